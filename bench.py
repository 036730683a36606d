"""Benchmark of the batched multi-adapter LoRA path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|prefill] [--impl ours|reference]

A step is one pass of the adapter path (shrink + expand at each of the block's four sites) over one
batch of synthetic input. The default workload is the decode mixed batch: hidden 4096 / intermediate
12288 block, 64 one-token sequences, 16 rank-16 adapters on all seven projections, 25% base-only tokens.
Under torchrun (N > 1) every rank runs that batch on its own GPU over its own disjoint adapter set
(adapter-affine partitioning, no collective on the data path): weak scaling.

L2: the step rotates over enough copies of the slot pool, inputs and outputs (>= 512 MB in total) that
every step reads its slabs from HBM, not from the 126 MB L2.

Prints ONE JSON line (rank 0).
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

METRIC = "mixed-adapter LoRA tokens/s (one transformer block's adapter path)"
UNIT = "tokens/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], "measured", d
    return 6650.0, "fallback", {}


PREFILL_SEQS = 8


def make_workload(name, seed, workloads=None):
    if workloads is None:
        from pocket_engine_b200 import workloads
    if name == "decode":
        return workloads.config2(seed=seed)
    if name == "prefill":
        return workloads.config3(seed=seed, seqs=PREFILL_SEQS)
    if name == "plumbing":
        return workloads.config1(seed=seed)
    raise SystemExit(f"unknown workload {name}")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                       "100", "-i", str(index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            c = [v.strip() for v in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for n, v in zip(names, c[5:9]):
                if v == "Active":
                    reasons.add(n)
        os.unlink(self.f.name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def shared_config(wl, work):
    """What both arms print as `config`: the workload, and how each arm keeps its inputs out of the caches."""
    return {"workload": wl.name, "tokens_per_step": wl.tokens, "lora_tokens": work["lora_tokens"], "adapters": wl.n_adapters,
            "slots_present": work["slots_present"], "sites": len(wl.sites),
            "partitioning": "adapter-affine, one batch per GPU, no collective",
            "l2": "inputs larger than L2: the GPU arm rotates over copies of pool + x + y of >= 512 MiB in total (126 MB L2); "
                  "the CPU arm streams its one copy (49 MB), larger than the host's L2",
            "metadata": "the step's grouping and launch records (built once per step and shared by all layers of a model) "
                        "run outside the device-timed `value` and inside `e2e`; their time is reported as meta_us"}


# ------------------------------------------------------------------------------------- ours

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the kernels that dominate the two block
# workloads, from the ncu captures summarised under profiles/ (decode_block_cluster_kernel_launch_records.md: the
# gate/up layer's cluster kernel at full size: its slabs, x and y are read once, and its y writes stay in L2.
# prefill_block_tile_kernels_tma_pipelines.md: the gate/up expand captured on 2 of the 8 sequences, traffic scaled by
# 4 since it grows with the token count).
NCU_TRAFFIC = {
    ("decode-4096x12288-64tok-16xr16", "site[2]"): 19.60e6,
    ("decode-4096x12288-64tok-16xr16", "expand[2]"): 15.02e6,
    ("prefill-4096x12288-8x2048-r64", "expand[2]"): 4 * (214.6e6 + 148.2e6),
}


def kernel_bytes(wl, si, which, f32_out=False):
    """Algorithmic bytes of one launch of the shrink or the expand of site si (true ranks)."""
    site = wl.sites[si]
    tslot = wl.token_slot()
    present = np.unique(tslot[tslot > 0])
    n_tot = sum(p.rows for p in site.parts)
    np_ = len(site.parts)
    ye = 8 if f32_out else 4
    b = 0
    for s in present:
        ta = int((tslot == s).sum())
        r = wl.ranks[s - 1]
        if which == "shrink":
            b += 2 * np_ * r * site.cols + ta * np_ * r * 4
        elif which == "expand":
            b += 2 * n_tot * r + ta * np_ * r * 4 + ta * n_tot * ye
        else:  # "site": one kernel per layer, the intermediate never leaves the chip
            b += 2 * np_ * r * site.cols + 2 * n_tot * r + ta * n_tot * ye
    if which in ("shrink", "site"):
        b += 2 * int((tslot > 0).sum()) * site.cols
    return b


def run_ours(args, rank, world, local_rank):
    import torch
    pe = entry.load_package()
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    wl = make_workload(args.workload, seed=1000 * rank)
    work = wl.work()
    ns = len(wl.sites)
    # enough rotating copies that the slabs of consecutive steps never sit in L2
    probe = pe.Loras(wl.sites, wl.n_adapters, wl.max_rank, wl.tokens, wl.n_seqs, device=-1)
    pool_bytes = probe.slot_bytes * wl.n_adapters
    probe.close()
    copies = int(min(32, max(2, -(-512 * 2 ** 20 // pool_bytes))))
    if work["bytes"] > 4 * 126 * 2 ** 20:
        copies = 1  # one step already streams several times the L2 size
    if args.copies:
        copies = args.copies
    main = torch.cuda.Stream(device=dev)
    side = torch.cuda.Stream(device=dev)
    decode = int(wl.row_n.max()) == 1  # a decoding step: only one-token sequences
    # streams == 1: shrink and expand in stream order on one stream (consecutive kernels overlap through
    # programmatic dependent launch); streams == 2: the engine's fork/join with the shrink on a side stream
    side_h = side.cuda_stream if args.streams == 2 else None
    facs = [wl.factors(i) for i in range(wl.n_adapters)]
    sets = []
    # One pinned host buffer holds the step's activations, x of every layer and then y_base of every layer, and one
    # device buffer per copy mirrors it (x[si], y[si] are views), so a step's inputs travel in one copy and its
    # results (the y region) in one. The step's sequence table (cu, then the slot of every sequence) likewise.
    x_np = [wl.x_bits(si).view(np.int16).reshape(-1) for si in range(ns)]
    y_np = [pe.bf16_bits(wl.y_base(si)).view(np.int16).reshape(-1) for si in range(ns)]
    in_host = torch.from_numpy(np.concatenate(x_np + y_np)).pin_memory()
    x_off = np.concatenate([[0], np.cumsum([a.size for a in x_np])])
    y_off = x_off[-1] + np.concatenate([[0], np.cumsum([a.size for a in y_np])])
    assert all(int(o) % 8 == 0 for o in list(x_off) + list(y_off))  # 16-byte aligned views
    meta_host = torch.from_numpy(np.concatenate([wl.cu(), wl.row_slot]).astype(np.int32)).pin_memory()
    n_cu = len(wl.cu())
    def make_set():
        L = pe.Loras(wl.sites, wl.n_adapters, wl.max_rank, wl.tokens, wl.n_seqs, device=local_rank)
        prep = L.prep()
        for i in range(wl.n_adapters):
            L.upload(i + 1, L.insert(prep.prepare(f"a{i}", facs[i])), main.cuda_stream)
        pack = in_host.to(dev, non_blocking=True)
        x = [pack[int(x_off[si]):int(x_off[si + 1])].view(torch.bfloat16).view(wl.tokens, -1) for si in range(ns)]
        y = [pack[int(y_off[si]):int(y_off[si + 1])].view(torch.bfloat16).view(wl.tokens, -1) for si in range(ns)]
        meta_dev = meta_host.to(dev)
        cu, ss = meta_dev[:n_cu], meta_dev[n_cu:]
        L.meta_build(cu.data_ptr(), ss.data_ptr(), wl.n_seqs, main.cuda_stream)
        step = L.lora_step(L.max_lora_tiles(), main.cuda_stream, decode=decode)
        lins = [pe.Linear(L, si) for si in range(ns)]
        L.set_apply_mode(0 if args.path == "apply-pair" else 1)
        L.set_early_x(args.early_x)
        return {"L": L, "x": x, "y": y, "cu": cu, "ss": ss, "step": step, "lins": lins, "pack": pack,
                "meta": meta_dev, "yreg": pack[int(y_off[0]):]}

    for c in range(copies):
        sets.append(make_set())
    torch.cuda.synchronize()

    fused = args.path != "pair"

    def block(S, m, s):
        for si in range(ns):
            S["lins"][si].forward(S["x"][si].data_ptr(), wl.tokens, S["y"][si].data_ptr(), S["y"][si].shape[1], False,
                                  lora=S["step"], main=m, side=s, fused=fused)

    # one CUDA graph per copy: the block's 8 launches with the engine's fork/join choreography
    graphs = []
    with torch.cuda.stream(main):
        for S in sets:
            block(S, main.cuda_stream, side_h)  # warm every kernel before capture
        torch.cuda.synchronize()
        for S in sets:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=main):
                block(S, main.cuda_stream, side_h)
            graphs.append(g)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: K steps, each `inner` passes of the block (graph replays over the rotating copies),
    # so that the timed region is long against launch and event jitter; reported per single pass
    inner = max(1, args.inner_repeats) if decode else 1
    with torch.cuda.stream(main):
        for i in range(args.warmup):
            graphs[i % copies].replay()
        barrier()
        sampler = ClockSampler(local_rank) if rank == 0 else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        for i in range(args.steps * inner):
            graphs[(args.warmup + i) % copies].replay()
        e1.record(main)
        barrier()
        ms = e0.elapsed_time(e1) / inner
    # keep the sampler alive a little longer for short runs so it sees load
    if sampler is not None and ms < 400:
        with torch.cuda.stream(main):
            t_end = time.time() + 0.5
            while time.time() < t_end:
                for i in range(copies):
                    graphs[i].replay()
                torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None

    # ---- the same with x vouched for (plora_set_early_x): here x was written long before the step, so the vouching
    # is true; reported beside the headline, which stays the form that is safe behind any producer
    early_variant = None
    if decode and fused and not args.early_x:
        with torch.cuda.stream(main):
            eg = []
            for S in sets:
                S["L"].set_early_x(True)
                block(S, main.cuda_stream, side_h)
            torch.cuda.synchronize()
            for S in sets:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=main):
                    block(S, main.cuda_stream, side_h)
                eg.append(g)
                S["L"].set_early_x(False)
            for i in range(args.warmup):
                eg[i % copies].replay()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(main)
            for i in range(args.steps * inner):
                eg[(args.warmup + i) % copies].replay()
            a1.record(main)
            barrier()
            early_ms = a0.elapsed_time(a1) / inner
            del eg
        early_variant = early_ms

    # ---- end to end through the C ABI with host buffers: H2D of x, y_base and the step's sequence table,
    # device metadata build + grouping, the block, D2H of y
    # Two steps are in flight at a time (two streams, two result buffers; consecutive steps use different copies),
    # so the copy of one step's inputs overlaps the other's kernels and result copy; the host waits for step i - 1
    # after issuing step i. (--e2e-depth: one step in flight runs at 312 us per step, two at 181, three at 188.)
    e2e_sets = list(sets)
    while len(e2e_sets) < max(2, args.e2e_depth):  # steps in flight need their own sets of buffers
        e2e_sets.append(make_set())
    torch.cuda.synchronize()
    depth = max(1, min(3, args.e2e_depth))
    lanes = [main] + [torch.cuda.Stream(device=dev) for _ in range(depth - 1)]
    y_out = [torch.empty(sets[0]["yreg"].numel(), dtype=torch.int16).pin_memory() for _ in range(depth)]
    h2d = in_host.numel() * 2 + meta_host.numel() * 4
    d2h = y_out[0].numel() * 2

    def e2e_issue(S, lane):
        stream = lanes[lane]
        m = stream.cuda_stream
        with torch.cuda.stream(stream):
            S["pack"].copy_(in_host, non_blocking=True)
            S["meta"].copy_(meta_host, non_blocking=True)
            S["L"].meta_build(S["cu"].data_ptr(), S["ss"].data_ptr(), wl.n_seqs, m)
            st = S["L"].lora_step(S["L"].max_lora_tiles(), m, decode=decode)
            for si in range(ns):
                S["lins"][si].forward(S["x"][si].data_ptr(), wl.tokens, S["y"][si].data_ptr(), S["y"][si].shape[1],
                                      False, lora=st, main=m, side=side_h if depth == 1 else None, fused=fused)
            y_out[lane].copy_(S["yreg"], non_blocking=True)

    # One CUDA graph per (copy, lane) holds the whole step as issued above (the two host-to-device copies, the metadata
    # kernels, the layers, the device-to-host copy), so that a step costs the host one replay instead of a dozen calls
    # through the binding: at 190 us per step the Python side of those calls was what bounded the rate, not PCIe.
    e2e_graphs = {}
    if not args.no_e2e_graph:
        torch.cuda.synchronize()
        for k in range(len(e2e_sets)):
            for lane in range(depth):
                if len(e2e_sets) % depth == 0 and k % depth != lane:
                    continue  # with an even number of copies a copy always meets the same lane
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=lanes[lane]):
                    e2e_issue(e2e_sets[k], lane)
                e2e_graphs[(k, lane)] = g
        torch.cuda.synchronize()

    ahead = max(1, args.e2e_ahead)
    done = [torch.cuda.Event() for _ in range(ahead + 1)]

    def e2e_run(first, count):
        for i in range(count):
            k, lane = (first + i) % len(e2e_sets), (first + i) % depth
            if (k, lane) in e2e_graphs:
                with torch.cuda.stream(lanes[lane]):
                    e2e_graphs[(k, lane)].replay()
            else:
                e2e_issue(e2e_sets[k], lane)
            # The host waits for the step issued `ahead` steps ago before it issues the next one. Stream order alone
            # keeps the buffers safe (a copy and a result buffer always meet the same lane); the wait only bounds how
            # far the host runs ahead of the device, and at one step ahead its wake-up and launch time (some 40 us)
            # showed up in every step.
            done[i % len(done)].record(lanes[lane])
            if depth == 1:
                lanes[0].synchronize()
            elif i >= ahead:
                done[(i - ahead) % len(done)].synchronize()
        for s in lanes:
            s.synchronize()

    e2e_run(0, args.warmup)
    barrier()
    t0 = time.perf_counter()
    e2e_run(args.warmup, args.steps)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3

    # ---- per-kernel durations: for every (layer, shrink | expand) one graph holding that launch once per
    # rotating copy (so each launch finds its slabs, x and y in HBM), CUDA events around replays on the launching
    # stream, divided by the number of launches. Single eager launches between two events would add several
    # microseconds of launch and event overhead to kernels that last about as long.
    kern = {}
    reps = 5 if decode else 2
    with torch.cuda.stream(main):
        m = main.cuda_stream
        for si in range(ns):
            for which in (("site",) if args.path == "apply" and decode else ("shrink", "expand")):
                def launches():
                    for S in sets:
                        hook = S["lins"][si].lora
                        if which == "shrink":
                            S["L"].shrink(hook, S["step"], S["x"][si].data_ptr(), wl.tokens, m)
                        elif which == "expand":
                            S["L"].expand(hook, S["step"], wl.tokens, S["y"][si].data_ptr(), S["y"][si].shape[1], False, m)
                        else:
                            S["L"].apply(hook, S["step"], S["x"][si].data_ptr(), wl.tokens, S["y"][si].data_ptr(),
                                         S["y"][si].shape[1], False, m)
                launches()
                main.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=main):
                    launches()
                g.replay()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(main)
                for _ in range(reps):
                    g.replay()
                b.record(main)
                main.synchronize()
                kern[f"{which}[{si}]"] = {"us": 1e3 * a.elapsed_time(b) / (reps * copies), "bytes": kernel_bytes(wl, si, which)}
                del g
        # the step's metadata kernels, for the record: device time of the two launches (tile list from the
        # sequence table; grouping with the launch records), replayed from a graph so that no host launch time is counted
        evs = []
        with torch.cuda.stream(main):
            for i in range(copies):
                S = sets[i]
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=main):
                    S["L"].meta_build(S["cu"].data_ptr(), S["ss"].data_ptr(), wl.n_seqs, m)
                    S["L"].lora_step(S["L"].max_lora_tiles(), m, decode=decode)
                g.replay()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(main)
                for _ in range(20):
                    g.replay()
                b.record(main)
                evs.append((a, b, g))
        torch.cuda.synchronize()
        meta_us = 1e3 * float(np.mean([a.elapsed_time(b) for a, b, _ in evs])) / 20
        del evs
    for S in e2e_sets:
        S["L"].device_status()

    # max over ranks
    if world > 1:
        t = torch.tensor([ms, e2e_ms, early_variant or 0.0], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
        early_variant = float(t[2]) if early_variant is not None else None
    if rank != 0:
        return None
    peak, peak_kind, _ = peaks()
    dom = max(kern, key=lambda k: kern[k]["us"])
    ach = kern[dom]["bytes"] / (kern[dom]["us"] * 1e-6) / 1e9
    step_us = 1e3 * ms / args.steps
    out = {
        "metric": METRIC, "value": world * wl.tokens * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": shared_config(wl, work),
        "run": {"copies": copies, "rotating_mib": round(copies * (pool_bytes + d2h + h2d // 2) / 2 ** 20),
                "graph": f"one CUDA graph per copy, {args.streams} stream(s)", "path": args.path,
                "early_x": bool(args.early_x), "inner_repeats": inner,
                "timed_region": f"{args.steps} steps x {inner} passes of the block; value and ms_per_step are per pass"},
        "e2e": {"value": world * wl.tokens * args.steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps, "steps_in_flight": depth, "host_runs_ahead": ahead,
                "launch": "one CUDA graph per copy and lane (copies, metadata kernels, layers)" if e2e_graphs else "individual calls"},
        "gpu_launches": ((4 if args.path == "apply" else 8) if decode else 16) * args.steps * inner,
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                     "peak_kind": peak_kind, "traffic": NCU_TRAFFIC.get((wl.name, dom)), "us_per_launch": kern[dom]["us"],
                     "algorithmic_bytes_per_launch": kern[dom]["bytes"]},
        "step_roofline": {"algorithmic_bytes_per_step": work["bytes"], "achieved_gbs": work["bytes"] / (step_us * 1e-6) / 1e9,
                          "frac": work["bytes"] / (step_us * 1e-6) / 1e9 / peak, "us_per_step": step_us},
        "kernels": {k: {"us": round(v["us"], 3), "gbs": round(v["bytes"] / (v["us"] * 1e-6) / 1e9, 1)} for k, v in kern.items()},
        "meta_us": meta_us,
        "clocks": clocks,
    }
    if early_variant is not None:
        eus = 1e3 * early_variant / args.steps
        out["x_vouched_variant"] = {
            "what": "plora_set_early_x(1): the caller vouches that x is complete before the kernel ahead of plora_apply starts, "
                    "so x is read and the shrink done ahead of the dependency wait; y is still read after it",
            "ms_per_step": early_variant / args.steps, "value": world * wl.tokens * args.steps / (early_variant * 1e-3),
            "step_roofline_frac": work["bytes"] / (eus * 1e-6) / 1e9 / peak}
    return out


# ------------------------------------------------------------------- FP8 fused layer, TP layer

def _event_time(torch, stream, fn, steps, warmup, barrier):
    with torch.cuda.stream(stream):
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(warmup + i)
        e1.record(stream)
        barrier()
    return e0.elapsed_time(e1)


def run_fp8(args, rank, world, local_rank):
    """Heterogeneous adapters over an FP8 base layer (4096 -> 12288, 256 decode tokens, 128 adapters of rank
    8..128, Zipf popularity): a step = row quantisation of x, shrink on the bf16 x, then the FP8 GEMM with the
    adapter expand fused into its epilogue. --tokens N runs the same layer at a prefill-sized M."""
    import torch
    pe = entry.load_package()
    from pocket_engine_b200 import workloads
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if args.tokens:
        seqs = max(1, args.tokens // 2048)
        wl = workloads.Workload(f"fp8-prefill-4096x12288-{seqs}x2048-r64", workloads.config4().sites, [64] * seqs, 1.0,
                                [2048] * seqs, list(range(1, seqs + 1)), 1000 * rank, max_rank=128)
    else:
        wl = workloads.config4(seed=1000 * rank, two_part=args.two_part)  # --two-part: the engine's gate + up layer
    site = wl.sites[0]
    K, N, T = site.cols, site.width(), wl.tokens
    main = torch.cuda.Stream(device=dev)
    rng = np.random.default_rng([wl.seed, 77])
    w = np.clip(rng.standard_normal((N, K), dtype=np.float32), -448, 448)
    wq_h = torch.from_numpy(w).to(torch.float8_e4m3fn).view(torch.uint8)
    sn_h = torch.from_numpy((rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32))
    x_h = torch.from_numpy(wl.x_bits(0).view(np.int16)).pin_memory()
    copies = args.copies or 2
    sets = []
    used = sorted(set(int(s) for s in wl.row_slot if s))
    for c in range(copies):
        L = pe.Loras(wl.sites, wl.n_adapters, wl.max_rank, T, wl.n_seqs, device=local_rank)
        prep = L.prep()
        for i in range(wl.n_adapters):
            L.upload(i + 1, L.insert(prep.prepare(f"a{i}", wl.factors(i))), main.cuda_stream)
        S = {"L": L, "x": x_h.to(dev).view(torch.bfloat16), "xq": torch.zeros(T, K, dtype=torch.uint8, device=dev),
             "st": torch.zeros(T, dtype=torch.float32, device=dev), "wq": wq_h.to(dev), "sn": sn_h.to(dev),
             "y": torch.zeros(T, N, dtype=torch.bfloat16, device=dev), "cu": torch.from_numpy(wl.cu()).to(dev),
             "ss": torch.from_numpy(wl.row_slot.copy()).to(dev), "hook": L.hook(0)}
        L.meta_build(S["cu"].data_ptr(), S["ss"].data_ptr(), wl.n_seqs, main.cuda_stream)
        S["step"] = L.lora_step(L.max_lora_tiles(), main.cuda_stream, decode=int(wl.row_n.max()) == 1)
        sets.append(S)
    torch.cuda.synchronize()

    def block(S, m):
        L = S["L"]
        L.fp8_quant_rows(S["x"].data_ptr(), T, K, S["xq"].data_ptr(), S["st"].data_ptr(), m)
        L.shrink(S["hook"], S["step"], S["x"].data_ptr(), T, m)
        L.linear_fp8_fused(S["hook"], S["step"], S["xq"].data_ptr(), S["st"].data_ptr(), S["wq"].data_ptr(),
                           S["sn"].data_ptr(), T, S["y"].data_ptr(), N, False, m)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms = _event_time(torch, main, lambda i: block(sets[i % copies], main.cuda_stream), args.steps, args.warmup, barrier)
    # the fused kernel alone
    evs = []
    with torch.cuda.stream(main):
        for i in range(12):
            S = sets[i % copies]
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            S["L"].shrink(S["hook"], S["step"], S["x"].data_ptr(), T, main.cuda_stream)
            a.record(main)
            S["L"].linear_fp8_fused(S["hook"], S["step"], S["xq"].data_ptr(), S["st"].data_ptr(), S["wq"].data_ptr(),
                                    S["sn"].data_ptr(), T, S["y"].data_ptr(), N, False, main.cuda_stream)
            b.record(main)
            evs.append((a, b))
        torch.cuda.synchronize()
    fused_us = 1e3 * float(np.mean([a.elapsed_time(b) for a, b in evs[2:]]))
    clocks = sampler.stop() if sampler is not None else None

    # ---- comparison rows (library kernels; not part of the product path)
    compare = {}
    try:
        # (a) what the engine does with an FP8 layer (src/gpu.rs:1183-1277, src/linear.rs:844-847): a library FP8 GEMM,
        # then the adapter as a separate read-modify-write pass over y. torch._scaled_mm with one scale per token and
        # per output channel is cuBLASLt's row-wise scaled FP8 GEMM.
        f8 = torch.float8_e4m3fn
        def library(S, m):
            L = S["L"]
            L.fp8_quant_rows(S["x"].data_ptr(), T, K, S["xq"].data_ptr(), S["st"].data_ptr(), m)
            torch._scaled_mm(S["xq"].view(f8), S["wq"].view(f8).t(), scale_a=S["st"].view(T, 1), scale_b=S["sn"].view(1, N),
                             out_dtype=torch.bfloat16, out=S["y"])
            L.apply(S["hook"], S["step"], S["x"].data_ptr(), T, S["y"].data_ptr(), N, False, m)
        t_lib = _event_time(torch, main, lambda i: library(sets[i % copies], main.cuda_stream), args.steps, args.warmup, barrier)
        compare["library_fp8_gemm_then_apply_us"] = 1e3 * t_lib / args.steps
    except Exception as e:  # noqa: BLE001
        compare["library_fp8_gemm_then_apply_us"] = f"unavailable: {type(e).__name__}: {e}"[:160]
    try:
        # (b) a measured FP8 dense peak for the tensor-pipe fractions: the same library GEMM at 8192^3, per-tensor scales
        n8 = 8192
        a8 = torch.randn(n8, n8, device=dev).to(torch.float8_e4m3fn)
        b8 = torch.randn(n8, n8, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        o8 = torch.empty(n8, n8, dtype=torch.bfloat16, device=dev)
        f = lambda i: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=o8)  # noqa: E731
        best = min(_event_time(torch, main, f, 1, 3 if r == 0 else 0, barrier) for r in range(8))
        t_sus = _event_time(torch, main, f, 200, 0, barrier) / 200
        compare["fp8_dense_peak_tflops_burst"] = 2.0 * n8 ** 3 / (best * 1e-3) / 1e12
        compare["fp8_dense_peak_tflops_sustained"] = 2.0 * n8 ** 3 / (t_sus * 1e-3) / 1e12
        del a8, b8, o8
    except Exception as e:  # noqa: BLE001
        compare["fp8_dense_peak_tflops_burst"] = f"unavailable: {type(e).__name__}: {e}"[:160]
    # end to end with host buffers: x in, y out
    y_out = torch.empty(T, N, dtype=torch.int16).pin_memory()

    def e2e(i):
        S = sets[i % copies]
        S["x"].view(torch.int16).copy_(x_h, non_blocking=True)
        block(S, main.cuda_stream)
        y_out.copy_(S["y"].view(torch.int16), non_blocking=True)

    with torch.cuda.stream(main):
        for i in range(args.warmup):
            e2e(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e(i)
            main.synchronize()
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    for S in sets:
        S["L"].device_status()
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if rank != 0:
        return None
    tslot = wl.token_slot()
    t_l = int((tslot > 0).sum())
    slab = sum(2 * wl.ranks[s - 1] * (K + N) for s in used)
    s_bytes = sum(int((tslot == s).sum()) * wl.ranks[s - 1] * 8 for s in used)
    fused_bytes = K * N + 4 * N + T * K + 4 * T + sum(2 * wl.ranks[s - 1] * N for s in used) + s_bytes // 2 + 2 * T * N
    step_bytes = fused_bytes + sum(2 * wl.ranks[s - 1] * K for s in used) + 2 * t_l * K + s_bytes // 2 + 2 * T * K + T * K
    flops = 2.0 * T * K * N + sum(int((tslot == s).sum()) * 2.0 * wl.ranks[s - 1] * (K + N) for s in used)
    peak, kind, pk = peaks()
    fp8_peak = 2 * pk.get("bf16_tflops", 1590.0)
    us = 1e3 * ms / args.steps
    meas = compare.get("fp8_dense_peak_tflops_burst")
    meas_sus = compare.get("fp8_dense_peak_tflops_sustained")
    return {"metric": METRIC, "value": world * T * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8 e4m3 base + bf16 adapters, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": wl.name, "tokens_per_step": T, "lora_tokens": t_l, "adapters": wl.n_adapters,
                       "slots_present": len(used), "layer": f"{K}->{N}", "l2": f"{copies} rotating copies of pool+W",
                       "step": "row quantisation + shrink + FP8 layer with the adapter term"},
            "e2e": {"value": world * T * args.steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 2 * T * K,
                    "d2h_bytes_per_step": 2 * T * N, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": 4 * args.steps,
            "roofline": {"bound": "hbm" if step_bytes / (peak * 1e9) > flops / (fp8_peak * 1e12) else "tensor",
                         "kernel": "plora_linear_fp8_fused: K-split reduction, plora_gemm_fused_kernel (base product + long "
                                   "runs' adapter term), gather expand for the other tokens", "achieved": fused_bytes / (fused_us * 1e-6) / 1e9, "peak": peak,
                         "unit": "GB/s", "frac": fused_bytes / (fused_us * 1e-6) / 1e9 / peak, "peak_kind": kind,
                         "traffic": None, "us_per_launch": fused_us, "algorithmic_bytes_per_launch": fused_bytes,
                         "tflops": flops / (fused_us * 1e-6) / 1e12,
                         "tensor_frac_of_2x_bf16_burst_peak": flops / (fused_us * 1e-6) / 1e12 / fp8_peak,
                         "tensor_frac_of_2x_bf16_sustained_peak": flops / (fused_us * 1e-6) / 1e12 /
                         (2 * pk.get("bf16_tflops_sustained", 1400.0)),
                         "tensor_frac_of_measured_fp8_burst_peak": flops / (fused_us * 1e-6) / 1e12 / meas
                         if isinstance(meas, float) else None,
                         "tensor_frac_of_measured_fp8_sustained_peak": flops / (fused_us * 1e-6) / 1e12 / meas_sus
                         if isinstance(meas_sus, float) else None},
            "compare": compare,
            "step_roofline": {"algorithmic_bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (us * 1e-6) / 1e9,
                              "frac": step_bytes / (us * 1e-6) / 1e9 / peak, "us_per_step": us,
                              "tflops": flops / (us * 1e-6) / 1e12},
            "clocks": clocks}


def run_fused_bf16(args, rank, world, local_rank):
    """The prefill block with its bf16 base layers: a step = the four layers of one transformer block over 8 x 2048
    tokens, each as y = x W^T + adapter term. Two ways, timed the same way: (a) the engine's order, a library bf16
    matrix multiply (cuBLAS through torch.matmul) followed by shrink and the read-modify-write expand; (b) shrink,
    then the library's one-kernel layer (base product and adapter term on the tensor cores, y written once)."""
    import torch
    pe = entry.load_package()
    from pocket_engine_b200 import workloads
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    wl = workloads.config3(seed=1000 * rank, seqs=args.seqs)
    ns, T = len(wl.sites), wl.tokens
    main = torch.cuda.Stream(device=dev)
    L = pe.Loras(wl.sites, wl.n_adapters, wl.max_rank, T, wl.n_seqs, device=local_rank)
    prep = L.prep()
    for i in range(wl.n_adapters):
        L.upload(i + 1, L.insert(prep.prepare(f"a{i}", wl.factors(i))), main.cuda_stream)
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    xs = [torch.from_numpy(wl.x_bits(si).view(np.int16)).to(dev).view(torch.bfloat16) for si in range(ns)]
    ws = [(torch.randn(s.width(), s.cols, device=dev, generator=g) / s.cols ** 0.5).to(torch.bfloat16) for s in wl.sites]
    ys = [torch.zeros(T, s.width(), dtype=torch.bfloat16, device=dev) for s in wl.sites]
    cu, ss = torch.from_numpy(wl.cu()).to(dev), torch.from_numpy(wl.row_slot.copy()).to(dev)
    L.meta_build(cu.data_ptr(), ss.data_ptr(), wl.n_seqs, main.cuda_stream)
    step = L.lora_step(L.max_lora_tiles(), main.cuda_stream)
    hooks = [L.hook(si) for si in range(ns)]
    torch.cuda.synchronize()

    def separate(i):
        for si in range(ns):
            torch.matmul(xs[si], ws[si].t(), out=ys[si])
            L.apply(hooks[si], step, xs[si].data_ptr(), T, ys[si].data_ptr(), ys[si].shape[1], False, main.cuda_stream)

    def fused(i):
        for si in range(ns):
            L.shrink(hooks[si], step, xs[si].data_ptr(), T, main.cuda_stream)
            L.linear_bf16_fused(hooks[si], step, xs[si].data_ptr(), ws[si].data_ptr(), T, ys[si].data_ptr(),
                                ys[si].shape[1], False, main.cuda_stream)

    def base_only(i):
        for si in range(ns):
            torch.matmul(xs[si], ws[si].t(), out=ys[si])

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    t_fused = _event_time(torch, main, fused, args.steps, args.warmup, barrier)
    clocks = sampler.stop() if sampler is not None else None
    t_sep = _event_time(torch, main, separate, args.steps, args.warmup, barrier)
    t_base = _event_time(torch, main, base_only, args.steps, args.warmup, barrier)
    L.device_status()
    if world > 1:
        t = torch.tensor([t_fused, t_sep, t_base], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        t_fused, t_sep, t_base = (float(v) for v in t)
    if rank != 0:
        return None
    flops = sum(2.0 * T * s.cols * s.width() for s in wl.sites) + wl.work()["flops"]
    _, _, pk = peaks()
    tf_peak = pk.get("bf16_tflops_sustained") or 1400.0
    us = 1e3 * t_fused / args.steps
    return {"metric": METRIC, "value": world * T * args.steps / (t_fused * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_fused / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl.name + "+bf16-base-layers", "tokens_per_step": T, "adapters": wl.n_adapters,
                       "step": "per layer: shrink, then base product + adapter term in one kernel (y written once)",
                       "l2": "inputs larger than L2 (x, W, y of the four layers)"},
            "gpu_launches": 4 * ns * args.steps,
            "roofline": {"bound": "tensor", "kernel": "plora_gemm_fused_kernel (bf16)", "achieved": flops / (us * 1e-6) / 1e12,
                         "peak": tf_peak, "unit": "TFLOP/s", "frac": flops / (us * 1e-6) / 1e12 / tf_peak if tf_peak else None,
                         "peak_kind": "measured, sustained bf16", "traffic": None},
            "compare": {"library_gemm_then_shrink_expand_ms": t_sep / args.steps, "library_gemm_alone_ms": t_base / args.steps,
                        "one_kernel_layers_ms": t_fused / args.steps},
            "clocks": clocks}


def tp_measure(args, rank, world, local_rank, exchanges, steps, warmup):
    """Tensor-parallel 27B-shaped layer set (q, o, gate/up, down; hidden 5120, intermediate 17408), 512 tokens,
    32 rank-32 adapters: column-parallel q and gate/up, row-parallel o and down whose [512, 32] shrink partials are
    summed over the ranks, per `exchanges`: "nccl" = an NCCL all-reduce, "fused" = the library's one-kernel exchange
    over peer memory. Strong scaling: the same batch over more GPUs. Returns {exchange: record}; every record carries
    a parity check of sampled token rows against the unsharded fp64 oracle (rank 0, outside the timed region)."""
    import torch
    import torch.distributed as dist
    pe = entry.load_package()
    from pocket_engine_b200 import tp, workloads
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    wl = workloads.config5()
    sh = tp.ShardedWorkload(wl, world, rank)
    ns = len(sh.sites)
    copies = args.copies or 4
    facs = [sh.factors(i) for i in range(sh.n_adapters)]
    x_h = [sh.x_bits(si) for si in range(ns)]
    y_h = [sh.y_base(si) for si in range(ns)]
    sets = []
    for c in range(copies):
        L = pe.Loras(sh.sites, sh.n_adapters, sh.max_rank, sh.tokens, sh.n_seqs, device=local_rank)
        prep = L.prep()
        for i in range(sh.n_adapters):
            L.upload(i + 1, L.insert(prep.prepare(f"a{i}", facs[i])))
        x = [torch.from_numpy(x_h[si].view(np.int16)).to(dev).view(torch.bfloat16) for si in range(ns)]
        y = [torch.from_numpy(pe.bf16_bits(y_h[si]).reshape(sh.tokens, -1).view(np.int16)).to(dev).view(torch.bfloat16)
             for si in range(ns)]
        L.meta_upload(pe.fill_tiles(sh.row_n, sh.row_slot, L.max_lora_tiles()))
        step = L.lora_step(L.max_lora_tiles())
        if "fused" in exchanges:
            tp.connect_exchange(L, rank, world)
        sets.append({"L": L, "x": x, "y": y, "step": step})
    torch.cuda.synchronize()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # sampled rows for the parity check: the first and last rows of the prompt chunks, and decode rows
    rng = np.random.default_rng(17)
    cu = wl.cu()
    rows = set(int(v) for v in rng.choice(wl.tokens, 56, replace=False))
    for i, n in enumerate(wl.row_n):
        if n > 1:
            rows.update([int(cu[i]), int(cu[i + 1]) - 1, int(cu[i]) + 15, int(cu[i]) + 16])
    rows = np.array(sorted(rows), np.int64)
    y32 = [torch.from_numpy(y_h[si].copy()).to(dev) for si in range(ns)]
    orc = entry.load_oracle() if rank == 0 else None  # the checker of the parity record, never the thing timed
    full_adapters = [orc.OracleAdapter(wl.sites, wl.factors(i), wl.max_rank) for i in range(wl.n_adapters)] if rank == 0 else []
    peak, kind, _ = peaks()
    shw = workloads.Workload(sh.name, sh.sites, sh.ranks, sh.scale, sh.row_n, sh.row_slot, sh.seed).work()
    out = {}
    for exchange in exchanges:
        for S in sets:
            S["lins"] = [tp.TPLinear(S["L"], si, sh.modes[si], exchange=exchange) for si in range(ns)]
        stream = torch.cuda.current_stream()

        def block(i, stream_handle=None):
            S = sets[i % copies]
            for si in range(ns):
                S["lins"][si].forward(S["x"][si].data_ptr(), sh.tokens, S["y"][si].data_ptr(), S["y"][si].shape[1], False,
                                      lora=S["step"], main=stream_handle if stream_handle is not None else stream.cuda_stream)

        # one CUDA graph per copy (kernels and the collectives), replayed; eager launches if capture is refused
        mode = "cuda graph per copy"
        cap = torch.cuda.Stream(device=dev)
        graphs = []
        try:
            with torch.cuda.stream(cap):
                for c in range(copies):
                    block(c, cap.cuda_stream)
                torch.cuda.synchronize()
                for c in range(copies):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=cap):
                        block(c, cap.cuda_stream)
                    graphs.append(g)
                torch.cuda.synchronize()
            stream = cap
            run = lambda i: graphs[i % copies].replay()  # noqa: E731
        except Exception as e:  # noqa: BLE001
            mode = f"eager launches (graph capture refused: {type(e).__name__})"
            stream = torch.cuda.current_stream()
            graphs = []
            run = block
        sampler = ClockSampler(local_rank) if rank == 0 else None
        ms = _event_time(torch, stream, run, steps, warmup, barrier)
        # the collective alone: one [512, lds] plane
        s0 = sets[0]["lins"][1]._s[:sh.tokens]
        if world == 1:
            ar = 0.0
        elif exchange == "fused":  # the exchange kernel alone (partials left over from the last step)
            L0, lin0 = sets[0]["L"], sets[0]["lins"][1]
            ar = _event_time(torch, stream, lambda i: L0.s_exchange(lin0.lora, sets[0]["step"], sh.tokens, stream.cuda_stream),
                             50, 5, barrier) / 50
        else:
            ar = _event_time(torch, stream, lambda i: dist.all_reduce(s0), 50, 5, barrier) / 50
        clocks = sampler.stop() if sampler is not None else None
        # parity: one pass in f32 on fresh outputs, sampled rows of every layer gathered on rank 0
        S = sets[0]
        worst = [0.0, 0.0]
        cur = torch.cuda.current_stream()
        for si in range(ns):
            y = y32[si].clone()
            S["lins"][si].forward(S["x"][si].data_ptr(), sh.tokens, y.data_ptr(), y.shape[1], True, lora=S["step"],
                                  main=cur.cuda_stream)
            torch.cuda.synchronize()
            outs = [None] * world
            dist.all_gather_object(outs, y[torch.from_numpy(rows).to(dev)].cpu().numpy())
            if rank == 0:
                got = sh.assemble(si, outs)
                table = orc.OracleTable(wl.sites, wl.n_adapters)
                for i, a in enumerate(full_adapters):
                    table.upload(i + 1, a)
                tslot = wl.token_slot()[rows]
                words = [int((tslot > 0).sum())]
                for i, sl in enumerate(tslot):
                    if sl:
                        words += [i, 1, int(sl)]
                want = wl.y_base(si)[rows].astype(np.float64)
                orc.site_f64(np.ascontiguousarray(wl.x_bits(si)[rows]), wl.sites[si].cols, np.array(words, np.int32),
                             table.tables[si], want)
                d = np.abs(got - want)
                rms = float(np.sqrt(np.mean(want ** 2)))
                worst = [max(worst[0], float(d.max()) / rms), max(worst[1], float(d.mean()) / rms)]
        for S2 in sets:
            S2["L"].device_status()
        t = torch.tensor([ms, ar], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ar = float(t[0]), float(t[1])
        us = 1e3 * ms / steps
        out[exchange] = {
            "ms_per_step": ms / steps, "tokens_per_s": sh.tokens * steps / (ms * 1e-3), "steps": steps, "warmup": warmup,
            "collective_us": 1e3 * ar, "collective_bytes": int(sh.tokens * sets[0]["L"].lds * 4),
            "collective": ("one exchange kernel per row-parallel layer: partials stored to every rank's staging memory over "
                           "NVLink, flags, sum in rank order" if exchange == "fused" else
                           "NCCL all-reduce(sum) of the f32 shrink partials") + ", 2 per step",
            "step_roofline": {"algorithmic_bytes_per_step_per_gpu": shw["bytes"],
                              "achieved_gbs_per_gpu": shw["bytes"] / (us * 1e-6) / 1e9,
                              "frac": shw["bytes"] / (us * 1e-6) / 1e9 / peak, "us_per_step": us},
            "parity": {"against": "unsharded fp64 oracle", "sampled_token_rows": int(len(rows)), "layers": ns,
                       "max_over_rms": worst[0], "mean_over_rms": worst[1],
                       "ok": bool(worst[0] <= 1e-2 and worst[1] <= 1e-3), "tolerance": "max 1e-2, mean 1e-3 of RMS(y)"},
            "launch": mode, "clocks": clocks}
        del graphs
    info = {"workload": wl.name, "tokens_per_step": sh.tokens, "adapters": sh.n_adapters, "scaling": "strong",
            "parallelism": f"tp{world}: column-parallel q, gate/up; row-parallel o, down", "l2": f"{copies} rotating copies"}
    for S in sets:
        S["L"].close()
    return info, out


def run_tp(args, rank, world, local_rank):
    """--workload tp: the tensor-parallel layer set alone, with the chosen exchange."""
    info, out = tp_measure(args, rank, world, local_rank, [args.exchange], args.steps, args.warmup)
    if rank != 0:
        return None
    r = out[args.exchange]
    return {"metric": METRIC, "value": r["tokens_per_s"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(info, collective=r["collective"], launch=r["launch"]),
            "gpu_launches": (2 * 4 + 2) * 2 * args.steps, "step_roofline": r["step_roofline"],
            "collective_us": r["collective_us"], "collective_bytes": r["collective_bytes"], "parity": r["parity"],
            "clocks": r["clocks"]}


# -------------------------------------------------------------------------------- CPU port

def cpu_port(wl_name, seconds, seed=0, threads=0, steps=None, warmup=0):
    """The oracle's multithreaded C restatement of the path, timed on the host cores. Returns
    (tokens/s, cores, sample description, ms per step). The prefill workload is sampled: one of its eight
    sequences (same shapes, one adapter), tokens/s counted on the tokens actually processed."""
    orc = entry.load_oracle()
    workloads = entry.load_inputs()  # the synthetic inputs only: the product library is not loaded by this arm
    bits = sys.modules["plora_inputs.sites"].bf16_bits
    wl = make_workload(wl_name, seed, workloads)
    full_name = wl.name
    if wl_name == "prefill":
        wl = workloads.config3(seed=seed, seqs=1)
    table = orc.OracleTable(wl.sites, wl.n_adapters)
    for i in range(wl.n_adapters):
        table.upload(i + 1, orc.OracleAdapter(wl.sites, wl.factors(i), wl.max_rank))
    tiles = orc.fill_tiles(wl.row_n, wl.row_slot, wl.tokens // 16 + wl.n_seqs)
    xs = [wl.x_bits(si) for si in range(len(wl.sites))]
    ys = [bits(wl.y_base(si)).reshape(wl.tokens, -1) for si in range(len(wl.sites))]
    s = np.zeros((wl.tokens, 4 * ((wl.max_rank + 15) // 16 * 16)), np.float32)
    threads = threads or orc.hw_threads()

    def one():
        for si, site in enumerate(wl.sites):
            orc.site_mt(xs[si], site.cols, tiles, table.tables[si], s, ys[si], False, threads)

    for _ in range(max(1, warmup) if wl.name == full_name else 0):
        one()
    n, t0 = 0, time.perf_counter()
    while True:
        one()
        n += 1
        el = time.perf_counter() - t0
        if (steps is not None and n >= steps) or (steps is None and el >= seconds):
            break
    what = "full steps" if wl.name == full_name else f"steps of a 1-of-8-sequences sample ({wl.name}) of {full_name}:"
    return wl.tokens * n / el, threads, f"{n} {what} in {el:.1f} s", 1e3 * el / n, wl


def run_reference(args, rank, world):
    """The reference has no CPU implementation of this path (it is GPU-only), so the timed CPU arm is the
    oracle's multithreaded port. When the reference's own kernels were compiled (oracle/_ref) and a GPU is
    visible, they are also timed on the same workload and reported beside it."""
    if rank != 0:
        return None
    v, cores, sample, ms, wl = cpu_port(args.workload, 0, steps=args.steps, warmup=args.warmup)
    wl = make_workload(args.workload, 0, entry.load_inputs())  # `config` names the whole workload (the sample says what ran)
    out = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic", "config": shared_config(wl, wl.work()),
           "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
           "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "note": "pocket-engine has no CPU path; this arm times the C port of its algorithm on the host cores"}
    try:
        out["reference_gpu_kernels"] = reference_gpu(args)
    except Exception as e:  # no GPU, no fatbin, or a driver error: report, do not fail the arm
        out["reference_gpu_kernels"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    try:  # the same launcher and grids over the drop-in kernel image this repository builds
        image = os.path.join(ROOT, "pocket-engine_b200", "plora_compat.fatbin")
        out["drop_in_image_same_grids"] = reference_gpu(args, image) if os.path.exists(image) else {"unavailable": "not built"}
    except Exception as e:
        out["drop_in_image_same_grids"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    return out


def reference_gpu(args, image=None):
    """pocket-engine's own lora_shrink / lora_expand (oracle/_ref fatbin; or another image with the same kernel
    names) on the same workload and the same rotation over pool copies, with the engine's grids and stream order;
    none of the product library's host code runs."""
    import importlib.util
    import torch
    spec = importlib.util.spec_from_file_location("plora_ref_kernels", os.path.join(ROOT, "oracle", "ref_kernels.py"))
    rk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rk)
    if image is None and not rk.available():
        return {"unavailable": "oracle/_ref fatbin not built"}
    if not torch.cuda.is_available():
        return {"unavailable": "no GPU"}
    orc = entry.load_oracle()
    workloads = entry.load_inputs()
    bits = sys.modules["plora_inputs.sites"].bf16_bits
    wl = make_workload(args.workload, 0, workloads)
    torch.cuda.set_device(0)
    ref = rk.RefKernels(image)
    max_rank = (wl.max_rank + 15) // 16 * 16
    lds = 4 * max_rank
    adapters = [orc.OracleAdapter(wl.sites, wl.factors(i), wl.max_rank) for i in range(wl.n_adapters)]
    slot_bytes = orc.lib().po_slot_bytes(orc.c_sites(wl.sites), len(wl.sites), max_rank)
    copies = int(min(32, max(2, -(-512 * 2 ** 20 // (slot_bytes * wl.n_adapters)))))
    tiles_h = orc.fill_tiles(wl.row_n, wl.row_slot, wl.tokens // 16 + wl.n_seqs)
    max_tiles = wl.tokens // 16 + wl.n_seqs
    sets = []
    for c in range(copies):
        pool = torch.empty(slot_bytes * wl.n_adapters, dtype=torch.uint8, device="cuda")
        tabs = []
        for si in range(len(wl.sites)):
            t = (orc.PoDesc * (wl.n_adapters + 1))()
            for i, a in enumerate(adapters):
                t[i + 1] = a.desc(si, pool.data_ptr() + i * slot_bytes)
            tabs.append(torch.frombuffer(bytearray(bytes(t)), dtype=torch.uint8).cuda())
        for i, a in enumerate(adapters):
            pool[i * slot_bytes:i * slot_bytes + a.len].copy_(torch.from_numpy(a.data[:a.len]))
        x = [torch.from_numpy(wl.x_bits(si).view(np.int16)).cuda() for si in range(len(wl.sites))]
        y = [torch.from_numpy(bits(wl.y_base(si)).reshape(wl.tokens, -1).view(np.int16)).cuda()
             for si in range(len(wl.sites))]
        sets.append({"pool": pool, "tabs": tabs, "x": x, "y": y, "tiles": torch.from_numpy(tiles_h.copy()).cuda(),
                     "s": torch.zeros(2, wl.tokens, lds, dtype=torch.float32, device="cuda")})
    main, side = torch.cuda.Stream(), torch.cuda.Stream()
    fork, join = torch.cuda.Event(), torch.cuda.Event()

    def block(S):
        for si, site in enumerate(wl.sites):
            cur, nxt = S["s"][si % 2], S["s"][1 - si % 2]
            parts, max_rows = len(site.parts), site.max_rows()
            fork.record(main)
            side.wait_event(fork)
            ref.launch_shrink(S["x"][si].data_ptr(), site.cols, site.cols, S["tiles"].data_ptr(), S["tabs"][si].data_ptr(),
                              cur.data_ptr(), lds, max_tiles, wl.tokens, parts, side.cuda_stream)
            join.record(side)
            main.wait_event(join)
            ref.launch_expand(cur.data_ptr(), lds, nxt.data_ptr(), S["tiles"].data_ptr(), S["tabs"][si].data_ptr(),
                              S["y"][si].data_ptr(), S["y"][si].shape[1], False, max_tiles, wl.tokens, max_rows, parts,
                              main.cuda_stream)

    graphs = []
    with torch.cuda.stream(main):
        for S in sets:
            block(S)
        torch.cuda.synchronize()
        for S in sets:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=main):
                block(S)
            graphs.append(g)
        torch.cuda.synchronize()
        for i in range(max(3, args.warmup)):
            graphs[i % copies].replay()
        torch.cuda.synchronize()
        steps = max(args.steps, 50)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        for i in range(steps):
            graphs[i % copies].replay()
        e1.record(main)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    work = wl.work()
    peak, kind, _ = peaks()
    return {"value": wl.tokens * steps / (ms * 1e-3), "unit": UNIT, "us_per_step": 1e3 * ms / steps, "steps": steps,
            "achieved_gbs": work["bytes"] / (ms / steps * 1e-3) / 1e9, "frac_of_peak": work["bytes"] / (ms / steps * 1e-3) / 1e9 / peak,
            "what": ("pocket-engine's lora_shrink/lora_expand compiled for sm_100a" if image is None else
                     "plora_compat.fatbin (same kernel names and grids)") + ", CUDA-graph replay, same rotation"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="default: 200 (decode), 10 (prefill)")
    ap.add_argument("--warmup", type=int, default=0, help="default: 20 (decode), 3 (prefill)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "plumbing", "fp8", "tp", "fused-bf16"])
    ap.add_argument("--tokens", type=int, default=0, help="fp8 workload only: run the layer at this prefill-sized M")
    ap.add_argument("--seqs", type=int, default=8, help="prefill workload only: sequences of 2048 tokens (8 = the "
                                                        "benchmark configuration; fewer for profiler captures)")
    ap.add_argument("--copies", type=int, default=0, help="override the number of rotating pool copies")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="tp workload only: how the row-parallel shrink partials are summed over the ranks: the "
                         "library's one-kernel exchange over peer memory, or an NCCL all-reduce")
    ap.add_argument("--path", default="apply", choices=["apply", "apply-pair", "pair"],
                    help="apply: plora_apply after the layer's own matrix multiply, one cluster kernel per layer; "
                         "apply-pair: plora_apply as the shrink / expand pair; pair: the engine's shrink-before / "
                         "expand-after bracket (plora_shrink, plora_expand)")
    ap.add_argument("--early-x", action="store_true",
                    help="plora_set_early_x(1): the caller vouches for x, which is then read ahead of the dependency wait")
    ap.add_argument("--inner-repeats", type=int, default=50,
                    help="decode workload: passes of the block per timed step (the result is reported per pass)")
    ap.add_argument("--two-part", action="store_true", help="fp8 workload: the engine's two-part gate + up layer (4096 -> 24576)")
    ap.add_argument("--e2e-ahead", type=int, default=4, help="steps the host may run ahead of the device in the end-to-end measurement")
    ap.add_argument("--e2e-depth", type=int, default=2, help="steps in flight in the end-to-end measurement (1 to 3)")
    ap.add_argument("--no-e2e-graph", action="store_true", help="end-to-end steps as individual calls instead of one CUDA graph per copy")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel layer set that the default run appends")
    ap.add_argument("--streams", type=int, default=1, choices=[1, 2],
                    help="1: one stream, kernels chained by programmatic dependent launch; 2: the engine's "
                         "side-stream shrink with fork/join events")
    args = ap.parse_args()
    global PREFILL_SEQS
    PREFILL_SEQS = args.seqs
    args.steps = args.steps or (10 if args.workload in ("prefill", "fused-bf16") else 200)
    args.warmup = max(args.warmup or (3 if args.workload in ("prefill", "fused-bf16") else 20), 3)
    if args.workload == "fp8" and args.tokens:
        args.steps, args.warmup = min(args.steps, 10), 3
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        out = run_reference(args, rank, world)
        if out is not None:
            print(json.dumps(out))
        return
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU fallback")
    with_tp = args.workload == "decode" and not args.no_tp  # the default run appends the tensor-parallel layer set
    if world > 1 or args.workload == "tp" or with_tp:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        torch.distributed.init_process_group("nccl", rank=rank, world_size=world,
                                             device_id=torch.device(f"cuda:{local_rank}"))
    if args.workload in ("fp8", "tp", "fused-bf16"):
        out = {"fp8": run_fp8, "tp": run_tp, "fused-bf16": run_fused_bf16}[args.workload](args, rank, world, local_rank)
        if rank == 0:
            print(json.dumps(out))
        if torch.distributed.is_initialized():
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()
        return
    out = run_ours(args, rank, world, local_rank)
    if with_tp:
        # configs[4] of the benchmark definition: NCCL all-reduce (the primary form) and, on more than one GPU, the
        # library's own exchange kernel; strong scaling, so its numbers sit beside the headline, not in `value`
        try:
            info, tp_out = tp_measure(args, rank, world, local_rank, ["nccl", "fused"] if world > 1 else ["nccl"],
                                      max(10, min(args.steps, 50)), 5)
            if rank == 0:
                out["tp"] = dict(info, **tp_out)
        except Exception as e:  # noqa: BLE001  (the headline line must still be printed)
            if rank == 0:
                out["tp"] = {"failed": f"{type(e).__name__}: {e}"[:300]}
    # The CPU baseline runs on rank 0 while the other ranks sleep on a store key (a collective barrier would have
    # them spin on the cores the baseline is timed on).
    store = None
    if torch.distributed.is_initialized():
        torch.cuda.synchronize()
        try:
            store = torch.distributed.distributed_c10d._get_default_store()
        except Exception:  # noqa: BLE001
            store = None
    if rank == 0:
        v, cores, sample, _, _ = cpu_port(args.workload, args.cpu_seconds)
        out["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        if store is not None:
            store.set("plora_cpu_baseline_done", "1")
        print(json.dumps(out))
    elif store is not None:
        import datetime
        store.wait(["plora_cpu_baseline_done"], datetime.timedelta(seconds=900))
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
