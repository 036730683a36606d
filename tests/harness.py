"""Shared test helpers: build the same registry in the product library and in the CPU oracle from one
synthetic workload, run the adapter path through the C ABI on the GPU, and compare.

Tolerances (stated by the benchmark definition): against the fp64 oracle, max |d| <= 1e-2 * RMS(y) and
mean |d| <= 1e-3 * RMS(y), measured in f32-out mode. In bf16-out mode the output is compared with the
oracle rounded to bf16 at the same point: at most one bf16 ulp apart, and all but a small fraction equal.
"""
import numpy as np

import __graft_entry__ as entry

MAX_TOL = 1e-2
MEAN_TOL = 1e-3


def oracle_registry(wl, max_slots=None):
    orc = entry.load_oracle()
    max_slots = max_slots or wl.n_adapters
    table = orc.OracleTable(wl.sites, max_slots)
    adapters = []
    for i in range(wl.n_adapters):
        a = orc.OracleAdapter(wl.sites, wl.factors(i), wl.max_rank)
        table.upload(i + 1, a)
        adapters.append(a)
    return table, adapters


def product_registry(pe, wl, device=0, max_slots=None, max_tokens=None, max_seqs=None):
    max_slots = max_slots or wl.n_adapters
    loras = pe.Loras(wl.sites, max_slots, wl.max_rank, max_tokens or wl.tokens, max_seqs or wl.n_seqs, device=device)
    prep = loras.prep()
    for i in range(wl.n_adapters):
        ad = prep.prepare(f"adapter-{i}", wl.factors(i))
        aid = loras.insert(ad)
        assert aid == i + 1
        if device >= 0:
            loras.upload(i + 1, aid)
    return loras


def tiles_of(pe, wl, cap=None):
    cap = cap or (wl.tokens // 16 + wl.n_seqs)
    return pe.fill_tiles(wl.row_n, wl.row_slot, cap)


def to_dev_bf16(bits, device):
    import torch
    return torch.from_numpy(bits.view(np.int16).copy()).to(f"cuda:{device}").view(torch.bfloat16)


def run_gpu(pe, loras, wl, f32_out, meta="host", device=0, y_base=None, xs=None, fused=False, early_x=False):
    """All sites of the workload once; returns [y numpy per site] (f32 values; bf16 outputs widened)."""
    import torch
    torch.cuda.set_device(device)
    dev = f"cuda:{device}"
    stream = torch.cuda.current_stream().cuda_stream
    if meta == "host":
        loras.meta_upload(tiles_of(pe, wl, loras.max_lora_tiles()), stream)
    else:
        cu = torch.from_numpy(wl.cu()).to(dev)
        ss = torch.from_numpy(wl.row_slot.copy()).to(dev)
        loras.meta_build(cu.data_ptr(), ss.data_ptr(), wl.n_seqs, stream)
    step = loras.lora_step(loras.max_lora_tiles(), stream)
    if fused:  # plora_apply: "early" = the shrink / expand pair, "cluster" = one cluster kernel per layer
        loras.set_apply_mode(1 if fused == "cluster" else 0)
        loras.set_early_x(early_x)  # the caller vouches for x (true here: x is a plain device copy made long before)
    outs = []
    for si in range(len(wl.sites)):
        xb = xs[si] if xs is not None else wl.x_bits(si)
        x = to_dev_bf16(xb, device)
        yb = y_base[si] if y_base is not None else wl.y_base(si)
        if f32_out:
            y = torch.from_numpy(yb.copy()).to(dev)
        else:
            y = to_dev_bf16(pe.bf16_bits(yb), device)
        lin = pe.Linear(loras, si)
        lin.forward(x.data_ptr(), wl.tokens, y.data_ptr(), y.shape[1], f32_out, lora=step, main=stream, fused=bool(fused))
        outs.append(y.float().cpu().numpy())
    torch.cuda.synchronize()
    loras.device_status()
    return outs


def oracle_f64(wl, table, tiles, y_base=None, xs=None, f32_out=True, pe=None):
    orc = entry.load_oracle()
    outs = []
    for si, site in enumerate(wl.sites):
        xb = xs[si] if xs is not None else wl.x_bits(si)
        yb = y_base[si] if y_base is not None else wl.y_base(si)
        if not f32_out:
            yb = pe.bf16_to_f32(pe.bf16_bits(yb)).reshape(yb.shape)
        y64 = yb.astype(np.float64)
        orc.site_f64(xb, site.cols, tiles, table.tables[si], y64)
        outs.append(y64)
    return outs


def oracle_rounded(wl, table, tiles, f32_out, pe, mode="f32s", y_base=None, xs=None):
    """The oracle with the kernels' rounding points (mode f32s) or the reference kernels' (mode emul)."""
    orc = entry.load_oracle()
    fn = orc.site_f32s if mode == "f32s" else orc.site_emul
    outs = []
    for si, site in enumerate(wl.sites):
        xb = xs[si] if xs is not None else wl.x_bits(si)
        yb = y_base[si] if y_base is not None else wl.y_base(si)
        if f32_out:
            y = yb.astype(np.float32).copy()
            fn(xb, site.cols, tiles, table.tables[si], y, True)
            outs.append(y)
        else:
            y = pe.bf16_bits(yb).reshape(yb.shape).copy()
            fn(xb, site.cols, tiles, table.tables[si], y, False)
            outs.append(pe.bf16_to_f32(y).reshape(yb.shape))
    return outs


def tolerance(y, y64):
    """(max |d| / RMS, mean |d| / RMS) over the whole output."""
    d = np.abs(y.astype(np.float64) - y64)
    rms = float(np.sqrt(np.mean(y64 ** 2)))
    return float(d.max()) / rms, float(d.mean()) / rms


def bf16_ulp_diff(a, b, pe, floor=2.0 ** -20):
    """Distance in bf16 steps between two arrays of bf16-representable f32 values. Values whose absolute
    difference is under `floor` count as equal: next to zero a bf16 step is far smaller than the f32
    rounding of the sums that feed it."""
    def key(v):
        u = pe.bf16_bits(v).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    d = np.abs(key(a) - key(b))
    d[np.abs(a.astype(np.float64) - b.astype(np.float64)) <= floor] = 0
    return d


def run_and_check(pe, wl, device=0, f32_out=True, meta="host", run_min=None, fused=False, early_x=False):
    table, _ = oracle_registry(wl)
    loras = product_registry(pe, wl, device)
    if run_min is not None:
        loras.set_run_min(run_min)  # runs at least this long take the tensor-core tile kernels
    tiles = tiles_of(pe, wl)
    ys = run_gpu(pe, loras, wl, f32_out, meta=meta, device=device, fused=fused, early_x=early_x)
    res = {}
    if f32_out:
        y64 = oracle_f64(wl, table, tiles)
        for si, (y, r) in enumerate(zip(ys, y64)):
            mx, mn = tolerance(y, r)
            assert mx <= MAX_TOL and mn <= MEAN_TOL, (wl.name, si, mx, mn)
            res[si] = (mx, mn)
    else:
        yr = oracle_rounded(wl, table, tiles, False, pe)
        # The tile path feeds S to the tensor cores as a bf16 high part plus a bf16 low part (about 16 bits of
        # mantissa instead of f32's 24) and the tensor cores' f32 accumulation over thousands of inputs is not
        # correctly rounded, so its y may sit about 1e-5 (of RMS(y) ~ 1) away from the rounded oracle: still a
        # thousand times inside the stated tolerance, but enough to move a value that lies within 1e-5 of a
        # bf16 rounding boundary (about 2 * 1e-5 / 2^-8 = 0.5% of the elements) to the neighbouring bf16.
        tile = run_min is not None and run_min < (1 << 30)
        floor, max_frac = (3e-5, 1e-2) if tile else (2.0 ** -20, 2e-3)
        for si, (y, r) in enumerate(zip(ys, yr)):
            ulp = bf16_ulp_diff(y, r, pe, floor)
            frac = float((ulp > 0).mean())
            assert ulp.max() <= 1 and frac < max_frac, (wl.name, si, int(ulp.max()), frac)
            res[si] = (int(ulp.max()), frac)
    loras.close()
    return res


# ---------------------------------------------------------------- device inspection

def dev_read(ptr, nbytes):
    """Copies nbytes from a raw device address to a numpy uint8 array (synchronous)."""
    import torch
    from cuda.bindings import runtime as rt
    torch.cuda.synchronize()
    out = np.zeros(nbytes, np.uint8)
    err, = rt.cudaMemcpy(out.ctypes.data, ptr, nbytes, rt.cudaMemcpyKind.cudaMemcpyDeviceToHost)
    assert int(err) == 0, err
    return out


class SegView:
    """The grouping kernel's output, decoded (word offsets as in csrc/plora_internal.h SegLayout)."""

    def __init__(self, loras, step):
        ms, mt, cap = loras.max_slots, loras.max_tokens, loras.max_lora_tiles()
        act, seg_off = 8, 8 + ms
        perm = seg_off + ms + 1
        work = (perm + mt + 31) // 32 * 32
        mma = work + 32 * cap
        words = dev_read(step.segs, (mma + 3 * cap) * 4).view(np.int32)
        self.n_act, self.n_work, self.n_mma, self.n_gather, self.n_tiles, self.status = words[:6]
        self.act = words[act:act + self.n_act]
        self.seg_off = words[seg_off:seg_off + self.n_act + 1]
        self.perm = words[perm:perm + self.n_gather]
        items = words[work:work + 32 * self.n_work].reshape(-1, 32)
        self.work = items[:, :3]
        self.work_tokens = [list(it[4:4 + it[2]]) for it in items]
        self.mma = words[mma:mma + 3 * self.n_mma].reshape(-1, 3)


def read_tiles(loras):
    cap = loras.max_lora_tiles()
    w = dev_read(loras.tiles, (1 + 3 * cap) * 4).view(np.int32)
    return w[:1 + 3 * int(w[0])]


def run_reference_kernels(pe, loras, wl, f32_out, device=0, y_base=None, xs=None, image=None):
    """pocket-engine's own lora_shrink / lora_expand (oracle/_ref) over the product's descriptor tables and
    tile words, with the engine's grids and its two-buffer S choreography (src/kernels/lora.cuh:69-73)."""
    import importlib.util
    import os
    import torch
    spec = importlib.util.spec_from_file_location("plora_ref_kernels", os.path.join(entry.ROOT, "oracle", "ref_kernels.py"))
    rk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rk)
    if image is None and not rk.available():
        return None
    torch.cuda.set_device(device)
    dev = f"cuda:{device}"
    ref = rk.RefKernels(image)
    stream = torch.cuda.current_stream().cuda_stream
    loras.meta_upload(tiles_of(pe, wl, loras.max_lora_tiles()), stream)
    lds = loras.lds
    s = torch.zeros(2, wl.tokens, lds, dtype=torch.float32, device=dev)
    max_tiles = loras.max_lora_tiles()
    outs = []
    for si, site in enumerate(wl.sites):
        xb = xs[si] if xs is not None else wl.x_bits(si)
        x = to_dev_bf16(xb, device)
        yb = y_base[si] if y_base is not None else wl.y_base(si)
        y = torch.from_numpy(yb.copy()).to(dev) if f32_out else to_dev_bf16(pe.bf16_bits(yb), device)
        hook = loras.hook(si)
        cur, nxt = s[si % 2], s[1 - si % 2]
        ref.launch_shrink(x.data_ptr(), site.cols, site.cols, loras.tiles, hook.table, cur.data_ptr(), lds, max_tiles,
                          wl.tokens, hook.parts, stream)
        ref.launch_expand(cur.data_ptr(), lds, nxt.data_ptr(), loras.tiles, hook.table, y.data_ptr(), y.shape[1],
                          f32_out, max_tiles, wl.tokens, hook.max_rows, hook.parts, stream)
        outs.append(y.float().cpu().numpy())
    torch.cuda.synchronize()
    return outs
