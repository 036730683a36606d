"""Graph sets per batch bucket (src/engine.rs:437-471, 698-721): the same captured graphs serve steps of different
sizes and different adapter-to-slot assignments; only tile words, slabs and descriptor tables change."""
import numpy as np
import pytest

import harness

pytestmark = pytest.mark.gpu


def test_bucket_graphs_survive_slot_swaps_and_batch_changes(pe, oracle):
    import torch
    from pocket_engine_b200 import graphs, workloads
    hidden, inter, n_adapters, n_slots, max_seqs = 512, 1024, 6, 3, 24
    sites = workloads.block_sites(hidden, inter, 128)
    wl = workloads.Workload("graph-set", sites, [16] * n_adapters, 1.0, [1], [0], 41)
    loras = pe.Loras(sites, n_slots, 16, max_seqs, max_seqs, device=0)
    prep = loras.prep()
    ids = [loras.insert(prep.prepare(f"a{i}", wl.factors(i))) for i in range(n_adapters)]
    adapters = [oracle.OracleAdapter(sites, wl.factors(i), 16) for i in range(n_adapters)]
    table = oracle.OracleTable(sites, n_slots)
    slots = pe.LoraSlots(n_slots)
    stream = torch.cuda.Stream()
    xs = [torch.zeros(max_seqs, s.cols, dtype=torch.bfloat16, device="cuda") for s in sites]
    ys = [torch.zeros(max_seqs, s.width(), dtype=torch.float32, device="cuda") for s in sites]
    lins = [pe.Linear(loras, si) for si in range(len(sites))]

    def body(step, rows, s):
        for si, lin in enumerate(lins):
            lin.forward(xs[si].data_ptr(), rows, ys[si].data_ptr(), ys[si].shape[1], True, lora=step, main=s, fused=True)

    gs = graphs.LoraGraphSet(loras, body, max_seqs, stream)
    assert sorted(gs.graphs) == [1, 2, 4, 8, 12, 16, 24]
    rng = np.random.default_rng(5)
    used = []
    for step_no, (n, wanted) in enumerate([(5, [0, 1, 2]), (10, [3, 1]), (5, [4, 5, 3]), (1, [0]), (24, [2, 5, 0])]):
        # which adapter each sequence runs (-1 = base only), and the slots they get (least recently used leave)
        seq_adapter = rng.choice(wanted + [-1], n)
        seq_slot = np.zeros(n, np.int32)
        held = []
        for i, a in enumerate(seq_adapter):
            if a >= 0:
                seq_slot[i] = slots.place(ids[a])
                held.append(seq_slot[i])
        with torch.cuda.stream(stream):
            for slot, aid in slots.take_loads():
                loras.upload(slot, aid, stream.cuda_stream)
                table.upload(slot, adapters[ids.index(aid)])
            x_bits = [pe.bf16_bits(rng.standard_normal((n, s.cols), dtype=np.float32)) for s in sites]
            y_base = [rng.standard_normal((n, s.width()), dtype=np.float32) for s in sites]
            for si in range(len(sites)):
                xs[si][:n].copy_(harness.to_dev_bf16(x_bits[si], 0))
                ys[si][:n].copy_(torch.from_numpy(y_base[si]).cuda())
        tiles = pe.fill_tiles(np.ones(n, np.int32), seq_slot, loras.max_lora_tiles())
        used.append(gs.replay(n, tiles))
        stream.synchronize()
        loras.device_status()
        for si, site in enumerate(sites):
            want = y_base[si].astype(np.float64)
            oracle.site_f64(x_bits[si], site.cols, tiles, table.tables[si], want)
            mx, mn = harness.tolerance(ys[si][:n].cpu().numpy(), want)
            assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL, (step_no, si, mx, mn)
        for s in held:
            slots.release(int(s))
    assert used == [8, 12, 8, 1, 24]  # the bucket-8 graph ran twice, with different adapters in the slots
    loras.close()


def test_adapter_from_a_peft_directory_through_a_worker_thread_to_a_gpu_slot(pe, oracle, tmp_path):
    """The whole way an adapter takes in the engine: read and laid out on a worker thread (pinned memory),
    registered by the engine thread, uploaded into a slot, applied; against the oracle fed the same factors."""
    import torch
    import test_adapter_files as files
    from pocket_engine_b200 import workloads
    sites = files.block_sites(pe, layers=1)
    rng = np.random.default_rng(8)
    mods = files.random_modules(pe, sites, 8, rng)
    files.write_peft(pe, str(tmp_path / "ad"), mods, 8, {"lora_alpha": 16})
    loras = pe.Loras(sites, 2, 16, 32, 32, device=0)
    mgr = pe.AdapterManager(loras, None, max_cpu_loras=4)
    assert mgr.settle(mgr.load("ad", tmp_path / "ad", on_demand=True)) == (pe.OK, "")
    aid = loras.id("ad")
    loras.upload(2, aid)
    fac = [pe.Factors.scaled(layer, module, a, b, 2.0) for (layer, module), (a, b) in mods.items()]
    table = oracle.OracleTable(sites, 2)
    table.upload(2, oracle.OracleAdapter(sites, fac, 16))
    rows, slots = [1, 5, 3], [2, 0, 2]
    wl = workloads.Workload("from-disk", sites, [8], 1.0, rows, slots, 3)
    tiles = pe.fill_tiles(wl.row_n, wl.row_slot, loras.max_lora_tiles())
    ys = harness.run_gpu(pe, loras, wl, True, meta="host")
    for si, site in enumerate(sites):
        want = wl.y_base(si).astype(np.float64)
        oracle.site_f64(wl.x_bits(si), site.cols, tiles, table.tables[si], want)
        mx, mn = harness.tolerance(ys[si], want)
        assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL and mx > 0
    mgr.close()
    loras.close()
