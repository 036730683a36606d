"""Tensor-parallel sharding on CPU ranks (gloo, world size 2): the shard definitions, the rank-local slabs,
and the exchange step. Each rank does its share of the arithmetic in numpy fp64 (no GPU here), all-reduces
the shrink partials of the row-parallel layers with torch.distributed, expands its own output slice, and
rank 0 checks the assembled result against the unsharded oracle."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    import harness
    pe = entry.load_package()
    orc = entry.load_oracle()
    from pocket_engine_b200 import tp, workloads
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wl = workloads.config5(adapters=3, rank=8, hidden=64, inter=128, q_width=96, decode=5, chunks=(18,))
        sh = tp.ShardedWorkload(wl, world, rank)
        # the rank's registry lays out exactly the sliced factors (layout-only handle: no GPU here)
        lay = pe.Loras(sh.sites, sh.n_adapters, sh.max_rank, sh.tokens, sh.n_seqs, device=-1)
        ads = []
        for i in range(sh.n_adapters):
            fac = sh.factors(i)
            ad = lay.prep().prepare(f"a{i}", fac)
            want = orc.OracleAdapter(sh.sites, fac, sh.max_rank)
            assert np.array_equal(ad.bytes(), want.data[:want.len])
            ads.append(want)
        tslot = sh.token_slot()
        ok = True
        for si, site in enumerate(sh.sites):
            mode = sh.modes[si]
            x = pe.bf16_to_f32(sh.x_bits(si)).reshape(sh.tokens, site.cols).astype(np.float64)
            y = sh.y_base(si).astype(np.float64)
            # shrink on the rank's slab: S[t, :] = x_local[t] . A_local^T
            S = np.zeros((sh.tokens, 4 * 16))
            for t in range(sh.tokens):
                if tslot[t] == 0:
                    continue
                a = ads[tslot[t] - 1]
                d = a.desc(si, 0)
                A = pe.bf16_to_f32(a.data[d.a:d.a + d.rank * site.cols * 2].view(np.uint16)).reshape(d.rank, site.cols)
                S[t, :d.rank] = A.astype(np.float64) @ x[t]
            if mode == tp.ROW:  # the exchange: partial sums over the input-column shards
                St = torch.from_numpy(S)
                dist.all_reduce(St, op=dist.ReduceOp.SUM)
                S = St.numpy()
            for t in range(sh.tokens):
                if tslot[t] == 0:
                    continue
                a = ads[tslot[t] - 1]
                d = a.desc(si, 0)
                for p in range(len(site.parts)):
                    r, rows = d.r[p], d.rows[p]
                    B = pe.bf16_to_f32(a.data[d.b[p]:d.b[p] + rows * r * 2].view(np.uint16)).reshape(rows, r)
                    y[t, d.off[p]:d.off[p] + rows] += B.astype(np.float64) @ S[t, d.r_off[p]:d.r_off[p] + r]
            # assemble on rank 0 and compare with the unsharded oracle
            gathered = [None] * world
            dist.all_gather_object(gathered, y)
            if rank == 0:
                got = sh.assemble(si, gathered)
                table, _ = harness.oracle_registry(wl)
                tiles = orc.fill_tiles(wl.row_n, wl.row_slot, 64)
                want = wl.y_base(si).astype(np.float64)
                orc.site_f64(wl.x_bits(si), wl.sites[si].cols, tiles, table.tables[si], want)
                err = float(np.abs(got - want).max())
                ok = ok and err < 1e-6
        if rank == 0:
            out.put(ok)
        lay.close()
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_sharding_two_ranks(pe, oracle):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


def test_shard_definitions(pe):
    from pocket_engine_b200 import tp
    site = pe.Site.fused(0, 5120, [("mlp.gate_proj", 17408), ("mlp.up_proj", 17408)])
    col = tp.shard_site(site, tp.COLUMN, 8, 3)
    assert col.cols == 5120 and [(p.rows, p.off) for p in col.parts] == [(2176, 0), (2176, 2176)]
    down = pe.Site.fused(0, 17408, [("mlp.down_proj", 5120)])
    row = tp.shard_site(down, tp.ROW, 8, 3)
    assert row.cols == 2176 and [(p.rows, p.off) for p in row.parts] == [(640, 1920)]
    with pytest.raises(ValueError):
        tp.shard_site(pe.Site.fused(0, 100, [("m", 64)]), tp.ROW, 8, 0)
    f = pe.Factors(0, "mlp.down_proj", np.arange(4 * 17408, dtype=np.float32).reshape(4, 17408),
                   np.arange(5120 * 4, dtype=np.float32).reshape(5120, 4))
    s = tp.shard_factors(f, down, tp.ROW, 8, 3)
    assert s.a.shape == (4, 2176) and s.a[0, 0] == 3 * 2176 and s.b.shape == (640, 4) and s.b[0, 0] == 1920 * 4
