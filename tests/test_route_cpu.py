"""Adapter-affine partitioning on CPU ranks (gloo, world size 2): the router sends every sequence to the GPU that
owns its adapter, each rank applies only its own adapters to its own sub-batch (here with the oracle: no GPU),
and the gathered rows equal the unpartitioned result bit for bit: there is no exchange on the data path."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _batch(seed=3, n_seq=23, n_adapters=7):
    rng = np.random.default_rng(seed)
    row_n = rng.choice([1, 1, 1, 2, 5, 17, 33], n_seq).astype(np.int32)
    row_adapter = rng.integers(-1, n_adapters, n_seq)
    return row_n, row_adapter


def test_router_places_every_sequence_once_and_balances_base_traffic(pe):
    from pocket_engine_b200 import route
    row_n, row_adapter = _batch()
    for world in (1, 2, 3, 8):
        for load in (None, np.array([100, 1, 1, 1, 50, 1, 1.0])):
            owner = route.assign_adapters(7, world, load)
            parts = route.split_batch(row_n, row_adapter, owner, world)
            allseq = np.sort(np.concatenate(parts))
            assert np.array_equal(allseq, np.arange(len(row_n)))  # each exactly once
            for g, p in enumerate(parts):
                assert np.all(np.diff(p) > 0)  # step order kept
                assert all(row_adapter[i] < 0 or owner[row_adapter[i]] == g for i in p)
    # load-aware placement spreads a skewed popularity: the two heavy adapters end on different GPUs
    owner = route.assign_adapters(7, 2, np.array([100, 1, 1, 1, 50, 1, 1.0]))
    assert owner[0] != owner[4]
    # base-only sequences even out the token counts
    row_n = np.array([64, 1, 1, 30, 30, 4], np.int32)
    row_adapter = np.array([0, -1, -1, -1, -1, -1])
    parts = route.split_batch(row_n, row_adapter, route.assign_adapters(1, 2), 2)
    assert abs(int(row_n[parts[0]].sum()) - int(row_n[parts[1]].sum())) <= 1 and 0 in parts[0]


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    import __graft_entry__ as entry
    pe = entry.load_package()
    orc = entry.load_oracle()
    from pocket_engine_b200 import route, workloads
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n_adapters = 7
        row_n, row_adapter = _batch()
        sites = workloads.block_sites(64, 128, 32)
        full = workloads.Workload("full", sites, [8, 16, 8, 16, 8, 8, 16], 1.5, row_n, row_adapter + 1, 5, max_rank=16)
        owner = route.assign_adapters(n_adapters, world)
        mine, slot_of = route.local_slots(row_adapter, owner, rank)
        seqs = route.split_batch(row_n, row_adapter, owner, world)[rank]
        # the rank's registry holds only its adapters, in its own slots
        lay = pe.Loras(sites, max(1, len(mine)), 16, int(row_n.sum()), len(row_n), device=-1)
        table = orc.OracleTable(sites, max(1, len(mine)))
        for a in mine:
            ad = lay.prep().prepare(f"a{a}", full.factors(a))
            assert lay.insert(ad) == slot_of(a)
            table.upload(slot_of(a), orc.OracleAdapter(sites, full.factors(a), 16))
        # its sub-batch: the rows of its sequences, with local slot numbers
        cu = full.cu()
        rows = np.concatenate([np.arange(cu[i], cu[i + 1]) for i in seqs]) if len(seqs) else np.zeros(0, np.int64)
        sub_n = row_n[seqs]
        sub_slot = np.array([slot_of(row_adapter[i]) for i in seqs], np.int32)
        tiles = pe.fill_tiles(sub_n, sub_slot, len(rows) // 16 + len(seqs) + 1)
        assert np.array_equal(tiles, orc.fill_tiles(sub_n, sub_slot, len(rows) // 16 + len(seqs) + 1))
        outs = []
        for si, site in enumerate(sites):
            y = full.y_base(si)[rows].astype(np.float64)
            if len(rows):
                orc.site_f64(np.ascontiguousarray(full.x_bits(si)[rows]), site.cols, tiles, table.tables[si], y)
            outs.append((rows, y))
        gathered = [None] * world
        dist.all_gather_object(gathered, outs)  # results only: nothing crossed ranks during the computation
        if rank == 0:
            import harness
            ftable, _ = harness.oracle_registry(full)
            ftiles = orc.fill_tiles(full.row_n, full.row_slot, full.tokens // 16 + full.n_seqs)
            ok = True
            for si, site in enumerate(sites):
                want = full.y_base(si).astype(np.float64)
                orc.site_f64(full.x_bits(si), site.cols, ftiles, ftable.tables[si], want)
                got = np.zeros_like(want)
                seen = np.zeros(full.tokens, bool)
                for part in gathered:
                    r, y = part[si]
                    got[r] = y
                    seen[r] = True
                ok = ok and bool(seen.all()) and np.array_equal(got, want)
            out.put(ok)
        lay.close()
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_adapter_affine_partitions_equal_the_whole_batch_gloo_world_2():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29655, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert out.get(timeout=10) is True
