"""Tensor-parallel mode on GPUs: one rank (exercises the K-split reduction, the collective call and the
expand from the reduced plane), two ranks over NCCL where the box has them, and the library's own exchange
kernel: all ranks in one cooperative launch on one GPU, one process per GPU where there are two."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def wls():
    from pocket_engine_b200 import workloads
    return workloads


def _run(nproc, port, exchange="nccl"):
    env = dict(os.environ, NCCL_DEBUG="WARN", PLORA_TP_EXCHANGE=exchange)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    return json.loads(line)


def test_row_and_column_parallel_layers_one_rank():
    res = _run(1, 29611)
    assert res["tp_check"] == "ok", res


def test_tensor_parallel_two_ranks():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = _run(2, 29612)
    assert res["tp_check"] == "ok" and res["world"] == 2, res


def test_two_ranks_own_exchange_kernel():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = _run(2, 29613, exchange="fused")
    assert res["tp_check"] == "ok" and res["world"] == 2 and res["exchange"] == "fused", res


def _emulated_ranks(pe, wls, world, rounds=3):
    """Every rank's shard on ONE GPU; the exchange of all ranks runs as a single cooperative launch."""
    import torch
    import __graft_entry__ as entry
    import harness
    from pocket_engine_b200 import tp
    orc = entry.load_oracle()
    wl = wls.config5(adapters=6, rank=16, hidden=512, inter=1024, q_width=768, decode=40, chunks=(128, 70))
    shards = [tp.ShardedWorkload(wl, world, r) for r in range(world)]
    ranks = [harness.product_registry(pe, sh, device=0) for sh in shards]
    stream = torch.cuda.current_stream().cuda_stream
    for r, L in enumerate(ranks):
        L.exchange_create(world, r, 2000)
    for r, L in enumerate(ranks):
        for p in range(world):
            if p != r:
                L.exchange_import_local(p, ranks[p])
    steps = []
    for sh, L in zip(shards, ranks):
        L.meta_upload(pe.fill_tiles(sh.row_n, sh.row_slot, L.max_lora_tiles()), stream)
        steps.append(L.lora_step(L.max_lora_tiles(), stream))
    table, _ = harness.oracle_registry(wl)
    tiles = orc.fill_tiles(wl.row_n, wl.row_slot, wl.tokens // 16 + wl.n_seqs)
    for rnd in range(rounds):  # several calls: both staging buffers and the call counter come into play
        for si in range(len(wl.sites)):
            if wl.modes[si] != tp.ROW:
                continue
            hooks = [L.hook(si) for L in ranks]
            xs = [harness.to_dev_bf16(sh.x_bits(si), 0) for sh in shards]
            ys = [torch.from_numpy(sh.y_base(si).copy()).cuda() for sh in shards]
            for L, h, st, x in zip(ranks, hooks, steps, xs):
                L.shrink(h, st, x.data_ptr(), wl.tokens, stream)
            pe.s_exchange_all_ranks(ranks, hooks, steps, wl.tokens, stream)
            planes = [harness.dev_read(L.s, wl.tokens * L.lds * 4) for L in ranks]
            for p in planes[1:]:
                assert np.array_equal(planes[0], p)  # every rank ends with the same bits
            for L, h, st, y in zip(ranks, hooks, steps, ys):
                L.expand_reduced(h, st, wl.tokens, y.data_ptr(), y.shape[1], True, stream)
            torch.cuda.synchronize()
            got = shards[0].assemble(si, [y.cpu().numpy() for y in ys])
            want = wl.y_base(si).astype(np.float64)
            orc.site_f64(wl.x_bits(si), wl.sites[si].cols, tiles, table.tables[si], want)
            mx, mn = harness.tolerance(got, want)
            assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL, (world, rnd, si, mx, mn)
    for L in ranks:
        L.device_status()
        L.close()


@pytest.mark.parametrize("world", [2, 4])
def test_exchange_kernel_all_ranks_in_one_launch(pe, wls, world):
    _emulated_ranks(pe, wls, world)


def test_exchange_wait_runs_out_and_reports(pe, wls):
    """A rank whose peer never arrives: the bounded wait gives up, the status word says so, and the device
    keeps working."""
    import torch
    import harness
    from pocket_engine_b200 import tp
    wl = wls.config5(adapters=3, rank=16, hidden=256, inter=512, q_width=256, decode=8, chunks=(64,))
    shards = [tp.ShardedWorkload(wl, 2, r) for r in range(2)]
    ranks = [harness.product_registry(pe, sh, device=0) for sh in shards]
    for r, L in enumerate(ranks):
        L.exchange_create(2, r, 30)  # 30 ms
    ranks[0].exchange_import_local(1, ranks[1])
    ranks[1].exchange_import_local(0, ranks[0])
    stream = torch.cuda.current_stream().cuda_stream
    L, sh = ranks[0], shards[0]
    L.meta_upload(pe.fill_tiles(sh.row_n, sh.row_slot, L.max_lora_tiles()), stream)
    step = L.lora_step(L.max_lora_tiles(), stream)
    si = wl.modes.index(tp.ROW)
    x = harness.to_dev_bf16(sh.x_bits(si), 0)
    L.shrink(L.hook(si), step, x.data_ptr(), wl.tokens, stream)
    L.s_exchange(L.hook(si), step, wl.tokens, stream)  # rank 1 never calls
    with pytest.raises(pe.PloraError) as err:
        L.device_status()
    assert err.value.code == pe.ERR_TIMEOUT
    L.device_status()  # the word was cleared and the context still answers
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0
    # rank 0 counted the failed call, rank 1 did not: without a reset every later exchange would time out as well
    for R in ranks:
        R.exchange_reset(stream)
    torch.cuda.synchronize()
    steps, hooks, xs = [], [], []
    for R, shd in zip(ranks, shards):
        R.meta_upload(pe.fill_tiles(shd.row_n, shd.row_slot, R.max_lora_tiles()), stream)
        steps.append(R.lora_step(R.max_lora_tiles(), stream))
        hooks.append(R.hook(si))
        xs.append(harness.to_dev_bf16(shd.x_bits(si), 0))
        R.shrink(hooks[-1], steps[-1], xs[-1].data_ptr(), wl.tokens, stream)
    pe.s_exchange_all_ranks(ranks, hooks, steps, wl.tokens, stream)
    torch.cuda.synchronize()
    for R in ranks:
        R.device_status()
    # both ranks now hold the same, complete sums: plane 0 of S, bit for bit
    s0 = harness.dev_read(ranks[0].s, wl.tokens * ranks[0].lds * 4)
    s1 = harness.dev_read(ranks[1].s, wl.tokens * ranks[1].lds * 4)
    assert np.array_equal(s0, s1) and np.any(s0 != 0)
    for R in ranks:
        R.close()
