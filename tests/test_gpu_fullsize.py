"""The benchmark configurations at their full sizes against the CPU oracle.

The prefill configuration (8 x 2048 tokens) and the FP8 layer (256 tokens, 128 adapters over 4096 -> 12288) are
too large for the oracle to recompute whole in seconds, so the device result is checked on a seeded sample of
token rows (the first and last rows of every sequence among them), all columns: a token's result depends on its
own row of x, its slot's slabs and its own row of y only (the property the engine tests at full model scale,
tests/gpu.rs:1083-1132), so the oracle recomputes exactly those rows. The activations are drawn on the device
and the sampled rows copied back, so the oracle sees the very bits the kernels saw. The tensor-parallel
configuration's layers (512 tokens) are recomputed whole."""
import numpy as np
import pytest

import harness

pytestmark = pytest.mark.gpu


def _sample_rows(wl, per_seq, rng):
    """Token rows to check: first and last of every sequence, plus random ones; sorted."""
    cu = wl.cu()
    rows = []
    for i, n in enumerate(wl.row_n):
        lo, hi = int(cu[i]), int(cu[i + 1])
        pick = {lo, hi - 1, lo + min(15, n - 1), lo + min(16, n - 1), hi - 1 - min(16, n - 1)}
        if n > 4:
            pick.update(int(v) for v in rng.integers(lo, hi, min(per_seq, n)))
        rows += sorted(pick)
    return np.array(sorted(set(rows)), np.int64)


def _one_token_tiles(slots):
    """Tile words that give every sampled row its own one-token tile (base-only rows get none)."""
    live = [(i, int(s)) for i, s in enumerate(slots) if s != 0]
    words = [len(live)]
    for i, s in live:
        words += [i, 1, s]
    return np.array(words, np.int32)


@pytest.mark.parametrize("f32_out", [True, False], ids=["f32", "bf16"])
@pytest.mark.parametrize("path", ["bracket", "apply"])
def test_prefill_segments_at_full_size(pe, oracle, wls_mod, f32_out, path):
    """8 sequences of 2048 tokens, one rank-64 adapter each, over the 4096 / 12288 block: 64+ sampled rows per
    sequence through the tensor-core tile kernels."""
    import torch
    wl = wls_mod.config3()
    assert wl.tokens == 16384
    loras = harness.product_registry(pe, wl)
    loras.set_run_min(64)
    table, _ = harness.oracle_registry(wl)
    rng = np.random.default_rng(3)
    rows = _sample_rows(wl, 64, rng)
    tslot = wl.token_slot()
    sub_tiles = _one_token_tiles(tslot[rows])
    dev = "cuda"
    gen = torch.Generator(device=dev)
    gen.manual_seed(33)
    stream = torch.cuda.current_stream().cuda_stream
    cu = torch.from_numpy(wl.cu()).to(dev)
    ss = torch.from_numpy(wl.row_slot.copy()).to(dev)
    loras.meta_build(cu.data_ptr(), ss.data_ptr(), wl.n_seqs, stream)
    step = loras.lora_step(loras.max_lora_tiles(), stream)
    ridx = torch.from_numpy(rows).to(dev)
    for si, site in enumerate(wl.sites):
        x = torch.randn(wl.tokens, site.cols, generator=gen, device=dev).to(torch.bfloat16)
        y = torch.randn(wl.tokens, site.width(), generator=gen, device=dev)
        if not f32_out:
            y = y.to(torch.bfloat16)
        before = y[ridx].clone()
        lin = pe.Linear(loras, si)
        lin.forward(x.data_ptr(), wl.tokens, y.data_ptr(), y.shape[1], f32_out, lora=step, main=stream,
                    fused=path == "apply")
        torch.cuda.synchronize()
        loras.device_status()
        xb = x[ridx].view(torch.int16).cpu().numpy().view(np.uint16)
        got = y[ridx].float().cpu().numpy()
        if f32_out:
            want = before.cpu().numpy().astype(np.float64)
            oracle.site_f64(xb, site.cols, sub_tiles, table.tables[si], want)
            mx, mn = harness.tolerance(got, want)
            assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL, (si, mx, mn)
            assert mx <= 2e-4, (si, mx)  # bf16 high + low terms on the tensor cores: about 1e-5 of RMS
        else:
            want = before.view(torch.int16).cpu().numpy().view(np.uint16).copy()
            oracle.site_f32s(xb, site.cols, sub_tiles, table.tables[si], want, False)
            ulp = harness.bf16_ulp_diff(got, pe.bf16_to_f32(want).reshape(got.shape), pe, floor=3e-5)
            assert ulp.max() <= 1 and (ulp > 0).mean() < 1e-2, (si, int(ulp.max()), float((ulp > 0).mean()))
        del x, y
    loras.close()


@pytest.mark.parametrize("two_part", [False, True], ids=["one-part", "gate-up"])
def test_heterogeneous_ranks_over_the_fp8_layer_at_full_size(pe, oracle, wls_mod, two_part):
    """256 decode tokens, 128 adapters of ranks 8..128 with Zipf popularity, FP8 base 4096 -> 12288 (and the
    engine's two-part gate + up layer, 4096 -> 24576): 64 sampled tokens against the fp64 oracle over the
    quantised operands."""
    import torch
    wl = wls_mod.config4(two_part=two_part)
    assert wl.tokens == 256 and wl.n_adapters == 128
    site = wl.sites[0]
    K, N, T = site.cols, site.width(), wl.tokens
    rng = np.random.default_rng([4, 77])
    w = np.clip(rng.standard_normal((N, K), dtype=np.float32), -448, 448)
    wq = torch.from_numpy(w).to(torch.float8_e4m3fn).view(torch.uint8).numpy().copy()
    sn = (rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32)
    xb = wl.x_bits(0)
    xq, st = oracle.fp8_quant_rows(xb)
    loras = harness.product_registry(pe, wl)
    table, _ = harness.oracle_registry(wl)
    tiles = harness.tiles_of(pe, wl)
    rows = np.sort(np.random.default_rng(5).choice(T, 64, replace=False))
    tslot = wl.token_slot()
    sub_tiles = _one_token_tiles(tslot[rows])
    want = oracle.fp8_base_f64(xq[rows].copy(), st[rows].copy(), wq, sn)
    base_abs = np.abs(want)
    oracle.site_f64(xb[rows].copy(), K, sub_tiles, table.tables[0], want)
    rms = float(np.sqrt(np.mean(want ** 2)))
    stream = torch.cuda.current_stream().cuda_stream
    x = harness.to_dev_bf16(xb, 0)
    xq_d = torch.zeros(T, K, dtype=torch.uint8, device="cuda")
    st_d = torch.zeros(T, dtype=torch.float32, device="cuda")
    wq_d, sn_d = torch.from_numpy(wq).cuda(), torch.from_numpy(sn).cuda()
    for f32_out in (True, False):
        y = torch.full((T, N), 7.0, dtype=torch.float32 if f32_out else torch.bfloat16, device="cuda")
        loras.meta_upload(tiles, stream)
        step = loras.lora_step(loras.max_lora_tiles(), stream, decode=True)
        hook = loras.hook(0)
        loras.fp8_quant_rows(x.data_ptr(), T, K, xq_d.data_ptr(), st_d.data_ptr(), stream)
        loras.shrink(hook, step, x.data_ptr(), T, stream)
        loras.linear_fp8_fused(hook, step, xq_d.data_ptr(), st_d.data_ptr(), wq_d.data_ptr(), sn_d.data_ptr(), T,
                               y.data_ptr(), N, f32_out, stream)
        torch.cuda.synchronize()
        loras.device_status()
        got = y.float().cpu().numpy()[rows].astype(np.float64)
        d = np.abs(got - want)
        if f32_out:
            assert d.max() <= harness.MAX_TOL * rms and d.mean() <= harness.MEAN_TOL * rms, (d.max() / rms, d.mean() / rms)
            assert d.max() <= 2e-4 * rms
        else:
            # the base is rounded to bf16 by the layer kernel, the sum with the adapter term once more
            assert np.all(d <= (np.abs(want) + base_abs) * 2.0 ** -8 + 2e-4 * rms), float((d / rms).max())
    assert np.array_equal(xq_d.cpu().numpy(), xq)
    loras.close()


@pytest.mark.parametrize("path", [False, "early", "cluster"], ids=["bracket", "apply-pair", "apply-cluster"])
def test_tensor_parallel_layers_at_full_size_unsharded(pe, wls_mod, path):
    """The 27B-shaped layers (5120 / 17408, 512 tokens = 256 decode tokens + 2 prompt chunks of 128, 32 rank-32
    adapters) on one GPU, every token against the oracle. (Sharded over ranks: tests/test_gpu_tp.py.)"""
    wl = wls_mod.config5()
    assert wl.tokens == 512
    for f32_out in (True, False):
        harness.run_and_check(pe, wl, f32_out=f32_out, meta="device", run_min=64, fused=path)


@pytest.fixture(scope="module")
def wls_mod():
    from pocket_engine_b200 import workloads
    return workloads
