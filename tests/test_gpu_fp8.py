"""The FP8 base layer with the adapter expand fused into its epilogue, against the CPU oracle over the same
quantised operands (so quantisation error is not charged to the kernel)."""
import numpy as np
import pytest

import harness

pytestmark = pytest.mark.gpu


def _weights(N, K, seed):
    """W ~ N(0,1) clipped to +-448 as e4m3 bits, per-output-channel scales ~ U(0.5, 2) / 448."""
    import torch
    rng = np.random.default_rng([seed, 77])
    w = np.clip(rng.standard_normal((N, K), dtype=np.float32), -448, 448)
    wq = torch.from_numpy(w).to(torch.float8_e4m3fn).view(torch.uint8).numpy().copy()
    sn = (rng.uniform(0.5, 2.0, N) / 448.0).astype(np.float32)
    return wq, sn


def test_row_quantisation_is_bit_exact(pe, oracle):
    import torch
    rng = np.random.default_rng(3)
    x = rng.standard_normal((37, 1096), dtype=np.float32) * rng.uniform(0.01, 30, (37, 1)).astype(np.float32)
    x[5] = 0
    xb = pe.bf16_bits(x).reshape(x.shape)
    sites = [pe.Site.fused(0, 1096, [("a", 64)])]
    loras = pe.Loras(sites, 2, 16, 64, device=0)
    xd = harness.to_dev_bf16(xb, 0)
    xq = torch.zeros(37, 1096, dtype=torch.uint8, device="cuda")
    st = torch.zeros(37, dtype=torch.float32, device="cuda")
    loras.fp8_quant_rows(xd.data_ptr(), 37, 1096, xq.data_ptr(), st.data_ptr())
    torch.cuda.synchronize()
    want_q, want_s = oracle.fp8_quant_rows(xb)
    assert np.array_equal(st.cpu().numpy(), want_s)
    assert np.array_equal(xq.cpu().numpy(), want_q)
    loras.close()


CASES = [
    # name, rows per sequence, slot per sequence, ranks, K, parts
    ("decode-hetero", [1] * 96, None, [8, 16, 32, 64, 128] * 4, 1024, [("gate", 320)]),
    ("two-parts-ragged", [1] * 70 + [40, 3], None, [16, 128, 32], 512, [("gate", 192), ("up", 130)]),
    ("prompt-tiles", [128, 200], [1, 2], [64, 64], 640, [("gate", 256)]),
    ("all-base", [5, 9], [0, 0], [16], 256, [("gate", 64)]),
]

# shapes the one-kernel prefill form takes (parts starting at multiples of 256 columns, aligned pitches): runs of
# all lengths against the 128-row blocks, decode tokens in between, a rank over 64 (two passes), a ragged edge
TILE_CASES = [
    ("prompts-and-decode-two-parts", [1] * 30 + [128, 200, 70, 64] + [1] * 5, None, [64, 128, 16], 640,
     [("gate", 512), ("up", 296)]),
    ("one-long-prompt", [700], [1], [32], 1024, [("gate", 256)]),
    ("short-prompts-only", [40, 63, 17], [1, 2, 1], [16, 48], 256, [("gate", 520)]),
]


def _slots(case):
    name, rows, slots, ranks, K, mods = case
    if slots is None:
        rng = np.random.default_rng(len(rows))
        slots = rng.integers(0, len(ranks) + 1, len(rows))
    return slots


ALL_CASES = [(c, False) for c in CASES] + [(c, True) for c in TILE_CASES]


@pytest.mark.parametrize("case,tile_form", ALL_CASES, ids=[c[0] + ("-one-kernel" if t else "") for c, t in ALL_CASES])
def test_fused_fp8_layer_matches_the_oracle(pe, oracle, case, tile_form):
    from pocket_engine_b200 import workloads as wls
    import torch
    name, rows, slots, ranks, K, mods = case
    sites = [pe.Site.fused(0, K, mods)]
    slots = _slots(case)
    wl = wls.Workload(name, sites, ranks, 1.0, rows, slots, 13, max_rank=128)
    N = sites[0].width()
    wq, sn = _weights(N, K, 5)
    xb = wl.x_bits(0)
    xq, st = oracle.fp8_quant_rows(xb)
    table, _ = harness.oracle_registry(wl)
    tiles = harness.tiles_of(pe, wl)
    y64 = oracle.fp8_base_f64(xq, st, wq, sn)
    base_abs = np.abs(y64)
    oracle.site_f64(xb, K, tiles, table.tables[0], y64)
    rms = float(np.sqrt(np.mean(y64 ** 2)))

    loras = harness.product_registry(pe, wl)
    # the tensor-core form (base product + long runs in one kernel, gather kernel for the rest), or the
    # decode-shaped kernel that builds every token's adapter term inside its tiles
    loras.set_fused_tile_rows(1 if tile_form else 1 << 30)
    stream = torch.cuda.current_stream().cuda_stream
    x = harness.to_dev_bf16(xb, 0)
    xq_d = torch.zeros(wl.tokens, K, dtype=torch.uint8, device="cuda")
    st_d = torch.zeros(wl.tokens, dtype=torch.float32, device="cuda")
    wq_d = torch.from_numpy(wq).cuda()
    sn_d = torch.from_numpy(sn).cuda()
    for f32_out in (True, False):
        y = torch.full((wl.tokens, N), 7.0, dtype=torch.float32 if f32_out else torch.bfloat16, device="cuda")
        loras.meta_upload(tiles, stream)
        step = loras.lora_step(loras.max_lora_tiles(), stream)
        hook = loras.hook(0)
        loras.fp8_quant_rows(x.data_ptr(), wl.tokens, K, xq_d.data_ptr(), st_d.data_ptr(), stream)
        loras.shrink(hook, step, x.data_ptr(), wl.tokens, stream)
        loras.linear_fp8_fused(hook, step, xq_d.data_ptr(), st_d.data_ptr(), wq_d.data_ptr(), sn_d.data_ptr(), wl.tokens,
                               y.data_ptr(), N, f32_out, stream)
        torch.cuda.synchronize()
        loras.device_status()
        got = y.float().cpu().numpy().astype(np.float64)
        d = np.abs(got - y64)
        if f32_out:
            assert d.max() <= harness.MAX_TOL * rms and d.mean() <= harness.MEAN_TOL * rms, (name, d.max() / rms, d.mean() / rms)
            assert d.max() <= 2e-4 * rms, (name, d.max() / rms)  # f32 accumulation: far inside the stated bound
        else:
            # one bf16 rounding of the result: within half a bf16 step (2^-9 relative) plus the f32 error. In the
            # one-kernel form the tokens outside long runs get their adapter term from the gather kernel afterwards,
            # as in the engine (lora_expand after the layer's GEMM): the base is rounded to bf16 first, then the sum.
            slack = base_abs * 2.0 ** -8 if tile_form else 0.0
            assert np.all(d <= np.abs(y64) * 2.0 ** -8 + slack + 2e-4 * rms), (name, float((d / rms).max()))
    assert np.array_equal(xq_d.cpu().numpy(), xq)
    loras.close()


@pytest.mark.parametrize("case", TILE_CASES, ids=[c[0] for c in TILE_CASES])
def test_fused_bf16_layer_matches_the_oracle(pe, oracle, case):
    """y = x W^T + adapter term written once by the one-kernel layer, against the fp64 product of the same bf16
    operands plus the oracle's adapter term."""
    from pocket_engine_b200 import workloads as wls
    import torch
    name, rows, slots, ranks, K, mods = case
    sites = [pe.Site.fused(0, K, mods)]
    wl = wls.Workload(name, sites, ranks, 1.0, rows, _slots(case), 17, max_rank=128)
    N = sites[0].width()
    rng = np.random.default_rng(23)
    wb = pe.bf16_bits(rng.standard_normal((N, K), dtype=np.float32) / np.float32(np.sqrt(K)))
    xb = wl.x_bits(0)
    xf = pe.bf16_to_f32(xb).reshape(wl.tokens, K).astype(np.float64)
    wf = pe.bf16_to_f32(wb).reshape(N, K).astype(np.float64)
    table, _ = harness.oracle_registry(wl)
    tiles = harness.tiles_of(pe, wl)
    y64 = xf @ wf.T
    base_abs = np.abs(y64)
    oracle.site_f64(xb, K, tiles, table.tables[0], y64)
    rms = float(np.sqrt(np.mean(y64 ** 2)))
    loras = harness.product_registry(pe, wl)
    stream = torch.cuda.current_stream().cuda_stream
    x = harness.to_dev_bf16(xb, 0)
    w = harness.to_dev_bf16(wb, 0)
    for f32_out in (True, False):
        y = torch.full((wl.tokens, N), 7.0, dtype=torch.float32 if f32_out else torch.bfloat16, device="cuda")
        loras.meta_upload(tiles, stream)
        step = loras.lora_step(loras.max_lora_tiles(), stream)
        hook = loras.hook(0)
        loras.shrink(hook, step, x.data_ptr(), wl.tokens, stream)
        loras.linear_bf16_fused(hook, step, x.data_ptr(), w.data_ptr(), wl.tokens, y.data_ptr(), N, f32_out, stream)
        torch.cuda.synchronize()
        loras.device_status()
        d = np.abs(y.float().cpu().numpy().astype(np.float64) - y64)
        if f32_out:
            assert d.max() <= 2e-4 * rms and d.mean() <= harness.MEAN_TOL * rms, (name, d.max() / rms, d.mean() / rms)
        else:
            # tokens outside long runs: base rounded to bf16, then the sum rounded again (as in the engine)
            assert np.all(d <= (np.abs(y64) + base_abs) * 2.0 ** -8 + 2e-4 * rms), (name, float((d / rms).max()))
    loras.close()


def test_fused_bf16_layer_rejects_unaligned_shapes(pe):
    import torch
    sites = [pe.Site.fused(0, 256, [("gate", 130), ("up", 64)])]  # the second part starts at column 130
    loras = pe.Loras(sites, 2, 16, 64, 4, device=0)
    x = torch.zeros(8, 256, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(194, 256, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(8, 200, dtype=torch.bfloat16, device="cuda")
    loras.meta_upload(pe.fill_tiles([8], [0], loras.max_lora_tiles()))
    step = loras.lora_step(loras.max_lora_tiles())
    with pytest.raises(pe.PloraError) as err:
        loras.linear_bf16_fused(loras.hook(0), step, x.data_ptr(), w.data_ptr(), 8, y.data_ptr(), 200)
    assert err.value.code == pe.ERR_ARG
    loras.close()
