"""plora_apply right behind the kernel that writes y (src/linear.rs:844-847: lora_expand is issued straight after
the layer's own matrix multiply). The kernels of plora_apply are launched with programmatic stream serialization
and release their own dependents early, so they must not bind any value of y (or of x, unless the caller vouched
for it) before their dependency wait: a producer that is still running, or that releases its dependents early
itself, would otherwise be read half-written. Every iteration changes x, so a stale read cannot hide."""
import numpy as np
import pytest

import harness

pytestmark = pytest.mark.gpu

ITERS = 200


def _setup(pe, oracle, K, widths, tokens, n_adapters, rank, seed):
    from pocket_engine_b200 import workloads
    sites = [pe.Site.fused(0, K, [(f"m{i}", w) for i, w in enumerate(widths)]),
             pe.Site.fused(0, K, [(f"n{i}", w) for i, w in enumerate(widths)])]
    rng = np.random.default_rng(seed)
    slots = rng.integers(0, n_adapters + 1, tokens)
    wl = workloads.Workload("behind-a-gemm", sites, [rank] * n_adapters, 2.0, [1] * tokens, slots, seed)
    loras = harness.product_registry(pe, wl)
    table, _ = harness.oracle_registry(wl)
    tiles = harness.tiles_of(pe, wl)
    return wl, loras, table, tiles


@pytest.mark.parametrize("mode", ["cluster", "pair"])
def test_apply_right_behind_a_library_gemm(pe, oracle, mode):
    """torch.matmul(out=y) (a cuBLAS kernel) then plora_apply on the same y, 200 times with new x."""
    import torch
    K, widths, T = 2048, [4096, 2048], 48
    wl, loras, table, tiles = _setup(pe, oracle, K, widths, T, 5, 16, 61)
    N = sum(widths)
    dev = "cuda"
    stream = torch.cuda.Stream()
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    w = (torch.randn(N, K, generator=gen, device=dev) / K ** 0.5).to(torch.bfloat16)
    xs = [torch.randn(T, K, generator=gen, device=dev).to(torch.bfloat16) for _ in range(ITERS)]
    ys = [torch.empty(T, N, dtype=torch.bfloat16, device=dev) for _ in range(ITERS)]
    base = [torch.empty(T, N, dtype=torch.bfloat16, device=dev) for _ in range(ITERS)]
    loras.set_apply_mode(1 if mode == "cluster" else 0)
    with torch.cuda.stream(stream):
        s = stream.cuda_stream
        loras.meta_upload(tiles, s)
        step = loras.lora_step(loras.max_lora_tiles(), s, decode=True)
        hooks = [loras.hook(0), loras.hook(1)]
        for i in range(ITERS):
            torch.matmul(xs[i], w.t(), out=base[i])  # what the layer's GEMM alone gives (the oracle's input)
        for i in range(ITERS):
            torch.matmul(xs[i], w.t(), out=ys[i])
            loras.apply(hooks[i % 2], step, xs[i].data_ptr(), T, ys[i].data_ptr(), N, False, s)
    stream.synchronize()
    loras.device_status()
    for i in range(ITERS):
        xb = xs[i].view(torch.int16).cpu().numpy().view(np.uint16)
        yb = base[i].float().cpu().numpy()
        want = pe.bf16_bits(yb).reshape(yb.shape).copy()
        oracle.site_f32s(xb, K, tiles, table.tables[i % 2], want, False)
        got = ys[i].float().cpu().numpy()
        ulp = harness.bf16_ulp_diff(got, pe.bf16_to_f32(want).reshape(got.shape), pe, floor=3e-5)
        assert ulp.max() <= 1 and (ulp > 0).mean() < 1e-2, (i, int(ulp.max()), float((ulp > 0).mean()))
        # the adapter term is really there: rows with a slot differ from the GEMM's output
        has = wl.token_slot() > 0
        assert np.any(got[has] != yb[has]) and np.array_equal(got[~has], yb[~has])
    loras.close()


def test_apply_right_behind_the_one_kernel_layer(pe, oracle):
    """The library's own plora_linear_bf16_fused (which is launched with programmatic stream serialization itself)
    writes y, then plora_apply of a second layer updates the same y."""
    import torch
    K, widths, T = 1024, [1024, 512], 40
    wl, loras, table, tiles = _setup(pe, oracle, K, widths, T, 4, 16, 62)
    N = sum(widths)
    dev = "cuda"
    stream = torch.cuda.Stream()
    gen = torch.Generator(device=dev)
    gen.manual_seed(8)
    w = (torch.randn(N, K, generator=gen, device=dev) / K ** 0.5).to(torch.bfloat16)
    iters = 50
    xs = [torch.randn(T, K, generator=gen, device=dev).to(torch.bfloat16) for _ in range(iters)]
    ys = [torch.empty(T, N, dtype=torch.float32, device=dev) for _ in range(iters)]
    with torch.cuda.stream(stream):
        s = stream.cuda_stream
        loras.meta_upload(tiles, s)
        step = loras.lora_step(loras.max_lora_tiles(), s, decode=True)
        h0, h1 = loras.hook(0), loras.hook(1)
        for i in range(iters):
            loras.shrink(h0, step, xs[i].data_ptr(), T, s)
            loras.linear_bf16_fused(h0, step, xs[i].data_ptr(), w.data_ptr(), T, ys[i].data_ptr(), N, True, s)
            loras.apply(h1, step, xs[i].data_ptr(), T, ys[i].data_ptr(), N, True, s)
    stream.synchronize()
    loras.device_status()
    wf = w.float().cpu().numpy().astype(np.float64)
    for i in range(iters):
        xb = xs[i].view(torch.int16).cpu().numpy().view(np.uint16)
        want = pe.bf16_to_f32(xb).reshape(T, K).astype(np.float64) @ wf.T
        oracle.site_f64(xb, K, tiles, table.tables[0], want)
        oracle.site_f64(xb, K, tiles, table.tables[1], want)
        mx, mn = harness.tolerance(ys[i].cpu().numpy(), want)
        assert mx <= 2e-4 and mn <= harness.MEAN_TOL, (i, mx, mn)
    loras.close()
