"""The allocation-free entry point, for callers that cannot allocate device memory (an engine whose memory is
fully claimed at start-up, plugin hosts that forbid allocation after initialisation): it must give what the
handle-based path gives and what the CPU oracle gives, on two calls in a row (the second call finds the first
call's leftovers in the shared static scratch), must leave device memory as it found it, must skip tiles whose
numbers make no sense, and must refuse sizes over its scratch.
Collected last on purpose, so a run that stops at the first failure has already run every other test."""
import numpy as np
import pytest

import harness

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_the_handle_path_and_the_oracle_twice(pe):
    import torch
    from pocket_engine_b200 import workloads
    wl = workloads.config2(tokens=40, adapters=5)
    loras = harness.product_registry(pe, wl, max_tokens=64, max_seqs=64)
    table, _ = harness.oracle_registry(wl)
    tiles = harness.tiles_of(pe, wl)
    stream = torch.cuda.current_stream().cuda_stream
    free0 = None
    for f32_out in (False, True):
        want = harness.run_gpu(pe, loras, wl, f32_out)  # also leaves the step's tile words on the device
        y64 = harness.oracle_f64(wl, table, tiles, f32_out=f32_out, pe=pe)
        rounded = harness.oracle_rounded(wl, table, tiles, f32_out, pe)
        for call in range(2):
            for si, site in enumerate(wl.sites):
                x = harness.to_dev_bf16(wl.x_bits(si), 0)
                yb = wl.y_base(si)
                y = torch.from_numpy(yb.copy()).cuda() if f32_out else harness.to_dev_bf16(pe.bf16_bits(yb), 0)
                pe.site_apply_static(x.data_ptr(), wl.tokens, site.cols, loras.tiles, loras.max_lora_tiles(),
                                     loras.hook(si), loras.lds, y.data_ptr(), y.shape[1], f32_out, stream)
                got = y.float().cpu().numpy()
                if f32_out:
                    mx, mn = harness.tolerance(got, want[si].astype(np.float64))
                    assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL, (call, si, mx, mn)
                    mx, mn = harness.tolerance(got, y64[si])  # and against the fp64 oracle
                    assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL, (call, si, mx, mn)
                else:
                    ulp = harness.bf16_ulp_diff(got, want[si], pe)
                    assert ulp.max() <= 1 and (ulp > 0).mean() < 2e-3, (call, si, int(ulp.max()))
                    ulp = harness.bf16_ulp_diff(got, rounded[si], pe)
                    assert ulp.max() <= 1 and (ulp > 0).mean() < 2e-3, (call, si, int(ulp.max()))
            torch.cuda.synchronize()
            free = torch.cuda.mem_get_info()[0]
            if free0 is None:
                free0 = free  # after the first round of calls (the array's address is resolved by now)
    # nothing was allocated by any later call: free device memory never fell below what the first round left
    assert torch.cuda.mem_get_info()[0] >= free0 - (4 << 20)
    assert pe.lib.plora_static_bad_tiles() == 0
    loras.close()


def test_static_scratch_entry_skips_tiles_that_make_no_sense(pe):
    """A tile past the rows, with more than 16 tokens, with a negative start or slot: skipped and counted, y untouched
    for it, the good tile next to it still applied. Nothing is read or written through the bad numbers."""
    import torch
    from pocket_engine_b200 import workloads
    wl = workloads.config1()
    loras = harness.product_registry(pe, wl)
    site = wl.sites[0]
    x = harness.to_dev_bf16(wl.x_bits(0), 0)
    yb = wl.y_base(0)
    before = pe.lib.plora_static_bad_tiles()
    words = np.array([5, 14, 4, 1, 0, 17, 2, -3, 2, 1, 3, 1, -1, 2, 1, 2], np.int32)  # only the last tile (row 2, slot 2) is good
    tiles = torch.from_numpy(words).cuda()
    y = torch.from_numpy(yb.copy()).cuda()
    pe.site_apply_static(x.data_ptr(), wl.tokens, site.cols, tiles.data_ptr(), 8, loras.hook(0), loras.lds,
                         y.data_ptr(), y.shape[1], True)
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    assert pe.lib.plora_static_bad_tiles() == before + 4
    changed = np.nonzero(np.any(got != yb, axis=1))[0]
    assert list(changed) == [2]
    table, _ = harness.oracle_registry(wl)
    orc = __import__("__graft_entry__").load_oracle()
    want = yb.astype(np.float64)
    orc.site_f64(wl.x_bits(0), site.cols, np.array([1, 2, 1, 2], np.int32), table.tables[0], want)
    mx, mn = harness.tolerance(got, want)
    assert mx <= harness.MAX_TOL and mn <= harness.MEAN_TOL
    loras.close()


def test_static_scratch_entry_rejects_what_does_not_fit(pe):
    import torch
    assert pe.lib.plora_static_scratch_bytes() == 8 << 20
    assert pe.lib.plora_static_splits(4096) == 8 and pe.lib.plora_static_splits(1024) == 2
    x = torch.zeros(16, 4096, dtype=torch.bfloat16, device="cuda")
    hook = pe.Hook(table=x.data_ptr(), parts=1, max_rows=64, parity=0, cols=4096, site=0)
    with pytest.raises(pe.PloraError) as e:  # 8 splits * 4096 rows * 512 * 4 bytes = 64 MiB
        pe.site_apply_static(x.data_ptr(), 4096, 4096, x.data_ptr(), 64, hook, 512, x.data_ptr(), 64)
    assert e.value.code == pe.ERR_CAPACITY and "static scratch" in e.value.text
    with pytest.raises(pe.PloraError) as e:
        pe.site_apply_static(x.data_ptr() + 2, 16, 4096, x.data_ptr(), 64, hook, 64, x.data_ptr(), 64)
    assert e.value.code == pe.ERR_ARG
