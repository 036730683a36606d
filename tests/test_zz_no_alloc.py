"""The allocation-free entry point, for callers that cannot allocate device memory (an engine whose memory
is fully claimed at start-up, code inside a stream capture, plugin hosts that forbid allocation after
initialisation): it must give what the handle-based path gives, on two calls in a row (the second call
finds the first call's leftovers in the shared static scratch), and must refuse sizes over its scratch.
Collected last on purpose, so a run that stops at the first failure has already run every other test."""
import numpy as np
import pytest

import harness

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_the_handle_path_twice(pe):
    import torch
    from pocket_engine_b200 import workloads
    wl = workloads.config2(tokens=40, adapters=5)
    loras = harness.product_registry(pe, wl, max_tokens=64, max_seqs=64)
    stream = torch.cuda.current_stream().cuda_stream
    for f32_out in (False, True):
        want = harness.run_gpu(pe, loras, wl, f32_out)  # also leaves the step's tile words on the device
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
                else:
                    ulp = harness.bf16_ulp_diff(got, want[si], pe)
                    assert ulp.max() <= 1 and (ulp > 0).mean() < 2e-3, (call, si, int(ulp.max()))
    loras.close()


def test_static_scratch_entry_rejects_what_does_not_fit(pe):
    import torch
    assert pe.lib.plora_static_scratch_bytes() == 8 << 20
    x = torch.zeros(16, 4096, dtype=torch.bfloat16, device="cuda")
    hook = pe.Hook(table=x.data_ptr(), parts=1, max_rows=64, parity=0, cols=4096, site=0)
    with pytest.raises(pe.PloraError) as e:  # 8 splits * 4096 rows * 512 * 4 bytes = 64 MiB
        pe.site_apply_static(x.data_ptr(), 4096, 4096, x.data_ptr(), 64, hook, 512, x.data_ptr(), 64)
    assert e.value.code == pe.ERR_CAPACITY and "static scratch" in e.value.text
    with pytest.raises(pe.PloraError) as e:
        pe.site_apply_static(x.data_ptr() + 2, 16, 4096, x.data_ptr(), 64, hook, 64, x.data_ptr(), 64)
    assert e.value.code == pe.ERR_ARG
