"""Runs in a process of its own with PLORA_LIB pointing at the range-checked build of the library
(libplora_bounds.so, -DPLORA_BOUNDS): the plumbing configuration and the odd shapes through every form of the
few-token path must pass their oracle checks with the checks compiled in, and a launch whose records reach past
the rows it names must be refused record by record (status word, y untouched) instead of touching memory."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import torch
    import __graft_entry__ as entry
    import harness
    pe = entry.load_package()
    from pocket_engine_b200 import workloads
    assert pe.lib.plora_bounds_build() == 1, "PLORA_LIB must name the range-checked build"
    done = []
    for fused in (False, "early", "cluster"):
        for f32_out in (True, False):
            harness.run_and_check(pe, workloads.config1(), f32_out=f32_out, meta="device", fused=fused)
    done.append("plumbing")
    import test_gpu_parity as tp
    for name, rows, slots, ranks, K, mods in tp.RAGGED:
        sites = [pe.Site.fused(0, K, mods), pe.Site.fused(0, K, [("z", 48)])]
        wl = workloads.Workload(name, sites, ranks, 1.5, rows, slots, 3)
        for fused in (False, "early", "cluster"):
            harness.run_and_check(pe, wl, f32_out=True, meta="host", fused=fused)
            harness.run_and_check(pe, wl, f32_out=False, meta="device", fused=fused)
        done.append(name)
    harness.run_and_check(pe, workloads.config2(), f32_out=False, meta="device", fused="cluster")
    done.append("decode block")
    # records that reach past the rows the launch names: 16 tokens grouped, but the calls say rows = 8
    wl = workloads.config1()
    loras = harness.product_registry(pe, wl)
    stream = torch.cuda.current_stream().cuda_stream
    refused = {}
    for fused in (False, "early", "cluster"):
        loras.meta_upload(harness.tiles_of(pe, wl, loras.max_lora_tiles()), stream)
        step = loras.lora_step(loras.max_lora_tiles(), stream)
        x = harness.to_dev_bf16(wl.x_bits(0), 0)
        yb = wl.y_base(0)
        y = torch.from_numpy(yb.copy()).cuda()
        if fused:
            loras.set_apply_mode(1 if fused == "cluster" else 0)
        pe.Linear(loras, 0).forward(x.data_ptr(), 8, y.data_ptr(), y.shape[1], True, lora=step, main=stream, fused=bool(fused))
        torch.cuda.synchronize()
        try:
            loras.device_status()
            code = 0
        except pe.PloraError as e:
            code = e.code
        got = y.cpu().numpy()
        # work items whose tokens all lie below row 8 were applied, the others were skipped whole: no row at or past
        # 8 changed, and every row either kept its base value or got its full update
        refused[str(fused)] = {"code": code, "rows_changed_past_8": int(np.any(got[8:] != yb[8:], axis=1).sum()),
                               "rows_changed_below_8": int(np.any(got[:8] != yb[:8], axis=1).sum())}
    loras.close()
    print(json.dumps({"bounds_check": "ok", "cases": done, "refused": refused}))


if __name__ == "__main__":
    main()
