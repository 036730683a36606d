"""One rank of the tensor-parallel GPU check (launched by torchrun from test_gpu_tp.py or by hand):
every rank runs its shard of a 27B-shaped layer set through TPLinear (NCCL all-reduce of the shrink
partials in the row-parallel layers); rank 0 assembles the outputs and compares them with the unsharded
fp64 oracle. Prints one JSON line on rank 0."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    import harness
    pe = entry.load_package()
    orc = entry.load_oracle()
    from pocket_engine_b200 import tp, workloads
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    full = os.environ.get("PLORA_TP_FULL") == "1"
    wl = workloads.config5() if full else workloads.config5(adapters=6, rank=16, hidden=512, inter=1024, q_width=768,
                                                            decode=40, chunks=(128, 70))
    sh = tp.ShardedWorkload(wl, world, rank)
    loras = harness.product_registry(pe, sh, device=local)
    stream = torch.cuda.current_stream().cuda_stream
    loras.meta_upload(pe.fill_tiles(sh.row_n, sh.row_slot, loras.max_lora_tiles()), stream)
    step = loras.lora_step(loras.max_lora_tiles(), stream)
    exchange = os.environ.get("PLORA_TP_EXCHANGE", "nccl")
    if exchange == "fused":
        tp.connect_exchange(loras, rank, world)
    worst = (0.0, 0.0)
    for si in range(len(sh.sites)):
        x = harness.to_dev_bf16(sh.x_bits(si), local)
        y = torch.from_numpy(sh.y_base(si).copy()).cuda()
        lin = tp.TPLinear(loras, si, sh.modes[si], exchange=exchange)
        lin.forward(x.data_ptr(), sh.tokens, y.data_ptr(), y.shape[1], True, lora=step, main=stream)
        torch.cuda.synchronize()
        outs = [None] * world
        dist.all_gather_object(outs, y.cpu().numpy())
        if rank == 0:
            got = sh.assemble(si, outs)
            table, _ = harness.oracle_registry(wl)
            tiles = orc.fill_tiles(wl.row_n, wl.row_slot, wl.tokens // 16 + wl.n_seqs)
            want = wl.y_base(si).astype(np.float64)
            orc.site_f64(wl.x_bits(si), wl.sites[si].cols, tiles, table.tables[si], want)
            mx, mn = harness.tolerance(got, want)
            worst = (max(worst[0], mx), max(worst[1], mn))
    loras.device_status()
    if rank == 0:
        ok = worst[0] <= harness.MAX_TOL and worst[1] <= harness.MEAN_TOL
        print(json.dumps({"tp_check": "ok" if ok else "FAILED", "world": world, "exchange": exchange, "max_over_rms": worst[0],
                          "mean_over_rms": worst[1], "workload": wl.name}))
    loras.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
