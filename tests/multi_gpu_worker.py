"""Worker for tests/test_gpu_multi.py: launched by torch.distributed.run, one rank per GPU (NCCL)."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from dirotq_b200 import backend, dit, ops, parallel
    from dirotq_b200.synth import synth_activations
    backend.patch_forward()
    res = {}
    for quant in ("int4", "nvfp4"):
        hidden, inner, M = 1152, 4608, 1024
        ffn = parallel.build_flux_tp_ffn(world, rank, quant, dev, seed=3000, hidden=hidden, inner=inner, k=64)
        ffn.reduce_dtype = torch.float32
        x = synth_activations(M, hidden, torch.Generator().manual_seed(5)).reshape(2, M // 2, hidden).to(dev)
        y_tp = ffn(x)
        full = parallel.build_flux_tp_ffn(1, 0, quant, dev, seed=3000, hidden=hidden, inner=inner, k=64)
        h = full.act_fn(full.up_fn(x))
        y_ref = full.down_fn(h)
        err = float((y_tp.float() - y_ref.float()).norm() / y_ref.float().norm())
        # data parallel: this rank's batch shard through the unsplit layer == its slice of the full result
        xs = parallel.shard_batch(x, world, rank)
        y_dp = full.down_fn(full.act_fn(full.up_fn(xs)))
        b, e = parallel.shard_range(x.shape[0], world, rank)
        dp_equal = bool(torch.equal(y_dp, y_ref[b:e]))
        t = torch.tensor([err, 0.0 if dp_equal else 1.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[quant] = {"tp_rel_l2": float(t[0]), "dp_equal": float(t[1]) == 0.0}
    ops.check_status(dev)
    if rank == 0:
        print("RESULT " + json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
