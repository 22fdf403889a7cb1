"""world_size-2 gloo tests (CPU) of the multi-GPU host logic: batch sharding needs no collective,
a column/row-split quantised FFN plus ONE all-reduce equals the unsplit layer."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dirotq_oracle as O


def _ffn_pieces(seed=0, D=128, Fdim=256, k=32):
    g = torch.Generator().manual_seed(seed)
    U = O.random_orthogonal(D, g).float()
    W_up = torch.randn(Fdim, D, generator=g) * 0.05
    low, _, _ = O.weight_quant_int((W_up @ U)[:, : D - k], 4, 64)
    W_up_f = torch.cat([low, (W_up @ U)[:, D - k:]], 1).to(torch.bfloat16)
    b_up = (torch.randn(Fdim, generator=g) * 0.1).to(torch.bfloat16)
    W_dn = torch.randn(D, Fdim, generator=g) * 0.05
    W_dn_q, _, _ = O.weight_quant_int(W_dn, 4, 64)
    W_dn_q = W_dn_q.to(torch.bfloat16)
    b_dn = (torch.randn(D, generator=g) * 0.1).to(torch.bfloat16)
    x = O.synth_activations(64, D, g).reshape(4, 16, D)
    return U, W_up_f, b_up, W_dn_q, b_dn, x, k


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from dirotq_b200.parallel import TPFeedForward, shard_batch, shard_range, tp_slices
        U, W_up, b_up, W_dn, b_dn, x, k = _ffn_pieces()
        Fdim = W_up.shape[0]
        c0, c1 = tp_slices(Fdim, world, rank, 64)
        cfg_up = O.QuantCfg(4, 64, True, 1.0, k, "int")
        cfg_dn = O.QuantCfg(4, 64, True, 1.0, 0, "int")
        up_spec = O.LayerSpec(W_up[c0:c1], b_up[c0:c1], cfg_up, rotation=U)
        dn_spec = O.LayerSpec(W_dn[:, c0:c1].contiguous(), b_dn if rank == 0 else None, cfg_dn)
        ffn = TPFeedForward(lambda t: O.fused_forward(t, up_spec), lambda h: O.fused_forward(h, dn_spec),
                            lambda t: torch.nn.functional.gelu(t, approximate="tanh"), reduce_dtype=torch.float32)
        y_tp = ffn(x)
        # data parallel: each rank's shard through the SAME (unsplit) layer, gathered only to check
        full_up = O.LayerSpec(W_up, b_up, cfg_up, rotation=U)
        full_dn = O.LayerSpec(W_dn, b_dn, cfg_dn)
        unsplit = lambda t: O.fused_forward(torch.nn.functional.gelu(O.fused_forward(t, full_up), approximate="tanh"), full_dn)
        xs = shard_batch(x, world, rank)
        y_dp = unsplit(xs)
        gathered = [torch.empty_like(y_dp) for _ in range(world)]
        dist.all_gather(gathered, y_dp)
        if rank == 0:
            y_ref = unsplit(x)
            q.put({"tp_err": float((y_tp.float() - y_ref.float()).norm() / y_ref.float().norm()),
                   "dp_equal": bool(torch.equal(torch.cat(gathered), y_ref)),
                   "ranges": [shard_range(7, 2, r) for r in range(2)]})
    finally:
        dist.destroy_process_group()


def test_tp_ffn_and_dp_shard_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res["dp_equal"], "batch-sharded outputs differ from the unsharded layer"
    assert res["tp_err"] < 1e-2, res          # partial sums are rounded to bf16 per rank before the reduce
    assert res["ranges"] == [(0, 4), (4, 7)]


def test_tp_slices_reject_split_groups():
    from dirotq_b200.parallel import tp_slices
    assert tp_slices(12288, 8, 3, 64) == (4608, 6144)
    with pytest.raises(ValueError):
        tp_slices(1152, 8, 0, 64)
