"""Two-rank tests on two GPUs (skipped on a single-GPU box): the tensor-parallel schedules
on real NCCL and on the fused multimem kernel, one process per GPU, against the oracle.

No rank is made to fail here: every process runs the same plans and leaves between steps."""

import os
import socket

import numpy as np
import pytest
import torch

from oracle import inputs as I
from oracle import reference_ops as R
from oracle.check import TOL_BF16, max_rel_err, assert_parity

pytestmark = pytest.mark.gpu

CFG = dict(n_layer=2, dim=256, n_heads=4, n_kv_heads=2, ffn=512, batch=2, seq=256)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import torch.distributed as dist

    from lighthouse_b200.context import CudaContext, find_torch_nccl, nccl_unique_id
    from lighthouse_b200.workloads import decoder as D
    from lighthouse_b200.workloads.session import PlanSession
    from lighthouse_b200.workloads.symmetric import SymmetricBuffers

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ctx = CudaContext(rank)
    try:
        nccl = find_torch_nccl()
        ids = [None] * world
        dist.all_gather_object(ids, nccl_unique_id(nccl) if rank == 0 else None)
        ctx.comm_init(ids[0], rank, world, nccl)
        symm = SymmetricBuffers(ctx)

        # 1. the fused operator alone: ragged row count, full-width rows
        rows, n = 50, 4096
        g = torch.Generator().manual_seed(11)
        parts = [torch.randn(rows * world, n, generator=g).to(torch.bfloat16) for _ in range(world)]
        h_all = torch.randn(rows * world, n, generator=g).to(torch.bfloat16)
        wgt = (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)
        part_s, xn_s = symm.empty((rows * world, n), torch.bfloat16), symm.empty((rows * world, n), torch.bfloat16)
        part_s.copy_(parts[rank])
        xn_s.zero_()
        h_mine, wgt_dev = h_all[rank * rows : (rank + 1) * rows].cuda(), wgt.cuda()
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(3):  # repeated launches exercise the epoch flags; h accumulates the sum each time
            ctx.reduce_norm_gather(xn_s, part_s, h_mine, wgt_dev, 1e-5)
        ctx.sync()
        op_xn, op_h = xn_s.float().cpu().numpy(), h_mine.float().cpu().numpy()

        # 2. the decoder: synchronous all-reduce, NCCL overlapped, fused overlapped
        cfg = D.LlamaConfig(**CFG)
        w = I.llama_weights(cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=7, std=0.05)
        x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
        weights = [t.cuda().contiguous() for t in D.flatten_llama_args(D.shard_llama_weights(w, cfg, rank, world))]
        outs = {}
        for name in ("allreduce", "nccl_overlapped", "fused_overlapped"):
            if name == "allreduce":
                plan, extra = D.build_llama_plan(cfg, rank, world), []
            else:
                fused = name == "fused_overlapped"
                plan = D.build_llama_plan_overlapped(cfg, rank, world, microbatches=2, reserve_sms=16, fused=fused)
                extra = [symm.empty(shape, torch.bfloat16) for shape in D.llama_symmetric_args(cfg, 2)] if fused else []
            out, x_dev = torch.zeros(cfg.tokens, cfg.dim, device="cuda", dtype=torch.bfloat16), x.cuda()
            torch.cuda.synchronize()
            sess = PlanSession(plan, ctx=ctx)
            for _ in range(2):
                sess.run([out, x_dev] + weights + extra, sync=True)
            sess.close()
            outs[name] = out.float().cpu().numpy()
        symm.close()
        q.put((rank, op_xn, op_h, outs, None))
    except Exception as e:  # the parent reports it; the process still leaves cleanly
        q.put((rank, None, None, None, repr(e)))
    finally:
        ctx.close()
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_on_two_gpus_match_the_oracle():
    import torch.multiprocessing as mp

    world = 2
    mpctx = mp.get_context("spawn")
    q = mpctx.Queue()
    port = _free_port()
    procs = [mpctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([q.get(timeout=600) for _ in range(world)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for r in results:
        assert r[4] is None, f"rank {r[0]}: {r[4]}"

    # fused operator: three accumulating launches
    rows, n = 50, 4096
    g = torch.Generator().manual_seed(11)
    parts = [I.to_np(torch.randn(rows * world, n, generator=g).to(torch.bfloat16)) for _ in range(world)]
    h = I.to_np(torch.randn(rows * world, n, generator=g).to(torch.bfloat16))
    wgt = I.to_np((1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16))
    total = R.round_to(sum(p.astype(np.float32) for p in parts), "bf16")
    for _ in range(3):
        h = R.round_to(h + total, "bf16")
    want_xn = R.rmsnorm(h, wgt, 1e-5, "bf16")
    for rank, op_xn, op_h, _, _ in results:
        # the switch returns its f32 sum in the activation type with a rounding of its own:
        # the residual rows agree to bf16 precision, not bit for bit
        assert_parity(op_h, h[rank * rows : (rank + 1) * rows], "bf16")
        assert_parity(op_xn, want_xn, "bf16")  # every rank holds every rank's rows
    assert np.array_equal(results[0][1], results[1][1])

    # decoder: all three schedules against the single-rank oracle, and replicated across ranks
    from lighthouse_b200.workloads import decoder as D

    cfg = D.LlamaConfig(**CFG)
    w = I.llama_weights(cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=7, std=0.05)
    x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    wn = I.tree_to_np(w)
    ref = R.llama_forward(I.to_np(x).reshape(cfg.batch, cfg.seq, cfg.dim), wn["layers"], wn["norm"], cfg.n_heads, cfg.n_kv_heads, cfg.theta, cfg.eps, "bf16", fused_swiglu=True, fused_residual=True)
    ref = ref.reshape(cfg.tokens, cfg.dim)
    for name in ("allreduce", "nccl_overlapped", "fused_overlapped"):
        for r in results:
            assert_parity(r[3][name], ref, "bf16")
        assert np.array_equal(results[0][3][name], results[1][3][name]), name
