"""nanoGPT / Llama decoder plans and their tensor-parallel sharding, checked on the CPU:
the plans are executed with the oracle's arithmetic (tests/cpu_plan.py); the multi-rank path
runs as two gloo ranks whose all-reduce is ``torch.distributed.all_reduce``."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cpu_plan import CpuPlanRunner
from oracle import inputs as I
from oracle import reference_ops as R
from oracle.check import max_rel_err

from lighthouse_b200.workloads import decoder as D

GPT = D.NanoGptConfig(n_layer=2, n_head=4, n_embd=64, vocab=128, block_size=16, batch=2, seq=16, act="gelu", causal=True)
GPT4 = D.NanoGptConfig(n_layer=2, n_head=4, n_embd=64, vocab=128, block_size=16, batch=4, seq=16, act="gelu", causal=True)  # 2 micro-batches x 2 ranks x whole sequences
LLAMA = D.LlamaConfig(n_layer=2, dim=128, n_heads=8, n_kv_heads=2, ffn=256, batch=2, seq=16)


def gpt_reference(cfg, w, ids):
    wn = I.tree_to_np(w)
    x = R.embed(ids.reshape(cfg.batch, cfg.seq), wn["wte"], wn["wpe"])
    return R.nanogpt_forward(x, wn["layers"], wn["gf_g"], wn["gf_b"], wn["lmw"], wn["lmb"], cfg.n_head, cfg.eps, cfg.causal, cfg.act, "bf16", cfg.batch)


def llama_reference(cfg, w, x):
    wn = I.tree_to_np(w)
    xr = I.to_np(x).reshape(cfg.batch, cfg.seq, cfg.dim)
    out = R.llama_forward(xr, wn["layers"], wn["norm"], cfg.n_heads, cfg.n_kv_heads, cfg.theta, cfg.eps, "bf16", fused_swiglu=True, fused_residual=True)
    return out.reshape(cfg.tokens, cfg.dim)


def run_gpt_rank(cfg, w, ids, rank, tp, allreduce=None, overlapped=False):
    plan = D.build_nanogpt_plan_overlapped(cfg, rank, tp, microbatches=2) if overlapped else D.build_nanogpt_plan(cfg, rank, tp)
    sw = D.shard_nanogpt_weights(w, cfg, rank, tp, full_bias=overlapped)
    args = [np.zeros((cfg.tokens, cfg.vocab // tp), np.float32), ids.astype(np.int64)] + [I.to_np(t) for t in D.flatten_nanogpt_args(sw)]
    return CpuPlanRunner(plan, allreduce, rank, tp).run(args)[0]


def run_llama_rank(cfg, w, x, rank, tp, allreduce=None, overlapped=False, fused=False, result_symmetric=False):
    plan = D.build_llama_plan_overlapped(cfg, rank, tp, microbatches=2, fused=fused, result_symmetric=result_symmetric) if overlapped else D.build_llama_plan(cfg, rank, tp)
    sw = D.shard_llama_weights(w, cfg, rank, tp)
    args = [np.zeros((cfg.tokens, cfg.dim), np.float32), I.to_np(x)] + [I.to_np(t) for t in D.flatten_llama_args(sw)]
    if fused:
        args += [np.zeros(shape, np.float32) for shape in D.llama_symmetric_args(cfg, 2)]
    return CpuPlanRunner(plan, allreduce, rank, tp).run(args)[0]


def gpt_inputs(cfg):
    w = I.nanogpt_weights(cfg.n_layer, cfg.n_embd, cfg.hidden, cfg.vocab, cfg.block_size, seed=4, std=0.1)
    ids = torch.randint(0, cfg.vocab, (cfg.tokens,), generator=torch.Generator().manual_seed(1)).numpy()
    return w, ids


def llama_inputs(cfg):
    w = I.llama_weights(cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=5, std=0.1)
    x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    return w, x


def test_flop_model_matches_the_published_per_token_counts():
    assert D.NanoGptConfig().flops_per_token() == pytest.approx(266.0e6, rel=1e-3)
    assert D.LlamaConfig().flops_per_token() == pytest.approx(3.758e9, rel=1e-3)
    assert D.build_nanogpt_plan(D.NanoGptConfig()).total_flops() == pytest.approx(4.358e12, rel=2e-3)
    assert D.build_llama_plan(D.LlamaConfig()).total_flops() == pytest.approx(61.57e12, rel=2e-3)


def test_nanogpt_plan_single_rank_matches_oracle():
    w, ids = gpt_inputs(GPT)
    got = run_gpt_rank(GPT, w, ids, 0, 1)
    assert max_rel_err(got, gpt_reference(GPT, w, ids)) < 2e-2


def test_llama_plan_single_rank_matches_oracle():
    w, x = llama_inputs(LLAMA)
    got = run_llama_rank(LLAMA, w, x, 0, 1)
    assert max_rel_err(got, llama_reference(LLAMA, w, x)) < 2e-2


def test_tp_degrees_that_do_not_divide_are_rejected():
    with pytest.raises(ValueError):
        D.check_tp(D.NanoGptConfig(), 8)  # 12 heads
    with pytest.raises(ValueError):
        D.check_tp(D.LlamaConfig(), 16)
    D.check_tp(D.NanoGptConfig(), 4)
    D.check_tp(D.LlamaConfig(), 8)


def test_swiglu_packing_layout():
    g = torch.arange(256 * 4, dtype=torch.float32).view(256, 4)
    u = -g
    p = D.pack_swiglu(g, u)
    assert p.shape == (512, 4)
    assert torch.equal(p[:128], g[:128]) and torch.equal(p[128:256], u[:128]) and torch.equal(p[256:384], g[128:])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _tp_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        def allreduce(a):
            t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float64))
            dist.all_reduce(t)
            return t.numpy()

        w, ids = gpt_inputs(GPT)
        logits = run_gpt_rank(GPT, w, ids, rank, world, allreduce)
        w4, ids4 = gpt_inputs(GPT4)
        logits_overlapped = run_gpt_rank(GPT4, w4, ids4, rank, world, allreduce, overlapped=True)
        # batch split: this rank's sequences through the plain single-rank plan, no collective;
        # the ranks' logits are gathered only to be checked
        import dataclasses

        part = dataclasses.replace(GPT4, batch=GPT4.batch // world)
        mine = run_gpt_rank(part, w4, ids4[rank * part.tokens : (rank + 1) * part.tokens], 0, 1)
        gathered = [torch.zeros(mine.shape, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(np.ascontiguousarray(mine, dtype=np.float32)))
        logits_dp = torch.cat(gathered, dim=0).numpy()
        lw, x = llama_inputs(LLAMA)
        hidden = run_llama_rank(LLAMA, lw, x, rank, world, allreduce)
        hidden_overlapped = run_llama_rank(LLAMA, lw, x, rank, world, allreduce, overlapped=True)
        hidden_fused = run_llama_rank(LLAMA, lw, x, rank, world, allreduce, overlapped=True, fused=True, result_symmetric=True)
        q.put((rank, logits, hidden, hidden_overlapped, hidden_fused, logits_overlapped, logits_dp))
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_matches_single_rank():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted([q.get(timeout=300) for _ in range(world)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    w, ids = gpt_inputs(GPT)
    full = gpt_reference(GPT, w, ids)
    logits = np.concatenate([r[1] for r in results], axis=1)  # vocab-sharded logits
    assert max_rel_err(logits, full) < 2e-2
    lw, x = llama_inputs(LLAMA)
    want = llama_reference(LLAMA, lw, x)
    w4, ids4 = gpt_inputs(GPT4)
    logits4 = np.concatenate([r[5] for r in results], axis=1)
    assert max_rel_err(logits4, gpt_reference(GPT4, w4, ids4)) < 2e-2  # row-sharded residual, overlapped collectives
    for r in results:  # sequences split over the ranks: every rank's gathered logits are the full batch's
        assert max_rel_err(r[6], gpt_reference(GPT4, w4, ids4)) < 2e-2
    for _, _, hidden, hidden_overlapped, hidden_fused, _, _ in results:  # the residual stream is replicated after each all-reduce
        assert max_rel_err(hidden, want) < 2e-2
        assert max_rel_err(hidden_overlapped, want) < 2e-2  # reduce-scatter / all-gather schedule
        assert max_rel_err(hidden_fused, want) < 2e-2  # one fused reduce + norm + gather per sub-block
    for i in (2, 3, 4):
        assert np.array_equal(results[0][i], results[1][i])


def test_overlapped_schedule_is_the_same_computation_and_is_fully_ordered():
    """Micro-batched reduce-scatter / all-gather schedule on one rank: same result as the plain
    plan up to the extra bf16 roundings of the sharded residual add; the interpreter's
    vector clocks accept its event ordering, and reject it once a wait is taken out."""
    w, x = llama_inputs(LLAMA)
    plain = run_llama_rank(LLAMA, w, x, 0, 1)
    assert max_rel_err(run_llama_rank(LLAMA, w, x, 0, 1, overlapped=True), plain) < 2e-2
    plan = D.build_llama_plan_overlapped(LLAMA, 0, 1, microbatches=2)
    kinds = plan.kinds()
    n_sub = 2 * LLAMA.n_layer * 2
    # one gather per contraction, plus the first norm of every micro-batch but the first (whose
    # rows each rank normalises itself: the input is replicated)
    assert kinds.count("reducescatter") == n_sub and kinds.count("allgather") == n_sub + 1
    assert kinds.count("reserve_sms") == 2 and plan.ops[[i for i, k in enumerate(kinds) if k == "reserve_sms"][-1]].attrs["index"] == 0
    # drop the main stream's wait for the first gathered activations: a read-before-write race
    waits = [i for i, op in enumerate(plan.ops) if op.kind == "event_wait" and i + 1 < len(plan.ops) and plan.ops[i + 1].kind == "gemm"]
    del plan.ops[waits[0]]
    sw = D.shard_llama_weights(w, LLAMA, 0, 1)
    args = [np.zeros((LLAMA.tokens, LLAMA.dim), np.float32), I.to_np(x)] + [I.to_np(t) for t in D.flatten_llama_args(sw)]
    with pytest.raises(AssertionError, match="without waiting"):
        CpuPlanRunner(plan).run(args)
    with pytest.raises(ValueError):
        D.build_llama_plan_overlapped(LLAMA, 0, 1, microbatches=3)
    # the fused form: same schedule, one operator per side chain, symmetric buffers as arguments
    fused = D.build_llama_plan_overlapped(LLAMA, 0, 1, microbatches=2, fused=True)
    assert fused.kinds().count("reduce_norm_gather") == n_sub + 1 and "reducescatter" not in fused.kinds()
    assert len(fused.args) == len(plan.args) + 4 and fused.args[-1].name == "xn1"
    got = run_llama_rank(LLAMA, w, x, 0, 1, overlapped=True, fused=True)
    assert max_rel_err(got, plain) < 2e-2
    # with a symmetric result buffer the last layer gathers straight into it: no copy, same values
    direct = D.build_llama_plan_overlapped(LLAMA, 0, 1, microbatches=2, fused=True, result_symmetric=True)
    assert direct.kinds().count("reduce_norm_gather") == n_sub + 1 and direct.kinds().count("ew:copy") == fused.kinds().count("ew:copy") - 2
    assert np.array_equal(run_llama_rank(LLAMA, w, x, 0, 1, overlapped=True, fused=True, result_symmetric=True), got)


def test_nanogpt_overlapped_schedule_single_rank_and_limits():
    w, ids = gpt_inputs(GPT4)
    plain = run_gpt_rank(GPT4, w, ids, 0, 1)
    assert max_rel_err(run_gpt_rank(GPT4, w, ids, 0, 1, overlapped=True), plain) < 2e-2
    assert max_rel_err(plain, gpt_reference(GPT4, w, ids)) < 2e-2
    with pytest.raises(ValueError):  # one sequence per micro-batch cannot be cut into two row blocks of whole sequences
        D.build_nanogpt_plan_overlapped(GPT, 0, 2, microbatches=2)
