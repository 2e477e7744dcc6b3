"""Decoder forward passes on the GPU against the oracle: nanoGPT (config 4 architecture) and
the Llama-style stack (config 5 architecture) at sizes the oracle finishes in seconds, plus
size-independent properties at the full configurations."""

import numpy as np
import pytest
import torch

from oracle import inputs as I
from oracle import prefix as P
from oracle import reference_ops as R
from oracle.check import TOL_BF16, max_rel_err, assert_parity

from lighthouse_b200.plan import PlanOp
from lighthouse_b200.workloads import decoder as D
from lighthouse_b200.workloads.session import PlanSession

pytestmark = pytest.mark.gpu


def cuda_args(tensors):
    return [t.cuda().contiguous() for t in tensors]


def run_nanogpt(ctx, cfg, w, ids, use_graph=False):
    plan = D.build_nanogpt_plan(cfg)
    sw = D.shard_nanogpt_weights(w, cfg)
    logits = torch.zeros(cfg.tokens, cfg.vocab, device="cuda", dtype=torch.float32 if cfg.logits_dtype == "f32" else torch.bfloat16)
    args = [logits, ids.to(torch.int32).cuda()] + cuda_args(D.flatten_nanogpt_args(sw))
    s = PlanSession(plan, ctx=ctx, use_graph=use_graph)
    s.run(args, sync=True)
    if use_graph:  # second run replays the captured graph
        first = logits.clone()
        s.run(args, sync=True)
        assert torch.equal(first, logits)
    s.close()
    return logits


def run_llama(ctx, cfg, w, x):
    plan = D.build_llama_plan(cfg)
    sw = D.shard_llama_weights(w, cfg)
    out = torch.zeros(cfg.tokens, cfg.dim, device="cuda", dtype=torch.bfloat16)
    s = PlanSession(plan, ctx=ctx)
    s.run([out, x.cuda()] + cuda_args(D.flatten_llama_args(sw)), sync=True)
    s.close()
    return out


@pytest.mark.parametrize("act,causal", [("gelu", True), ("relu", False)])
def test_nanogpt_forward_matches_oracle(ctx, act, causal):
    cfg = D.NanoGptConfig(n_layer=2, n_head=4, n_embd=256, vocab=1024, block_size=128, batch=3, seq=128, act=act, causal=causal)
    w = I.nanogpt_weights(cfg.n_layer, cfg.n_embd, cfg.hidden, cfg.vocab, cfg.block_size, seed=4, std=0.05)
    ids = torch.randint(0, cfg.vocab, (cfg.tokens,), generator=torch.Generator().manual_seed(1))
    logits = run_nanogpt(ctx, cfg, w, ids, use_graph=(act == "gelu"))
    wn = I.tree_to_np(w)
    x = R.embed(ids.numpy().reshape(cfg.batch, cfg.seq), wn["wte"], wn["wpe"])
    ref = R.nanogpt_forward(x, wn["layers"], wn["gf_g"], wn["gf_b"], wn["lmw"], wn["lmb"], cfg.n_head, cfg.eps, causal, act, "bf16", cfg.batch)
    assert_parity(logits.cpu().numpy(), ref, "bf16")


def test_llama_forward_matches_oracle(ctx):
    cfg = D.LlamaConfig(n_layer=2, dim=512, n_heads=4, n_kv_heads=2, ffn=1024, batch=2, seq=192)
    w = I.llama_weights(cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=5, std=0.05)
    x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    out = run_llama(ctx, cfg, w, x)
    wn = I.tree_to_np(w)
    ref = R.llama_forward(I.to_np(x).reshape(cfg.batch, cfg.seq, cfg.dim), wn["layers"], wn["norm"], cfg.n_heads, cfg.n_kv_heads, cfg.theta, cfg.eps, "bf16", fused_swiglu=True, fused_residual=True)
    assert_parity(out.float().cpu().numpy(), ref.reshape(cfg.tokens, cfg.dim), "bf16")


def test_tensor_parallel_shards_sum_to_the_full_model_on_one_gpu(ctx):
    """tp=2 emulated on one GPU as two plans run back to back (never as concurrently waiting
    kernels): each rank's partial projection is summed on the host where the all-reduce sits.
    Checks the weight sharding and the rank-0-only residual/bias rule on the real kernels."""
    cfg = D.LlamaConfig(n_layer=1, dim=256, n_heads=4, n_kv_heads=2, ffn=512, batch=1, seq=128)
    w = I.llama_weights(1, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=7, std=0.05)
    x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    full = run_llama(ctx, cfg, w, x).float()
    # one attention sub-block per rank, stopping at the first all-reduce
    partial = []
    for rank in range(2):
        plan = D.build_llama_plan(cfg, rank, 2)
        cut = [i for i, op in enumerate(plan.ops) if op.kind == "allreduce"][0]
        h_view = plan.ops[cut].operands[0]
        plan.ops = plan.ops[:cut] + [PlanOp("elementwise", [plan.arg(0), h_view, None], {"ew": "copy", "act": "none", "scalar": 0.0})]
        sw = D.shard_llama_weights(w, cfg, rank, 2)
        out = torch.zeros(cfg.tokens, cfg.dim, device="cuda", dtype=torch.bfloat16)
        s = PlanSession(plan, ctx=ctx)
        s.run([out, x.cuda()] + cuda_args(D.flatten_llama_args(sw)), sync=True)
        s.close()
        partial.append(out.float())
    h_tp = (partial[0] + partial[1]).cpu().numpy()
    wn = I.tree_to_np(w)
    lw = wn["layers"][0]
    xr = I.to_np(x).reshape(1, cfg.seq, cfg.dim)
    want = xr + R.llama_attention(R.rmsnorm(xr, lw["attention_norm"], cfg.eps, "bf16"), lw["wq"], lw["wk"], lw["wv"], lw["wo"], cfg.n_heads, cfg.n_kv_heads, cfg.theta, True, "bf16")
    assert_parity(h_tp, want.reshape(cfg.tokens, cfg.dim), "bf16")
    assert bool(torch.isfinite(full).all())


def test_overlapped_schedule_on_one_gpu_matches_the_plain_plan(ctx):
    """The micro-batched two-stream schedule with tp=1 (collectives of a single rank are
    copies): side stream, numbered events and SM reservation on the real kernels."""
    cfg = D.LlamaConfig(n_layer=2, dim=256, n_heads=4, n_kv_heads=2, ffn=512, batch=2, seq=256)
    w = I.llama_weights(cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=7, std=0.05)
    x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    plain = run_llama(ctx, cfg, w, x).float()
    plan = D.build_llama_plan_overlapped(cfg, 0, 1, microbatches=2, reserve_sms=16)
    outs = []
    for _ in range(2):
        out = torch.zeros(cfg.tokens, cfg.dim, device="cuda", dtype=torch.bfloat16)
        s = PlanSession(plan, ctx=ctx)
        s.run([out, x.cuda()] + cuda_args(D.flatten_llama_args(D.shard_llama_weights(w, cfg))), sync=True)
        s.close()
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    assert_parity(outs[0].float().cpu().numpy(), plain.cpu().numpy(), "bf16")


def test_fused_schedule_on_one_gpu_matches_the_plain_plan(ctx):
    """The fused reduce + norm + gather operator in its single-rank form (plain loads and
    stores instead of multimem), inside the micro-batched schedule."""
    cfg = D.LlamaConfig(n_layer=2, dim=256, n_heads=4, n_kv_heads=2, ffn=512, batch=2, seq=256)
    w = I.llama_weights(cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=7, std=0.05)
    x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    plain = run_llama(ctx, cfg, w, x).float()
    plan = D.build_llama_plan_overlapped(cfg, 0, 1, microbatches=2, reserve_sms=16, fused=True)
    out = torch.zeros(cfg.tokens, cfg.dim, device="cuda", dtype=torch.bfloat16)
    extra = [torch.zeros(shape, device="cuda", dtype=torch.bfloat16) for shape in D.llama_symmetric_args(cfg, 2)]
    s = PlanSession(plan, ctx=ctx)
    s.run([out, x.cuda()] + cuda_args(D.flatten_llama_args(D.shard_llama_weights(w, cfg))) + extra, sync=True)
    s.close()
    assert_parity(out.float().cpu().numpy(), plain.cpu().numpy(), "bf16")


@pytest.mark.parametrize("rows,n,with_part", [(96, 4096, True), (7, 256, True), (130, 1024, False)])
def test_reduce_norm_gather_single_rank_matches_oracle(ctx, rows, n, with_part):
    g = torch.Generator().manual_seed(rows + n)
    h = torch.randn(rows, n, generator=g).to(torch.bfloat16)
    part = torch.randn(rows, n, generator=g).to(torch.bfloat16)
    wgt = (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)
    hd, pd, wd, xn = h.cuda(), part.cuda(), wgt.cuda(), torch.zeros(rows, n, device="cuda", dtype=torch.bfloat16)
    ctx.reduce_norm_gather(xn, pd if with_part else None, hd, wd, 1e-5)
    ctx.sync()
    h_ref = R.round_to(I.to_np(h) + I.to_np(part), "bf16") if with_part else I.to_np(h)
    assert np.array_equal(hd.float().cpu().numpy(), h_ref)  # the residual update is exact in bf16
    want = R.rmsnorm(h_ref, I.to_np(wgt), 1e-5, "bf16")
    assert_parity(xn.float().cpu().numpy(), want, "bf16")
    with pytest.raises(ValueError):
        ctx.reduce_norm_gather(xn, None, hd[:, : n - 4], wd, 1e-5)


def test_full_size_configs_run_and_are_deterministic(ctx):
    """Config 5 layer shapes (dim 4096, 32/8 heads, FFN 14336, seq 4096) with 1 layer and
    batch 1, and config 4 with 1 layer: finite outputs, bitwise-repeatable."""
    cfg = D.LlamaConfig(n_layer=1, batch=1)
    w = I.llama_weights(1, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=5)
    x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    a, b = run_llama(ctx, cfg, w, x), run_llama(ctx, cfg, w, x)
    assert torch.equal(a, b) and bool(torch.isfinite(a.float()).all())
    # RMS-normalised output with unit weight: every row has mean square ~ 1
    ms = a.float().pow(2).mean(-1)
    assert float((ms - 1).abs().max()) < 0.05
    gcfg = D.NanoGptConfig(n_layer=1, batch=2)
    gw = I.nanogpt_weights(1, gcfg.n_embd, gcfg.hidden, gcfg.vocab, gcfg.block_size, seed=4)
    ids = torch.randint(0, gcfg.vocab, (gcfg.tokens,), generator=torch.Generator().manual_seed(1))
    la, lb = run_nanogpt(ctx, gcfg, gw, ids), run_nanogpt(ctx, gcfg, gw, ids)
    assert torch.equal(la, lb) and bool(torch.isfinite(la).all())


def test_config5_full_depth_matches_oracle_on_causal_prefixes(ctx):
    """The whole Llama configuration (8 layers, d 4096, 32/8 heads, FFN 14336, batch 4, seq 4096)
    on the GPU; the first 256 positions of two sequences against the oracle run on those
    prefixes alone (a causal decoder's prefix depends on nothing after it)."""
    cfg = D.LlamaConfig()
    w = I.llama_weights(cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=5)
    x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    out = run_llama(ctx, cfg, w, x)
    seqs, prefix = (0, 3), 256
    rows = torch.from_numpy(P.prefix_rows(cfg.seq, seqs, prefix)).cuda()
    got = out[rows].float().cpu().numpy()
    # 8 layers: the one-layer bound times sqrt(8) (oracle/check.py::stack_scale)
    assert_parity(got, P.llama_prefix_reference(w, x, cfg, seqs, prefix), "bf16", n_layer=cfg.n_layer)


def test_config4_full_depth_matches_oracle_on_causal_prefixes(ctx):
    """The whole nanoGPT configuration (12 layers, d 768, 12 heads, batch 16, seq 1024, vocab
    50304): f32 logits of the first 256 positions of two sequences against the oracle."""
    cfg = D.NanoGptConfig()
    w = I.nanogpt_weights(cfg.n_layer, cfg.n_embd, cfg.hidden, cfg.vocab, cfg.block_size, seed=4)
    ids = torch.randint(0, cfg.vocab, (cfg.tokens,), generator=torch.Generator().manual_seed(1))
    logits = run_nanogpt(ctx, cfg, w, ids)
    seqs, prefix = (0, 11), 256
    rows = torch.from_numpy(P.prefix_rows(cfg.seq, seqs, prefix)).cuda()
    got = logits[rows].cpu().numpy()
    del logits
    assert_parity(got, P.nanogpt_prefix_reference(w, ids, cfg, seqs, prefix), "bf16")
