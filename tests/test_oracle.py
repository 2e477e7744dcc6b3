"""Pins the CPU oracle: against the reference's golden vectors, against fixtures generated
by running the reference's own torch model and its own numpy check functions, and against
torch where only a definition exists (GELU)."""

import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import build as oracle_build
from oracle import inputs as I
from oracle import reference_ops as R
from oracle.check import assert_close, max_rel_err


@pytest.fixture(scope="module")
def lh_run_golden():
    with open(os.path.join(GOLDEN, "lh_run_pipeline_check.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def llama_golden():
    return np.load(os.path.join(GOLDEN, "llama_ref.npz"))


@pytest.fixture(scope="module")
def numpy_checks():
    return np.load(os.path.join(GOLDEN, "numpy_checks.npz"))


def test_lh_run_known_answer(lh_run_golden):
    """The 16 row values of the reference's lh-run test: rnd(16x64) @ ones(64x32), seed 123."""
    g = lh_run_golden
    a, b, c = I.lh_run_args(g["input_shape"], g["seed"])
    for out in (R.matmul_f32_loops(a, b, c), oracle_build.matmul_loops(a, b, c), oracle_build.matmul_loops(a, b, c, interchange=False)):
        assert out.shape == (16, 32)
        for row, want in zip(out, g["row_values"]):
            assert np.all(row == row[0])
            # the test prints with numpy's default 8 significant digits
            assert float(np.format_float_positional(row[0], precision=8, unique=True, fractional=False)) == pytest.approx(want, rel=2e-7)


def test_c_loop_nest_matches_numpy_restatement():
    a, b, c = I.gemm_f32_uniform(37, 29, 53, seed=7)
    ref = R.matmul_f32_loops(a, b, c)
    assert np.array_equal(oracle_build.matmul_loops(a, b, c), ref)
    assert np.array_equal(oracle_build.matmul_loops(a, b, c, interchange=False), ref)
    assert max_rel_err(ref, a.astype(np.float64) @ b.astype(np.float64)) < 1e-6


def test_llama_ops_match_reference_model(llama_golden):
    g = llama_golden
    dim, nl, nh, nkv, B, S = (int(x) for x in g["meta"])
    assert_close(R.rmsnorm(g["rms_x"], g["rms_w"], 1e-5, "f32"), g["rms_out"], "f32", "RMSNorm")
    assert_close(R.rope(g["rope_xq"], 10000.0, 0, "f32"), g["rope_q_out"], "f32", "rotary q")
    assert_close(R.rope(g["rope_xk"], 10000.0, 0, "f32"), g["rope_k_out"], "f32", "rotary k")
    out = R.llama_attention(g["attn_x"], g["attn_wq"], g["attn_wk"], g["attn_wv"], g["attn_wo"], nh, nkv, 10000.0, True, "f32")
    assert_close(out, g["attn_out"], "f32", "Attention")
    assert_close(R.llama_feed_forward(g["ff_x"], g["ff_w1"], g["ff_w2"], g["ff_w3"], "f32"), g["ff_out"], "f32", "FeedForward")


def test_llama_stack_matches_reference_model(llama_golden):
    g = llama_golden
    dim, nl, nh, nkv, B, S = (int(x) for x in g["meta"])
    keys = ("wq", "wk", "wv", "wo", "w1", "w2", "w3", "attention_norm", "ffn_norm")
    layers = [{k: g[f"tf_l{i}_{k}"] for k in keys} for i in range(nl)]
    assert_close(R.llama_block(g["tf_x"], layers[0], nh, nkv, 10000.0, 1e-5, "f32"), g["tf_block0_out"], "f32", "TransformerBlock")
    assert_close(R.llama_forward(g["tf_x"], layers, g["tf_norm"], nh, nkv, 10000.0, 1e-5, "f32"), g["tf_out"], "f32", "Transformer trunk")
    assert_close(R.llama_forward(g["tf_x"], layers, g["tf_norm"], nh, nkv, 10000.0, 1e-5, "f32", fused_swiglu=True, fused_residual=True), g["tf_out"], "f32", "fused SwiGLU and residual")


def test_row_ops_match_torch():
    rng = np.random.RandomState(0)
    x = rng.randn(33, 96).astype(np.float32)
    gmm, bta = rng.randn(96).astype(np.float32), rng.randn(96).astype(np.float32)
    t = torch.from_numpy(x)
    assert_close(R.layernorm(x, gmm, bta, 1e-5), torch.nn.functional.layer_norm(t, (96,), torch.from_numpy(gmm), torch.from_numpy(bta), 1e-5).numpy(), "f32", "layernorm")
    assert_close(R.softmax(x), torch.softmax(t, -1).numpy(), "f32", "softmax")
    np.testing.assert_allclose(R.softmax(x).sum(-1), 1.0, rtol=1e-5)
    assert_close(R.gelu_erf(x), torch.nn.functional.gelu(t).numpy(), "f32", "gelu")
    assert_close(R.silu(x), torch.nn.functional.silu(t).numpy(), "f32", "silu")


def test_attention_matches_torch_sdpa():
    q, k, v = I.attention_qkv(2, 4, 2, 48, 80, 32, seed=11)
    for causal in (False, True):
        ref = R.attention(I.to_np(q), I.to_np(k), I.to_np(v), causal=causal, io_dtype="f32")
        kk, vv = k.float().repeat_interleave(2, 1), v.float().repeat_interleave(2, 1)
        mask = torch.ones(48, 80, dtype=torch.bool).tril(80 - 48) if causal else None
        want = torch.nn.functional.scaled_dot_product_attention(q.float(), kk, vv, attn_mask=mask)
        assert_close(ref, want.numpy(), "f32", f"attention causal={causal}")


def test_gemm_epilogue_order_and_rounding():
    a, b, bias = I.gemm_bf16_normal(24, 40, 64, seed=3)
    A, B, bv = I.to_np(a), I.to_np(b), I.to_np(bias)
    out = R.gemm_epilogue(A, B, bias=bv, act="relu", out_dtype="bf16")
    want = torch.relu(a.float() @ b.float() + bias.float()).to(torch.bfloat16).float().numpy()
    assert np.array_equal(out, want)
    c = np.ones((24, 40), np.float32)
    assert np.allclose(R.gemm_epilogue(A, B, c=c), A @ B + 1.0)
    assert np.allclose(R.gemm_epilogue(A.T, B.T, transpose_a=True, transpose_b=True), A @ B)


# ------------------------------------------------------------------------------------------
# Fixtures produced by executing the reference's own numpy check functions
# (tests/golden/make_golden.py::golden_numpy_checks). 16-bit cases: the oracle and the
# reference evaluate the same formula with differently ordered f32 operations, so a value that
# sits on a rounding boundary of the 16-bit type may round the other way; the bound is one
# f16 ulp at the output's scale, everything else agrees to f32 rounding.
F16_ULP = 2.0**-10


def test_nanogpt_helpers_match_reference_functions(numpy_checks):
    g = numpy_checks
    assert_close(R.layernorm(g["gpt_x"], g["gpt_l0_g1"], g["gpt_l0_b1n"], 1e-5), g["gpt_ln"], "f32", "_ln")
    assert np.array_equal(R.round_to(g["gpt_x"] * 3.3, "f16"), g["gpt_f16"])
    T, C, H, hid, vocab, L = (int(v) for v in g["gpt_meta"])
    heads = lambda t: t.reshape(1, T, H, C // H).transpose(0, 2, 1, 3)
    for causal, key in ((False, "mha_out"), (True, "mha_out_causal")):
        got = R.attention(heads(g["mha_q"]), heads(g["mha_k"]), heads(g["mha_v"]), causal=causal, io_dtype="f16")
        # the oracle also rounds O to the 16-bit type (the kernel's output type); _mha returns f32
        want = g[key].reshape(T, H, C // H).transpose(1, 0, 2)[None]
        assert max_rel_err(got, R.round_to(want, "f16")) <= F16_ULP, key


def _gpt_layers(g, L):
    keys = ("g1", "b1n", "wq", "wk", "wv", "wp", "bp", "g2", "b2n", "w1", "bb1", "w2", "bb2")
    return [{k: g[f"gpt_l{i}_{k}"].astype(np.float32) for k in keys} for i in range(L)]


def test_nanogpt_block_and_model_match_reference_functions(numpy_checks):
    g = numpy_checks
    T, C, H, hid, vocab, L = (int(v) for v in g["gpt_meta"])
    layers = _gpt_layers(g, L)
    for causal, key in ((False, "gpt_block"), (True, "gpt_block_causal")):
        got = R.nanogpt_block(g["gpt_x"], layers[0], H, act="relu", causal=causal, lowp="f16")
        assert max_rel_err(got, g[key]) <= F16_ULP, key
        assert np.median(np.abs(got - g[key])) <= 1e-6 * np.abs(g[key]).max()
    got = R.nanogpt_forward(g["gpt_x"], layers, g["gpt_gf_g"], g["gpt_gf_b"], g["gpt_lmw"].astype(np.float32), g["gpt_lmb"], H, act="relu", causal=False, lowp="f16")
    assert max_rel_err(got, g["gpt_logits"]) <= 2 * F16_ULP
    assert np.median(np.abs(got - g["gpt_logits"])) <= 1e-6 * np.abs(g["gpt_logits"]).max()


def test_attention_layernorm_softmax_match_reference_checks(numpy_checks):
    g = numpy_checks
    f = lambda a: a.astype(np.float32)
    assert_close(R.attention_unfused_f32(f(g["fa_q"]), f(g["fa_k"]), f(g["fa_v"])), g["fa_out"], "f32", "fused_attention check_correctness")
    assert_close(R.layernorm(g["ln_x"], g["ln_g"], g["ln_b"], 1e-5), g["ln_out"], "f32", "layer_norm check_correctness")
    assert_close(R.softmax(g["sm_x"]), g["sm_out"], "f32", "softmax check_correctness")


def test_matmul_workload_matches_reference_generator_and_check(numpy_checks):
    from lighthouse_b200.workloads.matmul import CudaMatMul, matmul_complexity

    g = numpy_checks
    M, N, K = (int(v) for v in g["mm_meta"])
    assert tuple(g["mm_complexity"]) == matmul_complexity(4096, 4096, 4096, True, True, False, 2, 2)
    for i, (bias, relu, acc, trunc, ta, tb, ints) in enumerate(g["mm_variants"].astype(bool)):
        wl = CudaMatMul(M=M, N=N, K=K, ab_type="f16", c_type="f32", has_bias=bool(bias), has_relu=bool(relu), accumulate_c=bool(acc),
                        truncate_c=bool(trunc), transpose_a=bool(ta), transpose_b=bool(tb))
        arrays = wl.get_input_arrays(bool(ints))
        names = ("C", "A", "B", "bias")[: len(arrays)]
        for name, arr in zip(names, arrays):  # the seeded inputs themselves
            assert arr.dtype == g[f"mm{i}_{name}"].dtype and np.array_equal(arr, g[f"mm{i}_{name}"]), (i, name)
        f = lambda a: a.astype(np.float32)
        got = R.gemm_epilogue(f(arrays[1]), f(arrays[2]), c=f(arrays[0]) if acc else None, bias=f(arrays[3]) if bias else None,
                              act="relu" if relu else "none", out_dtype="f16" if trunc else "f32", transpose_a=bool(ta), transpose_b=bool(tb))
        want = f(g[f"mm{i}_out"])
        if ints:
            assert np.array_equal(got, want), i  # small integers: every product and sum is exact
        else:
            assert max_rel_err(got, want) <= (F16_ULP if trunc else 1e-6), i


def test_mlp_chain_matches_reference_check(numpy_checks):
    g = numpy_checks
    f = lambda a: a.astype(np.float32)
    h = f(g["mlp_x"])
    for i in range(3):  # ReLU between layers only, every layer's result truncated (examples/xegpu/mlp.py:76-84)
        h = R.gemm_epilogue(h, f(g[f"mlp_w{i}"]), bias=f(g[f"mlp_b{i}"]), act="relu" if i < 2 else "none", out_dtype="f16")
    assert max_rel_err(h, f(g["mlp_out"])) <= 2 * F16_ULP
    assert np.median(np.abs(h - f(g["mlp_out"]))) == 0.0


def test_complexity_models_match_reference(numpy_checks):
    g = numpy_checks
    # attention: 4 Z H S^2 D flop, Q K V read + O written (examples/xegpu/fused_attention.py:26-43)
    Z, H, S, D, nb = 8, 16, 2048, 128, 2
    assert tuple(g["fa_complexity"]) == (4 * Z * H * S * S * D, 3 * Z * H * S * D * nb, Z * H * S * D * nb)
    # row kernels: one read and one write of the matrix (softmax.py:24-39); layer norm also reads gamma and beta
    Mr, Nr = 16384, 768
    assert tuple(g["sm_complexity"])[1:] == (Mr * Nr * 4, Mr * Nr * 4)
    assert g["ln_complexity"][2] == Mr * Nr * 4 and g["ln_complexity"][1] >= Mr * Nr * 4


def test_causal_prefix_property_of_the_decoder_oracles():
    """What the full-size GPU parity tests rely on: the first t positions of a causal decoder's
    output depend on the first t inputs only, so the oracle run on a prefix reproduces those
    rows of the oracle run on whole sequences."""
    from lighthouse_b200.workloads import decoder as D
    from oracle import prefix as P

    cfg = D.LlamaConfig(n_layer=2, dim=64, n_heads=4, n_kv_heads=2, ffn=128, batch=3, seq=24)
    w = I.llama_weights(cfg.n_layer, cfg.dim, cfg.n_heads, cfg.n_kv_heads, cfg.ffn, seed=5, std=0.1)
    x = torch.randn(cfg.tokens, cfg.dim, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    wn = I.tree_to_np(w)
    full = R.llama_forward(I.to_np(x).reshape(cfg.batch, cfg.seq, cfg.dim), wn["layers"], wn["norm"], cfg.n_heads, cfg.n_kv_heads, cfg.theta, cfg.eps, "bf16", fused_swiglu=True, fused_residual=True)
    rows = P.prefix_rows(cfg.seq, (0, 2), 9)
    got = P.llama_prefix_reference(w, x, cfg, (0, 2), 9)
    assert max_rel_err(got, full.reshape(cfg.tokens, cfg.dim)[rows]) <= 1e-6

    g = D.NanoGptConfig(n_layer=2, n_head=4, n_embd=64, vocab=96, block_size=32, batch=3, seq=24)
    gw = I.nanogpt_weights(g.n_layer, g.n_embd, g.hidden, g.vocab, g.block_size, seed=4, std=0.1)
    ids = torch.randint(0, g.vocab, (g.tokens,), generator=torch.Generator().manual_seed(1))
    gn = I.tree_to_np(gw)
    xe = R.embed(ids.numpy().reshape(g.batch, g.seq), gn["wte"], gn["wpe"])
    full = R.nanogpt_forward(xe, gn["layers"], gn["gf_g"], gn["gf_b"], gn["lmw"], gn["lmb"], g.n_head, g.eps, True, g.act, "bf16", g.batch)
    got = P.nanogpt_prefix_reference(gw, ids, g, (1, 2), 7, vocab_slice=slice(48, 96))
    assert max_rel_err(got, full[P.prefix_rows(g.seq, (1, 2), 7), 48:96]) <= 1e-6


def test_llama_linalg_restatement_matches_the_reference_tests_ground_truth():
    """The oracle's restatement of the reference's linalg Llama builders against the torch
    model run the way the reference's own tests run it (real frequencies, additive mask):
    attention, one block, the two-layer transformer. Tolerance: the oracle's f32 bound, far
    inside the 0.01 the reference's tests allow (examples/llama/test_llama3.py:1651,1812,1985)."""
    g = np.load(os.path.join(GOLDEN, "llama_linalg_ref.npz"))
    dim, nl, nh, nkv, B, S, hidden = (int(v) for v in g["meta"])
    layers = [{k: g[f"l{i}_{k}"] for k in ("wq", "wk", "wv", "wo", "w1", "w2", "w3")} for i in range(nl)]
    l0 = layers[0]
    assert_close(R.llama_linalg_attention(g["x"], l0["wq"], l0["wk"], l0["wv"], l0["wo"], g["freqs_real"], g["mask"], nh, nkv), g["attn_out"], "f32", "get_attention")
    assert_close(R.llama_linalg_block(g["x"], l0, g["freqs_real"], g["mask"], nh, nkv), g["block0_out"], "f32", "get_transformer_block")
    assert_close(R.llama_linalg_transformer(g["x"], layers, g["freqs_real"], g["mask"], nh, nkv), g["out"], "f32", "get_transformer")


def test_sharded_contraction_rounds_per_device_and_agrees_with_the_plain_product():
    """One shard is the rounded product; several shards round each partial sum and the total,
    which moves a bf16 result by a few units in the last place and an f32 one not at all
    beyond summation order."""
    rng = np.random.default_rng(5)
    a = R.round_bf16(rng.standard_normal((24, 64)).astype(np.float32))
    w = R.round_bf16(rng.standard_normal((16, 64)).astype(np.float32) * 0.1)
    plain = R.round_bf16(a @ w.T)
    assert np.array_equal(R.sharded_contraction(a, w, 1, "bf16"), plain)
    two = R.sharded_contraction(a, w, 2, "bf16")
    assert not np.array_equal(two, plain)
    assert np.max(np.abs(two - plain)) <= 3 * 2.0**-8 * np.max(np.abs(plain))
    np.testing.assert_allclose(R.sharded_contraction(a, w, 4, "f32"), a @ w.T, rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        R.sharded_contraction(a, w, 3, "bf16")


def test_depth_and_rounding_count_scale_the_bounds():
    """One layer keeps the stated bounds; n layers scale them by sqrt(n); a schedule that rounds
    more often along a layer (the tensor-parallel one) by the square root of that ratio too, and
    the report says so."""
    from oracle.check import LAYER_ROUNDINGS, SHARDED_LAYER_ROUNDINGS, parity_report, stack_scale

    assert stack_scale(1) == 1.0 and stack_scale(0) == 1.0
    assert abs(stack_scale(8) - 8**0.5) < 1e-12
    assert abs(stack_scale(8, SHARDED_LAYER_ROUNDINGS) - (8 * SHARDED_LAYER_ROUNDINGS / LAYER_ROUNDINGS) ** 0.5) < 1e-12
    ref = np.linspace(-1.0, 1.0, 4096, dtype=np.float32).reshape(64, 64)
    out = ref + 0.015  # 1.5 % of max|ref| everywhere, also where ref is 0: outside the one-layer per-element bound (0.7 %), inside the 8-layer one (2 %)
    one = parity_report(out, ref, "bf16")
    deep = parity_report(out, ref, "bf16", n_layer=8)
    sharded = parity_report(out, ref, "bf16", n_layer=8, roundings_per_layer=SHARDED_LAYER_ROUNDINGS)
    assert not one["ok"] and "tol_rule" not in one
    assert deep["ok"] and "sqrt(8 layers)" in deep["tol_rule"] and abs(deep["tol"] - 0.0566) < 1e-4
    assert sharded["ok"] and sharded["tol"] > deep["tol"] and "13" in sharded["tol_rule"]
    assert sharded["elementwise_excess"] < deep["elementwise_excess"] < one["elementwise_excess"]
