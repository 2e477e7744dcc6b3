"""Pins the CPU oracle: against the reference's golden vectors, against fixtures generated
by running the reference's own torch model, and against torch where only a definition exists."""

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
    assert_close(R.llama_forward(g["tf_x"], layers, g["tf_norm"], nh, nkv, 10000.0, 1e-5, "f32", fused_swiglu=True), g["tf_out"], "f32", "fused SwiGLU")


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


def test_nanogpt_block_equals_reference_formula():
    """nanogpt_block with f16 / ReLU / non-causal / batch 1 must reduce to the reference's own
    numpy formula (restated inline here from examples/xegpu/nanoGPT.py:84-127)."""
    rng = np.random.RandomState(5)
    T, C, H, hid = 16, 32, 4, 64
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    w = dict(
        g1=np.ones(C, np.float32), b1n=np.zeros(C, np.float32), g2=np.ones(C, np.float32), b2n=np.zeros(C, np.float32),
        wq=f16(rng.randn(C, C) * 0.1), wk=f16(rng.randn(C, C) * 0.1), wv=f16(rng.randn(C, C) * 0.1), wp=f16(rng.randn(C, C) * 0.1),
        bp=rng.randn(C).astype(np.float32), w1=f16(rng.randn(C, hid) * 0.1), bb1=rng.randn(hid).astype(np.float32),
        w2=f16(rng.randn(hid, C) * 0.1), bb2=rng.randn(C).astype(np.float32),
    )
    x = (rng.randn(T, C) * 0.5).astype(np.float32)

    def ln(z, g, b):
        mu, var = z.mean(-1, keepdims=True), z.var(-1, keepdims=True)
        return (z - mu) / np.sqrt(var + 1e-5) * g + b

    ln1 = f16(ln(x, w["g1"], w["b1n"]))
    q, k, v = f16(ln1 @ w["wq"]), f16(ln1 @ w["wk"]), f16(ln1 @ w["wv"])
    hs = C // H
    attn = np.zeros((T, C), np.float32)
    for h in range(H):
        sl = slice(h * hs, (h + 1) * hs)
        s = (q[:, sl] @ k[:, sl].T) / (hs**0.5)
        e = np.exp(s - s.max(-1, keepdims=True))
        attn[:, sl] = f16(e / e.sum(-1, keepdims=True)) @ v[:, sl]
    a = x + f16(attn) @ w["wp"] + w["bp"]
    ln2 = f16(ln(a, w["g2"], w["b2n"]))
    want = a + f16(np.maximum(ln2 @ w["w1"] + w["bb1"], 0.0)) @ w["w2"] + w["bb2"]
    got = R.nanogpt_block(x, w, H, act="relu", causal=False, lowp="f16")
    # the oracle rounds the attention output to the 16-bit type once more (the kernel's O type)
    assert max_rel_err(got, want) < 2e-3
