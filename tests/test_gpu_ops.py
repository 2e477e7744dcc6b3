"""Parity of the CUDA kernels, called through the C ABI, against the CPU oracle on the same
seeded inputs. Tolerances: max |out - ref| / max |ref| <= 1e-5 for f32, <= 2e-2 for bf16
operands with f32 accumulation (oracle/check.py)."""

import numpy as np
import pytest
import torch

from oracle import build as oracle_build
from oracle import inputs as I
from oracle import reference_ops as R
from oracle.check import TOL_BF16, TOL_F32, max_rel_err, assert_parity

from lighthouse_b200 import _native as N

pytestmark = pytest.mark.gpu

ACT = {"none": N.ACT_NONE, "relu": N.ACT_RELU, "gelu": N.ACT_GELU_ERF, "gelu_tanh": N.ACT_GELU_TANH, "silu": N.ACT_SILU}


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def host(t):
    return t.detach().float().cpu().numpy()


# ------------------------------------------------------------------------------------ f32 GEMM
@pytest.mark.parametrize("shape", [(16, 32, 64), (1, 1, 1), (130, 70, 33), (257, 129, 100)])
def test_gemm_f32_matches_loop_nest(ctx, shape):
    m, n, k = shape
    a, b, c = I.gemm_f32_uniform(m, n, k, seed=m + n)
    c = np.random.RandomState(1).rand(m, n).astype(np.float32)
    ref = oracle_build.matmul_loops(a, b, c)
    d = dev(c.copy())
    ctx.gemm(d, dev(a), dev(b), c=d)
    ctx.sync()
    assert_parity(host(d), ref, "f32")


@pytest.mark.parametrize("shape", [(300, 264, 77), (129, 512, 1000), (2048, 128, 9)])
def test_gemm_f32_tensor_core_split_path(ctx, shape):
    """Shapes large enough for the split-f32 (six bf16 products) tensor-core path (N a multiple of 8), ragged in M
    and K, accumulating into C, with bias, activation and residual, and with transposed
    operand views: within the f32 tolerance of the loop nest."""
    m, n, k = shape
    a, b, _ = I.gemm_f32_uniform(m, n, k, seed=m + k)
    c = np.random.RandomState(2).rand(m, n).astype(np.float32)
    ref = oracle_build.matmul_loops(a, b, c)
    d = dev(c.copy())
    ctx.gemm(d, dev(a), dev(b), c=d)
    ctx.sync()
    assert_parity(host(d), ref, "f32")
    d2 = dev(c.copy())
    ctx.gemm(d2, dev(np.ascontiguousarray(a.T)).t(), dev(np.ascontiguousarray(b.T)).t(), c=d2)
    ctx.sync()
    assert_parity(host(d2), ref, "f32")
    bias, res = np.random.RandomState(3).randn(n).astype(np.float32), np.random.RandomState(4).randn(m, n).astype(np.float32)
    d3 = torch.zeros(m, n, device="cuda")
    ctx.gemm(d3, dev(a), dev(b), bias=dev(bias), residual=dev(res), act=N.ACT_RELU)
    ctx.sync()
    want = np.maximum(oracle_build.matmul_loops(a, b, np.zeros((m, n), np.float32)) + bias, 0) + res
    assert_parity(host(d3), want, "f32")
    # the CUDA-core kernel on request, same answer
    d4 = dev(c.copy())
    ctx.gemm(d4, dev(a), dev(b), c=d4, flags=N.GEMM_FORCE_SIMT)
    ctx.sync()
    assert_parity(host(d4), host(d), "f32")


def test_gemm_f32_config1_full_size(ctx):
    """Config 1: 1024^3, A, B ~ U(-1, 1), zero C; the C loop-nest oracle is the reference."""
    a, b, c = I.gemm_f32_uniform(1024, 1024, 1024, seed=1)
    ref = oracle_build.matmul_loops(a, b, c)
    d = dev(c)
    ctx.gemm(d, dev(a), dev(b))
    ctx.sync()
    assert_parity(host(d), ref, "f32")
    # strided views: A^T given as a transposed view, same answer
    d2 = torch.zeros_like(d)
    ctx.gemm(d2, dev(np.ascontiguousarray(a.T)).t(), dev(b))
    ctx.sync()
    assert_parity(host(d2), ref, "f32")


def test_gemm_empty_and_degenerate(ctx):
    d = torch.full((4, 8), 3.0, device="cuda")
    ctx.gemm(d, torch.zeros(4, 0, device="cuda"), torch.zeros(0, 8, device="cuda"))
    ctx.sync()
    assert float(d.abs().max()) == 0.0
    ctx.gemm(torch.zeros(0, 8, device="cuda"), torch.zeros(0, 4, device="cuda"), torch.zeros(4, 8, device="cuda"))
    with pytest.raises(ValueError):
        ctx.gemm(torch.zeros(4, 8, device="cuda"), torch.zeros(4, 5, device="cuda"), torch.zeros(6, 8, device="cuda"))
    with pytest.raises(ValueError):
        ctx.gemm(torch.zeros(4, 8), torch.zeros(4, 5), torch.zeros(5, 8))  # host tensors: no CPU path


# ---------------------------------------------------------------------------- bf16 tensor-core GEMM
@pytest.mark.parametrize("layout", ["nn", "nt"])
@pytest.mark.parametrize("shape,out", [((128, 256, 64), "bf16"), ((384, 768, 512), "bf16"), ((1000, 1000, 1000), "f32"), ((777, 1000, 520), "bf16"), ((130, 72, 64), "f32"), ((4096, 4096, 256), "bf16"), ((3900, 3848, 136), "bf16")])
def test_gemm_bf16_bias_relu(ctx, layout, shape, out):
    m, n, k = shape
    a, b, bias = I.gemm_bf16_normal(m, n, k, seed=m)
    a, b = a * 25, b * 25  # N(0, 0.5): keeps bf16 outputs well away from the subnormal range
    A, B, bv = I.to_np(a), I.to_np(b), I.to_np(bias)
    ref = R.gemm_epilogue(A, B, bias=bv, act="relu", out_dtype=out)
    bd = dev(b.t().contiguous()).t() if layout == "nt" else dev(b)
    d = torch.full((m, n), 7.0, device="cuda", dtype=torch.bfloat16 if out == "bf16" else torch.float32)
    ctx.gemm(d, dev(a), bd, bias=dev(bias), act=N.ACT_RELU)
    ctx.sync()
    assert_parity(host(d), ref, out)
    # the CUDA-core kernel must agree with the tensor-core kernel
    d2 = torch.empty_like(d)
    ctx.gemm(d2, dev(a), bd, bias=dev(bias), act=N.ACT_RELU, flags=N.GEMM_FORCE_SIMT)
    ctx.sync()
    assert_parity(host(d2), ref, out)


@pytest.mark.parametrize("act", ["none", "gelu", "gelu_tanh", "silu"])
@pytest.mark.parametrize("out", ["bf16", "f32"])
def test_gemm_bf16_full_epilogue(ctx, act, out):
    """acc = C + A.B + bias; act; + residual (in place over the residual buffer)."""
    m, n, k = 300, 520, 192
    a, b, bias = I.gemm_bf16_normal(m, n, k, seed=9)
    a, b = a * 25, b * 25
    tdt = torch.bfloat16 if out == "bf16" else torch.float32
    g = torch.Generator().manual_seed(1)
    c, res = torch.randn(m, n, generator=g).to(tdt), torch.randn(m, n, generator=g).to(tdt)
    ref = R.gemm_epilogue(I.to_np(a), I.to_np(b), c=I.to_np(c), bias=I.to_np(bias), act=act, residual=I.to_np(res), out_dtype=out)
    d = dev(res.clone())
    ctx.gemm(d, dev(a), dev(b), c=dev(c), bias=dev(bias), residual=d, act=ACT[act])
    ctx.sync()
    assert_parity(host(d), ref, out, tol=TOL_BF16 if out == "bf16" else 2e-5)


def test_gemm_swiglu_epilogue(ctx):
    from lighthouse_b200.workloads.decoder import pack_swiglu

    m, k, f = 200, 256, 512
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16)
    w1, w3 = (torch.randn(f, k, generator=g) * 0.1).to(torch.bfloat16), (torch.randn(f, k, generator=g) * 0.1).to(torch.bfloat16)
    ref = R.swiglu_gemm(I.to_np(x), I.to_np(w1), I.to_np(w3), "bf16")
    d = torch.empty(m, f, device="cuda", dtype=torch.bfloat16)
    ctx.gemm(d, dev(x), dev(pack_swiglu(w1, w3)).t(), flags=N.GEMM_SWIGLU)
    ctx.sync()
    assert_parity(host(d), ref, "bf16")


def test_gemm_config2_full_size_properties(ctx):
    """4096^3 bias + ReLU: sampled rows against the oracle, linearity in A, run-to-run
    bitwise determinism."""
    a, b, bias = I.gemm_bf16_normal(4096, 4096, 4096, seed=2)
    ad, bd, biasd = dev(a), dev(b), dev(bias)
    d = torch.empty(4096, 4096, device="cuda", dtype=torch.bfloat16)
    ctx.gemm(d, ad, bd, bias=biasd, act=N.ACT_RELU)
    ctx.sync()
    rows = [0, 1, 127, 128, 2049, 4095]
    ref = R.gemm_epilogue(I.to_np(a[rows]), I.to_np(b), bias=I.to_np(bias), act="relu", out_dtype="bf16")
    assert_parity(host(d[rows]), ref, "bf16")
    d2 = torch.empty_like(d)
    ctx.gemm(d2, ad, bd, bias=biasd, act=N.ACT_RELU)
    ctx.sync()
    assert torch.equal(d, d2)
    # linearity: (2A).B == 2 (A.B) exactly (scaling by 2 is exact in bf16 and f32)
    p1, p2 = torch.empty(4096, 4096, device="cuda"), torch.empty(4096, 4096, device="cuda")
    ctx.gemm(p1, ad, bd)
    ctx.gemm(p2, ad * 2, bd)
    ctx.sync()
    assert torch.equal(p1 * 2, p2)


def test_batched_gemm(ctx):
    g = torch.Generator().manual_seed(5)
    a = (torch.randn(3, 40, 24, generator=g)).to(torch.bfloat16)
    b = (torch.randn(3, 24, 56, generator=g)).to(torch.bfloat16)
    d = torch.empty(3, 40, 56, device="cuda")
    ctx.gemm(d, dev(a), dev(b))
    ctx.sync()
    assert_parity(host(d), np.einsum("bmk,bkn->bmn", I.to_np(a), I.to_np(b)), "f32")


def test_launch_overlap_gives_the_same_bits(ctx):
    """Programmatic dependent launches (opt-in): a chain of GEMMs each reading its predecessor's
    result, and an attention call behind them, must give bit for bit what ordinary launches
    give - every thread waits for the previous kernel before its first global access."""
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(512, 512, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w = [(torch.randn(512, 512, generator=g) * 0.05).to(torch.bfloat16).cuda() for _ in range(6)]
    q = torch.randn(1, 4, 512, 128, generator=g).to(torch.bfloat16).cuda()

    def run():
        a = x
        for wi in w:
            d = torch.empty(512, 512, device="cuda", dtype=torch.bfloat16)
            ctx.gemm(d, a, wi, act=N.ACT_GELU_ERF)
            a = d
        kv = a.view(1, 2, 256, 512)[:, :, :, :128].contiguous().expand(1, 2, 256, 128).repeat(1, 2, 2, 1).contiguous()
        o = torch.empty_like(q)
        ctx.attention_fwd(o, q, kv, kv, 128**-0.5, True)
        ctx.sync()
        return a.clone(), o.clone()

    plain = run()
    ctx.set_launch_overlap(True)
    try:
        for _ in range(3):
            got = run()
            assert torch.equal(got[0], plain[0]) and torch.equal(got[1], plain[1])
    finally:
        ctx.set_launch_overlap(False)


# --------------------------------------------------------------------------------- attention
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 1, 1, 128, 128, 128), (1, 2, 1, 256, 256, 128), (2, 4, 2, 384, 384, 128), (1, 2, 2, 200, 333, 64), (2, 3, 3, 77, 77, 64), (1, 4, 1, 130, 514, 128)])
def test_attention_bf16(ctx, shape, causal):
    b, hq, hkv, sq, skv, d = shape
    q, k, v = I.attention_qkv(b, hq, hkv, sq, skv, d, seed=sq + d)
    ref = R.attention(I.to_np(q), I.to_np(k), I.to_np(v), causal=causal, io_dtype="bf16")
    o = torch.full_like(q, 5.0).cuda()
    ctx.attention_fwd(o, dev(q), dev(k), dev(v), d**-0.5, causal)
    ctx.sync()
    assert_parity(host(o), ref, "bf16")


def test_attention_strided_views_and_f32_output(ctx):
    """q/k/v as head views of (tokens, 3C) rows — the layout the decoders use — no copies."""
    bsz, s, h, hs = 2, 160, 4, 64
    c = h * hs
    g = torch.Generator().manual_seed(6)
    qkv = torch.randn(bsz * s, 3 * c, generator=g).to(torch.bfloat16)
    qkv_d = dev(qkv)
    out = torch.zeros(bsz * s, c, device="cuda", dtype=torch.bfloat16)

    def heads(t, col0):
        return t[:, col0 : col0 + c].view(bsz, s, h, hs).permute(0, 2, 1, 3)

    ctx.attention_fwd(heads(out, 0), heads(qkv_d, 0), heads(qkv_d, c), heads(qkv_d, 2 * c), hs**-0.5, True)
    ctx.sync()
    ref = R.attention(I.to_np(heads(qkv, 0)), I.to_np(heads(qkv, c)), I.to_np(heads(qkv, 2 * c)), causal=True, io_dtype="bf16")
    assert_parity(host(heads(out, 0)), ref, "bf16")


def test_attention_f32_unfused_path(ctx):
    q, k, v = (t.float() for t in I.attention_qkv(2, 2, 2, 64, 96, 32, seed=8))
    o = torch.empty(2, 2, 64, 32, device="cuda")
    ctx.attention_fwd(o, dev(q), dev(k), dev(v), 32**-0.5, False)
    ctx.sync()
    assert_parity(host(o), R.attention_unfused_f32(I.to_np(q), I.to_np(k), I.to_np(v)), "f32")


def test_attention_config3_full_size_properties(ctx):
    """B8 H16 S2048 D128: one (batch, head) slice against the oracle; determinism; V-linearity
    (attention is linear in V: doubling V doubles O exactly)."""
    q, k, v = I.attention_qkv(8, 16, 16, 2048, 2048, 128, seed=3)
    qd, kd, vd = dev(q), dev(k), dev(v)
    for causal in (False, True):
        o = torch.empty_like(qd)
        ctx.attention_fwd(o, qd, kd, vd, 128**-0.5, causal)
        ctx.sync()
        ref = R.attention(I.to_np(q[3:4, 5:6]), I.to_np(k[3:4, 5:6]), I.to_np(v[3:4, 5:6]), causal=causal, io_dtype="bf16")
        assert_parity(host(o[3:4, 5:6]), ref, "bf16")
        o2 = torch.empty_like(qd)
        ctx.attention_fwd(o2, qd, kd, vd * 2, 128**-0.5, causal)
        ctx.sync()
        assert torch.equal(o * 2, o2)
        assert bool(torch.isfinite(o.float()).all())


@pytest.mark.parametrize("shape,out", [((1, 2, 2, 4096, 4096, 128), "bf16"), ((1, 4, 2, 2048, 2048, 128), "f32"), ((1, 3, 3, 1000, 1300, 64), "bf16"), ((2, 4, 1, 3000, 3000, 128), "bf16")])
def test_attention_causal_small_grid_splits_key_ranges(ctx, shape, out):
    """Causal problems with few (batch, head) pairs and long rows: the kernel spreads a pair of
    query tiles' key range over several work items and the last one to finish merges the
    partial (O, m, l). Same oracle and bound as the un-split kernel; a second call must give
    the same bits (the arrival counters are back at zero, the merge order does not depend on
    which item came last)."""
    b, hq, hkv, sq, skv, d = shape
    q, k, v = I.attention_qkv(b, hq, hkv, sq, skv, d, seed=sq + hq)
    ref = R.attention(I.to_np(q), I.to_np(k), I.to_np(v), causal=True, io_dtype="bf16")  # an f32 result only lacks the last rounding
    qd, kd, vd = dev(q), dev(k), dev(v)
    o = torch.full((b, hq, sq, d), 5.0, device="cuda", dtype=torch.bfloat16 if out == "bf16" else torch.float32)
    ctx.attention_fwd(o, qd, kd, vd, d**-0.5, True)
    ctx.sync()
    assert_parity(host(o), ref, "bf16")
    o2 = torch.zeros_like(o)
    ctx.attention_fwd(o2, qd, kd, vd, d**-0.5, True)
    ctx.sync()
    assert torch.equal(o, o2)


# ----------------------------------------------------------------------------------- row kernels
@pytest.mark.parametrize("rows,n,xdt,odt", [(1000, 768, "f32", "bf16"), (64, 768, "f32", "f32"), (33, 100, "f32", "f32"), (17, 4096, "bf16", "bf16"), (5, 5000, "f32", "f32")])
def test_layernorm(ctx, rows, n, xdt, odt):
    rng = np.random.RandomState(rows)
    x = R.round_to(rng.randn(rows, n).astype(np.float32) * 2 + 0.5, xdt)
    g, b = rng.randn(n).astype(np.float32), rng.randn(n).astype(np.float32)
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16}
    out = torch.empty(rows, n, device="cuda", dtype=tdt[odt])
    ctx.layernorm(out, dev(x, tdt[xdt]), dev(g), dev(b), 1e-5)
    ctx.sync()
    assert_parity(host(out), R.round_to(R.layernorm(x, g, b, 1e-5), odt), odt)


@pytest.mark.parametrize("rows,n", [(512, 4096), (7, 128), (3, 1000)])
def test_rmsnorm(ctx, rows, n):
    rng = np.random.RandomState(n)
    x = R.round_bf16(rng.randn(rows, n).astype(np.float32))
    w = R.round_bf16(rng.randn(n).astype(np.float32))
    out = torch.empty(rows, n, device="cuda", dtype=torch.bfloat16)
    ctx.rmsnorm(out, dev(x, torch.bfloat16), dev(w, torch.bfloat16), 1e-5)
    ctx.sync()
    assert_parity(host(out), R.rmsnorm(x, w, 1e-5, "bf16"), "bf16")
    out32 = torch.empty(rows, n, device="cuda")
    ctx.rmsnorm(out32, dev(x), None, 1e-5)
    ctx.sync()
    assert_parity(host(out32), R.rmsnorm(x, None, 1e-5, "f32"), "f32")


@pytest.mark.parametrize("rows,n", [(300, 1000), (64, 768), (2, 9000)])
def test_softmax(ctx, rows, n):
    x = np.random.RandomState(n).randn(rows, n).astype(np.float32) * 3
    out = torch.empty(rows, n, device="cuda")
    ctx.softmax(out, dev(x))
    ctx.sync()
    assert_parity(host(out), R.softmax(x), "f32")
    np.testing.assert_allclose(host(out).sum(-1), 1.0, rtol=1e-5)


def test_rope(ctx):
    x = R.round_bf16(np.random.RandomState(2).randn(2, 300, 5, 128).astype(np.float32))
    t = dev(x, torch.bfloat16)
    ctx.rope(t, 10000.0, 0)
    ctx.sync()
    assert_parity(host(t), R.rope(x, 10000.0, 0, "bf16"), "bf16")
    t32 = dev(x)
    ctx.rope(t32, 10000.0, 7)
    ctx.sync()
    assert_parity(host(t32), R.rope(x, 10000.0, 7, "f32"), "f32", tol=1e-4)  # angles up to ~300 rad in f32


def test_elementwise_family_and_embedding(ctx):
    rng = np.random.RandomState(4)
    a, b, bias = rng.randn(64, 256).astype(np.float32), rng.randn(64, 256).astype(np.float32), rng.randn(256).astype(np.float32)
    ad, bd, biasd = dev(a), dev(b), dev(bias)
    out = torch.empty(64, 256, device="cuda")
    cases = [
        (N.EW_ADD, (ad, bd), {}, a + b), (N.EW_MUL, (ad, bd), {}, a * b), (N.EW_SUB, (ad, bd), {}, a - b), (N.EW_MAX, (ad, bd), {}, np.maximum(a, b)),
        (N.EW_ADD_ACT, (ad, biasd), {"act": N.ACT_RELU}, np.maximum(a + bias, 0)), (N.EW_ACT, (ad,), {"act": N.ACT_GELU_ERF}, R.gelu_erf(a)),
        (N.EW_SILU_MUL, (ad, bd), {}, R.silu(a) * b), (N.EW_SCALE, (ad,), {"scalar": 0.125}, a * 0.125), (N.EW_FILL, (), {"scalar": 2.5}, np.full_like(a, 2.5)),
    ]
    for kind, ops, kw, ref in cases:
        ctx.elementwise(kind, out, *ops, **kw)
        ctx.sync()
        assert_parity(host(out), ref, "f32")
    # cast + transposing copy through strided views
    o16 = torch.empty(256, 64, device="cuda", dtype=torch.bfloat16)
    ctx.elementwise(N.EW_COPY, o16, ad.t())
    ctx.sync()
    assert np.array_equal(host(o16), R.round_bf16(a.T))
    ids = rng.randint(0, 50, size=(3, 16))
    wte, wpe = R.round_bf16(rng.randn(50, 32).astype(np.float32)), R.round_bf16(rng.randn(16, 32).astype(np.float32))
    emb = torch.empty(48, 32, device="cuda")
    ctx.embedding(emb, dev(ids.reshape(-1).astype(np.int32)), dev(wte, torch.bfloat16), dev(wpe, torch.bfloat16), 16)
    ctx.sync()
    assert max_rel_err(host(emb), R.embed(ids, wte, wpe)) <= 1e-6


def test_launch_counter_and_status_word(ctx):
    before = ctx.launch_count
    t = torch.zeros(8, 8, device="cuda")
    ctx.elementwise(N.EW_FILL, t, scalar=1.0)
    ctx.sync()  # also reads the device status word: no bounded wait ran out
    assert ctx.launch_count == before + 1 and float(t.sum()) == 64.0


def test_bounded_wait_gives_up_and_the_context_survives(own_stream_ctx):
    """The give-up path of the device-side waits, exercised in its harmless form: waits on an
    mbarrier and on a local flag that nothing will ever satisfy, with a 1 ms limit. The kernel
    returns by itself, the next sync reports a device error once, and the same context then
    runs a GEMM correctly."""
    c = own_stream_ctx
    assert c.selftest_bounded_wait(1_000_000) == 64
    with pytest.raises(N.LighthouseCudaError, match="bounded wait"):
        c.sync()
    c.sync()  # the status word was cleared: no second report
    a, b, _ = I.gemm_bf16_normal(128, 128, 64, seed=3)
    a, b = a * 25, b * 25
    ad, bd = dev(a), dev(b)
    d = torch.empty(128, 128, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    c.gemm(d, ad, bd)
    c.sync()
    assert_parity(host(d), R.gemm_epilogue(I.to_np(a), I.to_np(b), out_dtype="bf16"), "bf16")
    with pytest.raises(ValueError):
        c.selftest_bounded_wait(10**12)  # limits beyond 100 ms are refused


def test_own_stream_mode_with_explicit_synchronisation(own_stream_ctx):
    """A context on its own non-blocking stream is ordered with torch by synchronising: torch's
    stream before the call (operands and the result buffer's fill are complete), the
    context's after it."""
    c = own_stream_ctx
    a, b, bias = I.gemm_bf16_normal(256, 384, 128, seed=17)
    a, b = a * 25, b * 25
    ad, bd, biasd = dev(a), dev(b), dev(bias)
    d = torch.full((256, 384), float("nan"), device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    c.gemm(d, ad, bd, bias=biasd, act=N.ACT_RELU)
    c.sync()
    assert_parity(host(d), R.gemm_epilogue(I.to_np(a), I.to_np(b), bias=I.to_np(bias), act="relu", out_dtype="bf16"), "bf16")


def test_side_stream_events_and_collectives_of_one_rank(ctx):
    """The two-stream mechanism the overlapped schedules use: work on the side stream starts
    after the main stream's record and the main stream resumes after the side stream's."""
    a = torch.ones(1 << 22, device="cuda")
    b, c = torch.zeros_like(a), torch.zeros_like(a)
    torch.cuda.synchronize()
    ctx.reserve_sms(8)
    ctx.elementwise(N.EW_SCALE, b, a, scalar=2.0)  # main: b = 2
    ctx.event_record(0)
    ctx.stream_select(1)
    ctx.event_wait(0)
    ctx.elementwise(N.EW_SCALE, c, b, scalar=3.0)  # side: c = 6
    ctx.event_record(1)
    ctx.stream_select(0)
    ctx.event_wait(1)
    ctx.elementwise(N.EW_ADD, a, c, b)  # main: a = 8
    ctx.reserve_sms(0)
    ctx.sync()
    assert float(a.min()) == 8.0 and float(a.max()) == 8.0
    # a single rank's collectives are copies (or nothing, in place)
    src = torch.arange(1024, device="cuda", dtype=torch.float32)
    dst = torch.zeros_like(src)
    ctx.reducescatter(dst, src)
    ctx.allgather(src, dst)
    ctx.allreduce(dst)
    ctx.sync()
    assert torch.equal(dst, src)
    with pytest.raises(ValueError):
        ctx.event_wait(77)  # never recorded
    with pytest.raises(ValueError):
        ctx.reserve_sms(10**6)


@pytest.mark.parametrize("m,n,k,cols,hd,seq", [(256, 768, 512, 640, 128, 128), (384, 320, 256, 256, 64, 96), (64, 48, 32, 32, 16, 32)])
def test_gemm_with_rotary_epilogue(ctx, m, n, k, cols, hd, seq):
    """Projection + rotary embedding of its leading columns in one call: the tensor-core
    epilogue (head sizes that are multiples of 64) and the two-kernel form (the rest) against
    the oracle's product -> round -> rotate."""
    rng = np.random.RandomState(m + n)
    a, b = R.round_bf16(rng.randn(m, k).astype(np.float32) * 0.5), R.round_bf16(rng.randn(k, n).astype(np.float32) * 0.2)
    d = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    ctx.gemm_rope(d, dev(a, torch.bfloat16), dev(b, torch.bfloat16), cols, hd, seq, 10000.0, 3)
    ctx.sync()
    want = R.round_bf16(a @ b)
    want[:, :cols] = R.rope(want[:, :cols].reshape(m // seq, seq, cols // hd, hd), 10000.0, 3, "bf16").reshape(m, cols)
    assert_parity(host(d), want, "bf16")
    # untouched columns are the plain product
    plain = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    ctx.gemm(plain, dev(a, torch.bfloat16), dev(b, torch.bfloat16))
    ctx.sync()
    assert torch.equal(plain[:, cols:], d[:, cols:])
    with pytest.raises(ValueError):
        ctx.gemm_rope(d, dev(a, torch.bfloat16), dev(b, torch.bfloat16), cols + 1, hd, seq)
