"""Host logic of the payload layer: MLIR text reader, printer round trip, recognition and
fusion. Plans are executed on the CPU with the oracle's arithmetic (tests/cpu_plan.py) and
compared with the oracle applied directly to the same inputs."""

import numpy as np
import pytest

from cpu_plan import CpuPlanRunner
from oracle import inputs as I
from oracle import reference_ops as R
from oracle.check import max_rel_err

from lighthouse_b200.payload import UnsupportedPayload, as_payload_module, parse_mlir
from lighthouse_b200.payload import generators as G


def plan_of(module, name="payload", **kw):
    pm = as_payload_module(str(module), lower=False)
    from lighthouse_b200.payload.lower import recognize

    return recognize(pm.funcs[name], **kw)


def rnd(shape, dtype="f32", seed=0, scale=1.0):
    x = (np.random.RandomState(seed).randn(*shape) * scale).astype(np.float32)
    return R.round_to(x, dtype)


# ----------------------------------------------------------------------------- reader / printer
def test_print_parse_round_trip_is_stable():
    mods = [
        G.generate_gpu_matmul_payload("payload", 64, 48, 32, "bf16", "f32", True, True, True, True, True, result_type="bf16"),
        G.generate_gpu_attention_payload("payload", 2, 3, 32, 16, "f32"),
        G.generate_gpu_layer_norm_payload("payload", 8, 32, "f32"),
        G.generate_gpu_softmax_payload("payload", 8, 32, "f32"),
        G.build_gpt_fused_payload("payload", 32, 32, 128, 64, 2, 4)[0],
    ]
    for m in mods:
        text = str(m)
        again = str(parse_mlir(text))
        assert again == text


REFERENCE_STYLE_TEXT = """
#map = affine_map<(d0, d1, d2) -> (d0, d2)>
#map1 = affine_map<(d0, d1, d2) -> (d2, d1)>
#map2 = affine_map<(d0, d1, d2) -> (d0, d1)>
#map3 = affine_map<(d0, d1) -> (d1)>
#map4 = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @entry(%arg0: tensor<24x40xf32>, %arg1: tensor<40x56xf32>, %arg2: tensor<56xf32>, %arg3: tensor<24x56xf32>) -> tensor<24x56xf32> {
    // matmul, bias add and ReLU written as generics, the results threaded through outs
    %0 = linalg.generic {indexing_maps = [#map, #map1, #map2], iterator_types = ["parallel", "parallel", "reduction"]} ins(%arg0, %arg1 : tensor<24x40xf32>, tensor<40x56xf32>) outs(%arg3 : tensor<24x56xf32>) {
    ^bb0(%in: f32, %in_2: f32, %out: f32):
      %9 = arith.mulf %in, %in_2 : f32
      %10 = arith.addf %9, %out : f32
      linalg.yield %10 : f32
    } -> tensor<24x56xf32>
    %1 = linalg.generic {indexing_maps = [#map3, #map4], iterator_types = ["parallel", "parallel"]} ins(%arg2 : tensor<56xf32>) outs(%0 : tensor<24x56xf32>) {
    ^bb0(%in: f32, %out: f32):
      %9 = arith.addf %in, %out : f32
      linalg.yield %9 : f32
    } -> tensor<24x56xf32>
    %cst = arith.constant 0.000000e+00 : f32
    %2 = linalg.generic {indexing_maps = [#map4], iterator_types = ["parallel", "parallel"]} outs(%1 : tensor<24x56xf32>) {
    ^bb0(%out: f32):
      %9 = arith.cmpf ugt, %out, %cst : f32
      %10 = arith.select %9, %out, %cst : f32
      linalg.yield %10 : f32
    } -> tensor<24x56xf32>
    return %2 : tensor<24x56xf32>
  }
}
"""


def test_generic_form_matmul_bias_relu_is_recognised():
    """Ops written as linalg.generic with affine-map aliases, ``outs`` used as an input, and
    ReLU as cmpf/select — the textual style of the reference's own test payloads."""
    pm = as_payload_module(REFERENCE_STYLE_TEXT)
    plan = pm.plans["entry"]
    a, b, bias, c = rnd((24, 40), seed=1), rnd((40, 56), seed=2), rnd((56,), seed=3), rnd((24, 56), seed=4)
    out = CpuPlanRunner(plan).run([a, b, bias, c])[3]
    want = np.maximum(a @ b + c + bias, 0.0)
    assert max_rel_err(out, want) < 1e-6
    # the three in-place generics (the form of test/opt/pipeline-check.mlir:21-47 in the
    # reference) become ONE operator: a GEMM accumulating into its output with bias and ReLU
    # in its epilogue
    assert [op.kind for op in plan.ops] == ["gemm"]
    assert plan.ops[0].operands[4] is not None and plan.ops[0].attrs["act"] == "relu"


def test_unsupported_payloads_raise_value_error():
    with pytest.raises(ValueError):
        parse_mlir("module {\n func.func @f(%a: tensor<4xf32>) {\n %0 = foo.bar %a : tensor<4xf32>\n return\n }\n}")
    with pytest.raises(ValueError):
        parse_mlir("module {\n func.func @f(%a: tensor<?x4xf32>) {\n return\n }\n}")
    with pytest.raises(ValueError):
        parse_mlir("")
    bad = "module {\n func.func @f(%a: tensor<4x4xf32>, %o: tensor<4x4xf32>) {\n %0 = linalg.softmax dimension(0) ins(%a : tensor<4x4xf32>) outs(%o : tensor<4x4xf32>) -> tensor<4x4xf32>\n return\n }\n}"
    with pytest.raises(UnsupportedPayload):
        as_payload_module(bad)


# ------------------------------------------------------------------------------------ matmul / MLP
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("bias,relu,acc,rt", [(False, False, False, None), (True, True, False, "bf16"), (True, False, True, None), (False, True, True, "bf16")])
def test_matmul_payload_plan_matches_oracle(ta, tb, bias, relu, acc, rt):
    M, N, K = 40, 24, 56
    m = G.generate_gpu_matmul_payload("payload", M, N, K, "bf16", "f32", ta, tb, bias, relu, acc, result_type=rt)
    out_dt = rt or "f32"
    a = rnd((K, M) if ta else (M, K), "bf16", 1, 0.5)
    b = rnd((N, K) if tb else (K, N), "bf16", 2, 0.5)
    c = rnd((M, N), out_dt, 3)
    bv = rnd((N,), out_dt, 4)
    args = [c.copy(), a, b] + ([bv] if bias else [])
    want = R.gemm_epilogue(a, b, c=c if acc else None, bias=bv if bias else None, act="relu" if relu else "none", out_dtype=out_dt, transpose_a=ta, transpose_b=tb)
    for fuse in (True, False):
        plan = plan_of(m, fuse=fuse)
        got = CpuPlanRunner(plan).run([x.copy() for x in args])[0]
        assert max_rel_err(got, want) <= (1e-2 if out_dt == "bf16" else 1e-6), (fuse, str(plan))
    fused = plan_of(m)
    if not acc:
        assert [op.kind for op in fused.ops] == ["gemm"], str(fused)


def test_mlp_payload_chains_layers_on_device():
    m = G.generate_gpu_mlp_payload("payload", 16, 32, 8, [64, 48], "bf16", "f32", "f32", "f32", False, False, True, True, False)
    plan = plan_of(m)
    assert [op.kind for op in plan.ops] == ["gemm", "gemm", "gemm"]
    assert [op.attrs["act"] for op in plan.ops] == ["relu", "relu", "none"]
    x, w0, w1, w2 = rnd((16, 32), "bf16", 1), rnd((32, 64), "bf16", 2, 0.2), rnd((64, 48), "bf16", 3, 0.2), rnd((48, 8), "bf16", 4, 0.2)
    b0, b1, b2 = rnd((64,), seed=5), rnd((48,), seed=6), rnd((8,), seed=7)
    got = CpuPlanRunner(plan).run([np.zeros((16, 8), np.float32), x, w0, w1, w2, b0, b1, b2])[0]
    h = R.gemm_epilogue(x, w0, bias=b0, act="relu", out_dtype="bf16")
    h = R.gemm_epilogue(h, w1, bias=b1, act="relu", out_dtype="bf16")
    assert max_rel_err(got, R.gemm_epilogue(h, w2, bias=b2)) < 1e-6


def test_lh_run_style_tensor_matmul_accumulates_in_place():
    plan = plan_of(G.generate_matmul_tensor_payload("main", 16, 32, 64), "main")
    assert len(plan.ops) == 1 and plan.ops[0].operands[3] == plan.ops[0].operands[0]
    a, b, c = I.lh_run_args("16x64xf32xrnd,64x32xf32x1,16x32xf32x0", 123)
    got = CpuPlanRunner(plan).run([a, b, c])[2]
    assert got[0, 0] == pytest.approx(32.873924, rel=1e-6)


# -------------------------------------------------------------------------- attention / norms
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_attention_payload_fuses_to_one_operator(dtype):
    Z, H, S, D = 2, 3, 40, 16
    m = G.generate_gpu_attention_payload("payload", Z, H, S, D, dtype)
    plan = plan_of(m)
    assert [op.kind for op in plan.ops] == ["attention"] and not plan.temp_bytes
    unfused = plan_of(m, fuse_attention_pattern=False)
    assert [op.kind for op in unfused.ops] == ["gemm", "elementwise", "softmax", "gemm"]
    q, k, v = (rnd((Z, H, S, D), dtype, s) for s in (1, 2, 3))
    want = R.attention(q, k, v, io_dtype=dtype)
    got = CpuPlanRunner(plan).run([np.zeros_like(q), q, k, v])[0]
    assert max_rel_err(got, want) < 1e-6
    got_unfused = CpuPlanRunner(unfused).run([np.zeros_like(q), q, k, v])[0]
    assert max_rel_err(got_unfused, want) < (3e-2 if dtype == "bf16" else 1e-5)


def test_layer_norm_and_softmax_payloads():
    x, g, b = rnd((12, 64), seed=1), rnd((64,), seed=2), rnd((64,), seed=3)
    plan = plan_of(G.generate_gpu_layer_norm_payload("payload", 12, 64, "f32", eps=1e-4))
    assert [op.kind for op in plan.ops] == ["layernorm"] and plan.ops[0].attrs["eps"] == pytest.approx(1e-4)
    got = CpuPlanRunner(plan).run([np.zeros_like(x), x, g, b])[0]
    assert max_rel_err(got, R.layernorm(x, g, b, 1e-4)) < 1e-6
    plan = plan_of(G.generate_gpu_softmax_payload("payload", 12, 64, "f32"))
    assert [op.kind for op in plan.ops] == ["softmax"]
    assert max_rel_err(CpuPlanRunner(plan).run([np.zeros_like(x), x])[0], R.softmax(x)) < 1e-6


def test_nanogpt_payload_recognition_and_numerics():
    T, C, hidden, vocab, L, H = 32, 32, 128, 64, 2, 4
    mod, kinds = G.build_gpt_fused_payload("payload", T, C, hidden, vocab, L, H, lowp="bf16")
    assert kinds.count("fa") == L and kinds.count("ln") == 2 * L + 1
    plan = plan_of(mod)
    # per block: ln, q, k, v, attention, proj, ln, fc1, fc2; then ln_f and lm_head
    assert [op.kind for op in plan.ops] == (["layernorm", "gemm", "gemm", "gemm", "attention", "gemm", "layernorm", "gemm", "gemm"] * L + ["layernorm", "gemm"])
    w = I.tree_to_np(I.nanogpt_weights(L, C, hidden, vocab, T, seed=9, std=0.2))
    x = rnd((T, C), seed=10, scale=0.5)
    args = [np.zeros((T, vocab), np.float32), x]
    for lw in w["layers"]:
        args += [lw[k] for k in G.GPT_LAYER_KEYS]
    args += [w["gf_g"], w["gf_b"], w["lmw"], w["lmb"]]
    got = CpuPlanRunner(plan).run(args)[0]
    want = R.nanogpt_forward(x, w["layers"], w["gf_g"], w["gf_b"], w["lmw"], w["lmb"], H, act="relu", causal=False, lowp="bf16")
    assert max_rel_err(got, want) < 2e-2
    # without fusion the same payload is one operator per payload op, same result
    unfused = plan_of(mod, fuse=False)
    assert len(unfused.ops) > len(plan.ops)
    assert max_rel_err(CpuPlanRunner(unfused).run(args)[0], want) < 3e-2
