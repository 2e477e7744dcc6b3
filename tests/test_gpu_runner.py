"""The reference-facing surface on a GPU: ``Runner.execute / benchmark`` with the three
argument modes (host numpy, device clones, torch pass-through), ``lh-run`` with the
reference's known-answer vector, and payload modules from the generators end to end."""

import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, PAYLOADS
from oracle import inputs as I
from oracle import reference_ops as R
from oracle.check import TOL_BF16, TOL_F32, max_rel_err, assert_parity

from lighthouse_b200.execution import GPUMemoryManager, Runner, TorchCudaMemoryManager
from lighthouse_b200.payload import generators as G
from lighthouse_b200.pipeline import CompilerDriver
from lighthouse_b200.utils.numpy import mlir_to_numpy_dtype
from lighthouse_b200.workloads.matmul import CudaMatMul

pytestmark = pytest.mark.gpu

MATMUL = os.path.join(PAYLOADS, "matmul_16x32x64_f32.mlir")


def as_np(x, dtype):
    return np.asarray(x, dtype=np.float32).astype(mlir_to_numpy_dtype(dtype))


def test_lh_run_reproduces_the_reference_known_answer(capsys):
    """`lh-run --seed=123 --print-tensor=3` on the 16x64 rnd @ 64x32 ones payload prints the
    16 row values the reference's test checks."""
    from lighthouse_b200 import lh_run

    with open(os.path.join(GOLDEN, "lh_run_pipeline_check.json")) as f:
        g = json.load(f)
    rc = lh_run.main([MATMUL, "--stage", "cuda/matmul/f32.yaml", "--entry-point", g["entry_point"], "--input-shape", g["input_shape"],
                      "--print-tensor", str(g["print_tensor"]), "--seed", str(g["seed"])])
    out = capsys.readouterr().out
    assert rc == 0 and out.startswith("Output: [[")
    import re

    first_of_row = [float(m) for m in re.findall(r"\[\s*([0-9]+\.[0-9]+)", out)]
    assert first_of_row == pytest.approx(g["row_values"], rel=1e-7), out[:400]  # same digits the reference's CHECK lines hold
    rc = lh_run.main([MATMUL, "--stage", "cuda/matmul/f32.yaml", "--entry-point", "main", "--input-shape", g["input_shape"], "--benchmark"])
    assert rc == 0 and "100 runs: " in capsys.readouterr().out


def test_runner_host_arrays_are_updated_in_place(ctx):
    a, b, c = I.lh_run_args("16x64xf32xrnd,64x32xf32x1,16x32xf32x0", 123)
    runner = Runner(CompilerDriver(MATMUL, stages=["cuda-dispatch.yaml"]).run(), context=ctx)
    runner.execute("main", [a, b, c])
    assert c[0, 0] == pytest.approx(32.873924, rel=1e-6) and c[15, 31] == pytest.approx(26.437485, rel=1e-6)
    with pytest.raises(ValueError):
        runner.execute("nope", [a, b, c])
    with pytest.raises(ValueError):
        runner.execute("main", [a, b])
    with pytest.raises(ValueError):
        runner.execute("main", [a, b, c[:8]])
    with pytest.raises(ValueError):
        runner.execute("main", [a, b, torch.zeros(16, 32)])  # non-numpy without a memory manager
    runner.close()


def test_runner_gpu_memory_manager_and_callback(ctx):
    """The reference's GPU flow: clone host buffers, run, read argument 0 back in a callback."""
    wl = CudaMatMul(M=256, N=384, K=128, ab_type="bf16", c_type="f32", has_bias=True, has_relu=True, accumulate_c=False, truncate_c=True)
    C, A, B, bias = wl.get_input_arrays()
    runner = Runner(wl.payload_module(), mem_manager_cls=GPUMemoryManager, context=ctx)
    out = np.zeros_like(C)
    runner.execute("payload", [C, A, B, bias], Runner.get_gpu_argument_access_callback(out, arg_index=0))
    f = lambda x: np.asarray(x, dtype=np.float32)
    ref = R.gemm_epilogue(f(A), f(B), bias=f(bias), act="relu", out_dtype="bf16")
    assert_parity(f(out), ref, "bf16")
    times = runner.benchmark([C, A, B, bias], nruns=7, nwarmup=2)
    assert times.shape == (7,) and times.dtype == np.float64 and np.all(times > 0) and np.all(times < 1.0)
    flops, reads, writes = wl.get_complexity()
    assert flops == 2 * 256 * 384 * 128 + 2 * 256 * 384
    runner.close()


@pytest.mark.parametrize("transpose_b,accumulate_c,hidden", [(False, False, [384, 640]), (True, False, [384, 640]), (False, True, []), (True, True, [])])
def test_mlp_payload_three_layers_through_runner(ctx, transpose_b, accumulate_c, hidden):
    """The chained MLP payload (generate_gpu_mlp_payload of the reference,
    lighthouse/ingress/mlir_gen/gpu_mlp_payload.py:10-107: three layers, bias, ReLU between
    layers, hidden activations never leaving the device) through the Runner with
    GPUMemoryManager, checked the way examples/xegpu/mlp.py:47-101 checks it: every layer's
    result truncated to the operand type, ReLU on all but the last. ``accumulate_c`` is run
    on the single-layer form: with hidden layers the reference's payload accumulates those
    into a ``tensor.empty`` (gpu_mlp_payload.py:83-88), whose content is undefined; this
    backend refuses that payload with a ValueError instead of reading uninitialised memory."""
    from lighthouse_b200.payload import generators as G
    from lighthouse_b200.utils.numpy import mlir_to_numpy_dtype

    batch, sizes = 256, [512] + hidden + [128]
    nl = len(sizes) - 1
    m = G.generate_gpu_mlp_payload("payload", batch, sizes[0], sizes[-1], sizes[1:-1], "bf16", "f32", "bf16", "bf16", False, transpose_b, True, True, accumulate_c)
    if accumulate_c:
        with pytest.raises(ValueError, match="uninitialised"):
            Runner(G.generate_gpu_mlp_payload("payload", batch, 512, 128, [384], "bf16", "f32", "bf16", "bf16", False, transpose_b, True, True, True), context=ctx)
    bf16 = mlir_to_numpy_dtype("bf16")
    rng = np.random.RandomState(11)
    x = (rng.rand(batch, sizes[0]) - 0.5).astype(bf16)
    ws = [(rng.rand(sizes[i], sizes[i + 1]) - 0.5).astype(bf16) for i in range(nl)]
    bs = [(rng.rand(sizes[i + 1]) - 0.5).astype(bf16) for i in range(nl)]
    c0 = (rng.rand(batch, sizes[-1]) - 0.5).astype(bf16) if accumulate_c else np.zeros((batch, sizes[-1]), bf16)
    host_ws = [np.ascontiguousarray(w.T) for w in ws] if transpose_b else ws
    out = np.zeros_like(c0)
    runner = Runner(m, mem_manager_cls=GPUMemoryManager, context=ctx)
    plan = runner.payload.plans["payload"]
    launches = ctx.launch_count
    runner.execute("payload", [c0, x] + host_ws + bs, Runner.get_gpu_argument_access_callback(out))
    if not accumulate_c:
        # one kernel per layer with its epilogue fused; hidden activations are device temporaries
        assert [op.kind for op in plan.ops] == ["gemm"] * nl
        assert ctx.launch_count - launches == nl
    f = lambda a: np.asarray(a, dtype=np.float32)
    h = f(x)
    for i in range(nl):
        h = R.gemm_epilogue(h, f(ws[i]), c=f(c0) if (accumulate_c and i == nl - 1) else None, bias=f(bs[i]), act="relu" if i < nl - 1 else "none", out_dtype="bf16")
    assert_parity(f(out), h, "bf16")
    runner.close()


@pytest.mark.parametrize("init_int", [True, False])
def test_matmul_example_defaults_accumulate_c(ctx, init_int):
    """The reference example's default: accumulate into a random C (exact with integer inputs)."""
    wl = CudaMatMul(M=128, N=256, K=192, ab_type="bf16", c_type="f32")
    C, A, B = wl.get_input_arrays(init_int=init_int)
    runner = Runner(wl.payload_module(), mem_manager_cls=GPUMemoryManager, context=ctx)
    out = np.zeros_like(C)
    runner.execute("payload", [C, A, B], Runner.get_gpu_argument_access_callback(out))
    f = lambda x: np.asarray(x, dtype=np.float32)
    ref = R.gemm_epilogue(f(A), f(B), c=f(C))
    if init_int:
        assert np.array_equal(out, ref)
    else:
        assert_parity(out, ref, "f32")
    runner.close()


def test_runner_torch_pass_through(ctx):
    """ExternalMemoryManager protocol: CUDA tensors in, results in place, no copies."""
    mod = G.generate_gpu_attention_payload("payload", 2, 4, 256, 64, "bf16")
    q, k, v = I.attention_qkv(2, 4, 4, 256, 256, 64, seed=5)
    o = torch.zeros_like(q).cuda()
    runner = Runner(mod, mem_manager_cls=TorchCudaMemoryManager, context=ctx)
    seen = {}
    runner.execute("payload", [o, q.cuda(), k.cuda(), v.cuda()], lambda inputs, **kw: seen.update(kw, n=len(inputs)))
    assert seen["n"] == 4 and seen["memory_manager"] is not None and seen["execution_engine"] is ctx
    ref = R.attention(I.to_np(q), I.to_np(k), I.to_np(v), io_dtype="bf16")
    assert_parity(o.float().cpu().numpy(), ref, "bf16")
    with pytest.raises(ValueError):
        runner.execute("payload", [o.cpu(), q, k, v])
    runner.close()


def test_generated_payloads_through_text(ctx):
    """Payloads printed as MLIR text, parsed back, recognised and run: layer norm, softmax,
    f32 attention (unfused op sequence), transposed operands."""
    rng = np.random.RandomState(0)
    x, g, b = rng.randn(96, 768).astype(np.float32), rng.randn(768).astype(np.float32), rng.randn(768).astype(np.float32)
    out = np.zeros_like(x)
    r = Runner(str(G.generate_gpu_layer_norm_payload("payload", 96, 768, "f32")), context=ctx)
    r.execute("payload", [out, x, g, b])
    assert_parity(out, R.layernorm(x, g, b), "f32")
    r.close()
    r = Runner(str(G.generate_gpu_softmax_payload("payload", 96, 768, "f32")), context=ctx)
    r.execute("payload", [out, x])
    assert_parity(out, R.softmax(x), "f32")
    r.close()
    q, k, v = (rng.randn(2, 2, 48, 32).astype(np.float32) for _ in range(3))
    o = np.zeros_like(q)
    r = Runner(str(G.generate_gpu_attention_payload("payload", 2, 2, 48, 32, "f32")), context=ctx)
    r.execute("payload", [o, q, k, v])
    assert_parity(o, R.attention_unfused_f32(q, k, v), "f32")
    r.close()
    wl = CudaMatMul(M=128, N=64, K=256, ab_type="bf16", c_type="f32", accumulate_c=False, transpose_a=True, transpose_b=True, has_relu=True)
    C, A, B = wl.get_input_arrays()
    r = Runner(str(wl.payload_module()), context=ctx)
    r.execute("payload", [C, A, B])
    f = lambda t: np.asarray(t, dtype=np.float32)
    assert_parity(C, R.gemm_epilogue(f(A), f(B), act="relu", transpose_a=True, transpose_b=True), "f32")
    r.close()


def test_fused_and_unfused_pipelines_agree(ctx):
    wl = CudaMatMul(M=256, N=256, K=256, ab_type="bf16", c_type="f32", has_bias=True, has_relu=True, accumulate_c=False, truncate_c=True)
    C, A, B, bias = wl.get_input_arrays()
    path = os.path.join(PAYLOADS, "_tmp_matmul.mlir")
    outs = []
    try:
        with open(path, "w") as fh:
            fh.write(str(wl.payload_module()))
        for stage in ("cuda-dispatch.yaml", "cuda-unfused.yaml", "cuda-staged.yaml"):
            mod = CompilerDriver(path, stages=[stage]).run()
            out = C.copy()
            r = Runner(mod, context=ctx)
            r.execute("payload", [out, A, B, bias])
            outs.append((len(mod.plans["payload"].ops), np.asarray(out, dtype=np.float32)))
            r.close()
    finally:
        os.remove(path)
    assert outs[0][0] == 1 and outs[1][0] > 1 and outs[2][0] == 1
    assert np.array_equal(outs[0][1], outs[2][1])
    assert_parity(outs[1][1], outs[0][1], "bf16")


def test_nanogpt_payload_module_end_to_end(ctx):
    """The reference's nanoGPT example shape (T = C = 256, 4 heads, ReLU, non-causal) through
    payload -> text -> recognise -> GPU, against its numpy reference restated in the oracle."""
    T, C, hidden, vocab, L, H = 256, 256, 1024, 256, 2, 4
    mod, kinds = G.build_gpt_fused_payload("payload", T, C, hidden, vocab, L, H, lowp="bf16")
    w = I.nanogpt_weights(L, C, hidden, vocab, T, seed=0, std=0.05)
    wn = I.tree_to_np(w)
    x = (np.random.RandomState(0).randn(T, C) * 0.5).astype(np.float32)
    out = np.zeros((T, vocab), np.float32)
    host = [out, x]
    for lw in w["layers"]:
        host += [as_np(I.to_np(lw[k]), "bf16" if lw[k].dtype == torch.bfloat16 else "f32") for k in G.GPT_LAYER_KEYS]
    host += [as_np(I.to_np(w["gf_g"]), "f32"), as_np(I.to_np(w["gf_b"]), "f32"), as_np(I.to_np(w["lmw"]), "bf16"), as_np(I.to_np(w["lmb"]), "f32")]
    runner = Runner(str(mod), mem_manager_cls=GPUMemoryManager, context=ctx)
    runner.execute("payload", host, Runner.get_gpu_argument_access_callback(out, 0))
    ref = R.nanogpt_forward(x, wn["layers"], wn["gf_g"], wn["gf_b"], wn["lmw"], wn["lmb"], H, act="relu", causal=False, lowp="bf16")
    rel = np.abs(out - ref).max() / (np.abs(ref).max() + 1e-6)
    assert rel < TOL_BF16  # the reference's own criterion is rel < 5e-2
    runner.close()
