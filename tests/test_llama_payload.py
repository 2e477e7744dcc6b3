"""The Llama block as MLIR payloads (lighthouse_b200/payload/llama_gen.py: the linalg builders
of the reference's examples/llama/test_llama3.py): printed, parsed back, recognised, and run.

Ground truth is what the reference's own tests compare those builders with - the torch model
run with a real frequency table and an additive mask (tests/golden/llama_linalg_ref.npz, made
by tests/golden/make_golden.py::golden_llama_linalg) - at the tolerance those tests use
(rtol = atol = 0.01, test_llama3.py:1651,1812,1985) and at this repository's f32 bound.
On the CPU the plans are executed by the plan interpreter with the oracle's arithmetic; the
``gpu`` tests run them through the Runner on the CUDA kernels."""

import os

import numpy as np
import pytest

from conftest import GOLDEN
from cpu_plan import CpuPlanRunner
from oracle import reference_ops as R
from oracle.check import assert_parity, max_rel_err

from lighthouse_b200.payload import as_payload_module
from lighthouse_b200.payload.llama_gen import LAYER_ARG_NAMES, generate_llama_attention_payload, generate_llama_transformer_payload, llama_hidden_dim
from lighthouse_b200.payload.parser import parse_mlir


@pytest.fixture(scope="module")
def g():
    return np.load(os.path.join(GOLDEN, "llama_linalg_ref.npz"))


def meta(g):
    return tuple(int(v) for v in g["meta"])  # dim, layers, heads, kv heads, batch, seq, hidden


def layer_args(g, i):
    dim, _, _, _, _, _, hidden = meta(g)
    w = {k: g[f"l{i}_{k}"] for k in ("wq", "wk", "wv", "wo", "w1", "w2", "w3")}
    w.update(b1=np.zeros(hidden, np.float32), b2=np.zeros(dim, np.float32), b3=np.zeros(hidden, np.float32))  # the torch model has no biases
    return [w[n] for n in LAYER_ARG_NAMES]


def transformer_args(g, n_layers, mask):
    dim, _, _, _, B, S, _ = meta(g)
    args = [np.zeros((B, S, dim), np.float32), g["x"], g["freqs_real"]] + ([g["mask"]] if mask == "operand" else [])
    for i in range(n_layers):
        args += layer_args(g, i)
    return args


def test_payload_text_round_trips_and_uses_the_builders_ops(g):
    dim, nl, nh, nkv, B, S, hidden = meta(g)
    assert hidden == llama_hidden_dim(dim, 16)
    text = str(generate_llama_transformer_payload("payload", B, S, dim, nh, nkv, hidden, nl))
    assert str(parse_mlir(text)) == text
    for needle in ("linalg.contract indexing_maps", "kind=#linalg.elementwise_kind<rsqrt>", "floordiv 2", "complex.mul", "complex.create", "linalg.softmax dimension(3)", "-> (d0, d1, 0)>"):
        assert needle in text, needle


@pytest.mark.parametrize("mask", ["operand", "causal"])
def test_attention_block_and_transformer_plans_match_the_reference_ground_truth(g, mask):
    dim, nl, nh, nkv, B, S, hidden = meta(g)
    l0 = {k: g[f"l0_{k}"] for k in ("wq", "wk", "wv", "wo")}
    plan = as_payload_module(str(generate_llama_attention_payload("payload", B, S, dim, nh, nkv, mask=mask))).plans["payload"]
    args = [np.zeros((B, S, dim), np.float32), g["x"], l0["wq"], l0["wk"], l0["wv"], l0["wo"], g["freqs_real"]] + ([g["mask"]] if mask == "operand" else [])
    out = CpuPlanRunner(plan).run(args)[0]
    assert max_rel_err(out, g["attn_out"]) < 1e-5
    # a mask built in the payload is provably causal: flash attention with the kv heads read in
    # place; a mask operand's values are unknown: the builders' own un-fused sequence
    assert plan.kinds().count("attention") == (1 if mask == "causal" else 0)
    block = as_payload_module(str(generate_llama_transformer_payload("payload", B, S, dim, nh, nkv, hidden, 1, mask=mask, final_norm=False))).plans["payload"]
    out = CpuPlanRunner(block).run(transformer_args(g, 1, mask))[0]
    assert max_rel_err(out, g["block0_out"]) < 1e-5
    assert np.allclose(out, g["block0_out"], rtol=0.01, atol=0.01)  # the reference's own criterion
    if mask == "causal":  # every builder group became one operator
        assert block.kinds() == ["rmsnorm", "gemm", "gemm", "gemm"] + ["ew:mul"] * (2 * B) + ["attention", "gemm", "rmsnorm", "gemm", "gemm", "ew:mul", "gemm", "ew:copy"]
    full = as_payload_module(str(generate_llama_transformer_payload("payload", B, S, dim, nh, nkv, hidden, nl, mask=mask))).plans["payload"]
    out = CpuPlanRunner(full).run(transformer_args(g, nl, mask))[0]
    assert max_rel_err(out, g["out"]) < 1e-5
    assert np.allclose(out, g["out"], rtol=0.01, atol=0.01)


def test_oracle_restatement_agrees_with_the_plans_on_other_data(g):
    """Another configuration (no grouped heads, no mask) than the fixture's, oracle against plan."""
    rng = np.random.RandomState(3)
    B, S, dim, nh = 1, 12, 48, 3
    x = rng.randn(B, S, dim).astype(np.float32)
    ws = [(rng.randn(dim, dim) * 0.2).astype(np.float32) for _ in range(4)]
    freqs = rng.randn(S, dim // nh // 2).astype(np.float32)
    plan = as_payload_module(str(generate_llama_attention_payload("payload", B, S, dim, nh, nh, mask="none"))).plans["payload"]
    out = CpuPlanRunner(plan).run([np.zeros((B, S, dim), np.float32), x] + ws + [freqs])[0]
    assert max_rel_err(out, R.llama_linalg_attention(x, *ws, freqs, None, nh, nh)) < 1e-5


# ------------------------------------------------------------------------------------------ GPU
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_index_built_causal_mask_is_recognised_at_every_float_width(dtype):
    """-inf prints as the bit pattern of the mask's own element type and reads back as -inf,
    so that the masked attention becomes one causal flash-attention operator."""
    from lighthouse_b200.payload import as_payload_module

    module = generate_llama_transformer_payload("payload", 1, 128, 256, 2, 1, llama_hidden_dim(256, 64), 1, dtype=dtype, mask="causal", final_norm=False)
    plan = as_payload_module(str(module)).plans["payload"]
    attn = [op for op in plan.ops if op.kind == "attention"]
    assert len(attn) == 1 and attn[0].attrs["causal"]


@pytest.mark.gpu
@pytest.mark.parametrize("mask", ["operand", "causal"])
def test_llama_transformer_payload_on_the_gpu_matches_the_reference_ground_truth(ctx, g, mask):
    from lighthouse_b200.execution import GPUMemoryManager, Runner

    dim, nl, nh, nkv, B, S, hidden = meta(g)
    module = generate_llama_transformer_payload("payload", B, S, dim, nh, nkv, hidden, nl, mask=mask)
    runner = Runner(str(module), mem_manager_cls=GPUMemoryManager, context=ctx)
    out = np.zeros((B, S, dim), np.float32)
    runner.execute("payload", transformer_args(g, nl, mask), Runner.get_gpu_argument_access_callback(out))
    runner.close()
    assert np.allclose(out, g["out"], rtol=0.01, atol=0.01)  # the reference's own criterion
    assert_parity(out, g["out"], "f32", tol=1e-4)  # f32 on the CUDA cores / six bf16 products: accumulation order differs from torch's


@pytest.mark.gpu
def test_llama_block_payload_bf16_at_head_dim_128_takes_the_flash_kernel(ctx):
    """bf16 operands at the benchmark configuration's head size (head_dim 128, 4 query heads per
    kv head) through the payload path: the projections and the attention run on the tensor-core
    kernels; checked against the oracle's restatement of the builders on the bf16-rounded inputs."""
    import torch

    from lighthouse_b200.execution import Runner, TorchCudaMemoryManager

    B, S, nh, nkv, hd = 2, 256, 8, 2, 128
    dim = nh * hd
    hidden = llama_hidden_dim(dim, 256)
    module = generate_llama_transformer_payload("payload", B, S, dim, nh, nkv, hidden, 1, dtype="bf16", mask="causal", final_norm=False)
    gen = torch.Generator().manual_seed(12)
    rnd = lambda *s, std=1.0: (torch.randn(*s, generator=gen) * std).to(torch.bfloat16)
    x, freqs = rnd(B, S, dim), rnd(S, hd // 2)
    w = dict(wq=rnd(nh * hd, dim, std=0.03), wk=rnd(nkv * hd, dim, std=0.03), wv=rnd(nkv * hd, dim, std=0.03), wo=rnd(dim, nh * hd, std=0.03),
             w1=rnd(hidden, dim, std=0.03), b1=rnd(hidden, std=0.1), w2=rnd(dim, hidden, std=0.03), b2=rnd(dim, std=0.1), w3=rnd(hidden, dim, std=0.03), b3=rnd(hidden, std=0.1))
    runner = Runner(str(module), mem_manager_cls=TorchCudaMemoryManager, context=ctx)
    plan = runner.payload.plans["payload"]
    assert plan.kinds().count("attention") == 1
    out = torch.zeros(B, S, dim, device="cuda", dtype=torch.bfloat16)
    runner.execute("payload", [out, x.cuda(), freqs.cuda()] + [w[n].cuda() for n in LAYER_ARG_NAMES])
    runner.close()
    f = lambda t: t.float().numpy()
    mask = np.triu(np.full((B, nh, S, S), -np.inf, np.float32), k=1)
    wn = {k: f(v) for k, v in w.items()}
    # the builders at f32 on the same (bf16-valued) inputs, biases included
    xr = f(x)
    h = xr + R.llama_linalg_attention(R.rmsnorm(xr, None, 1e-5, "f32"), wn["wq"], wn["wk"], wn["wv"], wn["wo"], f(freqs), mask, nh, nkv)
    hn = R.rmsnorm(h, None, 1e-5, "f32")
    ref = h + (R.silu(hn @ wn["w1"].T + wn["b1"]) * (hn @ wn["w3"].T + wn["b3"])) @ wn["w2"].T + wn["b2"]
    assert_parity(out.float().cpu().numpy(), ref, "bf16")
