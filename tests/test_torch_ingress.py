"""The ``torch.compile`` entry: FX graph -> plan -> kernels.

CPU part: the importer's plans are executed by the plan interpreter (oracle arithmetic) and
compared with eager torch on the same seeded inputs; calling convention and error behaviour
mirror lighthouse/ingress/torch/compile.py of the reference. GPU part: the same modules run
through ``torch.compile(backend=gpu_backend())`` on the CUDA kernels."""

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from cpu_plan import CpuPlanRunner
from oracle import inputs as I
from oracle.check import TOL_BF16, max_rel_err, assert_parity

from lighthouse_b200.ingress.torch import CudaBackend, JITFunction, UnsupportedGraph, gpu_backend, import_fx_graph


class Mlp(nn.Module):
    def __init__(self, d_in=64, hidden=128, d_out=32):
        super().__init__()
        self.fc1 = nn.Linear(d_in, hidden)
        self.fc2 = nn.Linear(hidden, d_out, bias=False)

    def forward(self, x):
        return self.fc2(torch.relu(self.fc1(x)))


class Block(nn.Module):
    """Pre-LayerNorm decoder block: causal attention over (B, H, S, hs) views of one packed
    projection, output projection + residual, GELU MLP + residual."""

    def __init__(self, c=128, heads=2, hidden=256):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = nn.LayerNorm(c), nn.LayerNorm(c)
        self.qkv = nn.Linear(c, 3 * c, bias=False)
        self.proj = nn.Linear(c, c)
        self.fc1, self.fc2 = nn.Linear(c, hidden), nn.Linear(hidden, c)

    def forward(self, x):
        b, s, c = x.shape
        hs = c // self.heads
        q, k, v = self._split(self.qkv(self.ln1(x)), b, s, hs)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(b, s, c))
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))

    def _split(self, qkv, b, s, hs):
        t = qkv.view(b, s, 3, self.heads, hs)
        return t[:, :, 0].transpose(1, 2), t[:, :, 1].transpose(1, 2), t[:, :, 2].transpose(1, 2)


def capture(model, *inputs):
    """Compiles ``model`` with a backend that imports the graph and then runs eagerly; returns
    (plan, result metadata, example inputs as given to the backend, eager outputs)."""
    got = {}

    def backend(gm, example_inputs):
        got["plan"], got["results"], got["n"] = import_fx_graph(gm, example_inputs)
        got["inputs"] = list(example_inputs)
        return gm.forward

    torch._dynamo.reset()
    with torch.no_grad():
        out = torch.compile(model, backend=backend, dynamic=False)(*inputs)
    return got["plan"], got["results"], got["inputs"], out


def interpret(plan, results, inputs):
    args = [I.to_np(t.detach()) for t in inputs] + [np.zeros(r.shape, np.float32) for r in results]
    return CpuPlanRunner(plan).run(args)[len(inputs) :]


def test_mlp_graph_becomes_two_fused_gemms_and_matches_eager():
    torch.manual_seed(0)
    model, x = Mlp().to(torch.bfloat16), torch.randn(48, 64).to(torch.bfloat16)
    plan, results, inputs, want = capture(model, x)
    assert plan.kinds() == ["gemm", "gemm"] and plan.ops[0].attrs["act"] == "relu" and plan.ops[0].operands[4] is not None
    # calling convention: graph inputs in placeholder order, result buffers appended last
    assert len(plan.args) == len(inputs) + 1 and plan.args[-1].name == "result0" and tuple(plan.args[-1].shape) == (48, 32)
    assert plan.ops[-1].operands[0].slot == len(inputs)  # the last GEMM writes the result buffer itself
    assert results[0].dtype == torch.bfloat16 and results[0].shape == [48, 32]
    (got,) = interpret(plan, results, inputs)
    assert_parity(got, want.float().numpy(), "bf16")


def test_decoder_block_graph_matches_eager():
    torch.manual_seed(1)
    model, x = Block().to(torch.bfloat16), torch.randn(2, 32, 128).to(torch.bfloat16)
    plan, results, inputs, want = capture(model, x)
    kinds = plan.kinds()
    assert kinds.count("attention") == 1 and kinds.count("layernorm") == 2 and kinds.count("gemm") == 4
    attn = next(op for op in plan.ops if op.kind == "attention")
    assert attn.attrs["causal"] and attn.operands[1].shape == (2, 2, 32, 64)  # strided (B, H, S, hs) views, no copies
    (got,) = interpret(plan, results, inputs)
    assert_parity(got, want.float().numpy(), "bf16")


def test_two_results_and_f32_graph():
    class Two(nn.Module):
        def forward(self, a, b):
            c = torch.matmul(a, b)
            return c, torch.softmax(c, dim=-1)

    torch.manual_seed(2)
    a, b = torch.randn(24, 40), torch.randn(40, 16)
    plan, results, inputs, want = capture(Two(), a, b)
    assert [tuple(s.shape) for s in plan.args[-2:]] == [(24, 16), (24, 16)]
    got = interpret(plan, results, inputs)
    for g, w in zip(got, want):
        assert_parity(g, w.numpy(), "f32")


def test_embedding_rms_norm_and_split_views():
    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(50, 64)
            self.norm = nn.RMSNorm(64, eps=1e-5)
            self.up = nn.Linear(64, 256, bias=False)
            self.down = nn.Linear(128, 64, bias=False)

        def forward(self, ids):
            h = self.emb(ids)
            gate, up = self.up(self.norm(h)).chunk(2, dim=-1)
            return h + self.down(F.silu(gate) * up)

    torch.manual_seed(4)
    model = Tiny().to(torch.bfloat16)
    ids = torch.randint(0, 50, (2, 24))
    plan, results, inputs, want = capture(model, ids)
    kinds = plan.kinds()
    assert "embedding" in kinds and "rmsnorm" in kinds and kinds.count("gemm") == 2
    (got,) = interpret(plan, results, inputs)
    assert_parity(got, want.float().numpy(), "bf16")


def test_unsupported_graphs_are_value_errors_and_nothing_runs_on_cpu():
    class Sin(nn.Module):
        def forward(self, x):
            return torch.sin(x) @ x.t()

    gm = torch.fx.symbolic_trace(Sin())
    with pytest.raises(UnsupportedGraph, match="no kernel for 'sin'"):
        import_fx_graph(gm, [torch.randn(4, 4)])
    assert issubclass(UnsupportedGraph, ValueError)
    # masks other than the causal flag are not silently dropped
    class Masked(nn.Module):
        def forward(self, q, k, v, m):
            return F.scaled_dot_product_attention(q, k, v, attn_mask=m)

    q = torch.randn(1, 2, 8, 16)
    with pytest.raises(UnsupportedGraph, match="mask"):
        import_fx_graph(torch.fx.symbolic_trace(Masked()), [q, q, q, torch.zeros(8, 8)])
    # a compiled function refuses host tensors instead of computing them some other way
    plan, results, inputs, _ = capture(Mlp().to(torch.bfloat16), torch.randn(8, 64).to(torch.bfloat16))
    jit = JITFunction(plan, results)
    with pytest.raises(RuntimeError, match="no CPU path"):
        jit(*inputs)
    backend = gpu_backend()
    assert isinstance(backend, CudaBackend) and backend.entry_func == "main"


@pytest.mark.gpu
def test_torch_compile_on_the_cuda_backend_matches_eager(ctx):
    torch.manual_seed(3)
    for model, x in ((Mlp(256, 512, 128), torch.randn(384, 256)), (Block(256, 4, 512), torch.randn(2, 128, 256))):
        model = model.to(torch.bfloat16).cuda()
        x = x.to(torch.bfloat16).cuda()
        backend, seen = gpu_backend(context=ctx), {}

        def recording_backend(gm, example_inputs):
            seen["inputs"] = [t.detach() for t in example_inputs]
            return backend(gm, example_inputs)

        torch._dynamo.reset()
        with torch.no_grad():
            want = model(x)
            got = torch.compile(model, backend=recording_backend, dynamic=False)(x)
        torch.cuda.synchronize()
        assert_parity(got.float().cpu().numpy(), want.float().cpu().numpy(), "bf16")
        jit = backend._last_jit_function
        assert jit is not None and jit.plan.kinds().count("gemm") >= 2
        times = jit.benchmark(*seen["inputs"], nruns=3, nwarmup=1)  # parameters and inputs in graph order
        assert times.shape == (3,) and float(times.min()) > 0
    ctx.use_own_stream()  # the compiled functions had pointed the shared context at torch's stream


def test_view_algebra_agrees_with_torch_indexing():
    """Indexing, transposes and reshapes of the importer are stride arithmetic on ``PView``;
    the same operations on a torch tensor must select the same elements."""
    from hypothesis import given, settings, strategies as st

    from lighthouse_b200.ingress.torch.compile import _Importer
    from lighthouse_b200.plan import PView

    base = torch.arange(4 * 6 * 8).reshape(4, 6, 8)
    view = PView(0, (4, 6, 8), (48, 8, 1), "i64")

    def gather(v: PView) -> torch.Tensor:
        return torch.as_strided(base.reshape(-1), v.shape, v.strides, v.offset)

    index = st.one_of(st.integers(-4, 3), st.builds(slice, st.one_of(st.none(), st.integers(0, 3)), st.one_of(st.none(), st.integers(1, 6)), st.one_of(st.none(), st.integers(1, 3))))

    @settings(max_examples=150, deadline=None)
    @given(i0=index, i1=index, perm=st.permutations([0, 1, 2]))
    def check(i0, i1, perm):
        want = base[i0, i1]
        got = _Importer._index(view, (i0, i1))
        assert got.shape == tuple(want.shape) and torch.equal(gather(got), want)
        assert torch.equal(gather(view.permute(perm)), base.permute(perm))
        if want.dim() == 3 and want.shape[0] * want.shape[1] > 0:
            try:
                merged = got.reshape((want.shape[0] * want.shape[1], want.shape[2]))
            except ValueError:
                return  # needs a copy: the importer then materialises first
            assert torch.equal(gather(merged), want.reshape(-1, want.shape[2]))

    check()
