"""Generates the committed golden fixtures from the reference checkout.

Run where the reference is mounted (it is not on the GPU box):

    python tests/golden/make_golden.py <path of the reference checkout>

Four fixtures:

* ``lh_run_pipeline_check.json`` — the 16 known-answer row values of the reference's own
  ``lh-run`` test, read as text from test/run/pipeline-check.mlir (CHECK lines), with the
  command-line parameters of its RUN line.
* ``llama_ref.npz`` — inputs and outputs of the reference's torch model
  (examples/llama/ref_model.py, imported and executed here): RMSNorm, rotary embedding,
  Attention, FeedForward, TransformerBlock and a 2-layer Transformer trunk, on small seeded
  f32 configurations. These pin the oracle's Llama restatement against the reference itself.
* ``llama_linalg_ref.npz`` — the same torch model run the way the reference's tests of its
  linalg Llama builders run it (real frequency table, additive mask): see
  ``golden_llama_linalg``.
* ``numpy_checks.npz`` — inputs and outputs of the reference's own pure-numpy check code:
  ``_ln``, ``_f16``, ``_mha``, ``numpy_ref_block_fused``, ``numpy_ref_gpt_fused``
  (examples/xegpu/nanoGPT.py:84-135), ``check_correctness`` of fused_attention.py:46-106,
  layer_norm.py:43-78 and softmax.py:42-83, ``check_results`` of matmul.py:233-279,
  ``check_correctness`` of mlp.py:47-101, the seeded input generator of matmul.py:135-164 and
  the flop/byte models. Those modules import the MLIR bindings at the top, so they cannot be
  imported; the function definitions are taken out of the source text with ``ast`` and
  executed unmodified in a namespace that holds numpy only. A check function compares an
  output with a reference it computes inside and returns a bool: it is handed a numpy
  stand-in whose ``allclose`` records its second argument, which is that reference.
"""

from __future__ import annotations

import ast
import importlib.util
import json
import re
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def golden_lh_run(ref: Path) -> None:
    text = (ref / "test/run/pipeline-check.mlir").read_text()
    rows = [float(m.group(1)) for m in re.finditer(r"// CHECK: \[(\d+\.\d+)", text)]
    run = re.search(r"--input-shape=(\S+) --print-tensor=(\d+) --seed=(\d+)", text)
    out = {
        "source": "test/run/pipeline-check.mlir:1-31",
        "input_shape": run.group(1),
        "print_tensor": int(run.group(2)),
        "seed": int(run.group(3)),
        "entry_point": "main",
        "row_values": rows,
    }
    assert len(rows) == 16
    (HERE / "lh_run_pipeline_check.json").write_text(json.dumps(out, indent=1) + "\n")


def golden_llama(ref: Path) -> None:
    spec = importlib.util.spec_from_file_location("ref_model", ref / "examples/llama/ref_model.py")
    rm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rm)
    torch.manual_seed(1234)
    out: dict[str, np.ndarray] = {}
    args = rm.ModelArgs(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=97, multiple_of=32, norm_eps=1e-5, rope_theta=10000.0, max_batch_size=2, max_seq_len=16)
    B, S = 2, 8
    hd = args.dim // args.n_heads

    def randomise(mod):
        for p in mod.parameters():
            with torch.no_grad():
                p.copy_(torch.randn_like(p) * (0.2 if p.ndim > 1 else 1.0) + (0.0 if p.ndim > 1 else 1.0))

    # RMSNorm
    norm = rm.RMSNorm(args.dim, eps=args.norm_eps)
    randomise(norm)
    x = torch.randn(B, S, args.dim)
    out["rms_x"], out["rms_w"], out["rms_out"] = x.numpy(), norm.weight.detach().numpy(), norm(x).detach().numpy()
    # rotary
    freqs = rm.precompute_freqs_cis(hd, S, args.rope_theta)
    xq = torch.randn(B, S, args.n_heads, hd)
    xk = torch.randn(B, S, args.n_kv_heads, hd)
    q2, k2 = rm.apply_rotary_emb(xq, xk, freqs)
    out["rope_xq"], out["rope_xk"], out["rope_q_out"], out["rope_k_out"] = xq.numpy(), xk.numpy(), q2.numpy(), k2.numpy()
    # mask as Transformer.forward builds it
    mask = torch.triu(torch.full((S, S), float("-inf")), diagonal=1)
    # Attention
    attn = rm.Attention(args)
    randomise(attn)
    x = torch.randn(B, S, args.dim)
    with torch.no_grad():
        y = attn(x, 0, freqs, mask)
    out["attn_x"], out["attn_out"] = x.numpy(), y.numpy()
    for n in ("wq", "wk", "wv", "wo"):
        out[f"attn_{n}"] = getattr(attn, n).weight.detach().numpy()
    # FeedForward
    ff = rm.FeedForward(args.dim, 4 * args.dim, args.multiple_of, None)
    randomise(ff)
    x = torch.randn(B, S, args.dim)
    with torch.no_grad():
        y = ff(x)
    out["ff_x"], out["ff_out"] = x.numpy(), y.numpy()
    for n in ("w1", "w2", "w3"):
        out[f"ff_{n}"] = getattr(ff, n).weight.detach().numpy()
    # Transformer trunk: 2 blocks + final norm, fed with embeddings
    model = rm.Transformer(args)
    randomise(model)
    x = torch.randn(B, S, args.dim)
    with torch.no_grad():
        h = x
        blocks = []
        for layer in model.layers:
            h = layer(h, 0, model.freqs_cis[:S], mask)
            blocks.append(h)
        hn = model.norm(h)
    out["tf_x"], out["tf_block0_out"], out["tf_out"] = x.numpy(), blocks[0].numpy(), hn.numpy()
    out["tf_norm"] = model.norm.weight.detach().numpy()
    for i, layer in enumerate(model.layers):
        a, f = layer.attention, layer.feed_forward
        for n in ("wq", "wk", "wv", "wo"):
            out[f"tf_l{i}_{n}"] = getattr(a, n).weight.detach().numpy()
        for n in ("w1", "w2", "w3"):
            out[f"tf_l{i}_{n}"] = getattr(f, n).weight.detach().numpy()
        out[f"tf_l{i}_attention_norm"] = layer.attention_norm.weight.detach().numpy()
        out[f"tf_l{i}_ffn_norm"] = layer.ffn_norm.weight.detach().numpy()
    out["meta"] = np.array([args.dim, args.n_layers, args.n_heads, args.n_kv_heads, B, S], dtype=np.int64)
    np.savez_compressed(HERE / "llama_ref.npz", **out)


def golden_llama_linalg(ref: Path) -> None:
    """The configuration of the reference's own test_transformer_block_fwd / test_transformer_fwd
    (examples/llama/test_llama3.py:1655-1985): the torch model run with the REAL frequency table
    those tests feed it (a complex tensor with zero imaginary part, so the "rotary embedding" is
    a plain scaling of the (even, odd) pairs), an additive -inf upper-triangular mask, unit norm
    weights and no biases. These are the outputs the reference's linalg builders are checked
    against, so they pin the oracle's restatement of those builders."""
    spec = importlib.util.spec_from_file_location("ref_model", ref / "examples/llama/ref_model.py")
    rm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rm)
    torch.manual_seed(4321)
    args = rm.ModelArgs(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=97, multiple_of=16, norm_eps=1e-5, max_batch_size=2, max_seq_len=16)
    B, S = 2, 8
    hd = args.dim // args.n_heads
    out: dict[str, np.ndarray] = {}
    model = rm.Transformer(args)
    for name, prm in model.named_parameters():
        if prm.ndim > 1:
            with torch.no_grad():
                prm.copy_(torch.randn_like(prm) * 0.2)
    x = torch.randn(B, S, args.dim)
    freqs_real = torch.randn(S, hd // 2)
    freqs = torch.complex(freqs_real, torch.zeros_like(freqs_real))
    mask = torch.triu(torch.full((B, args.n_heads, S, S), float("-inf")), diagonal=1)
    with torch.no_grad():
        attn_out = model.layers[0].attention(x, 0, freqs, mask)
        h = x
        blocks = []
        for layer in model.layers:
            h = layer(h, 0, freqs, mask)
            blocks.append(h)
        final = model.norm(h)
    out["x"], out["freqs_real"], out["mask"] = x.numpy(), freqs_real.numpy(), mask.numpy()
    out["attn_out"], out["block0_out"], out["out"] = attn_out.numpy(), blocks[0].numpy(), final.numpy()
    for i, layer in enumerate(model.layers):
        for n in ("wq", "wk", "wv", "wo"):
            out[f"l{i}_{n}"] = getattr(layer.attention, n).weight.detach().numpy()
        for n in ("w1", "w2", "w3"):
            out[f"l{i}_{n}"] = getattr(layer.feed_forward, n).weight.detach().numpy()
    out["meta"] = np.array([args.dim, args.n_layers, args.n_heads, args.n_kv_heads, B, S, out["l0_w1"].shape[0]], dtype=np.int64)
    np.savez_compressed(HERE / "llama_linalg_ref.npz", **out)


class _RecordingNumpy:
    """numpy, except that ``allclose`` also keeps what it was asked to compare with."""

    def __init__(self):
        self.seen = []

    def __getattr__(self, name):
        return getattr(np, name)

    def allclose(self, a, b, *args, **kwargs):
        self.seen.append((np.array(b), dict(kwargs)))
        return np.allclose(a, b, *args, **kwargs)


def _extract(path: Path, names, recorder=None) -> dict:
    """Executes the named top-level functions (or ``Class.method``) of a source file, and
    nothing else of it, in a namespace holding numpy."""
    tree = ast.parse(path.read_text())
    wanted = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            wanted.append(node)
        if isinstance(node, ast.ClassDef):
            for sub in node.body:
                if isinstance(sub, ast.FunctionDef) and f"{node.name}.{sub.name}" in names:
                    sub.decorator_list = []
                    wanted.append(sub)
    for fn in wanted:  # annotations may name classes that are not extracted
        fn.returns = None
        for a in fn.args.args + fn.args.kwonlyargs:
            a.annotation = None
    missing = set(n.split(".")[-1] for n in names) - {fn.name for fn in wanted}
    if missing:
        raise SystemExit(f"{path}: not found: {sorted(missing)}")
    ns = {"np": recorder if recorder is not None else np}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), str(path), "exec"), ns)
    return ns


def golden_numpy_checks(ref: Path) -> None:
    ex = ref / "examples/xegpu"
    rng = np.random.RandomState(20240607)
    out: dict[str, np.ndarray] = {}
    f32 = np.float32

    # ---- nanoGPT numpy reference (f16 rounding points, optional causal switch)
    ns = _extract(ex / "nanoGPT.py", ["_ln", "_f16", "_mha", "numpy_ref_block_fused", "numpy_ref_gpt_fused"])
    T, C, H, hid, vocab, L = 32, 64, 4, 128, 96, 2
    f16w = lambda *s: (rng.randn(*s) * 0.1).astype(np.float16)
    layers = []
    for _ in range(L):
        layers.append(dict(
            g1=(1 + 0.1 * rng.randn(C)).astype(f32), b1n=(0.1 * rng.randn(C)).astype(f32),
            wq=f16w(C, C), wk=f16w(C, C), wv=f16w(C, C), wp=f16w(C, C), bp=(0.1 * rng.randn(C)).astype(f32),
            g2=(1 + 0.1 * rng.randn(C)).astype(f32), b2n=(0.1 * rng.randn(C)).astype(f32),
            w1=f16w(C, hid), bb1=(0.1 * rng.randn(hid)).astype(f32), w2=f16w(hid, C), bb2=(0.1 * rng.randn(C)).astype(f32),
        ))
    gf_g, gf_b = (1 + 0.1 * rng.randn(C)).astype(f32), (0.1 * rng.randn(C)).astype(f32)
    lmw, lmb = f16w(C, vocab), (0.1 * rng.randn(vocab)).astype(f32)
    x = (rng.randn(T, C) * 0.5).astype(f32)
    out["gpt_meta"] = np.array([T, C, H, hid, vocab, L], dtype=np.int64)
    out["gpt_x"] = x
    for i, w in enumerate(layers):
        for k, v in w.items():
            out[f"gpt_l{i}_{k}"] = v
    out["gpt_gf_g"], out["gpt_gf_b"], out["gpt_lmw"], out["gpt_lmb"] = gf_g, gf_b, lmw, lmb
    out["gpt_ln"] = ns["_ln"](x, layers[0]["g1"], layers[0]["b1n"], 1e-5)
    out["gpt_f16"] = ns["_f16"](x * 3.3)
    q, k, v = (ns["_f16"](rng.randn(T, C).astype(f32)) for _ in range(3))
    out["mha_q"], out["mha_k"], out["mha_v"] = q, k, v
    out["mha_out"] = ns["_mha"](q, k, v, H)
    out["mha_out_causal"] = ns["_mha"](q, k, v, H, causal=True)
    out["gpt_block"] = ns["numpy_ref_block_fused"](x, layers[0], H)
    out["gpt_block_causal"] = ns["numpy_ref_block_fused"](x, layers[0], H, causal=True)
    out["gpt_logits"] = ns["numpy_ref_gpt_fused"](x, layers, gf_g, gf_b, lmw, lmb, H)

    # ---- fused attention check (f32 statement; the reference feeds f16 arrays)
    rec = _RecordingNumpy()
    ns = _extract(ex / "fused_attention.py", ["fused_attention_complexity", "check_correctness"], rec)
    Q, K, V = (rng.randn(2, 3, 48, 32).astype(np.float16) for _ in range(3))
    assert not ns["check_correctness"](Q, K, V, np.zeros(Q.shape, f32))
    out["fa_q"], out["fa_k"], out["fa_v"], out["fa_out"] = Q, K, V, rec.seen[-1][0]
    out["fa_complexity"] = np.array(ns["fused_attention_complexity"](8, 16, 2048, 128, 2), dtype=np.int64)

    # ---- layer norm check
    rec = _RecordingNumpy()
    ns = _extract(ex / "layer_norm.py", ["layer_norm_complexity", "check_correctness"], rec)
    xin, g, b = rng.randn(24, 80).astype(f32) * 2 + 0.5, rng.randn(80).astype(f32), rng.randn(80).astype(f32)
    ns["check_correctness"](xin, g, b, np.zeros_like(xin), 1e-5)
    out["ln_x"], out["ln_g"], out["ln_b"], out["ln_out"] = xin, g, b, rec.seen[-1][0]
    out["ln_complexity"] = np.array(ns["layer_norm_complexity"](16384, 768, 4), dtype=np.int64)

    # ---- softmax check (its last allclose is the value comparison)
    rec = _RecordingNumpy()
    ns = _extract(ex / "softmax.py", ["softmax_complexity", "check_correctness"], rec)
    xin = rng.randn(24, 80).astype(f32) * 3
    ns["check_correctness"](xin, np.zeros_like(xin))
    out["sm_x"], out["sm_out"] = xin, rec.seen[-1][0]
    out["sm_complexity"] = np.array(ns["softmax_complexity"](16384, 768, 4), dtype=np.int64)

    # ---- matmul: seeded inputs, flop/byte model, reference result per post-op combination
    rec = _RecordingNumpy()
    ns = _extract(ex / "matmul.py", ["matmul_complexity", "check_results", "XeGPUMatMul.get_input_arrays"], rec)
    out["mm_complexity"] = np.array(ns["matmul_complexity"](4096, 4096, 4096, True, True, False, 2, 2), dtype=np.int64)
    variants = [  # (bias, relu, accumulate_c, truncate_c, transpose_a, transpose_b, init_int)
        (False, False, True, False, False, False, False),
        (True, True, False, True, False, False, False),
        (True, False, True, False, True, True, True),
        (False, True, False, True, False, True, True),
    ]
    M, N, K = 24, 40, 56
    out["mm_meta"] = np.array([M, N, K], dtype=np.int64)
    out["mm_variants"] = np.array(variants, dtype=np.int64)
    for i, (bias, relu, acc, trunc, ta, tb, ints) in enumerate(variants):
        mm = SimpleNamespace(
            M=M, N=N, K=K, has_bias=bias, has_relu=relu, accumulate_c=acc, truncate_c=trunc, transpose_a=ta, transpose_b=tb,
            ab_dtype=np.float16, c_dtype=np.float16 if trunc else f32,
            a_shape=(M, K) if not ta else (K, M), b_shape=(K, N) if not tb else (N, K), c_shape=(M, N), bias_shape=(N,),
            _input_arrays_cache={},
        )
        arrays = ns["get_input_arrays"](mm, ints)
        ns["check_results"](mm, arrays, np.zeros((M, N), f32))
        for name, arr in zip(("C", "A", "B", "bias"), arrays):
            out[f"mm{i}_{name}"] = arr
        out[f"mm{i}_out"] = rec.seen[-1][0]

    # ---- chained MLP check: 3 layers, bias, ReLU between layers
    rec = _RecordingNumpy()
    ns = _extract(ex / "mlp.py", ["check_correctness"], rec)
    sizes = [48, 64, 32, 40]
    xin = (rng.rand(16, sizes[0]) - 0.5).astype(np.float16)
    ws = [(rng.rand(sizes[i], sizes[i + 1]) - 0.5).astype(np.float16) for i in range(3)]
    bs = [(rng.rand(sizes[i + 1]) - 0.5).astype(np.float16) for i in range(3)]
    ns["check_correctness"]([np.zeros((16, sizes[-1]), np.float16), xin] + ws + bs, np.zeros((16, sizes[-1]), np.float16), np.float16, has_bias=True, has_relu=True)
    out["mlp_x"] = xin
    for i in range(3):
        out[f"mlp_w{i}"], out[f"mlp_b{i}"] = ws[i], bs[i]
    out["mlp_out"] = rec.seen[-1][0]
    np.savez_compressed(HERE / "numpy_checks.npz", **out)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    ref = Path(sys.argv[1])
    golden_lh_run(ref)
    golden_llama(ref)
    golden_numpy_checks(ref)
    golden_llama_linalg(ref)
    print("wrote", sorted(p.name for p in HERE.iterdir()))
