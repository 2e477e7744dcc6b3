"""Generates the committed golden fixtures from the reference checkout.

Run where the reference is mounted (it is not on the GPU box):

    python tests/golden/make_golden.py <path of the reference checkout>

Two fixtures:

* ``lh_run_pipeline_check.json`` — the 16 known-answer row values of the reference's own
  ``lh-run`` test, read as text from test/run/pipeline-check.mlir (CHECK lines), with the
  command-line parameters of its RUN line.
* ``llama_ref.npz`` — inputs and outputs of the reference's torch model
  (examples/llama/ref_model.py, imported and executed here): RMSNorm, rotary embedding,
  Attention, FeedForward, TransformerBlock and a 2-layer Transformer trunk, on small seeded
  f32 configurations. These pin the oracle's Llama restatement against the reference itself.
"""

from __future__ import annotations

import importlib.util
import json
import re
import sys
from pathlib import Path

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


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    ref = Path(sys.argv[1])
    golden_lh_run(ref)
    golden_llama(ref)
    print("wrote", sorted(p.name for p in HERE.iterdir()))
