"""Full-depth parity of the decoder workloads at their real sizes (test infrastructure only).

A causal decoder's output at positions 0..t-1 of a sequence depends only on that sequence's
first t inputs: every operator is either per token (norms, projections, feed-forward, rotary
embedding at absolute positions) or causal attention. So the oracle is run on the first
``prefix`` tokens of a few sequences - seconds on the host at any model width and depth - and
the GPU result of the whole batch at full sequence length must agree with it on those rows.
The oracle functions are the pinned ones of ``oracle.reference_ops`` (ref_model.py:204-284 of
examples/llama, nanoGPT.py:114-135 of examples/xegpu in the reference); only the row
selection is new.
"""

from __future__ import annotations

import numpy as np

from . import reference_ops as R
from .inputs import to_np, tree_to_np


def prefix_rows(seq_len: int, sequences, prefix: int) -> np.ndarray:
    """Row indices, in a (batch * seq_len, width) activation matrix, of the first ``prefix``
    positions of the given sequences."""
    return np.concatenate([np.arange(s * seq_len, s * seq_len + prefix) for s in sequences])


class _LazyLayers:
    """Layers converted to f32 numpy one at a time (a full-size stack is several GB in f32)."""

    def __init__(self, layers):
        self.layers = layers

    def __iter__(self):
        for lw in self.layers:
            yield tree_to_np(lw)


def llama_prefix_reference(weights: dict, x, cfg, sequences=(0, 1), prefix: int = 256, shards: int = 1) -> np.ndarray:
    """(len(sequences) * prefix, dim) oracle output for the first ``prefix`` positions of the
    chosen sequences of ``x`` ((batch * seq, dim), torch bf16 or numpy); ``weights`` in the
    reference's (out, in) layout as ``workloads.synthetic.llama_weights`` makes them.
    ``shards``: the tensor-parallel degree of the run under test (the contracting products'
    partial sums are then rounded per device, see ``reference_ops.sharded_contraction``)."""
    xs = to_np(x).reshape(cfg.batch, cfg.seq, cfg.dim)[list(sequences), :prefix]
    out = R.llama_forward(xs, _LazyLayers(weights["layers"]), to_np(weights["norm"]), cfg.n_heads, cfg.n_kv_heads, cfg.theta, cfg.eps, "bf16", fused_swiglu=True, fused_residual=True, shards=shards)
    return out.reshape(len(sequences) * prefix, cfg.dim)


def nanogpt_prefix_reference(weights: dict, ids, cfg, sequences=(0, 1), prefix: int = 256, vocab_slice: slice | None = None) -> np.ndarray:
    """(len(sequences) * prefix, vocab) oracle logits for the first ``prefix`` positions of the
    chosen sequences of ``ids`` ((batch * seq,) token ids); ``vocab_slice`` selects the columns
    a tensor-parallel rank holds."""
    ids = np.asarray(to_np(ids)).reshape(cfg.batch, cfg.seq)[list(sequences), :prefix]
    x = R.embed(ids, to_np(weights["wte"]), to_np(weights["wpe"]))
    lmw, lmb = to_np(weights["lmw"]), to_np(weights["lmb"])
    if vocab_slice is not None:
        lmw, lmb = lmw[:, vocab_slice], lmb[vocab_slice]
    return R.nanogpt_forward(x, _LazyLayers(weights["layers"]), to_np(weights["gf_g"]), to_np(weights["gf_b"]), lmw, lmb, cfg.n_head, cfg.eps, cfg.causal, cfg.act, "bf16", len(sequences))
