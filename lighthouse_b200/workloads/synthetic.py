"""Seeded synthetic inputs for the five benchmark configurations: shapes, distributions and
seeds of the configuration list the benchmarks are quoted on. Used by ``bench.py`` and by the
tests (through ``oracle.inputs``) so both see the same data."""

from __future__ import annotations

import numpy as np
import torch


def gemm_f32_uniform(m: int, n: int, k: int, seed: int = 1):
    """Config 1: A, B ~ U(-1, 1) f32 row-major, C zeros."""
    rng = np.random.RandomState(seed)
    a = (rng.rand(m, k) * 2.0 - 1.0).astype(np.float32)
    b = (rng.rand(k, n) * 2.0 - 1.0).astype(np.float32)
    return a, b, np.zeros((m, n), np.float32)


def gemm_bf16_normal(m: int, n: int, k: int, seed: int = 2):
    """Config 2: A, B ~ N(0, 0.02) rounded to bf16, bias ~ N(0, 1) in the result type (bf16)."""
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(m, k, generator=g) * 0.02).to(torch.bfloat16)
    b = (torch.randn(k, n, generator=g) * 0.02).to(torch.bfloat16)
    bias = torch.randn(n, generator=g).to(torch.bfloat16)
    return a, b, bias


def attention_qkv(b: int, hq: int, hkv: int, sq: int, skv: int, d: int, seed: int = 3):
    """Config 3: Q, K, V ~ N(0, 1) rounded to bf16, contiguous (B, H, S, D)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, hq, sq, d, generator=g).to(torch.bfloat16)
    k = torch.randn(b, hkv, skv, d, generator=g).to(torch.bfloat16)
    v = torch.randn(b, hkv, skv, d, generator=g).to(torch.bfloat16)
    return q, k, v


def nanogpt_weights(n_layer: int, c: int, hidden: int, vocab: int, block_size: int, seed: int = 4, std: float = 0.02):
    """Config 4: linear weights ~ N(0, 0.02) bf16 in (in, out) layout, LayerNorm gamma=1 beta=0,
    biases 0 (the reference's initialisation, examples/xegpu/nanoGPT.py:249-292), plus token
    and position tables (an extension: the reference builds embeddings on the host)."""
    g = torch.Generator().manual_seed(seed)

    def w(*shape):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    layers = []
    for _ in range(n_layer):
        layers.append(
            dict(
                g1=torch.ones(c), b1n=torch.zeros(c),
                wq=w(c, c), wk=w(c, c), wv=w(c, c), wp=w(c, c), bp=torch.zeros(c),
                g2=torch.ones(c), b2n=torch.zeros(c),
                w1=w(c, hidden), bb1=torch.zeros(hidden), w2=w(hidden, c), bb2=torch.zeros(c),
            )
        )
    return dict(
        layers=layers,
        gf_g=torch.ones(c), gf_b=torch.zeros(c),
        lmw=w(c, vocab), lmb=torch.zeros(vocab),
        wte=w(vocab, c), wpe=w(block_size, c),
    )


def llama_weights(n_layer: int, dim: int, n_heads: int, n_kv_heads: int, ffn: int, seed: int = 5, std: float = 0.02):
    """Config 5: weights ~ N(0, 0.02) bf16 in (out, in) layout, RMSNorm weight 1."""
    g = torch.Generator().manual_seed(seed)
    hd = dim // n_heads

    def w(*shape):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    layers = []
    for _ in range(n_layer):
        layers.append(
            dict(
                attention_norm=torch.ones(dim, dtype=torch.bfloat16), ffn_norm=torch.ones(dim, dtype=torch.bfloat16),
                wq=w(n_heads * hd, dim), wk=w(n_kv_heads * hd, dim), wv=w(n_kv_heads * hd, dim), wo=w(dim, n_heads * hd),
                w1=w(ffn, dim), w3=w(ffn, dim), w2=w(dim, ffn),
            )
        )
    return dict(layers=layers, norm=torch.ones(dim, dtype=torch.bfloat16))
