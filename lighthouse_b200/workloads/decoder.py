"""nanoGPT and Llama decoder forward passes as plans, with tensor parallelism.

* nanoGPT follows the reference's fused block
  (examples/xegpu/nanoGPT_payload.py:299-317: ln1 -> q,k,v -> flash attention -> proj + bias
  -> +x -> ln2 -> fc1 + bias, activation -> fc2 + bias -> +a; model: blocks -> ln_f -> lm_head
  + bias, f32 residual stream, 16-bit matmul operands, weights in (in, out) layout), extended
  with a batch dimension, a causal mask, GELU and the token/position embedding gather (the
  reference does embeddings on the host, examples/xegpu/nanoGPT.py:249-253).
* Llama follows the reference's torch model (examples/llama/ref_model.py:114-231: RMSNorm,
  q/k/v projections, rotary embedding, grouped-query causal attention, output projection,
  SwiGLU feed-forward, residuals; weights in (out, in) layout) fed with embeddings and ending
  at the final norm (examples/llama/test_llama3.py:906-947).

Tensor parallelism is the reference's 1-D weight-stationary scheme
(examples/mpi/feed-forward-mpi.py:213-224): projections that expand are split on the output
dimension, projections that contract on the input dimension, one sum all-reduce after each
contraction. The residual add rides in the contracting GEMM's epilogue on rank 0 only, so the
all-reduce of the partial sums also delivers ``x + sum``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

from ..plan import ArgSpec, Plan, PView

GPT_LAYER_KEYS = ["g1", "b1n", "wqkv", "wp", "bp", "g2", "b2n", "w1", "bb1", "w2", "bb2"]
LLAMA_LAYER_KEYS = ["attention_norm", "wqkv", "wo", "ffn_norm", "w13", "w2"]


@dataclass(frozen=True)
class NanoGptConfig:
    n_layer: int = 12
    n_head: int = 12
    n_embd: int = 768
    vocab: int = 50304
    block_size: int = 1024
    batch: int = 16
    seq: int = 1024
    hidden_mult: int = 4
    causal: bool = True
    act: str = "gelu"
    eps: float = 1e-5
    logits_dtype: str = "f32"

    @property
    def hidden(self) -> int:
        return self.hidden_mult * self.n_embd

    @property
    def tokens(self) -> int:
        return self.batch * self.seq

    def flops_per_token(self) -> float:
        """Linear layers 2 * params, attention 4 * S * C per layer (halved when causal):
        the reference's counting conventions applied to the decoder."""
        c, h = self.n_embd, self.hidden
        linear = 2 * (4 * c * c + 2 * c * h)
        attn = 4 * self.seq * c * (0.5 if self.causal else 1.0)
        return self.n_layer * (linear + attn) + 2 * c * self.vocab


@dataclass(frozen=True)
class LlamaConfig:
    n_layer: int = 8
    dim: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    batch: int = 4
    seq: int = 4096
    eps: float = 1e-5
    theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def tokens(self) -> int:
        return self.batch * self.seq

    def flops_per_token(self) -> float:
        hd = self.head_dim
        linear = 2 * (self.dim * self.n_heads * hd + 2 * self.dim * self.n_kv_heads * hd + self.n_heads * hd * self.dim + 3 * self.dim * self.ffn)
        attn = 4 * self.seq * self.n_heads * hd * 0.5
        return self.n_layer * (linear + attn)


def check_tp(cfg, tp: int) -> None:
    if tp < 1:
        raise ValueError("tensor-parallel degree must be >= 1")
    if isinstance(cfg, NanoGptConfig):
        if cfg.n_head % tp or cfg.hidden % tp or cfg.vocab % tp:
            raise ValueError(f"nanoGPT with {cfg.n_head} heads / hidden {cfg.hidden} / vocab {cfg.vocab} does not split {tp} ways")
        if (cfg.vocab // tp) % 8 or (cfg.hidden // tp) % 8:
            raise ValueError("per-rank widths must stay multiples of 8")
    else:
        if cfg.n_heads % tp or cfg.n_kv_heads % tp or cfg.ffn % tp:
            raise ValueError(f"Llama with {cfg.n_heads}/{cfg.n_kv_heads} heads, ffn {cfg.ffn} does not split {tp} ways")
        if (cfg.ffn // tp) % 128:
            raise ValueError("per-rank FFN width must be a multiple of 128 (SwiGLU column blocks)")


# ------------------------------------------------------------------------- weight layout
def shard_nanogpt_weights(w: dict, cfg: NanoGptConfig, rank: int = 0, tp: int = 1, full_bias: bool = False) -> dict:
    """Reference-layout weights (``oracle.inputs.nanogpt_weights`` keys) -> this rank's
    arrays: q/k/v column blocks of the rank's heads packed side by side into ``wqkv``;
    ``wp`` / ``w2`` row blocks; ``w1`` / ``lmw`` column blocks with their biases. Biases of
    contracting layers are kept whole on rank 0 and zeroed elsewhere (they are added once,
    before the all-reduce) unless ``full_bias``: the row-sharded schedule adds them after the
    reduce-scatter, each rank on its own rows."""
    import torch

    check_tp(cfg, tp)
    c = cfg.n_embd
    cl, hl, vl = c // tp, cfg.hidden // tp, cfg.vocab // tp
    cs, hs, vs = slice(rank * cl, (rank + 1) * cl), slice(rank * hl, (rank + 1) * hl), slice(rank * vl, (rank + 1) * vl)
    first = rank == 0 or full_bias
    layers = []
    for lw in w["layers"]:
        layers.append(
            dict(
                g1=lw["g1"].float(), b1n=lw["b1n"].float(),
                wqkv=torch.cat([lw["wq"][:, cs], lw["wk"][:, cs], lw["wv"][:, cs]], dim=1).contiguous(),
                wp=lw["wp"][cs, :].contiguous(),
                bp=lw["bp"].float() if first else torch.zeros_like(lw["bp"]).float(),
                g2=lw["g2"].float(), b2n=lw["b2n"].float(),
                w1=lw["w1"][:, hs].contiguous(), bb1=lw["bb1"][hs].float().contiguous(),
                w2=lw["w2"][hs, :].contiguous(),
                bb2=lw["bb2"].float() if first else torch.zeros_like(lw["bb2"]).float(),
            )
        )
    return dict(
        layers=layers, gf_g=w["gf_g"].float(), gf_b=w["gf_b"].float(),
        lmw=w["lmw"][:, vs].contiguous(), lmb=w["lmb"][vs].float().contiguous(),
        wte=w["wte"], wpe=w["wpe"],
    )


def pack_swiglu(w_gate, w_up, block: int = 128):
    """Rows of ``w1`` (gate) and ``w3`` (up), both (ffn, dim), interleaved in blocks of 128:
    [gate 0:128 | up 0:128 | gate 128:256 | ...] — the column layout the SwiGLU GEMM epilogue
    expects from its B operand (``LH_GEMM_SWIGLU`` in include/lh_b200.h)."""
    import torch

    f, k = w_gate.shape
    assert f % block == 0
    return torch.stack([w_gate.view(f // block, block, k), w_up.view(f // block, block, k)], dim=1).reshape(2 * f, k).contiguous()


def shard_llama_weights(w: dict, cfg: LlamaConfig, rank: int = 0, tp: int = 1) -> dict:
    """(out, in)-layout weights -> this rank's packed arrays: ``wqkv`` = rows of the rank's
    query heads, then its kv heads' k rows, then v rows; ``wo`` / ``w2`` column blocks;
    ``w13`` = SwiGLU-interleaved gate/up rows."""
    import torch

    check_tp(cfg, tp)
    hd = cfg.head_dim
    ql, kl, fl = cfg.n_heads // tp * hd, cfg.n_kv_heads // tp * hd, cfg.ffn // tp
    qs, ks, fs = slice(rank * ql, (rank + 1) * ql), slice(rank * kl, (rank + 1) * kl), slice(rank * fl, (rank + 1) * fl)
    layers = []
    for lw in w["layers"]:
        layers.append(
            dict(
                attention_norm=lw["attention_norm"],
                wqkv=torch.cat([lw["wq"][qs], lw["wk"][ks], lw["wv"][ks]], dim=0).contiguous(),
                wo=lw["wo"][:, qs].contiguous(),
                ffn_norm=lw["ffn_norm"],
                w13=pack_swiglu(lw["w1"][fs].contiguous(), lw["w3"][fs].contiguous()),
                w2=lw["w2"][:, fs].contiguous(),
            )
        )
    return dict(layers=layers, norm=w["norm"])


# --------------------------------------------------------------------------------- plans
def build_nanogpt_plan(cfg: NanoGptConfig, rank: int = 0, tp: int = 1, name: str = "nanogpt_forward") -> Plan:
    """Args: ``logits (tokens, vocab/tp), ids (tokens) i32, wte, wpe,
    [g1,b1n,wqkv,wp,bp,g2,b2n,w1,bb1,w2,bb2] * n_layer, gf_g, gf_b, lmw, lmb``."""
    check_tp(cfg, tp)
    c, t, hs = cfg.n_embd, cfg.tokens, cfg.n_embd // cfg.n_head
    cl, hl, vl, heads_l = c // tp, cfg.hidden // tp, cfg.vocab // tp, cfg.n_head // tp
    args = [ArgSpec((t, vl), cfg.logits_dtype, "logits"), ArgSpec((t,), "i32", "ids"), ArgSpec((cfg.vocab, c), "bf16", "wte"), ArgSpec((cfg.block_size, c), "bf16", "wpe")]
    per_layer = [
        ((c,), "f32"), ((c,), "f32"), ((c, 3 * cl), "bf16"), ((cl, c), "bf16"), ((c,), "f32"), ((c,), "f32"), ((c,), "f32"),
        ((c, hl), "bf16"), ((hl,), "f32"), ((hl, c), "bf16"), ((c,), "f32"),
    ]
    for li in range(cfg.n_layer):
        args += [ArgSpec(s, d, f"l{li}.{k}") for (s, d), k in zip(per_layer, GPT_LAYER_KEYS)]
    args += [ArgSpec((c,), "f32", "gf_g"), ArgSpec((c,), "f32", "gf_b"), ArgSpec((c, vl), "bf16", "lmw"), ArgSpec((vl,), "f32", "lmb")]
    p = Plan(name, args)
    x = p.temp((t, c), "f32")          # residual stream
    ln = p.temp((t, c), "bf16")
    qkv = p.temp((t, 3 * cl), "bf16")
    att = p.temp((t, cl), "bf16")
    hbuf = p.temp((t, hl), "bf16")
    p.embedding(x, p.arg(1), p.arg(2), p.arg(3), period=cfg.seq)

    def heads(view2d: PView, col0: int) -> PView:
        """(tokens, width) columns [col0, col0 + cl) as (batch, heads, seq, hs) without a copy."""
        v = view2d.slice(1, col0, cl)
        return PView(v.slot, (cfg.batch, heads_l, cfg.seq, hs), (cfg.seq * v.strides[0], hs, v.strides[0], 1), v.dtype, v.offset)

    first = rank == 0
    base = 4
    for li in range(cfg.n_layer):
        a = {k: p.arg(base + li * len(GPT_LAYER_KEYS) + i) for i, k in enumerate(GPT_LAYER_KEYS)}
        p.layernorm(ln, x, a["g1"], a["b1n"], cfg.eps)
        p.gemm(qkv, ln, a["wqkv"])
        p.attention(heads(att, 0), heads(qkv, 0), heads(qkv, cl), heads(qkv, 2 * cl), 1.0 / math.sqrt(hs), cfg.causal)
        p.gemm(x, att, a["wp"], bias=a["bp"], residual=x if first else None)
        if tp > 1:
            p.allreduce(x)
        p.layernorm(ln, x, a["g2"], a["b2n"], cfg.eps)
        p.gemm(hbuf, ln, a["w1"], bias=a["bb1"], act=cfg.act)
        p.gemm(x, hbuf, a["w2"], bias=a["bb2"], residual=x if first else None)
        if tp > 1:
            p.allreduce(x)
    tail = base + cfg.n_layer * len(GPT_LAYER_KEYS)
    p.layernorm(ln, x, p.arg(tail), p.arg(tail + 1), cfg.eps)
    p.gemm(p.arg(0), ln, p.arg(tail + 2), bias=p.arg(tail + 3))
    return p


def build_nanogpt_plan_overlapped(cfg: NanoGptConfig, rank: int, tp: int, microbatches: int = 2, reserve_sms: int = 8,
                                  name: str = "nanogpt_forward") -> Plan:
    """Same arguments and logits as ``build_nanogpt_plan`` (weights sharded with
    ``full_bias=True``), with the schedule of ``build_llama_plan_overlapped`` on NCCL calls: the
    f32 residual stream is sharded by rows, each contraction's bf16 partial sums are
    reduce-scattered, the rank adds them and the layer's bias to its rows, LayerNorm runs on
    those rows, and the normalised bf16 rows are all-gathered - on the side stream, under
    the other micro-batch's GEMMs."""
    check_tp(cfg, tp)
    check_overlap(cfg.tokens, cfg.batch, tp, microbatches)
    m = microbatches
    if (cfg.batch // m) % tp:
        raise ValueError(f"{cfg.batch // m} sequences per micro-batch do not split into {tp} row blocks of whole sequences")
    c, t, hs = cfg.n_embd, cfg.tokens, cfg.n_embd // cfg.n_head
    cl, hl, vl, heads_l = c // tp, cfg.hidden // tp, cfg.vocab // tp, cfg.n_head // tp
    args = [ArgSpec((t, vl), cfg.logits_dtype, "logits"), ArgSpec((t,), "i32", "ids"), ArgSpec((cfg.vocab, c), "bf16", "wte"), ArgSpec((cfg.block_size, c), "bf16", "wpe")]
    per_layer = [
        ((c,), "f32"), ((c,), "f32"), ((c, 3 * cl), "bf16"), ((cl, c), "bf16"), ((c,), "f32"), ((c,), "f32"), ((c,), "f32"),
        ((c, hl), "bf16"), ((hl,), "f32"), ((hl, c), "bf16"), ((c,), "f32"),
    ]
    for li in range(cfg.n_layer):
        args += [ArgSpec(s_, d_, f"l{li}.{k}") for (s_, d_), k in zip(per_layer, GPT_LAYER_KEYS)]
    args += [ArgSpec((c,), "f32", "gf_g"), ArgSpec((c,), "f32", "gf_b"), ArgSpec((c, vl), "bf16", "lmw"), ArgSpec((vl,), "f32", "lmb")]
    p = Plan(name, args)
    bm, tm = cfg.batch // m, t // m
    ts = tm // tp
    x = [p.temp((ts, c), "f32") for _ in range(m)]         # this rank's rows of the residual stream
    ln = [p.temp((tm, c), "bf16") for _ in range(m)]       # gathered normalised activations
    qkv = [p.temp((tm, 3 * cl), "bf16") for _ in range(m)]
    att = [p.temp((tm, cl), "bf16") for _ in range(m)]
    hbuf = [p.temp((tm, hl), "bf16") for _ in range(m)]
    part = [p.temp((tm, c), "bf16") for _ in range(m)]     # partial sums of a contraction
    rs = [p.temp((ts, c), "bf16") for _ in range(m)]
    chain = _SideChain(p, m)
    base = 4
    layer_args = lambda li: {k: p.arg(base + li * len(GPT_LAYER_KEYS) + i) for i, k in enumerate(GPT_LAYER_KEYS)}
    tail = base + cfg.n_layer * len(GPT_LAYER_KEYS)

    def heads(view2d: PView, col0: int) -> PView:
        v = view2d.slice(1, col0, cl)
        return PView(v.slot, (bm, heads_l, cfg.seq, hs), (cfg.seq * v.strides[0], hs, v.strides[0], 1), v.dtype, v.offset)

    def norm_and_gather(mb: int, gamma: PView, beta: PView) -> None:
        mine = ln[mb].slice(0, rank * ts, ts)
        p.layernorm(mine, x[mb], gamma, beta, cfg.eps)
        p.allgather(ln[mb], mine)

    def reduce_into_residual(mb: int, bias: PView) -> None:
        p.reducescatter(rs[mb], part[mb])
        p.elementwise("add", x[mb], x[mb], rs[mb])
        p.elementwise("add", x[mb], x[mb], bias)

    for mb in range(m):
        chain.fork()
        # rows of whole sequences: positions restart with each sequence, as in the full batch
        p.embedding(x[mb], p.arg(1).slice(0, mb * tm + rank * ts, ts), p.arg(2), p.arg(3), period=cfg.seq)
        norm_and_gather(mb, layer_args(0)["g1"], layer_args(0)["b1n"])
        chain.join(mb)
        if mb == 0:
            p.reserve_sms(reserve_sms)
    for li in range(cfg.n_layer):
        a = layer_args(li)
        for mb in range(m):
            p.event_wait(chain.ready[mb])
            p.gemm(qkv[mb], ln[mb], a["wqkv"])
            p.attention(heads(att[mb], 0), heads(qkv[mb], 0), heads(qkv[mb], cl), heads(qkv[mb], 2 * cl), 1.0 / math.sqrt(hs), cfg.causal)
            p.gemm(part[mb], att[mb], a["wp"])
            chain.fork()
            reduce_into_residual(mb, a["bp"])
            norm_and_gather(mb, a["g2"], a["b2n"])
            chain.join(mb)
        last = li == cfg.n_layer - 1
        for mb in range(m):
            p.event_wait(chain.ready[mb])
            p.gemm(hbuf[mb], ln[mb], a["w1"], bias=a["bb1"], act=cfg.act)
            p.gemm(part[mb], hbuf[mb], a["w2"])
            chain.fork()
            reduce_into_residual(mb, a["bb2"])
            nxt = (p.arg(tail), p.arg(tail + 1)) if last else (layer_args(li + 1)["g1"], layer_args(li + 1)["b1n"])
            norm_and_gather(mb, *nxt)
            chain.join(mb)
    p.reserve_sms(0)
    for mb in range(m):
        p.event_wait(chain.ready[mb])
        p.gemm(p.arg(0).slice(0, mb * tm, tm), ln[mb], p.arg(tail + 2), bias=p.arg(tail + 3))
    return p


def build_llama_plan(cfg: LlamaConfig, rank: int = 0, tp: int = 1, name: str = "llama_forward") -> Plan:
    """Args: ``out (tokens, dim) bf16, x (tokens, dim) bf16,
    [attention_norm, wqkv, wo, ffn_norm, w13, w2] * n_layer, norm``."""
    check_tp(cfg, tp)
    d, t, hd = cfg.dim, cfg.tokens, cfg.head_dim
    hq, hkv, fl = cfg.n_heads // tp, cfg.n_kv_heads // tp, cfg.ffn // tp
    ql, kl = hq * hd, hkv * hd
    width = ql + 2 * kl
    args = [ArgSpec((t, d), "bf16", "out"), ArgSpec((t, d), "bf16", "x")]
    per_layer = [((d,), "bf16"), ((width, d), "bf16"), ((d, ql), "bf16"), ((d,), "bf16"), ((2 * fl, d), "bf16"), ((d, fl), "bf16")]
    for li in range(cfg.n_layer):
        args += [ArgSpec(s, dt, f"l{li}.{k}") for (s, dt), k in zip(per_layer, LLAMA_LAYER_KEYS)]
    args.append(ArgSpec((d,), "bf16", "norm"))
    p = Plan(name, args)
    h = p.temp((t, d), "bf16")      # residual stream
    hn = p.temp((t, d), "bf16")
    qkv = p.temp((t, width), "bf16")
    att = p.temp((t, ql), "bf16")
    ff = p.temp((t, fl), "bf16")
    p.elementwise("copy", h, p.arg(1))

    def bshd(view2d: PView, col0: int, nheads: int) -> PView:
        v = view2d.slice(1, col0, nheads * hd)
        return PView(v.slot, (cfg.batch, cfg.seq, nheads, hd), (cfg.seq * v.strides[0], v.strides[0], hd, 1), v.dtype, v.offset)

    first = rank == 0
    for li in range(cfg.n_layer):
        a = {k: p.arg(2 + li * len(LLAMA_LAYER_KEYS) + i) for i, k in enumerate(LLAMA_LAYER_KEYS)}
        p.rmsnorm(hn, h, a["attention_norm"], cfg.eps)
        # q and k heads are the leading columns of the packed projection: rotated in its epilogue
        p.gemm_rope(qkv, hn, a["wqkv"].t(), ql + kl, hd, cfg.seq, cfg.theta, 0)
        q, k, v = bshd(qkv, 0, hq), bshd(qkv, ql, hkv), bshd(qkv, ql + kl, hkv)
        to_bhsd = lambda z: z.permute((0, 2, 1, 3))
        p.attention(to_bhsd(bshd(att, 0, hq)), to_bhsd(q), to_bhsd(k), to_bhsd(v), 1.0 / math.sqrt(hd), True)
        p.gemm(h, att, a["wo"].t(), residual=h if first else None)
        if tp > 1:
            p.allreduce(h)
        p.rmsnorm(hn, h, a["ffn_norm"], cfg.eps)
        p.gemm(ff, hn, a["w13"].t(), swiglu=True)
        p.gemm(h, ff, a["w2"].t(), residual=h if first else None)
        if tp > 1:
            p.allreduce(h)
    p.rmsnorm(p.arg(0), h, p.arg(len(args) - 1), cfg.eps)
    return p


class _SideChain:
    """Bookkeeping for plans that overlap collectives with compute: each micro-batch's
    contracting GEMM on the main stream is followed, on the side stream, by reduce-scatter ->
    residual add -> norm on this rank's rows -> all-gather, while the main stream runs the
    other micro-batch. ``ready[mb]`` is the event after which ``xn[mb]`` holds the gathered,
    normalised activations."""

    def __init__(self, p: Plan, microbatches: int):
        self.p = p
        self.next_event = 0
        self.ready = [None] * microbatches

    def event(self) -> int:
        self.next_event += 1
        return self.next_event - 1

    def fork(self) -> None:
        """Side stream continues from the main stream's current position."""
        e = self.event()
        self.p.event_record(e)
        self.p.stream(1)
        self.p.event_wait(e)

    def join(self, mb: int) -> None:
        """Back to the main stream; ``ready[mb]`` marks the side chain's end."""
        self.ready[mb] = self.event()
        self.p.event_record(self.ready[mb])
        self.p.stream(0)


def check_overlap(tokens: int, batch: int, tp: int, microbatches: int) -> None:
    if microbatches < 1 or batch % microbatches:
        raise ValueError(f"batch {batch} does not split into {microbatches} micro-batches of whole sequences")
    if (tokens // microbatches) % tp:
        raise ValueError(f"{tokens // microbatches} tokens per micro-batch do not split into {tp} row blocks")


def build_llama_plan_overlapped(cfg: LlamaConfig, rank: int, tp: int, microbatches: int = 2, reserve_sms: int = 16,
                                name: str = "llama_forward", fused: bool = False, result_symmetric: bool = False) -> Plan:
    """Same arguments and result as ``build_llama_plan``; different schedule for ``tp`` > 1.

    The all-reduce after each contraction is split into reduce-scatter + all-gather with the
    residual stream sharded by rows between them (each rank adds the residual and normalises
    1/tp of the tokens instead of all of them), and the batch is cut into micro-batches of
    whole sequences so that one micro-batch's collectives run on the side stream under the
    other's GEMMs and attention. Only the last collective of the step is exposed.

    ``fused``: reduce-scatter, residual add, RMSNorm and all-gather are ONE kernel over NVSwitch
    multicast memory (``lh_b200_reduce_norm_gather``) instead of two NCCL calls around two
    row kernels. The partial-sum and gathered-activation buffers are then symmetric memory
    the caller allocates: ``2 * microbatches`` extra arguments after ``norm``, per micro-batch
    ``part (tokens/microbatches, dim)`` then ``xn`` (same shape), see ``llama_symmetric_args``.
    ``result_symmetric`` (fused only): the caller's result buffer is symmetric memory registered
    with the context too, so the last layer's kernel gathers straight into it; otherwise the
    gathered rows are copied there from ``xn``."""
    check_tp(cfg, tp)
    check_overlap(cfg.tokens, cfg.batch, tp, microbatches)
    d, t, hd = cfg.dim, cfg.tokens, cfg.head_dim
    hq, hkv, fl = cfg.n_heads // tp, cfg.n_kv_heads // tp, cfg.ffn // tp
    ql, kl = hq * hd, hkv * hd
    width = ql + 2 * kl
    args = [ArgSpec((t, d), "bf16", "out"), ArgSpec((t, d), "bf16", "x")]
    per_layer = [((d,), "bf16"), ((width, d), "bf16"), ((d, ql), "bf16"), ((d,), "bf16"), ((2 * fl, d), "bf16"), ((d, fl), "bf16")]
    for li in range(cfg.n_layer):
        args += [ArgSpec(s, dt, f"l{li}.{k}") for (s, dt), k in zip(per_layer, LLAMA_LAYER_KEYS)]
    args.append(ArgSpec((d,), "bf16", "norm"))
    norm_index = len(args) - 1
    m = microbatches
    bm, tm = cfg.batch // m, t // m
    ts = tm // tp
    if fused:
        for mb in range(m):
            args += [ArgSpec((tm, d), "bf16", f"part{mb}"), ArgSpec((tm, d), "bf16", f"xn{mb}")]
    p = Plan(name, args)
    h = [p.temp((ts, d), "bf16") for _ in range(m)]       # this rank's rows of the residual stream
    # gathered normalised activations and this rank's partial sums of a contraction
    xn = [p.arg(norm_index + 2 + 2 * mb) if fused else p.temp((tm, d), "bf16") for mb in range(m)]
    part = [p.arg(norm_index + 1 + 2 * mb) if fused else p.temp((tm, d), "bf16") for mb in range(m)]
    qkv = [p.temp((tm, width), "bf16") for _ in range(m)]
    att = [p.temp((tm, ql), "bf16") for _ in range(m)]
    ff = [p.temp((tm, fl), "bf16") for _ in range(m)]
    rs = [None if fused else p.temp((ts, d), "bf16") for _ in range(m)]
    chain = _SideChain(p, m)
    layer_args = lambda li: {k: p.arg(2 + li * len(LLAMA_LAYER_KEYS) + i) for i, k in enumerate(LLAMA_LAYER_KEYS)}
    final_norm = p.arg(norm_index)

    def bshd(view2d: PView, col0: int, nheads: int) -> PView:
        v = view2d.slice(1, col0, nheads * hd)
        return PView(v.slot, (bm, cfg.seq, nheads, hd), (cfg.seq * v.strides[0], v.strides[0], hd, 1), v.dtype, v.offset)

    def norm_and_gather(mb: int, weight: PView, last: bool, reduce: bool = True) -> None:
        """On the side stream: (sum the partial sums of this rank's rows into the residual
        stream,) normalise those rows into their place in the gathered buffer (the result
        argument itself after the last layer) and gather."""
        if fused:
            if last and result_symmetric:
                p.reduce_norm_gather(p.arg(0).slice(0, mb * tm, tm), part[mb] if reduce else None, h[mb], weight, cfg.eps)
                return
            p.reduce_norm_gather(xn[mb], part[mb] if reduce else None, h[mb], weight, cfg.eps)
            if last:
                p.elementwise("copy", p.arg(0).slice(0, mb * tm, tm), xn[mb])
            return
        if reduce:
            p.reducescatter(rs[mb], part[mb])
            p.elementwise("add", h[mb], h[mb], rs[mb])
        full = p.arg(0).slice(0, mb * tm, tm) if last else xn[mb]
        mine = full.slice(0, rank * ts, ts)
        p.rmsnorm(mine, h[mb], weight, cfg.eps)
        p.allgather(full, mine)

    # Nothing runs beside the last micro-batch's last chain: it gets the whole GPU; before that
    # the GEMMs leave ``reserve_sms`` SMs to the side stream.
    # The input is replicated, so the first micro-batch's first norm needs no exchange: every rank
    # normalises all of its rows itself, on the main stream, which has nothing else to do yet
    # (a norm-and-gather there made the first GEMM wait for the slowest rank to arrive: 0.15 ms
    # at 8 GPUs). The other micro-batches' first chains run beside the first one's GEMMs.
    for mb in range(m):
        if mb == 0:
            p.elementwise("copy", h[0], p.arg(1).slice(0, rank * ts, ts))
            p.rmsnorm(xn[0], p.arg(1).slice(0, 0, tm), layer_args(0)["attention_norm"], cfg.eps)
            chain.ready[0] = chain.event()
            p.event_record(chain.ready[0])
            p.reserve_sms(reserve_sms)
            continue
        chain.fork()
        p.elementwise("copy", h[mb], p.arg(1).slice(0, mb * tm + rank * ts, ts))
        norm_and_gather(mb, layer_args(0)["attention_norm"], False, reduce=False)
        chain.join(mb)
    to_bhsd = lambda z: z.permute((0, 2, 1, 3))
    for li in range(cfg.n_layer):
        a = layer_args(li)
        for mb in range(m):
            p.event_wait(chain.ready[mb])
            # q and k heads are the leading columns of the packed projection: rotated in its epilogue
            p.gemm_rope(qkv[mb], xn[mb], a["wqkv"].t(), ql + kl, hd, cfg.seq, cfg.theta, 0)
            q, k, v = bshd(qkv[mb], 0, hq), bshd(qkv[mb], ql, hkv), bshd(qkv[mb], ql + kl, hkv)
            p.attention(to_bhsd(bshd(att[mb], 0, hq)), to_bhsd(q), to_bhsd(k), to_bhsd(v), 1.0 / math.sqrt(hd), True)
            p.gemm(part[mb], att[mb], a["wo"].t())
            chain.fork()
            norm_and_gather(mb, a["ffn_norm"], False)
            chain.join(mb)
        last = li == cfg.n_layer - 1
        for mb in range(m):
            p.event_wait(chain.ready[mb])
            p.gemm(ff[mb], xn[mb], a["w13"].t(), swiglu=True)
            p.gemm(part[mb], ff[mb], a["w2"].t())
            if last and mb == m - 1:
                p.reserve_sms(0)
            chain.fork()
            norm_and_gather(mb, final_norm if last else layer_args(li + 1)["attention_norm"], last)
            chain.join(mb)
    for mb in range(m):
        p.event_wait(chain.ready[mb])
    return p


def llama_symmetric_args(cfg: LlamaConfig, microbatches: int) -> list[tuple[int, int]]:
    """Shapes (bf16) of the symmetric buffers the fused schedule takes after ``norm``."""
    tm = cfg.tokens // microbatches
    return [(tm, cfg.dim)] * (2 * microbatches)


def flatten_nanogpt_args(w: dict) -> list:
    """Sharded weight dict -> argument list after ``logits, ids`` in plan order."""
    out = [w["wte"], w["wpe"]]
    for lw in w["layers"]:
        out += [lw[k] for k in GPT_LAYER_KEYS]
    return out + [w["gf_g"], w["gf_b"], w["lmw"], w["lmb"]]


def flatten_llama_args(w: dict) -> list:
    out = []
    for lw in w["layers"]:
        out += [lw[k] for k in LLAMA_LAYER_KEYS]
    return out + [w["norm"]]
