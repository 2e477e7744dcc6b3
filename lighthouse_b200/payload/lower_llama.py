"""Recognition of the Llama builders' op sequences (``llama_gen.py``, i.e. the linalg builders
of examples/llama/test_llama3.py in the reference) on top of the generic recogniser.

The builders spell every torch operation out of small linalg ops. What they compute per group:

* ``get_l2_norm``: square, scaled row reduction into (..., 1), + eps, rsqrt, broadcast, multiply
  -> ONE weight-less RMS norm operator;
* ``get_linear``: zero fill, ``linalg.contract`` over the last dims of a[..., k] and w[j, k],
  broadcast bias, add -> ONE GEMM with W read as (out, in) and the bias in its epilogue (a
  bias that is a zero fill is dropped);
* ``get_silu`` -> the SiLU activation; the product with the up projection stays an
  elementwise multiply (the epilogue fusion pass may fold what follows);
* ``get_rotary_emb``: pairs viewed as complex, multiplied by ``complex(freqs, 0)``, viewed as
  real again -> one elementwise multiply per batch entry of the (seq, heads, pairs, 2) view by
  the (seq, 1, pairs, 1) frequencies: nothing complex ever exists in memory;
* ``get_repeat_kv`` (``h floordiv n_rep``) -> no data movement: the attention operator reads
  kv head h / n_rep itself;
* transposes and reshapes -> views;
* scores contraction, scale, additive mask, softmax, weights-times-values contraction -> the
  flash-attention operator when the mask is absent or provably causal (built in the payload
  from ``linalg.index``); with a mask OPERAND, whose values the backend cannot know, the
  un-fused sequence per batch entry: batched GEMM, scale, add mask, softmax, batched GEMM.

Symbolic values carry the partial patterns between ops (kinds ``sq``, ``meansq``,
``meansq_eps``, ``rstd``, ``rstd_bcast``, ``cplx``, ``cplx_real``, ``cplx_scaled``,
``cplx_re_written``, ``repeat_kv``, ``causal_mask``, ``scores``, ``probs``).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

from ..plan import PView


@dataclass
class Scores:
    """Q K^T of (B, H, S, D) views, with what has been applied to it so far."""

    q: PView          # (B, H, Sq, D)
    k: PView          # (B, Hkv, Skv, D): before repeat_kv
    n_rep: int
    scale: float = 1.0
    mask: object = None  # None | "causal" | PView (additive operand)


def _as_matrix(v: PView):
    """(d0, ..., dk, n) -> (d0 * ... * dk, n) without moving data, or None: the leading dims must
    nest (or all be broadcast with stride 0)."""
    if v.rank <= 2:
        return v
    lead_shape, lead_strides = v.shape[:-1], v.strides[:-1]
    rows = math.prod(lead_shape)
    if all(s == 0 or d == 1 for d, s in zip(lead_shape, lead_strides)):
        return PView(v.slot, (rows, v.shape[-1]), (0, v.strides[-1]), v.dtype, v.offset)
    stride = None
    expect = None
    for d, s in zip(reversed(lead_shape), reversed(lead_strides)):
        if d == 1:
            continue
        if expect is None:
            stride, expect = s, s * d
        elif s != expect:
            return None
        else:
            expect *= d
    return PView(v.slot, (rows, v.shape[-1]), (stride if stride is not None else v.shape[-1], v.strides[-1]), v.dtype, v.offset)


class LlamaPatterns:
    # ------------------------------------------------------------------ linalg.elementwise
    def op_linalg_elementwise(self, op):
        from . import lower as L

        kind = op.attrs["kind"]
        ins = [self.tv(v) for v in op.ins]
        out_tv = self.tv(op.outs[0])
        out_t = op.outs[0].type
        TV = L.TV

        def plain(ew, a, b=None, **kw):
            dst = self.dest_for(out_tv, out_t.shape, out_t.dtype)
            va, vb = self.as_view(a, op.name), None if b is None else self.as_view(b, op.name)
            # (batch, seq, n) operands as (rows, n) matrices where their strides allow it: the
            # form in which the epilogue fusion recognises a bias, an activation or a residual
            flat = [_as_matrix(v) for v in (dst, va, vb) if v is not None]
            if dst.rank > 2 and all(f is not None for f in flat):
                self.plan.elementwise(ew, flat[0], flat[1], flat[2] if vb is not None else None, **kw)
            else:
                self.plan.elementwise(ew, dst, va, vb, **kw)
            self.bind(op, TV("view", dst.shape, dst.dtype, dst))

        if kind == "square":
            return self.bind(op, TV("sq", out_t.shape, out_t.dtype, src=ins[0]))
        if kind == "rsqrt":
            if ins[0].kind != "meansq_eps":
                raise L.UnsupportedPayload("linalg.elementwise rsqrt outside an RMS-norm pattern")
            return self.bind(op, TV("rstd", out_t.shape, out_t.dtype, src=ins[0].src))
        if kind == "add":
            a, b = ins
            for x, y in ((a, b), (b, a)):
                if x.kind == "meansq" and y.kind == "fill":
                    return self.bind(op, TV("meansq_eps", out_t.shape, out_t.dtype, src=(x.src[0], float(y.scalar))))
                if x.kind == "scores":
                    sc: Scores = x.src
                    if sc.mask is not None:
                        raise L.UnsupportedPayload("attention scores with two masks")
                    mask = "causal" if y.kind == "causal_mask" else self.as_view(y, "attention mask")
                    return self.bind(op, TV("scores", out_t.shape, out_t.dtype, src=Scores(sc.q, sc.k, sc.n_rep, sc.scale, mask)))
                if y.kind == "fill" and y.scalar == 0.0 and x.kind == "view":
                    return self.bind(op, x)  # + zero bias
            return plain("add", a, b)
        if kind == "mul":
            a, b = ins
            for x, y in ((a, b), (b, a)):
                if y.kind == "rstd_bcast":
                    if y.src[0] is not x:
                        raise L.UnsupportedPayload("RMS-norm pattern: the scale was computed from another tensor")
                    dst = self.dest_for(out_tv, out_t.shape, out_t.dtype)
                    xv = self.as_view(x, "rms norm")
                    rows = math.prod(dst.shape[:-1])
                    self.plan.rmsnorm(dst.reshape((rows, dst.shape[-1])), xv.reshape((rows, xv.shape[-1])), None, y.src[1])
                    return self.bind(op, TV("view", dst.shape, dst.dtype, dst))
                if x.kind == "scores" and y.kind == "fill":
                    sc = x.src
                    return self.bind(op, TV("scores", out_t.shape, out_t.dtype, src=Scores(sc.q, sc.k, sc.n_rep, sc.scale * float(y.scalar), sc.mask)))
            return plain("mul", a, b)
        raise L.UnsupportedPayload(f"linalg.elementwise kind '{kind}' is not supported")

    # ------------------------------------------------------------------------ linalg.generic
    def try_llama_generic(self, op, e, maps, iters) -> bool:
        """True if the generic was one of the Llama builders' and has been handled."""
        from . import lower as L

        TV = L.TV
        ins = [self.tv(v) for v in op.ins]
        out_t = op.outs[0].type
        out_tv = self.tv(op.outs[0])
        n_in = len(ins)
        rank = maps[-1].n_dims

        def const_last(m, value):
            return m.special == {len(m.results) - 1: ("const", value)} and m.results[:-1] == tuple(range(len(m.results) - 1))

        # causal mask from indices: select(cmpi sgt(index last, index last-1), -inf, 0)
        if n_in == 0 and L._is(e, "arith.select", 3):
            c, a, b = e[2], e[3], e[4]
            if (isinstance(c, tuple) and c[:3] == ("op", "arith.cmpi", "sgt") and c[3] == ("op", "linalg.index", rank - 1) and c[4] == ("op", "linalg.index", rank - 2)
                    and L._const(a) and a[1] == float("-inf") and L._const(b, 0.0) and rank >= 2 and out_t.shape[-1] == out_t.shape[-2]):
                self.bind(op, TV("causal_mask", out_t.shape, out_t.dtype))
                return True
            return False
        if n_in == 0:
            return False
        # mean of squares: addf(mulf(x, 1/N), acc) reduced over the last dim into (..., 1)
        if ins[0].kind == "sq":
            if not (n_in == 1 and iters[-1] == "reduction" and maps[0].is_identity() and const_last(maps[1], 0) and out_tv.kind == "fill" and out_tv.scalar == 0.0 and L._is(e, "arith.addf", 2)):
                raise L.UnsupportedPayload("a squared tensor is only recognised inside the RMS-norm pattern")
            pair = L._commutative_pair(e, lambda t: L._is(t, "arith.mulf", 2), lambda t: L._arg(t, 1))
            scaled = pair and L._commutative_pair(pair[0], lambda t: L._arg(t, 0), lambda t: L._const(t))
            n = ins[0].shape[-1]
            if not scaled or abs(scaled[1][1] * n - 1.0) > 1e-6:
                raise L.UnsupportedPayload("RMS-norm pattern: the reduction does not scale by 1/N")
            self.bind(op, TV("meansq", out_t.shape, out_t.dtype, src=(ins[0].src,)))
            return True
        # rstd (..., 1) broadcast along the last dim
        if ins[0].kind == "rstd":
            if not (n_in == 1 and L._arg(e, 0) and const_last(maps[0], 0) and maps[1].is_identity()):
                raise L.UnsupportedPayload("RMS-norm pattern: unexpected use of the reciprocal norm")
            self.bind(op, TV("rstd_bcast", out_t.shape, out_t.dtype, src=ins[0].src))
            return True
        all_par = all(i == "parallel" for i in iters)
        # silu: x * (1 / (1 + exp(-x)))
        if all_par and n_in == 1 and ins[0].kind == "view" and all(m.is_identity() for m in maps) and L._is(e, "arith.mulf", 2):
            pair = L._commutative_pair(e, lambda t: L._arg(t, 0), lambda t: L._is(t, "arith.divf", 2))
            if pair:
                d = pair[1]
                den = d[3]
                if L._const(d[2], 1.0) and L._is(den, "arith.addf", 2):
                    ex = L._commutative_pair(den, lambda t: L._const(t, 1.0), lambda t: L._is(t, "math.exp", 1))
                    if ex and L._is(ex[1][2], "arith.negf", 1) and L._arg(ex[1][2][2], 0):
                        dst = self.dest_for(out_tv, out_t.shape, out_t.dtype)
                        d2, x2 = _as_matrix(dst), _as_matrix(ins[0].view)
                        if d2 is not None and x2 is not None:
                            self.plan.elementwise("act", d2, x2, act="silu")
                        else:
                            self.plan.elementwise("act", dst, ins[0].view, act="silu")
                        self.bind(op, TV("view", dst.shape, dst.dtype, dst))
                        return True
        # repeat_kv: out[b, s, h, d] = x[b, s, h floordiv n_rep, d]
        if all_par and n_in == 1 and L._arg(e, 0) and maps[0].special and list(maps[0].special.values())[0][0] == "floordiv":
            (pos, (_, n_rep)), = maps[0].special.items()
            if not (rank == 4 and pos == 2 and maps[0].results == (0, 1, 2, 3) and maps[1].is_identity() and ins[0].kind == "view"):
                raise L.UnsupportedPayload("floordiv index map outside the repeat_kv pattern")
            self.bind(op, TV("repeat_kv", out_t.shape, out_t.dtype, src=(ins[0].view, int(n_rep))))
            return True
        # pure re-indexing of a real tensor (reshape_for_broadcast: freqs[s, p] -> (1, s, 1, p))
        if all_par and n_in == 1 and L._arg(e, 0) and ins[0].kind == "view" and maps[0].is_plain() and maps[1].is_identity() and not str(out_t.dtype).startswith("complex"):
            if out_tv.kind == "empty" and len(maps[0].results) == ins[0].view.rank and list(maps[0].results) == sorted(maps[0].results):
                missing = set(range(rank)) - set(maps[0].results)
                v = ins[0].view.broadcast_to(out_t.shape, missing)
                # the added dims have extent 1 here or are true broadcasts: either way a view
                self.bind(op, TV("view", out_t.shape, out_t.dtype, v))
                return True
            return False
        # ---- the complex detour of get_rotary_emb
        if L._is(e, "complex.create", 2):
            if n_in == 2 and op.ins[0] is op.ins[1] and L._arg(e[2], 0) and L._arg(e[3], 1) and const_last(maps[0], 0) and const_last(maps[1], 1) and ins[0].kind == "view":
                self.bind(op, TV("cplx", out_t.shape, out_t.dtype, src=ins[0].view))  # (..., pairs, 2) real view
                return True
            if n_in == 1 and L._arg(e[2], 0) and L._const(e[3], 0.0) and ins[0].kind == "view" and all(m.is_identity() for m in maps):
                self.bind(op, TV("cplx_real", out_t.shape, out_t.dtype, src=ins[0].view))
                return True
            raise L.UnsupportedPayload("complex.create outside the rotary-embedding pattern")
        if L._is(e, "complex.mul", 2):
            kinds = sorted(t.kind for t in ins)
            if not (n_in == 2 and kinds == ["cplx", "cplx_real"] and {e[2], e[3]} == {("arg", 0), ("arg", 1)}):
                raise L.UnsupportedPayload("complex.mul is only supported as (pairs) x (real frequencies)")
            xi = 0 if ins[0].kind == "cplx" else 1
            fmap = maps[1 - xi]
            if not maps[xi].is_identity() or any(sp[0] != "const" or sp[1] != 0 for sp in fmap.special.values()):
                raise L.UnsupportedPayload("rotary embedding: unexpected broadcast of the frequencies")
            f = ins[1 - xi].src  # real view, rank == out rank, extent 1 where broadcast
            strides = tuple(0 if (i in fmap.special or f.shape[i] == 1) else f.strides[i] for i in range(f.rank))
            fb = PView(f.slot, tuple(out_t.shape), strides, f.dtype, f.offset)
            self.bind(op, TV("cplx_scaled", out_t.shape, out_t.dtype, src=(ins[xi].src, fb)))
            return True
        if L._is(e, "complex.re", 1) or L._is(e, "complex.im", 1):
            part = 0 if e[1] == "complex.re" else 1
            if not (n_in == 1 and ins[0].kind == "cplx_scaled" and L._arg(e[2], 0) and maps[0].is_identity() and const_last(maps[1], part)):
                raise L.UnsupportedPayload("complex.re / complex.im outside the rotary-embedding pattern")
            if part == 0:
                self.bind(op, TV("cplx_re_written", out_t.shape, out_t.dtype, src=ins[0].src))
                return True
            if out_tv.kind != "cplx_re_written" or out_tv.src is not ins[0].src:
                raise L.UnsupportedPayload("rotary embedding: imaginary parts must complete the tensor the real parts went to")
            x5, f4 = ins[0].src  # (B, S, H, P, 2) real view; (B, S, H, P) frequencies with zero strides
            dst = self.plan.temp(out_t.shape, out_t.dtype)
            for b in range(x5.shape[0]):  # operators take at most rank-4 views: one per batch entry
                xb, db = x5.slice(0, b, 1), dst.slice(0, b, 1)
                fbv = f4.slice(0, b, 1)
                drop = lambda v: PView(v.slot, v.shape[1:], v.strides[1:], v.dtype, v.offset)
                f5 = PView(fbv.slot, fbv.shape[1:] + (2,), fbv.strides[1:] + (0,), fbv.dtype, fbv.offset)
                self.plan.elementwise("mul", drop(db), drop(xb), f5)
            self.bind(op, TV("view", dst.shape, dst.dtype, dst))
            return True
        return False

    # -------------------------------------------------------------------- views of markers
    def llama_transpose(self, op) -> bool:
        """linalg.transpose of a repeat_kv marker keeps the marker (on the permuted view)."""
        from . import lower as L

        src = self.tv(op.ins[0])
        if src.kind != "repeat_kv":
            return False
        v, n_rep = src.src
        perm = op.attrs["permutation"]
        out_t = op.outs[0].type
        self.bind(op, L.TV("repeat_kv", out_t.shape, out_t.dtype, src=(v.permute(perm), n_rep)))
        return True

    # ----------------------------------------------------------------------- linalg.contract
    def op_linalg_contract(self, op):
        from . import lower as L

        TV = L.TV
        maps = [m.results for m in op.attrs["indexing_maps"]]
        if any(not m.is_plain() for m in op.attrs["indexing_maps"]):
            raise L.UnsupportedPayload("linalg.contract with non-trivial index expressions")
        a_tv, b_tv = self.tv(op.ins[0]), self.tv(op.ins[1])
        acc = self.tv(op.outs[0])
        out_t = op.outs[0].type
        if acc.kind != "fill" or acc.scalar != 0.0:
            raise L.UnsupportedPayload("linalg.contract must accumulate into a zero fill")
        n = op.attrs["indexing_maps"][0].n_dims
        # linear: a[..., k] w[j, k] -> out[..., j]
        ar = len(maps[0])
        if n == ar + 1 and maps[0] == tuple(range(ar - 1)) + (n - 1,) and maps[1] == (ar - 1, n - 1) and maps[2] == tuple(range(ar)):
            a = self.as_view(a_tv, op.name)
            w = self.as_view(b_tv, op.name)
            dst = acc.view if acc.view is not None else self.plan.temp(out_t.shape, out_t.dtype)
            rows = math.prod(a.shape[:-1])
            try:
                a2, d2 = a.reshape((rows, a.shape[-1])), dst.reshape((rows, dst.shape[-1]))
            except ValueError as err:
                raise L.UnsupportedPayload(f"linalg.contract (linear): {err}")
            self.plan.gemm(d2, a2, w.t())
            return self.bind(op, TV("view", dst.shape, dst.dtype, dst))
        # scores: q[b, h, s1, d] k[b, h, s2, d] -> [b, h, s1, s2]
        if n == 5 and maps == [(0, 1, 2, 4), (0, 1, 3, 4), (0, 1, 2, 3)]:
            q = self.as_view(a_tv, op.name)
            if b_tv.kind == "repeat_kv":
                k, n_rep = b_tv.src
            else:
                k, n_rep = self.as_view(b_tv, op.name), 1
            return self.bind(op, TV("scores", out_t.shape, out_t.dtype, src=Scores(q, k, n_rep)))
        # weighted values: p[b, h, s1, s2] v[b, h, s2, d] -> [b, h, s1, d]
        if n == 5 and maps == [(0, 1, 2, 3), (0, 1, 3, 4), (0, 1, 2, 4)] and a_tv.kind == "probs":
            sc: Scores = a_tv.src
            if b_tv.kind == "repeat_kv":
                v, v_rep = b_tv.src
            else:
                v, v_rep = self.as_view(b_tv, op.name), 1
            if v_rep != sc.n_rep:
                raise L.UnsupportedPayload("attention: keys and values are repeated differently")
            if acc.view is not None:
                dst = acc.view
            else:
                # stored (B, S, H, D): the transpose and the collapse to (B, S, H D) that follow in
                # the builders are then views, and the output projection reads it as a matrix
                b_, h_, s_, d_ = out_t.shape
                dst = self.plan.temp((b_, s_, h_, d_), out_t.dtype).permute((0, 2, 1, 3))
            if sc.mask is None or sc.mask == "causal":
                self.plan.attention(dst, sc.q, sc.k, v, sc.scale, sc.mask == "causal")
            else:
                self._unfused_attention(dst, sc, v)
            return self.bind(op, TV("view", dst.shape, dst.dtype, dst))
        raise L.UnsupportedPayload(f"linalg.contract with maps {maps} is not a pattern this backend knows")

    def llama_softmax(self, op) -> bool:
        from . import lower as L

        x = self.tv(op.ins[0])
        if x.kind != "scores":
            return False
        out_t = op.outs[0].type
        if op.attrs.get("dimension") != len(out_t.shape) - 1:
            raise L.UnsupportedPayload("attention: softmax must run over the keys")
        self.bind(op, L.TV("probs", out_t.shape, out_t.dtype, src=x.src))
        return True

    def _unfused_attention(self, dst: PView, sc: Scores, v: PView) -> None:
        """Additive mask given as data: the builders' own sequence, per batch entry (operators
        take rank-3 batched products and rank-4 views): scores = q k^T, * scale, + mask, softmax,
        times v. Grouped heads are expanded into a temporary the way ``get_repeat_kv`` writes
        them out."""
        B, H, Sq, D = sc.q.shape
        Skv = sc.k.shape[2]
        dt = sc.q.dtype
        drop = lambda t: PView(t.slot, t.shape[1:], t.strides[1:], t.dtype, t.offset)

        def repeated(t: PView, b: int) -> PView:
            """(Hkv, S, D) view of batch entry b -> (H, S, D) with head h reading kv head h // n_rep."""
            tb = drop(t.slice(0, b, 1))
            if sc.n_rep == 1:
                return tb
            hkv = tb.shape[0]
            rep = self.plan.temp((hkv, sc.n_rep, tb.shape[1], D), dt)
            src = PView(tb.slot, (hkv, sc.n_rep, tb.shape[1], D), (tb.strides[0], 0, tb.strides[1], tb.strides[2]), tb.dtype, tb.offset)
            self.plan.elementwise("copy", rep, src)
            return rep.reshape((H, tb.shape[1], D))

        scores = self.plan.temp((H, Sq, Skv), dt)
        for b in range(B):
            kb, vb = repeated(sc.k, b), repeated(v, b)
            self.plan.gemm(scores, drop(sc.q.slice(0, b, 1)), kb.t())
            self.plan.elementwise("scale", scores, scores, scalar=sc.scale)
            self.plan.elementwise("add", scores, scores, drop(sc.mask.slice(0, b, 1)))
            self.plan.softmax(scores, scores)
            self.plan.gemm(drop(dst.slice(0, b, 1)), scores, vb)
