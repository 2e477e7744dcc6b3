"""The Llama block as MLIR payloads: the linalg builders of the reference's Llama example
(examples/llama/test_llama3.py:140-947), emitted op for op on the in-memory IR.

Each ``l_*`` function follows the builder it names: ``get_linear`` (W in (out, in) layout as a
``linalg.contract`` over the last dims, plus a broadcast bias), ``get_l2_norm`` (square, mean
as a scaled reduction, + eps, rsqrt, broadcast, multiply: an RMS norm without learned weight),
``get_silu`` (x * 1 / (1 + exp(-x))), ``get_rotary_emb`` (pairs viewed as complex numbers and
multiplied by ``complex(freqs, 0)``: a scaling of each pair by a real frequency, as the
reference has it), ``get_repeat_kv`` (``h floordiv n_rep`` index map), ``get_attention``
(projections, rotary, repeat, transposes, scores as a contraction, scale, additive mask,
softmax, weighted values, output projection), ``get_transformer_block`` and
``get_transformer``.

The payload functions take buffers GPU-payload style: the result first, then the inputs.
``mask`` selects how the attention mask reaches the payload: ``"operand"`` (an additive
(B, H, S, S) tensor argument, what the reference's tests pass), ``"none"``, or ``"causal"``
(an extension: the additive -inf strictly-upper-triangular mask is built inside the payload
from ``linalg.index``, which lets the backend prove causality and take the flash kernel).
"""

from __future__ import annotations

import math

from .builder import PARALLEL, REDUCTION, FuncBuilder, affine_map, identity_map
from .ir import AffineMap, PayloadModule, memref_t


def _shape(v):
    return tuple(v.type.shape)


def l_add(fb, a, b, out):
    return fb.elementwise("add", [a, b], out)


def l_mul(fb, a, b, out):
    return fb.elementwise("mul", [a, b], out)


def l_sqr(fb, a, out):
    return fb.elementwise("square", [a], out)


def l_rsqrt(fb, a, out):
    return fb.elementwise("rsqrt", [a], out)


def l_mean(fb, a, out):
    """get_mean (test_llama3.py:156-195): torch.mean(-1, keepdim=True) as a reduction that
    adds ``a * (1 / N)`` into a zero-filled (..., 1) tensor."""
    dt, rank = a.type.dtype, a.type.rank
    zero = fb.constant(0.0, dt)
    filled = fb.fill(zero, out)
    in_map = identity_map(rank)
    out_map = AffineMap(rank, tuple(range(rank - 1)) + (-1,), {rank - 1: ("const", 0)})
    scale = fb.constant(1.0 / _shape(a)[-1], dt)
    return fb.generic([a], [filled], [in_map, out_map], [PARALLEL] * (rank - 1) + [REDUCTION], lambda rb, v, acc: rb.addf(rb.mulf(v, scale), acc))


def l_l2_norm(fb, a, out, eps: float = 1e-5):
    """get_l2_norm (test_llama3.py:328-370): x * rsqrt(mean(x^2, -1, keepdim) + eps)."""
    dt, rank = a.type.dtype, a.type.rank
    reduced = _shape(a)[:-1] + (1,)
    eps_t = fb.fill(fb.constant(eps, dt), fb.empty(reduced, dt))
    sqr = l_sqr(fb, a, fb.empty(_shape(a), dt))
    mean_buf = fb.empty(reduced, dt)
    mean = l_mean(fb, sqr, mean_buf)
    mean_eps = l_add(fb, mean, eps_t, mean_buf)
    rstd = l_rsqrt(fb, mean_eps, mean_buf)
    in_map = AffineMap(rank, tuple(range(rank - 1)) + (-1,), {rank - 1: ("const", 0)})
    bcast = fb.generic([rstd], [out], [in_map, identity_map(rank)], [PARALLEL] * rank, lambda rb, v, _o: v)
    return l_mul(fb, a, bcast, out)


def l_linear(fb, a, w, b, out):
    """get_linear (test_llama3.py:290-324): a[..., k] * w[j, k] -> out[..., j] as a contraction
    into a zero fill, plus the bias broadcast over the leading dims."""
    dt = out.type.dtype
    zeroed = fb.fill(fb.constant(0.0, dt), out)
    ar = a.type.rank
    n = ar + 1
    batch = tuple(range(ar - 1))
    k, j = n - 1, ar - 1
    res = fb.contract(a, w, zeroed, [affine_map(n, batch + (k,)), affine_map(n, (j, k)), affine_map(n, batch + (j,))])
    bias = fb.broadcast(b, out, list(range(out.type.rank - 1)))
    return l_add(fb, res, bias, out)


def l_silu(fb, x, out):
    """get_silu (test_llama3.py:225-249): x * (1 / (1 + exp(-x)))."""
    dt, rank = x.type.dtype, x.type.rank
    one = fb.constant(1.0, dt)
    return fb.generic([x], [out], [identity_map(rank)] * 2, [PARALLEL] * rank, lambda rb, a, _o: rb.mulf(a, rb.divf(one, rb.addf(one, rb.exp(rb.negf(a))))))


def l_repeat_kv(fb, x, n_rep: int, out):
    """get_repeat_kv (test_llama3.py:198-221): output head h reads input head h floordiv n_rep."""
    if n_rep == 1:
        return x
    x_map = AffineMap(4, (0, 1, 2, 3), {2: ("floordiv", n_rep)})
    return fb.generic([x], [out], [x_map, identity_map(4)], [PARALLEL] * 4, lambda rb, a, _o: a)


def _view_as_complex(fb, x5, out):
    """get_view_as_complex (test_llama3.py:576-604): (..., 2) -> complex (...)."""
    r = x5.type.rank - 1
    dims = tuple(range(r))
    m_re = AffineMap(r, dims + (-1,), {r: ("const", 0)})
    m_im = AffineMap(r, dims + (-1,), {r: ("const", 1)})
    return fb.generic([x5, x5], [out], [m_re, m_im, identity_map(r)], [PARALLEL] * r, lambda rb, re, im, _o: rb.complex_create(re, im))


def _view_as_real(fb, xc, out):
    """get_view_as_real (test_llama3.py:607-646): real parts to [..., 0], then imaginary parts
    to [..., 1] of the same tensor."""
    r = xc.type.rank
    dims = tuple(range(r))
    m_re = AffineMap(r, dims + (-1,), {r: ("const", 0)})
    m_im = AffineMap(r, dims + (-1,), {r: ("const", 1)})
    re = fb.generic([xc], [out], [identity_map(r), m_re], [PARALLEL] * r, lambda rb, c, _o: rb.complex_re(c))
    return fb.generic([xc], [re], [identity_map(r), m_im], [PARALLEL] * r, lambda rb, c, _o: rb.complex_im(c))


def _complex_mul(fb, a, b, out):
    """get_complex_mul (test_llama3.py:424-454), b broadcast along its size-1 dims."""
    r = out.type.rank
    b_special = {i: ("const", 0) for i, d in enumerate(_shape(b)) if d == 1}
    b_map = AffineMap(r, tuple(-1 if i in b_special else i for i in range(r)), b_special)
    return fb.generic([a, b], [out], [identity_map(r), b_map, identity_map(r)], [PARALLEL] * r, lambda rb, x, y, _o: rb.complex_mul(x, y))


def l_rotary_emb(fb, xq, xk, freqs, xq_out, xk_out):
    """get_rotary_emb (test_llama3.py:457-558)."""
    dt = xq.type.dtype
    cdt = f"complex<{dt}>"
    seq, half = _shape(freqs)
    # freqs[seq, half] -> (1, seq, 1, half), then complex with a zero imaginary part
    fshape = (1, seq, 1, half)
    fb_real = fb.generic([freqs], [fb.empty(fshape, dt)], [affine_map(4, (1, 3)), identity_map(4)], [PARALLEL] * 4, lambda rb, v, _o: v)
    zero = fb.constant(0.0, dt)
    fb_cplx = fb.generic([fb_real], [fb.empty(fshape, cdt)], [identity_map(4)] * 2, [PARALLEL] * 4, lambda rb, r, _o: rb.complex_create(r, zero))
    outs = []
    for x, x_out in ((xq, xq_out), (xk, xk_out)):
        b, s, h, d = _shape(x)
        x5 = fb.expand_shape(x, (b, s, h, d // 2, 2), [[0], [1], [2], [3, 4]])
        xc = _view_as_complex(fb, x5, fb.empty((b, s, h, d // 2), cdt))
        rot = _complex_mul(fb, xc, fb_cplx, fb.empty((b, s, h, d // 2), cdt))
        real = _view_as_real(fb, rot, fb.empty((b, s, h, d // 2, 2), dt))
        flat = fb.collapse_shape(real, (b, s, h, d), [[0], [1], [2], [3, 4]])
        outs.append(fb.copy(flat, x_out))
    return outs


def l_causal_mask(fb, shape, dt):
    """Extension: the additive mask of the torch model (``triu(full(-inf), diagonal=1)``,
    examples/llama/ref_model.py:266-278) built inside the payload."""
    rank = len(shape)
    ninf, zero = fb.constant(float("-inf"), dt), fb.constant(0.0, dt)

    def body(rb, _o):
        return rb.select(rb.cmpi("sgt", rb.index(rank - 1), rb.index(rank - 2)), ninf, zero)

    return fb.generic([], [fb.empty(shape, dt)], [identity_map(rank)], [PARALLEL] * rank, body)


def l_attention(fb, x, wq, wk, wv, wo, freqs, mask, out, n_heads: int, n_kv_heads: int):
    """get_attention (test_llama3.py:650-839)."""
    dt = x.type.dtype
    batch, seq, dim = _shape(x)
    hd = dim // n_heads
    n_rep = n_heads // n_kv_heads
    zero = fb.constant(0.0, dt)

    def proj(w, heads):
        bias = fb.fill(zero, fb.empty((heads * hd,), dt))
        flat = l_linear(fb, x, w, bias, fb.empty((batch, seq, heads * hd), dt))
        return fb.expand_shape(flat, (batch, seq, heads, hd), [[0], [1], [2, 3]])

    xq, xk, xv = proj(wq, n_heads), proj(wk, n_kv_heads), proj(wv, n_kv_heads)
    xq_rot, xk_rot = l_rotary_emb(fb, xq, xk, freqs, fb.empty((batch, seq, n_heads, hd), dt), fb.empty((batch, seq, n_kv_heads, hd), dt))
    keys = l_repeat_kv(fb, xk_rot, n_rep, fb.empty((batch, seq, n_heads, hd), dt))
    values = l_repeat_kv(fb, xv, n_rep, fb.empty((batch, seq, n_heads, hd), dt))
    bhsd = (batch, n_heads, seq, hd)
    perm = [0, 2, 1, 3]
    q_t = fb.transpose(xq_rot, fb.empty(bhsd, dt), perm)
    k_t = fb.transpose(keys, fb.empty(bhsd, dt), perm)
    v_t = fb.transpose(values, fb.empty(bhsd, dt), perm)
    sshape = (batch, n_heads, seq, seq)
    scores0 = fb.fill(zero, fb.empty(sshape, dt))
    # b, h, s1, s2, d
    scores = fb.contract(q_t, k_t, scores0, [affine_map(5, (0, 1, 2, 4)), affine_map(5, (0, 1, 3, 4)), affine_map(5, (0, 1, 2, 3))])
    scaled_buf = fb.empty(sshape, dt)
    scale_t = fb.fill(fb.constant(1.0 / math.sqrt(hd), dt), scaled_buf)
    scaled = l_mul(fb, scores, scale_t, scaled_buf)
    final = l_add(fb, scaled, mask, scaled) if mask is not None else scaled
    weights = fb.softmax(final, fb.empty(sshape, dt), 3)
    out0 = fb.fill(zero, fb.empty(bhsd, dt))
    attn = fb.contract(weights, v_t, out0, [affine_map(5, (0, 1, 2, 3)), affine_map(5, (0, 1, 3, 4)), affine_map(5, (0, 1, 2, 4))])
    attn_t = fb.transpose(attn, fb.empty((batch, seq, n_heads, hd), dt), perm)
    flat = fb.collapse_shape(attn_t, (batch, seq, n_heads * hd), [[0], [1], [2, 3]])
    bo = fb.fill(zero, fb.empty((dim,), dt))
    return l_linear(fb, flat, wo, bo, out)


def l_transformer_block(fb, x, w, freqs, mask, out, n_heads, n_kv_heads, eps):
    """get_transformer_block (test_llama3.py:842-903); ``w`` maps wq, wk, wv, wo, w1, b1, w2,
    b2, w3, b3 to values."""
    dt = x.type.dtype
    shape = _shape(x)
    x_norm = l_l2_norm(fb, x, fb.empty(shape, dt), eps)
    attn_buf = fb.empty(shape, dt)
    attn = l_attention(fb, x_norm, w["wq"], w["wk"], w["wv"], w["wo"], freqs, mask, attn_buf, n_heads, n_kv_heads)
    h = l_add(fb, x, attn, attn_buf)
    h_norm = l_l2_norm(fb, h, fb.empty(shape, dt), eps)
    hidden = _shape(w["w1"])[0]
    inter = shape[:-1] + (hidden,)
    w1_buf = fb.empty(inter, dt)
    gate = l_silu(fb, l_linear(fb, h_norm, w["w1"], w["b1"], w1_buf), w1_buf)
    w3_buf = fb.empty(inter, dt)
    gated = l_mul(fb, gate, l_linear(fb, h_norm, w["w3"], w["b3"], w3_buf), w3_buf)
    ffn = l_linear(fb, gated, w["w2"], w["b2"], out)
    return l_add(fb, h, ffn, out)


LAYER_ARG_NAMES = ("wq", "wk", "wv", "wo", "w1", "b1", "w2", "b2", "w3", "b3")


def llama_hidden_dim(dim: int, multiple_of: int, ffn_dim_multiplier: float | None = None) -> int:
    """The feed-forward width of the reference (test_llama3.py:880-886)."""
    hidden = int(2 * (4 * dim) / 3)
    if ffn_dim_multiplier is not None:
        hidden = int(ffn_dim_multiplier * hidden)
    return multiple_of * ((hidden + multiple_of - 1) // multiple_of)


def generate_llama_transformer_payload(func_name: str, batch: int, seq: int, dim: int, n_heads: int, n_kv_heads: int, hidden: int, n_layers: int,
                                       dtype: str = "f32", eps: float = 1e-5, mask: str = "operand", final_norm: bool = True) -> PayloadModule:
    """``payload(out, x, freqs, [mask,] (wq, wk, wv, wo, w1, b1, w2, b2, w3, b3) * n_layers)``:
    get_transformer (test_llama3.py:906-947): the blocks, then the weight-less final norm.
    With ``n_layers = 1`` and ``final_norm=False`` it is one get_transformer_block."""
    if mask not in ("operand", "none", "causal"):
        raise ValueError("mask must be 'operand', 'none' or 'causal'")
    hd = dim // n_heads
    mod = PayloadModule()
    xt = memref_t((batch, seq, dim), dtype)
    per_layer = [
        memref_t((n_heads * hd, dim), dtype), memref_t((n_kv_heads * hd, dim), dtype), memref_t((n_kv_heads * hd, dim), dtype), memref_t((dim, n_heads * hd), dtype),
        memref_t((hidden, dim), dtype), memref_t((hidden,), dtype), memref_t((dim, hidden), dtype), memref_t((dim,), dtype), memref_t((hidden, dim), dtype), memref_t((hidden,), dtype),
    ]
    types = [xt, xt, memref_t((seq, hd // 2), dtype)]
    if mask == "operand":
        types.append(memref_t((batch, n_heads, seq, seq), dtype))
    fb = FuncBuilder(mod, func_name, types + per_layer * n_layers)
    args = fb.args
    out_buf = args[0]
    fb.to_tensor(out_buf, restrict=True, writable=True)
    x = fb.to_tensor(args[1], restrict=True)
    freqs = fb.to_tensor(args[2], restrict=True)
    pos = 3
    if mask == "operand":
        mask_t = fb.to_tensor(args[3], restrict=True)
        pos = 4
    elif mask == "causal":
        mask_t = l_causal_mask(fb, (batch, n_heads, seq, seq), dtype)
    else:
        mask_t = None
    h = x
    for _ in range(n_layers):
        w = {name: fb.to_tensor(args[pos + i], restrict=True) for i, name in enumerate(LAYER_ARG_NAMES)}
        pos += len(LAYER_ARG_NAMES)
        h = l_transformer_block(fb, h, w, freqs, mask_t, fb.empty((batch, seq, dim), dtype), n_heads, n_kv_heads, eps)
    if final_norm:
        h = l_l2_norm(fb, h, fb.empty((batch, seq, dim), dtype), eps)
    fb.materialize_in_destination(h, out_buf)
    fb.ret()
    return mod


def generate_llama_attention_payload(func_name: str, batch: int, seq: int, dim: int, n_heads: int, n_kv_heads: int, dtype: str = "f32", mask: str = "operand") -> PayloadModule:
    """``payload(out, x, wq, wk, wv, wo, freqs[, mask])``: get_attention alone."""
    hd = dim // n_heads
    mod = PayloadModule()
    xt = memref_t((batch, seq, dim), dtype)
    types = [xt, xt, memref_t((n_heads * hd, dim), dtype), memref_t((n_kv_heads * hd, dim), dtype), memref_t((n_kv_heads * hd, dim), dtype),
             memref_t((dim, n_heads * hd), dtype), memref_t((seq, hd // 2), dtype)]
    if mask == "operand":
        types.append(memref_t((batch, n_heads, seq, seq), dtype))
    fb = FuncBuilder(mod, func_name, types)
    a = fb.args
    fb.to_tensor(a[0], restrict=True, writable=True)
    x, wq, wk, wv, wo, freqs = (fb.to_tensor(v, restrict=True) for v in a[1:7])
    if mask == "operand":
        mask_t = fb.to_tensor(a[7], restrict=True)
    elif mask == "causal":
        mask_t = l_causal_mask(fb, (batch, n_heads, seq, seq), dtype)
    else:
        mask_t = None
    res = l_attention(fb, x, wq, wk, wv, wo, freqs, mask_t, fb.empty((batch, seq, dim), dtype), n_heads, n_kv_heads)
    fb.materialize_in_destination(res, a[0])
    fb.ret()
    return mod
