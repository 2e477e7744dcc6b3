"""Payload generators with the names, arguments and op sequences of the reference's
``lighthouse.ingress.mlir_gen`` package, producing ``PayloadModule`` objects (printable as
MLIR text) instead of ``ir.Module``. Element types are given by name.

  generate_gpu_matmul_payload     lighthouse/ingress/mlir_gen/gpu_matmul_payload.py:5-36
  generate_gpu_mlp_payload        lighthouse/ingress/mlir_gen/gpu_mlp_payload.py:10-156
  generate_gpu_attention_payload  lighthouse/ingress/mlir_gen/gpu_attention_payload.py:12-132
  generate_gpu_layer_norm_payload lighthouse/ingress/mlir_gen/gpu_layer_norm_payload.py:90-143
  generate_gpu_softmax_payload    lighthouse/ingress/mlir_gen/gpu_softmax_payload.py:11-65
  generate_matmul_tensor_payload  the tensor-argument form of test/run/pipeline-check.mlir:7-14
  build_gpt_fused_payload         examples/xegpu/nanoGPT_payload.py:58-414

Argument order is the reference's: outputs first for the memref-style payloads.
"""

from __future__ import annotations

import math

from .builder import PARALLEL, REDUCTION, FuncBuilder, affine_map, identity_map
from .ir import PayloadModule, memref_t, tensor_t

_WIDTH = {"f16": 16, "bf16": 16, "f32": 32, "f64": 64}


def convert_float_type(fb: FuncBuilder, value, out):
    """Elementwise truncf / extf generic (generic.py:179-188 of the reference)."""
    src, dst = value.type.dtype, out.type.dtype
    assert src != dst, "Cannot cast to same type."
    rank = out.type.rank
    idm = identity_map(rank)
    narrowing = _WIDTH[src] > _WIDTH[dst]
    return fb.generic([value], [out], [idm, idm], [PARALLEL] * rank, lambda rb, a, _o: rb.truncf(a, dst) if narrowing else rb.extf(a, dst))


def add_bias(fb: FuncBuilder, inputs, bias):
    """broadcast(bias) over rows + linalg.add (named.py:20-26)."""
    t = inputs.type
    out = fb.empty(t.shape, t.dtype)
    bcast = fb.broadcast(bias, out, [0])
    return fb.add(bcast, inputs, out)


def relu(fb: FuncBuilder, inputs):
    """linalg.max(x, fill(0)) (named.py:28-32)."""
    t = inputs.type
    zero = fb.constant(0.0, t.dtype)
    out = fb.empty(t.shape, t.dtype)
    filled = fb.fill(zero, out)
    return fb.max(inputs, filled, out)


def emit_mlp_layer(fb, a, b, acc_type, result_type, acc_tensor=None, bias_tensor=None, transpose_a=False, transpose_b=False, has_relu=False):
    """One layer: [transposes] -> matmul into (C or zeros) -> + bias -> cast -> ReLU
    (gpu_mlp_payload.py:110-156)."""
    M, K = a.type.shape[::-1] if transpose_a else a.type.shape
    K, N = b.type.shape[::-1] if transpose_b else b.type.shape
    convert_result = acc_type != result_type
    if acc_tensor is not None:
        if acc_tensor.type.dtype != acc_type:
            acc_tensor = convert_float_type(fb, acc_tensor, fb.empty((M, N), acc_type))
    else:
        zero = fb.constant(0.0, acc_type)
        acc_tensor = fb.fill(zero, fb.empty((M, N), acc_type))
    if transpose_a:
        a = fb.transpose(a, fb.empty((M, K), a.type.dtype), [1, 0])
    if transpose_b:
        b = fb.transpose(b, fb.empty((K, N), b.type.dtype), [1, 0])
    terminal = fb.matmul(a, b, acc_tensor)
    if bias_tensor is not None:
        if bias_tensor.type.dtype != acc_type:
            bias_tensor = convert_float_type(fb, bias_tensor, fb.empty((N,), acc_type))
        terminal = add_bias(fb, terminal, bias_tensor)
    if convert_result:
        terminal = convert_float_type(fb, terminal, fb.empty((M, N), result_type))
    if has_relu:
        terminal = relu(fb, terminal)
    return terminal


def generate_gpu_mlp_payload(
    func_name: str,
    batch_size: int,
    input_size: int,
    output_size: int,
    hidden_layer_sizes: list[int],
    ab_type: str,
    acc_type: str,
    bias_type: str,
    result_type: str,
    transpose_a: bool,
    transpose_b: bool,
    has_bias: bool,
    has_relu: bool,
    accumulate_c: bool,
    relu_on_final_layer: bool = False,
) -> PayloadModule:
    mod = PayloadModule()
    a_shape = (batch_size, input_size) if not transpose_a else (input_size, batch_size)
    layer_sizes = [input_size] + list(hidden_layer_sizes) + [output_size]
    feature_sizes = list(zip(layer_sizes[:-1], layer_sizes[1:]))
    weight_types, bias_types = [], []
    for in_size, out_size in feature_sizes:
        shape = (in_size, out_size) if not transpose_b else (out_size, in_size)
        weight_types.append(memref_t(shape, ab_type))
        if has_bias:
            bias_types.append(memref_t((out_size,), bias_type))
    # function argument order: output, input, weights..., [biases...]
    fargs = [memref_t((batch_size, output_size), result_type), memref_t(a_shape, ab_type)] + weight_types + bias_types
    fb = FuncBuilder(mod, func_name, fargs)
    args = fb.args
    output, inp = args[0], args[1]
    nlayers = len(hidden_layer_sizes) + 1
    weights = args[2 : 2 + nlayers]
    biases = args[2 + nlayers :] if has_bias else [None] * nlayers
    output_tensor = fb.to_tensor(output, restrict=True, writable=True)
    layer_input = fb.to_tensor(inp, restrict=True)
    weight_tensors = [fb.to_tensor(w, restrict=True) for w in weights]
    bias_tensors = [fb.to_tensor(b, restrict=True) if has_bias else None for b in biases]
    for i, (w, b) in enumerate(zip(weight_tensors, bias_tensors)):
        layer_transpose_a = transpose_a and i == 0
        M, K = layer_input.type.shape[::-1] if layer_transpose_a else layer_input.type.shape
        K, N = w.type.shape[::-1] if transpose_b else w.type.shape
        c_tensor = None
        if accumulate_c:
            c_tensor = output_tensor if i == nlayers - 1 else fb.empty((M, N), ab_type)
        hidden = i < nlayers - 1
        out = emit_mlp_layer(
            fb, layer_input, w, acc_type=acc_type, result_type=ab_type if hidden else result_type, acc_tensor=c_tensor,
            bias_tensor=b, transpose_a=layer_transpose_a, transpose_b=transpose_b, has_relu=(hidden or relu_on_final_layer) and has_relu,
        )
        if i == nlayers - 1:
            fb.materialize_in_destination(out, output)
        layer_input = out
    fb.ret()
    return mod


def generate_gpu_matmul_payload(func_name, M, N, K, ab_type, c_type, transpose_a, transpose_b, has_bias, has_relu, accumulate_c, result_type=None) -> PayloadModule:
    return generate_gpu_mlp_payload(
        func_name, batch_size=M, input_size=K, output_size=N, hidden_layer_sizes=[], ab_type=ab_type, acc_type=c_type,
        bias_type=c_type if result_type is None else result_type, result_type=c_type if result_type is None else result_type,
        transpose_a=transpose_a, transpose_b=transpose_b, has_bias=has_bias, has_relu=has_relu, accumulate_c=accumulate_c, relu_on_final_layer=True,
    )


def generate_gpu_attention_payload(func_name: str, Z: int, H: int, n_ctx: int, n_head: int, dtype: str) -> PayloadModule:
    """payload(out, Q, K, V): collapse (Z,H) -> batch; K^T; batch_matmul; * fill(1/sqrt d);
    linalg.softmax dim 2; batch_matmul with V; materialise into out."""
    mod = PayloadModule()
    t4 = memref_t((Z, H, n_ctx, n_head), dtype)
    fb = FuncBuilder(mod, func_name, [t4, t4, t4, t4])
    out, q_arg, k_arg, v_arg = fb.args
    batch = Z * H
    s3 = (batch, n_ctx, n_head)
    reassoc = [[0, 1], [2], [3]]
    q3m = fb.collapse_shape(q_arg, s3, reassoc)
    k3m = fb.collapse_shape(k_arg, s3, reassoc)
    v3m = fb.collapse_shape(v_arg, s3, reassoc)
    o3m = fb.collapse_shape(out, s3, reassoc)
    q3, k3, v3 = (fb.to_tensor(m, restrict=True) for m in (q3m, k3m, v3m))
    kt = fb.transpose(k3, fb.empty((batch, n_head, n_ctx), dtype), [0, 2, 1])
    qk_shape = (batch, n_ctx, n_ctx)
    zero = fb.constant(0.0, dtype)
    qkt = fb.batch_matmul(q3, kt, fb.fill(zero, fb.empty(qk_shape, dtype)))
    scale = fb.constant(1.0 / math.sqrt(n_head), dtype)
    scale_t = fb.fill(scale, fb.empty(qk_shape, dtype))
    scaled = fb.mul(qkt, scale_t, fb.empty(qk_shape, dtype))
    weights = fb.softmax(scaled, fb.empty(qk_shape, dtype), 2)
    res = fb.batch_matmul(weights, v3, fb.fill(zero, fb.empty(s3, dtype)))
    fb.materialize_in_destination(res, o3m)
    fb.ret()
    return mod


def emit_layer_norm_generics(fb: FuncBuilder, x, gamma, beta, out_init, N: int, dtype: str, eps: float = 1e-5):
    """The three generics of the reference's layer norm (gpu_layer_norm_payload.py:15-87):
    row sum; row sum of squared deviations; normalise with gamma and beta."""
    par2 = affine_map(2, [0, 1])
    red2 = affine_map(2, [0])
    bias2 = affine_map(2, [1])
    zero = fb.constant(0.0, dtype)
    inv_n = fb.constant(1.0 / float(N), dtype)
    eps_c = fb.constant(eps, dtype)
    rows = (out_init.type.shape[0],)
    mean_acc = fb.fill(zero, fb.empty(rows, dtype))
    mean_sum = fb.generic([x], [mean_acc], [par2, red2], [PARALLEL, REDUCTION], lambda rb, v, acc: rb.addf(v, acc))
    var_acc = fb.fill(zero, fb.empty(rows, dtype))

    def var_body(rb, v, m_sum, acc):
        centered = rb.subf(v, rb.mulf(m_sum, inv_n))
        return rb.addf(rb.mulf(centered, centered), acc)

    var_sum = fb.generic([x, mean_sum], [var_acc], [par2, red2, red2], [PARALLEL, REDUCTION], var_body)

    def norm_body(rb, v, m_sum, v_sum, g, b, _out):
        mean = rb.mulf(m_sum, inv_n)
        var_eps = rb.addf(rb.mulf(v_sum, inv_n), eps_c)
        scaled = rb.mulf(rb.subf(v, mean), rb.rsqrt(var_eps))
        return rb.addf(rb.mulf(scaled, g), b)

    return fb.generic([x, mean_sum, var_sum, gamma, beta], [out_init], [par2, red2, red2, bias2, bias2, par2], [PARALLEL, PARALLEL], norm_body)


def generate_gpu_layer_norm_payload(func_name: str, M: int, N: int, dtype: str, eps: float = 1e-5) -> PayloadModule:
    mod = PayloadModule()
    mt, bt = memref_t((M, N), dtype), memref_t((N,), dtype)
    fb = FuncBuilder(mod, func_name, [mt, mt, bt, bt])
    out, x_arg, g_arg, b_arg = fb.args
    fb.to_tensor(out, restrict=True, writable=True)
    x, g, b = (fb.to_tensor(a, restrict=True) for a in (x_arg, g_arg, b_arg))
    normed = emit_layer_norm_generics(fb, x, g, b, fb.empty((M, N), dtype), N, dtype, eps)
    fb.materialize_in_destination(normed, out)
    fb.ret()
    return mod


def generate_gpu_softmax_payload(func_name: str, M: int, N: int, dtype: str) -> PayloadModule:
    mod = PayloadModule()
    mt = memref_t((M, N), dtype)
    fb = FuncBuilder(mod, func_name, [mt, mt])
    out, x_arg = fb.args
    fb.to_tensor(out, restrict=True, writable=True)
    x = fb.to_tensor(x_arg, restrict=True)
    res = fb.softmax(x, fb.empty((M, N), dtype), 1)
    fb.materialize_in_destination(res, out)
    fb.ret()
    return mod


def generate_matmul_tensor_payload(func_name: str, M: int, N: int, K: int, dtype: str = "f32") -> PayloadModule:
    """``@main(A, B, out)`` on tensors: fill(0) of ``out`` (result unused) and
    ``linalg.matmul ins(A, B) outs(out)`` — the payload shape of the reference's lh-run
    known-answer test. The product accumulates into the ``out`` argument in place."""
    mod = PayloadModule()
    fb = FuncBuilder(mod, func_name, [tensor_t((M, K), dtype), tensor_t((K, N), dtype), tensor_t((M, N), dtype)], arg_names=["arg0", "arg1", "out"], c_interface=False)
    a, b, out = fb.args
    zero = fb.constant(0.0, dtype)
    fb.fill(zero, out)
    fb.matmul(a, b, out)
    fb.ret()
    return mod


# ------------------------------------------------------------------------------ nanoGPT
class GptBuilder:
    """Op emitters of the reference's nanoGPT ``Builder`` (examples/xegpu/nanoGPT_payload.py:58-286):
    every op writes a fresh ``gpu.alloc`` buffer; ``kinds`` records the class of each op in
    emission order ('mm', 'ln', 'ew', 'fa'). ``lowp`` is the 16-bit type (the reference uses f16)."""

    def __init__(self, fb: FuncBuilder, T: int, lowp: str = "bf16"):
        self.fb, self.T, self.lowp = fb, T, lowp
        self.kinds: list[str] = []
        self.to_dealloc = []

    def _buf(self, shape, dtype):
        b = self.fb.gpu_alloc(shape, dtype)
        self.to_dealloc.append(b)
        return b

    def matmul(self, a, b, M, N, out_buf=None):
        fb = self.fb
        buf = out_buf if out_buf is not None else self._buf((M, N), "f32")
        out_t = fb.to_tensor(buf, restrict=True, writable=True)
        acc = fb.fill(fb.constant(0.0, "f32"), out_t)
        res = fb.matmul(a, b, acc)
        fb.materialize_in_destination(res, buf)
        self.kinds.append("mm")
        return None if out_buf is not None else fb.to_tensor(buf, restrict=True)

    def layernorm(self, x, gamma, beta, M, N, eps=1e-5):
        fb = self.fb
        buf = self._buf((M, N), "f32")
        out_t = fb.to_tensor(buf, restrict=True, writable=True)
        normed = emit_layer_norm_generics(fb, x, gamma, beta, out_t, N, "f32", eps)
        fb.materialize_in_destination(normed, buf)
        self.kinds.append("ln")
        return fb.to_tensor(buf, restrict=True)

    def _cast(self, x, M, N):
        fb = self.fb
        buf = self._buf((M, N), self.lowp)
        out_t = fb.to_tensor(buf, restrict=True, writable=True)
        idm = identity_map(2)
        c = fb.generic([x], [out_t], [idm, idm], [PARALLEL, PARALLEL], lambda rb, s, _o: rb.truncf(s, self.lowp))
        fb.materialize_in_destination(c, buf)
        self.kinds.append("ew")
        return buf

    def cast_lowp(self, x, M, N):
        return self.fb.to_tensor(self._cast(x, M, N), restrict=True)

    def cast_lowp_buf(self, x, T, C):
        return self._cast(x, T, C)

    def bias(self, x, bias_vec, M, N, relu=False, out_buf=None):
        fb = self.fb
        par2, bias2 = identity_map(2), affine_map(2, [1])
        zero = fb.constant(0.0, "f32")
        buf = out_buf if out_buf is not None else self._buf((M, N), "f32")
        out_t = fb.to_tensor(buf, restrict=True, writable=True)

        def body(rb, v, bb, _o):
            s = rb.addf(v, bb)
            return rb.maximumf(s, zero) if relu else rb.addf(s, zero)

        b = fb.generic([x, bias_vec], [out_t], [par2, bias2, par2], [PARALLEL, PARALLEL], body)
        fb.materialize_in_destination(b, buf)
        self.kinds.append("ew")
        return None if out_buf is not None else fb.to_tensor(buf, restrict=True)

    def add(self, a, b, M, N, out_buf=None):
        fb = self.fb
        par2 = identity_map(2)
        buf = out_buf if out_buf is not None else self._buf((M, N), "f32")
        out_t = fb.to_tensor(buf, restrict=True, writable=True)
        r = fb.generic([a, b], [out_t], [par2, par2, par2], [PARALLEL, PARALLEL], lambda rb, x, y, _o: rb.addf(x, y))
        fb.materialize_in_destination(r, buf)
        self.kinds.append("ew")
        return None if out_buf is not None else fb.to_tensor(buf, restrict=True)

    def _heads_view_of(self, buf2d, T, H, hs):
        e = self.fb.expand_shape(buf2d, (T, H, hs), [[0], [1, 2]])
        return self.fb.memref_transpose(e, [1, 0, 2])  # (H, T, hs) strided view, no copy

    def heads_view(self, buf2d, T, H, hs):
        return self.fb.to_tensor(self._heads_view_of(buf2d, T, H, hs), restrict=True)

    def attention_4d(self, Qh, Kh, Vh, H, T, hs, out_view, out_view_memref):
        fb, lp = self.fb, self.lowp
        zero = fb.constant(0.0, lp)
        Kt = fb.transpose(Kh, fb.empty((H, hs, T), lp), [0, 2, 1])
        qkt = fb.batch_matmul(Qh, Kt, fb.fill(zero, fb.empty((H, T, T), lp)))
        scale_t = fb.fill(fb.constant(1.0 / (hs**0.5), lp), fb.empty((H, T, T), lp))
        scaled = fb.mul(qkt, scale_t, fb.empty((H, T, T), lp))
        aw = fb.softmax(scaled, fb.empty((H, T, T), lp), 2)
        out = fb.batch_matmul(aw, Vh, fb.fill(zero, out_view))
        fb.materialize_in_destination(out, out_view_memref)
        self.kinds.append("fa")

    def fused_attention(self, x, wq, wk, wv, T, C, H):
        hs = C // H
        x16 = self.cast_lowp(x, T, C)
        qbuf = self.cast_lowp_buf(self.matmul(x16, wq, T, C), T, C)
        kbuf = self.cast_lowp_buf(self.matmul(x16, wk, T, C), T, C)
        vbuf = self.cast_lowp_buf(self.matmul(x16, wv, T, C), T, C)
        Qh, Kh, Vh = (self.heads_view(b, T, H, hs) for b in (qbuf, kbuf, vbuf))
        out_buf = self._buf((T, C), self.lowp)
        out_view_memref = self._heads_view_of(out_buf, T, H, hs)
        out_view = self.fb.to_tensor(out_view_memref, restrict=True, writable=True)
        self.attention_4d(Qh, Kh, Vh, H, T, hs, out_view, out_view_memref)
        return self.fb.to_tensor(out_buf, restrict=True)


def _emit_block_fused(bld: GptBuilder, x, w, T, C, hidden, H, eps, out_buf=None):
    ln1 = bld.layernorm(x, w["g1"], w["b1n"], T, C, eps)
    attn16 = bld.fused_attention(ln1, w["wq"], w["wk"], w["wv"], T, C, H)
    proj = bld.matmul(attn16, w["wp"], T, C)
    proj = bld.bias(proj, w["bp"], T, C, relu=False)
    a = bld.add(x, proj, T, C)
    ln2 = bld.layernorm(a, w["g2"], w["b2n"], T, C, eps)
    ln2_16 = bld.cast_lowp(ln2, T, C)
    h = bld.matmul(ln2_16, w["w1"], T, hidden)
    h = bld.bias(h, w["bb1"], T, hidden, relu=True)
    h16 = bld.cast_lowp(h, T, hidden)
    o = bld.matmul(h16, w["w2"], T, C)
    o = bld.bias(o, w["bb2"], T, C, relu=False)
    return bld.add(a, o, T, C, out_buf=out_buf)


GPT_LAYER_KEYS = ["g1", "b1n", "wq", "wk", "wv", "wp", "bp", "g2", "b2n", "w1", "bb1", "w2", "bb2"]


def build_gpt_fused_payload(func_name, T, C, hidden, vocab, n_layer, H, eps=1e-5, lowp="bf16"):
    """Full nanoGPT forward as one module (examples/xegpu/nanoGPT_payload.py:320-414):
    args ``out, x, [g1,b1n,wq,wk,wv,wp,bp,g2,b2n,w1,bb1,w2,bb2] * n_layer, gf_g, gf_b, lmw, lmb``.
    Returns (module, kinds)."""
    mod = PayloadModule()
    x_t, g_t = memref_t((T, C), "f32"), memref_t((C,), "f32")
    wcc, w1_t, w2_t = memref_t((C, C), lowp), memref_t((C, hidden), lowp), memref_t((hidden, C), lowp)
    b1_t = memref_t((hidden,), "f32")
    per_layer = [g_t, g_t, wcc, wcc, wcc, wcc, g_t, g_t, g_t, w1_t, b1_t, w2_t, g_t]
    fargs = [memref_t((T, vocab), "f32"), x_t] + per_layer * n_layer + [g_t, g_t, memref_t((C, vocab), lowp), memref_t((vocab,), "f32")]
    fb = FuncBuilder(mod, func_name, fargs)
    bld = GptBuilder(fb, T, lowp)
    args = fb.args
    output = args[0]
    fb.to_tensor(output, restrict=True, writable=True)
    h = fb.to_tensor(args[1], restrict=True)
    idx = 2
    layers = []
    for _ in range(n_layer):
        layers.append({k: fb.to_tensor(args[idx + i], restrict=True) for i, k in enumerate(GPT_LAYER_KEYS)})
        idx += len(GPT_LAYER_KEYS)
    gf_g, gf_b, lmw, lmb = (fb.to_tensor(args[idx + i], restrict=True) for i in range(4))
    for w in layers:
        h = _emit_block_fused(bld, h, w, T, C, hidden, H, eps)
    hf = bld.layernorm(h, gf_g, gf_b, T, C, eps)
    hf16 = bld.cast_lowp(hf, T, C)
    logits = bld.matmul(hf16, lmw, T, vocab)
    bld.bias(logits, lmb, T, vocab, relu=False, out_buf=output)
    for b in bld.to_dealloc:
        fb.gpu_dealloc(b)
    fb.ret()
    return mod, bld.kinds
