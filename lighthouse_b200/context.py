"""``CudaContext``: the Python handle on an ``lh_ctx_t`` plus operator calls that
accept torch CUDA tensors (or raw ``MemRef`` descriptors) and pass them through
the C ABI. PyTorch is used only to own device memory; every kernel that runs is
the library's own.
"""

from __future__ import annotations

import ctypes
from ctypes import byref, c_int, c_void_p

from . import _native as N


def _torch():
    import torch

    return torch


_TORCH_DTYPES = None


def torch_dtype_code(dtype) -> int:
    global _TORCH_DTYPES
    torch = _torch()
    if _TORCH_DTYPES is None:
        _TORCH_DTYPES = {
            torch.float32: N.LH_F32,
            torch.bfloat16: N.LH_BF16,
            torch.float16: N.LH_F16,
            torch.int32: N.LH_I32,
            torch.int64: N.LH_I64,
            torch.float64: N.LH_F64,
        }
    if dtype not in _TORCH_DTYPES:
        raise ValueError(f"Unsupported dtype: {dtype}")
    return _TORCH_DTYPES[dtype]


def as_memref(t) -> N.MemRef | None:
    """torch CUDA tensor (any strides) -> ``lh_memref_t``; ``MemRef`` and ``None`` pass through.

    Same convention as ``lighthouse.utils.torch.to_memref`` (lighthouse/utils/torch.py:41-66):
    strides in elements, data pointer in both ``allocated`` and ``aligned``.
    """
    if t is None or isinstance(t, N.MemRef):
        return t
    if not t.is_cuda:
        raise ValueError("operands must be CUDA tensors: this backend has no CPU path")
    return N.memref(t.data_ptr(), tuple(t.shape), tuple(t.stride()), torch_dtype_code(t.dtype))


def _ref(m):
    return byref(m) if m is not None else None


class CudaContext:
    """One ``lh_ctx_t``: a device, a stream, the device status word, NCCL state."""

    def __init__(self, device: int = 0, use_torch_stream: bool = False):
        self._lib = N.load()
        handle = c_void_p()
        rc = self._lib.lh_b200_ctx_create(int(device), byref(handle))
        N.check(rc, None, "lh_b200_ctx_create")
        self.handle = handle
        self.device = int(device)
        sm, major, minor = c_int(), c_int(), c_int()
        N.check(self._lib.lh_b200_device_info(self.handle, byref(sm), byref(major), byref(minor)), self.handle)
        self.sm_count, self.cc = sm.value, (major.value, minor.value)
        if use_torch_stream:
            self.use_torch_stream()

    # -- lifetime ---------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "handle", None):
            self._lib.lh_b200_ctx_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):  # best effort
        try:
            self.close()
        except Exception:
            pass

    # -- stream / status --------------------------------------------------------
    def use_torch_stream(self) -> None:
        """Launch on torch's current stream so library kernels order with torch ops."""
        torch = _torch()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        N.check(self._lib.lh_b200_ctx_set_stream(self.handle, c_void_p(stream), 1), self.handle)

    def use_own_stream(self) -> None:
        N.check(self._lib.lh_b200_ctx_set_stream(self.handle, None, 0), self.handle)

    def stream_handle(self) -> int:
        return self._lib.lh_b200_ctx_get_stream(self.handle) or 0

    def sync(self) -> None:
        N.check(self._lib.lh_b200_sync(self.handle), self.handle, "lh_b200_sync")

    def selftest_bounded_wait(self, limit_ns: int = 1_000_000) -> int:
        """Lets 64 bounded waits run out on purpose (``lh_b200_selftest_bounded_wait``); returns
        how many gave up. The next ``sync()`` raises once, then the context is usable again."""
        n = c_int()
        N.check(self._lib.lh_b200_selftest_bounded_wait(self.handle, int(limit_ns), byref(n)), self.handle, "lh_b200_selftest_bounded_wait")
        return n.value

    @property
    def launch_count(self) -> int:
        return int(self._lib.lh_b200_launch_count(self.handle))

    # -- memory -----------------------------------------------------------------
    def malloc(self, nbytes: int) -> int:
        out = c_void_p()
        N.check(self._lib.lh_b200_malloc(self.handle, int(nbytes), byref(out)), self.handle, "lh_b200_malloc")
        return out.value or 0

    def free(self, ptr: int) -> None:
        N.check(self._lib.lh_b200_free(self.handle, c_void_p(ptr)), self.handle, "lh_b200_free")

    def memcpy_h2d(self, dst: int, src_host_ptr: int, nbytes: int) -> None:
        N.check(self._lib.lh_b200_memcpy(self.handle, c_void_p(dst), c_void_p(src_host_ptr), int(nbytes), 0), self.handle)

    def memcpy_d2h(self, dst_host_ptr: int, src: int, nbytes: int) -> None:
        N.check(self._lib.lh_b200_memcpy(self.handle, c_void_p(dst_host_ptr), c_void_p(src), int(nbytes), 1), self.handle)

    def memcpy_d2d(self, dst: int, src: int, nbytes: int) -> None:
        N.check(self._lib.lh_b200_memcpy(self.handle, c_void_p(dst), c_void_p(src), int(nbytes), 2), self.handle)

    def memset(self, dst: int, value: int, nbytes: int) -> None:
        N.check(self._lib.lh_b200_memset(self.handle, c_void_p(dst), int(value), int(nbytes)), self.handle)

    # -- operators (see include/lh_b200.h for semantics) ---------------------------
    def gemm(self, d, a, b, c=None, bias=None, residual=None, act: int = N.ACT_NONE, flags: int = 0) -> None:
        md, ma, mb, mc, mbias, mres = (as_memref(x) for x in (d, a, b, c, bias, residual))
        if mc is not None:
            flags |= N.GEMM_ACCUMULATE_C
        rc = self._lib.lh_b200_gemm(self.handle, _ref(md), _ref(ma), _ref(mb), _ref(mc), _ref(mbias), _ref(mres), int(act), int(flags))
        N.check(rc, self.handle, "lh_b200_gemm")

    def attention_fwd(self, o, q, k, v, scale: float, causal: bool = False) -> None:
        mo, mq, mk, mv = (as_memref(x) for x in (o, q, k, v))
        rc = self._lib.lh_b200_attention_fwd(self.handle, _ref(mo), _ref(mq), _ref(mk), _ref(mv), float(scale), int(bool(causal)))
        N.check(rc, self.handle, "lh_b200_attention_fwd")

    def attention_fwd_noalloc(self, o, q, k, v, scale: float, causal: bool = False) -> None:
        """Un-fused attention that performs no device allocation (score scratch lives in the
        library image; Sq * Skv <= 1 Mi). For callers whose memory is fully owned by their own
        pool or that must not allocate once warm."""
        mo, mq, mk, mv = (as_memref(x) for x in (o, q, k, v))
        rc = self._lib.lh_b200_attention_fwd_noalloc(self.handle, _ref(mo), _ref(mq), _ref(mk), _ref(mv), float(scale), int(bool(causal)))
        N.check(rc, self.handle, "lh_b200_attention_fwd_noalloc")

    def gemm_rope(self, d, a, b, rope_cols: int, head_dim: int, seq: int, theta: float = 10000.0, pos0: int = 0) -> None:
        md, ma, mb = as_memref(d), as_memref(a), as_memref(b)
        rc = self._lib.lh_b200_gemm_rope(self.handle, _ref(md), _ref(ma), _ref(mb), int(rope_cols), int(head_dim), int(seq), float(theta), int(pos0))
        N.check(rc, self.handle, "lh_b200_gemm_rope")

    def layernorm(self, out, x, gamma=None, beta=None, eps: float = 1e-5) -> None:
        mo, mx, mg, mb = (as_memref(t) for t in (out, x, gamma, beta))
        N.check(self._lib.lh_b200_layernorm(self.handle, _ref(mo), _ref(mx), _ref(mg), _ref(mb), float(eps)), self.handle, "lh_b200_layernorm")

    def rmsnorm(self, out, x, weight=None, eps: float = 1e-5) -> None:
        mo, mx, mw = (as_memref(t) for t in (out, x, weight))
        N.check(self._lib.lh_b200_rmsnorm(self.handle, _ref(mo), _ref(mx), _ref(mw), float(eps)), self.handle, "lh_b200_rmsnorm")

    def softmax(self, out, x) -> None:
        mo, mx = as_memref(out), as_memref(x)
        N.check(self._lib.lh_b200_softmax(self.handle, _ref(mo), _ref(mx)), self.handle, "lh_b200_softmax")

    def rope(self, x, theta: float = 10000.0, pos0: int = 0) -> None:
        mx = as_memref(x)
        N.check(self._lib.lh_b200_rope(self.handle, _ref(mx), float(theta), int(pos0)), self.handle, "lh_b200_rope")

    def elementwise(self, kind: int, out, a=None, b=None, act: int = N.ACT_NONE, scalar: float = 0.0) -> None:
        mo, ma, mb = as_memref(out), as_memref(a), as_memref(b)
        rc = self._lib.lh_b200_elementwise(self.handle, int(kind), _ref(mo), _ref(ma), _ref(mb), int(act), float(scalar))
        N.check(rc, self.handle, "lh_b200_elementwise")

    def embedding(self, out, ids, wte, wpe=None, period: int = 0) -> None:
        mo, mi, mw, mp = (as_memref(t) for t in (out, ids, wte, wpe))
        N.check(self._lib.lh_b200_embedding(self.handle, _ref(mo), _ref(mi), _ref(mw), _ref(mp), int(period)), self.handle, "lh_b200_embedding")

    # -- collectives ---------------------------------------------------------------
    def comm_init(self, unique_id: bytes, rank: int, world: int, nccl_path: str | None = None) -> None:
        buf = ctypes.create_string_buffer(unique_id, 128)
        path = nccl_path.encode() if nccl_path else None
        N.check(self._lib.lh_b200_comm_init(self.handle, path, buf, int(rank), int(world)), self.handle, "lh_b200_comm_init")
        self.rank, self.world = rank, world

    def allreduce(self, buf) -> None:
        m = as_memref(buf)
        N.check(self._lib.lh_b200_allreduce(self.handle, _ref(m)), self.handle, "lh_b200_allreduce")

    def allgather(self, out, inp) -> None:
        mo, mi = as_memref(out), as_memref(inp)
        N.check(self._lib.lh_b200_allgather(self.handle, _ref(mo), _ref(mi)), self.handle, "lh_b200_allgather")


    def reducescatter(self, out, inp) -> None:
        mo, mi = as_memref(out), as_memref(inp)
        N.check(self._lib.lh_b200_reducescatter(self.handle, _ref(mo), _ref(mi)), self.handle, "lh_b200_reducescatter")

    # -- side stream ------------------------------------------------------------------
    def stream_select(self, side: int) -> None:
        N.check(self._lib.lh_b200_stream_select(self.handle, int(side)), self.handle, "lh_b200_stream_select")

    def event_record(self, number: int) -> None:
        N.check(self._lib.lh_b200_event_record(self.handle, int(number)), self.handle, "lh_b200_event_record")

    def event_wait(self, number: int) -> None:
        N.check(self._lib.lh_b200_event_wait(self.handle, int(number)), self.handle, "lh_b200_event_wait")

    def reserve_sms(self, n: int) -> None:
        N.check(self._lib.lh_b200_reserve_sms(self.handle, int(n)), self.handle, "lh_b200_reserve_sms")

    def set_launch_overlap(self, enabled: bool) -> None:
        """Tensor-core kernels as programmatic dependents of their predecessor in the stream
        (their set-up runs under its tail). Off by default: it pays for kernels queued back to
        back on one stream and costs where other streams' copies and events interleave."""
        N.check(self._lib.lh_b200_set_launch_overlap(self.handle, 1 if enabled else 0), self.handle, "lh_b200_set_launch_overlap")

    # -- symmetric memory and the fused collective ------------------------------------------
    def symm_register(self, local_ptr: int, nbytes: int, multicast_ptr: int, peer_ptrs: list[int]) -> None:
        """Registers one symmetric buffer: this rank's address, its multicast mapping (0: none)
        and every rank's copy as mapped into this process."""
        peers = (ctypes.c_void_p * len(peer_ptrs))(*peer_ptrs)
        rc = self._lib.lh_b200_symm_register(self.handle, ctypes.c_void_p(local_ptr), int(nbytes), ctypes.c_void_p(multicast_ptr or None), peers, len(peer_ptrs))
        N.check(rc, self.handle, "lh_b200_symm_register")

    def symm_set_flags(self, rank: int, world: int, pad_ptrs: list[int]) -> None:
        pads = (ctypes.c_void_p * len(pad_ptrs))(*pad_ptrs)
        N.check(self._lib.lh_b200_symm_set_flags(self.handle, int(rank), int(world), pads), self.handle, "lh_b200_symm_set_flags")

    def symm_clear(self) -> None:
        N.check(self._lib.lh_b200_symm_clear(self.handle), self.handle, "lh_b200_symm_clear")

    def reduce_norm_gather(self, xn, part, h, weight, eps: float = 1e-5) -> None:
        mx, mp, mh, mw = (as_memref(t) for t in (xn, part, h, weight))
        rc = self._lib.lh_b200_reduce_norm_gather(self.handle, _ref(mx), _ref(mp), _ref(mh), _ref(mw), float(eps))
        N.check(rc, self.handle, "lh_b200_reduce_norm_gather")


def nccl_unique_id(nccl_path: str | None = None) -> bytes:
    """128-byte NCCL unique id for ``CudaContext.comm_init`` (rank 0 creates, everyone receives)."""
    buf = ctypes.create_string_buffer(128)
    path = nccl_path.encode() if nccl_path else None
    N.check(N.load().lh_b200_comm_unique_id(path, buf), None, "lh_b200_comm_unique_id")
    return buf.raw


def find_torch_nccl() -> str | None:
    """Path of the libnccl torch bundles, so the library and torch agree on the NCCL build."""
    import glob
    import os
    import site

    for sp in site.getsitepackages():
        hits = glob.glob(os.path.join(sp, "nvidia", "nccl", "lib", "libnccl.so*"))
        if hits:
            return sorted(hits)[0]
    return None
