"""ctypes binding of ``liblh_b200.so`` (the C ABI declared in ``include/lh_b200.h``).

The library is the product: there is no Python or CPU fallback behind any call
here. If the shared object has not been built, loading raises ``RuntimeError``
with the command that builds it.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import (
    POINTER,
    Structure,
    c_char_p,
    c_double,
    c_float,
    c_int,
    c_int32,
    c_int64,
    c_size_t,
    c_uint32,
    c_void_p,
)
from pathlib import Path

import numpy as np

LH_MAX_RANK = 4
LH_MAX_OPERANDS = 8

# lh_status_t
LH_OK = 0
LH_ERR_INVALID = -1
LH_ERR_UNSUPPORTED = -2
LH_ERR_CUDA = -3
LH_ERR_DEVICE = -4
LH_ERR_COMM = -5
LH_ERR_NOMEM = -6

# lh_dtype_t
LH_F32, LH_BF16, LH_F16, LH_I32, LH_I64, LH_F64 = 0, 1, 2, 3, 4, 5
DTYPE_SIZE = {LH_F32: 4, LH_BF16: 2, LH_F16: 2, LH_I32: 4, LH_I64: 8, LH_F64: 8}
DTYPE_NAME = {LH_F32: "f32", LH_BF16: "bf16", LH_F16: "f16", LH_I32: "i32", LH_I64: "i64", LH_F64: "f64"}
DTYPE_FROM_NAME = {v: k for k, v in DTYPE_NAME.items()}

# lh_act_t
ACT_NONE, ACT_RELU, ACT_GELU_ERF, ACT_GELU_TANH, ACT_SILU, ACT_SIGMOID = 0, 1, 2, 3, 4, 5

# GEMM flags
GEMM_ACCUMULATE_C = 1
GEMM_FORCE_SIMT = 2
GEMM_SWIGLU = 4

# lh_ew_t
EW_COPY, EW_ADD, EW_MUL, EW_ACT, EW_ADD_ACT, EW_SILU_MUL, EW_SCALE, EW_FILL, EW_SUB, EW_MAX = range(10)

# lh_op_kind_t
(
    OP_GEMM,
    OP_ATTENTION,
    OP_LAYERNORM,
    OP_RMSNORM,
    OP_SOFTMAX,
    OP_ROPE,
    OP_ELEMENTWISE,
    OP_EMBEDDING,
    OP_ALLREDUCE,
    OP_ALLGATHER,
    OP_REDUCESCATTER,
    OP_STREAM,
    OP_EVENT_RECORD,
    OP_EVENT_WAIT,
    OP_RESERVE_SMS,
    OP_REDUCE_NORM_GATHER,
    OP_GEMM_ROPE,
) = range(1, 18)


class MemRef(Structure):
    """``lh_memref_t``: a ranked strided memref plus its rank and element type."""

    _fields_ = [
        ("allocated", c_void_p),
        ("aligned", c_void_p),
        ("offset", c_int64),
        ("rank", c_int32),
        ("dtype", c_int32),
        ("shape", c_int64 * LH_MAX_RANK),
        ("strides", c_int64 * LH_MAX_RANK),
    ]


class View(Structure):
    """``lh_view_t``: an operand of a module operator, a view into a buffer slot."""

    _fields_ = [
        ("slot", c_int32),
        ("rank", c_int32),
        ("dtype", c_int32),
        ("pad_", c_int32),
        ("offset", c_int64),
        ("shape", c_int64 * LH_MAX_RANK),
        ("strides", c_int64 * LH_MAX_RANK),
    ]


class Op(Structure):
    """``lh_op_t``: one operator record of a module."""

    _fields_ = [
        ("kind", c_int32),
        ("i0", c_int32),
        ("i1", c_int32),
        ("i2", c_int32),
        ("f0", c_float),
        ("f1", c_float),
        ("operands", View * LH_MAX_OPERANDS),
    ]


class ArgSig(Structure):
    _fields_ = [("rank", c_int32), ("dtype", c_int32)]


LIB_PATH = Path(__file__).resolve().parent / "_lib" / "liblh_b200.so"

# name -> (restype, argtypes); every symbol include/lh_b200.h declares.
_PROTOTYPES = {
    "lh_b200_ctx_create": (c_int, [c_int, POINTER(c_void_p)]),
    "lh_b200_ctx_destroy": (c_int, [c_void_p]),
    "lh_b200_ctx_set_stream": (c_int, [c_void_p, c_void_p, c_int]),
    "lh_b200_ctx_get_stream": (c_void_p, [c_void_p]),
    "lh_b200_sync": (c_int, [c_void_p]),
    "lh_b200_last_error": (c_char_p, [c_void_p]),
    "lh_b200_launch_count": (c_int64, [c_void_p]),
    "lh_b200_device_info": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "lh_b200_selftest_bounded_wait": (c_int, [c_void_p, ctypes.c_uint64, POINTER(c_int)]),
    "lh_b200_malloc": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "lh_b200_free": (c_int, [c_void_p, c_void_p]),
    "lh_b200_memcpy": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int]),
    "lh_b200_memset": (c_int, [c_void_p, c_void_p, c_int, c_size_t]),
    "lh_b200_host_alloc": (c_int, [c_size_t, POINTER(c_void_p)]),
    "lh_b200_host_free": (c_int, [c_void_p]),
    "lh_b200_gemm": (
        c_int,
        [c_void_p] + [POINTER(MemRef)] * 6 + [c_int, c_uint32],
    ),
    "lh_b200_attention_fwd": (c_int, [c_void_p] + [POINTER(MemRef)] * 4 + [c_float, c_int]),
    "lh_b200_attention_fwd_noalloc": (c_int, [c_void_p] + [POINTER(MemRef)] * 4 + [c_float, c_int]),
    "lh_b200_layernorm": (c_int, [c_void_p] + [POINTER(MemRef)] * 4 + [c_float]),
    "lh_b200_rmsnorm": (c_int, [c_void_p] + [POINTER(MemRef)] * 3 + [c_float]),
    "lh_b200_softmax": (c_int, [c_void_p] + [POINTER(MemRef)] * 2),
    "lh_b200_rope": (c_int, [c_void_p, POINTER(MemRef), c_float, c_int]),
    "lh_b200_elementwise": (c_int, [c_void_p, c_int] + [POINTER(MemRef)] * 3 + [c_int, c_float]),
    "lh_b200_embedding": (c_int, [c_void_p] + [POINTER(MemRef)] * 4 + [c_int]),
    "lh_b200_comm_unique_id": (c_int, [c_char_p, c_void_p]),
    "lh_b200_comm_init": (c_int, [c_void_p, c_char_p, c_void_p, c_int, c_int]),
    "lh_b200_comm_destroy": (c_int, [c_void_p]),
    "lh_b200_allreduce": (c_int, [c_void_p, POINTER(MemRef)]),
    "lh_b200_reducescatter": (c_int, [c_void_p, POINTER(MemRef), POINTER(MemRef)]),
    "lh_b200_gemm_rope": (c_int, [c_void_p, POINTER(MemRef), POINTER(MemRef), POINTER(MemRef), c_int, c_int, c_int, c_float, c_int]),
    "lh_b200_symm_register": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, POINTER(c_void_p), c_int]),
    "lh_b200_symm_set_flags": (c_int, [c_void_p, c_int, c_int, POINTER(c_void_p)]),
    "lh_b200_symm_clear": (c_int, [c_void_p]),
    "lh_b200_reduce_norm_gather": (c_int, [c_void_p, POINTER(MemRef), POINTER(MemRef), POINTER(MemRef), POINTER(MemRef), c_float]),
    "lh_b200_stream_select": (c_int, [c_void_p, c_int]),
    "lh_b200_event_record": (c_int, [c_void_p, c_int]),
    "lh_b200_event_wait": (c_int, [c_void_p, c_int]),
    "lh_b200_reserve_sms": (c_int, [c_void_p, c_int]),
    "lh_b200_set_launch_overlap": (c_int, [c_void_p, c_int]),
    "lh_b200_allgather": (c_int, [c_void_p, POINTER(MemRef), POINTER(MemRef)]),
    "lh_b200_module_create": (
        c_int,
        [
            c_void_p,
            c_char_p,
            POINTER(ArgSig),
            c_int,
            POINTER(c_size_t),
            c_int,
            POINTER(Op),
            c_int,
            POINTER(c_void_p),
        ],
    ),
    "lh_b200_module_destroy": (c_int, [c_void_p]),
    "lh_b200_invoke": (c_int, [c_void_p, c_char_p, POINTER(c_void_p), c_int]),
    "lh_b200_module_run": (c_int, [c_void_p, POINTER(c_void_p), c_int]),
    "lh_b200_benchmark": (
        c_int,
        [c_void_p, POINTER(c_void_p), c_int, POINTER(c_double), c_int64, c_int64, c_size_t],
    ),
    "lh_b200_module_use_graph": (c_int, [c_void_p, c_int]),
    "lh_b200_module_set_profiling": (c_int, [c_void_p, c_int]),
    "lh_b200_module_op_times": (c_int, [c_void_p, POINTER(c_float), c_int]),
    "lh_b200_module_op_end_times": (c_int, [c_void_p, POINTER(c_float), c_int]),
}

EXPORTED_SYMBOLS = tuple(_PROTOTYPES)

_lib = None


def lib_path() -> Path:
    return Path(os.environ.get("LH_B200_LIB", str(LIB_PATH)))


def load() -> ctypes.CDLL:
    """Loads the shared library (once) and sets the prototypes of every export."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not path.exists():
        raise RuntimeError(
            f"lighthouse_b200: native library {path} is missing; build it with "
            "`python -m lighthouse_b200.build` (needs nvcc). There is no CPU fallback."
        )
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in _PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the export is missing
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


class LighthouseCudaError(RuntimeError):
    """A CUDA, device-status or NCCL failure reported by the native library."""


def check(rc: int, ctx=None, what: str = "") -> None:
    """Maps a status code to the exception the reference's Runner would raise:
    ``ValueError`` for bad/unsupported requests, ``RuntimeError`` for device failures."""
    if rc == LH_OK:
        return
    msg = load().lh_b200_last_error(ctx)
    text = msg.decode("utf-8", "replace") if msg else ""
    text = f"{what}: {text}" if what else text
    if rc in (LH_ERR_INVALID, LH_ERR_UNSUPPORTED):
        raise ValueError(text or f"lh_b200 status {rc}")
    if rc == LH_ERR_NOMEM:
        raise MemoryError(text)
    raise LighthouseCudaError(text or f"lh_b200 status {rc}")


def memref(ptr: int, shape, strides, dtype: int, offset: int = 0) -> MemRef:
    """Builds an ``lh_memref_t`` from a device pointer and element strides."""
    rank = len(shape)
    if rank > LH_MAX_RANK:
        raise ValueError(f"rank {rank} exceeds LH_MAX_RANK={LH_MAX_RANK}")
    m = MemRef()
    m.allocated = ptr
    m.aligned = ptr
    m.offset = offset
    m.rank = rank
    m.dtype = dtype
    for i in range(rank):
        m.shape[i] = int(shape[i])
        m.strides[i] = int(strides[i])
    return m


def contiguous_strides(shape) -> list[int]:
    strides, acc = [], 1
    for d in reversed(shape):
        strides.append(acc)
        acc *= int(d)
    return list(reversed(strides))


def numpy_dtype_code(dt) -> int:
    """Maps a numpy dtype (``ml_dtypes.bfloat16`` included) to ``lh_dtype_t``."""
    dt = np.dtype(dt)
    if dt == np.float32:
        return LH_F32
    if dt == np.float16:
        return LH_F16
    if dt == np.float64:
        return LH_F64
    if dt == np.int32:
        return LH_I32
    if dt == np.int64:
        return LH_I64
    if dt.name == "bfloat16":
        return LH_BF16
    raise ValueError(f"unsupported numpy dtype {dt}")


def numpy_dtype_from_code(code: int):
    if code == LH_BF16:
        import ml_dtypes

        return np.dtype(ml_dtypes.bfloat16)
    return np.dtype({LH_F32: np.float32, LH_F16: np.float16, LH_F64: np.float64, LH_I32: np.int32, LH_I64: np.int64}[code])
