"""MLIR-style ranked memref descriptors and the packed-argument convention.

Same layout and calling convention as lighthouse/utils/memref.py:5-44 and
``mlir.runtime.np_to_memref`` in the reference: a descriptor is
``{T* allocated; T* aligned; int64 offset; int64 shape[r]; int64 strides[r]}`` with
strides in elements, an argument is a pointer to a pointer to the descriptor, and the
call takes one ``void*`` array.
"""

from __future__ import annotations

import ctypes
from collections.abc import Sequence
from functools import lru_cache


@lru_cache(maxsize=None)
def make_nd_memref_descriptor(rank: int):
    """ctypes structure type of a rank-``rank`` memref descriptor (element type erased:
    the pointers are ``void*``; rank 0 has no shape/strides)."""
    fields = [("allocated", ctypes.c_void_p), ("aligned", ctypes.c_void_p), ("offset", ctypes.c_longlong)]
    if rank > 0:
        fields += [("shape", ctypes.c_longlong * rank), ("strides", ctypes.c_longlong * rank)]
    return type(f"MemRefDescriptor{rank}D", (ctypes.Structure,), {"_fields_": fields})


def make_descriptor(ptr: int, shape, strides, offset: int = 0) -> ctypes.Structure:
    rank = len(shape)
    d = make_nd_memref_descriptor(rank)()
    d.allocated = ptr
    d.aligned = ptr
    d.offset = offset
    if rank:
        d.shape = (ctypes.c_longlong * rank)(*[int(s) for s in shape])
        d.strides = (ctypes.c_longlong * rank)(*[int(s) for s in strides])
    return d


def to_ctype(memref_desc) -> ctypes._Pointer:
    """Descriptor -> pointer-to-pointer argument."""
    return ctypes.pointer(ctypes.pointer(memref_desc))


def get_packed_arg(ctypes_args: Sequence) -> ctypes.Array:
    packed = (ctypes.c_void_p * max(len(ctypes_args), 1))()
    for i, a in enumerate(ctypes_args):
        packed[i] = ctypes.cast(a, ctypes.c_void_p)
    return packed


def to_packed_args(args) -> ctypes.Array:
    """Descriptors and/or Python ints -> packed ``void*[]`` (ints become ``int64*``)."""
    keep = []
    for arg in args:
        if isinstance(arg, int):
            keep.append(ctypes.pointer(ctypes.c_int64(arg)))
        else:
            keep.append(to_ctype(arg))
    packed = get_packed_arg(keep)
    packed._keepalive = keep  # the pointers must outlive the call
    return packed
