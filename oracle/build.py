"""Builds the C part of the oracle: ``oracle/_build/liblh_oracle.so`` (test infrastructure).

    python -m oracle.build

``-ffp-contract=off`` keeps multiply and add as two roundings, as the loop nest the
reference lowers to does before any vectorising stage.
"""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SRC = HERE / "loops" / "matmul_loops.c"
OUT_DIR = HERE / "_build"
LIB = OUT_DIR / "liblh_oracle.so"


def build(force: bool = False) -> Path:
    OUT_DIR.mkdir(exist_ok=True)
    if force or not LIB.exists() or LIB.stat().st_mtime < SRC.stat().st_mtime:
        cmd = ["gcc", "-O3", "-march=native", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", str(SRC), "-o", str(LIB)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"gcc failed:\n{res.stderr}")
    return LIB


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = LIB if LIB.exists() else build()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError:
            # built with -march=native on another machine: rebuild for this CPU
            lib = ctypes.CDLL(str(build(force=True)))
        fp = ctypes.POINTER(ctypes.c_float)
        i64 = ctypes.c_int64
        lib.lh_oracle_num_threads.restype = ctypes.c_int
        for name in ("lh_oracle_matmul_loops", "lh_oracle_matmul_loops_ikj"):
            getattr(lib, name).argtypes = [fp, fp, fp, i64, i64, i64]
            getattr(lib, name).restype = None
        lib.lh_oracle_matmul_bias_relu.argtypes = [fp, fp, fp, fp, i64, i64, i64, ctypes.c_int]
        lib.lh_oracle_matmul_bias_relu.restype = None
        _lib = lib
    return _lib


def _fp(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def matmul_loops(a: np.ndarray, b: np.ndarray, c: np.ndarray | None = None, interchange: bool = True) -> np.ndarray:
    """C += A @ B by the loop nest; returns C (a fresh zero matrix when c is None)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    m, k = a.shape
    n = b.shape[1]
    out = np.zeros((m, n), np.float32) if c is None else np.ascontiguousarray(c, dtype=np.float32).copy()
    fn = load().lh_oracle_matmul_loops_ikj if interchange else load().lh_oracle_matmul_loops
    fn(_fp(a), _fp(b), _fp(out), m, n, k)
    return out


def matmul_bias_relu(a: np.ndarray, b: np.ndarray, bias: np.ndarray | None, relu: bool = True) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    m, k = a.shape
    n = b.shape[1]
    out = np.empty((m, n), np.float32)
    bp = _fp(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
    load().lh_oracle_matmul_bias_relu(_fp(a), _fp(b), bp, _fp(out), m, n, k, int(relu))
    return out


def num_threads() -> int:
    return int(load().lh_oracle_num_threads())


if __name__ == "__main__":
    print(build(force=True))
