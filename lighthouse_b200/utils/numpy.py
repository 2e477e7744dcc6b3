"""numpy <-> MLIR element type names (the mapping of lighthouse/utils/numpy.py:15-84)."""

from __future__ import annotations

import numpy as np

_NAMES = {
    "f16": np.float16,
    "f32": np.float32,
    "f64": np.float64,
    "i8": np.int8,
    "i16": np.int16,
    "i32": np.int32,
    "i64": np.int64,
    "index": np.int64,
}


def mlir_to_numpy_dtype(name) -> np.dtype:
    """``"f32"`` -> ``np.float32``; ``"bf16"`` -> ``ml_dtypes.bfloat16``. Raises ValueError otherwise."""
    name = str(name)
    if name == "bf16":
        import ml_dtypes

        return np.dtype(ml_dtypes.bfloat16)
    if name not in _NAMES:
        raise ValueError(f"Unsupported MLIR element type: {name}")
    return np.dtype(_NAMES[name])


def numpy_to_mlir_type(dtype) -> str:
    dt = np.dtype(dtype)
    if dt.name == "bfloat16":
        return "bf16"
    for k, v in _NAMES.items():
        if k != "index" and np.dtype(v) == dt:
            return k
    raise ValueError(f"Unsupported numpy dtype: {dt}")
