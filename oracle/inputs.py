"""Seeded synthetic inputs for the five benchmark configurations (test infrastructure
only). Shapes, distributions and seeds follow the configuration list the benchmarks are
quoted on; the ``lh-run`` style initialisers follow lighthouse/execution/init.py:63-80
(``rnd`` is ``np.random.rand`` in [0, 1) after ``np.random.seed``, lh_run.py:82-85).
"""

from __future__ import annotations

import numpy as np
import torch


def lh_run_args(spec: str, seed: int) -> list[np.ndarray]:
    """``--input-shape`` parsing + init of KernelArgumentParser (execution/init.py:83-118)."""
    if seed:
        np.random.seed(seed)
    out = []
    for s in spec.split(","):
        parts = s.split("x")
        dims = [int(d) for d in parts[:-2]]
        dt = {"f32": np.float32, "f64": np.float64, "f16": np.float16, "i32": np.int32, "i64": np.int64}[parts[-2]]
        init = parts[-1]
        if init == "0":
            out.append(np.zeros(dims, dt))
        elif init == "1":
            out.append(np.ones(dims, dt))
        elif init == "rnd":
            out.append(np.random.rand(*dims).astype(dt))
        elif init == "id":
            out.append(np.eye(dims[0], dtype=dt))
        else:
            raise ValueError(init)
    return out


from lighthouse_b200.workloads.synthetic import (  # noqa: E402,F401  (one definition, shared with bench.py)
    attention_qkv,
    gemm_bf16_normal,
    gemm_f32_uniform,
    llama_weights,
    nanogpt_weights,
)


def to_np(t) -> np.ndarray:
    """torch tensor (bf16 included) -> float32 numpy holding the same values."""
    if isinstance(t, np.ndarray):
        return t
    if t.dtype in (torch.int32, torch.int64):
        return t.numpy()
    return t.to(torch.float32).numpy()


def tree_to_np(obj):
    if isinstance(obj, dict):
        return {k: tree_to_np(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [tree_to_np(v) for v in obj]
    return to_np(obj)
