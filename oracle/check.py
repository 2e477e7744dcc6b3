"""Error metrics and tolerances of the parity tests (test infrastructure only).

The north-star tolerances are "max relative error <= 1e-5 for f32 and <= 2e-2 for bf16
with f32 accumulation". "Relative" is taken the way the reference's own nanoGPT check
takes it (examples/xegpu/nanoGPT.py:300-302): max |out - ref| / max |ref|, which stays
meaningful for outputs that cross zero.
"""

from __future__ import annotations

import numpy as np

TOL_F32 = 1e-5
TOL_BF16 = 2e-2


def max_rel_err(out, ref) -> float:
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    if out.shape != ref.shape:
        raise ValueError(f"shape mismatch {out.shape} vs {ref.shape}")
    if ref.size == 0:
        return 0.0
    if not np.all(np.isfinite(out)):
        return float("inf")
    return float(np.abs(out - ref).max() / (np.abs(ref).max() + 1e-30))


def tolerance_for(dtype: str) -> float:
    return TOL_F32 if dtype in ("f32", "f64") else TOL_BF16


def assert_close(out, ref, dtype: str, what: str = "") -> float:
    err = max_rel_err(out, ref)
    tol = tolerance_for(dtype)
    assert err <= tol, f"{what}: max relative error {err:.3e} exceeds {tol:.0e} for {dtype}"
    return err
