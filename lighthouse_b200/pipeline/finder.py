"""Target-based descriptor lookup, the directory convention of lighthouse/pipeline/finder.py:12-92:
``<base>/<arch>/<feature>/<pipeline>/<dtype>.yaml`` first, then ``<base>/<arch>/<pipeline>/<dtype>.yaml``;
an external ``base_path`` is searched before the packaged descriptors."""

from __future__ import annotations

import os
from pathlib import Path

from ..execution.target import TargetInfo

DESCRIPTORS_REPO = Path(__file__).parent / "descriptors"


def find_pipeline_file(target: TargetInfo, pipeline: str, dtype: str = "f32", base_path: str | None = None):
    """Returns (path, feature) or (None, None)."""
    if not pipeline or not target:
        return None, None
    if base_path is not None:
        file, feature = _find_pipeline_in_base(target, base_path, pipeline, dtype)
        if file is not None:
            return file, feature
    return _find_pipeline_in_base(target, DESCRIPTORS_REPO, pipeline, dtype)


def _find_pipeline_in_base(target: TargetInfo, base_path, pipeline: str, dtype: str):
    base_path = Path(base_path)
    arch_path = base_path / target.arch
    if not base_path.exists() or not arch_path.exists():
        return None, None
    available = [n for n in os.listdir(arch_path) if (arch_path / n).is_dir()]
    for feature in target.has_features(available):
        p = arch_path / feature / pipeline / f"{dtype}.yaml"
        if p.exists():
            return str(p), feature
    p = arch_path / pipeline / f"{dtype}.yaml"
    if p.exists():
        return str(p), None
    return None, None
