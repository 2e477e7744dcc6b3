"""Which machine a pipeline is being chosen for.

``TargetInfo`` plays the part of lighthouse/execution/target.py:13-132 in the reference: an
architecture name plus a feature list that ``find_pipeline_file`` matches descriptor
directories against. The reference reads ``platform.machine()`` and ``lscpu``; this backend
knows one architecture, ``cuda``, whose features are compute-capability names (``sm_100a`` and
``sm_100`` on a B200). Tests fake a target with ``TargetInfo.override(...)`` the way the
reference's do (test/execution/target_info_host_override.py:10-40).
"""

from __future__ import annotations

from contextlib import contextmanager

_BUILD_TARGET = "sm_100a"


def _visible_gpu_features() -> list[str]:
    """Capability names of device 0 if one is visible, else what the library is built for."""
    try:
        import torch

        if torch.cuda.is_available():
            major, minor = torch.cuda.get_device_capability(0)
            base = f"sm_{major}{minor}"
            return [base + "a", base] if major >= 9 else [base]
    except Exception:  # no torch, no driver: describe the build target
        pass
    return [_BUILD_TARGET]


class TargetInfo:
    """``arch`` and ``features``; ``filter`` keeps only the listed features."""

    _host: "TargetInfo | None" = None
    _overrides: list[dict] = []  # innermost ``override(...)`` last

    def __init__(self, arch: str | None = None, features: list[str] | None = None, filter: list[str] | None = None):
        faked = self._overrides[-1] if self._overrides else {}
        if arch is None:
            arch = faked.get("arch") or "cuda"
        if features is None:
            features = list(faked["features"]) if faked.get("features") is not None else _visible_gpu_features()
        self.arch, self.features = arch, features
        if filter is not None:
            self.features = self.has_features(filter)

    # -- constructors ------------------------------------------------------------------
    @classmethod
    def host(cls) -> "TargetInfo":
        """The machine we are on (cached), or the faked one inside ``override``."""
        if cls._overrides:
            return cls()
        if cls._host is None:
            cls._host = cls()
        return cls._host

    @classmethod
    def cuda(cls) -> "TargetInfo":
        """The target this backend's kernels are compiled for."""
        return cls(arch="cuda", features=[_BUILD_TARGET])

    @classmethod
    def reset_host_cache(cls) -> None:
        cls._host = None

    @classmethod
    @contextmanager
    def override(cls, *, features: list[str] | None = None, arch: str | None = None):
        cls._overrides.append({"arch": arch, "features": None if features is None else list(features)})
        cls.reset_host_cache()
        try:
            yield
        finally:
            cls._overrides.pop()
            cls.reset_host_cache()

    # -- queries -------------------------------------------------------------------------
    def has_features(self, filter: list[str]) -> list[str]:
        return [f for f in self.features if f in filter]

    def is_supported(self, hw_extension: str) -> bool:
        """True if some feature starts with the name (``sm_100`` matches ``sm_100a``)."""
        wanted = hw_extension.lower()
        return any(f.startswith(wanted) for f in self.features)
