"""Target description (the role of lighthouse/execution/target.py:13-132 in the reference).

The reference derives ``arch`` from ``platform.machine()`` and ``features`` from ``lscpu``;
this backend has one target: ``arch="cuda"`` with the compute capability as a feature
(``sm_100a`` on B200). ``TargetInfo.override`` is kept so tests can fake a target the same
way the reference's tests do (test/execution/target_info_host_override.py:10-40).
"""

from __future__ import annotations

from contextlib import contextmanager


class TargetInfo:
    _cached_host: "TargetInfo | None" = None
    _override_features_stack: list = []
    _override_arch_stack: list = []

    def __init__(self, arch: str | None = None, features: list[str] | None = None, filter: list[str] | None = None):
        if arch is None and self._override_arch_stack:
            arch = self._override_arch_stack[-1]
        if features is None and self._override_features_stack:
            override = self._override_features_stack[-1]
            if override is not None:
                features = list(override)
        self.arch = arch if arch is not None else "cuda"
        self.features = features if features is not None else self._get_feature_list()
        if filter is not None:
            self.features = self.has_features(filter)

    @classmethod
    def host(cls) -> "TargetInfo":
        if cls._override_features_stack or cls._override_arch_stack:
            return cls()
        if cls._cached_host is None:
            cls._cached_host = cls()
        return cls._cached_host

    @classmethod
    def cuda(cls) -> "TargetInfo":
        """The one target this backend executes on."""
        return cls(arch="cuda", features=["sm_100a"])

    @classmethod
    def reset_host_cache(cls) -> None:
        cls._cached_host = None

    @classmethod
    @contextmanager
    def override(cls, *, features: list[str] | None = None, arch: str | None = None):
        cls._override_features_stack.append(None if features is None else list(features))
        cls._override_arch_stack.append(arch)
        cls.reset_host_cache()
        try:
            yield
        finally:
            cls._override_features_stack.pop()
            cls._override_arch_stack.pop()
            cls.reset_host_cache()

    def _get_feature_list(self) -> list[str]:
        """``sm_<major><minor>[a]`` of device 0 when a GPU is visible, else the build target."""
        try:
            import torch

            if torch.cuda.is_available():
                major, minor = torch.cuda.get_device_capability(0)
                name = f"sm_{major}{minor}"
                return [name + "a", name] if major >= 9 else [name]
        except Exception:
            pass
        return ["sm_100a"]

    def has_features(self, filter: list[str]) -> list[str]:
        return [f for f in self.features if f in filter]

    def is_supported(self, hw_extension: str) -> bool:
        hw_extension = hw_extension.lower()
        return any(f.startswith(hw_extension) for f in self.features)
