"""``ScheduleParameters``: per-layer parameter dictionaries with JSON persistence, the
interface of lighthouse/schedule/parameters.py:6-128 of the reference (a list of dicts, each
with a ``layer_kind`` string and values that are scalars or flat sequences of scalars)."""

from __future__ import annotations

import json
import os
from collections.abc import Iterator

_SCALARS = (int, float, str, bool)


def _check_entry(entry) -> None:
    if not isinstance(entry, dict):
        raise ValueError(f"Each parameter entry must be a dictionary: found '{entry}'.")
    kind = entry.get("layer_kind")
    if kind is None:
        raise ValueError("Each parameter dictionary must contain a 'layer_kind' key.")
    if not isinstance(kind, str):
        raise ValueError("'layer_kind' must be a string.")
    for key, value in entry.items():
        if not isinstance(key, str):
            raise ValueError(f"Parameter dictionary keys must be strings: found '{key}'.")
        ok = isinstance(value, _SCALARS) or (isinstance(value, (list, tuple)) and all(isinstance(v, _SCALARS) for v in value))
        if not ok:
            raise ValueError(f"Parameter dictionary values must be an int, float, str, bool, list, or tuple: found '{value}' for key '{key}'.")


class ScheduleParameters:
    """Behaves as a list of parameter dictionaries, one per layer of the payload in walk
    order; what the keys mean is up to the schedule that consumes them (here: ``tile_n`` of a
    ``matmul`` layer is the GEMM kernel's tile width)."""

    def __init__(self, list_of_parameters: list[dict] | None = None):
        if list_of_parameters is not None and not isinstance(list_of_parameters, list):
            raise ValueError(f"list_of_parameters must be a list of dictionaries or None, got {type(list_of_parameters)}")
        for entry in list_of_parameters or []:
            _check_entry(entry)
        self.list_of_parameters: list[dict] = list(list_of_parameters or [])

    def __iter__(self) -> Iterator[dict]:
        return iter(self.list_of_parameters)

    def __len__(self) -> int:
        return len(self.list_of_parameters)

    def __getitem__(self, index: int) -> dict:
        return self.list_of_parameters[index]

    def __setitem__(self, index: int, value: dict) -> None:
        _check_entry(value)
        self.list_of_parameters[index] = value

    def __delitem__(self, index: int) -> None:
        del self.list_of_parameters[index]

    def append(self, value: dict) -> None:
        _check_entry(value)
        self.list_of_parameters.append(value)

    def extend(self, values: list[dict]) -> None:
        for v in values:
            _check_entry(v)
        self.list_of_parameters.extend(values)

    def insert(self, index: int, value: dict) -> None:
        _check_entry(value)
        self.list_of_parameters.insert(index, value)

    def to_json(self, filename, overwrite: bool = False) -> None:
        if not overwrite and os.path.exists(filename):
            raise FileExistsError(f"File '{filename}' already exists. Use 'overwrite=True' to overwrite it.")
        with open(filename, "w") as f:
            json.dump(self.list_of_parameters, f, indent=4)

    @classmethod
    def from_json(cls, filename: str) -> "ScheduleParameters":
        with open(filename) as f:
            return cls(json.load(f))
