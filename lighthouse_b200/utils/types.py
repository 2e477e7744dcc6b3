"""String -> value coercion for descriptor options (the role of
lighthouse/utils/types.py:30-80 in the reference: ``k=v`` options arrive as text)."""

from __future__ import annotations


def string_to_type(value: str):
    """``"true"/"false"`` -> bool, ints, floats, ``[a,b]`` lists (recursively), else the string."""
    v = value.strip()
    low = v.lower()
    if low in ("true", "false"):
        return low == "true"
    if v.startswith("[") and v.endswith("]"):
        inner = v[1:-1].strip()
        return [string_to_type(p) for p in inner.split(",")] if inner else []
    for cast in (int, float):
        try:
            return cast(v)
        except ValueError:
            pass
    if len(v) >= 2 and v[0] == v[-1] and v[0] in "\"'":
        return v[1:-1]
    return v
