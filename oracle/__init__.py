"""CPU oracle for the lighthouse_b200 parity tests (test infrastructure only).

See ``oracle/reference_ops.py`` for what each function restates and how it is pinned.
Nothing under ``lighthouse_b200/`` may import this package.
"""
