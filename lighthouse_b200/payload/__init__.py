"""Payload layer: MLIR text <-> in-memory payloads <-> plans."""

from __future__ import annotations

import os

from .ir import PayloadModule
from .lower import UnsupportedPayload, lower_module, recognize
from .parser import ParseError, parse_mlir

__all__ = ["PayloadModule", "ParseError", "UnsupportedPayload", "as_payload_module", "lower_module", "parse_mlir", "recognize"]


def as_payload_module(module, lower: bool = True) -> PayloadModule:
    """Accepts a ``PayloadModule``, a ``Plan``, MLIR text, a path to an ``.mlir`` file, or any
    object whose ``str()`` is MLIR text (an ``ir.Module`` of the upstream bindings). With
    ``lower`` the result carries plans (the CUDA dispatch stage is applied if it was not yet)."""
    from ..plan import Plan

    if isinstance(module, Plan):
        pm = PayloadModule()
        pm.plans[module.entry] = module
        return pm
    if isinstance(module, PayloadModule):
        pm = module
    elif isinstance(module, (str, os.PathLike)):
        text = os.fspath(module)
        if "\n" not in text and os.path.exists(text):
            with open(text) as f:
                pm = parse_mlir(f.read())
            pm.source_path = text
        elif "func.func" in text or "module" in text:
            pm = parse_mlir(text)
        else:
            raise ValueError(f"Path to the module does not exist: {text}")
    elif module is None:
        raise ValueError("module must be provided")
    else:
        pm = parse_mlir(str(module))
    if lower and not pm.plans:
        lower_module(pm)
    return pm
