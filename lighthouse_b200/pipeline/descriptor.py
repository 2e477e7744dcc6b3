"""Pipeline descriptors.

A *descriptor* is one stage written in the mini-syntax of the reference
(lighthouse/pipeline/descriptor.py:8-287)::

    name[arg=value,arg=value]{opt=value flag opt=[1,2,3]}

and a *pipeline descriptor* is a YAML file whose ``Pipeline`` list names such stages, may
include other files, and substitutes ``$var`` with the options of the including descriptor::

    Pipeline:
      - include: other.yaml{fuse=false}
      - pass: cuda-fuse-epilogues
      - backend: cuda{fuse=$fuse fuse_attention}

The reference's stage keys ``pass`` / ``transform`` / ``schedule`` / ``include`` name MLIR passes
and transform-dialect schedules. This backend adds one key, ``backend``, which selects the CUDA
dispatch stage; any other key is rejected as upstream rejects unknown keys.
"""

from __future__ import annotations

import os
import re

import yaml

from ..utils.types import string_to_type

_KINDS = ("pass", "transform", "include", "backend")
# where a file named without a directory is looked for, by extension (relative to this package)
_PACKAGED = {".py": "../schedule", ".yaml": "./descriptors"}
_HEAD = re.compile(r"^[^\[{]*")           # everything before the first '[' or '{'
_ARGS = re.compile(r"^[^{]*?\[([^\]]*)\]")  # a '[...]' that comes before any '{'
_OPTS = re.compile(r"\{([^}]+)\}")


def _assignments(text: str, separator: str) -> dict:
    """``k=v`` items (values typed by ``string_to_type``); a bare item is a true flag."""
    out = {}
    for item in (piece.strip() for piece in text.split(separator)):
        if item:
            key, eq, value = item.partition("=")
            out[key.strip()] = string_to_type(value.strip()) if eq else True
    return out


class Descriptor:
    """``basename``, ``args`` (from ``[...]``), ``opts`` (from ``{...}``) and ``type`` of one
    stage. The type is given by the YAML key, or inferred from the name: a ``.yaml`` file is an
    include, a ``.mlir`` / ``.py`` file a transform, a bare name a pass."""

    search_path = _PACKAGED

    def __init__(self, descriptor: str = "", args: dict | None = None, opts: dict | None = None, type: str | None = None, base_path: str | None = None):
        self.type = "transform" if type == "schedule" else type
        self.base_path = base_path
        if descriptor and not args and not opts:
            self.basename, self.args, self.opts = self._parse_args_and_opts(descriptor)
        else:
            self.basename, self.args, self.opts = descriptor, dict(args or {}), dict(opts or {})
        if self.is_include() or self.is_transform():
            self.basename = self._locate(self.basename)
        if self.base_path is None and self.basename:
            self.base_path = os.path.dirname(self.basename)

    # -- what kind of stage ------------------------------------------------------------
    def _infer(self) -> str | None:
        name = self.basename or ""
        if name.endswith(".yaml") and not self.args and not self.opts:
            return "include"
        if name.endswith((".mlir", ".py")):
            return "transform"
        if name and not self.args and not self.opts and not re.search(r"\.\w+$", name):
            return "pass"
        return None

    def _is(self, kind: str) -> bool:
        if self.type is None:
            inferred = self._infer()
            if inferred == kind:
                self.type = kind
        return self.type == kind

    def is_pass(self) -> bool:
        return self._is("pass")

    def is_include(self) -> bool:
        return self._is("include")

    def is_transform(self) -> bool:
        return self._is("transform")

    def is_backend(self) -> bool:
        return self.type == "backend"

    # -- files ---------------------------------------------------------------------------
    def _locate(self, name: str) -> str:
        """A file as given, else beside the including file, else in the packaged directory
        for its extension."""
        if os.path.exists(os.path.abspath(name)):
            return name
        filename = _HEAD.match(str(name)).group(0)
        tried = []
        if self.base_path and os.path.exists(self.base_path):
            tried.append(self.base_path)
        packaged = self.search_path.get(os.path.splitext(filename)[1])
        if packaged is not None:
            tried.append(os.path.normpath(os.path.join(os.path.dirname(__file__), packaged)))
        for directory in tried:
            candidate = os.path.join(directory, filename)
            if os.path.exists(candidate):
                return candidate
        raise ValueError(f"Included pipeline descriptor file does not exist: {filename} (searched in {' and '.join(map(str, tried)) or self.base_path})")

    # -- the mini-syntax -------------------------------------------------------------------
    @staticmethod
    def _parse_args_and_opts(line: str):
        line = str(line)
        args = _ARGS.search(line)
        opts = _OPTS.search(line)
        return (
            _HEAD.match(line).group(0).strip(),
            _assignments(args.group(1), ",") if args else {},
            _assignments(" ".join(opts.group(1).split()), " ") if opts else {},
        )

    def __str__(self) -> str:
        text = self.basename
        if self.args:
            text += "[" + ",".join(f"{k}={v}" for k, v in self.args.items()) + "]"
        if self.opts:
            text += "{" + " ".join(k if v is True else f"{k}={v}" for k, v in self.opts.items()) + "}"
        return text


class PipelineDescriptor:
    """A YAML pipeline file as a flat list of stage descriptors: includes are expanded in
    place (recursively) and ``$var`` is replaced by the including descriptor's options."""

    STAGE_KEYS = ("pass", "transform", "schedule", "include", "backend")

    def __init__(self, desc: Descriptor):
        if not isinstance(desc, Descriptor):
            raise ValueError(f"PipelineDescriptor requires a Descriptor as input, got {type(desc)}")
        self.descriptor = desc
        self.base_path = os.path.dirname(desc.basename) if desc.basename else desc.base_path
        with open(desc.basename) as f:
            self.pipeline_desc = yaml.safe_load(f) or {}
        entries = self.pipeline_desc.get("Pipeline")
        if not entries:
            raise ValueError(f"Pipeline description file {desc.basename} does not contain a 'Pipeline' key.")
        self.stages: list[Descriptor] = []
        for entry in entries:
            (key, value), = entry.items()
            self.stages.extend(self._stage(key, self._substitute(str(value))))
        if not self.stages:
            raise ValueError(f"Pipeline description file {desc.basename} does not contain a valid 'Pipeline'.")

    def _substitute(self, line: str) -> str:
        for var, value in self.descriptor.opts.items():
            line = line.replace("$" + var, str(value).replace(" ", ""))
        return line

    def _stage(self, key: str, line: str) -> list[Descriptor]:
        if key not in self.STAGE_KEYS:
            raise ValueError(f"Invalid stage in pipeline description: {key}: {line}.")
        desc = Descriptor(line, type=key, base_path=self.base_path)
        if desc.is_include():
            return PipelineDescriptor(desc).get_stages()
        if desc.type in _KINDS:
            return [desc]
        raise ValueError(f"Invalid stage in pipeline description: {desc}.")

    def get_stages(self) -> list[Descriptor]:
        return self.stages
