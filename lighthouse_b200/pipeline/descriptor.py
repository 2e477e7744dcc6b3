"""Pipeline descriptors: the ``name[arg=...]{opt=... opt}`` mini-syntax and YAML pipeline
files, with the grammar of lighthouse/pipeline/descriptor.py:8-287 in the reference.

One stage key is added to the YAML grammar: ``backend: cuda{...}`` selects the CUDA dispatch
stage (the reference's keys ``pass`` / ``transform`` / ``schedule`` / ``include`` name MLIR
passes and transform-dialect schedules, which this backend does not run).

    Pipeline:
      - include: other.yaml
      - pass: cuda-fuse-epilogues
      - backend: cuda{fuse=true fuse_attention=true}
"""

from __future__ import annotations

import os
import re

import yaml

from ..utils.types import string_to_type


class Descriptor:
    """basename + ``[args]`` + ``{opts}`` + type (pass | transform | include | backend)."""

    search_path = {".py": "../schedule", ".yaml": "./descriptors"}

    def __init__(self, descriptor: str = "", args: dict | None = None, opts: dict | None = None, type: str | None = None, base_path: str | None = None):
        self.type = "transform" if type == "schedule" else type
        self.base_path = base_path
        if descriptor and not args and not opts:
            self.basename, self.args, self.opts = self._parse_args_and_opts(descriptor)
        else:
            self.basename = descriptor
            self.args = args if args is not None else {}
            self.opts = opts if opts is not None else {}
        if self.is_include() or self.is_transform():
            self.basename = self._normalize_include_path()
        if self.base_path is None and self.basename:
            self.base_path = os.path.dirname(self.basename)

    def is_backend(self) -> bool:
        return self.type == "backend"

    def is_pass(self) -> bool:
        if self.type == "pass":
            return True
        if self.type in ("transform", "include", "backend"):
            return False
        if self.basename and not self.args and not self.opts and not re.search(r"\.\w+$", self.basename):
            self.type = "pass"
            return True
        return False

    def is_include(self) -> bool:
        if self.type == "include":
            return True
        if self.type in ("pass", "transform", "backend"):
            return False
        if self.basename and not self.args and not self.opts and self.basename.endswith(".yaml"):
            self.type = "include"
            return True
        return False

    def is_transform(self) -> bool:
        if self.type == "transform":
            return True
        if self.type in ("pass", "include", "backend"):
            return False
        if self.basename and (self.basename.endswith(".mlir") or self.basename.endswith(".py")):
            self.type = "transform"
            return True
        return False

    def _normalize_include_path(self) -> str:
        """Looks beside the including file first, then in the packaged directory for the extension."""
        if os.path.exists(os.path.abspath(self.basename)):
            return self.basename
        filename = self._remove_args_and_opts(self.basename)
        if self.base_path and os.path.exists(self.base_path):
            candidate = os.path.join(self.base_path, filename)
            if os.path.exists(candidate):
                return candidate
        ext = os.path.splitext(filename)[1]
        if ext not in self.search_path:
            raise ValueError(f"Included pipeline descriptor file does not exist: {filename} (searched in {self.base_path})")
        root = os.path.normpath(os.path.join(os.path.dirname(__file__), self.search_path[ext]))
        candidate = os.path.join(root, filename)
        if os.path.exists(candidate):
            return candidate
        raise ValueError(f"Included pipeline descriptor file does not exist: {filename} (searched in {self.base_path} and {root})")

    @staticmethod
    def _parse_csv(line: str, separator: str = ",") -> dict:
        result = {}
        for item in str(line).split(separator):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                key, value = item.split("=", 1)
                result[key.strip()] = string_to_type(value.strip())
            else:
                result[item] = True
        return result

    @staticmethod
    def _remove_args_and_opts(line: str) -> str:
        m = re.search(r"^([^[{]*)", str(line))
        return m.group(1) if m else str(line)

    @staticmethod
    def _parse_args_and_opts(line: str):
        line = str(line)
        args, options = {}, {}
        if re.match(r"[^{]+\[", line):  # '[...]' that is not inside '{...}'
            m = re.search(r"\[([^]]*)\]", line)
            if m:
                args = Descriptor._parse_csv(m.group(1).strip(), ",")
        m = re.search(r"\{([^}]+)\}", line)
        if m:
            options = Descriptor._parse_csv(" ".join(m.group(1).split()), " ")
        return Descriptor._remove_args_and_opts(line).strip(), args, options

    def __str__(self) -> str:
        args_str = "[" + ",".join(f"{k}={v}" for k, v in self.args.items()) + "]" if self.args else ""
        opts_str = ""
        if self.opts:
            opts_str = "{" + " ".join(k if isinstance(v, bool) and v else f"{k}={v}" for k, v in self.opts.items()) + "}"
        return f"{self.basename}{args_str}{opts_str}"


class PipelineDescriptor:
    """A YAML pipeline file flattened (includes resolved, ``$var`` substituted) into stages."""

    STAGE_KEYS = ("pass", "transform", "schedule", "include", "backend")

    def __init__(self, desc: Descriptor):
        if not isinstance(desc, Descriptor):
            raise ValueError(f"PipelineDescriptor requires a Descriptor as input, got {type(desc)}")
        self.descriptor = desc
        self.base_path = os.path.dirname(desc.basename) if desc.basename else desc.base_path
        with open(desc.basename) as f:
            self.pipeline_desc = yaml.safe_load(f) or {}
        self._apply_variables()
        self.stages: list[Descriptor] = []
        self._parse_stages()
        if not self.stages:
            raise ValueError(f"Pipeline description file {desc.basename} does not contain a valid 'Pipeline'.")

    def _apply_variables(self) -> None:
        pipeline = self.pipeline_desc.get("Pipeline") or []
        for idx, item in enumerate(pipeline):
            key, line = next(iter(item.items()))
            line = str(line)
            for var, value in self.descriptor.opts.items():
                line = line.replace("$" + var, str(value).replace(" ", ""))
            pipeline[idx] = {key: line}

    def _parse_stages(self) -> None:
        pipeline = self.pipeline_desc.get("Pipeline")
        if not pipeline:
            raise ValueError(f"Pipeline description file {self.descriptor.basename} does not contain a 'Pipeline' key.")
        for stage in pipeline:
            key, value = next(iter(stage.items()))
            if key not in self.STAGE_KEYS:
                raise ValueError(f"Invalid stage in pipeline description: {key}: {value}.")
            desc = Descriptor(value, type=key, base_path=self.base_path)
            if desc.is_include():
                self.stages.extend(PipelineDescriptor(desc).get_stages())
            elif desc.is_transform() or desc.is_pass() or desc.is_backend():
                self.stages.append(desc)
            else:
                raise ValueError(f"Invalid stage in pipeline description: {desc}.")

    def get_stages(self) -> list[Descriptor]:
        return self.stages
