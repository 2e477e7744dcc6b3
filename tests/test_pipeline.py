"""Descriptors, finder, drivers, argument parsing and the lh-run / lh-opt CLIs (host logic;
the reference tests the same layer in test/pipeline/ and test/execution/)."""

import os
from unittest import mock

import numpy as np
import pytest

from conftest import PAYLOADS

from lighthouse_b200.execution import KernelArgumentParser, TargetInfo
from lighthouse_b200.execution.init import InitType
from lighthouse_b200.payload import as_payload_module
from lighthouse_b200.payload import generators as G
from lighthouse_b200.pipeline import (
    CompilerDriver, CudaDispatchStage, Descriptor, PipelineDescriptor, PipelineDriver, Stage, TransformDriver, find_pipeline_file,
)
from lighthouse_b200.pipeline import finder as finder_mod

MATMUL = os.path.join(PAYLOADS, "matmul_16x32x64_f32.mlir")


def test_descriptor_mini_syntax():
    d = Descriptor("cuda-fuse-epilogues")
    assert d.is_pass() and str(d) == "cuda-fuse-epilogues"
    d = Descriptor("cuda{fuse=false fuse_attention}", type="backend")
    assert d.is_backend() and d.opts == {"fuse": False, "fuse_attention": True}
    name, args, opts = Descriptor._parse_args_and_opts("sched.py[gen=make,seq=x]{m=4096 tiles=[1,2,3] flag}")
    assert name == "sched.py" and args == {"gen": "make", "seq": "x"} and opts == {"m": 4096, "tiles": [1, 2, 3], "flag": True}


def test_yaml_pipeline_includes_and_variables(tmp_path):
    (tmp_path / "inner.yaml").write_text("Pipeline:\n  - backend: \"cuda{fuse=$fuse}\"\n")
    (tmp_path / "outer.yaml").write_text("Pipeline:\n  - pass: cuda-recognize\n  - include: inner.yaml{fuse=false}\n")
    stages = PipelineDescriptor(Descriptor(str(tmp_path / "outer.yaml"))).get_stages()
    assert [s.type for s in stages] == ["pass", "backend"] and stages[1].opts == {"fuse": False}
    (tmp_path / "bad.yaml").write_text("Pipeline:\n  - frobnicate: x\n")
    with pytest.raises(ValueError):
        PipelineDescriptor(Descriptor(str(tmp_path / "bad.yaml")))
    (tmp_path / "empty.yaml").write_text("Other: 1\n")
    with pytest.raises(ValueError):
        PipelineDescriptor(Descriptor(str(tmp_path / "empty.yaml")))
    with pytest.raises(ValueError):
        Descriptor("does-not-exist.yaml")


def test_packaged_descriptors_resolve_by_name():
    stages = PipelineDescriptor(Descriptor("cuda/matmul/bf16.yaml")).get_stages()
    assert len(stages) == 1 and stages[0].is_backend() and stages[0].basename == "cuda"
    staged = PipelineDescriptor(Descriptor("cuda-staged.yaml")).get_stages()
    assert [s.basename for s in staged] == ["cuda-recognize", "cuda-fuse-epilogues", "cuda-fuse-norm-cast", "cuda-fuse-attention"]


def test_find_pipeline_file_with_fixture_tree(tmp_path):
    (tmp_path / "cuda" / "sm_100a" / "matmul").mkdir(parents=True)
    (tmp_path / "cuda" / "matmul").mkdir(parents=True)
    (tmp_path / "cuda" / "sm_100a" / "matmul" / "bf16.yaml").write_text("Pipeline: []\n")
    (tmp_path / "cuda" / "matmul" / "f32.yaml").write_text("Pipeline: []\n")
    b200 = TargetInfo(arch="cuda", features=["sm_100a"])
    with mock.patch.object(finder_mod, "DESCRIPTORS_REPO", tmp_path):
        assert find_pipeline_file(b200, "matmul", "bf16") == (str(tmp_path / "cuda" / "sm_100a" / "matmul" / "bf16.yaml"), "sm_100a")
        assert find_pipeline_file(b200, "matmul", "f32") == (str(tmp_path / "cuda" / "matmul" / "f32.yaml"), None)
        assert find_pipeline_file(TargetInfo(arch="cuda", features=["sm_90"]), "matmul", "bf16") == (None, None)
        assert find_pipeline_file(TargetInfo(arch="x86_64", features=[]), "matmul", "f32") == (None, None)
    # packaged tree, and an external base path taking precedence
    path, feature = find_pipeline_file(TargetInfo.cuda(), "attention", "bf16")
    assert path.endswith(os.path.join("cuda", "attention", "bf16.yaml")) and feature is None
    assert find_pipeline_file(b200, "matmul", "f32", base_path=str(tmp_path))[0].startswith(str(tmp_path))
    assert find_pipeline_file(None, "matmul") == (None, None)


def test_target_info_override():
    with TargetInfo.override(features=["sm_90"], arch="cuda"):
        t = TargetInfo.host()
        assert t.arch == "cuda" and t.features == ["sm_90"] and not t.is_supported("sm_100")
    assert TargetInfo.cuda().is_supported("sm_100")


def test_kernel_argument_parser():
    np.random.seed(123)
    args = KernelArgumentParser.parse_all("16x64xf32xrnd,64x32xf32x1,16x32xf32x0,4x4xbf16xid")
    assert [a.arg.shape for a in args] == [(16, 64), (64, 32), (16, 32), (4, 4)]
    assert args[0].init_type == InitType.RANDOM and 0.0 <= args[0].arg.min() and args[0].arg.max() < 1.0
    assert args[1].arg.sum() == 64 * 32 and args[2].arg.sum() == 0 and args[3].arg.dtype.name == "bfloat16"
    for bad in ("16x64xf33xrnd", "axbxf32x0", "4x4xf32xfoo", "0x4xf32x0", "3x4xf32xid"):
        with pytest.raises(ValueError):
            KernelArgumentParser.parse(bad)


def test_drivers_and_stages(tmp_path):
    drv = CompilerDriver(MATMUL, stages=["cuda-staged.yaml"])
    mod = drv.run()
    assert list(mod.plans) == ["main"] and [op.kind for op in mod.plans["main"].ops] == ["gemm"]
    with pytest.raises(ValueError):
        drv.add_stage("cuda-recognize")  # fixed after run
    with pytest.raises(ValueError):
        drv.run()  # module consumed
    with pytest.raises(ValueError):
        CompilerDriver(str(tmp_path / "nope.mlir"))
    with pytest.raises(ValueError):
        CompilerDriver(MATMUL).run()  # no stages
    with pytest.raises(ValueError):
        CompilerDriver(MATMUL, stages=["not-a-known-pass"])
    # upstream lowering pass names are accepted and ignored
    mod = CompilerDriver(MATMUL, stages=["canonicalize", "cuda-dispatch.yaml", "convert-linalg-to-loops"]).run()
    assert mod.plans

    class Counter(Stage):
        seen = 0

        def apply(self, module):
            Counter.seen += 1
            return module

    pm = as_payload_module(str(G.generate_gpu_softmax_payload("payload", 4, 8, "f32")), lower=False)
    out = TransformDriver([Counter(), CudaDispatchStage(fuse=False)]).apply(pm)
    assert Counter.seen == 1 and out.plans["payload"].ops[0].kind == "softmax"
    # a Python schedule file whose generator returns a stage
    sched = tmp_path / "sched.py"
    sched.write_text("from lighthouse_b200.pipeline import CudaDispatchStage\n\ndef create_schedule(fuse=True):\n    return CudaDispatchStage(fuse=fuse)\n")
    d = PipelineDriver()
    d.add_stage(Descriptor(f"{sched}{{fuse=false}}"))
    assert d.apply(as_payload_module(MATMUL, lower=False)).plans
    with pytest.raises(ValueError):
        PipelineDriver().add_stage(Descriptor("cuda{bogus=1}", type="backend"))


def test_lh_run_cli_errors_map_to_exit_code_1(capsys):
    from lighthouse_b200 import lh_opt, lh_run

    assert lh_run.main(["/no/such/file.mlir", "--stage", "cuda-dispatch.yaml", "--entry-point", "main", "--input-shape", "4x4xf32x0"]) == 1
    assert "Error:" in capsys.readouterr().err
    assert lh_run.main([MATMUL, "--stage", "cuda-dispatch.yaml", "--entry-point", "missing", "--input-shape", "4x4xf32x0"]) == 1
    assert lh_run.main([MATMUL, "--stage", "bogus-pass", "--entry-point", "main", "--input-shape", "4x4xf32x0"]) == 1
    capsys.readouterr()
    assert lh_opt.main([MATMUL, "--stage", "cuda-dispatch.yaml"]) == 0
    out = capsys.readouterr().out
    assert "linalg.matmul" in out and "plan @main" in out
