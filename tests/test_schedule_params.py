"""Schedule parameters and the GEMM tile database: container and JSON round trip as the
reference's ScheduleParameters (lighthouse/schedule/parameters.py:6-128), lookup / model
fallback / apply / autotune of the selector, and the hint's way into the native operator."""

import json

import numpy as np
import pytest

from lighthouse_b200 import _native as N
from lighthouse_b200.plan import ArgSpec, Plan
from lighthouse_b200.schedule import TILE_WIDTHS, CudaTileSelector, ScheduleParameters


def gemm_plan(m, n, k, dtype="bf16"):
    p = Plan("gemm", [ArgSpec((m, n), dtype, "d"), ArgSpec((m, k), dtype, "a"), ArgSpec((k, n), dtype, "b")])
    p.gemm(p.arg(0), p.arg(1), p.arg(2))
    return p


def test_schedule_parameters_container_and_json(tmp_path):
    params = ScheduleParameters([{"layer_kind": "matmul", "wg_tile": [256, 256]}])
    params.append({"layer_kind": "elemwise", "vector": 8, "fast": True})
    assert len(params) == 2 and params[0]["wg_tile"] == [256, 256] and [p["layer_kind"] for p in params] == ["matmul", "elemwise"]
    params[1] = {"layer_kind": "reduction", "rows": 4}
    params.insert(0, {"layer_kind": "matmul", "tile_n": 128})
    del params[1]
    assert [p["layer_kind"] for p in params] == ["matmul", "reduction"]
    path = tmp_path / "params.json"
    params.to_json(path)
    with pytest.raises(FileExistsError):
        params.to_json(path)
    params.to_json(path, overwrite=True)
    assert ScheduleParameters.from_json(path).list_of_parameters == params.list_of_parameters
    for bad in ([{"wg_tile": [1]}], [{"layer_kind": 3}], [{"layer_kind": "matmul", "x": {"nested": 1}}], ["matmul"], "matmul"):
        with pytest.raises(ValueError):
            ScheduleParameters(bad)
    with pytest.raises(ValueError):
        params.append({"tile_n": 64})
    assert len(ScheduleParameters(None)) == 0


def test_selector_database_model_and_apply(tmp_path):
    sel = CudaTileSelector()  # the committed database
    hit = sel.lookup(4096, 4096, 4096)
    assert hit["source"] == "database" and hit["tile_n"] == 256 and hit["layer_kind"] == "matmul"
    miss = sel.lookup(8192, 768, 2048)  # 64 x 3 tiles of 256 = 2 waves; 64 x 4 tiles of 192 = 2 cheaper waves
    assert miss["source"] == "model" and miss["tile_n"] == 192
    assert sel.model_choice(16384, 4096, 4096) == 256

    plan = gemm_plan(8192, 768, 2048)
    params = sel.select(plan)
    assert len(params) == 1 and params[0]["shape"] == [8192, 768, 2048]
    sel.apply(plan, params)
    assert plan.ops[0].attrs["tile_n"] == 192
    # the hint travels in bits 8-15 of the native flags, the documented flags stay in the low bits
    _, _, _, _, ops, nops = plan.to_native()
    assert nops == 1 and ops[0].kind == N.OP_GEMM and ops[0].i1 == (192 // 8) << 8
    plan.ops[0].attrs["flags"] = N.GEMM_ACCUMULATE_C
    assert plan.to_native()[4][0].i1 == ((192 // 8) << 8) | N.GEMM_ACCUMULATE_C
    with pytest.raises(ValueError):
        sel.apply(plan, ScheduleParameters([{"layer_kind": "matmul", "shape": [8192, 768, 4096], "tile_n": 100}]))
    with pytest.raises(ValueError):
        sel.apply(plan, ScheduleParameters([]))
    # f32 GEMMs are not the tensor-core bf16 kernel's: no entries, nothing set
    f32 = gemm_plan(256, 256, 256, "f32")
    assert len(sel.select(f32)) == 0 and "tile_n" not in sel.apply(f32).ops[0].attrs


def test_autotune_records_the_fastest_width(tmp_path):
    db = tmp_path / "tiles.json"
    sel = CudaTileSelector(str(db))
    assert sel.lookup(1024, 512, 256)["source"] == "model"
    calls = []

    def measure(m, n, k, tile_n):  # stands in for a GPU timing: 128-wide tiles win
        calls.append(tile_n)
        return 1e-3 * (1.0 + abs(tile_n - 128) / 256)

    tuned = sel.autotune([(1024, 512, 256)], measure)
    assert sorted(calls) == sorted(TILE_WIDTHS) and tuned[0]["tile_n"] == 128 and tuned[0]["source"] == "autotune"
    stored = json.loads(db.read_text())
    assert stored[0]["shape"] == [1024, 512, 256] and stored[0]["tile_n"] == 128 and set(stored[0]["seconds"]) == {"256", "192", "128", "64"}
    assert stored[0]["tflops"] == pytest.approx(2 * 1024 * 512 * 256 / 1e-3 / 1e12, abs=0.06)  # stored to one decimal
    again = CudaTileSelector(str(db)).lookup(1024, 512, 256)
    assert again["source"] == "database" and again["tile_n"] == 128


@pytest.mark.gpu
def test_every_tile_width_hint_gives_the_same_product(ctx):
    import torch

    from oracle import reference_ops as R
    from oracle.check import TOL_BF16, max_rel_err, assert_parity
    from lighthouse_b200.workloads.session import PlanSession

    rng = np.random.RandomState(5)
    m, n, k = 384, 448, 320
    a, b = R.round_bf16(rng.randn(m, k).astype(np.float32) * 0.5), R.round_bf16(rng.randn(k, n).astype(np.float32) * 0.2)
    ad, bd = torch.from_numpy(a).to(torch.bfloat16).cuda(), torch.from_numpy(b).to(torch.bfloat16).cuda()
    want = R.round_bf16(a @ b)
    for tile_n in TILE_WIDTHS:
        plan = gemm_plan(m, n, k)
        plan.ops[0].attrs["tile_n"] = tile_n
        d = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
        s = PlanSession(plan, ctx=ctx)
        s.run([d, ad, bd], sync=True)
        s.close()
        assert_parity(d.float().cpu().numpy(), want, "bf16")


def test_selector_covers_a_decoder_plan():
    from lighthouse_b200.workloads import decoder as D

    cfg = D.LlamaConfig(n_layer=2)
    plan = D.build_llama_plan(cfg)
    sel = CudaTileSelector()
    params = sel.select(plan)
    gemms = [op for op in plan.ops if op.kind == "gemm"]
    assert len(params) == len(gemms) == 6  # per layer: output projection, gate/up (SwiGLU), down (the q/k/v projection is a gemm_rope)
    assert {tuple(p["shape"]) for p in params} == {(16384, 4096, 4096), (16384, 28672, 4096), (16384, 4096, 14336)}
    sel.apply(plan, params)
    hinted = [op for op in gemms if "tile_n" in op.attrs]
    assert len(hinted) == 4 and all(op.attrs["tile_n"] == 256 for op in hinted)  # SwiGLU GEMMs keep their fixed width
