"""Tile database and selector for the tensor-core GEMM, in the shape of the reference's
``XeGPUParameterSelector`` (lighthouse/schedule/xegpu/xegpu_parameter_selector.py:26-85 with its
``matmul_params.json``): a JSON file of per-(M, N, K) tile parameters, a lookup that falls
back to a model for shapes the file does not hold, and an autotune pass that fills the file
from measurements.

The only free parameter of ``gemm_bf16_tc_kernel`` is its tile width (128 x {64,128,192,256}
output tiles; the pipeline depth follows from it). Without a hint the library chooses by a
wave model; a plan operator with ``attrs["tile_n"]`` carries the database's choice to the
kernel in bits 8-15 of the GEMM flags.
"""

from __future__ import annotations

import json
import math
import os
from typing import Callable, Iterable

from ..plan import Plan
from .parameters import ScheduleParameters

TILE_WIDTHS = (256, 192, 128, 64)
_DEFAULT_DB = os.path.join(os.path.dirname(__file__), "matmul_params.json")
# relative efficiency of a tile of each width at equal wave counts (4096 x 4096 x K measurements)
_WIDTH_EFFICIENCY = {256: 1.0, 192: 0.88, 128: 0.72, 64: 0.5}


def _key(m: int, n: int, k: int) -> str:
    return f"{m}x{n}x{k}"


class CudaTileSelector:
    """``select(plan)`` gives one parameter dictionary per GEMM of the plan; ``apply`` writes
    the tile widths into the plan; ``autotune`` measures the candidates and records the best."""

    def __init__(self, db_path: str | None = None, sm_count: int = 148):
        self.db_path = db_path or _DEFAULT_DB
        self.sm_count = sm_count
        self.db: dict[str, dict] = {}
        if os.path.exists(self.db_path):
            with open(self.db_path) as f:
                self.db = {_key(*e["shape"]): e for e in json.load(f)}

    # -- lookup ------------------------------------------------------------------------
    def model_choice(self, m: int, n: int, k: int) -> int:
        """Waves of tiles over the SMs times the relative cost of a tile of that width (the
        model the library itself applies when it gets no hint)."""
        best, best_cost = 256, math.inf
        for bn in (256, 192, 128):
            tiles = math.ceil(m / 128) * math.ceil(n / bn)
            cost = math.ceil(tiles / self.sm_count) * bn / _WIDTH_EFFICIENCY[bn]
            if cost < best_cost - 1e-9:
                best, best_cost = bn, cost
        return best

    def lookup(self, m: int, n: int, k: int) -> dict:
        entry = self.db.get(_key(m, n, k))
        if entry is not None:
            return {"layer_kind": "matmul", "shape": [m, n, k], "tile_n": int(entry["tile_n"]), "source": "database"}
        return {"layer_kind": "matmul", "shape": [m, n, k], "tile_n": self.model_choice(m, n, k), "source": "model"}

    @staticmethod
    def _gemm_shapes(plan: Plan) -> Iterable[tuple[int, tuple[int, int, int]]]:
        for i, op in enumerate(plan.ops):
            if op.kind == "gemm" and op.operands[1].rank == 2 and op.operands[1].dtype == "bf16":
                a, b = op.operands[1], op.operands[2]
                yield i, (a.shape[0], b.shape[1], a.shape[1])

    def select(self, plan: Plan) -> ScheduleParameters:
        return ScheduleParameters([self.lookup(*shape) for _, shape in self._gemm_shapes(plan)])

    def apply(self, plan: Plan, params: ScheduleParameters | None = None) -> Plan:
        """Sets ``tile_n`` on the plan's bf16 GEMMs, in walk order. SwiGLU GEMMs keep the
        256-wide tile their packed [gate | up] column blocks need."""
        params = params if params is not None else self.select(plan)
        gemms = list(self._gemm_shapes(plan))
        if len(params) != len(gemms):
            raise ValueError(f"{len(params)} parameter entries for {len(gemms)} GEMMs")
        for (i, shape), entry in zip(gemms, params):
            if entry["layer_kind"] != "matmul" or list(entry.get("shape", shape)) != list(shape):
                raise ValueError(f"parameter entry {entry} does not describe the GEMM {shape}")
            tile_n = int(entry["tile_n"])
            if tile_n not in TILE_WIDTHS:
                raise ValueError(f"tile_n must be one of {TILE_WIDTHS}, got {tile_n}")
            if not plan.ops[i].attrs.get("flags", 0) & 4:
                plan.ops[i].attrs["tile_n"] = tile_n
        return plan

    # -- autotune ----------------------------------------------------------------------
    def autotune(self, shapes: Iterable[tuple[int, int, int]], measure: Callable[[int, int, int, int], float], save: bool = True) -> ScheduleParameters:
        """``measure(m, n, k, tile_n)`` returns seconds per launch (on a GPU: a one-GEMM plan
        with that ``tile_n`` timed by ``PlanSession.benchmark``, see ``measure_on_gpu``). The
        fastest width per shape goes into the database with its TFLOP/s."""
        out = ScheduleParameters()
        for m, n, k in shapes:
            timings = {bn: float(measure(m, n, k, bn)) for bn in TILE_WIDTHS if bn <= max(64, 8 * math.ceil(n / 8))}
            best = min(timings, key=timings.get)
            entry = {"shape": [m, n, k], "tile_n": best, "tflops": round(2.0 * m * n * k / timings[best] / 1e12, 1),
                     "seconds": {str(bn): round(t, 9) for bn, t in timings.items()}, "source": "autotune"}
            self.db[_key(m, n, k)] = entry
            out.append({"layer_kind": "matmul", "shape": [m, n, k], "tile_n": best, "source": "autotune"})
        if save:
            with open(self.db_path, "w") as f:
                json.dump(sorted(self.db.values(), key=lambda e: e["shape"]), f, indent=1)
        return out


def measure_on_gpu(ctx, nruns: int = 10, nwarmup: int = 3, l2_flush_bytes: int = 256 << 20, reserved_sms: int = 0) -> Callable[[int, int, int, int], float]:
    """The ``measure`` callback of ``CudaTileSelector.autotune`` on a CUDA context: seeded bf16
    operands, one GEMM per launch, L2 flushed between launches. ``reserved_sms``: the SMs the
    persistent grid leaves free, as in the overlapped tensor-parallel schedules."""
    import torch

    from ..plan import ArgSpec
    from ..workloads.session import PlanSession

    def measure(m: int, n: int, k: int, tile_n: int) -> float:
        g = torch.Generator().manual_seed(2)
        a = (torch.randn(m, k, generator=g) * 0.02).to(torch.bfloat16).cuda()
        b = (torch.randn(k, n, generator=g) * 0.02).to(torch.bfloat16).cuda()
        d = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        plan = Plan("gemm", [ArgSpec((m, n), "bf16", "d"), ArgSpec((m, k), "bf16", "a"), ArgSpec((k, n), "bf16", "b")])
        if reserved_sms:
            plan.reserve_sms(reserved_sms)
        plan.gemm(plan.arg(0), plan.arg(1), plan.arg(2))
        plan.ops[-1].attrs["tile_n"] = tile_n
        if reserved_sms:
            plan.reserve_sms(0)
        session = PlanSession(plan, ctx=ctx)
        torch.cuda.synchronize()
        try:
            return float(session.benchmark([d, a, b], nruns=nruns, nwarmup=nwarmup, l2_flush_bytes=l2_flush_bytes).mean())
        finally:
            session.close()

    return measure


def decoder_gemm_shapes() -> list[tuple[int, int, int, int]]:
    """(M, N, K, reserved SMs) of the GEMMs the benchmark configurations launch whose tile width
    is free (the SwiGLU product keeps its 256-wide tiles): the K sweep of the GEMM
    configuration, the Llama stack at tensor-parallel degrees 1, 2, 4, 8 (micro-batches of half
    the tokens and 8 reserved SMs where it is parallel), nanoGPT on one GPU and with its batch
    split 2, 4 and 8 ways."""
    shapes = [(4096, 4096, k, 0) for k in (512, 1024, 2048, 4096, 8192, 16384)]
    for tp in (1, 2, 4, 8):
        m, r = (16384, 0) if tp == 1 else (8192, 8)
        q, kv, f = 4096 // tp, 1024 // tp, 14336 // tp
        shapes += [(m, q + 2 * kv, 4096, r), (m, 4096, q, r), (m, 4096, f, r)]
    for dp in (1, 2, 4, 8):
        m = 16384 // dp
        shapes += [(m, 2304, 768, 0), (m, 768, 768, 0), (m, 3072, 768, 0), (m, 768, 3072, 0), (m, 50304, 768, 0)]
    return shapes


def main(argv=None) -> int:
    """``python -m lighthouse_b200.schedule.tile_selector --autotune`` measures every tile
    width on the GPU for the benchmark configurations' GEMM shapes and rewrites the database."""
    import argparse

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--autotune", action="store_true")
    ap.add_argument("--db", default=None, help="database file to update (default: the packaged one)")
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    if not args.autotune:
        ap.print_help()
        return 0
    from ..context import CudaContext

    ctx = CudaContext(args.device)
    sel = CudaTileSelector(args.db, sm_count=ctx.sm_count)
    by_reserve: dict[int, list] = {}
    for m, n, k, r in decoder_gemm_shapes():
        by_reserve.setdefault(r, []).append((m, n, k))
    for r, shapes in by_reserve.items():
        for entry in sel.autotune(shapes, measure_on_gpu(ctx, reserved_sms=r)):
            e = sel.db[_key(*entry["shape"])]
            e["reserved_sms"] = r
            print(f"{entry['shape']} reserved {r}: tile_n {entry['tile_n']}  {e['tflops']} TFLOP/s  {e['seconds']}", flush=True)
    with open(sel.db_path, "w") as f:
        json.dump(sorted(sel.db.values(), key=lambda e: e["shape"]), f, indent=1)
    ctx.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
