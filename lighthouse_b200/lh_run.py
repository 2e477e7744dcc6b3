"""``lh-run`` for the CUDA backend: same flags, output strings and exit codes as the
reference's runner CLI (lighthouse/lh_run.py:14-144).

    python -m lighthouse_b200.lh_run payload.mlir --stage cuda-dispatch.yaml \\
        --entry-point main --input-shape 16x64xf32xrnd,64x32xf32x1,16x32xf32x0 \\
        --seed 123 --print-tensor 3

Differences forced by the target: the reference always appends ``convert-linalg-to-loops``
and ``llvm-lowering.yaml`` to reach the LLVM JIT (lh_run.py:106-107); here the pipeline must
end with plans for the native library instead, so if no stage produced them the CUDA
dispatch stage is appended. ``-O`` is accepted and has no effect.
"""

from __future__ import annotations

import argparse
import sys
from datetime import datetime

import numpy as np


# (flag, argparse keywords): the reference CLI's flags, described in this backend's terms
_ON_OFF = argparse.BooleanOptionalAction
_FLAGS = [
    ("payload_module", dict(type=str, help="MLIR text of the payload (a file path).")),
    ("--entry-point", dict(type=str, required=True, help="Function of the payload to run.")),
    ("--input-shape", dict(required=True, help="One DIMSxTYPExINIT field per argument, comma separated: 16x64xf32xrnd,64x32xf32x1 (INIT: 0, 1, rnd, id).")),
    ("--seed", dict(type=int, default=0, help="Seed of numpy's generator for 'rnd' arguments; 0 takes the clock.")),
    ("--stage", dict(action="append", required=True, help="A pass name, a pipeline YAML or a backend descriptor; may be given several times, applied in order.")),
    ("-O", dict(type=int, default=3, help="Kept for command-line compatibility; the kernels are not re-optimised.")),
    ("--benchmark", dict(action=_ON_OFF, help="Time the entry point instead of running it once.")),
    ("--print-optimized-module", dict(action=_ON_OFF, help="Print the plan each function was recognised as.")),
    ("--print-tensor", dict(type=int, default=0, help="Print argument N (1-based) after the run; 0 prints nothing.")),
    ("--print-mlir-after-all", dict(action=_ON_OFF, help="Print the module after every stage.")),
]


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="lh-run", description="Runs an MLIR payload module on a B200 through the CUDA dispatch pipeline.")
    for flag, keywords in _FLAGS:
        parser.add_argument(flag, **keywords)
    return parser


def main(argv=None) -> int:
    try:
        args = build_parser().parse_args(argv)
        from .execution.init import KernelArgumentParser
        from .execution.runner import Runner
        from .pipeline.driver import CompilerDriver
        from .pipeline.stage import CudaDispatchStage

        # A zero seed means "no seed given": seed from the clock, as the reference does.
        np.random.seed(args.seed if args.seed else int(datetime.now().timestamp()))

        driver = CompilerDriver(args.payload_module)
        if args.benchmark:
            driver.add_module_stage(Runner.get_bench_wrapper_schedule(args.entry_point))
        else:
            Runner.make_function_callable(driver.module, args.entry_point)
        driver.add_stages(args.stage)
        module = driver.run(print_after_all=bool(args.print_mlir_after_all))
        if not module.plans:
            module = CudaDispatchStage().apply(module)
        if args.print_optimized_module:
            for plan in module.plans.values():
                print(plan)

        buffers = [a.arg for a in KernelArgumentParser.parse_all(args.input_shape)]
        runner = Runner(module, opt_level=args.O)
        try:
            if args.benchmark:
                time_array = runner.benchmark(host_input_buffers=buffers)
                print(f"{len(time_array)} runs: {np.mean(time_array)} seconds")
            else:
                runner.execute(payload_function_name=args.entry_point, host_input_buffers=buffers)
        finally:
            runner.close()

        if args.print_tensor > 0:
            print(f"Output: {buffers[args.print_tensor - 1]}")
        return 0
    except KeyboardInterrupt:
        print("\nInterrupted", file=sys.stderr)
        return 130
    except (FileNotFoundError, OSError, ValueError, RuntimeError) as exc:  # RuntimeError: no GPU / CUDA failure
        print(f"Error: {exc}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
