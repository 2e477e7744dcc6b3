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


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(
        prog="lh-run",
        description="Lighthouse runner on B200: optionally applies pipeline stages to an input MLIR payload module and executes it on the GPU.",
    )
    p.add_argument("payload_module", type=str, help="Path to the payload MLIR module.")
    p.add_argument("--entry-point", type=str, required=True, help="Name of the entrypoint function in the payload MLIR module.")
    p.add_argument(
        "--input-shape",
        required=True,
        help="Shape of the input tensors in format: DIMS(MxNx...)xTYPE(f16/f32/f64/bf16/i8)xINIT(0/1/rnd/id). For multiple inputs, separate by comma.",
    )
    p.add_argument("--seed", type=int, default=0, help="Random seed for initializing input tensors.")
    p.add_argument("--stage", action="append", required=True, help="Pipeline stages to apply to the input module.")
    p.add_argument("-O", type=int, default=3, help="Optimization level (accepted for compatibility).")
    p.add_argument("--benchmark", action=argparse.BooleanOptionalAction, help="Whether to run the benchmark. Default is False.")
    p.add_argument("--print-optimized-module", action=argparse.BooleanOptionalAction, help="Whether to print the recognised module (its plans). Default is False.")
    p.add_argument("--print-tensor", type=int, default=0, help="Print the Nth tensor. Default is 0 (no print).")
    p.add_argument("--print-mlir-after-all", action=argparse.BooleanOptionalAction, help="Whether to print the module after every stage. Default is False.")
    return p


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
