"""``lh-opt`` for the CUDA backend: applies pipeline stages to a payload and prints the
result (the module and the plans the stages attached), like the reference's optimizer CLI
(lighthouse/lh_opt.py) prints the transformed IR."""

from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    try:
        p = argparse.ArgumentParser(prog="lh-opt", description="Applies pipeline stages to an MLIR payload module and prints the result.")
        p.add_argument("payload_module", type=str)
        p.add_argument("--stage", action="append", required=True)
        p.add_argument("--print-mlir-after-all", action=argparse.BooleanOptionalAction)
        args = p.parse_args(argv)
        from .pipeline.driver import CompilerDriver

        driver = CompilerDriver(args.payload_module, stages=args.stage)
        module = driver.run(print_after_all=bool(args.print_mlir_after_all))
        print(module)
        for plan in module.plans.values():
            print(plan)
        return 0
    except KeyboardInterrupt:
        print("\nInterrupted", file=sys.stderr)
        return 130
    except (FileNotFoundError, OSError, ValueError) as exc:
        print(f"Error: {exc}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
