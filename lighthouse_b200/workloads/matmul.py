"""Matmul workload: the parameter set, seeded inputs and flop/byte accounting of the
reference's ``XeGPUMatMul`` example (examples/xegpu/matmul.py:41-164), producing the same
payload through ``generate_gpu_matmul_payload``."""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..payload.generators import generate_gpu_matmul_payload
from ..utils.numpy import mlir_to_numpy_dtype


def matmul_complexity(M, N, K, bias, relu, accumulate_c, nbytes_ab, nbytes_c):
    """(flops, bytes read, bytes written): 2MNK (+MN for bias, +MN for ReLU); post-ops are
    assumed fused and add no traffic beyond the bias vector and an accumulated C."""
    flops = 2 * M * N * K
    reads = (M * K + K * N) * nbytes_ab
    writes = M * N * nbytes_c
    if bias:
        flops += M * N
        reads += N * nbytes_c
    if relu:
        flops += M * N
    if accumulate_c:
        reads += M * N * nbytes_c
    return flops, reads, writes


@dataclass
class CudaMatMul:
    M: int = 4096
    N: int = 4096
    K: int = 4096
    ab_type: str = "bf16"
    c_type: str = "f32"
    has_bias: bool = False
    has_relu: bool = False
    accumulate_c: bool = True
    truncate_c: bool = False
    transpose_a: bool = False
    transpose_b: bool = False
    payload_function_name: str = "payload"

    @property
    def result_type(self) -> str:
        return self.ab_type if self.truncate_c else self.c_type

    def payload_module(self):
        return generate_gpu_matmul_payload(
            self.payload_function_name, self.M, self.N, self.K, self.ab_type, self.c_type, self.transpose_a, self.transpose_b,
            self.has_bias, self.has_relu, self.accumulate_c, result_type=self.result_type,
        )

    def get_input_arrays(self, init_int: bool = False) -> list[np.ndarray]:
        """[C, A, B(, bias)] from ``np.random.seed(2)``: U(-0.5, 0.5), or integers in [-3, 3]
        for exact comparisons (the reference's generator, examples/xegpu/matmul.py:135-164)."""
        ab, ct = mlir_to_numpy_dtype(self.ab_type), mlir_to_numpy_dtype(self.result_type)

        def gen(shape, dtype):
            a = np.random.randint(-3, 4, shape) if init_int else np.random.rand(*shape) - 0.5
            return a.astype(dtype)

        np.random.seed(2)
        a_shape = (self.M, self.K) if not self.transpose_a else (self.K, self.M)
        b_shape = (self.K, self.N) if not self.transpose_b else (self.N, self.K)
        A, B, C = gen(a_shape, ab), gen(b_shape, ab), gen((self.M, self.N), ct)
        return [C, A, B] + ([gen((self.N,), ct)] if self.has_bias else [])

    def get_complexity(self):
        return matmul_complexity(self.M, self.N, self.K, self.has_bias, self.has_relu, self.accumulate_c,
                                 mlir_to_numpy_dtype(self.ab_type).itemsize, mlir_to_numpy_dtype(self.result_type).itemsize)
