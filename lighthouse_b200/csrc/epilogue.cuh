// Device-side epilogue arithmetic shared by the GEMM kernels and the
// elementwise kernels: typed loads/stores, activations.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/lh_b200.h"

namespace lh {

__device__ __forceinline__ float load_as_f32(const void* p, int dtype, int64_t idx) {
  switch (dtype) {
    case LH_F32: return static_cast<const float*>(p)[idx];
    case LH_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
    case LH_F16: return __half2float(static_cast<const __half*>(p)[idx]);
    case LH_F64: return static_cast<float>(static_cast<const double*>(p)[idx]);
    case LH_I32: return static_cast<float>(static_cast<const int32_t*>(p)[idx]);
    case LH_I64: return static_cast<float>(static_cast<const int64_t*>(p)[idx]);
  }
  return 0.f;
}

__device__ __forceinline__ void store_from_f32(void* p, int dtype, int64_t idx, float v) {
  switch (dtype) {
    case LH_F32: static_cast<float*>(p)[idx] = v; break;
    case LH_BF16: static_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v); break;
    case LH_F16: static_cast<__half*>(p)[idx] = __float2half_rn(v); break;
    case LH_F64: static_cast<double*>(p)[idx] = static_cast<double>(v); break;
    case LH_I32: static_cast<int32_t*>(p)[idx] = static_cast<int32_t>(v); break;
    case LH_I64: static_cast<int64_t*>(p)[idx] = static_cast<int64_t>(v); break;
  }
}

// erf by Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7, two special-function instructions and
// a short polynomial, no branches): an epilogue applies it to every element of a tile, where
// the library erff's length and divergent ranges cost more than the tile's main loop.
__device__ __forceinline__ float erf_as(float z) {
  const float a = fabsf(z);
  const float t = __fdividef(1.f, fmaf(0.3275911f, a, 1.f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float r = 1.f - poly * t * __expf(-a * a);
  return copysignf(r, z);
}

__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case LH_ACT_RELU: return fmaxf(x, 0.f);
    case LH_ACT_GELU_ERF: return 0.5f * x * (1.f + erf_as(x * 0.70710678118654752440f));
    case LH_ACT_GELU_TANH: {
      // 0.5 x (1 + tanh u) = x / (1 + exp(-2u))
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return __fdividef(x, 1.f + __expf(-2.f * u));
    }
    // (fast division: two special-function instructions and a multiply; the IEEE divide is a
    // dozen instructions with a slow path, which made an epilogue three times its main loop)
    case LH_ACT_SILU: return __fdividef(x, 1.f + __expf(-x));
    case LH_ACT_SIGMOID: return __fdividef(1.f, 1.f + __expf(-x));
    default: return x;
  }
}

// Loads 8 consecutive elements (16-byte aligned for 2-byte types, 32 for f32) as floats.
__device__ __forceinline__ void load8_as_f32(const void* p, int dtype, int64_t idx, float (&v)[8]) {
  if (dtype == LH_BF16) {
    const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p) + idx);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  } else if (dtype == LH_F32) {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = load_as_f32(p, dtype, idx + i);
  }
}

__device__ __forceinline__ void store8_from_f32(void* p, int dtype, int64_t idx, const float (&v)[8]) {
  if (dtype == LH_BF16) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p) + idx) = raw;
  } else if (dtype == LH_F32) {
    *reinterpret_cast<float4*>(static_cast<float*>(p) + idx) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(static_cast<float*>(p) + idx + 4) = make_float4(v[4], v[5], v[6], v[7]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) store_from_f32(p, dtype, idx + i, v[i]);
  }
}

}  // namespace lh
