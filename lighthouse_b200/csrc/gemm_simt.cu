// Generic CUDA-core GEMM with the same fused epilogue as the tensor-core kernel.
//
// It is the kernel for everything the tensor-core path does not take: f32
// operands (linalg.matmul on f32 tensors, test/run/pipeline-check.mlir:8-12 of the
// reference, where products are accumulated in f32 with k ascending as
// convert-linalg-to-loops orders them), arbitrary element strides (transposed
// views), batched products (linalg.batch_matmul) and shapes whose rows are not
// 16-byte aligned. Classic shared-memory tiling: BMxBNx16 tiles, 256 threads, each
// thread a TMxTN register block, register-staged double buffering.
#include "common.cuh"
#include "epilogue.cuh"

namespace lh {

namespace {

constexpr int SBK = 16;

struct SimtParams {
  int M, N, K;
  const void* A; int a_dtype; int64_t sam, sak, sab;
  const void* B; int b_dtype; int64_t sbk, sbn, sbb;
  void* D; int d_dtype; int64_t sdm, sdn, sdb;
  const void* C; int c_dtype; int64_t scm, scn, scb;
  const void* bias; int bias_dtype;
  const void* R; int r_dtype; int64_t srm, srn, srb;
  int act;
};

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename TA, typename TB, int BM_, int BN_, int TM, int TN>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
  constexpr int THREADS = 256;
  static_assert((BM_ / TM) * (BN_ / TN) == THREADS, "thread tiling must cover the block tile");
  constexpr int A_PER_THREAD = BM_ * SBK / THREADS;
  constexpr int B_PER_THREAD = BN_ * SBK / THREADS;
  __shared__ float As[2][SBK][BM_ + 4];
  __shared__ float Bs[2][SBK][BN_ + 4];

  const int tid = threadIdx.x;
  const int batch = blockIdx.z;
  const int m0 = blockIdx.y * BM_;
  const int n0 = blockIdx.x * BN_;
  const TA* A = static_cast<const TA*>(p.A) + batch * p.sab;
  const TB* B = static_cast<const TB*>(p.B) + batch * p.sbb;
  const bool a_kfast = (p.sak == 1);  // consecutive threads walk k (row-major A) or m
  const bool b_nfast = (p.sbn == 1);

  float a_reg[A_PER_THREAD], b_reg[B_PER_THREAD];
  auto load_tiles = [&](int k0) {
#pragma unroll
    for (int i = 0; i < A_PER_THREAD; ++i) {
      const int e = tid + i * THREADS;
      const int kk = a_kfast ? (e % SBK) : (e / BM_);
      const int mm = a_kfast ? (e / SBK) : (e % BM_);
      const int m = m0 + mm, k = k0 + kk;
      a_reg[i] = (m < p.M && k < p.K) ? to_f32<TA>(A[m * p.sam + k * p.sak]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < B_PER_THREAD; ++i) {
      const int e = tid + i * THREADS;
      const int kk = b_nfast ? (e / BN_) : (e % SBK);
      const int nn = b_nfast ? (e % BN_) : (e / SBK);
      const int n = n0 + nn, k = k0 + kk;
      b_reg[i] = (n < p.N && k < p.K) ? to_f32<TB>(B[k * p.sbk + n * p.sbn]) : 0.f;
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int i = 0; i < A_PER_THREAD; ++i) {
      const int e = tid + i * THREADS;
      const int kk = a_kfast ? (e % SBK) : (e / BM_);
      const int mm = a_kfast ? (e / SBK) : (e % BM_);
      As[buf][kk][mm] = a_reg[i];
    }
#pragma unroll
    for (int i = 0; i < B_PER_THREAD; ++i) {
      const int e = tid + i * THREADS;
      const int kk = b_nfast ? (e / BN_) : (e % SBK);
      const int nn = b_nfast ? (e % BN_) : (e / SBK);
      Bs[buf][kk][nn] = b_reg[i];
    }
  };

  const int tx = tid % (BN_ / TN);
  const int ty = tid / (BN_ / TN);
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  const int num_k = (p.K + SBK - 1) / SBK;
  load_tiles(0);
  store_tiles(0);
  __syncthreads();
  for (int kb = 0; kb < num_k; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < num_k) load_tiles((kb + 1) * SBK);
#pragma unroll
    for (int kk = 0; kk < SBK; ++kk) {
      float av[TM], bv[TN];
#pragma unroll
      for (int i = 0; i < TM; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(&As[buf][kk][ty * TM + i]);
        av[i] = t.x; av[i + 1] = t.y; av[i + 2] = t.z; av[i + 3] = t.w;
      }
#pragma unroll
      for (int j = 0; j < TN; j += 4) {
        const float4 t = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * TN + j]);
        bv[j] = t.x; bv[j + 1] = t.y; bv[j + 2] = t.z; bv[j + 3] = t.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (kb + 1 < num_k) {
      store_tiles(buf ^ 1);
      __syncthreads();
    }
  }

  char* D = static_cast<char*>(p.D);
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= p.N) continue;
      float v = acc[i][j];
      if (p.C) v += load_as_f32(p.C, p.c_dtype, batch * p.scb + m * p.scm + n * p.scn);
      if (p.bias) v += load_as_f32(p.bias, p.bias_dtype, n);
      v = apply_act(v, p.act);
      if (p.R) v += load_as_f32(p.R, p.r_dtype, batch * p.srb + m * p.srm + n * p.srn);
      store_from_f32(D, p.d_dtype, batch * p.sdb + m * p.sdm + n * p.sdn, v);
    }
  }
}

template <typename TA, typename TB>
int launch_typed(lh_ctx* ctx, const SimtParams& sp, int batch) {
  const int64_t big_tiles = static_cast<int64_t>((sp.M + 127) / 128) * ((sp.N + 127) / 128) * batch;
  if (big_tiles >= ctx->sm_count) {
    dim3 grid((sp.N + 127) / 128, (sp.M + 127) / 128, batch);
    gemm_simt_kernel<TA, TB, 128, 128, 8, 8><<<grid, 256, 0, ctx->stream>>>(sp);
  } else {
    dim3 grid((sp.N + 63) / 64, (sp.M + 63) / 64, batch);
    gemm_simt_kernel<TA, TB, 64, 64, 4, 4><<<grid, 256, 0, ctx->stream>>>(sp);
  }
  LH_CHECK_LAUNCH(ctx, "gemm_simt_kernel");
  return LH_OK;
}

}  // namespace

int gemm_simt_launch(lh_ctx* ctx, const GemmProblem& g) {
  if (g.flags & LH_GEMM_SWIGLU)
    return set_error(ctx, LH_ERR_UNSUPPORTED, "the SwiGLU epilogue needs the tensor-core GEMM path");
  if (g.batch > 65535 || (g.M + 63) / 64 > 65535)
    return set_error(ctx, LH_ERR_UNSUPPORTED, "GEMM grid too large for the CUDA-core kernel");
  SimtParams sp;
  sp.M = g.M; sp.N = g.N; sp.K = g.K;
  sp.A = g.A; sp.a_dtype = g.a_dtype; sp.sam = g.sam; sp.sak = g.sak; sp.sab = g.sab;
  sp.B = g.B; sp.b_dtype = g.b_dtype; sp.sbk = g.sbk; sp.sbn = g.sbn; sp.sbb = g.sbb;
  sp.D = g.D; sp.d_dtype = g.d_dtype; sp.sdm = g.sdm; sp.sdn = g.sdn; sp.sdb = g.sdb;
  sp.C = g.C; sp.c_dtype = g.c_dtype; sp.scm = g.scm; sp.scn = g.scn; sp.scb = g.scb;
  sp.bias = g.bias; sp.bias_dtype = g.bias_dtype;
  sp.R = g.R; sp.r_dtype = g.r_dtype; sp.srm = g.srm; sp.srn = g.srn; sp.srb = g.srb;
  sp.act = g.act;
  if (g.a_dtype == LH_F32 && g.b_dtype == LH_F32) return launch_typed<float, float>(ctx, sp, g.batch);
  if (g.a_dtype == LH_BF16 && g.b_dtype == LH_BF16)
    return launch_typed<__nv_bfloat16, __nv_bfloat16>(ctx, sp, g.batch);
  if (g.a_dtype == LH_F16 && g.b_dtype == LH_F16) return launch_typed<__half, __half>(ctx, sp, g.batch);
  if (g.a_dtype == LH_BF16 && g.b_dtype == LH_F32) return launch_typed<__nv_bfloat16, float>(ctx, sp, g.batch);
  if (g.a_dtype == LH_F32 && g.b_dtype == LH_BF16) return launch_typed<float, __nv_bfloat16>(ctx, sp, g.batch);
  return set_error(ctx, LH_ERR_UNSUPPORTED, "GEMM operand dtypes %d x %d are not supported", g.a_dtype,
                   g.b_dtype);
}

}  // namespace lh
