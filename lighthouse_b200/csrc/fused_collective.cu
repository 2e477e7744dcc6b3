// Reduce-scatter + residual add + RMSNorm + all-gather as ONE kernel over NVSwitch multicast
// memory. Between two tensor-parallel projections every rank needs
//     h   += sum over ranks of the contraction's partial sums        (residual stream)
//     xn   = rmsnorm(h) * weight                                      (input of the next GEMM)
// for all tokens. Each rank owns 1/world of the rows: it reads the switch-reduced sum of its
// rows with multimem.ld_reduce (one load returns the sum over all GPUs' buffers), updates its
// rows of h in local memory, normalises them and writes the result into every GPU's xn buffer
// with multimem.st (one store, replicated by the switch). Per direction the links carry the
// bytes of one all-reduce's reduce-scatter half and one all-gather half, the activations never
// take an extra trip through HBM, and the row work is not replicated.
//
// Cross-rank ordering is by epoch-numbered flags in a symmetric flag pad: "my partial sums
// are complete" before anyone reduces, "my stores are issued and fenced" before anyone's
// kernel ends. Every wait is bounded (2 s on the device clock); on a timeout the kernel
// records DEV_TIMEOUT_PEER in the context's status word and returns.
//
// The reference's tensor-parallel example does this with a synchronous MPI all-reduce followed
// by separate kernels (examples/mpi/feed-forward-mpi.py:213-228).
#include "common.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"

namespace lh {
namespace {

constexpr int RNG_THREADS = 512;
constexpr int RNG_ROWS = 8;  // rows a block keeps in flight
// Dynamic shared memory the kernel asks for without using it: with it a block cannot share an SM
// with a GEMM block (which takes nearly all of the SM's shared memory), so the two kernels
// split the GPU cleanly by SMs instead of delaying some of each other's blocks.
constexpr int RNG_SMEM_FENCE = 40 * 1024;  // + the static arrays stays under the 48 KB a kernel gets without opting in

struct RngParams {
  const char* part;   // my rows of the partial sums: multicast address (MC) or local; null = no reduce
  int64_t part_ld;    // elements
  char* h;            // my rows of the residual stream (local)
  int64_t h_ld;
  char* xn;           // my rows of the destination: multicast address (MC) or local
  int64_t xn_ld;
  const void* weight; int weight_dtype;
  int rows, n;
  float eps;
  int rank, world;
  uint32_t epoch;
  uint32_t* pads[LH_MAX_RANKS];  // every rank's flag pad as mapped here; [rank] is local
  uint32_t* counter;             // local: blocks finished in this launch
  int* dev_status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Sum over all GPUs' copies of 8 bf16 values, accumulated in f32 inside the switch.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc)
               : "memory");
  return r;
}
// One 16-byte store replicated into every GPU's copy.
__device__ __forceinline__ void multimem_st_16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void unpack8(uint4 u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// Waits until flag `slot` of every rank in the local pad has reached `epoch`. Threads
// 0..world-1 poll one flag each. Returns false (for the whole block) after the time limit.
__device__ bool wait_all_ranks(const RngParams& p, int slot, int* s_abort) {
  if (threadIdx.x < p.world)
    flag_wait_limit(p.pads[p.rank] + slot * LH_MAX_RANKS + threadIdx.x, p.epoch, reinterpret_cast<volatile int*>(s_abort), p.dev_status,
                    DEV_TIMEOUT_PEER, LH_WAIT_TIMEOUT_NS);
  __syncthreads();
  return *reinterpret_cast<volatile int*>(s_abort) == 0;
}

template <bool MC>
__global__ void __launch_bounds__(RNG_THREADS, 1) reduce_norm_gather_kernel(const RngParams p) {
  __shared__ float red[2][RNG_ROWS][RNG_THREADS / 32];
  __shared__ int s_abort;
  __shared__ int s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) s_abort = 0;
  __syncthreads();
  bool ok = true;
  if (MC) {
    // phase 0: tell every rank that this rank's partial sums are complete (they are: this
    // kernel is ordered after the GEMM on its stream), then wait for everyone's.
    if (blockIdx.x == 0 && tid < p.world) {
      __threadfence_system();
      st_release_sys(p.pads[tid] + 0 * LH_MAX_RANKS + p.rank, p.epoch);
    }
    ok = wait_all_ranks(p, 0, &s_abort);
  }
  const int c = tid * 8;
  const bool active = c < p.n;
  float g[8];
  if (active) load8_as_f32(p.weight, p.weight_dtype, c, g);
  const float inv_n = 1.f / static_cast<float>(p.n);
  int phase = 0;
  for (int row0 = blockIdx.x * RNG_ROWS; ok && row0 < p.rows; row0 += gridDim.x * RNG_ROWS, phase ^= 1) {
    uint4 pr[RNG_ROWS], hr[RNG_ROWS];
#pragma unroll
    for (int u = 0; u < RNG_ROWS; ++u) {
      const int row = row0 + u;
      pr[u] = make_uint4(0, 0, 0, 0);
      if (active && row < p.rows && p.part) {
        const char* src = p.part + (static_cast<int64_t>(row) * p.part_ld + c) * 2;
        pr[u] = MC ? multimem_ld_reduce_bf16x8(src) : *reinterpret_cast<const uint4*>(src);
      }
    }
#pragma unroll
    for (int u = 0; u < RNG_ROWS; ++u) {
      const int row = row0 + u;
      hr[u] = make_uint4(0, 0, 0, 0);
      if (active && row < p.rows) hr[u] = *reinterpret_cast<const uint4*>(p.h + (static_cast<int64_t>(row) * p.h_ld + c) * 2);
    }
    // h <- bf16(h + sum): the residual stream keeps the activation type, and the norm sees the
    // rounded value exactly as a separate RMSNorm kernel reading h would. The rows stay packed
    // (4 registers each) across the block reduction.
    float sq[RNG_ROWS];
#pragma unroll
    for (int u = 0; u < RNG_ROWS; ++u) {
      const int row = row0 + u;
      float a[8];
      unpack8(hr[u], a);
      if (p.part) {
        float b[8];
        unpack8(pr[u], b);
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] += b[k];
        hr[u] = pack8(a);
        unpack8(hr[u], a);
        if (active && row < p.rows) *reinterpret_cast<uint4*>(p.h + (static_cast<int64_t>(row) * p.h_ld + c) * 2) = hr[u];
      }
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) s += a[k] * a[k];
      sq[u] = s;
    }
#pragma unroll
    for (int u = 0; u < RNG_ROWS; ++u) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sq[u] += __shfl_xor_sync(0xffffffffu, sq[u], o);
      if (lane == 0) red[phase][u][warp] = sq[u];
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < RNG_ROWS; ++u) {
      const int row = row0 + u;
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < RNG_THREADS / 32; ++w) tot += red[phase][u][w];
      const float rstd = rsqrtf(tot * inv_n + p.eps);
      if (active && row < p.rows) {
        float y[8];
        unpack8(hr[u], y);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // normalised value rounded to the activation type before the weight multiply
          // (examples/llama/ref_model.py:44-47 of the reference)
          y[k] = __bfloat162float(__float2bfloat16_rn(y[k] * rstd)) * g[k];
        }
        char* dst = p.xn + (static_cast<int64_t>(row) * p.xn_ld + c) * 2;
        if (MC) multimem_st_16(dst, pack8(y));
        else *reinterpret_cast<uint4*>(dst) = pack8(y);
      }
    }
  }
  if (!MC) return;
  // phase 1: when the last block of this rank has issued and fenced its stores, tell every
  // rank; that block then waits for everyone's, so the kernel ends only when every rank's
  // rows have arrived here.
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const uint32_t done = atomicAdd(p.counter, 1u) + 1u;
    s_last = (done == gridDim.x);
    if (s_last) *p.counter = 0;  // re-armed for the next launch (launches on one stream do not overlap)
  }
  __syncthreads();
  if (!s_last) return;
  if (*reinterpret_cast<volatile int*>(&s_abort) == 0 && tid < p.world) {
    __threadfence_system();
    st_release_sys(p.pads[tid] + 1 * LH_MAX_RANKS + p.rank, p.epoch);
  }
  wait_all_ranks(p, 1, &s_abort);
}

const SymmRegion* find_region(const lh_ctx* ctx, const void* ptr, size_t bytes) {
  const char* q = static_cast<const char*>(ptr);
  for (const SymmRegion& r : ctx->symm)
    if (q >= r.local && q + bytes <= r.local + r.bytes) return &r;
  return nullptr;
}

}  // namespace
}  // namespace lh

using namespace lh;

extern "C" int lh_b200_symm_register(lh_ctx_t* ctx, void* local, size_t bytes, void* multicast, void* const* peers, int world) {
  if (!ctx || !local || !bytes || world < 1 || world > LH_MAX_RANKS) return LH_ERR_INVALID;
  SymmRegion r{};
  r.local = static_cast<char*>(local);
  r.bytes = bytes;
  r.multicast = static_cast<char*>(multicast);
  for (int i = 0; i < world; ++i) r.peers[i] = peers ? static_cast<char*>(peers[i]) : nullptr;
  ctx->symm.push_back(r);
  return LH_OK;
}

extern "C" int lh_b200_symm_set_flags(lh_ctx_t* ctx, int rank, int world, void* const* pads) {
  if (!ctx || !pads || world < 1 || world > LH_MAX_RANKS || rank < 0 || rank >= world) return LH_ERR_INVALID;
  cudaSetDevice(ctx->device);
  for (int i = 0; i < LH_MAX_RANKS; ++i) ctx->symm_pads[i] = i < world ? static_cast<uint32_t*>(pads[i]) : nullptr;
  ctx->symm_rank = rank;
  ctx->symm_world = world;
  ctx->symm_epoch = 0;
  ctx->symm_broken = false;
  // The launch numbering restarts, so this rank's pad must read zero again. The caller runs a
  // barrier over all ranks after this call and before the first fused launch: no rank may
  // signal into a pad its owner has not cleared yet.
  LH_CUDA_CHECK(ctx, cudaMemset(pads[rank], 0, 2 * LH_MAX_RANKS * sizeof(uint32_t)));
  if (!ctx->symm_counter) {
    LH_CUDA_CHECK(ctx, cudaMalloc(&ctx->symm_counter, sizeof(uint32_t)));
    LH_CUDA_CHECK(ctx, cudaMemset(ctx->symm_counter, 0, sizeof(uint32_t)));
  }
  return LH_OK;
}

extern "C" int lh_b200_symm_clear(lh_ctx_t* ctx) {
  if (!ctx) return LH_ERR_INVALID;
  ctx->symm.clear();
  for (int i = 0; i < LH_MAX_RANKS; ++i) ctx->symm_pads[i] = nullptr;
  ctx->symm_world = 0;
  ctx->symm_rank = 0;
  return LH_OK;
}

extern "C" int lh_b200_reduce_norm_gather(lh_ctx_t* ctx, const lh_memref_t* xn, const lh_memref_t* part, const lh_memref_t* h,
                                          const lh_memref_t* weight, float eps) {
  if (!ctx || !xn || !h || !weight) return LH_ERR_INVALID;
  const int world = ctx->symm_world > 0 ? ctx->symm_world : 1;
  const int rank = ctx->symm_world > 0 ? ctx->symm_rank : 0;
  if (xn->rank != 2 || h->rank != 2 || (part && part->rank != 2) || weight->rank != 1)
    return set_error(ctx, LH_ERR_INVALID, "reduce_norm_gather: xn, part, h are matrices and weight a vector");
  const int64_t rows = h->shape[0], n = h->shape[1];
  if (xn->shape[0] != rows * world || xn->shape[1] != n || (part && (part->shape[0] != rows * world || part->shape[1] != n)) || weight->shape[0] != n)
    return set_error(ctx, LH_ERR_INVALID, "reduce_norm_gather: xn/part must be (%d * %lld, %lld)", world, (long long)rows, (long long)n);
  if (xn->dtype != LH_BF16 || h->dtype != LH_BF16 || (part && part->dtype != LH_BF16))
    return set_error(ctx, LH_ERR_UNSUPPORTED, "reduce_norm_gather: activations must be bf16");
  if (n % 8 || n > RNG_THREADS * 8) return set_error(ctx, LH_ERR_UNSUPPORTED, "reduce_norm_gather: row length %lld (multiple of 8, at most %d)", (long long)n, RNG_THREADS * 8);
  if (xn->strides[1] != 1 || h->strides[1] != 1 || (part && part->strides[1] != 1) || (weight->shape[0] > 1 && weight->strides[0] != 1))
    return set_error(ctx, LH_ERR_UNSUPPORTED, "reduce_norm_gather: unit inner strides required");
  if (xn->strides[0] % 8 || h->strides[0] % 8 || (part && part->strides[0] % 8) ||
      (reinterpret_cast<uintptr_t>(data_ptr(xn)) | reinterpret_cast<uintptr_t>(data_ptr(h)) | (part ? reinterpret_cast<uintptr_t>(data_ptr(part)) : 0)) % 16)
    return set_error(ctx, LH_ERR_UNSUPPORTED, "reduce_norm_gather: rows must be 16-byte aligned");
  if (rows == 0) return LH_OK;

  RngParams p{};
  p.rows = static_cast<int>(rows);
  p.n = static_cast<int>(n);
  p.eps = eps;
  p.rank = rank;
  p.world = world;
  p.h = data_ptr(h);
  p.h_ld = h->strides[0];
  p.weight = data_ptr(weight);
  p.weight_dtype = weight->dtype;
  p.part_ld = part ? part->strides[0] : 0;
  p.xn_ld = xn->strides[0];
  p.dev_status = ctx->dev_status;
  const int64_t my_row0 = static_cast<int64_t>(rank) * rows;
  char* xn_mine = data_ptr(xn) + my_row0 * xn->strides[0] * 2;
  const char* part_mine = part ? data_ptr(part) + my_row0 * part->strides[0] * 2 : nullptr;
  const unsigned want = static_cast<unsigned>((rows + RNG_ROWS - 1) / RNG_ROWS);
  if (world == 1) {
    p.xn = xn_mine;
    p.part = part_mine;
    const unsigned grid = want < 2u * ctx->sm_count ? want : 2u * ctx->sm_count;
    reduce_norm_gather_kernel<false><<<grid, RNG_THREADS, 0, ctx->stream>>>(p);
    LH_CHECK_LAUNCH(ctx, "reduce_norm_gather_kernel");
    return LH_OK;
  }
  // multi-rank: both buffers must lie in registered symmetric regions with a multicast mapping
  const size_t span = static_cast<size_t>((rows - 1) * xn->strides[0] + n) * 2;
  const SymmRegion* rx = find_region(ctx, xn_mine, span);
  if (!rx || !rx->multicast) return set_error(ctx, LH_ERR_INVALID, "reduce_norm_gather: xn is not in a registered multicast region");
  p.xn = rx->multicast + (xn_mine - rx->local);
  if (part) {
    const SymmRegion* rp = find_region(ctx, part_mine, static_cast<size_t>((rows - 1) * part->strides[0] + n) * 2);
    if (!rp || !rp->multicast) return set_error(ctx, LH_ERR_INVALID, "reduce_norm_gather: part is not in a registered multicast region");
    p.part = rp->multicast + (part_mine - rp->local);
  }
  for (int i = 0; i < world; ++i) {
    if (!ctx->symm_pads[i]) return set_error(ctx, LH_ERR_INVALID, "reduce_norm_gather: flag pads not set");
    p.pads[i] = ctx->symm_pads[i];
  }
  if (ctx->symm_broken)
    return set_error(ctx, LH_ERR_DEVICE, "reduce_norm_gather: a launch on this context failed, so the ranks' launch numbers may have parted; set the flags up again (lh_b200_symm_set_flags on every rank)");
  p.counter = ctx->symm_counter;
  p.epoch = ctx->symm_epoch + 1;  // counted only once the launch is known to have gone out
  // The kernel shares the GPU with a persistent GEMM on the main stream: stay within the
  // SMs that GEMM leaves free, so that no block waits for an SM behind it.
  // (one block per SM; alone on the GPU the kernel takes all of it).
  const unsigned cap = static_cast<unsigned>(ctx->reserved_sms > 0 ? ctx->reserved_sms : ctx->sm_count);
  const unsigned grid = want < cap ? want : cap;
  reduce_norm_gather_kernel<true><<<grid, RNG_THREADS, RNG_SMEM_FENCE, ctx->stream>>>(p);
  {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      ctx->symm_broken = true;  // the other ranks launched and this one did not
      return set_error(ctx, LH_ERR_CUDA, "launch of reduce_norm_gather_kernel failed: %s", cudaGetErrorString(e));
    }
  }
  ctx->launches++;
  ctx->symm_epoch++;
  return LH_OK;
}
