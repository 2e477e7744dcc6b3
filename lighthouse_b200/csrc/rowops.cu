// HBM-bound row and elementwise kernels: LayerNorm, RMSNorm, row softmax, rotary
// embedding, the elementwise family and the embedding gather.
//
// Row reductions keep a row in the registers of one warp (or of 4 / 8 warps for long rows):
// 16-byte vector loads, warp shuffles for the reductions, a few words of shared memory
// only to combine warps; rows longer than 8192 elements or not vectorisable fall back to
// a block-per-row kernel that re-reads the row from L2.
#include "common.cuh"
#include "ptx.cuh"
#include "epilogue.cuh"

namespace lh {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float round_through(float v, int dtype) {
  if (dtype == LH_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (dtype == LH_F16) return __half2float(__float2half_rn(v));
  return v;
}

struct RowParams {
  const void* x; int x_dtype; int64_t x_row_stride;
  void* out; int out_dtype; int64_t out_row_stride;
  const void* gamma; int gamma_dtype;
  const void* beta; int beta_dtype;
  int64_t rows;
  int n;
  float eps;
  int mode;  // 0 layernorm, 1 rmsnorm, 2 softmax
};

// A group of TPR threads per row (one warp, or 4 / 8 warps of a 256-thread block); thread t
// of the group owns VPL vectors of 8 consecutive elements, vector i covering columns
// [(i*TPR + t)*8, +8), so a row of up to TPR*VPL*8 elements lives in registers once.
// SD fixes the element types at compile time (0: read from the parameters; 1: bf16 rows in
// and out with bf16 scale / shift, the Llama RMSNorm; 2: f32 rows in, bf16 out, f32 scale /
// shift, the nanoGPT LayerNorm). With run-time types every load, store and rounding carries
// its type switch, and the kernel is bound by instruction issue and fetch instead of HBM.
template <int VPL, int TPR, int SD = 0>
__global__ void __launch_bounds__(256, 4) row_group_kernel(const RowParams p) {
  // a kernel launched as a programmatic dependent may set its CTAs up under this kernel's last
  // wave of blocks (it still waits for this kernel's completion before it reads anything)
  grid_dependency_trigger();
  const int x_dtype = SD == 1 ? LH_BF16 : SD == 2 ? LH_F32 : p.x_dtype;
  const int out_dtype = SD != 0 ? LH_BF16 : p.out_dtype;
  const int gamma_dtype = SD == 1 ? LH_BF16 : SD == 2 ? LH_F32 : p.gamma_dtype;
  const int beta_dtype = SD == 1 ? LH_BF16 : SD == 2 ? LH_F32 : p.beta_dtype;
  constexpr int GROUPS = 256 / TPR;
  constexpr int WARPS_PER_GROUP = TPR / 32;
  __shared__ float red[2][8];
  const int t = threadIdx.x % TPR;
  const int group = threadIdx.x / TPR;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int64_t row = static_cast<int64_t>(blockIdx.x) * GROUPS + group;
  const bool valid = row < p.rows;
  if (!valid) row = p.rows - 1;  // keep every thread in the block-wide barriers
  int phase = 0;
  auto group_reduce = [&](float val, bool is_max) -> float {
    val = is_max ? warp_max(val) : warp_sum(val);
    if (WARPS_PER_GROUP == 1) return val;
    if (lane == 0) red[phase][warp] = val;
    __syncthreads();
    float r = is_max ? -INFINITY : 0.f;
#pragma unroll
    for (int w = 0; w < WARPS_PER_GROUP; ++w) {
      const float o = red[phase][group * WARPS_PER_GROUP + w];
      r = is_max ? fmaxf(r, o) : r + o;
    }
    phase ^= 1;
    return r;
  };
  float v[VPL][8];
  const int64_t xoff = row * p.x_row_stride;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * TPR + t) * 8;
    if (c < p.n) {
      load8_as_f32(p.x, x_dtype, xoff + c, v[i]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[i][k] = (p.mode == 2) ? -INFINITY : 0.f;
    }
  }
  const float inv_n = 1.f / static_cast<float>(p.n);
  if (p.mode == 2) {
    // softmax: max, exp, sum, divide (gpu_softmax_payload.py:11-65 of the reference)
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
#pragma unroll
      for (int k = 0; k < 8; ++k) mx = fmaxf(mx, v[i][k]);
    mx = group_reduce(mx, true);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[i][k] = __expf(v[i][k] - mx);
        sum += v[i][k];
      }
    sum = group_reduce(sum, false);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
#pragma unroll
      for (int k = 0; k < 8; ++k) v[i][k] *= inv;
  } else {
    float mean = 0.f;
    if (p.mode == 0) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) s += v[i][k];
      mean = group_reduce(s, false) * inv_n;
    }
    // second pass over registers: sum of squared deviations (biased variance)
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = (i * TPR + t) * 8;
      if (c < p.n) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float d = v[i][k] - mean;
          sq += d * d;
        }
      }
    }
    const float rstd = rsqrtf(group_reduce(sq, false) * inv_n + p.eps);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = (i * TPR + t) * 8;
      if (c < p.n) {
        float g[8], bt[8];
        if (p.gamma) load8_as_f32(p.gamma, gamma_dtype, c, g);
        if (p.beta) load8_as_f32(p.beta, beta_dtype, c, bt);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float y = (v[i][k] - mean) * rstd;
          // RMSNorm casts the normalised value to the activation type before the weight
          // multiply (examples/llama/ref_model.py:44-47 of the reference)
          if (p.mode == 1 && p.gamma) y = round_through(y, out_dtype);
          if (p.gamma) y *= g[k];
          if (p.beta) y += bt[k];
          v[i][k] = y;
        }
      }
    }
  }
  if (!valid) return;
  const int64_t ooff = row * p.out_row_stride;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = (i * TPR + t) * 8;
    if (c < p.n) store8_from_f32(p.out, out_dtype, ooff + c, v[i]);
  }
}

template <int TPR, int SD>
void launch_row_group_sd(const RowParams& p, cudaStream_t stream) {
  const int vpl = (p.n / 8 + TPR - 1) / TPR;
  const unsigned blocks = static_cast<unsigned>((p.rows + (256 / TPR) - 1) / (256 / TPR));
  if (vpl <= 1) row_group_kernel<1, TPR, SD><<<blocks, 256, 0, stream>>>(p);
  else if (vpl <= 2) row_group_kernel<2, TPR, SD><<<blocks, 256, 0, stream>>>(p);
  else if (vpl <= 3) row_group_kernel<3, TPR, SD><<<blocks, 256, 0, stream>>>(p);
  else row_group_kernel<4, TPR, SD><<<blocks, 256, 0, stream>>>(p);
}

template <int TPR>
void launch_row_group(const RowParams& p, cudaStream_t stream) {
  // the two type combinations of the decoder workloads get kernels with the types compiled in
  const bool gb_bf16 = (!p.gamma || p.gamma_dtype == LH_BF16) && (!p.beta || p.beta_dtype == LH_BF16);
  const bool gb_f32 = (!p.gamma || p.gamma_dtype == LH_F32) && (!p.beta || p.beta_dtype == LH_F32);
  if (p.mode != 2 && p.x_dtype == LH_BF16 && p.out_dtype == LH_BF16 && gb_bf16) launch_row_group_sd<TPR, 1>(p, stream);
  else if (p.mode != 2 && p.x_dtype == LH_F32 && p.out_dtype == LH_BF16 && gb_f32) launch_row_group_sd<TPR, 2>(p, stream);
  else launch_row_group_sd<TPR, 0>(p, stream);
}

// Block per row, any length / alignment; three passes over the row.
__global__ void __launch_bounds__(256) row_block_kernel(const RowParams p) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int64_t xoff = row * p.x_row_stride;
  const int64_t ooff = row * p.out_row_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  auto block_reduce = [&](float val, bool is_max) -> float {
    val = is_max ? warp_max(val) : warp_sum(val);
    __syncthreads();
    if (lane == 0) red[warp] = val;
    __syncthreads();
    float r = (lane < nwarps) ? red[lane] : (is_max ? -INFINITY : 0.f);
    r = is_max ? warp_max(r) : warp_sum(r);
    return r;
  };
  const float inv_n = 1.f / static_cast<float>(p.n);
  if (p.mode == 2) {
    float mx = -INFINITY;
    for (int c = tid; c < p.n; c += blockDim.x) mx = fmaxf(mx, load_as_f32(p.x, p.x_dtype, xoff + c));
    mx = block_reduce(mx, true);
    float s = 0.f;
    for (int c = tid; c < p.n; c += blockDim.x) s += __expf(load_as_f32(p.x, p.x_dtype, xoff + c) - mx);
    s = block_reduce(s, false);
    const float inv = 1.f / s;
    for (int c = tid; c < p.n; c += blockDim.x)
      store_from_f32(p.out, p.out_dtype, ooff + c, __expf(load_as_f32(p.x, p.x_dtype, xoff + c) - mx) * inv);
    return;
  }
  float mean = 0.f;
  if (p.mode == 0) {
    float s = 0.f;
    for (int c = tid; c < p.n; c += blockDim.x) s += load_as_f32(p.x, p.x_dtype, xoff + c);
    mean = block_reduce(s, false) * inv_n;
  }
  float sq = 0.f;
  for (int c = tid; c < p.n; c += blockDim.x) {
    const float d = load_as_f32(p.x, p.x_dtype, xoff + c) - mean;
    sq += d * d;
  }
  const float rstd = rsqrtf(block_reduce(sq, false) * inv_n + p.eps);
  for (int c = tid; c < p.n; c += blockDim.x) {
    float y = (load_as_f32(p.x, p.x_dtype, xoff + c) - mean) * rstd;
    if (p.mode == 1 && p.gamma) y = round_through(y, p.out_dtype);
    if (p.gamma) y *= load_as_f32(p.gamma, p.gamma_dtype, c);
    if (p.beta) y += load_as_f32(p.beta, p.beta_dtype, c);
    store_from_f32(p.out, p.out_dtype, ooff + c, y);
  }
}

// Collapses a view with unit stride in its last dim into (rows, n, row_stride).
bool collapse_rows(const lh_memref_t* m, int64_t* rows, int* n, int64_t* row_stride) {
  if (m->rank < 1) return false;
  const int r = m->rank;
  if (m->shape[r - 1] != 1 && m->strides[r - 1] != 1) return false;
  *n = static_cast<int>(m->shape[r - 1]);
  int64_t nrows = 1;
  for (int i = 0; i < r - 1; ++i) nrows *= m->shape[i];
  *rows = nrows;
  if (r == 1) {
    *row_stride = *n;
    return true;
  }
  // leading dims must nest: stride[i] == stride[i+1] * shape[i+1]
  int64_t stride = m->strides[r - 2];
  for (int i = r - 3; i >= 0; --i) {
    if (m->shape[i] == 1) continue;
    if (m->strides[i] != m->strides[i + 1] * m->shape[i + 1]) return false;
  }
  *row_stride = stride;
  return true;
}

bool vec_ok(const void* ptr, int dtype, int64_t row_stride) {
  if (dtype != LH_F32 && dtype != LH_BF16 && dtype != LH_F16) return false;
  const uintptr_t a = reinterpret_cast<uintptr_t>(ptr);
  const size_t bytes = dtype_size(dtype) * 8;  // one 8-element vector (two 16-byte halves for f32)
  return (a % 16) == 0 && ((row_stride * (int64_t)dtype_size(dtype)) % 16) == 0 && bytes >= 16;
}

int row_launch(lh_ctx* ctx, const lh_memref_t* out, const lh_memref_t* x, const lh_memref_t* gamma,
               const lh_memref_t* beta, float eps, int mode, const char* what) {
  if (!out || !x) return set_error(ctx, LH_ERR_INVALID, "%s: null operand", what);
  RowParams p;
  int n2 = 0;
  int64_t rows2 = 0;
  if (!collapse_rows(x, &p.rows, &p.n, &p.x_row_stride) || !collapse_rows(out, &rows2, &n2, &p.out_row_stride))
    return set_error(ctx, LH_ERR_UNSUPPORTED, "%s: operands must have unit stride in the last dim and nested leading dims", what);
  if (rows2 != p.rows || n2 != p.n) return set_error(ctx, LH_ERR_INVALID, "%s: shape mismatch", what);
  if (p.rows == 0 || p.n == 0) return LH_OK;
  p.x = data_ptr(x); p.x_dtype = x->dtype;
  p.out = data_ptr(out); p.out_dtype = out->dtype;
  p.gamma = gamma ? data_ptr(gamma) : nullptr; p.gamma_dtype = gamma ? gamma->dtype : 0;
  p.beta = beta ? data_ptr(beta) : nullptr; p.beta_dtype = beta ? beta->dtype : 0;
  p.eps = eps;
  p.mode = mode;
  if (gamma && numel(gamma) != p.n) return set_error(ctx, LH_ERR_INVALID, "%s: scale length mismatch", what);
  if (beta && numel(beta) != p.n) return set_error(ctx, LH_ERR_INVALID, "%s: shift length mismatch", what);
  bool vec = (p.n % 8) == 0 && p.n <= 256 * 8 * 4 && vec_ok(p.x, p.x_dtype, p.x_row_stride) &&
             vec_ok(p.out, p.out_dtype, p.out_row_stride);
  if (gamma) vec = vec && vec_ok(p.gamma, p.gamma_dtype, 8) && is_contiguous(gamma);
  if (beta) vec = vec && vec_ok(p.beta, p.beta_dtype, 8) && is_contiguous(beta);
  if (vec) {
    const int nvec = p.n / 8;
    if (nvec <= 32 * 4) launch_row_group<32>(p, ctx->stream);
    else if (nvec <= 128 * 4) launch_row_group<128>(p, ctx->stream);
    else launch_row_group<256>(p, ctx->stream);
    LH_CHECK_LAUNCH(ctx, "row_group_kernel");
  } else {
    if (p.rows > 0x7fffffffLL) return set_error(ctx, LH_ERR_UNSUPPORTED, "%s: too many rows", what);
    row_block_kernel<<<static_cast<unsigned>(p.rows), 256, 0, ctx->stream>>>(p);
    LH_CHECK_LAUNCH(ctx, "row_block_kernel");
  }
  return LH_OK;
}

// ------------------------------------------------------------------- rotary
struct RopeParams {
  void* x; int dtype;
  int64_t sb, ss, sh;
  int B, S, H, D;
  float theta;
  int pos0;
};
__global__ void __launch_bounds__(256) rope_kernel(const RopeParams p) {
  // One thread per (position, pair): the angle and its sine / cosine are computed once and
  // reused for every batch entry and head.
  const int half = p.D / 2;
  const int64_t total = static_cast<int64_t>(p.S) * half;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx % half);
    const int s = static_cast<int>(idx / half);
    // freqs = 1 / theta^(2i/D); angle = position * freq, all in f32 as torch computes it
    const float freq = 1.0f / powf(p.theta, static_cast<float>(2 * i) / static_cast<float>(p.D));
    const float ang = static_cast<float>(p.pos0 + s) * freq;
    float sn, cs;
    sincosf(ang, &sn, &cs);
    for (int b = 0; b < p.B; ++b) {
      for (int h = 0; h < p.H; ++h) {
        const int64_t off = b * p.sb + s * p.ss + h * p.sh + 2 * i;
        if (p.dtype == LH_BF16) {
          __nv_bfloat162* ptr = reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(p.x) + off);
          const float2 x = __bfloat1622float2(*ptr);
          *ptr = __floats2bfloat162_rn(x.x * cs - x.y * sn, x.x * sn + x.y * cs);
        } else if (p.dtype == LH_F32) {
          float2* ptr = reinterpret_cast<float2*>(static_cast<float*>(p.x) + off);
          const float2 x = *ptr;
          *ptr = make_float2(x.x * cs - x.y * sn, x.x * sn + x.y * cs);
        } else {
          const float x0 = load_as_f32(p.x, p.dtype, off);
          const float x1 = load_as_f32(p.x, p.dtype, off + 1);
          store_from_f32(p.x, p.dtype, off, x0 * cs - x1 * sn);
          store_from_f32(p.x, p.dtype, off + 1, x0 * sn + x1 * cs);
        }
      }
    }
  }
}

// Table of (cos, sin) per (position, pair), with exactly rope_kernel's arithmetic, for the
// GEMM epilogue that rotates q and k columns on their way out.
__global__ void __launch_bounds__(256) rope_table_kernel(float2* table, int seq, int dim, float theta, int pos0) {
  const int half = dim / 2;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= seq * half) return;
  const int i = idx % half, s = idx / half;
  const float freq = 1.0f / powf(theta, static_cast<float>(2 * i) / static_cast<float>(dim));
  const float ang = static_cast<float>(pos0 + s) * freq;
  float sn, cs;
  sincosf(ang, &sn, &cs);
  table[idx] = make_float2(cs, sn);
}

// -------------------------------------------------------------- elementwise
struct EwParams {
  int kind, act;
  float scalar;
  void* out; int out_dtype;
  const void* a; int a_dtype;
  const void* b; int b_dtype;
  int rank;
  int64_t shape[LH_MAX_RANK];
  int64_t so[LH_MAX_RANK], sa[LH_MAX_RANK], sbb[LH_MAX_RANK];
  int64_t total;
  int n_inner;  // fast path: b indexed by (i % n_inner) when b_row_vector
  int b_row_vector;
};

__device__ __forceinline__ float ew_apply(int kind, int act, float scalar, float a, float b) {
  switch (kind) {
    case LH_EW_COPY: return a;
    case LH_EW_ADD: return a + b;
    case LH_EW_MUL: return a * b;
    case LH_EW_ACT: return apply_act(a, act);
    case LH_EW_ADD_ACT: return apply_act(a + b, act);
    case LH_EW_SILU_MUL: return apply_act(a, LH_ACT_SILU) * b;
    case LH_EW_SCALE: return a * scalar;
    case LH_EW_FILL: return scalar;
    case LH_EW_SUB: return a - b;
    case LH_EW_MAX: return fmaxf(a, b);
  }
  return a;
}

// All operands contiguous (b optionally a last-dim vector): 8 elements per thread.
__global__ void __launch_bounds__(256) ew_vec_kernel(const EwParams p) {
  // a kernel launched as a programmatic dependent may set its CTAs up under this kernel's last
  // wave of blocks (it still waits for this kernel's completion before it reads anything)
  grid_dependency_trigger();
  const int64_t nvec = p.total / 8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = i * 8;
    float a[8], b[8], o[8];
    if (p.a) load8_as_f32(p.a, p.a_dtype, e, a);
    if (p.b) load8_as_f32(p.b, p.b_dtype, p.b_row_vector ? (e % p.n_inner) : e, b);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = ew_apply(p.kind, p.act, p.scalar, p.a ? a[k] : 0.f, p.b ? b[k] : 0.f);
    store8_from_f32(p.out, p.out_dtype, e, o);
  }
}

// Arbitrary strides / broadcasting.
__global__ void __launch_bounds__(256) ew_generic_kernel(const EwParams p) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < p.total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t rem = i, oo = 0, oa = 0, ob = 0;
#pragma unroll
    for (int d = LH_MAX_RANK - 1; d >= 0; --d) {
      if (d < p.rank) {
        const int64_t c = rem % p.shape[d];
        rem /= p.shape[d];
        oo += c * p.so[d];
        oa += c * p.sa[d];
        ob += c * p.sbb[d];
      }
    }
    const float a = p.a ? load_as_f32(p.a, p.a_dtype, oa) : 0.f;
    const float b = p.b ? load_as_f32(p.b, p.b_dtype, ob) : 0.f;
    store_from_f32(p.out, p.out_dtype, oo, ew_apply(p.kind, p.act, p.scalar, a, b));
  }
}

// ---------------------------------------------------------------- embedding
struct EmbParams {
  void* out; int out_dtype; int64_t out_stride;
  const void* ids; int ids_dtype;
  const void* wte; int wte_dtype; int64_t wte_stride;
  const void* wpe; int wpe_dtype; int64_t wpe_stride;
  int64_t tokens;
  int dim, period;
  int64_t vocab;
};
__global__ void __launch_bounds__(128) embedding_kernel(const EmbParams p) {
  const int64_t t = blockIdx.x;
  int64_t id = (p.ids_dtype == LH_I64) ? static_cast<const int64_t*>(p.ids)[t]
                                        : static_cast<int64_t>(static_cast<const int32_t*>(p.ids)[t]);
  if (id < 0) id = 0;
  if (id >= p.vocab) id = p.vocab - 1;
  const int64_t pos = p.period > 0 ? (t % p.period) : 0;
  for (int c = threadIdx.x; c < p.dim; c += blockDim.x) {
    float v = load_as_f32(p.wte, p.wte_dtype, id * p.wte_stride + c);
    if (p.wpe) v += load_as_f32(p.wpe, p.wpe_dtype, pos * p.wpe_stride + c);
    store_from_f32(p.out, p.out_dtype, t * p.out_stride + c, v);
  }
}

unsigned grid_for(const lh_ctx* ctx, int64_t work_items, int threads) {
  int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = static_cast<int64_t>(ctx->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<unsigned>(blocks);
}

}  // namespace

int layernorm_launch(lh_ctx* ctx, const lh_memref_t* out, const lh_memref_t* x, const lh_memref_t* gamma,
                     const lh_memref_t* beta, float eps, int rms) {
  return row_launch(ctx, out, x, gamma, beta, eps, rms ? 1 : 0, rms ? "rmsnorm" : "layernorm");
}

int softmax_launch(lh_ctx* ctx, const lh_memref_t* out, const lh_memref_t* x) {
  return row_launch(ctx, out, x, nullptr, nullptr, 0.f, 2, "softmax");
}

int rope_launch(lh_ctx* ctx, const lh_memref_t* x, float theta, int pos0) {
  if (!x || x->rank != 4) return set_error(ctx, LH_ERR_INVALID, "rope: x must be a rank-4 (B,S,H,D) view");
  if (x->strides[3] != 1 || (x->shape[3] % 2) != 0)
    return set_error(ctx, LH_ERR_UNSUPPORTED, "rope: last dim must be even with unit stride");
  RopeParams p;
  p.x = data_ptr(x); p.dtype = x->dtype;
  p.B = (int)x->shape[0]; p.S = (int)x->shape[1]; p.H = (int)x->shape[2]; p.D = (int)x->shape[3];
  p.sb = x->strides[0]; p.ss = x->strides[1]; p.sh = x->strides[2];
  p.theta = theta; p.pos0 = pos0;
  if (numel(x) == 0) return LH_OK;
  if ((p.sb | p.ss | p.sh) & 1 || (reinterpret_cast<uintptr_t>(p.x) & 7))
    return set_error(ctx, LH_ERR_UNSUPPORTED, "rope: strides must be even and the base 8-byte aligned");
  const int64_t total = static_cast<int64_t>(p.S) * (p.D / 2);
  rope_kernel<<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>(p);
  LH_CHECK_LAUNCH(ctx, "rope_kernel");
  return LH_OK;
}

// One table per (theta, head size), covering positions [0, positions): a call for positions
// [pos0, pos0 + seq) indexes into it, so a decode loop with a moving pos0 neither allocates nor
// rebuilds. A table that is too short is replaced by one at least twice as long; the old one
// is retired with the outgrown scratch buffers (freed at the next lh_b200_sync, and captured
// graphs see the generation change). The build is ordered before later work of BOTH streams.
int rope_table_for(lh_ctx* ctx, float theta, int pos0, int seq, int dim, const float** table) {
  if (seq < 1 || dim < 2 || dim % 2 || pos0 < 0) return set_error(ctx, LH_ERR_INVALID, "rope table: positions %d + %d, head size %d", pos0, seq, dim);
  const int need = pos0 + seq;
  lh_ctx::RopeTable* slot = nullptr;
  for (auto& t : ctx->rope_tables)
    if (t.theta == theta && t.dim == dim) slot = &t;
  if (slot && slot->positions >= need) {
    *table = slot->data + static_cast<size_t>(pos0) * dim;  // (cos, sin) pairs: dim floats per position
    return LH_OK;
  }
  int positions = 256;
  while (positions < need) positions *= 2;
  if (slot && positions < 2 * slot->positions) positions = 2 * slot->positions;
  void* mem = nullptr;
  const int64_t n = static_cast<int64_t>(positions) * (dim / 2);
  int rc = lh_b200_malloc(ctx, static_cast<size_t>(n) * sizeof(float2), &mem);
  if (rc) return rc;
  rope_table_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, ctx->stream>>>(static_cast<float2*>(mem), positions, dim, theta, 0);
  LH_CHECK_LAUNCH(ctx, "rope_table_kernel");
  cudaStream_t other = ctx->side_selected ? ctx->main_saved : ctx->side_stream;
  if (other) {
    if (!ctx->rope_built) LH_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&ctx->rope_built, cudaEventDisableTiming));
    LH_CUDA_CHECK(ctx, cudaEventRecord(ctx->rope_built, ctx->stream));
    LH_CUDA_CHECK(ctx, cudaStreamWaitEvent(other, ctx->rope_built, 0));
  }
  if (slot) {
    ctx->retired_scratch.push_back(slot->data);
    ctx->scratch_generation++;
    slot->data = static_cast<float*>(mem);
    slot->positions = positions;
  } else {
    ctx->rope_tables.push_back({theta, dim, positions, static_cast<float*>(mem)});
  }
  *table = static_cast<float*>(mem) + static_cast<size_t>(pos0) * dim;
  return LH_OK;
}

int elementwise_launch(lh_ctx* ctx, int kind, const lh_memref_t* out, const lh_memref_t* a,
                       const lh_memref_t* b, int act, float scalar) {
  if (!out) return set_error(ctx, LH_ERR_INVALID, "elementwise: null output");
  if (kind < LH_EW_COPY || kind > LH_EW_MAX) return set_error(ctx, LH_ERR_INVALID, "elementwise: bad kind %d", kind);
  const bool needs_a = kind != LH_EW_FILL;
  const bool needs_b = kind == LH_EW_ADD || kind == LH_EW_MUL || kind == LH_EW_ADD_ACT ||
                       kind == LH_EW_SILU_MUL || kind == LH_EW_SUB || kind == LH_EW_MAX;
  if (needs_a && !a) return set_error(ctx, LH_ERR_INVALID, "elementwise: operand a missing");
  if (needs_b && !b) return set_error(ctx, LH_ERR_INVALID, "elementwise: operand b missing");
  if (!needs_a) a = nullptr;
  if (!needs_b) b = nullptr;
  EwParams p;
  memset(&p, 0, sizeof(p));
  p.kind = kind; p.act = act; p.scalar = scalar;
  p.out = data_ptr(out); p.out_dtype = out->dtype;
  p.a = a ? data_ptr(a) : nullptr; p.a_dtype = a ? a->dtype : 0;
  p.b = b ? data_ptr(b) : nullptr; p.b_dtype = b ? b->dtype : 0;
  p.rank = out->rank;
  p.total = numel(out);
  if (p.total == 0) return LH_OK;
  if (out->rank > LH_MAX_RANK) return set_error(ctx, LH_ERR_UNSUPPORTED, "elementwise: rank > %d", LH_MAX_RANK);
  // Right-align lower-rank operands (numpy broadcasting); size-1 dims broadcast.
  auto fill_strides = [&](const lh_memref_t* m, int64_t* dst) -> bool {
    for (int d = 0; d < LH_MAX_RANK; ++d) dst[d] = 0;
    if (!m) return true;
    if (m->rank > out->rank) return false;
    const int shift = out->rank - m->rank;
    for (int d = 0; d < m->rank; ++d) {
      if (m->shape[d] == out->shape[d + shift]) dst[d + shift] = m->strides[d];
      else if (m->shape[d] == 1) dst[d + shift] = 0;
      else return false;
    }
    return true;
  };
  for (int d = 0; d < out->rank; ++d) {
    p.shape[d] = out->shape[d];
    p.so[d] = out->strides[d];
  }
  if (!fill_strides(a, p.sa) || !fill_strides(b, p.sbb))
    return set_error(ctx, LH_ERR_INVALID, "elementwise: operand shapes do not broadcast to the output");
  // Fast path test.
  auto same_shape = [&](const lh_memref_t* m) {
    if (m->rank != out->rank) return false;
    for (int d = 0; d < out->rank; ++d)
      if (m->shape[d] != out->shape[d]) return false;
    return true;
  };
  auto vec_ptr = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) % 16) == 0; };
  auto vec_dtype = [](int dt) { return dt == LH_F32 || dt == LH_BF16 || dt == LH_F16; };
  const int n_inner = static_cast<int>(out->shape[out->rank > 0 ? out->rank - 1 : 0]);
  bool fast = out->rank >= 1 && is_contiguous(out) && vec_ptr(p.out) && vec_dtype(out->dtype) && (p.total % 8) == 0;
  if (a) fast = fast && same_shape(a) && is_contiguous(a) && vec_ptr(p.a) && vec_dtype(a->dtype);
  if (b) {
    const bool b_full = same_shape(b) && is_contiguous(b);
    const bool b_vec = (numel(b) == n_inner) && is_contiguous(b) && b->shape[b->rank - 1] == n_inner && (n_inner % 8) == 0;
    fast = fast && (b_full || b_vec) && vec_ptr(p.b) && vec_dtype(b->dtype);
    p.b_row_vector = (!b_full && b_vec) ? 1 : 0;
    p.n_inner = n_inner;
  }
  if (fast) {
    ew_vec_kernel<<<grid_for(ctx, p.total / 8, 256), 256, 0, ctx->stream>>>(p);
    LH_CHECK_LAUNCH(ctx, "ew_vec_kernel");
  } else {
    ew_generic_kernel<<<grid_for(ctx, p.total, 256), 256, 0, ctx->stream>>>(p);
    LH_CHECK_LAUNCH(ctx, "ew_generic_kernel");
  }
  return LH_OK;
}

int embedding_launch(lh_ctx* ctx, const lh_memref_t* out, const lh_memref_t* ids, const lh_memref_t* wte,
                     const lh_memref_t* wpe, int period) {
  if (!out || !ids || !wte) return set_error(ctx, LH_ERR_INVALID, "embedding: null operand");
  if (wte->rank != 2 || wte->strides[1] != 1) return set_error(ctx, LH_ERR_UNSUPPORTED, "embedding: table must be (vocab, dim) with unit inner stride");
  if (ids->dtype != LH_I32 && ids->dtype != LH_I64) return set_error(ctx, LH_ERR_INVALID, "embedding: ids must be i32 or i64");
  if (!is_contiguous(ids)) return set_error(ctx, LH_ERR_UNSUPPORTED, "embedding: ids must be contiguous");
  EmbParams p;
  int n = 0;
  int64_t rows = 0;
  if (!collapse_rows(out, &rows, &n, &p.out_stride)) return set_error(ctx, LH_ERR_UNSUPPORTED, "embedding: output rows must be nested");
  p.tokens = numel(ids);
  p.dim = static_cast<int>(wte->shape[1]);
  if (rows != p.tokens || n != p.dim) return set_error(ctx, LH_ERR_INVALID, "embedding: output shape mismatch");
  p.out = data_ptr(out); p.out_dtype = out->dtype;
  p.ids = data_ptr(ids); p.ids_dtype = ids->dtype;
  p.wte = data_ptr(wte); p.wte_dtype = wte->dtype; p.wte_stride = wte->strides[0];
  p.vocab = wte->shape[0];
  p.wpe = nullptr; p.wpe_dtype = 0; p.wpe_stride = 0;
  if (wpe) {
    if (wpe->rank != 2 || wpe->strides[1] != 1 || wpe->shape[1] != p.dim)
      return set_error(ctx, LH_ERR_INVALID, "embedding: positional table must be (period, dim)");
    p.wpe = data_ptr(wpe); p.wpe_dtype = wpe->dtype; p.wpe_stride = wpe->strides[0];
    if (period <= 0 || period > wpe->shape[0]) return set_error(ctx, LH_ERR_INVALID, "embedding: bad period");
  }
  p.period = period;
  if (p.tokens == 0) return LH_OK;
  if (p.tokens > 0x7fffffffLL) return set_error(ctx, LH_ERR_UNSUPPORTED, "embedding: too many tokens");
  embedding_kernel<<<static_cast<unsigned>(p.tokens), 128, 0, ctx->stream>>>(p);
  LH_CHECK_LAUNCH(ctx, "embedding_kernel");
  return LH_OK;
}

}  // namespace lh
