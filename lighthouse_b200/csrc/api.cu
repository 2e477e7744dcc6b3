// The extern "C" surface declared in include/lh_b200.h: context, memory, operator
// entry points, recognised-payload modules, packed invocation and benchmarking.
#include <dlfcn.h>
#include <stdlib.h>

#include <string>
#include <vector>

#include "common.cuh"

namespace lh {

static thread_local char g_error[512] = {0};
char* global_error_buffer() { return g_error; }

int set_error(lh_ctx* ctx, int code, const char* fmt, ...) {
  char* dst = ctx ? ctx->err : g_error;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(dst, 512, fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_tensor_map(lh_ctx* ctx, CUtensorMap* out, int dtype, int rank, void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, int swizzle128) {
  if (!ctx->encode_tiled) return set_error(ctx, LH_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMapDataType dt;
  switch (dtype) {
    case LH_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case LH_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case LH_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: return set_error(ctx, LH_ERR_UNSUPPORTED, "tensor map: unsupported dtype %d", dtype);
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      gstrides[i - 1] = strides_bytes[i - 1];
      if (gstrides[i - 1] % 16) return set_error(ctx, LH_ERR_UNSUPPORTED, "tensor map: stride %llu is not a multiple of 16 bytes", (unsigned long long)gstrides[i - 1]);
    }
  }
  if (reinterpret_cast<uintptr_t>(base) % 16) return set_error(ctx, LH_ERR_UNSUPPORTED, "tensor map: base address is not 16-byte aligned");
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
      out, dt, static_cast<cuuint32_t>(rank), base, gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(ctx, LH_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return LH_OK;
}

// Grows the context's scratch buffer. A buffer that is too small is not freed here - kernels
// already queued may still use it, and freeing would need a device-wide wait in the middle of
// a plan - but retired until the next lh_b200_sync, where the stream is idle anyway. Modules
// size the scratch once at creation (module_scratch_bytes), so a plan never grows it mid-run.
// The generation number lets a captured CUDA graph notice that the pointer it baked in is stale.
int ensure_scratch(lh_ctx* ctx, size_t bytes) {
  if (ctx->scratch_bytes >= bytes) return LH_OK;
  void* fresh = nullptr;
  LH_CUDA_CHECK(ctx, cudaMalloc(&fresh, bytes));
  if (ctx->scratch) ctx->retired_scratch.push_back(ctx->scratch);
  ctx->scratch = fresh;
  ctx->scratch_bytes = bytes;
  ctx->scratch_generation++;
  return LH_OK;
}

static void free_retired_scratch(lh_ctx* ctx) {
  for (void* ptr : ctx->retired_scratch) cudaFree(ptr);
  ctx->retired_scratch.clear();
}

// Unfused attention for what the tensor-core kernel does not take (f32 operands,
// odd head sizes): exactly the op sequence of the un-fused payload,
// lighthouse/ingress/mlir_gen/gpu_attention_payload.py:76-129 — batched Q K^T, scale,
// (mask), row softmax, batched P V — with the scores in f32 scratch memory.
__global__ void scale_mask_kernel(float* s, int64_t total, int Sq, int Skv, float scale, int causal) {
  const int offset = Skv - Sq;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int col = static_cast<int>(i % Skv);
    const int row = static_cast<int>((i / Skv) % Sq);
    float v = s[i] * scale;
    if (causal && col > row + offset) v = -INFINITY;
    s[i] = v;
  }
}

int attn_simt_launch(lh_ctx* ctx, const AttnProblem& a) {
  const int64_t score_elems = static_cast<int64_t>(a.Sq) * a.Skv;
  const size_t need = static_cast<size_t>(score_elems) * sizeof(float);
  if (need > (size_t(2) << 30))
    return set_error(ctx, LH_ERR_UNSUPPORTED, "unfused attention would need %zu bytes of score scratch per head", need);
  int rc = ensure_scratch(ctx, need);
  if (rc) return rc;
  const int n_rep = a.Hq / a.Hkv;
  const size_t esz = dtype_size(a.dtype);
  for (int b = 0; b < a.B; ++b) {
    for (int h = 0; h < a.Hq; ++h) {
      const int hk = h / n_rep;
      const char* q = static_cast<const char*>(a.Q) + (b * a.sqb + h * a.sqh) * (int64_t)esz;
      const char* k = static_cast<const char*>(a.K) + (b * a.skb + hk * a.skh) * (int64_t)esz;
      const char* v = static_cast<const char*>(a.V) + (b * a.svb + hk * a.svh) * (int64_t)esz;
      char* o = static_cast<char*>(a.O) + (b * a.sob + h * a.soh) * (int64_t)dtype_size(a.o_dtype);
      GemmProblem g;
      memset(&g, 0, sizeof(g));
      g.batch = 1;
      g.M = a.Sq; g.N = a.Skv; g.K = a.D;
      g.A = q; g.a_dtype = a.dtype; g.sam = a.sqs; g.sak = 1;
      g.B = k; g.b_dtype = a.dtype; g.sbk = 1; g.sbn = a.sks;  // K^T as a strided view
      g.D = ctx->scratch; g.d_dtype = LH_F32; g.sdm = a.Skv; g.sdn = 1;
      rc = gemm_simt_launch(ctx, g);
      if (rc) return rc;
      int64_t blocks = (score_elems + 255) / 256;
      if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
      scale_mask_kernel<<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(
          static_cast<float*>(ctx->scratch), score_elems, a.Sq, a.Skv, a.scale, a.causal);
      LH_CHECK_LAUNCH(ctx, "scale_mask_kernel");
      lh_memref_t s;
      memset(&s, 0, sizeof(s));
      s.allocated = s.aligned = ctx->scratch;
      s.rank = 2; s.dtype = LH_F32;
      s.shape[0] = a.Sq; s.shape[1] = a.Skv; s.strides[0] = a.Skv; s.strides[1] = 1;
      rc = softmax_launch(ctx, &s, &s);
      if (rc) return rc;
      memset(&g, 0, sizeof(g));
      g.batch = 1;
      g.M = a.Sq; g.N = a.D; g.K = a.Skv;
      g.A = ctx->scratch; g.a_dtype = LH_F32; g.sam = a.Skv; g.sak = 1;
      g.B = v; g.b_dtype = a.dtype; g.sbk = a.svs; g.sbn = 1;
      g.D = o; g.d_dtype = a.o_dtype; g.sdm = a.sos; g.sdn = 1;
      rc = gemm_simt_launch(ctx, g);
      if (rc) return rc;
    }
  }
  return LH_OK;
}

}  // namespace lh

using namespace lh;

// ------------------------------------------------------------------- context
extern "C" int lh_b200_ctx_create(int device, lh_ctx_t** out) {
  if (!out) return set_error(nullptr, LH_ERR_INVALID, "ctx_create: out is NULL");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return set_error(nullptr, LH_ERR_CUDA, "no CUDA device available: %s", cudaGetErrorString(e));
  if (device < 0 || device >= count) return set_error(nullptr, LH_ERR_INVALID, "device %d out of range (%d devices)", device, count);
  lh_ctx* ctx = new lh_ctx();
  ctx->device = device;
#define CTX_CHECK(expr)                                                                          \
  do {                                                                                           \
    cudaError_t e__ = (expr);                                                                    \
    if (e__ != cudaSuccess) {                                                                    \
      set_error(nullptr, LH_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));          \
      delete ctx;                                                                                \
      return LH_ERR_CUDA;                                                                        \
    }                                                                                            \
  } while (0)
  CTX_CHECK(cudaSetDevice(device));
  cudaDeviceProp prop;
  CTX_CHECK(cudaGetDeviceProperties(&prop, device));
  ctx->sm_count = prop.multiProcessorCount;
  ctx->cc_major = prop.major;
  ctx->cc_minor = prop.minor;
  CTX_CHECK(cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking));
  ctx->stream = ctx->own_stream;
  CTX_CHECK(cudaMalloc(&ctx->dev_status, sizeof(int)));
  CTX_CHECK(cudaMemset(ctx->dev_status, 0, sizeof(int)));
  CTX_CHECK(cudaMallocHost(&ctx->host_status, sizeof(int)));
  *ctx->host_status = 0;
  cudaDriverEntryPointQueryResult qres;
  void* fn = nullptr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    ctx->encode_tiled = fn;
  (void)cudaGetLastError();
#undef CTX_CHECK
  *out = ctx;
  return LH_OK;
}

extern "C" int lh_b200_comm_destroy(lh_ctx_t* ctx);

extern "C" int lh_b200_ctx_destroy(lh_ctx_t* ctx) {
  if (!ctx) return LH_OK;
  cudaSetDevice(ctx->device);
  lh_b200_comm_destroy(ctx);
  if (ctx->own_stream) {
    cudaStreamSynchronize(ctx->own_stream);
    cudaStreamDestroy(ctx->own_stream);
  }
  if (ctx->side_stream) {
    cudaStreamSynchronize(ctx->side_stream);
    cudaStreamDestroy(ctx->side_stream);
  }
  for (cudaEvent_t e : ctx->events)
    if (e) cudaEventDestroy(e);
  if (ctx->scratch) cudaFree(ctx->scratch);
  for (void* ptr : ctx->retired_scratch) cudaFree(ptr);
  if (ctx->symm_counter) cudaFree(ctx->symm_counter);
  for (auto& t : ctx->rope_tables) cudaFree(t.data);
  for (auto& pl : ctx->attn_plans) {
    if (pl.table) cudaFree(pl.table);
    if (pl.counters) cudaFree(pl.counters);
  }
  if (ctx->rope_built) cudaEventDestroy(ctx->rope_built);
  if (ctx->dev_status) cudaFree(ctx->dev_status);
  if (ctx->host_status) cudaFreeHost(ctx->host_status);
  delete ctx;
  return LH_OK;
}

extern "C" int lh_b200_ctx_set_stream(lh_ctx_t* ctx, void* cuda_stream, int use_external) {
  if (!ctx) return LH_ERR_INVALID;
  if (ctx->side_selected) return set_error(ctx, LH_ERR_INVALID, "ctx_set_stream while the side stream is selected");
  ctx->stream = use_external ? static_cast<cudaStream_t>(cuda_stream) : ctx->own_stream;
  return LH_OK;
}

extern "C" void* lh_b200_ctx_get_stream(lh_ctx_t* ctx) { return ctx ? ctx->stream : nullptr; }

extern "C" int lh_b200_sync(lh_ctx_t* ctx) {
  if (!ctx) return LH_ERR_INVALID;
  if (ctx->side_selected) lh_b200_stream_select(ctx, 0);
  if (ctx->side_stream) LH_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->side_stream));
  LH_CUDA_CHECK(ctx, cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  LH_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
  lh::free_retired_scratch(ctx);  // both streams are idle: nothing can still use an outgrown scratch buffer
  const int st = *ctx->host_status;
  if (st != 0) {
    if (st == 106) ctx->symm_broken = true;  // a peer's flag never came: the ranks are out of step until the flags are set up again
    cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), ctx->stream);
    // an attention launch that gave up may have left its tiles' arrival counters part-way:
    // back to zero, or the next launch's merge would trigger on the wrong item
    for (const AttnSplitPlan& pl : ctx->attn_plans)
      if (pl.counters) cudaMemsetAsync(pl.counters, 0, static_cast<size_t>(pl.n_slots) * 2 * sizeof(int), ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    return set_error(ctx, LH_ERR_DEVICE, "a kernel gave up on a bounded wait (device status %d)", st);
  }
  return LH_OK;
}

extern "C" const char* lh_b200_last_error(lh_ctx_t* ctx) { return ctx ? ctx->err : global_error_buffer(); }
extern "C" int64_t lh_b200_launch_count(lh_ctx_t* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int lh_b200_device_info(lh_ctx_t* ctx, int* sm_count, int* cc_major, int* cc_minor) {
  if (!ctx) return LH_ERR_INVALID;
  if (sm_count) *sm_count = ctx->sm_count;
  if (cc_major) *cc_major = ctx->cc_major;
  if (cc_minor) *cc_minor = ctx->cc_minor;
  return LH_OK;
}

// -------------------------------------------------------------------- memory
extern "C" int lh_b200_malloc(lh_ctx_t* ctx, size_t bytes, void** out) {
  if (!ctx || !out) return LH_ERR_INVALID;
  *out = nullptr;
  if (bytes == 0) bytes = 16;
  cudaError_t e = cudaMalloc(out, bytes);
  if (e == cudaErrorMemoryAllocation) {
    (void)cudaGetLastError();
    return set_error(ctx, LH_ERR_NOMEM, "cudaMalloc of %zu bytes failed: out of memory", bytes);
  }
  LH_CUDA_CHECK(ctx, e);
  return LH_OK;
}

extern "C" int lh_b200_free(lh_ctx_t* ctx, void* ptr) {
  if (!ctx) return LH_ERR_INVALID;
  if (!ptr) return LH_OK;
  LH_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
  LH_CUDA_CHECK(ctx, cudaFree(ptr));
  return LH_OK;
}

extern "C" int lh_b200_memcpy(lh_ctx_t* ctx, void* dst, const void* src, size_t bytes, int kind) {
  if (!ctx || (bytes && (!dst || !src))) return LH_ERR_INVALID;
  if (bytes == 0) return LH_OK;
  cudaMemcpyKind k = kind == 0 ? cudaMemcpyHostToDevice : kind == 1 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
  LH_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, src, bytes, k, ctx->stream));
  if (kind == 1) LH_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
  return LH_OK;
}

extern "C" int lh_b200_memset(lh_ctx_t* ctx, void* dst, int value, size_t bytes) {
  if (!ctx || (bytes && !dst)) return LH_ERR_INVALID;
  if (bytes == 0) return LH_OK;
  LH_CUDA_CHECK(ctx, cudaMemsetAsync(dst, value, bytes, ctx->stream));
  return LH_OK;
}

extern "C" int lh_b200_host_alloc(size_t bytes, void** out) {
  if (!out) return LH_ERR_INVALID;
  cudaError_t e = cudaMallocHost(out, bytes ? bytes : 16);
  if (e != cudaSuccess) return set_error(nullptr, LH_ERR_CUDA, "cudaMallocHost failed: %s", cudaGetErrorString(e));
  return LH_OK;
}
extern "C" int lh_b200_host_free(void* ptr) {
  if (ptr) cudaFreeHost(ptr);
  return LH_OK;
}

// ----------------------------------------------------------------- operators
static int build_gemm(lh_ctx* ctx, GemmProblem& g, const lh_memref_t* d, const lh_memref_t* a, const lh_memref_t* b,
                      const lh_memref_t* c, const lh_memref_t* bias, const lh_memref_t* residual, int act,
                      uint32_t flags) {
  if (!d || !a || !b) return set_error(ctx, LH_ERR_INVALID, "gemm: d, a and b are required");
  if (a->rank != b->rank || a->rank != d->rank || (a->rank != 2 && a->rank != 3))
    return set_error(ctx, LH_ERR_INVALID, "gemm: operands must all be rank 2 or all rank 3 (got %d, %d, %d)", d->rank, a->rank, b->rank);
  const int o = a->rank - 2;
  memset(&g, 0, sizeof(g));
  g.batch = o ? static_cast<int>(a->shape[0]) : 1;
  g.M = static_cast<int>(a->shape[o]);
  g.K = static_cast<int>(a->shape[o + 1]);
  g.N = static_cast<int>(b->shape[o + 1]);
  const int n_out = (flags & LH_GEMM_SWIGLU) ? g.N / 2 : g.N;
  if (b->shape[o] != g.K || d->shape[o] != g.M || d->shape[o + 1] != n_out || (o && (b->shape[0] != g.batch || d->shape[0] != g.batch)))
    return set_error(ctx, LH_ERR_INVALID, "gemm: shape mismatch A(%lld,%lld) B(%lld,%lld) D(%lld,%lld)", (long long)a->shape[o],
                     (long long)a->shape[o + 1], (long long)b->shape[o], (long long)b->shape[o + 1], (long long)d->shape[o],
                     (long long)d->shape[o + 1]);
  g.A = data_ptr(a); g.a_dtype = a->dtype; g.sam = a->strides[o]; g.sak = a->strides[o + 1]; g.sab = o ? a->strides[0] : 0;
  g.B = data_ptr(b); g.b_dtype = b->dtype; g.sbk = b->strides[o]; g.sbn = b->strides[o + 1]; g.sbb = o ? b->strides[0] : 0;
  g.D = data_ptr(d); g.d_dtype = d->dtype; g.sdm = d->strides[o]; g.sdn = d->strides[o + 1]; g.sdb = o ? d->strides[0] : 0;
  auto same2d = [&](const lh_memref_t* m) {
    return m->rank == d->rank && m->shape[o] == g.M && m->shape[o + 1] == n_out && (!o || m->shape[0] == g.batch);
  };
  if (c && (flags & LH_GEMM_ACCUMULATE_C)) {
    if (!same2d(c)) return set_error(ctx, LH_ERR_INVALID, "gemm: C must have D's shape");
    g.C = data_ptr(c); g.c_dtype = c->dtype; g.scm = c->strides[o]; g.scn = c->strides[o + 1]; g.scb = o ? c->strides[0] : 0;
  }
  if (residual) {
    if (!same2d(residual)) return set_error(ctx, LH_ERR_INVALID, "gemm: residual must have D's shape");
    g.R = data_ptr(residual); g.r_dtype = residual->dtype; g.srm = residual->strides[o]; g.srn = residual->strides[o + 1];
    g.srb = o ? residual->strides[0] : 0;
  }
  if (bias) {
    if (numel(bias) != g.N || !is_contiguous(bias)) return set_error(ctx, LH_ERR_INVALID, "gemm: bias must be a contiguous vector of N elements");
    g.bias = data_ptr(bias); g.bias_dtype = bias->dtype;
  }
  g.act = act;
  g.flags = flags;
  return LH_OK;
}

extern "C" int lh_b200_gemm(lh_ctx_t* ctx, const lh_memref_t* d, const lh_memref_t* a, const lh_memref_t* b,
                            const lh_memref_t* c, const lh_memref_t* bias, const lh_memref_t* residual, int act,
                            uint32_t flags) {
  if (!ctx) return LH_ERR_INVALID;
  GemmProblem g;
  int rc = build_gemm(ctx, g, d, a, b, c, bias, residual, act, flags);
  if (rc) return rc;
  if (g.M == 0 || g.N == 0 || g.batch == 0) return LH_OK;
  if (g.K == 0 && !g.C && !g.bias && !g.R && act == LH_ACT_NONE && is_contiguous(d)) {
    return lh_b200_memset(ctx, g.D, 0, static_cast<size_t>(numel(d)) * dtype_size(d->dtype));
  }
  if (gemm_tc_bf16_supported(ctx, g)) return gemm_tc_bf16_launch(ctx, g);
  if (gemm_tc_split_f32_supported(ctx, g)) return gemm_tc_split_f32_launch(ctx, g);
  return gemm_simt_launch(ctx, g);
}

extern "C" int lh_b200_gemm_rope(lh_ctx_t* ctx, const lh_memref_t* d, const lh_memref_t* a, const lh_memref_t* b,
                                 int rope_cols, int head_dim, int seq, float theta, int pos0) {
  if (!ctx) return LH_ERR_INVALID;
  GemmProblem g;
  int rc = build_gemm(ctx, g, d, a, b, nullptr, nullptr, nullptr, LH_ACT_NONE, 0);
  if (rc) return rc;
  if (head_dim < 2 || head_dim % 2 || seq < 1 || rope_cols < 0 || rope_cols % head_dim || rope_cols > g.N || g.batch != 1 || g.M % seq)
    return set_error(ctx, LH_ERR_INVALID, "gemm_rope: %d rotary columns of heads of %d, sequence %d, for a %d x %d product", rope_cols, head_dim, seq, g.M, g.N);
  if (g.M == 0 || g.N == 0) return LH_OK;
  if (rope_cols > 0 && d->dtype == LH_BF16 && head_dim % 64 == 0 && gemm_tc_bf16_supported(ctx, g)) {
    rc = rope_table_for(ctx, theta, pos0, seq, head_dim, &g.rope_table);
    if (rc) return rc;
    g.rope_cols = rope_cols;
    g.rope_dim = head_dim;
    g.rope_seq = seq;
    return gemm_tc_bf16_launch(ctx, g);
  }
  // shapes the fused epilogue does not take: the projection, then the rotary kernel on
  // its leading columns viewed as (batch, seq, heads, head_dim)
  rc = lh_b200_gemm(ctx, d, a, b, nullptr, nullptr, nullptr, LH_ACT_NONE, 0);
  if (rc || rope_cols == 0) return rc;
  lh_memref_t x = *d;
  x.rank = 4;
  x.shape[0] = g.M / seq; x.shape[1] = seq; x.shape[2] = rope_cols / head_dim; x.shape[3] = head_dim;
  x.strides[0] = seq * d->strides[0]; x.strides[1] = d->strides[0]; x.strides[2] = head_dim * d->strides[1]; x.strides[3] = d->strides[1];
  return lh_b200_rope(ctx, &x, theta, pos0);
}

extern "C" int lh_b200_attention_fwd(lh_ctx_t* ctx, const lh_memref_t* o, const lh_memref_t* q, const lh_memref_t* k,
                                     const lh_memref_t* v, float scale, int causal) {
  if (!ctx) return LH_ERR_INVALID;
  if (!o || !q || !k || !v) return set_error(ctx, LH_ERR_INVALID, "attention: null operand");
  if (q->rank != k->rank || q->rank != v->rank || q->rank != o->rank || (q->rank != 3 && q->rank != 4))
    return set_error(ctx, LH_ERR_INVALID, "attention: operands must all be rank 3 (Z,S,D) or rank 4 (B,H,S,D)");
  const int r = q->rank;
  AttnProblem a;
  memset(&a, 0, sizeof(a));
  auto dim = [&](const lh_memref_t* m, int i) { return static_cast<int>(m->shape[i]); };
  if (r == 4) {
    a.B = dim(q, 0); a.Hq = dim(q, 1); a.Sq = dim(q, 2); a.D = dim(q, 3);
    a.Hkv = dim(k, 1); a.Skv = dim(k, 2);
    a.sqb = q->strides[0]; a.sqh = q->strides[1]; a.sqs = q->strides[2];
    a.skb = k->strides[0]; a.skh = k->strides[1]; a.sks = k->strides[2];
    a.svb = v->strides[0]; a.svh = v->strides[1]; a.svs = v->strides[2];
    a.sob = o->strides[0]; a.soh = o->strides[1]; a.sos = o->strides[2];
  } else {
    a.B = dim(q, 0); a.Hq = 1; a.Sq = dim(q, 1); a.D = dim(q, 2);
    a.Hkv = 1; a.Skv = dim(k, 1);
    a.sqb = q->strides[0]; a.sqs = q->strides[1];
    a.skb = k->strides[0]; a.sks = k->strides[1];
    a.svb = v->strides[0]; a.svs = v->strides[1];
    a.sob = o->strides[0]; a.sos = o->strides[1];
  }
  for (int i = 0; i < r; ++i) {
    if (o->shape[i] != q->shape[i]) return set_error(ctx, LH_ERR_INVALID, "attention: O must have Q's shape");
    if (v->shape[i] != k->shape[i]) return set_error(ctx, LH_ERR_INVALID, "attention: V must have K's shape");
  }
  if (k->shape[0] != q->shape[0] || k->shape[r - 1] != q->shape[r - 1])
    return set_error(ctx, LH_ERR_INVALID, "attention: K batch/head_dim must match Q");
  if (a.Hkv < 1 || a.Hq % a.Hkv) return set_error(ctx, LH_ERR_INVALID, "attention: %d query heads are not a multiple of %d kv heads", a.Hq, a.Hkv);
  if (q->strides[r - 1] != 1 || k->strides[r - 1] != 1 || v->strides[r - 1] != 1 || o->strides[r - 1] != 1)
    return set_error(ctx, LH_ERR_UNSUPPORTED, "attention: head_dim must have unit stride");
  if (q->dtype != k->dtype || q->dtype != v->dtype) return set_error(ctx, LH_ERR_INVALID, "attention: Q, K, V dtypes differ");
  a.dtype = q->dtype; a.o_dtype = o->dtype;
  a.Q = data_ptr(q); a.K = data_ptr(k); a.V = data_ptr(v); a.O = data_ptr(o);
  a.scale = scale; a.causal = causal;
  if (a.B == 0 || a.Sq == 0) return LH_OK;
  if (a.Skv == 0) return set_error(ctx, LH_ERR_INVALID, "attention: empty key sequence");
  if (attn_tc_supported(ctx, a)) return attn_tc_launch(ctx, a);
  return attn_simt_launch(ctx, a);
}

extern "C" int lh_b200_layernorm(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* x, const lh_memref_t* gamma,
                                 const lh_memref_t* beta, float eps) {
  if (!ctx) return LH_ERR_INVALID;
  return layernorm_launch(ctx, out, x, gamma, beta, eps, 0);
}
extern "C" int lh_b200_rmsnorm(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* x, const lh_memref_t* weight,
                               float eps) {
  if (!ctx) return LH_ERR_INVALID;
  return layernorm_launch(ctx, out, x, weight, nullptr, eps, 1);
}
extern "C" int lh_b200_softmax(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* x) {
  if (!ctx) return LH_ERR_INVALID;
  return softmax_launch(ctx, out, x);
}
extern "C" int lh_b200_rope(lh_ctx_t* ctx, const lh_memref_t* x, float theta, int pos0) {
  if (!ctx) return LH_ERR_INVALID;
  return rope_launch(ctx, x, theta, pos0);
}
extern "C" int lh_b200_elementwise(lh_ctx_t* ctx, int kind, const lh_memref_t* out, const lh_memref_t* a,
                                   const lh_memref_t* b, int act, float scalar) {
  if (!ctx) return LH_ERR_INVALID;
  return elementwise_launch(ctx, kind, out, a, b, act, scalar);
}
extern "C" int lh_b200_embedding(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* ids, const lh_memref_t* wte,
                                 const lh_memref_t* wpe, int period) {
  if (!ctx) return LH_ERR_INVALID;
  return embedding_launch(ctx, out, ids, wte, wpe, period);
}

// --------------------------------------------------------------- collectives
// NCCL is bound at run time so the library has no link-time dependency on a
// particular libnccl; only the handful of entry points below are used.
namespace {
struct NcclId { char internal[128]; };
typedef int (*nccl_get_id_t)(NcclId*);
typedef int (*nccl_init_rank_t)(void**, int, NcclId, int);
typedef int (*nccl_destroy_t)(void*);
typedef int (*nccl_allreduce_t)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*nccl_allgather_t)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*nccl_reducescatter_t)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef const char* (*nccl_errstr_t)(int);

void* open_nccl(const char* path) {
  void* h = nullptr;
  if (path && *path) h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  return h;
}

int nccl_dtype(int dt) {
  switch (dt) {
    case LH_F32: return 7;   // ncclFloat32
    case LH_BF16: return 9;  // ncclBfloat16
    case LH_F16: return 6;   // ncclFloat16
    case LH_I32: return 2;   // ncclInt32
    case LH_I64: return 4;   // ncclInt64
    case LH_F64: return 8;   // ncclFloat64
  }
  return -1;
}
}  // namespace

extern "C" int lh_b200_comm_unique_id(const char* nccl_path, void* id128) {
  if (!id128) return LH_ERR_INVALID;
  void* h = open_nccl(nccl_path);
  if (!h) return set_error(nullptr, LH_ERR_COMM, "cannot load NCCL: %s", dlerror());
  auto get_id = reinterpret_cast<nccl_get_id_t>(dlsym(h, "ncclGetUniqueId"));
  if (!get_id) return set_error(nullptr, LH_ERR_COMM, "ncclGetUniqueId not found");
  NcclId id;
  int r = get_id(&id);
  if (r != 0) return set_error(nullptr, LH_ERR_COMM, "ncclGetUniqueId failed (%d)", r);
  memcpy(id128, &id, sizeof(id));
  return LH_OK;
}

extern "C" int lh_b200_comm_init(lh_ctx_t* ctx, const char* nccl_path, const void* id128, int rank, int world) {
  if (!ctx || !id128 || world < 1 || rank < 0 || rank >= world) return LH_ERR_INVALID;
  if (ctx->nccl_comm) return set_error(ctx, LH_ERR_COMM, "communicator already initialised");
  void* h = open_nccl(nccl_path);
  if (!h) return set_error(ctx, LH_ERR_COMM, "cannot load NCCL: %s", dlerror());
  auto init_rank = reinterpret_cast<nccl_init_rank_t>(dlsym(h, "ncclCommInitRank"));
  if (!init_rank) return set_error(ctx, LH_ERR_COMM, "ncclCommInitRank not found");
  LH_CUDA_CHECK(ctx, cudaSetDevice(ctx->device));
  NcclId id;
  memcpy(&id, id128, sizeof(id));
  void* comm = nullptr;
  int r = init_rank(&comm, world, id, rank);
  if (r != 0) return set_error(ctx, LH_ERR_COMM, "ncclCommInitRank failed (%d)", r);
  ctx->nccl_lib = h;
  ctx->nccl_comm = comm;
  ctx->rank = rank;
  ctx->world = world;
  return LH_OK;
}

extern "C" int lh_b200_comm_destroy(lh_ctx_t* ctx) {
  if (!ctx || !ctx->nccl_comm) return LH_OK;
  auto destroy = reinterpret_cast<nccl_destroy_t>(dlsym(ctx->nccl_lib, "ncclCommDestroy"));
  if (destroy) destroy(ctx->nccl_comm);
  ctx->nccl_comm = nullptr;
  ctx->world = 1;
  ctx->rank = 0;
  return LH_OK;
}

extern "C" int lh_b200_allreduce(lh_ctx_t* ctx, const lh_memref_t* buf) {
  if (!ctx || !buf) return LH_ERR_INVALID;
  if (ctx->world == 1 && !ctx->nccl_comm) return LH_OK;  // single rank: the sum over one rank is the buffer itself
  if (!ctx->nccl_comm) return set_error(ctx, LH_ERR_COMM, "allreduce: communicator not initialised");
  if (!is_contiguous(buf)) return set_error(ctx, LH_ERR_UNSUPPORTED, "allreduce: buffer must be contiguous");
  const int dt = nccl_dtype(buf->dtype);
  if (dt < 0) return set_error(ctx, LH_ERR_UNSUPPORTED, "allreduce: dtype %d", buf->dtype);
  auto fn = reinterpret_cast<nccl_allreduce_t>(dlsym(ctx->nccl_lib, "ncclAllReduce"));
  if (!fn) return set_error(ctx, LH_ERR_COMM, "ncclAllReduce not found");
  void* p = data_ptr(buf);
  int r = fn(p, p, static_cast<size_t>(numel(buf)), dt, /*ncclSum*/ 0, ctx->nccl_comm, ctx->stream);
  if (r != 0) return set_error(ctx, LH_ERR_COMM, "ncclAllReduce failed (%d)", r);
  return LH_OK;
}

extern "C" int lh_b200_reducescatter(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* in) {
  if (!ctx || !out || !in) return LH_ERR_INVALID;
  if (!is_contiguous(out) || !is_contiguous(in)) return set_error(ctx, LH_ERR_UNSUPPORTED, "reducescatter: buffers must be contiguous");
  if (out->dtype != in->dtype || numel(in) != numel(out) * ctx->world) return set_error(ctx, LH_ERR_INVALID, "reducescatter: size mismatch");
  if (ctx->world == 1 && !ctx->nccl_comm) {
    if (data_ptr(out) == data_ptr(in)) return LH_OK;
    return lh_b200_memcpy(ctx, data_ptr(out), data_ptr(in), static_cast<size_t>(numel(in)) * dtype_size(in->dtype), 2);
  }
  if (!ctx->nccl_comm) return set_error(ctx, LH_ERR_COMM, "reducescatter: communicator not initialised");
  const int dt = nccl_dtype(in->dtype);
  auto fn = reinterpret_cast<nccl_reducescatter_t>(dlsym(ctx->nccl_lib, "ncclReduceScatter"));
  if (!fn || dt < 0) return set_error(ctx, LH_ERR_COMM, "ncclReduceScatter unavailable");
  int r = fn(data_ptr(in), data_ptr(out), static_cast<size_t>(numel(out)), dt, /*ncclSum*/ 0, ctx->nccl_comm, ctx->stream);
  if (r != 0) return set_error(ctx, LH_ERR_COMM, "ncclReduceScatter failed (%d)", r);
  return LH_OK;
}

// ------------------------------------------------------- side stream / events
extern "C" int lh_b200_stream_select(lh_ctx_t* ctx, int side) {
  if (!ctx) return LH_ERR_INVALID;
  if ((side != 0) == ctx->side_selected) return LH_OK;
  if (side) {
    if (!ctx->side_stream) {
      int least = 0, greatest = 0;
      LH_CUDA_CHECK(ctx, cudaDeviceGetStreamPriorityRange(&least, &greatest));
      LH_CUDA_CHECK(ctx, cudaStreamCreateWithPriority(&ctx->side_stream, cudaStreamNonBlocking, greatest));
    }
    ctx->main_saved = ctx->stream;
    ctx->stream = ctx->side_stream;
    ctx->side_selected = true;
  } else {
    ctx->stream = ctx->main_saved;
    ctx->side_selected = false;
  }
  return LH_OK;
}

static int numbered_event(lh_ctx* ctx, int id, bool create, cudaEvent_t* out) {
  if (id < 0 || id >= 4096) return set_error(ctx, LH_ERR_INVALID, "event number %d out of range [0, 4096)", id);
  if (static_cast<size_t>(id) >= ctx->events.size()) ctx->events.resize(id + 1, nullptr);
  if (!ctx->events[id]) {
    if (!create) return set_error(ctx, LH_ERR_INVALID, "event %d waited for before any record", id);
    LH_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&ctx->events[id], cudaEventDisableTiming));
  }
  *out = ctx->events[id];
  return LH_OK;
}

extern "C" int lh_b200_event_record(lh_ctx_t* ctx, int id) {
  if (!ctx) return LH_ERR_INVALID;
  cudaEvent_t e;
  int rc = numbered_event(ctx, id, true, &e);
  if (rc) return rc;
  LH_CUDA_CHECK(ctx, cudaEventRecord(e, ctx->stream));
  return LH_OK;
}

extern "C" int lh_b200_event_wait(lh_ctx_t* ctx, int id) {
  if (!ctx) return LH_ERR_INVALID;
  cudaEvent_t e;
  int rc = numbered_event(ctx, id, false, &e);
  if (rc) return rc;
  LH_CUDA_CHECK(ctx, cudaStreamWaitEvent(ctx->stream, e, 0));
  return LH_OK;
}

extern "C" int lh_b200_reserve_sms(lh_ctx_t* ctx, int n) {
  if (!ctx) return LH_ERR_INVALID;
  if (n < 0 || n >= ctx->sm_count) return set_error(ctx, LH_ERR_INVALID, "reserve_sms: %d of %d SMs", n, ctx->sm_count);
  ctx->reserved_sms = n;
  return LH_OK;
}

extern "C" int lh_b200_set_launch_overlap(lh_ctx_t* ctx, int enabled) {
  if (!ctx) return LH_ERR_INVALID;
  ctx->launch_overlap = enabled != 0;
  return LH_OK;
}

extern "C" int lh_b200_allgather(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* in) {
  if (!ctx || !out || !in) return LH_ERR_INVALID;
  if (!is_contiguous(out) || !is_contiguous(in)) return set_error(ctx, LH_ERR_UNSUPPORTED, "allgather: buffers must be contiguous");
  if (out->dtype != in->dtype || numel(out) != numel(in) * ctx->world) return set_error(ctx, LH_ERR_INVALID, "allgather: size mismatch");
  if (ctx->world == 1 && !ctx->nccl_comm) {
    if (data_ptr(out) == data_ptr(in)) return LH_OK;
    return lh_b200_memcpy(ctx, data_ptr(out), data_ptr(in), static_cast<size_t>(numel(in)) * dtype_size(in->dtype), 2);
  }
  if (!ctx->nccl_comm) return set_error(ctx, LH_ERR_COMM, "allgather: communicator not initialised");
  const int dt = nccl_dtype(in->dtype);
  auto fn = reinterpret_cast<nccl_allgather_t>(dlsym(ctx->nccl_lib, "ncclAllGather"));
  if (!fn || dt < 0) return set_error(ctx, LH_ERR_COMM, "ncclAllGather unavailable");
  int r = fn(data_ptr(in), data_ptr(out), static_cast<size_t>(numel(in)), dt, ctx->nccl_comm, ctx->stream);
  if (r != 0) return set_error(ctx, LH_ERR_COMM, "ncclAllGather failed (%d)", r);
  return LH_OK;
}

// ------------------------------------------------------------------- modules
namespace lh {
// Upper bound of the context scratch an operator can ask for, from its operand views alone
// (the choice between kernels also looks at pointer alignment, which is not known yet).
size_t op_scratch_bytes(lh_ctx* ctx, const lh_op_t& op) {
  if (op.kind == LH_OP_ATTENTION) {
    const lh_view_t& q = op.operands[1];
    const lh_view_t& k = op.operands[2];
    if (q.slot < 0 || k.slot < 0 || q.rank < 3) return 0;
    const int64_t d = q.shape[q.rank - 1];
    if (q.dtype == LH_BF16 && (d == 64 || d == 128)) {
      // tensor-core kernel: no score matrix; partial results where a small causal grid is split
      const int64_t heads = q.rank >= 3 ? q.shape[q.rank - 3] : 1;
      const int64_t batch = q.rank >= 4 ? q.shape[0] : 1;
      if (q.rank > 4 || batch * heads > 0x7fffffffLL) return 0;
      return attn_tc_scratch_bytes(ctx, static_cast<int>(batch), static_cast<int>(heads), static_cast<int>(q.shape[q.rank - 2]),
                                   static_cast<int>(k.shape[k.rank - 2]), static_cast<int>(d), op.i0);
    }
    return static_cast<size_t>(q.shape[q.rank - 2]) * static_cast<size_t>(k.shape[k.rank - 2]) * sizeof(float);
  }
  if (op.kind == LH_OP_GEMM) {
    const lh_view_t& a = op.operands[1];
    const lh_view_t& b = op.operands[2];
    if (a.slot < 0 || b.slot < 0 || a.rank != 2 || a.dtype != LH_F32 || b.dtype != LH_F32) return 0;
    return gemm_tc_split_f32_scratch_bytes(static_cast<int>(a.shape[0]), static_cast<int>(b.shape[1]), static_cast<int>(a.shape[1]));
  }
  return 0;
}
}  // namespace lh

struct lh_module {
  lh_ctx* ctx = nullptr;
  std::string entry;
  std::vector<lh_arg_sig_t> args;
  std::vector<size_t> temp_bytes;
  std::vector<void*> temps;
  std::vector<lh_op_t> ops;
  bool use_graph = false;
  cudaGraphExec_t graph_exec = nullptr;
  std::vector<void*> graph_args;
  uint64_t graph_scratch_generation = 0;  // ctx->scratch_generation the graph was captured under
  // per-operator timing: one event before the first operator and one after each
  bool profiling = false;
  std::vector<cudaEvent_t> op_events;
};

extern "C" int lh_b200_module_create(lh_ctx_t* ctx, const char* entry_name, const lh_arg_sig_t* args, int nargs,
                                     const size_t* temp_bytes, int ntemps, const lh_op_t* ops, int nops,
                                     lh_module_t** out) {
  if (!ctx || !out || nargs < 0 || ntemps < 0 || nops < 0 || (nargs && !args) || (ntemps && !temp_bytes) || (nops && !ops))
    return ctx ? set_error(ctx, LH_ERR_INVALID, "module_create: bad arguments") : LH_ERR_INVALID;
  *out = nullptr;
  const int nslots = nargs + ntemps;
  for (int i = 0; i < nops; ++i) {
    if (ops[i].kind < LH_OP_GEMM || ops[i].kind > LH_OP_GEMM_ROPE) return set_error(ctx, LH_ERR_INVALID, "module_create: op %d has unknown kind %d", i, ops[i].kind);
    for (int j = 0; j < LH_MAX_OPERANDS; ++j) {
      const lh_view_t& v = ops[i].operands[j];
      if (v.slot >= nslots) return set_error(ctx, LH_ERR_INVALID, "module_create: op %d operand %d names slot %d of %d", i, j, v.slot, nslots);
      if (v.slot >= 0 && (v.rank < 0 || v.rank > LH_MAX_RANK)) return set_error(ctx, LH_ERR_INVALID, "module_create: op %d operand %d has rank %d", i, j, v.rank);
    }
  }
  // scratch the operators will ask for, allocated now instead of in the middle of a run
  {
    size_t need = 0;
    const int reserved_now = ctx->reserved_sms;
    for (int i = 0; i < nops; ++i) {
      // persistent kernels size their work lists by the SMs they may take: follow the plan's
      // own reservations while sizing
      if (ops[i].kind == LH_OP_RESERVE_SMS) ctx->reserved_sms = ops[i].i0 > 0 && ops[i].i0 < ctx->sm_count ? ops[i].i0 : 0;
      const size_t b = lh::op_scratch_bytes(ctx, ops[i]);
      if (b > need) need = b;
    }
    ctx->reserved_sms = reserved_now;
    if (need) {
      int rc = ensure_scratch(ctx, need);
      if (rc) return rc;
    }
  }
  lh_module* m = new lh_module();
  m->ctx = ctx;
  m->entry = entry_name ? entry_name : "";
  m->args.assign(args, args + nargs);
  m->temp_bytes.assign(temp_bytes, temp_bytes + ntemps);
  m->ops.assign(ops, ops + nops);
  m->temps.assign(ntemps, nullptr);
  for (int i = 0; i < ntemps; ++i) {
    int rc = lh_b200_malloc(ctx, m->temp_bytes[i], &m->temps[i]);
    if (rc) {
      for (int j = 0; j < i; ++j) cudaFree(m->temps[j]);
      delete m;
      return rc;
    }
  }
  *out = m;
  return LH_OK;
}

extern "C" int lh_b200_module_destroy(lh_module_t* m) {
  if (!m) return LH_OK;
  cudaStreamSynchronize(m->ctx->stream);
  if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
  for (auto& e : m->op_events) cudaEventDestroy(e);
  for (void* t : m->temps)
    if (t) cudaFree(t);
  delete m;
  return LH_OK;
}

static int run_ops(lh_module* m, void* const* arg_ptrs) {
  lh_ctx* ctx = m->ctx;
  const int nargs = static_cast<int>(m->args.size());
  auto resolve = [&](const lh_view_t& v, lh_memref_t& mr) -> const lh_memref_t* {
    if (v.slot < 0) return nullptr;
    void* base = v.slot < nargs ? arg_ptrs[v.slot] : m->temps[v.slot - nargs];
    mr.allocated = base;
    mr.aligned = base;
    mr.offset = v.offset;
    mr.rank = v.rank;
    mr.dtype = v.dtype;
    for (int i = 0; i < LH_MAX_RANK; ++i) {
      mr.shape[i] = v.shape[i];
      mr.strides[i] = v.strides[i];
    }
    return &mr;
  };
  for (size_t i = 0; i < m->ops.size(); ++i) {
    const lh_op_t& op = m->ops[i];
    lh_memref_t mr[LH_MAX_OPERANDS];
    const lh_memref_t* o[LH_MAX_OPERANDS];
    for (int j = 0; j < LH_MAX_OPERANDS; ++j) o[j] = resolve(op.operands[j], mr[j]);
    int rc = LH_OK;
    if (m->profiling && i == 0) cudaEventRecord(m->op_events[0], ctx->stream);
    switch (op.kind) {
      case LH_OP_GEMM: rc = lh_b200_gemm(ctx, o[0], o[1], o[2], o[3], o[4], o[5], op.i0, static_cast<uint32_t>(op.i1)); break;
      case LH_OP_ATTENTION: rc = lh_b200_attention_fwd(ctx, o[0], o[1], o[2], o[3], op.f0, op.i0); break;
      case LH_OP_LAYERNORM: rc = lh_b200_layernorm(ctx, o[0], o[1], o[2], o[3], op.f0); break;
      case LH_OP_RMSNORM: rc = lh_b200_rmsnorm(ctx, o[0], o[1], o[2], op.f0); break;
      case LH_OP_SOFTMAX: rc = lh_b200_softmax(ctx, o[0], o[1]); break;
      case LH_OP_ROPE: rc = lh_b200_rope(ctx, o[0], op.f0, op.i0); break;
      case LH_OP_ELEMENTWISE: rc = lh_b200_elementwise(ctx, op.i0, o[0], o[1], o[2], op.i1, op.f0); break;
      case LH_OP_EMBEDDING: rc = lh_b200_embedding(ctx, o[0], o[1], o[2], o[3], op.i0); break;
      case LH_OP_ALLREDUCE: rc = lh_b200_allreduce(ctx, o[0]); break;
      case LH_OP_REDUCESCATTER: rc = lh_b200_reducescatter(ctx, o[0], o[1]); break;
      case LH_OP_STREAM: rc = lh_b200_stream_select(ctx, op.i0); break;
      case LH_OP_EVENT_RECORD: rc = lh_b200_event_record(ctx, op.i0); break;
      case LH_OP_EVENT_WAIT: rc = lh_b200_event_wait(ctx, op.i0); break;
      case LH_OP_RESERVE_SMS: rc = lh_b200_reserve_sms(ctx, op.i0); break;
      case LH_OP_REDUCE_NORM_GATHER: rc = lh_b200_reduce_norm_gather(ctx, o[0], o[1], o[2], o[3], op.f0); break;
      case LH_OP_ALLGATHER: rc = lh_b200_allgather(ctx, o[0], o[1]); break;
      case LH_OP_GEMM_ROPE: rc = lh_b200_gemm_rope(ctx, o[0], o[1], o[2], op.i0, op.i1, op.i2, op.f0, static_cast<int>(op.f1)); break;
      default: rc = set_error(ctx, LH_ERR_INVALID, "unknown op kind %d", op.kind);
    }
    if (rc) {
      char msg[400];
      snprintf(msg, sizeof(msg), "%s", ctx->err);
      lh_b200_stream_select(ctx, 0);
      ctx->reserved_sms = 0;
      return set_error(ctx, rc, "op %zu (kind %d): %s", i, op.kind, msg);
    }
    if (m->profiling) cudaEventRecord(m->op_events[i + 1], ctx->stream);
  }
  if (ctx->side_selected || ctx->reserved_sms) {
    lh_b200_stream_select(ctx, 0);
    ctx->reserved_sms = 0;
    return set_error(ctx, LH_ERR_INVALID, "module '%s' ends with the side stream selected or SMs reserved", m->entry.c_str());
  }
  return LH_OK;
}

extern "C" int lh_b200_module_run(lh_module_t* m, void* const* arg_ptrs, int nargs) {
  if (!m) return LH_ERR_INVALID;
  lh_ctx* ctx = m->ctx;
  if (nargs != static_cast<int>(m->args.size()) || (nargs && !arg_ptrs))
    return set_error(ctx, LH_ERR_INVALID, "module '%s' takes %zu arguments, got %d", m->entry.c_str(), m->args.size(), nargs);
  if (!m->use_graph) return run_ops(m, arg_ptrs);
  // a captured graph holds raw pointers: the arguments' and the context scratch's
  bool same = m->graph_exec && m->graph_args.size() == static_cast<size_t>(nargs) && m->graph_scratch_generation == ctx->scratch_generation;
  for (int i = 0; same && i < nargs; ++i) same = (m->graph_args[i] == arg_ptrs[i]);
  if (!same) {
    if (m->graph_exec) {
      cudaGraphExecDestroy(m->graph_exec);
      m->graph_exec = nullptr;
    }
    // One eager run first: it sizes scratch buffers and sets kernel attributes outside the capture.
    int rc = run_ops(m, arg_ptrs);
    if (rc) return rc;
    LH_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    LH_CUDA_CHECK(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    rc = run_ops(m, arg_ptrs);
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (rc) {
      if (graph) cudaGraphDestroy(graph);
      return rc;
    }
    LH_CUDA_CHECK(ctx, e);
    e = cudaGraphInstantiate(&m->graph_exec, graph, 0);
    cudaGraphDestroy(graph);
    LH_CUDA_CHECK(ctx, e);
    m->graph_args.assign(arg_ptrs, arg_ptrs + nargs);
    m->graph_scratch_generation = ctx->scratch_generation;
    return LH_OK;  // the eager run above already produced this call's results
  }
  LH_CUDA_CHECK(ctx, cudaGraphLaunch(m->graph_exec, ctx->stream));
  ctx->launches += static_cast<int64_t>(m->ops.size());
  return LH_OK;
}

extern "C" int lh_b200_module_set_profiling(lh_module_t* m, int enable) {
  if (!m) return LH_ERR_INVALID;
  lh_ctx* ctx = m->ctx;
  if (enable && m->use_graph) return set_error(ctx, LH_ERR_INVALID, "per-operator timing is not available in graph mode");
  if (enable && m->op_events.empty()) {
    m->op_events.resize(m->ops.size() + 1);
    for (auto& e : m->op_events) LH_CUDA_CHECK(ctx, cudaEventCreate(&e));
  }
  m->profiling = enable != 0;
  return LH_OK;
}

extern "C" int lh_b200_module_op_times(lh_module_t* m, float* ms, int n) {
  if (!m || !ms) return LH_ERR_INVALID;
  lh_ctx* ctx = m->ctx;
  if (m->op_events.empty() || n != static_cast<int>(m->ops.size()))
    return set_error(ctx, LH_ERR_INVALID, "op_times: profiling was not enabled or n != number of operators");
  LH_CUDA_CHECK(ctx, cudaEventSynchronize(m->op_events.back()));
  for (int i = 0; i < n; ++i) LH_CUDA_CHECK(ctx, cudaEventElapsedTime(&ms[i], m->op_events[i], m->op_events[i + 1]));
  return LH_OK;
}

extern "C" int lh_b200_module_op_end_times(lh_module_t* m, float* ms, int n) {
  if (!m || !ms) return LH_ERR_INVALID;
  lh_ctx* ctx = m->ctx;
  if (m->op_events.empty() || n != static_cast<int>(m->ops.size()))
    return set_error(ctx, LH_ERR_INVALID, "op_end_times: profiling was not enabled or n != number of operators");
  for (int i = 0; i < n; ++i) {
    LH_CUDA_CHECK(ctx, cudaEventSynchronize(m->op_events[i + 1]));
    LH_CUDA_CHECK(ctx, cudaEventElapsedTime(&ms[i], m->op_events[0], m->op_events[i + 1]));
  }
  return LH_OK;
}

extern "C" int lh_b200_module_use_graph(lh_module_t* m, int enable) {
  if (!m) return LH_ERR_INVALID;
  if (enable)
    for (const lh_op_t& op : m->ops) {
      if (op.kind == LH_OP_STREAM) return set_error(m->ctx, LH_ERR_UNSUPPORTED, "graph mode is not available for modules that use the side stream");
      // the cross-rank kernel takes a launch number that every replay would repeat: its flag
      // waits would pass at once from the second replay on and the ranks would run unordered
      if (op.kind == LH_OP_REDUCE_NORM_GATHER && m->ctx->symm_world > 1)
        return set_error(m->ctx, LH_ERR_UNSUPPORTED, "graph mode is not available for modules with the multi-rank reduce_norm_gather operator");
    }
  m->use_graph = enable != 0;
  return LH_OK;
}

// Rank-specific MLIR memref descriptor header: {allocated, aligned, offset, sizes[r], strides[r]}.
struct MlirMemrefHeader {
  void* allocated;
  void* aligned;
  int64_t offset;
};

extern "C" int lh_b200_invoke(lh_module_t* m, const char* fn, void** packed_args, int nargs) {
  if (!m) return LH_ERR_INVALID;
  lh_ctx* ctx = m->ctx;
  if (fn && m->entry != fn) return set_error(ctx, LH_ERR_INVALID, "module has no function '%s' (entry is '%s')", fn, m->entry.c_str());
  if (nargs != static_cast<int>(m->args.size()) || (nargs && !packed_args))
    return set_error(ctx, LH_ERR_INVALID, "function '%s' takes %zu arguments, got %d", m->entry.c_str(), m->args.size(), nargs);
  std::vector<void*> ptrs(nargs);
  for (int i = 0; i < nargs; ++i) {
    // packed_args[i] -> pointer to descriptor pointer -> descriptor
    void** pp = static_cast<void**>(packed_args[i]);
    if (!pp || !*pp) return set_error(ctx, LH_ERR_INVALID, "argument %d is NULL", i);
    const MlirMemrefHeader* h = static_cast<const MlirMemrefHeader*>(*pp);
    ptrs[i] = static_cast<char*>(h->aligned) + h->offset * (int64_t)dtype_size(m->args[i].dtype);
  }
  return lh_b200_module_run(m, ptrs.data(), nargs);
}

__global__ void l2_flush_kernel(float* buf, size_t n, float v) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
    buf[i] = v;
}

extern "C" int lh_b200_benchmark(lh_module_t* m, void* const* arg_ptrs, int nargs, double* times, int64_t nruns,
                                 int64_t nwarmup, size_t l2_flush_bytes) {
  if (!m || !times || nruns < 0 || nwarmup < 0) return LH_ERR_INVALID;
  lh_ctx* ctx = m->ctx;
  if (l2_flush_bytes) {
    int rc = ensure_scratch(ctx, l2_flush_bytes);
    if (rc) return rc;
  }
  for (int64_t i = 0; i < nwarmup; ++i) {
    int rc = lh_b200_module_run(m, arg_ptrs, nargs);
    if (rc) return rc;
  }
  cudaEvent_t e0, e1;
  LH_CUDA_CHECK(ctx, cudaEventCreate(&e0));
  LH_CUDA_CHECK(ctx, cudaEventCreate(&e1));
  int rc = LH_OK;
  for (int64_t i = 0; i < nruns && rc == LH_OK; ++i) {
    if (l2_flush_bytes) {
      l2_flush_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(static_cast<float*>(ctx->scratch), l2_flush_bytes / 4, static_cast<float>(i));
    }
    cudaEventRecord(e0, ctx->stream);
    rc = lh_b200_module_run(m, arg_ptrs, nargs);
    cudaEventRecord(e1, ctx->stream);
    if (cudaEventSynchronize(e1) != cudaSuccess) rc = set_error(ctx, LH_ERR_CUDA, "benchmark: event synchronisation failed: %s", cudaGetErrorString(cudaGetLastError()));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    times[i] = static_cast<double>(ms) * 1e-3;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (rc) return rc;
  return lh_b200_sync(ctx);
}

// --------------------------------------------------- attention without allocation
// Some callers must not trigger device allocation at all: a serving loop that has handed
// the whole memory budget to its own pool, a host thread that must never block on the
// implicit device synchronisation an allocation can cause, code that runs after a
// "no allocation past warm-up" gate. For them this entry point runs the un-fused attention
// (batched Q K^T, scale, mask, row softmax, batched P V) with its score matrix in a buffer
// that is part of the library image instead of one obtained at run time.
namespace {

constexpr int64_t NOALLOC_MAX_SCORES = int64_t(1) << 20;  // Sq * Skv <= 1 Mi f32 = 4 MiB per GPU
static __device__ __align__(256) float g_noalloc_scores[NOALLOC_MAX_SCORES];

constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};

// The array's name is only a host-side handle; the kernels need its address on the device
// they run on, which the runtime reports for the device that is current. The look-up runs
// once per device with that device made current for its duration (the calling thread's
// current device is put back before returning).
int noalloc_scores_ptr(lh_ctx* ctx, float** out) {
  if (ctx->device < 0 || ctx->device >= NOALLOC_MAX_DEVICES)
    return set_error(ctx, LH_ERR_UNSUPPORTED, "attention_fwd_noalloc: device ordinal %d out of range", ctx->device);
  if (!g_noalloc_ptr[ctx->device]) {
    int prev = -1;
    LH_CUDA_CHECK(ctx, cudaGetDevice(&prev));
    if (prev != ctx->device) LH_CUDA_CHECK(ctx, cudaSetDevice(ctx->device));
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scores);
    if (prev != ctx->device) (void)cudaSetDevice(prev);
    LH_CUDA_CHECK(ctx, e);
    g_noalloc_ptr[ctx->device] = ptr;
  }
  *out = g_noalloc_ptr[ctx->device];
  return LH_OK;
}

}  // namespace

extern "C" int lh_b200_attention_fwd_noalloc(lh_ctx_t* ctx, const lh_memref_t* o, const lh_memref_t* q,
                                             const lh_memref_t* k, const lh_memref_t* v, float scale, int causal) {
  if (!ctx) return LH_ERR_INVALID;
  if (!o || !q || !k || !v) return set_error(ctx, LH_ERR_INVALID, "attention_fwd_noalloc: null operand");
  if (q->rank != 4 || k->rank != 4 || v->rank != 4 || o->rank != 4)
    return set_error(ctx, LH_ERR_INVALID, "attention_fwd_noalloc: operands must be rank-4 (B, H, S, D) views");
  for (int i = 0; i < 4; ++i) {
    if (o->shape[i] != q->shape[i] || v->shape[i] != k->shape[i])
      return set_error(ctx, LH_ERR_INVALID, "attention_fwd_noalloc: O must match Q and V must match K in shape");
  }
  if (k->shape[0] != q->shape[0] || k->shape[3] != q->shape[3] || k->shape[1] < 1 || q->shape[1] % k->shape[1])
    return set_error(ctx, LH_ERR_INVALID, "attention_fwd_noalloc: batch / head_dim / head grouping mismatch");
  if (q->strides[3] != 1 || k->strides[3] != 1 || v->strides[3] != 1 || o->strides[3] != 1)
    return set_error(ctx, LH_ERR_UNSUPPORTED, "attention_fwd_noalloc: head_dim must have unit stride");
  if (q->dtype != k->dtype || q->dtype != v->dtype)
    return set_error(ctx, LH_ERR_INVALID, "attention_fwd_noalloc: Q, K, V dtypes differ");
  // every check comes before the first launch, so a rejected call leaves nothing half done
  if (q->dtype != LH_F32 && q->dtype != LH_BF16)
    return set_error(ctx, LH_ERR_UNSUPPORTED, "attention_fwd_noalloc: Q, K, V must be f32 or bf16 (dtype %d)", q->dtype);
  if (o->dtype != LH_F32 && o->dtype != LH_BF16)
    return set_error(ctx, LH_ERR_UNSUPPORTED, "attention_fwd_noalloc: O must be f32 or bf16 (dtype %d)", o->dtype);
  for (int i = 0; i < 4; ++i)
    if (q->shape[i] < 0 || k->shape[i] < 0 || q->shape[i] > 0x7fffffffll || k->shape[i] > 0x7fffffffll)
      return set_error(ctx, LH_ERR_INVALID, "attention_fwd_noalloc: extent out of range");
  if (q->shape[0] == 0 || q->shape[2] == 0) return LH_OK;
  if (k->shape[2] == 0) return set_error(ctx, LH_ERR_INVALID, "attention_fwd_noalloc: empty key sequence");
  const int64_t score_elems = q->shape[2] * k->shape[2];  // both below 2^31: no overflow
  if (score_elems > NOALLOC_MAX_SCORES)
    return set_error(ctx, LH_ERR_UNSUPPORTED,
                     "attention_fwd_noalloc: Sq * Skv = %lld exceeds the built-in score buffer of %lld elements; use lh_b200_attention_fwd",
                     (long long)score_elems, (long long)NOALLOC_MAX_SCORES);
  const int B = static_cast<int>(q->shape[0]), Hq = static_cast<int>(q->shape[1]), Sq = static_cast<int>(q->shape[2]);
  const int D = static_cast<int>(q->shape[3]), Hkv = static_cast<int>(k->shape[1]), Skv = static_cast<int>(k->shape[2]);
  float* scores = nullptr;
  int rc = noalloc_scores_ptr(ctx, &scores);
  if (rc) return rc;
  const int n_rep = Hq / Hkv;
  const int64_t esz = static_cast<int64_t>(dtype_size(q->dtype)), osz = static_cast<int64_t>(dtype_size(o->dtype));
  // The buffer keeps whatever the previous call left; every element a head reads is
  // written first by that head's Q K^T product (no accumulation), so nothing needs clearing.
  for (int b = 0; b < B; ++b) {
    for (int h = 0; h < Hq; ++h) {
      const int hk = h / n_rep;
      GemmProblem g;
      memset(&g, 0, sizeof(g));
      g.batch = 1;
      g.M = Sq; g.N = Skv; g.K = D;
      g.A = data_ptr(q) + (b * q->strides[0] + h * q->strides[1]) * esz; g.a_dtype = q->dtype; g.sam = q->strides[2]; g.sak = 1;
      g.B = data_ptr(k) + (b * k->strides[0] + hk * k->strides[1]) * esz; g.b_dtype = k->dtype; g.sbk = 1; g.sbn = k->strides[2];
      g.D = scores; g.d_dtype = LH_F32; g.sdm = Skv; g.sdn = 1;
      rc = gemm_simt_launch(ctx, g);
      if (rc) return rc;
      int64_t blocks = (score_elems + 255) / 256;
      if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
      scale_mask_kernel<<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(scores, score_elems, Sq, Skv, scale, causal);
      LH_CHECK_LAUNCH(ctx, "scale_mask_kernel");
      lh_memref_t s;
      memset(&s, 0, sizeof(s));
      s.allocated = s.aligned = scores;
      s.rank = 2; s.dtype = LH_F32;
      s.shape[0] = Sq; s.shape[1] = Skv; s.strides[0] = Skv; s.strides[1] = 1;
      rc = softmax_launch(ctx, &s, &s);
      if (rc) return rc;
      memset(&g, 0, sizeof(g));
      g.batch = 1;
      g.M = Sq; g.N = D; g.K = Skv;
      g.A = scores; g.a_dtype = LH_F32; g.sam = Skv; g.sak = 1;
      g.B = data_ptr(v) + (b * v->strides[0] + hk * v->strides[1]) * esz; g.b_dtype = v->dtype; g.sbk = v->strides[2]; g.sbn = 1;
      g.D = data_ptr(o) + (b * o->strides[0] + h * o->strides[1]) * osz; g.d_dtype = o->dtype; g.sdm = o->strides[2]; g.sdn = 1;
      rc = gemm_simt_launch(ctx, g);
      if (rc) return rc;
    }
  }
  return LH_OK;
}
