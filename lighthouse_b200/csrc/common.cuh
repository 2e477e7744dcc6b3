// Shared host-side definitions for the library's translation units: the
// context object, error reporting, dtype helpers and the internal kernel
// launch entry points each .cu file provides.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <vector>

#include "../../include/lh_b200.h"

// A buffer allocated symmetrically on every rank (same size, same role): its address here,
// its NVSwitch multicast mapping (one address that reaches all ranks' copies) and the ranks'
// copies as mapped into this process.
struct SymmRegion {
  char* local;
  size_t bytes;
  char* multicast;
  char* peers[LH_MAX_RANKS];
};

// How a small causal attention grid is cut into work items whose key ranges are parts of a
// pair of query tiles' range (attention_tc3.cu). Built once per problem shape, kept until the
// context goes.
struct AttnSplitPlan {
  int bh, sq, skv, hd, grid;  // the shape it was built for
  int chunk;                  // key tiles per item; 0: this shape is not split
  int max_chunks, n_items, n_slots;
  void* table;                // device, n_items x int4
  int* counters;              // device, n_slots x 2, zero between launches
  size_t part_bytes;          // partial results in the context's scratch
};

struct lh_ctx {
  int device = 0;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;  // the stream launches go to (own or external)
  int* dev_status = nullptr;      // device word kernels write a DeviceError into
  int* host_status = nullptr;     // pinned mirror read by lh_b200_sync
  int64_t launches = 0;
  char err[512] = {0};
  // tensor-map encoder resolved from the driver at context creation
  void* encode_tiled = nullptr;
  // scratch for split/partial results and for L2 flushing in benchmarks
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  uint64_t scratch_generation = 0;        // bumped whenever `scratch` is replaced
  std::vector<void*> retired_scratch;     // outgrown buffers, freed at the next lh_b200_sync
  // NCCL
  void* nccl_lib = nullptr;
  void* nccl_comm = nullptr;
  int rank = 0, world = 1;
  // side stream (collectives overlapping the main stream) and the numbered events ordering the two
  cudaStream_t side_stream = nullptr;
  cudaStream_t main_saved = nullptr;  // the main stream while the side stream is selected
  bool side_selected = false;
  std::vector<cudaEvent_t> events;    // indexed by event number, created on first use
  int reserved_sms = 0;               // SMs persistent kernels leave free
  bool launch_overlap = false;        // tensor-core kernels launched as programmatic dependents (lh_b200_set_launch_overlap)
  // symmetric memory for the fused collectives
  std::vector<SymmRegion> symm;
  uint32_t* symm_pads[LH_MAX_RANKS] = {nullptr};  // every rank's flag pad as mapped here
  int symm_rank = 0, symm_world = 0;
  uint32_t symm_epoch = 0;            // launches of flag-synchronised kernels so far (same on every rank)
  bool symm_broken = false;           // a fused launch failed here: launch numbers may differ between ranks
  uint32_t* symm_counter = nullptr;   // device word: blocks finished in the running launch
  // rotary tables built so far
  struct RopeTable { float theta; int dim, positions; float* data; };  // (cos, sin) of positions [0, positions)
  std::vector<RopeTable> rope_tables;
  cudaEvent_t rope_built = nullptr;   // orders a table's build before the other stream's later work
  std::vector<AttnSplitPlan> attn_plans;
};

namespace lh {

int set_error(lh_ctx* ctx, int code, const char* fmt, ...);
char* global_error_buffer();

#define LH_CUDA_CHECK(ctx, expr)                                                                   \
  do {                                                                                             \
    cudaError_t e__ = (expr);                                                                      \
    if (e__ != cudaSuccess)                                                                        \
      return lh::set_error((ctx), LH_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                           __FILE__, __LINE__);                                                    \
  } while (0)

#define LH_CHECK_LAUNCH(ctx, name)                                                                 \
  do {                                                                                             \
    cudaError_t e__ = cudaGetLastError();                                                          \
    if (e__ != cudaSuccess)                                                                        \
      return lh::set_error((ctx), LH_ERR_CUDA, "launch of %s failed: %s", (name), cudaGetErrorString(e__)); \
    (ctx)->launches++;                                                                             \
  } while (0)

inline size_t dtype_size(int dt) {
  switch (dt) {
    case LH_F32: return 4;
    case LH_BF16: return 2;
    case LH_F16: return 2;
    case LH_I32: return 4;
    case LH_I64: return 8;
    case LH_F64: return 8;
  }
  return 0;
}

inline char* data_ptr(const lh_memref_t* m) {
  return static_cast<char*>(m->aligned) + m->offset * (int64_t)dtype_size(m->dtype);
}

inline bool is_contiguous(const lh_memref_t* m) {
  int64_t expect = 1;
  for (int i = m->rank - 1; i >= 0; --i) {
    if (m->shape[i] != 1 && m->strides[i] != expect) return false;
    expect *= m->shape[i];
  }
  return true;
}

inline int64_t numel(const lh_memref_t* m) {
  int64_t n = 1;
  for (int i = 0; i < m->rank; ++i) n *= m->shape[i];
  return n;
}

// ------------------------------------------------------------- GEMM problem
// One (possibly batched) product with its epilogue, in element strides.
struct GemmProblem {
  int M, N, K, batch;
  const void* A; int a_dtype; int64_t sam, sak, sab;  // A(m,k) at A + m*sam + k*sak (+ b*sab)
  const void* B; int b_dtype; int64_t sbk, sbn, sbb;  // B(k,n)
  void* D; int d_dtype; int64_t sdm, sdn, sdb;
  const void* C; int c_dtype; int64_t scm, scn, scb;      // added before bias/act (may be null)
  const void* bias; int bias_dtype;                        // [N] (may be null)
  const void* R; int r_dtype; int64_t srm, srn, srb;      // added after act (may be null)
  int act;
  uint32_t flags;
  // rotary embedding applied to output columns [0, rope_cols) in the epilogue (0: none):
  // heads of rope_dim columns, position = row mod rope_seq; rope_table[pos][pair] = (cos, sin)
  int rope_cols = 0, rope_dim = 0, rope_seq = 0;
  const float* rope_table = nullptr;
};

// Epilogue parameters passed by value to the kernels.
struct EpiParams {
  void* D; int d_dtype; int64_t ldd;
  const void* C; int c_dtype; int64_t ldc;
  const void* bias; int bias_dtype;
  const void* R; int r_dtype; int64_t ldr;
  int act;
  int swiglu;
  const float* rope_table; int rope_cols, rope_dim, rope_seq;
};

int gemm_tc_bf16_supported(const lh_ctx* ctx, const GemmProblem& p);
int gemm_tc_bf16_launch(lh_ctx* ctx, const GemmProblem& p);
int gemm_tc_split_f32_supported(const lh_ctx* ctx, const GemmProblem& p);
int gemm_tc_split_f32_launch(lh_ctx* ctx, const GemmProblem& p);
size_t gemm_tc_split_f32_scratch_bytes(int M, int N, int K);  // 0 where the split-f32 tensor-core path does not apply
int gemm_simt_launch(lh_ctx* ctx, const GemmProblem& p);

// -------------------------------------------------------- attention problem
struct AttnProblem {
  int B, Hq, Hkv, Sq, Skv, D;
  int dtype;  // Q/K/V/O element type
  const void* Q; int64_t sqb, sqh, sqs;  // unit stride in D
  const void* K; int64_t skb, skh, sks;
  const void* V; int64_t svb, svh, svs;
  void* O; int64_t sob, soh, sos;
  int o_dtype;
  float scale;
  int causal;
};
int attn_tc_supported(const lh_ctx* ctx, const AttnProblem& p);
int attn_tc_launch(lh_ctx* ctx, const AttnProblem& p);
int attn_tc2_launch(lh_ctx* ctx, const AttnProblem& p);
int attn_tc3_launch(lh_ctx* ctx, const AttnProblem& p);
// Scratch the tensor-core attention needs for this shape (0 unless its key ranges are split);
// builds and uploads the shape's work-item table on first use (allocates: not under capture).
size_t attn_tc_scratch_bytes(lh_ctx* ctx, int B, int Hq, int Sq, int Skv, int D, int causal);
int attn_simt_launch(lh_ctx* ctx, const AttnProblem& p);

// ------------------------------------------------------------ row operators
int layernorm_launch(lh_ctx* ctx, const lh_memref_t* out, const lh_memref_t* x, const lh_memref_t* gamma,
                     const lh_memref_t* beta, float eps, int rms);
int softmax_launch(lh_ctx* ctx, const lh_memref_t* out, const lh_memref_t* x);
int rope_launch(lh_ctx* ctx, const lh_memref_t* x, float theta, int pos0);
// (cos, sin) of every (position, pair) for rope_launch's arithmetic, cached per context.
int rope_table_for(lh_ctx* ctx, float theta, int pos0, int seq, int dim, const float** table);
int elementwise_launch(lh_ctx* ctx, int kind, const lh_memref_t* out, const lh_memref_t* a,
                       const lh_memref_t* b, int act, float scalar);
int embedding_launch(lh_ctx* ctx, const lh_memref_t* out, const lh_memref_t* ids, const lh_memref_t* wte,
                     const lh_memref_t* wpe, int period);

// Encodes a tiled tensor map through the driver entry point the context resolved.
// dims/strides are innermost-first; strides_bytes[0] is implied by the element size.
int encode_tensor_map(lh_ctx* ctx, CUtensorMap* out, int dtype, int rank, void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, int swizzle128);

int ensure_scratch(lh_ctx* ctx, size_t bytes);

}  // namespace lh
