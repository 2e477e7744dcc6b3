/*
 * lh_b200 — C ABI of the sm_100a execution backend for Lighthouse payloads.
 *
 * Lighthouse (llvm/lighthouse) has no C ABI of its own for this path: its
 * Runner JIT-compiles the lowered payload with the MLIR ExecutionEngine and
 * calls `_mlir_ciface_<fn>` through ctypes with "packed" arguments
 * (lighthouse/execution/runner.py:146-224, lighthouse/utils/memref.py:5-44).
 * This header is the replacement for that boundary: the same memref
 * descriptors and packed-argument convention, but the callee is a fixed
 * library of hand-written CUDA kernels instead of JIT'd code.
 *
 * Conventions
 *   - every entry point is extern "C", returns int (0 = ok, <0 = lh_status_t)
 *     and never throws; lh_b200_last_error() gives the message of the last
 *     failing call on that context (or of ctx creation when ctx == NULL)
 *   - the caller owns every buffer it passes; the library borrows the pointers
 *     until the work is complete on the context's stream (lh_b200_sync)
 *   - one lh_ctx_t per (process, device); calls on one context are serialised
 *     on its stream
 *   - no entry point falls back to the CPU: an unsupported shape/dtype is
 *     LH_ERR_UNSUPPORTED
 */
#ifndef LH_B200_H
#define LH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LH_MAX_RANK 4
#define LH_MAX_OPERANDS 8

typedef struct lh_ctx lh_ctx_t;
typedef struct lh_module lh_module_t;

typedef enum {
  LH_OK = 0,
  LH_ERR_INVALID = -1,     /* bad argument (NULL, rank, shape mismatch)        */
  LH_ERR_UNSUPPORTED = -2, /* valid request this backend has no kernel for     */
  LH_ERR_CUDA = -3,        /* CUDA runtime / driver error                      */
  LH_ERR_DEVICE = -4,      /* a kernel reported a bounded wait that ran out    */
  LH_ERR_COMM = -5,        /* NCCL error or communicator not initialised       */
  LH_ERR_NOMEM = -6
} lh_status_t;

/* Element types. bf16/f16 are 2-byte storage, as in
 * lighthouse/utils/numpy.py:15-84 and lighthouse/utils/torch.py:15-38. */
typedef enum { LH_F32 = 0, LH_BF16 = 1, LH_F16 = 2, LH_I32 = 3, LH_I64 = 4, LH_F64 = 5 } lh_dtype_t;

/*
 * Ranked strided memref with its rank and element type carried alongside.
 * `allocated/aligned/offset/shape/strides` have the meaning of the MLIR memref
 * descriptor that lighthouse/utils/torch.py:41-66 and
 * mlir.runtime.np_to_memref build: strides and offset are in ELEMENTS.
 */
typedef struct {
  void* allocated;
  void* aligned;
  int64_t offset;
  int32_t rank;
  int32_t dtype; /* lh_dtype_t */
  int64_t shape[LH_MAX_RANK];
  int64_t strides[LH_MAX_RANK];
} lh_memref_t;

/* Activation applied in a GEMM epilogue or by lh_b200_elementwise. */
typedef enum {
  LH_ACT_NONE = 0,
  LH_ACT_RELU = 1,      /* max(x, 0): lighthouse/ingress/mlir_gen/named.py:28-32 */
  LH_ACT_GELU_ERF = 2,  /* 0.5 x (1 + erf(x / sqrt 2)); no counterpart in the reference */
  LH_ACT_GELU_TANH = 3, /* tanh approximation; no counterpart in the reference */
  LH_ACT_SILU = 4,      /* x / (1 + exp(-x)): examples/llama/test_llama3.py:225-249 */
  LH_ACT_SIGMOID = 5    /* examples/mpi/feed-forward-mpi.py:213-228 */
} lh_act_t;

/* GEMM flags. */
#define LH_GEMM_ACCUMULATE_C 1u /* add `c` BEFORE bias/activation (accumulate_c of gpu_mlp_payload.py:110-156) */
#define LH_GEMM_FORCE_SIMT 2u   /* use the CUDA-core kernel even if the tensor-core one applies */
#define LH_GEMM_SWIGLU 4u       /* B holds [gate | up] column blocks; D = silu(gate) * up (N_out = N / 2) */
/* Bits 8-15: tile width of the tensor-core kernel divided by 8 (64, 128, 192 or 256 columns;
 * 0 = let the library choose). The hook for a tile database, as the reference's schedules
 * take wg_tile from matmul_params.json (lighthouse/schedule/xegpu/xegpu_parameter_selector.py:26-85). */
#define LH_GEMM_TILE_N(n) (((uint32_t)(n) / 8u) << 8)

/* Elementwise op kinds for lh_b200_elementwise. `b` broadcasts over leading
 * dims when its rank is lower than `a`'s (bias add). */
typedef enum {
  LH_EW_COPY = 0,     /* out = cast(a) — also the strided/transposing copy        */
  LH_EW_ADD = 1,      /* out = a + b                                             */
  LH_EW_MUL = 2,      /* out = a * b                                             */
  LH_EW_ACT = 3,      /* out = act(a)                                            */
  LH_EW_ADD_ACT = 4,  /* out = act(a + b)                                        */
  LH_EW_SILU_MUL = 5, /* out = silu(a) * b                                       */
  LH_EW_SCALE = 6,    /* out = a * scalar                                        */
  LH_EW_FILL = 7,     /* out = scalar                                            */
  LH_EW_SUB = 8,      /* out = a - b                                             */
  LH_EW_MAX = 9       /* out = max(a, b)                                         */
} lh_ew_t;

/* ------------------------------------------------------------------ context */

/* Creates a context on `device` with its own non-blocking stream. Replaces the
 * ExecutionEngine construction of lighthouse/execution/runner.py:129-137. */
int lh_b200_ctx_create(int device, lh_ctx_t** out);
int lh_b200_ctx_destroy(lh_ctx_t* ctx);
/* use_external != 0: launch on the externally owned CUDA stream `cuda_stream`
 * (e.g. torch's current stream; NULL is the legacy default stream).
 * use_external == 0: return to the context's own stream (cuda_stream ignored). */
int lh_b200_ctx_set_stream(lh_ctx_t* ctx, void* cuda_stream, int use_external);
void* lh_b200_ctx_get_stream(lh_ctx_t* ctx);
/* Blocks until the stream is idle, then reads the device status word: returns
 * LH_ERR_DEVICE if a kernel gave up on a bounded wait since the last sync. */
int lh_b200_sync(lh_ctx_t* ctx);
const char* lh_b200_last_error(lh_ctx_t* ctx);
/* Number of kernels this library has launched on the context since creation. */
int64_t lh_b200_launch_count(lh_ctx_t* ctx);
/* Device properties the host side needs: SM count, and whether the device is sm_100. */
int lh_b200_device_info(lh_ctx_t* ctx, int* sm_count, int* cc_major, int* cc_minor);

/* Runs one small kernel whose 64 waits can never be satisfied (an mbarrier nothing arrives on,
 * a flag in this GPU's own memory nothing writes) through the bounded-wait helpers every kernel
 * of this library uses, with `limit_ns` (at most 100 ms) as their limit. The kernel returns
 * normally once the waits have given up; `timed_out_waits` receives how many did (64). The
 * context's status word then holds the self-test's code, so the NEXT lh_b200_sync returns
 * LH_ERR_DEVICE once and clears it; the context stays usable. This is how the give-up path
 * is exercised without making any GPU hang or fault. No counterpart in the reference. */
int lh_b200_selftest_bounded_wait(lh_ctx_t* ctx, uint64_t limit_ns, int* timed_out_waits);

/* ------------------------------------------------------------------- memory */
/* Device buffers for the DeviceMemoryManager protocol
 * (lighthouse/execution/memory_manager.py:70-85,89-168: alloc / copy / dealloc). */
int lh_b200_malloc(lh_ctx_t* ctx, size_t bytes, void** out);
int lh_b200_free(lh_ctx_t* ctx, void* ptr);
/* kind: 0 = host->device, 1 = device->host, 2 = device->device. Asynchronous on
 * the context stream when the host pointer is pinned; ordered with kernels. */
int lh_b200_memcpy(lh_ctx_t* ctx, void* dst, const void* src, size_t bytes, int kind);
int lh_b200_memset(lh_ctx_t* ctx, void* dst, int value, size_t bytes);
int lh_b200_host_alloc(size_t bytes, void** out); /* pinned host memory */
int lh_b200_host_free(void* ptr);

/* ---------------------------------------------------------------- operators */

/*
 * D = epilogue(A . B [+ C] [+ bias]).
 * Semantics of emit_mlp_layer, lighthouse/ingress/mlir_gen/gpu_mlp_payload.py:110-156,
 * and of `linalg.matmul` in test/run/pipeline-check.mlir:8-12:
 *   acc(f32)  = (flags & ACCUMULATE_C) ? extf(C) : 0;  acc += A . B  (f32 accumulate)
 *   acc      += extf(bias)[col]                      (bias may be NULL)
 *   acc       = act(acc)
 *   acc      += extf(residual)                       (residual may be NULL; added AFTER act)
 *   D         = round-to-nearest-even(acc) in D's dtype
 * A is an (M,K) view, B a (K,N) view, both with arbitrary element strides, so a
 * transposed operand is a view with swapped strides (transpose_a / transpose_b of
 * lighthouse/utils/mlir.py:146-173). Rank-3 operands are a batched product
 * (linalg.batch_matmul). bf16 operands whose rows are 16-byte aligned with unit
 * inner stride run on the tcgen05 tensor-core kernel; f32 operands run on the
 * tensor cores as six bf16 products (each operand split into three bf16 terms,
 * f32 accumulation) or on the FFMA kernel; everything else runs on the
 * generic CUDA-core kernel.
 * `c` and `residual` may alias `d`.
 */
int lh_b200_gemm(lh_ctx_t* ctx, const lh_memref_t* d, const lh_memref_t* a, const lh_memref_t* b,
                 const lh_memref_t* c, const lh_memref_t* bias, const lh_memref_t* residual, int act,
                 uint32_t flags);

/*
 * D = A @ B with the rotary embedding of lh_b200_rope applied to output columns
 * [0, rope_cols) on the way out: the fused q/k/v projection of the Llama block
 * (wq, wk, wv followed by apply_rotary_emb, examples/llama/ref_model.py:50-97 and :139-160).
 * Columns are heads of `head_dim`; row r is position pos0 + (r mod seq). The product is
 * rounded to D's type before the rotation, as the separate kernels do. bf16 on the
 * tensor-core kernel rotates in its epilogue from a cached (cos, sin) table; other shapes
 * run lh_b200_gemm followed by lh_b200_rope.
 */
int lh_b200_gemm_rope(lh_ctx_t* ctx, const lh_memref_t* d, const lh_memref_t* a, const lh_memref_t* b,
                      int rope_cols, int head_dim, int seq, float theta, int pos0);

/*
 * O = softmax(scale . Q K^T [+ causal mask]) V, flash style (never materialises
 * the score matrix). Algorithm of ReplaceWithFusedAttentionOp,
 * lighthouse/dialects/transform/transform_ext/ops/replace_with_fused_attention.py:334-455:
 * f32 scores / running max / running sum / accumulator, P rounded to the input
 * dtype before P.V, O = acc / l rounded to the output dtype.
 * Q, O: (B, Hq, Sq, D) views; K, V: (B, Hkv, Skv, D) views with unit stride in D.
 * Hq must be a multiple of Hkv; query head h reads kv head h / (Hq / Hkv)
 * (repeat_kv of examples/llama/ref_model.py:100-111 without materialising it).
 * causal != 0 masks key j > query i + (Skv - Sq)
 * (examples/xegpu/nanoGPT.py:95-111, examples/llama/ref_model.py:266-278).
 */
int lh_b200_attention_fwd(lh_ctx_t* ctx, const lh_memref_t* o, const lh_memref_t* q, const lh_memref_t* k,
                          const lh_memref_t* v, float scale, int causal);

/*
 * The same attention for callers that are not allowed to allocate device memory: a
 * process whose memory pool owns every free byte, a latency-critical thread that must not
 * hit the device-wide synchronisation an allocation may imply, anything running behind a
 * "no allocation after warm-up" rule. It has no counterpart in the reference.
 * It always takes the un-fused route (batched Q K^T, scale, mask, row softmax, batched P V)
 * and keeps the f32 score matrix of one head in a 4 MiB buffer built into the library
 * (every GPU that loads the library holds it until the process exits), so it needs
 * Sq * Skv <= 1,048,576 and returns LH_ERR_UNSUPPORTED with a message beyond that.
 * Operands are rank-4 (B, H, S, D) views as above; results match lh_b200_attention_fwd's
 * un-fused path. It calls no cudaMalloc / cudaFree and no allocating library routine.
 * Q, K, V are f32 or bf16, O is f32 or bf16; anything else is rejected before the first
 * launch. The first call on a device looks up the buffer's device address, and if nothing of
 * this library has run on that device yet it is also the call on which the CUDA runtime loads
 * the library's device image, the 4 MiB buffer included: that first call is the warm-up, it
 * may allocate inside the runtime, and it belongs before any "no allocation" gate and outside
 * any stream capture. Every later call allocates nothing. All calls share the one buffer: two calls whose kernels can
 * overlap on the GPU (different streams or contexts on one device) race on it.
 */
int lh_b200_attention_fwd_noalloc(lh_ctx_t* ctx, const lh_memref_t* o, const lh_memref_t* q, const lh_memref_t* k,
                                  const lh_memref_t* v, float scale, int causal);

/* out = (x - mean) * rsqrt(var + eps) * gamma + beta over the last dim, biased
 * variance, two-pass: emit_layer_norm_generics,
 * lighthouse/ingress/mlir_gen/gpu_layer_norm_payload.py:15-87. gamma/beta may be NULL. */
int lh_b200_layernorm(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* x, const lh_memref_t* gamma,
                      const lh_memref_t* beta, float eps);

/* out = x * rsqrt(mean(x^2) + eps) [* weight]: RMSNorm of
 * examples/llama/ref_model.py:32-47 (weight) / get_l2_norm of
 * examples/llama/test_llama3.py:328-370 (weight == NULL). */
int lh_b200_rmsnorm(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* x, const lh_memref_t* weight,
                    float eps);

/* Row softmax over the last dim: linalg.softmax of
 * lighthouse/ingress/mlir_gen/gpu_softmax_payload.py:11-65. */
int lh_b200_softmax(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* x);

/* Rotary embedding, in place on x (B, S, H, D): pairs (2i, 2i+1) rotated by
 * angle (pos0 + s) * theta^(-2i/D): precompute_freqs_cis / apply_rotary_emb of
 * examples/llama/ref_model.py:50-97. */
int lh_b200_rope(lh_ctx_t* ctx, const lh_memref_t* x, float theta, int pos0);

/* Elementwise family (lh_ew_t): named.add_bias / relu and convert_float_type of
 * lighthouse/ingress/mlir_gen/named.py:20-32, generic.py:160-188, and the
 * Builder.{cast_f16,bias,add} emitters of examples/xegpu/nanoGPT_payload.py:58-286. */
int lh_b200_elementwise(lh_ctx_t* ctx, int kind, const lh_memref_t* out, const lh_memref_t* a,
                        const lh_memref_t* b, int act, float scalar);

/* out[t, :] = wte[ids[t], :] (+ wpe[t mod period, :]); ids are i32 or i64.
 * The reference builds embeddings on the host (examples/xegpu/nanoGPT.py:249-253). */
int lh_b200_embedding(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* ids, const lh_memref_t* wte,
                      const lh_memref_t* wpe, int period);

/* ------------------------------------------------------------- collectives */
/* Tensor-parallel plumbing: the reference's only precedent is the MPI
 * weight-stationary example (examples/mpi/feed-forward-mpi.py:213-228). NCCL is
 * loaded at run time from `nccl_path` (NULL: the loader's default search). */
int lh_b200_comm_unique_id(const char* nccl_path, void* id128); /* fills 128 bytes */
int lh_b200_comm_init(lh_ctx_t* ctx, const char* nccl_path, const void* id128, int rank, int world);
int lh_b200_comm_destroy(lh_ctx_t* ctx);
/* In-place sum all-reduce of the (contiguous) view on the context stream. */
int lh_b200_allreduce(lh_ctx_t* ctx, const lh_memref_t* buf);
/* out (n) = this rank's block of the element-wise sum over ranks of in (world * n); both
 * contiguous. Together with lh_b200_allgather it splits the all-reduce in two, so that the
 * work between them (residual add, normalisation) runs on 1/world of the rows. */
int lh_b200_reducescatter(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* in);
/* out (world * n) = concatenation over ranks of in (n), contiguous. */
int lh_b200_allgather(lh_ctx_t* ctx, const lh_memref_t* out, const lh_memref_t* in);

/* ------------------------------------------------ fused collective kernels */
/*
 * Symmetric memory: buffers that every rank allocates with the same size and role, mapped
 * into every process (peer pointers) and bound to an NVSwitch multicast object (one address
 * whose loads can return the sum over all ranks' copies and whose stores reach all of them).
 * The host allocates and exchanges them (torch.distributed._symmetric_memory in this
 * repository's workloads) and registers the raw addresses here; the library never maps peer
 * memory itself. `pads` are the ranks' flag pads (>= 2 * LH_MAX_RANKS * 4 bytes each) through
 * which the kernels order themselves across ranks; lh_b200_symm_set_flags zeroes this rank's
 * own pad and restarts the launch numbering, so all ranks call it together and pass a barrier
 * before the first fused launch. Every wait on the pads is bounded and ends in LH_ERR_DEVICE at
 * the next lh_b200_sync; after that (or after a failed launch of a fused kernel on any rank)
 * the ranks' launch numbers may differ, further fused calls on that context are refused, and
 * the flags have to be set up again on every rank.
 */
#define LH_MAX_RANKS 8
int lh_b200_symm_register(lh_ctx_t* ctx, void* local, size_t bytes, void* multicast, void* const* peers, int world);
int lh_b200_symm_set_flags(lh_ctx_t* ctx, int rank, int world, void* const* pads);
int lh_b200_symm_clear(lh_ctx_t* ctx);
/*
 * What follows a tensor-parallel contraction, as one kernel on world ranks (rows = h's rows;
 * this rank owns rows [rank * rows, (rank + 1) * rows) of xn and part):
 *   h   <- h + sum over ranks of part[my rows]        (part == NULL: h unchanged)
 *   xn[my rows] on EVERY rank <- rmsnorm(h) * weight
 * i.e. reduce-scatter, residual add, RMSNorm (ref_model.py:24-47) and all-gather. xn and part
 * must lie in registered regions with a multicast mapping; with one rank and no
 * registration the same arithmetic runs on local memory. bf16 activations, row length a
 * multiple of 8 and at most 4096. Every rank must make the same sequence of these calls.
 */
int lh_b200_reduce_norm_gather(lh_ctx_t* ctx, const lh_memref_t* xn, const lh_memref_t* part, const lh_memref_t* h,
                               const lh_memref_t* weight, float eps);

/* ----------------------------------------------------- side stream / events */
/*
 * A context owns a second, high-priority stream for work that should overlap the main
 * stream (a collective and the small kernels around it, while the GEMMs of another
 * micro-batch run). lh_b200_stream_select(ctx, 1) routes every following call of this
 * library to the side stream, (ctx, 0) back to the main one. Ordering between the two is
 * by numbered events: lh_b200_event_record marks the selected stream's position,
 * lh_b200_event_wait makes the selected stream wait for the last record of that number.
 * lh_b200_sync waits for both streams. lh_b200_reserve_sms(ctx, n) makes persistent kernels
 * (the tcgen05 GEMM) launch sm_count - n blocks, so that side-stream kernels find free SMs
 * while a GEMM runs; 0 restores the full grid. The reference has no counterpart: its MPI
 * example communicates synchronously (examples/mpi/feed-forward-mpi.py:213-228).
 */
int lh_b200_stream_select(lh_ctx_t* ctx, int side);
int lh_b200_event_record(lh_ctx_t* ctx, int id);
int lh_b200_event_wait(lh_ctx_t* ctx, int id);
int lh_b200_reserve_sms(lh_ctx_t* ctx, int n);

/*
 * Launch overlap (off by default). With it on, the tensor-core GEMM and attention kernels are
 * launched as programmatic dependents of the kernel before them in the stream: their blocks
 * start on SMs that kernel has already left, set up, and wait for its completion before their
 * first access to global memory. That hides a launch's set-up under its predecessor's tail (a
 * 4096 x 4096 x 1024 GEMM back to back: 33.9 -> 31.2 us), but with copies and event waits of
 * other streams interleaved (a pipelined serving loop) it was measured to cost 4 % of the
 * end-to-end rate, which is why a caller opts in. No counterpart in the reference.
 */
int lh_b200_set_launch_overlap(lh_ctx_t* ctx, int enabled);

/* ------------------------------------------------------------------ modules */
/*
 * A module is a recognised payload: a list of operator records over numbered
 * buffer slots. Slots [0, nargs) are the entry function's arguments in
 * signature order (results are written in place, never re-ordered:
 * gpu_mlp_payload.py:44-48, lh_run.py:110-132); slots >= nargs are temporaries
 * the module allocates once.
 */
typedef enum {
  LH_OP_GEMM = 1,
  LH_OP_ATTENTION = 2,
  LH_OP_LAYERNORM = 3,
  LH_OP_RMSNORM = 4,
  LH_OP_SOFTMAX = 5,
  LH_OP_ROPE = 6,
  LH_OP_ELEMENTWISE = 7,
  LH_OP_EMBEDDING = 8,
  LH_OP_ALLREDUCE = 9,
  LH_OP_ALLGATHER = 10,
  LH_OP_REDUCESCATTER = 11,
  LH_OP_STREAM = 12,
  LH_OP_EVENT_RECORD = 13,
  LH_OP_EVENT_WAIT = 14,
  LH_OP_RESERVE_SMS = 15,
  LH_OP_REDUCE_NORM_GATHER = 16,
  LH_OP_GEMM_ROPE = 17
} lh_op_kind_t;

/* An operand: a view into a slot. slot < 0 means "absent". */
typedef struct {
  int32_t slot;
  int32_t rank;
  int32_t dtype;
  int32_t pad_;
  int64_t offset; /* elements, relative to the slot's base */
  int64_t shape[LH_MAX_RANK];
  int64_t strides[LH_MAX_RANK];
} lh_view_t;

/*
 * Operand order per kind (same as the per-operator entry points):
 *   GEMM        d, a, b, c, bias, residual      i0 = act, i1 = flags
 *   ATTENTION   o, q, k, v                      f0 = scale, i0 = causal
 *   LAYERNORM   out, x, gamma, beta             f0 = eps
 *   RMSNORM     out, x, weight                  f0 = eps
 *   SOFTMAX     out, x
 *   ROPE        x                               f0 = theta, i0 = pos0
 *   ELEMENTWISE out, a, b                       i0 = kind, i1 = act, f0 = scalar
 *   EMBEDDING   out, ids, wte, wpe              i0 = period
 *   ALLREDUCE   buf
 *   ALLGATHER   out, in
 *   REDUCESCATTER out, in
 *   STREAM      (none)                          i0 = 0 main / 1 side
 *   EVENT_RECORD, EVENT_WAIT (none)             i0 = event number
 *   RESERVE_SMS (none)                          i0 = SMs left free by persistent kernels
 *   REDUCE_NORM_GATHER xn, part, h, weight      f0 = eps
 *   GEMM_ROPE   d, a, b                         i0 = rotary columns, i1 = head size, i2 = sequence
 *                                               length, f0 = theta, f1 = first position
 */
typedef struct {
  int32_t kind;
  int32_t i0, i1, i2;
  float f0, f1;
  lh_view_t operands[LH_MAX_OPERANDS];
} lh_op_t;

/* Describes one entry-function argument (rank and dtype are needed to read
 * the rank-specific MLIR descriptors in packed calls). */
typedef struct {
  int32_t rank;
  int32_t dtype;
} lh_arg_sig_t;

/* `temp_bytes[i]` is the size of temporary slot nargs + i. */
int lh_b200_module_create(lh_ctx_t* ctx, const char* entry_name, const lh_arg_sig_t* args, int nargs,
                          const size_t* temp_bytes, int ntemps, const lh_op_t* ops, int nops,
                          lh_module_t** out);
int lh_b200_module_destroy(lh_module_t* m);

/*
 * Packed call, the convention of lighthouse/utils/memref.py:5-44 and the
 * `_mlir_ciface_` entry the Runner looks up (runner.py:214-215):
 * packed_args[i] points to a pointer to the i-th argument's MLIR memref
 * descriptor {T* allocated; T* aligned; int64 offset; int64 shape[r]; int64 strides[r]}.
 * The data pointers must be DEVICE pointers. Launches the module's operators on
 * the context stream; does not synchronise.
 */
int lh_b200_invoke(lh_module_t* m, const char* fn, void** packed_args, int nargs);
/* Same with the argument base pointers given directly (slot i = ptrs[i]). */
int lh_b200_module_run(lh_module_t* m, void* const* arg_ptrs, int nargs);

/*
 * The `__benchmark` contract of
 * lighthouse/dialects/transform/transform_ext/ops/wrap_in_benching_func.py:29-65:
 * nwarmup untimed calls, then nruns calls timed one by one; times[i] is seconds
 * (CUDA events on the context stream instead of rtclock). Synchronises.
 * l2_flush_bytes > 0 overwrites a scratch buffer of that size between timed calls.
 */
int lh_b200_benchmark(lh_module_t* m, void* const* arg_ptrs, int nargs, double* times, int64_t nruns,
                      int64_t nwarmup, size_t l2_flush_bytes);
/* Per-operator timing: with profiling on, module_run records a CUDA event on the context
 * stream before the first operator and after each one; op_times waits for the last run and
 * fills ms[i] with operator i's duration in milliseconds (n = number of operators). */
int lh_b200_module_set_profiling(lh_module_t* m, int enable);
int lh_b200_module_op_times(lh_module_t* m, float* ms, int n);
/* The same events read as a timeline: ms[i] = when operator i ended, measured from the start
 * of the run. With operators on two streams this shows what overlapped what. */
int lh_b200_module_op_end_times(lh_module_t* m, float* ms, int n);
/* Captures one module_run into a CUDA graph and replays it on later runs. */
int lh_b200_module_use_graph(lh_module_t* m, int enable);

#ifdef __cplusplus
}
#endif
#endif /* LH_B200_H */
