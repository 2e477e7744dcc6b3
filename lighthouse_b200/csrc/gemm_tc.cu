// bf16 GEMM with fused epilogue on the sm_100a tensor cores.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer: fills a STAGES-deep ring of {A 128x64, B BNx64} bf16
//               tiles in shared memory (128-byte swizzle)
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) into one
//               of two f32 accumulators in tensor memory, so the epilogue of tile t
//               overlaps the main loop of tile t+1
//   warps 2-5   epilogue: each warp owns 32 accumulator rows; per 64 columns it reads
//               them with tcgen05.ld, adds C / bias, applies the activation, adds the
//               residual, rounds, writes a 32-row x 128-byte block into its own
//               swizzled staging buffer and hands it to a TMA store (coalesced,
//               clipped at the matrix edge, asynchronous)
// Hand-offs are mbarriers; every wait is bounded (ptx.cuh) and a wait that runs out
// raises a status word instead of hanging.
//
// What it computes is the layer of emit_mlp_layer
// (lighthouse/ingress/mlir_gen/gpu_mlp_payload.py:110-156): f32 accumulation of
// bf16 products, + bias, activation, round-to-nearest-even to the result type.
#include "common.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"

namespace lh {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                      // 64 bf16 = one 128-byte swizzle row
constexpr int A_TILE_BYTES = BM * BK * 2;   // 16 KiB
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M_MIN = 16;             // tile rasterisation: at least 16 row-blocks share B column-blocks in L2
constexpr size_t GROUP_A_PANEL_BYTES = 36u << 20;  // how much of A a group may keep resident in L2
constexpr int STAGING_BUF_BYTES = 32 * 128; // 32 rows x 128 bytes
constexpr int STAGING_BYTES = 4 * 2 * STAGING_BUF_BYTES;  // 4 epilogue warps x 2 buffers

struct GemmTcParams {
  int M, N, K;
  int n_out;  // columns of D (N, or N/2 with the SwiGLU epilogue)
  int num_m_blocks, num_n_blocks, num_k_blocks;
  int group_m;  // row-blocks per rasterisation group
  int seg_k_blocks;  // SEGS > 1: k-blocks per accumulator
  int num_items;        // work items: full tiles, then the last partial wave's tiles as two half-width items each
  int first_half_item;  // items from here on are half tiles (== num_items when the tail is not split)
  EpiParams epi;
  int* dev_status;
};

__host__ __device__ constexpr int tmem_cols_for(int bn) {
  return (2 * bn <= 32) ? 32 : (2 * bn <= 64) ? 64 : (2 * bn <= 128) ? 128 : (2 * bn <= 256) ? 256 : 512;
}

// TERMS = 3 (the split-f32 path): a stage holds three A tiles and three B tiles, the bf16
// terms of the f32 operands' k-block.
template <int BN, int STAGES, int TERMS = 1>
struct SmemLayout {
  static constexpr int B_TILE_BYTES = BN * BK * 2;
  static constexpr int B_BOX_ROWS = BN == 256 ? 128 : BN;  // k-major B: rows per TMA box (a half tile is one box of the widest tile)
  static constexpr int STAGE_BYTES = TERMS * (A_TILE_BYTES + B_TILE_BYTES);
  static constexpr int STAGING_OFFSET = STAGES * STAGE_BYTES;  // multiple of 1024
  static constexpr int BAR_OFFSET = STAGING_OFFSET + STAGING_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack for the 1024-byte alignment of the ring
  static_assert(DYN_BYTES <= 232448, "exceeds the 227 KiB of shared memory a CTA can opt into");
};

// Tiles are walked group by group: a group is `group_m` row-blocks times all column-blocks,
// row-blocks fastest. Within a group every A row-panel is fetched from HBM once and found in
// L2 by the later column-blocks; B is streamed once per group, so the fewer groups the less
// B traffic - as long as the group's A panel still fits in L2 beside the stream.
__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int group_m, int& m_blk, int& n_blk) {
  const int group_size = group_m * num_n;
  const int group = tile / group_size;
  const int first_m = group * group_m;
  const int rows = min(num_m - first_m, group_m);
  const int in_group = tile - group * group_size;
  m_blk = first_m + in_group % rows;
  n_blk = in_group / rows;
}

// Work item -> (tile, which half, is it a half). When the tiles do not fill the grid's last
// wave and twice the remainder still fits the grid, the remaining tiles are walked as two
// half-width items each: the last wave then takes about 0.6 of a tile's time instead of a
// whole one while most of the SMs idle.
struct WorkItem {
  int tile, half;
  bool is_half;
};
__device__ __forceinline__ WorkItem work_item(int it, int first_half_item) {
  if (it < first_half_item) return {it, 0, false};
  const int h = it - first_half_item;
  return {first_half_item + (h >> 1), h & 1, true};
}

// Every lane observes the phase itself (its later accesses are ordered after it); the warp
// agrees on the verdict so that a wait that ran out never splits it.
__device__ __forceinline__ bool mbar_wait_all(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* dev_status, int code) {
  const bool ok = mbar_wait(bar, parity, abort_flag, dev_status, code);
  return __all_sync(0xffffffffu, ok);
}

// Warp-uniform bounded wait: lane 0 spins, the verdict is broadcast, then every lane
// observes the completed phase itself so that its later reads are ordered after it.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               int* dev_status, int code, int lane) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag, dev_status, code) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (ok) {
    // lane 0 saw the phase complete, so this returns at once; the cap is only a guard
    for (int i = 0; i < (1 << 20) && !mbar_try_wait(bar, parity); ++i) {
    }
  }
  return ok != 0;
}

// 16-byte chunk j of this lane's 128-byte row in a 32-row staging buffer laid out with
// the 128-byte swizzle the output tensor map expects (chunk index XOR row mod 8).
__device__ __forceinline__ void stage_chunk(uint8_t* buf, int lane, int j, uint4 val) {
  *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = val;
}

// Activation over a register block; the switch is outside the loop so that only the
// selected activation's code is ever fetched.
template <int N_>
__device__ __forceinline__ void activate_block(float (&v)[N_], int act) {
  switch (act) {
    case LH_ACT_NONE: break;
    case LH_ACT_RELU:
#pragma unroll
      for (int i = 0; i < N_; ++i) v[i] = fmaxf(v[i], 0.f);
      break;
    case LH_ACT_GELU_ERF:
#pragma unroll
      for (int i = 0; i < N_; ++i) v[i] = apply_act(v[i], LH_ACT_GELU_ERF);
      break;
    case LH_ACT_GELU_TANH:
#pragma unroll
      for (int i = 0; i < N_; ++i) v[i] = apply_act(v[i], LH_ACT_GELU_TANH);
      break;
    case LH_ACT_SILU:
#pragma unroll
      for (int i = 0; i < N_; ++i) v[i] = apply_act(v[i], LH_ACT_SILU);
      break;
    default:
#pragma unroll
      for (int i = 0; i < N_; ++i) v[i] = apply_act(v[i], LH_ACT_SIGMOID);
      break;
  }
}

// Adds a row segment of N_ values held in 16-byte registers (4 f32 or 8 bf16 each).
template <bool F32, int N_>
__device__ __forceinline__ void add_row_segment(float (&v)[N_], const uint4 (&seg)[8]) {
  if (F32) {
#pragma unroll
    for (int j = 0; j < N_ / 4; ++j) {
      v[j * 4 + 0] += __uint_as_float(seg[j].x);
      v[j * 4 + 1] += __uint_as_float(seg[j].y);
      v[j * 4 + 2] += __uint_as_float(seg[j].z);
      v[j * 4 + 3] += __uint_as_float(seg[j].w);
    }
  } else {
#pragma unroll
    for (int j = 0; j < N_ / 8; ++j) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&seg[j]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        v[j * 8 + q * 2] += f.x;
        v[j * 8 + q * 2 + 1] += f.y;
      }
    }
  }
}

// Loads this lane's row segment of N_ values (16-byte vectors of 4 f32 or 8 bf16) starting at
// element `elem0`; vectors past column `n_out` are skipped (n_out is a multiple of 8).
template <bool F32, int N_>
__device__ __forceinline__ void load_row_segment(uint4 (&seg)[8], const void* base, int64_t elem0, int col0, int n_out) {
  constexpr int EPV = F32 ? 4 : 8;
  constexpr int NV = N_ / EPV;
  const char* ptr = static_cast<const char*>(base) + elem0 * (F32 ? 4 : 2);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    seg[j] = (col0 + j * EPV < n_out) ? __ldg(reinterpret_cast<const uint4*>(ptr) + j) : make_uint4(0u, 0u, 0u, 0u);
  }
}

// SEGS > 1 (the split-f32 path below): the k range is cut into up to SEGS segments, each summed
// in its own accumulator (SEGS * BN columns of tensor memory, no double buffering across tiles)
// and the segments' sums are added with correctly rounded f32 adds in the epilogue: the tensor
// core adds into an accumulator with truncation, which biases long sums.
// EPI32: bf16 results in units of 32 columns instead of 64 (launch_variant picks it when the
// epilogue applies an activation with special-function work).
template <int BN, bool B_KMAJOR, int STAGES, bool OUT_F32, int SEGS = 1, int TERMS = 1, bool EPI32 = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmD, const GemmTcParams p) {
  using L = SmemLayout<BN, STAGES, TERMS>;
  static_assert(TERMS == 1 || (TERMS == 3 && B_KMAJOR && SEGS > 1), "three-term stages are the split-f32 path's");
  constexpr int TMEM_COLS = SEGS > 1 ? tmem_cols_for((SEGS * BN + 1) / 2) : tmem_cols_for(BN);
  static_assert(SEGS == 1 || (B_KMAJOR && OUT_F32 && SEGS * BN <= 512), "segmented accumulation is the split-f32 path's");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 128);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched only this CTA's shared and tensor memory, so it may run while the
  // kernel before this one in the stream drains (the launch below asks for that). Every CTA of
  // this persistent grid is resident by now: the next kernel may take SMs as they fall free.
  // From here on global memory is read, by every role: all threads wait for the predecessor.
  grid_dependency_trigger();
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // (warp-uniform like the MMA issuer: every lane waits, one elected lane issues)
    {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < p.num_items && ok; it += gridDim.x) {
        const WorkItem w = work_item(it, p.first_half_item);
        int m_blk, n_blk;
        tile_coords(w.tile, p.num_m_blocks, p.num_n_blocks, p.group_m, m_blk, n_blk);
        const int n0 = n_blk * BN + w.half * (BN / 2);
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!mbar_wait_all(&empty_bar[stage], phase ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * L::STAGE_BYTES;
          uint8_t* sB = sA + TERMS * A_TILE_BYTES;
          // (the two cases are spelled out so that the full tile's loads stay unrolled with
          // constant offsets: this thread's issue rate is on the main loop's critical path)
          if (TERMS == 3) {
            // tensor maps (k, row, term): term t of the k-block into tile t of the stage
            if (elect_one()) {
              mbar_arrive_expect_tx(&full_bar[stage], L::STAGE_BYTES);
#pragma unroll
              for (int t = 0; t < 3; ++t) {
                tma_load_3d(sA + t * A_TILE_BYTES, &tmA, &full_bar[stage], kb * BK, m_blk * BM, t);
                tma_load_3d(sB + t * L::B_TILE_BYTES, &tmB, &full_bar[stage], kb * BK, n0, t);
              }
            }
          } else if (elect_one()) {
          if (!w.is_half) {
            mbar_arrive_expect_tx(&full_bar[stage], L::STAGE_BYTES);
            tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, m_blk * BM);
            if (B_KMAJOR) {
#pragma unroll
              for (int j = 0; j < BN / L::B_BOX_ROWS; ++j)
                tma_load_2d(sB + j * (L::B_BOX_ROWS * BK * 2), &tmB, &full_bar[stage], kb * BK, n0 + j * L::B_BOX_ROWS);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sB + j * (64 * BK * 2), &tmB, &full_bar[stage], n0 + j * 64, kb * BK);
            }
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], A_TILE_BYTES + (BN / 2) * BK * 2);
            tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, m_blk * BM);
            if (B_KMAJOR) {
              tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, n0);  // half tiles exist at BN = 256 only: one box
            } else {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j)
                tma_load_2d(sB + j * (64 * BK * 2), &tmB, &full_bar[stage], n0 + j * 64, kb * BK);
            }
          }
          }
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    // The whole warp walks the loop (waits included) and one elected lane issues: a lone
    // divergent thread pays its address arithmetic per instruction, which bounds tiles of
    // 128 columns and fewer (measured per k-block at 128 / 64 columns: 310 / 292 ns with one
    // thread, 257 / 224 ns this way; 256-wide tiles are bound by the tensor pipe either way).
    constexpr uint32_t idesc_full = make_idesc(UMMA_BF16, BM, BN, false, !B_KMAJOR);
    constexpr uint32_t idesc_half = make_idesc(UMMA_BF16, BM, BN / 2, false, !B_KMAJOR);
    // descriptors of stage 0; a stage / k step is an addition to the 16-byte-unit address field
    const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(smem), 16, 1024);
    const uint64_t b_desc0 = B_KMAJOR ? make_smem_desc_sw128(smem_u32(smem) + TERMS * A_TILE_BYTES, 16, 1024)
                                      : make_smem_desc_sw128(smem_u32(smem) + A_TILE_BYTES, 64 * BK * 2, 1024);
    constexpr uint64_t B_K_STEP = B_KMAJOR ? (32 >> 4) : (2048 >> 4);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int t = 0;
    for (int it = blockIdx.x; it < p.num_items && ok; it += gridDim.x, ++t) {
      const uint32_t idesc = it < p.first_half_item ? idesc_full : idesc_half;
      const int buf = SEGS > 1 ? 0 : (t & 1);
      const uint32_t acc_phase = SEGS > 1 ? (t & 1u) : ((t >> 1) & 1u);
      if (!mbar_wait_all(&tmem_empty[buf], acc_phase ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) break;
      tc_fence_after_sync();
      for (int kb = 0; kb < p.num_k_blocks; ++kb) {
        const int seg = SEGS > 1 ? kb / p.seg_k_blocks : 0;
        const int kb_in_seg = SEGS > 1 ? kb - seg * p.seg_k_blocks : kb;
        const uint32_t d_tmem = tmem_base + (SEGS > 1 ? seg : buf) * BN;
        if (!mbar_wait_all(&full_bar[stage], phase, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (elect_one()) {
          const uint64_t so = static_cast<uint64_t>((stage * L::STAGE_BYTES) >> 4);
          if (TERMS == 3) {
            // x = h + m + l per operand: the six products of weight >= 2^-16, smallest first
            constexpr int TA[6] = {0, 2, 1, 0, 1, 0}, TB[6] = {2, 0, 1, 1, 0, 0};
#pragma unroll
            for (int q = 0; q < 6; ++q) {
              const uint64_t ad = a_desc0 + so + static_cast<uint64_t>((TA[q] * A_TILE_BYTES) >> 4);
              const uint64_t bd = b_desc0 + so + static_cast<uint64_t>((TB[q] * L::B_TILE_BYTES) >> 4);
#pragma unroll
              for (int k = 0; k < BK / 16; ++k)
                umma_f16_ss(d_tmem, ad + static_cast<uint64_t>(k * 2), bd + static_cast<uint64_t>(k * 2), idesc, (kb_in_seg | q | k) != 0 ? 1u : 0u);
            }
          } else {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_f16_ss(d_tmem, a_desc0 + so + static_cast<uint64_t>(k * 2), b_desc0 + so + k * B_K_STEP, idesc, (kb_in_seg | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok && elect_one()) umma_commit(&tmem_full[buf]);
      __syncwarp();
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // tensor-memory lanes [32*quarter, +32) belong to this warp
    const EpiParams& e = p.epi;
    uint8_t* stage_bufs = smem + L::STAGING_OFFSET + quarter * (2 * STAGING_BUF_BYTES);
    int sbuf = 0;
    int t = 0;
    for (int it = blockIdx.x; it < p.num_items; it += gridDim.x, ++t) {
      const WorkItem w = work_item(it, p.first_half_item);
      int m_blk, n_blk;
      tile_coords(w.tile, p.num_m_blocks, p.num_n_blocks, p.group_m, m_blk, n_blk);
      const int buf = SEGS > 1 ? 0 : (t & 1);
      const uint32_t acc_phase = SEGS > 1 ? (t & 1u) : ((t >> 1) & 1u);
      const int nseg = SEGS > 1 ? (p.num_k_blocks + p.seg_k_blocks - 1) / p.seg_k_blocks : 1;
      if (!mbar_wait_warp(&tmem_full[buf], acc_phase, abort_flag, p.dev_status, DEV_TIMEOUT_EPILOGUE, lane))
        break;
      tc_fence_after_sync();
      const int row0 = m_blk * BM + quarter * 32;
      const int row = row0 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      // Output columns of this tile, CHUNK at a time. bf16 results normally go 64 at a time (one
      // stored block per unit: the least per-unit overhead). With an activation that has
      // special-function work, units of 64 left an epilogue warp, alone on its scheduler, with a
      // dependent chain per element that the compiler, at its register limit, did not interleave
      // (erf-GELU on bf16 results 150 us where f32 results, 32 wide, took 112): those launches use
      // units of 32, two per stored block (121 us; without an activation 32-wide units cost 10 %).
      constexpr int CHUNK = (OUT_F32 || EPI32) ? 32 : 64;  // columns per unit of work
      constexpr int PER_STORE = OUT_F32 ? 1 : 64 / CHUNK;  // units per stored block (a 128-byte row segment)
      const int out_cols = (e.swiglu || w.is_half) ? BN / 2 : BN;
      const int out_col_base = e.swiglu ? n_blk * (BN / 2) : n_blk * BN + w.half * (BN / 2);
      const int units = out_cols / CHUNK;
      // The tile's bias, 8 columns per lane, fetched once per tile with one coalesced load and
      // handed round by shuffles (a per-unit load by every lane of the same address costs an L2
      // round trip per group of 8 columns).
      float bq[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (e.bias && lane * 8 < out_cols && out_col_base + lane * 8 < p.n_out) {
        const int bc = out_col_base + lane * 8;
        if (e.bias_dtype == LH_BF16) {
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(e.bias) + bc));
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h2[i]);
            bq[2 * i] = f.x;
            bq[2 * i + 1] = f.y;
          }
        } else {
          const float4 b0 = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(e.bias) + bc));
          const float4 b1 = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(e.bias) + bc + 4));
          bq[0] = b0.x; bq[1] = b0.y; bq[2] = b0.z; bq[3] = b0.w;
          bq[4] = b1.x; bq[5] = b1.y; bq[6] = b1.z; bq[7] = b1.w;
        }
      }
      bool pending = false;  // bf16 results: the first half of a 64-column store block is staged
#pragma unroll 1
      for (int u = 0; u < units; ++u) {
        const int col0 = out_col_base + u * CHUNK;
        const bool active = row0 < p.M && col0 < p.n_out;  // warp-uniform: block intersects D
        float v[CHUNK];
        uint4 cseg[8], rseg[8];
        const bool use_c = e.C != nullptr && active;
        const bool use_r = e.R != nullptr && active;
        if (!e.swiglu) {
          uint32_t raw[CHUNK];
#pragma unroll
          for (int h = 0; h < CHUNK / 32; ++h) tmem_ld_32x32b_x32(taddr + u * CHUNK + h * 32, *reinterpret_cast<uint32_t(*)[32]>(&raw[h * 32]));
          // C / residual rows travel while the tensor-memory load is in flight
          if (use_c) load_row_segment<OUT_F32, CHUNK>(cseg, e.C, row_ok ? static_cast<int64_t>(row) * e.ldc + col0 : 0, row_ok ? col0 : p.n_out, p.n_out);
          if (use_r) load_row_segment<OUT_F32, CHUNK>(rseg, e.R, row_ok ? static_cast<int64_t>(row) * e.ldr + col0 : 0, row_ok ? col0 : p.n_out, p.n_out);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < CHUNK; ++i) v[i] = __uint_as_float(raw[i]);
          if (SEGS > 1) {
            // the later segments' sums, added one by one with rounded f32 adds
            for (int sg = 1; sg < nseg; ++sg) {
              tmem_ld_32x32b_x32(taddr + sg * BN + u * CHUNK, *reinterpret_cast<uint32_t(*)[32]>(&raw[0]));  // f32 results: CHUNK = 32
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < CHUNK; ++i) v[i] += __uint_as_float(raw[i]);
            }
          }
        } else {
          // B columns of this tile are [gate (BN/2) | up (BN/2)]: D = silu(gate) * up.
#pragma unroll
          for (int h = 0; h < CHUNK / 32; ++h) {
            uint32_t g_[32], u_[32];
            tmem_ld_32x32b_x32(taddr + u * CHUNK + h * 32, g_);
            tmem_ld_32x32b_x32(taddr + BN / 2 + u * CHUNK + h * 32, u_);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              // IEEE divide here (this epilogue hides under a main loop over K >= 4096 and the
              // product feeds a contraction over 14336 terms)
              const float gv = __uint_as_float(g_[i]);
              v[h * 32 + i] = gv / (1.f + __expf(-gv)) * __uint_as_float(u_[i]);
            }
          }
        }
        if (u == units - 1) {
          // every accumulator column of this tile is now in registers
          tc_fence_before_sync();
          mbar_arrive(&tmem_empty[buf]);
        }
        // bf16 results leave in blocks of 64 columns (one 128-byte row segment): two units
        // share a staging buffer and a store
        const int part = u % PER_STORE;
        uint8_t* sb = stage_bufs + sbuf * STAGING_BUF_BYTES;
        if (active) {
          if (!e.swiglu) {
            if (use_c) add_row_segment<OUT_F32>(v, cseg);
            if (e.bias) {
              // lane (u * CHUNK) / 8 + g holds the bias of this unit's g-th group of 8 columns
#pragma unroll
              for (int g = 0; g < CHUNK / 8; ++g) {
                const int src = u * (CHUNK / 8) + g;
#pragma unroll
                for (int i = 0; i < 8; ++i) v[g * 8 + i] += __shfl_sync(0xffffffffu, bq[i], src);
              }
            }
#pragma unroll
            for (int h = 0; h < CHUNK / 32; ++h) activate_block(*reinterpret_cast<float(*)[32]>(&v[h * 32]), e.act);
            if (use_r) add_row_segment<OUT_F32>(v, rseg);
            if (!OUT_F32 && col0 < e.rope_cols) {
              // Rotary embedding on the way out: pairs (2i, 2i+1) of a head are neighbours in
              // this thread's registers. The value is first rounded to the output type, as a
              // separate rotary kernel reading the stored projection would see it.
              const int pos = row_ok ? row % e.rope_seq : 0;
              const float4* tab = reinterpret_cast<const float4*>(e.rope_table) +
                                  (static_cast<int64_t>(pos) * (e.rope_dim / 2) + (col0 % e.rope_dim) / 2) / 2;
#pragma unroll
              for (int j = 0; j < CHUNK / 4; ++j) {
                const float4 cs = __ldg(tab + j);  // (cos, sin) of two pairs
                const float x0 = __bfloat162float(__float2bfloat16_rn(v[4 * j])), x1 = __bfloat162float(__float2bfloat16_rn(v[4 * j + 1]));
                const float x2 = __bfloat162float(__float2bfloat16_rn(v[4 * j + 2])), x3 = __bfloat162float(__float2bfloat16_rn(v[4 * j + 3]));
                v[4 * j] = x0 * cs.x - x1 * cs.y;
                v[4 * j + 1] = x0 * cs.y + x1 * cs.x;
                v[4 * j + 2] = x2 * cs.z - x3 * cs.w;
                v[4 * j + 3] = x2 * cs.w + x3 * cs.z;
              }
            }
          }
          if (part == 0) {
            if (lane == 0) bulk_wait_group_read<1>();  // the store that last read this buffer is done
            __syncwarp();
          }
          if (!OUT_F32) {
#pragma unroll
            for (int j = 0; j < CHUNK / 8; ++j) {
              uint4 q;
              q.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
              q.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
              q.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
              q.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
              stage_chunk(sb, lane, part * (CHUNK / 8) + j, q);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              stage_chunk(sb, lane, j, make_uint4(__float_as_uint(v[j * 4]), __float_as_uint(v[j * 4 + 1]), __float_as_uint(v[j * 4 + 2]), __float_as_uint(v[j * 4 + 3])));
          }
          pending = true;
        }
        // the block goes out after its last unit (columns past the edge of D are clipped by
        // the store, so a first half alone is complete)
        const bool last_of_block = part == PER_STORE - 1 || u == units - 1;
        if (pending && last_of_block) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmD, sb, col0 - part * CHUNK, row0);
            bulk_commit_group();
          }
          sbuf ^= 1;
          pending = false;
        }
      }
    }
    if (lane == 0) bulk_wait_group<0>();  // all stores of this warp have landed
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if (*abort_flag) {
      // A role gave up: let copies and MMAs already in flight drain before the
      // tensor memory goes back to the allocator.
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// TERMS = 3: pr.A / pr.B point at three consecutive (rows, ld) bf16 arrays, the terms of the f32
// operands, `term_stride_a` / `term_stride_b` elements apart; pr.K is the f32 operands' k range.
template <int BN, bool B_KMAJOR, int STAGES, bool OUT_F32, int SEGS = 1, int TERMS = 1, bool EPI32 = false>
int launch_variant(lh_ctx* ctx, const GemmProblem& pr, const EpiParams& epi, int seg_k_blocks = 0, int64_t term_stride_a = 0,
                   int64_t term_stride_b = 0, bool follows_own_kernel = false) {
  using L = SmemLayout<BN, STAGES, TERMS>;
  CUtensorMap tmA, tmB, tmD;
  const int n_out = epi.swiglu ? pr.N / 2 : pr.N;
  constexpr uint64_t ab_size = 2;
  constexpr int ab_dtype = LH_BF16;
  if (TERMS == 3) {
    const uint64_t dims_a[3] = {static_cast<uint64_t>(pr.K), static_cast<uint64_t>(pr.M), 3};
    const uint64_t strides_a[2] = {static_cast<uint64_t>(pr.sam) * ab_size, static_cast<uint64_t>(term_stride_a) * ab_size};
    const uint32_t box_a[3] = {BK, BM, 1};
    int rc = encode_tensor_map(ctx, &tmA, ab_dtype, 3, const_cast<void*>(pr.A), dims_a, strides_a, box_a, 1);
    if (rc) return rc;
    const uint64_t dims_b[3] = {static_cast<uint64_t>(pr.K), static_cast<uint64_t>(pr.N), 3};
    const uint64_t strides_b[2] = {static_cast<uint64_t>(pr.sbn) * ab_size, static_cast<uint64_t>(term_stride_b) * ab_size};
    const uint32_t box_b[3] = {BK, BN, 1};
    rc = encode_tensor_map(ctx, &tmB, ab_dtype, 3, const_cast<void*>(pr.B), dims_b, strides_b, box_b, 1);
    if (rc) return rc;
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(pr.K), static_cast<uint64_t>(pr.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(pr.sam) * ab_size};
    const uint32_t box[2] = {BK, BM};
    int rc = encode_tensor_map(ctx, &tmA, ab_dtype, 2, const_cast<void*>(pr.A), dims, strides, box, 1);
    if (rc) return rc;
  }
  if (TERMS == 3) {
  } else if (B_KMAJOR) {  // B(k,n) with unit k stride: a row-major (N,K) array
    const uint64_t dims[2] = {static_cast<uint64_t>(pr.K), static_cast<uint64_t>(pr.N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(pr.sbn) * ab_size};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(L::B_BOX_ROWS)};
    int rc = encode_tensor_map(ctx, &tmB, ab_dtype, 2, const_cast<void*>(pr.B), dims, strides, box, 1);
    if (rc) return rc;
  } else {  // B(k,n) with unit n stride: a row-major (K,N) array
    const uint64_t dims[2] = {static_cast<uint64_t>(pr.N), static_cast<uint64_t>(pr.K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(pr.sbk) * 2};
    const uint32_t box[2] = {64, BK};
    int rc = encode_tensor_map(ctx, &tmB, LH_BF16, 2, const_cast<void*>(pr.B), dims, strides, box, 1);
    if (rc) return rc;
  }
  {
    const uint64_t esz = OUT_F32 ? 4 : 2;
    const uint64_t dims[2] = {static_cast<uint64_t>(n_out), static_cast<uint64_t>(pr.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(pr.sdm) * esz};
    const uint32_t box[2] = {OUT_F32 ? 32u : 64u, 32u};
    int rc = encode_tensor_map(ctx, &tmD, pr.d_dtype, 2, pr.D, dims, strides, box, 1);
    if (rc) return rc;
  }
  GemmTcParams p;
  p.M = pr.M;
  p.N = pr.N;
  p.K = pr.K;
  p.n_out = n_out;
  p.num_m_blocks = (pr.M + BM - 1) / BM;
  p.num_n_blocks = (pr.N + BN - 1) / BN;
  p.num_k_blocks = (pr.K + BK - 1) / BK;
  // Widest group whose A panel (group_m x 128 rows x K) stays within a quarter of L2: 64
  // row-blocks up to K = 2048, 32 up to 4096, 16 beyond (measured at 16 with K = 4096,
  // N = 28672: B read 8 times, 2.0 GB of DRAM reads for 0.37 GB of operands).
  p.group_m = GROUP_M_MIN;
  {
    const size_t row_block_bytes = static_cast<size_t>(BM) * pr.K * ab_size;
    while (p.group_m < 64 && 2 * static_cast<size_t>(p.group_m) * row_block_bytes <= GROUP_A_PANEL_BYTES && p.num_m_blocks > p.group_m) p.group_m *= 2;
  }
  p.epi = epi;
  p.seg_k_blocks = seg_k_blocks > 0 ? seg_k_blocks : p.num_k_blocks;
  p.dev_status = ctx->dev_status;
  auto kernel = gemm_bf16_tc_kernel<BN, B_KMAJOR, STAGES, OUT_F32, SEGS, TERMS, EPI32>;
  LH_CUDA_CHECK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;
  // A persistent grid that fills the GPU would make side-stream kernels (collectives) wait for
  // this kernel's end; lh_b200_reserve_sms leaves them room.
  const int sms = ctx->sm_count - ctx->reserved_sms > 0 ? ctx->sm_count - ctx->reserved_sms : 1;
  const int grid = num_tiles < sms ? num_tiles : sms;
  // the last partial wave as half tiles, when both halves of each of its tiles get an SM
  const int leftover = num_tiles % grid;
  const bool split_tail = BN == 256 && SEGS == 1 && !epi.swiglu && leftover > 0 && 2 * leftover <= grid;
  p.first_half_item = split_tail ? num_tiles - leftover : num_tiles;
  p.num_items = split_tail ? num_tiles + leftover : num_tiles;
  // With launch overlap on (lh_b200_set_launch_overlap): programmatic dependent launch. This
  // kernel's CTAs may start (barrier set-up, tensor-memory allocation) on SMs the previous
  // kernel in the stream has already left; they wait for its completion before their first
  // global access (grid_dependency_wait in the kernel).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = L::DYN_BYTES;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (ctx->launch_overlap || follows_own_kernel) ? 1 : 0;  // off: an ordinary launch, the kernel's grid-dependency calls are no-ops
  LH_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmD, p));
  LH_CHECK_LAUNCH(ctx, "gemm_bf16_tc_kernel");
  return LH_OK;
}

template <bool B_KMAJOR, bool OUT_F32>
int launch_bn(lh_ctx* ctx, const GemmProblem& p, const EpiParams& epi, int bn) {
  // bf16 results through an activation with special-function work: 32-column epilogue units
  const bool epi32 = !OUT_F32 && !epi.swiglu && epi.act != LH_ACT_NONE && epi.act != LH_ACT_RELU;
  if (epi32) {
    switch (bn) {
      case 256: return launch_variant<256, B_KMAJOR, 4, OUT_F32, 1, 1, !OUT_F32>(ctx, p, epi);
      case 192: return launch_variant<192, B_KMAJOR, 4, OUT_F32, 1, 1, !OUT_F32>(ctx, p, epi);
      case 128: return launch_variant<128, B_KMAJOR, 6, OUT_F32, 1, 1, !OUT_F32>(ctx, p, epi);
      default: return launch_variant<64, B_KMAJOR, 8, OUT_F32, 1, 1, !OUT_F32>(ctx, p, epi);
    }
  }
  switch (bn) {
    case 256: return launch_variant<256, B_KMAJOR, 4, OUT_F32>(ctx, p, epi);
    case 192: return launch_variant<192, B_KMAJOR, 4, OUT_F32>(ctx, p, epi);
    case 128: return launch_variant<128, B_KMAJOR, 6, OUT_F32>(ctx, p, epi);
    default: return launch_variant<64, B_KMAJOR, 8, OUT_F32>(ctx, p, epi);
  }
}

int pick_bn(const lh_ctx* ctx, const GemmProblem& p) {
  if (p.flags & LH_GEMM_SWIGLU) return 256;
  const int hint = static_cast<int>((p.flags >> 8) & 0xffu) * 8;  // the caller's tile database
  if (hint == 64 || hint == 128 || hint == 192 || hint == 256) return hint;
  // Cost model: waves of tiles over the SMs times the per-tile time; narrower tiles
  // re-read A more often per flop, which the relative efficiencies account for.
  const int cand[3] = {256, 192, 128};
  const double eff[3] = {1.0, 0.88, 0.72};  // measured on 4096 x 4096 x K problems
  const int num_m = (p.M + BM - 1) / BM;
  const int sms = ctx->sm_count - ctx->reserved_sms > 0 ? ctx->sm_count - ctx->reserved_sms : 1;  // the grid's size
  int best = 256;
  double best_cost = 1e300;
  for (int i = 0; i < 3; ++i) {
    const int bn = cand[i];
    const int64_t tiles = static_cast<int64_t>(num_m) * ((p.N + bn - 1) / bn);
    const int64_t waves = (tiles + sms - 1) / sms;
    const double cost = static_cast<double>(waves) * bn / eff[i];
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

}  // namespace

int gemm_tc_bf16_supported(const lh_ctx* ctx, const GemmProblem& p) {
  if (ctx->cc_major != 10) return 0;
  if (p.flags & LH_GEMM_FORCE_SIMT) return 0;
  if (p.batch != 1) return 0;
  if (p.a_dtype != LH_BF16 || p.b_dtype != LH_BF16) return 0;
  if (p.M < 1 || p.N < 8 || p.K < 8) return 0;
  auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  // A must be k-contiguous with 16-byte aligned rows.
  if (p.sak != 1 || (p.sam % 8) != 0 || p.sam < p.K || !aligned16(p.A)) return 0;
  const bool b_kmajor = (p.sbk == 1 && p.N > 1 && p.sbn >= p.K);
  const bool b_nmajor = (p.sbn == 1 && p.sbk >= p.N);
  if (!b_kmajor && !b_nmajor) return 0;
  if (b_nmajor && !b_kmajor && (p.sbk % 8) != 0) return 0;
  if (b_kmajor && (p.sbn % 8) != 0) return 0;
  if (!aligned16(p.B)) return 0;
  const int n_out = (p.flags & LH_GEMM_SWIGLU) ? p.N / 2 : p.N;
  if ((p.flags & LH_GEMM_SWIGLU) && ((p.N % 256) != 0 || p.C || p.bias || p.R)) return 0;
  if (p.N % 8) return 0;
  // D goes out through a tensor map; C / bias / residual use 8-element vectors.
  if (p.d_dtype != LH_BF16 && p.d_dtype != LH_F32) return 0;
  if (p.sdn != 1 || (p.sdm % 8) != 0 || p.sdm < n_out || !aligned16(p.D)) return 0;
  if (p.C) {
    if (p.c_dtype != p.d_dtype) return 0;  // the epilogue reads C rows as D-typed 128-byte segments
    if (p.scn != 1 || (p.scm % 8) != 0 || !aligned16(p.C)) return 0;
  }
  if (p.R) {
    if (p.r_dtype != p.d_dtype) return 0;
    if (p.srn != 1 || (p.srm % 8) != 0 || !aligned16(p.R)) return 0;
  }
  if (p.bias) {
    if (p.bias_dtype != LH_BF16 && p.bias_dtype != LH_F32) return 0;
    if (!aligned16(p.bias)) return 0;
  }
  return 1;
}

int gemm_tc_bf16_launch(lh_ctx* ctx, const GemmProblem& p) {
  EpiParams epi;
  epi.D = p.D; epi.d_dtype = p.d_dtype; epi.ldd = p.sdm;
  epi.C = p.C; epi.c_dtype = p.c_dtype; epi.ldc = p.scm;
  epi.bias = p.bias; epi.bias_dtype = p.bias_dtype;
  epi.R = p.R; epi.r_dtype = p.r_dtype; epi.ldr = p.srm;
  epi.rope_table = p.rope_table; epi.rope_cols = p.rope_table ? p.rope_cols : 0; epi.rope_dim = p.rope_dim; epi.rope_seq = p.rope_seq;
  epi.act = p.act;
  epi.swiglu = (p.flags & LH_GEMM_SWIGLU) ? 1 : 0;
  const bool b_kmajor = (p.sbk == 1 && p.N > 1 && p.sbn >= p.K);
  const bool out_f32 = p.d_dtype == LH_F32;
  const int bn = pick_bn(ctx, p);
  if (b_kmajor) return out_f32 ? launch_bn<true, true>(ctx, p, epi, bn) : launch_bn<true, false>(ctx, p, epi, bn);
  return out_f32 ? launch_bn<false, true>(ctx, p, epi, bn) : launch_bn<false, false>(ctx, p, epi, bn);
}

// ------------------------------------------------------------- f32 GEMM as six bf16 products
// Each f32 operand is split into three bf16 terms, x = h + m + l exactly up to 2^-24 |x|:
// h = bf16(x), m = bf16(x - h), l = bf16(x - h - m) (both differences are exact in f32). The
// f32 product is summed from the six bf16 products whose weight is at least 2^-16,
//   h*h + h*m + m*h + m*m + h*l + l*h     (dropped: m*l, l*m, l*l, about 2^-24 relative),
// with f32 accumulation in tensor memory. split_bf16x3_kernel writes the terms of both operands
// as three k-major bf16 arrays each into context scratch (transposing B as needed): 6 bytes per
// operand element. The GEMM kernel's three-term instantiation loads the three A tiles and three
// B tiles of a k-block into one stage and issues the six products from them - the operand
// bytes into the SM, which bound this path, are half of what one concatenated [h h m m h l] x
// [h m h m l h] k dimension would move, and a quarter of the barrier rounds.
// The tensor core adds into its f32 accumulator with truncation, a bias towards zero of about
// 3e-8 of the sum per instruction. So k is cut into segments of SPLIT_SEGMENT columns (96
// instructions), each summed in its own accumulator, and the segments' sums are added with
// correctly rounded f32 adds in the epilogue. A k range beyond what one launch's accumulators
// hold takes further launches whose epilogue adds the running result as C.
namespace {

struct SplitOperand {
  const float* src;
  int64_t s_row, s_k;
  int rows;
  __nv_bfloat16* dst;  // [3 terms][rows][ld]
};

constexpr int SPLIT_SEGMENT = 256;                    // k per accumulator: 4 k-blocks x 6 products x 4 instructions
constexpr int64_t SPLIT_MIN_WORK = 1ll << 21;         // below this the CUDA-core kernel's single launch wins
constexpr size_t SPLIT_MAX_SCRATCH = 3ull << 30;      // split copies larger than this stay on the CUDA cores

// Both operands in one launch: blockIdx.z selects A or B. A block handles 32 rows x 64 k
// through shared memory, so that the read (along whichever of row / k is contiguous in src) is
// coalesced; each thread then splits 8 consecutive k of one row and writes three 16-byte vectors.
__global__ void __launch_bounds__(256) split_bf16x3_kernel(const SplitOperand oa, const SplitOperand ob, int K, int64_t ld) {
  __shared__ float tile[32][65];
  grid_dependency_trigger();  // the GEMM behind this kernel may set its CTAs up under the last wave of blocks
  const SplitOperand& o = blockIdx.z == 0 ? oa : ob;
  const int r0 = blockIdx.y * 32, k0 = blockIdx.x * 64;
  if (r0 >= o.rows) return;
  if (o.s_k == 1) {
    // k contiguous: 64 consecutive k of a row per pair of warps
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
    for (int i = ty; i < 32; i += 4) {
      const int r = r0 + i, k = k0 + tx;
      tile[i][tx] = (r < o.rows && k < K) ? o.src[r * o.s_row + k] : 0.f;
    }
  } else {
    // rows contiguous: 32 consecutive rows of one k per warp
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (int i = ty; i < 64; i += 8) {
      const int r = r0 + tx, k = k0 + i;
      tile[tx][i] = (r < o.rows && k < K) ? o.src[r * o.s_row + k * o.s_k] : 0.f;
    }
  }
  __syncthreads();
  const int i = threadIdx.x >> 3, g = threadIdx.x & 7;  // row in the tile, group of 8 k
  const int r = r0 + i, k = k0 + g * 8;
  if (r >= o.rows || k >= K) return;
  __nv_bfloat16 term[3][8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float x = tile[i][g * 8 + e];  // zero beyond K
    const __nv_bfloat16 h = __float2bfloat16_rn(x);
    const float x1 = x - __bfloat162float(h);
    const __nv_bfloat16 m = __float2bfloat16_rn(x1);
    const float x2 = x1 - __bfloat162float(m);
    term[0][e] = h;
    term[1][e] = m;
    term[2][e] = __float2bfloat16_rn(x2);
  }
  // rows are `ld` (a multiple of 8) long, so the whole group of 8 is inside the row
  __nv_bfloat16* out = o.dst + r * ld + k;
  const int64_t term_stride = static_cast<int64_t>(o.rows) * ld;
#pragma unroll
  for (int t = 0; t < 3; ++t) *reinterpret_cast<uint4*>(out + t * term_stride) = *reinterpret_cast<const uint4*>(term[t]);
}

inline int64_t split_ld(int K) { return (static_cast<int64_t>(K) + 7) & ~7ll; }  // rows 16-byte aligned
inline size_t split_operand_bytes(int rows, int K) { return (static_cast<size_t>(rows) * split_ld(K) * 2 * 3 + 255) & ~static_cast<size_t>(255); }

}  // namespace

int gemm_tc_split_f32_supported(const lh_ctx* ctx, const GemmProblem& p) {
  if (ctx->cc_major != 10) return 0;
  if (p.flags & (LH_GEMM_FORCE_SIMT | LH_GEMM_SWIGLU)) return 0;
  if (p.batch != 1) return 0;
  if (p.a_dtype != LH_F32 || p.b_dtype != LH_F32 || p.d_dtype != LH_F32) return 0;
  if (p.M < 1 || p.K < 1 || p.N < 8 || p.N % 8) return 0;
  if (static_cast<int64_t>(p.M) * p.N * p.K < SPLIT_MIN_WORK) return 0;
  if (split_operand_bytes(p.M, p.K) + split_operand_bytes(p.N, p.K) > SPLIT_MAX_SCRATCH) return 0;
  auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  if (p.sdn != 1 || (p.sdm % 4) != 0 || p.sdm < p.N || !aligned16(p.D)) return 0;
  if (p.C && (p.c_dtype != LH_F32 || p.scn != 1 || (p.scm % 4) != 0 || !aligned16(p.C))) return 0;
  if (p.R && (p.r_dtype != LH_F32 || p.srn != 1 || (p.srm % 4) != 0 || !aligned16(p.R))) return 0;
  if (p.bias && ((p.bias_dtype != LH_BF16 && p.bias_dtype != LH_F32) || !aligned16(p.bias))) return 0;
  return 1;
}

size_t gemm_tc_split_f32_scratch_bytes(int M, int N, int K) {
  if (M < 1 || K < 1 || N < 8 || N % 8 || static_cast<int64_t>(M) * N * K < SPLIT_MIN_WORK) return 0;
  const size_t total = split_operand_bytes(M, K) + split_operand_bytes(N, K);
  return total > SPLIT_MAX_SCRATCH ? 0 : total;
}

int gemm_tc_split_f32_launch(lh_ctx* ctx, const GemmProblem& p) {
  const int64_t ld = split_ld(p.K);
  const size_t a_bytes = split_operand_bytes(p.M, p.K), b_bytes = split_operand_bytes(p.N, p.K);
  int rc = ensure_scratch(ctx, a_bytes + b_bytes);
  if (rc) return rc;
  __nv_bfloat16* a3 = static_cast<__nv_bfloat16*>(ctx->scratch);
  __nv_bfloat16* b3 = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ctx->scratch) + a_bytes);
  {
    const SplitOperand oa{static_cast<const float*>(p.A), p.sam, p.sak, p.M, a3};
    const SplitOperand ob{static_cast<const float*>(p.B), p.sbn, p.sbk, p.N, b3};
    const int max_rows = p.M > p.N ? p.M : p.N;
    const dim3 grid((p.K + 63) / 64, (max_rows + 31) / 32, 2);
    split_bf16x3_kernel<<<grid, 256, 0, ctx->stream>>>(oa, ob, p.K, ld);
    LH_CHECK_LAUNCH(ctx, "split_bf16x3_kernel");
  }
  const int sms = ctx->sm_count - ctx->reserved_sms > 0 ? ctx->sm_count - ctx->reserved_sms : 1;
  const int64_t num_m = (p.M + BM - 1) / BM;
  const int64_t tiles128 = num_m * ((p.N + 127) / 128);
  const int nseg = (p.K + SPLIT_SEGMENT - 1) / SPLIT_SEGMENT;
  // 128-wide tiles (two three-term stages of 96 KB) once they fill the GPU, 64-wide ones (two
  // stages of 72 KB, twice the CTAs) below that; four segment accumulators per tile either way,
  // so a k range of 1024 is ONE GEMM launch. The caller's tile hint (bits 8-15 of the flags)
  // overrides the choice.
  const int hint = static_cast<int>((p.flags >> 8) & 0xffu) * 8;
  const int bn = (hint == 64 || hint == 128) ? hint : tiles128 >= sms ? 128 : 64;
  const int per_launch = 4;
  for (int s0 = 0; s0 < nseg; s0 += per_launch) {
    const int s1 = s0 + per_launch < nseg ? s0 + per_launch : nseg;
    const int first = s0 * SPLIT_SEGMENT;
    const int last_k = s1 * SPLIT_SEGMENT < p.K ? s1 * SPLIT_SEGMENT : p.K;
    const bool is_first = s0 == 0, is_last = s1 == nseg;
    GemmProblem q = p;
    q.a_dtype = LH_BF16; q.b_dtype = LH_BF16;
    q.K = last_k - first;
    q.A = a3 + first; q.sam = ld; q.sak = 1;
    q.B = b3 + first; q.sbn = ld; q.sbk = 1;
    EpiParams epi;
    epi.D = p.D; epi.d_dtype = p.d_dtype; epi.ldd = p.sdm;
    // the caller's C enters with the first launch, the running sum (D) with the later ones;
    // bias, activation and residual belong to the last
    epi.C = is_first ? p.C : p.D; epi.c_dtype = LH_F32; epi.ldc = is_first ? p.scm : p.sdm;
    epi.bias = is_last ? p.bias : nullptr; epi.bias_dtype = p.bias_dtype;
    epi.R = is_last ? p.R : nullptr; epi.r_dtype = p.r_dtype; epi.ldr = p.srm;
    epi.act = is_last ? p.act : LH_ACT_NONE;
    epi.swiglu = 0;
    epi.rope_table = nullptr; epi.rope_cols = 0; epi.rope_dim = 0; epi.rope_seq = 0;
    const int seg_k_blocks = SPLIT_SEGMENT / BK;
    const int64_t ts_a = static_cast<int64_t>(p.M) * ld, ts_b = static_cast<int64_t>(p.N) * ld;
    // (always a programmatic dependent: what precedes it in the stream is this call's own split
    // kernel or previous segment launch, and its set-up is a third of a 1024^3 product's time)
    rc = bn == 128 ? launch_variant<128, true, 2, true, 4, 3>(ctx, q, epi, seg_k_blocks, ts_a, ts_b, true)
                   : launch_variant<64, true, 2, true, 4, 3>(ctx, q, epi, seg_k_blocks, ts_a, ts_b, true);
    if (rc) return rc;
  }
  return LH_OK;
}

}  // namespace lh
