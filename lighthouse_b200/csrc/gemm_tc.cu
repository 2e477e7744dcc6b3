// bf16 GEMM with fused epilogue on the sm_100a tensor cores.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer: fills a STAGES-deep ring of {A 128x64, B BNx64} bf16
//               tiles in shared memory (128-byte swizzle)
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) into one
//               of two f32 accumulators in tensor memory, so the epilogue of tile t
//               overlaps the main loop of tile t+1
//   warps 2-5   epilogue: tcgen05.ld the accumulator (one row per thread), add
//               C / bias, activation, residual, round, 16-byte global stores
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
constexpr int GROUP_M = 16;                 // tile rasterisation: 16 row-blocks share B column-blocks in L2

struct GemmTcParams {
  int M, N, K;
  int num_m_blocks, num_n_blocks, num_k_blocks;
  EpiParams epi;
  int* dev_status;
};

__host__ __device__ constexpr int tmem_cols_for(int bn) {
  return (2 * bn <= 32) ? 32 : (2 * bn <= 64) ? 64 : (2 * bn <= 128) ? 128 : (2 * bn <= 256) ? 256 : 512;
}

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int B_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack for the 1024-byte alignment of the ring
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int group_size = GROUP_M * num_n;
  const int group = tile / group_size;
  const int first_m = group * GROUP_M;
  const int rows = min(num_m - first_m, GROUP_M);
  const int in_group = tile - group * group_size;
  m_blk = first_m + in_group % rows;
  n_blk = in_group / rows;
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

template <int BN, bool B_KMAJOR, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmTcParams p) {
  using L = SmemLayout<BN, STAGES>;
  constexpr int TMEM_COLS = tmem_cols_for(BN);
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
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;

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
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, p.num_m_blocks, p.num_n_blocks, m_blk, n_blk);
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * L::STAGE_BYTES;
          uint8_t* sB = sA + A_TILE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, m_blk * BM);
          if (B_KMAJOR) {
            tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, n_blk * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sB + j * (64 * BK * 2), &tmB, &full_bar[stage], n_blk * BN + j * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(UMMA_BF16, BM, BN, false, !B_KMAJOR);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int t = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
        const int buf = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_KMAJOR ? make_smem_desc_sw128(b_addr + k * 32, 16, 1024)
                                            : make_smem_desc_sw128(b_addr + k * 2048, 64 * BK * 2, 1024);
            umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(&tmem_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // tensor-memory lanes [32*quarter, +32) belong to this warp
    const EpiParams& e = p.epi;
    int t = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      int m_blk, n_blk;
      tile_coords(tile, p.num_m_blocks, p.num_n_blocks, m_blk, n_blk);
      const int buf = t & 1;
      const uint32_t acc_phase = (t >> 1) & 1u;
      if (!mbar_wait_warp(&tmem_full[buf], acc_phase, abort_flag, p.dev_status, DEV_TIMEOUT_EPILOGUE, lane))
        break;
      tc_fence_after_sync();
      const int row = m_blk * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (!e.swiglu) {
#pragma unroll 1
        for (int chunk = 0; chunk < BN / 32; ++chunk) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + chunk * 32, r);
          tmem_ld_wait();
          const int col0 = n_blk * BN + chunk * 32;
          if (row < p.M) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int c = col0 + g * 8;
              if (c < p.N) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]);
                if (e.C) {
                  float cv[8];
                  load8_as_f32(e.C, e.c_dtype, static_cast<int64_t>(row) * e.ldc + c, cv);
#pragma unroll
                  for (int i = 0; i < 8; ++i) v[i] += cv[i];
                }
                if (e.bias) {
                  float bv[8];
                  load8_as_f32(e.bias, e.bias_dtype, c, bv);
#pragma unroll
                  for (int i = 0; i < 8; ++i) v[i] += bv[i];
                }
                if (e.act != LH_ACT_NONE) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) v[i] = apply_act(v[i], e.act);
                }
                if (e.R) {
                  float rv[8];
                  load8_as_f32(e.R, e.r_dtype, static_cast<int64_t>(row) * e.ldr + c, rv);
#pragma unroll
                  for (int i = 0; i < 8; ++i) v[i] += rv[i];
                }
                store8_from_f32(e.D, e.d_dtype, static_cast<int64_t>(row) * e.ldd + c, v);
              }
            }
          }
        }
      } else {
        // B columns of this tile are [gate(BN/2) | up(BN/2)]; D has N/2 columns.
        constexpr int HALF = BN / 2;
#pragma unroll 1
        for (int chunk = 0; chunk < HALF / 32; ++chunk) {
          uint32_t g_[32], u_[32];
          tmem_ld_32x32b_x32(taddr + chunk * 32, g_);
          tmem_ld_32x32b_x32(taddr + HALF + chunk * 32, u_);
          tmem_ld_wait();
          const int col0 = n_blk * HALF + chunk * 32;
          if (row < p.M) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int c = col0 + g * 8;
              if (c < p.N / 2) {
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float gate = __uint_as_float(g_[g * 8 + i]);
                  const float up = __uint_as_float(u_[g * 8 + i]);
                  v[i] = apply_act(gate, LH_ACT_SILU) * up;
                }
                store8_from_f32(e.D, e.d_dtype, static_cast<int64_t>(row) * e.ldd + c, v);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tmem_empty[buf]);
    }
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

template <int BN, bool B_KMAJOR, int STAGES>
int launch_variant(lh_ctx* ctx, const GemmProblem& pr, const EpiParams& epi) {
  using L = SmemLayout<BN, STAGES>;
  CUtensorMap tmA, tmB;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(pr.K), static_cast<uint64_t>(pr.M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(pr.sam) * 2};
    const uint32_t box[2] = {BK, BM};
    int rc = encode_tensor_map(ctx, &tmA, LH_BF16, 2, const_cast<void*>(pr.A), dims, strides, box, 1);
    if (rc) return rc;
  }
  if (B_KMAJOR) {  // B(k,n) with unit k stride: a row-major (N,K) array
    const uint64_t dims[2] = {static_cast<uint64_t>(pr.K), static_cast<uint64_t>(pr.N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(pr.sbn) * 2};
    const uint32_t box[2] = {BK, BN};
    int rc = encode_tensor_map(ctx, &tmB, LH_BF16, 2, const_cast<void*>(pr.B), dims, strides, box, 1);
    if (rc) return rc;
  } else {  // B(k,n) with unit n stride: a row-major (K,N) array
    const uint64_t dims[2] = {static_cast<uint64_t>(pr.N), static_cast<uint64_t>(pr.K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(pr.sbk) * 2};
    const uint32_t box[2] = {64, BK};
    int rc = encode_tensor_map(ctx, &tmB, LH_BF16, 2, const_cast<void*>(pr.B), dims, strides, box, 1);
    if (rc) return rc;
  }
  GemmTcParams p;
  p.M = pr.M;
  p.N = pr.N;
  p.K = pr.K;
  p.num_m_blocks = (pr.M + BM - 1) / BM;
  p.num_n_blocks = (pr.N + BN - 1) / BN;
  p.num_k_blocks = (pr.K + BK - 1) / BK;
  p.epi = epi;
  p.dev_status = ctx->dev_status;
  auto kernel = gemm_bf16_tc_kernel<BN, B_KMAJOR, STAGES>;
  LH_CUDA_CHECK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;
  const int grid = num_tiles < ctx->sm_count ? num_tiles : ctx->sm_count;
  kernel<<<grid, NUM_THREADS, L::DYN_BYTES, ctx->stream>>>(tmA, tmB, p);
  LH_CHECK_LAUNCH(ctx, "gemm_bf16_tc_kernel");
  return LH_OK;
}

int pick_bn(const lh_ctx* ctx, const GemmProblem& p) {
  if (p.flags & LH_GEMM_SWIGLU) return 256;
  static const char* env = getenv("LH_B200_GEMM_BN");
  if (env) {
    const int v = atoi(env);
    if (v == 64 || v == 128 || v == 192 || v == 256) return v;
  }
  // Cost model: waves of tiles over the SMs times the per-tile time; narrower tiles
  // re-read A more often per flop, which the relative efficiencies account for.
  const int cand[3] = {256, 192, 128};
  const double eff[3] = {1.0, 0.97, 0.86};
  const int num_m = (p.M + BM - 1) / BM;
  int best = 256;
  double best_cost = 1e300;
  for (int i = 0; i < 3; ++i) {
    const int bn = cand[i];
    const int64_t tiles = static_cast<int64_t>(num_m) * ((p.N + bn - 1) / bn);
    const int64_t waves = (tiles + ctx->sm_count - 1) / ctx->sm_count;
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
  // Epilogue operands use 8-element vectors.
  if (p.d_dtype != LH_BF16 && p.d_dtype != LH_F32) return 0;
  if (p.sdn != 1 || (p.sdm % 8) != 0 || p.sdm < n_out || !aligned16(p.D)) return 0;
  if (p.C) {
    if (p.c_dtype != LH_BF16 && p.c_dtype != LH_F32) return 0;
    if (p.scn != 1 || (p.scm % 8) != 0 || !aligned16(p.C)) return 0;
  }
  if (p.R) {
    if (p.r_dtype != LH_BF16 && p.r_dtype != LH_F32) return 0;
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
  epi.act = p.act;
  epi.swiglu = (p.flags & LH_GEMM_SWIGLU) ? 1 : 0;
  const bool b_kmajor = (p.sbk == 1 && p.N > 1 && p.sbn >= p.K);
  const int bn = pick_bn(ctx, p);
  if (b_kmajor) {
    switch (bn) {
      case 256: return launch_variant<256, true, 4>(ctx, p, epi);
      case 192: return launch_variant<192, true, 5>(ctx, p, epi);
      case 128: return launch_variant<128, true, 6>(ctx, p, epi);
      default: return launch_variant<64, true, 8>(ctx, p, epi);
    }
  } else {
    switch (bn) {
      case 256: return launch_variant<256, false, 4>(ctx, p, epi);
      case 192: return launch_variant<192, false, 5>(ctx, p, epi);
      case 128: return launch_variant<128, false, 6>(ctx, p, epi);
      default: return launch_variant<64, false, 8>(ctx, p, epi);
    }
  }
}

int gemm_tc_tf32x3_supported(const lh_ctx*, const GemmProblem&) { return 0; }
int gemm_tc_tf32x3_launch(lh_ctx* ctx, const GemmProblem&) {
  return set_error(ctx, LH_ERR_UNSUPPORTED, "3xTF32 tensor-core GEMM is not built");
}

}  // namespace lh
