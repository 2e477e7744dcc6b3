// Flash-attention forward, one query tile per CTA, P kept in tensor memory.
//
// Online softmax of replace_with_fused_attention.py:334-455 in the reference: f32 scores /
// max / sum / accumulator, P rounded to bf16 before P.V, O = acc / l. The data path:
//   * the softmax warps write P (bf16 pairs) back into the tensor-memory columns the scores
//     came from, and the second MMA reads its A operand from tensor memory, so P never
//     crosses shared memory and the P.V product loads only V from it;
//   * scores are read from tensor memory twice (row max, then exponentials), which keeps the
//     softmax threads under 128 registers;
//   * K and V each have one shared-memory buffer released separately (K when Q K^T has
//     finished, V when P V has), 96 KB per CTA at head_dim 128, and a CTA uses 256 of the
//     512 tensor-memory columns, so TWO CTAs share an SM: while one CTA's softmax runs, the
//     other CTA's MMAs keep the tensor pipe busy.
// One CTA per (batch, query head, 128 query rows); warp 0 TMA, warp 1 MMA issue, warps 2-5
// softmax (one row per thread). All waits are bounded.
#include "common.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"

namespace lh {

namespace {

constexpr int BQ2 = 128;
constexpr int BKV2 = 128;
constexpr int ATT2_THREADS = 192;
constexpr int SUBTILE2 = 128 * 128;  // 128 rows x 64 bf16

struct Attn2Params {
  int B, Hq, Hkv, Sq, Skv;
  void* O;
  int o_dtype;
  int64_t sob, soh, sos;
  float scale_log2;
  int causal;
  int num_q_tiles;
  int pair_slots;  // causal: blocks below this count are placed one per SM first (0: plain order)
  int* dev_status;
};

template <int HD>
struct Attn2Smem {
  static constexpr int Q_BYTES = BQ2 * HD * 2;
  static constexpr int KV_BYTES = BKV2 * HD * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;
  static constexpr int V_OFF = K_OFF + KV_BYTES;
  static constexpr int BAR_OFF = V_OFF + KV_BYTES;
  static constexpr int NUM_BARS = 9;
  static constexpr int DYN_BYTES = BAR_OFF + NUM_BARS * 8 + 16 + 1024;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ bool wait_warp2(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* dev_status,
                                           int code, int lane) {
  // every lane observes the phase itself (its later reads are ordered after it); the warp
  // agrees on the verdict so that a timeout never splits it
  (void)lane;
  const bool ok = mbar_wait(bar, parity, abort_flag, dev_status, code);
  return __all_sync(0xffffffffu, ok);
}

template <int HD>
__global__ void __launch_bounds__(ATT2_THREADS, 2)
attn_fwd_tc2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const Attn2Params p) {
  using L = Attn2Smem<HD>;
  constexpr int TMEM_COLS = 256;
  constexpr uint32_t S_COL = 0, O_COL = 128;  // P (bf16 pairs) overwrites S columns [0, 64)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 2;
  uint64_t* v_full = bars + 3;
  uint64_t* v_empty = bars + 4;
  uint64_t* s_full = bars + 5;
  uint64_t* p_half = bars + 6;  // [2]: keys [0,64) of P written / keys [64,128) written
  uint64_t* pv_done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Work order. A causal query tile qt visits qt + 1 key tiles, so tiles are handed out
  // heaviest first (every (batch, head) of the last tile, then of the one before, ...): late
  // blocks are short and the tail of the grid is too. When the whole grid is resident at once
  // (two blocks per SM), the second block of each SM instead comes from the light end, so
  // that a long block shares its SM with a short one and has it alone for most of its run.
  int bh, qt;
  if (p.causal) {
    const int total = gridDim.x, nbh = total / p.num_q_tiles;
    int r = blockIdx.x;
    if (p.pair_slots > 0 && r >= p.pair_slots) r = total - 1 - (r - p.pair_slots);
    qt = p.num_q_tiles - 1 - r / nbh;
    bh = r % nbh;
  } else {
    bh = blockIdx.x / p.num_q_tiles;
    qt = blockIdx.x % p.num_q_tiles;
  }
  const int b = bh / p.Hq;
  const int hq = bh % p.Hq;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int q0 = qt * BQ2;
  const int offset = p.Skv - p.Sq;
  int n_kv = (p.Skv + BKV2 - 1) / BKV2;
  if (p.causal) {
    const int last_col = min(q0 + BQ2 - 1 + offset, p.Skv - 1);
    n_kv = min(n_kv, max(last_col, 0) / BKV2 + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(&p_half[0], 128);
    mbar_init(&p_half[1], 128);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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
      mbar_arrive_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int h = 0; h < HD / 64; ++h) tma_load_4d(smem + L::Q_OFF + h * SUBTILE2, &tmQ, q_full, h * 64, q0, hq, b);
      for (int j = 0; j < n_kv; ++j) {
        const uint32_t ph = j & 1u;
        if (!mbar_wait(k_empty, ph ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(k_full, L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) tma_load_4d(smem + L::K_OFF + h * SUBTILE2, &tmK, k_full, h * 64, j * BKV2, hkv, b);
        if (!mbar_wait(v_empty, ph ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(v_full, L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) tma_load_4d(smem + L::V_OFF + h * SUBTILE2, &tmV, v_full, h * 64, j * BKV2, hkv, b);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(UMMA_BF16, BQ2, BKV2, false, false);
      constexpr uint32_t idesc_pv = make_idesc(UMMA_BF16, BQ2, HD, false, true);
      const uint32_t q_addr = smem_u32(smem + L::Q_OFF);
      const uint32_t k_addr = smem_u32(smem + L::K_OFF);
      const uint32_t v_addr = smem_u32(smem + L::V_OFF);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.dev_status, DEV_TIMEOUT_MMA);
      for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t ph = j & 1u;
        // S_j = Q K_j^T (overwrites the columns P_{j-1} lived in; P_{j-1} V_{j-1} has completed)
        if (!mbar_wait(k_full, ph, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k / 4) * SUBTILE2 + (k % 4) * 32;
          umma_f16_ss(tmem_base + S_COL, make_smem_desc_sw128(q_addr + off, 16, 1024), make_smem_desc_sw128(k_addr + off, 16, 1024),
                      idesc_qk, k != 0 ? 1u : 0u);
        }
        umma_commit(k_empty);
        umma_commit(s_full);
        // O += P_j V_j with P_j read from tensor memory
        if (!mbar_wait(v_full, ph, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) break;
        // the first 64 keys of P are consumed while the softmax warps still produce the rest
        bool half_ok = true;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          if (!mbar_wait(&p_half[hf], ph, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) {
            half_ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int k = hf * 4; k < hf * 4 + 4; ++k) {
            // 16 keys of P = 8 packed columns; V rows are keys, 64 head-dim elements per 128-byte row
            umma_f16_ts(tmem_base + O_COL, tmem_base + S_COL + k * 8, make_smem_desc_sw128(v_addr + k * 2048, SUBTILE2, 1024), idesc_pv,
                        (j | k) != 0 ? 1u : 0u);
          }
        }
        if (!half_ok) break;
        umma_commit(v_empty);
        umma_commit(pv_done);
        // The next Q K^T overwrites the columns this product reads P from; the two MMAs use
        // different accumulators, so wait for this one instead of relying on issue order.
        if (j + 1 < n_kv && !mbar_wait(pv_done, ph, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) break;
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int q_row = q0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + S_COL + lane_off;
    const uint32_t o_addr = tmem_base + O_COL + lane_off;
    float m_used = -INFINITY;
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!wait_warp2(s_full, j & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_SOFTMAX, lane)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int col0 = j * BKV2;
      const bool need_mask = (col0 + BKV2 > p.Skv) || (p.causal && (col0 + BKV2 - 1 > q0 + offset));
      const int limit = need_mask ? (p.causal ? min(p.Skv - 1, q_row + offset) : (p.Skv - 1)) - col0 : BKV2;  // last visible column in this tile
      // pass 1: row max of the scores
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;  // independent chains
#pragma unroll
      for (int c = 0; c < 4; c += 2) {
        uint32_t s0[32], s1[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, s0);
        tmem_ld_32x32b_x32(s_addr + c * 32 + 32, s1);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (c * 32 + i > limit) s0[i] = 0xff800000u;  // -inf
            if (c * 32 + 32 + i > limit) s1[i] = 0xff800000u;
          }
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          mx0 = fmaxf(mx0, __uint_as_float(s0[i]));
          mx1 = fmaxf(mx1, __uint_as_float(s0[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(s1[i]));
          mx3 = fmaxf(mx3, __uint_as_float(s1[i + 1]));
        }
      }
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      mx *= p.scale_log2;  // scale > 0: max commutes with the scaling
      // lazy rescale: move the reference max only when it grew by more than 8 (2^8 headroom)
      float alpha = 1.f;
      const bool need = (mx > m_used + 8.f) || (m_used == -INFINITY && mx > -INFINITY);
      if (need) {
        alpha = (m_used == -INFINITY) ? 0.f : ex2(m_used - mx);
        m_used = mx;
      }
      const bool warp_need = __any_sync(0xffffffffu, need);
      if (j > 0 && warp_need) {
        // s_full(j) fired after every earlier MMA, P_{j-1} V_{j-1} included: O is up to date
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(o_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32b_x32(o_addr + c * 32, o);
        }
      }
      // pass 2: P = exp2(scale*S - m), row sum, bf16 pairs written over the S columns; each
      // half (64 keys) is handed to the MMA warp as soon as it is in tensor memory
      const float msub = (m_used == -INFINITY) ? 0.f : m_used;
      float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t s0[32], s1[32];
        tmem_ld_32x32b_x32(s_addr + hf * 64, s0);
        tmem_ld_32x32b_x32(s_addr + hf * 64 + 32, s1);
        tmem_ld_wait();
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2(fmaf(__uint_as_float(s0[2 * i]), p.scale_log2, -msub));
          float p1 = ex2(fmaf(__uint_as_float(s0[2 * i + 1]), p.scale_log2, -msub));
          float p2 = ex2(fmaf(__uint_as_float(s1[2 * i]), p.scale_log2, -msub));
          float p3 = ex2(fmaf(__uint_as_float(s1[2 * i + 1]), p.scale_log2, -msub));
          if (need_mask) {
            const int cbase = hf * 64 + 2 * i;
            p0 = (cbase <= limit) ? p0 : 0.f;
            p1 = (cbase + 1 <= limit) ? p1 : 0.f;
            p2 = (cbase + 32 <= limit) ? p2 : 0.f;
            p3 = (cbase + 33 <= limit) ? p3 : 0.f;
          }
          rs0 += p0;
          rs1 += p1;
          rs2 += p2;
          rs3 += p3;
          pk[i] = pack_bf16x2(p0, p1);
          pk[16 + i] = pack_bf16x2(p2, p3);
        }
        tmem_st_32x32b_x32(s_addr + hf * 32, pk);
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(&p_half[hf]);
      }
      l = l * alpha + ((rs0 + rs1) + (rs2 + rs3));
    }
    if (ok && wait_warp2(pv_done, (n_kv - 1) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_SOFTMAX, lane)) {
      tc_fence_after_sync();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      char* obase = static_cast<char*>(p.O);
      const int64_t oidx = static_cast<int64_t>(b) * p.sob + static_cast<int64_t>(hq) * p.soh + static_cast<int64_t>(q_row) * p.sos;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(o_addr + c * 32, o);
        tmem_ld_wait();
        if (q_row < p.Sq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(o[g * 8 + i]) * inv_l;
            store8_from_f32(obase, p.o_dtype, oidx + c * 32 + g * 8, v);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if (*abort_flag) {
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int HD>
int launch2_hd(lh_ctx* ctx, const AttnProblem& a) {
  using L = Attn2Smem<HD>;
  CUtensorMap tmQ, tmK, tmV;
  const uint32_t box[4] = {64, 128, 1, 1};
  {
    const uint64_t dims[4] = {(uint64_t)a.D, (uint64_t)a.Sq, (uint64_t)a.Hq, (uint64_t)a.B};
    const uint64_t st[3] = {(uint64_t)a.sqs * 2, (uint64_t)a.sqh * 2, (uint64_t)a.sqb * 2};
    int rc = encode_tensor_map(ctx, &tmQ, LH_BF16, 4, const_cast<void*>(a.Q), dims, st, box, 1);
    if (rc) return rc;
  }
  {
    const uint64_t dims[4] = {(uint64_t)a.D, (uint64_t)a.Skv, (uint64_t)a.Hkv, (uint64_t)a.B};
    const uint64_t stk[3] = {(uint64_t)a.sks * 2, (uint64_t)a.skh * 2, (uint64_t)a.skb * 2};
    const uint64_t stv[3] = {(uint64_t)a.svs * 2, (uint64_t)a.svh * 2, (uint64_t)a.svb * 2};
    int rc = encode_tensor_map(ctx, &tmK, LH_BF16, 4, const_cast<void*>(a.K), dims, stk, box, 1);
    if (rc) return rc;
    rc = encode_tensor_map(ctx, &tmV, LH_BF16, 4, const_cast<void*>(a.V), dims, stv, box, 1);
    if (rc) return rc;
  }
  Attn2Params p;
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Sq = a.Sq; p.Skv = a.Skv;
  p.O = a.O; p.o_dtype = a.o_dtype; p.sob = a.sob; p.soh = a.soh; p.sos = a.sos;
  p.scale_log2 = a.scale * 1.44269504088896340736f;
  p.causal = a.causal;
  p.num_q_tiles = (a.Sq + BQ2 - 1) / BQ2;
  p.dev_status = ctx->dev_status;
  auto kernel = attn_fwd_tc2_kernel<HD>;
  LH_CUDA_CHECK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
  const int64_t grid = static_cast<int64_t>(a.B) * a.Hq * p.num_q_tiles;
  p.pair_slots = (grid > ctx->sm_count && grid <= 2 * static_cast<int64_t>(ctx->sm_count)) ? ctx->sm_count : 0;
  kernel<<<static_cast<unsigned>(grid), ATT2_THREADS, L::DYN_BYTES, ctx->stream>>>(tmQ, tmK, tmV, p);
  LH_CHECK_LAUNCH(ctx, "attn_fwd_tc2_kernel");
  return LH_OK;
}

}  // namespace

int attn_tc2_launch(lh_ctx* ctx, const AttnProblem& a) {
  if (a.scale <= 0.f) return set_error(ctx, LH_ERR_UNSUPPORTED, "attention: scale must be positive");
  if (a.D == 128) return launch2_hd<128>(ctx, a);
  return launch2_hd<64>(ctx, a);
}

}  // namespace lh
