// Flash-attention forward on the sm_100a tensor cores.
//
// The algorithm is the online-softmax loop the reference emits as IR in
// ReplaceWithFusedAttentionOp
// (lighthouse/dialects/transform/transform_ext/ops/replace_with_fused_attention.py:334-455):
// per 128-row query tile, for each 128-row key/value tile: S = Q K^T (f32), running
// row max m and row sum l in f32, P = exp(scale S - m) rounded to bf16, acc += P V
// in f32, and at the end O = acc / l rounded to the output type. Causal masking and
// grouped-query head mapping follow examples/xegpu/nanoGPT.py:95-111 and
// examples/llama/ref_model.py:100-111,266-278.
//
// One CTA per (batch, query head, 128 query rows), 192 threads:
//   warp 0     TMA producer: Q once, then K/V tiles into a 2-deep ring
//   warp 1     MMA issuer: S_j = Q K_j^T into one of two S buffers in tensor memory
//              (so S_{j+1} is computed while the softmax of S_j runs), then
//              O += P_j V_j with O resident in tensor memory
//   warps 2-5  softmax: one query row per thread; read S from tensor memory, update
//              m and l, write P as bf16 into shared memory in the swizzled operand
//              layout, rescale O in tensor memory only when the running max moved by
//              more than 2^8 (the final division by l absorbs the stale scale)
// All waits are bounded; a wait that runs out raises the status word.
#include "common.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"

namespace lh {

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int KV_STAGES = 2;
constexpr int ATT_THREADS = 192;
constexpr int SUBTILE_BYTES = 128 * 128;  // 128 rows x 64 bf16 (one 128-byte swizzle row each)

struct AttnTcParams {
  int B, Hq, Hkv, Sq, Skv;
  void* O;
  int o_dtype;
  int64_t sob, soh, sos;
  float scale_log2;  // scale * log2(e)
  int causal;
  int num_q_tiles;
  int* dev_status;
};

template <int HD>
struct AttnSmem {
  static constexpr int Q_BYTES = BQ * HD * 2;
  static constexpr int KV_BYTES = BKV * HD * 2;  // one of K or V
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * KV_BYTES;
  static constexpr int P_OFF = V_OFF + KV_STAGES * KV_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int NUM_BARS = 1 + 3 * KV_STAGES + 2 + 2 + 2;
  static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ bool wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
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

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const AttnTcParams p) {
  using L = AttnSmem<HD>;
  constexpr int TMEM_COLS = 512;
  constexpr uint32_t S_COL0 = 0, S_COL1 = 128, O_COL = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 1;               // [KV_STAGES]
  uint64_t* v_full = k_full + KV_STAGES;       // [KV_STAGES]
  uint64_t* kv_empty = v_full + KV_STAGES;     // [KV_STAGES]
  uint64_t* s_full = kv_empty + KV_STAGES;     // [2]
  uint64_t* s_free = s_full + 2;               // [2]
  uint64_t* p_full = s_free + 2;               // [1]
  uint64_t* pv_done = p_full + 1;              // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Work item: consecutive CTAs share a (batch, head); longest causal rows first.
  const int bh = blockIdx.x / p.num_q_tiles;
  const int qt = p.num_q_tiles - 1 - (blockIdx.x % p.num_q_tiles);
  const int b = bh / p.Hq;
  const int hq = bh % p.Hq;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int q0 = qt * BQ;
  const int offset = p.Skv - p.Sq;  // causal: key j visible to query i iff j <= i + offset
  int n_kv = (p.Skv + BKV - 1) / BKV;
  if (p.causal) {
    const int last_col = min(q0 + BQ - 1 + offset, p.Skv - 1);
    n_kv = min(n_kv, max(last_col, 0) / BKV + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 128);
    }
    mbar_init(p_full, 128);
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
      for (int h = 0; h < HD / 64; ++h)
        tma_load_4d(smem + L::Q_OFF + h * SUBTILE_BYTES, &tmQ, q_full, h * 64, q0, hq, b);
      for (int j = 0; j < n_kv; ++j) {
        const int stage = j % KV_STAGES;
        const uint32_t phase = (j / KV_STAGES) & 1u;
        if (!mbar_wait(&kv_empty[stage], phase ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(&k_full[stage], L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h)
          tma_load_4d(smem + L::K_OFF + stage * L::KV_BYTES + h * SUBTILE_BYTES, &tmK, &k_full[stage], h * 64,
                      j * BKV, hkv, b);
        mbar_arrive_expect_tx(&v_full[stage], L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h)
          tma_load_4d(smem + L::V_OFF + stage * L::KV_BYTES + h * SUBTILE_BYTES, &tmV, &v_full[stage], h * 64,
                      j * BKV, hkv, b);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(UMMA_BF16, BQ, BKV, false, false);
      constexpr uint32_t idesc_pv = make_idesc(UMMA_BF16, BQ, HD, false, true);
      const uint32_t q_addr = smem_u32(smem + L::Q_OFF);
      const uint32_t p_addr = smem_u32(smem + L::P_OFF);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.dev_status, DEV_TIMEOUT_MMA);
      auto issue_qk = [&](int j) -> bool {
        const int stage = j % KV_STAGES;
        const uint32_t phase = (j / KV_STAGES) & 1u;
        const int sb = j & 1;
        if (!mbar_wait(&k_full[stage], phase, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) return false;
        if (!mbar_wait(&s_free[sb], ((j >> 1) & 1u) ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + L::K_OFF + stage * L::KV_BYTES);
        const uint32_t d_tmem = tmem_base + (sb ? S_COL1 : S_COL0);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k / 4) * SUBTILE_BYTES + (k % 4) * 32;
          umma_f16_ss(d_tmem, make_smem_desc_sw128(q_addr + off, 16, 1024),
                      make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          if (!issue_qk(j + 1)) break;
        }
        const int stage = j % KV_STAGES;
        const uint32_t phase = (j / KV_STAGES) & 1u;
        if (!mbar_wait(&v_full[stage], phase, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) break;
        if (!mbar_wait(p_full, j & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) break;
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(smem + L::V_OFF + stage * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint32_t a_off = (k / 4) * SUBTILE_BYTES + (k % 4) * 32;
          // V tile: rows are keys (the MMA's K), 64 head-dim elements per 128-byte row.
          umma_f16_ss(tmem_base + O_COL, make_smem_desc_sw128(p_addr + a_off, 16, 1024),
                      make_smem_desc_sw128(v_addr + k * 2048, SUBTILE_BYTES, 1024), idesc_pv,
                      (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&kv_empty[stage]);
        umma_commit(pv_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int q_row = q0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    float m_used = -INFINITY;
    float l = 0.f;
    bool ok = true;
    uint8_t* sP = smem + L::P_OFF;
    for (int j = 0; j < n_kv; ++j) {
      const int sb = j & 1;
      if (!wait_warp(&s_full[sb], (j >> 1) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_SOFTMAX, lane)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t s[128];
      {
        const uint32_t ta = tmem_base + (sb ? S_COL1 : S_COL0) + lane_off;
        uint32_t(&s0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
        uint32_t(&s1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[32]);
        uint32_t(&s2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[64]);
        uint32_t(&s3)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[96]);
        tmem_ld_32x32b_x32(ta, s0);
        tmem_ld_32x32b_x32(ta + 32, s1);
        tmem_ld_32x32b_x32(ta + 64, s2);
        tmem_ld_32x32b_x32(ta + 96, s3);
        tmem_ld_wait();
      }
      tc_fence_before_sync();
      mbar_arrive(&s_free[sb]);

      const int col0 = j * BKV;
      const bool need_mask = (col0 + BKV > p.Skv) || (p.causal && (col0 + BKV - 1 > q0 + offset));
      float mx = -INFINITY;
      if (need_mask) {
        const int limit = p.causal ? min(p.Skv - 1, q_row + offset) : (p.Skv - 1);
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          float v = __uint_as_float(s[i]) * p.scale_log2;
          v = (col0 + i <= limit) ? v : -INFINITY;
          s[i] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const float v = __uint_as_float(s[i]) * p.scale_log2;
          s[i] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      }
      // Lazy rescale: move the reference max only when it grew by more than 8 (2^8 headroom).
      float alpha = 1.f;
      const bool need = (mx > m_used + 8.f) || (m_used == -INFINITY && mx > -INFINITY);
      if (need) {
        alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - mx);
        m_used = mx;
      }
      const bool warp_need = __any_sync(0xffffffffu, need);
      const float msub = (m_used == -INFINITY) ? 0.f : m_used;
      float rowsum = 0.f;
      uint32_t pk[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const float p0 = fast_exp2(__uint_as_float(s[2 * i]) - msub);
        const float p1 = fast_exp2(__uint_as_float(s[2 * i + 1]) - msub);
        rowsum += p0 + p1;
        pk[i] = pack_bf16x2(p0, p1);
      }
      l = l * alpha + rowsum;

      if (j > 0) {
        if (!wait_warp(pv_done, (j - 1) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_SOFTMAX, lane)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (warp_need) {
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(tmem_base + O_COL + c * 32 + lane_off, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(tmem_base + O_COL + c * 32 + lane_off, o);
          }
          tmem_st_wait();
        }
      }
      // P row -> shared memory, K-major 128-byte-swizzled operand layout:
      // 16-byte chunk c of row r lives at r*128 + ((c ^ (r & 7)) * 16) inside its 64-column sub-tile.
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint32_t off = (c >> 3) * SUBTILE_BYTES + row * 128 + (((c & 7) ^ (row & 7)) << 4);
        *reinterpret_cast<uint4*>(sP + off) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_full);
    }
    if (ok && wait_warp(pv_done, (n_kv - 1) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_SOFTMAX, lane)) {
      tc_fence_after_sync();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      char* obase = static_cast<char*>(p.O);
      const int64_t oidx = static_cast<int64_t>(b) * p.sob + static_cast<int64_t>(hq) * p.soh +
                           static_cast<int64_t>(q_row) * p.sos;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_base + O_COL + c * 32 + lane_off, o);
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
int launch_hd(lh_ctx* ctx, const AttnProblem& a) {
  using L = AttnSmem<HD>;
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
  AttnTcParams p;
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Sq = a.Sq; p.Skv = a.Skv;
  p.O = a.O; p.o_dtype = a.o_dtype; p.sob = a.sob; p.soh = a.soh; p.sos = a.sos;
  p.scale_log2 = a.scale * 1.44269504088896340736f;
  p.causal = a.causal;
  p.num_q_tiles = (a.Sq + BQ - 1) / BQ;
  p.dev_status = ctx->dev_status;
  auto kernel = attn_fwd_tc_kernel<HD>;
  LH_CUDA_CHECK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
  const int64_t grid = static_cast<int64_t>(a.B) * a.Hq * p.num_q_tiles;
  kernel<<<static_cast<unsigned>(grid), ATT_THREADS, L::DYN_BYTES, ctx->stream>>>(tmQ, tmK, tmV, p);
  LH_CHECK_LAUNCH(ctx, "attn_fwd_tc_kernel");
  return LH_OK;
}

}  // namespace

int attn_tc_supported(const lh_ctx* ctx, const AttnProblem& a) {
  if (ctx->cc_major != 10) return 0;
  if (a.dtype != LH_BF16) return 0;
  if (a.o_dtype != LH_BF16 && a.o_dtype != LH_F32) return 0;
  if (a.D != 64 && a.D != 128) return 0;
  if (a.Hkv < 1 || a.Hq % a.Hkv) return 0;
  if (a.causal && a.Skv < a.Sq) return 0;
  auto ok8 = [](int64_t s) { return (s % 8) == 0; };
  if (!ok8(a.sqb) || !ok8(a.sqh) || !ok8(a.sqs) || !ok8(a.skb) || !ok8(a.skh) || !ok8(a.sks) || !ok8(a.svb) ||
      !ok8(a.svh) || !ok8(a.svs) || !ok8(a.sob) || !ok8(a.soh) || !ok8(a.sos))
    return 0;
  auto al = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  if (!al(a.Q) || !al(a.K) || !al(a.V) || !al(a.O)) return 0;
  if (static_cast<int64_t>(a.B) * a.Hq * ((a.Sq + BQ - 1) / BQ) > 0x7fffffffLL) return 0;
  return 1;
}

int attn_tc_launch(lh_ctx* ctx, const AttnProblem& a) {
  // Default: the kernel that keeps P in tensor memory (attention_tc2.cu). This file's kernel
  // (P through shared memory, one CTA per SM) stays selectable for comparison.
  const char* v1 = getenv("LH_B200_ATTN_V1");
  if (!(v1 && v1[0] == '1') && a.scale > 0.f) return attn_tc2_launch(ctx, a);
  if (a.D == 128) return launch_hd<128>(ctx, a);
  return launch_hd<64>(ctx, a);
}

}  // namespace lh
