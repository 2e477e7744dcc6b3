// Flash-attention forward: two query tiles per CTA in explicit ping-pong, one persistent CTA
// per SM.
//
// Algorithm and numerics are those of attention_tc2.cu (online softmax of
// replace_with_fused_attention.py:334-455 in the reference: f32 scores / max / sum /
// accumulator, P rounded to bf16 before P.V, O = acc / l; P kept in tensor memory over the
// score columns, TS-form MMA). What changes is the schedule:
//   * ONE MMA warp serves two query tiles A and B of the same (batch, head) and fixes the order
//         ... P_A V -> Q_A K' -> P_B V -> Q_B K' -> P_A' V' -> ...
//     so that tile A's softmax runs under tile B's two products and vice versa, and both tiles
//     read the same K / V tiles from shared memory (loaded once for 256 query rows). Two
//     independent CTAs on an SM do not settle into that order by themselves.
//   * The whole MMA warp walks the schedule and one elected lane issues, so descriptor
//     arithmetic stays warp-uniform: an MMA of 128 x 128 x 16 runs for about 64 clocks, and a
//     single divergent thread building two descriptors per instruction could not feed the
//     tensor core that fast (measured: ~92 clocks per issue).
//   * CTAs are persistent: a CTA walks work items (batch, head, pair of query tiles) with its
//     barriers' phases running on. The next item's Q is fetched during the last key tiles of
//     the current one, its first Q K^T is issued right behind the current item's last P V, and
//     only the softmax warps' write-out of O (tensor memory -> registers -> global) separates
//     two items, per tile and under the other tile's work. One CTA per work item left ~10 us of
//     set-up and drain per item exposed (a quarter of the run at sequence length 2048).
//
// Warps: 0 TMA producer (Q_A, Q_B per item; K and V in two-stage rings), 1 MMA issuer, 2-5
// softmax of tile A, 6-9 softmax of tile B (one row per thread). Tensor memory: S_A, S_B, O_A,
// O_B, 128 columns each = all 512. Every wait is bounded.
#include "common.cuh"
#include "epilogue.cuh"
#include "ptx.cuh"

#include <algorithm>
#include <vector>

namespace lh {

namespace {

constexpr int BQ3 = 128;   // query rows per tile; two tiles per work item
constexpr int BKV3 = 128;
constexpr int ATT3_THREADS = 320;
constexpr int SUBTILE3 = 128 * 128;  // 128 rows x 64 bf16

struct Attn3Params {
  int B, Hq, Hkv, Sq, Skv;
  void* O;
  int o_dtype;
  int64_t sob, soh, sos;
  float scale_log2;
  int causal;
  int num_q_pairs;
  int num_items;  // B * Hq * num_q_pairs, or the length of `table`
  int* dev_status;
  // Split key ranges (small causal grids, see AttnSplitPlan): work items come from a table,
  // an item covers `chunk` key tiles of its pair of query tiles, and a tile whose key range is
  // spread over several items is put together by whichever of them finishes last.
  const int4* table;  // nullptr: items are whole pairs, numbered arithmetically
  float* part;        // [(slot * 2 + tile) * max_chunks + chunk index] blocks of 128 x (HD + 4) floats: O unnormalised, m, l
  int* counters;      // [slot * 2 + tile]: items of that tile finished so far (zero between launches)
  int chunk, max_chunks;
};

template <int HD>
struct Attn3Smem {
  static constexpr int Q_BYTES = BQ3 * HD * 2;   // one query tile
  static constexpr int KV_BYTES = BKV3 * HD * 2;
  static constexpr int Q_OFF = 0;                      // tiles A, B
  static constexpr int K_OFF = Q_OFF + 2 * Q_BYTES;    // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * KV_BYTES;   // 2 stages
  static constexpr int BAR_OFF = V_OFF + 2 * KV_BYTES;
  static constexpr int NUM_BARS = 18;
  static constexpr int DYN_BYTES = BAR_OFF + NUM_BARS * 8 + 16 + 1024;
  static_assert(DYN_BYTES <= 232448, "exceeds the shared memory a CTA can opt into");
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ bool wait_warp3(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* dev_status, int code) {
  // every lane observes the phase itself (its later reads are ordered after it); the warp
  // agrees on the verdict so that a timeout never splits it
  const bool ok = mbar_wait(bar, parity, abort_flag, dev_status, code);
  return __all_sync(0xffffffffu, ok);
}

// One work item: which (batch, query head, pair of query tiles), and how many key tiles each
// of its two query tiles visits (0 for a tile that lies outside the queries).
struct Item3 {
  int b, hq, hkv, q0, n_a, n_b, n_max;
  int j0;            // first key tile this item visits
  int cidx, slot;    // split items: which chunk of the pair's key range, and the pair's slot in the partial buffers
  int nch_a, nch_b;  // over how many items each tile's key range is spread (1: this item writes the result itself)
};

__device__ __forceinline__ int kv_tiles_for(const Attn3Params& p, int q0) {
  if (q0 >= p.Sq) return 0;
  int n = (p.Skv + BKV3 - 1) / BKV3;
  if (p.causal) {
    const int last_col = min(q0 + BQ3 - 1 + (p.Skv - p.Sq), p.Skv - 1);
    n = min(n, max(last_col, 0) / BKV3 + 1);
  }
  return n;
}

// Which item CTA `cta` of `grid` takes in round r, or -1 if none: rounds alternate direction
// (c, 2 grid - 1 - c, 2 grid + c, ...). Causal items are numbered heaviest first (a pair of
// query tiles (2i, 2i + 1) visits up to 2i + 2 key tiles), so a CTA that got an early, heavy
// item of one round gets a late, light one of the next, and the CTAs' totals stay within a
// few key tiles of each other (plain round-robin leaves 70 against a mean of 62 at batch 8,
// 16 heads, sequence 2048; this order 64).
__device__ __forceinline__ int item_of_round(int r, int cta, int grid, int num_items) {
  const int idx = r * grid + ((r & 1) ? grid - 1 - cta : cta);
  return idx < num_items ? idx : -1;
}
#define FOR_EACH_ITEM(item)                                                                          \
  for (int r_ = 0, item = 0; r_ * static_cast<int>(gridDim.x) < p.num_items; ++r_)                     \
    if ((item = item_of_round(r_, blockIdx.x, gridDim.x, p.num_items)) >= 0)

__device__ __forceinline__ Item3 decode_item(const Attn3Params& p, int item) {
  const int nbh = p.B * p.Hq;
  int bh, qp;
  Item3 w;
  w.j0 = 0; w.cidx = 0; w.slot = -1; w.nch_a = 1; w.nch_b = 1;
  if (p.table) {
    const int4 e = __ldg(&p.table[item]);
    bh = e.x;
    qp = e.y & 0xffff;
    w.cidx = e.y >> 16;
    w.j0 = e.z;
    w.slot = e.w;
  } else if (p.causal) {
    qp = p.num_q_pairs - 1 - item / nbh;
    bh = item % nbh;
  } else {
    bh = item / p.num_q_pairs;
    qp = item % p.num_q_pairs;
  }
  w.b = bh / p.Hq;
  w.hq = bh % p.Hq;
  w.hkv = w.hq / (p.Hq / p.Hkv);
  w.q0 = qp * (2 * BQ3);
  w.n_a = kv_tiles_for(p, w.q0);
  w.n_b = kv_tiles_for(p, w.q0 + BQ3);
  if (p.table) {
    w.nch_a = (w.n_a + p.chunk - 1) / p.chunk;
    w.nch_b = (w.n_b + p.chunk - 1) / p.chunk;
    w.n_a = min(max(w.n_a - w.j0, 0), p.chunk);
    w.n_b = min(max(w.n_b - w.j0, 0), p.chunk);
  }
  w.n_max = max(w.n_a, w.n_b);
  return w;
}

template <int HD>
__global__ void __launch_bounds__(ATT3_THREADS, 1)
attn_fwd_tc3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const Attn3Params p) {
  using L = Attn3Smem<HD>;
  constexpr int TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, O_COL = 256;  // tile t: scores at S_COL + 128 t, accumulator at O_COL + 128 t
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars + 0;
  uint64_t* q_empty = bars + 1;   // the item's last Q K^T has read Q
  uint64_t* k_full = bars + 2;    // [2] stages
  uint64_t* k_empty = bars + 4;   // [2]
  uint64_t* v_full = bars + 6;    // [2]
  uint64_t* v_empty = bars + 8;   // [2]
  uint64_t* s_full = bars + 10;   // [2] tiles
  uint64_t* p_half = bars + 12;   // [tile][half]: keys [0,64) / [64,128) of P written
  uint64_t* pv_done = bars + 16;  // [2] tiles
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* arrivals = abort_flag + 1;  // [2] tiles: how many items of a split tile had finished before this one

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int offset = p.Skv - p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_half[2 * s], 128);
      mbar_init(&p_half[2 * s + 1], 128);
      mbar_init(&pv_done[s], 1);
    }
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
  // Set-up above touched only this CTA's shared and tensor memory and may run while the kernel
  // before this one drains (programmatic dependent launch, see the launch); every CTA of this
  // persistent grid is resident, so the next kernel may take SMs as they fall free. Global
  // memory is read from here on: all threads wait for the predecessor first.
  grid_dependency_trigger();
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t kv = 0;  // key tiles loaded so far: ring position, running across items
      bool ok = true;
      int it = -1;
      FOR_EACH_ITEM(item) {
        if (!ok) break;
        ++it;
        const Item3 w = decode_item(p, item);
        // Q of the previous item is no longer read once its last Q K^T has completed
        if (it > 0 && !mbar_wait(q_empty, (it - 1) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_PRODUCER)) {
          ok = false;
          break;
        }
        // Both query tiles; rows beyond the queries arrive as zeros (their results are never stored).
        mbar_arrive_expect_tx(q_full, 2 * L::Q_BYTES);
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int h = 0; h < HD / 64; ++h)
            tma_load_4d(smem + L::Q_OFF + t * L::Q_BYTES + h * SUBTILE3, &tmQ, q_full, h * 64, w.q0 + t * BQ3, w.hq, w.b);
        for (int j = 0; j < w.n_max; ++j, ++kv) {
          const int st = kv & 1;
          const uint32_t ph = (kv >> 1) & 1u;
          if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&k_full[st], L::KV_BYTES);
#pragma unroll
          for (int h = 0; h < HD / 64; ++h)
            tma_load_4d(smem + L::K_OFF + st * L::KV_BYTES + h * SUBTILE3, &tmK, &k_full[st], h * 64, (w.j0 + j) * BKV3, w.hkv, w.b);
          if (!mbar_wait(&v_empty[st], ph ^ 1u, abort_flag, p.dev_status, DEV_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&v_full[st], L::KV_BYTES);
#pragma unroll
          for (int h = 0; h < HD / 64; ++h)
            tma_load_4d(smem + L::V_OFF + st * L::KV_BYTES + h * SUBTILE3, &tmV, &v_full[st], h * 64, (w.j0 + j) * BKV3, w.hkv, w.b);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc_qk = make_idesc(UMMA_BF16, BQ3, BKV3, false, false);
    constexpr uint32_t idesc_pv = make_idesc(UMMA_BF16, BQ3, HD, false, true);
    const uint32_t q_addr = smem_u32(smem + L::Q_OFF);
    const uint32_t k_addr = smem_u32(smem + L::K_OFF);
    const uint32_t v_addr = smem_u32(smem + L::V_OFF);
    // S_t = Q_t K^T with K in ring stage `st`, into tile t's score columns
    auto issue_qk = [&](int t, int st) {
      const uint64_t qd = make_smem_desc_sw128(q_addr + t * L::Q_BYTES, 16, 1024);
      const uint64_t kd = make_smem_desc_sw128(k_addr + st * L::KV_BYTES, 16, 1024);
      const uint32_t d = tmem_base + S_COL + t * 128;
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t off = static_cast<uint64_t>(((k / 4) * SUBTILE3 + (k % 4) * 32) >> 4);  // the address field counts 16-byte units
          umma_f16_ss(d, qd + off, kd + off, idesc_qk, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      }
      __syncwarp();
    };
    uint32_t kv = 0;            // key tiles consumed so far (ring position)
    uint32_t cnt[2] = {0u, 0u};  // key tiles each query tile has been through: phase of its barriers
    bool ok = true;
    int it = -1;
    FOR_EACH_ITEM(item) {
      if (!ok) break;
      ++it;
      const Item3 w = decode_item(p, item);
      auto n_of = [&](int t) { return t == 0 ? w.n_a : w.n_b; };
      if (!wait_warp3(q_full, it & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_MMA) ||
          !wait_warp3(&k_full[kv & 1], (kv >> 1) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // The item's first scores overwrite the columns the previous item's last P V reads P from;
      // the tensor core runs one thread's MMAs in issue order.
      for (int t = 0; t < 2; ++t)
        if (n_of(t) > 0) issue_qk(t, kv & 1);
      if (elect_one()) {
        umma_commit(&k_empty[kv & 1]);
        if (w.n_max == 1) umma_commit(q_empty);
      }
      __syncwarp();
      for (int j = 0; j < w.n_max && ok; ++j, ++kv) {
        const int st = kv & 1;
        const bool have_next = j + 1 < w.n_max;
        if (!wait_warp3(&v_full[st], (kv >> 1) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        bool next_k_seen = false;
        const uint64_t vd = make_smem_desc_sw128(v_addr + st * L::KV_BYTES, SUBTILE3, 1024);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (!ok) break;
          if (j < n_of(t)) {
            // O_t += P_t V_j, P_t read from tensor memory, its first 64 keys consumed while the
            // softmax warps still produce the rest. (The first product of an item overwrites
            // O_t: the softmax warps hand over P only after they have read the previous item's
            // result out of it.)
            const uint32_t od = tmem_base + O_COL + t * 128, pa = tmem_base + S_COL + t * 128;
            const uint32_t tph = (cnt[t] + j) & 1u;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              if (!wait_warp3(&p_half[2 * t + hf], tph, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) {
                ok = false;
                break;
              }
              tc_fence_after_sync();
              if (elect_one()) {
#pragma unroll
                for (int k = hf * 4; k < hf * 4 + 4; ++k)  // 16 keys of P = 8 packed columns; V rows are keys, 2048 bytes per 16 keys and 64 head-dim elements
                  umma_f16_ts(od, pa + k * 8, vd + static_cast<uint64_t>((k * 2048) >> 4), idesc_pv, (j | k) != 0 ? 1u : 0u);
                if (hf == 1) umma_commit(&pv_done[t]);
              }
              __syncwarp();
            }
            if (!ok) break;
          }
          if (j + 1 < n_of(t)) {
            // The next scores of this tile overwrite the columns the product just issued reads P from.
            if (!next_k_seen) {
              if (!wait_warp3(&k_full[(kv + 1) & 1], ((kv + 1) >> 1) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_MMA)) {
                ok = false;
                break;
              }
              tc_fence_after_sync();
              next_k_seen = true;
            }
            issue_qk(t, (kv + 1) & 1);
          }
        }
        if (!ok) break;
        if (elect_one()) {
          umma_commit(&v_empty[st]);                           // both tiles' P V of this stage are issued
          if (have_next) umma_commit(&k_empty[(kv + 1) & 1]);  // and both tiles' Q K^T on the next K
          if (j + 2 == w.n_max) umma_commit(q_empty);          // those were the item's last Q K^T
        }
        __syncwarp();
      }
      cnt[0] += w.n_a;
      cnt[1] += w.n_b;
    }
  } else {
    // ---------------------------------------------------------------- softmax
    const int t = (warp - 2) >> 2;  // which query tile this warp group serves
    const int quarter = warp & 3;   // tensor-memory lanes [32 quarter, +32) are this warp's
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + S_COL + t * 128 + lane_off;
    const uint32_t o_addr = tmem_base + O_COL + t * 128 + lane_off;
    uint64_t* my_s_full = &s_full[t];
    uint64_t* my_p_half = &p_half[2 * t];
    uint32_t cnt = 0;  // key tiles this query tile has been through over all items
    bool ok = true;
    FOR_EACH_ITEM(item) {
      if (!ok) break;
      // (only what the key loop needs stays live through it; the item is decoded again for the
      // write-out, which keeps the loop free of spills)
      int n_mine, q0t, key0;
      {
        const Item3 w = decode_item(p, item);
        n_mine = t == 0 ? w.n_a : w.n_b;
        q0t = w.q0 + t * BQ3;
        key0 = w.j0 * BKV3;
      }
      const int q_row = q0t + row;
      float m_used = -INFINITY;
      float l = 0.f;
      for (int j = 0; j < n_mine; ++j) {
        if (!wait_warp3(my_s_full, (cnt + j) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_SOFTMAX)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const int col0 = key0 + j * BKV3;
        const bool need_mask = (col0 + BKV3 > p.Skv) || (p.causal && (col0 + BKV3 - 1 > q0t + offset));
        const int limit = need_mask ? (p.causal ? min(p.Skv - 1, q_row + offset) : (p.Skv - 1)) - col0 : BKV3;  // last visible column in this tile
        // pass 1: row max of the scores, two 32-column loads in flight at a time
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
          for (int i = 0; i < 32; i += 4) {
            mx0 = fmax3(mx0, __uint_as_float(s0[i]), __uint_as_float(s0[i + 1]));
            mx1 = fmax3(mx1, __uint_as_float(s0[i + 2]), __uint_as_float(s0[i + 3]));
            mx2 = fmax3(mx2, __uint_as_float(s1[i]), __uint_as_float(s1[i + 1]));
            mx3 = fmax3(mx3, __uint_as_float(s1[i + 2]), __uint_as_float(s1[i + 3]));
          }
        }
        float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        mx *= p.scale_log2;  // scale > 0: max commutes with the scaling
        // lazy rescale: move the reference max only when it grew by more than 8 (2^8 headroom)
        float alpha = 1.f;
        const bool need = (mx > m_used + 8.f) || (m_used == -INFINITY && mx > -INFINITY);
        if (need) {
          alpha = (m_used == -INFINITY) ? 0.f : ex2_approx(m_used - mx);
          m_used = mx;
        }
        const bool warp_need = __any_sync(0xffffffffu, need);
        if (j > 0 && warp_need) {
          // s_full(j) fired after every MMA issued before it, this tile's P V of key tile j - 1
          // included: the accumulator is up to date and nothing writes it until P(j) is handed over
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
            float p0 = ex2_approx(fmaf(__uint_as_float(s0[2 * i]), p.scale_log2, -msub));
            float p1 = ex2_approx(fmaf(__uint_as_float(s0[2 * i + 1]), p.scale_log2, -msub));
            float p2 = ex2_approx(fmaf(__uint_as_float(s1[2 * i]), p.scale_log2, -msub));
            float p3 = ex2_approx(fmaf(__uint_as_float(s1[2 * i + 1]), p.scale_log2, -msub));
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
          mbar_arrive(&my_p_half[hf]);
        }
        l = l * alpha + ((rs0 + rs1) + (rs2 + rs3));
      }
      if (!ok) break;
      if (n_mine > 0) {
        // O_t is final once this tile's last P V has completed. Its columns are read out here
        // before these threads hand over the next item's first P, which is what the MMA warp
        // waits for before it overwrites them.
        if (!wait_warp3(&pv_done[t], (cnt + n_mine - 1) & 1u, abort_flag, p.dev_status, DEV_TIMEOUT_SOFTMAX)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const Item3 w = decode_item(p, item);
        char* obase = static_cast<char*>(p.O);
        const int64_t oidx = static_cast<int64_t>(w.b) * p.sob + static_cast<int64_t>(w.hq) * p.soh + static_cast<int64_t>(q_row) * p.sos;
        const int nch_mine = t == 0 ? w.nch_a : w.nch_b;
        if (nch_mine <= 1) {
          const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
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
        } else {
          // This tile's keys are spread over nch_mine items. Every one of them leaves its
          // un-normalised accumulator, reference maximum and row sum in global memory and counts
          // itself in; the one that finds all the others counted puts the rows together:
          // O = sum_c 2^(m_c - M) O_c / sum_c 2^(m_c - M) l_c with M = max_c m_c. Nobody waits.
          // One item's block: [HD / 4 groups of 4 columns][128 rows][4] then m[128], l[128]: a
          // warp's 32 rows of one group are 512 contiguous bytes, for the writes here and the
          // reads of the merge alike (a row per thread with rows 528 bytes apart made each
          // 16-byte access its own transaction: 25 us per item).
          constexpr int BLOCK = BQ3 * (HD + 4);
          float* tile_part = p.part + static_cast<int64_t>(w.slot * 2 + t) * p.max_chunks * BLOCK;
          float* mine = tile_part + static_cast<int64_t>(w.cidx) * BLOCK;
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(o_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int g = 0; g < 8; ++g)
              __stcg(reinterpret_cast<uint4*>(mine) + (c * 8 + g) * BQ3 + row, make_uint4(o[4 * g], o[4 * g + 1], o[4 * g + 2], o[4 * g + 3]));
          }
          __stcg(mine + HD * BQ3 + row, m_used);
          __stcg(mine + (HD + 1) * BQ3 + row, l);
          __threadfence();
          asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");  // the tile's 128 rows are written
          if (row == 0) arrivals[t] = atomicAdd(&p.counters[w.slot * 2 + t], 1);
          asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");
          const bool last = arrivals[t] == nch_mine - 1;
          asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");  // everyone has read the verdict before the next item overwrites it
          if (last) {
            __threadfence();
            if (row == 0) p.counters[w.slot * 2 + t] = 0;  // ready for the next launch
            float M = -INFINITY;
            for (int c = 0; c < nch_mine; ++c) M = fmaxf(M, __ldcg(tile_part + static_cast<int64_t>(c) * BLOCK + HD * BQ3 + row));
            float L = 0.f;
            for (int c = 0; c < nch_mine; ++c) {
              const float* blk = tile_part + static_cast<int64_t>(c) * BLOCK;
              const float mc = __ldcg(blk + HD * BQ3 + row), lc = __ldcg(blk + (HD + 1) * BQ3 + row);
              L += (mc == -INFINITY) ? 0.f : ex2_approx(mc - M) * lc;
            }
            const float inv_l = (L > 0.f) ? 1.f / L : 0.f;
            if (q_row < p.Sq) {
#pragma unroll 1
              for (int cb = 0; cb < HD / 32; ++cb) {
                float acc[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = 0.f;
                for (int c = 0; c < nch_mine; ++c) {
                  const float* blk = tile_part + static_cast<int64_t>(c) * BLOCK;
                  const float mc = __ldcg(blk + HD * BQ3 + row);
                  const float wgt = (mc == -INFINITY) ? 0.f : ex2_approx(mc - M);
#pragma unroll
                  for (int g = 0; g < 8; ++g) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(blk) + (cb * 8 + g) * BQ3 + row);
                    acc[4 * g] = fmaf(wgt, v.x, acc[4 * g]);
                    acc[4 * g + 1] = fmaf(wgt, v.y, acc[4 * g + 1]);
                    acc[4 * g + 2] = fmaf(wgt, v.z, acc[4 * g + 2]);
                    acc[4 * g + 3] = fmaf(wgt, v.w, acc[4 * g + 3]);
                  }
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  float v[8];
#pragma unroll
                  for (int i = 0; i < 8; ++i) v[i] = acc[g * 8 + i] * inv_l;
                  store8_from_f32(obase, p.o_dtype, oidx + cb * 32 + g * 8, v);
                }
              }
            }
          }
        }
        tc_fence_before_sync();
      }
      cnt += n_mine;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if (*abort_flag) {
      // a role gave up: let copies and MMAs already in flight drain before the tensor memory
      // goes back to the allocator
      const uint64_t t0 = global_timer_ns();
      while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Key tiles a 128-row query tile starting at q0 visits (host copy of kv_tiles_for).
int host_kv_tiles(int Sq, int Skv, int causal, int q0) {
  if (q0 >= Sq) return 0;
  int n = (Skv + BKV3 - 1) / BKV3;
  if (causal) {
    int last_col = q0 + BQ3 - 1 + (Skv - Sq);
    if (last_col > Skv - 1) last_col = Skv - 1;
    if (last_col < 0) last_col = 0;
    const int m = last_col / BKV3 + 1;
    if (m < n) n = m;
  }
  return n;
}

// The plan for this shape, built on first use. A causal grid is split when there are no more
// pairs of query tiles than SMs - every SM then gets at most one pair and the heaviest pair
// sets the time (8 sequences-times-heads of 4096 positions: 128 pairs on 148 SMs, the heaviest
// 32 key tiles against a mean of 14.7 per SM: 77 us, 69 us with chunks of 8 key tiles, and
// less with chunks of the mean load). An item costs about 10 us beyond its key tiles (pipeline
// fill and drain, 134 KB of partial results written and read back), so grids with more pairs
// than SMs, which snake order already balances to within a few key tiles, stay whole: split
// they were measured 25-35 % slower. Items are `chunk` key tiles of a pair, chunk = the mean
// load per SM rounded up to even, sorted heaviest first for the kernel's snake order.
// SMs this kernel's persistent grid may take: like the GEMM it leaves the reserved ones to a
// collective running beside it (a CTA that found its SM taken would start when another
// finished, and its items with it).
inline int usable_sms(const lh_ctx* ctx) { return ctx->sm_count - ctx->reserved_sms > 0 ? ctx->sm_count - ctx->reserved_sms : 1; }

const AttnSplitPlan* split_plan(lh_ctx* ctx, int BH, int Sq, int Skv, int HD, int causal) {
  const int pairs = (Sq + 2 * BQ3 - 1) / (2 * BQ3);
  const int64_t whole_items = static_cast<int64_t>(BH) * pairs;
  const int sms = usable_sms(ctx);
  const int grid = whole_items < sms ? static_cast<int>(whole_items) : sms;
  for (const AttnSplitPlan& pl : ctx->attn_plans)
    if (pl.bh == BH && pl.sq == Sq && pl.skv == Skv && pl.hd == HD && pl.grid == grid) return pl.chunk ? &pl : nullptr;
  AttnSplitPlan pl{};
  pl.bh = BH; pl.sq = Sq; pl.skv = Skv; pl.hd = HD; pl.grid = grid;
  std::vector<int> n_max(pairs);
  int64_t work = 0;
  int heaviest = 0;
  for (int qp = 0; qp < pairs; ++qp) {
    const int na = host_kv_tiles(Sq, Skv, causal, qp * 2 * BQ3), nb = host_kv_tiles(Sq, Skv, causal, qp * 2 * BQ3 + BQ3);
    n_max[qp] = na > nb ? na : nb;
    work += n_max[qp];
    if (n_max[qp] > heaviest) heaviest = n_max[qp];
  }
  work *= BH;
  const double mean = static_cast<double>(work) / sms;
  if (causal && heaviest >= 8 && whole_items <= sms && heaviest > 1.25 * mean && pairs < 0x10000) {
    int chunk = 2 * static_cast<int>((mean + 1.999) / 2.0);
    chunk = chunk < 4 ? 4 : chunk > 16 ? 16 : chunk;
    struct Entry { int size, bh, qp, c, j0, slot; };
    std::vector<Entry> entries;
    int slots = 0, max_chunks = 1;
    for (int bh = 0; bh < BH; ++bh)
      for (int qp = 0; qp < pairs; ++qp) {
        const int nch = (n_max[qp] + chunk - 1) / chunk;
        if (nch > max_chunks) max_chunks = nch;
        const int slot = nch > 1 ? slots++ : -1;
        for (int c = 0; c < nch; ++c) {
          const int left = n_max[qp] - c * chunk;
          entries.push_back({left < chunk ? left : chunk, bh, qp, c, c * chunk, slot});
        }
      }
    std::stable_sort(entries.begin(), entries.end(), [](const Entry& x, const Entry& y) { return x.size > y.size; });
    const size_t part_bytes = static_cast<size_t>(slots) * 2 * max_chunks * BQ3 * (HD + 4) * sizeof(float);
    if (slots > 0 && part_bytes <= (512ull << 20)) {
      std::vector<int4> table(entries.size());
      for (size_t i = 0; i < entries.size(); ++i) table[i] = make_int4(entries[i].bh, entries[i].qp | (entries[i].c << 16), entries[i].j0, entries[i].slot);
      void* dev_table = nullptr;
      int* dev_counters = nullptr;
      if (cudaMalloc(&dev_table, table.size() * sizeof(int4)) == cudaSuccess && cudaMalloc(&dev_counters, static_cast<size_t>(slots) * 2 * sizeof(int)) == cudaSuccess &&
          cudaMemcpy(dev_table, table.data(), table.size() * sizeof(int4), cudaMemcpyHostToDevice) == cudaSuccess &&
          cudaMemset(dev_counters, 0, static_cast<size_t>(slots) * 2 * sizeof(int)) == cudaSuccess) {
        pl.chunk = chunk; pl.max_chunks = max_chunks; pl.n_items = static_cast<int>(entries.size()); pl.n_slots = slots;
        pl.table = dev_table; pl.counters = dev_counters; pl.part_bytes = part_bytes;
      } else {
        cudaGetLastError();  // no table: the shape runs as whole pairs
        if (dev_table) cudaFree(dev_table);
        if (dev_counters) cudaFree(dev_counters);
      }
    }
  }
  ctx->attn_plans.push_back(pl);
  return ctx->attn_plans.back().chunk ? &ctx->attn_plans.back() : nullptr;
}

template <int HD>
int launch3_hd(lh_ctx* ctx, const AttnProblem& a) {
  using L = Attn3Smem<HD>;
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
  Attn3Params p;
  p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Sq = a.Sq; p.Skv = a.Skv;
  p.O = a.O; p.o_dtype = a.o_dtype; p.sob = a.sob; p.soh = a.soh; p.sos = a.sos;
  p.scale_log2 = a.scale * 1.44269504088896340736f;
  p.causal = a.causal;
  p.num_q_pairs = (a.Sq + 2 * BQ3 - 1) / (2 * BQ3);
  int64_t items = static_cast<int64_t>(a.B) * a.Hq * p.num_q_pairs;
  p.table = nullptr; p.part = nullptr; p.counters = nullptr; p.chunk = 0; p.max_chunks = 1;
  if (const AttnSplitPlan* pl = split_plan(ctx, a.B * a.Hq, a.Sq, a.Skv, HD, a.causal)) {
    int rc = ensure_scratch(ctx, pl->part_bytes);
    if (rc) return rc;
    p.table = static_cast<const int4*>(pl->table);
    p.part = static_cast<float*>(ctx->scratch);
    p.counters = pl->counters;
    p.chunk = pl->chunk;
    p.max_chunks = pl->max_chunks;
    items = pl->n_items;
  }
  p.num_items = static_cast<int>(items);
  p.dev_status = ctx->dev_status;
  auto kernel = attn_fwd_tc3_kernel<HD>;
  LH_CUDA_CHECK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES));
  const int grid = items < usable_sms(ctx) ? static_cast<int>(items) : usable_sms(ctx);  // one persistent CTA per SM
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(ATT3_THREADS);
  cfg.dynamicSmemBytes = L::DYN_BYTES;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // CTAs may set up while the previous kernel drains
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->launch_overlap ? 1 : 0;  // off: an ordinary launch, the kernel's grid-dependency calls are no-ops
  LH_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, kernel, tmQ, tmK, tmV, p));
  LH_CHECK_LAUNCH(ctx, "attn_fwd_tc3_kernel");
  return LH_OK;
}

}  // namespace

size_t attn_tc_scratch_bytes(lh_ctx* ctx, int B, int Hq, int Sq, int Skv, int D, int causal) {
  if (ctx->cc_major != 10 || (D != 64 && D != 128) || Sq <= BQ3 || B < 1 || Hq < 1) return 0;
  const AttnSplitPlan* pl = split_plan(ctx, B * Hq, Sq, Skv, D, causal);
  return pl ? pl->part_bytes : 0;
}

int attn_tc3_launch(lh_ctx* ctx, const AttnProblem& a) {
  if (a.scale <= 0.f) return set_error(ctx, LH_ERR_UNSUPPORTED, "attention: scale must be positive");
  if (a.D == 128) return launch3_hd<128>(ctx, a);
  return launch3_hd<64>(ctx, a);
}

// What the tensor-core kernels take: bf16 Q / K / V with unit stride in the head dimension,
// head sizes 64 and 128, 16-byte aligned rows (tensor maps), grouped heads, and for a causal
// mask at least as many keys as queries.
int attn_tc_supported(const lh_ctx* ctx, const AttnProblem& a) {
  if (ctx->cc_major != 10) return 0;
  if (a.dtype != LH_BF16) return 0;
  if (a.o_dtype != LH_BF16 && a.o_dtype != LH_F32) return 0;
  if (a.D != 64 && a.D != 128) return 0;
  if (a.Hkv < 1 || a.Hq % a.Hkv) return 0;
  if (a.causal && a.Skv < a.Sq) return 0;
  if (a.scale <= 0.f) return 0;
  auto ok8 = [](int64_t s) { return (s % 8) == 0; };
  if (!ok8(a.sqb) || !ok8(a.sqh) || !ok8(a.sqs) || !ok8(a.skb) || !ok8(a.skh) || !ok8(a.sks) || !ok8(a.svb) ||
      !ok8(a.svh) || !ok8(a.svs) || !ok8(a.sob) || !ok8(a.soh) || !ok8(a.sos))
    return 0;
  auto al = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  if (!al(a.Q) || !al(a.K) || !al(a.V) || !al(a.O)) return 0;
  if (static_cast<int64_t>(a.B) * a.Hq * ((a.Sq + BQ3 - 1) / BQ3) > 0x7fffffffLL) return 0;
  return 1;
}

int attn_tc_launch(lh_ctx* ctx, const AttnProblem& a) {
  // One query tile per (batch, head): nothing to ping-pong with, two independent blocks per SM
  // serve such problems better.
  if (a.Sq <= BQ3) return attn_tc2_launch(ctx, a);
  return attn_tc3_launch(ctx, a);
}

}  // namespace lh
