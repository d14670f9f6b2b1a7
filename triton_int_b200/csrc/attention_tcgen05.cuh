// Fused int8 attention for sm_100a: O = int8(alpha_pv * (P . V)),
// P = int8(p_mul * softmax(mask(alpha_qk * Q . K^T))), head_dim 128.
//
// The score matrix S and the quantised probabilities P never leave the SM.  Because P
// is quantised with the FINAL row maximum and row sum, every 128-row query tile makes
// two passes over its key tiles:
//   pass 1  S_j = Q K_j^T on the tensor cores; running integer row maximum and the row
//           sum of 2^((s - max) * c) (c = alpha_qk * log2 e)
//   pass 2  S_j again; P_j = round(p_mul * 2^((s - max) * c) / sum) written as int8 into
//           128B-swizzled shared memory, from where the second MMA accumulates
//           O += P_j V_j in TMEM (V tiles are read in their natural [key][d] layout as
//           an MN-major operand, so no V^T copy exists anywhere)
// Roles (576 threads, one persistent CTA per SM): warp 0 TMA producer, warp 1 MMA
// issuer, warps 2-9 and 10-17 two softmax groups that alternate key tiles; inside a group
// a thread owns half a query row of the 128x128 score tile (64 columns, pulled out of TMEM
// in one go), so four softmax warps share each scheduler and hide each other's latencies.
// int32 -> fp32 uses the exact "add 1.5*2^23 as integer bits" form (|s - max| < 2^22 for
// head_dim 128), so one exp2 per element is the only special-function operation.
// Every wait is bounded; on expiry a status bit is set and the CTA drains and returns.
#pragma once

#include "gemm_tcgen05.cuh"

namespace ti {
namespace attn {

using namespace ti::tc;

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = 128 * 128;  // every operand tile: 128 rows x 128 bytes
constexpr int KS = 4;                  // K ring stages
constexpr int VS = 3;                  // V ring stages
constexpr int ATT_THREADS = 576;
constexpr int GROUP_THREADS = 256;  // one softmax group: 128 rows x 2 column halves
constexpr int GROUP_WARPS = GROUP_THREADS / 32;  // barriers signalled by a group count one arrival per warp
constexpr uint32_t MAGIC_BITS = 0x4B400000u;  // bits of 12582912.0f = 1.5 * 2^23
constexpr float MAGIC_F = 12582912.0f;

struct Params {
  const float* alpha_qk;
  const float* alpha_pv;
  int batch, heads, seq_q, seq_k;
  int q_tiles, kv_tiles, num_items;
  int causal, rounding;
  float p_mul;
};

struct Smem {
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KS * TILE_BYTES;
  static constexpr int P_OFF = V_OFF + VS * TILE_BYTES;
  static constexpr int O_OFF = P_OFF + 2 * TILE_BYTES;
  static constexpr int STAT_OFF = O_OFF + TILE_BYTES;          // [2 groups x 2 halves][128 rows] x (int max, float sum)
  static constexpr int BAR_OFF = STAT_OFF + 4 * 128 * 8;
  // q_full, q_empty, k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], s_full[2], s_empty[2],
  // p_full[2], p_empty[2], o_full, o_empty, stat, stg_free, stg_full
  static constexpr int NUM_BARS = 2 + 2 * KS + 2 * VS + 8 + 2 + 3;
  static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
  static_assert(DYN_BYTES <= 232448, "exceeds the shared memory of one CTA");
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x));
  return e;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float e;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x));
  return e;
}
// MN-major, 128B-swizzled operand: rows are k (keys), each row 128 contiguous bytes of n (d);
// groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(TILE_BYTES >> 4) << 16;  // leading byte offset: next 128-wide n chunk (only one is used)
  d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset: next group of 8 k rows
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

struct Item {
  int b, h, qi, n_kv;
};
__device__ __forceinline__ Item decode_item(const Params& p, int w) {
  // heaviest query tiles (most key tiles) first
  Item it;
  const int bh = p.batch * p.heads;
  it.qi = p.q_tiles - 1 - w / bh;
  const int r = w % bh;
  it.b = r / p.heads;
  it.h = r - it.b * p.heads;
  int n = p.kv_tiles;
  if (p.causal) {
    const int last_key = min(p.seq_k - 1, it.qi * BQ + BQ - 1 + (p.seq_k - p.seq_q));
    n = last_key < 0 ? 0 : min(p.kv_tiles, last_key / BKV + 1);
  }
  it.n_kv = n;
  return it;
}

__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_i8_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                    const Params p) {
  using S = Smem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sb = smem_u32(smem);
  const uint32_t bar0 = sb + S::BAR_OFF;
  int bi = 0;
  const uint32_t q_full = bar0 + 8 * bi++, q_empty = bar0 + 8 * bi++;
  const uint32_t k_full0 = bar0 + 8 * bi; bi += KS;
  const uint32_t k_empty0 = bar0 + 8 * bi; bi += KS;
  const uint32_t v_full0 = bar0 + 8 * bi; bi += VS;
  const uint32_t v_empty0 = bar0 + 8 * bi; bi += VS;
  const uint32_t s_full0 = bar0 + 8 * bi; bi += 2;
  const uint32_t s_empty0 = bar0 + 8 * bi; bi += 2;
  const uint32_t p_full0 = bar0 + 8 * bi; bi += 2;
  const uint32_t p_empty0 = bar0 + 8 * bi; bi += 2;
  const uint32_t o_full = bar0 + 8 * bi++, o_empty = bar0 + 8 * bi++;
  const uint32_t stat_bar = bar0 + 8 * bi++, stg_free = bar0 + 8 * bi++, stg_full = bar0 + 8 * bi++;
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + S::BAR_OFF + S::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::BAR_OFF + S::NUM_BARS * 8 + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(q_empty, 1);
    for (int i = 0; i < KS; ++i) { mbar_init(k_full0 + 8 * i, 1); mbar_init(k_empty0 + 8 * i, 1); }
    for (int i = 0; i < VS; ++i) { mbar_init(v_full0 + 8 * i, 1); mbar_init(v_empty0 + 8 * i, 1); }
    for (int g = 0; g < 2; ++g) {
      mbar_init(s_full0 + 8 * g, 1); mbar_init(s_empty0 + 8 * g, GROUP_WARPS);
      mbar_init(p_full0 + 8 * g, GROUP_WARPS); mbar_init(p_empty0 + 8 * g, 1);
    }
    mbar_init(o_full, 1); mbar_init(o_empty, 2 * GROUP_WARPS);
    mbar_init(stat_bar, 2 * GROUP_WARPS); mbar_init(stg_free, 2 * GROUP_WARPS); mbar_init(stg_full, 2 * GROUP_WARPS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32((const void*)tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s0 = tmem_base;          // S buffers: columns [0,128) and [128,256)
  const uint32_t tmem_o = tmem_base + 256;     // O accumulator: columns [256,384)

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0, item_par = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, item_par ^= 1u) {
        const Item it = decode_item(p, w);
        if (!mbar_wait(q_empty, item_par ^ 1u, abort_flag)) { atomicOr(&g_status, STATUS_PRODUCER); break; }
        mbar_expect_tx(q_full, TILE_BYTES);
        tma_load_4d(sb + S::Q_OFF, &map_q, q_full, 0, it.h, it.qi * BQ, it.b);
        for (int pass = 0; pass < 2 && ok; ++pass) {
          for (int j = 0; j < it.n_kv; ++j) {
            if (!mbar_wait(k_empty0 + 8 * ks, kph ^ 1u, abort_flag)) { atomicOr(&g_status, STATUS_PRODUCER); ok = false; break; }
            mbar_expect_tx(k_full0 + 8 * ks, TILE_BYTES);
            tma_load_4d(sb + S::K_OFF + ks * TILE_BYTES, &map_k, k_full0 + 8 * ks, 0, it.h, j * BKV, it.b);
            if (++ks == KS) { ks = 0; kph ^= 1u; }
            if (pass == 1) {
              if (!mbar_wait(v_empty0 + 8 * vs, vph ^ 1u, abort_flag)) { atomicOr(&g_status, STATUS_PRODUCER); ok = false; break; }
              mbar_expect_tx(v_full0 + 8 * vs, TILE_BYTES);
              tma_load_4d(sb + S::V_OFF + vs * TILE_BYTES, &map_v, v_full0 + 8 * vs, 0, it.h, j * BKV, it.b);
              if (++vs == VS) { vs = 0; vph ^= 1u; }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_i8(BQ, BKV);
      constexpr uint32_t idesc_pv = make_idesc_i8(BQ, HD) | (1u << 16);  // B operand MN-major
      int ks = 0, vs = 0;
      uint32_t kph = 0, vph = 0, item_par = 0;
      uint32_t s_cnt[2] = {0, 0}, p_cnt[2] = {0, 0};
      bool ok = true;
      const uint64_t qdesc = make_smem_desc(sb + S::Q_OFF);
      auto issue_qk = [&](int g) -> bool {
        // S[g] must have been pulled out of TMEM by its softmax group
        if (!mbar_wait(s_empty0 + 8 * g, (s_cnt[g] & 1u) ^ 1u, abort_flag)) return false;
        if (!mbar_wait(k_full0 + 8 * ks, kph, abort_flag)) return false;
        tc_fence_after();
        const uint64_t kdesc = make_smem_desc(sb + S::K_OFF + ks * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < HD / UMMA_K; ++k)
          umma_i8(tmem_s0 + (uint32_t)(g * BKV), qdesc + (uint64_t)(2 * k), kdesc + (uint64_t)(2 * k), idesc_qk, k > 0 ? 1u : 0u);
        umma_commit(k_empty0 + 8 * ks);
        umma_commit(s_full0 + 8 * g);
        if (++ks == KS) { ks = 0; kph ^= 1u; }
        ++s_cnt[g];
        return true;
      };
      for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, item_par ^= 1u) {
        const Item it = decode_item(p, w);
        const int n = it.n_kv;
        if (!mbar_wait(q_full, item_par, abort_flag)) { atomicOr(&g_status, STATUS_MMA); break; }
        // pass 1: scores only
        for (int j = 0; j < n && ok; ++j) ok = issue_qk(j & 1);
        // pass 2: scores again, then P V
        for (int j = 0; j < 2 && j < n && ok; ++j) ok = issue_qk(j & 1);
        if (n <= 2 && ok) umma_commit(q_empty);
        for (int j = 0; j < n && ok; ++j) {
          const int g = j & 1;
          // scores of tile j+2 first: its group has S_j in registers long before P_j is ready,
          // so the next score tile is computed while the group still works on this one
          if (j + 2 < n) {
            ok = issue_qk(g);
            if (!ok) break;
            if (j + 3 == n) umma_commit(q_empty);  // that was the last read of Q
          }
          if (!mbar_wait(p_full0 + 8 * g, p_cnt[g] & 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(v_full0 + 8 * vs, vph, abort_flag)) { ok = false; break; }
          if (j == 0 && !mbar_wait(o_empty, item_par ^ 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t pdesc = make_smem_desc(sb + S::P_OFF + g * TILE_BYTES);
          const uint64_t vdesc = make_smem_desc_mn(sb + S::V_OFF + vs * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < BKV / UMMA_K; ++k)
            umma_i8(tmem_o, pdesc + (uint64_t)(2 * k), vdesc + (uint64_t)(256 * k), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(v_empty0 + 8 * vs);
          umma_commit(p_empty0 + 8 * g);
          if (++vs == VS) { vs = 0; vph ^= 1u; }
          ++p_cnt[g];
        }
        if (ok) umma_commit(o_full);
        if (!ok) atomicOr(&g_status, STATUS_MMA);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax groups
    const int g = (warp - 2) >> 3;          // which key tiles (even / odd)
    const int half = ((warp - 2) >> 2) & 1; // which 64 columns of the score tile
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;      // query row inside the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float c = (p.alpha_qk ? *p.alpha_qk : 1.0f) * 1.4426950408889634f;
    const float negK = -(MAGIC_F * c);
    const float2 c2 = make_float2(c, c), negK2 = make_float2(negK, negK), magic2 = make_float2(MAGIC_F, MAGIC_F);
    const bool clamp_p = p.p_mul > 127.0f;  // p <= 1, so p_mul * p only needs a clamp beyond 127
    const float alpha_pv = p.alpha_pv ? *p.alpha_pv : 1.0f;
    int* stat_m = reinterpret_cast<int*>(smem + S::STAT_OFF);
    float* stat_l = reinterpret_cast<float*>(smem + S::STAT_OFF + 4 * 128 * 4);
    const int slot = (g * 2 + half) * 128 + r;
    uint32_t s_cnt = 0, p_cnt = 0, item_par = 0;
    bool ok = true;
    const int INT_LOW = -(1 << 30);

    for (int w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, item_par ^= 1u) {
      const Item it = decode_item(p, w);
      const int n = it.n_kv;
      const int qrow = it.qi * BQ + r;
      // keys [0, limit) are visible to this row
      const int limit = p.causal ? min(p.seq_k, qrow + (p.seq_k - p.seq_q) + 1) : p.seq_k;
      uint32_t acc[2][32];

      auto load_scores = [&]() -> bool {
        if (!mbar_wait_warp(s_full0 + 8 * g, s_cnt & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t ta = tmem_s0 + lane_addr + (uint32_t)(g * BKV + half * 64);
        tmem_ld32(ta, acc[0]); tmem_ld32(ta + 32, acc[1]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive_warp(s_empty0 + 8 * g);
        ++s_cnt;
        return true;
      };

      // ---- pass 1: integer row maximum and the sum of 2^((s - max) c) over this thread's columns
      int m_run = INT_LOW;
      float l_run = 0.f;
      for (int j = g; j < n; j += 2) {
        if (!load_scores()) { ok = false; break; }
        const int nvalid = limit - j * BKV - half * 64;  // columns [0, nvalid) of this thread's 64 are visible
        int tmax = INT_LOW;
        if (nvalid >= 64) {
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
            for (int i = 0; i < 32; ++i) tmax = max(tmax, (int)acc[q2][i]);
        } else {
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
            for (int i = 0; i < 32; ++i) tmax = max(tmax, (q2 * 32 + i) < nvalid ? (int)acc[q2][i] : INT_LOW);
        }
        if (tmax > m_run) {
          if (l_run != 0.f) l_run *= ex2_approx((float)(m_run - tmax) * c);
          m_run = tmax;
        }
        const uint32_t ic = MAGIC_BITS - (uint32_t)m_run;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        if (nvalid >= 64) {
          // packed fp32 pairs (fma.rn.f32x2 / add.rn.f32x2) halve the multiply-add and add count
          float2 sa = make_float2(0.f, 0.f), sb2 = make_float2(0.f, 0.f);
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float2 xa = __ffma2_rn(make_float2(__uint_as_float(acc[q2][i] + ic), __uint_as_float(acc[q2][i + 1] + ic)), c2, negK2);
              const float2 xb = __ffma2_rn(make_float2(__uint_as_float(acc[q2][i + 2] + ic), __uint_as_float(acc[q2][i + 3] + ic)), c2, negK2);
              sa = __fadd2_rn(sa, make_float2(ex2_approx(xa.x), ex2_approx(xa.y)));
              sb2 = __fadd2_rn(sb2, make_float2(ex2_approx(xb.x), ex2_approx(xb.y)));
            }
          s0 = sa.x; s1 = sa.y; s2 = sb2.x; s3 = sb2.y;
        } else if (nvalid > 0) {
#pragma unroll
          for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float e = ex2_approx(__fmaf_rn(__uint_as_float(acc[q2][i] + ic), c, negK));
              s0 += (q2 * 32 + i) < nvalid ? e : 0.f;
            }
        }
        l_run += (s0 + s1) + (s2 + s3);
      }
      if (!ok) break;
      // ---- combine the four partial statistics of the row (2 groups x 2 halves)
      stat_m[slot] = m_run;
      stat_l[slot] = l_run;
      mbar_arrive_warp(stat_bar);
      if (!mbar_wait_warp(stat_bar, item_par, abort_flag)) { ok = false; break; }
      {
        int m = INT_LOW;
#pragma unroll
        for (int k = 0; k < 4; ++k) m = max(m, stat_m[k * 128 + r]);
        float l = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float lk = stat_l[k * 128 + r];
          if (lk != 0.f) l += lk * ex2_approx((float)(stat_m[k * 128 + r] - m) * c);
        }
        m_run = m;
        l_run = l;
      }
      // p_mul * 2^(x) / l = 2^(x + log2(p_mul / l)): the normalisation becomes an exponent offset
      // (added after the fused multiply-add: the large constant inside it would swallow its low bits)
      const float lgn = l_run > 0.f ? lg2_approx(p.p_mul / l_run) : -1.0e30f;
      const uint32_t ic = MAGIC_BITS - (uint32_t)m_run;

      // ---- pass 2: quantised probabilities into shared memory
      for (int j = g; j < n; j += 2) {
        if (!load_scores()) { ok = false; break; }
        if (!mbar_wait_warp(p_empty0 + 8 * g, (p_cnt & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        const int nvalid = limit - j * BKV - half * 64;
        const uint32_t prow = sb + S::P_OFF + (uint32_t)(g * TILE_BYTES + r * 128);
        const float2 lgn2 = make_float2(lgn, lgn);
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
#pragma unroll
          for (int h16 = 0; h16 < 2; ++h16) {
            uint32_t wv[4];
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4) {
              uint32_t b[4];
#pragma unroll
              for (int i = 0; i < 4; i += 2) {
                const int k0 = h16 * 16 + w4 * 4 + i;
                float2 x = __ffma2_rn(make_float2(__uint_as_float(acc[q2][k0] + ic), __uint_as_float(acc[q2][k0 + 1] + ic)), c2, negK2);
                x = __fadd2_rn(x, lgn2);
                float2 e = make_float2(ex2_approx(x.x), ex2_approx(x.y));
                if (nvalid < 64) {
                  const int col = q2 * 32 + k0;
                  e.x = col < nvalid ? e.x : 0.f;
                  e.y = col + 1 < nvalid ? e.y : 0.f;
                }
                if (clamp_p) { e.x = fminf(e.x, 127.0f); e.y = fminf(e.y, 127.0f); }
                const float2 rr = __fadd2_rn(e, magic2);  // round half even; low byte = int8
                b[i] = __float_as_uint(rr.x);
                b[i + 1] = __float_as_uint(rr.y);
              }
              wv[w4] = pack4_low_bytes(b[0], b[1], b[2], b[3]);
            }
            const int lc = half * 4 + q2 * 2 + h16;  // 16-byte piece inside the 128-byte row
            st_shared_v4(prow + (uint32_t)((lc ^ (r & 7)) * 16), wv[0], wv[1], wv[2], wv[3]);
          }
        }
        fence_async_smem();
        mbar_arrive_warp(p_full0 + 8 * g);
        ++p_cnt;
      }
      if (!ok) break;

      // ---- epilogue: O (int32 in TMEM) -> int8, 32 of the 128 head-dimension columns per thread
      if (!mbar_wait_warp(o_full, item_par, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int oq = g * 2 + half;  // which 32 columns
      uint32_t o32[32];
      tmem_ld32(tmem_o + lane_addr + (uint32_t)(oq * 32), o32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(o_empty);
      if (threadIdx.x == 64) tma_store_wait_read<0>();  // the previous item's store has left the staging tile
      mbar_arrive_warp(stg_free);
      if (!mbar_wait_warp(stg_free, item_par, abort_flag)) { ok = false; break; }
      {
        const uint32_t orow = sb + S::O_OFF + (uint32_t)(r * 128);
#pragma unroll
        for (int h16 = 0; h16 < 2; ++h16) {
          uint32_t wv[4];
#pragma unroll
          for (int w4 = 0; w4 < 4; ++w4) {
            uint32_t b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float f = __fmul_rn(__int2float_rn((int32_t)o32[h16 * 16 + w4 * 4 + i]), alpha_pv);
              b[i] = (p.rounding == TI_ROUND_RNE_SAT) ? quant_rne_sat_bits(f)
                                                      : (uint32_t)(uint8_t)cast_i8(f, TI_ROUND_TRUNC_WRAP);
            }
            wv[w4] = pack4_low_bytes(b[0], b[1], b[2], b[3]);
          }
          const int lc = oq * 2 + h16;
          st_shared_v4(orow + (uint32_t)((lc ^ (r & 7)) * 16), wv[0], wv[1], wv[2], wv[3]);
        }
      }
      fence_async_smem();
      mbar_arrive_warp(stg_full);
      if (warp == 2) {  // the warp whose first lane owns the output stores
        if (!mbar_wait_warp(stg_full, item_par, abort_flag)) { ok = false; break; }
        if (lane == 0) {
          tma_store_4d(&map_o, sb + S::O_OFF, 0, it.h, it.qi * BQ, it.b);
          tma_store_commit();
        }
      }
    }
    if (!ok && lane == 0) atomicOr(&g_status, STATUS_EPILOGUE);
    if (threadIdx.x == 64) tma_store_wait_all();
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------- host side
// [batch][seq][heads][128] int8 operand with arbitrary batch / row / head strides, viewed
// by TMA as {d, head, seq, batch}; one box = 128 rows of one head.
inline int make_head_map(CUtensorMap* map, const void* base, int64_t batch, int64_t seq, int64_t heads,
                         int64_t stride_b, int64_t stride_s, int64_t stride_h) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return TI_ERR_CUDA; }
  cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)heads, (cuuint64_t)seq, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)stride_h, (cuuint64_t)stride_s, (cuuint64_t)stride_b};
  cuuint32_t box[4] = {(cuuint32_t)HD, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("attention: cuTensorMapEncodeTiled failed with CUresult %d (strides b=%lld s=%lld h=%lld)", (int)r,
              (long long)stride_b, (long long)stride_s, (long long)stride_h);
    return TI_ERR_CUDA;
  }
  return TI_OK;
}

inline int launch(const ti_attention_params& a, int num_sms) {
  if (a.batch <= 0 || a.heads <= 0 || a.seq_q <= 0 || a.seq_k <= 0) return TI_OK;
  if (a.head_dim != HD) { set_error("attention: head_dim must be 128 (got %lld)", (long long)a.head_dim); return TI_ERR_UNSUPPORTED; }
  if (a.causal && a.seq_k < a.seq_q) { set_error("attention: causal mode needs seq_k >= seq_q"); return TI_ERR_UNSUPPORTED; }
  const int64_t st[12] = {a.q_stride_b, a.q_stride_s, a.q_stride_h, a.k_stride_b, a.k_stride_s, a.k_stride_h,
                          a.v_stride_b, a.v_stride_s, a.v_stride_h, a.o_stride_b, a.o_stride_s, a.o_stride_h};
  for (int i = 0; i < 12; ++i)
    if (st[i] <= 0 || (st[i] % 16) != 0) { set_error("attention: strides must be positive multiples of 16 bytes"); return TI_ERR_ALIGN; }
  if (((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.o) & 15) { set_error("attention: pointers must be 16-byte aligned"); return TI_ERR_ALIGN; }
  if (a.batch >= (1 << 20) || a.heads >= (1 << 16) || a.seq_q >= (1 << 24) || a.seq_k >= (1 << 24)) { set_error("attention: extent too large"); return TI_ERR_SHAPE; }
  CUtensorMap mq, mk, mv, mo;
  int rc;
  if ((rc = make_head_map(&mq, a.q, a.batch, a.seq_q, a.heads, a.q_stride_b, a.q_stride_s, a.q_stride_h)) != TI_OK) return rc;
  if ((rc = make_head_map(&mk, a.k, a.batch, a.seq_k, a.heads, a.k_stride_b, a.k_stride_s, a.k_stride_h)) != TI_OK) return rc;
  if ((rc = make_head_map(&mv, a.v, a.batch, a.seq_k, a.heads, a.v_stride_b, a.v_stride_s, a.v_stride_h)) != TI_OK) return rc;
  if ((rc = make_head_map(&mo, a.o, a.batch, a.seq_q, a.heads, a.o_stride_b, a.o_stride_s, a.o_stride_h)) != TI_OK) return rc;
  Params p;
  p.alpha_qk = a.alpha_qk; p.alpha_pv = a.alpha_pv;
  p.batch = (int)a.batch; p.heads = (int)a.heads; p.seq_q = (int)a.seq_q; p.seq_k = (int)a.seq_k;
  p.q_tiles = (int)((a.seq_q + BQ - 1) / BQ);
  p.kv_tiles = (int)((a.seq_k + BKV - 1) / BKV);
  const int64_t items = (int64_t)p.q_tiles * a.batch * a.heads;
  if (items >= (1ll << 31)) { set_error("attention: too many tiles"); return TI_ERR_SHAPE; }
  p.num_items = (int)items;
  p.causal = a.causal; p.rounding = a.rounding; p.p_mul = a.p_mul;
  static bool attr_set = false;
  if (!attr_set) {
    TI_CUDA_CHECK(cudaFuncSetAttribute(attention_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::DYN_BYTES));
    attr_set = true;
  }
  const int grid = p.num_items < num_sms ? p.num_items : num_sms;
  attention_i8_kernel<<<grid, ATT_THREADS, Smem::DYN_BYTES, (cudaStream_t)a.stream>>>(mq, mk, mv, mo, p);
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

}  // namespace attn
}  // namespace ti
