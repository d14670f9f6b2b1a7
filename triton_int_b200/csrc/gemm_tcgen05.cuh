// int8 x int8 -> int32 GEMM / batched GEMM for sm_100a.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: 128B-swizzled tiles of A [BM x 128 B] and B [BN x 128 B]
//               into a ring of shared-memory stages (plain per-CTA tensor loads)
//   warp 1      allocates TMEM, then one lane issues tcgen05.mma kind::i8
//               (M=128, N=BN, K=32 per instruction, 4 per stage) into one of two
//               TMEM accumulator buffers and commits stage/accumulator barriers
//   warps 2..9  epilogue: tcgen05.ld the int32 accumulator (warp w owns the 32 TMEM
//               lanes of quarter w%4 and one half of the tile's columns; two warps
//               per scheduler hide each other's latencies), apply the fused fp32 epilogue, stage
//               128-byte output rows in swizzled shared memory and write them
//               with TMA tensor stores (which clip ragged edges); outputs TMA
//               cannot address fall back to per-row vector/scalar stores
// Every mbarrier wait is bounded; on expiry the kernel records a status bit,
// drains and returns instead of hanging.
#pragma once

#include <cuda.h>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "ti_common.cuh"

namespace ti {
namespace tc {

constexpr int BM = 128;          // rows of A per tile = TMEM lanes
constexpr int BK = 128;          // bytes of K per stage = one 128B swizzle row
constexpr int UMMA_K = 32;       // K per tcgen05.mma kind::i8
constexpr int NUM_THREADS = 320; // 10 warps
constexpr int NUM_EPI_THREADS = 256;
constexpr int NUM_EPI_WARPS = NUM_EPI_THREADS / 32;  // barriers the epilogue signals count one arrival per warp
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s

struct Params {
  void* c;
  const void* bias;
  const float* alpha;
  const float* beta;
  int64_t c_stride_m, c_stride_n, c_stride_batch;
  int m, n, k, batch;
  int tiles_m, tiles_n, num_tiles, num_kb;
  int bias_dtype, epilogue, rounding, causal;
  int c_vec_ok;  // c_stride_n == 1 and rows start on 16-byte boundaries
  int c_tma_ok;  // map_c is valid: output written with tensor stores
  int b_mn_major;           // B is [K, N] with N contiguous ("s8t" second operand): MN-major smem tiles
  int rows_per_rank, rank;  // scatter mode: rows [r*rows_per_rank, ...) belong to rank r; this rank's slot index
  const float* residual;    // TI_EPI_DQ_ADD: fp32 [m, n] added after the dequantisation
  int64_t res_stride_m;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// SUSPEND: give the hardware a suspend-time hint, so that a waiting thread sleeps until the
// phase completes instead of re-polling.  On the power-capped GEMMs the eight epilogue
// warps wait most of every tile and their polling costs clock (measured 5 % on large
// linears); the attention kernel's waits are short and latency-critical and keep the plain form.
template <bool SUSPEND = false>
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  if constexpr (SUSPEND) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(100000u)   // nanoseconds
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  }
  return ok != 0;
}
// Bounded wait.  Returns false when the limit expired or another role already
// gave up (abort flag in shared memory).
template <bool SUSPEND = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait<SUSPEND>(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait<SUSPEND>(bar, parity)) {
    if ((++spins & (SUSPEND ? 3u : 255u)) == 0u) {   // a suspended poll already lasts up to 0.1 ms
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// ---- CTA-pair (cta_group::2) forms: the two CTAs of a cluster compute one 256-row tile;
// the even CTA issues the MMAs, each CTA loads its own A rows and its half of the B rows.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// One arrival for a whole warp: the lanes meet first, so everything each of them did
// before the call (shared-memory writes, TMEM loads, proxy fences) is ordered before the
// single arrive.  Barriers that every thread of a role signals are initialised with the
// number of WARPS (measured 2 % faster on the attention kernel than 32 arrivals per warp).
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
// Bounded wait of a whole warp with one result for all lanes, so that a later
// mbar_arrive_warp never meets a warp that has split.
template <bool SUSPEND = false>
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  // every lane polls (one elected lane polling measured a third slower on the attention kernel)
  const bool r = mbar_wait<SUSPEND>(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, r);
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tensor load whose completion is signalled on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major, 128B-swizzled shared-memory operand descriptor: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                     // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset
  d |= (uint64_t)1 << 46;                     // version
  d |= (uint64_t)2 << 61;                     // SWIZZLE_128B
  return d;
}
// MN-major, 128B-swizzled operand tile: rows are k, each row 128 contiguous bytes of n;
// groups of 8 k-rows 1024 bytes apart (stride byte offset); the next 128-wide n chunk
// `lbo_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t make_smem_desc_mn_major(uint32_t saddr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::i8 instruction descriptor: D = s32, A = B = signed int8, both K-major.
__host__ __device__ constexpr uint32_t make_idesc_i8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------ tile schedule
struct Tile {
  int batch, m_blk, n_blk;
};
constexpr int GROUP_M = 8;
__device__ __forceinline__ Tile decode_tile(int t, int tiles_m, int tiles_n) {
  Tile r;
  const int per_batch = tiles_m * tiles_n;
  r.batch = t / per_batch;
  int i = t - r.batch * per_batch;
  const int per_group = GROUP_M * tiles_n;
  const int group = i / per_group;
  const int first_m = group * GROUP_M;
  const int gsize = min(tiles_m - first_m, GROUP_M);
  const int j = i - group * per_group;
  r.m_blk = first_m + (j % gsize);
  r.n_blk = j / gsize;
  return r;
}
// Output tiles a causal consumer never reads: every column lies right of the
// diagonal of every row in the tile.
template <int BN>
__device__ __forceinline__ bool tile_skipped(const Params& p, const Tile& t) {
  if (!p.causal) return false;
  const int row_last = min(t.m_blk * BM + BM - 1, p.m - 1);
  return t.n_blk * BN > row_last + (p.n - p.m);
}

// ------------------------------------------------------------------ shared memory
template <int BN, int STAGES, bool TWO_CTA = false>
struct Smem {
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = (TWO_CTA ? BN / 2 : BN) * BK;   // a CTA pair splits the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  // output staging: 8 epilogue warps x (32 rows x 128 bytes)
  static constexpr int OUT_BUF_BYTES = 32 * 128;
  static constexpr int OUT_OFFSET = TILE_BYTES;
  static constexpr int OUT_BYTES = 8 * OUT_BUF_BYTES;
  // per-tile bias row (fp32 or raw int32 bits)
  static constexpr int BIAS_OFFSET = OUT_OFFSET + OUT_BYTES;
  static constexpr int BIAS_BYTES = BN * 4;
  // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], bias_ready, bias_free;
  // then tmem base, abort flag
  static constexpr int BAR_OFFSET = BIAS_OFFSET + BIAS_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 6;
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack to align the base to 1024
  static_assert(DYN_BYTES <= 232448, "exceeds the 227 KB shared memory of one CTA");
};

// ------------------------------------------------------------------ epilogue
template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* dst, const OutT (&v)[32], int ncols, bool vec_ok, int64_t stride_n) {
  if (vec_ok && ncols == 32) {
    constexpr int PER16 = 16 / (int)sizeof(OutT);
    const uint4* src = reinterpret_cast<const uint4*>(v);
    uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 32 / PER16; ++i) d[i] = src[i];
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) dst[(int64_t)j * stride_n] = v[j];
  }
}

// float -> int8 (round half to even, saturate) without the conversion unit: clamp,
// then add 1.5 * 2^23 so the fp32 adder rounds to an integer that sits in the low
// mantissa bits; the low byte of the result is the two's-complement int8.
__device__ __forceinline__ uint32_t quant_rne_sat_bits(float f) {
  f = fminf(fmaxf(f, -128.0f), 127.0f);
  return __float_as_uint(__fadd_rn(f, 12582912.0f));
}
__device__ __forceinline__ uint32_t pack4_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// Packed fp32 pairs with explicit rounding in the instruction, so that a multiply and the
// add that follows it are never contracted into one fused multiply-add (the epilogues
// round after every operation, as the reference's element-wise arithmetic does).
__device__ __forceinline__ float2 mul2_rn(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 add2_rn(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 fma2_rn(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}

// GELU-quant value before the int8 cast: gelu_tanh(x) * scale with
// 0.5*x*(1+tanh(u)) rewritten as x - x / (exp(2u) + 1) (two special-function
// operations per element).  Differs from the operation-by-operation form of
// ti::gelu_tanh_scaled by a few fp32 ulps.
__device__ __forceinline__ float gelu_q_fast(float x, float scale) {
  const float c2 = 2.302208198f;       // 2 * sqrt(2/pi) * log2(e)
  const float c2k = 0.1029432397f;     // c2 * 0.044715
  const float u = __fmul_rn(x, __fmaf_rn(__fmul_rn(x, x), c2k, c2));
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(u));
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__fadd_rn(e, 1.0f)));
  return __fmul_rn(__fmaf_rn(-x, r, x), scale);
}

// 32 accumulators of one row -> 32 outputs packed into 32-bit words (8 words of
// int8, 16 of fp16/bf16, 32 of fp32/int32).  `bias_c` points at this chunk's 32
// staged bias values in shared memory (already multiplied by beta for the
// scale+bias epilogues; raw int32 bits for the int32 epilogue) or is null.
template <typename OutT, int epilogue>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[32], const float* bias_c, float alpha, float beta,
                                               int rounding, uint32_t (&vw)[8 * sizeof(OutT)],
                                               const float* res = nullptr, int res_n = 0) {
  float f[32];
  if constexpr (epilogue == TI_EPI_DQ_ADD) {
    // residual + alpha * (acc + bias_i32) with one rounding: the arithmetic the dequantising
    // LayerNorm kernel does per element, so the two forms return the same bits.
    // `res` points at this thread's 32 residual values (res_n of them exist), or is null.
    float rv[32];
    if (res && res_n >= 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 t = __ldcs(reinterpret_cast<const float4*>(res + j));
        rv[j] = t.x; rv[j + 1] = t.y; rv[j + 2] = t.z; rv[j + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) rv[j] = (res && j < res_n) ? res[j] : 0.f;
    }
    if constexpr (std::is_same<OutT, float>::value) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int a = (int)r[j] + (bias_c ? __float_as_int(bias_c[j]) : 0);
        vw[j] = __float_as_uint(__fmaf_rn(__int2float_rn(a), alpha, rv[j]));
      }
    }
    return;
  }
  if constexpr (epilogue == TI_EPI_I32) {
    if constexpr (std::is_same<OutT, int32_t>::value) {
#pragma unroll
      for (int j = 0; j < 32; ++j) vw[j] = r[j] + (bias_c ? __float_as_uint(bias_c[j]) : 0u);
    }
    return;
  }
  if constexpr (epilogue == TI_EPI_SCALE) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __fmul_rn(__int2float_rn((int32_t)r[j]), alpha);
  } else if constexpr (epilogue == TI_EPI_GELU_Q) {
    // gelu_q_fast on two elements at a time with the packed fp32 instructions: every
    // operation rounds as its scalar form does, so the results are those of gelu_q_fast
    const float2 a2 = make_float2(alpha, alpha), s2 = make_float2(beta, beta);
    const float2 c2 = make_float2(2.302208198f, 2.302208198f), c2k = make_float2(0.1029432397f, 0.1029432397f);
    const float2 neg1 = make_float2(-1.0f, -1.0f);
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      float2 x = mul2_rn(make_float2(__int2float_rn((int32_t)r[j]), __int2float_rn((int32_t)r[j + 1])), a2);
      x = add2_rn(x, bias_c ? *reinterpret_cast<const float2*>(bias_c + j) : make_float2(0.f, 0.f));
      const float2 u = mul2_rn(x, fma2_rn(mul2_rn(x, x), c2k, c2));
      float e0, e1, r0, r1;
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(u.x));
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(u.y));
      const float2 d = fma2_rn(make_float2(e0, e1), neg1, neg1);   // -(e + 1): its reciprocal is -1/(e + 1)
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(d.x));
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(d.y));
      const float2 g = mul2_rn(fma2_rn(x, make_float2(r0, r1), x), s2);
      f[j] = g.x;
      f[j + 1] = g.y;
    }
  } else {  // scale + bias (+ ReLU)
    const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const float2 x = mul2_rn(make_float2(__int2float_rn((int32_t)r[j]), __int2float_rn((int32_t)r[j + 1])), a2);
      const float2 y = add2_rn(bias_c ? *reinterpret_cast<const float2*>(bias_c + j) : make_float2(0.f, 0.f), x);
      f[j] = y.x;
      f[j + 1] = y.y;
    }
  }
  if constexpr (std::is_same<OutT, int8_t>::value) {
    constexpr bool relu = (epilogue == TI_EPI_SCALE_BIAS_RELU);
    if (rounding == TI_ROUND_RNE_SAT) {
      const float2 magic2 = make_float2(12582912.0f, 12582912.0f);
      const float lo = relu ? 0.f : -128.0f;   // ReLU folded into the lower clamp
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) c[i] = fminf(fmaxf(f[j + i], lo), 127.0f);
        const float2 b01 = add2_rn(make_float2(c[0], c[1]), magic2);   // round half even; low byte = int8
        const float2 b23 = add2_rn(make_float2(c[2], c[3]), magic2);
        vw[j >> 2] = pack4_low_bytes(__float_as_uint(b01.x), __float_as_uint(b01.y), __float_as_uint(b23.x), __float_as_uint(b23.y));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        uint32_t b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          int8_t o = cast_i8(f[j + i], TI_ROUND_TRUNC_WRAP);
          if (relu && o < 0) o = 0;  // ReLU after the wrapping cast, as the reference orders it
          b[i] = (uint32_t)(uint8_t)o;
        }
        vw[j >> 2] = pack4_low_bytes(b[0], b[1], b[2], b[3]);
      }
    }
  } else if constexpr (std::is_same<OutT, int32_t>::value) {
#pragma unroll
    for (int j = 0; j < 32; ++j) vw[j] = (uint32_t)__float2int_rz(f[j]);
  } else if constexpr (std::is_same<OutT, float>::value) {
#pragma unroll
    for (int j = 0; j < 32; ++j) vw[j] = __float_as_uint(f[j]);
  } else if constexpr (std::is_same<OutT, __half>::value) {
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const __half2 h = __floats2half2_rn(f[j], f[j + 1]);
      vw[j >> 1] = *reinterpret_cast<const uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[j], f[j + 1]);
      vw[j >> 1] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
}

// `peer_maps` (scatter mode, else null): one output tensor map per tensor-parallel rank over
// that rank's receive buffer [world][rows_per_rank][n]; a finished tile is stored straight
// into the buffer of the rank that owns its rows (over NVLink for a peer), in the slot of
// the storing rank, so the reduce-scatter traffic overlaps the remaining tiles' MMAs.
template <int BN, int STAGES, typename OutT, int EPI, bool TWO_CTA = false>
__device__ __forceinline__ void gemm_body(const CUtensorMap* pa, const CUtensorMap* pb, const CUtensorMap* pc,
                                          const CUtensorMap* peer_maps, const Params& p) {
  using S = Smem<BN, STAGES, TWO_CTA>;
  // CTA pair: rank 0 issues the MMAs for both; a work unit is a 256-row tile shared by the pair
  const uint32_t pair_rank = TWO_CTA ? cluster_ctarank() : 0u;
  const int unit = TWO_CTA ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int unit_stride = TWO_CTA ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  constexpr int TILE_M = TWO_CTA ? 2 * BM : BM;
  constexpr int B_ROWS = TWO_CTA ? BN / 2 : BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + S::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  const uint32_t bias_ready_bar = bar_base + 8u * (2 * STAGES + 4);
  const uint32_t bias_free_bar = bar_base + 8u * (2 * STAGES + 5);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + S::BAR_OFFSET + S::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::BAR_OFFSET + S::NUM_BARS * 8 + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), TWO_CTA ? 2 * NUM_EPI_WARPS : NUM_EPI_WARPS);  // pair: both CTAs' epilogues
    }
    mbar_init(bias_ready_bar, NUM_EPI_WARPS);
    mbar_init(bias_free_bar, NUM_EPI_WARPS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (TWO_CTA) {
      tmem_alloc_pair(smem_u32((const void*)tmem_holder), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32((const void*)tmem_holder), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (TWO_CTA) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = unit; t < p.num_tiles && ok; t += unit_stride) {
        const Tile tile = decode_tile(t, p.tiles_m, p.tiles_n);
        if (tile_skipped<BN>(p, tile)) continue;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait<true>(empty_bar(stage), phase ^ 1u, abort_flag)) {
            atomicOr(&g_status, STATUS_PRODUCER);
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
          const uint32_t b_dst = a_dst + S::A_BYTES;
          if constexpr (TWO_CTA) {
            // both CTAs' loads complete on the even CTA's barrier, which expects the pair's bytes
            const uint32_t full_leader = map_to_cta(full_bar(stage), 0);
            if (pair_rank == 0) mbar_expect_tx(full_bar(stage), 2 * S::STAGE_BYTES);
            tma_load_3d_pair(a_dst, pa, full_leader, kb * BK, tile.m_blk * TILE_M + (int)pair_rank * BM, tile.batch);
            tma_load_3d_pair(b_dst, pb, full_leader, kb * BK, tile.n_blk * BN + (int)pair_rank * B_ROWS, tile.batch);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          mbar_expect_tx(full_bar(stage), S::STAGE_BYTES);
          tma_load_3d(a_dst, pa, full_bar(stage), kb * BK, tile.m_blk * BM, tile.batch);
          if (p.b_mn_major) {
            // [k rows][128 bytes of n] sub-tiles, one per 128 columns
#pragma unroll
            for (int c = 0; c < BN / 128; ++c)
              tma_load_3d(b_dst + (uint32_t)(c * BK * 128), pb, full_bar(stage), tile.n_blk * BN + c * 128, kb * BK, tile.batch);
          } else {
            tma_load_3d(b_dst, pb, full_bar(stage), kb * BK, tile.n_blk * BN, tile.batch);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && pair_rank == 0) {
      constexpr uint32_t idesc = make_idesc_i8(TILE_M, BN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int t = unit; t < p.num_tiles && ok; t += unit_stride) {
        const Tile tile = decode_tile(t, p.tiles_m, p.tiles_n);
        if (tile_skipped<BN>(p, tile)) continue;
        const int buf = local & 1;
        const uint32_t use = (uint32_t)(local >> 1);
        // wait until the epilogue has drained this accumulator buffer
        if (!mbar_wait<true>(acc_empty_bar(buf), (use & 1u) ^ 1u, abort_flag)) {
          atomicOr(&g_status, STATUS_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait<true>(full_bar(stage), phase, abort_flag)) {
            atomicOr(&g_status, STATUS_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * S::STAGE_BYTES;
          const uint32_t b_src = a_src + S::A_BYTES;
          const uint64_t adesc = make_smem_desc(a_src);
          if constexpr (TWO_CTA) {
            const uint64_t bdesc = make_smem_desc(b_src);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_i8_pair(tmem_d, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
            // the stage is free in both CTAs once these MMAs have read it
            umma_commit_pair(empty_bar(stage));
            umma_commit_pair(map_to_cta(empty_bar(stage), 1));
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          if (p.b_mn_major) {
            const uint64_t bdesc = make_smem_desc_mn_major(b_src, BK * 128);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)  // 32 k-rows of 128 bytes per step: +4096 bytes
              umma_i8(tmem_d, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(256 * k), idesc | (1u << 16),
                      (kb > 0 || k > 0) ? 1u : 0u);
          } else {
            const uint64_t bdesc = make_smem_desc(b_src);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // advance 32 bytes of K inside the 128-byte swizzle row: +2 in 16-byte units
              umma_i8(tmem_d, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(empty_bar(stage));  // the stage may be refilled once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if constexpr (TWO_CTA) {
            umma_commit_pair(acc_full_bar(buf));
            umma_commit_pair(map_to_cta(acc_full_bar(buf), 1));
          } else {
            umma_commit(acc_full_bar(buf));
          }
        }
        ++local;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;       // TMEM lanes [32*quarter, 32*quarter+32)
    const int half = (warp - 2) >> 2;   // which half of the tile's columns
    const int epi_tid = threadIdx.x - 64;
    const float alpha = p.alpha ? *p.alpha : 1.0f;
    const float beta = p.beta ? *p.beta : 1.0f;
    constexpr int ESZ = (int)sizeof(OutT);
    constexpr int HALF_N = BN / 2;
    constexpr int ROW_BYTES = (HALF_N * ESZ < 128) ? HALF_N * ESZ : 128;  // one staged output row
    constexpr int COLS_PER_BUF = ROW_BYTES / ESZ;
    constexpr int CHUNKS_PER_BUF = COLS_PER_BUF / 32;
    constexpr bool SWZ = (ROW_BYTES == 128);
    constexpr int NV = 32 * ESZ / 16;  // 16-byte pieces per 32-column chunk
    constexpr int NCH = HALF_N / 32;   // 32-column chunks per warp
    static_assert(CHUNKS_PER_BUF >= 1 && NCH >= 1, "tile width");
    float* bias_s = reinterpret_cast<float*>(smem + S::BIAS_OFFSET);
    const uint32_t buf_addr = smem_base + S::OUT_OFFSET + (uint32_t)((warp - 2) * S::OUT_BUF_BYTES);
    const bool has_bias = p.bias != nullptr;
    int local = 0;
    bool ok = true;
    for (int t = unit; t < p.num_tiles && ok; t += unit_stride) {
      const Tile tile = decode_tile(t, p.tiles_m, p.tiles_n);
      if (tile_skipped<BN>(p, tile)) continue;
      const int buf = local & 1;
      const uint32_t use = (uint32_t)(local >> 1);
      const int col0 = tile.n_blk * BN;
      if (has_bias) {
        // stage this tile's bias row once the previous tile's readers are done
        if (!mbar_wait_warp<true>(bias_free_bar, ((uint32_t)local & 1u) ^ 1u, abort_flag)) {
          if (lane == 0) atomicOr(&g_status, STATUS_EPILOGUE);
          ok = false;
          break;
        }
        for (int c = epi_tid; c < BN; c += NUM_EPI_THREADS) {
          const int col = col0 + c;
          float bv = 0.f;
          if (col < p.n) {
            if constexpr (EPI == TI_EPI_I32 || EPI == TI_EPI_DQ_ADD) {
              bv = __int_as_float(((const int32_t*)p.bias)[col]);
            } else {
              bv = load_bias_f32(p.bias, p.bias_dtype, col);
              if constexpr (EPI == TI_EPI_SCALE_BIAS || EPI == TI_EPI_SCALE_BIAS_RELU) bv = __fmul_rn(bv, beta);
            }
          }
          bias_s[c] = bv;
        }
        mbar_arrive_warp(bias_ready_bar);
        if (!mbar_wait_warp<true>(bias_ready_bar, (uint32_t)local & 1u, abort_flag)) {
          if (lane == 0) atomicOr(&g_status, STATUS_EPILOGUE);
          ok = false;
          break;
        }
      }
      if (!mbar_wait_warp<true>(acc_full_bar(buf), use & 1u, abort_flag)) {
        if (lane == 0) atomicOr(&g_status, STATUS_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row0 = tile.m_blk * TILE_M + (int)pair_rank * BM + quarter * 32;
      const int row = row0 + lane;
      const bool row_ok = row < p.m;
      OutT* c_row = reinterpret_cast<OutT*>(p.c) + (int64_t)tile.batch * p.c_stride_batch + (int64_t)row * p.c_stride_m;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * HALF_N);

      auto emit = [&](const int chunk, const uint32_t (&r)[32]) {
        const int ccol = half * HALF_N + chunk * 32;  // column inside the tile
        const int col = col0 + ccol;
        alignas(16) uint32_t vw[8 * ESZ];
        if (col < p.n) {
          if constexpr (EPI == TI_EPI_DQ_ADD) {
            const float* res = row_ok ? p.residual + (int64_t)row * p.res_stride_m + col : nullptr;
            epilogue_chunk<OutT, EPI>(r, has_bias ? bias_s + ccol : nullptr, alpha, beta, p.rounding, vw, res, p.n - col);
          } else {
            epilogue_chunk<OutT, EPI>(r, has_bias ? bias_s + ccol : nullptr, alpha, beta, p.rounding, vw);
          }
        }
        if (p.c_tma_ok) {
          const int sub = chunk % CHUNKS_PER_BUF;
          if (sub == 0) {
            // the previous store issued from this warp's buffer must have finished reading it
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
          }
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int lc = sub * NV + i;
            const int pc = SWZ ? (lc ^ (lane & 7)) : lc;
            st_shared_v4(buf_addr + (uint32_t)(lane * ROW_BYTES + pc * 16), vw[4 * i], vw[4 * i + 1], vw[4 * i + 2], vw[4 * i + 3]);
          }
          if (sub == CHUNKS_PER_BUF - 1) {
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int bcol = col0 + half * HALF_N + (chunk / CHUNKS_PER_BUF) * COLS_PER_BUF;
              if (bcol < p.n && row0 < p.m) {
                if (peer_maps) {
                  const int owner = row0 / p.rows_per_rank;
                  tma_store_3d(peer_maps + owner, buf_addr, bcol, row0 - owner * p.rows_per_rank, p.rank);
                } else {
                  tma_store_3d(pc, buf_addr, bcol, row0, tile.batch);
                }
              }
              tma_store_commit();
            }
          }
        } else if (row_ok && col < p.n) {
          store_row32<OutT>(c_row + (int64_t)col * p.c_stride_n, *reinterpret_cast<const OutT(*)[32]>(vw),
                            min(32, p.n - col), p.c_vec_ok != 0, p.c_stride_n);
        }
      };
      auto release_acc = [&]() {
        // every accumulator this warp needs is in registers: hand the buffer back to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (TWO_CTA) mbar_arrive_cluster(map_to_cta(acc_empty_bar(buf), 0));  // the MMA issuer lives in the even CTA
          else mbar_arrive(acc_empty_bar(buf));
        }
      };

      // one call site for the chunk body keeps the instruction footprint small; the two
      // epilogue warps of each scheduler cover each other's TMEM-load latency
#pragma unroll 1
      for (int c = 0; c < NCH; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), r);
        tmem_ld_wait();
        if (c == NCH - 1) release_acc();
        emit(c, r);
      }
      if (has_bias) mbar_arrive_warp(bias_free_bar);
      ++local;
    }
    if (lane == 0) tma_store_wait_all();
    __syncwarp();
  }

  // ---------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag) {
    // let loads already in flight land before the shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if constexpr (TWO_CTA) cluster_sync_all();  // neither CTA frees TMEM or exits while its peer may still signal it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (TWO_CTA) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// CTA-pair variant: clusters of two CTAs, 256 x 256 output tile per pair (each CTA 128 rows),
// K-major B only, six 32 KB stages per CTA.
template <int STAGES, typename OutT, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_i8_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                            const __grid_constant__ CUtensorMap map_c, const Params p) {
  gemm_body<256, STAGES, OutT, EPI, true>(&map_a, &map_b, &map_c, nullptr, p);
}

template <int BN, int STAGES, typename OutT, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_c, const Params p) {
  gemm_body<BN, STAGES, OutT, EPI>(&map_a, &map_b, &map_c, nullptr, p);
}

struct PeerMaps {
  CUtensorMap m[8];
};
template <int BN, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_i8_tcgen05_scatter_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                               const __grid_constant__ PeerMaps peers, const Params p) {
  gemm_body<BN, STAGES, int32_t, TI_EPI_I32>(&map_a, &map_b, &peers.m[0], &peers.m[0], p);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// Tensor map over an int8 operand viewed as [batch][rows][k] with k contiguous.
inline int make_operand_map(CUtensorMap* map, const void* base, int64_t k, int64_t rows, int64_t batch,
                            int64_t row_stride, int64_t batch_stride, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return TI_ERR_CUDA;
  }
  cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)row_stride, (cuuint64_t)(batch > 1 ? batch_stride : row_stride * rows)};
  if (strides[1] == 0 || (strides[1] % 16) != 0) strides[1] = 16;  // single batch: never used to address
  cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (k=%lld rows=%lld batch=%lld row_stride=%lld)", (int)r,
              (long long)k, (long long)rows, (long long)batch, (long long)row_stride);
    return TI_ERR_CUDA;
  }
  return TI_OK;
}

// Tensor map over the output viewed as [batch][m][n], n contiguous; box = 32 rows x one
// staged row (128 bytes, 128B-swizzled, or a narrower unswizzled row for small tiles).
inline int make_output_map(CUtensorMap* map, void* base, int esz, int64_t n, int64_t m, int64_t batch,
                           int64_t row_stride, int64_t batch_stride, int box_cols, bool swizzle128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return TI_ERR_CUDA;
  const CUtensorMapDataType dt = esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                               : esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)(row_stride * esz), (cuuint64_t)((batch > 1 ? batch_stride : row_stride * m) * esz)};
  if (strides[1] == 0 || (strides[1] % 16) != 0) strides[1] = 16;
  cuuint32_t box[3] = {(cuuint32_t)box_cols, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TI_OK : TI_ERR_CUDA;
}

// True when the tensor-map path can address this problem: both operands K-contiguous,
// 16-byte aligned bases and 16-byte multiple row/batch strides.
// B given as [K, N] with N contiguous and not also K-contiguous.
inline bool b_is_mn_major(const ti_gemm_params& g) { return g.b_stride_k != 1 && g.b_stride_n == 1; }

inline bool eligible(const ti_gemm_params& g) {
  if (g.m <= 0 || g.n <= 0 || g.k <= 0 || g.batch <= 0) return false;
  if (g.a_stride_k != 1) return false;
  if (((uintptr_t)g.a & 15) || ((uintptr_t)g.b & 15)) return false;
  if ((g.a_stride_m % 16) || g.a_stride_m < g.k) return false;
  if (b_is_mn_major(g)) {
    if ((g.b_stride_k % 16) || g.b_stride_k < g.n) return false;   // rows of K, 16-byte multiples
  } else {
    if (g.b_stride_k != 1 || (g.b_stride_n % 16) || g.b_stride_n < g.k) return false;
  }
  if (g.batch > 1 && ((g.a_stride_batch % 16) || (g.b_stride_batch % 16))) return false;
  if (g.batch > 1 && (g.a_stride_batch <= 0 || g.b_stride_batch <= 0)) return false;
  if (g.m >= (1ll << 31) || g.n >= (1ll << 31) || g.k >= (1ll << 31) || g.batch >= (1ll << 31)) return false;
  return true;
}

// Tensor map over an MN-major B operand viewed as [batch][k][n] with n contiguous; box = 128 k-rows x 128 bytes of n.
inline int make_operand_map_mn(CUtensorMap* map, const void* base, int64_t n, int64_t k, int64_t batch,
                               int64_t k_stride, int64_t batch_stride) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return TI_ERR_CUDA; }
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)k, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)k_stride, (cuuint64_t)(batch > 1 ? batch_stride : k_stride * k)};
  if (strides[1] == 0 || (strides[1] % 16) != 0) strides[1] = 16;
  cuuint32_t box[3] = {128, (cuuint32_t)BK, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (MN-major B) failed with CUresult %d", (int)r); return TI_ERR_CUDA; }
  return TI_OK;
}

template <int BN, int STAGES, typename OutT, int EPI>
int launch_cfg(const ti_gemm_params& g, int num_sms) {
  using S = Smem<BN, STAGES>;
  CUtensorMap map_a, map_b;
  int rc = make_operand_map(&map_a, g.a, g.k, g.m, g.batch, g.a_stride_m, g.a_stride_batch, BM);
  if (rc != TI_OK) return rc;
  const bool mn = b_is_mn_major(g);
  rc = mn ? make_operand_map_mn(&map_b, g.b, g.n, g.k, g.batch, g.b_stride_k, g.b_stride_batch)
          : make_operand_map(&map_b, g.b, g.k, g.n, g.batch, g.b_stride_n, g.b_stride_batch, BN);
  if (rc != TI_OK) return rc;

  Params p;
  p.b_mn_major = mn ? 1 : 0;
  p.c = g.c;
  p.bias = g.bias;
  p.alpha = g.alpha;
  p.beta = g.beta;
  p.c_stride_m = g.c_stride_m;
  p.c_stride_n = g.c_stride_n;
  p.c_stride_batch = g.c_stride_batch;
  p.m = (int)g.m; p.n = (int)g.n; p.k = (int)g.k; p.batch = (int)g.batch;
  p.tiles_m = (int)((g.m + BM - 1) / BM);
  p.tiles_n = (int)((g.n + BN - 1) / BN);
  const int64_t nt = (int64_t)p.tiles_m * p.tiles_n * g.batch;
  if (nt >= (1ll << 31)) { set_error("too many tiles"); return TI_ERR_SHAPE; }
  p.num_tiles = (int)nt;
  p.num_kb = (int)((g.k + BK - 1) / BK);
  p.bias_dtype = g.bias_dtype;
  p.epilogue = g.epilogue;
  p.rounding = g.rounding;
  p.causal = g.causal;
  p.rows_per_rank = 0; p.rank = 0;
  p.residual = g.residual; p.res_stride_m = g.residual_stride_m;
  const int64_t esz = (int64_t)sizeof(OutT);
  p.c_vec_ok = (g.c_stride_n == 1) && (((uintptr_t)g.c & 15) == 0) && ((g.c_stride_m * esz) % 16 == 0) &&
               ((g.c_stride_batch * esz) % 16 == 0);

  auto kern = gemm_i8_tcgen05_kernel<BN, STAGES, OutT, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    TI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::DYN_BYTES));
    attr_set = true;
  }
  CUtensorMap map_c;
  memset(&map_c, 0, sizeof(map_c));
  p.c_tma_ok = 0;
  if (p.c_vec_ok) {
    constexpr int ROW_BYTES = ((BN / 2) * (int)sizeof(OutT) < 128) ? (BN / 2) * (int)sizeof(OutT) : 128;
    if (make_output_map(&map_c, g.c, (int)sizeof(OutT), g.n, g.m, g.batch, g.c_stride_m, g.c_stride_batch,
                        ROW_BYTES / (int)sizeof(OutT), ROW_BYTES == 128) == TI_OK)
      p.c_tma_ok = 1;
  }
  const int grid = p.num_tiles < num_sms ? p.num_tiles : num_sms;
  kern<<<grid, NUM_THREADS, S::DYN_BYTES, (cudaStream_t)g.stream>>>(map_a, map_b, map_c, p);
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

// CTA-pair launch: 256 x 256 tiles, one per cluster of two CTAs.
template <typename OutT, int EPI>
int launch_pair_cfg(const ti_gemm_params& g, int num_sms) {
  constexpr int STAGES = 6;
  using S = Smem<256, STAGES, true>;
  CUtensorMap map_a, map_b, map_c;
  int rc = make_operand_map(&map_a, g.a, g.k, g.m, g.batch, g.a_stride_m, g.a_stride_batch, BM);
  if (rc != TI_OK) return rc;
  rc = make_operand_map(&map_b, g.b, g.k, g.n, g.batch, g.b_stride_n, g.b_stride_batch, 128);
  if (rc != TI_OK) return rc;
  Params p;
  p.c = g.c; p.bias = g.bias; p.alpha = g.alpha; p.beta = g.beta;
  p.c_stride_m = g.c_stride_m; p.c_stride_n = g.c_stride_n; p.c_stride_batch = g.c_stride_batch;
  p.m = (int)g.m; p.n = (int)g.n; p.k = (int)g.k; p.batch = (int)g.batch;
  p.tiles_m = (int)((g.m + 2 * BM - 1) / (2 * BM));
  p.tiles_n = (int)((g.n + 255) / 256);
  const int64_t nt = (int64_t)p.tiles_m * p.tiles_n * g.batch;
  if (nt >= (1ll << 31)) { set_error("too many tiles"); return TI_ERR_SHAPE; }
  p.num_tiles = (int)nt;
  p.num_kb = (int)((g.k + BK - 1) / BK);
  p.bias_dtype = g.bias_dtype; p.epilogue = g.epilogue; p.rounding = g.rounding; p.causal = 0;
  p.b_mn_major = 0; p.rows_per_rank = 0; p.rank = 0;
  p.residual = g.residual; p.res_stride_m = g.residual_stride_m;
  const int64_t esz = (int64_t)sizeof(OutT);
  p.c_vec_ok = (g.c_stride_n == 1) && (((uintptr_t)g.c & 15) == 0) && ((g.c_stride_m * esz) % 16 == 0) &&
               ((g.c_stride_batch * esz) % 16 == 0);
  memset(&map_c, 0, sizeof(map_c));
  p.c_tma_ok = 0;
  if (p.c_vec_ok) {
    constexpr int ROW_BYTES = (128 * (int)sizeof(OutT) < 128) ? 128 * (int)sizeof(OutT) : 128;
    if (make_output_map(&map_c, g.c, (int)sizeof(OutT), g.n, g.m, g.batch, g.c_stride_m, g.c_stride_batch,
                        ROW_BYTES / (int)sizeof(OutT), true) == TI_OK)
      p.c_tma_ok = 1;
  }
  auto kern = gemm_i8_tcgen05_pair_kernel<STAGES, OutT, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    TI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::DYN_BYTES));
    attr_set = true;
  }
  const int pairs = num_sms / 2;
  const int clusters = p.num_tiles < pairs ? p.num_tiles : pairs;
  kern<<<2 * clusters, NUM_THREADS, S::DYN_BYTES, (cudaStream_t)g.stream>>>(map_a, map_b, map_c, p);
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

// 0: never; 1: when the problem fills the pairs (default); 2: always when addressable
inline int pair_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("TRITON_INT_GEMM_PAIR");
    mode = e ? atoi(e) : 1;
  }
  return mode;
}
inline bool use_pair(const ti_gemm_params& g, int num_sms) {
  const int mode = pair_mode();
  if (mode == 0 || b_is_mn_major(g) || g.causal || g.n <= 128 || g.m <= 128) return false;
  if (mode == 2) return true;
  const int64_t tiles = ((g.m + 255) / 256) * ((g.n + 255) / 256) * g.batch;
  return tiles >= num_sms / 2 && g.k >= 1024;
}

// Row-parallel linear whose int32 tiles go straight to the ranks that own their rows.
template <int BN, int STAGES>
int launch_scatter_cfg(const ti_gemm_params& g, const ti_gemm_scatter& sc, int num_sms) {
  using S = Smem<BN, STAGES>;
  CUtensorMap map_a, map_b;
  int rc = make_operand_map(&map_a, g.a, g.k, g.m, 1, g.a_stride_m, 0, BM);
  if (rc != TI_OK) return rc;
  rc = make_operand_map(&map_b, g.b, g.k, g.n, 1, g.b_stride_n, 0, BN);
  if (rc != TI_OK) return rc;
  PeerMaps peers;
  memset(&peers, 0, sizeof(peers));
  constexpr int ROW_BYTES = ((BN / 2) * 4 < 128) ? (BN / 2) * 4 : 128;
  for (int r = 0; r < sc.world; ++r) {
    rc = make_output_map(&peers.m[r], sc.recv[r], 4, g.n, sc.rows_per_rank, sc.world, g.n, sc.rows_per_rank * g.n,
                         ROW_BYTES / 4, ROW_BYTES == 128);
    if (rc != TI_OK) { set_error("scatter: tensor map over rank %d's receive buffer could not be encoded", r); return rc; }
  }
  Params p;
  p.c = nullptr; p.bias = nullptr; p.alpha = nullptr; p.beta = nullptr;
  p.c_stride_m = g.n; p.c_stride_n = 1; p.c_stride_batch = 0;
  p.m = (int)g.m; p.n = (int)g.n; p.k = (int)g.k; p.batch = 1;
  p.tiles_m = (int)((g.m + BM - 1) / BM);
  p.tiles_n = (int)((g.n + BN - 1) / BN);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.num_kb = (int)((g.k + BK - 1) / BK);
  p.bias_dtype = TI_I32; p.epilogue = TI_EPI_I32; p.rounding = g.rounding; p.causal = 0;
  p.c_vec_ok = 1; p.c_tma_ok = 1;
  p.rows_per_rank = (int)sc.rows_per_rank; p.rank = sc.rank; p.b_mn_major = 0;
  p.residual = nullptr; p.res_stride_m = 0;
  auto kern = gemm_i8_tcgen05_scatter_kernel<BN, STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    TI_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::DYN_BYTES));
    attr_set = true;
  }
  const int grid = p.num_tiles < num_sms ? p.num_tiles : num_sms;
  kern<<<grid, NUM_THREADS, S::DYN_BYTES, (cudaStream_t)g.stream>>>(map_a, map_b, peers, p);
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

inline int launch_scatter(const ti_gemm_params& g, const ti_gemm_scatter& sc, int num_sms) {
  if (g.batch != 1 || !eligible(g) || b_is_mn_major(g)) { set_error("scatter: needs one K-contiguous, 16-byte aligned problem"); return TI_ERR_ALIGN; }
  if (sc.world < 1 || sc.world > 8 || sc.rank < 0 || sc.rank >= sc.world) { set_error("scatter: bad world/rank"); return TI_ERR_UNSUPPORTED; }
  if (sc.rows_per_rank <= 0 || sc.rows_per_rank % BM != 0 || sc.rows_per_rank * sc.world != g.m || (g.n % 4) != 0) {
    set_error("scatter: rows_per_rank must be a multiple of 128 with world * rows_per_rank == m, and n a multiple of 4");
    return TI_ERR_SHAPE;
  }
  for (int r = 0; r < sc.world; ++r)
    if (!sc.recv[r] || ((uintptr_t)sc.recv[r] & 15)) { set_error("scatter: null or misaligned receive buffer %d", r); return TI_ERR_ALIGN; }
  if (g.n > 128) return launch_scatter_cfg<256, 4>(g, sc, num_sms);
  if (g.n > 64) return launch_scatter_cfg<128, 6>(g, sc, num_sms);
  return launch_scatter_cfg<64, 8>(g, sc, num_sms);
}

template <typename OutT, int EPI>
int launch_epi(const ti_gemm_params& g, int num_sms) {
  if (use_pair(g, num_sms)) return launch_pair_cfg<OutT, EPI>(g, num_sms);
  // 128x256 tiles when N is wide enough to fill them, else 128x128 / 128x64
  if (g.n > 128) return launch_cfg<256, 4, OutT, EPI>(g, num_sms);
  if (g.n > 64 || b_is_mn_major(g)) return launch_cfg<128, 6, OutT, EPI>(g, num_sms);  // MN-major tiles are 128 columns wide
  return launch_cfg<64, 8, OutT, EPI>(g, num_sms);
}

// ------------------------------------------------------------------ split-K
// Second step of a split-K GEMM: out = epilogue(sum_s ws[s][m][n]).  The int32 sum is
// exact in any order; the epilogue arithmetic is the one of the fused epilogue.
struct ReduceParams {
  const int32_t* ws;
  void* c;
  const void* bias;
  const float* alpha;
  const float* beta;
  int64_t m, n, c_stride_m, c_stride_n;
  int splits, bias_dtype, epilogue, rounding;
};

template <typename OutT>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const ReduceParams p) {
  const int64_t quads = p.n >> 2;  // n is a multiple of 4 on this path
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.m * quads) return;
  const int64_t row = idx / quads;
  const int64_t col = (idx - row * quads) << 2;
  const int64_t plane = p.m * p.n;
  const int32_t* src = p.ws + row * p.n + col;
  int4 a = make_int4(0, 0, 0, 0);
  for (int s = 0; s < p.splits; ++s) {
    const int4 v = __ldcs(reinterpret_cast<const int4*>(src + (int64_t)s * plane));
    a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
  }
  const int32_t acc[4] = {a.x, a.y, a.z, a.w};
  const float alpha = p.alpha ? *p.alpha : 1.0f;
  const float beta = p.beta ? *p.beta : 1.0f;
  OutT* dst = reinterpret_cast<OutT*>(p.c) + row * p.c_stride_m + col * p.c_stride_n;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    OutT o;
    if (p.epilogue == TI_EPI_I32) {
      int32_t v = acc[j];
      if (p.bias) v += ((const int32_t*)p.bias)[col + j];
      if constexpr (sizeof(OutT) == 4) *reinterpret_cast<int32_t*>(&o) = v; else o = OutT();
    } else {
      const float b = p.bias ? load_bias_f32(p.bias, p.bias_dtype, col + j) : 0.f;
      float f;
      if (p.epilogue == TI_EPI_GELU_Q) {
        f = gelu_q_fast(__fadd_rn(__fmul_rn(__int2float_rn(acc[j]), alpha), b), beta);
      } else {
        f = epilogue_f32(acc[j], b, alpha, beta, p.epilogue);
      }
      o = OutCast<OutT>::from(f, p.rounding);
      if constexpr (sizeof(OutT) == 1) {
        if (p.epilogue == TI_EPI_SCALE_BIAS_RELU) o = o < 0 ? (OutT)0 : o;
      }
    }
    dst[j * p.c_stride_n] = o;
  }
}

// How many ways to split K: only for single (non-batched) problems whose tiles leave more
// than half of the SMs idle, K at least 8 stages long, N a multiple of 4.  The split count
// divides the number of 128-byte K blocks so every part is whole.
inline int pick_splits(const ti_gemm_params& g, int num_sms) {
  if (g.batch != 1 || g.causal || (g.n % 4) != 0 || (g.k % BK) != 0 || b_is_mn_major(g) || g.epilogue == TI_EPI_DQ_ADD) return 1;
  const int bn = g.n > 128 ? 256 : (g.n > 64 ? 128 : 64);
  const int64_t tiles = ((g.m + BM - 1) / BM) * ((g.n + bn - 1) / bn);
  const int64_t kb = g.k / BK;
  if (tiles * 2 > num_sms || kb < 8) return 1;
  int best = 1;
  for (int s = 2; s <= 32; ++s)
    if (kb % s == 0 && kb / s >= 2 && tiles * s <= num_sms) best = s;
  return best;
}

inline int64_t workspace_bytes(const ti_gemm_params& g, int num_sms) {
  if (!eligible(g)) return 0;
  const int s = pick_splits(g, num_sms);
  return s > 1 ? (int64_t)s * g.m * g.n * 4 : 0;
}

inline int launch_plain(const ti_gemm_params& g, int num_sms);

inline int launch(const ti_gemm_params& g, int num_sms) {
  const int splits = pick_splits(g, num_sms);
  const int64_t need = splits > 1 ? (int64_t)splits * g.m * g.n * 4 : 0;
  if (splits <= 1 || !g.workspace || g.workspace_bytes < need || ((uintptr_t)g.workspace & 15)) return launch_plain(g, num_sms);
  // step 1: the K parts as a batched GEMM into the workspace (raw int32 accumulators)
  ti_gemm_params part = g;
  const int64_t ks = g.k / splits;
  part.k = ks;
  part.batch = splits;
  part.a_stride_batch = ks;   // part s starts ks elements further along K
  part.b_stride_batch = ks;
  part.c = g.workspace;
  part.c_stride_m = g.n; part.c_stride_n = 1; part.c_stride_batch = g.m * g.n;
  part.bias = nullptr; part.alpha = nullptr; part.beta = nullptr;
  part.out_dtype = TI_I32; part.epilogue = TI_EPI_I32;
  part.workspace = nullptr; part.workspace_bytes = 0;
  int rc = launch_plain(part, num_sms);
  if (rc != TI_OK) return launch_plain(g, num_sms);  // (a driver that refuses the K-part view: unsplit)
  // step 2: exact sum + epilogue
  ReduceParams r;
  r.ws = (const int32_t*)g.workspace; r.c = g.c; r.bias = g.bias; r.alpha = g.alpha; r.beta = g.beta;
  r.m = g.m; r.n = g.n; r.c_stride_m = g.c_stride_m; r.c_stride_n = g.c_stride_n;
  r.splits = splits; r.bias_dtype = g.bias_dtype; r.epilogue = g.epilogue; r.rounding = g.rounding;
  const int64_t threads = g.m * (g.n >> 2);
  const unsigned grid = (unsigned)((threads + 255) / 256);
  cudaStream_t st = (cudaStream_t)g.stream;
  switch (g.out_dtype) {
    case TI_I8: splitk_reduce_kernel<int8_t><<<grid, 256, 0, st>>>(r); break;
    case TI_I32: splitk_reduce_kernel<int32_t><<<grid, 256, 0, st>>>(r); break;
    case TI_F32: splitk_reduce_kernel<float><<<grid, 256, 0, st>>>(r); break;
    case TI_F16: splitk_reduce_kernel<__half><<<grid, 256, 0, st>>>(r); break;
    case TI_BF16: splitk_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(r); break;
    default: set_error("unsupported output dtype %d", g.out_dtype); return TI_ERR_DTYPE;
  }
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

inline int launch_plain(const ti_gemm_params& g, int num_sms) {
  const int ep = g.epilogue;
  switch (g.out_dtype) {
    case TI_I8:
      if (ep == TI_EPI_SCALE) return launch_epi<int8_t, TI_EPI_SCALE>(g, num_sms);
      if (ep == TI_EPI_SCALE_BIAS) return launch_epi<int8_t, TI_EPI_SCALE_BIAS>(g, num_sms);
      if (ep == TI_EPI_SCALE_BIAS_RELU) return launch_epi<int8_t, TI_EPI_SCALE_BIAS_RELU>(g, num_sms);
      if (ep == TI_EPI_GELU_Q) return launch_epi<int8_t, TI_EPI_GELU_Q>(g, num_sms);
      break;
    case TI_I32:
      if (ep == TI_EPI_I32) return launch_epi<int32_t, TI_EPI_I32>(g, num_sms);
      if (ep == TI_EPI_SCALE) return launch_epi<int32_t, TI_EPI_SCALE>(g, num_sms);
      if (ep == TI_EPI_SCALE_BIAS) return launch_epi<int32_t, TI_EPI_SCALE_BIAS>(g, num_sms);
      break;
    case TI_F32:
      if (ep == TI_EPI_SCALE) return launch_epi<float, TI_EPI_SCALE>(g, num_sms);
      if (ep == TI_EPI_SCALE_BIAS) return launch_epi<float, TI_EPI_SCALE_BIAS>(g, num_sms);
      if (ep == TI_EPI_DQ_ADD) return launch_epi<float, TI_EPI_DQ_ADD>(g, num_sms);
      break;
    case TI_F16:
      if (ep == TI_EPI_SCALE) return launch_epi<__half, TI_EPI_SCALE>(g, num_sms);
      if (ep == TI_EPI_SCALE_BIAS) return launch_epi<__half, TI_EPI_SCALE_BIAS>(g, num_sms);
      break;
    case TI_BF16:
      if (ep == TI_EPI_SCALE) return launch_epi<__nv_bfloat16, TI_EPI_SCALE>(g, num_sms);
      if (ep == TI_EPI_SCALE_BIAS) return launch_epi<__nv_bfloat16, TI_EPI_SCALE_BIAS>(g, num_sms);
      break;
  }
  set_error("unsupported output dtype / epilogue combination (%d, %d)", g.out_dtype, ep);
  return TI_ERR_DTYPE;
}

}  // namespace tc
}  // namespace ti
