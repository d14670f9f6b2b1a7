// Memory-bound row kernels: the LayerNorm family (with optional int32 dequant +
// residual add in front and int8 quantisation behind), the stand-alone int8 GELU
// and the causal softmax -> int8 step between the two attention BMMs.
// All of them read each input byte once with 16-byte (or 8-byte) vector loads,
// keep the row in registers, reduce with warp shuffles + one shared-memory hop,
// and write each output byte once.
#pragma once

#include <type_traits>

#include "ti_common.cuh"

namespace ti {
namespace row {

// ------------------------------------------------------------------ reductions
// A row is owned by `tpr` consecutive threads (a multiple of 32) of the CTA.
template <bool IS_MAX>
__device__ __forceinline__ float row_reduce(float v, int tpr, int tid_in_row, int row_in_cta, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, other) : v + other;
  }
  if (tpr == 32) return v;
  const int warps = tpr >> 5;
  float* r = red + row_in_cta * 32;
  __syncthreads();  // previous use of `red` is over
  if ((tid_in_row & 31) == 0) r[tid_in_row >> 5] = v;
  __syncthreads();
  float t = r[0];
  for (int w = 1; w < warps; ++w) t = IS_MAX ? fmaxf(t, r[w]) : t + r[w];
  return t;
}

// ------------------------------------------------------------------ typed 4-element access
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&o)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&o)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  }
};
template <> struct Vec4<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&o)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __half2 a = *reinterpret_cast<const __half2*>(&v.x), b = *reinterpret_cast<const __half2*>(&v.y);
    o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(__half* p, const float (&o)[4]) {
    __half2 a = __halves2half2(__float2half_rn(o[0]), __float2half_rn(o[1]));
    __half2 b = __halves2half2(__float2half_rn(o[2]), __float2half_rn(o[3]));
    uint2 v;
    v.x = *reinterpret_cast<unsigned*>(&a); v.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = v;
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&o)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
    o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&o)[4]) {
    __nv_bfloat16 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __float2bfloat16_rn(o[i]);
    *reinterpret_cast<uint2*>(p) = *reinterpret_cast<uint2*>(h);
  }
};
template <> struct Vec4<int8_t> {
  static __device__ __forceinline__ void store_q(int8_t* p, const float (&o)[4], int rounding) {
    char4 c;
    c.x = cast_i8(o[0], rounding); c.y = cast_i8(o[1], rounding);
    c.z = cast_i8(o[2], rounding); c.w = cast_i8(o[3], rounding);
    *reinterpret_cast<char4*>(p) = c;
  }
};

// round a float to the storage type and back (the skip variants add the skip
// tensor to the already-rounded LayerNorm output, kernels/fused.py:622-635)
template <typename T> __device__ __forceinline__ float round_through(float f);
template <> __device__ __forceinline__ float round_through<float>(float f) { return f; }
template <> __device__ __forceinline__ float round_through<__half>(float f) { return __half2float(__float2half_rn(f)); }
template <> __device__ __forceinline__ float round_through<__nv_bfloat16>(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }

struct LnParams {
  const void* x;
  const float* residual_in;
  float* residual_out;
  const int32_t* bias_i32;
  const void* gamma;
  const void* beta;
  const void* skip;
  void* out;
  void* out2;
  const float* dq_scale_dev;
  int64_t rows, n;
  int64_t x_row_stride, x_col_stride, out_row_stride, out_col_stride;
  float eps, dq_scale;
  int rounding, rms;
};

// ------------------------------------------------------------------ LayerNorm, vector path
// XT: float / half / bf16 / int32 (dequant+residual).  PT: dtype of gamma, beta, skip and
// of a non-int8 output.  QOUT: int8 output.  MAXV float4-groups per thread.
template <typename XT, typename PT, bool QOUT, int MAXV>
__global__ void __launch_bounds__(512, (MAXV <= 4 ? 3 : (MAXV == 8 ? 2 : 1)))
layernorm_vec_kernel(const LnParams p, const int tpr) {
  __shared__ float red[32 * 32];
  const int rows_per_cta = blockDim.x / tpr;
  const int row_in_cta = threadIdx.x / tpr;
  const int tid = threadIdx.x - row_in_cta * tpr;
  const int64_t row = (int64_t)blockIdx.x * rows_per_cta + row_in_cta;
  const bool row_ok = row < p.rows;
  const int n = (int)p.n;
  float v[MAXV][4];

  // ---- load (and dequantise + add the residual) ----
  float dq = p.dq_scale;
  if constexpr (std::is_same<XT, int32_t>::value) {
    if (p.dq_scale_dev) dq = *p.dq_scale_dev;
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int col = (i * tpr + tid) * 4;
    if (row_ok && col < n) {
      if constexpr (std::is_same<XT, int32_t>::value) {
        int4 a = __ldcs(reinterpret_cast<const int4*>((const int32_t*)p.x + row * p.x_row_stride + col));
        if (p.bias_i32) {
          const int4 b = *reinterpret_cast<const int4*>(p.bias_i32 + col);
          a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        const float4 r = __ldcs(reinterpret_cast<const float4*>(p.residual_in + row * n + col));
        // residual + scale * int32 as one fused multiply-add: what torch.add(residual,
        // int32, alpha=scale) evaluates (functional/fused.py:9)
        v[i][0] = __fmaf_rn(__int2float_rn(a.x), dq, r.x);
        v[i][1] = __fmaf_rn(__int2float_rn(a.y), dq, r.y);
        v[i][2] = __fmaf_rn(__int2float_rn(a.z), dq, r.z);
        v[i][3] = __fmaf_rn(__int2float_rn(a.w), dq, r.w);
        if (p.residual_out) Vec4<float>::store(p.residual_out + row * n + col, v[i]);
      } else {
        Vec4<XT>::load((const XT*)p.x + row * p.x_row_stride + col, v[i]);
      }
    } else {
      v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
    }
  }

  // ---- statistics: mean, then the centred second moment, both over registers ----
  float mean = 0.f;
  if (!p.rms) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) s += (v[i][0] + v[i][1]) + (v[i][2] + v[i][3]);
    s = row_reduce<false>(s, tpr, tid, row_in_cta, red);
    mean = s / (float)n;
  }
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int col = (i * tpr + tid) * 4;
    if (col < n) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float d = v[i][j] - mean;
        q += d * d;
      }
    }
  }
  q = row_reduce<false>(q, tpr, tid, row_in_cta, red);
  const float rstd = 1.0f / sqrtf(q / (float)n + p.eps);

  // ---- normalise, scale, shift, store ----
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int col = (i * tpr + tid) * 4;
    if (!(row_ok && col < n)) continue;
    float g[4], o[4];
    Vec4<PT>::load((const PT*)p.gamma + col, g);
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = ((v[i][j] - mean) * rstd) * g[j];
    if (p.beta) {
      float b[4];
      Vec4<PT>::load((const PT*)p.beta + col, b);
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] += b[j];
    }
    if constexpr (QOUT) {
      Vec4<int8_t>::store_q((int8_t*)p.out + row * p.out_row_stride + col, o, p.rounding);
    } else {
      if (p.out) Vec4<PT>::store((PT*)p.out + row * p.out_row_stride + col, o);
      if (p.out2) {
        float s[4];
        Vec4<PT>::load((const PT*)p.skip + row * p.x_row_stride + col, s);
#pragma unroll
        for (int j = 0; j < 4; ++j) s[j] += round_through<PT>(o[j]);
        Vec4<PT>::store((PT*)p.out2 + row * p.out_row_stride + col, s);
      }
    }
  }
}

// ------------------------------------------------------------------ LayerNorm, any strides / any N
template <typename XT, typename PT, bool QOUT>
__global__ void __launch_bounds__(256)
layernorm_any_kernel(const LnParams p) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const int64_t n = p.n;
  float dq = p.dq_scale;
  if constexpr (std::is_same<XT, int32_t>::value) {
    if (p.dq_scale_dev) dq = *p.dq_scale_dev;
  }
  auto load = [&](int64_t col) -> float {
    if constexpr (std::is_same<XT, int32_t>::value) {
      int32_t a = ((const int32_t*)p.x)[row * p.x_row_stride + col * p.x_col_stride];
      if (p.bias_i32) a += p.bias_i32[col];
      return __fmaf_rn(__int2float_rn(a), dq, p.residual_in[row * n + col]);
    } else if constexpr (std::is_same<XT, float>::value) {
      return ((const float*)p.x)[row * p.x_row_stride + col * p.x_col_stride];
    } else if constexpr (std::is_same<XT, __half>::value) {
      return __half2float(((const __half*)p.x)[row * p.x_row_stride + col * p.x_col_stride]);
    } else {
      return __bfloat162float(((const __nv_bfloat16*)p.x)[row * p.x_row_stride + col * p.x_col_stride]);
    }
  };
  auto loadp = [&](const void* base, int64_t idx) -> float {
    if constexpr (std::is_same<PT, float>::value) return ((const float*)base)[idx];
    else if constexpr (std::is_same<PT, __half>::value) return __half2float(((const __half*)base)[idx]);
    else return __bfloat162float(((const __nv_bfloat16*)base)[idx]);
  };
  float mean = 0.f;
  if (!p.rms) {
    float s = 0.f;
    for (int64_t c = threadIdx.x; c < n; c += blockDim.x) s += load(c);
    s = row_reduce<false>(s, blockDim.x, threadIdx.x, 0, red);
    mean = s / (float)n;
  }
  float q = 0.f;
  for (int64_t c = threadIdx.x; c < n; c += blockDim.x) {
    const float d = load(c) - mean;
    q += d * d;
  }
  q = row_reduce<false>(q, blockDim.x, threadIdx.x, 0, red);
  const float rstd = 1.0f / sqrtf(q / (float)n + p.eps);
  for (int64_t c = threadIdx.x; c < n; c += blockDim.x) {
    const float x = load(c);
    if constexpr (std::is_same<XT, int32_t>::value) {
      if (p.residual_out) p.residual_out[row * n + c] = x;
    }
    float o = ((x - mean) * rstd) * loadp(p.gamma, c);
    if (p.beta) o += loadp(p.beta, c);
    const int64_t oi = row * p.out_row_stride + c * p.out_col_stride;
    if constexpr (QOUT) {
      ((int8_t*)p.out)[oi] = cast_i8(o, p.rounding);
    } else {
      if (p.out) ((PT*)p.out)[oi] = OutCast<PT>::from(o, 0);
      if (p.out2) {
        const float s = loadp(p.skip, row * p.x_row_stride + c * p.x_col_stride);
        ((PT*)p.out2)[oi] = OutCast<PT>::from(round_through<PT>(o) + s, 0);
      }
    }
  }
}

// ------------------------------------------------------------------ LayerNorm, TMA-streamed rows
// The two hot instantiations (int32 dequant + residual add -> int8, and fp32 -> int8)
// as a persistent kernel: a producer warp streams whole rows into a shared-memory ring
// with bulk asynchronous copies, so the bytes in flight per SM are set by the ring depth
// and not by how many threads happen to be between their load and their store.  256
// consumer threads pull a row into registers, free its slot, and run the same
// arithmetic as layernorm_vec_kernel.  Several CTAs share an SM so that one CTA's
// reductions overlap another's loads.  All mbarrier waits are bounded.
namespace stream {

constexpr int CONSUMERS = 256;
constexpr int THREADS = CONSUMERS + 32;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (try_wait(bar, parity)) return true;
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  uint32_t spins = 0;
  while (!try_wait(bar, parity)) {
    if ((++spins & 255u) == 0u) {
      if (*abort_flag) return false;
      uint64_t t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
    }
  }
  return true;
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// sum over the 256 consumer threads (named barrier 1; the producer warp never joins it)
__device__ __forceinline__ float consumer_sum(float v, float* red, int tid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((tid & 31) == 0) red[tid >> 5] = v;
  asm volatile("bar.sync 1, 256;" ::: "memory");
  // same left-to-right order over warps as row_reduce, so every LayerNorm kernel of this
  // library produces the same statistics for the same row
  float t = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) t += red[w];
  return t;
}

template <bool DQ, int MAXV>
__global__ void __launch_bounds__(THREADS, 2)
layernorm_stream_kernel(const LnParams p, const int stages) {
  extern __shared__ __align__(128) uint8_t sm[];
  const int n = (int)p.n;
  const uint32_t row_bytes = (uint32_t)n * 4u;
  const uint32_t stage_bytes = DQ ? 2u * row_bytes : row_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + (size_t)stages * stage_bytes);
  float* red = reinterpret_cast<float*>(bars + 2 * stages);   // two banks of 8 partial sums
  volatile int* abort_flag = reinterpret_cast<volatile int*>(red + 16);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + stages);
  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full0 + 8 * s), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty0 + 8 * s), "r"(CONSUMERS / 32) : "memory");  // one arrival per consumer warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (tid >= CONSUMERS) {
    // ---- producer: one lane streams this CTA's rows into the ring
    if (tid == CONSUMERS) {
      int s = 0;
      uint32_t ph = 0;
      for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        if (!wait(empty0 + 8 * s, ph ^ 1u, abort_flag)) { atomicOr(&g_status, STATUS_PRODUCER); break; }
        const uint32_t dst = smem_u32(sm + (size_t)s * stage_bytes);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full0 + 8 * s), "r"(stage_bytes) : "memory");
        bulk_load(dst, (const uint8_t*)p.x + row * p.x_row_stride * 4, row_bytes, full0 + 8 * s);
        if (DQ) bulk_load(dst + row_bytes, p.residual_in + row * n, row_bytes, full0 + 8 * s);
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
    return;  // the producer warp takes no part in the consumers' named barrier
  }

  // ---- consumers
  float dq = p.dq_scale;
  if (DQ && p.dq_scale_dev) dq = *p.dq_scale_dev;
  const float inv_n = 1.0f / (float)n;
  // gamma / beta of this thread's columns stay in registers for all rows
  float g[MAXV][4], bt[MAXV][4];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int col = (i * CONSUMERS + tid) * 4;
    g[i][0] = g[i][1] = g[i][2] = g[i][3] = 0.f;
    bt[i][0] = bt[i][1] = bt[i][2] = bt[i][3] = 0.f;
    if (col < n) {
      Vec4<float>::load((const float*)p.gamma + col, g[i]);
      if (p.beta) Vec4<float>::load((const float*)p.beta + col, bt[i]);
    }
  }
  int s = 0;
  uint32_t ph = 0;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const bool got = wait(full0 + 8 * s, ph, abort_flag);
    // agree on the outcome before anyone can diverge around the named barriers below
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (!got || *abort_flag) {
      if (tid == 0) atomicOr(&g_status, STATUS_EPILOGUE);
      break;
    }
    const uint8_t* base = sm + (size_t)s * stage_bytes;
    float v[MAXV][4];
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int col = (i * CONSUMERS + tid) * 4;
      v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
      if (col < n) {
        if (DQ) {
          int4 a = *reinterpret_cast<const int4*>(base + col * 4);
          if (p.bias_i32) {
            const int4 b = __ldg(reinterpret_cast<const int4*>(p.bias_i32 + col));
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
          }
          const float4 r = *reinterpret_cast<const float4*>(base + row_bytes + col * 4);
          v[i][0] = __fmaf_rn(__int2float_rn(a.x), dq, r.x);
          v[i][1] = __fmaf_rn(__int2float_rn(a.y), dq, r.y);
          v[i][2] = __fmaf_rn(__int2float_rn(a.z), dq, r.z);
          v[i][3] = __fmaf_rn(__int2float_rn(a.w), dq, r.w);
        } else {
          Vec4<float>::load(reinterpret_cast<const float*>(base + col * 4), v[i]);
        }
      }
    }
    // the row is in registers: hand the slot back to the producer (the warp meets first, so
    // every lane's reads are ordered before the one arrival)
    __syncwarp();
    if ((tid & 31) == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty0 + 8 * s) : "memory");
    if (++s == stages) { s = 0; ph ^= 1u; }
    if (DQ && p.residual_out) {
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int col = (i * CONSUMERS + tid) * 4;
        if (col < n) __stcs(reinterpret_cast<float4*>(p.residual_out + row * n + col), make_float4(v[i][0], v[i][1], v[i][2], v[i][3]));
      }
    }
    float mean = 0.f;
    if (!p.rms) {
      float t = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) t += (v[i][0] + v[i][1]) + (v[i][2] + v[i][3]);
      mean = consumer_sum(t, red, tid) * inv_n;
    }
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      if ((i * CONSUMERS + tid) * 4 < n) {
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float d = v[i][j] - mean; q += d * d; }
      }
    }
    q = consumer_sum(q, red + 8, tid);
    const float rstd = 1.0f / sqrtf(q * inv_n + p.eps);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int col = (i * CONSUMERS + tid) * 4;
      if (col >= n) continue;
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = ((v[i][j] - mean) * rstd) * g[i][j] + bt[i][j];
      Vec4<int8_t>::store_q((int8_t*)p.out + row * p.out_row_stride + col, o, p.rounding);
    }
  }
}

template <bool DQ>
inline int launch(const LnParams& p, int num_sms, cudaStream_t st) {
  const int64_t n = p.n;
  int maxv = 1;
  while ((int64_t)maxv * CONSUMERS * 4 < n) maxv <<= 1;
  const size_t stage = (size_t)(DQ ? 8 : 4) * n;
  // two CTAs per SM (one CTA's reductions overlap the other's loads), rings as deep as
  // half the shared memory allows, at most 4 rows (measured best on 4096-wide rows)
  const int per_sm = 2;
  int stages = (int)((108 * 1024 - 256) / stage);
  if (stages > 4) stages = 4;
  if (stages < 2) stages = 2;
  const size_t smem = (size_t)stages * stage + 2 * (size_t)stages * 8 + 16 * 4 + 16;
  const int64_t want = (int64_t)num_sms * per_sm;
  const int grid = (int)(p.rows < want ? p.rows : want);
#define TI_LNS(MV)                                                                                         \
  {                                                                                                        \
    auto k = layernorm_stream_kernel<DQ, MV>;                                                              \
    static bool attr = false;                                                                              \
    if (!attr) { TI_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024)); attr = true; } \
    k<<<grid, THREADS, smem, st>>>(p, stages);                                                             \
  }
  switch (maxv) {
    case 1: TI_LNS(1); break;
    case 2: TI_LNS(2); break;
    case 4: TI_LNS(4); break;
    default: TI_LNS(8); break;
  }
#undef TI_LNS
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

// rows whose operands are contiguous fp32/int32 of a 16-byte multiple and fit the ring
inline bool eligible(const ti_layernorm_params& g, bool vec_ok) {
  if (!vec_ok || g.out_dtype != TI_I8 || g.param_dtype != TI_F32) return false;
  if (g.x_dtype != TI_I32 && g.x_dtype != TI_F32) return false;
  if (g.n > 6144 || g.n < 1024 || g.rows < 256) return false;
  if (((uintptr_t)g.x & 15) || (g.x_row_stride % 4) != 0) return false;
  return true;
}

}  // namespace stream

inline int pick_tpr(int64_t n, int* maxv, int per_thread = 16) {
  // about `per_thread` elements per thread, 32..512 threads per row
  int tpr = 32;
  while (tpr < 512 && (int64_t)tpr * per_thread < n) tpr <<= 1;
  int64_t v = (n + (int64_t)tpr * 4 - 1) / ((int64_t)tpr * 4);
  int mv = 1;
  while (mv < v) mv <<= 1;
  *maxv = mv;
  return tpr;
}

template <typename XT, typename PT, bool QOUT>
int launch_ln_typed(const ti_layernorm_params& g, const LnParams& p, bool vec_ok) {
  cudaStream_t st = (cudaStream_t)g.stream;
  int maxv = 0;
  const int tpr = pick_tpr(g.n, &maxv);
  if (vec_ok && maxv <= 16) {
    const int threads = tpr < 128 ? 128 : tpr;
    const int rows_per_cta = threads / tpr;
    const int64_t grid = (g.rows + rows_per_cta - 1) / rows_per_cta;
    if (grid >= (1ll << 31)) { set_error("too many rows"); return TI_ERR_SHAPE; }
    switch (maxv) {
      case 1: layernorm_vec_kernel<XT, PT, QOUT, 1><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
      case 2: layernorm_vec_kernel<XT, PT, QOUT, 2><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
      case 4: layernorm_vec_kernel<XT, PT, QOUT, 4><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
      case 8: layernorm_vec_kernel<XT, PT, QOUT, 8><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
      default: layernorm_vec_kernel<XT, PT, QOUT, 16><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
    }
  } else {
    if (g.rows >= (1ll << 31)) { set_error("too many rows"); return TI_ERR_SHAPE; }
    layernorm_any_kernel<XT, PT, QOUT><<<(unsigned)g.rows, 256, 0, st>>>(p);
  }
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

inline bool aligned(const void* p, int a) { return p == nullptr || ((uintptr_t)p % a) == 0; }

inline int launch_layernorm(const ti_layernorm_params& g) {
  if (g.rows < 0 || g.n <= 0) { set_error("layernorm: bad extents rows=%lld n=%lld", (long long)g.rows, (long long)g.n); return TI_ERR_SHAPE; }
  if (g.rows == 0) return TI_OK;
  if (!g.x || !g.gamma || (!g.out && !g.out2)) { set_error("layernorm: null pointer"); return TI_ERR_DEVICE; }
  const bool is_dq = g.x_dtype == TI_I32;
  if (is_dq && !g.residual_in) { set_error("layernorm: int32 input needs residual_in"); return TI_ERR_DEVICE; }
  if (g.out2 && !g.skip) { set_error("layernorm: out2 needs skip"); return TI_ERR_DEVICE; }
  const bool qout = g.out_dtype == TI_I8;
  if (qout && (g.out2 || !g.out)) { set_error("layernorm: int8 output has no skip variant"); return TI_ERR_UNSUPPORTED; }
  if (!qout && g.out_dtype != g.param_dtype) { set_error("layernorm: float output dtype must equal the parameter dtype"); return TI_ERR_DTYPE; }
  if (!is_dq && g.x_dtype != g.param_dtype) { set_error("layernorm: input and parameter dtypes differ"); return TI_ERR_DTYPE; }
  if (is_dq && g.param_dtype != TI_F32) { set_error("layernorm: dequantising path needs fp32 parameters"); return TI_ERR_DTYPE; }

  LnParams p;
  p.x = g.x; p.residual_in = g.residual_in; p.residual_out = g.residual_out; p.bias_i32 = g.bias_i32;
  p.gamma = g.gamma; p.beta = g.beta; p.skip = g.skip; p.out = g.out; p.out2 = g.out2;
  p.dq_scale_dev = g.dq_scale_dev;
  p.rows = g.rows; p.n = g.n;
  p.x_row_stride = g.x_row_stride; p.x_col_stride = g.x_col_stride;
  p.out_row_stride = g.out_row_stride; p.out_col_stride = g.out_col_stride;
  p.eps = g.eps; p.dq_scale = g.dq_scale; p.rounding = g.rounding; p.rms = g.rms;

  const int xs = dtype_size(g.x_dtype), ps = dtype_size(g.param_dtype), os = dtype_size(g.out_dtype);
  if (!xs || !ps || !os) { set_error("layernorm: bad dtype"); return TI_ERR_DTYPE; }
  bool vec_ok = (g.n % 4 == 0) && g.x_col_stride == 1 && g.out_col_stride == 1 &&
                aligned(g.x, 4 * xs) && (g.x_row_stride * xs) % (4 * xs) == 0 &&
                aligned(g.out, 4 * os) && aligned(g.out2, 4 * os) && (g.out_row_stride * os) % (4 * os) == 0 &&
                aligned(g.gamma, 4 * ps) && aligned(g.beta, 4 * ps) && aligned(g.skip, 4 * ps) &&
                aligned(g.residual_in, 16) && aligned(g.residual_out, 16) && aligned(g.bias_i32, 16);

  if (stream::eligible(g, vec_ok)) {
    int dev = 0, sms = 0;
    TI_CUDA_CHECK(cudaGetDevice(&dev));
    TI_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    return is_dq ? stream::launch<true>(p, sms, (cudaStream_t)g.stream) : stream::launch<false>(p, sms, (cudaStream_t)g.stream);
  }
#define TI_LN_DISPATCH(XT, PT)                                                   \
  return qout ? launch_ln_typed<XT, PT, true>(g, p, vec_ok) : launch_ln_typed<XT, PT, false>(g, p, vec_ok)
  if (is_dq) { TI_LN_DISPATCH(int32_t, float); }
  switch (g.param_dtype) {
    case TI_F32: TI_LN_DISPATCH(float, float);
    case TI_F16: TI_LN_DISPATCH(__half, __half);
    case TI_BF16: TI_LN_DISPATCH(__nv_bfloat16, __nv_bfloat16);
  }
#undef TI_LN_DISPATCH
  set_error("layernorm: unsupported parameter dtype %d", g.param_dtype);
  return TI_ERR_DTYPE;
}

// ------------------------------------------------------------------ int8 GELU
// Only 256 distinct inputs exist, so each CTA tabulates the function once
// (accurate tanhf) and then streams: 16 bytes in, 16 look-ups, 16 bytes out.
// The table is replicated per lane (entry = value*32 + lane) so that the 32
// look-ups of a warp never collide on a shared-memory bank.
__global__ void __launch_bounds__(256)
gelu_q_kernel(const int8_t* __restrict__ x, int8_t* __restrict__ y, int64_t n, float in_scale, float out_mul,
              int rounding, int vec_ok) {
  __shared__ uint32_t lut[256 * 32];
  {
    const int val = (int)(int8_t)threadIdx.x;  // blockDim.x == 256: one input value per thread
    const float f = gelu_tanh_scaled(__fmul_rn((float)val, in_scale), out_mul);
    const uint32_t q = (uint32_t)(uint8_t)cast_i8(f, rounding);
#pragma unroll 8
    for (int l = 0; l < 32; ++l) lut[threadIdx.x * 32 + l] = q;
  }
  __syncthreads();
  const uint32_t* my = lut + (threadIdx.x & 31);
  auto look = [&](uint32_t byte) -> uint32_t { return my[byte << 5]; };
  auto word = [&](uint32_t w) -> uint32_t {
    return look(w & 0xffu) | (look((w >> 8) & 0xffu) << 8) | (look((w >> 16) & 0xffu) << 16) | (look(w >> 24) << 24);
  };
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec_ok) {
    const int64_t nvec = n >> 4;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    uint4* yv = reinterpret_cast<uint4*>(y);
    // four independent 16-byte loads in flight per thread
    int64_t i = gtid;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcs(xv + i + u * stride);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        v[u].x = word(v[u].x); v[u].y = word(v[u].y); v[u].z = word(v[u].z); v[u].w = word(v[u].w);
        __stcs(yv + i + u * stride, v[u]);
      }
    }
    for (; i < nvec; i += stride) {
      uint4 v = __ldcs(xv + i);
      v.x = word(v.x); v.y = word(v.y); v.z = word(v.z); v.w = word(v.w);
      __stcs(yv + i, v);
    }
    for (int64_t j = (nvec << 4) + gtid; j < n; j += stride) y[j] = (int8_t)look((uint8_t)x[j]);
  } else {
    for (int64_t i = gtid; i < n; i += stride) y[i] = (int8_t)look((uint8_t)x[i]);
  }
}

inline int launch_gelu_q(const int8_t* x, int8_t* y, int64_t n, float in_scale, float out_mul, int rounding,
                         void* stream, int num_sms) {
  if (n < 0) { set_error("gelu_q: negative size"); return TI_ERR_SHAPE; }
  if (n == 0) return TI_OK;
  if (!x || !y) { set_error("gelu_q: null pointer"); return TI_ERR_DEVICE; }
  const int vec_ok = (((uintptr_t)x | (uintptr_t)y) & 15) == 0;
  int64_t want = (n / 16 + 255) / 256;
  int64_t cap = (int64_t)num_sms * 8;
  int grid = (int)(want < 1 ? 1 : (want > cap ? cap : want));
  gelu_q_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, y, n, in_scale, out_mul, rounding, vec_ok);
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

// ------------------------------------------------------------------ causal softmax -> int8
struct SmParams {
  const float* s;
  int8_t* p;
  int64_t batch, m, n;
  int64_t s_row_stride, s_batch_stride, p_row_stride, p_batch_stride;
  float out_mul;
  int causal, rounding;
};

__device__ __forceinline__ float exp2_approx(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x));
  return e;
}

template <int MAXV, bool VEC>
__global__ void __launch_bounds__(512, (MAXV <= 4 ? 3 : (MAXV == 8 ? 2 : 1)))
softmax_q_kernel(const SmParams p, const int tpr) {
  __shared__ float red[32 * 32];
  const int rows_per_cta = blockDim.x / tpr;
  const int row_in_cta = threadIdx.x / tpr;
  const int tid = threadIdx.x - row_in_cta * tpr;
  const int64_t grow = (int64_t)blockIdx.x * rows_per_cta + row_in_cta;  // over batch*m
  const bool row_ok = grow < p.batch * p.m;
  const int64_t b = row_ok ? grow / p.m : 0;
  const int64_t i = row_ok ? grow - b * p.m : 0;
  const int n = (int)p.n;
  // number of visible keys of this query row
  int64_t vis64 = p.causal ? (i + (p.n - p.m) + 1) : p.n;
  const int vis = row_ok ? (int)(vis64 < 0 ? 0 : (vis64 > p.n ? p.n : vis64)) : 0;
  const float* srow = p.s + b * p.s_batch_stride + i * p.s_row_stride;
  int8_t* prow = p.p + b * p.p_batch_stride + i * p.p_row_stride;
  const float NEG_INF = __int_as_float(0xff800000);
  const float LOG2E = 1.4426950408889634f;

  // masked positions are never loaded; they hold -inf and come out as exact zeros
  float v[MAXV][4];
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int col = (k * tpr + tid) * 4;
    v[k][0] = v[k][1] = v[k][2] = v[k][3] = NEG_INF;
    if (col < vis) {
      if (VEC && col + 4 <= n) {
        Vec4<float>::load(srow + col, v[k]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) if (col + j < n) v[k][j] = srow[col + j];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) if (col + j >= vis) v[k][j] = NEG_INF;
    }
  }
  float mx = NEG_INF;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) mx = fmaxf(mx, fmaxf(fmaxf(v[k][0], v[k][1]), fmaxf(v[k][2], v[k][3])));
  mx = row_reduce<true>(mx, tpr, tid, row_in_cta, red);
  // exp(s - max) = 2^((s - max) * log2 e); 2^-inf = 0 covers the masked positions
  const float mxl = (vis > 0) ? mx * LOG2E : 0.f;
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int col = (k * tpr + tid) * 4;
    if (col < vis) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float e = exp2_approx(v[k][j] * LOG2E - mxl);
        v[k][j] = e;
        sum += e;
      }
    }
  }
  sum = row_reduce<false>(sum, tpr, tid, row_in_cta, red);
  const float inv = (vis > 0) ? p.out_mul / sum : 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int col = (k * tpr + tid) * 4;
    if (!(row_ok && col < n)) continue;
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    if (col < vis) {
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = v[k][j] * inv;
    }
    if (VEC && col + 4 <= n) {
      if (col < vis) Vec4<int8_t>::store_q(prow + col, o, p.rounding);
      else *reinterpret_cast<uint32_t*>(prow + col) = 0u;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) if (col + j < n) prow[col + j] = cast_i8(o[j], p.rounding);
    }
  }
}

inline int launch_softmax_q(const SmParams& p, void* stream) {
  if (p.batch < 0 || p.m < 0 || p.n <= 0) { set_error("softmax_q: bad extents"); return TI_ERR_SHAPE; }
  if (p.batch == 0 || p.m == 0) return TI_OK;
  if (!p.s || !p.p) { set_error("softmax_q: null pointer"); return TI_ERR_DEVICE; }
  int maxv = 0;
  const int tpr = pick_tpr(p.n, &maxv, 16);
  if (maxv > 16) { set_error("softmax_q: rows longer than 32768 are not supported"); return TI_ERR_UNSUPPORTED; }
  const bool vec = (((uintptr_t)p.s & 15) == 0) && (p.s_row_stride % 4 == 0) && (p.s_batch_stride % 4 == 0) &&
                   (((uintptr_t)p.p & 3) == 0) && (p.p_row_stride % 4 == 0) && (p.p_batch_stride % 4 == 0);
  const int threads = tpr < 128 ? 128 : tpr;
  const int rows_per_cta = threads / tpr;
  const int64_t grid = (p.batch * p.m + rows_per_cta - 1) / rows_per_cta;
  if (grid >= (1ll << 31)) { set_error("softmax_q: too many rows"); return TI_ERR_SHAPE; }
  cudaStream_t st = (cudaStream_t)stream;
#define TI_SM_LAUNCH(MV)                                                                  \
  if (vec) softmax_q_kernel<MV, true><<<(unsigned)grid, threads, 0, st>>>(p, tpr);        \
  else softmax_q_kernel<MV, false><<<(unsigned)grid, threads, 0, st>>>(p, tpr)
  switch (maxv) {
    case 1: TI_SM_LAUNCH(1); break;
    case 2: TI_SM_LAUNCH(2); break;
    case 4: TI_SM_LAUNCH(4); break;
    case 8: TI_SM_LAUNCH(8); break;
    default: TI_SM_LAUNCH(16); break;
  }
#undef TI_SM_LAUNCH
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

}  // namespace row
}  // namespace ti
