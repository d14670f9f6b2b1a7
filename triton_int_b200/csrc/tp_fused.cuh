// Tensor-parallel exchange fused with the row kernel that consumes it:
//   reduce-scatter (int32 partial sums of a row-parallel linear, read from every
//   rank's buffer over NVLink with plain peer loads, added exactly)
//   -> + int32 bias -> dequantise -> + residual -> LayerNorm -> int8
//   -> all-gather (the int8 row is stored into every rank's activation buffer).
// Each rank runs this kernel over its own slice of the rows; the fp32 residual
// stream stays row-sharded.  There is no wait inside the kernel: ordering against
// the producers of the partial sums and the consumers of the gathered rows is a
// stream-level barrier supplied by the caller.  Plain loads and stores only.
#pragma once

#include "rowwise.cuh"

namespace ti {
namespace tp {

constexpr int MAX_WORLD = 8;

struct Params {
  const int32_t* parts[MAX_WORLD];  // every rank's [rows_total, n] partial-sum buffer as mapped here
  int8_t* outs[MAX_WORLD];          // every rank's [rows_total, n] int8 buffer as mapped here
  const float* residual_in;         // this rank's rows: [row_count, n]
  float* residual_out;              // this rank's rows: [row_count, n]
  const int32_t* bias_i32;
  const float* gamma;
  const float* beta;
  const float* dq_scale_dev;
  int64_t row_begin, row_count, n, parts_row_begin;
  float eps, dq_scale;
  int world, rank, rounding;
};

template <int MAXV>
__global__ void __launch_bounds__(512, 1)
tp_reduce_layernorm_q_kernel(const Params p, const int tpr) {
  __shared__ float red[32 * 32];
  const int rows_per_cta = blockDim.x / tpr;
  const int row_in_cta = threadIdx.x / tpr;
  const int tid = threadIdx.x - row_in_cta * tpr;
  const int64_t lrow = (int64_t)blockIdx.x * rows_per_cta + row_in_cta;  // row inside this rank's slice
  const bool row_ok = lrow < p.row_count;
  const int64_t grow = p.row_begin + lrow;                               // row of the full matrix
  const int n = (int)p.n;
  const float dq = p.dq_scale_dev ? *p.dq_scale_dev : p.dq_scale;
  float v[MAXV][4];

  // All ranks' partial sums for this thread's columns are requested before any is used.
  // Rank q starts with rank q+1's buffer and ends with its own, so that at any moment
  // the ranks pull from different sources instead of all draining the same GPU's links.
  // Peers are visited four at a time: four peers' loads are in flight together.
  int4 acc[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) acc[i] = make_int4(0, 0, 0, 0);
#pragma unroll
  for (int s0 = 0; s0 < MAX_WORLD; s0 += 4) {
    if (s0 < p.world) {
      int4 part[4][MAXV];
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        if (s0 + s < p.world) {
          int r = p.rank + 1 + s0 + s;
          if (r >= p.world) r -= p.world;
          const int32_t* src = p.parts[r] + (p.parts_row_begin + lrow) * n;
#pragma unroll
          for (int i = 0; i < MAXV; ++i) {
            const int col = (i * tpr + tid) * 4;
            part[s][i] = (row_ok && col < n) ? __ldcs(reinterpret_cast<const int4*>(src + col)) : make_int4(0, 0, 0, 0);
          }
        }
      }
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        if (s0 + s < p.world) {
#pragma unroll
          for (int i = 0; i < MAXV; ++i) {
            acc[i].x += part[s][i].x; acc[i].y += part[s][i].y; acc[i].z += part[s][i].z; acc[i].w += part[s][i].w;
          }
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int col = (i * tpr + tid) * 4;
    v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
    if (row_ok && col < n) {
      int4 a = acc[i];
      if (p.bias_i32) {
        const int4 b = *reinterpret_cast<const int4*>(p.bias_i32 + col);
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
      }
      const float4 r = __ldcs(reinterpret_cast<const float4*>(p.residual_in + lrow * n + col));
      v[i][0] = __fmaf_rn(__int2float_rn(a.x), dq, r.x);
      v[i][1] = __fmaf_rn(__int2float_rn(a.y), dq, r.y);
      v[i][2] = __fmaf_rn(__int2float_rn(a.z), dq, r.z);
      v[i][3] = __fmaf_rn(__int2float_rn(a.w), dq, r.w);
      if (p.residual_out) row::Vec4<float>::store(p.residual_out + lrow * n + col, v[i]);
    }
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) s += (v[i][0] + v[i][1]) + (v[i][2] + v[i][3]);
  s = row::row_reduce<false>(s, tpr, tid, row_in_cta, red);
  const float mean = s / (float)n;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    if ((i * tpr + tid) * 4 < n) {
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float d = v[i][j] - mean; q += d * d; }
    }
  }
  q = row::row_reduce<false>(q, tpr, tid, row_in_cta, red);
  const float rstd = 1.0f / sqrtf(q / (float)n + p.eps);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int col = (i * tpr + tid) * 4;
    if (!(row_ok && col < n)) continue;
    float g[4], o[4];
    row::Vec4<float>::load(p.gamma + col, g);
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = ((v[i][j] - mean) * rstd) * g[j];
    if (p.beta) {
      float b[4];
      row::Vec4<float>::load(p.beta + col, b);
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] += b[j];
    }
    char4 c;
    c.x = cast_i8(o[0], p.rounding); c.y = cast_i8(o[1], p.rounding);
    c.z = cast_i8(o[2], p.rounding); c.w = cast_i8(o[3], p.rounding);
#pragma unroll
    for (int s = 0; s < MAX_WORLD; ++s) {
      if (s < p.world) {
        int r = p.rank + 1 + s;
        if (r >= p.world) r -= p.world;
        *reinterpret_cast<char4*>(p.outs[r] + grow * n + col) = c;
      }
    }
  }
}

// Device-side barrier between the ranks of one node, ordered on a stream.  Every rank
// owns a pad of MAX_WORLD 32-bit flags in peer-mapped memory; rank r stores the epoch
// number into flag r of every rank's pad (system-scope release) and then waits until
// all flags of its own pad have reached the epoch (system-scope acquire).  The wait is
// bounded: after the limit the kernel records STATUS_TP_PEER and returns.
struct BarrierParams {
  uint32_t* pads[MAX_WORLD];
  int world, rank;
  uint32_t epoch;
};
__global__ void tp_barrier_kernel(const BarrierParams p) {
  const int q = threadIdx.x;
  if (q >= p.world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.pads[q] + p.rank), "r"(p.epoch) : "memory");
  const uint32_t* mine = p.pads[p.rank] + q;
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  uint32_t spins = 0;
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int32_t)(v - p.epoch) >= 0) break;
    if ((++spins & 63u) == 0u) {
      uint64_t t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > 2000000000ull) {
        atomicOr(&g_status, STATUS_TP_PEER);
        break;
      }
    }
  }
  __threadfence_system();
}

inline int launch_barrier(uint32_t* const* pads, int world, int rank, uint32_t epoch, void* stream) {
  if (world < 1 || world > MAX_WORLD || rank < 0 || rank >= world) { set_error("tp barrier: bad world/rank"); return TI_ERR_UNSUPPORTED; }
  BarrierParams p;
  for (int r = 0; r < MAX_WORLD; ++r) p.pads[r] = nullptr;
  for (int r = 0; r < world; ++r) {
    if (!pads[r] || ((uintptr_t)pads[r] & 3)) { set_error("tp barrier: null or misaligned pad for rank %d", r); return TI_ERR_ALIGN; }
    p.pads[r] = pads[r];
  }
  p.world = world; p.rank = rank; p.epoch = epoch;
  tp_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p);
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

inline int launch(const ti_tp_reduce_ln_params& g) {
  if (g.world < 1 || g.world > MAX_WORLD || g.rank < 0 || g.rank >= g.world) { set_error("tp: world size must be 1..8 and rank inside it"); return TI_ERR_UNSUPPORTED; }
  if (g.row_count < 0 || g.n <= 0 || g.row_begin < 0) { set_error("tp: bad extents"); return TI_ERR_SHAPE; }
  if (g.row_count == 0) return TI_OK;
  if (g.n % 4 != 0) { set_error("tp: row length must be a multiple of 4"); return TI_ERR_ALIGN; }
  Params p;
  for (int r = 0; r < MAX_WORLD; ++r) { p.parts[r] = nullptr; p.outs[r] = nullptr; }
  for (int r = 0; r < g.world; ++r) {
    if (!g.parts[r] || !g.outs[r] || ((uintptr_t)g.parts[r] & 15) || ((uintptr_t)g.outs[r] & 3)) {
      set_error("tp: null or misaligned peer buffer for rank %d", r);
      return TI_ERR_ALIGN;
    }
    p.parts[r] = g.parts[r];
    p.outs[r] = g.outs[r];
  }
  if (!g.residual_in || !g.gamma || ((uintptr_t)g.residual_in & 15) || ((uintptr_t)g.residual_out & 15) ||
      ((uintptr_t)g.gamma & 15) || ((uintptr_t)g.beta & 15) || ((uintptr_t)g.bias_i32 & 15)) {
    set_error("tp: null or misaligned local operand");
    return TI_ERR_ALIGN;
  }
  p.residual_in = g.residual_in; p.residual_out = g.residual_out; p.bias_i32 = g.bias_i32;
  p.gamma = g.gamma; p.beta = g.beta; p.dq_scale_dev = g.dq_scale_dev;
  p.row_begin = g.row_begin; p.row_count = g.row_count; p.n = g.n; p.parts_row_begin = g.parts_row_begin;
  p.eps = g.eps; p.dq_scale = g.dq_scale; p.world = g.world; p.rank = g.rank; p.rounding = g.rounding;
  int maxv = 0;
  // same thread layout as layernorm_vec_kernel, hence the same reduction order and the same bits
  const int tpr = row::pick_tpr(g.n, &maxv);
  if (maxv > 8) { set_error("tp: rows longer than 16384 are not supported"); return TI_ERR_UNSUPPORTED; }
  const int threads = tpr < 128 ? 128 : tpr;
  const int rows_per_cta = threads / tpr;
  const int64_t grid = (g.row_count + rows_per_cta - 1) / rows_per_cta;
  if (grid >= (1ll << 31)) { set_error("tp: too many rows"); return TI_ERR_SHAPE; }
  cudaStream_t st = (cudaStream_t)g.stream;
  switch (maxv) {
    case 1: tp_reduce_layernorm_q_kernel<1><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
    case 2: tp_reduce_layernorm_q_kernel<2><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
    case 4: tp_reduce_layernorm_q_kernel<4><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
    default: tp_reduce_layernorm_q_kernel<8><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
  }
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

}  // namespace tp
}  // namespace ti
