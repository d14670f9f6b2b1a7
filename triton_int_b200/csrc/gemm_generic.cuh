// Stride-agnostic int8 GEMM / batched GEMM.  Serves operands the tensor-map path
// cannot address (element strides other than 1 along K, rows that do not start on
// 16-byte boundaries, "s8t" [K,N] operands) with the same epilogue arithmetic.
// 64x64 output tile per CTA, 256 threads, 4x4 outputs per thread, dp4a over K.
#pragma once

#include "ti_common.cuh"

namespace ti {
namespace generic {

constexpr int TM = 64, TN = 64, TK = 32;

struct Params {
  const int8_t* a;
  const int8_t* b;
  void* c;
  const void* bias;
  const float* alpha;
  const float* beta;
  int64_t m, n, k;
  int64_t a_stride_m, a_stride_k, a_stride_batch;
  int64_t b_stride_n, b_stride_k, b_stride_batch;
  int64_t c_stride_m, c_stride_n, c_stride_batch;
  int bias_dtype, epilogue, rounding, causal;
  int tiles_n;
};

template <typename OutT>
__global__ void __launch_bounds__(256)
gemm_i8_generic_kernel(const Params p) {
  __shared__ __align__(16) int8_t As[TM][TK + 4];
  __shared__ __align__(16) int8_t Bs[TN][TK + 4];
  const int tile = blockIdx.x;
  const int64_t batch = blockIdx.y;
  const int m0 = (tile / p.tiles_n) * TM;
  const int n0 = (tile % p.tiles_n) * TN;
  if (p.causal) {
    const int64_t row_last = min((int64_t)m0 + TM - 1, p.m - 1);
    if (n0 > row_last + (p.n - p.m)) return;
  }
  const int8_t* A = p.a + batch * p.a_stride_batch;
  const int8_t* B = p.b + batch * p.b_stride_batch;
  const int tx = threadIdx.x & 15;  // columns tx*4 .. tx*4+3
  const int ty = threadIdx.x >> 4;  // rows    ty*4 .. ty*4+3
  int32_t acc[4][4] = {};

  for (int64_t k0 = 0; k0 < p.k; k0 += TK) {
    // 64x32 bytes per operand, 256 threads: 8 bytes each
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      const int r = i / TK, kk = i % TK;
      const int64_t gm = m0 + r, gn = n0 + r, gk = k0 + kk;
      As[r][kk] = (gm < p.m && gk < p.k) ? A[gm * p.a_stride_m + gk * p.a_stride_k] : (int8_t)0;
      Bs[r][kk] = (gn < p.n && gk < p.k) ? B[gn * p.b_stride_n + gk * p.b_stride_k] : (int8_t)0;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk += 4) {
      int av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = *reinterpret_cast<const int*>(&As[ty * 4 + i][kk]);
        bv[i] = *reinterpret_cast<const int*>(&Bs[tx * 4 + i][kk]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }

  const float alpha = p.alpha ? *p.alpha : 1.0f;
  const float beta = p.beta ? *p.beta : 1.0f;
  OutT* C = reinterpret_cast<OutT*>(p.c) + batch * p.c_stride_batch;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t row = m0 + ty * 4 + i;
    if (row >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t col = n0 + tx * 4 + j;
      if (col >= p.n) continue;
      OutT o;
      if (p.epilogue == TI_EPI_I32) {
        int32_t a = acc[i][j];
        if (p.bias) a += ((const int32_t*)p.bias)[col];
        if constexpr (sizeof(OutT) == 4) {
          *reinterpret_cast<int32_t*>(&o) = a;
        } else {
          o = OutT();
        }
      } else {
        const float b = p.bias ? load_bias_f32(p.bias, p.bias_dtype, col) : 0.f;
        const float f = epilogue_f32(acc[i][j], b, alpha, beta, p.epilogue);
        o = OutCast<OutT>::from(f, p.rounding);
        if constexpr (sizeof(OutT) == 1) {
          if (p.epilogue == TI_EPI_SCALE_BIAS_RELU) o = o < 0 ? (OutT)0 : o;
        }
      }
      C[row * p.c_stride_m + col * p.c_stride_n] = o;
    }
  }
}

template <typename OutT>
int launch_out(const ti_gemm_params& g) {
  Params p;
  p.a = g.a; p.b = g.b; p.c = g.c; p.bias = g.bias; p.alpha = g.alpha; p.beta = g.beta;
  p.m = g.m; p.n = g.n; p.k = g.k;
  p.a_stride_m = g.a_stride_m; p.a_stride_k = g.a_stride_k; p.a_stride_batch = g.a_stride_batch;
  p.b_stride_n = g.b_stride_n; p.b_stride_k = g.b_stride_k; p.b_stride_batch = g.b_stride_batch;
  p.c_stride_m = g.c_stride_m; p.c_stride_n = g.c_stride_n; p.c_stride_batch = g.c_stride_batch;
  p.bias_dtype = g.bias_dtype; p.epilogue = g.epilogue; p.rounding = g.rounding; p.causal = g.causal;
  const int64_t tiles_m = (g.m + TM - 1) / TM;
  p.tiles_n = (int)((g.n + TN - 1) / TN);
  const int64_t tiles = tiles_m * p.tiles_n;
  if (tiles >= (1ll << 31) || g.batch > 65535) {
    set_error("generic GEMM grid too large (tiles=%lld batch=%lld)", (long long)tiles, (long long)g.batch);
    return TI_ERR_SHAPE;
  }
  dim3 grid((unsigned)tiles, (unsigned)g.batch);
  gemm_i8_generic_kernel<OutT><<<grid, 256, 0, (cudaStream_t)g.stream>>>(p);
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

inline int launch(const ti_gemm_params& g) {
  switch (g.out_dtype) {
    case TI_I8: return launch_out<int8_t>(g);
    case TI_I32: return launch_out<int32_t>(g);
    case TI_F32: return launch_out<float>(g);
    case TI_F16: return launch_out<__half>(g);
    case TI_BF16: return launch_out<__nv_bfloat16>(g);
  }
  set_error("unsupported output dtype %d", g.out_dtype);
  return TI_ERR_DTYPE;
}

}  // namespace generic
}  // namespace ti
