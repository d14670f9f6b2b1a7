// Dynamic activation quantisers on the GPU: the step in front of the W8A8 linears when
// no static input scale exists (reference functional/quantization.py:5-61).
//   per token : scale_r = max(absmax(x[r,:]), 1e-8) / 127 ; q = clamp(rint(x / scale_r), -128, 127)
//   per tensor: one scale from the absolute maximum of the whole tensor
// One pass per row for the per-token form (row in registers); two small kernels for the
// per-tensor form (absolute maximum via an integer atomic on the float bits, then the
// element-wise quantisation).  Division and rounding happen in the input's own dtype,
// as torch's in-place `div_().round_()` does: for fp16/bf16 the quotient is rounded to
// that type before it is rounded to an integer.
#pragma once

#include "rowwise.cuh"

namespace ti {
namespace quant {

template <typename T> __device__ __forceinline__ float quotient_in_type(float x, float s);
template <> __device__ __forceinline__ float quotient_in_type<float>(float x, float s) { return x / s; }
template <> __device__ __forceinline__ float quotient_in_type<__half>(float x, float s) { return __half2float(__float2half_rn(x / s)); }
template <> __device__ __forceinline__ float quotient_in_type<__nv_bfloat16>(float x, float s) { return __bfloat162float(__float2bfloat16_rn(x / s)); }
template <typename T> __device__ __forceinline__ float round_to_type(float x);
template <> __device__ __forceinline__ float round_to_type<float>(float x) { return x; }
template <> __device__ __forceinline__ float round_to_type<__half>(float x) { return __half2float(__float2half_rn(x)); }
template <> __device__ __forceinline__ float round_to_type<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ int8_t q_rne_sat(float v) {
  int i = __float2int_rn(v);
  return (int8_t)max(-128, min(127, i));
}

struct Params {
  const void* x;
  int8_t* q;
  void* scales;          // per token: [rows] in x's dtype; per tensor: float[2] = {scale, bits of the absolute maximum}
  int64_t rows, n, x_row_stride, q_row_stride;
  int clamp_min;         // 1: absmax is clamped to >= 1e-8 before the division by 127
};

template <typename T, int MAXV>
__global__ void __launch_bounds__(512)
quantize_per_token_kernel(const Params p, const int tpr) {
  __shared__ float red[32 * 32];
  const int rows_per_cta = blockDim.x / tpr;
  const int row_in_cta = threadIdx.x / tpr;
  const int tid = threadIdx.x - row_in_cta * tpr;
  const int64_t row = (int64_t)blockIdx.x * rows_per_cta + row_in_cta;
  const bool row_ok = row < p.rows;
  const int n = (int)p.n;
  float v[MAXV][4];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int col = (i * tpr + tid) * 4;
    v[i][0] = v[i][1] = v[i][2] = v[i][3] = 0.f;
    if (row_ok && col < n) row::Vec4<T>::load((const T*)p.x + row * p.x_row_stride + col, v[i]);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i][0]), fabsf(v[i][1])), fmaxf(fabsf(v[i][2]), fabsf(v[i][3]))));
  }
  amax = row::row_reduce<true>(amax, tpr, tid, row_in_cta, red);
  // max_val = clamp(absmax, 1e-8) / 127, computed and stored in the input's dtype
  float scale = round_to_type<T>(p.clamp_min ? fmaxf(amax, round_to_type<T>(1e-8f)) : amax);
  // torch divides a CUDA tensor by a Python scalar as a multiplication by the fp32 reciprocal
  scale = round_to_type<T>(__fmul_rn(scale, 1.0f / 127.0f));
  if (row_ok && tid == 0) ((T*)p.scales)[row] = OutCast<T>::from(scale, 0);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int col = (i * tpr + tid) * 4;
    if (!(row_ok && col < n)) continue;
    char4 c;
    c.x = q_rne_sat(quotient_in_type<T>(v[i][0], scale)); c.y = q_rne_sat(quotient_in_type<T>(v[i][1], scale));
    c.z = q_rne_sat(quotient_in_type<T>(v[i][2], scale)); c.w = q_rne_sat(quotient_in_type<T>(v[i][3], scale));
    *reinterpret_cast<char4*>(p.q + row * p.q_row_stride + col) = c;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
absmax_kernel(const T* __restrict__ x, int64_t n, unsigned int* __restrict__ out_bits) {
  __shared__ float red[8];
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float f;
    if constexpr (std::is_same<T, float>::value) f = x[i];
    else if constexpr (std::is_same<T, __half>::value) f = __half2float(x[i]);
    else f = __bfloat162float(x[i]);
    m = fmaxf(m, fabsf(f));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    atomicMax(out_bits, __float_as_uint(m));  // non-negative floats order like their bit patterns
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
quantize_per_tensor_kernel(const T* __restrict__ x, int8_t* __restrict__ q, int64_t n, float* scales, int clamp_min) {
  const float amax = __uint_as_float(reinterpret_cast<const unsigned int*>(scales)[1]);
  float scale = round_to_type<T>(clamp_min ? fmaxf(amax, round_to_type<T>(1e-8f)) : amax);
  scale = round_to_type<T>(__fmul_rn(scale, 1.0f / 127.0f));
  if (blockIdx.x == 0 && threadIdx.x == 0) scales[0] = scale;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float f;
    if constexpr (std::is_same<T, float>::value) f = x[i];
    else if constexpr (std::is_same<T, __half>::value) f = __half2float(x[i]);
    else f = __bfloat162float(x[i]);
    q[i] = q_rne_sat(quotient_in_type<T>(f, scale));
  }
}

template <typename T>
int launch_typed(const ti_quantize_params& g, int num_sms) {
  cudaStream_t st = (cudaStream_t)g.stream;
  if (g.per_token) {
    Params p;
    p.x = g.x; p.q = g.q; p.scales = g.scales; p.rows = g.rows; p.n = g.n;
    p.x_row_stride = g.x_row_stride; p.q_row_stride = g.q_row_stride; p.clamp_min = g.clamp_min;
    int maxv = 0;
    const int tpr = row::pick_tpr(g.n, &maxv);
    if (maxv > 16) { set_error("quantize: rows longer than 32768 are not supported"); return TI_ERR_UNSUPPORTED; }
    const int threads = tpr < 128 ? 128 : tpr;
    const int rpc = threads / tpr;
    const int64_t grid = (g.rows + rpc - 1) / rpc;
    if (grid >= (1ll << 31)) { set_error("quantize: too many rows"); return TI_ERR_SHAPE; }
    switch (maxv) {
      case 1: quantize_per_token_kernel<T, 1><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
      case 2: quantize_per_token_kernel<T, 2><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
      case 4: quantize_per_token_kernel<T, 4><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
      case 8: quantize_per_token_kernel<T, 8><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
      default: quantize_per_token_kernel<T, 16><<<(unsigned)grid, threads, 0, st>>>(p, tpr); break;
    }
    count_launch();
  } else {
    const int64_t total = g.rows * g.n;
    TI_CUDA_CHECK(cudaMemsetAsync(g.scales, 0, 8, st));
    int64_t want = (total + 256 * 8 - 1) / (256 * 8);
    const int grid = (int)(want < 1 ? 1 : (want > (int64_t)num_sms * 8 ? (int64_t)num_sms * 8 : want));
    absmax_kernel<T><<<grid, 256, 0, st>>>((const T*)g.x, total, reinterpret_cast<unsigned int*>(g.scales) + 1);
    quantize_per_tensor_kernel<T><<<grid, 256, 0, st>>>((const T*)g.x, g.q, total, (float*)g.scales, g.clamp_min);
    count_launch(2);
  }
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

inline int launch(const ti_quantize_params& g, int num_sms) {
  if (g.rows < 0 || g.n <= 0) { set_error("quantize: bad extents"); return TI_ERR_SHAPE; }
  if (g.rows == 0) return TI_OK;
  if (!g.x || !g.q || !g.scales) { set_error("quantize: null pointer"); return TI_ERR_DEVICE; }
  const int es = dtype_size(g.x_dtype);
  if (g.x_dtype != TI_F32 && g.x_dtype != TI_F16 && g.x_dtype != TI_BF16) { set_error("quantize: input must be fp32, fp16 or bf16"); return TI_ERR_DTYPE; }
  if (g.per_token) {
    if ((g.n % 4) || ((uintptr_t)g.x % (4 * es)) || ((g.x_row_stride * es) % (4 * es)) || ((uintptr_t)g.q & 3) || (g.q_row_stride & 3)) {
      set_error("quantize (per token): rows must be multiples of 4 elements on 4-element boundaries");
      return TI_ERR_ALIGN;
    }
  } else if (g.x_row_stride != g.n || g.q_row_stride != g.n) {
    set_error("quantize (per tensor): contiguous tensors expected");
    return TI_ERR_ALIGN;
  }
  switch (g.x_dtype) {
    case TI_F32: return launch_typed<float>(g, num_sms);
    case TI_F16: return launch_typed<__half>(g, num_sms);
    default: return launch_typed<__nv_bfloat16>(g, num_sms);
  }
}

}  // namespace quant
}  // namespace ti
