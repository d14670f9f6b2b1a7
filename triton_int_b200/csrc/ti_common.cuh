// Shared host/device helpers of the sm_100a INT8 operator library: status
// handling, the fp32 epilogue arithmetic and the float -> int8 cast policies.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/triton_int_b200.h"

namespace ti {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
void count_launch(int n = 1);
int cuda_fail(cudaError_t e, const char* what);  // records the message, returns TI_ERR_CUDA

#define TI_CUDA_CHECK(expr)                                   \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return ::ti::cuda_fail(_e, #expr); \
  } while (0)

// device status word (one per device that loaded the library); bits say which
// bounded wait gave up.  The library is a single translation unit, so the
// definition lives here.
__device__ unsigned int g_status = 0;
enum : unsigned { STATUS_PRODUCER = 1u, STATUS_MMA = 2u, STATUS_EPILOGUE = 4u, STATUS_TP_PEER = 8u };

// ---------------------------------------------------------------- device side
__device__ __forceinline__ int8_t cast_i8(float f, int rounding) {
  if (rounding == TI_ROUND_TRUNC_WRAP) {
    // fptosi then low byte: the reference kernels' `.to(tl.int8)`
    return (int8_t)(__float2int_rz(f) & 0xff);
  }
  int i = __float2int_rn(f);  // round half to even
  i = max(-128, min(127, i));
  return (int8_t)i;
}

template <typename T> struct OutCast;
template <> struct OutCast<int8_t> {
  static __device__ __forceinline__ int8_t from(float f, int rounding) { return cast_i8(f, rounding); }
};
template <> struct OutCast<int32_t> {
  // `.to(tl.int32)`: truncation toward zero
  static __device__ __forceinline__ int32_t from(float f, int) { return __float2int_rz(f); }
};
template <> struct OutCast<float> {
  static __device__ __forceinline__ float from(float f, int) { return f; }
};
template <> struct OutCast<__half> {
  static __device__ __forceinline__ __half from(float f, int) { return __float2half_rn(f); }
};
template <> struct OutCast<__nv_bfloat16> {
  static __device__ __forceinline__ __nv_bfloat16 from(float f, int) { return __float2bfloat16_rn(f); }
};

// tanh(x) = 1 - 2 / (exp(2x) + 1) with the hardware exp2 and reciprocal
// approximations (two special-function operations, absolute error of a few 1e-7,
// far below half an int8 step after the GELU scaling).  Saturates cleanly:
// exp2 -> inf gives 1, exp2 -> 0 gives -1.
__device__ __forceinline__ float tanh_fast(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(__fmul_rn(x, 2.885390081777927f)));  // exp(2x)
  return __fsub_rn(1.0f, __fdividef(2.0f, __fadd_rn(e, 1.0f)));
}

// 0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715*x*x*x)))*scale, evaluated left to right in
// fp32 with no contraction.
__device__ __forceinline__ float gelu_tanh_scaled(float v, float scale) {
  const float c = 0.7978845608028654f;  // sqrt(2/pi)
  float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
  float inner = __fmul_rn(c, __fadd_rn(v, cube));
  inner = fminf(fmaxf(inner, -15.0f), 15.0f);  // tanh is +-1 to fp32 precision beyond |x| ~ 9
  float t = tanh_fast(inner);
  float r = __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, t));
  return __fmul_rn(r, scale);
}

// fp32 value of one output element before the final cast
__device__ __forceinline__ float epilogue_f32(int32_t acc, float biasf, float alpha, float beta, int epilogue) {
  float a = __int2float_rn(acc);
  switch (epilogue) {
    case TI_EPI_SCALE:
      return __fmul_rn(a, alpha);
    case TI_EPI_SCALE_BIAS:
    case TI_EPI_SCALE_BIAS_RELU:
      return __fadd_rn(__fmul_rn(biasf, beta), __fmul_rn(a, alpha));
    case TI_EPI_GELU_Q:
      return gelu_tanh_scaled(__fadd_rn(__fmul_rn(a, alpha), biasf), beta);
    default:
      return a;
  }
}

__device__ __forceinline__ float load_bias_f32(const void* bias, int bias_dtype, int64_t col) {
  switch (bias_dtype) {
    case TI_I8:   return (float)((const int8_t*)bias)[col];
    case TI_I32:  return __int2float_rn(((const int32_t*)bias)[col]);
    case TI_F32:  return ((const float*)bias)[col];
    case TI_F16:  return __half2float(((const __half*)bias)[col]);
    case TI_BF16: return __bfloat162float(((const __nv_bfloat16*)bias)[col]);
  }
  return 0.f;
}

inline int dtype_size(int dt) {
  switch (dt) {
    case TI_I8: return 1;
    case TI_I32: case TI_F32: return 4;
    case TI_F16: case TI_BF16: return 2;
  }
  return 0;
}

}  // namespace ti
