/*
 * triton_int_b200 -- C ABI of the sm_100a INT8 operator library.
 *
 * Plain pointers and sizes only; no exceptions cross this boundary.  Every entry
 * point returns a ti_status, launches asynchronously on the given CUDA stream
 * and never allocates memory the caller can see.  All data pointers are device
 * pointers on the current device unless stated otherwise; there is no CPU path.
 *
 * Each declaration names the reference interface (file:line inside the
 * reference project) that it replaces.
 */
#ifndef TRITON_INT_B200_H
#define TRITON_INT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TI_OK = 0,
  TI_ERR_SHAPE = 1,       /* rank / extent mismatch (the reference raises AssertionError) */
  TI_ERR_DTYPE = 2,
  TI_ERR_ALIGN = 3,       /* a pointer or stride the requested path cannot take */
  TI_ERR_DEVICE = 4,      /* null or non-device pointer, wrong architecture */
  TI_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up (see ti_device_status) */
  TI_ERR_CUDA = 6,        /* a CUDA runtime/driver call failed (see ti_last_error_string) */
  TI_ERR_UNSUPPORTED = 7
} ti_status;

typedef enum { TI_I8 = 0, TI_I32 = 1, TI_F32 = 2, TI_F16 = 3, TI_BF16 = 4 } ti_dtype;

/* float -> int8 policy of every quantising epilogue.
 *   TI_ROUND_RNE_SAT    round half to even, saturate to [-128,127]
 *   TI_ROUND_TRUNC_WRAP truncate toward zero, keep the low byte: the behaviour of
 *                       the reference kernels' `.to(tl.int8)` (kernels/linear.py:254) */
typedef enum { TI_ROUND_RNE_SAT = 0, TI_ROUND_TRUNC_WRAP = 1 } ti_rounding;

typedef enum {
  TI_EPI_I32 = 0,             /* C = acc (+ bias_i32)            kernels/linear.py:505-507,534; kernels/bmm.py:163-273 */
  TI_EPI_SCALE = 1,           /* C = cast(alpha*f32(acc))        kernels/linear.py:107; kernels/bmm.py:414,562,710 */
  TI_EPI_SCALE_BIAS = 2,      /* C = cast(beta*f32(bias) + alpha*f32(acc))   kernels/linear.py:225-227,247,254,674,817 */
  TI_EPI_SCALE_BIAS_RELU = 3, /* C = max(cast_i8(...), 0)        kernels/linear.py:396 */
  TI_EPI_GELU_Q = 4,          /* C = cast_i8(gelu_tanh(alpha*f32(acc) + bias) * beta)   kernels/fused.py:184-187 */
  TI_EPI_DQ_ADD = 5           /* C(fp32) = fma(f32(acc + bias_i32), alpha, residual[m,n]): the dequantise + residual-add
                                 front half of DQ_Add_LayerNorm_Q (functional/fused.py:6-15, nn/fused.py:59-78) done by
                                 the GEMM that produced acc; C is then the new residual stream and the input of a plain
                                 LayerNorm -> int8.  fp32 output, batch == 1, tensor-map path only. */
} ti_epilogue;

typedef enum { TI_PATH_AUTO = 0, TI_PATH_TCGEN05 = 1, TI_PATH_GENERIC = 2 } ti_gemm_path;

/*
 * One int8 x int8 -> int32 GEMM / batched GEMM with a fused epilogue:
 *     acc[b,m,n] = sum_k A[b,m,k] * B[b,n,k]          (B addressed through its strides)
 * Replaces the 6 linear kernels of kernels/linear.py:24-853, the GELU-Q linear of
 * kernels/fused.py:88-231 and the 5 BMM kernels of kernels/bmm.py:12-760.
 * Strides are in elements.  A linear is batch == 1.  "s8n" operands ([N,K]) have
 * b_stride_k == 1; "s8t" operands ([K,N]) have b_stride_n == 1.
 * alpha/beta are DEVICE pointers to one float each (the reference reads its
 * scales with tl.load, kernels/linear.py:227,247); NULL means 1.0.
 */
typedef struct {
  const int8_t* a;
  const int8_t* b;
  void* c;
  const void* bias;        /* [n], dtype bias_dtype; may be NULL (treated as 0) */
  const float* alpha;
  const float* beta;
  int64_t m, n, k, batch;
  int64_t a_stride_m, a_stride_k, a_stride_batch;
  int64_t b_stride_n, b_stride_k, b_stride_batch;
  int64_t c_stride_m, c_stride_n, c_stride_batch;
  int32_t bias_dtype;      /* ti_dtype */
  int32_t out_dtype;       /* ti_dtype */
  int32_t epilogue;        /* ti_epilogue */
  int32_t rounding;        /* ti_rounding */
  int32_t path;            /* ti_gemm_path */
  int32_t causal;          /* 1: skip output tiles with n0 > m0 + BM - 1 + (n - m) (never read by a causal softmax) */
  void* stream;            /* cudaStream_t */
  /* Optional scratch for split-K (few output tiles, long K: the M <= 128 weight-streaming
   * shapes).  When workspace_bytes >= ti_gemm_workspace_bytes(p) the K range is divided
   * over several CTAs per tile, int32 partial sums go to the workspace and a second
   * kernel adds them (exactly) and applies the epilogue.  NULL / 0: never split. */
  void* workspace;
  int64_t workspace_bytes;
  /* TI_EPI_DQ_ADD only: fp32 [m, n] residual read by the epilogue, row stride in elements
   * (a multiple of 4), columns contiguous, 16-byte aligned; must not overlap c. */
  const float* residual;
  int64_t residual_stride_m;
} ti_gemm_params;

/* Bytes of workspace with which ti_gemm_i8 would split K for this problem on the
 * current device; 0 when it would not split. */
int64_t ti_gemm_workspace_bytes(const ti_gemm_params* p);

int ti_gemm_i8(const ti_gemm_params* p);

/*
 * ti_gemm_i8 for callers that cannot hand over (or obtain) device memory.
 *
 * Some hosts of this library must not call cudaMalloc on the hot path: a serving
 * process that reserved the whole HBM for its own pools at start-up (a later
 * cudaMalloc simply fails), a latency-critical loop (cudaMalloc synchronises the whole
 * device), or a plugin that is not allowed to own device memory.  Without scratch,
 * ti_gemm_i8 runs small-M problems unsplit and leaves most SMs idle.  This variant
 * takes the same struct, ignores its workspace fields and, when the problem would
 * split K, keeps the int32 partial sums in an array that is part of the library image
 * (ti_static_scratch_bytes() bytes, 8 MiB: enough for M up to about 48 rows of the
 * config-5 layers; every GPU that loads the library holds it
 * until the process exits).  It calls no allocator of any kind.
 *   - Problems whose partial sums need more than that are refused with
 *     TI_ERR_UNSUPPORTED and a message naming both sizes.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call, with the device current, before
 *     any stream capture begins.
 *   - All calls on a device share the one array: two calls whose kernels can overlap on
 *     the GPU (different streams) race on it.  Serialise them on one stream.  Nothing in
 *     the array needs to start at zero: every partial sum a call reads, it wrote itself.
 * It has no counterpart in the reference.
 */
int ti_gemm_i8_static_scratch(const ti_gemm_params* p);
int64_t ti_static_scratch_bytes(void);

/*
 * Row-wise normalisation family.  One struct covers
 *   layer_norm_fwd_fused_single_pass_q      kernels/fused.py:235-382   (out int8)
 *   layer_norm_fwd_fused_single_pass        kernels/fused.py:385-532   (out = input dtype)
 *   skip_layer_norm_fwd_fused_single_pass   kernels/fused.py:535-693   (out2 = out + skip)
 *   skip_layer_norm_fwd_fused_single_pass2  kernels/fused.py:696-862   (out and out2)
 *   dq_add_layernorm_q                      functional/fused.py:6-15,27-32; nn/fused.py:59-78
 * With x_dtype == TI_I32 the row is first dequantised and added to the residual:
 *     r = residual_in + dq_scale * (x + bias_i32) ; residual_out = r ; y = LN(r).
 * Strides are in elements; the column stride of x and out may differ from 1.
 */
typedef struct {
  const void* x;
  const float* residual_in;   /* fp32 [rows,n], row stride n; required when x_dtype == TI_I32 */
  float* residual_out;        /* optional fp32 [rows,n] */
  const int32_t* bias_i32;    /* optional [n], added to the int32 row before dequantisation */
  const void* gamma;          /* [n] */
  const void* beta;           /* [n] or NULL */
  const void* skip;           /* [rows,n] in x's layout or NULL */
  void* out;                  /* may be NULL when only out2 is wanted */
  void* out2;                 /* out + skip, or NULL */
  const float* dq_scale_dev;  /* optional device scalar overriding dq_scale */
  int64_t rows, n;
  int64_t x_row_stride, x_col_stride;
  int64_t out_row_stride, out_col_stride;
  float eps;
  float dq_scale;
  int32_t x_dtype;            /* TI_F32 / TI_F16 / TI_BF16 / TI_I32 */
  int32_t param_dtype;        /* dtype of gamma/beta/skip */
  int32_t out_dtype;          /* TI_I8 or a float dtype */
  int32_t rounding;
  int32_t rms;                /* 1: RMSNorm (kernels/fused.py:291-292) */
  void* stream;
} ti_layernorm_params;

int ti_layernorm(const ti_layernorm_params* p);

/* Stand-alone int8 GELU: y = cast_i8(gelu_tanh(in_scale * x) * out_mul), the
 * formula of fast_geluQ (kernels/fused.py:76-79) that nn/fused.py:81-87 (GeLu_Q)
 * was meant to expose.  x and y are contiguous, n_elems bytes each. */
int ti_gelu_q(const int8_t* x, int8_t* y, int64_t n_elems, float in_scale, float out_mul,
              int32_t rounding, void* stream);

/* Causal softmax over the last dimension of fp32 scores, quantised to int8:
 * p = cast_i8(out_mul * softmax(mask(s))), query row i sees keys j <= i + (n - m).
 * The step a caller performs between bmm_s8t_s8n_f32t (kernels/bmm.py:428-464)
 * and bmm_s8t_s8n_s8t (kernels/bmm.py:576-612); the reference leaves it to user
 * code.  s is [batch,m,n] with row stride s_row_stride and batch stride
 * s_batch_stride (elements), p likewise. causal == 0 gives a plain softmax. */
int ti_softmax_q(const float* s, int8_t* p, int64_t batch, int64_t m, int64_t n,
                 int64_t s_row_stride, int64_t s_batch_stride,
                 int64_t p_row_stride, int64_t p_batch_stride,
                 int32_t causal, float out_mul, int32_t rounding, void* stream);

/*
 * Fused int8 attention for one layer (head_dim 128):
 *     S = alpha_qk * Q K^T ; P = int8(p_mul * softmax(mask(S))) ; O = int8(alpha_pv * P V)
 * The composition of bmm_s8t_s8n_f32t (kernels/bmm.py:428-464), the caller's softmax
 * and bmm_s8t_s8n_s8t (kernels/bmm.py:576-612) without materialising S or P, and
 * without the [B*h,S,D] / V^T copies those operators need: q, k, v and o are addressed
 * as [batch][seq][head][128] through their batch / row / head strides (elements).
 * It has no single counterpart in the reference.  causal != 0 masks keys
 * j > i + (seq_k - seq_q).  alpha_* are device pointers to one float each.
 */
typedef struct {
  const int8_t* q;
  const int8_t* k;
  const int8_t* v;
  int8_t* o;
  const float* alpha_qk;
  const float* alpha_pv;
  int64_t batch, heads, seq_q, seq_k, head_dim;
  int64_t q_stride_b, q_stride_s, q_stride_h;
  int64_t k_stride_b, k_stride_s, k_stride_h;
  int64_t v_stride_b, v_stride_s, v_stride_h;
  int64_t o_stride_b, o_stride_s, o_stride_h;
  float p_mul;
  int32_t causal;
  int32_t rounding;
  void* stream;
} ti_attention_params;

int ti_attention_i8(const ti_attention_params* p);

/*
 * Tensor-parallel exchange fused with its consumer, one launch per rank:
 *   sum over ranks of the int32 partial sums of a row-parallel linear (read from
 *   every rank's buffer with peer loads) + int32 bias -> dequantise -> + residual
 *   -> LayerNorm -> int8, the int8 row stored into every rank's activation buffer.
 * Rank r processes rows [row_begin, row_begin + row_count) of the [rows, n] matrix;
 * residual_in / residual_out hold only those rows.  parts[i] / outs[i] are rank i's
 * buffers as mapped into this process (peer-accessible device memory); entries at
 * index >= world are ignored.  The caller orders this launch after every rank's
 * producer of parts and orders every rank's consumer of outs after it (a stream
 * barrier).  The reference has no distributed code; the arithmetic is that of
 * dq_add_layernorm_q (functional/fused.py:6-15) applied to the exact integer sum.
 */
typedef struct {
  const int32_t* parts[8];
  int8_t* outs[8];
  const float* residual_in;
  float* residual_out;         /* optional */
  const int32_t* bias_i32;     /* optional [n] */
  const float* gamma;
  const float* beta;           /* optional */
  const float* dq_scale_dev;   /* optional device scalar overriding dq_scale */
  int64_t row_begin, row_count, n;
  int64_t parts_row_begin;     /* row of parts[i] that holds matrix row row_begin (row_begin for full-size
                                  buffers, 0 for receive slots that only hold this rank's rows) */
  float eps;
  float dq_scale;
  int32_t world;
  int32_t rank;                /* this process's rank: sets the order in which peers are visited */
  int32_t rounding;
  void* stream;
} ti_tp_reduce_ln_params;

int ti_tp_reduce_layernorm_q(const ti_tp_reduce_ln_params* p);

/*
 * Row-parallel linear fused with the first half of its reduce-scatter: the raw int32
 * accumulators acc = A . B^T (no bias, no scaling; p->c, bias, alpha, beta are ignored)
 * are not written to a local [m, n] matrix but, tile by tile as they finish, into the
 * receive buffer of the rank that owns the tile's rows:
 *     recv[owner][rank][row - owner * rows_per_rank][col],  owner = row / rows_per_rank
 * recv[i] is rank i's buffer of world * rows_per_rank * n int32 as mapped into this
 * process (peer-accessible memory).  The stores are TMA tensor stores issued from the
 * GEMM's epilogue, so the NVLink traffic overlaps the remaining tiles' MMAs.  After a
 * barrier, ti_tp_reduce_layernorm_q with parts[s] = recv[rank] + s * rows_per_rank * n
 * adds the world slices locally.  The reference has no distributed code.
 */
typedef struct {
  int32_t* recv[8];
  int32_t world;
  int32_t rank;
  int64_t rows_per_rank;   /* multiple of 128; world * rows_per_rank == m */
} ti_gemm_scatter;

int ti_gemm_i8_scatter(const ti_gemm_params* p, const ti_gemm_scatter* sc);

/* Stream-ordered barrier between the `world` ranks of one node.  pads[i] is rank i's
 * pad of 8 zero-initialised uint32 flags in peer-mapped memory, as mapped into this
 * process.  `epoch` must increase by one on every call and be the same on every rank.
 * The wait on the device is bounded (2 s); on expiry bit 3 of the status word is set.
 * Part of the tensor-parallel plumbing; the reference has no counterpart. */
int ti_tp_barrier(uint32_t* const* pads, int32_t world, int32_t rank, uint32_t epoch, void* stream);

/* Reads and clears the device-side status word of the current device.  Non-zero
 * means a bounded wait inside a kernel expired (bit 0: TMA producer, bit 1: MMA
 * issuer, bit 2: epilogue).  Synchronises the device. */
int ti_device_status(uint32_t* status_out);

/*
 * Dynamic activation quantisation on the GPU (absolute-maximum scaling), the step in front
 * of a W8A8 linear when no static input scale exists:
 *   per_token != 0: dynamic_quantize_activation_per_token_absmax  functional/quantization.py:54-61
 *                   scales = [rows] in x's dtype
 *   per_token == 0: dynamic_quantize_activation_per_tensor_absmax (clamp_min = 1, :46-51) or
 *                   quantize_per_tensor_absmax (clamp_min = 0, :5-14); scales = float[2]:
 *                   scales[0] receives the scale, scales[1] is working storage
 * q = clamp(rint(x / scale), -128, 127) with the quotient rounded to x's dtype first, as
 * torch's in-place div_().round_() does.  x is not modified (the reference helpers
 * overwrite their argument).
 */
typedef struct {
  const void* x;
  int8_t* q;
  void* scales;
  int64_t rows, n;
  int64_t x_row_stride, q_row_stride;   /* elements */
  int32_t x_dtype;                      /* TI_F32 / TI_F16 / TI_BF16 */
  int32_t per_token;
  int32_t clamp_min;
  void* stream;
} ti_quantize_params;

int ti_quantize_absmax(const ti_quantize_params* p);

/* Test hook for the failure-reporting path: launches one thread that waits, with the
 * library's bounded-wait loop, on a barrier nothing arrives at; after limit_us
 * microseconds (1..100000) it sets bit 2 of the status word and returns.  The GPU is
 * neither hung nor faulted and the context stays usable. */
int ti_debug_expire_wait(uint32_t limit_us, void* stream);

/* Library facts. */
int ti_version(void);
const char* ti_last_error_string(void);
/* Number of kernels this library has launched since load (host-side counter). */
int64_t ti_launch_count(void);
/* 1 when the current device can run the tcgen05 path (compute capability 10.x). */
int ti_device_supported(void);

#ifdef __cplusplus
}
#endif
#endif /* TRITON_INT_B200_H */
