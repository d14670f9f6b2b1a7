// C ABI of the sm_100a INT8 operator library (single translation unit).
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "ti_common.cuh"

namespace ti {

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return TI_ERR_CUDA;
}

struct DeviceInfo {
  int device = -1;
  int sms = 0;
  int cc_major = 0;
  bool ok = false;
};
// One process drives one GPU; the record is refreshed if the current device changes.
static int device_info(DeviceInfo* out) {
  static thread_local DeviceInfo cache;
  int dev = -1;
  TI_CUDA_CHECK(cudaGetDevice(&dev));
  if (cache.device != dev) {
    cudaDeviceProp prop;
    TI_CUDA_CHECK(cudaGetDeviceProperties(&prop, dev));
    cache.device = dev;
    cache.sms = prop.multiProcessorCount;
    cache.cc_major = prop.major;
    cache.ok = (prop.major == 10);
  }
  *out = cache;
  return TI_OK;
}

}  // namespace ti

#include "gemm_generic.cuh"
#include "gemm_tcgen05.cuh"
#include "rowwise.cuh"
#include "attention_tcgen05.cuh"
#include "tp_fused.cuh"
#include "quantize.cuh"

using namespace ti;

static int require_device(DeviceInfo* di) {
  int rc = device_info(di);
  if (rc != TI_OK) return rc;
  if (!di->ok) {
    set_error("this library runs on compute capability 10.x (sm_100a) only; current device is %d.x", di->cc_major);
    return TI_ERR_DEVICE;
  }
  return TI_OK;
}

static bool is_device_ptr(const void* p) {
  if (!p) return false;
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

extern "C" {

int ti_version(void) { return 100; }

const char* ti_last_error_string(void) { return ti::g_error; }

int64_t ti_launch_count(void) { return (int64_t)ti::g_launches.load(); }

int ti_device_supported(void) {
  DeviceInfo di;
  if (device_info(&di) != TI_OK) return 0;
  return di.ok ? 1 : 0;
}

int ti_device_status(uint32_t* status_out) {
  unsigned int h = 0, zero = 0;
  TI_CUDA_CHECK(cudaDeviceSynchronize());
  TI_CUDA_CHECK(cudaMemcpyFromSymbol(&h, ti::g_status, sizeof(h)));
  if (h) TI_CUDA_CHECK(cudaMemcpyToSymbol(ti::g_status, &zero, sizeof(zero)));
  if (status_out) *status_out = h;
  if (h) {
    set_error("a bounded device-side wait expired (status bits 0x%x)", h);
    return TI_ERR_TIMEOUT;
  }
  return TI_OK;
}

int ti_gemm_i8(const ti_gemm_params* g) {
  if (!g) { set_error("gemm: null params"); return TI_ERR_DEVICE; }
  if (g->m < 0 || g->n < 0 || g->k < 0 || g->batch < 0) {
    set_error("gemm: negative extent m=%lld n=%lld k=%lld batch=%lld", (long long)g->m, (long long)g->n,
              (long long)g->k, (long long)g->batch);
    return TI_ERR_SHAPE;
  }
  // dtype / epilogue combinations
  const int od = g->out_dtype, ep = g->epilogue;
  if (od < TI_I8 || od > TI_BF16) { set_error("gemm: bad out dtype %d", od); return TI_ERR_DTYPE; }
  if (ep < TI_EPI_I32 || ep > TI_EPI_DQ_ADD) { set_error("gemm: bad epilogue %d", ep); return TI_ERR_UNSUPPORTED; }
  if (ep == TI_EPI_DQ_ADD) {
    if (od != TI_F32) { set_error("gemm: the dequantise + residual epilogue stores fp32"); return TI_ERR_DTYPE; }
    if (g->bias && g->bias_dtype != TI_I32) { set_error("gemm: the dequantise + residual epilogue takes an int32 bias"); return TI_ERR_DTYPE; }
    if (g->batch != 1 || g->causal) { set_error("gemm: the dequantise + residual epilogue is for single (non-batched) linears"); return TI_ERR_UNSUPPORTED; }
    if (!g->residual || ((uintptr_t)g->residual & 15) || (g->residual_stride_m & 3) || g->residual_stride_m < g->n) {
      set_error("gemm: residual must be a 16-byte aligned fp32 [m, n] matrix with a row stride that is a multiple of 4 elements");
      return TI_ERR_ALIGN;
    }
  }
  if (ep == TI_EPI_I32 && od != TI_I32) { set_error("gemm: the raw accumulator epilogue stores int32"); return TI_ERR_DTYPE; }
  if (ep == TI_EPI_I32 && g->bias && g->bias_dtype != TI_I32) { set_error("gemm: int32 epilogue takes an int32 bias"); return TI_ERR_DTYPE; }
  if ((ep == TI_EPI_SCALE_BIAS_RELU || ep == TI_EPI_GELU_Q) && od != TI_I8) {
    set_error("gemm: ReLU / GELU-Q epilogues store int8");
    return TI_ERR_DTYPE;
  }
  if (g->bias && (g->bias_dtype < TI_I8 || g->bias_dtype > TI_BF16)) { set_error("gemm: bad bias dtype"); return TI_ERR_DTYPE; }
  if (g->rounding != TI_ROUND_RNE_SAT && g->rounding != TI_ROUND_TRUNC_WRAP) { set_error("gemm: bad rounding mode"); return TI_ERR_UNSUPPORTED; }
  if (g->m == 0 || g->n == 0 || g->batch == 0) return TI_OK;  // nothing to write
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  if (!is_device_ptr(g->c) || (g->k > 0 && (!is_device_ptr(g->a) || !is_device_ptr(g->b)))) {
    set_error("gemm: a, b and c must be device pointers (there is no CPU path)");
    return TI_ERR_DEVICE;
  }
  bool fast = ti::tc::eligible(*g);
  if (g->path == TI_PATH_TCGEN05 && !fast) {
    set_error("gemm: operands not addressable by tensor maps (need K-contiguous rows on 16-byte boundaries)");
    return TI_ERR_ALIGN;
  }
  if (g->path == TI_PATH_GENERIC) fast = false;
  if (ep == TI_EPI_DQ_ADD) {
    if (!is_device_ptr(g->residual)) { set_error("gemm: residual must be a device pointer"); return TI_ERR_DEVICE; }
    if (!fast) {
      set_error("gemm: the dequantise + residual epilogue exists on the tensor-map path only "
                "(K-contiguous operands on 16-byte boundaries); use TI_EPI_I32 and ti_layernorm otherwise");
      return TI_ERR_UNSUPPORTED;
    }
  }
  return fast ? ti::tc::launch(*g, di.sms) : ti::generic::launch(*g);
}

// ---------------------------------------------------------------------------
// Split-K scratch that lives inside the library image, for ti_gemm_i8_static_scratch.
// The name below is only a host-side handle for the symbol; the device address is
// looked up once per device with cudaGetSymbolAddress and that pointer is what the
// kernels receive.
#define TI_STATIC_SCRATCH_BYTES (8ll * 1024 * 1024)
static __device__ __align__(256) unsigned char g_static_scratch[TI_STATIC_SCRATCH_BYTES];

static int static_scratch_ptr(void** out) {
  static void* per_device[64] = {nullptr};
  int dev = -1;
  TI_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { set_error("static scratch: device index %d out of range", dev); return TI_ERR_DEVICE; }
  if (!per_device[dev]) {
    void* ptr = nullptr;
    // resolves the symbol in the context of the CURRENT device (dev)
    TI_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (!ptr) { set_error("static scratch: cudaGetSymbolAddress returned a null address"); return TI_ERR_CUDA; }
    per_device[dev] = ptr;
  }
  *out = per_device[dev];
  return TI_OK;
}

int64_t ti_static_scratch_bytes(void) { return TI_STATIC_SCRATCH_BYTES; }

int ti_gemm_i8_static_scratch(const ti_gemm_params* g) {
  if (!g) { set_error("gemm: null params"); return TI_ERR_DEVICE; }
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  ti_gemm_params local = *g;
  local.workspace = nullptr;
  local.workspace_bytes = 0;
  const int64_t need = (g->path == TI_PATH_GENERIC) ? 0 : ti::tc::workspace_bytes(local, di.sms);
  if (need > TI_STATIC_SCRATCH_BYTES) {
    set_error("gemm (static scratch): this problem splits K into partial sums of %lld bytes, the built-in scratch holds %lld; "
              "use ti_gemm_i8 with a caller-provided workspace, or without one (unsplit)",
              (long long)need, (long long)TI_STATIC_SCRATCH_BYTES);
    return TI_ERR_UNSUPPORTED;
  }
  if (need > 0) {
    void* ptr = nullptr;
    rc = static_scratch_ptr(&ptr);
    if (rc != TI_OK) return rc;
    local.workspace = ptr;
    local.workspace_bytes = TI_STATIC_SCRATCH_BYTES;
  }
  return ti_gemm_i8(&local);
}

// A kernel whose only job is to wait on a barrier that nothing ever arrives at, with the same
// bounded-wait code path as the real kernels but a caller-chosen, short limit.  It lets a test
// see the failure-reporting path (status word, context still usable) without hanging or
// faulting the GPU.
__global__ void ti_expire_wait_kernel(unsigned long long limit_ns) {
  __shared__ unsigned long long bar;
  const unsigned addr = (unsigned)__cvta_generic_to_shared(&bar);
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(addr) : "memory");
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    if (ti::tc::mbar_try_wait(addr, 0)) return;  // cannot happen: nobody arrives
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (t1 - t0 > limit_ns) {
      atomicOr(&ti::g_status, ti::STATUS_EPILOGUE);
      return;
    }
  }
}

int ti_quantize_absmax(const ti_quantize_params* p) {
  if (!p) { set_error("quantize: null params"); return TI_ERR_DEVICE; }
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  if (p->rows > 0 && (!is_device_ptr(p->x) || !is_device_ptr(p->q))) {
    set_error("quantize: x and q must be device pointers (there is no CPU path)");
    return TI_ERR_DEVICE;
  }
  return ti::quant::launch(*p, di.sms);
}

int ti_debug_expire_wait(uint32_t limit_us, void* stream) {
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  if (limit_us == 0 || limit_us > 100000) { set_error("debug wait: limit must be 1..100000 microseconds"); return TI_ERR_UNSUPPORTED; }
  ti_expire_wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((unsigned long long)limit_us * 1000ull);
  count_launch();
  TI_CUDA_CHECK(cudaGetLastError());
  return TI_OK;
}

int64_t ti_gemm_workspace_bytes(const ti_gemm_params* g) {
  if (!g) return 0;
  DeviceInfo di;
  if (device_info(&di) != TI_OK || !di.ok) return 0;
  if (g->path == TI_PATH_GENERIC) return 0;
  return ti::tc::workspace_bytes(*g, di.sms);
}

int ti_layernorm(const ti_layernorm_params* p) {
  if (!p) { set_error("layernorm: null params"); return TI_ERR_DEVICE; }
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  if (p->rows > 0 && (!is_device_ptr(p->x) || !is_device_ptr(p->gamma))) {
    set_error("layernorm: x and gamma must be device pointers (there is no CPU path)");
    return TI_ERR_DEVICE;
  }
  return ti::row::launch_layernorm(*p);
}

int ti_gelu_q(const int8_t* x, int8_t* y, int64_t n_elems, float in_scale, float out_mul, int32_t rounding,
              void* stream) {
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  if (n_elems > 0 && (!is_device_ptr(x) || !is_device_ptr(y))) {
    set_error("gelu_q: x and y must be device pointers (there is no CPU path)");
    return TI_ERR_DEVICE;
  }
  return ti::row::launch_gelu_q(x, y, n_elems, in_scale, out_mul, rounding, stream, di.sms);
}

int ti_softmax_q(const float* s, int8_t* p, int64_t batch, int64_t m, int64_t n, int64_t s_row_stride,
                 int64_t s_batch_stride, int64_t p_row_stride, int64_t p_batch_stride, int32_t causal, float out_mul,
                 int32_t rounding, void* stream) {
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  if (batch > 0 && m > 0 && (!is_device_ptr(s) || !is_device_ptr(p))) {
    set_error("softmax_q: s and p must be device pointers (there is no CPU path)");
    return TI_ERR_DEVICE;
  }
  ti::row::SmParams sp;
  sp.s = s; sp.p = p; sp.batch = batch; sp.m = m; sp.n = n;
  sp.s_row_stride = s_row_stride; sp.s_batch_stride = s_batch_stride;
  sp.p_row_stride = p_row_stride; sp.p_batch_stride = p_batch_stride;
  sp.out_mul = out_mul; sp.causal = causal; sp.rounding = rounding;
  return ti::row::launch_softmax_q(sp, stream);
}

int ti_attention_i8(const ti_attention_params* a) {
  if (!a) { set_error("attention: null params"); return TI_ERR_DEVICE; }
  if (a->batch < 0 || a->heads < 0 || a->seq_q < 0 || a->seq_k < 0) { set_error("attention: negative extent"); return TI_ERR_SHAPE; }
  if (a->rounding != TI_ROUND_RNE_SAT && a->rounding != TI_ROUND_TRUNC_WRAP) { set_error("attention: bad rounding mode"); return TI_ERR_UNSUPPORTED; }
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  if (a->batch * a->heads * a->seq_q > 0 &&
      (!is_device_ptr(a->q) || !is_device_ptr(a->k) || !is_device_ptr(a->v) || !is_device_ptr(a->o))) {
    set_error("attention: q, k, v and o must be device pointers (there is no CPU path)");
    return TI_ERR_DEVICE;
  }
  return ti::attn::launch(*a, di.sms);
}

int ti_tp_reduce_layernorm_q(const ti_tp_reduce_ln_params* p) {
  if (!p) { set_error("tp: null params"); return TI_ERR_DEVICE; }
  if (p->rounding != TI_ROUND_RNE_SAT && p->rounding != TI_ROUND_TRUNC_WRAP) { set_error("tp: bad rounding mode"); return TI_ERR_UNSUPPORTED; }
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  return ti::tp::launch(*p);
}

int ti_gemm_i8_scatter(const ti_gemm_params* g, const ti_gemm_scatter* sc) {
  if (!g || !sc) { set_error("scatter: null params"); return TI_ERR_DEVICE; }
  if (g->m <= 0 || g->n <= 0 || g->k <= 0) { set_error("scatter: empty problem"); return TI_ERR_SHAPE; }
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  if (!is_device_ptr(g->a) || !is_device_ptr(g->b)) { set_error("scatter: a and b must be device pointers"); return TI_ERR_DEVICE; }
  return ti::tc::launch_scatter(*g, *sc, di.sms);
}

int ti_tp_barrier(uint32_t* const* pads, int32_t world, int32_t rank, uint32_t epoch, void* stream) {
  if (!pads) { set_error("tp barrier: null pads"); return TI_ERR_DEVICE; }
  DeviceInfo di;
  int rc = require_device(&di);
  if (rc != TI_OK) return rc;
  return ti::tp::launch_barrier(pads, world, rank, epoch, stream);
}

}  // extern "C"
