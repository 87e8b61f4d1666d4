// Context, device memory and timing entry points.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

thread_local std::string g_ruai_global_err;

int ruai_fail(ruai_ctx* ctx, int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  g_ruai_global_err = buf;
  return code;
}

RUAI_API const char* ruai_version(void) { return "ruai_b200 0.1 (sm_100a)"; }

RUAI_API int ruai_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

RUAI_API const char* ruai_last_error(const ruai_ctx* ctx) { return ctx ? ctx->err.c_str() : g_ruai_global_err.c_str(); }

RUAI_API int ruai_ctx_create(int ordinal, void* stream_or_null, ruai_ctx** out) {
  if (!out) return ruai_fail(nullptr, RUAI_ERR_ARG, "ruai_ctx_create: out is NULL");
  *out = nullptr;
  int n = ruai_device_count();
  if (n <= 0) return ruai_fail(nullptr, RUAI_ERR_CUDA, "no CUDA device: this library has no CPU fallback");
  if (ordinal < 0 || ordinal >= n) return ruai_fail(nullptr, RUAI_ERR_ARG, "device ordinal %d out of range (%d devices)", ordinal, n);
  RUAI_CUDA(nullptr, cudaSetDevice(ordinal));
  cudaDeviceProp prop;
  RUAI_CUDA(nullptr, cudaGetDeviceProperties(&prop, ordinal));
  if (prop.major != 10)
    return ruai_fail(nullptr, RUAI_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", ordinal, prop.major, prop.minor);
  ruai_ctx* c = new ruai_ctx();
  c->ordinal = ordinal;
  c->sm_count = prop.multiProcessorCount;
  if (stream_or_null) c->stream = (cudaStream_t)stream_or_null;
  else {
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete c; return ruai_fail(nullptr, RUAI_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)); }
    c->own_stream = true;
  }
  cudaEventCreate(&c->ev0);
  cudaEventCreate(&c->ev1);
  const char* pdl = getenv("RUAI_B200_PDL");
  if (pdl && pdl[0] == '0') c->use_pdl = false;
  const char* bulk = getenv("RUAI_B200_BULK");
  if (bulk && bulk[0] == '0') c->use_bulk = false;
  const char* tc = getenv("RUAI_B200_TC");
  if (tc && tc[0] == '0') c->use_tc = false;
  if (cudaMalloc(&c->status, sizeof(int)) != cudaSuccess || cudaMemset(c->status, 0, sizeof(int)) != cudaSuccess) {
    delete c;
    return ruai_fail(nullptr, RUAI_ERR_CUDA, "cannot allocate the status word");
  }
  int rc = ruai_ctx_reserve(c, 8u << 20, 4096);
  if (rc != RUAI_OK) { g_ruai_global_err = c->err; delete c; return rc; }
  *out = c;
  return RUAI_OK;
}

RUAI_API int ruai_ctx_destroy(ruai_ctx* c) {
  if (!c) return RUAI_OK;
  DeviceGuard g(c->ordinal);
  cudaStreamSynchronize(c->stream);
  cudaFree(c->partial);
  cudaFree(c->counters);
  cudaFree(c->status);
  cudaFree(c->ps_sync);
  cudaFree(c->sample_buf);
  cudaEventDestroy(c->ev0);
  cudaEventDestroy(c->ev1);
  if (c->own_stream) cudaStreamDestroy(c->stream);
  delete c;
  return RUAI_OK;
}

int ruai_ctx_reserve(ruai_ctx* c, size_t partial_bytes, size_t counters) {
  DeviceGuard g(c->ordinal);
  if (partial_bytes > c->partial_bytes) {
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->partial) cudaFree(c->partial);
    c->partial = nullptr;
    c->partial_bytes = 0;
    RUAI_CUDA(c, cudaMalloc(&c->partial, partial_bytes));
    c->partial_bytes = partial_bytes;
    c->scratch_epoch++;
  }
  if (counters > c->counters_n) {
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    if (c->counters) cudaFree(c->counters);
    c->counters = nullptr;
    c->counters_n = 0;
    RUAI_CUDA(c, cudaMalloc(&c->counters, counters * sizeof(unsigned)));
    RUAI_CUDA(c, cudaMemset(c->counters, 0, counters * sizeof(unsigned)));
    c->counters_n = counters;
    c->scratch_epoch++;
  }
  return RUAI_OK;
}

int ruai_ctx_check_status(ruai_ctx* c) {
  int st = 0;
  RUAI_CUDA(c, cudaMemcpyAsync(&st, c->status, sizeof st, cudaMemcpyDeviceToHost, c->stream));
  RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
  if (st == 0) return RUAI_OK;
  cudaMemsetAsync(c->status, 0, sizeof(int), c->stream);
  if (c->ps_sync) {  // a persistent launch that gave up leaves its barrier count undefined: start over
    cudaMemsetAsync(c->ps_sync, 0, 64, c->stream);
    c->ps_bar_base = 0;
  }
  if (st == 5) return ruai_fail(c, RUAI_ERR_SHAPE, "a decode step was launched at a position beyond the cache capacity; nothing was written there");
  return ruai_fail(c, RUAI_ERR_TIMEOUT, "a bounded wait inside a kernel ran out (status %d); results of that launch are invalid", st);
}

RUAI_API int ruai_ctx_synchronize(ruai_ctx* c) {
  if (!c) return ruai_fail(nullptr, RUAI_ERR_ARG, "ctx is NULL");
  DeviceGuard g(c->ordinal);
  return ruai_ctx_check_status(c);
}

RUAI_API int ruai_malloc(ruai_ctx* c, size_t bytes, void** out) {
  if (!c || !out) return ruai_fail(c, RUAI_ERR_ARG, "ruai_malloc: NULL argument");
  DeviceGuard g(c->ordinal);
  *out = nullptr;
  RUAI_CUDA(c, cudaMalloc(out, bytes ? bytes : 1));
  return RUAI_OK;
}

RUAI_API int ruai_free(ruai_ctx* c, void* p) {
  if (!c) return ruai_fail(nullptr, RUAI_ERR_ARG, "ctx is NULL");
  DeviceGuard g(c->ordinal);
  RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
  RUAI_CUDA(c, cudaFree(p));
  return RUAI_OK;
}

RUAI_API int ruai_memcpy_h2d(ruai_ctx* c, void* dst, const void* src, size_t bytes) {
  if (!c) return ruai_fail(nullptr, RUAI_ERR_ARG, "ctx is NULL");
  DeviceGuard g(c->ordinal);
  RUAI_CUDA(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
  RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
  return RUAI_OK;
}

RUAI_API int ruai_memcpy_d2h(ruai_ctx* c, void* dst, const void* src, size_t bytes) {
  if (!c) return ruai_fail(nullptr, RUAI_ERR_ARG, "ctx is NULL");
  DeviceGuard g(c->ordinal);
  RUAI_CUDA(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
  RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
  return RUAI_OK;
}

RUAI_API int ruai_timer_start(ruai_ctx* c) {
  if (!c) return ruai_fail(nullptr, RUAI_ERR_ARG, "ctx is NULL");
  RUAI_CUDA(c, cudaEventRecord(c->ev0, c->stream));
  return RUAI_OK;
}

RUAI_API int ruai_timer_stop_ms(ruai_ctx* c, float* ms) {
  if (!c || !ms) return ruai_fail(c, RUAI_ERR_ARG, "NULL argument");
  RUAI_CUDA(c, cudaEventRecord(c->ev1, c->stream));
  RUAI_CUDA(c, cudaEventSynchronize(c->ev1));
  RUAI_CUDA(c, cudaEventElapsedTime(ms, c->ev0, c->ev1));
  return RUAI_OK;
}

// Tuning knob: the split-k count of the tensor-core GEMVs (0 = the chooser decides).
RUAI_API int ruai_ctx_force_splits(ruai_ctx* c, unsigned splits) {
  if (!c) return ruai_fail(c, RUAI_ERR_ARG, "NULL argument");
  if (splits > 8) return ruai_fail(c, RUAI_ERR_ARG, "splits %u: 0 (automatic) or 1..8", splits);
  c->force_splits = splits;
  return RUAI_OK;
}

// Profiling hooks, present only in builds made with RUAI_B200_TRACE=1 (never in the library as shipped).
#ifdef RUAI_B200_TRACE
RUAI_API int ruai_debug_force_splits(ruai_ctx* c, unsigned splits) {  // also the profiling bits above the count
  c->force_splits = splits;
  return RUAI_OK;
}

RUAI_API int ruai_debug_trace(ruai_ctx* c, void* dev_buf, unsigned slots) {
  c->trace = (unsigned long long*)dev_buf;
  c->trace_slots = slots;
  c->trace_seq = 0;
  return RUAI_OK;
}
#endif
