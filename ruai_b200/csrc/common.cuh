// Shared declarations of the library's translation units.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/ruai_b200.h"
#include "../../include/ruai_b200_synth.h"

#define RUAI_API extern "C" __attribute__((visibility("default")))

// Number of SMs of the target part; grids are sized in multiples of it.
constexpr int kSmCountB200 = 148;

struct ruai_ctx {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int sm_count = kSmCountB200;
  std::string err;
  // split-K scratch: partial sums [splits][m][n] and one arrival counter per column tile
  float* partial = nullptr;
  size_t partial_bytes = 0;
  unsigned long long scratch_epoch = 0;  // counts reallocations of the scratch: captured graphs hold its address
  unsigned* counters = nullptr;
  size_t counters_n = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  bool use_pdl = true;  // programmatic dependent launch between consecutive kernels
  bool use_bulk = true; // bulk-copy staged GEMV (gemv_bulk.cu) where the weight allows it
  bool use_tc = true;   // tensor-core GEMV (gemv_tc.cu, gemv_tc8.cu) for chunk-layout weights and up to 16 rows
  unsigned force_splits = 0;  // debug: overrides the split-K choice of the tensor-core GEMVs (0 = automatic)
  unsigned long long* trace = nullptr;  // debug: per-launch [first entry, first past the dependency wait, last exit] in ns
  unsigned trace_slots = 0, trace_seq = 0;
  int* status = nullptr;  // device word: 0 ok, 3 / 4 = a bounded wait inside a kernel ran out (mbarrier / grid barrier), 5 = cache position out of range
  unsigned long long launches = 0;
  // persistent kernels (pstep.cu)
  unsigned spin_limit = 1u << 20;  // polls of a bounded device-side wait (about a second)
  unsigned barrier_skew = 0;       // failure injection: extra arrivals (in grids) the next persistent launch will wait for in vain
  unsigned tx_shortfall = 0;       // failure injection: bytes the first bulk copy of the next persistent launch is announced too large by
  unsigned* ps_sync = nullptr;     // [0] grid barrier counter, [1] abort flag, [2..3] poison, for ruai_matmul_q_stream
  unsigned ps_bar_base = 0;
  // sampler scratch (sample.cu): sort keys, probabilities, the sort's temporary storage
  void* sample_buf = nullptr;
  size_t sample_bytes = 0;
};

enum QLayout : uint32_t {
  QL_CHUNK16 = 0,  // 16-byte chunks at ((c * n + j) * 16); int8: 16 rows, int4: one group of 32 rows
  QL_REFERENCE = 1 // the reference's row-major buffers, for shapes the chunk layout does not cover
};

struct ruai_sweight;
struct ruai_qweight {
  ruai_ctx* ctx = nullptr;
  ruai_sweight* stream = nullptr;  // tile-stream copy, built on the first ruai_matmul_q_stream
  uint32_t k = 0, n = 0, bits = 0, group = 0;
  QLayout layout = QL_CHUNK16;
  uint32_t chunks = 0;      // 16-byte chunks per column
  uint8_t* data = nullptr;  // device
  float* scale = nullptr;   // device; int8 [n], int4 [k/group][n]
  size_t data_bytes = 0, scale_bytes = 0;
};

extern thread_local std::string g_ruai_global_err;

int ruai_fail(ruai_ctx* ctx, int code, const char* fmt, ...);

#define RUAI_CUDA(ctx, call)                                                                   \
  do {                                                                                         \
    cudaError_t e__ = (call);                                                                  \
    if (e__ != cudaSuccess)                                                                    \
      return ruai_fail((ctx), RUAI_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), \
                       __FILE__, __LINE__);                                                    \
  } while (0)

#define RUAI_TRY(call)           \
  do {                           \
    int rc__ = (call);           \
    if (rc__ != RUAI_OK) return rc__; \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int ordinal) {
    cudaGetDevice(&prev);
    if (prev != ordinal) cudaSetDevice(ordinal);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// Grows the split-K scratch when a launch needs more (never inside a graph capture).
int ruai_ctx_reserve(ruai_ctx* ctx, size_t partial_bytes, size_t counters);

// ---- launches ---------------------------------------------------------------

// Launches `kernel` on the context stream; with PDL the grid may start while its
// predecessor drains, and must call grid_dependency_wait() before touching
// anything the predecessor writes.
template <typename... KArgs, typename... Args>
inline cudaError_t ruai_launch(ruai_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, bool pdl,
                               Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl && ctx->use_pdl) ? 1 : 0;
  ctx->launches++;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Debug timeline: slot[0] = earliest entry, slot[1] = earliest return from the dependency wait, slot[2] = latest exit.
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#ifdef RUAI_B200_TRACE
__device__ __forceinline__ void trace_min(unsigned long long* slot, int i) { if (slot) atomicMin(slot + i, global_ns()); }
__device__ __forceinline__ void trace_max(unsigned long long* slot, int i) { if (slot) atomicMax(slot + i, global_ns()); }
#else  // the stamps exist in profiling builds only
__device__ __forceinline__ void trace_min(unsigned long long*, int) {}
__device__ __forceinline__ void trace_max(unsigned long long*, int) {}
#endif
inline unsigned long long* ruai_trace_slot(ruai_ctx* c) {
  if (!c->trace || c->trace_seq >= c->trace_slots) return nullptr;
  return c->trace + 4ull * (c->trace_seq++);
}

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- element helpers ----------------------------------------------------------

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
  if (dtype == RUAI_F32) return ((const float*)p)[i];
  if (dtype == RUAI_F16) return __half2float(((const __half*)p)[i]);
  return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void store_from_f32(void* p, int dtype, size_t i, float v) {
  if (dtype == RUAI_F32) ((float*)p)[i] = v;
  else if (dtype == RUAI_F16) ((__half*)p)[i] = __float2half_rn(v);
  else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

// Sign-extended 4-bit value of a packed byte (backend/mod.rs:98-102).
__host__ __device__ __forceinline__ int int4_of(uint8_t b, bool hi) {
  int v = hi ? (b >> 4) : (b & 0xF);
  return v >= 8 ? v - 16 : v;
}

// ---- GEMV (gemv.cu) -------------------------------------------------------------

enum GemvAct : int { ACT_NONE = 0, ACT_GELU = 1, ACT_SWIGLU = 2 };

struct GemvEpilogue {
  const float* bias = nullptr;   // f32 [n]
  const float* resid = nullptr;  // f32 [m, out_ld]; out = resid + y (may alias out)
  int act = ACT_NONE;            // ACT_SWIGLU: columns (2i, 2i+1) = (gate_i, up_i), out is [m, n/2]
  int out_dtype = RUAI_F32;
  uint32_t out_ld = 0;           // row stride of out in elements (0: n, or n/2 for SWIGLU)
  float* sumsq = nullptr;        // optional [col_tiles][m]: per 256-column tile, the sum of squares of the stored row
  // optional greedy pick over the stored rows (generation.rs:6-8, last maximum): every column tile leaves its
  // best (ordered value, column) in argmax_slots [col_tiles][m]; the last tile to finish picks per row, writes
  // argmax_out [m] and adds len_add to *len_ptr.  Needs m <= 16.
  int32_t* argmax_out = nullptr;
  int2* argmax_slots = nullptr;
  unsigned* argmax_counter = nullptr;
  int32_t* len_ptr = nullptr;
  int32_t len_add = 0;
};

// RMSNorm folded into the GEMV's load of x (functional.rs:151-165): x * rstd * w with
// rstd = 1/sqrt(sum(x^2) * (1/k) + eps), the sum given as per-tile partial sums [tiles][m].
struct GemvPrologue {
  const float* norm_w = nullptr;  // f32 [k]; NULL: x is used as it is
  const float* sumsq = nullptr;
  uint32_t tiles = 0;
  float eps = 0.0f;
  unsigned long long* trace = nullptr;  // debug timeline slot of this launch
};

constexpr int kGemvTileCols = 256;      // columns per CTA of gemv.cu, and per sumsq / argmax tile it writes
constexpr int kGemvBulkTileCols = 128;  // the same for gemv_bulk.cu
// Number of sumsq / argmax tiles a GEMV over `w` writes (depends on which kernel serves it).
uint32_t ruai_gemv_tiles(const ruai_ctx* ctx, const ruai_qweight* w);
bool ruai_gemv_bulk_eligible(const ruai_qweight* w);
int ruai_gemv_bulk_launch(ruai_ctx* ctx, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                          const GemvEpilogue& epi, const GemvPrologue& pro);
bool ruai_gemv_tc_eligible(const ruai_qweight* w, uint32_t m);
int ruai_gemv_tc_launch(ruai_ctx* ctx, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                        const GemvEpilogue& epi, const GemvPrologue& pro);
bool ruai_gemv_tc8_eligible(const ruai_qweight* w, uint32_t m);
int ruai_gemv_tc8_launch(ruai_ctx* ctx, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                         const GemvEpilogue& epi, const GemvPrologue& pro);
// Bytes of the context's scratch that a Linear over `w` with m rows may use for its split activations.
size_t ruai_gemv_xs_bytes(const ruai_qweight* w, uint32_t m);
bool ruai_gemv_wide_eligible(const ruai_ctx* ctx, const ruai_qweight* w, uint32_t m);
int ruai_gemv_wide_launch(ruai_ctx* ctx, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                          const GemvEpilogue& epi, const GemvPrologue& pro);
bool ruai_gemm_tc_eligible(const ruai_qweight* w, uint32_t m);
int ruai_gemm_tc_launch(ruai_ctx* ctx, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                        const GemvEpilogue& epi, const GemvPrologue& pro);
// Reads and clears the context's device status word (synchronizes the stream).
int ruai_ctx_check_status(ruai_ctx* ctx);

// y = x @ W for m rows; x is [m, k] (row stride x_ld) in x_dtype.
int ruai_gemv_launch(ruai_ctx* ctx, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                     const GemvEpilogue& epi, const GemvPrologue& pro = GemvPrologue());
