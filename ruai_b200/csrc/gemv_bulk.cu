// Fused dequantize + GEMV, second generation: weights staged through shared memory with
// bulk asynchronous copies, split-K inside a thread-block cluster.
//
// Same arithmetic and the same epilogues as gemv.cu (the CPU definition of
// matmul_int8 / matmul_int4, src/nn/backend/cpu.rs:897-927, 1035-1067); what changes is how
// the bytes move:
//  - a CTA of 128 threads owns 128 neighbouring columns.  In the chunk layout one chunk row
//    of that tile is 2 KB contiguous (plus 512 B of int4 scales), so one thread issues
//    `cp.async.bulk` copies into a ring of kStages x kStageChunks chunk rows and the copies
//    signal an mbarrier per ring slot.  The bytes in flight no longer depend on registers
//    or occupancy: every resident CTA keeps up to 40 KB requested, and it requests the first
//    ring-full before the grid-dependency wait, while the previous kernel is still running.
//  - k is split over the CTAs of a cluster (1, S, 1), S <= 8.  Partial sums travel through
//    distributed shared memory to the cluster's first CTA, which adds them in rank order
//    (deterministic) and runs the epilogue.  No global scratch, no atomics, no second pass.
//  - every wait on an mbarrier is bounded; on a timeout the kernel records status 3 in the
//    context's status word and leaves without hanging.
#include "common.cuh"
#include "pipeline.cuh"
#include "gemv_epilogue.cuh"

namespace gemv_bulk {

using namespace pipe;

constexpr int kCols = kGemvBulkTileCols;  // 128 columns (= threads) per CTA
constexpr int kStageChunks = 4;           // chunk rows per ring slot
constexpr int kStages = 4;                // ring slots
constexpr int kStageK = 512;              // activations per row staged at a time

struct Params {
  const uint4* w;
  const float* scale;
  const void* x;
  int x_dtype;
  uint32_t x_ld, m, k, n, chunks, chunks_per_cta, splits;
  void* out;
  int* status;
  GemvEpilogue epi;
  GemvPrologue pro;
};

template <int B>
__device__ __forceinline__ float byte_f32(uint32_t w, float magic) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + B)) - magic;
}
// One chunk (16 bytes of one column) against the staged activations.
template <int BITS, int MT>
__device__ __forceinline__ void consume_chunk(const uint4 wv, const float sv, const float* xr, float (&acc)[MT]) {
  const uint32_t wd[4] = {wv.x, wv.y, wv.z, wv.w};
  if (BITS == 8) {
    float f[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t t = wd[i] ^ 0x80808080u;
      f[4 * i + 0] = byte_f32<0>(t, 8388736.0f);
      f[4 * i + 1] = byte_f32<1>(t, 8388736.0f);
      f[4 * i + 2] = byte_f32<2>(t, 8388736.0f);
      f[4 * i + 3] = byte_f32<3>(t, 8388736.0f);
    }
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      float a = acc[r];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 xv = *reinterpret_cast<const float4*>(xr + r * kStageK + 4 * i);
        a = fmaf(xv.x, f[4 * i + 0], a);
        a = fmaf(xv.y, f[4 * i + 1], a);
        a = fmaf(xv.z, f[4 * i + 2], a);
        a = fmaf(xv.w, f[4 * i + 3], a);
      }
      acc[r] = a;
    }
  } else {
    float f[32];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = wd[i] & 0x0F0F0F0Fu, hi = (wd[i] >> 4) & 0x0F0F0F0Fu;
      f[4 * i + 0] = byte_f32<0>(lo, 8388616.0f);
      f[4 * i + 1] = byte_f32<1>(lo, 8388616.0f);
      f[4 * i + 2] = byte_f32<2>(lo, 8388616.0f);
      f[4 * i + 3] = byte_f32<3>(lo, 8388616.0f);
      f[16 + 4 * i + 0] = byte_f32<0>(hi, 8388616.0f);
      f[16 + 4 * i + 1] = byte_f32<1>(hi, 8388616.0f);
      f[16 + 4 * i + 2] = byte_f32<2>(hi, 8388616.0f);
      f[16 + 4 * i + 3] = byte_f32<3>(hi, 8388616.0f);
    }
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      float p0 = 0.0f, p1 = 0.0f;  // two chains: rows 0-15 and 16-31 of the group
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 xa = *reinterpret_cast<const float4*>(xr + r * kStageK + 4 * i);
        const float4 xb = *reinterpret_cast<const float4*>(xr + r * kStageK + 16 + 4 * i);
        p0 = fmaf(xa.x, f[4 * i + 0], p0);
        p1 = fmaf(xb.x, f[16 + 4 * i + 0], p1);
        p0 = fmaf(xa.y, f[4 * i + 1], p0);
        p1 = fmaf(xb.y, f[16 + 4 * i + 1], p1);
        p0 = fmaf(xa.z, f[4 * i + 2], p0);
        p1 = fmaf(xb.z, f[16 + 4 * i + 2], p1);
        p0 = fmaf(xa.w, f[4 * i + 3], p0);
        p1 = fmaf(xb.w, f[16 + 4 * i + 3], p1);
      }
      acc[r] = fmaf(p0 + p1, sv, acc[r]);
    }
  }
}

// Dynamic shared memory layout.
template <int BITS, int MT>
struct Smem {
  static constexpr size_t kW = (size_t)kStages * kStageChunks * kCols * 16;
  static constexpr size_t kS = BITS == 4 ? (size_t)kStages * kStageChunks * kCols * 4 : 0;
  static constexpr size_t kX = (size_t)MT * kStageK * 4;
  static constexpr size_t off_w = 0, off_s = kW, off_x = kW + kS, off_red = kW + kS + kX;
  static size_t bytes(uint32_t splits) { return off_red + (size_t)splits * MT * kCols * 4 + 128; }
};

template <int BITS, int MT>
__global__ void __launch_bounds__(kCols) gemv_bulk_kernel(const Params p) {
  constexpr int CK = BITS == 8 ? 16 : 32;           // rows of W per chunk
  constexpr int kRoundStages = kStageK / (CK * kStageChunks);  // ring stages per staged round of x
  using L = Smem<BITS, MT>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[kStages];
  __shared__ float s_rstd[MT];
  __shared__ float s_red[kCols / 32];
  __shared__ int2 s_arg[kCols / 32];
  __shared__ unsigned s_flag;
  uint4* wring = reinterpret_cast<uint4*>(smem + L::off_w);
  float* sring = reinterpret_cast<float*>(smem + L::off_s);
  float* xs = reinterpret_cast<float*>(smem + L::off_x);
  float* red = reinterpret_cast<float*>(smem + L::off_red);

  const int tid = threadIdx.x;
  const uint32_t j0 = blockIdx.x * kCols;
  const uint32_t j = j0 + tid;
  const bool active = j < p.n;
  const uint32_t cols = min((uint32_t)kCols, p.n - j0);
  const uint32_t split = p.splits > 1 ? cluster_ctarank() : 0u;
  const uint32_t m0 = blockIdx.z * MT;
  const uint32_t rows = min((uint32_t)MT, p.m - m0);
  const uint32_t c_begin = min(p.chunks, split * p.chunks_per_cta);
  const uint32_t c_end = min(p.chunks, c_begin + p.chunks_per_cta);
  const uint32_t nst = (c_end - c_begin + kStageChunks - 1) / kStageChunks;

  auto issue = [&](uint32_t i) {  // one thread: request ring stage i
    const uint32_t slot = i % kStages;
    const uint32_t c0 = c_begin + i * kStageChunks;
    const uint32_t nch = min((uint32_t)kStageChunks, c_end - c0);
    mbar_expect_tx(&full[slot], nch * cols * (BITS == 4 ? 20u : 16u));
    for (uint32_t u = 0; u < nch; ++u) {
      bulk_load(wring + (size_t)(slot * kStageChunks + u) * kCols, p.w + (size_t)(c0 + u) * p.n + j0, cols * 16u, &full[slot]);
      if (BITS == 4) bulk_load(sring + (size_t)(slot * kStageChunks + u) * kCols, p.scale + (size_t)(c0 + u) * p.n + j0, cols * 4u, &full[slot]);
    }
  };

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_flag = 1;
  }
  __syncthreads();
  // weights do not depend on the predecessor kernel: fill the ring before waiting for it
  if (tid == 0)
    for (uint32_t i = 0; i < nst && i < (uint32_t)kStages; ++i) issue(i);
  if (tid == 0) trace_min(p.pro.trace, 0);
  grid_dependency_wait();
  if (tid == 0) trace_min(p.pro.trace, 1);
  grid_launch_dependents();
  const bool normed = p.pro.norm_w != nullptr;
  if (normed && tid < MT) {
    float ss = 0.0f;
    if (tid < (int)rows)
      for (uint32_t t = 0; t < p.pro.tiles; ++t) ss += p.pro.sumsq[(size_t)t * p.m + m0 + tid];
    s_rstd[tid] = 1.0f / sqrtf(ss * (1.0f / (float)p.k) + p.pro.eps);
  }

  float acc[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) acc[r] = 0.0f;

  for (uint32_t i = 0; i < nst; ++i) {
    if (i % kRoundStages == 0) {  // stage the next kStageK activations of every row
      __syncthreads();
      const uint32_t kbase = (c_begin + i * kStageChunks) * CK;
      const uint32_t len = min((uint32_t)kStageK, (c_end - c_begin - i * kStageChunks) * CK);
      for (uint32_t idx = tid; idx < MT * len; idx += kCols) {
        const uint32_t r = idx / len, kk = idx - r * len;
        const uint32_t kidx = kbase + kk;
        float v = 0.0f;
        if (r < rows && kidx < p.k) {
          v = load_as_f32(p.x, p.x_dtype, (size_t)(m0 + r) * p.x_ld + kidx);
          if (normed) v = v * s_rstd[r] * p.pro.norm_w[kidx];
        }
        xs[r * kStageK + kk] = v;
      }
      __syncthreads();
    }
    const uint32_t slot = i % kStages;
    if (!mbar_wait(&full[slot], (i / kStages) & 1u)) s_flag = 0;  // bounded; every thread waits on its own
    if (s_flag) {
      const uint32_t c0 = c_begin + i * kStageChunks;
      const uint32_t nch = min((uint32_t)kStageChunks, c_end - c0);
      const float* xr = xs + (i % kRoundStages) * kStageChunks * CK;
#pragma unroll
      for (int u = 0; u < kStageChunks; ++u) {
        if ((uint32_t)u < nch && active) {
          const uint4 wv = wring[(size_t)(slot * kStageChunks + u) * kCols + tid];
          const float sv = BITS == 4 ? sring[(size_t)(slot * kStageChunks + u) * kCols + tid] : 0.0f;
          consume_chunk<BITS, MT>(wv, sv, xr + u * CK, acc);
        }
      }
    }
    __syncthreads();  // everyone is done with this slot
    if (tid == 0 && s_flag && i + kStages < nst) issue(i + kStages);
  }
  if (!s_flag && tid == 0) atomicExch(p.status, 3);

  // ---- split-K inside the cluster: partial sums go to the first CTA through distributed shared memory ----
  if (p.splits > 1) {
    if (split != 0) {
#pragma unroll
      for (int r = 0; r < MT; ++r) st_cluster_f32(red + ((size_t)split * MT + r) * kCols + tid, 0, acc[r]);
    }
    cluster_sync_all();
    if (split != 0) { if (tid == 0) trace_max(p.pro.trace, 2); return; }
    for (uint32_t s = 1; s < p.splits; ++s) {
#pragma unroll
      for (int r = 0; r < MT; ++r) acc[r] += red[((size_t)s * MT + r) * kCols + tid];
    }
  }

  // ---- epilogue ----
  const float col_scale = (BITS == 8 && active) ? p.scale[j] : 1.0f;
  gemv_epilogue<MT, kCols>(p.epi, acc, rows, m0, p.m, j, active, BITS == 8, col_scale, p.out, s_red, s_arg, &s_flag);
  if (tid == 0) trace_max(p.pro.trace, 2);
}

template <int BITS, int MT>
cudaError_t launch_one(ruai_ctx* c, const Params& p, dim3 grid) {
  const size_t smem = Smem<BITS, MT>::bytes(p.splits);
  static bool attr_done[64] = {};  // per instantiation and device
  if (!attr_done[c->ordinal & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_bulk_kernel<BITS, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<BITS, MT>::bytes(8));
    if (e != cudaSuccess) return e;
    attr_done[c->ordinal & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kCols);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = c->stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (c->use_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (p.splits > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = p.splits;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  c->launches++;
  return cudaLaunchKernelEx(&cfg, gemv_bulk_kernel<BITS, MT>, p);
}

template <int BITS>
cudaError_t launch_mt(ruai_ctx* c, const Params& p, dim3 grid, int mt) {
  switch (mt) {
    case 1: return launch_one<BITS, 1>(c, p, grid);
    case 2: return launch_one<BITS, 2>(c, p, grid);
    case 4: return launch_one<BITS, 4>(c, p, grid);
    case 8: return launch_one<BITS, 8>(c, p, grid);
    default: return launch_one<BITS, 16>(c, p, grid);
  }
}

}  // namespace gemv_bulk

bool ruai_gemv_bulk_eligible(const ruai_qweight* w) {
  return w->layout == QL_CHUNK16 && (w->bits == 8 || w->n % 4 == 0);
}

int ruai_gemv_bulk_launch(ruai_ctx* c, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                          const GemvEpilogue& epi_in, const GemvPrologue& pro) {
  using namespace gemv_bulk;
  if (m == 0) return RUAI_OK;
  GemvEpilogue epi = epi_in;
  if (epi.act == ACT_SWIGLU && (w->n & 1)) return ruai_fail(c, RUAI_ERR_SHAPE, "SwiGLU epilogue needs an even column count, got %u", w->n);
  if (epi.out_ld == 0) epi.out_ld = epi.act == ACT_SWIGLU ? w->n / 2 : w->n;
  const int mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16;
  const uint32_t row_tiles = (m + mt - 1) / mt;
  const uint32_t col_tiles = (w->n + kCols - 1) / kCols;
  if (row_tiles > 65535) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "m too large");
  if (epi.argmax_out && (row_tiles != 1 || epi.act == ACT_SWIGLU)) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "fused argmax needs m <= 16");
  if (epi.sumsq && epi.act == ACT_SWIGLU) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "sum of squares with the SwiGLU epilogue");
  // split k over a cluster until there are about two CTAs per SM, keeping at least two ring stages per CTA
  uint32_t splits = 1;
  while (splits < 8 && col_tiles * row_tiles * splits < 2u * (uint32_t)c->sm_count && w->chunks / (splits * 2) >= 2u * kStageChunks) splits *= 2;
  uint32_t cpc = (w->chunks + splits - 1) / splits;
  cpc = (cpc + kStageChunks - 1) / kStageChunks * kStageChunks;
  Params p;
  p.w = (const uint4*)w->data; p.scale = w->scale; p.x = x; p.x_dtype = x_dtype; p.x_ld = x_ld;
  p.m = m; p.k = w->k; p.n = w->n; p.chunks = w->chunks; p.chunks_per_cta = cpc; p.splits = splits;
  p.out = out; p.status = c->status; p.epi = epi; p.pro = pro;
  p.pro.trace = ruai_trace_slot(c);
  const dim3 grid(col_tiles, splits, row_tiles);
  cudaError_t e = w->bits == 8 ? launch_mt<8>(c, p, grid, mt) : launch_mt<4>(c, p, grid, mt);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "bulk gemv launch failed: %s", cudaGetErrorString(e));
  return RUAI_OK;
}
