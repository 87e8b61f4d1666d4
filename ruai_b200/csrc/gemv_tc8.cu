// Fused GEMV on the tensor cores for int8 weights and up to 8 rows of activations per CTA.
//
// matmul_int8 (src/nn/backend/cpu.rs:897-927) is out[i,j] = scale[j] * sum_p x[i,p] * q[p,j].
// In the chunk layout (pack.cu) one chunk row of a 128-column tile is 2 KB holding, for each
// of 16 groups of 8 columns, 8 rows of 16 bytes: exactly the canonical K-major, unswizzled
// operand layout of `tcgen05.mma`.  So the packed weights need no work at all: a warp streams
// them HBM -> shared memory with bulk asynchronous copies (ring of stages, mbarrier per slot),
// another issues one `kind::i8` MMA per 32 rows of W straight on the ring, accumulating over
// this CTA's whole slice of k in tensor memory.
//
// The activations of the slice are written once per CTA as block fixed point with ONE scale
// per row: x = f * 2^(e-27), |f| <= 2^27, e from the row's largest magnitude in the slice, and f as
// four balanced base-128 digits (int8).  The tensor core returns D_t = sum_p q * d_t exactly
// (|D_t| < 2^25 for k <= 4096 per CTA); the epilogue forms ((D3*128 + D2)*128 + D1)*128 + D0 in f32 and
// multiplies by 2^(e-27) * scale[j].  An element much smaller than the row maximum keeps fewer
// significant bits, but its absolute error stays below 2^-28 of the largest product, which is
// inside the rounding of an f32 accumulation.  Split-K over a cluster, bounded waits and epilogues
// are those of gemv_tc.cu.
#include "common.cuh"
#include "gemv_epilogue.cuh"
#include "pipeline.cuh"

namespace gemv_tc8 {

using namespace pipe;

constexpr int kCols = kGemvBulkTileCols;  // 128
constexpr int kStageChunks = 4;           // chunk rows (16 k each) per ring stage: two MMAs of K = 32
constexpr int kLimbs = 4;
constexpr int kThreads = kCols + 64;
constexpr int kMaxSliceK = 4096;          // k per CTA (bounds the digit buffer and the s32 sums)

// ring stages (8 KB each): 10 for long slices of k with few rows (the digit buffer leaves room), 6 otherwise
constexpr int kStagesShort = 6, kStagesLong = 10;
constexpr int n_of(int mt) { return mt <= 4 ? 16 : 32; }
// Rows of the digit operand that are stored.  In the long-slice variant, with at most 8 rows in use (two rows of
// activations x four digits), only the first 8-row group is kept and the descriptor's stride between 8-row groups is
// 0: the MMA reads it twice and leaves a copy of columns 0-7 in columns 8-15 of the accumulator, which nobody reads.
// That halves the digit buffer and makes room for the longer ring.
constexpr int nb_of(int mt, int stages) { return mt <= 2 && stages == kStagesLong ? 8 : n_of(mt); }

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

template <int MT, int STAGES>
struct Smem {
  static constexpr int kNB = nb_of(MT, STAGES);
  static constexpr int kStages = STAGES;
  static constexpr size_t off_ring = 0;
  static constexpr size_t off_b = off_ring + (size_t)kStages * kStageChunks * kCols * 16;
  __host__ __device__ static size_t off_red(uint32_t slice_k) { return off_b + (size_t)(slice_k / 32) * kNB * 32; }
  __host__ __device__ static size_t bytes(uint32_t slice_k, uint32_t splits) { return off_red(slice_k) + (size_t)splits * MT * kCols * 4 + 128; }
};

template <int MT, int STAGES>
__global__ void __launch_bounds__(kThreads) gemv_tc_int8_kernel(const Params p, uint32_t slice_k) {
  constexpr int kN = n_of(MT);
  constexpr int kNB = nb_of(MT, STAGES);
  constexpr int kStages = STAGES;
  static_assert(MT * kLimbs <= kNB, "rows x limbs must fit the stored rows of the digit operand");
  using L = Smem<MT, STAGES>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[kStages];   // ring stage landed
  __shared__ __align__(8) uint64_t empty[kStages];  // MMAs that read the stage completed
  __shared__ __align__(8) uint64_t b_ready;         // digits written (4 warp arrivals)
  __shared__ __align__(8) uint64_t all_done;        // every MMA completed
  __shared__ uint32_t s_tmem;
  __shared__ float s_rstd[MT];
  __shared__ float s_max[MT][kCols / 32];
  __shared__ float s_xscale[MT];
  __shared__ float s_red[kThreads / 32];
  __shared__ int2 s_arg[kThreads / 32];
  __shared__ unsigned s_flag;
  __shared__ volatile int s_abort;
  uint4* ring = reinterpret_cast<uint4*>(smem + L::off_ring);
  unsigned char* bop = smem + L::off_b;
  float* red = reinterpret_cast<float*>(smem + L::off_red(slice_k));

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t j0 = blockIdx.x * kCols;
  const uint32_t j = j0 + tid;
  const bool active = tid < kCols && j < p.n;
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
    mbar_expect_tx(&full[slot], nch * cols * 16u);
    for (uint32_t u = 0; u < nch; ++u)
      bulk_load(ring + (size_t)(slot * kStageChunks + u) * kCols, p.w + (size_t)(c0 + u) * p.n + j0, cols * 16u, &full[slot]);
  };

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(&b_ready, kCols / 32);
    mbar_init(&all_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_abort = 0;
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(&s_tmem, 32);
  // the digit buffer starts as zeros (rows beyond rows x limbs, and k beyond the slice, stay zero)
  for (uint32_t i = tid; i < (slice_k / 32) * kNB * 32 / 16; i += kThreads) reinterpret_cast<uint4*>(bop)[i] = make_uint4(0, 0, 0, 0);
  // (an odd slice makes the last MMA read one chunk row that was never loaded: its digits are zero, so it adds nothing)
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s_tmem;
  // weights do not depend on the predecessor kernel: fill the ring before waiting for it
  if (tid == kCols + 32) {
    for (uint32_t i = 0; i < nst && i < (uint32_t)kStages; ++i) issue(i);
  }
  if (tid == 0) trace_min(p.pro.trace, 0);
  grid_dependency_wait();
  if (tid == 0) trace_min(p.pro.trace, 1);
  grid_launch_dependents();
  const bool normed = p.pro.norm_w != nullptr;
  if (normed && warp == kCols / 32 && lane < MT) {
    float ss = 0.0f;
    if (lane < (int)rows)
      for (uint32_t t = 0; t < p.pro.tiles; ++t) ss += p.pro.sumsq[(size_t)t * p.m + m0 + lane];
    s_rstd[lane] = 1.0f / sqrtf(ss * (1.0f / (float)p.k) + p.pro.eps);
  }
  float resid_pre[MT];
  const bool pre = p.epi.resid != nullptr && p.epi.act != ACT_SWIGLU && split == 0 && active;
#pragma unroll
  for (int r = 0; r < MT; ++r) resid_pre[r] = (pre && r < (int)rows) ? p.epi.resid[(size_t)(m0 + r) * p.epi.out_ld + j] : 0.0f;

  float acc[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) acc[r] = 0.0f;

  if (warp == kCols / 32) {
    // ===== MMA issuer =====
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_i8(kN, true);
      const uint64_t ad0 = umma_desc_kmajor(smem_u32(ring), kCols * 16, 128);
      const uint64_t bd0 = umma_desc_kmajor(smem_u32(bop), kNB / 8 * 128, kNB == kN ? 128 : 0);
      bool ok = mbar_wait(&b_ready, 0);
      uint32_t left = c_end - c_begin, slot = 0, par = 0;
      uint64_t bd = bd0;
      for (uint32_t i = 0; i < nst && ok; ++i, left -= kStageChunks) {
        if (!mbar_wait(&full[slot], par)) { ok = false; break; }
        tc_fence_after_sync();
        const uint64_t ad = umma_desc_advance(ad0, slot * (kStageChunks * kCols * 16));
        // one MMA per two chunk rows (K = 32); an odd last chunk is paired with digits that are zero
        umma_i8(tmem_base, ad, bd, idesc, i != 0u ? 1u : 0u);
        if (left > 2) umma_i8(tmem_base, umma_desc_advance(ad, 2 * kCols * 16), umma_desc_advance(bd, kNB * 32), idesc, 1u);
        bd = umma_desc_advance(bd, 2 * kNB * 32);
        umma_commit(&empty[slot]);
        if (++slot == (uint32_t)kStages) { slot = 0; par ^= 1u; }
      }
      if (ok) umma_commit(&all_done);
      else s_abort = 1;
    }
  } else if (warp == kCols / 32 + 1) {
    // ===== copy issuer: refill a ring slot once its MMAs are done =====
    if (lane == 0) {
      for (uint32_t i = kStages; i < nst; ++i) {
        if (s_abort || !mbar_wait(&empty[i % kStages], ((i / kStages) - 1) & 1u)) { s_abort = 1; break; }
        issue(i);
      }
    }
  } else {
    // ===== four warps: activations -> four int8 digits per value, one scale per row =====
    const uint32_t kbeg = c_begin * 16, kend = min(p.k, c_end * 16);
    const bool vec = p.x_dtype == RUAI_F32 && (p.x_ld & 3u) == 0 && (p.k & 3u) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0 &&
                     (!normed || (reinterpret_cast<uintptr_t>(p.pro.norm_w) & 15u) == 0);
    const uint32_t nvec = kend > kbeg ? (kend - kbeg) >> 2 : 0u;  // float4 per row in the slice
    constexpr int R = 8 / MT;                                      // float4 per row a thread can keep in registers
    const float4* xv = reinterpret_cast<const float4*>(p.x);
    const float4* nv = reinterpret_cast<const float4*>(p.pro.norm_w);
    auto load4 = [&](uint32_t r, uint32_t idx) -> float4 {  // float4 number idx of row r of the slice, normed
      float4 v = __ldg(xv + (((size_t)(m0 + r) * p.x_ld + kbeg) >> 2) + idx);
      if (normed) {
        const float4 g = __ldg(nv + (kbeg >> 2) + idx);
        v.x *= g.x; v.y *= g.y; v.z *= g.z; v.w *= g.w;
      }
      return v;
    };
    // (fmaxf drops NaN: a NaN or an infinity in the row is looked for on its own and makes the maximum infinite, which
    // turns the row's scale and with it its sums into NaN, as f32 arithmetic would: cpu.rs:1002-1029 propagates them)
    auto max4 = [](float mx, const float4& v) {
      const bool fin = fabsf(v.x) <= 3.402823466e38f && fabsf(v.y) <= 3.402823466e38f && fabsf(v.z) <= 3.402823466e38f && fabsf(v.w) <= 3.402823466e38f;
      return fin ? fmaxf(fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w))) : INFINITY;
    };
    auto row_max = [&](int r, float mx) {  // 128-thread maximum of one row: warp part here, the rest after the barrier
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
      if (lane == 0) s_max[r][warp] = mx;
    };
    auto row_scale = [&](int r) -> float {  // 2^(27 - e) for the row, and its inverse for the epilogue
      float gmax = 0.0f;
#pragma unroll
      for (int w2 = 0; w2 < kCols / 32; ++w2) gmax = fmaxf(gmax, s_max[r][w2]);
      const uint32_t eb = __float_as_uint(gmax) >> 23;
      const bool nz = eb >= 27u && eb < 255u;
      if (tid == 0) s_xscale[r] = eb == 255u ? __int_as_float(0x7fc00000) : (nz ? __uint_as_float((eb - 26u) << 23) : 0.0f);  // 2^(e - 27), e = eb - 126
      return nz ? __uint_as_float((280u - eb) << 23) : 0.0f;
    };
    // digits of four consecutive k of row r into the B operand: group g = 32 k, [k-half][n/8][n%8][16 bytes]
    auto put4 = [&](int r, uint32_t idx, const float4& v, float up) {
      int f[4] = {__float2int_rn(v.x * up), __float2int_rn(v.y * up), __float2int_rn(v.z * up), __float2int_rn(v.w * up)};
      const uint32_t rel = idx << 2, g = rel >> 5, l = rel & 31u;
      unsigned char* bg = bop + (size_t)g * (kNB * 32) + (l >> 4) * (kNB / 8 * 128) + (l & 15u);
#pragma unroll
      for (int t = kLimbs - 1; t >= 0; --t) {  // least significant digit first; operand rows: most significant first
        uint32_t pack = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int dgt = t > 0 ? ((f[e] + 64) & 127) - 64 : f[e];
          f[e] = (f[e] - dgt) >> 7;
          pack |= (uint32_t)(dgt & 255) << (8 * e);
        }
        const uint32_t nrow = r * kLimbs + t;
        *reinterpret_cast<uint32_t*>(bg + (nrow >> 3) * 128 + (nrow & 7u) * 16) = pack;
      }
    };
    if (vec && nvec <= (uint32_t)(R * kCols)) {
      // the whole slice of every row fits this thread's registers: one round of loads
      float4 v[MT][R];
#pragma unroll
      for (int r = 0; r < MT; ++r)
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const uint32_t idx = i * kCols + tid;
          v[r][i] = (r < (int)rows && idx < nvec) ? load4(r, idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        float mx = 0.0f;
#pragma unroll
        for (int i = 0; i < R; ++i) mx = max4(mx, v[r][i]);
        row_max(r, mx);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        const float up = row_scale(r);
        if (r < (int)rows)
#pragma unroll
          for (int i = 0; i < R; ++i) {
            const uint32_t idx = i * kCols + tid;
            if (idx < nvec) put4(r, idx, v[r][i], up);
          }
      }
    } else if (vec) {
      // two passes, eight independent 16-byte loads in flight per thread
      const uint32_t per_row = (nvec + kCols - 1) / kCols;
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        float mx = 0.0f;
        if (r < (int)rows)
          for (uint32_t i0 = 0; i0 < per_row; i0 += 8) {
            float4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t idx = (i0 + i) * kCols + tid;
              v[i] = idx < nvec ? load4(r, idx) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) mx = max4(mx, v[i]);
          }
        row_max(r, mx);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        const float up = row_scale(r);
        if (r < (int)rows)
          for (uint32_t i0 = 0; i0 < per_row; i0 += 8) {
            float4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t idx = (i0 + i) * kCols + tid;
              v[i] = idx < nvec ? load4(r, idx) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t idx = (i0 + i) * kCols + tid;
              if (idx < nvec) put4(r, idx, v[i], up);
            }
          }
      }
    } else {
      // any dtype, any alignment: one value at a time
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        float mx = 0.0f;
        if (r < (int)rows)
          for (uint32_t kk = kbeg + tid; kk < kend; kk += kCols) {
            float v = load_as_f32(p.x, p.x_dtype, (size_t)(m0 + r) * p.x_ld + kk);
            if (normed) v *= p.pro.norm_w[kk];
            mx = fabsf(v) <= 3.402823466e38f ? fmaxf(mx, fabsf(v)) : INFINITY;
          }
        row_max(r, mx);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        const float up = row_scale(r);
        if (r < (int)rows)
          for (uint32_t kk = kbeg + tid; kk < kend; kk += kCols) {
            float v = load_as_f32(p.x, p.x_dtype, (size_t)(m0 + r) * p.x_ld + kk);
            if (normed) v *= p.pro.norm_w[kk];
            int f = __float2int_rn(v * up);
            const uint32_t rel = kk - kbeg, g = rel >> 5, l = rel & 31;
            unsigned char* bg = bop + (size_t)g * (kNB * 32) + (l >> 4) * (kNB / 8 * 128) + (l & 15);
#pragma unroll
            for (int t = kLimbs - 1; t >= 0; --t) {
              const int dgt = t > 0 ? ((f + 64) & 127) - 64 : f;
              f = (f - dgt) >> 7;
              const uint32_t nrow = r * kLimbs + t;
              bg[(nrow >> 3) * 128 + (nrow & 7) * 16] = (unsigned char)(signed char)dgt;
            }
          }
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&b_ready);
    // ---- the sums, once every MMA has completed ----
    if (!mbar_wait(&all_done, 0)) s_abort = 1;
    else if (nst > 0) {
      tc_fence_after_sync();
      const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        int32_t d[4];
        tmem_ld4(tmem_base + lane_base + kLimbs * r, d);
        tmem_ld_wait();
        float v = (float)d[0];
        v = fmaf(v, 128.0f, (float)d[1]);
        v = fmaf(v, 128.0f, (float)d[2]);
        v = fmaf(v, 128.0f, (float)d[3]);
        acc[r] = v * s_xscale[r];
      }
      tc_fence_before_sync();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (s_abort && tid == 0) atomicExch(p.status, 3);
  if (warp == 0) tmem_dealloc(tmem_base, 32);

  // ---- split-K inside the cluster ----
  if (p.splits > 1) {
    if (split != 0 && tid < kCols) {
#pragma unroll
      for (int r = 0; r < MT; ++r) st_cluster_f32(red + ((size_t)split * MT + r) * kCols + tid, 0, acc[r]);
    }
    cluster_sync_all();
    if (split != 0) { if (tid == 0) trace_max(p.pro.trace, 2); return; }
    if (tid < kCols) {
      for (uint32_t s = 1; s < p.splits; ++s) {
#pragma unroll
        for (int r = 0; r < MT; ++r) acc[r] += red[((size_t)s * MT + r) * kCols + tid];
      }
    }
  }
  if (normed) {
#pragma unroll
    for (int r = 0; r < MT; ++r) acc[r] *= s_rstd[r];
  }
  const float col_scale = active ? p.scale[j] : 1.0f;
  gemv_epilogue<MT, kThreads>(p.epi, acc, rows, m0, p.m, j, active, true, col_scale, p.out, s_red, s_arg, &s_flag, pre ? resid_pre : nullptr);
  if (tid == 0) trace_max(p.pro.trace, 2);
}

template <int MT, int STAGES>
cudaError_t launch_one(ruai_ctx* c, const Params& p, dim3 grid, uint32_t slice_k) {
  static bool attr_done[64] = {};
  if (!attr_done[c->ordinal & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_tc_int8_kernel<MT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<MT, STAGES>::bytes(kMaxSliceK, 8));
    if (e != cudaSuccess) return e;
    attr_done[c->ordinal & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Smem<MT, STAGES>::bytes(slice_k, p.splits);
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
  return cudaLaunchKernelEx(&cfg, gemv_tc_int8_kernel<MT, STAGES>, p, slice_k);
}

}  // namespace gemv_tc8

bool ruai_gemv_tc8_eligible(const ruai_qweight* w, uint32_t m) {
  return w->layout == QL_CHUNK16 && w->bits == 8 && m >= 1 && m <= 16 && w->k <= 8u * (uint32_t)gemv_tc8::kMaxSliceK;
}

int ruai_gemv_tc8_launch(ruai_ctx* c, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                         const GemvEpilogue& epi_in, const GemvPrologue& pro) {
  using namespace gemv_tc8;
  GemvEpilogue epi = epi_in;
  if (epi.act == ACT_SWIGLU && (w->n & 1)) return ruai_fail(c, RUAI_ERR_SHAPE, "SwiGLU epilogue needs an even column count, got %u", w->n);
  if (epi.out_ld == 0) epi.out_ld = epi.act == ACT_SWIGLU ? w->n / 2 : w->n;
  if (epi.sumsq && epi.act == ACT_SWIGLU) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "sum of squares with the SwiGLU epilogue");
  const int mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : 8;
  const uint32_t row_tiles = (m + mt - 1) / mt;
  if (epi.argmax_out && (row_tiles != 1 || epi.act == ACT_SWIGLU)) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "fused argmax needs a single row tile");
  const uint32_t col_tiles = (w->n + kCols - 1) / kCols;
  // the slice of k per CTA is bounded (digit buffer, 32-bit sums); beyond that, split over a cluster
  uint32_t splits = 1;
  // and short enough that a thread converts its part of every row from registers (4096 / rows values of k)
  while (splits < 8 && (w->chunks + splits - 1) / splits * 16 > (uint32_t)kMaxSliceK / mt) splits *= 2;
  const uint32_t slots = 3u * (uint32_t)c->sm_count;
  double best = 1e30;
  uint32_t best_s = splits;
  for (uint32_t s2 = splits; s2 <= 8; s2 *= 2) {
    const uint32_t per = (w->chunks + s2 - 1) / s2;
    if (s2 > splits && per < 2u * kStageChunks) break;
    const uint32_t stages = (per + kStageChunks - 1) / kStageChunks;
    const uint32_t waves = (col_tiles * row_tiles * s2 + slots - 1) / slots;
    const double t = waves * (6.0 + 0.4 * stages + 0.15 * s2);
    if (t < best) { best = t; best_s = s2; }
  }
  splits = best_s;
  if ((c->force_splits & 255u) && (c->force_splits & 255u) >= splits && (c->force_splits & 255u) <= 8) splits = c->force_splits & 255u;
  uint32_t cpc = (w->chunks + splits - 1) / splits;
  cpc = (cpc + kStageChunks - 1) / kStageChunks * kStageChunks;
  if (cpc * 16 > (uint32_t)kMaxSliceK) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "k = %u is too large for the int8 tensor-core GEMV", w->k);
  const uint32_t slice_k = (cpc * 16 + 31) / 32 * 32;
  Params p;
  p.w = (const uint4*)w->data; p.scale = w->scale; p.x = x; p.x_dtype = x_dtype; p.x_ld = x_ld;
  p.m = m; p.k = w->k; p.n = w->n; p.chunks = w->chunks; p.chunks_per_cta = cpc; p.splits = splits;
  p.out = out; p.status = c->status; p.epi = epi; p.pro = pro;
  p.pro.trace = ruai_trace_slot(c);
  const dim3 grid(col_tiles, splits, row_tiles);
  const bool deep = mt <= 2 && slice_k >= 4096;  // a long slice of k and a small digit buffer: the deeper ring pays
  cudaError_t e = mt == 1 ? (deep ? launch_one<1, kStagesLong>(c, p, grid, slice_k) : launch_one<1, kStagesShort>(c, p, grid, slice_k))
                : mt == 2 ? (deep ? launch_one<2, kStagesLong>(c, p, grid, slice_k) : launch_one<2, kStagesShort>(c, p, grid, slice_k))
                : mt == 4 ? launch_one<4, kStagesShort>(c, p, grid, slice_k) : launch_one<8, kStagesShort>(c, p, grid, slice_k);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "int8 tensor-core gemv launch failed: %s", cudaGetErrorString(e));
  return RUAI_OK;
}
