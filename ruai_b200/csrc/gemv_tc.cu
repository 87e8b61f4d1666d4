// Fused dequantize + GEMV on the tensor cores (tcgen05, accumulators in tensor memory) for
// int4 group-32 weights and up to four rows of activations: the decode hot path.
//
// Why tensor cores for a memory-bound kernel: at full HBM speed one SM has to consume about
// 46 int4 weights per clock.  On the CUDA cores every weight costs a byte permute, a
// subtract and a fused multiply-add, which is more than the SM can issue; here a weight
// costs 3/8 of a logic instruction (nibbles -> bytes) and the multiply-adds run as
// `tcgen05.mma kind::i8`, integer and therefore exact.
//
// Arithmetic.  matmul_int4 (src/nn/backend/cpu.rs:1035-1067) is
//     out[i,j] = sum_g scale[g,j] * sum_{l in g} x[i,l] * q[l,j],   q in [-8, 7].
// Per row and group of 32 the activations are written as block fixed point,
// x = f * 2^(e-20) with |f| <= 2^20 (e from the group's largest magnitude), and f as three
// balanced base-128 digits f = d0*2^14 + d1*2^7 + d2, each an int8.  The stored weights are
// u = q + 8 (0..15, see pack.cu), so
//     sum_l x*q = 2^(e-20) * (2^14*D0 + 2^7*D1 + D2 - 8*sum_l f),  D_t = sum_l u*d_t,
// where D_t is what one MMA (M = 128 columns of W, N = 16, K = 32) leaves in TMEM, exactly.
// The integer is converted to f32 once per (group, column, row) and multiplied by
// scale[g,j] * 2^(e-20).  The rounding of x to 21 significant bits relative to its group
// maximum is the only approximation (relative error of a group sum about 2^-21).
//
// Data movement is that of gemv_bulk.cu: a ring of bulk asynchronous copies of the chunk
// layout (2 KB of packed weights + 512 B of scales per group and 128-column tile), filled
// before the grid-dependency wait; split-K over a cluster with the partial sums sent
// through distributed shared memory; bounded waits everywhere.
#include "common.cuh"
#include "gemv_epilogue.cuh"
#include "pipeline.cuh"

namespace gemv_tc {

using namespace pipe;

constexpr int kCols = kGemvBulkTileCols;  // 128 = MMA M = TMEM lanes = threads
constexpr int kStageGroups = 4;           // scale groups (chunks) per ring stage
constexpr int kRoundGroups = 16;          // groups per conversion round of the activations
constexpr int kLimbs = 3;
// MMA N (rows x limbs, padded to a multiple of 16) and the TMEM columns of two stages of accumulators
constexpr int n_of(int mt) { return mt <= 4 ? 16 : mt <= 8 ? 32 : 48; }
constexpr int tmem_cols_of(int mt) { return 2 * kStageGroups * n_of(mt) <= 128 ? 128 : 2 * kStageGroups * n_of(mt) <= 256 ? 256 : 512; }

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
  long long* prof;  // debug: cycle stamps of one CTA (NULL in normal use)
};

template <int MT>
struct Smem {
  static constexpr int kN = n_of(MT);
  static constexpr size_t off_a = 0;
  static constexpr size_t off_b = off_a + 2 * (size_t)kStageGroups * kCols * 32;
  static constexpr size_t off_meta = off_b + 2 * (size_t)kRoundGroups * kN * 32;
  static constexpr size_t off_red = off_meta + 2 * (size_t)kRoundGroups * MT * 8;
  static size_t bytes(uint32_t splits) { return off_red + (size_t)splits * MT * kCols * 4 + 128; }
};

constexpr int kThreads = kCols + 32;  // four loading / converting / draining warps and one MMA-issuing warp

// kAheadStages: stages of packed weights held in registers ahead of their use (2: more CTAs per SM; 4: more
// bytes in flight per CTA, for launches with few CTAs per SM).
template <int MT, int kAheadStages>
__global__ void __launch_bounds__(kThreads) gemv_tc_int4_kernel(const Params p) {
  constexpr int kN = n_of(MT);
  constexpr int kTmemCols = tmem_cols_of(MT);
  static_assert(MT * kLimbs <= kN, "rows x limbs must fit the MMA N");
  using L = Smem<MT>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t a_ready[2];      // A operand (and digits) of a stage written (4 warp arrivals)
  __shared__ __align__(8) uint64_t mma_done[2];     // MMAs of a stage completed
  __shared__ uint32_t s_tmem;
  __shared__ float s_rstd[MT];
  __shared__ float s_red[kThreads / 32];
  __shared__ int2 s_arg[kThreads / 32];
  __shared__ unsigned s_flag;
  __shared__ volatile int s_abort;
  unsigned char* abuf = smem + L::off_a;
  unsigned char* bop = smem + L::off_b;
  float* meta_scale = reinterpret_cast<float*>(smem + L::off_meta);        // [2][kRoundGroups][MT]
  int* meta_sum = reinterpret_cast<int*>(smem + L::off_meta) + 2 * kRoundGroups * MT;
  float* red = reinterpret_cast<float*>(smem + L::off_red);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  long long* prof = (p.prof && blockIdx.x == 7 && blockIdx.y == 0 && (tid == 0 || tid == 64)) ? p.prof + (tid ? 512 : 0) : nullptr;
  int pn = 0;
#define STAMP() do { if (prof && pn < 500) prof[pn++] = clock64(); } while (0)
  STAMP();
  const uint32_t j0 = blockIdx.x * kCols;
  const uint32_t j = j0 + tid;
  const bool active = tid < kCols && j < p.n;
  const uint32_t cols = min((uint32_t)kCols, p.n - j0);
  const uint32_t split = p.splits > 1 ? cluster_ctarank() : 0u;
  const uint32_t m0 = blockIdx.z * MT;
  const uint32_t rows = min((uint32_t)MT, p.m - m0);
  const uint32_t c_begin = min(p.chunks, split * p.chunks_per_cta);
  const uint32_t c_end = min(p.chunks, c_begin + p.chunks_per_cta);
  const uint32_t nst = (c_end - c_begin + kStageGroups - 1) / kStageGroups;
  constexpr uint32_t kRoundStages = kRoundGroups / kStageGroups;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) { mbar_init(&a_ready[s], kCols / 32); mbar_init(&mma_done[s], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_abort = 0;
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(&s_tmem, kTmemCols);
  // rows of the B operand beyond rows x limbs stay zero for the whole kernel
  for (uint32_t i = tid; i < 2 * kRoundGroups * kN * 32 / 16; i += kThreads) reinterpret_cast<uint4*>(bop)[i] = make_uint4(0, 0, 0, 0);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s_tmem;
  STAMP();
  // packed weights and scales of this thread's column, kAheadStages stages ahead of their use.  They do not
  // depend on the predecessor kernel: the first ones are requested before waiting for it.
  uint4 wq[kAheadStages][kStageGroups];
  float sq[kAheadStages][kStageGroups];
  auto load_stage = [&](uint32_t i, uint4 (&wv)[kStageGroups], float (&sv)[kStageGroups]) {
#pragma unroll
    for (int u = 0; u < kStageGroups; ++u) {
      const uint32_t c = c_begin + i * kStageGroups + u;
      const bool in = tid < kCols && j < p.n && i < nst && c < c_end;
      wv[u] = in ? __ldcs(&p.w[(size_t)c * p.n + j]) : make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
      sv[u] = in ? __ldcs(&p.scale[(size_t)c * p.n + j]) : 0.0f;
    }
  };
  if (tid < kCols) {
#pragma unroll
    for (int a = 0; a < kAheadStages; ++a) load_stage(a, wq[a], sq[a]);
  }
  if (tid == 0) {  // warm the L2 for the kernel after this one
    const uint32_t cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, n_ctas = gridDim.x * gridDim.y * gridDim.z;
    l2_prefetch_share(p.pro.next_data, p.pro.next_data_bytes, cta, n_ctas);
    l2_prefetch_share(p.pro.next_scale, p.pro.next_scale_bytes, cta, n_ctas);
  }
  if (tid == 0) trace_min(p.pro.trace, 0);
  grid_dependency_wait();
  if (tid == 0) trace_min(p.pro.trace, 1);
  grid_launch_dependents();
  // RMSNorm: x * rstd * w with rstd a per-row scalar, so the digits are taken from x * w and rstd multiplies
  // the finished sums; its inputs are fetched now and not needed before the end.
  const bool normed = p.pro.norm_w != nullptr;
  if (normed && warp == kCols / 32 && lane < MT) {
    float ss = 0.0f;
    if (lane < (int)rows)
      for (uint32_t t = 0; t < p.pro.tiles; ++t) ss += p.pro.sumsq[(size_t)t * p.m + m0 + lane];
    s_rstd[lane] = 1.0f / sqrtf(ss * (1.0f / (float)p.k) + p.pro.eps);
  }
  // the residual this CTA will add in its epilogue, fetched before the main loop
  float resid_pre[MT];
  const bool pre = p.epi.resid != nullptr && p.epi.act != ACT_SWIGLU && split == 0 && active;
#pragma unroll
  for (int r = 0; r < MT; ++r) resid_pre[r] = (pre && r < (int)rows) ? p.epi.resid[(size_t)(m0 + r) * p.epi.out_ld + j] : 0.0f;

  float acc[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) acc[r] = 0.0f;

  if (warp == kCols / 32) {
    // ===== MMA issuer: one thread =====
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_i8(kN, false);
      for (uint32_t i = 0; i < nst; ++i) {
        if (s_abort || !mbar_wait(&a_ready[i & 1], (i >> 1) & 1u)) { s_abort = 1; break; }
        tc_fence_after_sync();
        const uint32_t rb = (i / kRoundStages) & 1u, g0 = (i % kRoundStages) * kStageGroups;
        const uint32_t nch = min((uint32_t)kStageGroups, c_end - (c_begin + i * kStageGroups));
        for (uint32_t u = 0; u < nch; ++u) {
          const uint64_t ad = umma_desc_kmajor(smem_u32(abuf + ((size_t)(i & 1) * kStageGroups + u) * (kCols * 32)), kCols * 16, 128);
          const uint64_t bd = umma_desc_kmajor(smem_u32(bop + ((size_t)rb * kRoundGroups + g0 + u) * (kN * 32)), kN / 8 * 128, 128);
          umma_i8(tmem_base + ((i & 1) * kStageGroups + u) * kN, ad, bd, idesc, 0u);
        }
        umma_commit(&mma_done[i & 1]);
      }
    }
  } else {
    // ===== four warps: activations -> digits, nibbles -> bytes, scaled sums out of TMEM =====
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float sv_prev[kStageGroups] = {0.f, 0.f, 0.f, 0.f};
    // activations of one round (16 groups = 512 values per row): 4 consecutive values per thread, fetched a round ahead
    float4 xnext[MT];
    auto fetch_round = [&](uint32_t stage0) {
      const uint32_t kidx = (c_begin + stage0 * kStageGroups) * 32 + 4 * tid;
      const bool in = stage0 < nst && c_begin + stage0 * kStageGroups + tid / 8 < c_end;
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (in && r < (int)rows) {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            if (kidx + t < p.k) {
              v[t] = load_as_f32(p.x, p.x_dtype, (size_t)(m0 + r) * p.x_ld + kidx + t);
              if (normed) v[t] = v[t] * p.pro.norm_w[kidx + t];
            }
          }
        }
        xnext[r] = make_float4(v[0], v[1], v[2], v[3]);
      }
    };
    fetch_round(0);
    STAMP();

    // scaled sums of stage s (its MMAs must have completed) into acc
    auto drain = [&](uint32_t s, const float (&sv)[kStageGroups]) -> bool {
      if (!mbar_wait(&mma_done[s & 1], (s >> 1) & 1u)) return false;
      tc_fence_after_sync();
      const uint32_t rb = (s / kRoundStages) & 1u;
      const uint32_t g0 = (s % kRoundStages) * kStageGroups;
      const uint32_t nch = min((uint32_t)kStageGroups, c_end - (c_begin + s * kStageGroups));
      constexpr int kQ = (MT * kLimbs + 3) / 4;  // 4-column loads per group
      constexpr int kBatch = MT <= 4 ? kStageGroups : 1;  // groups whose sums are in registers at once
#pragma unroll
      for (int u0 = 0; u0 < kStageGroups; u0 += kBatch) {
        int32_t d[kBatch][kQ * 4];
#pragma unroll
        for (int ub = 0; ub < kBatch; ++ub) {
          const uint32_t col = tmem_base + lane_base + ((s & 1) * kStageGroups + u0 + ub) * kN;
#pragma unroll
          for (int q4 = 0; q4 < kQ; ++q4) {
            int32_t t4[4];
            tmem_ld4(col + 4 * q4, t4);  // groups past the end hold stale sums; they are not used below
            d[ub][4 * q4 + 0] = t4[0]; d[ub][4 * q4 + 1] = t4[1]; d[ub][4 * q4 + 2] = t4[2]; d[ub][4 * q4 + 3] = t4[3];
          }
        }
        tmem_ld_wait();
#pragma unroll
        for (int ub = 0; ub < kBatch; ++ub) {
          const int u = u0 + ub;
          if ((uint32_t)u < nch) {
#pragma unroll
            for (int r = 0; r < MT; ++r) {
              const uint32_t mi = (rb * kRoundGroups + g0 + u) * MT + r;
              const int val = d[ub][kLimbs * r] * 16384 + d[ub][kLimbs * r + 1] * 128 + d[ub][kLimbs * r + 2] - 8 * meta_sum[mi];
              acc[r] = fmaf((float)val, sv[u] * meta_scale[mi], acc[r]);
            }
          }
        }
      }
      tc_fence_before_sync();
      return true;
    };

    bool ok = true;
    for (uint32_t i = 0; i < nst && ok; ++i) {
      if (s_abort) { ok = false; break; }
      const uint32_t rb = (i / kRoundStages) & 1u;
      if (i % kRoundStages == 0) {
        // ---- this warp's 4 groups of the round (8 lanes per group): block fixed point, three int8 digits ----
        const uint32_t gi = warp * 4 + (lane >> 3);
#pragma unroll
        for (int r = 0; r < MT; ++r) {
          const float4 xv = xnext[r];
          float gmax = fmaxf(fmaxf(fabsf(xv.x), fabsf(xv.y)), fmaxf(fabsf(xv.z), fabsf(xv.w)));
          gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 1));
          gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 2));
          gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 4));
          // gmax < 2^e with e = biased exponent - 126; f = round(v * 2^(20-e)), x = f * 2^(e-20)
          const uint32_t eb = __float_as_uint(gmax) >> 23;
          const bool nz = eb >= 20u && eb < 255u;
          const float up = nz ? __uint_as_float((273u - eb) << 23) : 0.0f;
          const float xscale = nz ? __uint_as_float((eb - 19u) << 23) : 0.0f;
          const float vv[4] = {xv.x, xv.y, xv.z, xv.w};
          uint32_t w0 = 0, w1 = 0, w2 = 0;
          int fs = 0;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int f = __float2int_rn(vv[t] * up);
            const int d2 = ((f + 64) & 127) - 64;
            const int t1 = (f - d2) >> 7;
            const int d1 = ((t1 + 64) & 127) - 64;
            const int d0 = (t1 - d1) >> 7;
            fs += f;
            w0 |= (uint32_t)(d0 & 0xFF) << (8 * t);
            w1 |= (uint32_t)(d1 & 0xFF) << (8 * t);
            w2 |= (uint32_t)(d2 & 0xFF) << (8 * t);
          }
          fs += __shfl_xor_sync(0xFFFFFFFFu, fs, 1);
          fs += __shfl_xor_sync(0xFFFFFFFFu, fs, 2);
          fs += __shfl_xor_sync(0xFFFFFFFFu, fs, 4);
          unsigned char* bg = bop + ((size_t)rb * kRoundGroups + gi) * (kN * 32) + ((lane & 7) >> 2) * (kN / 8 * 128) + ((4 * (lane & 7)) & 15);
          const uint32_t ww[kLimbs] = {w0, w1, w2};
#pragma unroll
          for (int t = 0; t < kLimbs; ++t) {
            const uint32_t nrow = r * kLimbs + t;
            *reinterpret_cast<uint32_t*>(bg + (nrow >> 3) * 128 + (nrow & 7) * 16) = ww[t];
          }
          if ((lane & 7) == 0) {
            meta_scale[(rb * kRoundGroups + gi) * MT + r] = xscale;
            meta_sum[(rb * kRoundGroups + gi) * MT + r] = fs;
          }
        }
        fetch_round(i + kRoundStages);
      }
      STAMP();
      float sv_cur[kStageGroups];
      // nibbles -> bytes: 32 rows of this thread's column become one row of two 16-byte k-halves of A
#pragma unroll
      for (int u = 0; u < kStageGroups; ++u) {
        const uint4 wv = wq[0][u];
        sv_cur[u] = sq[0][u];
        uint4 lo, hi;
        lo.x = wv.x & 0x0F0F0F0Fu; hi.x = (wv.x >> 4) & 0x0F0F0F0Fu;
        lo.y = wv.y & 0x0F0F0F0Fu; hi.y = (wv.y >> 4) & 0x0F0F0F0Fu;
        lo.z = wv.z & 0x0F0F0F0Fu; hi.z = (wv.z >> 4) & 0x0F0F0F0Fu;
        lo.w = wv.w & 0x0F0F0F0Fu; hi.w = (wv.w >> 4) & 0x0F0F0F0Fu;
        unsigned char* a = abuf + ((size_t)(i & 1) * kStageGroups + u) * (kCols * 32) + (size_t)tid * 16;
        *reinterpret_cast<uint4*>(a) = lo;
        *reinterpret_cast<uint4*>(a + kCols * 16) = hi;
      }
      // shift the register queue and request the stage kAheadStages further on
#pragma unroll
      for (int a = 0; a + 1 < kAheadStages; ++a) {
#pragma unroll
        for (int u = 0; u < kStageGroups; ++u) { wq[a][u] = wq[a + 1][u]; sq[a][u] = sq[a + 1][u]; }
      }
      load_stage(i + kAheadStages, wq[kAheadStages - 1], sq[kAheadStages - 1]);
      STAMP();
      // this warp's part of the A operand (and of the digits) is in place and its reads of the raw slot are done
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_ready[i & 1]);
      STAMP();
      if (i > 0) ok = drain(i - 1, sv_prev);
      STAMP();
#pragma unroll
      for (int u = 0; u < kStageGroups; ++u) sv_prev[u] = sv_cur[u];
    }
    if (ok && nst > 0) ok = drain(nst - 1, sv_prev);
    if (!ok) s_abort = 1;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (s_abort && tid == 0) atomicExch(p.status, 3);
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);

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
  gemv_epilogue<MT, kThreads>(p.epi, acc, rows, m0, p.m, j, active, false, 1.0f, p.out, s_red, s_arg, &s_flag, pre ? resid_pre : nullptr);
  if (tid == 0) trace_max(p.pro.trace, 2);
  STAMP();
  if (prof) prof[511] = pn;
#undef STAMP
}

template <int MT, int AHEAD>
cudaError_t launch_one(ruai_ctx* c, const Params& p, dim3 grid) {
  static bool attr_done[64] = {};
  if (!attr_done[c->ordinal & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_tc_int4_kernel<MT, AHEAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<MT>::bytes(8));
    if (e != cudaSuccess) return e;

    attr_done[c->ordinal & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Smem<MT>::bytes(p.splits);
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
  return cudaLaunchKernelEx(&cfg, gemv_tc_int4_kernel<MT, AHEAD>, p);
}

}  // namespace gemv_tc

bool ruai_gemv_tc_eligible(const ruai_qweight* w, uint32_t m) {
  return w->layout == QL_CHUNK16 && w->bits == 4 && w->n % 4 == 0 && m >= 1 && m <= 16;
}

int ruai_gemv_tc_launch(ruai_ctx* c, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                        const GemvEpilogue& epi_in, const GemvPrologue& pro) {
  using namespace gemv_tc;
  GemvEpilogue epi = epi_in;
  if (epi.act == ACT_SWIGLU && (w->n & 1)) return ruai_fail(c, RUAI_ERR_SHAPE, "SwiGLU epilogue needs an even column count, got %u", w->n);
  if (epi.out_ld == 0) epi.out_ld = epi.act == ACT_SWIGLU ? w->n / 2 : w->n;
  if (epi.sumsq && epi.act == ACT_SWIGLU) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "sum of squares with the SwiGLU epilogue");
  if (epi.argmax_out && epi.act == ACT_SWIGLU) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "argmax with the SwiGLU epilogue");
  // up to 8 rows per CTA; 9..16 rows run as two row tiles (the second pass over the weights mostly hits the L2)
  const int mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : 8;
  const uint32_t row_tiles = (m + mt - 1) / mt;
  if (epi.argmax_out && row_tiles != 1) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "fused argmax needs a single row tile");
  const uint32_t col_tiles = (w->n + kCols - 1) / kCols;
  // Split k over a cluster of up to 8 CTAs.  A launch is a link in a chain of
  // dependent kernels, so what counts is its latency: waves x (fixed cost + stages per CTA x time per stage).
  const uint32_t slots = 4u * (uint32_t)c->sm_count;
  uint32_t splits = 1;
  double best = 1e30;
  for (uint32_t s2 = 1; s2 <= 8; s2 *= 2) {  // 16-CTA clusters were tried: fewer clusters fit at once and the launch got slower
    const uint32_t per = (w->chunks + s2 - 1) / s2;
    if (s2 > 1 && per < (uint32_t)kStageGroups) break;
    const uint32_t stages = (per + kStageGroups - 1) / kStageGroups;
    const uint32_t waves = (col_tiles * row_tiles * s2 + slots - 1) / slots;
    const double t = waves * (4.7 + 1.5 * stages + 0.15 * s2);
    if (t < best) { best = t; splits = s2; }
  }
  uint32_t cpc = (w->chunks + splits - 1) / splits;
  cpc = (cpc + kStageGroups - 1) / kStageGroups * kStageGroups;
  Params p;
  p.w = (const uint4*)w->data; p.scale = w->scale; p.x = x; p.x_dtype = x_dtype; p.x_ld = x_ld;
  p.m = m; p.k = w->k; p.n = w->n; p.chunks = w->chunks; p.chunks_per_cta = cpc; p.splits = splits;
  p.out = out; p.status = c->status; p.epi = epi; p.pro = pro;
  p.pro.trace = ruai_trace_slot(c);
  p.prof = (long long*)c->prof;
  const dim3 grid(col_tiles, splits, row_tiles);
  // few CTAs per SM: spend the free registers on a deeper weight queue
  const bool deep = col_tiles * row_tiles * splits <= 2u * (uint32_t)c->sm_count;
  cudaError_t e = mt == 1 ? (deep ? launch_one<1, 4>(c, p, grid) : launch_one<1, 2>(c, p, grid))
                : mt == 2 ? (deep ? launch_one<2, 4>(c, p, grid) : launch_one<2, 2>(c, p, grid))
                : mt == 4 ? launch_one<4, 2>(c, p, grid)
                          : launch_one<8, 2>(c, p, grid);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "tensor-core gemv launch failed: %s", cudaGetErrorString(e));
  return RUAI_OK;
}
