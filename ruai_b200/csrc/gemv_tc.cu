// Fused dequantize + GEMV on the tensor cores (tcgen05, accumulators in tensor memory) for
// int4 group-32 weights and up to sixteen rows of activations (eight per CTA): the decode hot path.
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
// Organisation of a CTA (128 columns of W, a slice of k): three kinds of warps that only meet at mbarriers,
// so that the latency of one kind's work hides behind the others'.
//   * four expanding warps (thread = column): the packed weights of their column come straight from global memory
//     into registers, some stages ahead of their use and requested before the grid-dependency wait (weights do not
//     depend on the predecessor); nibbles -> bytes into one of kBufs A operand buffers in shared memory;
//   * one warp whose first lane issues the MMAs of a stage (one per scale group) and commits them;
//   * four draining warps (thread = column): digits of the activations a round (16 groups) ahead, and per stage
//     the sums out of tensor memory, scaled and accumulated in f32; they run the epilogue.
// Split-K over a cluster with the partial sums sent through distributed shared memory; bounded waits everywhere.
#include "common.cuh"
#include "gemv_epilogue.cuh"
#include "pipeline.cuh"

namespace gemv_tc {

using namespace pipe;

constexpr int kCols = kGemvBulkTileCols;  // 128 = MMA M = TMEM lanes
constexpr int kStageGroups = 4;           // scale groups (chunks) per stage
constexpr int kRoundGroups = 16;          // groups per conversion round of the activations
constexpr int kRoundStages = kRoundGroups / kStageGroups;
constexpr int kLimbs = 3;
constexpr int kThreads = 2 * kCols + 32;  // draining warps 0-3, issuing warp 4, expanding warps 5-8
constexpr int kExpand0 = kCols + 32;      // first expanding thread
// MMA N (rows x limbs, padded to a multiple of 16), stage buffers (A operand + accumulators), TMEM columns
constexpr int n_of(int mt) { return mt <= 4 ? 16 : 32; }
// The variant with a 2-stage register queue and up to two rows is the small one: two stage buffers, 128 TMEM columns,
// about 52 KB of shared memory and 72 registers, so that three CTAs fit an SM; it serves launches of few stages per CTA.
constexpr bool small_of(int mt, int ahead) { return mt <= 2 && ahead == 2; }
constexpr int bufs_of(int mt, int ahead) { return mt <= 4 && !small_of(mt, ahead) ? 4 : 2; }
// The standard variant for up to four rows keeps its A operand in TENSOR memory: an expanding thread's 32 bytes of a
// group (its column's 32 rows of W) are exactly the 8 words of its lane there (lane = row of A, column c, byte b =
// A[row][4 c + b]), so one tcgen05.st replaces the two 16-byte shared-memory stores, the proxy fence, and the tensor
// core's own read of 16 KB of shared memory per stage.  Tensor memory per CTA stays 256 columns (two CTAs per SM): four
// A buffers (4 x 4 groups x 8 columns) and two accumulator buffers (2 x 4 groups x 16 columns).
constexpr bool a_in_tmem(int mt, int ahead) { return mt <= 4 && !small_of(mt, ahead); }
constexpr int acc_bufs_of(int mt, int ahead) { return a_in_tmem(mt, ahead) ? 2 : bufs_of(mt, ahead); }
constexpr int tmem_cols_of(int mt, int ahead) {  // 256 or 128
  return a_in_tmem(mt, ahead) ? acc_bufs_of(mt, ahead) * kStageGroups * n_of(mt) + bufs_of(mt, ahead) * kStageGroups * 8
                              : bufs_of(mt, ahead) * kStageGroups * n_of(mt);
}

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

template <int MT, int AHEAD>
struct Smem {
  static constexpr int kN = n_of(MT);
  static constexpr int kBufs = bufs_of(MT, AHEAD);
  static constexpr size_t off_a = 0;
  static constexpr size_t off_b = off_a + (a_in_tmem(MT, AHEAD) ? 0 : (size_t)kBufs * kStageGroups * kCols * 32);  // no A buffers in shared memory where A is in tensor memory
  static constexpr size_t off_meta = off_b + 2 * (size_t)kRoundGroups * kN * 32;
  static constexpr size_t off_red = off_meta + 2 * (size_t)kRoundGroups * MT * 8;
  static size_t bytes(uint32_t splits) { return off_red + (size_t)splits * MT * kCols * 4 + 128; }
};

// Activations of one round for layouts the 16-byte path cannot take (any dtype, any alignment): one value at a time.
// For one or two rows it is inlined and unrolled, so that the row array stays in registers (handing it to a function by
// address puts it, and the fast path's copy with it, into per-thread local memory); for more rows the function call
// keeps the kernel small and the array is in local memory either way.
template <int MT>
static __device__ __forceinline__ void fetch_round_scalar_body(float4* dst, const void* x, int x_dtype, uint32_t x_ld, uint32_t m0, uint32_t rows,
                                                               uint32_t kidx, uint32_t k, bool in, const float* norm_w) {
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (in && r < (int)rows) {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        if (kidx + t < k) {
          v[t] = load_as_f32(x, x_dtype, (size_t)(m0 + r) * x_ld + kidx + t);
          if (norm_w) v[t] = v[t] * norm_w[kidx + t];
        }
      }
    }
    dst[r] = make_float4(v[0], v[1], v[2], v[3]);
  }
}
template <int MT>
static __device__ __noinline__ void fetch_round_scalar_call(float4* dst, const void* x, int x_dtype, uint32_t x_ld, uint32_t m0, uint32_t rows,
                                                            uint32_t kidx, uint32_t k, bool in, const float* norm_w) {
  fetch_round_scalar_body<MT>(dst, x, x_dtype, x_ld, m0, rows, kidx, k, in, norm_w);
}
template <int MT>
static __device__ __forceinline__ void fetch_round_scalar(float4 (&dst)[MT], const void* x, int x_dtype, uint32_t x_ld, uint32_t m0, uint32_t rows,
                                                          uint32_t kidx, uint32_t k, bool in, const float* norm_w) {
  if constexpr (MT <= 2) fetch_round_scalar_body<MT>(dst, x, x_dtype, x_ld, m0, rows, kidx, k, in, norm_w);
  else fetch_round_scalar_call<MT>(dst, x, x_dtype, x_ld, m0, rows, kidx, k, in, norm_w);
}

// kAhead: stages of packed weights an expanding thread holds in registers ahead of their use.
template <int MT, int kAhead>
__global__ void __launch_bounds__(kThreads, small_of(MT, kAhead) ? 3 : 2) gemv_tc_int4_kernel(const Params p) {
  constexpr int kN = n_of(MT);
  constexpr int kBufs = bufs_of(MT, kAhead);
  constexpr int kTmemCols = tmem_cols_of(MT, kAhead);
  constexpr bool kATmem = a_in_tmem(MT, kAhead);
  constexpr int kAccBufs = acc_bufs_of(MT, kAhead);
  constexpr uint32_t kATmemCol0 = kAccBufs * kStageGroups * kN;  // first column of the A buffers (kATmem)
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols >= 32, "tensor memory is allotted in powers of two");
  static_assert(kRoundStages % kAccBufs == 0, "accumulator buffers must divide a round");
  static_assert(MT * kLimbs <= kN, "rows x limbs must fit the MMA N");
  static_assert((kBufs & (kBufs - 1)) == 0 && kRoundStages % kBufs == 0, "stage buffers must divide a round");
  using L = Smem<MT, kAhead>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t a_ready[kBufs];   // A operand of a stage written (4 expanding warps)
  __shared__ __align__(8) uint64_t mma_done[kBufs];  // MMAs of a stage completed: sums valid, A buffer free
  __shared__ __align__(8) uint64_t acc_free[kBufs];  // sums of a stage read out of tensor memory (4 draining warps)
  __shared__ __align__(8) uint64_t b_ready[2];       // digits of a round written (4 draining warps)
  __shared__ uint32_t s_tmem;
  __shared__ float s_rstd[MT];
  __shared__ float s_red[kThreads / 32];
  __shared__ int2 s_arg[kThreads / 32];
  __shared__ unsigned s_flag;
  __shared__ volatile int s_abort;
  unsigned char* abuf = smem + L::off_a;
  unsigned char* bop = smem + L::off_b;
  float* meta_scale = reinterpret_cast<float*>(smem + L::off_meta);  // [2][kRoundGroups][MT]
  int* meta_sum = reinterpret_cast<int*>(smem + L::off_meta) + 2 * kRoundGroups * MT;
  float* red = reinterpret_cast<float*>(smem + L::off_red);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t j0 = blockIdx.x * kCols;
  const uint32_t j = j0 + tid;
  const bool active = tid < kCols && j < p.n;
  const uint32_t split = p.splits > 1 ? cluster_ctarank() : 0u;
  const uint32_t m0 = blockIdx.z * MT;
  const uint32_t rows = min((uint32_t)MT, p.m - m0);
  const uint32_t c_begin = min(p.chunks, split * p.chunks_per_cta);
  const uint32_t c_end = min(p.chunks, c_begin + p.chunks_per_cta);
  const uint32_t nst = (c_end - c_begin + kStageGroups - 1) / kStageGroups;
  const uint32_t nrounds = (nst + kRoundStages - 1) / kRoundStages;

  // The expanding warps' first stages of packed weights are requested before anything else: they depend on nothing,
  // not on the predecessor kernel and not on this CTA's own set-up (barriers, tensor memory, the zeroed operand rows).
  const bool expander = warp > kCols / 32;
  // (A in tensor memory: a warp reaches only the lanes 32 (warp % 4) .., so its threads take those columns)
  const int te = kATmem ? (warp & 3) * 32 + lane : tid - kExpand0;
  const uint32_t je = j0 + te;
  const bool in_col = je < p.n;
  uint4 wq[kAhead][kStageGroups];
  auto load_stage = [&](uint32_t i, uint4 (&wv)[kStageGroups]) {
#pragma unroll
    for (int u = 0; u < kStageGroups; ++u) {
      const uint32_t c = c_begin + i * kStageGroups + u;
      // beyond the slice or the matrix: stored value 8 is weight 0
      wv[u] = (in_col && c < c_end) ? ldg_stream_u4(&p.w[(size_t)c * p.n + je]) : make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
    }
  };
  if (expander) {
#pragma unroll
    for (int a = 0; a < kAhead; ++a) load_stage(a, wq[a]);
  }

  if (tid == 0) {
    for (int s = 0; s < kBufs; ++s) { mbar_init(&a_ready[s], kCols / 32); mbar_init(&mma_done[s], 1); mbar_init(&acc_free[s], kCols / 32); }
    mbar_init(&b_ready[0], kCols / 32);
    mbar_init(&b_ready[1], kCols / 32);
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
  const bool normed = p.pro.norm_w != nullptr;
  float acc[MT];
  float resid_pre[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) { acc[r] = 0.0f; resid_pre[r] = 0.0f; }
  const bool pre = p.epi.resid != nullptr && p.epi.act != ACT_SWIGLU && split == 0 && active;

  if (expander) {
    // ===== expanding warps: packed weights -> A operand.  Nothing here depends on the predecessor kernel, so
    // these warps do not wait for it: the first kBufs stages are in place before the activations exist. =====
    bool ok = true;
    // the register queue is addressed statically (stage i sits in wq[i % kAhead]): moving it along would make every
    // stage wait for the newest loads
    for (uint32_t i0 = 0; i0 < nst && ok; i0 += kAhead) {
#pragma unroll
      for (int a = 0; a < kAhead; ++a) {
        const uint32_t i = i0 + a;
        if (i >= nst) break;
        const uint32_t b = i & (kBufs - 1), q = i / kBufs;
        if (q > 0 && (s_abort || !mbar_wait(&mma_done[b], (q - 1) & 1u))) { ok = false; break; }  // the MMAs that read this buffer last are done
        // nibbles -> bytes: 32 rows of this thread's column become one row of two 16-byte k-halves of A
#pragma unroll
        for (int u = 0; u < kStageGroups; ++u) {
          const uint4 wv = wq[a][u];
          uint4 lo, hi;
          lo.x = wv.x & 0x0F0F0F0Fu; hi.x = (wv.x >> 4) & 0x0F0F0F0Fu;
          lo.y = wv.y & 0x0F0F0F0Fu; hi.y = (wv.y >> 4) & 0x0F0F0F0Fu;
          lo.z = wv.z & 0x0F0F0F0Fu; hi.z = (wv.z >> 4) & 0x0F0F0F0Fu;
          lo.w = wv.w & 0x0F0F0F0Fu; hi.w = (wv.w >> 4) & 0x0F0F0F0Fu;
          if constexpr (kATmem) {
            const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + kATmemCol0 + (b * kStageGroups + u) * 8u;
            asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(lo.x), "r"(lo.y), "r"(lo.z),
                         "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                         : "memory");
          } else {
            unsigned char* dst = abuf + ((size_t)b * kStageGroups + u) * (kCols * 32) + (size_t)te * 16;
            *reinterpret_cast<uint4*>(dst) = lo;
            *reinterpret_cast<uint4*>(dst + kCols * 16) = hi;
          }
        }
        load_stage(i + kAhead, wq[a]);  // the stage kAhead further on, into the registers just consumed
        if constexpr (kATmem) {
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          tc_fence_before_sync();
        } else {
          fence_proxy_async_smem();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_ready[b]);
      }
    }
    if (!ok) s_abort = 1;
  } else if (warp == kCols / 32) {
    // ===== issuing warp =====
    if (tid == kCols) trace_min(p.pro.trace, 0);
    grid_dependency_wait();
    if (tid == kCols) trace_min(p.pro.trace, 1);
    grid_launch_dependents();
    // RMSNorm: x * rstd * w with rstd a per-row scalar, so the digits are taken from x * w and rstd multiplies
    // the finished sums
    if (normed && lane < MT) {
      float ss = 0.0f;
      if (lane < (int)rows)
        for (uint32_t t = 0; t < p.pro.tiles; ++t) ss += p.pro.sumsq[(size_t)t * p.m + m0 + lane];
      s_rstd[lane] = 1.0f / sqrtf(ss * (1.0f / (float)p.k) + p.pro.eps);
    }
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_i8(kN, false);
      // descriptors of the first operand slots; the loop only adds to their address fields
      const uint64_t ad0 = umma_desc_kmajor(smem_u32(abuf), kCols * 16, 128);
      const uint64_t bd0 = umma_desc_kmajor(smem_u32(bop), kN / 8 * 128, 128);
      uint32_t left = c_end - c_begin;
      for (uint32_t i = 0; i < nst; ++i, left -= kStageGroups) {
        const uint32_t b = i & (kBufs - 1), q = i / kBufs;
        bool ok = !s_abort;
        if (ok && (i % kRoundStages) == 0) ok = mbar_wait(&b_ready[(i / kRoundStages) & 1u], (i / (2 * kRoundStages)) & 1u);  // digits of the round
        const uint32_t ab = i & (kAccBufs - 1), aq = i / kAccBufs;  // accumulator buffer of this stage
        if (ok && aq > 0) ok = mbar_wait(&acc_free[ab], (aq - 1) & 1u);  // the sums these MMAs overwrite have been read
        if (ok) ok = mbar_wait(&a_ready[b], q & 1u);
        if (!ok) { s_abort = 1; break; }
        tc_fence_after_sync();
        const uint32_t slot = b * kStageGroups;                            // A and accumulator slots of this stage
        const uint32_t gb = (i & (2 * kRoundStages - 1)) * kStageGroups;   // first group in the two rounds of digits
        const uint64_t ad = umma_desc_advance(ad0, slot * (kCols * 32));
        const uint64_t bd = umma_desc_advance(bd0, gb * (kN * 32));
        const uint32_t d = tmem_base + ab * kStageGroups * kN;
        const uint32_t at = tmem_base + kATmemCol0 + slot * 8u;  // kATmem: the stage's A buffer in tensor memory
        auto mma = [&](uint32_t u) {
          if constexpr (kATmem) umma_i8_ts(d + u * kN, at + u * 8u, umma_desc_advance(bd, u * (kN * 32)), idesc, 0u);
          else umma_i8(d + u * kN, umma_desc_advance(ad, u * (kCols * 32)), umma_desc_advance(bd, u * (kN * 32)), idesc, 0u);
        };
        if (left >= (uint32_t)kStageGroups) {
#pragma unroll
          for (uint32_t u = 0; u < (uint32_t)kStageGroups; ++u) mma(u);
        } else {
          for (uint32_t u = 0; u < left; ++u) mma(u);
        }
        umma_commit(&mma_done[b]);
      }
    }
  } else {
    // ===== draining warps: digits of the activations, scaled sums out of tensor memory =====
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    // scales of this thread's column one round ahead of their use; they do not depend on the predecessor
    float sq[kRoundStages][kStageGroups];
    auto load_scales = [&](uint32_t i, float (&sv)[kStageGroups]) {
#pragma unroll
      for (int u = 0; u < kStageGroups; ++u) {
        const uint32_t c = c_begin + i * kStageGroups + u;
        sv[u] = (active && c < c_end) ? ldg_stream_f32(&p.scale[(size_t)c * p.n + j]) : 0.0f;
      }
    };
#pragma unroll
    for (int a = 0; a < kRoundStages; ++a) load_scales(a, sq[a]);
    grid_dependency_wait();
#pragma unroll
    for (int r = 0; r < MT; ++r) resid_pre[r] = (pre && r < (int)rows) ? p.epi.resid[(size_t)(m0 + r) * p.epi.out_ld + j] : 0.0f;
    // activations of one round (16 groups = 512 values per row): 4 consecutive values per thread
    // 16-byte loads when the layout allows; the RMSNorm weights of the same columns ride along and multiply at conversion
    const bool vec = p.x_dtype == RUAI_F32 && (p.x_ld & 3u) == 0 && (p.k & 3u) == 0 && (reinterpret_cast<uintptr_t>(p.x) & 15u) == 0 &&
                     (!normed || (reinterpret_cast<uintptr_t>(p.pro.norm_w) & 15u) == 0);
    auto fetch_round = [&](uint32_t round, float4 (&dst)[MT], float4& nw) {
      const uint32_t g = c_begin + round * kRoundGroups + tid / 8;
      const uint32_t kidx = (c_begin + round * kRoundGroups) * 32 + 4 * tid;
      const bool in = round < nrounds && g < c_end;
      nw = make_float4(1.f, 1.f, 1.f, 1.f);
      if (vec) {
        const bool ld = in && kidx < p.k;
        if (ld && normed) nw = ldg_f4(reinterpret_cast<const float4*>(p.pro.norm_w + kidx));
#pragma unroll
        for (int r = 0; r < MT; ++r)
          dst[r] = (ld && r < (int)rows) ? ldg_f4(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + (size_t)(m0 + r) * p.x_ld + kidx))
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
        return;
      }
      fetch_round_scalar<MT>(dst, p.x, p.x_dtype, p.x_ld, m0, rows, kidx, p.k, in, normed ? p.pro.norm_w : nullptr);
    };
    // this warp's 4 groups of a round (8 lanes per group): block fixed point, three int8 digits into the B operand
    auto convert = [&](uint32_t round, const float4 (&src)[MT], const float4& nw) {
      const uint32_t rb = round & 1u;
      const uint32_t gi = warp * 4 + (lane >> 3);
#pragma unroll
      for (int r = 0; r < MT; ++r) {
        const float4 xv = make_float4(src[r].x * nw.x, src[r].y * nw.y, src[r].z * nw.z, src[r].w * nw.w);
        float gmax = fmaxf(fmaxf(fabsf(xv.x), fabsf(xv.y)), fmaxf(fabsf(xv.z), fabsf(xv.w)));
        gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 1));
        gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 2));
        gmax = fmaxf(gmax, __shfl_xor_sync(0xFFFFFFFFu, gmax, 4));
        // gmax < 2^e with e = biased exponent - 126; f = round(v * 2^(20-e)), x = f * 2^(e-20)
        const uint32_t eb = __float_as_uint(gmax) >> 23;
        // a NaN or an infinity anywhere in the group (fmaxf drops NaN, so it is looked for on its own): the group's
        // scale becomes NaN and with it this row's sums, as in f32 arithmetic (cpu.rs:1035-1067 propagates them)
        bool bad = !(fabsf(xv.x) <= 3.402823466e38f && fabsf(xv.y) <= 3.402823466e38f && fabsf(xv.z) <= 3.402823466e38f && fabsf(xv.w) <= 3.402823466e38f);
        bad = ((__ballot_sync(0xFFFFFFFFu, bad) >> (lane & 24)) & 0xFFu) != 0u;
        const bool nz = eb >= 20u && eb < 255u && !bad;
        const float up = nz ? __uint_as_float((273u - eb) << 23) : 0.0f;
        const float xscale = bad ? __int_as_float(0x7fc00000) : (nz ? __uint_as_float((eb - 19u) << 23) : 0.0f);
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
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&b_ready[rb]);
    };
    float4 xa[MT], xb[MT], na, nb;
    fetch_round(0, xa, na);
    fetch_round(1, xb, nb);
    convert(0, xa, na);
    if (nrounds > 1) convert(1, xb, nb);
    fetch_round(2, xa, na);
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the rounds' scales and sums are visible to the four warps

    bool ok = true;
    // a warp whose wait ran out still walks the rounds, so that the four warps meet at every barrier below
    for (uint32_t round = 0; round < nrounds; ++round) {
      const uint32_t rb = round & 1u;
#pragma unroll
      for (int a = 0; a < kRoundStages; ++a) {
        const uint32_t i = round * kRoundStages + a;
        if (i >= nst || !ok) break;
        const uint32_t b = a & (kBufs - 1), q = i / kBufs;
        if (s_abort || !mbar_wait(&mma_done[b], q & 1u)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t nch = min((uint32_t)kStageGroups, c_end - (c_begin + i * kStageGroups));
        constexpr int kQ = (MT * kLimbs + 3) / 4;            // 4-column loads per group
        constexpr int kBatch = MT <= 2 ? kStageGroups : 1;  // groups whose sums are in registers at once
#pragma unroll
        for (int u0 = 0; u0 < kStageGroups; u0 += kBatch) {
          int32_t d[kBatch][kQ * 4];
#pragma unroll
          for (int ub = 0; ub < kBatch; ++ub) {
            const uint32_t col = tmem_base + lane_base + ((a & (kAccBufs - 1)) * kStageGroups + u0 + ub) * kN;
#pragma unroll
            for (int q4 = 0; q4 < kQ; ++q4) {
              int32_t t4[4];
              tmem_ld4(col + 4 * q4, t4);  // groups past the end hold stale sums; they are not used below
              d[ub][4 * q4 + 0] = t4[0]; d[ub][4 * q4 + 1] = t4[1]; d[ub][4 * q4 + 2] = t4[2]; d[ub][4 * q4 + 3] = t4[3];
            }
          }
          tmem_ld_wait();
          if (u0 + kBatch >= kStageGroups) {  // the last sums of the stage are out: the next MMAs into this buffer may go
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_free[a & (kAccBufs - 1)]);
          }
#pragma unroll
          for (int ub = 0; ub < kBatch; ++ub) {
            const int u = u0 + ub;
            if ((uint32_t)u < nch) {
#pragma unroll
              for (int r = 0; r < MT; ++r) {
                const uint32_t mi = (rb * kRoundGroups + a * kStageGroups + u) * MT + r;
                const int val = d[ub][kLimbs * r] * 16384 + d[ub][kLimbs * r + 1] * 128 + d[ub][kLimbs * r + 2] - 8 * meta_sum[mi];
                acc[r] = fmaf((float)val, sq[a][u] * meta_scale[mi], acc[r]);
              }
            }
          }
        }
        load_scales(i + kRoundStages, sq[a]);
      }
      if (round + 2 < nrounds) {
        // every MMA of this round is complete and (after the barrier) every warp has used its scales and sums:
        // the round after next takes its place
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ok) {
          convert(round + 2, xa, na);
          fetch_round(round + 3, xa, na);
        }
      }
    }
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
}

template <int MT, int AHEAD>
cudaError_t launch_one(ruai_ctx* c, const Params& p, dim3 grid) {
  static bool attr_done[64] = {};
  if (!attr_done[c->ordinal & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_tc_int4_kernel<MT, AHEAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<MT, AHEAD>::bytes(8));
    if (e != cudaSuccess) return e;

    attr_done[c->ordinal & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Smem<MT, AHEAD>::bytes(p.splits);
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
  // Split k over a cluster of up to 8 CTAs.  A launch is a link in a chain of dependent kernels, so what counts is its
  // latency.  Measured on the 8B shapes, in microseconds: about 5.5 per wave of CTAs that is fixed, 0.45 per stage
  // (more with more rows) and 0.15 per CTA of the cluster for the reduction.
  const double per_stage = 0.45 * (mt == 1 ? 1.0 : mt == 2 ? 1.4 : mt == 4 ? 2.0 : 3.2);
  uint32_t splits = 1;
  bool small = false;  // the three-CTAs-per-SM variant
  double best = 1e30;
  for (int variant = 0; variant < (mt <= 2 ? 2 : 1); ++variant) {
    const uint32_t slots = (variant ? 3u : 2u) * (uint32_t)c->sm_count;
    for (uint32_t s2 = 1; s2 <= 8; s2 *= 2) {  // 16-CTA clusters were tried: fewer clusters fit at once and the launch got slower
      const uint32_t per = (w->chunks + s2 - 1) / s2;
      if (s2 > 1 && per < (uint32_t)kStageGroups) break;
      const uint32_t stages = (per + kStageGroups - 1) / kStageGroups;
      if (variant && stages > 8) continue;  // the small variant's short queues are for short slices
      const uint32_t ctas = col_tiles * row_tiles * s2;
      const uint32_t waves = (ctas + slots - 1) / slots;
      // clusters of 8 that nearly fill the machine do not always find their places at once (measured on o_proj: 256 CTAs,
      // 5.7 or 9.8 us from launch to launch; as 128 CTAs in clusters of 4 always 6.5)
      const double crowd = (s2 == 8 && (variant ? 10u * ctas > 9u * slots : 4u * ctas > 3u * slots)) ? 2.0 : 0.0;
      const double t = waves * (5.5 + per_stage * stages) + 0.15 * s2 + crowd + (variant ? 0.2 : 0.0);
      if (t < best) { best = t; splits = s2; small = variant != 0; }
    }
  }
  uint32_t cpc = (w->chunks + splits - 1) / splits;
  cpc = (cpc + kStageGroups - 1) / kStageGroups * kStageGroups;
  Params p;
  p.w = (const uint4*)w->data; p.scale = w->scale; p.x = x; p.x_dtype = x_dtype; p.x_ld = x_ld;
  p.m = m; p.k = w->k; p.n = w->n; p.chunks = w->chunks; p.chunks_per_cta = cpc; p.splits = splits;
  p.out = out; p.status = c->status; p.epi = epi; p.pro = pro;
  p.pro.trace = ruai_trace_slot(c);
  if ((c->force_splits & 255u) && (c->force_splits & 255u) <= 8) {
    p.splits = splits = c->force_splits & 255u;
    cpc = (w->chunks + splits - 1) / splits;
    p.chunks_per_cta = cpc = (cpc + kStageGroups - 1) / kStageGroups * kStageGroups;
  }
  const dim3 grid(col_tiles, splits, row_tiles);
  // few CTAs per SM: spend the free registers on a deeper weight queue
  const bool deep = !(c->force_splits & 256u);
  cudaError_t e = mt == 1 ? (deep && !small ? launch_one<1, 4>(c, p, grid) : launch_one<1, 2>(c, p, grid))
                : mt == 2 ? (deep && !small ? launch_one<2, 4>(c, p, grid) : launch_one<2, 2>(c, p, grid))
                : mt == 4 ? launch_one<4, 2>(c, p, grid)
                          : launch_one<8, 2>(c, p, grid);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "tensor-core gemv launch failed: %s", cudaGetErrorString(e));
  return RUAI_OK;
}
