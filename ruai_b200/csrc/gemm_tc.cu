// Prefill / large-batch quantized GEMM on the tensor cores: out[m,n] = x[m,k] @ dequant(W)[k,n], m > 16.
//
// Replaces the reference's "dequantize the whole weight to f32, cast, cuBLAS" route for m > 16
// (src/nn/backend/cuda.rs:812-826) with one kernel that keeps the weight packed in HBM:
//   - the packed tile (128 columns of W, the chunk layout of pack.cu) is fetched into registers a
//     stage ahead, expanded to bf16 in shared memory (int4 and int8 values are exact in bf16),
//   - the activations are split once, by a small pre-kernel, into two bf16 pieces x = hi + lo
//     (16 significant bits) stored in the tensor core's B-operand layout; a warp streams them
//     into a shared-memory ring with bulk asynchronous copies,
//   - `tcgen05.mma kind::f16` accumulates hi and lo into the same f32 accumulator in tensor
//     memory: D[128 columns of W][128 rows of x].
// int4: one accumulator per scale group of 32 rows of W; the epilogue warps read it back and add
// scale[g, j] * D into registers, which is exactly the reference's per-group sum
// (cpu.rs:1045-1063).  int8: one accumulator over all of k, scaled per column at the end
// (cpu.rs:903-920).  RMSNorm, when folded in, contributes x * w here and its per-row factor at the end.
// Every mbarrier wait is bounded.
#include "common.cuh"
#include "gemv_epilogue.cuh"
#include "pipeline.cuh"

namespace gemm_tc {

using namespace pipe;

constexpr int kCols = 128;        // columns of W per CTA = MMA M = TMEM lanes
constexpr int kRows = 128;        // rows of x per CTA = MMA N
constexpr int kStageGroups = 2;   // groups of 32 k per pipeline stage
constexpr int kBStages = 3;       // ring of B stages in shared memory (five change nothing: measured)
constexpr int kParts = 4;             // worker threads per column
constexpr int kWorkers = kParts * kCols;  // sixteen warps: thread = (column, part); a part expands one k-step of one of a stage's two groups
                                          // (16 of the group's 32 rows of W) and reads a quarter of the rows of x out of tensor memory
constexpr int kIssuers = kStageGroups;  // issuing warps, one per group of a stage: a tcgen05.mma costs its issuing thread about 116 clocks (measured,
                                        // kind::f16 up to N = 128) against the 64 the tensor core needs for 128 x 128 x 16, so one thread cannot keep it busy
constexpr int kThreads = kWorkers + 32 + 32 * kIssuers;  // workers, the B producer's warp, the issuing warps
constexpr uint32_t kBGroupBytes = 2 * 2 * kRows * 32;  // pieces x k-steps x rows x 32 B = 16 KB per group of 32 k

// ---- activations -> two bf16 pieces in B-operand layout --------------------------------------------
// xs[row_block][group][piece][kstep][kchunk][row/8][row%8][8 bf16]; one CTA per (group, row block), one thread per row.
__global__ void __launch_bounds__(kRows) xsplit_kernel(const void* __restrict__ x, int x_dtype, uint32_t x_ld, uint32_t m, uint32_t k,
                                                       const float* __restrict__ norm_w, uint32_t groups, unsigned char* __restrict__ xs) {
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t g = blockIdx.x, rb = blockIdx.y, r = threadIdx.x, row = rb * kRows + r;
  unsigned char* dst = xs + ((size_t)rb * groups + g) * kBGroupBytes + (r >> 3) * 128 + (r & 7) * 16;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float v[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint32_t kidx = g * 32 + s * 16 + c * 8 + 2 * t + q;
          v[q] = 0.0f;
          if (row < m && kidx < k) {
            v[q] = load_as_f32(x, x_dtype, (size_t)row * x_ld + kidx);
            if (norm_w) v[q] *= norm_w[kidx];
          }
        }
        const __nv_bfloat16 h0 = __float2bfloat16_rn(v[0]), h1 = __float2bfloat16_rn(v[1]);
        const __nv_bfloat16 l0 = __float2bfloat16_rn(v[0] - __bfloat162float(h0)), l1 = __float2bfloat16_rn(v[1] - __bfloat162float(h1));
        hi[t] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
        lo[t] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
      }
      *reinterpret_cast<uint4*>(dst + 0 * 8192 + s * 4096 + c * 2048) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(dst + 1 * 8192 + s * 4096 + c * 2048) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
  }
}

struct Params {
  const uint4* w;
  const float* scale;
  const unsigned char* xs;  // split activations
  uint32_t m, k, n, chunks, groups;  // groups of 32 k (int8: two chunks each)
  void* out;
  int* status;
  GemvEpilogue epi;
  const float* rstd_sumsq;  // RMSNorm folded in: per-tile sums of squares [tiles][m] (NULL: none)
  uint32_t rstd_tiles;
  float eps;
};

// Instruction descriptor of kind::f16 with bf16 operands, f32 accumulate, both K-major, M = 128.
__host__ __device__ constexpr uint32_t idesc_bf16(uint32_t n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24); }

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(adesc),
               "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
      "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared memory: A (bf16 tile) double buffered, B ring.
constexpr size_t kAGroupBytes = 2 * kCols * 32;  // two k-steps x 128 rows x 32 B = 8 KB
constexpr size_t off_a = 0;
constexpr size_t off_b = off_a + 2 * kStageGroups * kAGroupBytes;
constexpr size_t kSmemBytes = off_b + (size_t)kBStages * kStageGroups * kBGroupBytes + 128;

template <int BITS>
__global__ void __launch_bounds__(kThreads) gemm_tc_kernel(const Params p) {
  constexpr int kTmemCols = BITS == 4 ? 512 : kIssuers * kRows;  // int8: one accumulator per issuing warp
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t b_full[kBStages];  // B stage landed
  __shared__ __align__(8) uint64_t b_empty[kBStages]; // MMAs that read a B slot completed
  __shared__ __align__(8) uint64_t a_ready[2];        // A stage written (4 warp arrivals)
  __shared__ __align__(8) uint64_t mma_done[2];       // MMAs of a stage completed (frees A buffer, B slot; int4: accumulators ready)
  __shared__ uint32_t s_tmem;
  __shared__ volatile int s_abort;
  __shared__ float s_rstd[kRows];
  unsigned char* abuf = smem + off_a;
  unsigned char* bring = smem + off_b;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t col = (uint32_t)tid & (kCols - 1), part = (uint32_t)tid >> 7;  // workers only
  const uint32_t pg = part >> 1, pstep = part & 1u;  // the group of the stage and the k-step of the group this thread expands
  const uint32_t j0 = blockIdx.x * kCols, j = j0 + col, rb = blockIdx.y, row0 = rb * kRows;
  const bool active = tid < kWorkers && j < p.n;
  const uint32_t nst = (p.groups + kStageGroups - 1) / kStageGroups;

  if (tid == 0) {
    for (int s = 0; s < kBStages; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], kIssuers); }
    for (int s = 0; s < 2; ++s) { mbar_init(&a_ready[s], kWorkers / 32); mbar_init(&mma_done[s], kIssuers); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_abort = 0;
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(&s_tmem, kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s_tmem;

  // packed weights of this thread's column, kAhead stages ahead of their use in a register queue addressed statically
  // (they do not depend on the predecessor kernel).  One stage ahead was not enough: a worker is through with a stage long
  // before the next stage's weights have made their way from the L2 or from HBM, and waited for them every time.
  constexpr int kChunksPerGroup = BITS == 4 ? 1 : 2;
  constexpr int kAhead = BITS == 4 ? 2 : 3;
  uint4 wq[kAhead];                    // int4: the chunk of this thread's group; int8: the chunk that is its k-step of the group
  float sq[kAhead][kStageGroups];      // the column's scales of both groups (the read-out needs both)
  auto load_stage = [&](uint32_t i, uint4& wv, float (&sv)[kStageGroups]) {
    const uint32_t g = i * kStageGroups + pg;
    const uint32_t c = BITS == 4 ? g : g * kChunksPerGroup + pstep;
    const bool in = active && c < p.chunks;
    wv = in ? __ldg(&p.w[(size_t)c * p.n + j]) : (BITS == 4 ? make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u) : make_uint4(0, 0, 0, 0));
#pragma unroll
    for (int u = 0; u < kStageGroups; ++u) {
      const uint32_t gu = i * kStageGroups + u;
      sv[u] = (BITS == 4 && active && gu < p.groups) ? __ldg(&p.scale[(size_t)gu * p.n + j]) : 0.0f;
    }
  };
  if (tid < kWorkers) {
#pragma unroll
    for (int a = 0; a < kAhead; ++a) load_stage(a, wq[a], sq[a]);
  }
  grid_dependency_wait();
  grid_launch_dependents();

  constexpr int kHalfRows = kRows / kParts;
  float acc[kHalfRows];  // worker threads: this column's sums for the thread's 32 rows
  if (warp == kWorkers / 32 || warp > kWorkers / 32 + 1) {
    // ===== MMA issuers: warp wi takes group wi of every stage =====
    const uint32_t wi = warp == kWorkers / 32 ? 0u : (uint32_t)warp - kWorkers / 32 - 1;
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(kRows);
      for (uint32_t i = 0; i < nst; ++i) {
        if (s_abort || !mbar_wait(&a_ready[i & 1], (i >> 1) & 1u) || !mbar_wait(&b_full[i % kBStages], (i / kBStages) & 1u)) { s_abort = 1; break; }
        tc_fence_after_sync();
        const uint32_t ng = min((uint32_t)kStageGroups, p.groups - i * kStageGroups);
        if (const uint32_t u = wi; u < ng) {
          // int8: an accumulator per issuing warp (MMAs of two threads are not ordered among themselves)
          const uint32_t d = tmem_base + (BITS == 4 ? ((i & 1) * kStageGroups + u) * kRows : wi * kRows);
          const unsigned char* a = abuf + ((size_t)(i & 1) * kStageGroups + u) * kAGroupBytes;
          const unsigned char* b = bring + ((size_t)(i % kBStages) * kStageGroups + u) * kBGroupBytes;
          for (uint32_t s = 0; s < 2; ++s)
            for (uint32_t pc = 0; pc < 2; ++pc) {
              const uint64_t ad = umma_desc_kmajor(smem_u32(a + s * 4096), 2048, 128);
              const uint64_t bd = umma_desc_kmajor(smem_u32(b + pc * 8192 + s * 4096), 2048, 128);
              const uint32_t accumulate = BITS == 4 ? (s | pc) : ((i | s | pc) != 0u ? 1u : 0u);
              umma_bf16(d, ad, bd, idesc, accumulate);
            }
        }
        umma_commit(&mma_done[i & 1]);
        umma_commit(&b_empty[i % kBStages]);
      }
    }
  } else if (warp == kWorkers / 32 + 1) {
    // ===== B producer: bulk copies of the split activations =====
    if (lane == 0) {
      for (uint32_t i = 0; i < nst; ++i) {
        if (i >= (uint32_t)kBStages) {
          // slot reuse: the MMAs of stage i - kBStages must be done (a barrier per slot, so it cannot be lapped)
          if (s_abort || !mbar_wait(&b_empty[i % kBStages], ((i / kBStages) - 1) & 1u)) { s_abort = 1; break; }
        }
        const uint32_t ng = min((uint32_t)kStageGroups, p.groups - i * kStageGroups);
        mbar_expect_tx(&b_full[i % kBStages], ng * kBGroupBytes);
        for (uint32_t u = 0; u < ng; ++u)
          bulk_load(bring + ((size_t)(i % kBStages) * kStageGroups + u) * kBGroupBytes,
                    p.xs + ((size_t)rb * p.groups + i * kStageGroups + u) * kBGroupBytes, kBGroupBytes, &b_full[i % kBStages]);
      }
    }
  } else {
    // ===== sixteen warps: packed weights -> bf16 A tile; accumulators -> scaled sums =====
#pragma unroll
    for (int r = 0; r < kHalfRows; ++r) acc[r] = 0.0f;
    if (tid < kRows) {  // per-row RMS factor of this CTA's rows (needed only in the epilogue)
      float rs = 1.0f;
      if (p.rstd_sumsq && row0 + tid < p.m) {
        float ss = 0.0f;
        for (uint32_t t = 0; t < p.rstd_tiles; ++t) ss += p.rstd_sumsq[(size_t)t * p.m + row0 + tid];
        rs = 1.0f / sqrtf(ss * (1.0f / (float)p.k) + p.eps);
      }
      s_rstd[tid] = rs;
    }
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    float sv_prev[kStageGroups] = {0.f, 0.f};
    auto drain = [&](uint32_t s, const float (&sv)[kStageGroups]) -> bool {  // int4: stage s's accumulators into acc
      if (!mbar_wait(&mma_done[s & 1], (s >> 1) & 1u)) return false;
      tc_fence_after_sync();
      const uint32_t ng = min((uint32_t)kStageGroups, p.groups - s * kStageGroups);
#pragma unroll
      for (int u = 0; u < kStageGroups; ++u) {
        if ((uint32_t)u < ng) {
#pragma unroll
          for (int q = 0; q < kHalfRows / 32; ++q) {
            float d[32];
            tmem_ld32(tmem_base + lane_base + ((s & 1) * kStageGroups + u) * kRows + part * kHalfRows + 32 * q, d);
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < 32; ++t) acc[32 * q + t] = fmaf(d[t], sv[u], acc[32 * q + t]);
          }
        }
      }
      tc_fence_before_sync();
      return true;
    };
    bool ok = true;
    for (uint32_t i0 = 0; i0 < nst && ok; i0 += kAhead) {
#pragma unroll
     for (int qa = 0; qa < kAhead; ++qa) {
      const uint32_t i = i0 + qa;
      if (i >= nst) break;
      if (s_abort) { ok = false; break; }
      // the A buffer of stage i was last read by the MMAs of stage i - 2
      if (i >= 2 && BITS == 8) { if (!mbar_wait(&mma_done[i & 1], ((i - 2) >> 1) & 1u)) { ok = false; break; } }
      float sv_cur[kStageGroups];
#pragma unroll
      for (int u = 0; u < kStageGroups; ++u) sv_cur[u] = sq[qa][u];
      {
        unsigned char* a = abuf + ((size_t)(i & 1) * kStageGroups + pg) * kAGroupBytes + (size_t)col * 16 + pstep * 4096;
        const uint32_t wd[4] = {wq[qa].x, wq[qa].y, wq[qa].z, wq[qa].w};
        uint32_t o[8];
        if (BITS == 4) {
          // 16 nibbles (value + 8) -> 16 bf16: (128 + u) has the bit pattern 0x4300 | u; subtract 136 in bf16 pairs.
          // The low nibbles of the chunk are rows 0..15 of the group (k-step 0), the high nibbles rows 16..31 (k-step 1).
          const __nv_bfloat162 off = __floats2bfloat162_rn(136.0f, 136.0f);
#pragma unroll
          for (int w4 = 0; w4 < 4; ++w4) {
            const uint32_t nib = (pstep ? (wd[w4] >> 4) : wd[w4]) & 0x0F0F0F0Fu;  // rows 4w..4w+3 of the k-step
            const uint32_t pl[2] = {__byte_perm(nib, 0x43434343u, 0x4140), __byte_perm(nib, 0x43434343u, 0x4342)};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              __nv_bfloat162 a2 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&pl[h]), off);
              o[2 * w4 + h] = *reinterpret_cast<uint32_t*>(&a2);  // rows 4w + 2h, +1
            }
          }
        } else {
          // int8: the chunk is the k-step; 16 bytes -> 16 bf16
#pragma unroll
          for (int w4 = 0; w4 < 4; ++w4) {
            const int b0 = (int)(signed char)(wd[w4] & 0xFF), b1 = (int)(signed char)((wd[w4] >> 8) & 0xFF);
            const int b2 = (int)(signed char)((wd[w4] >> 16) & 0xFF), b3 = (int)(signed char)(wd[w4] >> 24);
            __nv_bfloat162 p0 = __floats2bfloat162_rn((float)b0, (float)b1), p1 = __floats2bfloat162_rn((float)b2, (float)b3);
            o[2 * w4] = *reinterpret_cast<uint32_t*>(&p0);
            o[2 * w4 + 1] = *reinterpret_cast<uint32_t*>(&p1);
          }
        }
        // k-chunk c of the k-step holds its rows 8c .. 8c+7 = o[4c .. 4c+3]
        *reinterpret_cast<uint4*>(a) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(a + 2048) = make_uint4(o[4], o[5], o[6], o[7]);
      }
      load_stage(i + kAhead, wq[qa], sq[qa]);  // into the registers just consumed
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_ready[i & 1]);
      if (BITS == 4 && i > 0) ok = drain(i - 1, sv_prev);
#pragma unroll
      for (int u = 0; u < kStageGroups; ++u) sv_prev[u] = sv_cur[u];
      if (!ok) break;
     }
    }
    if (ok && nst > 0) {
      if (BITS == 4) ok = drain(nst - 1, sv_prev);
      else {
        // int8: the issuing warps' accumulators (warp u had groups if there are more than u of them), scaled per column (cpu.rs:918-920)
        const uint32_t s = nst - 1;
        if (!mbar_wait(&mma_done[s & 1], (s >> 1) & 1u)) ok = false;
        else {
          tc_fence_after_sync();
          const float cs = active ? p.scale[j] : 0.0f;
#pragma unroll
          for (int q = 0; q < kHalfRows / 32; ++q) {
#pragma unroll
            for (int u = 0; u < kIssuers; ++u) {
              if ((uint32_t)u < p.groups) {
                float d[32];
                tmem_ld32(tmem_base + lane_base + u * kRows + part * kHalfRows + 32 * q, d);
                tmem_ld_wait();
#pragma unroll
                for (int t = 0; t < 32; ++t) acc[32 * q + t] += d[t];
              }
            }
#pragma unroll
            for (int t = 0; t < 32; ++t) acc[32 * q + t] *= cs;
          }
          tc_fence_before_sync();
        }
      }
    }
    if (!ok) s_abort = 1;
    // ---- epilogue: per-row RMS factor, bias, activation, residual, store (one row at a time: coalesced) ----
    asm volatile("bar.sync 1, 512;" ::: "memory");  // s_rstd is written by the first four warps, read by all sixteen
    if (ok) {
      const GemvEpilogue& e = p.epi;
      const float bias = (e.bias && active) ? e.bias[j] : 0.0f;
#pragma unroll
      for (int r = 0; r < kHalfRows; ++r) {
        const uint32_t row = row0 + part * kHalfRows + r;
        if (row >= p.m) break;
        float v = acc[r] * s_rstd[part * kHalfRows + r];
        if (e.bias) v += bias;
        if (e.act == ACT_SWIGLU) {
          const float other = __shfl_xor_sync(0xFFFFFFFFu, v, 1);
          if (active && (j & 1u) == 0) {
            const float h = silu_ref(v) * other;
            const size_t o = (size_t)row * e.out_ld + (j >> 1);
            store_from_f32(p.out, e.out_dtype, o, e.resid ? e.resid[o] + h : h);
          }
        } else if (active) {
          if (e.act == ACT_GELU) v = gelu_ref(v);
          const size_t o = (size_t)row * e.out_ld + j;
          if (e.resid) v = e.resid[o] + v;
          store_from_f32(p.out, e.out_dtype, o, v);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (s_abort && tid == 0) atomicExch(p.status, 3);
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace gemm_tc

bool ruai_gemm_tc_eligible(const ruai_qweight* w, uint32_t m) {
  return w->layout == QL_CHUNK16 && m > 16 && (w->bits == 8 || w->n % 4 == 0);
}

int ruai_gemm_tc_launch(ruai_ctx* c, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                        const GemvEpilogue& epi_in, const GemvPrologue& pro) {
  using namespace gemm_tc;
  GemvEpilogue epi = epi_in;
  if (epi.act == ACT_SWIGLU && (w->n & 1)) return ruai_fail(c, RUAI_ERR_SHAPE, "SwiGLU epilogue needs an even column count, got %u", w->n);
  if (epi.out_ld == 0) epi.out_ld = epi.act == ACT_SWIGLU ? w->n / 2 : w->n;
  if (epi.sumsq || epi.argmax_out) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "the prefill GEMM has no fused sum of squares / argmax");
  const uint32_t groups = (w->k + 31) / 32, row_blocks = (m + kRows - 1) / kRows, col_tiles = (w->n + kCols - 1) / kCols;
  if (row_blocks > 65535) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "m too large");
  // the split activations live in the context's scratch
  const size_t xs_bytes = (size_t)row_blocks * groups * kBGroupBytes;
  RUAI_TRY(ruai_ctx_reserve(c, xs_bytes, 0));
  unsigned char* xs = reinterpret_cast<unsigned char*>(c->partial);
  RUAI_CUDA(c, ruai_launch(c, xsplit_kernel, dim3(groups, row_blocks), dim3(kRows), 0, true, x, x_dtype, x_ld, m, w->k, pro.norm_w, groups, xs));
  Params p;
  p.w = (const uint4*)w->data; p.scale = w->scale; p.xs = xs; p.m = m; p.k = w->k; p.n = w->n; p.chunks = w->chunks; p.groups = groups;
  p.out = out; p.status = c->status; p.epi = epi;
  p.rstd_sumsq = pro.norm_w ? pro.sumsq : nullptr; p.rstd_tiles = pro.tiles; p.eps = pro.eps;
  static bool attr_done[64][2] = {};
  const int bi = w->bits == 8 ? 1 : 0;
  if (!attr_done[c->ordinal & 63][bi]) {
    cudaError_t e = bi ? cudaFuncSetAttribute(gemm_tc_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes)
                       : cudaFuncSetAttribute(gemm_tc_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done[c->ordinal & 63][bi] = true;
  }
  const dim3 grid(col_tiles, row_blocks);
  cudaError_t e = bi ? ruai_launch(c, gemm_tc_kernel<8>, grid, dim3(kThreads), kSmemBytes, true, p)
                     : ruai_launch(c, gemm_tc_kernel<4>, grid, dim3(kThreads), kSmemBytes, true, p);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "prefill GEMM launch failed: %s", cudaGetErrorString(e));
  return RUAI_OK;
}

