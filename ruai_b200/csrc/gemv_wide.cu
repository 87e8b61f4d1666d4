// Fused dequantize + matmul for 5..16 rows of activations (a decode step of 5..16 sequences), int4 group-32 and
// int8 weights: out[m,n] = x[m,k] @ dequant(W)[k,n] with the packed weight streamed from HBM exactly once.
//
// The digit scheme of the narrow GEMV (three int8 digits per activation, one s32 sum per digit to read back and
// combine) costs work per (group, column, ROW); at sixteen rows that read-out, not HBM, sets the time.  Here the
// activations are split once, by a small pre-kernel, into two bf16 pieces x = hi + lo (16 significant bits) laid
// out as the tensor core's B operand, the weights become bf16 (every int4 / int8 value is exact in bf16), and
// `tcgen05.mma kind::f16` accumulates both pieces in f32: per (group, column) the read-out is sixteen f32 words
// and sixteen FMAs with scale[g, j] (int4: cpu.rs:1045-1063), or nothing until the end (int8: cpu.rs:903-920).
//
// A CTA owns 128 columns of W and a slice of k; two CTAs share an SM.
//   * four expanding warps (thread = column): the packed weights of their column go global -> registers, some stages
//     ahead of their use and without waiting for the predecessor kernel; nibbles / bytes -> bf16 pairs, written
//     straight into TENSOR memory as the A operand (lane = column of W, sixteen 32-bit words per group of 32 k); one
//     of their threads keeps the ring of split activations full with bulk copies;
//   * two issuing warps, each with every other group of a stage (per group: two k-steps x two pieces, M = 128,
//     N = 16, K = 16).  Issuing an MMA costs its thread about 116 clocks whatever N is (measured up to N = 128), so
//     the sixteen MMAs of a stage are what a stage costs: two threads issue them side by side.  (Tried and measured
//     slower: both pieces side by side in one MMA of N = 32, which needs single-buffered sums and so a hand-off per
//     stage between issue and read-out; the same with a hand-off per group; four issuing warps, whose 384 threads
//     leave 80 registers and make the expanding warps spill.)
//   * four draining warps (thread = column): int4: per stage the groups' sums out of tensor memory (double
//     buffered), times the group's scale, into sixteen f32 registers; they run the epilogue shared with the narrow GEMV.
// Split-k over a cluster (<= 8) with the partial sums sent through distributed shared memory.  Every mbarrier wait
// is bounded; a wait that runs out sets status 3 and the kernel still leaves through its barriers.
#include "common.cuh"
#include "gemv_epilogue.cuh"
#include "pipeline.cuh"

namespace gemv_wide {

using namespace pipe;

constexpr int kCols = 128;            // columns of W per CTA = MMA M = TMEM lanes
constexpr int kRows = 16;             // rows of x = MMA N
constexpr int kStageGroups = 4;       // groups of 32 k per stage
constexpr int kXsGroupBytes = 2 * 2 * kRows * 32;           // pieces x k-steps x rows x 32 B = 2 KB per group
constexpr int kXsTileBytes = 2 * kXsGroupBytes;             // a swizzled tile: 64 k (two groups) x 32 rows x 2 B = 4 KB
constexpr int kXsStageBytes = kStageGroups * kXsGroupBytes;  // 8 KB: two tiles
constexpr int kXsSlots = 6;           // ring of activation stages
constexpr int kIssuers = 2;           // issuing warps; each takes every kIssuers-th group of a stage (four of them need 384 threads,
                                      // 80 registers each, and the expanding warps then spill and set the pace)
constexpr int kThreads = 2 * kCols + 32 * kIssuers;  // draining warps 0-3, expanding warps 5-8, issuing warps 4 and 9 ..
constexpr int kTmemCols = 256;        // accumulators in columns 0..127 (int4: 2 stages x 4 groups x 16), A operand in 128..255 (2 stages x 4 groups x 16)
constexpr uint32_t kACol0 = 128;
constexpr int kPartialBytes = kRows * kCols * 4;  // one CTA's partial sums (split-k)

// ---- activations -> two bf16 pieces in B-operand layout ------------------------------------------------------
// The B operand of the MMAs, K-major with the 128-byte swizzle: per 64 k (two groups) a tile of 32 rows x 128 bytes,
// rows 0..15 the hi pieces of the sixteen rows of x and rows 16..31 their lo pieces.  Within the tile, row t lies at
// (t / 8) * 1024 + (t % 8) * 128 and its 16-byte chunk c (8 k) at position c ^ (t % 8).  An MMA takes 16 k of
// sixteen rows: the tile's address plus 32 bytes per k-step, plus 2 KB for the lo pieces.
// One thread per (8-k chunk, row): it reads one 32-byte sector of x and writes two 16-byte chunks.
__global__ void __launch_bounds__(256) xsplit16_kernel(const void* __restrict__ x, int x_dtype, uint32_t x_ld, uint32_t m, uint32_t k,
                                                       const float* __restrict__ norm_w, uint32_t groups, unsigned char* __restrict__ xs) {
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t idx = blockIdx.x * 256u + threadIdx.x, r = idx & 15u, kc = idx >> 4;
  if (kc >= ((groups + 1u) & ~1u) * 4u) return;  // whole tiles: an odd last group is followed by 32 k of zeros
  const uint32_t k0 = kc * 8u;
  float v[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) v[t] = 0.0f;
  if (r < m) {
    const bool fast = x_dtype == RUAI_F32 && (x_ld & 3u) == 0 && ((uintptr_t)x & 15u) == 0 && k0 + 8u <= k;
    if (fast) {
      const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)r * x_ld + k0);
      const float4 a = src[0], b = src[1];
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int t = 0; t < 8; ++t)
        if (k0 + t < k) v[t] = load_as_f32(x, x_dtype, (size_t)r * x_ld + k0 + t);
    }
    if (norm_w) {
#pragma unroll
      for (int t = 0; t < 8; ++t)
        if (k0 + t < k) v[t] *= norm_w[k0 + t];
    }
  }
  uint32_t hi[4], lo[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(v[2 * t]), h1 = __float2bfloat16_rn(v[2 * t + 1]);
    const __nv_bfloat16 l0 = __float2bfloat16_rn(v[2 * t] - __bfloat162float(h0)), l1 = __float2bfloat16_rn(v[2 * t + 1] - __bfloat162float(h1));
    hi[t] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
    lo[t] = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
  }
  // tile kc / 8 (64 k), chunk kc % 8 of the row; the lo piece's row is 16 further on, two 8-row blocks = 2 KB
  unsigned char* dst = xs + (size_t)(kc >> 3) * kXsTileBytes + (r >> 3) * 1024u + (r & 7u) * 128u + (((kc & 7u) ^ (r & 7u)) << 4);
  *reinterpret_cast<uint4*>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  *reinterpret_cast<uint4*>(dst + 2048) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
}

struct Params {
  const uint4* w;
  const float* scale;
  const unsigned char* xs;
  uint32_t m, k, n, chunks, groups, groups_per_cta, splits;
  void* out;
  int* status;
  GemvEpilogue epi;
  GemvPrologue pro;
};

// Shared-memory operand descriptor, K-major, 128-byte swizzle: rows of 128 bytes, 1024 bytes between 8-row blocks; the
// tile starts on a 1024-byte boundary and an MMA's 32 bytes of k are addressed by adding them to the start address.
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: bf16 operands, f32 accumulate, both K-major, M = 128.
__host__ __device__ constexpr uint32_t idesc_bf16(uint32_t n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24); }
// D[tmem] (+)= A[tmem] * B[smem]: A's lane = row of A, 32-bit column c holds A[row][2 c], A[row][2 c + 1] (low half first).
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem), "r"(a_tmem),
               "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}
// The same, executed by the lanes whose `lead` is non-zero (the warp stays converged around it).
__device__ __forceinline__ void umma_bf16_ts_if(uint32_t lead, uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(lead)
      : "memory");
}
__device__ __forceinline__ void umma_commit_if(uint32_t lead, uint64_t* bar) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_u32(bar)),
               "r"(lead)
               : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr), "r"(v[0]),
      "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]),
      "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16f(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Sixteen packed weights of one column -> eight words of bf16 pairs (consecutive k in the low and high half).
// int4: the chunk's word w4 holds rows 4 w4 .. 4 w4 + 3 of k-step 0 in its low nibbles and of k-step 1 in its high
// nibbles, as value + 8; (128 + u) has the bf16 bit pattern 0x4300 | u, and subtracting 136 gives the weight exactly.
__device__ __forceinline__ void expand_int4(const uint4& wv, uint32_t (&o)[16]) {
  const uint32_t wd[4] = {wv.x, wv.y, wv.z, wv.w};
  const __nv_bfloat162 off = __floats2bfloat162_rn(136.0f, 136.0f);
#pragma unroll
  for (int s = 0; s < 2; ++s) {
#pragma unroll
    for (int w4 = 0; w4 < 4; ++w4) {
      const uint32_t nib = (s ? (wd[w4] >> 4) : wd[w4]) & 0x0F0F0F0Fu;
      const uint32_t pl[2] = {__byte_perm(nib, 0x43434343u, 0x4140), __byte_perm(nib, 0x43434343u, 0x4342)};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __nv_bfloat162 a2 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&pl[h]), off);
        o[8 * s + 2 * w4 + h] = *reinterpret_cast<const uint32_t*>(&a2);
      }
    }
  }
}
// int8: a chunk is one k-step (16 rows).  (byte ^ 0x80) is value + 128; 2^23 + that has the f32 bit pattern
// 0x4B000000 | byte, so one subtraction gives the value exactly and one conversion packs two of them.
__device__ __forceinline__ void expand_int8(const uint4& wv, uint32_t* o) {
  const uint32_t wd[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
  for (int w4 = 0; w4 < 4; ++w4) {
    const uint32_t u = wd[w4] ^ 0x80808080u;
    const float f0 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
    const float f1 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
    const float f2 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
    const float f3 = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(f0, f1), p1 = __floats2bfloat162_rn(f2, f3);
    o[2 * w4] = *reinterpret_cast<const uint32_t*>(&p0);
    o[2 * w4 + 1] = *reinterpret_cast<const uint32_t*>(&p1);
  }
}

constexpr size_t smem_bytes(uint32_t splits) {
  const size_t ring = (size_t)kXsSlots * kXsStageBytes, red = (size_t)(splits > 1 ? splits - 1 : 0) * kPartialBytes;
  return ring + red + 1024;
}

template <int BITS>
__global__ void __launch_bounds__(kThreads, 2) gemv_wide_kernel(const Params p) {
  constexpr int kAhead = BITS == 4 ? 3 : 2;                    // stages of packed weights in registers
  constexpr int kStageChunks = BITS == 4 ? kStageGroups : 2 * kStageGroups;  // 16-byte chunks per column and stage
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // the swizzled tiles start on 1024-byte boundaries (same offset in every CTA of a cluster: the window bases are alike)
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t xs_full[kXsSlots];   // activations of a stage landed
  __shared__ __align__(8) uint64_t a_ready[2];          // A operand of a stage written (4 expanding warps)
  __shared__ __align__(8) uint64_t mma_done[2];         // MMAs of a stage completed (both issuing warps): A buffer and ring slot free; int4: sums valid
  __shared__ __align__(8) uint64_t acc_free[2];         // int4: the sums of a stage read out (4 draining warps)
  __shared__ __align__(8) uint64_t all_done;            // int8: every MMA of the slice completed
  __shared__ uint32_t s_tmem;
  __shared__ float s_rstd[kRows];
  __shared__ float s_red[kThreads / 32];
  __shared__ int2 s_arg[kThreads / 32];
  __shared__ unsigned s_flag;
  __shared__ volatile int s_abort;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t j0 = blockIdx.x * kCols, j = j0 + tid;
  const bool active = tid < kCols && j < p.n;
  const uint32_t split = p.splits > 1 ? cluster_ctarank() : 0u;
  const uint32_t g_begin = min(p.groups, split * p.groups_per_cta);
  const uint32_t g_end = min(p.groups, g_begin + p.groups_per_cta);
  const uint32_t nst = (g_end - g_begin + kStageGroups - 1) / kStageGroups;
  const uint32_t rows = p.m;

  if (tid == 0) {
    for (int s = 0; s < kXsSlots; ++s) { mbar_init(&xs_full[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&a_ready[s], kCols / 32); mbar_init(&mma_done[s], kIssuers); mbar_init(&acc_free[s], kCols / 32); }
    mbar_init(&all_done, kIssuers);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_abort = 0;
  }
  __syncwarp();
  if (warp == 0) tmem_alloc(&s_tmem, kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s_tmem;
  const bool normed = p.pro.norm_w != nullptr;
  float acc[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) acc[r] = 0.0f;
  // one stage of the split activations into its slot of the ring (one thread)
  auto xs_copy = [&](uint32_t i) {
    const uint32_t slot = i % kXsSlots, g0 = g_begin + i * kStageGroups, ng = min((uint32_t)kStageGroups, g_end - g0);
    const uint32_t bytes = ((ng + 1u) >> 1) * kXsTileBytes;  // whole tiles (g0 is even)
    mbar_expect_tx(&xs_full[slot], bytes);
    bulk_load(smem + (size_t)slot * kXsStageBytes, p.xs + (size_t)g0 * kXsGroupBytes, bytes, &xs_full[slot]);
  };

  if (warp > kCols / 32 && warp <= 2 * kCols / 32) {
    // ===== expanding warps: packed weights -> bf16 A operand in tensor memory.  Nothing here depends on the
    // predecessor kernel.  A warp reaches the lanes 32 (warp % 4) .. of tensor memory, so its threads take those columns.
    const uint32_t te = (uint32_t)(warp & 3) * 32u + lane, je = j0 + te;
    const bool in_col = je < p.n;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    uint4 wq[kAhead][kStageChunks];
    auto load_stage = [&](uint32_t i, uint4 (&wv)[kStageChunks]) {
#pragma unroll
      for (int u = 0; u < kStageChunks; ++u) {
        // int4: chunk = group; int8: chunks 2 g and 2 g + 1 are the group's two k-steps
        const uint32_t g = g_begin + i * kStageGroups + (BITS == 4 ? u : u >> 1);
        const uint32_t c = BITS == 4 ? g : 2 * g + (u & 1);
        // beyond the slice or the matrix: weight 0 (int4 stores value + 8)
        const uint32_t zero = BITS == 4 ? 0x88888888u : 0u;
        wv[u] = (in_col && g < g_end && c < p.chunks) ? ldg_stream_u4(&p.w[(size_t)c * p.n + je]) : make_uint4(zero, zero, zero, zero);
      }
    };
#pragma unroll
    for (int a = 0; a < kAhead; ++a) load_stage(a, wq[a]);
    bool ok = true;
    for (uint32_t i0 = 0; i0 < nst && ok; i0 += kAhead) {
#pragma unroll
      for (int a = 0; a < kAhead; ++a) {
        const uint32_t i = i0 + a;
        if (i >= nst) break;
        const uint32_t b = i & 1u, q = i >> 1;
        if (q > 0 && (s_abort || !mbar_wait(&mma_done[b], (q - 1) & 1u))) { ok = false; break; }  // the MMAs that read this buffer last are done
        tc_fence_after_sync();
        // the MMAs of stage i - 2 are done, so its slot of the activation ring is free: the stage kXsSlots after it goes there
        // (griddepcontrol.wait: the copy reads the predecessor's output; it has long returned by now)
        if (tid == 5 * 32 && q > 0 && i - 2 + kXsSlots < nst) { grid_dependency_wait(); xs_copy(i - 2 + kXsSlots); }
#pragma unroll
        for (int u = 0; u < kStageGroups; ++u) {
          uint32_t o[16];
          if constexpr (BITS == 4) expand_int4(wq[a][u], o);
          else { expand_int8(wq[a][2 * u], o); expand_int8(wq[a][2 * u + 1], o + 8); }
          tmem_st16(tmem_base + lane_base + kACol0 + (b * kStageGroups + u) * 16u, o);
        }
        load_stage(i + kAhead, wq[a]);  // the stage kAhead further on, into the registers just consumed
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_ready[b]);
      }
    }
    if (!ok) s_abort = 1;
  } else if (warp == kCols / 32 || warp > 2 * kCols / 32) {
    // ===== issuing warps, each with its share of a stage's groups: issuing one MMA costs its thread more than a hundred
    // clocks whatever the MMA's size (measured: 116 for kind::f16 up to N = 128), and a stage has sixteen of them =====
    const uint32_t wi = warp == kCols / 32 ? 0u : (uint32_t)warp - 2 * kCols / 32;
    grid_dependency_wait();
    if (wi == 0) {
      grid_launch_dependents();
      // RMSNorm: x * rstd * w with rstd a per-row scalar: the pieces are taken from x * w, rstd multiplies the finished sums
      if (normed && lane < kRows) {
        float ss = 0.0f;
        if (lane < (int)rows)
          for (uint32_t t = 0; t < p.pro.tiles; ++t) ss += p.pro.sumsq[(size_t)t * p.m + lane];
        s_rstd[lane] = 1.0f / sqrtf(ss * (1.0f / (float)p.k) + p.pro.eps);
      }
      // the first stages of the split activations (the predecessor's output); an expanding thread refills the ring
      if (lane == 0) {
        for (uint32_t i = 0; i < nst && i < (uint32_t)kXsSlots; ++i) xs_copy(i);
      }
      __syncwarp();
    }
    {
      // The whole warp runs the issuing loop, converged, so that the operands of the MMAs (descriptors, tensor-memory
      // addresses) are warp-uniform values; only the instructions themselves are predicated on the first lane.
      constexpr uint32_t idesc = idesc_bf16(kRows);
      const uint32_t lead = lane == 0 ? 1u : 0u;
      const uint32_t tb = __shfl_sync(0xFFFFFFFFu, tmem_base, 0);
      const uint64_t bd0 = umma_desc_kmajor_sw128(smem_u32(smem));
      for (uint32_t i = 0; i < nst; ++i) {
        const uint32_t b = i & 1u, q = i >> 1, slot = i % kXsSlots, lap = i / kXsSlots;
        bool ok = !s_abort;
        if (ok && BITS == 4 && q > 0) ok = mbar_wait(&acc_free[b], (q - 1) & 1u);  // the sums these MMAs overwrite have been read
        if (ok) ok = mbar_wait(&xs_full[slot], lap & 1u);
        if (ok) ok = mbar_wait(&a_ready[b], q & 1u);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) { s_abort = 1; break; }
        tc_fence_after_sync();
        const uint32_t ng = min((uint32_t)kStageGroups, g_end - (g_begin + i * kStageGroups));
        for (uint32_t u = wi; u < ng; u += kIssuers) {
          // int4: one accumulator per group, two stages of them; int8: one per issuing warp over the whole slice (MMAs
          // of two threads are not ordered among themselves)
          const uint32_t d = tb + (BITS == 4 ? (b * kStageGroups + u) * kRows : wi * kRows);
          const uint32_t at = tb + kACol0 + (b * kStageGroups + u) * 16u;
          // group u of the stage: tile u / 2, and in its rows the 64 bytes from (u % 2) * 64 on; the lo pieces' rows 2 KB further
          const uint64_t bd = umma_desc_advance(bd0, slot * kXsStageBytes + (u >> 1) * kXsTileBytes + (u & 1u) * 64u);
#pragma unroll
          for (uint32_t s = 0; s < 2; ++s)
#pragma unroll
            for (uint32_t pc = 0; pc < 2; ++pc) {
              const uint32_t accumulate = BITS == 4 ? (s | pc) : ((i | (u - wi) | s | pc) != 0u ? 1u : 0u);
              umma_bf16_ts_if(lead, d, at + s * 8u, umma_desc_advance(bd, s * 32u + pc * 2048u), idesc, accumulate);
            }
        }
        umma_commit_if(lead, &mma_done[b]);
        if (BITS == 8 && i + 1 == nst) umma_commit_if(lead, &all_done);
      }
    }
  } else {
    // ===== draining warps =====
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    if constexpr (BITS == 4) {
      // scales of this thread's column kAhead stages ahead of their use; they do not depend on the predecessor
      float sq[kAhead][kStageGroups];
      auto load_scales = [&](uint32_t i, float (&sv)[kStageGroups]) {
#pragma unroll
        for (int u = 0; u < kStageGroups; ++u) {
          const uint32_t g = g_begin + i * kStageGroups + u;
          sv[u] = (active && g < g_end) ? ldg_stream_f32(&p.scale[(size_t)g * p.n + j]) : 0.0f;
        }
      };
#pragma unroll
      for (int a = 0; a < kAhead; ++a) load_scales(a, sq[a]);
      grid_dependency_wait();
      bool ok = true;
      for (uint32_t i0 = 0; i0 < nst && ok; i0 += kAhead) {
#pragma unroll
        for (int a = 0; a < kAhead; ++a) {
          const uint32_t i = i0 + a;
          if (i >= nst) break;
          const uint32_t b = i & 1u, q = i >> 1;
          if (s_abort || !mbar_wait(&mma_done[b], q & 1u)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t ng = min((uint32_t)kStageGroups, g_end - (g_begin + i * kStageGroups));  // groups beyond the slice have no MMA
#pragma unroll
          for (int u2 = 0; u2 < kStageGroups; u2 += 2) {
            float d0[kRows], d1[kRows];
            const bool in0 = (uint32_t)u2 < ng, in1 = (uint32_t)u2 + 1 < ng;
            if (in0) tmem_ld16f(tmem_base + lane_base + (b * kStageGroups + u2) * kRows, d0);
            if (in1) tmem_ld16f(tmem_base + lane_base + (b * kStageGroups + u2 + 1) * kRows, d1);
            tmem_ld_wait();
            if (u2 + 2 == kStageGroups) {
              // all the sums of the stage are in registers: the issuing warps may overwrite them
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_free[b]);
            }
            if (in0) {
#pragma unroll
              for (int r = 0; r < kRows; ++r) acc[r] = fmaf(d0[r], sq[a][u2], acc[r]);
            }
            if (in1) {
#pragma unroll
              for (int r = 0; r < kRows; ++r) acc[r] = fmaf(d1[r], sq[a][u2 + 1], acc[r]);
            }
          }
          load_scales(i + kAhead, sq[a]);
        }
      }
      if (!ok) s_abort = 1;
    } else {
      // int8: one accumulator over the whole slice, scaled per column at the end (cpu.rs:918-920)
      const float cs = active ? p.scale[j] : 0.0f;
      grid_dependency_wait();
      if (nst > 0) {
        // (a barrier of its own: the stage barriers alternate and a wait for a late phase of one cannot tell it from an early one)
        if (!mbar_wait(&all_done, 0u) || s_abort) s_abort = 1;
        else {
          tc_fence_after_sync();
          // issuing warp u had groups at all if the slice has more than u of them
          const uint32_t had = min((uint32_t)kIssuers, g_end - g_begin);
#pragma unroll
          for (int u = 0; u < kIssuers; ++u) {
            float d[kRows];
            if ((uint32_t)u < had) {
              tmem_ld16f(tmem_base + lane_base + u * kRows, d);
              tmem_ld_wait();
#pragma unroll
              for (int r = 0; r < kRows; ++r) acc[r] += d[r];
            }
          }
#pragma unroll
          for (int r = 0; r < kRows; ++r) acc[r] *= cs;
          tc_fence_before_sync();
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (s_abort && tid == 0) atomicExch(p.status, 3);
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);

  // ---- split-k inside the cluster: the partial sums go to the first CTA's shared memory (a region after its ring) ----
  if (p.splits > 1) {
    float* red = reinterpret_cast<float*>(smem + (size_t)kXsSlots * kXsStageBytes);
    if (split != 0 && tid < kCols) {
#pragma unroll
      for (int r = 0; r < kRows; ++r) st_cluster_f32(red + ((size_t)(split - 1) * kRows + r) * kCols + tid, 0, acc[r]);
    }
    cluster_sync_all();
    if (split != 0) return;
    if (tid < kCols) {
      for (uint32_t s = 0; s + 1 < p.splits; ++s) {
#pragma unroll
        for (int r = 0; r < kRows; ++r) acc[r] += red[((size_t)s * kRows + r) * kCols + tid];
      }
    }
  }
  if (normed) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[r] *= s_rstd[r];
  }
  gemv_epilogue<kRows, kThreads>(p.epi, acc, rows, 0u, p.m, j, active, false, 1.0f, p.out, s_red, s_arg, &s_flag, nullptr);
}

template <int BITS>
cudaError_t launch_one(ruai_ctx* c, const Params& p, dim3 grid) {
  static bool attr_done[64] = {};
  if (!attr_done[c->ordinal & 63]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_wide_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes(8));
    if (e != cudaSuccess) return e;
    attr_done[c->ordinal & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_bytes(p.splits);
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
  return cudaLaunchKernelEx(&cfg, gemv_wide_kernel<BITS>, p);
}

}  // namespace gemv_wide

// From five rows on: measured on the 8B shapes, this kernel at 9 rows is faster than the narrow kernels at 5 .. 8 rows for
// every Linear (int4 gate/up 39 against 53 us, down_proj 23 against 38; int8 head 163 against 261); up to four rows the
// narrow kernels win (gate/up 33 us).  And from four million weights on: a smaller Linear is over before the pre-kernel
// that splits the activations has paid for itself (135M-parameter shapes, 16 sequences: 1.44 ms per step without, 1.94 with).
bool ruai_gemv_wide_eligible(const ruai_ctx* c, const ruai_qweight* w, uint32_t m) {
  (void)c;
  // int8 with a long k also at four rows: the narrow int8 kernel converts its whole slice of the activations before its first
  // MMA, which at 4 x 14336 costs more than this kernel in all (down_proj of the 8B shape: 43 us there, 28 here)
  const uint32_t from = (w->bits == 8 && w->k >= 8192) ? 4u : 5u;
  return w->layout == QL_CHUNK16 && ((w->bits == 4 && w->group == 32) || w->bits == 8) && m >= from && m <= (uint32_t)gemv_wide::kRows &&
         (uint64_t)w->k * w->n >= (1ull << 22);
}

int ruai_gemv_wide_launch(ruai_ctx* c, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                          const GemvEpilogue& epi_in, const GemvPrologue& pro) {
  using namespace gemv_wide;
  GemvEpilogue epi = epi_in;
  if (epi.act == ACT_SWIGLU && (w->n & 1)) return ruai_fail(c, RUAI_ERR_SHAPE, "SwiGLU epilogue needs an even column count, got %u", w->n);
  if (epi.out_ld == 0) epi.out_ld = epi.act == ACT_SWIGLU ? w->n / 2 : w->n;
  if (epi.sumsq && epi.act == ACT_SWIGLU) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "sum of squares with the SwiGLU epilogue");
  if (epi.argmax_out && epi.act == ACT_SWIGLU) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "argmax with the SwiGLU epilogue");
  const uint32_t groups = (w->k + 31) / 32, col_tiles = (w->n + kCols - 1) / kCols;
  // the split activations live in the context's scratch
  RUAI_TRY(ruai_ctx_reserve(c, (size_t)((groups + 1u) & ~1u) * kXsGroupBytes, 0));
  unsigned char* xs = reinterpret_cast<unsigned char*>(c->partial);
  RUAI_CUDA(c, ruai_launch(c, xsplit16_kernel, dim3((((groups + 1u) & ~1u) * 4u * kRows + 255u) / 256u), dim3(256), 0, true, x, x_dtype, x_ld, m, w->k, pro.norm_w, groups, xs));
  // Split k over a cluster of up to 8 CTAs so that the launch fills the two CTA places of every SM; what counts is the
  // launch's latency: a fixed part per wave of CTAs, a part per stage, a part per CTA of the cluster for the reduction.
  const double per_stage = w->bits == 4 ? 0.5 : 0.8;
  const uint32_t slots = 2u * (uint32_t)c->sm_count;
  uint32_t splits = 1;
  double best = 1e30;
  for (uint32_t s2 = 1; s2 <= 8; s2 *= 2) {
    const uint32_t per = (groups + s2 - 1) / s2;
    if (s2 > 1 && per < 2u * kStageGroups) break;
    const uint32_t stages = (per + kStageGroups - 1) / kStageGroups;
    const uint32_t ctas = col_tiles * s2, waves = (ctas + slots - 1) / slots;
    const double t = waves * (5.5 + per_stage * stages) + 0.3 * s2;
    if (t < best) { best = t; splits = s2; }
  }
  if ((c->force_splits & 255u) && (c->force_splits & 255u) <= 8) splits = c->force_splits & 255u;
  uint32_t gpc = (groups + splits - 1) / splits;
  gpc = (gpc + kStageGroups - 1) / kStageGroups * kStageGroups;
  Params p;
  p.w = (const uint4*)w->data; p.scale = w->scale; p.xs = xs; p.m = m; p.k = w->k; p.n = w->n; p.chunks = w->chunks;
  p.groups = groups; p.groups_per_cta = gpc; p.splits = splits;
  p.out = out; p.status = c->status; p.epi = epi; p.pro = pro;
  const dim3 grid(col_tiles, splits, 1);
  cudaError_t e = w->bits == 4 ? launch_one<4>(c, p, grid) : launch_one<8>(c, p, grid);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "wide gemv launch failed: %s", cudaGetErrorString(e));
  return RUAI_OK;
}

