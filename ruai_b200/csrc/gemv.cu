// Fused dequantize + GEMV for small row counts (decode): y[m,n] = x[m,k] @ W[k,n].
//
// Replaces the reference's one-thread-per-output kernels matmul_int8_* / matmul_int4_*
// (src/nn/backend/cuda_kernels.cu:499-552, dispatched from cuda.rs:788-833) with the
// arithmetic of the CPU definition (cpu.rs:897-927, 1035-1067): f32 products of the
// activations with the integer weights, int8 scaled once per column at the end,
// int4 scaled per group of 32 rows before accumulation.
//
// Work split.  The weight is stored as 16-byte chunks, chunk c of column j at
// (c*n + j)*16 (pack.cu).  A CTA of 256 threads owns 256 neighbouring columns (one
// per thread, so a warp streams 512 contiguous bytes per chunk) and one slice of
// the chunks (split-K across CTAs, so that every SM streams a share of the matrix
// even when n is small).  The slice of x is staged in shared memory and read as
// broadcast float4s.  Weight chunks are requested four ahead, and the first four
// before the grid-dependency wait, so the fetch overlaps the predecessor's tail.
// Split-K partials go to a scratch buffer; the last CTA to arrive for a column
// tile adds them in split order (deterministic) and applies the epilogue:
// int8 scale, bias, GELU or SwiGLU, residual add, output cast.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;   // columns per CTA
constexpr int kStageK = 512;    // activations per row staged in shared memory at a time
constexpr int kAhead = 4;       // weight chunks in flight per thread

struct GemvParams {
  const uint4* w;
  const float* scale;
  const void* x;
  int x_dtype;
  uint32_t x_ld, m, k, n, chunks, chunks_per_split, splits;
  float* partial;
  unsigned* counters;
  void* out;
  GemvEpilogue epi;
  GemvPrologue pro;
};

__device__ __forceinline__ int32_t ordered_bits(float v) {  // total_cmp order as a signed integer
  int32_t i = __float_as_int(v);
  return i ^ (int32_t)(((uint32_t)(i >> 31)) >> 1);
}

// Byte `b` of `w` as an exact float: the byte becomes the low mantissa byte of
// 2^23, then 2^23 + offset is subtracted.
template <int B>
__device__ __forceinline__ float byte_f32(uint32_t w, float magic) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + B)) - magic;
}

// cpu.rs:229-239 (`1 - 2/(exp(2u)+1)` with u clamped to +-15).
__device__ __forceinline__ float gelu_ref(float x) {
  float u = 0.7978846f * (x + 0.044715f * x * x * x);
  u = fminf(fmaxf(u, -15.0f), 15.0f);
  const float t = 1.0f - 2.0f / (expf(2.0f * u) + 1.0f);
  return 0.5f * x * (1.0f + t);
}
// ops.rs:158-160 over cpu.rs:376.
__device__ __forceinline__ float silu_ref(float v) { return v * (1.0f / (1.0f + expf(-v))); }

template <int BITS, int MT>
__global__ void __launch_bounds__(kThreads) gemv_kernel(const GemvParams p) {
  constexpr int CK = BITS == 8 ? 16 : 32;       // rows of W per chunk
  constexpr int kStageChunks = kStageK / CK;    // chunks per shared-memory stage
  extern __shared__ __align__(16) float xs[];   // [MT][kStageK]
  __shared__ unsigned s_last;
  __shared__ float s_rstd[MT];
  __shared__ float s_red[kThreads / 32];
  __shared__ int2 s_arg[kThreads / 32];

  const int tid = threadIdx.x;
  const uint32_t j = blockIdx.x * kThreads + tid;
  const bool active = j < p.n;
  const uint32_t split = blockIdx.y;
  const uint32_t m0 = blockIdx.z * MT;
  const uint32_t rows = min((uint32_t)MT, p.m - m0);
  const uint32_t c_begin = split * p.chunks_per_split;
  const uint32_t c_end = min(p.chunks, c_begin + p.chunks_per_split);

  float acc[MT];
#pragma unroll
  for (int r = 0; r < MT; ++r) acc[r] = 0.0f;

  // weights do not depend on the predecessor kernel: request them before waiting for it
  uint4 wbuf[kAhead];
  float sbuf[kAhead];
#pragma unroll
  for (int u = 0; u < kAhead; ++u) {
    const uint32_t c = c_begin + u;
    wbuf[u] = make_uint4(0, 0, 0, 0);
    sbuf[u] = 0.0f;
    if (active && c < c_end) {
      wbuf[u] = __ldcs(&p.w[(size_t)c * p.n + j]);
      if (BITS == 4) sbuf[u] = __ldcs(&p.scale[(size_t)c * p.n + j]);
    }
  }
  grid_dependency_wait();
  grid_launch_dependents();
  const bool normed = p.pro.norm_w != nullptr;
  if (normed && tid < MT) {
    float ss = 0.0f;
    if (tid < (int)rows)
      for (uint32_t t = 0; t < p.pro.tiles; ++t) ss += p.pro.sumsq[(size_t)t * p.m + m0 + tid];
    s_rstd[tid] = 1.0f / sqrtf(ss * (1.0f / (float)p.k) + p.pro.eps);
  }

  for (uint32_t c0 = c_begin; c0 < c_end; c0 += kStageChunks) {
    const uint32_t c1 = min(c_end, c0 + kStageChunks);
    const uint32_t len = (c1 - c0) * CK;
    __syncthreads();
    for (uint32_t idx = tid; idx < MT * len; idx += kThreads) {
      const uint32_t r = idx / len, kk = idx - r * len;
      const uint32_t kidx = c0 * CK + kk;
      float v = 0.0f;
      if (r < rows && kidx < p.k) {
        v = load_as_f32(p.x, p.x_dtype, (size_t)(m0 + r) * p.x_ld + kidx);
        if (normed) v = v * s_rstd[r] * p.pro.norm_w[kidx];
      }
      xs[r * kStageK + kk] = v;
    }
    __syncthreads();
    for (uint32_t cb = c0; cb < c1; cb += kAhead) {
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const uint32_t c = cb + u;
        if (c < c1) {
          const uint4 wv = wbuf[u];
          const float sv = sbuf[u];
          // refill this slot with the chunk kAhead further on
          const uint32_t cn = c + kAhead;
          if (active && cn < c_end) {
            wbuf[u] = __ldcs(&p.w[(size_t)cn * p.n + j]);
            if (BITS == 4) sbuf[u] = __ldcs(&p.scale[(size_t)cn * p.n + j]);
          }
          const float* xr = xs + (c - c0) * CK;
          const uint32_t wd[4] = {wv.x, wv.y, wv.z, wv.w};
          if (BITS == 8) {
            float f[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t t = wd[i] ^ 0x80808080u;  // two's complement -> offset binary
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
            float f[32];  // rows 0..31 of the group, values -8..7
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
              float part = 0.0f;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 xv = *reinterpret_cast<const float4*>(xr + r * kStageK + 4 * i);
                part = fmaf(xv.x, f[4 * i + 0], part);
                part = fmaf(xv.y, f[4 * i + 1], part);
                part = fmaf(xv.z, f[4 * i + 2], part);
                part = fmaf(xv.w, f[4 * i + 3], part);
              }
              acc[r] = fmaf(part, sv, acc[r]);
            }
          }
        }
      }
    }
  }

  // ---- split-K: the last CTA of a column tile adds the partials in split order ----
  if (p.splits > 1) {
    if (active) {
#pragma unroll
      for (int r = 0; r < MT; ++r)
        if (r < (int)rows) __stcg(&p.partial[((size_t)split * p.m + m0 + r) * p.n + j], acc[r]);
    }
    __threadfence();
    __syncthreads();
    const uint32_t tile = blockIdx.z * gridDim.x + blockIdx.x;
    if (tid == 0) {
      const unsigned t = atomicAdd(&p.counters[tile], 1u);
      s_last = (t == p.splits - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) p.counters[tile] = 0;  // ready for the next launch
#pragma unroll
    for (int r = 0; r < MT; ++r) acc[r] = 0.0f;
    if (active) {
      if (MT == 1) {  // eight independent loads in flight, added in split order
        for (uint32_t s0 = 0; s0 < p.splits; s0 += 8) {
          float v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = s0 + u < p.splits ? __ldcg(&p.partial[((size_t)(s0 + u) * p.m + m0) * p.n + j]) : 0.0f;
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (s0 + u < p.splits) acc[0] += v[u];
        }
      } else {
        for (uint32_t s = 0; s < p.splits; ++s) {
#pragma unroll
          for (int r = 0; r < MT; ++r)
            if (r < (int)rows) acc[r] += __ldcg(&p.partial[((size_t)s * p.m + m0 + r) * p.n + j]);
        }
      }
    }
  }

  // ---- epilogue ----
  const GemvEpilogue& e = p.epi;
  const float col_scale = (BITS == 8 && active) ? p.scale[j] : 1.0f;
  const float bias = (e.bias && active) ? e.bias[j] : 0.0f;
  const int lane = tid & 31, warp = tid >> 5;
  bool last_tile = false;
#pragma unroll
  for (int r = 0; r < MT; ++r) {
    if (r >= (int)rows) break;  // uniform across the CTA
    float v = acc[r];
    if (BITS == 8) v *= col_scale;
    if (e.bias) v += bias;
    const size_t row = (size_t)(m0 + r);
    if (e.act == ACT_SWIGLU) {
      // columns (2i, 2i+1) hold (gate_i, up_i): layers.rs:573-576
      const float other = __shfl_xor_sync(0xFFFFFFFFu, v, 1);
      if (active && (j & 1u) == 0) {
        const float h = silu_ref(v) * other;
        const size_t o = row * e.out_ld + (j >> 1);
        store_from_f32(p.out, e.out_dtype, o, e.resid ? e.resid[o] + h : h);
      }
      continue;
    }
    if (active) {
      if (e.act == ACT_GELU) v = gelu_ref(v);
      const size_t o = row * e.out_ld + j;
      if (e.resid) v = e.resid[o] + v;
      store_from_f32(p.out, e.out_dtype, o, v);
    }
    if (e.sumsq) {  // sum of squares of this tile's part of the stored row, in a fixed order
      float q = active ? v * v : 0.0f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) q += __shfl_xor_sync(0xFFFFFFFFu, q, off);
      __syncthreads();
      if (lane == 0) s_red[warp] = q;
      __syncthreads();
      if (tid == 0) {
        float t = 0.0f;
        for (int w = 0; w < kThreads / 32; ++w) t += s_red[w];
        e.sumsq[(size_t)blockIdx.x * p.m + row] = t;
      }
    }
    if (e.argmax_out) {  // best (value, column) of this tile; ties go to the larger column
      int32_t bv = active ? ordered_bits(v) : INT32_MIN;
      int32_t bj = active ? (int32_t)j : -1;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const int32_t ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
        const int32_t oj = __shfl_xor_sync(0xFFFFFFFFu, bj, off);
        if (ov > bv || (ov == bv && oj > bj)) { bv = ov; bj = oj; }
      }
      __syncthreads();
      if (lane == 0) s_arg[warp] = make_int2(bv, bj);
      __syncthreads();
      if (tid == 0) {
        int2 b = s_arg[0];
        for (int w = 1; w < kThreads / 32; ++w)
          if (s_arg[w].x > b.x || (s_arg[w].x == b.x && s_arg[w].y > b.y)) b = s_arg[w];
        e.argmax_slots[(size_t)blockIdx.x * p.m + row] = b;
      }
    }
  }
  if (e.argmax_out) {
    // the last column tile to finish picks the winners
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned a = atomicAdd(e.argmax_counter, 1u);
      s_last = a == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    last_tile = s_last != 0;
    if (last_tile) {
      __threadfence();
      if (tid < (int)p.m) {
        const volatile int* sl = (const volatile int*)e.argmax_slots;
        int bv = INT32_MIN, bj = -1;
        for (uint32_t t = 0; t < gridDim.x; ++t) {
          const int v = sl[2 * ((size_t)t * p.m + tid)], jj = sl[2 * ((size_t)t * p.m + tid) + 1];
          if (v > bv || (v == bv && jj > bj)) { bv = v; bj = jj; }
        }
        e.argmax_out[tid] = bj;
      }
      if (tid == 0) {
        *e.argmax_counter = 0;
        if (e.len_ptr) *e.len_ptr += e.len_add;
      }
    }
  }
}

// Shapes outside the chunk layout (int4 with a group other than 32): one thread per
// output element over the reference layout, the reference kernel's own decomposition
// (cuda_kernels.cu:520-552) with the CPU path's per-group summation.
__global__ void gemv_int4_reference_layout_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale, const void* x, int x_dtype,
                                                  uint32_t x_ld, uint32_t m, uint32_t k, uint32_t n, uint32_t group, void* out,
                                                  GemvEpilogue e) {
  grid_dependency_wait();
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x, i = blockIdx.y;
  const bool glu = e.act == ACT_SWIGLU;
  const uint32_t j = glu ? 2 * t : t;
  if (j >= n || i >= m) return;
  auto column = [&](uint32_t col) {
    float acc = 0.0f;
    for (uint32_t g = 0; g < k / group; ++g) {
      float part = 0.0f;
      for (uint32_t l = g * group; l < (g + 1) * group; ++l)
        part = fmaf(load_as_f32(x, x_dtype, (size_t)i * x_ld + l), (float)int4_of((uint8_t)q[(size_t)(l / 2) * n + col], l & 1), part);
      acc = fmaf(part, scale[(size_t)g * n + col], acc);
    }
    return e.bias ? acc + e.bias[col] : acc;
  };
  float acc = column(j);
  size_t o = (size_t)i * e.out_ld + j;
  if (glu) {
    acc = silu_ref(acc) * column(j + 1);
    o = (size_t)i * e.out_ld + t;
  } else if (e.act == ACT_GELU) acc = gelu_ref(acc);
  if (e.resid) acc = e.resid[o] + acc;
  store_from_f32(out, e.out_dtype, o, acc);
}

template <int BITS, int MT>
cudaError_t launch_one(ruai_ctx* c, const GemvParams& p, dim3 grid) {
  return ruai_launch(c, gemv_kernel<BITS, MT>, grid, dim3(kThreads), (size_t)MT * kStageK * sizeof(float), true, p);
}

template <int BITS>
cudaError_t launch_mt(ruai_ctx* c, const GemvParams& p, dim3 grid, int mt) {
  switch (mt) {
    case 1: return launch_one<BITS, 1>(c, p, grid);
    case 2: return launch_one<BITS, 2>(c, p, grid);
    case 4: return launch_one<BITS, 4>(c, p, grid);
    case 8: return launch_one<BITS, 8>(c, p, grid);
    default: return launch_one<BITS, 16>(c, p, grid);
  }
}

}  // namespace

int ruai_gemv_launch(ruai_ctx* c, const ruai_qweight* w, const void* x, int x_dtype, uint32_t x_ld, uint32_t m, void* out,
                     const GemvEpilogue& epi_in, const GemvPrologue& pro) {
  if (m == 0) return RUAI_OK;
  if (c->use_bulk && c->use_tc && ruai_gemm_tc_eligible(w, m) && !epi_in.sumsq && !epi_in.argmax_out)
    return ruai_gemm_tc_launch(c, w, x, x_dtype, x_ld, m, out, epi_in, pro);
  if (c->use_bulk && c->use_tc && ruai_gemv_wide_eligible(c, w, m)) return ruai_gemv_wide_launch(c, w, x, x_dtype, x_ld, m, out, epi_in, pro);
  if (c->use_bulk && c->use_tc && ruai_gemv_tc8_eligible(w, m) && !(epi_in.argmax_out && m > 8)) return ruai_gemv_tc8_launch(c, w, x, x_dtype, x_ld, m, out, epi_in, pro);
  if (c->use_bulk && c->use_tc && ruai_gemv_tc_eligible(w, m)) return ruai_gemv_tc_launch(c, w, x, x_dtype, x_ld, m, out, epi_in, pro);
  if (c->use_bulk && ruai_gemv_bulk_eligible(w)) return ruai_gemv_bulk_launch(c, w, x, x_dtype, x_ld, m, out, epi_in, pro);
  GemvEpilogue epi = epi_in;
  if (epi.act == ACT_SWIGLU && (w->n & 1)) return ruai_fail(c, RUAI_ERR_SHAPE, "SwiGLU epilogue needs an even column count, got %u", w->n);
  if (epi.out_ld == 0) epi.out_ld = epi.act == ACT_SWIGLU ? w->n / 2 : w->n;
  if (w->layout == QL_REFERENCE) {
    if (pro.norm_w || epi.sumsq || epi.argmax_out) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "fused norm / argmax on a reference-layout weight");
    if (m > 65535) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "m too large");
    RUAI_CUDA(c, ruai_launch(c, gemv_int4_reference_layout_kernel, dim3((w->n + 127) / 128, m), dim3(128), 0, true, (const int8_t*)w->data,
                             (const float*)w->scale, x, x_dtype, x_ld, m, w->k, w->n, w->group, out, epi));
    return RUAI_OK;
  }
  const int mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16;
  const uint32_t row_tiles = (m + mt - 1) / mt;
  const uint32_t col_tiles = (w->n + kThreads - 1) / kThreads;
  if (row_tiles > 65535) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "m too large");
  // enough CTAs for three per SM, but at least kAhead chunks per split
  const uint32_t want = (uint32_t)c->sm_count * 3u;
  uint32_t splits = (want + col_tiles * row_tiles - 1) / (col_tiles * row_tiles);
  const uint32_t max_splits = (w->chunks + kAhead - 1) / kAhead;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  uint32_t cps = (w->chunks + splits - 1) / splits;
  cps = (cps + kAhead - 1) / kAhead * kAhead;  // keeps stage boundaries aligned with the prefetch ring
  splits = (w->chunks + cps - 1) / cps;
  GemvParams p;
  p.w = (const uint4*)w->data; p.scale = w->scale; p.x = x; p.x_dtype = x_dtype; p.x_ld = x_ld;
  p.m = m; p.k = w->k; p.n = w->n; p.chunks = w->chunks; p.chunks_per_split = cps; p.splits = splits;
  p.out = out; p.epi = epi; p.pro = pro;
  if (epi.argmax_out && (row_tiles != 1 || epi.act == ACT_SWIGLU)) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "fused argmax needs m <= 16");
  if (epi.sumsq && epi.act == ACT_SWIGLU) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "sum of squares with the SwiGLU epilogue");
  if (splits > 1) RUAI_TRY(ruai_ctx_reserve(c, (size_t)splits * m * w->n * sizeof(float), (size_t)col_tiles * row_tiles));
  p.partial = c->partial; p.counters = c->counters;
  const dim3 grid(col_tiles, splits, row_tiles);
  cudaError_t e = w->bits == 8 ? launch_mt<8>(c, p, grid, mt) : launch_mt<4>(c, p, grid, mt);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "gemv launch failed: %s", cudaGetErrorString(e));
  return RUAI_OK;
}

size_t ruai_gemv_xs_bytes(const ruai_qweight* w, uint32_t m) {
  const size_t groups = (w->k + 31) / 32;
  // up to 16 rows: one 16-row tile, 2 KB per group, whole 64-k tiles; beyond: 16 KB per group and block of 128 rows
  return m <= 16 ? ((groups + 1) & ~(size_t)1) * 2048 : (size_t)((m + 127) / 128) * groups * 16384;
}

uint32_t ruai_gemv_tiles(const ruai_ctx* c, const ruai_qweight* w) {
  const uint32_t t = c->use_bulk && ruai_gemv_bulk_eligible(w) ? kGemvBulkTileCols : kGemvTileCols;
  return (w->n + t - 1) / t;
}

// Backend::matmul_int8 / matmul_int4 (mod.rs:675-704) + Linear::forward's bias (layers.rs:184-189).
RUAI_API int ruai_matmul_q(ruai_ctx* c, int x_dtype, const void* x, const ruai_qweight* w, const float* bias, void* out, uint32_t m) {
  if (!c || !w || (m && (!x || !out))) return ruai_fail(c, RUAI_ERR_ARG, "ruai_matmul_q: NULL argument");
  if (x_dtype != RUAI_F32 && x_dtype != RUAI_F16 && x_dtype != RUAI_BF16) return ruai_fail(c, RUAI_ERR_ARG, "ruai_matmul_q: bad dtype %d", x_dtype);
  if (w->ctx != c) return ruai_fail(c, RUAI_ERR_ARG, "ruai_matmul_q: weight belongs to another context");
  DeviceGuard g(c->ordinal);
  GemvEpilogue e;
  e.bias = bias;
  e.out_dtype = x_dtype;
  return ruai_gemv_launch(c, w, x, x_dtype, w->k, m, out, e);
}

// ---------------------------------------------------------------------------------------
// Quantized matmul for callers that must not allocate.
//
// Some hosts of this library cannot let it call cudaMalloc at run time: a serving process
// whose framework has already claimed the whole device for its own caching allocator (a
// later cudaMalloc simply fails), or a latency-critical loop in which the implicit device
// synchronisation of cudaMalloc / cudaFree is not acceptable.  ruai_matmul_q grows the
// context's split-K scratch on demand; this variant instead keeps its split-K scratch in a
// fixed array that is part of the loaded module, so it never allocates.
//
// The array costs kStaticScratchBytes (8 MiB + 16 KiB) of device memory on every GPU that
// loads the library, from load until exit.  All calls on a device share it, and it keeps
// whatever the last call left: the arrival counters are cleared on the stream before every
// launch, the partial sums are always written before they are read.  Two calls that overlap
// on the GPU (different streams or contexts on one device) would race on it.
namespace {

constexpr size_t kStaticCounters = 4096;                                 // column tiles x row tiles
constexpr size_t kStaticPartialBytes = 8u << 20;                         // split-K partial sums
constexpr size_t kStaticScratchBytes = kStaticCounters * sizeof(unsigned) + kStaticPartialBytes;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device ordinal.  In host code the array's name is
// only a handle for the runtime, never an address a kernel may be given.
static void* g_static_scratch_addr[kMaxDevices] = {};

}  // namespace

RUAI_API int ruai_matmul_q_static(ruai_ctx* c, int x_dtype, const void* x, const ruai_qweight* w, const float* bias, void* out, uint32_t m) {
  if (!c || !w || (m && (!x || !out))) return ruai_fail(c, RUAI_ERR_ARG, "ruai_matmul_q_static: NULL argument");
  if (x_dtype != RUAI_F32 && x_dtype != RUAI_F16 && x_dtype != RUAI_BF16) return ruai_fail(c, RUAI_ERR_ARG, "ruai_matmul_q_static: bad dtype %d", x_dtype);
  if (w->ctx != c) return ruai_fail(c, RUAI_ERR_ARG, "ruai_matmul_q_static: weight belongs to another context");
  if (w->layout != QL_CHUNK16) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "ruai_matmul_q_static: int4 weights need group 32");
  if (c->ordinal < 0 || c->ordinal >= kMaxDevices) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "ruai_matmul_q_static: device ordinal %d", c->ordinal);
  if (m == 0) return RUAI_OK;
  DeviceGuard g(c->ordinal);
  // set-up, once per device, with that device current: ask the runtime where the array lives
  if (!g_static_scratch_addr[c->ordinal]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) return ruai_fail(c, RUAI_ERR_CUDA, "ruai_matmul_q_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_static_scratch_addr[c->ordinal] = p;
  }
  unsigned char* base = (unsigned char*)g_static_scratch_addr[c->ordinal];
  // the work split of the first-generation kernel: the same bits as ruai_matmul_q gives when the tensor-core and bulk-copy
  // kernels are off (RUAI_B200_TC=0, RUAI_B200_BULK=0); against the default dispatch the results agree within the
  // GPU-vs-CPU tolerance (other activation rounding, other order of the partial sums)
  const int mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16;
  const uint32_t row_tiles = (m + mt - 1) / mt;
  const uint32_t col_tiles = (w->n + kThreads - 1) / kThreads;
  if (row_tiles > 65535) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "m too large");
  const uint32_t want = (uint32_t)c->sm_count * 3u;
  uint32_t splits = (want + col_tiles * row_tiles - 1) / (col_tiles * row_tiles);
  const uint32_t max_splits = (w->chunks + kAhead - 1) / kAhead;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  uint32_t cps = (w->chunks + splits - 1) / splits;
  cps = (cps + kAhead - 1) / kAhead * kAhead;
  splits = (w->chunks + cps - 1) / cps;
  const size_t need_partial = splits > 1 ? (size_t)splits * m * w->n * sizeof(float) : 0;
  const size_t need_counters = splits > 1 ? (size_t)col_tiles * row_tiles : 0;
  if (need_partial > kStaticPartialBytes || need_counters > kStaticCounters)
    return ruai_fail(c, RUAI_ERR_UNSUPPORTED,
                     "ruai_matmul_q_static: m=%u x n=%u needs %zu bytes of split-K scratch and %zu counters; the fixed scratch holds %zu bytes and %zu "
                     "counters (use ruai_matmul_q, which allocates)",
                     m, w->n, need_partial, need_counters, kStaticPartialBytes, kStaticCounters);
  GemvParams p;
  p.w = (const uint4*)w->data; p.scale = w->scale; p.x = x; p.x_dtype = x_dtype; p.x_ld = w->k;
  p.m = m; p.k = w->k; p.n = w->n; p.chunks = w->chunks; p.chunks_per_split = cps; p.splits = splits;
  p.out = out;
  p.epi = GemvEpilogue();
  p.pro = GemvPrologue();
  p.epi.bias = bias;
  p.epi.out_dtype = x_dtype;
  p.epi.out_ld = w->n;
  p.counters = (unsigned*)base;
  p.partial = (float*)(base + kStaticCounters * sizeof(unsigned));
  if (need_counters) RUAI_CUDA(c, cudaMemsetAsync(p.counters, 0, need_counters * sizeof(unsigned), c->stream));
  const dim3 grid(col_tiles, splits, row_tiles);
  cudaError_t e = w->bits == 8 ? launch_mt<8>(c, p, grid, mt) : launch_mt<4>(c, p, grid, mt);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "ruai_matmul_q_static: launch failed: %s", cudaGetErrorString(e));
  return RUAI_OK;
}
