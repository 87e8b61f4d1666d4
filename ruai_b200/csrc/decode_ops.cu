// The non-matmul kernels of one decode / prefill step: embedding gather, RMSNorm and
// LayerNorm, RoPE + KV-cache append, attention over the cache, greedy argmax.
//
// They replace the chains of generic elementwise launches the reference's CUDA
// backend issues for the same functions (binary_*/unary_*/reduce_rows_*/cat_copy_*/
// softmax_rows in src/nn/backend/cuda_kernels.cu, driven by src/nn/functional.rs) and
// the host round trips around them (rope tables rebuilt and uploaded every step,
// functional.rs:176-192; logits copied out for the host argmax, generation.rs:104).
// Positions and token ids are read from device memory so that a captured graph of
// the step can be replayed without host involvement.
#include "decode_ops.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// Sum over the CTA (blockDim.x <= 1024, multiple of 32); every thread gets the result.
__device__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.0f;
  for (int i = 0; i < nw; ++i) t += red[i];  // fixed order: deterministic
  return t;
}

// Embedding::forward (layers.rs:436-446); GPT-2 adds wpe[pos] (gpt2.rs:225-226).
// Row r = b*T + t; position = *len + t.
__global__ void embed_kernel(const int32_t* __restrict__ ids, const float* __restrict__ embed, const float* __restrict__ wpe,
                             const int32_t* __restrict__ len, uint32_t T, uint32_t d, uint32_t vocab, float* __restrict__ x,
                             int* __restrict__ err) {
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t r = blockIdx.x;
  int32_t id = ids[r];
  if (id < 0 || (uint32_t)id >= vocab) {  // the reference's index_select would panic; flag it and stay in bounds
    if (threadIdx.x == 0) atomicExch(err, 1);
    id = 0;
  }
  const float* e = embed + (size_t)id * d;
  const float* p = wpe ? wpe + (size_t)(*len + (r % T)) * d : nullptr;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) x[(size_t)r * d + i] = p ? e[i] + p[i] : e[i];
}

// F::rms_norm (functional.rs:151-165): x * (1/sqrt(sum(x^2) * (1/d) + eps)) * w.
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, uint32_t d, float eps, float* __restrict__ y) {
  __shared__ float red[32];
  grid_dependency_wait();
  grid_launch_dependents();
  const float* xr = x + (size_t)blockIdx.x * d;
  float s = 0.0f;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) s = fmaf(xr[i], xr[i], s);
  s = block_sum(s, red);
  const float rstd = 1.0f / sqrtf(s * (1.0f / (float)d) + eps);
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) y[(size_t)blockIdx.x * d + i] = xr[i] * rstd * w[i];
}

// F::layer_norm (functional.rs:137-146) over cpu.rs:855-876: two-pass mean, biased variance.
__global__ void layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, uint32_t d, float eps,
                                  float* __restrict__ y) {
  __shared__ float red[32];
  grid_dependency_wait();
  grid_launch_dependents();
  const float* xr = x + (size_t)blockIdx.x * d;
  float s = 0.0f;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) s += xr[i];
  const float mean = block_sum(s, red) / (float)d;
  float v = 0.0f;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) v = fmaf(xr[i] - mean, xr[i] - mean, v);
  const float rstd = 1.0f / sqrtf(block_sum(v, red) / (float)d + eps);
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) y[(size_t)blockIdx.x * d + i] = (xr[i] - mean) * rstd * w[i] + b[i];
}

// rope_cos_sin (functional.rs:176-192): angle = pos * inv_freq in f64, cos/sin rounded to f32.
// table[pos][i] = (cos, sin), i < hd/2.
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, uint32_t half, uint32_t max_pos, float2* __restrict__ table) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)max_pos * half) return;
  const uint32_t pos = (uint32_t)(idx / half), i = (uint32_t)(idx % half);
  const double a = (double)pos * (double)inv_freq[i];
  double s, c;
  sincos(a, &s, &c);
  table[idx] = make_float2((float)c, (float)s);
}

// apply_rope (functional.rs:197-204) on q in place and on k while appending k, v to the
// cache (KvBuf::append, transformer.rs:27-53).  qkv row layout: [q heads | k heads | v heads].
// grid (B*T, Hq + KV); thread i < hd/2 handles the pair (i, i + hd/2).
__global__ void rope_kv_kernel(float* __restrict__ qkv, uint32_t qkv_ld, uint32_t k_off, uint32_t v_off, const float2* __restrict__ table,
                               const int32_t* __restrict__ len, uint32_t T, uint32_t Hq, uint32_t KV, uint32_t hd, uint32_t cap,
                               float* __restrict__ kcache, float* __restrict__ vcache) {
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t r = blockIdx.x, b = r / T, t = r % T, head = blockIdx.y, half = hd / 2;
  const uint32_t pos = (uint32_t)*len + t;
  float* row = qkv + (size_t)r * qkv_ld;
  if (head < Hq) {
    if (!table) return;
    float* q = row + (size_t)head * hd;
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
      const float2 cs = table[(size_t)pos * half + i];
      const float x1 = q[i], x2 = q[i + half];
      q[i] = x1 * cs.x + (-x2) * cs.y;
      q[i + half] = x2 * cs.x + x1 * cs.y;
    }
  } else {
    const uint32_t h = head - Hq;
    const float* k = row + k_off + (size_t)h * hd;
    const float* v = row + v_off + (size_t)h * hd;
    float* kd = kcache + (((size_t)b * KV + h) * cap + pos) * hd;
    float* vd = vcache + (((size_t)b * KV + h) * cap + pos) * hd;
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
      const float x1 = k[i], x2 = k[i + half];
      if (table) {
        const float2 cs = table[(size_t)pos * half + i];
        kd[i] = x1 * cs.x + (-x2) * cs.y;
        kd[i + half] = x2 * cs.x + x1 * cs.y;
      } else {
        kd[i] = x1;
        kd[i + half] = x2;
      }
      vd[i] = v[i];
      vd[i + half] = v[i + half];
    }
  }
}

// scaled_dot_product_attention over the cache (functional.rs:264-296, llama.rs:248-277):
// softmax(q k^T / sqrt(hd) + causal mask) v.  The `rep` query heads of one KV head are
// handled together so the cached rows are read once (the reference's
// [B, H_kv, rep*T, hd] view, llama.rs:264-268).  Keys are split over gridDim.z CTAs and
// over the warps of a CTA; each keeps an online-softmax state (max, sum, weighted V)
// and the states are merged at the end: within the CTA through shared memory, across
// CTAs by the last one to arrive.
template <int EPL, int REP>
__global__ void __launch_bounds__(128) attention_kernel(const AttnParams p) {
  constexpr int kWarps = 4;
  extern __shared__ float sm[];  // q [REP][hd] | merge [kWarps][REP][hd + 2]
  __shared__ unsigned s_last;
  const uint32_t hd = p.hd;
  float* qs = sm;
  float* mg = sm + REP * hd;
  const uint32_t bk = blockIdx.x, b = bk / p.KV, kvh = bk % p.KV, t = blockIdx.y, split = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t past = (uint32_t)*p.len;
  const uint32_t n_keys = past + t + 1;  // causal_mask_offset, functional.rs:238-247
  const uint32_t per = (n_keys + gridDim.z - 1) / gridDim.z;
  const uint32_t k0 = split * per, k1 = min(n_keys, k0 + per);
  const float* qrow = p.q + (size_t)(b * p.T + t) * p.q_ld + (size_t)kvh * REP * hd;
  for (uint32_t i = threadIdx.x; i < REP * hd; i += blockDim.x) qs[i] = qrow[i];
  __syncthreads();
  const float* kbase = p.kcache + ((size_t)b * p.KV + kvh) * p.cap * hd;
  const float* vbase = p.vcache + ((size_t)b * p.KV + kvh) * p.cap * hd;
  float mx[REP], l[REP], o[REP][EPL];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    mx[r] = -INFINITY;
    l[r] = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) o[r][i] = 0.0f;
  }
  for (uint32_t key = k0 + warp; key < k1; key += kWarps) {
    float kv[EPL], vv[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const uint32_t e = lane + 32 * i;
      kv[i] = e < hd ? kbase[(size_t)key * hd + e] : 0.0f;
      vv[i] = e < hd ? vbase[(size_t)key * hd + e] : 0.0f;
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float s = 0.0f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const uint32_t e = lane + 32 * i;
        if (e < hd) s = fmaf(qs[r * hd + e], kv[i], s);
      }
      s = warp_sum(s) * p.scale;
      const float nm = fmaxf(mx[r], s);
      const float c = expf(mx[r] - nm);  // exp(-inf) = 0 on the first key
      const float pr = expf(s - nm);
      l[r] = l[r] * c + pr;
#pragma unroll
      for (int i = 0; i < EPL; ++i) o[r][i] = o[r][i] * c + pr * vv[i];
      mx[r] = nm;
    }
  }
  // ---- merge the warps ----
  const uint32_t stride = hd + 2;
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    float* dst = mg + ((size_t)warp * REP + r) * stride;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const uint32_t e = lane + 32 * i;
      if (e < hd) dst[e] = o[r][i];
    }
    if (lane == 0) { dst[hd] = mx[r]; dst[hd + 1] = l[r]; }
  }
  __syncthreads();
  const uint32_t rows = REP, total = rows * hd;
  float* sc = p.scratch + ((((size_t)bk * p.T + t) * gridDim.z + split) * REP) * stride;
  for (uint32_t idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const uint32_t r = idx / hd, e = idx % hd;
    float M = -INFINITY;
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, mg[((size_t)w * REP + r) * stride + hd]);
    float L = 0.0f, O = 0.0f;
    for (int w = 0; w < kWarps; ++w) {
      const float* src = mg + ((size_t)w * REP + r) * stride;
      const float c = src[hd] == -INFINITY ? 0.0f : expf(src[hd] - M);
      L += src[hd + 1] * c;
      O += src[e] * c;
    }
    if (gridDim.z == 1) {
      p.out[(size_t)(b * p.T + t) * p.out_ld + ((size_t)kvh * REP + r) * hd + e] = O / L;
    } else {
      sc[(size_t)r * stride + e] = O;
      if (e == 0) { sc[(size_t)r * stride + hd] = M; sc[(size_t)r * stride + hd + 1] = L; }
    }
  }
  if (gridDim.z == 1) return;
  // ---- merge the key splits: last CTA to arrive ----
  __threadfence();
  __syncthreads();
  unsigned* counter = p.counters + (size_t)bk * p.T + t;
  if (threadIdx.x == 0) {
    const unsigned a = atomicAdd(counter, 1u);
    s_last = a == gridDim.z - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x == 0) *counter = 0;
  const float* base = p.scratch + (((size_t)bk * p.T + t) * gridDim.z) * REP * stride;
  for (uint32_t idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const uint32_t r = idx / hd, e = idx % hd;
    float M = -INFINITY;
    for (uint32_t s = 0; s < gridDim.z; ++s) M = fmaxf(M, __ldcg(base + ((size_t)s * REP + r) * stride + hd));
    float L = 0.0f, O = 0.0f;
    for (uint32_t s = 0; s < gridDim.z; ++s) {
      const float* src = base + ((size_t)s * REP + r) * stride;
      const float ms = __ldcg(src + hd);
      const float c = ms == -INFINITY ? 0.0f : expf(ms - M);
      L += __ldcg(src + hd + 1) * c;
      O += __ldcg(src + e) * c;
    }
    p.out[(size_t)(b * p.T + t) * p.out_ld + ((size_t)kvh * REP + r) * hd + e] = O / L;
  }
}

// generation::argmax (generation.rs:6-8): the LAST index among equal maxima, in
// total_cmp order (sign-magnitude bits mapped to a signed integer order).
__device__ __forceinline__ int32_t total_order(float v) {
  int32_t i = __float_as_int(v);
  return i ^ (int32_t)(((uint32_t)(i >> 31)) >> 1);
}
__global__ void argmax_kernel(const float* __restrict__ logits, uint32_t ld, uint32_t n, int32_t* __restrict__ out, uint32_t out_offset) {
  __shared__ int32_t sv[32];
  __shared__ uint32_t si[32];
  grid_dependency_wait();
  grid_launch_dependents();
  const float* row = logits + (size_t)blockIdx.x * ld;
  int32_t bv = INT32_MIN;
  uint32_t bi = 0;
  bool any = false;
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
    const int32_t v = total_order(row[i]);
    if (!any || v >= bv) { bv = v; bi = i; any = true; }  // ascending i per thread: >= keeps the last
  }
  auto better = [](int32_t v, uint32_t i, bool a, int32_t bv2, uint32_t bi2, bool b2) {
    if (!b2) return false;
    if (!a) return true;
    return bv2 > v || (bv2 == v && bi2 > i);
  };
  for (int o = 16; o > 0; o >>= 1) {
    const int32_t ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
    const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
    const bool oa = __shfl_xor_sync(0xFFFFFFFFu, (int)any, o) != 0;
    if (better(bv, bi, any, ov, oi, oa)) { bv = ov; bi = oi; any = true; }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) { sv[w] = any ? bv : INT32_MIN; si[w] = any ? bi : 0xFFFFFFFFu; }
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t v = INT32_MIN;
    uint32_t idx = 0;
    bool a = false;
    for (int i = 0; i < nw; ++i) {
      if (si[i] == 0xFFFFFFFFu) continue;
      if (!a || sv[i] > v || (sv[i] == v && si[i] > idx)) { v = sv[i]; idx = si[i]; a = true; }
    }
    out[blockIdx.x] = (int32_t)(idx + out_offset);
  }
}

__global__ void add_scalar_kernel(int32_t* p, int32_t v) {
  grid_dependency_wait();
  grid_launch_dependents();
  if (threadIdx.x == 0 && blockIdx.x == 0) *p += v;
}

// Copies rows (b*T + T-1) of x [B*T, d] to y [B, d].
__global__ void take_last_rows_kernel(const float* __restrict__ x, uint32_t T, uint32_t d, float* __restrict__ y) {
  grid_dependency_wait();
  grid_launch_dependents();
  const float* src = x + ((size_t)blockIdx.x * T + T - 1) * d;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) y[(size_t)blockIdx.x * d + i] = src[i];
}

template <int EPL>
cudaError_t launch_attn_rep(ruai_ctx* c, const AttnParams& p, dim3 grid, size_t smem, uint32_t rep) {
  switch (rep) {
    case 1: return ruai_launch(c, attention_kernel<EPL, 1>, grid, dim3(128), smem, true, p);
    case 2: return ruai_launch(c, attention_kernel<EPL, 2>, grid, dim3(128), smem, true, p);
    case 3: return ruai_launch(c, attention_kernel<EPL, 3>, grid, dim3(128), smem, true, p);
    case 4: return ruai_launch(c, attention_kernel<EPL, 4>, grid, dim3(128), smem, true, p);
    case 8: return ruai_launch(c, attention_kernel<EPL, 8>, grid, dim3(128), smem, true, p);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

int ruai_embed(ruai_ctx* c, const int32_t* ids, const float* embed, const float* wpe, const int32_t* len, uint32_t rows, uint32_t T, uint32_t d,
               uint32_t vocab, float* x, int* err) {
  RUAI_CUDA(c, ruai_launch(c, embed_kernel, dim3(rows), dim3(256), 0, true, ids, embed, wpe, len, T, d, vocab, x, err));
  return RUAI_OK;
}

int ruai_rms_norm(ruai_ctx* c, const float* x, const float* w, uint32_t rows, uint32_t d, float eps, float* y) {
  RUAI_CUDA(c, ruai_launch(c, rms_norm_kernel, dim3(rows), dim3(d >= 2048 ? 512 : 256), 0, true, x, w, d, eps, y));
  return RUAI_OK;
}

int ruai_layer_norm(ruai_ctx* c, const float* x, const float* w, const float* b, uint32_t rows, uint32_t d, float eps, float* y) {
  RUAI_CUDA(c, ruai_launch(c, layer_norm_kernel, dim3(rows), dim3(256), 0, true, x, w, b, d, eps, y));
  return RUAI_OK;
}

int ruai_rope_table(ruai_ctx* c, const float* inv_freq, uint32_t half, uint32_t max_pos, float2* table) {
  const size_t total = (size_t)max_pos * half;
  rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, c->stream>>>(inv_freq, half, max_pos, table);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

int ruai_rope_kv(ruai_ctx* c, float* qkv, uint32_t qkv_ld, uint32_t k_off, uint32_t v_off, const float2* table, const int32_t* len, uint32_t rows,
                 uint32_t T, uint32_t Hq, uint32_t KV, uint32_t hd, uint32_t cap, float* kcache, float* vcache) {
  const unsigned threads = hd / 2 >= 64 ? 64 : 32;
  RUAI_CUDA(c, ruai_launch(c, rope_kv_kernel, dim3(rows, Hq + KV), dim3(threads), 0, true, qkv, qkv_ld, k_off, v_off, table, len, T, Hq, KV, hd, cap,
                           kcache, vcache));
  return RUAI_OK;
}

int ruai_attention(ruai_ctx* c, const AttnParams& p, uint32_t B, uint32_t rep, uint32_t splits) {
  const uint32_t epl = (p.hd + 31) / 32;
  const size_t smem = ((size_t)rep * p.hd + 4 * (size_t)rep * (p.hd + 2)) * sizeof(float);
  const dim3 grid(B * p.KV, p.T, splits);
  cudaError_t e;
  if (epl <= 1) e = launch_attn_rep<1>(c, p, grid, smem, rep);
  else if (epl <= 2) e = launch_attn_rep<2>(c, p, grid, smem, rep);
  else if (epl <= 4) e = launch_attn_rep<4>(c, p, grid, smem, rep);
  else if (epl <= 8) e = launch_attn_rep<8>(c, p, grid, smem, rep);
  else return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "head_dim %u > 256", p.hd);
  if (e != cudaSuccess) return ruai_fail(c, e == cudaErrorInvalidValue ? RUAI_ERR_UNSUPPORTED : RUAI_ERR_CUDA,
                                         "attention launch (heads per KV head = %u): %s", rep, cudaGetErrorString(e));
  return RUAI_OK;
}

int ruai_argmax(ruai_ctx* c, const float* logits, uint32_t ld, uint32_t rows, uint32_t n, int32_t* out, uint32_t out_offset) {
  RUAI_CUDA(c, ruai_launch(c, argmax_kernel, dim3(rows), dim3(1024), 0, true, logits, ld, n, out, out_offset));
  return RUAI_OK;
}

int ruai_add_scalar(ruai_ctx* c, int32_t* p, int32_t v) {
  RUAI_CUDA(c, ruai_launch(c, add_scalar_kernel, dim3(1), dim3(32), 0, true, p, v));
  return RUAI_OK;
}

int ruai_take_last_rows(ruai_ctx* c, const float* x, uint32_t B, uint32_t T, uint32_t d, float* y) {
  RUAI_CUDA(c, ruai_launch(c, take_last_rows_kernel, dim3(B), dim3(256), 0, true, x, T, d, y));
  return RUAI_OK;
}
