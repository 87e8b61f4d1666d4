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
#include <algorithm>

#include "decode_ops.cuh"
#include "pipeline.cuh"

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
                             int* __restrict__ err, float* __restrict__ sumsq) {
  __shared__ float red[32];
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
  float ss = 0.0f;
  for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = p ? e[i] + p[i] : e[i];
    x[(size_t)r * d + i] = v;
    ss = fmaf(v, v, ss);
  }
  if (sumsq) {  // one tile per row: the sum of squares the next RMSNorm needs
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) sumsq[r] = ss;
  }
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
                               float* __restrict__ kcache, float* __restrict__ vcache, int* __restrict__ status) {
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
    if (pos >= cap) {  // never write past the cache (see attention_kernel)
      if (threadIdx.x == 0 && status) atomicCAS(status, 0, 5);
      return;
    }
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
// handled by one CTA so the cached rows are read once (the reference's [B, H_kv, rep*T, hd]
// view, llama.rs:264-268).  Keys are split over gridDim.z CTAs; a CTA brings its keys and
// values into shared memory with bulk copies, 64 at a time, requested before the
// grid-dependency wait in the fused step.
//   scores : warp (block of 32 keys, head): one key per lane, the lane walks its key row
//            starting at its own 16-byte column (no bank conflicts, no cross-lane sums);
//            block maximum and sum by shuffles.
//   values : thread (head, element): sums p * V over the chunk's keys, rows read conflict-free.
// Every thread keeps a running (max, sum, weighted value) for its outputs across chunks; the
// splits are merged by the last CTA to arrive.
// With p.fuse (single new token per sequence) the kernel also does apply_rope
// (functional.rs:197-204) on q and on the new key and appends the new key / value to the
// cache (KvBuf::append, transformer.rs:27-53): the last key split owns the new position.

// SUB: warps per (32 keys, query head).  2 (more warps than the work needs, to hide each other's latencies) for grids of
// about one CTA per SM; 1 for large grids, where two or three smaller CTAs per SM hide them instead.
template <int REP, int SUB>
__global__ void __launch_bounds__(kAttnChunkKeys * REP * SUB) attention_kernel(const AttnParams p) {
  constexpr int kThreads = kAttnChunkKeys * REP * SUB, kBlocks = kAttnChunkKeys / 32, kParts = REP * SUB;
  extern __shared__ __align__(128) float sm[];  // K chunk | V chunk | q [REP][hd] | new k | new v | probs | stats | parts | merge
  __shared__ __align__(8) uint64_t kv_bar;
  __shared__ unsigned s_last;
  const uint32_t hd = p.hd, half = hd / 2;
  float* ks = sm;
  float* vs = ks + (size_t)kAttnChunkKeys * hd;
  float* qs = vs + (size_t)kAttnChunkKeys * hd;
  float* knew = qs + REP * hd;
  float* vnew = knew + hd;
  float* probs = vnew + hd;                       // [kBlocks][REP][32]
  float* bmax = probs + kBlocks * REP * 32;       // [kBlocks + 1][REP]: block maxima; the last row is the new key's score
  float* bsum = bmax + (kBlocks + 1) * REP;       // [kBlocks][REP]
  float* part = bsum + kBlocks * REP;             // [kParts][REP heads][64 keys] partial scores
  float* mg = part + kParts * REP * kAttnChunkKeys;  // split merge: [64][REP] weights, [64][REP] sums, [REP]
  const uint32_t bk = blockIdx.x, b = bk / p.KV, kvh = bk % p.KV, t = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* kbase = p.kcache + ((size_t)b * p.KV + kvh) * p.cap * hd;
  float* vbase = p.vcache + ((size_t)b * p.KV + kvh) * p.cap * hd;
  if (tid == 0) {
    pipe::mbar_init(&kv_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  uint32_t past = 0, pos = 0, n_keys = 0, n_cached = 0, k0 = 0, k1 = 0;
  bool over = false;
  auto plan = [&]() {
    past = (uint32_t)*p.len;
    pos = past + t;
    n_keys = pos + 1;  // causal_mask_offset, functional.rs:238-247
    n_cached = p.fuse ? n_keys - 1 : n_keys;
    // The host grows the cache before the step, so a position at or past the capacity means the device's position
    // word is not the host's: touch nothing of the cache, leave an error for the host (the step's output is void).
    over = pos >= p.cap;
    if (over) n_cached = 0;
    const uint32_t per = (n_cached + gridDim.z - 1) / gridDim.z;
    k0 = min(n_cached, split * per);
    k1 = min(n_cached, k0 + per);
  };
  auto fetch_chunk = [&](uint32_t c0) {  // one thread
    const uint32_t nk = min((uint32_t)kAttnChunkKeys, k1 - c0);
    const uint32_t bytes = nk * hd * 4u;
    pipe::mbar_expect_tx(&kv_bar, 2u * bytes);
    pipe::bulk_load(ks, kbase + (size_t)c0 * hd, bytes, &kv_bar);
    pipe::bulk_load(vs, vbase + (size_t)c0 * hd, bytes, &kv_bar);
  };
  // In the fused single-token step the cached rows were written by earlier steps, and the position by the
  // previous step's last kernel: both are safe to read while the predecessor (the q/k/v GEMV) still runs.
  if (p.fuse) {
    plan();
    if (tid == 0 && k1 > k0) fetch_chunk(k0);
  }
  if (tid == 0) trace_min(p.trace, 0);
  grid_dependency_wait();
  if (tid == 0) trace_min(p.trace, 1);
  grid_launch_dependents();
  if (!p.fuse) {
    plan();
    if (tid == 0 && k1 > k0) fetch_chunk(k0);
  }
  const bool owns_new = p.fuse && split == gridDim.z - 1;
  if (over && tid == 0 && p.status) atomicCAS(p.status, 0, 5);
  const float* row = p.q + (size_t)(b * p.T + t) * p.q_ld;
  const float* qrow = row + (size_t)kvh * REP * hd;
  const bool rot = p.fuse && p.table != nullptr;
  for (uint32_t i = tid; i < REP * hd; i += kThreads) {
    float v = qrow[i];
    if (rot) {
      const uint32_t r = i / hd, e = i % hd, f = e < half ? e : e - half;
      const float2 cs = p.table[(size_t)pos * half + f];
      const float x1 = qrow[r * hd + f], x2 = qrow[r * hd + f + half];
      v = e < half ? x1 * cs.x + (-x2) * cs.y : x2 * cs.x + x1 * cs.y;
    }
    qs[i] = v;
  }
  if (owns_new) {
    const float* kr = row + p.k_off + (size_t)kvh * hd;
    const float* vr = row + p.v_off + (size_t)kvh * hd;
    for (uint32_t e = tid; e < hd; e += kThreads) {
      float kvv = kr[e];
      if (rot) {
        const uint32_t f = e < half ? e : e - half;
        const float2 cs = p.table[(size_t)pos * half + f];
        const float x1 = kr[f], x2 = kr[f + half];
        kvv = e < half ? x1 * cs.x + (-x2) * cs.y : x2 * cs.x + x1 * cs.y;
      }
      const float vv = vr[e];
      knew[e] = kvv;
      vnew[e] = vv;
      if (!over) {
        kbase[(size_t)pos * hd + e] = kvv;
        vbase[(size_t)pos * hd + e] = vv;
      }
    }
  }
  __syncthreads();
  // ---- thread roles ----
  // partial scores: warp (key block, part of the head dimension), lane = key, all REP heads at once
  // softmax stats : warp (key block, head), lane = key
  // values        : thread (key group, head, 4 consecutive elements)
  const uint32_t nq4 = hd / 4;
  const int wblk = warp / kParts, wpart = warp % kParts, wr = wpart;  // wr: the head, for the warps with wpart < REP
  const uint32_t cper = (nq4 + kParts - 1) / kParts;
  const uint32_t c_lo = min(nq4, (uint32_t)wpart * cper), c_hi = min(nq4, c_lo + cper), ncols = c_hi - c_lo;
  const uint32_t vthreads = REP * nq4;                 // threads that cover one full set of outputs
  const uint32_t G = max(1u, (uint32_t)kThreads / vthreads);  // key groups in the value phase
  const uint32_t vg = tid / vthreads, vrem = tid % vthreads, vr = vrem / nq4, vc = vrem % nq4;
  const bool vact = (uint32_t)tid < G * vthreads;
  float run_m = -INFINITY, run_l = 0.0f;
  float4 run_o = make_float4(0.f, 0.f, 0.f, 0.f);
  uint32_t phase = 0;
  bool ok = true;
  for (uint32_t c0 = k0; c0 < k1 || (c0 == k0 && owns_new); c0 += kAttnChunkKeys) {
    const bool have_keys = c0 < k1;
    if (c0 != k0) {
      __syncthreads();  // everyone is done with the previous chunk
      if (tid == 0) fetch_chunk(c0);
    }
    if (have_keys) {
      // the whole CTA leaves together if the copy did not arrive for any of its threads: the barriers below are for all
      const bool got = pipe::mbar_wait(&kv_bar, phase & 1u);
      if (__syncthreads_or(!got)) { ok = false; break; }
      ++phase;
    }
    const uint32_t c1 = have_keys ? min(k1, c0 + kAttnChunkKeys) : c0;
    const uint32_t nkeys = c1 - c0;
    // ---- partial scores: this lane's key against this warp's columns of every head ----
    {
      const uint32_t key = wblk * 32 + lane;
      const float4* krow = reinterpret_cast<const float4*>(ks + (size_t)(key < nkeys ? key : 0) * hd);
      const float4* q4 = reinterpret_cast<const float4*>(qs);
      float acc[REP][2];
#pragma unroll
      for (int r = 0; r < REP; ++r) { acc[r][0] = 0.0f; acc[r][1] = 0.0f; }
      auto dot4 = [](const float4& a, const float4& b2, float s) {
        s = fmaf(a.x, b2.x, s); s = fmaf(a.y, b2.y, s); s = fmaf(a.z, b2.z, s); return fmaf(a.w, b2.w, s);
      };
      if (ncols > 0) {
        // each lane starts at its own column: the eight lanes of a quarter warp read eight different 16-byte columns
        uint32_t cc = c_lo + lane % ncols;
        uint32_t it = 0;
        for (; it + 2 <= ncols; it += 2) {
          const uint32_t ca = cc, cb = ca + 1 == c_hi ? c_lo : ca + 1;
          const float4 ka = krow[ca], kb = krow[cb];
#pragma unroll
          for (int r = 0; r < REP; ++r) {
            acc[r][0] = dot4(q4[r * nq4 + ca], ka, acc[r][0]);
            acc[r][1] = dot4(q4[r * nq4 + cb], kb, acc[r][1]);
          }
          cc = cb + 1 == c_hi ? c_lo : cb + 1;
        }
        if (it < ncols) {
          const float4 ka = krow[cc];
#pragma unroll
          for (int r = 0; r < REP; ++r) acc[r][0] = dot4(q4[r * nq4 + cc], ka, acc[r][0]);
        }
      }
#pragma unroll
      for (int r = 0; r < REP; ++r) part[(wpart * REP + r) * kAttnChunkKeys + key] = acc[r][0] + acc[r][1];
    }
    __syncthreads();
    // ---- scores of (key block, head): sum of the parts, block maximum and sum by shuffles ----
    if (wpart < REP) {
      const uint32_t key = wblk * 32 + lane;
      const bool valid = key < nkeys;
      float sc = 0.0f;
#pragma unroll
      for (int pt = 0; pt < kParts; ++pt) sc += part[(pt * REP + wr) * kAttnChunkKeys + key];
      const float sv = valid ? sc * p.scale : -INFINITY;
      float bm = sv;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, off));
      const float pr = valid ? expf(sv - bm) : 0.0f;
      float bs = pr;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) bs += __shfl_xor_sync(0xFFFFFFFFu, bs, off);
      probs[(wblk * REP + wr) * 32 + lane] = pr;
      if (lane == 0) { bmax[wblk * REP + wr] = bm; bsum[wblk * REP + wr] = bs; }
      // the token's own key: one more score per head, computed by the first block's warps on the first chunk
      if (owns_new && c0 == k0 && wblk == 0) {
        float a = 0.0f;
        for (uint32_t e = lane; e < hd; e += 32) a = fmaf(qs[wr * hd + e], knew[e], a);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, off);
        if (lane == 0) bmax[kBlocks * REP + wr] = a * p.scale;
      }
    }
    __syncthreads();
    // ---- weighted values: this thread's four elements over its group's keys ----
    if (vact) {
      const bool with_new = owns_new && c0 == k0;
      float M = run_m;
#pragma unroll
      for (int bl = 0; bl < kBlocks; ++bl) M = fmaxf(M, bmax[bl * REP + vr]);
      const float snew = with_new ? bmax[kBlocks * REP + vr] : -INFINITY;
      M = fmaxf(M, snew);
      const float cr = expf(run_m - M);  // 0 on the first chunk
      float L = run_l * cr;
      float4 O = make_float4(run_o.x * cr, run_o.y * cr, run_o.z * cr, run_o.w * cr);
#pragma unroll
      for (int bl = 0; bl < kBlocks; ++bl) {
        const float bm = bmax[bl * REP + vr];
        if (bm != -INFINITY) {
          const float cb = expf(bm - M);
          L = fmaf(bsum[bl * REP + vr], cb, L);
          const uint32_t nb = min(32u, nkeys - min(nkeys, (uint32_t)bl * 32u));
          const float* pp = probs + (bl * REP + vr) * 32;
          const float4* vp = reinterpret_cast<const float4*>(vs + (size_t)bl * 32 * hd) + vc;
          float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
          uint32_t kk = vg;
          for (; kk + G < nb; kk += 2 * G) {  // two keys per step: independent reads and sums
            const float p0 = pp[kk], p1 = pp[kk + G];
            const float4 v0 = vp[(size_t)kk * nq4], v1 = vp[(size_t)(kk + G) * nq4];
            a0.x = fmaf(p0, v0.x, a0.x); a0.y = fmaf(p0, v0.y, a0.y); a0.z = fmaf(p0, v0.z, a0.z); a0.w = fmaf(p0, v0.w, a0.w);
            a1.x = fmaf(p1, v1.x, a1.x); a1.y = fmaf(p1, v1.y, a1.y); a1.z = fmaf(p1, v1.z, a1.z); a1.w = fmaf(p1, v1.w, a1.w);
          }
          if (kk < nb) {
            const float p0 = pp[kk];
            const float4 v0 = vp[(size_t)kk * nq4];
            a0.x = fmaf(p0, v0.x, a0.x); a0.y = fmaf(p0, v0.y, a0.y); a0.z = fmaf(p0, v0.z, a0.z); a0.w = fmaf(p0, v0.w, a0.w);
          }
          O.x = fmaf(a0.x + a1.x, cb, O.x); O.y = fmaf(a0.y + a1.y, cb, O.y); O.z = fmaf(a0.z + a1.z, cb, O.z); O.w = fmaf(a0.w + a1.w, cb, O.w);
        }
      }
      if (with_new) {
        const float cn = expf(snew - M);
        L += cn;
        if (vg == 0) {
          const float4 vn = reinterpret_cast<const float4*>(vnew)[vc];
          O.x = fmaf(cn, vn.x, O.x); O.y = fmaf(cn, vn.y, O.y); O.z = fmaf(cn, vn.z, O.z); O.w = fmaf(cn, vn.w, O.w);
        }
      }
      run_m = M; run_l = L; run_o = O;
    }
  }
  if (!ok && p.status && tid == 0) atomicExch(p.status, 3);
  // ---- the key groups' sums come together in group 0 (through the K staging area, no longer needed) ----
  if (G > 1) {
    __syncthreads();
    float4* comb = reinterpret_cast<float4*>(ks);
    if (vact && vg > 0) comb[(vg - 1) * vthreads + vrem] = run_o;
    __syncthreads();
    if (vact && vg == 0) {
      for (uint32_t g2 = 1; g2 < G; ++g2) {
        const float4 o2 = comb[(g2 - 1) * vthreads + vrem];
        run_o.x += o2.x; run_o.y += o2.y; run_o.z += o2.z; run_o.w += o2.w;
      }
    }
  }
  // ---- this CTA's result: straight out, or into the split scratch ----
  const uint32_t stride = hd + 4;  // a row of sums, then its maximum and total; 16-byte aligned rows
  const bool writer = vact && vg == 0;
  float* sc = p.scratch + ((((size_t)bk * p.T + t) * gridDim.z + split) * REP) * stride;
  if (writer) {
    if (gridDim.z == 1) {
      float* o = p.out + (size_t)(b * p.T + t) * p.out_ld + ((size_t)kvh * REP + vr) * hd + 4 * vc;
      const float inv = 1.0f / run_l;
      o[0] = run_o.x * inv; o[1] = run_o.y * inv; o[2] = run_o.z * inv; o[3] = run_o.w * inv;
    } else {
      *reinterpret_cast<float4*>(sc + (size_t)vr * stride + 4 * vc) = run_o;
      if (vc == 0) { sc[(size_t)vr * stride + hd] = run_m; sc[(size_t)vr * stride + hd + 1] = run_l; }
    }
  }
  if (gridDim.z == 1) { if (tid == 0) trace_max(p.trace, 2); return; }
  // ---- merge the key splits: last CTA to arrive ----
  __threadfence();
  __syncthreads();
  unsigned* counter = p.counters + (size_t)bk * p.T + t;
  if (tid == 0) {
    const unsigned a = atomicAdd(counter, 1u);
    s_last = a == gridDim.z - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (!s_last) { if (tid == 0) trace_max(p.trace, 2); return; }
  __threadfence();
  if (tid == 0) *counter = 0;
  const float* base = p.scratch + (((size_t)bk * p.T + t) * gridDim.z) * REP * stride;
  const uint32_t ns = gridDim.z;  // <= 64
  float* wgt = mg;                // [ns][REP] max, then coefficient
  float* lsum = mg + 64 * REP;    // [ns][REP]
  // the splits' sums for this thread's elements are requested first; the weights are worked out while they travel
  float4 part_o[8];
  if (writer) {
#pragma unroll
    for (int u = 0; u < 8; ++u)
      part_o[u] = (uint32_t)u < ns ? __ldcg(reinterpret_cast<const float4*>(base + ((size_t)u * REP + vr) * stride + 4 * vc)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (uint32_t i = tid; i < ns * REP; i += kThreads) {
    const float* src = base + (size_t)i * stride;  // i = s * REP + r
    wgt[i] = __ldcg(src + hd);
    lsum[i] = __ldcg(src + hd + 1);
  }
  __syncthreads();
  float* inv = lsum + 64 * REP;   // [REP] 1 / total
  if (warp < REP) {  // one warp per head: the lanes share the splits (ns <= 64)
    const uint32_t r = warp;
    const float m0 = (uint32_t)lane < ns ? wgt[lane * REP + r] : -INFINITY;
    const float m1 = (uint32_t)lane + 32 < ns ? wgt[(lane + 32) * REP + r] : -INFINITY;
    float M = fmaxf(m0, m1);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, off));
    const float c0 = m0 == -INFINITY ? 0.0f : expf(m0 - M), c1 = m1 == -INFINITY ? 0.0f : expf(m1 - M);
    float L = 0.0f;
    if ((uint32_t)lane < ns) { L = lsum[lane * REP + r] * c0; wgt[lane * REP + r] = c0; }
    if ((uint32_t)lane + 32 < ns) { L = fmaf(lsum[(lane + 32) * REP + r], c1, L); wgt[(lane + 32) * REP + r] = c1; }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xFFFFFFFFu, L, off);
    if (lane == 0) inv[r] = 1.0f / L;
  }
  __syncthreads();
  if (writer) {
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t s0 = 0; s0 < ns; s0 += 8) {
      if (s0 > 0) {
#pragma unroll
        for (int u = 0; u < 8; ++u)
          part_o[u] = s0 + u < ns ? __ldcg(reinterpret_cast<const float4*>(base + ((size_t)(s0 + u) * REP + vr) * stride + 4 * vc)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (s0 + u < ns) {
          const float w = wgt[(s0 + u) * REP + vr];
          O.x = fmaf(part_o[u].x, w, O.x); O.y = fmaf(part_o[u].y, w, O.y); O.z = fmaf(part_o[u].z, w, O.z); O.w = fmaf(part_o[u].w, w, O.w);
        }
      }
    }
    float* o = p.out + (size_t)(b * p.T + t) * p.out_ld + ((size_t)kvh * REP + vr) * hd + 4 * vc;
    const float iv = inv[vr];
    o[0] = O.x * iv; o[1] = O.y * iv; o[2] = O.z * iv; o[3] = O.w * iv;
  }
  if (tid == 0) trace_max(p.trace, 2);
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

template <int REP, int SUB>
cudaError_t launch_attn_sub(ruai_ctx* c, const AttnParams& p, dim3 grid, size_t smem) {
  static bool attr_done[64] = {};
  if (!attr_done[c->ordinal & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attention_kernel<REP, SUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    attr_done[c->ordinal & 63] = true;
  }
  return ruai_launch(c, attention_kernel<REP, SUB>, grid, dim3(kAttnChunkKeys * REP * SUB), smem, true, p);
}
template <int REP>
cudaError_t launch_attn(ruai_ctx* c, const AttnParams& p, dim3 grid, size_t smem_per_sub) {
  // smem_per_sub: bytes without the partial scores; those take REP * REP * SUB * 64 floats more
  const bool big = (size_t)grid.x * grid.y * grid.z > 2u * (size_t)c->sm_count;
  const size_t parts = (size_t)REP * REP * kAttnChunkKeys * sizeof(float);
  return big ? launch_attn_sub<REP, 1>(c, p, grid, smem_per_sub + parts) : launch_attn_sub<REP, 2>(c, p, grid, smem_per_sub + 2 * parts);
}

}  // namespace

int ruai_embed(ruai_ctx* c, const int32_t* ids, const float* embed, const float* wpe, const int32_t* len, uint32_t rows, uint32_t T, uint32_t d,
               uint32_t vocab, float* x, int* err, float* sumsq) {
  RUAI_CUDA(c, ruai_launch(c, embed_kernel, dim3(rows), dim3(256), 0, true, ids, embed, wpe, len, T, d, vocab, x, err, sumsq));
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
                           kcache, vcache, c->status));
  return RUAI_OK;
}

int ruai_attention(ruai_ctx* c, const AttnParams& p_in, uint32_t B, uint32_t rep, uint32_t splits) {
  AttnParams p = p_in;
  p.trace = ruai_trace_slot(c);
  if (p.hd % 4 || p.hd > 256) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "head_dim %u must be a multiple of 4 and at most 256", p.hd);
  constexpr size_t kb = kAttnChunkKeys / 32;
  const size_t floats = 2 * (size_t)kAttnChunkKeys * p.hd + (size_t)rep * p.hd + 2 * (size_t)p.hd + kb * rep * 32 + (kb + 1) * rep + kb * rep +
                        128 * (size_t)rep + rep;  // + the partial scores, added per variant at the launch
  const size_t smem = floats * sizeof(float);
  const dim3 grid(B * p.KV, p.T, splits);
  cudaError_t e;
  switch (rep) {
    case 1: e = launch_attn<1>(c, p, grid, smem); break;
    case 2: e = launch_attn<2>(c, p, grid, smem); break;
    case 3: e = launch_attn<3>(c, p, grid, smem); break;
    case 4: e = launch_attn<4>(c, p, grid, smem); break;
    case 8: e = launch_attn<8>(c, p, grid, smem); break;
    default: return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "%u query heads per KV head (supported: 1, 2, 3, 4, 8)", rep);
  }
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "attention launch: %s", cudaGetErrorString(e));
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
