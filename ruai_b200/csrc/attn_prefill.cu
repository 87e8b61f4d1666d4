// Causal attention over the KV cache for MANY query positions at once (prefill): queries in tiles, so that a cached key
// or value is read from memory once per tile of 16 queries instead of once per query.
//
// Semantics are those of attention_kernel (decode_ops.cu), i.e. of `scaled_dot_product_attention` with the causal
// offset of functional.rs:238-247 / 281-296: query t of the new block sees keys 0 .. past + t.  q is rotated and the
// new keys / values are appended before (rope_kv_kernel).  Everything is f32 on the CUDA cores: softmax(q k^T / sqrt(hd)) v
// with a running maximum and sum per row (the order of the additions differs from the CPU's, as every GPU kernel's does;
// the parity tests bound the difference).
//
// A CTA owns (sequence, KV head, tile of QT queries): rows = QT queries x the REP query heads of the group, 64 rows
// (48 for groups of three).  Eight computing warps own an eighth of the rows each and never need each other after the query tile is in shared memory; a ninth warp's
// first lane streams the keys and values, 64 at a time, through two shared-memory buffers with bulk copies (keys row by
// row into rows padded by four floats, so that a lane per key reads them without bank conflicts).  Per chunk a warp
// computes its rows' scores (a lane per key, two keys per lane, all of the warp's rows at once: a key row is read from
// shared memory once per warp), updates the rows' running softmax, leaves the probabilities in its own rows of a
// shared tile and accumulates probabilities x values (a lane per four elements of the head dimension).
#include "common.cuh"
#include "decode_ops.cuh"
#include "pipeline.cuh"

namespace {

using namespace pipe;

constexpr int kKC = 64;        // keys per chunk
constexpr int kWarps = 8;      // computing warps
constexpr int kThreads = (kWarps + 1) * 32;

template <int REP, int kQT>
__global__ void __launch_bounds__(kThreads) attention_prefill_kernel(const AttnParams p, uint32_t hd4_per_lane) {
  constexpr int kRows = kQT * REP;
  constexpr int R = kRows / kWarps;     // rows per warp
  static_assert(kRows % kWarps == 0, "rows must share out over the warps");
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[2], empty[2];
  __shared__ int s_abort;
  const uint32_t hd = p.hd, kstride = hd + 4u;
  float* qs = reinterpret_cast<float*>(smem_raw);                  // [kRows][hd]
  float* ks = qs + (size_t)kRows * hd;                              // [2][kKC][hd + 4]
  float* vs = ks + 2 * (size_t)kKC * kstride;                       // [2][kKC][hd]
  float* ps = vs + 2 * (size_t)kKC * hd;                            // [kRows][kKC]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // the tiles with the most keys first: they are the long ones
  const uint32_t bk = blockIdx.y, b = bk / p.KV, kvh = bk % p.KV, q0 = (gridDim.x - 1u - blockIdx.x) * kQT;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], kWarps); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_abort = 0;
  }
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t past = (uint32_t)*p.len;
  const uint32_t nq = min((uint32_t)kQT, p.T - q0);
  uint32_t kmax = past + q0 + nq;  // keys 0 .. kmax - 1 are seen by the tile's last query
  const bool over = kmax > p.cap;  // the device's position is not the host's: touch nothing beyond the cache, tell the host
  if (over) {
    kmax = 0;
    if (tid == 0 && p.status) atomicCAS(p.status, 0, 5);
  }
  const uint32_t nchunks = (kmax + kKC - 1) / kKC;
  // the query tile: row r = qi * REP + h
  for (uint32_t i = tid; i < (uint32_t)kRows * (hd / 4); i += kThreads) {
    const uint32_t r = i / (hd / 4), e4 = i % (hd / 4), qi = r / REP, h = r % REP;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (qi < nq) v = *reinterpret_cast<const float4*>(p.q + (size_t)(b * p.T + q0 + qi) * p.q_ld + (size_t)(kvh * REP + h) * hd + 4 * e4);
    reinterpret_cast<float4*>(qs)[i] = v;
  }
  __syncthreads();
  const float* kbase = p.kcache + (size_t)bk * p.cap * hd;
  const float* vbase = p.vcache + (size_t)bk * p.cap * hd;

  if (warp == kWarps) {
    // ===== the copying warp =====
    if (lane == 0) {
      for (uint32_t c = 0; c < nchunks; ++c) {
        const uint32_t buf = c & 1u;
        if (c >= 2 && (s_abort || !mbar_wait(&empty[buf], ((c >> 1) - 1u) & 1u))) { s_abort = 1; break; }
        const uint32_t k0 = c * kKC, nk = min((uint32_t)kKC, kmax - k0), row = hd * 4u;
        mbar_expect_tx(&full[buf], 2u * nk * row);
        for (uint32_t k = 0; k < nk; ++k) bulk_load(ks + ((size_t)buf * kKC + k) * kstride, kbase + (size_t)(k0 + k) * hd, row, &full[buf]);
        bulk_load(vs + (size_t)buf * kKC * hd, vbase + (size_t)k0 * hd, nk * row, &full[buf]);
      }
    }
    return;
  }

  // ===== computing warps =====
  const uint32_t row0 = (uint32_t)warp * R;
  float m_run[R], l_run[R];
  float4 o[R][2];  // this lane's elements 4 (lane + 32 j) .. of the head dimension, j < hd4_per_lane <= 2
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m_run[r] = -INFINITY; l_run[r] = 0.0f;
    o[r][0] = make_float4(0.f, 0.f, 0.f, 0.f); o[r][1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (uint32_t c = 0; c < nchunks; ++c) {
    const uint32_t buf = c & 1u, k0 = c * kKC, nk = min((uint32_t)kKC, kmax - k0);
    if (s_abort || !mbar_wait(&full[buf], (c >> 1) & 1u)) { s_abort = 1; break; }
    const float* kb = ks + (size_t)buf * kKC * kstride;
    const float* vb = vs + (size_t)buf * kKC * hd;
    // ---- scores: this lane's keys `lane` and `lane + 32` against the warp's R rows ----
    float s0[R], s1[R];
#pragma unroll
    for (int r = 0; r < R; ++r) { s0[r] = 0.0f; s1[r] = 0.0f; }
    const float4* k0p = reinterpret_cast<const float4*>(kb + (size_t)lane * kstride);
    const float4* k1p = reinterpret_cast<const float4*>(kb + (size_t)(lane + 32) * kstride);
    const float4* qp = reinterpret_cast<const float4*>(qs + (size_t)row0 * hd);
    for (uint32_t e4 = 0; e4 < hd / 4; ++e4) {
      const float4 a = k0p[e4], bq = k1p[e4];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float4 qv = qp[(size_t)r * (hd / 4) + e4];
        s0[r] = fmaf(qv.x, a.x, s0[r]); s0[r] = fmaf(qv.y, a.y, s0[r]); s0[r] = fmaf(qv.z, a.z, s0[r]); s0[r] = fmaf(qv.w, a.w, s0[r]);
        s1[r] = fmaf(qv.x, bq.x, s1[r]); s1[r] = fmaf(qv.y, bq.y, s1[r]); s1[r] = fmaf(qv.z, bq.z, s1[r]); s1[r] = fmaf(qv.w, bq.w, s1[r]);
      }
    }
    // ---- running softmax per row; probabilities into the warp's rows of the shared tile ----
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint32_t qpos = past + q0 + (row0 + r) / REP;  // the last key this row's query sees
      const uint32_t key0 = k0 + lane, key1 = key0 + 32u;
      float a = (key0 <= qpos && (uint32_t)lane < nk) ? s0[r] * p.scale : -INFINITY;
      float bq = (key1 <= qpos && (uint32_t)lane + 32u < nk) ? s1[r] * p.scale : -INFINITY;
      float mx = fmaxf(a, bq);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
      const float m_new = fmaxf(m_run[r], mx);
      const float p0 = a == -INFINITY ? 0.0f : expf(a - m_new), p1 = bq == -INFINITY ? 0.0f : expf(bq - m_new);
      float sum = p0 + p1;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
      const float corr = m_run[r] == -INFINITY ? 0.0f : expf(m_run[r] - m_new);
      l_run[r] = fmaf(l_run[r], corr, sum);
      m_run[r] = m_new;
      o[r][0].x *= corr; o[r][0].y *= corr; o[r][0].z *= corr; o[r][0].w *= corr;
      o[r][1].x *= corr; o[r][1].y *= corr; o[r][1].z *= corr; o[r][1].w *= corr;
      ps[(size_t)(row0 + r) * kKC + lane] = p0;
      ps[(size_t)(row0 + r) * kKC + lane + 32] = p1;
    }
    __syncwarp();
    // ---- values: o[r] += sum_k p[r][k] v[k], four keys at a time (keys past nk carry probability 0) ----
    const uint32_t nk4 = (nk + 3u) & ~3u;
    for (uint32_t k = 0; k < nk4; k += 4) {
      float4 pr[R];
#pragma unroll
      for (int r = 0; r < R; ++r) pr[r] = *reinterpret_cast<const float4*>(ps + (size_t)(row0 + r) * kKC + k);
#pragma unroll
      for (uint32_t j = 0; j < 2; ++j) {
        if (j < hd4_per_lane) {
          const uint32_t e4 = lane + 32u * j;
          if (e4 < hd / 4) {
            const float4 v0 = reinterpret_cast<const float4*>(vb + (size_t)(k + 0) * hd)[e4];
            const float4 v1 = k + 1 < nk ? reinterpret_cast<const float4*>(vb + (size_t)(k + 1) * hd)[e4] : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 v2 = k + 2 < nk ? reinterpret_cast<const float4*>(vb + (size_t)(k + 2) * hd)[e4] : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 v3 = k + 3 < nk ? reinterpret_cast<const float4*>(vb + (size_t)(k + 3) * hd)[e4] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < R; ++r) {
              o[r][j].x = fmaf(pr[r].x, v0.x, o[r][j].x); o[r][j].y = fmaf(pr[r].x, v0.y, o[r][j].y); o[r][j].z = fmaf(pr[r].x, v0.z, o[r][j].z); o[r][j].w = fmaf(pr[r].x, v0.w, o[r][j].w);
              o[r][j].x = fmaf(pr[r].y, v1.x, o[r][j].x); o[r][j].y = fmaf(pr[r].y, v1.y, o[r][j].y); o[r][j].z = fmaf(pr[r].y, v1.z, o[r][j].z); o[r][j].w = fmaf(pr[r].y, v1.w, o[r][j].w);
              o[r][j].x = fmaf(pr[r].z, v2.x, o[r][j].x); o[r][j].y = fmaf(pr[r].z, v2.y, o[r][j].y); o[r][j].z = fmaf(pr[r].z, v2.z, o[r][j].z); o[r][j].w = fmaf(pr[r].z, v2.w, o[r][j].w);
              o[r][j].x = fmaf(pr[r].w, v3.x, o[r][j].x); o[r][j].y = fmaf(pr[r].w, v3.y, o[r][j].y); o[r][j].z = fmaf(pr[r].w, v3.z, o[r][j].z); o[r][j].w = fmaf(pr[r].w, v3.w, o[r][j].w);
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[buf]);  // this warp is done with the chunk's keys and values
  }
  if (s_abort) {
    if (lane == 0 && p.status) atomicCAS(p.status, 0, 3);
    return;
  }
  // ---- out = o / l ----
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t row = row0 + r, qi = row / REP, h = row % REP;
    if (qi >= nq || over) continue;
    const float inv = 1.0f / l_run[r];
    float* dst = p.out + (size_t)(b * p.T + q0 + qi) * p.out_ld + (size_t)(kvh * REP + h) * hd;
#pragma unroll
    for (uint32_t j = 0; j < 2; ++j) {
      const uint32_t e4 = lane + 32u * j;
      if (j < hd4_per_lane && e4 < hd / 4)
        reinterpret_cast<float4*>(dst)[e4] = make_float4(o[r][j].x * inv, o[r][j].y * inv, o[r][j].z * inv, o[r][j].w * inv);
    }
  }
}

template <int REP, int kQT>
cudaError_t launch(ruai_ctx* c, const AttnParams& p, uint32_t B, size_t smem, uint32_t hd4_per_lane) {
  static bool done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<REP, kQT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    done[dev & 63] = true;
  }
  const dim3 grid((p.T + kQT - 1) / kQT, B * p.KV);
  return ruai_launch(c, attention_prefill_kernel<REP, kQT>, grid, dim3(kThreads), smem, true, p, hd4_per_lane);
}

constexpr int tile_queries(int rep) { return rep == 3 ? 16 : 64 / rep; }

}  // namespace

// 1: launched; 0: this shape is not taken (the caller uses attention_kernel); < 0: error.
int ruai_attention_prefill(ruai_ctx* c, const AttnParams& p, uint32_t B, uint32_t rep) {
  if (p.fuse || p.T < 8 || p.hd % 4 || p.hd > 256) return 0;
  if (rep != 1 && rep != 2 && rep != 3 && rep != 4 && rep != 8) return 0;
  const size_t rows = (size_t)tile_queries((int)rep) * rep;
  const size_t floats = rows * p.hd + 2 * (size_t)kKC * (p.hd + 4) + 2 * (size_t)kKC * p.hd + rows * kKC;
  const size_t smem = floats * sizeof(float);
  if (smem > 200 * 1024) return 0;
  const uint32_t hd4_per_lane = (p.hd / 4 + 31) / 32;
  cudaError_t e;
  switch (rep) {
    case 1: e = launch<1, tile_queries(1)>(c, p, B, smem, hd4_per_lane); break;
    case 2: e = launch<2, tile_queries(2)>(c, p, B, smem, hd4_per_lane); break;
    case 3: e = launch<3, tile_queries(3)>(c, p, B, smem, hd4_per_lane); break;
    case 4: e = launch<4, tile_queries(4)>(c, p, B, smem, hd4_per_lane); break;
    default: e = launch<8, tile_queries(8)>(c, p, B, smem, hd4_per_lane); break;
  }
  if (e != cudaSuccess) { ruai_fail(c, RUAI_ERR_CUDA, "prefill attention launch: %s", cudaGetErrorString(e)); return -1; }
  return 1;
}
