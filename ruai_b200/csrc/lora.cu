// LoRA on a quantized base and the input gradient of the quantized matmul: what the reference's
// QLoRA-style fine-tuning runs on top of the same packed weights.
//
//   Linear::forward with an adapter (src/nn/modules/layers.rs:169-190, add_lora 84-97):
//       y = matmul_int8/int4(x)        (frozen quantized base)
//       y = y + (x @ A @ B) * scale    (A [k, r], B [r, n], scale = alpha / r)
//       y = y + bias
//   Backward of Tensor::matmul_int8 / matmul_int4 (src/nn/ops.rs:705-709, 731-734): the weights are frozen, the
//   only gradient is dx = g @ dequant(W)^T.  The reference materialises the f32 [k, n] weight for it; here the
//   packed weight is read once per row of g and dequantised in registers.
// These are training-side kernels (a handful of rows, run once per step), written for correctness and coalesced
// reads, not tuned like the decode path.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.0f;
  for (int i = 0; i < kThreads / 32; ++i) t += red[i];  // fixed order
  return t;
}

// dx[i, rows of chunk c] = sum_j g[i, j] * scale * q[row, j]; chunk layout (pack.cu).  grid (chunks, m).
template <int BITS>
__global__ void __launch_bounds__(kThreads) grad_input_chunk_kernel(const uint4* __restrict__ w, const float* __restrict__ scale, const float* __restrict__ g,
                                                                    uint32_t k, uint32_t n, float* __restrict__ dx) {
  constexpr int R = BITS == 4 ? 32 : 16;
  __shared__ float red[kThreads / 32];
  const uint32_t c = blockIdx.x, i = blockIdx.y;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.0f;
  for (uint32_t j = threadIdx.x; j < n; j += kThreads) {
    const uint4 q = w[(size_t)c * n + j];
    const float v = g[(size_t)i * n + j] * (BITS == 4 ? scale[(size_t)c * n + j] : scale[j]);
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (words[wi] >> (8 * b)) & 0xFFu;
        if (BITS == 4) {  // low nibble: row 4 wi + b, high nibble: row 16 + 4 wi + b, stored value + 8
          acc[4 * wi + b] = fmaf(v, (float)((int)(byte & 0xFu) - 8), acc[4 * wi + b]);
          acc[16 + 4 * wi + b] = fmaf(v, (float)((int)(byte >> 4) - 8), acc[16 + 4 * wi + b]);
        } else {
          acc[4 * wi + b] = fmaf(v, (float)(int)(int8_t)byte, acc[4 * wi + b]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float t = block_sum(acc[r], red);
    const uint32_t row = c * R + r;
    if (threadIdx.x == 0 && row < k) dx[(size_t)i * k + row] = t;
  }
}

// The same for int4 weights kept in the reference layout (groups other than 32): one packed row (two rows of k)
// per block.  grid (k / 2, m).
__global__ void __launch_bounds__(kThreads) grad_input_ref4_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale, const float* __restrict__ g,
                                                                   uint32_t k, uint32_t n, uint32_t group, float* __restrict__ dx) {
  __shared__ float red[kThreads / 32];
  const uint32_t r = blockIdx.x, i = blockIdx.y;
  const float* s0 = scale + (size_t)((2 * r) / group) * n;
  const float* s1 = scale + (size_t)((2 * r + 1) / group) * n;
  float a0 = 0.0f, a1 = 0.0f;
  for (uint32_t j = threadIdx.x; j < n; j += kThreads) {
    const uint8_t b = (uint8_t)q[(size_t)r * n + j];
    const float gv = g[(size_t)i * n + j];
    a0 = fmaf(gv * s0[j], (float)int4_of(b, false), a0);
    a1 = fmaf(gv * s1[j], (float)int4_of(b, true), a1);
  }
  const float t0 = block_sum(a0, red), t1 = block_sum(a1, red);
  if (threadIdx.x == 0) { dx[(size_t)i * k + 2 * r] = t0; dx[(size_t)i * k + 2 * r + 1] = t1; }
}

// t[i, r0 .. r0+7] = sum_p x[i, p] * A[p, r]; grid (m, ceil(rank / 8)).
__global__ void __launch_bounds__(kThreads) lora_xa_kernel(const float* __restrict__ x, const float* __restrict__ a, uint32_t k, uint32_t rank,
                                                           float* __restrict__ t) {
  __shared__ float red[kThreads / 32];
  const uint32_t i = blockIdx.x, r0 = blockIdx.y * 8;
  float acc[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) acc[u] = 0.0f;
  for (uint32_t p = threadIdx.x; p < k; p += kThreads) {
    const float xv = x[(size_t)i * k + p];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (r0 + u < rank) acc[u] = fmaf(xv, a[(size_t)p * rank + r0 + u], acc[u]);
  }
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const float s = block_sum(acc[u], red);
    if (threadIdx.x == 0 && r0 + u < rank) t[(size_t)i * rank + r0 + u] = s;
  }
}

// y[i, j] = (y[i, j] + (sum_r t[i, r] * B[r, j]) * scale) + bias[j]: the order of layers.rs:175-189.
__global__ void lora_add_kernel(float* __restrict__ y, const float* __restrict__ t, const float* __restrict__ b, const float* __restrict__ bias, uint32_t n,
                                uint32_t rank, float scale) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, i = blockIdx.y;
  if (j >= n) return;
  float d = 0.0f;
  for (uint32_t r = 0; r < rank; ++r) d = fmaf(t[(size_t)i * rank + r], b[(size_t)r * n + j], d);
  float v = y[(size_t)i * n + j] + d * scale;
  if (bias) v += bias[j];
  y[(size_t)i * n + j] = v;
}

}  // namespace

RUAI_API int ruai_matmul_q_grad_input(ruai_ctx* c, const float* g_dev, const ruai_qweight* w, float* dx_dev, uint32_t m) {
  if (!c || !g_dev || !w || !dx_dev) return ruai_fail(c, RUAI_ERR_ARG, "ruai_matmul_q_grad_input: NULL argument");
  if (m == 0) return RUAI_OK;
  if (m > 65535u) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "ruai_matmul_q_grad_input: %u rows exceed 65535", m);
  DeviceGuard g(c->ordinal);
  if (w->layout == QL_CHUNK16) {
    const dim3 grid(w->chunks, m);
    if (w->bits == 4) grad_input_chunk_kernel<4><<<grid, kThreads, 0, c->stream>>>((const uint4*)w->data, w->scale, g_dev, w->k, w->n, dx_dev);
    else grad_input_chunk_kernel<8><<<grid, kThreads, 0, c->stream>>>((const uint4*)w->data, w->scale, g_dev, w->k, w->n, dx_dev);
  } else {
    if (w->k / 2 > 65535u * 32768u) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "k too large");
    grad_input_ref4_kernel<<<dim3(w->k / 2, m), kThreads, 0, c->stream>>>((const int8_t*)w->data, w->scale, g_dev, w->k, w->n, w->group, dx_dev);
  }
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

RUAI_API int ruai_linear_lora_forward(ruai_ctx* c, const float* x_dev, const ruai_qweight* w, const float* lora_a_dev, const float* lora_b_dev,
                                      uint32_t rank, float scale, const float* bias_dev_or_null, float* out_dev, uint32_t m) {
  if (!c || !x_dev || !w || !lora_a_dev || !lora_b_dev || !out_dev) return ruai_fail(c, RUAI_ERR_ARG, "ruai_linear_lora_forward: NULL argument");
  if (rank == 0 || rank > 1024) return ruai_fail(c, RUAI_ERR_SHAPE, "LoRA rank %u must be in 1..1024", rank);
  if (m == 0) return RUAI_OK;
  if (m > 65535u) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "ruai_linear_lora_forward: %u rows exceed 65535", m);
  DeviceGuard g(c->ordinal);
  // the frozen base first (no bias: the reference adds it after the adapter), then the low-rank path into the scratch
  RUAI_TRY(ruai_matmul_q(c, RUAI_F32, x_dev, w, nullptr, out_dev, m));
  RUAI_TRY(ruai_ctx_reserve(c, (size_t)m * rank * sizeof(float), 0));
  float* t = c->partial;
  lora_xa_kernel<<<dim3(m, (rank + 7) / 8), kThreads, 0, c->stream>>>(x_dev, lora_a_dev, w->k, rank, t);
  RUAI_CUDA(c, cudaGetLastError());
  lora_add_kernel<<<dim3((w->n + 255) / 256, m), 256, 0, c->stream>>>(out_dev, t, lora_b_dev, bias_dev_or_null, w->n, rank, scale);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}
