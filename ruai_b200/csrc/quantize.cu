// Device-side quantizer and synthetic-tensor generator.
//
// The quantizers reproduce Linear::quantize_int8 (src/nn/modules/layers.rs:112-129)
// and Linear::quantize_int4 (layers.rs:139-165) bit for bit: the column / group
// maximum of |w| is order independent, the scale is one IEEE f32 division, each
// value is an IEEE f32 division followed by round-half-away (roundf) and a clamp.
// This file must not be compiled with fast-math.
#include "common.cuh"

namespace {

__global__ void synth_normal_kernel(float* out, size_t count, uint64_t key, float mult) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < count; i += stride) out[i] = ruai_synth_normal(key, i, mult);
}

__global__ void synth_tokens_kernel(int32_t* out, size_t count, uint64_t key, uint32_t vocab) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = ruai_synth_token(key, i, vocab);
}

__global__ void fill_kernel(float* out, size_t count, float v) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < count; i += stride) out[i] = v;
}

// out[c, r] = in[r, c]; in is [rows, cols].
__global__ void transpose_kernel(const float* __restrict__ in, float* __restrict__ out, uint32_t rows, uint32_t cols) {
  __shared__ float tile[32][33];
  uint32_t c = blockIdx.x * 32 + threadIdx.x, r0 = blockIdx.y * 32;
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y)
    if (r0 + i < rows && c < cols) tile[i][threadIdx.x] = in[(size_t)(r0 + i) * cols + c];
  __syncthreads();
  uint32_t r = r0 + threadIdx.x, c0 = blockIdx.x * 32;
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y)
    if (c0 + i < cols && r < rows) out[(size_t)(c0 + i) * rows + r] = tile[threadIdx.x][i];
}

// Column maxima of |w| over a band of rows; non-negative floats order like their bit patterns.
__global__ void absmax_cols_kernel(const float* __restrict__ w, uint32_t k, uint32_t n, uint32_t rows_per_block,
                                   unsigned* __restrict__ mx_bits) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const uint32_t r0 = blockIdx.y * rows_per_block, r1 = min(k, r0 + rows_per_block);
  float m = 0.0f;
  for (uint32_t r = r0; r < r1; ++r) m = fmaxf(m, fabsf(w[(size_t)r * n + j]));
  atomicMax(&mx_bits[j], __float_as_uint(m));
}

__global__ void finish_scale_kernel(float* scale, size_t count, float qmax) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const float s = scale[i];
  scale[i] = s > 0.0f ? __fdiv_rn(s, qmax) : 1.0f;
}

__global__ void quant8_kernel(const float* __restrict__ w, const float* __restrict__ scale, uint32_t k, uint32_t n,
                              int8_t* __restrict__ q) {
  const size_t total = (size_t)k * n;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    float r = roundf(__fdiv_rn(w[i], scale[i % n]));
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    q[i] = (int8_t)r;
  }
}

// One thread per (group, column): the group's maximum.
__global__ void absmax_groups_kernel(const float* __restrict__ w, uint32_t k, uint32_t n, uint32_t group, float* __restrict__ scale) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, g = blockIdx.y;
  if (j >= n) return;
  float m = 0.0f;
  for (uint32_t l = g * group; l < (g + 1) * group; ++l) m = fmaxf(m, fabsf(w[(size_t)l * n + j]));
  scale[(size_t)g * n + j] = m > 0.0f ? __fdiv_rn(m, 7.0f) : 1.0f;
}

__global__ void quant4_kernel(const float* __restrict__ w, const float* __restrict__ scale, uint32_t k, uint32_t n, uint32_t group,
                              int8_t* __restrict__ packed) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
  if (j >= n) return;
  auto qv = [&](uint32_t l) -> int {
    float v = roundf(__fdiv_rn(w[(size_t)l * n + j], scale[(size_t)(l / group) * n + j]));
    v = fminf(fmaxf(v, -8.0f), 7.0f);
    return (int)v;
  };
  const unsigned lo = (unsigned)qv(2 * r) & 0xF, hi = (unsigned)qv(2 * r + 1) & 0xF;
  packed[(size_t)r * n + j] = (int8_t)(lo | (hi << 4));
}

inline unsigned blocks_for(size_t count, unsigned threads, unsigned cap = 148 * 16) {
  size_t b = (count + threads - 1) / threads;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

int ruai_synth_normal_dev(ruai_ctx* c, float* out, size_t count, uint64_t seed, uint64_t tensor_id, double std_dev) {
  if (!count) return RUAI_OK;
  synth_normal_kernel<<<blocks_for(count, 256), 256, 0, c->stream>>>(out, count, ruai_synth_key(seed, tensor_id), ruai_synth_mult(std_dev));
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

int ruai_synth_tokens_dev(ruai_ctx* c, int32_t* out, size_t count, uint64_t seed, uint64_t tensor_id, uint32_t vocab) {
  if (!count) return RUAI_OK;
  synth_tokens_kernel<<<(unsigned)((count + 255) / 256), 256, 0, c->stream>>>(out, count, ruai_synth_key(seed, tensor_id), vocab);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

int ruai_fill_dev(ruai_ctx* c, float* out, size_t count, float v) {
  if (!count) return RUAI_OK;
  fill_kernel<<<blocks_for(count, 256), 256, 0, c->stream>>>(out, count, v);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

int ruai_transpose_dev(ruai_ctx* c, const float* in, float* out, uint32_t rows, uint32_t cols) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  transpose_kernel<<<grid, block, 0, c->stream>>>(in, out, rows, cols);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

RUAI_API int ruai_quantize_int8(ruai_ctx* c, const float* w, uint32_t k, uint32_t n, int8_t* q, float* scale) {
  if (!c || !w || !q || !scale) return ruai_fail(c, RUAI_ERR_ARG, "ruai_quantize_int8: NULL argument");
  if (k == 0 || n == 0) return RUAI_OK;
  DeviceGuard g(c->ordinal);
  RUAI_CUDA(c, cudaMemsetAsync(scale, 0, (size_t)n * sizeof(float), c->stream));
  const uint32_t rows_per_block = 128;
  dim3 grid((n + 127) / 128, (k + rows_per_block - 1) / rows_per_block);
  absmax_cols_kernel<<<grid, 128, 0, c->stream>>>(w, k, n, rows_per_block, (unsigned*)scale);
  finish_scale_kernel<<<(n + 255) / 256, 256, 0, c->stream>>>(scale, n, 127.0f);
  quant8_kernel<<<blocks_for((size_t)k * n, 256), 256, 0, c->stream>>>(w, scale, k, n, q);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

RUAI_API int ruai_quantize_int4(ruai_ctx* c, const float* w, uint32_t k, uint32_t n, uint32_t group, int8_t* q, float* scale) {
  if (!c || !w || !q || !scale) return ruai_fail(c, RUAI_ERR_ARG, "ruai_quantize_int4: NULL argument");
  // layers.rs:144
  if (!(group >= 2 && group % 2 == 0 && k % group == 0))
    return ruai_fail(c, RUAI_ERR_SHAPE, "int4 group %u must be even and divide in_features %u", group, k);
  if (k == 0 || n == 0) return RUAI_OK;
  if (k / group > 65535 || k / 2 > 65535) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "ruai_quantize_int4: k too large");
  DeviceGuard g(c->ordinal);
  absmax_groups_kernel<<<dim3((n + 127) / 128, k / group), 128, 0, c->stream>>>(w, k, n, group, scale);
  quant4_kernel<<<dim3((n + 127) / 128, k / 2), 128, 0, c->stream>>>(w, scale, k, n, group, q);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}
