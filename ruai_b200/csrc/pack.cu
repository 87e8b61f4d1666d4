// Repack between the reference's quantized buffers and the kernel layout.
//
// Reference layout (src/nn/modules/layers.rs:34-38, 205-211):
//   int8: q [k, n] i8 row-major, scale [n]
//   int4: q [k/2, n] bytes, byte (r, j) = row 2r in the low nibble, row 2r+1 in the
//         high nibble, two's complement; scale [k/group, n]
// Kernel layout ("chunk16"): for column j and chunk c the 16 bytes at (c*n + j)*16.
//   int8: byte b of chunk c = q[16c + b, j] (rows past k are zero)
//   int4 (group 32): chunk c is scale group c.  32-bit word i (0..3), byte b (0..3):
//         low nibble = row 32c + 4i + b, high nibble = row 32c + 16 + 4i + b, each
//         stored as value + 8 (0..15) so that `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F`
//         give four consecutive rows as four unsigned bytes.
// Scales are copied unchanged.  Shapes the chunk layout does not cover (int4 with a
// group other than 32) keep the reference layout.
#include "common.cuh"
#include "pstep.cuh"

namespace {

__global__ void repack8_kernel(const int8_t* __restrict__ q, uint32_t k, uint32_t n, uint32_t chunks, uint4* __restrict__ out) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (j >= n) return;
  uint32_t w[4] = {0, 0, 0, 0};
  for (uint32_t b = 0; b < 16; ++b) {
    const uint32_t row = 16 * c + b;
    const uint32_t v = row < k ? (uint8_t)q[(size_t)row * n + j] : 0u;
    w[b >> 2] |= v << (8 * (b & 3));
  }
  out[(size_t)c * n + j] = make_uint4(w[0], w[1], w[2], w[3]);
}

__global__ void unpack8_kernel(const uint4* __restrict__ in, uint32_t k, uint32_t n, int8_t* __restrict__ q) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (j >= n) return;
  const uint4 v = in[(size_t)c * n + j];
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  for (uint32_t b = 0; b < 16; ++b) {
    const uint32_t row = 16 * c + b;
    if (row < k) q[(size_t)row * n + j] = (int8_t)((w[b >> 2] >> (8 * (b & 3))) & 0xFF);
  }
}

__global__ void repack4_kernel(const int8_t* __restrict__ q, uint32_t n, uint4* __restrict__ out) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (j >= n) return;
  // offset-binary values of the group's 32 rows
  uint32_t u[32];
  for (uint32_t r = 0; r < 16; ++r) {
    const uint8_t b = (uint8_t)q[(size_t)(16 * c + r) * n + j];
    u[2 * r] = (b & 0xF) ^ 8u;
    u[2 * r + 1] = (b >> 4) ^ 8u;
  }
  uint32_t w[4];
  for (uint32_t i = 0; i < 4; ++i) {
    w[i] = 0;
    for (uint32_t b = 0; b < 4; ++b) w[i] |= (u[4 * i + b] | (u[16 + 4 * i + b] << 4)) << (8 * b);
  }
  out[(size_t)c * n + j] = make_uint4(w[0], w[1], w[2], w[3]);
}

__global__ void unpack4_kernel(const uint4* __restrict__ in, uint32_t n, int8_t* __restrict__ q) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (j >= n) return;
  const uint4 v = in[(size_t)c * n + j];
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t u[32];
  for (uint32_t i = 0; i < 4; ++i)
    for (uint32_t b = 0; b < 4; ++b) {
      const uint32_t byte = (w[i] >> (8 * b)) & 0xFF;
      u[4 * i + b] = (byte & 0xF) ^ 8u;
      u[16 + 4 * i + b] = (byte >> 4) ^ 8u;
    }
  for (uint32_t r = 0; r < 16; ++r) q[(size_t)(16 * c + r) * n + j] = (int8_t)(u[2 * r] | (u[2 * r + 1] << 4));
}

// Backend::dequant_int4 (mod.rs:689-693): w[l, j] = nibble(l, j) * scale[l / group, j].
__global__ void dequant4_chunk_kernel(const uint4* __restrict__ in, const float* __restrict__ scale, uint32_t n, float* __restrict__ out) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, c = blockIdx.y;
  if (j >= n) return;
  const uint4 v = in[(size_t)c * n + j];
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  const float s = scale[(size_t)c * n + j];
  for (uint32_t i = 0; i < 4; ++i)
    for (uint32_t b = 0; b < 4; ++b) {
      const uint32_t byte = (w[i] >> (8 * b)) & 0xFF;
      out[(size_t)(32 * c + 4 * i + b) * n + j] = (float)((int)(byte & 0xF) - 8) * s;
      out[(size_t)(32 * c + 16 + 4 * i + b) * n + j] = (float)((int)(byte >> 4) - 8) * s;
    }
}

__global__ void dequant4_ref_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale, uint32_t k, uint32_t n, uint32_t group,
                                    float* __restrict__ out) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x, l = blockIdx.y;
  if (j >= n) return;
  out[(size_t)l * n + j] = (float)int4_of((uint8_t)q[(size_t)(l / 2) * n + j], l & 1) * scale[(size_t)(l / group) * n + j];
}

bool is_device_ptr(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// A device copy of `src` (host or device); *owned tells whether to free it.
int stage_in(ruai_ctx* c, const void* src, size_t bytes, void** dev, bool* owned) {
  if (is_device_ptr(src)) { *dev = const_cast<void*>(src); *owned = false; return RUAI_OK; }
  *owned = true;
  RUAI_CUDA(c, cudaMalloc(dev, bytes ? bytes : 1));
  RUAI_CUDA(c, cudaMemcpyAsync(*dev, src, bytes, cudaMemcpyHostToDevice, c->stream));
  return RUAI_OK;
}

}  // namespace

static int make_qweight(ruai_ctx* c, const int8_t* q, const float* scale, uint32_t k, uint32_t n, uint32_t bits, uint32_t group,
                        ruai_qweight** out) {
  if (!c || !q || !scale || !out) return ruai_fail(c, RUAI_ERR_ARG, "repack: NULL argument");
  *out = nullptr;
  if (k == 0 || n == 0) return ruai_fail(c, RUAI_ERR_SHAPE, "repack: empty weight [%u, %u]", k, n);
  // element counts must fit u32 as in the reference (cuda.rs:178-180)
  if ((uint64_t)k * n > 0xFFFFFFFFull) return ruai_fail(c, RUAI_ERR_SHAPE, "repack: %u x %u elements exceed u32", k, n);
  if (bits == 4 && !(group >= 2 && group % 2 == 0 && k % group == 0))
    return ruai_fail(c, RUAI_ERR_SHAPE, "int4 group %u must be even and divide in_features %u", group, k);
  DeviceGuard g(c->ordinal);
  ruai_qweight* w = new ruai_qweight();
  w->ctx = c; w->k = k; w->n = n; w->bits = bits; w->group = bits == 4 ? group : 0;
  const size_t q_bytes = bits == 8 ? (size_t)k * n : (size_t)(k / 2) * n;
  w->scale_bytes = (bits == 8 ? (size_t)n : (size_t)(k / group) * n) * sizeof(float);
  if (bits == 8) { w->layout = QL_CHUNK16; w->chunks = (k + 15) / 16; }
  else if (group == 32) { w->layout = QL_CHUNK16; w->chunks = k / 32; }
  else { w->layout = QL_REFERENCE; w->chunks = 0; }
  w->data_bytes = w->layout == QL_CHUNK16 ? (size_t)w->chunks * n * 16 : q_bytes;
  if (w->chunks > 65535) { delete w; return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "repack: k = %u too large", k); }
  void *qd = nullptr, *sd = nullptr;
  bool qo = false, so = false;
  int rc = RUAI_OK;
  auto fail = [&](int code) {
    if (qo && qd) cudaFree(qd);
    if (so && sd) cudaFree(sd);
    cudaFree(w->data); cudaFree(w->scale);
    delete w;
    return code;
  };
  if ((rc = stage_in(c, q, q_bytes, &qd, &qo)) != RUAI_OK) return fail(rc);
  if ((rc = stage_in(c, scale, w->scale_bytes, &sd, &so)) != RUAI_OK) return fail(rc);
  if (cudaMalloc(&w->data, w->data_bytes) != cudaSuccess || cudaMalloc(&w->scale, w->scale_bytes) != cudaSuccess)
    return fail(ruai_fail(c, RUAI_ERR_CUDA, "repack: out of device memory (%zu bytes)", w->data_bytes + w->scale_bytes));
  cudaMemcpyAsync(w->scale, sd, w->scale_bytes, cudaMemcpyDeviceToDevice, c->stream);
  dim3 grid((n + 127) / 128, w->chunks ? w->chunks : 1);
  if (w->layout == QL_REFERENCE) cudaMemcpyAsync(w->data, qd, q_bytes, cudaMemcpyDeviceToDevice, c->stream);
  else if (bits == 8) repack8_kernel<<<grid, 128, 0, c->stream>>>((const int8_t*)qd, k, n, w->chunks, (uint4*)w->data);
  else repack4_kernel<<<grid, 128, 0, c->stream>>>((const int8_t*)qd, n, (uint4*)w->data);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
  if (e != cudaSuccess) return fail(ruai_fail(c, RUAI_ERR_CUDA, "repack: %s", cudaGetErrorString(e)));
  if (qo) cudaFree(qd);
  if (so) cudaFree(sd);
  *out = w;
  return RUAI_OK;
}

RUAI_API int ruai_repack_int8(ruai_ctx* c, const int8_t* q, const float* scale, uint32_t k, uint32_t n, ruai_qweight** out) {
  return make_qweight(c, q, scale, k, n, 8, 0, out);
}

RUAI_API int ruai_repack_int4(ruai_ctx* c, const int8_t* q, const float* scale, uint32_t k, uint32_t n, uint32_t group,
                              ruai_qweight** out) {
  return make_qweight(c, q, scale, k, n, 4, group, out);
}

RUAI_API int ruai_qweight_free(ruai_qweight* w) {
  if (!w) return RUAI_OK;
  DeviceGuard g(w->ctx->ordinal);
  cudaStreamSynchronize(w->ctx->stream);
  if (w->stream) { ruai_sweight_free(w->stream); delete w->stream; }
  cudaFree(w->data);
  cudaFree(w->scale);
  delete w;
  return RUAI_OK;
}

RUAI_API int ruai_qweight_info(const ruai_qweight* w, uint32_t* k, uint32_t* n, uint32_t* bits, uint32_t* group) {
  if (!w) return ruai_fail(nullptr, RUAI_ERR_ARG, "qweight is NULL");
  if (k) *k = w->k;
  if (n) *n = w->n;
  if (bits) *bits = w->bits;
  if (group) *group = w->group;
  return RUAI_OK;
}

RUAI_API int ruai_unpack(ruai_ctx* c, const ruai_qweight* w, int8_t* q_out, float* scale_out) {
  if (!c || !w || !q_out || !scale_out) return ruai_fail(c, RUAI_ERR_ARG, "ruai_unpack: NULL argument");
  DeviceGuard g(c->ordinal);
  const size_t q_bytes = w->bits == 8 ? (size_t)w->k * w->n : (size_t)(w->k / 2) * w->n;
  const bool q_dev = is_device_ptr(q_out), s_dev = is_device_ptr(scale_out);
  int8_t* qd = q_out;
  if (!q_dev) RUAI_CUDA(c, cudaMalloc(&qd, q_bytes));
  dim3 grid((w->n + 127) / 128, w->chunks ? w->chunks : 1);
  if (w->layout == QL_REFERENCE) cudaMemcpyAsync(qd, w->data, q_bytes, cudaMemcpyDeviceToDevice, c->stream);
  else if (w->bits == 8) unpack8_kernel<<<grid, 128, 0, c->stream>>>((const uint4*)w->data, w->k, w->n, qd);
  else unpack4_kernel<<<grid, 128, 0, c->stream>>>((const uint4*)w->data, w->n, qd);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && !q_dev) e = cudaMemcpyAsync(q_out, qd, q_bytes, cudaMemcpyDeviceToHost, c->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(scale_out, w->scale, w->scale_bytes, s_dev ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, c->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
  if (!q_dev) cudaFree(qd);
  if (e != cudaSuccess) return ruai_fail(c, RUAI_ERR_CUDA, "ruai_unpack: %s", cudaGetErrorString(e));
  return RUAI_OK;
}

RUAI_API int ruai_dequant_int4_ref(ruai_ctx* c, const int8_t* q, const float* scale, uint32_t k, uint32_t n, uint32_t group, float* out) {
  if (!c || !q || !scale || !out) return ruai_fail(c, RUAI_ERR_ARG, "ruai_dequant_int4_ref: NULL argument");
  if (!(group >= 2 && group % 2 == 0 && k % group == 0))
    return ruai_fail(c, RUAI_ERR_SHAPE, "int4 group %u must be even and divide in_features %u", group, k);
  if (k == 0 || n == 0) return RUAI_OK;
  if (k > 65535) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "ruai_dequant_int4_ref: k too large");
  DeviceGuard g(c->ordinal);
  dequant4_ref_kernel<<<dim3((n + 127) / 128, k), 128, 0, c->stream>>>(q, scale, k, n, group, out);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

RUAI_API int ruai_dequant_int4(ruai_ctx* c, const ruai_qweight* w, float* out) {
  if (!c || !w || !out) return ruai_fail(c, RUAI_ERR_ARG, "ruai_dequant_int4: NULL argument");
  if (w->bits != 4) return ruai_fail(c, RUAI_ERR_SHAPE, "ruai_dequant_int4: weight is int%u", w->bits);
  if (w->layout == QL_REFERENCE) return ruai_dequant_int4_ref(c, (const int8_t*)w->data, w->scale, w->k, w->n, w->group, out);
  DeviceGuard g(c->ordinal);
  dequant4_chunk_kernel<<<dim3((w->n + 127) / 128, w->chunks), 128, 0, c->stream>>>((const uint4*)w->data, w->scale, w->n, out);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}
