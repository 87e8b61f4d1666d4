// Tile-stream layout for the persistent decode kernel (see pstep.cuh), built from the chunk layout.
#include "pstep.cuh"

namespace {

// int4: record (tile, group) = [128 columns][16 packed bytes] then [128] f32 scales.
__global__ void stream4_kernel(const uint4* __restrict__ chunk, const float* __restrict__ scale, uint32_t n, uint32_t ngroups,
                               uint8_t* __restrict__ out) {
  const uint32_t col = threadIdx.x, g = blockIdx.x, tile = blockIdx.y;
  const uint32_t j = tile * kStreamTileCols + col;
  uint8_t* rec = out + ((size_t)tile * ngroups + g) * kStreamRec4;
  const bool in = j < n;
  // stored nibble 8 is weight 0 (pack.cu stores value + 8)
  const uint4 v = in ? chunk[(size_t)g * n + j] : make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
  reinterpret_cast<uint4*>(rec)[col] = v;
  reinterpret_cast<float*>(rec + kStreamTileCols * 16)[col] = in ? scale[(size_t)g * n + j] : 0.0f;
}

// int8: record (tile, block of 32 rows) = [2 halves of 16 rows][128 columns][16 bytes].
__global__ void stream8_kernel(const uint4* __restrict__ chunk, uint32_t n, uint32_t chunks, uint32_t nblk, uint8_t* __restrict__ out) {
  const uint32_t col = threadIdx.x, b = blockIdx.x, tile = blockIdx.y;
  const uint32_t j = tile * kStreamTileCols + col;
  uint4* rec = reinterpret_cast<uint4*>(out + ((size_t)tile * nblk + b) * kStreamRec8);
  for (uint32_t h = 0; h < 2; ++h) {
    const uint32_t c = 2 * b + h;
    rec[h * kStreamTileCols + col] = (j < n && c < chunks) ? chunk[(size_t)c * n + j] : make_uint4(0, 0, 0, 0);
  }
}

}  // namespace

bool ruai_sweight_supported(const ruai_qweight* w) {
  return w && w->layout == QL_CHUNK16 && (w->bits == 8 || (w->bits == 4 && w->group == 32)) && w->k % 4 == 0;
}

int ruai_sweight_create(ruai_ctx* c, const ruai_qweight* w, ruai_sweight* out) {
  if (!ruai_sweight_supported(w)) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "the tile-stream layout takes int8 or int4 group-32 weights with k a multiple of 4");
  ruai_sweight_free(out);
  out->k = w->k; out->n = w->n; out->bits = w->bits;
  out->ntiles = (w->n + kStreamTileCols - 1) / kStreamTileCols;
  out->nblk = w->bits == 4 ? w->k / 32 : (w->k + 31) / 32;
  out->rec_bytes = w->bits == 4 ? kStreamRec4 : kStreamRec8;
  out->bytes = (size_t)out->ntiles * out->nblk * out->rec_bytes;
  out->colscale = w->bits == 8 ? w->scale : nullptr;
  if (out->nblk > 65535u || out->ntiles > 65535u) return ruai_fail(c, RUAI_ERR_UNSUPPORTED, "weight [%u, %u] is too large for the tile-stream layout", w->k, w->n);
  RUAI_CUDA(c, cudaMalloc(&out->data, out->bytes));
  const dim3 grid(out->nblk, out->ntiles);
  if (w->bits == 4) stream4_kernel<<<grid, kStreamTileCols, 0, c->stream>>>((const uint4*)w->data, w->scale, w->n, out->nblk, out->data);
  else stream8_kernel<<<grid, kStreamTileCols, 0, c->stream>>>((const uint4*)w->data, w->n, w->chunks, out->nblk, out->data);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

void ruai_sweight_free(ruai_sweight* s) {
  if (s->data) cudaFree(s->data);
  *s = ruai_sweight();
}
