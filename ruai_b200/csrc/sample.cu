// Token sampling on the device: `Sampler::sample` (src/nn/generation.rs:38-73) for one row of logits that already
// sits in device memory, so that sampled generation moves four bytes per token to the host, not the vocabulary.
//
//   temperature <= 0 : argmax (the last maximum, generation.rs:6-8);
//   otherwise        : candidates sorted by logit, descending; keep top_k (0 = all); p_i = exp((l_i - l_0) / T),
//                      normalised by their sum; keep the shortest prefix whose mass reaches top_p (1 = all);
//                      r = unit() * (sum of the kept p); the first candidate whose running sum exceeds r.
// The reference sorts with sort_unstable_by, which leaves the order of equal logits open; here equal logits go by
// ascending index (the checker does the same).  Every sum the reference takes front to back in f32 is taken front to
// back in f32 here too (one warp walks the candidates 32 at a time and adds them in order), so that the comparisons
// `acc >= top_p` and `r < acc` see the same numbers as on the CPU up to the rounding of expf.  The random number comes
// from the caller's SplitMix64 state on the host (src/nn/rand.rs:29-41), advanced once per sampled token.
//
// The sort is cub::DeviceRadixSort on 64-bit keys (inverted order-preserving image of the logit in the high word, the
// index in the low word): library code, as the sampler is not on the step's critical path.
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"
#include "decode_ops.cuh"

namespace {

__global__ void sample_keys_kernel(const float* __restrict__ logits, uint32_t n, unsigned long long* __restrict__ keys) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t u = __float_as_uint(logits[i]);
  u ^= (u >> 31) ? 0xFFFFFFFFu : 0x80000000u;  // f32::total_cmp order as an ascending unsigned integer
  keys[i] = ((unsigned long long)(~u) << 32) | i;
}

// One warp.  `acc` sums are taken in candidate order: the 32 values of a chunk are added one after the other (every
// lane does the same additions, so all lanes hold the same running sum).
__global__ void __launch_bounds__(32) sample_walk_kernel(const float* __restrict__ logits, const unsigned long long* __restrict__ sorted, uint32_t n,
                                                         float temperature, float top_p, float r_unit, float* __restrict__ probs,
                                                         int32_t* __restrict__ token_out) {
  const int lane = threadIdx.x;
  const float m = logits[(uint32_t)sorted[0]];
  // p_i = exp((l_i - m) / T) and their sum
  float total = 0.0f;
  for (uint32_t i0 = 0; i0 < n; i0 += 32) {
    const uint32_t i = i0 + lane;
    float p = 0.0f;
    if (i < n) {
      p = expf((logits[(uint32_t)sorted[i]] - m) / temperature);
      probs[i] = p;
    }
    const uint32_t cnt = min(32u, n - i0);
    for (uint32_t j = 0; j < cnt; ++j) total += __shfl_sync(0xFFFFFFFFu, p, (int)j);
  }
  // normalise; the nucleus: the first position where the running sum reaches top_p
  uint32_t keep = n;
  float acc = 0.0f;
  bool cut = false;
  for (uint32_t i0 = 0; i0 < n && !cut; i0 += 32) {
    const uint32_t i = i0 + lane;
    float p = 0.0f;
    if (i < n) {
      p = probs[i] / total;
      probs[i] = p;
    }
    const uint32_t cnt = min(32u, n - i0);
    for (uint32_t j = 0; j < cnt; ++j) {
      acc += __shfl_sync(0xFFFFFFFFu, p, (int)j);
      if (top_p < 1.0f && acc >= top_p) { keep = i0 + j + 1; cut = true; break; }
    }
  }
  // acc is now the sum of the kept probabilities, added front to back as `probs.iter().sum()` does
  const float r = r_unit * acc;
  float run = 0.0f;
  uint32_t pick = keep - 1;
  bool found = false;
  for (uint32_t i0 = 0; i0 < keep && !found; i0 += 32) {
    const uint32_t i = i0 + lane;
    const float p = i < keep ? probs[i] : 0.0f;
    const uint32_t cnt = min(32u, keep - i0);
    for (uint32_t j = 0; j < cnt; ++j) {
      run += __shfl_sync(0xFFFFFFFFu, p, (int)j);
      if (r < run) { pick = i0 + j; found = true; break; }
    }
  }
  if (lane == 0) *token_out = (int32_t)(uint32_t)sorted[pick];
}

inline float splitmix_unit(uint64_t* state) {  // rand.rs:29-41
  *state += 0x9e3779b97f4a7c15ull;
  uint64_t z = *state;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  z ^= z >> 31;
  return (float)(z >> 40) / (float)(1ull << 24);
}

}  // namespace

int ruai_sample_device(ruai_ctx* c, const float* logits_dev, uint32_t vocab, float temperature, uint32_t top_k, float top_p, uint64_t* rng_state,
                       int32_t* token_dev) {
  if (temperature <= 0.0f) return ruai_argmax(c, logits_dev, vocab, 1, vocab, token_dev, 0);
  size_t temp_bytes = 0;
  unsigned long long* nullkeys = nullptr;
  RUAI_CUDA(c, cub::DeviceRadixSort::SortKeys(nullptr, temp_bytes, nullkeys, nullkeys, (int)vocab, 0, 64, c->stream));
  const size_t keys_bytes = ((size_t)vocab * 8 + 255) & ~(size_t)255, probs_bytes = ((size_t)vocab * 4 + 255) & ~(size_t)255;
  const size_t need = 2 * keys_bytes + probs_bytes + temp_bytes;
  if (need > c->sample_bytes) {
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    cudaFree(c->sample_buf);
    c->sample_buf = nullptr;
    c->sample_bytes = 0;
    RUAI_CUDA(c, cudaMalloc(&c->sample_buf, need));
    c->sample_bytes = need;
  }
  unsigned char* base = static_cast<unsigned char*>(c->sample_buf);
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(base);
  unsigned long long* sorted = reinterpret_cast<unsigned long long*>(base + keys_bytes);
  float* probs = reinterpret_cast<float*>(base + 2 * keys_bytes);
  void* temp = base + 2 * keys_bytes + probs_bytes;
  sample_keys_kernel<<<(vocab + 255) / 256, 256, 0, c->stream>>>(logits_dev, vocab, keys);
  RUAI_CUDA(c, cudaGetLastError());
  RUAI_CUDA(c, cub::DeviceRadixSort::SortKeys(temp, temp_bytes, keys, sorted, (int)vocab, 0, 64, c->stream));
  const uint32_t n = top_k > 0 ? std::min(top_k, vocab) : vocab;
  const float r = splitmix_unit(rng_state);
  sample_walk_kernel<<<1, 32, 0, c->stream>>>(logits_dev, sorted, n, temperature, top_p, r, probs, token_dev);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

RUAI_API int ruai_sample(ruai_ctx* c, const float* logits_dev, uint32_t vocab, float temperature, uint32_t top_k, float top_p, uint64_t* rng_state,
                         int32_t* token_host) {
  if (!c || !logits_dev || !rng_state || !token_host) return ruai_fail(c, RUAI_ERR_ARG, "ruai_sample: NULL argument");
  if (vocab == 0 || vocab > 0x7FFFFFFFu) return ruai_fail(c, RUAI_ERR_SHAPE, "ruai_sample: vocabulary of %u", vocab);
  DeviceGuard g(c->ordinal);
  int32_t* tok = nullptr;
  RUAI_CUDA(c, cudaMallocAsync(reinterpret_cast<void**>(&tok), sizeof(int32_t), c->stream));
  int rc = ruai_sample_device(c, logits_dev, vocab, temperature, top_k, top_p, rng_state, tok);
  if (rc == RUAI_OK) {
    cudaError_t e = cudaMemcpyAsync(token_host, tok, sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) rc = ruai_fail(c, RUAI_ERR_CUDA, "ruai_sample: %s", cudaGetErrorString(e));
  }
  cudaFreeAsync(tok, c->stream);
  return rc;
}
