/* Deterministic synthetic tensors shared by the CUDA library and the CPU checker.
 *
 * The benchmark configurations use random-initialised weights ~N(0, 0.02^2) and
 * uniform token ids from a fixed seed; no checkpoint or tokenizer is involved.
 * To make "the same seeded input" mean bit-identical f32 values on the host and
 * on the device, the generator uses integer hashing only: twelve 16-bit uniform
 * fields are summed (Irwin-Hall, n = 12; support +-6 sigma, excess kurtosis -0.1)
 * and the centred integer is multiplied once by an f32 constant.  No libm call
 * is involved, so host and device agree to the last bit.
 *
 * Everything here is `static inline` and compiles as C, C++ and CUDA.
 */
#ifndef RUAI_B200_SYNTH_H
#define RUAI_B200_SYNTH_H

#include <stdint.h>

#if defined(__CUDACC__)
#define RUAI_HD __host__ __device__ static inline
#else
#define RUAI_HD static inline
#endif

/* SplitMix64 finaliser (public-domain mixing function). */
RUAI_HD uint64_t ruai_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

/* Key of one tensor: a function of the run seed and a tensor id. */
RUAI_HD uint64_t ruai_synth_key(uint64_t seed, uint64_t tensor_id) {
  return ruai_mix64(seed * 0xD6E8FEB86659FD93ull + tensor_id);
}

/* Centred sum of twelve 16-bit uniforms: an integer in [-393210, 393210]. */
RUAI_HD int32_t ruai_synth_isum(uint64_t key, uint64_t idx) {
  uint32_t s = 0;
  for (int r = 0; r < 3; ++r) {
    uint64_t h = ruai_mix64(key + 3ull * idx + (uint64_t)r);
    s += (uint32_t)(h & 0xFFFF) + (uint32_t)((h >> 16) & 0xFFFF) +
         (uint32_t)((h >> 32) & 0xFFFF) + (uint32_t)(h >> 48);
  }
  /* 12 * 32767.5 = 393210 */
  return (int32_t)s - 393210;
}

/* Standard deviation of the integer sum: sqrt(12 * (65536^2 - 1) / 12). */
#define RUAI_SYNTH_ISUM_SIGMA 65535.99999237060546875

/* f32 multiplier that turns the integer sum into N(0, std^2).  Computed in
 * double on the host and rounded once, then passed to whoever generates. */
static inline float ruai_synth_mult(double std_dev) {
  return (float)(std_dev / RUAI_SYNTH_ISUM_SIGMA);
}

/* One element of a synthetic normal tensor. */
RUAI_HD float ruai_synth_normal(uint64_t key, uint64_t idx, float mult) {
  return (float)ruai_synth_isum(key, idx) * mult;
}

/* One synthetic token id in [0, vocab). */
RUAI_HD int32_t ruai_synth_token(uint64_t key, uint64_t idx, uint32_t vocab) {
  return (int32_t)(ruai_mix64(key + idx) % (uint64_t)vocab);
}

/* Tensor ids of the model weights.  Layer tensors: layer * 16 + kind. */
enum {
  RUAI_T_Q = 0, RUAI_T_K = 1, RUAI_T_V = 2, RUAI_T_O = 3,
  RUAI_T_GATE = 4, RUAI_T_UP = 5, RUAI_T_DOWN = 6,
  /* GPT-2 block tensors */
  RUAI_T_CATTN = 7, RUAI_T_CPROJ = 8, RUAI_T_CFC = 9, RUAI_T_MPROJ = 10,
  RUAI_T_CATTN_B = 11, RUAI_T_CPROJ_B = 12, RUAI_T_CFC_B = 13, RUAI_T_MPROJ_B = 14
};
#define RUAI_T_EMBED   0x10000000ull /* token embedding [vocab, d] */
#define RUAI_T_LMHEAD  0x10000001ull /* untied head [d, vocab] */
#define RUAI_T_WPE     0x10000002ull /* GPT-2 position embedding [n_pos, d] */
#define RUAI_T_PROMPT  0x20000000ull /* + sequence index: prompt token ids */
#define RUAI_T_INPUT   0x30000000ull /* microbenchmark activations */

RUAI_HD uint64_t ruai_layer_tensor(uint32_t layer, uint32_t kind) {
  return (uint64_t)layer * 16ull + (uint64_t)kind;
}

#endif /* RUAI_B200_SYNTH_H */
