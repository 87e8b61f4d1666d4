// TEST INFRASTRUCTURE — not part of the product.
//
// CPU restatement of ruai's quantized-inference path, used only as the checker
// for the CUDA library and as the timed CPU baseline.  The reference is Rust
// and cannot be compiled where this is built, so each function below restates
// the reference's algorithm and cites the file:line it follows (paths inside
// the ruai source tree).  Pinned against the closed-form definitions and the
// synthetic-pattern cases of the reference's own tests (tests/quant.rs:29-61,
// tests/devices.rs:444-502, tests/llama.rs:34-74).
//
// Build: g++ -O2 -ffp-contract=off -fopenmp -shared -fPIC (rustc neither fuses
// a*b+c nor relaxes IEEE division; f32::round is C roundf).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <omp.h>
#include <vector>

#include "../include/ruai_b200.h"
#include "../include/ruai_b200_synth.h"

#define ORC extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------
// Quantizer
// ---------------------------------------------------------------------------

// Linear::quantize_int8, src/nn/modules/layers.rs:112-129.
// scale[j] = max_i |W[i,j]| / 127 (1.0 when the column is all zero);
// q[i,j] = clamp(round(W[i,j] / scale[j]), -127, 127) as i8.
ORC void orc_quantize_int8(const float* w, uint32_t k, uint32_t n, int8_t* q, float* scale) {
  for (uint32_t j = 0; j < n; ++j) scale[j] = 0.0f;
  for (uint32_t i = 0; i < k; ++i)
    for (uint32_t j = 0; j < n; ++j) scale[j] = std::fmax(scale[j], std::fabs(w[(size_t)i * n + j]));
  for (uint32_t j = 0; j < n; ++j) scale[j] = scale[j] > 0.0f ? scale[j] / 127.0f : 1.0f;
#pragma omp parallel for schedule(static)
  for (uint32_t i = 0; i < k; ++i)
    for (uint32_t j = 0; j < n; ++j) {
      float r = std::roundf(w[(size_t)i * n + j] / scale[j]);
      r = std::fmin(std::fmax(r, -127.0f), 127.0f);
      q[(size_t)i * n + j] = (int8_t)r;
    }
}

// Linear::quantize_int4, src/nn/modules/layers.rs:139-165.
// Returns 1 on the reference's assert failure ("must be even and divide").
ORC int orc_quantize_int4(const float* w, uint32_t k, uint32_t n, uint32_t group, int8_t* packed, float* scale) {
  if (!(group >= 2 && group % 2 == 0 && k % group == 0)) return 1;
  const uint32_t groups = k / group;
  for (size_t t = 0; t < (size_t)groups * n; ++t) scale[t] = 0.0f;
  for (uint32_t l = 0; l < k; ++l) {
    float* s = scale + (size_t)(l / group) * n;
    for (uint32_t j = 0; j < n; ++j) s[j] = std::fmax(s[j], std::fabs(w[(size_t)l * n + j]));
  }
  for (size_t t = 0; t < (size_t)groups * n; ++t) scale[t] = scale[t] > 0.0f ? scale[t] / 7.0f : 1.0f;
  auto qv = [&](uint32_t l, uint32_t j) -> int8_t {
    float r = std::roundf(w[(size_t)l * n + j] / scale[(size_t)(l / group) * n + j]);
    r = std::fmin(std::fmax(r, -8.0f), 7.0f);
    return (int8_t)r;
  };
#pragma omp parallel for schedule(static)
  for (uint32_t r = 0; r < k / 2; ++r)
    for (uint32_t j = 0; j < n; ++j) {
      uint8_t lo = (uint8_t)qv(2 * r, j) & 0xF, hi = (uint8_t)qv(2 * r + 1, j) & 0xF;
      packed[(size_t)r * n + j] = (int8_t)(lo | (hi << 4));
    }
  return 0;
}

// nibble, src/nn/backend/cpu.rs:61-65 (same value as int4_value, backend/mod.rs:98-102).
static inline float nibble(int8_t b, bool hi) {
  return (float)(hi ? (int8_t)(b >> 4) : (int8_t)((int8_t)((uint8_t)b << 4) >> 4));
}

// CpuCore::dequant_int4, src/nn/backend/cpu.rs:1023-1033.
ORC void orc_dequant_int4(const int8_t* q, const float* sc, uint32_t k, uint32_t n, uint32_t group, float* w) {
#pragma omp parallel for schedule(static)
  for (uint32_t l = 0; l < k; ++l) {
    const float* s = sc + (size_t)(l / group) * n;
    for (uint32_t j = 0; j < n; ++j) w[(size_t)l * n + j] = nibble(q[(size_t)(l / 2) * n + j], l % 2 == 1) * s[j];
  }
}

// ---------------------------------------------------------------------------
// Quantized matmuls
// ---------------------------------------------------------------------------

// CpuCore::matmul_int8, src/nn/backend/cpu.rs:897-927.
// out[i,j] = scale[j] * sum_p x[i,p] * q[p,j]; column blocks of 256, p ascending,
// zero activations skipped, scale applied last.
ORC void orc_matmul_int8(const float* x, const int8_t* q, const float* sc, uint32_t m, uint32_t k, uint32_t n, float* out) {
  if ((size_t)m * n == 0) return;
  const uint32_t cw = std::min<uint32_t>(256, std::max<uint32_t>(n, 1));
  const uint32_t nblk = (n + cw - 1) / cw;
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t i = 0; i < m; ++i)
    for (uint32_t cb = 0; cb < nblk; ++cb) {
      const float* xr = x + (size_t)i * k;
      const uint32_t j0 = cb * cw, w = std::min(cw, n - j0);
      float* acc = out + (size_t)i * n + j0;
      for (uint32_t t = 0; t < w; ++t) acc[t] = 0.0f;
      for (uint32_t p = 0; p < k; ++p) {
        const float xv = xr[p];
        if (xv == 0.0f) continue;
        const int8_t* qr = q + (size_t)p * n + j0;
        for (uint32_t t = 0; t < w; ++t) acc[t] += xv * (float)qr[t];
      }
      for (uint32_t t = 0; t < w; ++t) acc[t] *= sc[j0 + t];
    }
}

// CpuCore::matmul_int4, src/nn/backend/cpu.rs:1035-1067.
// out[i,j] = sum_g scale[g,j] * (sum_{l in g} x[i,l] * nibble(l,j)).
ORC void orc_matmul_int4(const float* x, const int8_t* q, const float* sc, uint32_t m, uint32_t k, uint32_t n, uint32_t group, float* out) {
  if ((size_t)m * n == 0) return;
  const uint32_t cw = std::min<uint32_t>(256, std::max<uint32_t>(n, 1));
  const uint32_t nblk = (n + cw - 1) / cw;
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t i = 0; i < m; ++i)
    for (uint32_t cb = 0; cb < nblk; ++cb) {
      const float* xr = x + (size_t)i * k;
      const uint32_t j0 = cb * cw, w = std::min(cw, n - j0);
      float* acc = out + (size_t)i * n + j0;
      float part[256];
      for (uint32_t t = 0; t < w; ++t) acc[t] = 0.0f;
      for (uint32_t g = 0; g < k / group; ++g) {
        for (uint32_t t = 0; t < w; ++t) part[t] = 0.0f;
        for (uint32_t l = g * group; l < (g + 1) * group; ++l) {
          const float xv = xr[l];
          if (xv == 0.0f) continue;
          const int8_t* qr = q + (size_t)(l / 2) * n + j0;
          const bool hi = l % 2 == 1;
          for (uint32_t t = 0; t < w; ++t) part[t] += xv * nibble(qr[t], hi);
        }
        const float* s = sc + (size_t)g * n + j0;
        for (uint32_t t = 0; t < w; ++t) acc[t] += part[t] * s[t];
      }
    }
}

// ---------------------------------------------------------------------------
// Decode-step functions
// ---------------------------------------------------------------------------

// F::rms_norm, src/nn/functional.rs:151-165: y = x * (1/sqrt(mean(x^2)+eps)) * w,
// mean = sum * (1/n) (Tensor::mean, src/nn/ops.rs:397-400).
ORC void orc_rms_norm(const float* x, const float* w, uint32_t rows, uint32_t d, float eps, float* y) {
  for (uint32_t r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * d;
    float s = 0.0f;
    for (uint32_t i = 0; i < d; ++i) s += xr[i] * xr[i];
    const float rstd = 1.0f / std::sqrt(s * (1.0f / (float)d) + eps);
    for (uint32_t i = 0; i < d; ++i) {
      float v = xr[i] * rstd;
      y[(size_t)r * d + i] = w ? v * w[i] : v;
    }
  }
}

// F::layer_norm, src/nn/functional.rs:137-146 over CpuCore::layer_norm,
// src/nn/backend/cpu.rs:855-876: two-pass mean, biased variance.
ORC void orc_layer_norm(const float* x, const float* w, const float* b, uint32_t rows, uint32_t d, float eps, float* y) {
  for (uint32_t r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * d;
    float s = 0.0f;
    for (uint32_t i = 0; i < d; ++i) s += xr[i];
    const float mean = s / (float)d;
    float v = 0.0f;
    for (uint32_t i = 0; i < d; ++i) v += (xr[i] - mean) * (xr[i] - mean);
    const float rstd = 1.0f / std::sqrt(v / (float)d + eps);
    for (uint32_t i = 0; i < d; ++i) {
      float t = (xr[i] - mean) * rstd;
      if (w) t = t * w[i];
      if (b) t = t + b[i];
      y[(size_t)r * d + i] = t;
    }
  }
}

// gelu with fast_tanh, src/nn/backend/cpu.rs:229-239.
static inline float fast_tanh(float u) {
  u = std::fmin(std::fmax(u, -15.0f), 15.0f);
  return 1.0f - 2.0f / (std::exp(2.0f * u) + 1.0f);
}
static inline float gelu(float x) {
  const float S = 0.7978846f;
  return 0.5f * x * (1.0f + fast_tanh(S * (x + 0.044715f * x * x * x)));
}
ORC void orc_gelu(const float* x, size_t n, float* y) {
  for (size_t i = 0; i < n; ++i) y[i] = gelu(x[i]);
}
// Tensor::silu = x * sigmoid(x), src/nn/ops.rs:158-160; sigmoid cpu.rs:376.
static inline float silu(float v) { return v * (1.0f / (1.0f + std::exp(-v))); }

// F::rope_inv_freq, src/nn/functional.rs:168-171.
ORC void orc_rope_inv_freq(uint32_t head_dim, float theta, float* inv) {
  for (uint32_t i = 0; i < head_dim / 2; ++i) inv[i] = std::pow(theta, -((float)(2 * i)) / (float)head_dim);
}
// F::rope_cos_sin, src/nn/functional.rs:176-192: f64 angles, halves duplicated.
ORC void orc_rope_cos_sin(const float* inv, uint32_t half, uint32_t start, uint32_t t, float* cosv, float* sinv) {
  const uint32_t d = 2 * half;
  for (uint32_t p = 0; p < t; ++p)
    for (uint32_t i = 0; i < half; ++i) {
      const double a = (double)(start + p) * (double)inv[i];
      const float c = (float)std::cos(a), s = (float)std::sin(a);
      cosv[p * d + i] = c; cosv[p * d + i + half] = c;
      sinv[p * d + i] = s; sinv[p * d + i + half] = s;
    }
}
// F::apply_rope, src/nn/functional.rs:197-204: x*cos + rotate_half(x)*sin,
// rotate_half([x1,x2]) = [-x2, x1].  One vector of length d, in place.
ORC void orc_apply_rope(float* x, const float* cosv, const float* sinv, uint32_t d) {
  const uint32_t half = d / 2;
  float tmp[512];
  for (uint32_t i = 0; i < d; ++i) {
    const float rot = i < half ? -x[i + half] : x[i - half];
    tmp[i] = x[i] * cosv[i] + rot * sinv[i];
  }
  std::memcpy(x, tmp, d * sizeof(float));
}

// attention_composed, src/nn/functional.rs:281-296:
// softmax(q k^T * (1/sqrt(d)) + mask) v for one (batch, head) pair.
// q [tq,d], k/v [tk,d] with row stride d; causal mask with `past` cached
// positions (causal_mask_offset, functional.rs:238-247), applied only when
// use_mask (the models pass a mask only for t > 1: llama.rs:269, gpt2.rs:117).
static void attention_head(const float* q, const float* k, const float* v, uint32_t tq, uint32_t tk, uint32_t d,
                           uint32_t past, bool use_mask, float* o, std::vector<float>& sc) {
  const float scale = 1.0f / std::sqrt((float)d);
  sc.resize(tk);
  for (uint32_t i = 0; i < tq; ++i) {
    float mx = -INFINITY;
    for (uint32_t j = 0; j < tk; ++j) {
      float s = 0.0f;
      for (uint32_t c = 0; c < d; ++c) s += q[(size_t)i * d + c] * k[(size_t)j * d + c];
      s = s * scale;
      if (use_mask && j > past + i) s = s + -1e9f;
      sc[j] = s;
      mx = std::fmax(mx, s);
    }
    float sum = 0.0f;
    for (uint32_t j = 0; j < tk; ++j) { sc[j] = std::exp(sc[j] - mx); sum += sc[j]; }
    for (uint32_t c = 0; c < d; ++c) o[(size_t)i * d + c] = 0.0f;
    for (uint32_t j = 0; j < tk; ++j) {
      const float p = sc[j] / sum;
      for (uint32_t c = 0; c < d; ++c) o[(size_t)i * d + c] += p * v[(size_t)j * d + c];
    }
  }
}
ORC void orc_attention(const float* q, const float* k, const float* v, uint32_t tq, uint32_t tk, uint32_t d,
                       uint32_t past, int use_mask, float* o) {
  std::vector<float> sc;
  attention_head(q, k, v, tq, tk, d, past, use_mask != 0, o, sc);
}

// argmax, src/nn/generation.rs:6-8: max_by(total_cmp) keeps the LAST maximum.
ORC uint32_t orc_argmax(const float* logits, uint32_t n) {
  uint32_t best = 0;
  for (uint32_t i = 1; i < n; ++i) {
    // total_cmp order for non-NaN values equals numeric order except -0 < +0.
    const float a = logits[i], b = logits[best];
    int32_t ia, ib;
    std::memcpy(&ia, &a, 4); std::memcpy(&ib, &b, 4);
    ia ^= (int32_t)(((uint32_t)(ia >> 31)) >> 1);
    ib ^= (int32_t)(((uint32_t)(ib >> 31)) >> 1);
    if (ia >= ib) best = i;
  }
  return best;
}

// ---------------------------------------------------------------------------
// Synthetic tensors (include/ruai_b200_synth.h)
// ---------------------------------------------------------------------------
ORC void orc_synth_normal(uint64_t seed, uint64_t tensor_id, size_t count, double std_dev, float* out) {
  const uint64_t key = ruai_synth_key(seed, tensor_id);
  const float mult = ruai_synth_mult(std_dev);
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < count; ++i) out[i] = ruai_synth_normal(key, i, mult);
}
ORC void orc_synth_tokens(uint64_t seed, uint64_t tensor_id, size_t count, uint32_t vocab, int32_t* out) {
  const uint64_t key = ruai_synth_key(seed, tensor_id);
  for (size_t i = 0; i < count; ++i) out[i] = ruai_synth_token(key, i, vocab);
}

// ---------------------------------------------------------------------------
// Models
// ---------------------------------------------------------------------------
namespace {

struct QLinear {  // Linear after quantize_int8 / quantize_int4 (layers.rs:24-41)
  uint32_t k = 0, n = 0, bits = 0, group = 0;
  std::vector<int8_t> q;
  std::vector<float> scale, bias;
  // Linear::forward, layers.rs:169-190: quantized matmul then bias.
  void forward(const float* x, uint32_t m, float* y) const {
    if (bits == 8) orc_matmul_int8(x, q.data(), scale.data(), m, k, n, y);
    else orc_matmul_int4(x, q.data(), scale.data(), m, k, n, group, y);
    if (!bias.empty())
      for (uint32_t i = 0; i < m; ++i)
        for (uint32_t j = 0; j < n; ++j) y[(size_t)i * n + j] += bias[j];
  }
  void quantize(const std::vector<float>& w, uint32_t k_, uint32_t n_, uint32_t bits_, uint32_t group_) {
    k = k_; n = n_; bits = bits_; group = bits_ == 4 ? group_ : 0;
    if (bits == 8) { q.resize((size_t)k * n); scale.resize(n); orc_quantize_int8(w.data(), k, n, q.data(), scale.data()); }
    else { q.resize((size_t)k / 2 * n); scale.resize((size_t)(k / group) * n); orc_quantize_int4(w.data(), k, n, group, q.data(), scale.data()); }
  }
};

// KvBuf / LayerKv, src/nn/modules/transformer.rs:10-128: per layer K and V
// [B, H_kv, cap, hd], capacity max(need, 2*cap, 16), append in place.
struct LayerKv {
  std::vector<float> k, v;
  uint32_t cap = 0;
};

struct Model {
  bool is_llama = true;
  ruai_llama_config lc{};
  ruai_gpt2_config gc{};
  uint32_t L = 0, d = 0, H = 0, KV = 0, hd = 0, ffn = 0, V = 0, max_pos = 0;
  std::vector<float> embed, wpe, final_w, final_b, inv_freq;
  struct Layer {
    std::vector<float> n1w, n1b, n2w, n2b;
    QLinear q, k, v, o, gate, up, down;   // llama
    QLinear c_attn, c_proj, c_fc, m_proj; // gpt2
  };
  std::vector<Layer> layers;
  QLinear head;
  // cache
  std::vector<LayerKv> kv;
  uint32_t len = 0, B = 0;
};

std::vector<float> synth(uint64_t seed, uint64_t id, size_t count, double sd) {
  std::vector<float> v(count);
  orc_synth_normal(seed, id, count, sd, v.data());
  return v;
}

void kv_append(LayerKv& c, uint32_t B, uint32_t KV, uint32_t hd, uint32_t len, uint32_t t) {
  const uint32_t need = len + t;
  if (c.cap >= need) return;
  const uint32_t cap = std::max(std::max(need, 2 * c.cap), 16u);
  std::vector<float> nk((size_t)B * KV * cap * hd, 0.0f), nv(nk.size(), 0.0f);
  for (uint32_t bh = 0; bh < B * KV; ++bh)
    for (uint32_t p = 0; p < len; ++p)
      for (uint32_t c2 = 0; c2 < hd; ++c2) {
        nk[((size_t)bh * cap + p) * hd + c2] = c.k[((size_t)bh * c.cap + p) * hd + c2];
        nv[((size_t)bh * cap + p) * hd + c2] = c.v[((size_t)bh * c.cap + p) * hd + c2];
      }
  c.k.swap(nk); c.v.swap(nv); c.cap = cap;
}

// Attention::forward, src/nn/modules/llama.rs:248-277 (rope = true) and
// src/nn/modules/gpt2.rs:102-121 (rope = false).  q [B,T,H*hd], k/v [B,T,KV*hd]
// are the projections; out [B,T,H*hd] is the input of o_proj / c_proj.
void attend(Model& M, uint32_t layer, uint32_t B, uint32_t T, const float* q, uint32_t qs, const float* k,
            uint32_t ks, const float* v, uint32_t vs, bool rope, float* out) {
  const uint32_t H = M.H, KV = M.KV, hd = M.hd, rep = H / KV, past = M.len;
  LayerKv& c = M.kv[layer];
  kv_append(c, B, KV, hd, past, T);
  std::vector<float> cosv, sinv;
  if (rope) { cosv.resize((size_t)T * hd); sinv.resize((size_t)T * hd); orc_rope_cos_sin(M.inv_freq.data(), hd / 2, past, T, cosv.data(), sinv.data()); }
  // write new keys / values (keys rotated) into the cache
  for (uint32_t b = 0; b < B; ++b)
    for (uint32_t t = 0; t < T; ++t)
      for (uint32_t h = 0; h < KV; ++h) {
        float* kd = &c.k[(((size_t)b * KV + h) * c.cap + past + t) * hd];
        float* vd = &c.v[(((size_t)b * KV + h) * c.cap + past + t) * hd];
        std::memcpy(kd, k + ((size_t)b * T + t) * ks + (size_t)h * hd, hd * sizeof(float));
        std::memcpy(vd, v + ((size_t)b * T + t) * vs + (size_t)h * hd, hd * sizeof(float));
        if (rope) orc_apply_rope(kd, &cosv[(size_t)t * hd], &sinv[(size_t)t * hd], hd);
      }
  const uint32_t tk = past + T;
#pragma omp parallel
  {
    std::vector<float> sc, qh((size_t)T * hd), oh((size_t)T * hd);
#pragma omp for collapse(2) schedule(static)
    for (uint32_t b = 0; b < B; ++b)
      for (uint32_t h = 0; h < H; ++h) {
        for (uint32_t t = 0; t < T; ++t) {
          std::memcpy(&qh[(size_t)t * hd], q + ((size_t)b * T + t) * qs + (size_t)h * hd, hd * sizeof(float));
          if (rope) orc_apply_rope(&qh[(size_t)t * hd], &cosv[(size_t)t * hd], &sinv[(size_t)t * hd], hd);
        }
        const uint32_t g = h / rep;  // query head h reads KV head h / rep (llama.rs:264-268)
        attention_head(qh.data(), &c.k[((size_t)b * KV + g) * c.cap * hd], &c.v[((size_t)b * KV + g) * c.cap * hd], T, tk, hd,
                       past, T > 1, oh.data(), sc);
        for (uint32_t t = 0; t < T; ++t)
          std::memcpy(out + ((size_t)b * T + t) * (H * hd) + (size_t)h * hd, &oh[(size_t)t * hd], hd * sizeof(float));
      }
  }
}

// Llama::run, src/nn/modules/llama.rs:441-463; DecoderLayer::forward 306-309;
// SwiGLU::forward, layers.rs:573-576.  GPT2::run, gpt2.rs:221-241; Block::forward 142-146.
int forward_cached(Model& M, const int32_t* ids, uint32_t B, uint32_t T, float* logits, bool all_pos) {
  if (M.len == 0 && B != M.B) {  // a new batch shape starts new buffers (transformer.rs:31-32)
    for (auto& c : M.kv) { c.k.clear(); c.v.clear(); c.cap = 0; }
    M.B = B;
  }
  if (B != M.B || M.len + T > M.max_pos) return 1;
  const uint32_t d = M.d, m = B * T;
  std::vector<float> x((size_t)m * d), xn((size_t)m * d), tmp((size_t)m * d);
  for (uint32_t r = 0; r < m; ++r) {
    const int32_t id = ids[r];
    if (id < 0 || (uint32_t)id >= M.V) return 2;
    std::memcpy(&x[(size_t)r * d], &M.embed[(size_t)id * d], d * sizeof(float));
    if (!M.is_llama) {
      const uint32_t pos = M.len + r % T;
      for (uint32_t i = 0; i < d; ++i) x[(size_t)r * d + i] += M.wpe[(size_t)pos * d + i];
    }
  }
  for (uint32_t l = 0; l < M.L; ++l) {
    Model::Layer& Ly = M.layers[l];
    if (M.is_llama) {
      orc_rms_norm(x.data(), Ly.n1w.data(), m, d, M.lc.rms_norm_eps, xn.data());
      const uint32_t nq = M.H * M.hd, nkv = M.KV * M.hd;
      std::vector<float> q((size_t)m * nq), k((size_t)m * nkv), v((size_t)m * nkv), a((size_t)m * nq);
      Ly.q.forward(xn.data(), m, q.data()); Ly.k.forward(xn.data(), m, k.data()); Ly.v.forward(xn.data(), m, v.data());
      attend(M, l, B, T, q.data(), nq, k.data(), nkv, v.data(), nkv, true, a.data());
      Ly.o.forward(a.data(), m, tmp.data());
      for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + tmp[i];
      orc_rms_norm(x.data(), Ly.n2w.data(), m, d, M.lc.rms_norm_eps, xn.data());
      std::vector<float> g((size_t)m * M.ffn), u((size_t)m * M.ffn);
      Ly.gate.forward(xn.data(), m, g.data()); Ly.up.forward(xn.data(), m, u.data());
      for (size_t i = 0; i < g.size(); ++i) g[i] = silu(g[i]) * u[i];
      Ly.down.forward(g.data(), m, tmp.data());
      for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + tmp[i];
    } else {
      orc_layer_norm(x.data(), Ly.n1w.data(), Ly.n1b.data(), m, d, 1e-5f, xn.data());
      std::vector<float> qkv((size_t)m * 3 * d), a((size_t)m * d);
      Ly.c_attn.forward(xn.data(), m, qkv.data());
      attend(M, l, B, T, qkv.data(), 3 * d, qkv.data() + d, 3 * d, qkv.data() + 2 * d, 3 * d, false, a.data());
      Ly.c_proj.forward(a.data(), m, tmp.data());
      for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + tmp[i];
      orc_layer_norm(x.data(), Ly.n2w.data(), Ly.n2b.data(), m, d, 1e-5f, xn.data());
      std::vector<float> h((size_t)m * M.ffn);
      Ly.c_fc.forward(xn.data(), m, h.data());
      for (size_t i = 0; i < h.size(); ++i) h[i] = gelu(h[i]);
      Ly.m_proj.forward(h.data(), m, tmp.data());
      for (size_t i = 0; i < x.size(); ++i) x[i] = x[i] + tmp[i];
    }
  }
  M.len += T;
  if (M.is_llama) orc_rms_norm(x.data(), M.final_w.data(), m, d, M.lc.rms_norm_eps, xn.data());
  else orc_layer_norm(x.data(), M.final_w.data(), M.final_b.data(), m, d, 1e-5f, xn.data());
  if (logits) {
    if (all_pos) M.head.forward(xn.data(), m, logits);
    else {
      // the reference computes every position (llama.rs:457-462) and generate
      // keeps the last row (generation.rs:103-104); rows are independent.
      std::vector<float> last((size_t)B * d);
      for (uint32_t b = 0; b < B; ++b) std::memcpy(&last[(size_t)b * d], &xn[((size_t)b * T + T - 1) * d], d * sizeof(float));
      M.head.forward(last.data(), B, logits);
    }
  }
  return 0;
}

}  // namespace

// Llama::new + quantize_int8 / quantize_int4(group) (llama.rs:522-554) over the
// seeded synthetic weights; n_layers_override > 0 builds a layer-reduced model.
ORC void* orc_llama_create(const ruai_llama_config* c, uint64_t seed, uint32_t bits, uint32_t group) {
  Model* M = new Model();
  M->is_llama = true; M->lc = *c;
  M->L = c->num_hidden_layers; M->d = c->hidden_size; M->H = c->num_attention_heads; M->KV = c->num_key_value_heads;
  M->hd = c->head_dim; M->ffn = c->intermediate_size; M->V = c->vocab_size; M->max_pos = c->max_position_embeddings;
  const uint32_t d = M->d, nq = M->H * M->hd, nkv = M->KV * M->hd, f = M->ffn;
  M->embed = synth(seed, RUAI_T_EMBED, (size_t)M->V * d, 0.02);
  M->final_w.assign(d, 1.0f);
  M->inv_freq.resize(M->hd / 2); orc_rope_inv_freq(M->hd, c->rope_theta, M->inv_freq.data());
  M->layers.resize(M->L); M->kv.resize(M->L);
  for (uint32_t l = 0; l < M->L; ++l) {
    auto& Ly = M->layers[l];
    Ly.n1w.assign(d, 1.0f); Ly.n2w.assign(d, 1.0f);
    Ly.q.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_Q), (size_t)d * nq, 0.02), d, nq, bits, group);
    Ly.k.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_K), (size_t)d * nkv, 0.02), d, nkv, bits, group);
    Ly.v.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_V), (size_t)d * nkv, 0.02), d, nkv, bits, group);
    Ly.o.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_O), (size_t)nq * d, 0.02), nq, d, bits, group);
    Ly.gate.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_GATE), (size_t)d * f, 0.02), d, f, bits, group);
    Ly.up.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_UP), (size_t)d * f, 0.02), d, f, bits, group);
    Ly.down.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_DOWN), (size_t)f * d, 0.02), f, d, bits, group);
  }
  // quantize_head_int8, llama.rs:544-554: untied lm_head, or the transposed embedding.
  std::vector<float> hw;
  if (c->tie_word_embeddings) {
    hw.resize((size_t)d * M->V);
    for (uint32_t t = 0; t < M->V; ++t)
      for (uint32_t i = 0; i < d; ++i) hw[(size_t)i * M->V + t] = M->embed[(size_t)t * d + i];
  } else hw = synth(seed, RUAI_T_LMHEAD, (size_t)d * M->V, 0.02);
  M->head.quantize(hw, d, M->V, 8, 0);
  return M;
}

// GPT2::new + quantize_int8 / quantize_int4 (gpt2.rs:306-335).
ORC void* orc_gpt2_create(const ruai_gpt2_config* c, uint64_t seed, uint32_t bits, uint32_t group) {
  Model* M = new Model();
  M->is_llama = false; M->gc = *c;
  M->L = c->n_layer; M->d = c->n_embd; M->H = c->n_head; M->KV = c->n_head; M->hd = c->n_embd / c->n_head;
  M->ffn = 4 * c->n_embd; M->V = c->vocab_size; M->max_pos = c->n_positions;
  const uint32_t d = M->d, f = M->ffn;
  M->embed = synth(seed, RUAI_T_EMBED, (size_t)M->V * d, 0.02);
  M->wpe = synth(seed, RUAI_T_WPE, (size_t)M->max_pos * d, 0.02);
  M->final_w.assign(d, 1.0f); M->final_b.assign(d, 0.0f);
  M->layers.resize(M->L); M->kv.resize(M->L);
  for (uint32_t l = 0; l < M->L; ++l) {
    auto& Ly = M->layers[l];
    Ly.n1w.assign(d, 1.0f); Ly.n1b.assign(d, 0.0f); Ly.n2w.assign(d, 1.0f); Ly.n2b.assign(d, 0.0f);
    Ly.c_attn.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_CATTN), (size_t)d * 3 * d, 0.02), d, 3 * d, bits, group);
    Ly.c_attn.bias = synth(seed, ruai_layer_tensor(l, RUAI_T_CATTN_B), 3 * d, 0.02);
    Ly.c_proj.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_CPROJ), (size_t)d * d, 0.02), d, d, bits, group);
    Ly.c_proj.bias = synth(seed, ruai_layer_tensor(l, RUAI_T_CPROJ_B), d, 0.02);
    Ly.c_fc.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_CFC), (size_t)d * f, 0.02), d, f, bits, group);
    Ly.c_fc.bias = synth(seed, ruai_layer_tensor(l, RUAI_T_CFC_B), f, 0.02);
    Ly.m_proj.quantize(synth(seed, ruai_layer_tensor(l, RUAI_T_MPROJ), (size_t)f * d, 0.02), f, d, bits, group);
    Ly.m_proj.bias = synth(seed, ruai_layer_tensor(l, RUAI_T_MPROJ_B), d, 0.02);
  }
  std::vector<float> hw((size_t)d * M->V);
  for (uint32_t t = 0; t < M->V; ++t)
    for (uint32_t i = 0; i < d; ++i) hw[(size_t)i * M->V + t] = M->embed[(size_t)t * d + i];
  M->head.quantize(hw, d, M->V, 8, 0);
  return M;
}

ORC void orc_model_destroy(void* h) { delete (Model*)h; }

// Threads the OpenMP loops of this library use, and a way to set them (a launcher may have exported
// OMP_NUM_THREADS=1 for its children).
ORC int orc_threads(void) { return omp_get_max_threads(); }
ORC void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }

// Pretends `len` positions are cached for batch B (zero keys and values): times a decode step at a given
// context without running the prompt.  Same capacity rule as an append of `len` positions.
ORC int orc_model_cache_assume(void* h, uint32_t B, uint32_t len) {
  Model* M = (Model*)h;
  if (len + 1 > M->max_pos) return 1;
  for (auto& c : M->kv) { c.k.clear(); c.v.clear(); c.cap = 0; }
  M->B = B; M->len = 0;
  for (auto& c : M->kv) kv_append(c, B, M->KV, M->hd, 0, len + 1);
  M->len = len;
  return 0;
}
ORC void orc_model_cache_clear(void* h) { Model* M = (Model*)h; M->len = 0; }
ORC uint32_t orc_model_cache_len(void* h) { return ((Model*)h)->len; }
ORC uint32_t orc_model_cache_capacity(void* h) { return ((Model*)h)->kv.empty() ? 0 : ((Model*)h)->kv[0].cap; }
ORC int orc_model_forward_cached(void* h, const int32_t* ids, uint32_t B, uint32_t T, float* logits, int all_pos) {
  return forward_cached(*(Model*)h, ids, B, T, logits, all_pos != 0);
}

// Read one quantized Linear of the model in the reference's buffer layout.
// which: layer * 16 + kind (include/ruai_b200_synth.h) or RUAI_T_LMHEAD.
ORC int orc_model_get_linear(void* h, uint64_t id, int8_t* q, float* scale, uint32_t* k, uint32_t* n) {
  Model* M = (Model*)h;
  const QLinear* L = nullptr;
  if (id == RUAI_T_LMHEAD) L = &M->head;
  else {
    const uint32_t l = (uint32_t)(id / 16), kind = (uint32_t)(id % 16);
    if (l >= M->L) return 1;
    auto& Ly = M->layers[l];
    const QLinear* tab[11] = {&Ly.q, &Ly.k, &Ly.v, &Ly.o, &Ly.gate, &Ly.up, &Ly.down, &Ly.c_attn, &Ly.c_proj, &Ly.c_fc, &Ly.m_proj};
    if (kind > 10) return 1;
    L = tab[kind];
  }
  if (k) *k = L->k;
  if (n) *n = L->n;
  if (q) std::memcpy(q, L->q.data(), L->q.size());
  if (scale) std::memcpy(scale, L->scale.data(), L->scale.size() * sizeof(float));
  return 0;
}

// Rng::next_u64 / Rng::unit, src/nn/rand.rs:29-41 (SplitMix64; 24 random bits).
static float rng_unit(uint64_t* state) {
  *state += 0x9e3779b97f4a7c15ull;
  uint64_t z = *state;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  z ^= z >> 31;
  return (float)(z >> 40) / (float)(1ull << 24);
}
ORC float orc_rng_unit(uint64_t* state) { return rng_unit(state); }

// Sampler::sample, src/nn/generation.rs:38-73.  The reference's sort_unstable_by leaves the order of equal logits
// open; equal logits go by ascending index here.  margin (optional) receives the smallest distance, in probability
// mass, between a comparison the sampler made and its threshold at the position it decided on (top_p cut, draw): a draw
// whose margin is below the rounding differences of exp may fall the other way on another implementation.
ORC uint32_t orc_sample(const float* logits, uint32_t n, float temperature, uint32_t top_k, float top_p, uint64_t* state, float* margin) {
  if (margin) *margin = 1.0f;
  if (temperature <= 0.0f) return orc_argmax(logits, n);
  auto key = [&](uint32_t i) {
    int32_t b;
    std::memcpy(&b, &logits[i], 4);
    return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);  // total_cmp
  };
  std::vector<uint32_t> idx(n);
  for (uint32_t i = 0; i < n; ++i) idx[i] = i;
  std::sort(idx.begin(), idx.end(), [&](uint32_t a, uint32_t b) {
    const int32_t ka = key(a), kb = key(b);
    return ka != kb ? ka > kb : a < b;
  });
  if (top_k > 0) idx.resize(std::min<size_t>(top_k, idx.size()));
  const float m = logits[idx[0]];
  std::vector<float> probs(idx.size());
  for (size_t i = 0; i < idx.size(); ++i) probs[i] = std::exp((logits[idx[i]] - m) / temperature);
  float total = 0.0f;
  for (float p : probs) total += p;
  for (float& p : probs) p /= total;
  float mg = 1.0f;
  if (top_p < 1.0f) {
    float acc = 0.0f;
    size_t keep = probs.size();
    for (size_t i = 0; i < probs.size(); ++i) {
      const float before = acc;
      acc += probs[i];
      if (acc >= top_p) {
        keep = i + 1;
        mg = std::min(mg, std::min(acc - top_p, top_p - before));
        break;
      }
    }
    probs.resize(keep);
    idx.resize(keep);
  }
  float sum = 0.0f;
  for (float p : probs) sum += p;
  const float r = rng_unit(state) * sum;
  float acc = 0.0f;
  uint32_t pick = idx.back();
  for (size_t i = 0; i < probs.size(); ++i) {
    const float before = acc;
    acc += probs[i];
    if (r < acc) {
      pick = idx[i];
      mg = std::min(mg, std::min(acc - r, r - before));
      break;
    }
  }
  if (margin) *margin = mg;
  return pick;
}

// generate_cached with Sampler::greedy, src/nn/generation.rs:83-113.
// out receives T + n ids; logits_trace (optional) receives the n logit rows.
static int generate_with(void* h, const int32_t* prompt, uint32_t T, uint32_t n, int32_t* out, float* logits_trace, bool sampled, float temperature,
                         uint32_t top_k, float top_p, uint64_t seed, float* margins);
ORC int orc_model_generate(void* h, const int32_t* prompt, uint32_t T, uint32_t n, int32_t* out, float* logits_trace) {
  return generate_with(h, prompt, T, n, out, logits_trace, false, 0.0f, 0, 1.0f, 0, nullptr);
}
// generate_cached with Sampler::new(temperature, top_k, top_p, seed); margins (optional) [n]: see orc_sample.
ORC int orc_model_generate_sampled(void* h, const int32_t* prompt, uint32_t T, uint32_t n, float temperature, uint32_t top_k, float top_p, uint64_t seed,
                                   int32_t* out, float* margins) {
  return generate_with(h, prompt, T, n, out, nullptr, true, temperature, top_k, top_p, seed, margins);
}
static int generate_with(void* h, const int32_t* prompt, uint32_t T, uint32_t n, int32_t* out, float* logits_trace, bool sampled, float temperature,
                         uint32_t top_k, float top_p, uint64_t seed, float* margins) {
  Model* M = (Model*)h;
  uint64_t state = seed;
  if (T == 0) return 1;
  const uint32_t max_len = M->max_pos;
  std::vector<int32_t> ids(prompt, prompt + T);
  M->len = 0;
  std::vector<int32_t> pending(ids.begin() + (ids.size() > max_len ? ids.size() - max_len : 0), ids.end());
  std::vector<float> logits(M->V);
  for (uint32_t s = 0; s < n; ++s) {
    if (M->len + pending.size() > max_len) {
      M->len = 0;
      pending.assign(ids.end() - max_len, ids.end());
    }
    int rc = forward_cached(*M, pending.data(), 1, (uint32_t)pending.size(), logits.data(), false);
    if (rc) return rc;
    if (logits_trace) std::memcpy(logits_trace + (size_t)s * M->V, logits.data(), M->V * sizeof(float));
    float mg = 1.0f;
    const int32_t next = sampled ? (int32_t)orc_sample(logits.data(), M->V, temperature, top_k, top_p, &state, &mg) : (int32_t)orc_argmax(logits.data(), M->V);
    if (margins) margins[s] = mg;
    ids.push_back(next);
    pending.assign(1, next);
  }
  std::memcpy(out, ids.data(), ids.size() * sizeof(int32_t));
  return 0;
}
