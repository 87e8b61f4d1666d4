// Host-callable launchers of decode_ops.cu and quantize.cu used by the model code.
#pragma once
#include "common.cuh"

constexpr int kAttnChunkKeys = 64;  // keys (and values) staged in shared memory at a time

struct AttnParams {
  const float* q;       // [B*T, q_ld]; the rep query heads of KV head g at column g*rep*hd
  uint32_t q_ld;
  float* kcache;        // [B, KV, cap, hd]
  float* vcache;
  // fuse != 0 (T == 1 only): rotate q and the new key with `table` (may be NULL: no RoPE) and append the
  // new key / value, read from the row of q at columns k_off / v_off, to the cache at position *len
  int fuse;
  const float2* table;
  uint32_t k_off, v_off;
  const int32_t* len;   // device: positions already cached before this step
  uint32_t T, KV, hd, cap;
  float scale;          // 1/sqrt(hd)
  float* out;           // [B*T, out_ld]
  uint32_t out_ld;
  float* scratch;       // split merge: [B*KV*T][splits][rep][hd+2]
  unsigned* counters;   // [B*KV*T], zero between launches
  int* status;          // context status word (bounded waits)
  unsigned long long* trace;  // debug timeline slot
};

int ruai_embed(ruai_ctx* c, const int32_t* ids, const float* embed, const float* wpe, const int32_t* len, uint32_t rows, uint32_t T, uint32_t d,
               uint32_t vocab, float* x, int* err, float* sumsq);
int ruai_rms_norm(ruai_ctx* c, const float* x, const float* w, uint32_t rows, uint32_t d, float eps, float* y);
int ruai_layer_norm(ruai_ctx* c, const float* x, const float* w, const float* b, uint32_t rows, uint32_t d, float eps, float* y);
int ruai_rope_table(ruai_ctx* c, const float* inv_freq, uint32_t half, uint32_t max_pos, float2* table);
int ruai_rope_kv(ruai_ctx* c, float* qkv, uint32_t qkv_ld, uint32_t k_off, uint32_t v_off, const float2* table, const int32_t* len, uint32_t rows,
                 uint32_t T, uint32_t Hq, uint32_t KV, uint32_t hd, uint32_t cap, float* kcache, float* vcache);
int ruai_attention(ruai_ctx* c, const AttnParams& p, uint32_t B, uint32_t rep, uint32_t splits);
// Many query positions at once, queries in tiles (attn_prefill.cu).  1: launched; 0: not taken for this shape; < 0: error.
int ruai_attention_prefill(ruai_ctx* c, const AttnParams& p, uint32_t B, uint32_t rep);
int ruai_argmax(ruai_ctx* c, const float* logits, uint32_t ld, uint32_t rows, uint32_t n, int32_t* out, uint32_t out_offset);
// Sampler::sample (generation.rs:38-73) on one row of device logits; the token is left at token_dev (sample.cu).
int ruai_sample_device(ruai_ctx* c, const float* logits_dev, uint32_t vocab, float temperature, uint32_t top_k, float top_p, uint64_t* rng_state,
                       int32_t* token_dev);
int ruai_add_scalar(ruai_ctx* c, int32_t* p, int32_t v);
int ruai_take_last_rows(ruai_ctx* c, const float* x, uint32_t B, uint32_t T, uint32_t d, float* y);

// quantize.cu
int ruai_synth_normal_dev(ruai_ctx* c, float* out, size_t count, uint64_t seed, uint64_t tensor_id, double std_dev);
int ruai_synth_tokens_dev(ruai_ctx* c, int32_t* out, size_t count, uint64_t seed, uint64_t tensor_id, uint32_t vocab);
int ruai_fill_dev(ruai_ctx* c, float* out, size_t count, float v);
int ruai_transpose_dev(ruai_ctx* c, const float* in, float* out, uint32_t rows, uint32_t cols);
