// Llama and GPT-2 inference over the quantized Linear: weights, KV cache, the per-step
// kernel sequence, CUDA-graph replay of the decode step, greedy generation.
//
// Mirrors, for inference only, Llama::run / forward_cached / generate / quantize_int8 /
// quantize_int4 (src/nn/modules/llama.rs:434-554), GPT2 (src/nn/modules/gpt2.rs:214-335),
// KvCache (src/nn/modules/transformer.rs:10-166) and generate_cached
// (src/nn/generation.rs:83-113).  Differences in mechanism, not in results:
//  - q/k/v (and gate/up) of a layer are quantized separately, exactly as the reference
//    does, and then stored side by side as one weight so that one kernel reads x once;
//    gate and up columns are interleaved so SwiGLU runs in the GEMV epilogue;
//  - RoPE tables are computed once on the device (same f64 angles) instead of per step
//    on the host; position and token ids live in device memory;
//  - the decode step is captured once into a CUDA graph and replayed.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <vector>

#include "decode_ops.cuh"
#include "pstep.cuh"
#include "tp.cuh"

namespace {

template <typename T>
__global__ void copy2d_kernel(T* __restrict__ dst, size_t dst_ld, size_t dst_c0, size_t dst_cstride, const T* __restrict__ src, size_t src_ld,
                              size_t src_r0, size_t src_c0, uint32_t rows, uint32_t cols) {
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  for (uint32_t r = blockIdx.y; r < rows; r += gridDim.y)
    dst[(size_t)r * dst_ld + dst_c0 + (size_t)c * dst_cstride] = src[(src_r0 + r) * src_ld + src_c0 + c];
}

template <typename T>
int copy2d(ruai_ctx* c, T* dst, size_t dst_ld, size_t dst_c0, size_t dst_cstride, const T* src, size_t src_ld, size_t src_r0, size_t src_c0,
           uint32_t rows, uint32_t cols) {
  if (!rows || !cols) return RUAI_OK;
  dim3 grid((cols + 255) / 256, std::min<uint32_t>(rows, 4096));
  copy2d_kernel<T><<<grid, 256, 0, c->stream>>>(dst, dst_ld, dst_c0, dst_cstride, src, src_ld, src_r0, src_c0, rows, cols);
  RUAI_CUDA(c, cudaGetLastError());
  return RUAI_OK;
}

struct DevBuf {
  void* p = nullptr;
  size_t bytes = 0;
  int alloc(ruai_ctx* c, size_t n) {
    release();
    RUAI_CUDA(c, cudaMalloc(&p, n ? n : 1));
    bytes = n;
    return RUAI_OK;
  }
  int reserve(ruai_ctx* c, size_t n) { return n <= bytes && p ? RUAI_OK : alloc(c, n); }
  void release() {
    if (p) cudaFree(p);
    p = nullptr;
    bytes = 0;
  }
  template <typename T> T* as() const { return (T*)p; }
};

// A reference Linear after quantize_int8 / quantize_int4: full (unsharded) buffers in the
// reference layout, on the device.  Lives only while a layer is being loaded.
struct RefQ {
  uint32_t k = 0, n = 0, bits = 0, group = 0;
  DevBuf q, scale;
  uint32_t q_rows() const { return bits == 8 ? k : k / 2; }
  uint32_t s_rows() const { return bits == 8 ? 1 : k / group; }
  RefQ() = default;
  RefQ(const RefQ&) = delete;
  RefQ& operator=(const RefQ&) = delete;
  ~RefQ() { q.release(); scale.release(); }
};

struct Lin {
  ruai_qweight* w = nullptr;
  ruai_sweight sw;  // the same weight in the tile-stream layout of the persistent decode kernel (Llama only)
  DevBuf bias;
  double bytes() const { return w ? (double)w->k * w->n * w->bits / 8.0 + (double)w->scale_bytes + (double)bias.bytes : 0.0; }
};

struct Layer {
  DevBuf n1w, n1b, n2w, n2b;
  Lin qkv, o, up, down;  // up = gate/up interleaved (Llama) or c_fc (GPT-2)
  DevBuf kc, vc;         // KV cache [B, KVl, cap, hd]
};

// Device state of the persistent decode step (pstep.cu).
struct PStep {
  bool tried = false, usable = false;
  int wanted = -1;  // -1: the environment decides (RUAI_B200_PSTEP=1 turns it on), 0 / 1: ruai_model_use_persistent_step
  DevBuf layers, x, ss, acc, poison, att_part, arg_slots, sync;  // sync: [0] barrier counter, [1] abort flag
  unsigned bar_base = 0;
  uint32_t table_cap = 0, table_B = 0, splits = 0, att_rows = 0;
  size_t acc_elems = 0;
};

}  // namespace

struct ruai_model {
  ruai_ctx* ctx = nullptr;
  bool llama = true;
  ruai_llama_config lc{};
  ruai_gpt2_config gc{};
  uint32_t L = 0, d = 0, H = 0, KV = 0, hd = 0, ffn = 0, V = 0, max_pos = 0;
  uint32_t rank = 0, world = 1, Hl = 0, KVl = 0, fl = 0, Vl = 0;
  float eps = 1e-5f;
  bool tied = false;
  // weights
  DevBuf embed, wpe, final_w, final_b, rope_table;
  std::vector<Layer> layers;
  Lin head;
  bool quantized = false;
  uint32_t bits = 0, group = 0;
  std::map<uint64_t, DevBuf> staged;  // f32 tensors set before quantizing
  std::map<uint64_t, RefQ*> staged_q; // Linears that arrived already quantized (a checkpoint in the reference's format)
  // cache state
  uint32_t B = 0, len = 0, cap = 0;
  // device state
  DevBuf d_ids, d_len, d_err, x, xn, qkv, att, hbuf, xl, logits, attn_scratch, attn_counters, sumsq, arg_slots, arg_counter;
  uint32_t act_rows = 0, logit_rows = 0;
  // decode graph
  cudaGraphExec_t graph = nullptr;
  uint32_t graph_B = 0, graph_cap = 0, graph_launches = 0;
  unsigned long long graph_epoch = 0;  // the context's scratch_epoch at capture: the graph holds the scratch's address
  bool len_dirty = true;  // the device copy of `len` may differ from the host's
  PStep ps;
  ruai_tp_state tp;
};

namespace {

int model_fail(ruai_model* m, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  return ruai_fail(m ? m->ctx : nullptr, code, "%s", buf);
}

void drop_graph(ruai_model* m) {
  if (m->graph) cudaGraphExecDestroy(m->graph);
  m->graph = nullptr;
}

// ---- tensor ids -----------------------------------------------------------------

struct TensorShape { size_t rows, cols; };

bool tensor_shape(const ruai_model* m, uint64_t id, TensorShape* s) {
  const size_t d = m->d, nq = (size_t)m->H * m->hd, nkv = (size_t)m->KV * m->hd, f = m->ffn;
  if (id == RUAI_T_EMBED) { *s = {m->V, d}; return true; }
  if (id == RUAI_T_LMHEAD) { *s = {d, m->V}; return m->llama && !m->tied; }
  if (id == RUAI_T_WPE) { *s = {m->max_pos, d}; return !m->llama; }
  if (id == RUAI_TN_FINAL_NORM) { *s = {1, d}; return true; }
  if (id == RUAI_TN_FINAL_NORM_B) { *s = {1, d}; return !m->llama; }
  for (uint64_t base : {RUAI_TN_LAYER_NORM1, RUAI_TN_LAYER_NORM1B, RUAI_TN_LAYER_NORM2, RUAI_TN_LAYER_NORM2B})
    if (id >= base && id < base + m->L) {
      *s = {1, d};
      return m->llama ? (base == RUAI_TN_LAYER_NORM1 || base == RUAI_TN_LAYER_NORM2) : true;
    }
  if (id < (uint64_t)m->L * 16) {
    const uint32_t kind = (uint32_t)(id % 16);
    if (m->llama) switch (kind) {
      case RUAI_T_Q: *s = {d, nq}; return true;
      case RUAI_T_K: case RUAI_T_V: *s = {d, nkv}; return true;
      case RUAI_T_O: *s = {nq, d}; return true;
      case RUAI_T_GATE: case RUAI_T_UP: *s = {d, f}; return true;
      case RUAI_T_DOWN: *s = {f, d}; return true;
      default: return false;
    }
    switch (kind) {
      case RUAI_T_CATTN: *s = {d, 3 * d}; return true;
      case RUAI_T_CPROJ: *s = {d, d}; return true;
      case RUAI_T_CFC: *s = {d, f}; return true;
      case RUAI_T_MPROJ: *s = {f, d}; return true;
      case RUAI_T_CATTN_B: *s = {1, 3 * d}; return true;
      case RUAI_T_CPROJ_B: *s = {1, d}; return true;
      case RUAI_T_CFC_B: *s = {1, f}; return true;
      case RUAI_T_MPROJ_B: *s = {1, d}; return true;
      default: return false;
    }
  }
  return false;
}

int staged_get(ruai_model* m, uint64_t id, DevBuf** out) {
  auto it = m->staged.find(id);
  if (it == m->staged.end()) return model_fail(m, RUAI_ERR_ARG, "tensor 0x%llx was not set before quantizing", (unsigned long long)id);
  *out = &it->second;
  return RUAI_OK;
}

void staged_drop(ruai_model* m, uint64_t id) {
  auto it = m->staged.find(id);
  if (it != m->staged.end()) {
    it->second.release();
    m->staged.erase(it);
  }
}

// ---- quantization pipeline ----------------------------------------------------------

// Linear::quantize_int8 / quantize_int4 of one full f32 matrix [k, n] (layers.rs:112-165).
int quantize_ref(ruai_model* m, const float* w, uint32_t k, uint32_t n, uint32_t bits, uint32_t group, RefQ* out) {
  ruai_ctx* c = m->ctx;
  out->k = k; out->n = n; out->bits = bits; out->group = bits == 4 ? group : 0;
  if (bits == 4 && !(group >= 2 && group % 2 == 0 && k % group == 0))
    return model_fail(m, RUAI_ERR_SHAPE, "int4 group %u must be even and divide in_features %u", group, k);
  RUAI_TRY(out->q.alloc(c, (size_t)out->q_rows() * n));
  RUAI_TRY(out->scale.alloc(c, (size_t)out->s_rows() * n * sizeof(float)));
  if (bits == 8) return ruai_quantize_int8(c, w, k, n, out->q.as<int8_t>(), out->scale.as<float>());
  return ruai_quantize_int4(c, w, k, n, group, out->q.as<int8_t>(), out->scale.as<float>());
}

// The reference-layout quantized form of Linear `id`: the buffers a checkpoint supplied, or the quantizer run
// over the f32 tensor that was set.
int obtain_ref(ruai_model* m, uint64_t id, uint32_t k, uint32_t n, uint32_t bits, uint32_t group, RefQ* out) {
  auto it = m->staged_q.find(id);
  if (it != m->staged_q.end()) {
    RefQ* r = it->second;
    const uint32_t g = bits == 4 ? group : 0;
    if (r->k != k || r->n != n || r->bits != bits || r->group != g)
      return model_fail(m, RUAI_ERR_SHAPE, "quantized tensor 0x%llx is int%u [%u, %u] group %u; the model needs int%u [%u, %u] group %u",
                        (unsigned long long)id, r->bits, r->k, r->n, r->group, bits, k, n, g);
    out->k = k; out->n = n; out->bits = bits; out->group = g;
    out->q = r->q; out->scale = r->scale;
    r->q = DevBuf(); r->scale = DevBuf();
    delete r;
    m->staged_q.erase(it);
    return RUAI_OK;
  }
  DevBuf* t = nullptr;
  RUAI_TRY(staged_get(m, id, &t));
  RUAI_TRY(quantize_ref(m, t->as<float>(), k, n, bits, group, out));
  staged_drop(m, id);
  return RUAI_OK;
}

// One part of a fused local weight: columns [c0, c0+cols) and rows [r0, r0+rows) of a
// reference Linear, placed at column dst_c0 with column stride dst_cs.
struct Part { const RefQ* src; uint32_t r0, rows, c0, cols, dst_c0, dst_cs; };

// Builds the local weight from parts (all with the same rows) and repacks it.
int build_lin(ruai_model* m, const std::vector<Part>& parts, uint32_t n_local, Lin* out) {
  ruai_ctx* c = m->ctx;
  const RefQ* s0 = parts[0].src;
  const uint32_t bits = s0->bits, group = s0->group, rows = parts[0].rows;
  if (bits == 4 && (parts[0].r0 % group || rows % group))
    return model_fail(m, RUAI_ERR_SHAPE, "int4 row shard [%u, +%u) does not align with group %u", parts[0].r0, rows, group);
  const uint32_t q_rows = bits == 8 ? rows : rows / 2, s_rows = bits == 8 ? 1 : rows / group;
  DevBuf q, s;
  RUAI_TRY(q.alloc(c, (size_t)q_rows * n_local));
  RUAI_TRY(s.alloc(c, (size_t)s_rows * n_local * sizeof(float)));
  int rc = RUAI_OK;
  for (const Part& p : parts) {
    const uint32_t qr0 = bits == 8 ? p.r0 : p.r0 / 2, sr0 = bits == 8 ? 0 : p.r0 / group;
    if ((rc = copy2d<int8_t>(c, q.as<int8_t>(), n_local, p.dst_c0, p.dst_cs, p.src->q.as<int8_t>(), p.src->n, qr0, p.c0, q_rows, p.cols)) != RUAI_OK) break;
    if ((rc = copy2d<float>(c, s.as<float>(), n_local, p.dst_c0, p.dst_cs, p.src->scale.as<float>(), p.src->n, sr0, p.c0, s_rows, p.cols)) != RUAI_OK) break;
  }
  if (rc == RUAI_OK) {
    if (out->w) ruai_qweight_free(out->w);
    out->w = nullptr;
    rc = bits == 8 ? ruai_repack_int8(c, q.as<int8_t>(), s.as<float>(), rows, n_local, &out->w)
                   : ruai_repack_int4(c, q.as<int8_t>(), s.as<float>(), rows, n_local, group, &out->w);
  }
  if (rc == RUAI_OK && m->llama && ruai_sweight_supported(out->w)) rc = ruai_sweight_create(c, out->w, &out->sw);
  cudaStreamSynchronize(c->stream);
  q.release();
  s.release();
  return rc;
}

int copy_vec(ruai_model* m, DevBuf* dst, const DevBuf* src, size_t off, size_t count) {
  RUAI_TRY(dst->alloc(m->ctx, count * sizeof(float)));
  RUAI_CUDA(m->ctx, cudaMemcpyAsync(dst->p, src->as<float>() + off, count * sizeof(float), cudaMemcpyDeviceToDevice, m->ctx->stream));
  return RUAI_OK;
}

int quantize_layer(ruai_model* m, uint32_t l, uint32_t bits, uint32_t group) {
  Layer& Ly = m->layers[l];
  const uint32_t d = m->d, hd = m->hd, r = m->rank;
  DevBuf* t = nullptr;
  if (m->llama) {
    RefQ q, k, v, o, g, u, dn;
    const uint32_t nq = m->H * hd, nkv = m->KV * hd, nql = m->Hl * hd, nkvl = m->KVl * hd, f = m->ffn, fl = m->fl;
    RUAI_TRY(obtain_ref(m, ruai_layer_tensor(l, RUAI_T_Q), d, nq, bits, group, &q));
    RUAI_TRY(obtain_ref(m, ruai_layer_tensor(l, RUAI_T_K), d, nkv, bits, group, &k));
    RUAI_TRY(obtain_ref(m, ruai_layer_tensor(l, RUAI_T_V), d, nkv, bits, group, &v));
    RUAI_TRY(build_lin(m, {{&q, 0, d, r * nql, nql, 0, 1}, {&k, 0, d, r * nkvl, nkvl, nql, 1}, {&v, 0, d, r * nkvl, nkvl, nql + nkvl, 1}}, nql + 2 * nkvl, &Ly.qkv));
    q.q.release(); k.q.release(); v.q.release(); q.scale.release(); k.scale.release(); v.scale.release();
    RUAI_TRY(obtain_ref(m, ruai_layer_tensor(l, RUAI_T_O), nq, d, bits, group, &o));
    RUAI_TRY(build_lin(m, {{&o, r * nql, nql, 0, d, 0, 1}}, d, &Ly.o));
    o.q.release(); o.scale.release();
    RUAI_TRY(obtain_ref(m, ruai_layer_tensor(l, RUAI_T_GATE), d, f, bits, group, &g));
    RUAI_TRY(obtain_ref(m, ruai_layer_tensor(l, RUAI_T_UP), d, f, bits, group, &u));
    RUAI_TRY(build_lin(m, {{&g, 0, d, r * fl, fl, 0, 2}, {&u, 0, d, r * fl, fl, 1, 2}}, 2 * fl, &Ly.up));
    g.q.release(); u.q.release(); g.scale.release(); u.scale.release();
    RUAI_TRY(obtain_ref(m, ruai_layer_tensor(l, RUAI_T_DOWN), f, d, bits, group, &dn));
    RUAI_TRY(build_lin(m, {{&dn, r * fl, fl, 0, d, 0, 1}}, d, &Ly.down));
  } else {
    const uint32_t f = m->ffn;
    struct Item { uint32_t kind, bias_kind, k, n; Lin* dst; };
    const Item items[4] = {{RUAI_T_CATTN, RUAI_T_CATTN_B, d, 3 * d, &Ly.qkv}, {RUAI_T_CPROJ, RUAI_T_CPROJ_B, d, d, &Ly.o},
                           {RUAI_T_CFC, RUAI_T_CFC_B, d, f, &Ly.up}, {RUAI_T_MPROJ, RUAI_T_MPROJ_B, f, d, &Ly.down}};
    for (const Item& it : items) {
      RefQ q;
      RUAI_TRY(obtain_ref(m, ruai_layer_tensor(l, it.kind), it.k, it.n, bits, group, &q));
      RUAI_TRY(build_lin(m, {{&q, 0, it.k, 0, it.n, 0, 1}}, it.n, it.dst));
      RUAI_TRY(staged_get(m, ruai_layer_tensor(l, it.bias_kind), &t));
      RUAI_TRY(copy_vec(m, &it.dst->bias, t, 0, it.n));
      cudaStreamSynchronize(m->ctx->stream);
      staged_drop(m, ruai_layer_tensor(l, it.bias_kind));
    }
  }
  // norm parameters
  RUAI_TRY(staged_get(m, RUAI_TN_LAYER_NORM1 + l, &t)); RUAI_TRY(copy_vec(m, &Ly.n1w, t, 0, d));
  RUAI_TRY(staged_get(m, RUAI_TN_LAYER_NORM2 + l, &t)); RUAI_TRY(copy_vec(m, &Ly.n2w, t, 0, d));
  if (!m->llama) {
    RUAI_TRY(staged_get(m, RUAI_TN_LAYER_NORM1B + l, &t)); RUAI_TRY(copy_vec(m, &Ly.n1b, t, 0, d));
    RUAI_TRY(staged_get(m, RUAI_TN_LAYER_NORM2B + l, &t)); RUAI_TRY(copy_vec(m, &Ly.n2b, t, 0, d));
  }
  cudaStreamSynchronize(m->ctx->stream);
  for (uint64_t base : {RUAI_TN_LAYER_NORM1, RUAI_TN_LAYER_NORM1B, RUAI_TN_LAYER_NORM2, RUAI_TN_LAYER_NORM2B}) staged_drop(m, base + l);
  return RUAI_OK;
}

// quantize_head_int8 (llama.rs:544-554, gpt2.rs:327-335): int8 of lm_head, or of the
// transposed embedding when tied; the embedding itself stays f32.
int quantize_head(ruai_model* m) {
  ruai_ctx* c = m->ctx;
  DevBuf* t = nullptr;
  RUAI_TRY(staged_get(m, RUAI_T_EMBED, &t));
  RefQ h;
  if (m->staged_q.count(RUAI_T_LMHEAD)) {  // `lm_head.weight_int8` of a quantized checkpoint (tied or not)
    RUAI_TRY(obtain_ref(m, RUAI_T_LMHEAD, m->d, m->V, 8, 0, &h));
    staged_drop(m, RUAI_T_LMHEAD);
  } else if (m->llama && !m->tied) {
    DevBuf* lh = nullptr;
    RUAI_TRY(staged_get(m, RUAI_T_LMHEAD, &lh));
    RUAI_TRY(quantize_ref(m, lh->as<float>(), m->d, m->V, 8, 0, &h));
    staged_drop(m, RUAI_T_LMHEAD);
  } else {
    DevBuf tr;
    RUAI_TRY(tr.alloc(c, (size_t)m->d * m->V * sizeof(float)));
    RUAI_TRY(ruai_transpose_dev(c, t->as<float>(), tr.as<float>(), m->V, m->d));
    int rc = quantize_ref(m, tr.as<float>(), m->d, m->V, 8, 0, &h);
    cudaStreamSynchronize(c->stream);
    tr.release();
    RUAI_TRY(rc);
  }
  RUAI_TRY(build_lin(m, {{&h, 0, m->d, m->rank * m->Vl, m->Vl, 0, 1}}, m->Vl, &m->head));
  // the embedding table moves from the staging map into the model
  m->embed.release();
  m->embed = *t;
  m->staged.erase(RUAI_T_EMBED);
  if (!m->llama) {
    RUAI_TRY(staged_get(m, RUAI_T_WPE, &t));
    m->wpe.release();
    m->wpe = *t;
    m->staged.erase(RUAI_T_WPE);
    RUAI_TRY(staged_get(m, RUAI_TN_FINAL_NORM_B, &t)); RUAI_TRY(copy_vec(m, &m->final_b, t, 0, m->d));
  }
  RUAI_TRY(staged_get(m, RUAI_TN_FINAL_NORM, &t)); RUAI_TRY(copy_vec(m, &m->final_w, t, 0, m->d));
  cudaStreamSynchronize(c->stream);
  staged_drop(m, RUAI_TN_FINAL_NORM);
  staged_drop(m, RUAI_TN_FINAL_NORM_B);
  return RUAI_OK;
}

int stage_alloc(ruai_model* m, uint64_t id, size_t count, DevBuf** out) {
  DevBuf& b = m->staged[id];
  RUAI_TRY(b.alloc(m->ctx, count * sizeof(float)));
  *out = &b;
  return RUAI_OK;
}

int stage_synth(ruai_model* m, uint64_t seed, uint64_t id, double std_dev) {
  TensorShape s;
  if (!tensor_shape(m, id, &s)) return model_fail(m, RUAI_ERR_ARG, "bad tensor id 0x%llx", (unsigned long long)id);
  DevBuf* b;
  RUAI_TRY(stage_alloc(m, id, s.rows * s.cols, &b));
  return ruai_synth_normal_dev(m->ctx, b->as<float>(), s.rows * s.cols, seed, id, std_dev);
}

int stage_fill(ruai_model* m, uint64_t id, float v) {
  TensorShape s;
  if (!tensor_shape(m, id, &s)) return model_fail(m, RUAI_ERR_ARG, "bad tensor id 0x%llx", (unsigned long long)id);
  DevBuf* b;
  RUAI_TRY(stage_alloc(m, id, s.rows * s.cols, &b));
  return ruai_fill_dev(m->ctx, b->as<float>(), s.rows * s.cols, v);
}

int finish_create(ruai_model* m) {
  ruai_ctx* c = m->ctx;
  m->layers.resize(m->L);
  RUAI_TRY(m->d_len.alloc(c, sizeof(int32_t)));
  RUAI_TRY(m->d_err.alloc(c, sizeof(int32_t)));
  RUAI_CUDA(c, cudaMemsetAsync(m->d_len.p, 0, sizeof(int32_t), c->stream));
  RUAI_CUDA(c, cudaMemsetAsync(m->d_err.p, 0, sizeof(int32_t), c->stream));
  if (m->llama) {
    // rope_inv_freq (functional.rs:168-171): theta^(-2i/hd) in f32 powf, on the host like the reference
    std::vector<float> inv(m->hd / 2);
    for (uint32_t i = 0; i < m->hd / 2; ++i) inv[i] = powf(m->lc.rope_theta, -((float)(2 * i)) / (float)m->hd);
    DevBuf dinv;
    RUAI_TRY(dinv.alloc(c, inv.size() * sizeof(float)));
    RUAI_CUDA(c, cudaMemcpyAsync(dinv.p, inv.data(), inv.size() * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    RUAI_TRY(m->rope_table.alloc(c, (size_t)m->max_pos * (m->hd / 2) * sizeof(float2)));
    RUAI_TRY(ruai_rope_table(c, dinv.as<float>(), m->hd / 2, m->max_pos, m->rope_table.as<float2>()));
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    dinv.release();
  }
  RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
  return RUAI_OK;
}

// ---- cache --------------------------------------------------------------------------

// KvBuf::append's growth rule (transformer.rs:38-49): capacity max(need, 2*cap, 16),
// old contents copied.
int ensure_cache(ruai_model* m, uint32_t B, uint32_t need) {
  ruai_ctx* c = m->ctx;
  if (m->len == 0 && B != m->B) {  // a new batch shape starts new buffers (transformer.rs:31-32)
    for (Layer& L : m->layers) { L.kc.release(); L.vc.release(); }
    m->cap = 0;
    m->B = B;
    drop_graph(m);
  }
  if (B != m->B) return model_fail(m, RUAI_ERR_SHAPE, "KV cache: new keys/values for batch %u do not match the cached batch %u", B, m->B);
  if (m->cap >= need) return RUAI_OK;
  const uint32_t cap = std::max(std::max(need, 2 * m->cap), 16u);
  const size_t per = (size_t)B * m->KVl * cap * m->hd * sizeof(float);
  RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
  // Layer by layer (at most one layer's old and new buffers exist together).  If an allocation or copy fails half way
  // the layers would disagree about their capacity: the whole cache is dropped then (as after cache_clear, contents
  // lost) and the error says so, so that the model stays usable.
  auto grow_layer = [&](Layer& L) -> int {
    DevBuf nk, nv;
    auto bail = [&](int rc) { nk.release(); nv.release(); return rc; };
    if (nk.alloc(c, per) != RUAI_OK || nv.alloc(c, per) != RUAI_OK) return bail(RUAI_ERR_CUDA);
    cudaError_t e = cudaMemsetAsync(nk.p, 0, per, c->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(nv.p, 0, per, c->stream);
    if (e == cudaSuccess && m->len > 0 && L.kc.p) {
      const size_t row = (size_t)m->hd * sizeof(float);
      e = cudaMemcpy2DAsync(nk.p, (size_t)cap * row, L.kc.p, (size_t)m->cap * row, (size_t)m->len * row, (size_t)B * m->KVl, cudaMemcpyDeviceToDevice, c->stream);
      if (e == cudaSuccess)
        e = cudaMemcpy2DAsync(nv.p, (size_t)cap * row, L.vc.p, (size_t)m->cap * row, (size_t)m->len * row, (size_t)B * m->KVl, cudaMemcpyDeviceToDevice, c->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) return bail(ruai_fail(c, RUAI_ERR_CUDA, "KV cache growth: %s", cudaGetErrorString(e)));
    L.kc.release(); L.vc.release();
    L.kc = nk; L.vc = nv;
    return RUAI_OK;
  };
  for (Layer& L : m->layers) {
    if (grow_layer(L) != RUAI_OK) {
      (void)cudaGetLastError();  // an allocation failure is not sticky; later launch checks must not see it
      for (Layer& L2 : m->layers) { L2.kc.release(); L2.vc.release(); }
      m->cap = 0; m->len = 0; m->len_dirty = true; m->B = 0;
      drop_graph(m);
      m->ps.table_cap = 0;
      return model_fail(m, RUAI_ERR_CUDA, "KV cache: growing to %u positions for batch %u failed (%zu bytes per layer and tensor); the cache was dropped", cap, B, per);
    }
  }
  m->cap = cap;
  drop_graph(m);
  return RUAI_OK;
}

uint32_t attn_splits(const ruai_model* m, uint32_t B, uint32_t T) {
  if (T > 1) return 1;
  // one chunk of 64 keys per CTA where the capacity allows it (a single round trip to memory per CTA); with many
  // (sequence, KV head) items there are CTAs enough without it, and fewer splits mean fewer partial results to merge
  // (measured, 8B shape, 1024 positions: 16 sequences 5.65 -> 5.49 ms with two chunks per CTA, 128 sequences 27.2 -> 26.1
  // with two splits in all)
  const uint32_t by_len = (m->cap + kAttnChunkKeys - 1) / kAttnChunkKeys;
  const uint32_t items = B * m->KVl;
  if (items >= 512) return std::max(1u, std::min(by_len, 2u));
  if (B >= 5) return std::max(1u, std::min((by_len + 1) / 2, 64u));
  return std::max(1u, std::min(by_len, 64u));
}

int ensure_activations(ruai_model* m, uint32_t rows, uint32_t out_rows, uint32_t B, uint32_t T) {
  ruai_ctx* c = m->ctx;
  if (rows > m->act_rows) {
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    const size_t nqkv = (size_t)(m->Hl + 2 * m->KVl) * m->hd;
    RUAI_TRY(m->d_ids.alloc(c, (size_t)rows * sizeof(int32_t)));
    RUAI_TRY(m->x.alloc(c, (size_t)rows * m->d * sizeof(float)));
    RUAI_TRY(m->xn.alloc(c, (size_t)rows * m->d * sizeof(float)));
    RUAI_TRY(m->qkv.alloc(c, (size_t)rows * nqkv * sizeof(float)));
    RUAI_TRY(m->att.alloc(c, (size_t)rows * m->Hl * m->hd * sizeof(float)));
    RUAI_TRY(m->hbuf.alloc(c, (size_t)rows * m->fl * sizeof(float)));
    RUAI_TRY(m->xl.alloc(c, (size_t)rows * m->d * sizeof(float)));
    RUAI_TRY(m->sumsq.alloc(c, (size_t)rows * ((m->d + kGemvBulkTileCols - 1) / kGemvBulkTileCols) * sizeof(float)));
    RUAI_TRY(m->arg_slots.alloc(c, (size_t)16 * ((m->Vl + kGemvBulkTileCols - 1) / kGemvBulkTileCols) * sizeof(int2)));
    if (!m->arg_counter.p) {
      RUAI_TRY(m->arg_counter.alloc(c, sizeof(unsigned)));
      RUAI_CUDA(c, cudaMemsetAsync(m->arg_counter.p, 0, sizeof(unsigned), c->stream));
    }
    m->act_rows = rows;
    drop_graph(m);
  }
  if (out_rows > m->logit_rows) {
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    RUAI_TRY(m->logits.alloc(c, (size_t)out_rows * m->Vl * sizeof(float)));
    m->logit_rows = out_rows;
    drop_graph(m);
  }
  const uint32_t splits = attn_splits(m, B, T);
  const uint32_t rep = m->Hl / m->KVl;
  const size_t need = (size_t)B * m->KVl * T * splits * rep * (m->hd + 4) * sizeof(float);
  const size_t cnt = (size_t)B * m->KVl * T * sizeof(unsigned);
  if (need > m->attn_scratch.bytes || cnt > m->attn_counters.bytes) {
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    RUAI_TRY(m->attn_scratch.reserve(c, need));
    if (cnt > m->attn_counters.bytes) {
      RUAI_TRY(m->attn_counters.alloc(c, cnt));
      RUAI_CUDA(c, cudaMemsetAsync(m->attn_counters.p, 0, cnt, c->stream));
    }
    drop_graph(m);
  }
  return RUAI_OK;
}

// ---- the step ---------------------------------------------------------------------------

// Issues every kernel of one forward over rows = B*T new tokens whose ids are in d_ids and
// whose first position is *d_len.  Logits for the last position of each sequence (or all
// positions) land in m->logits.  With want_argmax the greedy next ids are written to d_ids[0..B).
int issue_step(ruai_model* m, uint32_t B, uint32_t T, bool all_positions, bool want_argmax) {
  ruai_ctx* c = m->ctx;
  const uint32_t rows = B * T, d = m->d, hd = m->hd;
  const uint32_t nql = m->Hl * hd, nkvl = m->KVl * hd, nqkv = nql + 2 * nkvl, rep = m->Hl / m->KVl;
  int32_t* len = m->d_len.as<int32_t>();
  float *x = m->x.as<float>(), *xn = m->xn.as<float>(), *qkv = m->qkv.as<float>(), *att = m->att.as<float>(), *hb = m->hbuf.as<float>();
  const uint32_t splits = attn_splits(m, B, T);
  const bool tp = m->world > 1;
  // RMSNorm rides in the prologue of the GEMV that consumes it: the producer of x (embedding, o_proj, down_proj)
  // leaves per-tile sums of squares.  LayerNorm (GPT-2) and the sharded model (x is produced by the exchange
  // kernel) keep the standalone norm kernels.
  // decode-sized steps on the chunk-layout kernels; sharded: only where the exchange kernel can supply the sum of squares
  const bool fold = m->llama && (m->bits == 8 || m->group == 32) && rows <= 16 && (!tp || ruai_tp_allreduce_gives_sumsq(rows, d));
  float* ss = fold ? m->sumsq.as<float>() : nullptr;
  const uint32_t d_tiles = tp ? 1u : ruai_gemv_tiles(c, m->layers[0].o.w);  // o_proj and down_proj both write [.., d]; sharded: the exchange writes one tile
  uint32_t ss_tiles = 1;
  RUAI_TRY(ruai_embed(c, m->d_ids.as<int32_t>(), m->embed.as<float>(), m->llama ? nullptr : m->wpe.as<float>(), len, rows, T, d, m->V, x,
                      m->d_err.as<int>(), ss));
  for (uint32_t l = 0; l < m->L; ++l) {
    Layer& Ly = m->layers[l];
    GemvEpilogue e;
    e.bias = Ly.qkv.bias.as<float>();
    if (fold) {
      GemvPrologue pr;
      pr.norm_w = Ly.n1w.as<float>(); pr.sumsq = ss; pr.tiles = ss_tiles; pr.eps = m->eps;
      RUAI_TRY(ruai_gemv_launch(c, Ly.qkv.w, x, RUAI_F32, d, rows, qkv, e, pr));
    } else {
      if (m->llama) RUAI_TRY(ruai_rms_norm(c, x, Ly.n1w.as<float>(), rows, d, m->eps, xn));
      else RUAI_TRY(ruai_layer_norm(c, x, Ly.n1w.as<float>(), Ly.n1b.as<float>(), rows, d, 1e-5f, xn));
      RUAI_TRY(ruai_gemv_launch(c, Ly.qkv.w, xn, RUAI_F32, d, rows, qkv, e));
    }
    const float2* table = m->llama ? m->rope_table.as<float2>() : nullptr;
    const bool fuse = T == 1;  // rotate + append inside the attention kernel
    if (!fuse)
      RUAI_TRY(ruai_rope_kv(c, qkv, nqkv, nql, nql + nkvl, table, len, rows, T, m->Hl, m->KVl, hd, m->cap, Ly.kc.as<float>(), Ly.vc.as<float>()));
    AttnParams ap;
    ap.q = qkv; ap.q_ld = nqkv; ap.kcache = Ly.kc.as<float>(); ap.vcache = Ly.vc.as<float>(); ap.len = len;
    ap.fuse = fuse ? 1 : 0; ap.table = table; ap.k_off = nql; ap.v_off = nql + nkvl;
    ap.T = T; ap.KV = m->KVl; ap.hd = hd; ap.cap = m->cap; ap.scale = 1.0f / sqrtf((float)hd);
    ap.out = att; ap.out_ld = nql; ap.scratch = m->attn_scratch.as<float>(); ap.counters = m->attn_counters.as<unsigned>(); ap.status = c->status;
    {
      const int took = ruai_attention_prefill(c, ap, B, rep);  // many query positions: queries in tiles
      if (took < 0) return RUAI_ERR_CUDA;
      if (took == 0) RUAI_TRY(ruai_attention(c, ap, B, rep, splits));
    }
    GemvEpilogue eo;
    eo.bias = Ly.o.bias.as<float>();
    if (!tp) {
      eo.resid = x;
      eo.sumsq = ss;
      GemvPrologue po;
      RUAI_TRY(ruai_gemv_launch(c, Ly.o.w, att, RUAI_F32, nql, rows, x, eo, po));
    } else {
      RUAI_TRY(ruai_gemv_launch(c, Ly.o.w, att, RUAI_F32, nql, rows, m->tp.local_partial(), eo));
      RUAI_TRY(ruai_tp_allreduce_add(c, &m->tp, x, rows, d, m->d_err.as<int>(), ss));
    }
    ss_tiles = d_tiles;
    GemvEpilogue eu;
    eu.bias = Ly.up.bias.as<float>();
    eu.act = m->llama ? ACT_SWIGLU : ACT_GELU;
    if (fold) {
      GemvPrologue pr;
      pr.norm_w = Ly.n2w.as<float>(); pr.sumsq = ss; pr.tiles = ss_tiles; pr.eps = m->eps;
      RUAI_TRY(ruai_gemv_launch(c, Ly.up.w, x, RUAI_F32, d, rows, hb, eu, pr));
    } else {
      if (m->llama) RUAI_TRY(ruai_rms_norm(c, x, Ly.n2w.as<float>(), rows, d, m->eps, xn));
      else RUAI_TRY(ruai_layer_norm(c, x, Ly.n2w.as<float>(), Ly.n2b.as<float>(), rows, d, 1e-5f, xn));
      RUAI_TRY(ruai_gemv_launch(c, Ly.up.w, xn, RUAI_F32, d, rows, hb, eu));
    }
    GemvEpilogue ed;
    ed.bias = Ly.down.bias.as<float>();
    if (!tp) {
      ed.resid = x;
      ed.sumsq = ss;
      GemvPrologue pd;
      RUAI_TRY(ruai_gemv_launch(c, Ly.down.w, hb, RUAI_F32, m->fl, rows, x, ed, pd));
    } else {
      RUAI_TRY(ruai_gemv_launch(c, Ly.down.w, hb, RUAI_F32, m->fl, rows, m->tp.local_partial(), ed));
      RUAI_TRY(ruai_tp_allreduce_add(c, &m->tp, x, rows, d, m->d_err.as<int>(), ss));
    }
  }
  const float* hx = x;
  uint32_t out_rows = rows;
  const bool last_only = !all_positions && T > 1;
  if (last_only) {
    RUAI_TRY(ruai_take_last_rows(c, x, B, T, d, m->xl.as<float>()));
    hx = m->xl.as<float>();
    out_rows = B;
  }
  GemvEpilogue eh;
  // the pick rides in the head GEMV's epilogue where that runs as one row tile on a tensor-core kernel (up to 4 rows, or
  // 5..16 on the 16-row tile); otherwise the separate argmax kernel beats the CUDA-core kernel that could fuse it
  const bool fused_pick = want_argmax && !tp && (out_rows <= 8 || (c->use_bulk && c->use_tc && ruai_gemv_wide_eligible(c, m->head.w, out_rows)));
  if (fused_pick) {
    eh.argmax_out = m->d_ids.as<int32_t>(); eh.argmax_slots = m->arg_slots.as<int2>(); eh.argmax_counter = m->arg_counter.as<unsigned>();
    eh.len_ptr = len; eh.len_add = (int32_t)T;
  }
  if (fold && !last_only) {
    GemvPrologue pr;
    pr.norm_w = m->final_w.as<float>(); pr.sumsq = ss; pr.tiles = ss_tiles; pr.eps = m->eps;
    RUAI_TRY(ruai_gemv_launch(c, m->head.w, hx, RUAI_F32, d, out_rows, m->logits.as<float>(), eh, pr));
  } else {
    if (m->llama) RUAI_TRY(ruai_rms_norm(c, hx, m->final_w.as<float>(), out_rows, d, m->eps, xn));
    else RUAI_TRY(ruai_layer_norm(c, hx, m->final_w.as<float>(), m->final_b.as<float>(), out_rows, d, 1e-5f, xn));
    RUAI_TRY(ruai_gemv_launch(c, m->head.w, xn, RUAI_F32, d, out_rows, m->logits.as<float>(), eh));
  }
  if (!fused_pick) {
    RUAI_TRY(ruai_add_scalar(c, len, (int32_t)T));
    if (want_argmax) {
      if (!tp) RUAI_TRY(ruai_argmax(c, m->logits.as<float>(), m->Vl, B, m->Vl, m->d_ids.as<int32_t>(), 0));
      else RUAI_TRY(ruai_tp_argmax(c, &m->tp, m->logits.as<float>(), m->Vl, B, m->rank * m->Vl, m->d_ids.as<int32_t>(), m->d_err.as<int>()));
    }
  }
  return RUAI_OK;
}

int pstep_reset(ruai_model* m);

int check_device_status(ruai_model* m) {
  int32_t e = 0;
  RUAI_CUDA(m->ctx, cudaMemcpyAsync(&e, m->d_err.p, sizeof e, cudaMemcpyDeviceToHost, m->ctx->stream));
  RUAI_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
  if (e == 0) {
    const int rc = ruai_ctx_check_status(m->ctx);
    if (rc != RUAI_OK) pstep_reset(m);  // a step that gave up leaves its accumulators and barrier count undefined
    return rc;
  }
  cudaMemsetAsync(m->d_err.p, 0, sizeof(int32_t), m->ctx->stream);
  if (e == 1) return model_fail(m, RUAI_ERR_ARG, "token id out of range [0, %u)", m->V);
  return model_fail(m, RUAI_ERR_TIMEOUT, "tensor-parallel exchange timed out waiting for a peer (status %d)", e);
}

// ---- the persistent decode step (pstep.cu) ---------------------------------------------------

// Whether single-token steps of this model for B sequences run as the one persistent kernel.
bool pstep_eligible(ruai_model* m, uint32_t B) {
  PStep& S = m->ps;
  if (!S.tried) {
    S.tried = true;
    const char* env = getenv("RUAI_B200_PSTEP");
    const bool wanted = S.wanted >= 0 ? S.wanted == 1 : (env && env[0] == '1');  // the launch chain is the default
    bool ok = wanted && m->llama && m->world == 1 && m->quantized && m->L >= 1 && m->L <= (uint32_t)ps::kMaxLayers;
    ok = ok && m->d % 32 == 0 && m->hd % 4 == 0 && m->hd <= 256 && m->KVl > 0;
    const uint32_t rep = m->KVl ? m->Hl / m->KVl : 0;
    ok = ok && rep >= 1 && rep <= 8 && rep * (m->hd / 4) <= 448u && m->fl % 4 == 0;
    for (Layer& L : m->layers)
      for (Lin* l : {&L.qkv, &L.o, &L.up, &L.down}) ok = ok && l->sw.data != nullptr;
    ok = ok && m->head.sw.data != nullptr;
    ok = ok && ruai_pstep_grid(m->ctx) > 0;
    S.usable = ok;
  }
  return S.usable && B >= 1 && B <= (uint32_t)ps::kMaxRows;
}

int pstep_reset(ruai_model* m) {
  PStep& S = m->ps;
  ruai_ctx* c = m->ctx;
  if (!S.acc.p) return RUAI_OK;
  RUAI_CUDA(c, cudaMemsetAsync(S.acc.p, 0, S.acc.bytes, c->stream));
  RUAI_CUDA(c, cudaMemsetAsync(S.poison.p, 0, S.poison.bytes, c->stream));
  RUAI_CUDA(c, cudaMemsetAsync(S.sync.p, 0, S.sync.bytes, c->stream));
  S.bar_base = 0;
  return RUAI_OK;
}

int pstep_run(ruai_model* m, uint32_t B) {
  PStep& S = m->ps;
  ruai_ctx* c = m->ctx;
  const uint32_t MR = ps::kMaxRows, d = m->d, hd = m->hd, nq = m->Hl * hd, nkv = m->KVl * hd, nqkv = nq + 2 * nkv, rep = m->Hl / m->KVl;
  const int grid = ruai_pstep_grid(c);
  if (!S.acc.p) {
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    S.acc_elems = (size_t)MR * ((size_t)nqkv + d + 2 * (size_t)m->fl + d + m->Vl);
    RUAI_TRY(S.acc.alloc(c, S.acc_elems * sizeof(long long)));
    RUAI_TRY(S.poison.alloc(c, 5 * MR * sizeof(int)));
    RUAI_TRY(S.sync.alloc(c, 64 + (size_t)MR * m->KVl * sizeof(unsigned)));  // barrier counter, abort flag; from byte 64: attention item counters
    RUAI_TRY(S.x.alloc(c, (2 * (size_t)MR * d + (size_t)MR * nq) * sizeof(float)));
    RUAI_TRY(S.ss.alloc(c, 3 * (size_t)MR * (d / 32) * sizeof(float)));
    RUAI_TRY(S.arg_slots.alloc(c, (size_t)grid * MR * sizeof(int2)));
    RUAI_TRY(S.layers.alloc(c, (size_t)m->L * sizeof(ps::LayerPtrs)));
    // nothing below is read before the kernel writes it; zeroed all the same, so that no run depends on what an earlier
    // owner of the memory left there
    RUAI_CUDA(c, cudaMemsetAsync(S.x.p, 0, S.x.bytes, c->stream));
    RUAI_CUDA(c, cudaMemsetAsync(S.ss.p, 0, S.ss.bytes, c->stream));
    RUAI_CUDA(c, cudaMemsetAsync(S.arg_slots.p, 0, S.arg_slots.bytes, c->stream));
    RUAI_TRY(pstep_reset(m));
  }
  // key splits: one (sequence, KV head, split) item per CTA where the cache is long enough to share out
  const uint32_t splits = std::max(1u, std::min(32u, (uint32_t)grid / (B * m->KVl)));
  const size_t att_floats = (size_t)B * m->KVl * splits * rep * (hd + 4);
  if (att_floats * sizeof(float) > S.att_part.bytes) {
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    RUAI_TRY(S.att_part.alloc(c, att_floats * sizeof(float)));
    RUAI_CUDA(c, cudaMemsetAsync(S.att_part.p, 0, S.att_part.bytes, c->stream));
  }
  if (S.table_cap != m->cap || S.table_B != B) {  // the cache buffers moved (growth) or were made anew
    std::vector<ps::LayerPtrs> t(m->L);
    for (uint32_t l = 0; l < m->L; ++l) {
      Layer& Y = m->layers[l];
      t[l].w_qkv = Y.qkv.sw.data; t[l].w_o = Y.o.sw.data; t[l].w_gu = Y.up.sw.data; t[l].w_dn = Y.down.sw.data;
      t[l].s_qkv = Y.qkv.sw.colscale; t[l].s_o = Y.o.sw.colscale; t[l].s_gu = Y.up.sw.colscale; t[l].s_dn = Y.down.sw.colscale;
      t[l].n1 = Y.n1w.as<float>(); t[l].n2 = Y.n2w.as<float>();
      t[l].kc = Y.kc.as<float>(); t[l].vc = Y.vc.as<float>();
    }
    RUAI_CUDA(c, cudaMemcpyAsync(S.layers.p, t.data(), t.size() * sizeof(ps::LayerPtrs), cudaMemcpyHostToDevice, c->stream));
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));  // `t` is a stack object
    S.table_cap = m->cap; S.table_B = B;
  }
  ps::StepParams P{};
  P.m = B; P.L = m->L; P.d = d; P.nq = nq; P.nkv = nkv; P.hd = hd; P.Hl = m->Hl; P.KVl = m->KVl; P.rep = rep; P.fl = m->fl; P.Vl = m->Vl; P.V = m->V;
  P.cap = m->cap; P.bits = m->bits; P.splits = splits; P.keys_per_stage = (kRingSlotBytes / 2u) / (hd * 4u); P.col_offset = m->rank * m->Vl;
  P.eps = m->eps; P.attn_scale = 1.0f / sqrtf((float)hd);
  auto geom = [](const ruai_sweight& w) { return ps::Geom{w.ntiles, w.nblk, w.n, w.k}; };
  P.qkv = geom(m->layers[0].qkv.sw); P.o = geom(m->layers[0].o.sw); P.gu = geom(m->layers[0].up.sw); P.dn = geom(m->layers[0].down.sw);
  P.head = geom(m->head.sw);
  P.layers = S.layers.as<ps::LayerPtrs>();
  P.w_head = m->head.sw.data; P.s_head = m->head.sw.colscale;
  P.final_norm = m->final_w.as<float>(); P.embed = m->embed.as<float>(); P.rope = m->rope_table.as<float2>();
  P.ids = m->d_ids.as<int32_t>(); P.len = m->d_len.as<int32_t>(); P.err = m->d_err.as<int>();
  P.x0 = S.x.as<float>(); P.x1 = P.x0 + (size_t)MR * d;
  P.ss_a = S.ss.as<float>(); P.ss_b = P.ss_a + (size_t)MR * (d / 32); P.ss_c = P.ss_b + (size_t)MR * (d / 32);
  long long* a = S.acc.as<long long>();
  P.acc_qkv = a; a += (size_t)MR * nqkv;
  P.acc_o = a; a += (size_t)MR * d;
  P.acc_gu = a; a += (size_t)MR * 2 * m->fl;
  P.acc_dn = a; a += (size_t)MR * d;
  P.acc_logits = a;
  P.poison = S.poison.as<int>();
  P.att_part = S.att_part.as<float>();
  P.att_out = P.x1 + (size_t)MR * d;
  P.att_cnt = S.sync.as<unsigned>() + 16;
  P.logits = m->logits.as<float>();
  P.arg_slots = S.arg_slots.as<int2>();
  P.bar = S.sync.as<unsigned>(); P.bar_base = S.bar_base + c->barrier_skew * (unsigned)grid; P.status = c->status; P.abort_flag = S.sync.as<int>() + 1;
  P.spin_limit = c->spin_limit;
  P.tx_shortfall = c->tx_shortfall;
  c->tx_shortfall = 0;
  P.want_argmax = 1;
  P.trace = c->trace;
  c->barrier_skew = 0;
  RUAI_TRY(ruai_pstep_launch(c, P));
  S.bar_base += (5u * m->L + 2u) * (unsigned)grid;  // one arrival per CTA at each of the step's barriers
  m->graph_launches = 1;
  m->len += 1;
  return RUAI_OK;
}

int prepare_step(ruai_model* m, uint32_t B, uint32_t T, bool all_positions) {
  if (!m->quantized) return model_fail(m, RUAI_ERR_UNSUPPORTED, "only the quantized model is implemented on this path: call quantize first");
  if (B == 0 || T == 0) return model_fail(m, RUAI_ERR_SHAPE, "empty token batch [%u, %u]", B, T);
  // llama.rs:444-445 / gpt2.rs:224
  if (m->len + T > m->max_pos)
    return model_fail(m, RUAI_ERR_SHAPE, "context %u exceeds %s %u", m->len + T, m->llama ? "max_position_embeddings" : "n_positions", m->max_pos);
  RUAI_TRY(ensure_cache(m, B, m->len + T));
  RUAI_TRY(ensure_activations(m, B * T, all_positions ? B * T : B, B, T));
  if (m->world > 1) RUAI_TRY(ruai_tp_check_ready(m->ctx, &m->tp, B * T, m->d));
  return RUAI_OK;
}

}  // namespace

// ---- C ABI ---------------------------------------------------------------------------------

static int run_decode_graph(ruai_model* m, uint32_t B);

RUAI_API int ruai_model_use_persistent_step(ruai_model* m, int on) {
  if (!m) return RUAI_ERR_ARG;
  RUAI_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
  m->ps.wanted = on ? 1 : 0;
  m->ps.tried = false;
  m->len_dirty = true;  // the two paths keep the position in different places; the host's copy is uploaded again
  return RUAI_OK;
}

RUAI_API int ruai_model_uses_persistent_step(ruai_model* m, uint32_t B) {
  return m && pstep_eligible(m, B) ? 1 : 0;
}

RUAI_API int ruai_llama_create(ruai_ctx* c, const ruai_llama_config* cfg, const ruai_tp* tp, ruai_model** out) {
  if (!c || !cfg || !out) return ruai_fail(c, RUAI_ERR_ARG, "ruai_llama_create: NULL argument");
  *out = nullptr;
  const uint32_t world = tp ? tp->world : 1, rank = tp ? tp->rank : 0;
  if (world == 0 || rank >= world) return ruai_fail(c, RUAI_ERR_ARG, "bad tensor-parallel placement %u of %u", rank, world);
  if (!cfg->num_attention_heads || !cfg->num_key_value_heads || cfg->num_attention_heads % cfg->num_key_value_heads)
    return ruai_fail(c, RUAI_ERR_SHAPE, "heads %u must be a multiple of kv_heads %u", cfg->num_attention_heads, cfg->num_key_value_heads);
  if (cfg->head_dim == 0 || cfg->head_dim % 2) return ruai_fail(c, RUAI_ERR_SHAPE, "RoPE needs an even head_dim, got %u", cfg->head_dim);
  if (cfg->num_key_value_heads % world || cfg->intermediate_size % world || cfg->vocab_size % world)
    return ruai_fail(c, RUAI_ERR_SHAPE, "kv heads %u, intermediate %u and vocab %u must divide by the tensor-parallel world %u",
                     cfg->num_key_value_heads, cfg->intermediate_size, cfg->vocab_size, world);
  DeviceGuard g(c->ordinal);
  ruai_model* m = new ruai_model();
  m->ctx = c; m->llama = true; m->lc = *cfg;
  m->L = cfg->num_hidden_layers; m->d = cfg->hidden_size; m->H = cfg->num_attention_heads; m->KV = cfg->num_key_value_heads;
  m->hd = cfg->head_dim; m->ffn = cfg->intermediate_size; m->V = cfg->vocab_size; m->max_pos = cfg->max_position_embeddings;
  m->eps = cfg->rms_norm_eps; m->tied = cfg->tie_word_embeddings != 0;
  m->rank = rank; m->world = world;
  m->Hl = m->H / world; m->KVl = m->KV / world; m->fl = m->ffn / world; m->Vl = m->V / world;
  int rc = finish_create(m);
  if (rc == RUAI_OK && world > 1) rc = ruai_tp_init(c, &m->tp, rank, world, m->d);
  if (rc != RUAI_OK) { ruai_model_destroy(m); return rc; }
  *out = m;
  return RUAI_OK;
}

RUAI_API int ruai_gpt2_create(ruai_ctx* c, const ruai_gpt2_config* cfg, ruai_model** out) {
  if (!c || !cfg || !out) return ruai_fail(c, RUAI_ERR_ARG, "ruai_gpt2_create: NULL argument");
  *out = nullptr;
  if (!cfg->n_head || cfg->n_embd % cfg->n_head) return ruai_fail(c, RUAI_ERR_SHAPE, "n_embd %u must be divisible by n_head %u", cfg->n_embd, cfg->n_head);
  DeviceGuard g(c->ordinal);
  ruai_model* m = new ruai_model();
  m->ctx = c; m->llama = false; m->gc = *cfg;
  m->L = cfg->n_layer; m->d = cfg->n_embd; m->H = cfg->n_head; m->KV = cfg->n_head; m->hd = cfg->n_embd / cfg->n_head;
  m->ffn = 4 * cfg->n_embd; m->V = cfg->vocab_size; m->max_pos = cfg->n_positions; m->tied = true;
  m->Hl = m->H; m->KVl = m->KV; m->fl = m->ffn; m->Vl = m->V;
  int rc = finish_create(m);
  if (rc != RUAI_OK) { ruai_model_destroy(m); return rc; }
  *out = m;
  return RUAI_OK;
}

RUAI_API int ruai_model_destroy(ruai_model* m) {
  if (!m) return RUAI_OK;
  DeviceGuard g(m->ctx->ordinal);
  cudaStreamSynchronize(m->ctx->stream);
  drop_graph(m);
  ruai_tp_destroy(&m->tp);
  for (auto& kv : m->staged) kv.second.release();
  for (auto& kv : m->staged_q) delete kv.second;
  for (Layer& L : m->layers) {
    for (Lin* l : {&L.qkv, &L.o, &L.up, &L.down}) { if (l->w) ruai_qweight_free(l->w); ruai_sweight_free(&l->sw); l->bias.release(); }
    for (DevBuf* b : {&L.n1w, &L.n1b, &L.n2w, &L.n2b, &L.kc, &L.vc}) b->release();
  }
  if (m->head.w) ruai_qweight_free(m->head.w);
  ruai_sweight_free(&m->head.sw);
  for (DevBuf* b : {&m->ps.layers, &m->ps.x, &m->ps.ss, &m->ps.acc, &m->ps.poison, &m->ps.att_part, &m->ps.arg_slots, &m->ps.sync}) b->release();
  for (DevBuf* b : {&m->embed, &m->wpe, &m->final_w, &m->final_b, &m->rope_table, &m->d_ids, &m->d_len, &m->d_err, &m->x, &m->xn, &m->qkv, &m->att,
                    &m->hbuf, &m->xl, &m->logits, &m->attn_scratch, &m->attn_counters, &m->sumsq, &m->arg_slots, &m->arg_counter})
    b->release();
  delete m;
  return RUAI_OK;
}

RUAI_API int ruai_model_set_f32(ruai_model* m, uint64_t id, const float* data, size_t count) {
  if (!m || !data) return ruai_fail(m ? m->ctx : nullptr, RUAI_ERR_ARG, "ruai_model_set_f32: NULL argument");
  if (m->quantized) return model_fail(m, RUAI_ERR_UNSUPPORTED, "the model is already quantized");
  TensorShape s;
  if (!tensor_shape(m, id, &s)) return model_fail(m, RUAI_ERR_ARG, "tensor id 0x%llx does not exist in this model", (unsigned long long)id);
  if (s.rows * s.cols != count) return model_fail(m, RUAI_ERR_SHAPE, "tensor 0x%llx has %zu elements, got %zu", (unsigned long long)id, s.rows * s.cols, count);
  DeviceGuard g(m->ctx->ordinal);
  DevBuf* b;
  RUAI_TRY(stage_alloc(m, id, count, &b));
  RUAI_CUDA(m->ctx, cudaMemcpyAsync(b->p, data, count * sizeof(float), cudaMemcpyHostToDevice, m->ctx->stream));
  RUAI_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
  return RUAI_OK;
}

RUAI_API int ruai_model_set_quantized(ruai_model* m, uint64_t id, const int8_t* q_host, const float* scale_host, uint32_t bits, uint32_t group) {
  if (!m || !q_host || !scale_host) return ruai_fail(m ? m->ctx : nullptr, RUAI_ERR_ARG, "ruai_model_set_quantized: NULL argument");
  if (m->quantized) return model_fail(m, RUAI_ERR_UNSUPPORTED, "the model is already quantized");
  if (m->world > 1) return model_fail(m, RUAI_ERR_UNSUPPORTED, "loading quantized tensors into a sharded model is not implemented");
  TensorShape s;
  const bool is_linear = id == RUAI_T_LMHEAD || (id < (uint64_t)m->L * 16 && (m->llama ? (id % 16) <= RUAI_T_DOWN : ((id % 16) >= RUAI_T_CATTN && (id % 16) <= RUAI_T_MPROJ)));
  if (id == RUAI_T_LMHEAD) s = {m->d, m->V};
  else if (!is_linear || !tensor_shape(m, id, &s)) return model_fail(m, RUAI_ERR_ARG, "tensor id 0x%llx is not a Linear weight of this model", (unsigned long long)id);
  if (bits != 8 && bits != 4) return model_fail(m, RUAI_ERR_ARG, "bits must be 8 or 4, got %u", bits);
  const uint32_t k = (uint32_t)s.rows, n = (uint32_t)s.cols;
  if (bits == 4 && !(group >= 2 && group % 2 == 0 && k % group == 0))
    return model_fail(m, RUAI_ERR_SHAPE, "int4 group %u must be even and divide in_features %u", group, k);
  DeviceGuard g(m->ctx->ordinal);
  RefQ* r = new RefQ();
  r->k = k; r->n = n; r->bits = bits; r->group = bits == 4 ? group : 0;
  const size_t qb = (size_t)r->q_rows() * n, sb = (size_t)r->s_rows() * n * sizeof(float);
  int rc = r->q.alloc(m->ctx, qb);
  if (rc == RUAI_OK) rc = r->scale.alloc(m->ctx, sb);
  if (rc != RUAI_OK) { delete r; return rc; }
  cudaError_t e = cudaMemcpyAsync(r->q.p, q_host, qb, cudaMemcpyHostToDevice, m->ctx->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(r->scale.p, scale_host, sb, cudaMemcpyHostToDevice, m->ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(m->ctx->stream);
  if (e != cudaSuccess) { delete r; return model_fail(m, RUAI_ERR_CUDA, "ruai_model_set_quantized: %s", cudaGetErrorString(e)); }
  auto it = m->staged_q.find(id);
  if (it != m->staged_q.end()) { delete it->second; m->staged_q.erase(it); }
  m->staged_q[id] = r;
  return RUAI_OK;
}

RUAI_API int ruai_model_get_f32(ruai_model* m, uint64_t id, float* out_host, size_t count) {
  if (!m || !out_host) return ruai_fail(m ? m->ctx : nullptr, RUAI_ERR_ARG, "ruai_model_get_f32: NULL argument");
  if (!m->quantized) return model_fail(m, RUAI_ERR_UNSUPPORTED, "the model is not loaded");
  const DevBuf* b = nullptr;
  if (id == RUAI_T_EMBED) b = &m->embed;
  else if (id == RUAI_T_WPE && !m->llama) b = &m->wpe;
  else if (id == RUAI_TN_FINAL_NORM) b = &m->final_w;
  else if (id == RUAI_TN_FINAL_NORM_B && !m->llama) b = &m->final_b;
  else if (id >= RUAI_TN_LAYER_NORM1 && id < RUAI_TN_LAYER_NORM1 + m->L) b = &m->layers[id - RUAI_TN_LAYER_NORM1].n1w;
  else if (id >= RUAI_TN_LAYER_NORM2 && id < RUAI_TN_LAYER_NORM2 + m->L) b = &m->layers[id - RUAI_TN_LAYER_NORM2].n2w;
  else if (!m->llama && id >= RUAI_TN_LAYER_NORM1B && id < RUAI_TN_LAYER_NORM1B + m->L) b = &m->layers[id - RUAI_TN_LAYER_NORM1B].n1b;
  else if (!m->llama && id >= RUAI_TN_LAYER_NORM2B && id < RUAI_TN_LAYER_NORM2B + m->L) b = &m->layers[id - RUAI_TN_LAYER_NORM2B].n2b;
  else if (!m->llama && id < (uint64_t)m->L * 16) {
    Layer& Y = m->layers[id / 16];
    switch ((uint32_t)(id % 16)) {
      case RUAI_T_CATTN_B: b = &Y.qkv.bias; break;
      case RUAI_T_CPROJ_B: b = &Y.o.bias; break;
      case RUAI_T_CFC_B: b = &Y.up.bias; break;
      case RUAI_T_MPROJ_B: b = &Y.down.bias; break;
      default: break;
    }
  }
  if (!b || !b->p) return model_fail(m, RUAI_ERR_ARG, "no f32 tensor with id 0x%llx in this model", (unsigned long long)id);
  if (b->bytes != count * sizeof(float)) return model_fail(m, RUAI_ERR_SHAPE, "tensor 0x%llx has %zu elements, got %zu", (unsigned long long)id, b->bytes / sizeof(float), count);
  DeviceGuard g(m->ctx->ordinal);
  RUAI_CUDA(m->ctx, cudaMemcpyAsync(out_host, b->p, b->bytes, cudaMemcpyDeviceToHost, m->ctx->stream));
  RUAI_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
  return RUAI_OK;
}

RUAI_API int ruai_model_quantize(ruai_model* m, uint32_t bits, uint32_t group) {
  if (!m) return ruai_fail(nullptr, RUAI_ERR_ARG, "model is NULL");
  if (m->quantized) return RUAI_OK;  // quantize_* is a no-op on a quantized layer (layers.rs:113-115)
  if (bits != 8 && bits != 4) return model_fail(m, RUAI_ERR_ARG, "bits must be 8 or 4, got %u", bits);
  DeviceGuard g(m->ctx->ordinal);
  for (uint32_t l = 0; l < m->L; ++l) RUAI_TRY(quantize_layer(m, l, bits, group));
  RUAI_TRY(quantize_head(m));
  m->quantized = true; m->bits = bits; m->group = bits == 4 ? group : 0;
  return RUAI_OK;
}

RUAI_API int ruai_model_load_synthetic(ruai_model* m, uint64_t seed, uint32_t bits, uint32_t group) {
  if (!m) return ruai_fail(nullptr, RUAI_ERR_ARG, "model is NULL");
  if (m->quantized) return model_fail(m, RUAI_ERR_UNSUPPORTED, "the model is already loaded");
  if (bits != 8 && bits != 4) return model_fail(m, RUAI_ERR_ARG, "bits must be 8 or 4, got %u", bits);
  DeviceGuard g(m->ctx->ordinal);
  for (uint32_t l = 0; l < m->L; ++l) {
    if (m->llama) {
      for (uint32_t kind : {RUAI_T_Q, RUAI_T_K, RUAI_T_V, RUAI_T_O, RUAI_T_GATE, RUAI_T_UP, RUAI_T_DOWN}) RUAI_TRY(stage_synth(m, seed, ruai_layer_tensor(l, kind), 0.02));
    } else {
      for (uint32_t kind : {RUAI_T_CATTN, RUAI_T_CPROJ, RUAI_T_CFC, RUAI_T_MPROJ, RUAI_T_CATTN_B, RUAI_T_CPROJ_B, RUAI_T_CFC_B, RUAI_T_MPROJ_B})
        RUAI_TRY(stage_synth(m, seed, ruai_layer_tensor(l, kind), 0.02));
      RUAI_TRY(stage_fill(m, RUAI_TN_LAYER_NORM1B + l, 0.0f));
      RUAI_TRY(stage_fill(m, RUAI_TN_LAYER_NORM2B + l, 0.0f));
    }
    RUAI_TRY(stage_fill(m, RUAI_TN_LAYER_NORM1 + l, 1.0f));
    RUAI_TRY(stage_fill(m, RUAI_TN_LAYER_NORM2 + l, 1.0f));
    RUAI_TRY(quantize_layer(m, l, bits, group));
  }
  RUAI_TRY(stage_synth(m, seed, RUAI_T_EMBED, 0.02));
  if (m->llama && !m->tied) RUAI_TRY(stage_synth(m, seed, RUAI_T_LMHEAD, 0.02));
  if (!m->llama) { RUAI_TRY(stage_synth(m, seed, RUAI_T_WPE, 0.02)); RUAI_TRY(stage_fill(m, RUAI_TN_FINAL_NORM_B, 0.0f)); }
  RUAI_TRY(stage_fill(m, RUAI_TN_FINAL_NORM, 1.0f));
  RUAI_TRY(quantize_head(m));
  m->quantized = true; m->bits = bits; m->group = bits == 4 ? group : 0;
  return RUAI_OK;
}

RUAI_API int ruai_model_get_linear(ruai_model* m, uint64_t id, int8_t* q_host, float* scale_host) {
  if (!m || !q_host || !scale_host) return ruai_fail(m ? m->ctx : nullptr, RUAI_ERR_ARG, "ruai_model_get_linear: NULL argument");
  if (!m->quantized) return model_fail(m, RUAI_ERR_UNSUPPORTED, "the model is not quantized");
  if (m->world > 1) return model_fail(m, RUAI_ERR_UNSUPPORTED, "reading a Linear back needs an unsharded model");
  DeviceGuard g(m->ctx->ordinal);
  const Lin* lin = nullptr;
  uint32_t c0 = 0, cols = 0, cs = 1;
  const uint32_t hd = m->hd, nq = m->H * hd, nkv = m->KV * hd;
  if (id == RUAI_T_LMHEAD) { lin = &m->head; cols = m->V; }
  else if (id < (uint64_t)m->L * 16) {
    Layer& Ly = m->layers[id / 16];
    switch ((uint32_t)(id % 16)) {
      case RUAI_T_Q: lin = &Ly.qkv; c0 = 0; cols = nq; break;
      case RUAI_T_K: lin = &Ly.qkv; c0 = nq; cols = nkv; break;
      case RUAI_T_V: lin = &Ly.qkv; c0 = nq + nkv; cols = nkv; break;
      case RUAI_T_O: case RUAI_T_CPROJ: lin = &Ly.o; cols = m->d; break;
      case RUAI_T_GATE: lin = &Ly.up; c0 = 0; cols = m->ffn; cs = 2; break;
      case RUAI_T_UP: lin = &Ly.up; c0 = 1; cols = m->ffn; cs = 2; break;
      case RUAI_T_DOWN: case RUAI_T_MPROJ: lin = &Ly.down; cols = m->d; break;
      case RUAI_T_CATTN: lin = &Ly.qkv; cols = 3 * m->d; break;
      case RUAI_T_CFC: lin = &Ly.up; cols = m->ffn; break;
      default: break;
    }
    if (!m->llama && ((id % 16) < RUAI_T_CATTN)) lin = nullptr;
    if (m->llama && ((id % 16) > RUAI_T_DOWN)) lin = nullptr;
  }
  if (!lin || !lin->w) return model_fail(m, RUAI_ERR_ARG, "no Linear with id 0x%llx", (unsigned long long)id);
  const ruai_qweight* w = lin->w;
  const uint32_t q_rows = w->bits == 8 ? w->k : w->k / 2, s_rows = w->bits == 8 ? 1 : w->k / w->group;
  std::vector<int8_t> q((size_t)q_rows * w->n);
  std::vector<float> s((size_t)s_rows * w->n);
  RUAI_TRY(ruai_unpack(m->ctx, w, q.data(), s.data()));
  for (uint32_t r = 0; r < q_rows; ++r)
    for (uint32_t j = 0; j < cols; ++j) q_host[(size_t)r * cols + j] = q[(size_t)r * w->n + c0 + (size_t)j * cs];
  for (uint32_t r = 0; r < s_rows; ++r)
    for (uint32_t j = 0; j < cols; ++j) scale_host[(size_t)r * cols + j] = s[(size_t)r * w->n + c0 + (size_t)j * cs];
  return RUAI_OK;
}

RUAI_API int ruai_model_forward_cached(ruai_model* m, const int32_t* ids, uint32_t B, uint32_t T, float* logits_host, int all_positions) {
  if (!m || !ids) return ruai_fail(m ? m->ctx : nullptr, RUAI_ERR_ARG, "ruai_model_forward_cached: NULL argument");
  ruai_ctx* c = m->ctx;
  DeviceGuard g(c->ordinal);
  RUAI_TRY(prepare_step(m, B, T, all_positions != 0));
  RUAI_CUDA(c, cudaMemcpyAsync(m->d_ids.p, ids, (size_t)B * T * sizeof(int32_t), cudaMemcpyHostToDevice, c->stream));
  const int32_t len = (int32_t)m->len;
  RUAI_CUDA(c, cudaMemcpyAsync(m->d_len.p, &len, sizeof len, cudaMemcpyHostToDevice, c->stream));
  m->len_dirty = false;
  if (T == 1) RUAI_TRY(run_decode_graph(m, B));  // single-token steps: the persistent kernel, or the captured graph
  else {
    RUAI_TRY(issue_step(m, B, T, all_positions != 0, false));
    m->len += T;
  }
  if (logits_host) {
    if (m->world > 1) return model_fail(m, RUAI_ERR_UNSUPPORTED, "full logits of a sharded head are not gathered; use decode_step / generate");
    const size_t rows = all_positions ? (size_t)B * T : B;
    RUAI_CUDA(c, cudaMemcpyAsync(logits_host, m->logits.p, rows * m->V * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  }
  return check_device_status(m);
}

RUAI_API int ruai_model_cache_clear(ruai_model* m) {
  if (!m) return ruai_fail(nullptr, RUAI_ERR_ARG, "model is NULL");
  m->len = 0;  // KvCache::clear keeps the buffers (transformer.rs:160-165)
  m->len_dirty = true;
  return RUAI_OK;
}

RUAI_API int ruai_model_cache_len(const ruai_model* m, uint32_t* len, uint32_t* cap) {
  if (!m) return ruai_fail(nullptr, RUAI_ERR_ARG, "model is NULL");
  if (len) *len = m->len;
  if (cap) *cap = m->cap;
  return RUAI_OK;
}

RUAI_API int ruai_model_cache_reserve(ruai_model* m, uint32_t B, uint32_t positions) {
  if (!m) return ruai_fail(nullptr, RUAI_ERR_ARG, "model is NULL");
  if (positions > m->max_pos) return model_fail(m, RUAI_ERR_SHAPE, "context %u exceeds the maximum %u", positions, m->max_pos);
  DeviceGuard g(m->ctx->ordinal);
  return ensure_cache(m, B, positions);
}

RUAI_API int ruai_model_cache_assume(ruai_model* m, uint32_t B, uint32_t len) {
  if (!m) return ruai_fail(nullptr, RUAI_ERR_ARG, "model is NULL");
  if (len + 1 > m->max_pos) return model_fail(m, RUAI_ERR_SHAPE, "context %u exceeds the maximum %u", len + 1, m->max_pos);
  DeviceGuard g(m->ctx->ordinal);
  m->len = 0;
  RUAI_TRY(ensure_cache(m, B, len + 1));
  m->len = len;
  const int32_t l = (int32_t)len;
  RUAI_CUDA(m->ctx, cudaMemcpyAsync(m->d_len.p, &l, sizeof l, cudaMemcpyHostToDevice, m->ctx->stream));
  RUAI_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
  m->len_dirty = false;
  return RUAI_OK;
}

// Replays (capturing first if needed) the graph of one greedy decode step for batch B.
static int run_decode_graph(ruai_model* m, uint32_t B) {
  ruai_ctx* c = m->ctx;
  if (pstep_eligible(m, B)) return pstep_run(m, B);
  if (!m->graph || m->graph_B != B || m->graph_cap != m->cap || m->graph_epoch != c->scratch_epoch) {
    drop_graph(m);
    // split-K partials of one GEMV never exceed (3 * SMs + column tiles) * 256 floats per row;
    // reserve before capturing (no allocation inside a capture)
    uint32_t max_n = m->head.w->n;
    for (Layer& L : m->layers) max_n = std::max(max_n, std::max(L.up.w->n, L.qkv.w->n));
    const size_t tiles = (max_n + 255) / 256;
    size_t need = ((size_t)3 * c->sm_count + tiles + 1) * 256 * B * sizeof(float);
    need = std::max(need, ruai_gemv_xs_bytes(m->head.w, B));  // the split activations of the tensor-core tiles live there too
    for (Layer& L : m->layers)
      for (const ruai_qweight* w : {L.qkv.w, L.o.w, L.up.w, L.down.w})
        if (w) need = std::max(need, ruai_gemv_xs_bytes(w, B));
    RUAI_TRY(ruai_ctx_reserve(c, need, tiles * ((B + 15) / 16) + 16));
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    const unsigned long long before = c->launches;
    cudaGraph_t gr = nullptr;
    RUAI_CUDA(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    int rc = issue_step(m, B, 1, false, true);
    cudaError_t e = cudaStreamEndCapture(c->stream, &gr);
    if (rc != RUAI_OK) { if (gr) cudaGraphDestroy(gr); return rc; }
    if (e != cudaSuccess) return model_fail(m, RUAI_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    m->graph_launches = (uint32_t)(c->launches - before);
    e = cudaGraphInstantiate(&m->graph, gr, 0);
    cudaGraphDestroy(gr);
    if (e != cudaSuccess) { m->graph = nullptr; return model_fail(m, RUAI_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e)); }
    m->graph_B = B; m->graph_cap = m->cap; m->graph_epoch = c->scratch_epoch;
  }
  RUAI_CUDA(c, cudaGraphLaunch(m->graph, c->stream));
  m->len += 1;
  return RUAI_OK;
}

RUAI_API int ruai_model_decode_step(ruai_model* m, const int32_t* ids_dev, uint32_t B, int32_t* next_host) {
  if (!m) return ruai_fail(nullptr, RUAI_ERR_ARG, "model is NULL");
  ruai_ctx* c = m->ctx;
  DeviceGuard g(c->ordinal);
  RUAI_TRY(prepare_step(m, B, 1, false));
  if (ids_dev) RUAI_CUDA(c, cudaMemcpyAsync(m->d_ids.p, ids_dev, (size_t)B * sizeof(int32_t), cudaMemcpyDeviceToDevice, c->stream));
  if (m->len_dirty) {  // the host's position is the authority: a cleared or re-assumed cache has not reached the device yet
    const int32_t len = (int32_t)m->len;
    RUAI_CUDA(c, cudaMemcpyAsync(m->d_len.p, &len, sizeof len, cudaMemcpyHostToDevice, c->stream));
    RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
    m->len_dirty = false;
  }
  RUAI_TRY(run_decode_graph(m, B));
  if (next_host) {
    RUAI_CUDA(c, cudaMemcpyAsync(next_host, m->d_ids.p, (size_t)B * sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream));
    return check_device_status(m);
  }
  return RUAI_OK;
}

// Times `iters` passes over every quantized Linear of the model (the weight-streaming
// kernels of one decode step, nothing else) for B rows, with CUDA events on the stream.
RUAI_API int ruai_model_time_linears(ruai_model* m, uint32_t B, uint32_t iters, float* ms_total, uint32_t* launches, double* bytes_per_pass) {
  if (!m || !ms_total) return ruai_fail(nullptr, RUAI_ERR_ARG, "NULL argument");
  if (!m->quantized) return model_fail(m, RUAI_ERR_UNSUPPORTED, "the model is not quantized");
  ruai_ctx* c = m->ctx;
  DeviceGuard g(c->ordinal);
  RUAI_TRY(ensure_activations(m, B, B, B, 1));
  float *xn = m->xn.as<float>(), *qkv = m->qkv.as<float>(), *att = m->att.as<float>(), *hb = m->hbuf.as<float>(), *xl = m->xl.as<float>();
  RUAI_CUDA(c, cudaMemsetAsync(xn, 0, (size_t)B * m->d * sizeof(float), c->stream));
  RUAI_CUDA(c, cudaMemsetAsync(att, 0, (size_t)B * m->Hl * m->hd * sizeof(float), c->stream));
  RUAI_CUDA(c, cudaMemsetAsync(hb, 0, (size_t)B * m->fl * sizeof(float), c->stream));
  double bytes = 0.0;
  uint32_t n_launch = 0;
  auto pass = [&](bool count) -> int {
    for (Layer& Ly : m->layers) {
      GemvEpilogue e0, e1, e2, e3;
      e0.bias = Ly.qkv.bias.as<float>(); e1.bias = Ly.o.bias.as<float>(); e2.bias = Ly.up.bias.as<float>(); e3.bias = Ly.down.bias.as<float>();
      e2.act = m->llama ? ACT_SWIGLU : ACT_GELU;
      GemvPrologue p0, p1, p2, p3;
      const size_t li = (size_t)(&Ly - m->layers.data());
      RUAI_TRY(ruai_gemv_launch(c, Ly.qkv.w, xn, RUAI_F32, m->d, B, qkv, e0, p0));
      RUAI_TRY(ruai_gemv_launch(c, Ly.o.w, att, RUAI_F32, m->Hl * m->hd, B, xl, e1, p1));
      RUAI_TRY(ruai_gemv_launch(c, Ly.up.w, xn, RUAI_F32, m->d, B, hb, e2, p2));
      RUAI_TRY(ruai_gemv_launch(c, Ly.down.w, hb, RUAI_F32, m->fl, B, xl, e3, p3));
      if (count) {
        for (const Lin* l : {&Ly.qkv, &Ly.o, &Ly.up, &Ly.down}) bytes += l->bytes() + 4.0 * B * (l->w->k + l->w->n);
        n_launch += 4;
      }
    }
    GemvEpilogue eh;
    RUAI_TRY(ruai_gemv_launch(c, m->head.w, xn, RUAI_F32, m->d, B, m->logits.as<float>(), eh));
    if (count) { bytes += m->head.bytes() + 4.0 * B * (m->head.w->k + m->head.w->n); n_launch += 1; }
    return RUAI_OK;
  };
  RUAI_TRY(pass(true));  // warm-up, also sizes the scratch
  RUAI_CUDA(c, cudaStreamSynchronize(c->stream));
  RUAI_CUDA(c, cudaEventRecord(c->ev0, c->stream));
  for (uint32_t i = 0; i < iters; ++i) RUAI_TRY(pass(false));
  RUAI_CUDA(c, cudaEventRecord(c->ev1, c->stream));
  RUAI_CUDA(c, cudaEventSynchronize(c->ev1));
  RUAI_CUDA(c, cudaEventElapsedTime(ms_total, c->ev0, c->ev1));
  if (launches) *launches = n_launch;
  if (bytes_per_pass) *bytes_per_pass = bytes;
  return RUAI_OK;
}

RUAI_API int ruai_model_step_launches(const ruai_model* m, uint32_t* launches) {
  if (!m || !launches) return ruai_fail(nullptr, RUAI_ERR_ARG, "NULL argument");
  *launches = m->graph_launches;
  return RUAI_OK;
}

RUAI_API int ruai_model_step_bytes(const ruai_model* m, uint32_t B, uint32_t len, double* bytes) {
  if (!m || !bytes) return ruai_fail(nullptr, RUAI_ERR_ARG, "NULL argument");
  double w = 0.0;
  for (const Layer& L : m->layers) {
    w += L.qkv.bytes() + L.o.bytes() + L.up.bytes() + L.down.bytes();
    w += (double)(L.n1w.bytes + L.n1b.bytes + L.n2w.bytes + L.n2b.bytes);
  }
  w += m->head.bytes() + (double)(m->final_w.bytes + m->final_b.bytes);
  const double kv_pos = 2.0 * m->L * m->KVl * m->hd * sizeof(float);
  const double per_seq = 4.0 * m->d * (m->llama ? 1 : 2) + kv_pos * len + kv_pos;
  *bytes = w + (double)B * per_seq;
  return RUAI_OK;
}

// generate_cached with Sampler::greedy (generation.rs:83-113): batch 1, sliding window.
namespace {
struct SamplerArgs { float temperature; uint32_t top_k; float top_p; uint64_t state; };
}
static int generate_impl(ruai_model* m, const int32_t* prompt, uint32_t T, uint32_t n_new, SamplerArgs* sampler, int32_t* out);

RUAI_API int ruai_model_generate(ruai_model* m, const int32_t* prompt, uint32_t T, uint32_t n_new, int32_t* out) {
  return generate_impl(m, prompt, T, n_new, nullptr, out);
}

RUAI_API int ruai_model_generate_sampled(ruai_model* m, const int32_t* prompt, uint32_t T, uint32_t n_new, float temperature, uint32_t top_k, float top_p,
                                         uint64_t seed, int32_t* out) {
  SamplerArgs sa{temperature, top_k, top_p, seed};  // Sampler::new (generation.rs:28-30)
  if (m && m->world > 1) return model_fail(m, RUAI_ERR_UNSUPPORTED, "sampling needs the whole vocabulary on one GPU: the head of this model is sharded");
  return generate_impl(m, prompt, T, n_new, temperature > 0.0f ? &sa : nullptr, out);
}

static int generate_impl(ruai_model* m, const int32_t* prompt, uint32_t T, uint32_t n_new, SamplerArgs* sampler, int32_t* out) {
  if (!m || !prompt || !out) return ruai_fail(m ? m->ctx : nullptr, RUAI_ERR_ARG, "ruai_model_generate: NULL argument");
  if (T == 0) return model_fail(m, RUAI_ERR_ARG, "prompt must not be empty");
  ruai_ctx* c = m->ctx;
  DeviceGuard g(c->ordinal);
  const uint32_t max_len = m->max_pos;
  std::vector<int32_t> ids(prompt, prompt + T);
  m->len = 0;
  m->len_dirty = true;
  std::vector<int32_t> pending(ids.begin() + (ids.size() > max_len ? ids.size() - max_len : 0), ids.end());
  bool on_device = false;  // d_ids already holds the next token (written by the step's argmax)
  for (uint32_t s = 0; s < n_new; ++s) {
    if (m->len + pending.size() > max_len) {
      m->len = 0;
      m->len_dirty = true;
      pending.assign(ids.end() - max_len, ids.end());
      on_device = false;
    }
    int32_t next = 0;
    if (pending.size() == 1 && on_device) {
      RUAI_TRY(ruai_model_decode_step(m, nullptr, 1, &next));
    } else if (pending.size() == 1) {
      RUAI_TRY(prepare_step(m, 1, 1, false));
      RUAI_CUDA(c, cudaMemcpyAsync(m->d_ids.p, pending.data(), sizeof(int32_t), cudaMemcpyHostToDevice, c->stream));
      const int32_t len = (int32_t)m->len;
      RUAI_CUDA(c, cudaMemcpyAsync(m->d_len.p, &len, sizeof len, cudaMemcpyHostToDevice, c->stream));
      RUAI_TRY(ruai_model_decode_step(m, nullptr, 1, &next));
    } else {
      const uint32_t Tn = (uint32_t)pending.size();
      RUAI_TRY(prepare_step(m, 1, Tn, false));
      RUAI_CUDA(c, cudaMemcpyAsync(m->d_ids.p, pending.data(), (size_t)Tn * sizeof(int32_t), cudaMemcpyHostToDevice, c->stream));
      const int32_t len = (int32_t)m->len;
      RUAI_CUDA(c, cudaMemcpyAsync(m->d_len.p, &len, sizeof len, cudaMemcpyHostToDevice, c->stream));
      m->len_dirty = false;
      RUAI_TRY(issue_step(m, 1, Tn, false, true));
      m->len += Tn;
      RUAI_CUDA(c, cudaMemcpyAsync(&next, m->d_ids.p, sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream));
      RUAI_TRY(check_device_status(m));
    }
    if (sampler) {  // the step left the argmax in d_ids; the sampled token replaces it there
      RUAI_TRY(ruai_sample_device(c, m->logits.as<float>(), m->V, sampler->temperature, sampler->top_k, sampler->top_p, &sampler->state, m->d_ids.as<int32_t>()));
      RUAI_CUDA(c, cudaMemcpyAsync(&next, m->d_ids.p, sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream));
      RUAI_TRY(check_device_status(m));
    }
    on_device = true;
    ids.push_back(next);
    pending.assign(1, next);
  }
  memcpy(out, ids.data(), ids.size() * sizeof(int32_t));
  return RUAI_OK;
}

RUAI_API int ruai_tp_export(ruai_model* m, void* handle_out) {
  if (!m || !handle_out) return ruai_fail(nullptr, RUAI_ERR_ARG, "NULL argument");
  if (m->world <= 1) return model_fail(m, RUAI_ERR_UNSUPPORTED, "the model is not sharded");
  DeviceGuard g(m->ctx->ordinal);
  return ruai_tp_export_handle(m->ctx, &m->tp, handle_out);
}

RUAI_API int ruai_tp_resync(ruai_model* m) {
  if (!m) return ruai_fail(nullptr, RUAI_ERR_ARG, "NULL argument");
  if (m->world <= 1) return model_fail(m, RUAI_ERR_UNSUPPORTED, "the model is not sharded");
  DeviceGuard g(m->ctx->ordinal);
  RUAI_TRY(ruai_tp_resync_state(m->ctx, &m->tp));
  RUAI_CUDA(m->ctx, cudaMemset(m->d_err.p, 0, sizeof(int32_t)));
  (void)ruai_ctx_check_status(m->ctx);  // clears a pending status word
  return RUAI_OK;
}

RUAI_API int ruai_tp_connect(ruai_model* m, const void* handles) {
  if (!m || !handles) return ruai_fail(nullptr, RUAI_ERR_ARG, "NULL argument");
  if (m->world <= 1) return model_fail(m, RUAI_ERR_UNSUPPORTED, "the model is not sharded");
  DeviceGuard g(m->ctx->ordinal);
  return ruai_tp_connect_handles(m->ctx, &m->tp, handles);
}
