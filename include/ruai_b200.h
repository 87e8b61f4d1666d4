/* ruai_b200 — C ABI of the B200 (sm_100a) quantized-inference path.
 *
 * This library stands behind the three quantized-matmul methods of ruai's
 * `trait Backend` (src/nn/backend/mod.rs:675-704: matmul_int8, dequant_int4,
 * matmul_int4), whose CUDA bodies are src/nn/backend/cuda.rs:788-833, and behind
 * the model surface that drives them (`Linear::quantize_int8/int4`,
 * src/nn/modules/layers.rs:112-165; `Llama` / `GPT2` `forward_cached`,
 * `generate`, `quantize_int8/int4`, src/nn/modules/{llama,gpt2}.rs).
 *
 * Conventions
 *  - every entry point returns an int status (RUAI_OK == 0).  The reference
 *    panics on error (cuda.rs:256, ops.rs:694-699); a binding turns a non-zero
 *    status plus ruai_last_error() into that panic.
 *  - pointers named *_dev are device pointers on the context's GPU; pointers
 *    named *_host are host pointers; plain names accept either (the library
 *    asks the driver which it is).
 *  - all work is issued on the context's stream and is asynchronous unless a
 *    host buffer has to be filled.
 *  - matrices are row-major.  Weights are `[in, out]` = `[k, n]` as in the
 *    reference (`Linear::weight`, layers.rs:29).
 *  - there is no CPU fallback: without a CUDA device every call that touches
 *    data fails with RUAI_ERR_CUDA.
 */
#ifndef RUAI_B200_H
#define RUAI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ruai_ctx ruai_ctx;         /* one per device: stream, scratch, error text */
typedef struct ruai_qweight ruai_qweight; /* repacked quantized weight, device resident, immutable */
typedef struct ruai_model ruai_model;     /* a Llama or GPT-2 with its KV cache */

enum {
  RUAI_OK = 0,
  RUAI_ERR_SHAPE = 1,       /* the reference's shape / group asserts */
  RUAI_ERR_CUDA = 2,        /* a CUDA call failed or no device / library */
  RUAI_ERR_COMM = 3,        /* tensor-parallel exchange failed */
  RUAI_ERR_TIMEOUT = 4,     /* a bounded device-side wait ran out */
  RUAI_ERR_UNSUPPORTED = 5,
  RUAI_ERR_ARG = 6
};

/* Activation dtypes; mirrors DType::{F32,F16,BF16} (mod.rs:32-44). */
enum { RUAI_F32 = 0, RUAI_F16 = 1, RUAI_BF16 = 2 };

/* ---- context ------------------------------------------------------------ */

/* Replaces `cuda::backend(ordinal)` (cuda.rs:82-86, 262-281): one context and
 * stream per device ordinal.  `stream_or_null` is a cudaStream_t to adopt. */
int ruai_ctx_create(int ordinal, void* stream_or_null, ruai_ctx** out);
int ruai_ctx_destroy(ruai_ctx* ctx);
/* Text of the last failure on this context (or the last context-less failure
 * when ctx is NULL).  Valid until the next failing call. */
const char* ruai_last_error(const ruai_ctx* ctx);
/* `Backend::synchronize` (cuda.rs:447-452). */
int ruai_ctx_synchronize(ruai_ctx* ctx);
/* `Device::is_available` (cuda.rs:73-79): number of CUDA devices, 0 if none. */
int ruai_device_count(void);
/* Library version string. */
const char* ruai_version(void);

/* Bound of every device-side wait of the persistent kernels, in polls (0 restores the default,
 * about a second).  A wait that runs out makes the launch return early; the next status check
 * reports RUAI_ERR_TIMEOUT and the context stays usable.  The reference has no counterpart (its
 * kernels never wait on one another). */
int ruai_ctx_set_wait_limit(ruai_ctx* ctx, unsigned polls);
/* Failure injection, on the host: the next persistent launch on this context is told that `grids`
 * more grid-wide arrivals precede it than really do, so its first grid barrier can never
 * complete and its bounded wait runs out.  Nothing faults; used by the timeout tests. */
int ruai_ctx_inject_barrier_skew(ruai_ctx* ctx, unsigned grids);
/* The same for a shared-memory barrier: the first bulk copy of the next persistent launch is announced `bytes` larger
 * than it is, so the barrier it signals never completes and the consumers' bounded wait for that stage runs out. */
int ruai_ctx_inject_copy_shortfall(ruai_ctx* ctx, unsigned bytes);
/* Tuning knob: fixes the split-k count (1..8 CTAs of a cluster share the k of a column tile) of the tensor-core GEMVs
 * on this context; 0 gives the choice back to the library's cost model.  Results do not depend on it beyond the order
 * of a few f32 additions.  `python -m ruai_b200.sweep_splits` uses it to compare the cost model with every fixed split
 * on a list of shapes.  No counterpart in the reference. */
int ruai_ctx_force_splits(ruai_ctx* ctx, unsigned splits);

/* Device memory for callers without their own allocator (cuda.rs:288-300). */
int ruai_malloc(ruai_ctx* ctx, size_t bytes, void** out_dev);
int ruai_free(ruai_ctx* ctx, void* ptr_dev);
int ruai_memcpy_h2d(ruai_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int ruai_memcpy_d2h(ruai_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);

/* Timing on the context's stream with CUDA events. */
int ruai_timer_start(ruai_ctx* ctx);
int ruai_timer_stop_ms(ruai_ctx* ctx, float* ms_out); /* records, synchronizes, returns elapsed */

/* ---- quantizer (Linear::quantize_int8 / quantize_int4) --------------------
 * Bit-exact with layers.rs:112-129 and layers.rs:139-165: f32 absmax, true
 * division, round-half-away, clamp.  The reference runs these loops on the
 * host after a device-to-host copy; here they run on the device.
 *   int8: q[k,n] i8, scale[n] f32           (per output column)
 *   int4: q[k/2,n] packed, scale[k/group,n] (low nibble = even row)          */
int ruai_quantize_int8(ruai_ctx* ctx, const float* w_dev, uint32_t k, uint32_t n,
                       int8_t* q_dev, float* scale_dev);
int ruai_quantize_int4(ruai_ctx* ctx, const float* w_dev, uint32_t k, uint32_t n, uint32_t group,
                       int8_t* q_dev, float* scale_dev);

/* ---- repack: reference layout -> kernel layout ----------------------------
 * Inputs are the reference's buffers `weight_int8`/`weight_scale` and
 * `weight_int4`/`weight_int4_scale` (layers.rs:205-211), host or device.
 * The kernel layout stores, for every output column j and every run c of 16
 * bytes along k, one 16-byte chunk at ((c * n + j) * 16): a warp that owns 32
 * neighbouring columns reads 512 contiguous bytes, and one chunk is 16 int8
 * rows, or the 32 int4 rows of one scale group.  Scales keep the reference's
 * values and order.  ruai_unpack() restores the reference bytes exactly.     */
int ruai_repack_int8(ruai_ctx* ctx, const int8_t* q, const float* scale, uint32_t k, uint32_t n,
                     ruai_qweight** out);
int ruai_repack_int4(ruai_ctx* ctx, const int8_t* q, const float* scale, uint32_t k, uint32_t n,
                     uint32_t group, ruai_qweight** out);
int ruai_unpack(ruai_ctx* ctx, const ruai_qweight* w, int8_t* q_out, float* scale_out);
int ruai_qweight_free(ruai_qweight* w);
/* k, n, bits (8 or 4), group (0 for int8). */
int ruai_qweight_info(const ruai_qweight* w, uint32_t* k, uint32_t* n, uint32_t* bits, uint32_t* group);

/* ---- Backend-trait equivalents -------------------------------------------- */

/* `Backend::matmul_int8` / `matmul_int4` (mod.rs:675-682, 700-704; CPU
 * definition cpu.rs:897-927, 1035-1067) followed by `Linear::forward`'s bias
 * add (layers.rs:184-189).  x_dev is [m,k] in x_dtype, out_dev is [m,n] in
 * x_dtype, bias_dev_or_null is f32 [n].  Sums, scales and bias are f32.  The
 * products run on the tensor cores with the weights exact: up to 4 rows the
 * activations as block fixed point of 21 (int4) or 28 (int8) bits, results
 * within 1e-4 * (1 + |y|) of the reference's CPU path (tests/devices.rs); from
 * 5 rows on (Linears of 4M weights and more) and in the many-row GEMM the
 * activations as two bf16 pieces (16 significant bits): max-abs 1e-2, 1e-3 of
 * the output's scale, and all but about 1e-4 of the outputs inside the 1e-4.
 * A non-finite activation makes its row of the output non-finite.           */
int ruai_matmul_q(ruai_ctx* ctx, int x_dtype, const void* x_dev, const ruai_qweight* w,
                  const float* bias_dev_or_null, void* out_dev, uint32_t m);
/* Backward of `Tensor::matmul_int8` / `matmul_int4` (ops.rs:705-709, 731-734): the weights are frozen, the only
 * gradient is dx[m,k] = g[m,n] @ dequant(W)^T.  The reference materialises the f32 weight for it; here the packed
 * weight is read once per row of g.  f32 in, f32 out, m <= 65535.                                                   */
int ruai_matmul_q_grad_input(ruai_ctx* ctx, const float* g_dev, const ruai_qweight* w, float* dx_dev, uint32_t m);
/* `Linear::forward` of a quantized layer with a LoRA adapter (layers.rs:169-190; add_lora 84-97), QLoRA-style:
 * out = matmul_q(x) + (x @ A @ B) * scale + bias, A [k,rank], B [rank,n] row-major f32, scale = alpha / rank,
 * in the reference's order of additions.  f32 activations; rank 1..1024.                                           */
int ruai_linear_lora_forward(ruai_ctx* ctx, const float* x_dev, const ruai_qweight* w, const float* lora_a_dev,
                             const float* lora_b_dev, uint32_t rank, float scale, const float* bias_dev_or_null,
                             float* out_dev, uint32_t m);
/* ruai_matmul_q for hosts that cannot let this library allocate device memory at run time
 * (a serving process whose framework already owns the whole device, or a loop that cannot
 * afford cudaMalloc's implicit synchronisation).  Same arguments; results within the same
 * tolerance of the reference's CPU path (it always runs the first-generation f32 kernel, so the
 * bits equal ruai_matmul_q's only with RUAI_B200_TC=0 and RUAI_B200_BULK=0).  It has no
 * counterpart in the reference.  The split-K scratch lives in a fixed 8 MiB + 16 KiB array
 * inside the loaded module (held on every GPU that loads the library until exit); a call
 * whose split plan needs more fails with RUAI_ERR_UNSUPPORTED and says so.  The first call
 * on a device looks the array's address up once; make that call before starting any stream
 * capture.  All calls on a device share the array: calls that overlap on the GPU race.
 * Only chunk-layout weights (int8, or int4 with group 32). */
int ruai_matmul_q_static(ruai_ctx* ctx, int x_dtype, const void* x_dev, const ruai_qweight* w,
                         const float* bias_dev_or_null, void* out_dev, uint32_t m);
/* The same product for 1 or 2 rows of f32 activations through the data path of the persistent
 * decode kernel (one cooperative launch, one CTA per SM, weights streamed through a ring of bulk
 * copies in the tile-stream layout, split-k sums met in 64-bit fixed-point accumulators, so the
 * result is bit-identical from run to run).  The tile-stream copy of the weight is built on the
 * first call and kept with the qweight.  `repeat` >= 1 runs the product that many times inside
 * the one launch (the phases of a decode step in miniature; used to time the streaming rate).
 * Replaces the same reference methods as ruai_matmul_q (mod.rs:675-682, 700-704).           */
int ruai_matmul_q_stream(ruai_ctx* ctx, const float* x_dev, const ruai_qweight* w, float* out_dev,
                         uint32_t m, uint32_t repeat);
/* `Backend::dequant_int4` (mod.rs:689-693, cpu.rs:1023-1033): exact f32 [k,n]. */
int ruai_dequant_int4(ruai_ctx* ctx, const ruai_qweight* w, float* out_dev);
/* Same on reference-layout device buffers, without a repack (any even group). */
int ruai_dequant_int4_ref(ruai_ctx* ctx, const int8_t* q_dev, const float* scale_dev,
                          uint32_t k, uint32_t n, uint32_t group, float* out_dev);

/* ---- models ---------------------------------------------------------------- */

/* Field names follow `LlamaConfig` (llama.rs:48-75). */
typedef struct {
  uint32_t vocab_size, hidden_size, intermediate_size, num_hidden_layers;
  uint32_t num_attention_heads, num_key_value_heads, head_dim, max_position_embeddings;
  float rms_norm_eps, rope_theta;
  uint32_t tie_word_embeddings;
} ruai_llama_config;

/* Field names follow `GPT2Config` (gpt2.rs:30-44). */
typedef struct {
  uint32_t vocab_size, n_positions, n_embd, n_layer, n_head;
} ruai_gpt2_config;

/* Tensor-parallel placement of one model replica: this process owns rank
 * `rank` of `world` (1 = no sharding).  Column-split q/k/v/gate/up and the
 * head, row-split o/down, one sum exchange after o_proj and down_proj.      */
typedef struct {
  uint32_t rank, world;
} ruai_tp;

int ruai_llama_create(ruai_ctx* ctx, const ruai_llama_config* cfg, const ruai_tp* tp_or_null,
                      ruai_model** out);
int ruai_gpt2_create(ruai_ctx* ctx, const ruai_gpt2_config* cfg, ruai_model** out);
int ruai_model_destroy(ruai_model* m);

/* Fill the model with the seeded synthetic weights of include/ruai_b200_synth.h
 * (N(0, 0.02^2) matrices and GPT-2 biases, unit norm gains), generated in f32
 * on the device, then quantized exactly as `Llama::quantize_int8` /
 * `quantize_int4(group)` (llama.rs:522-554, gpt2.rs:306-335) do: every block
 * Linear to `bits`, the output head to int8, embeddings left in f32.        */
int ruai_model_load_synthetic(ruai_model* m, uint64_t seed, uint32_t bits, uint32_t group);

/* Set one f32 tensor from host memory before quantizing (ids: ruai_b200_synth.h,
 * plus RUAI_TN_* below for norm parameters). `count` must match the shape.  */
#define RUAI_TN_FINAL_NORM   0x40000000ull /* Llama `norm.weight` / GPT-2 `ln_f.weight` */
#define RUAI_TN_FINAL_NORM_B 0x40000001ull /* GPT-2 `ln_f.bias` */
#define RUAI_TN_LAYER_NORM1  0x50000000ull /* + layer: input_layernorm / ln_1 weight */
#define RUAI_TN_LAYER_NORM1B 0x51000000ull /* + layer: ln_1 bias */
#define RUAI_TN_LAYER_NORM2  0x52000000ull /* + layer: post_attention_layernorm / ln_2 weight */
#define RUAI_TN_LAYER_NORM2B 0x53000000ull /* + layer: ln_2 bias */
int ruai_model_set_f32(ruai_model* m, uint64_t tensor_id, const float* data_host, size_t count);
/* Hand one Linear over already quantized, in the reference's buffer layout (`weight_int8` [k,n] +
 * `weight_scale` [n], or `weight_int4` [k/2,n] + `weight_int4_scale` [k/group,n]; layers.rs:205-211),
 * as a checkpoint saved by `serialize::save` of a quantized model holds it (serialize.rs:239-241).
 * ids: block Linears and RUAI_T_LMHEAD (`lm_head.weight_int8`, also present for a tied model).  The
 * following ruai_model_quantize(bits, group) repacks these as they are and quantizes only what was
 * set as f32. */
int ruai_model_set_quantized(ruai_model* m, uint64_t tensor_id, const int8_t* q_host, const float* scale_host,
                             uint32_t bits, uint32_t group);
/* Read back one f32 tensor of a loaded model (embeddings, norm parameters, GPT-2 biases): the
 * parameters `state_dict()` of a quantized model still holds (llama.rs:559-578, gpt2.rs:344-358). */
int ruai_model_get_f32(ruai_model* m, uint64_t tensor_id, float* out_host, size_t count);
/* Which of the two implementations of a single-token greedy step (ruai_model_decode_step, ruai_model_generate) the
 * model uses: the chain of launches, one kernel per Linear / attention (default), or ONE persistent cooperative kernel
 * per token (on != 0; Llama-shaped quantized models, one GPU, at most two sequences; other cases keep the chain).
 * Both compute the reference's step (llama.rs:441-463); they differ in speed and in the last bits of the logits.
 * Without a call the environment decides (RUAI_B200_PSTEP=1 selects the persistent kernel).
 * ruai_model_uses_persistent_step: 1 if steps of B sequences would run as the persistent kernel now. */
int ruai_model_use_persistent_step(ruai_model* m, int on);
int ruai_model_uses_persistent_step(ruai_model* m, uint32_t B);
/* `Llama::quantize_int8` / `quantize_int4(group)` over the f32 tensors set so far. */
int ruai_model_quantize(ruai_model* m, uint32_t bits, uint32_t group);
/* Read back one block Linear (or the head, tensor id RUAI_T_LMHEAD) in the
 * reference's buffer layout — what `state_dict()` would hold (layers.rs:205-211). */
int ruai_model_get_linear(ruai_model* m, uint64_t tensor_id, int8_t* q_host, float* scale_host);

/* `forward_cached` (llama.rs:434-463, gpt2.rs:214-241): logits for the new
 * tokens `ids_host` [B,T] after the cached positions; the cache is extended.
 * logits_host_or_null receives [B,V] (last position) or, with all_positions,
 * [B,T,V].  The batch size is fixed by the first call after a cache reset.  */
int ruai_model_forward_cached(ruai_model* m, const int32_t* ids_host, uint32_t B, uint32_t T,
                              float* logits_host_or_null, int all_positions);
/* `KvCache::clear` (transformer.rs:160-165) and `KvCache::len`. */
int ruai_model_cache_clear(ruai_model* m);
int ruai_model_cache_len(const ruai_model* m, uint32_t* len, uint32_t* capacity);

/* `generate` with `Sampler::greedy()` (generation.rs:83-113, llama.rs:467-477):
 * batch 1, argmax with the last-maximum tie rule, sliding window past the
 * maximum context.  out_ids_host receives T + n_new ids (prompt first).     */
int ruai_model_generate(ruai_model* m, const int32_t* prompt_host, uint32_t T, uint32_t n_new,
                        int32_t* out_ids_host);

/* `generate` with `Sampler::new(temperature, top_k, top_p, seed)` (generation.rs:28-73, 83-113): as above, but the
 * next token is drawn on the device from the step's logits (temperature <= 0: greedy; top_k 0 = no limit; top_p 1 =
 * off).  Equal logits are ordered by ascending index (the reference's unstable sort leaves this open).  One GPU. */
int ruai_model_generate_sampled(ruai_model* m, const int32_t* prompt_host, uint32_t T, uint32_t n_new,
                                float temperature, uint32_t top_k, float top_p, uint64_t seed, int32_t* out_ids_host);
/* `Sampler::sample` on one row of f32 logits in device memory; *rng_state is the sampler's SplitMix64 state
 * (rand.rs:29-41), advanced by one draw when temperature > 0. */
int ruai_sample(ruai_ctx* ctx, const float* logits_dev, uint32_t vocab, float temperature, uint32_t top_k, float top_p,
                uint64_t* rng_state, int32_t* token_host);

/* One decode step that never leaves the device: the ids are read from
 * ids_dev_or_null [B] (NULL: the argmax of the previous step), the argmax of
 * the new logits is left on the device and, if next_ids_host_or_null is given,
 * copied out.  Batched greedy decode for B independent sequences.           */
int ruai_model_decode_step(ruai_model* m, const int32_t* ids_dev_or_null, uint32_t B,
                           int32_t* next_ids_host_or_null);
/* Grow the cache now to hold `positions` per sequence for batch B (same growth rule), so that
 * later steps neither reallocate nor re-capture the decode graph. */
int ruai_model_cache_reserve(ruai_model* m, uint32_t B, uint32_t positions);
/* Pretend `len` positions are cached for batch B (contents: whatever the
 * buffers hold, zero-filled when fresh); used to time decode at a given
 * context length without running the prompt. */
int ruai_model_cache_assume(ruai_model* m, uint32_t B, uint32_t len);
/* Algorithmic bytes of one decode step at batch B with `len` cached positions:
 * packed weights + scales + head + norm/bias parameters + B * (embedding row +
 * KV read + KV write). */
int ruai_model_step_bytes(const ruai_model* m, uint32_t B, uint32_t len, double* bytes);
/* Kernels launched by one decode step (for launch accounting). */
int ruai_model_step_launches(const ruai_model* m, uint32_t* launches);
/* Times `iters` passes over every quantized Linear of the model for B rows (the
 * weight-streaming kernels of a decode step and nothing else) with CUDA events on
 * the context stream.  Reports the elapsed milliseconds, the launches of one pass
 * and the algorithmic bytes of one pass (packed weights + scales + biases +
 * activations read and written). */
int ruai_model_time_linears(ruai_model* m, uint32_t B, uint32_t iters, float* ms_total,
                            uint32_t* launches_per_pass, double* bytes_per_pass);

/* ---- tensor parallel -------------------------------------------------------
 * The exchange buffers of every rank are mapped into every other rank through
 * CUDA IPC handles that the caller carries between processes (any transport:
 * torch.distributed object gather, a file, MPI).                            */
#define RUAI_IPC_HANDLE_BYTES 64
int ruai_tp_export(ruai_model* m, void* handle_out /* RUAI_IPC_HANDLE_BYTES */);
int ruai_tp_connect(ruai_model* m, const void* handles /* world * RUAI_IPC_HANDLE_BYTES */);
/* After a step that failed with RUAI_ERR_TIMEOUT on any rank (a peer did not take part): once every rank has
 * stopped stepping (the caller synchronises the ranks), each calls this to clear its side of the exchange; after a
 * second synchronisation of the ranks, and a cache clear, stepping can resume.                                   */
int ruai_tp_resync(ruai_model* m);

#ifdef __cplusplus
}
#endif
#endif /* RUAI_B200_H */
