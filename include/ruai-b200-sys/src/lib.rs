//! Raw bindings to `libruai_b200.so`, one declaration per entry point of `include/ruai_b200.h`.
//!
//! Every function returns an `i32` status (`RUAI_OK == 0`); on failure `ruai_last_error(ctx)`
//! holds the message.  The reference panics where these fail (src/nn/backend/cuda.rs:256,
//! src/nn/ops.rs:694-699), so the safe wrappers in the patch next to this crate turn a non-zero
//! status into `panic!("{}", last_error)`.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_int, c_uint, c_void};

pub mod backend;

#[repr(C)]
pub struct ruai_ctx {
    _private: [u8; 0],
}
#[repr(C)]
pub struct ruai_qweight {
    _private: [u8; 0],
}
#[repr(C)]
pub struct ruai_model {
    _private: [u8; 0],
}

pub const RUAI_OK: c_int = 0;
pub const RUAI_ERR_SHAPE: c_int = 1;
pub const RUAI_ERR_CUDA: c_int = 2;
pub const RUAI_ERR_COMM: c_int = 3;
pub const RUAI_ERR_TIMEOUT: c_int = 4;
pub const RUAI_ERR_UNSUPPORTED: c_int = 5;
pub const RUAI_ERR_ARG: c_int = 6;

/// `DType::{F32, F16, BF16}` (src/nn/backend/mod.rs:32-44).
pub const RUAI_F32: c_int = 0;
pub const RUAI_F16: c_int = 1;
pub const RUAI_BF16: c_int = 2;

pub const RUAI_IPC_HANDLE_BYTES: usize = 64;

/// `LlamaConfig` (src/nn/modules/llama.rs:48-75), the fields the path uses.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct ruai_llama_config {
    pub vocab_size: u32,
    pub hidden_size: u32,
    pub intermediate_size: u32,
    pub num_hidden_layers: u32,
    pub num_attention_heads: u32,
    pub num_key_value_heads: u32,
    pub head_dim: u32,
    pub max_position_embeddings: u32,
    pub rms_norm_eps: f32,
    pub rope_theta: f32,
    pub tie_word_embeddings: u32,
}

/// `GPT2Config` (src/nn/modules/gpt2.rs:30-44).
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct ruai_gpt2_config {
    pub vocab_size: u32,
    pub n_positions: u32,
    pub n_embd: u32,
    pub n_layer: u32,
    pub n_head: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct ruai_tp {
    pub rank: u32,
    pub world: u32,
}

extern "C" {
    // ---- context ----
    pub fn ruai_ctx_create(ordinal: c_int, stream_or_null: *mut c_void, out: *mut *mut ruai_ctx) -> c_int;
    pub fn ruai_ctx_destroy(ctx: *mut ruai_ctx) -> c_int;
    pub fn ruai_last_error(ctx: *const ruai_ctx) -> *const c_char;
    pub fn ruai_ctx_synchronize(ctx: *mut ruai_ctx) -> c_int;
    pub fn ruai_device_count() -> c_int;
    pub fn ruai_version() -> *const c_char;
    pub fn ruai_ctx_set_wait_limit(ctx: *mut ruai_ctx, polls: c_uint) -> c_int;
    pub fn ruai_ctx_inject_barrier_skew(ctx: *mut ruai_ctx, grids: c_uint) -> c_int;
    pub fn ruai_ctx_inject_copy_shortfall(ctx: *mut ruai_ctx, bytes: c_uint) -> c_int;
    pub fn ruai_ctx_force_splits(ctx: *mut ruai_ctx, splits: c_uint) -> c_int;
    pub fn ruai_malloc(ctx: *mut ruai_ctx, bytes: usize, out_dev: *mut *mut c_void) -> c_int;
    pub fn ruai_free(ctx: *mut ruai_ctx, ptr_dev: *mut c_void) -> c_int;
    pub fn ruai_memcpy_h2d(ctx: *mut ruai_ctx, dst_dev: *mut c_void, src_host: *const c_void, bytes: usize) -> c_int;
    pub fn ruai_memcpy_d2h(ctx: *mut ruai_ctx, dst_host: *mut c_void, src_dev: *const c_void, bytes: usize) -> c_int;
    pub fn ruai_timer_start(ctx: *mut ruai_ctx) -> c_int;
    pub fn ruai_timer_stop_ms(ctx: *mut ruai_ctx, ms_out: *mut f32) -> c_int;

    // ---- quantizer: Linear::quantize_int8 / quantize_int4 (layers.rs:112-165) ----
    pub fn ruai_quantize_int8(ctx: *mut ruai_ctx, w_dev: *const f32, k: u32, n: u32, q_dev: *mut i8, scale_dev: *mut f32) -> c_int;
    pub fn ruai_quantize_int4(ctx: *mut ruai_ctx, w_dev: *const f32, k: u32, n: u32, group: u32, q_dev: *mut i8, scale_dev: *mut f32) -> c_int;

    // ---- repack ----
    pub fn ruai_repack_int8(ctx: *mut ruai_ctx, q: *const i8, scale: *const f32, k: u32, n: u32, out: *mut *mut ruai_qweight) -> c_int;
    pub fn ruai_repack_int4(ctx: *mut ruai_ctx, q: *const i8, scale: *const f32, k: u32, n: u32, group: u32, out: *mut *mut ruai_qweight) -> c_int;
    pub fn ruai_unpack(ctx: *mut ruai_ctx, w: *const ruai_qweight, q_out: *mut i8, scale_out: *mut f32) -> c_int;
    pub fn ruai_qweight_free(w: *mut ruai_qweight) -> c_int;
    pub fn ruai_qweight_info(w: *const ruai_qweight, k: *mut u32, n: *mut u32, bits: *mut u32, group: *mut u32) -> c_int;

    // ---- Backend::matmul_int8 / dequant_int4 / matmul_int4 (backend/mod.rs:675-704) ----
    pub fn ruai_matmul_q(ctx: *mut ruai_ctx, x_dtype: c_int, x_dev: *const c_void, w: *const ruai_qweight, bias_dev_or_null: *const f32, out_dev: *mut c_void, m: u32) -> c_int;
    pub fn ruai_matmul_q_static(ctx: *mut ruai_ctx, x_dtype: c_int, x_dev: *const c_void, w: *const ruai_qweight, bias_dev_or_null: *const f32, out_dev: *mut c_void, m: u32) -> c_int;
    pub fn ruai_matmul_q_grad_input(ctx: *mut ruai_ctx, g_dev: *const f32, w: *const ruai_qweight, dx_dev: *mut f32, m: u32) -> c_int;
    pub fn ruai_linear_lora_forward(ctx: *mut ruai_ctx, x_dev: *const f32, w: *const ruai_qweight, lora_a_dev: *const f32, lora_b_dev: *const f32, rank: u32, scale: f32, bias_dev_or_null: *const f32, out_dev: *mut f32, m: u32) -> c_int;
    pub fn ruai_sample(ctx: *mut ruai_ctx, logits_dev: *const f32, vocab: u32, temperature: f32, top_k: u32, top_p: f32, rng_state: *mut u64, token_host: *mut i32) -> c_int;
    pub fn ruai_model_generate_sampled(m: *mut ruai_model, prompt_host: *const i32, T: u32, n_new: u32, temperature: f32, top_k: u32, top_p: f32, seed: u64, out_ids_host: *mut i32) -> c_int;
    pub fn ruai_matmul_q_stream(ctx: *mut ruai_ctx, x_dev: *const f32, w: *const ruai_qweight, out_dev: *mut f32, m: u32, repeat: u32) -> c_int;
    pub fn ruai_dequant_int4(ctx: *mut ruai_ctx, w: *const ruai_qweight, out_dev: *mut f32) -> c_int;
    pub fn ruai_dequant_int4_ref(ctx: *mut ruai_ctx, q_dev: *const i8, scale_dev: *const f32, k: u32, n: u32, group: u32, out_dev: *mut f32) -> c_int;

    // ---- models ----
    pub fn ruai_llama_create(ctx: *mut ruai_ctx, cfg: *const ruai_llama_config, tp_or_null: *const ruai_tp, out: *mut *mut ruai_model) -> c_int;
    pub fn ruai_gpt2_create(ctx: *mut ruai_ctx, cfg: *const ruai_gpt2_config, out: *mut *mut ruai_model) -> c_int;
    pub fn ruai_model_destroy(m: *mut ruai_model) -> c_int;
    pub fn ruai_model_load_synthetic(m: *mut ruai_model, seed: u64, bits: u32, group: u32) -> c_int;
    pub fn ruai_model_set_f32(m: *mut ruai_model, tensor_id: u64, data_host: *const f32, count: usize) -> c_int;
    pub fn ruai_model_set_quantized(m: *mut ruai_model, tensor_id: u64, q_host: *const i8, scale_host: *const f32, bits: u32, group: u32) -> c_int;
    pub fn ruai_model_get_f32(m: *mut ruai_model, tensor_id: u64, out_host: *mut f32, count: usize) -> c_int;
    pub fn ruai_model_use_persistent_step(m: *mut ruai_model, on: c_int) -> c_int;
    pub fn ruai_model_uses_persistent_step(m: *mut ruai_model, B: u32) -> c_int;
    pub fn ruai_model_quantize(m: *mut ruai_model, bits: u32, group: u32) -> c_int;
    pub fn ruai_model_get_linear(m: *mut ruai_model, tensor_id: u64, q_host: *mut i8, scale_host: *mut f32) -> c_int;
    pub fn ruai_model_forward_cached(m: *mut ruai_model, ids_host: *const i32, b: u32, t: u32, logits_host_or_null: *mut f32, all_positions: c_int) -> c_int;
    pub fn ruai_model_cache_clear(m: *mut ruai_model) -> c_int;
    pub fn ruai_model_cache_len(m: *const ruai_model, len: *mut u32, capacity: *mut u32) -> c_int;
    pub fn ruai_model_generate(m: *mut ruai_model, prompt_host: *const i32, t: u32, n_new: u32, out_ids_host: *mut i32) -> c_int;
    pub fn ruai_model_decode_step(m: *mut ruai_model, ids_dev_or_null: *const i32, b: u32, next_ids_host_or_null: *mut i32) -> c_int;
    pub fn ruai_model_cache_reserve(m: *mut ruai_model, b: u32, positions: u32) -> c_int;
    pub fn ruai_model_cache_assume(m: *mut ruai_model, b: u32, len: u32) -> c_int;
    pub fn ruai_model_step_bytes(m: *const ruai_model, b: u32, len: u32, bytes: *mut f64) -> c_int;
    pub fn ruai_model_step_launches(m: *const ruai_model, launches: *mut u32) -> c_int;
    pub fn ruai_model_time_linears(m: *mut ruai_model, b: u32, iters: u32, ms_total: *mut f32, launches_per_pass: *mut u32, bytes_per_pass: *mut f64) -> c_int;

    // ---- tensor parallel ----
    pub fn ruai_tp_export(m: *mut ruai_model, handle_out: *mut c_void) -> c_int;
    pub fn ruai_tp_resync(m: *mut ruai_model) -> c_int;
    pub fn ruai_tp_connect(m: *mut ruai_model, handles: *const c_void) -> c_int;
}
