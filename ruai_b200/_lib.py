"""ctypes binding of libruai_b200.so (the C ABI of include/ruai_b200.h).

The shared library is the product; this module only declares its prototypes.
There is no fallback: if the library is missing it is built with nvcc, and if a
call fails a RuaiError carrying ruai_last_error() is raised — the same place
where the reference panics (cuda.rs:256, ops.rs:694-699).
"""
import ctypes as C
import os

from . import _build

u32, u64, i32 = C.c_uint32, C.c_uint64, C.c_int32
vp = C.c_void_p

OK, ERR_SHAPE, ERR_CUDA, ERR_COMM, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_ARG = range(7)
F32, F16, BF16 = 0, 1, 2
IPC_HANDLE_BYTES = 64


class RuaiError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"ruai_b200 error {code}: {msg}")
        self.code = code


class LlamaConfig(C.Structure):
    """`ruai_llama_config`: the fields of `LlamaConfig` (llama.rs:48-75) the path uses."""
    _fields_ = [("vocab_size", u32), ("hidden_size", u32), ("intermediate_size", u32),
                ("num_hidden_layers", u32), ("num_attention_heads", u32), ("num_key_value_heads", u32),
                ("head_dim", u32), ("max_position_embeddings", u32), ("rms_norm_eps", C.c_float),
                ("rope_theta", C.c_float), ("tie_word_embeddings", u32)]


class GPT2Config(C.Structure):
    """`ruai_gpt2_config`: `GPT2Config` (gpt2.rs:30-44)."""
    _fields_ = [("vocab_size", u32), ("n_positions", u32), ("n_embd", u32), ("n_layer", u32), ("n_head", u32)]


class TP(C.Structure):
    _fields_ = [("rank", u32), ("world", u32)]


_PROTOS = {
    "ruai_ctx_create": (C.c_int, [C.c_int, vp, C.POINTER(vp)]),
    "ruai_ctx_destroy": (C.c_int, [vp]),
    "ruai_last_error": (C.c_char_p, [vp]),
    "ruai_ctx_synchronize": (C.c_int, [vp]),
    "ruai_device_count": (C.c_int, []),
    "ruai_version": (C.c_char_p, []),
    "ruai_malloc": (C.c_int, [vp, C.c_size_t, C.POINTER(vp)]),
    "ruai_free": (C.c_int, [vp, vp]),
    "ruai_memcpy_h2d": (C.c_int, [vp, vp, vp, C.c_size_t]),
    "ruai_memcpy_d2h": (C.c_int, [vp, vp, vp, C.c_size_t]),
    "ruai_timer_start": (C.c_int, [vp]),
    "ruai_timer_stop_ms": (C.c_int, [vp, C.POINTER(C.c_float)]),
    "ruai_quantize_int8": (C.c_int, [vp, vp, u32, u32, vp, vp]),
    "ruai_quantize_int4": (C.c_int, [vp, vp, u32, u32, u32, vp, vp]),
    "ruai_repack_int8": (C.c_int, [vp, vp, vp, u32, u32, C.POINTER(vp)]),
    "ruai_repack_int4": (C.c_int, [vp, vp, vp, u32, u32, u32, C.POINTER(vp)]),
    "ruai_unpack": (C.c_int, [vp, vp, vp, vp]),
    "ruai_qweight_free": (C.c_int, [vp]),
    "ruai_qweight_info": (C.c_int, [vp, C.POINTER(u32), C.POINTER(u32), C.POINTER(u32), C.POINTER(u32)]),
    "ruai_matmul_q": (C.c_int, [vp, C.c_int, vp, vp, vp, vp, u32]),
    "ruai_matmul_q_static": (C.c_int, [vp, C.c_int, vp, vp, vp, vp, u32]),
    "ruai_matmul_q_grad_input": (C.c_int, [vp, vp, vp, vp, u32]),
    "ruai_linear_lora_forward": (C.c_int, [vp, vp, vp, vp, vp, u32, C.c_float, vp, vp, u32]),
    "ruai_sample": (C.c_int, [vp, vp, u32, C.c_float, u32, C.c_float, C.POINTER(u64), C.POINTER(i32)]),
    "ruai_model_generate_sampled": (C.c_int, [vp, vp, u32, u32, C.c_float, u32, C.c_float, u64, vp]),
    "ruai_matmul_q_stream": (C.c_int, [vp, vp, vp, vp, u32, u32]),
    "ruai_ctx_set_wait_limit": (C.c_int, [vp, C.c_uint]),
    "ruai_ctx_inject_barrier_skew": (C.c_int, [vp, C.c_uint]),
    "ruai_ctx_inject_copy_shortfall": (C.c_int, [vp, C.c_uint]),
    "ruai_ctx_force_splits": (C.c_int, [vp, C.c_uint]),
    "ruai_dequant_int4": (C.c_int, [vp, vp, vp]),
    "ruai_dequant_int4_ref": (C.c_int, [vp, vp, vp, u32, u32, u32, vp]),
    "ruai_llama_create": (C.c_int, [vp, C.POINTER(LlamaConfig), C.POINTER(TP), C.POINTER(vp)]),
    "ruai_gpt2_create": (C.c_int, [vp, C.POINTER(GPT2Config), C.POINTER(vp)]),
    "ruai_model_destroy": (C.c_int, [vp]),
    "ruai_model_load_synthetic": (C.c_int, [vp, u64, u32, u32]),
    "ruai_model_set_f32": (C.c_int, [vp, u64, vp, C.c_size_t]),
    "ruai_model_quantize": (C.c_int, [vp, u32, u32]),
    "ruai_model_set_quantized": (C.c_int, [vp, u64, vp, vp, u32, u32]),
    "ruai_model_get_f32": (C.c_int, [vp, u64, vp, C.c_size_t]),
    "ruai_model_use_persistent_step": (C.c_int, [vp, C.c_int]),
    "ruai_model_uses_persistent_step": (C.c_int, [vp, u32]),
    "ruai_model_get_linear": (C.c_int, [vp, u64, vp, vp]),
    "ruai_model_forward_cached": (C.c_int, [vp, vp, u32, u32, vp, C.c_int]),
    "ruai_model_cache_clear": (C.c_int, [vp]),
    "ruai_model_cache_len": (C.c_int, [vp, C.POINTER(u32), C.POINTER(u32)]),
    "ruai_model_generate": (C.c_int, [vp, vp, u32, u32, vp]),
    "ruai_model_decode_step": (C.c_int, [vp, vp, u32, vp]),
    "ruai_model_cache_assume": (C.c_int, [vp, u32, u32]),
    "ruai_model_cache_reserve": (C.c_int, [vp, u32, u32]),
    "ruai_model_step_bytes": (C.c_int, [vp, u32, u32, C.POINTER(C.c_double)]),
    "ruai_model_step_launches": (C.c_int, [vp, C.POINTER(u32)]),
    "ruai_model_time_linears": (C.c_int, [vp, u32, u32, C.POINTER(C.c_float), C.POINTER(u32), C.POINTER(C.c_double)]),
    "ruai_tp_export": (C.c_int, [vp, vp]),
    "ruai_tp_resync": (C.c_int, [vp]),
    "ruai_tp_connect": (C.c_int, [vp, vp]),
}

_lib = None


def symbols():
    """Names of every entry point include/ruai_b200.h declares."""
    return sorted(_PROTOS)


def lib_path():
    return _build.LIB


def load():
    """Load (building first if stale or absent) and return the ctypes library."""
    global _lib
    if _lib is None:
        if _build.needs_build():
            _build.build()
        L = C.CDLL(_build.LIB)
        for name, (res, args) in _PROTOS.items():
            fn = getattr(L, name)  # AttributeError here = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc, ctx=None):
    if rc != OK:
        msg = load().ruai_last_error(ctx)
        raise RuaiError(rc, msg.decode() if msg else "")
