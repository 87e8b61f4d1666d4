"""ctypes front end of the CPU checker (TEST INFRASTRUCTURE, not the product).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs import
this package.  Every function forwards to oracle.cpp, which restates the
reference's CPU path and cites the reference lines it follows.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None

u32, u64, i32 = C.c_uint32, C.c_uint64, C.c_int32
_fp = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(dtype=np.int8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


class LlamaConfig(C.Structure):
    """Mirror of `ruai_llama_config` (include/ruai_b200.h), itself `LlamaConfig` of llama.rs:48-75."""
    _fields_ = [("vocab_size", u32), ("hidden_size", u32), ("intermediate_size", u32),
                ("num_hidden_layers", u32), ("num_attention_heads", u32), ("num_key_value_heads", u32),
                ("head_dim", u32), ("max_position_embeddings", u32), ("rms_norm_eps", C.c_float),
                ("rope_theta", C.c_float), ("tie_word_embeddings", u32)]


class GPT2Config(C.Structure):
    """Mirror of `ruai_gpt2_config`, itself `GPT2Config` of gpt2.rs:30-44."""
    _fields_ = [("vocab_size", u32), ("n_positions", u32), ("n_embd", u32), ("n_layer", u32), ("n_head", u32)]


def lib():
    global _lib
    if _lib is None:
        path = _build.build()
        L = C.CDLL(path)
        L.orc_quantize_int8.argtypes = [_fp, u32, u32, _i8p, _fp]
        L.orc_quantize_int4.argtypes = [_fp, u32, u32, u32, _i8p, _fp]
        L.orc_quantize_int4.restype = C.c_int
        L.orc_dequant_int4.argtypes = [_i8p, _fp, u32, u32, u32, _fp]
        L.orc_matmul_int8.argtypes = [_fp, _i8p, _fp, u32, u32, u32, _fp]
        L.orc_matmul_int4.argtypes = [_fp, _i8p, _fp, u32, u32, u32, u32, _fp]
        L.orc_rms_norm.argtypes = [_fp, C.c_void_p, u32, u32, C.c_float, _fp]
        L.orc_layer_norm.argtypes = [_fp, C.c_void_p, C.c_void_p, u32, u32, C.c_float, _fp]
        L.orc_gelu.argtypes = [_fp, C.c_size_t, _fp]
        L.orc_rope_inv_freq.argtypes = [u32, C.c_float, _fp]
        L.orc_rope_cos_sin.argtypes = [_fp, u32, u32, u32, _fp, _fp]
        L.orc_apply_rope.argtypes = [_fp, _fp, _fp, u32]
        L.orc_attention.argtypes = [_fp, _fp, _fp, u32, u32, u32, u32, C.c_int, _fp]
        L.orc_argmax.argtypes = [_fp, u32]
        L.orc_argmax.restype = u32
        L.orc_synth_normal.argtypes = [u64, u64, C.c_size_t, C.c_double, _fp]
        L.orc_synth_tokens.argtypes = [u64, u64, C.c_size_t, u32, _i32p]
        L.orc_llama_create.argtypes = [C.POINTER(LlamaConfig), u64, u32, u32]
        L.orc_llama_create.restype = C.c_void_p
        L.orc_gpt2_create.argtypes = [C.POINTER(GPT2Config), u64, u32, u32]
        L.orc_gpt2_create.restype = C.c_void_p
        L.orc_model_destroy.argtypes = [C.c_void_p]
        L.orc_threads.restype = C.c_int
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_model_cache_assume.argtypes = [C.c_void_p, u32, u32]
        L.orc_model_cache_assume.restype = C.c_int
        L.orc_model_cache_clear.argtypes = [C.c_void_p]
        L.orc_model_cache_len.argtypes = [C.c_void_p]
        L.orc_model_cache_len.restype = u32
        L.orc_model_cache_capacity.argtypes = [C.c_void_p]
        L.orc_model_cache_capacity.restype = u32
        L.orc_model_forward_cached.argtypes = [C.c_void_p, _i32p, u32, u32, C.c_void_p, C.c_int]
        L.orc_model_forward_cached.restype = C.c_int
        L.orc_model_get_linear.argtypes = [C.c_void_p, u64, C.c_void_p, C.c_void_p, C.POINTER(u32), C.POINTER(u32)]
        L.orc_model_get_linear.restype = C.c_int
        L.orc_model_generate.argtypes = [C.c_void_p, _i32p, u32, u32, _i32p, C.c_void_p]
        L.orc_model_generate.restype = C.c_int
        _lib = L
    return _lib


def threads():
    """Threads the checker's OpenMP loops run on."""
    return int(lib().orc_threads())


def set_threads(n):
    lib().orc_set_threads(int(n))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def quantize_int8(w):
    """`Linear::quantize_int8` (layers.rs:112-129): returns (q [k,n] int8, scale [n] f32)."""
    w = _f32(w)
    k, n = w.shape
    q, s = np.empty((k, n), np.int8), np.empty(n, np.float32)
    lib().orc_quantize_int8(w, k, n, q, s)
    return q, s


def quantize_int4(w, group):
    """`Linear::quantize_int4` (layers.rs:139-165): returns (packed [k/2,n] int8, scale [k/group,n])."""
    w = _f32(w)
    k, n = w.shape
    if not (group >= 2 and group % 2 == 0 and k % group == 0):
        raise ValueError(f"int4 group {group} must be even and divide in_features {k}")
    q, s = np.empty((k // 2, n), np.int8), np.empty((k // group, n), np.float32)
    rc = lib().orc_quantize_int4(w, k, n, group, q, s)
    assert rc == 0
    return q, s


def dequant_int4(q, scale, group):
    """`Backend::dequant_int4` (cpu.rs:1023-1033): f32 [k,n]."""
    q = np.ascontiguousarray(q, np.int8)
    scale = _f32(scale)
    k, n = 2 * q.shape[0], q.shape[1]
    w = np.empty((k, n), np.float32)
    lib().orc_dequant_int4(q, scale, k, n, group, w)
    return w


def matmul_int8(x, q, scale):
    """`Backend::matmul_int8` on the CPU (cpu.rs:897-927); x [m,k] f32."""
    x, q, scale = _f32(x), np.ascontiguousarray(q, np.int8), _f32(scale)
    m, k = x.shape
    n = q.shape[1]
    assert q.shape[0] == k and scale.shape == (n,)
    out = np.empty((m, n), np.float32)
    lib().orc_matmul_int8(x, q, scale, m, k, n, out)
    return out


def matmul_int4(x, q, scale):
    """`Backend::matmul_int4` on the CPU (cpu.rs:1035-1067); group = k / scale rows (ops.rs:724)."""
    x, q, scale = _f32(x), np.ascontiguousarray(q, np.int8), _f32(scale)
    m, k = x.shape
    n = q.shape[1]
    assert 2 * q.shape[0] == k and scale.shape[1] == n
    group = k // scale.shape[0]
    assert group * scale.shape[0] == k
    out = np.empty((m, n), np.float32)
    lib().orc_matmul_int4(x, q, scale, m, k, n, group, out)
    return out


def dequant(bits, q, scale, group=32):
    """The f32 weight the reference's backward materialises: q * scales (ops.rs:707) or dequant_int4 (ops.rs:732)."""
    if bits == 8:
        return np.ascontiguousarray(q, np.int8).astype(np.float32) * _f32(scale)[None, :]
    return dequant_int4(q, scale, group)


def matmul_q_grad_input(bits, g, q, scale, group=32):
    """Backward of matmul_int8 / matmul_int4 (ops.rs:705-709, 731-734): dx = g @ dequant(W)^T, f32."""
    return (_f32(g) @ dequant(bits, q, scale, group).T).astype(np.float32)


def linear_lora_forward(bits, x, q, scale, lora_a, lora_b, lora_scale, bias=None):
    """Linear::forward with an adapter (layers.rs:169-190): quantized base, + (x @ A @ B) * scale, + bias, in that order."""
    x = _f32(x)
    y = matmul_int8(x, q, scale) if bits == 8 else matmul_int4(x, q, scale)
    y = y + ((x @ _f32(lora_a)) @ _f32(lora_b)) * np.float32(lora_scale)
    if bias is not None:
        y = y + _f32(bias)
    return y.astype(np.float32)


def rms_norm(x, w, eps):
    x = _f32(x)
    y = np.empty_like(x)
    wp = None if w is None else _f32(w).ctypes.data_as(C.c_void_p)
    lib().orc_rms_norm(x.reshape(-1, x.shape[-1]), wp, x.size // x.shape[-1], x.shape[-1], eps, y.reshape(-1, x.shape[-1]))
    return y


def layer_norm(x, w, b, eps=1e-5):
    x = _f32(x)
    y = np.empty_like(x)
    w_, b_ = (None if w is None else _f32(w)), (None if b is None else _f32(b))
    lib().orc_layer_norm(x.reshape(-1, x.shape[-1]), None if w_ is None else w_.ctypes.data_as(C.c_void_p),
                         None if b_ is None else b_.ctypes.data_as(C.c_void_p), x.size // x.shape[-1], x.shape[-1], eps,
                         y.reshape(-1, x.shape[-1]))
    return y


def gelu(x):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_gelu(x.ravel(), x.size, y.ravel())
    return y


def rope_inv_freq(head_dim, theta):
    inv = np.empty(head_dim // 2, np.float32)
    lib().orc_rope_inv_freq(head_dim, theta, inv)
    return inv


def rope_cos_sin(inv, start, t):
    half = inv.shape[0]
    c, s = np.empty((t, 2 * half), np.float32), np.empty((t, 2 * half), np.float32)
    lib().orc_rope_cos_sin(_f32(inv), half, start, t, c, s)
    return c, s


def apply_rope(x, cos, sin):
    """x [T, d] with tables [T, d]."""
    x = _f32(x).copy()
    for t in range(x.shape[0]):
        lib().orc_apply_rope(x[t], _f32(cos[t]), _f32(sin[t]), x.shape[1])
    return x


def attention(q, k, v, past=0, use_mask=False):
    """One head: q [tq,d], k/v [tk,d]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    o = np.empty_like(q)
    lib().orc_attention(q, k, v, q.shape[0], k.shape[0], q.shape[1], past, int(use_mask), o)
    return o


def argmax(logits):
    """`generation::argmax` (generation.rs:6-8): last index among equal maxima."""
    logits = _f32(logits)
    return int(lib().orc_argmax(logits, logits.size))


class Sampler:
    """`Sampler` (generation.rs:15-73); equal logits ordered by ascending index."""

    def __init__(self, temperature, top_k=0, top_p=1.0, seed=0):
        self.temperature, self.top_k, self.top_p = float(temperature), int(top_k), float(top_p)
        self.state = C.c_uint64(seed)
        self.margin = 1.0

    def sample(self, logits):
        logits = _f32(logits)
        mg = C.c_float(1.0)
        L = lib()
        L.orc_sample.restype = u32
        L.orc_sample.argtypes = [_fp, u32, C.c_float, u32, C.c_float, C.POINTER(C.c_uint64), C.POINTER(C.c_float)]
        tok = L.orc_sample(logits, logits.size, self.temperature, self.top_k, self.top_p, C.byref(self.state), C.byref(mg))
        self.margin = float(mg.value)
        return int(tok)


def synth_normal(seed, tensor_id, shape, std=0.02):
    out = np.empty(int(np.prod(shape)), np.float32)
    lib().orc_synth_normal(seed, tensor_id, out.size, std, out)
    return out.reshape(shape)


def synth_tokens(seed, tensor_id, count, vocab):
    out = np.empty(count, np.int32)
    lib().orc_synth_tokens(seed, tensor_id, count, vocab, out)
    return out


class Model:
    """A Llama or GPT-2 over the seeded synthetic weights, quantized like the reference."""

    def __init__(self, cfg, seed=0, bits=8, group=32):
        self.cfg = cfg
        if isinstance(cfg, LlamaConfig):
            self.h = lib().orc_llama_create(C.byref(cfg), seed, bits, group)
        else:
            self.h = lib().orc_gpt2_create(C.byref(cfg), seed, bits, group)
        self.vocab = cfg.vocab_size

    def close(self):
        if self.h:
            lib().orc_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def cache_clear(self):
        lib().orc_model_cache_clear(self.h)

    def cache_assume(self, B, length):
        """Zero keys and values for `length` cached positions of batch B (timing aid)."""
        if lib().orc_model_cache_assume(self.h, B, length):
            raise RuntimeError("oracle cache_assume failed")

    def cache_len(self):
        return lib().orc_model_cache_len(self.h)

    def cache_capacity(self):
        return lib().orc_model_cache_capacity(self.h)

    def forward_cached(self, ids, all_positions=False):
        """`forward_cached` (llama.rs:434-463): ids [B,T] -> logits [B,V] or [B,T,V]."""
        ids = np.ascontiguousarray(ids, np.int32)
        B, T = ids.shape
        out = np.empty((B, T, self.vocab) if all_positions else (B, self.vocab), np.float32)
        rc = lib().orc_model_forward_cached(self.h, ids, B, T, out.ctypes.data_as(C.c_void_p), int(all_positions))
        if rc:
            raise RuntimeError(f"oracle forward_cached failed ({rc})")
        return out

    def generate(self, prompt, n, trace=False):
        """Greedy `generate` (generation.rs:83-113): returns ids (and the n logit rows)."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.empty(prompt.size + n, np.int32)
        tr = np.empty((n, self.vocab), np.float32) if trace else None
        rc = lib().orc_model_generate(self.h, prompt, prompt.size, n, out, None if tr is None else tr.ctypes.data_as(C.c_void_p))
        if rc:
            raise RuntimeError(f"oracle generate failed ({rc})")
        return (out, tr) if trace else out

    def generate_sampled(self, prompt, n, temperature, top_k=0, top_p=1.0, seed=0):
        """`generate` with `Sampler::new(...)`: returns (ids, margins [n]) (see orc_sample for the margin)."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.empty(prompt.size + n, np.int32)
        mg = np.empty(n, np.float32)
        L = lib()
        L.orc_model_generate_sampled.restype = C.c_int
        L.orc_model_generate_sampled.argtypes = [C.c_void_p, _i32p, u32, u32, C.c_float, u32, C.c_float, C.c_uint64, _i32p, _fp]
        rc = L.orc_model_generate_sampled(self.h, prompt, prompt.size, n, float(temperature), int(top_k), float(top_p), int(seed), out, mg)
        if rc:
            raise RuntimeError(f"oracle generate_sampled failed ({rc})")
        return out, mg

    def get_linear(self, tensor_id, bits, group=32):
        """(q, scale) of one Linear in the reference's buffer layout; tensor ids as in ruai_b200_synth.h."""
        k, n = u32(), u32()
        rc = lib().orc_model_get_linear(self.h, tensor_id, None, None, C.byref(k), C.byref(n))
        if rc:
            raise KeyError(tensor_id)
        k, n = k.value, n.value
        q = np.empty((k if bits == 8 else k // 2, n), np.int8)
        s = np.empty((n,) if bits == 8 else (k // group, n), np.float32)
        lib().orc_model_get_linear(self.h, tensor_id, q.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p), None, None)
        return q, s
