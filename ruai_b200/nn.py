"""Host-side mirror of the `ruai::nn` surface the quantized path goes through.

Same names, argument meaning and error behaviour as the reference:
`Device::Cuda(i)` (device.rs), `Tensor` as an immutable device buffer
(tensor.rs), `Linear::quantize_int8 / quantize_int4 / forward / dims /
state_dict` (layers.rs:24-212), `Tensor::matmul_int8 / matmul_int4`
(ops.rs:689-735) and the `Llama` / `GPT2` inference methods (llama.rs,
gpt2.rs).  Every computation is a call into libruai_b200.so through its C ABI;
nothing here computes on the host.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import F32, F16, BF16, GPT2Config, LlamaConfig, RuaiError, TP  # noqa: F401

_NP_OF = {F32: np.float32, F16: np.float16, BF16: np.uint16}  # bf16 travels as raw 16-bit words


class Device:
    """`Device::Cuda(ordinal)`; owns one library context (stream + scratch) like cuda.rs:82-86."""
    _by_ordinal = {}

    def __init__(self, ordinal=0):
        self.ordinal = ordinal
        self.L = _lib.load()
        h = C.c_void_p()
        _lib.check(self.L.ruai_ctx_create(ordinal, None, C.byref(h)))
        self.ctx = h

    @classmethod
    def cuda(cls, ordinal=0):
        if ordinal not in cls._by_ordinal:
            cls._by_ordinal[ordinal] = cls(ordinal)
        return cls._by_ordinal[ordinal]

    @staticmethod
    def is_available():
        """`Device::is_available` (cuda.rs:73-79)."""
        return _lib.load().ruai_device_count() > 0

    def check(self, rc):
        _lib.check(rc, self.ctx)

    def synchronize(self):
        self.check(self.L.ruai_ctx_synchronize(self.ctx))

    def set_wait_limit(self, polls):
        self.check(self.L.ruai_ctx_set_wait_limit(self.ctx, polls))

    def inject_barrier_skew(self, grids):
        self.check(self.L.ruai_ctx_inject_barrier_skew(self.ctx, grids))

    def inject_copy_shortfall(self, nbytes):
        self.check(self.L.ruai_ctx_inject_copy_shortfall(self.ctx, nbytes))

    def force_splits(self, splits):
        """Fix the split-k count of the tensor-core GEMVs (1..8), or 0 to let the library choose."""
        self.check(self.L.ruai_ctx_force_splits(self.ctx, splits))

    def timer_start(self):
        self.check(self.L.ruai_timer_start(self.ctx))

    def timer_stop_ms(self):
        ms = C.c_float()
        self.check(self.L.ruai_timer_stop_ms(self.ctx, C.byref(ms)))
        return ms.value


class Tensor:
    """A contiguous row-major device buffer with a shape and a dtype (F32 / F16 / BF16 / int8 / int32)."""

    def __init__(self, dev, shape, np_dtype, rdtype=None):
        self.dev, self.shape, self.np_dtype, self.rdtype = dev, tuple(int(s) for s in shape), np.dtype(np_dtype), rdtype
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.np_dtype.itemsize
        p = C.c_void_p()
        dev.check(dev.L.ruai_malloc(dev.ctx, self.nbytes, C.byref(p)))
        self.ptr = p

    @classmethod
    def from_numpy(cls, dev, a, rdtype=None):
        a = np.ascontiguousarray(a)
        if rdtype is None and a.dtype == np.float32:
            rdtype = F32
        if rdtype is None and a.dtype == np.float16:
            rdtype = F16
        t = cls(dev, a.shape, a.dtype, rdtype)
        if t.nbytes:
            dev.check(dev.L.ruai_memcpy_h2d(dev.ctx, t.ptr, a.ctypes.data_as(C.c_void_p), t.nbytes))
        return t

    def numpy(self):
        a = np.empty(self.shape, self.np_dtype)
        if self.nbytes:
            self.dev.check(self.dev.L.ruai_memcpy_d2h(self.dev.ctx, a.ctypes.data_as(C.c_void_p), self.ptr, self.nbytes))
        return a

    def free(self):
        if self.ptr:
            self.dev.L.ruai_free(self.dev.ctx, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    # ops.rs:693-710
    def matmul_int8(self, q, scales):
        return _matmul_q(self, QWeight.int8(self.dev, q, scales))

    # ops.rs:716-735
    def matmul_int4(self, q, scales):
        k = 2 * q.shape[0]
        if scales.ndim != 2 or q.ndim != 2:
            raise ValueError("matmul_int4: q must be [k/2, n] and scales [k/group, n]")
        if scales.shape[0] == 0 or k % scales.shape[0]:
            raise ValueError(f"matmul_int4: {scales.shape[0]} scale rows do not divide k = {k}")
        return _matmul_q(self, QWeight.int4(self.dev, q, scales, k // scales.shape[0]))


class QWeight:
    """A repacked quantized weight (`ruai_qweight`), built once from the reference-layout buffers."""

    def __init__(self, dev, handle, k, n, bits, group):
        self.dev, self.h, self.k, self.n, self.bits, self.group = dev, handle, k, n, bits, group

    @classmethod
    def int8(cls, dev, q, scale):
        q, scale = np.ascontiguousarray(q, np.int8), np.ascontiguousarray(scale, np.float32)
        if q.ndim != 2:
            raise ValueError("matmul_int8: weights must be [k, n]")
        k, n = q.shape
        if scale.shape != (n,):
            raise ValueError("matmul_int8: scales must be [n]")
        h = C.c_void_p()
        dev.check(dev.L.ruai_repack_int8(dev.ctx, q.ctypes.data_as(C.c_void_p), scale.ctypes.data_as(C.c_void_p), k, n, C.byref(h)))
        return cls(dev, h, k, n, 8, 0)

    @classmethod
    def int4(cls, dev, q, scale, group):
        q, scale = np.ascontiguousarray(q, np.int8), np.ascontiguousarray(scale, np.float32)
        k, n = 2 * q.shape[0], q.shape[1]
        if scale.shape[1] != n:
            raise ValueError(f"matmul_int4: scales must have {n} columns")
        h = C.c_void_p()
        dev.check(dev.L.ruai_repack_int4(dev.ctx, q.ctypes.data_as(C.c_void_p), scale.ctypes.data_as(C.c_void_p), k, n, group, C.byref(h)))
        return cls(dev, h, k, n, 4, group)

    def unpack(self):
        """The reference-layout buffers back, byte for byte."""
        q = np.empty((self.k if self.bits == 8 else self.k // 2, self.n), np.int8)
        s = np.empty((self.n,) if self.bits == 8 else (self.k // self.group, self.n), np.float32)
        self.dev.check(self.dev.L.ruai_unpack(self.dev.ctx, self.h, q.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p)))
        return q, s

    def dequant(self):
        """`Backend::dequant_int4` (mod.rs:689-693)."""
        out = Tensor(self.dev, (self.k, self.n), np.float32, F32)
        self.dev.check(self.dev.L.ruai_dequant_int4(self.dev.ctx, self.h, out.ptr))
        return out.numpy()

    def free(self):
        if self.h:
            self.dev.L.ruai_qweight_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _matmul_q(x, w, bias=None):
    if x.rdtype not in (F32, F16, BF16):
        raise TypeError("matmul_int8/int4: activations must be a float tensor")
    if x.shape[-1] != w.k:
        raise ValueError(f"inner dims differ ({x.shape} @ int{w.bits} [{w.k}, {w.n}])")
    m = int(np.prod(x.shape[:-1], dtype=np.int64))
    out = Tensor(x.dev, x.shape[:-1] + (w.n,), x.np_dtype, x.rdtype)
    x.dev.check(x.dev.L.ruai_matmul_q(x.dev.ctx, x.rdtype, x.ptr, w.h, bias.ptr if bias is not None else None, out.ptr, m))
    return out


def matmul_q_grad_input(g, w):
    """Gradient of `matmul_int8` / `matmul_int4` with respect to the activations (ops.rs:705-709, 731-734): g @ dequant(W)^T."""
    if g.rdtype != F32 or g.shape[-1] != w.n:
        raise ValueError(f"gradient must be f32 [..., {w.n}]")
    m = int(np.prod(g.shape[:-1], dtype=np.int64))
    out = Tensor(g.dev, g.shape[:-1] + (w.k,), np.float32, F32)
    g.dev.check(g.dev.L.ruai_matmul_q_grad_input(g.dev.ctx, g.ptr, w.h, out.ptr, m))
    return out


def linear_lora_forward(x, w, lora_a, lora_b, scale, bias=None):
    """`Linear::forward` of a quantized layer with a LoRA adapter (layers.rs:169-190)."""
    if x.rdtype != F32 or x.shape[-1] != w.k:
        raise ValueError(f"activations must be f32 [..., {w.k}]")
    rank = lora_a.shape[1]
    if lora_a.shape != (w.k, rank) or lora_b.shape != (rank, w.n):
        raise ValueError("lora_a must be [k, rank] and lora_b [rank, n]")
    m = int(np.prod(x.shape[:-1], dtype=np.int64))
    out = Tensor(x.dev, x.shape[:-1] + (w.n,), np.float32, F32)
    x.dev.check(x.dev.L.ruai_linear_lora_forward(x.dev.ctx, x.ptr, w.h, lora_a.ptr, lora_b.ptr, rank, float(scale),
                                                 bias.ptr if bias is not None else None, out.ptr, m))
    return out


class Sampler:
    """`Sampler` (generation.rs:15-73) over logits in device memory."""

    def __init__(self, temperature, top_k=0, top_p=1.0, seed=0):
        self.temperature, self.top_k, self.top_p = float(temperature), int(top_k), float(top_p)
        self.state = C.c_uint64(seed)

    def sample(self, logits):
        if logits.rdtype != F32 or len(logits.shape) != 1:
            raise ValueError("logits must be a 1-D f32 tensor")
        tok = C.c_int32(0)
        logits.dev.check(logits.dev.L.ruai_sample(logits.dev.ctx, logits.ptr, logits.shape[0], self.temperature, self.top_k, self.top_p,
                                                  C.byref(self.state), C.byref(tok)))
        return int(tok.value)


def matmul_q_stream(x, w, repeat=1):
    """`matmul_int8` / `matmul_int4` for 1 or 2 rows through the persistent kernel's data path (f32)."""
    if x.rdtype != F32:
        raise TypeError("matmul_q_stream: activations must be f32")
    if x.shape[-1] != w.k:
        raise ValueError(f"inner dims differ ({x.shape} @ int{w.bits} [{w.k}, {w.n}])")
    m = int(np.prod(x.shape[:-1], dtype=np.int64))
    out = Tensor(x.dev, x.shape[:-1] + (w.n,), np.float32, F32)
    x.dev.check(x.dev.L.ruai_matmul_q_stream(x.dev.ctx, x.ptr, w.h, out.ptr, m, repeat))
    return out


def quantize_int8_device(dev, w):
    """`Linear::quantize_int8`'s loops (layers.rs:112-129) run on the device; returns numpy (q, scale)."""
    w = np.ascontiguousarray(w, np.float32)
    k, n = w.shape
    wt = Tensor.from_numpy(dev, w)
    q, s = Tensor(dev, (k, n), np.int8), Tensor(dev, (n,), np.float32, F32)
    dev.check(dev.L.ruai_quantize_int8(dev.ctx, wt.ptr, k, n, q.ptr, s.ptr))
    return q.numpy(), s.numpy()


def quantize_int4_device(dev, w, group):
    """`Linear::quantize_int4` (layers.rs:139-165) on the device; returns numpy (packed, scale)."""
    w = np.ascontiguousarray(w, np.float32)
    k, n = w.shape
    if not (group >= 2 and group % 2 == 0 and k % group == 0):
        raise ValueError(f"int4 group {group} must be even and divide in_features {k}")
    wt = Tensor.from_numpy(dev, w)
    q, s = Tensor(dev, (k // 2, n), np.int8), Tensor(dev, (k // group, n), np.float32, F32)
    dev.check(dev.L.ruai_quantize_int4(dev.ctx, wt.ptr, k, n, group, q.ptr, s.ptr))
    return q.numpy(), s.numpy()


class Linear:
    """`Linear` (layers.rs:24-212): y = x @ W + b with W [in, out]; inference-only quantized forms."""

    def __init__(self, dev, weight, bias=None):
        self.dev = dev
        self.weight = np.ascontiguousarray(weight, np.float32)
        self.bias = None if bias is None else Tensor.from_numpy(dev, np.ascontiguousarray(bias, np.float32))
        self.int8 = self.int4 = None
        self._q = None

    def is_quantized(self):
        return self._q is not None

    def dims(self):
        return (self._q.k, self._q.n) if self._q else self.weight.shape

    def quantize_int8(self):
        if self.is_quantized():
            return
        q, s = quantize_int8_device(self.dev, self.weight)
        self.int8, self._q = (q, s), QWeight.int8(self.dev, q, s)
        self.weight = np.zeros((0,), np.float32)

    def quantize_int4(self, group):
        if self.is_quantized():
            return
        q, s = quantize_int4_device(self.dev, self.weight, group)
        self.int4, self._q = (q, s), QWeight.int4(self.dev, q, s, group)
        self.weight = np.zeros((0,), np.float32)

    def forward(self, x):
        if not self.is_quantized():
            raise RuaiError(_lib.ERR_UNSUPPORTED, "only the quantized Linear is implemented on this path")
        return _matmul_q(x, self._q, self.bias)

    def state_dict(self):
        """Buffer names of layers.rs:205-211."""
        d = {}
        if self.bias is not None:
            d["bias"] = self.bias.numpy()
        if self.int8:
            d["weight_int8"], d["weight_scale"] = self.int8
        if self.int4:
            d["weight_int4"], d["weight_int4_scale"] = self.int4
        return d


class _Model:
    """Shared inference surface of `Llama` and `GPT2`: quantize, forward_cached, generate."""

    def __init__(self, dev, handle, cfg):
        self.dev, self.h, self.config = dev, handle, cfg
        self.vocab = cfg.vocab_size

    def close(self):
        if self.h:
            self.dev.L.ruai_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_synthetic(self, seed=0, bits=8, group=32):
        """Seeded N(0, 0.02^2) weights generated and quantized on the device (see include/ruai_b200_synth.h)."""
        self.dev.check(self.dev.L.ruai_model_load_synthetic(self.h, seed, bits, group if bits == 4 else 0))

    def set_f32(self, tensor_id, a):
        a = np.ascontiguousarray(a, np.float32)
        self.dev.check(self.dev.L.ruai_model_set_f32(self.h, tensor_id, a.ctypes.data_as(C.c_void_p), a.size))

    def quantize_int8(self):
        """`Llama::quantize_int8` (llama.rs:522-531) / `GPT2::quantize_int8` (gpt2.rs:306-315)."""
        self.dev.check(self.dev.L.ruai_model_quantize(self.h, 8, 0))

    def quantize_int4(self, group):
        """`Llama::quantize_int4(group)` (llama.rs:533-542): block Linears int4, head int8."""
        self.dev.check(self.dev.L.ruai_model_quantize(self.h, 4, group))

    def get_linear(self, tensor_id, k, n, bits, group=32):
        """One quantized Linear in the reference's buffer layout (`weight_int8`/`weight_scale`, ...)."""
        q = np.empty((k if bits == 8 else k // 2, n), np.int8)
        s = np.empty((n,) if bits == 8 else (k // group, n), np.float32)
        self.dev.check(self.dev.L.ruai_model_get_linear(self.h, tensor_id, q.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p)))
        return q, s

    def forward_cached(self, ids, all_positions=False, want_logits=True):
        """`forward_cached` (llama.rs:434-463, gpt2.rs:214-241): ids [B,T] -> logits [B,V] (last) or [B,T,V]."""
        ids = np.ascontiguousarray(ids, np.int32)
        B, T = ids.shape
        out = np.empty((B, T, self.vocab) if all_positions else (B, self.vocab), np.float32) if want_logits else None
        self.dev.check(self.dev.L.ruai_model_forward_cached(self.h, ids.ctypes.data_as(C.c_void_p), B, T,
                                                           out.ctypes.data_as(C.c_void_p) if want_logits else None, int(all_positions)))
        return out

    def cache_clear(self):
        self.dev.check(self.dev.L.ruai_model_cache_clear(self.h))

    def cache_len(self):
        a, b = C.c_uint32(), C.c_uint32()
        self.dev.check(self.dev.L.ruai_model_cache_len(self.h, C.byref(a), C.byref(b)))
        return a.value

    def cache_capacity(self):
        a, b = C.c_uint32(), C.c_uint32()
        self.dev.check(self.dev.L.ruai_model_cache_len(self.h, C.byref(a), C.byref(b)))
        return b.value

    def generate(self, prompt, n):
        """Greedy `generate` (generation.rs:83-113): prompt followed by n new ids."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.empty(prompt.size + n, np.int32)
        self.dev.check(self.dev.L.ruai_model_generate(self.h, prompt.ctypes.data_as(C.c_void_p), prompt.size, n, out.ctypes.data_as(C.c_void_p)))
        return out

    def generate_sampled(self, prompt, n, temperature, top_k=0, top_p=1.0, seed=0):
        """`generate` with `Sampler::new(temperature, top_k, top_p, seed)` (generation.rs:28-73); the draw runs on the device."""
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.empty(prompt.size + n, np.int32)
        self.dev.check(self.dev.L.ruai_model_generate_sampled(self.h, prompt.ctypes.data_as(C.c_void_p), prompt.size, n, float(temperature), int(top_k),
                                                              float(top_p), int(seed), out.ctypes.data_as(C.c_void_p)))
        return out

    def decode_step(self, B, ids_dev=None, fetch=True):
        """One greedy step for B sequences that stays on the device; returns the next ids if fetch."""
        out = np.empty(B, np.int32) if fetch else None
        self.dev.check(self.dev.L.ruai_model_decode_step(self.h, ids_dev, B, out.ctypes.data_as(C.c_void_p) if fetch else None))
        return out

    def use_persistent_step(self, on=True):
        """Single-token greedy steps as ONE persistent kernel per token (on) or as the chain of launches (default)."""
        self.dev.check(self.dev.L.ruai_model_use_persistent_step(self.h, 1 if on else 0))

    def uses_persistent_step(self, B=1):
        return bool(self.dev.L.ruai_model_uses_persistent_step(self.h, B))

    def cache_reserve(self, B, positions):
        self.dev.check(self.dev.L.ruai_model_cache_reserve(self.h, B, positions))

    def cache_assume(self, B, length):
        self.dev.check(self.dev.L.ruai_model_cache_assume(self.h, B, length))

    def step_bytes(self, B, length):
        v = C.c_double()
        self.dev.check(self.dev.L.ruai_model_step_bytes(self.h, B, length, C.byref(v)))
        return v.value

    def step_launches(self):
        v = C.c_uint32()
        self.dev.check(self.dev.L.ruai_model_step_launches(self.h, C.byref(v)))
        return v.value

    def time_linears(self, B, iters):
        """(ms per pass, launches per pass, algorithmic bytes per pass) of the quantized Linears alone."""
        ms, n, b = C.c_float(), C.c_uint32(), C.c_double()
        self.dev.check(self.dev.L.ruai_model_time_linears(self.h, B, iters, C.byref(ms), C.byref(n), C.byref(b)))
        return ms.value / iters, n.value, b.value

    def tp_export(self):
        buf = C.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        self.dev.check(self.dev.L.ruai_tp_export(self.h, buf))
        return bytes(buf.raw)

    def tp_resync(self):
        """Clear this rank's side of the exchange after a timed-out step (see ruai_tp_resync for the protocol)."""
        self.dev.check(self.dev.L.ruai_tp_resync(self.h))

    def tp_connect(self, handles):
        blob = b"".join(handles)
        self.dev.check(self.dev.L.ruai_tp_connect(self.h, blob))


class Llama(_Model):
    """`Llama` (llama.rs): RMSNorm + RoPE + GQA + SwiGLU decoder, inference methods only."""

    def __init__(self, dev, cfg, tp=None):
        h = C.c_void_p()
        dev.check(dev.L.ruai_llama_create(dev.ctx, C.byref(cfg), C.byref(tp) if tp is not None else None, C.byref(h)))
        super().__init__(dev, h, cfg)


class GPT2(_Model):
    """`GPT2` (gpt2.rs): LayerNorm + learned positions + GELU decoder, inference methods only."""

    def __init__(self, dev, cfg):
        h = C.c_void_p()
        dev.check(dev.L.ruai_gpt2_create(dev.ctx, C.byref(cfg), C.byref(h)))
        super().__init__(dev, h, cfg)
