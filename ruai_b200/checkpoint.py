"""Safetensors I/O of the models in the reference's on-disk naming and layout.

A quantized model saved by the reference (`serialize::save`, src/nn/serialize.rs:239-241, over
`state_dict()` = parameters + buffers, modules/module.rs:58-62) holds

  Llama (llama.rs:559-594)                              GPT-2 (gpt2.rs:344-377)
    model.embed_tokens.weight              F32 [V,d]      wte.weight, wpe.weight           F32
    model.layers.{i}.input_layernorm.weight               h.{i}.ln_1.weight / .bias
    model.layers.{i}.self_attn.{q,k,v,o}_proj.<buffers>   h.{i}.attn.c_attn.bias + <buffers>
    model.layers.{i}.post_attention_layernorm.weight      h.{i}.attn.c_proj.bias + <buffers>
    model.layers.{i}.mlp.{gate,up,down}_proj.<buffers>    h.{i}.ln_2.weight / .bias
    model.norm.weight                                     h.{i}.mlp.c_fc / c_proj .bias + <buffers>
    lm_head.<int8 buffers>                                ln_f.weight / .bias, lm_head.<int8 buffers>

with <buffers> = `weight_int8` I8 [in,out] + `weight_scale` F32 [out], or `weight_int4` I8 [in/2,out] +
`weight_int4_scale` F32 [in/group,out] (layers.rs:205-211; I8 as serialize.rs:44, 95).  The head is
int8 even in an int4 model (llama.rs:535-542).  Unquantized checkpoints in Hugging Face layout store
Llama's `*_proj.weight` and `lm_head.weight` as [out,in] (transposed on load, llama.rs:319-321, 391-403)
and GPT-2's Conv1D weights as [in,out] (no transpose, gpt2.rs:4-7).

Quantized tensors go to the device exactly as stored (`ruai_model_set_quantized`, repacked there);
nothing is re-quantized, so saving a loaded model reproduces the file byte for byte.
"""
import ctypes as C
import json
import struct

import numpy as np
from safetensors.numpy import save_file

from . import nn

T_EMBED, T_LMHEAD, T_WPE = 0x10000000, 0x10000001, 0x10000002
TN_FINAL, TN_FINAL_B = 0x40000000, 0x40000001
TN_N1, TN_N1B, TN_N2, TN_N2B = 0x50000000, 0x51000000, 0x52000000, 0x53000000
LLAMA_LINEARS = [("self_attn.q_proj", 0), ("self_attn.k_proj", 1), ("self_attn.v_proj", 2), ("self_attn.o_proj", 3),
                 ("mlp.gate_proj", 4), ("mlp.up_proj", 5), ("mlp.down_proj", 6)]
GPT2_LINEARS = [("attn.c_attn", 7, 11), ("attn.c_proj", 8, 12), ("mlp.c_fc", 9, 13), ("mlp.c_proj", 10, 14)]


_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I8": np.int8, "I32": np.int32, "F64": np.float64}


def load_file(path):
    """Name -> array of a .safetensors file (8-byte header length, JSON header, raw little-endian data).  BF16 arrives
    as raw uint16 words (numpy has no bfloat16); `_as_f32` widens them exactly as serialize.rs:83-88 does."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        base = 8 + n
        out = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if info["dtype"] not in _ST_DTYPES:
                raise ValueError(f"'{name}': unsupported safetensors dtype {info['dtype']}")
            a, b = info["data_offsets"]
            f.seek(base + a)
            out[name] = np.frombuffer(f.read(b - a), dtype=_ST_DTYPES[info["dtype"]]).reshape(info["shape"])
    return out


def llama_linear_shapes(cfg):
    d, hd = cfg.hidden_size, cfg.head_dim
    nq, nkv, f = cfg.num_attention_heads * hd, cfg.num_key_value_heads * hd, cfg.intermediate_size
    return {0: (d, nq), 1: (d, nkv), 2: (d, nkv), 3: (nq, d), 4: (d, f), 5: (d, f), 6: (f, d)}


def gpt2_linear_shapes(cfg):
    d = cfg.n_embd
    return {7: (d, 3 * d), 8: (d, d), 9: (d, 4 * d), 10: (4 * d, d)}


def _quant_names(prefix, bits):
    return (prefix + ".weight_int8", prefix + ".weight_scale") if bits == 8 else (prefix + ".weight_int4", prefix + ".weight_int4_scale")


def detect_quantization(tensors):
    """(bits, group) of the block Linears of a quantized state dict, or (0, 0) for an unquantized one."""
    for name, t in tensors.items():
        if name.startswith("lm_head."):
            continue
        if name.endswith(".weight_int8"):
            return 8, 0
        if name.endswith(".weight_int4"):
            s = tensors[name[:-len("weight_int4")] + "weight_int4_scale"]
            return 4, 2 * t.shape[0] // s.shape[0]
    return 0, 0


def _set_quantized(model, tid, q, s, bits, group):
    q, s = np.ascontiguousarray(q, np.int8), np.ascontiguousarray(s, np.float32)
    model.dev.check(model.dev.L.ruai_model_set_quantized(model.h, tid, q.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p), bits, group))


def _get_f32(model, tid, shape):
    a = np.empty(shape, np.float32)
    model.dev.check(model.dev.L.ruai_model_get_f32(model.h, tid, a.ctypes.data_as(C.c_void_p), a.size))
    return a


def _as_f32(t):
    """F32 / F16 / F64 widen or narrow through numpy; BF16 words (uint16 from `load_file`) become the f32 with those high bits."""
    if t.dtype == np.uint16:
        return (t.astype(np.uint32) << 16).view(np.float32)
    return np.asarray(t, np.float32)


def load_llama(dev, cfg, path, bits=None, group=32):
    """A `Llama` from a safetensors file: a quantized state dict in the reference's format (loaded as stored), or an
    unquantized Hugging Face checkpoint (quantized on the device to `bits`, `group`)."""
    tensors = load_file(path)
    fbits, fgroup = detect_quantization(tensors)
    m = nn.Llama(dev, cfg)
    shapes = llama_linear_shapes(cfg)
    tied = bool(cfg.tie_word_embeddings)
    m.set_f32(T_EMBED, _as_f32(tensors["model.embed_tokens.weight"]))
    m.set_f32(TN_FINAL, _as_f32(tensors["model.norm.weight"]))
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        m.set_f32(TN_N1 + i, _as_f32(tensors[p + ".input_layernorm.weight"]))
        m.set_f32(TN_N2 + i, _as_f32(tensors[p + ".post_attention_layernorm.weight"]))
        for name, kind in LLAMA_LINEARS:
            if fbits:
                qn, sn = _quant_names(f"{p}.{name}", fbits)
                _set_quantized(m, i * 16 + kind, tensors[qn], tensors[sn], fbits, fgroup)
            else:
                w = _as_f32(tensors[f"{p}.{name}.weight"]).T  # Hugging Face [out, in] -> [in, out]
                assert w.shape == shapes[kind], (name, w.shape, shapes[kind])
                m.set_f32(i * 16 + kind, w)
    if fbits:
        _set_quantized(m, T_LMHEAD, tensors["lm_head.weight_int8"], tensors["lm_head.weight_scale"], 8, 0)
        m.dev.check(m.dev.L.ruai_model_quantize(m.h, fbits, fgroup))
    else:
        if not tied:
            m.set_f32(T_LMHEAD, _as_f32(tensors["lm_head.weight"]).T)
        if bits is None:
            raise ValueError("an unquantized checkpoint needs bits=8 or bits=4: this path runs quantized models only")
        m.dev.check(m.dev.L.ruai_model_quantize(m.h, bits, group if bits == 4 else 0))
    m.bits, m.group = (fbits, fgroup) if fbits else (bits, group if bits == 4 else 0)
    return m


def save_llama(m, cfg, path, bits, group=32):
    """`serialize::save` of a quantized `Llama`: every name, dtype and shape as the reference writes them."""
    shapes = llama_linear_shapes(cfg)
    d, V = cfg.hidden_size, cfg.vocab_size
    out = {"model.embed_tokens.weight": _get_f32(m, T_EMBED, (V, d)), "model.norm.weight": _get_f32(m, TN_FINAL, (d,))}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        out[p + ".input_layernorm.weight"] = _get_f32(m, TN_N1 + i, (d,))
        out[p + ".post_attention_layernorm.weight"] = _get_f32(m, TN_N2 + i, (d,))
        for name, kind in LLAMA_LINEARS:
            k, n = shapes[kind]
            qn, sn = _quant_names(f"{p}.{name}", bits)
            out[qn], out[sn] = m.get_linear(i * 16 + kind, k, n, bits, group)
    out["lm_head.weight_int8"], out["lm_head.weight_scale"] = m.get_linear(T_LMHEAD, d, V, 8)
    save_file(out, path)
    return sorted(out)


def load_gpt2(dev, cfg, path, bits=None, group=32):
    """A `GPT2` from a quantized state dict in the reference's format or an unquantized checkpoint (Conv1D [in, out])."""
    tensors = load_file(path)
    fbits, fgroup = detect_quantization(tensors)
    m = nn.GPT2(dev, cfg)
    m.set_f32(T_EMBED, _as_f32(tensors["wte.weight"]))
    m.set_f32(T_WPE, _as_f32(tensors["wpe.weight"]))
    m.set_f32(TN_FINAL, _as_f32(tensors["ln_f.weight"]))
    m.set_f32(TN_FINAL_B, _as_f32(tensors["ln_f.bias"]))
    for i in range(cfg.n_layer):
        p = f"h.{i}"
        for ln, w_id, b_id in (("ln_1", TN_N1, TN_N1B), ("ln_2", TN_N2, TN_N2B)):
            m.set_f32(w_id + i, _as_f32(tensors[f"{p}.{ln}.weight"]))
            m.set_f32(b_id + i, _as_f32(tensors[f"{p}.{ln}.bias"]))
        for name, kind, bias_kind in GPT2_LINEARS:
            m.set_f32(i * 16 + bias_kind, _as_f32(tensors[f"{p}.{name}.bias"]))
            if fbits:
                qn, sn = _quant_names(f"{p}.{name}", fbits)
                _set_quantized(m, i * 16 + kind, tensors[qn], tensors[sn], fbits, fgroup)
            else:
                m.set_f32(i * 16 + kind, _as_f32(tensors[f"{p}.{name}.weight"]))
    if fbits:
        _set_quantized(m, T_LMHEAD, tensors["lm_head.weight_int8"], tensors["lm_head.weight_scale"], 8, 0)
        m.dev.check(m.dev.L.ruai_model_quantize(m.h, fbits, fgroup))
    else:
        if bits is None:
            raise ValueError("an unquantized checkpoint needs bits=8 or bits=4: this path runs quantized models only")
        m.dev.check(m.dev.L.ruai_model_quantize(m.h, bits, group if bits == 4 else 0))
    return m


def save_gpt2(m, cfg, path, bits, group=32):
    shapes = gpt2_linear_shapes(cfg)
    d, V = cfg.n_embd, cfg.vocab_size
    out = {"wte.weight": _get_f32(m, T_EMBED, (V, d)), "wpe.weight": _get_f32(m, T_WPE, (cfg.n_positions, d)),
           "ln_f.weight": _get_f32(m, TN_FINAL, (d,)), "ln_f.bias": _get_f32(m, TN_FINAL_B, (d,))}
    for i in range(cfg.n_layer):
        p = f"h.{i}"
        for ln, w_id, b_id in (("ln_1", TN_N1, TN_N1B), ("ln_2", TN_N2, TN_N2B)):
            out[f"{p}.{ln}.weight"] = _get_f32(m, w_id + i, (d,))
            out[f"{p}.{ln}.bias"] = _get_f32(m, b_id + i, (d,))
        for name, kind, bias_kind in GPT2_LINEARS:
            k, n = shapes[kind]
            out[f"{p}.{name}.bias"] = _get_f32(m, i * 16 + bias_kind, (n,))
            qn, sn = _quant_names(f"{p}.{name}", bits)
            out[qn], out[sn] = m.get_linear(i * 16 + kind, k, n, bits, group)
    out["lm_head.weight_int8"], out["lm_head.weight_scale"] = m.get_linear(T_LMHEAD, d, V, 8)
    save_file(out, path)
    return sorted(out)
