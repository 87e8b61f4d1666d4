"""Safetensors I/O in the reference's on-disk format (names and layouts of layers.rs:205-211, llama.rs:559-594,
gpt2.rs:344-377; Hugging Face import with the Llama transpose, llama.rs:391-403).

CPU part: a quantized state dict written from the checker's model has exactly the reference's tensor names, dtypes
and shapes, and reads back unchanged.  GPU part: the file loads straight into the kernel layout (no re-quantizing),
the logits equal the checker's, and saving the loaded model reproduces the file byte for byte.
"""
import os

import numpy as np
import pytest
from safetensors.numpy import save_file

import oracle
from ruai_b200 import checkpoint as ck

T_EMBED, T_LMHEAD, T_WPE = 0x10000000, 0x10000001, 0x10000002
LLAMA = dict(V=41, d=32, ffn=96, L=2, H=4, KV=2, hd=8, max_pos=64)


def llama_cfgs(tied):
    from ruai_b200 import _lib
    c = LLAMA
    args = (c["V"], c["d"], c["ffn"], c["L"], c["H"], c["KV"], c["hd"], c["max_pos"], 1e-5, 10000.0, int(tied))
    return oracle.LlamaConfig(*args), _lib.LlamaConfig(*args)


def oracle_llama_state_dict(om, cfg, bits, group, seed):
    """What `serialize::save` of the quantized reference model would hold, built from the checker's model."""
    out = {"model.embed_tokens.weight": oracle.synth_normal(seed, T_EMBED, (cfg.vocab_size, cfg.hidden_size)),
           "model.norm.weight": np.ones(cfg.hidden_size, np.float32)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        out[p + ".input_layernorm.weight"] = np.ones(cfg.hidden_size, np.float32)
        out[p + ".post_attention_layernorm.weight"] = np.ones(cfg.hidden_size, np.float32)
        for name, kind in ck.LLAMA_LINEARS:
            qn, sn = ck._quant_names(f"{p}.{name}", bits)
            out[qn], out[sn] = om.get_linear(i * 16 + kind, bits, group)
    out["lm_head.weight_int8"], out["lm_head.weight_scale"] = om.get_linear(T_LMHEAD, 8)
    return out


def oracle_gpt2_state_dict(om, cfg, bits, group, seed):
    d = cfg.n_embd
    out = {"wte.weight": oracle.synth_normal(seed, T_EMBED, (cfg.vocab_size, d)), "wpe.weight": oracle.synth_normal(seed, T_WPE, (cfg.n_positions, d)),
           "ln_f.weight": np.ones(d, np.float32), "ln_f.bias": np.zeros(d, np.float32)}
    shapes = ck.gpt2_linear_shapes(cfg)
    for i in range(cfg.n_layer):
        p = f"h.{i}"
        for ln in ("ln_1", "ln_2"):
            out[f"{p}.{ln}.weight"], out[f"{p}.{ln}.bias"] = np.ones(d, np.float32), np.zeros(d, np.float32)
        for name, kind, bias_kind in ck.GPT2_LINEARS:
            out[f"{p}.{name}.bias"] = oracle.synth_normal(seed, i * 16 + bias_kind, (shapes[kind][1],))
            qn, sn = ck._quant_names(f"{p}.{name}", bits)
            out[qn], out[sn] = om.get_linear(i * 16 + kind, bits, group)
    out["lm_head.weight_int8"], out["lm_head.weight_scale"] = om.get_linear(T_LMHEAD, 8)
    return out


@pytest.mark.parametrize("bits,group", [(8, 0), (4, 32), (4, 16)])
def test_quantized_state_dict_names_and_layout(tmp_path, bits, group):
    oc, _ = llama_cfgs(False)
    om = oracle.Model(oc, seed=5, bits=bits, group=group or 32)
    sd = oracle_llama_state_dict(om, oc, bits, group, 5)
    c = LLAMA
    # the names tests/quant.rs:106-107 and tests/llama.rs:291 look for
    tag = "weight_int8" if bits == 8 else "weight_int4"
    assert f"model.layers.0.mlp.down_proj.{tag}" in sd and "lm_head.weight_int8" in sd
    assert not any(n.endswith("_proj.weight") for n in sd), "a quantized Linear keeps no f32 weight (layers.rs:126-128)"
    q = sd[f"model.layers.1.self_attn.k_proj.{tag}"]
    s = sd["model.layers.1.self_attn.k_proj." + ("weight_scale" if bits == 8 else "weight_int4_scale")]
    assert q.dtype == np.int8 and s.dtype == np.float32
    if bits == 8:
        assert q.shape == (c["d"], c["KV"] * c["hd"]) and s.shape == (c["KV"] * c["hd"],)
    else:
        assert q.shape == (c["d"] // 2, c["KV"] * c["hd"]) and s.shape == (c["d"] // group, c["KV"] * c["hd"])
    path = str(tmp_path / "m.safetensors")
    save_file(sd, path)
    back = ck.load_file(path)
    assert sorted(back) == sorted(sd)
    assert all(np.array_equal(back[n], sd[n]) and back[n].dtype == sd[n].dtype for n in sd)
    assert ck.detect_quantization(back) == (bits, group)


def test_reader_widens_half_formats(tmp_path):
    """F16 and BF16 tensors (serialize.rs:76-88) widen exactly."""
    import json
    import struct
    a = np.array([[1.5, -2.25, 3.0e-3], [0.0, 65280.0, -1.0]], np.float32)
    bf = (a.view(np.uint32) >> 16).astype(np.uint16)  # these values are exact in bf16
    raw = bf.tobytes() + a.astype(np.float16).tobytes()
    hdr = json.dumps({"b": {"dtype": "BF16", "shape": [2, 3], "data_offsets": [0, 12]}, "h": {"dtype": "F16", "shape": [2, 3], "data_offsets": [12, 24]}},
                     separators=(",", ":")).encode()
    hdr += b" " * (-len(hdr) % 8)
    path = tmp_path / "h.safetensors"
    path.write_bytes(struct.pack("<Q", len(hdr)) + hdr + raw)
    t = ck.load_file(str(path))
    assert np.array_equal(ck._as_f32(t["b"]), (bf.astype(np.uint32) << 16).view(np.float32))
    assert np.array_equal(ck._as_f32(t["h"]), a.astype(np.float16).astype(np.float32))


# ---- GPU ------------------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def dev():
    from ruai_b200 import nn
    assert nn.Device.is_available(), "these tests need a CUDA device"
    return nn.Device.cuda(0)


@pytest.mark.gpu
@pytest.mark.parametrize("tied", [False, True])
@pytest.mark.parametrize("bits,group", [(8, 0), (4, 32), (4, 16)])
def test_llama_quantized_checkpoint_round_trip(dev, tmp_path, bits, group, tied):
    oc, gc = llama_cfgs(tied)
    om = oracle.Model(oc, seed=5, bits=bits, group=group or 32)
    path, path2 = str(tmp_path / "a.safetensors"), str(tmp_path / "b.safetensors")
    save_file(oracle_llama_state_dict(om, oc, bits, group, 5), path)
    gm = ck.load_llama(dev, gc, path)
    ids = np.array([[3, 1, 4, 1, 5, 9, 2, 6]], np.int32)
    want, got = om.forward_cached(ids, all_positions=True), gm.forward_cached(ids, all_positions=True)
    assert np.abs(want - got).max() <= 1e-3 * max(np.abs(want).max(), 1e-6)
    ck.save_llama(gm, gc, path2, bits, group)
    assert open(path, "rb").read() == open(path2, "rb").read()


@pytest.mark.gpu
@pytest.mark.parametrize("bits,group", [(8, 0), (4, 32)])
def test_gpt2_quantized_checkpoint_round_trip(dev, tmp_path, bits, group):
    from ruai_b200 import _lib
    oc, gc = oracle.GPT2Config(41, 32, 64, 2, 2), _lib.GPT2Config(41, 32, 64, 2, 2)
    om = oracle.Model(oc, seed=6, bits=bits, group=group or 32)
    path, path2 = str(tmp_path / "a.safetensors"), str(tmp_path / "b.safetensors")
    save_file(oracle_gpt2_state_dict(om, oc, bits, group, 6), path)
    gm = ck.load_gpt2(dev, gc, path)
    ids = np.array([[3, 1, 4, 1, 5, 9, 2, 6]], np.int32)
    want, got = om.forward_cached(ids, all_positions=True), gm.forward_cached(ids, all_positions=True)
    assert np.abs(want - got).max() <= 1e-3 * max(np.abs(want).max(), 1e-6)
    ck.save_gpt2(gm, gc, path2, bits, group)
    assert open(path, "rb").read() == open(path2, "rb").read()


@pytest.mark.gpu
def test_llama_hugging_face_import_transposes_and_quantizes(dev, tmp_path):
    """An unquantized checkpoint in Hugging Face layout ([out, in] projections) quantized on load equals the checker's
    model built from the same f32 tensors."""
    oc, gc = llama_cfgs(False)
    c = LLAMA
    shapes = ck.llama_linear_shapes(gc)
    sd = {"model.embed_tokens.weight": oracle.synth_normal(5, T_EMBED, (c["V"], c["d"])), "model.norm.weight": np.ones(c["d"], np.float32),
          "lm_head.weight": np.ascontiguousarray(oracle.synth_normal(5, T_LMHEAD, (c["d"], c["V"])).T),
          "model.rotary_emb.inv_freq": np.zeros(c["hd"] // 2, np.float32)}
    for i in range(c["L"]):
        p = f"model.layers.{i}"
        sd[p + ".input_layernorm.weight"] = np.ones(c["d"], np.float32)
        sd[p + ".post_attention_layernorm.weight"] = np.ones(c["d"], np.float32)
        for name, kind in ck.LLAMA_LINEARS:
            sd[f"{p}.{name}.weight"] = np.ascontiguousarray(oracle.synth_normal(5, i * 16 + kind, shapes[kind]).T)
    path = str(tmp_path / "hf.safetensors")
    save_file(sd, path)
    gm = ck.load_llama(dev, gc, path, bits=4, group=32)
    om = oracle.Model(oc, seed=5, bits=4, group=32)
    ids = np.array([[3, 1, 4, 1, 5, 9, 2, 6]], np.int32)
    want, got = om.forward_cached(ids, all_positions=True), gm.forward_cached(ids, all_positions=True)
    assert np.abs(want - got).max() <= 1e-3 * max(np.abs(want).max(), 1e-6)
    q, s = gm.get_linear(0 * 16 + 6, c["ffn"], c["d"], 4, 32)
    qo, so = om.get_linear(0 * 16 + 6, 4, 32)
    assert np.array_equal(q, qo) and np.array_equal(s, so)
