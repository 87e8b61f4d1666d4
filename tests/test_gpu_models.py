"""GPU parity of the model-level C ABI (Llama / GPT-2 forward_cached, generate, decode_step) against the CPU checker.

Tolerance on logits is the one the task states for this path: max-abs 1e-2 and relative 1e-3
(relative to the largest |logit| of the row set), with identical greedy tokens for at least the
first 32 generated tokens.
"""
import numpy as np
import pytest

import oracle
from ruai_b200 import nn

pytestmark = pytest.mark.gpu

TOL_ABS, TOL_REL = 1e-2, 1e-3
T_LMHEAD = 0x10000001


@pytest.fixture(scope="module")
def dev():
    assert nn.Device.is_available(), "these tests need a CUDA device"
    return nn.Device.cuda(0)


def close(want, got, what=""):
    want, got = np.asarray(want, np.float64), np.asarray(got, np.float64)
    assert want.shape == got.shape
    err = np.abs(want - got).max()
    assert err <= TOL_ABS and err <= TOL_REL * max(np.abs(want).max(), 1e-6), f"{what}: max-abs {err}, scale {np.abs(want).max()}"
    return err


def llama_cfg(V, d, ffn, L, H, KV, hd, max_pos, theta=10000.0, tied=False):
    return (oracle.LlamaConfig(V, d, ffn, L, H, KV, hd, max_pos, 1e-5, theta, int(tied)),
            nn.LlamaConfig(V, d, ffn, L, H, KV, hd, max_pos, 1e-5, theta, int(tied)))


def gpt2_cfg(V, n_pos, d, L, H):
    return oracle.GPT2Config(V, n_pos, d, L, H), nn.GPT2Config(V, n_pos, d, L, H)


def build(dev, cfgs, seed, bits, group=32):
    oc, gc = cfgs
    om = oracle.Model(oc, seed=seed, bits=bits, group=group)
    gm = nn.Llama(dev, gc) if isinstance(gc, nn.LlamaConfig) else nn.GPT2(dev, gc)
    gm.load_synthetic(seed, bits, group)
    return om, gm


TINY_LLAMA = dict(V=41, d=32, ffn=96, L=2, H=4, KV=2, hd=8, max_pos=160)


@pytest.mark.parametrize("bits,group", [(8, 0), (4, 32), (4, 16)])
def test_tiny_llama_weights_are_bit_exact(dev, bits, group):
    om, gm = build(dev, llama_cfg(**TINY_LLAMA), 1, bits, group)
    c = TINY_LLAMA
    shapes = {0: (c["d"], c["H"] * c["hd"]), 1: (c["d"], c["KV"] * c["hd"]), 2: (c["d"], c["KV"] * c["hd"]), 3: (c["H"] * c["hd"], c["d"]),
              4: (c["d"], c["ffn"]), 5: (c["d"], c["ffn"]), 6: (c["ffn"], c["d"])}
    for layer in range(c["L"]):
        for kind, (k, n) in shapes.items():
            q, s = gm.get_linear(layer * 16 + kind, k, n, bits, group)
            qo, so = om.get_linear(layer * 16 + kind, bits, group)
            assert np.array_equal(q, qo) and np.array_equal(s, so), (layer, kind)
    q, s = gm.get_linear(T_LMHEAD, c["d"], c["V"], 8)
    qo, so = om.get_linear(T_LMHEAD, 8)
    assert np.array_equal(q, qo) and np.array_equal(s, so)  # the head stays int8 (llama.rs:535-542)


@pytest.mark.parametrize("kind", ["llama", "llama_tied", "gpt2"])
@pytest.mark.parametrize("bits,group", [(8, 0), (4, 32), (4, 16)])
def test_tiny_models_cached_decode(dev, kind, bits, group):
    """tests/llama.rs:139-170, tests/inference.rs:50-68: full forward, chunked [5,1,4,2] and 1-by-1, all vs the checker."""
    if kind == "gpt2":
        cfgs = gpt2_cfg(41, 160, 64, 2, 2)
    else:
        cfgs = llama_cfg(**dict(TINY_LLAMA, tied=(kind == "llama_tied")))
    om, gm = build(dev, cfgs, 2, bits, group)
    ids = np.array([[(i * 5 + 1) % 41 for i in range(12)]], np.int32)
    want = om.forward_cached(ids, all_positions=True)
    close(want, gm.forward_cached(ids, all_positions=True), "full")
    for chunks in ([5, 1, 4, 2], [1] * 12):
        gm.cache_clear()
        pos, rows = 0, []
        for c in chunks:
            rows.append(gm.forward_cached(ids[:, pos:pos + c], all_positions=True))
            pos += c
        close(want, np.concatenate(rows, 1), str(chunks))
    assert gm.cache_len() == 12


def test_cache_capacity_doubles_and_long_decode(dev):
    """tests/kvcache.rs:84-102: 100 single-token steps; capacity 16 -> 32 -> 64 -> 128; logits track the checker."""
    om, gm = build(dev, llama_cfg(**TINY_LLAMA), 3, 8)
    seen = set()
    tok = np.array([[1]], np.int32)
    for step in range(100):
        got = gm.forward_cached(tok)
        seen.add(gm.cache_capacity())
        want = om.forward_cached(tok)
        if step % 9 == 0 or step == 99:
            close(want, got, f"step {step}")
        tok = np.array([[int(np.argmax(want[0]))]], np.int32)
    assert seen == {16, 32, 64, 128}


def test_causal_and_batched(dev):
    """tests/llama.rs:172-191: a batch of 2 equals two separate passes."""
    om, gm = build(dev, llama_cfg(**TINY_LLAMA), 4, 8)
    a = np.array([[1, 2, 3, 4, 5]], np.int32)
    b = np.array([[7, 8, 9, 10, 11]], np.int32)
    both = gm.forward_cached(np.concatenate([a, b]), all_positions=True)
    close(om.forward_cached(np.concatenate([a, b]), all_positions=True), both, "batch")
    gm.cache_clear()
    la = gm.forward_cached(a, all_positions=True)
    gm.cache_clear()
    lb = gm.forward_cached(b, all_positions=True)
    assert np.abs(both[0] - la[0]).max() < 1e-5 and np.abs(both[1] - lb[0]).max() < 1e-5


STEP_CASES = [(kind, bits, B) for kind, bits in (("llama", 4), ("llama", 8), ("gpt2", 8)) for B in (5, 8, 9, 13, 16)] + \
             [("llama_wide", bits, B) for bits in (4, 8) for B in (5, 9, 16)]


@pytest.mark.parametrize("kind,bits,B", STEP_CASES)
def test_steps_of_five_to_sixteen_sequences(dev, kind, bits, B):
    """Decode steps of 5..16 sequences (one 16-row tile on the tensor cores, weights read once): logits of every row
    against the checker.  Layer-reduced models: of mid width (small Linears stay on the narrow kernels, two row tiles from
    nine rows on), and `llama_wide`, where every Linear has 4M weights or more and runs on the 16-row kernel with its fused
    epilogues and the fused greedy pick."""
    if kind == "llama_wide":
        cfgs = llama_cfg(V=4000, d=2048, ffn=5632, L=2, H=32, KV=4, hd=64, max_pos=64)
    elif kind == "llama":
        cfgs = llama_cfg(V=1000, d=576, ffn=1568, L=2, H=9, KV=3, hd=64, max_pos=64)
    else:
        cfgs = gpt2_cfg(V=1000, n_pos=64, d=192, L=2, H=6)
    om, gm = build(dev, cfgs, 5, bits, 32)
    V = 4000 if kind == "llama_wide" else 1000
    prompts = np.stack([oracle.synth_tokens(5, 0x20000000 + b, 2, V) for b in range(B)])
    lo = om.forward_cached(prompts)
    close(lo, gm.forward_cached(prompts), "prefill")
    for step in range(3):
        nxt = np.array([oracle.argmax(r) for r in lo], np.int32)[:, None]
        lo = om.forward_cached(nxt)
        close(lo, gm.forward_cached(nxt), f"{kind} int{bits} B={B} step {step}")
    # the greedy pick fused into the head's launch (one 16-row tile): ids of one more step
    nxt = np.array([oracle.argmax(r) for r in lo], np.int32)
    lo = om.forward_cached(nxt[:, None])
    ids_dev = nn.Tensor.from_numpy(dev, nxt)
    got = gm.decode_step(B, ids_dev.ptr)
    srt = np.sort(lo, axis=1)
    decisive = (srt[:, -1] - srt[:, -2]) > 1e-4
    want = np.array([oracle.argmax(r) for r in lo], np.int32)
    assert (got[decisive] == want[decisive]).all(), f"{kind} int{bits} B={B}: fused pick"


def test_decode_graph_survives_a_larger_scratch(dev):
    """The captured decode step holds the address of the context's scratch (split activations of the 16-row tile).  A
    later prefill of many rows needs a larger scratch, which moves it: the next decode step has to be captured anew, not
    replayed with the old address."""
    cfgs = llama_cfg(V=1000, d=576, ffn=1568, L=2, H=9, KV=3, hd=64, max_pos=256)
    om, gm = build(dev, cfgs, 6, 4, 32)
    B = 8

    def steps(T, n):
        prompts = np.stack([oracle.synth_tokens(6, 0x20000000 + b, T, 1000) for b in range(B)])
        om.cache_clear()
        gm.cache_clear()
        lo = om.forward_cached(prompts)
        close(lo, gm.forward_cached(prompts), f"prefill of {B} x {T}")
        nxt = np.array([oracle.argmax(r) for r in lo], np.int32)
        for step in range(n):
            lo = om.forward_cached(nxt[:, None])
            want = np.array([oracle.argmax(r) for r in lo], np.int32)
            ids_dev = nn.Tensor.from_numpy(dev, nxt)  # (kept alive across the call)
            got = gm.decode_step(B, ids_dev.ptr)
            srt = np.sort(lo, axis=1)
            decisive = (srt[:, -1] - srt[:, -2]) > 1e-4
            assert (got[decisive] == want[decisive]).all(), f"T={T} step {step}"
            nxt = want
        close(om.forward_cached(nxt[:, None]), gm.forward_cached(nxt[:, None]), f"T={T} step logits")

    steps(2, 2)     # captures the graph of a step of 8 sequences
    steps(128, 2)   # 1024 rows through the GEMM: the scratch grows; then steps of 8 sequences again


@pytest.mark.parametrize("H,KV,hd,B", [(4, 2, 96, 1), (6, 6, 24, 3), (8, 1, 40, 2), (4, 2, 96, 40)])
def test_attention_geometries(dev, H, KV, hd, B):
    """Head dimensions that are not powers of two, 1 / 2 / 8 query heads per KV head, and enough sequences to take the
    small-CTA variant of the attention kernel: prefill of 70 tokens (two chunks of keys, causal) and then single-token
    steps over several key splits, against the checker."""
    cfg = dict(V=53, d=H * hd, ffn=64, L=2, H=H, KV=KV, hd=hd, max_pos=256)
    om, gm = build(dev, llama_cfg(**cfg), 11, 8)
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, cfg["V"], (B, 70)).astype(np.int32)
    close(om.forward_cached(prompt), gm.forward_cached(prompt), "prefill")
    tok = rng.integers(0, cfg["V"], (B, 1)).astype(np.int32)
    for step in range(70):
        want, got = om.forward_cached(tok), gm.forward_cached(tok)
        if step % 23 == 0 or step == 69:
            close(want, got, f"step {step}")
        tok = np.argmax(want, axis=1).astype(np.int32).reshape(B, 1)


def test_errors_mirror_the_reference_asserts(dev):
    _, gm = build(dev, llama_cfg(**dict(TINY_LLAMA, max_pos=8)), 5, 8)
    with pytest.raises(nn.RuaiError, match="exceeds max_position_embeddings"):
        gm.forward_cached(np.zeros((1, 9), np.int32))
    with pytest.raises(nn.RuaiError, match="out of range"):
        gm.forward_cached(np.array([[41]], np.int32))
    gm.cache_clear()
    gm.forward_cached(np.array([[1, 2]], np.int32))
    with pytest.raises(nn.RuaiError, match="do not match the cached"):
        gm.forward_cached(np.array([[1], [2]], np.int32))
    fresh = nn.Llama(dev, llama_cfg(**TINY_LLAMA)[1])
    with pytest.raises(nn.RuaiError, match="quantize"):
        fresh.forward_cached(np.array([[1]], np.int32))


@pytest.mark.parametrize("kind", ["llama", "gpt2"])
def test_generate_slides_the_window(dev, kind):
    """generation.rs:96-101 with a context of 8."""
    cfgs = gpt2_cfg(41, 8, 64, 2, 2) if kind == "gpt2" else llama_cfg(**dict(TINY_LLAMA, max_pos=8))
    om, gm = build(dev, cfgs, 6, 8)
    prompt = np.array([1, 2, 3], np.int32)
    assert gm.generate(prompt, 14).tolist() == om.generate(prompt, 14).tolist()


def test_set_weights_then_quantize_matches_load_synthetic(dev):
    """The `set f32 weights -> quantize_int4(group)` route (what a checkpoint loader uses) equals the synthetic loader."""
    oc, gc = llama_cfg(**TINY_LLAMA)
    c = TINY_LLAMA
    gm = nn.Llama(dev, gc)
    shapes = {0: (c["d"], c["H"] * c["hd"]), 1: (c["d"], c["KV"] * c["hd"]), 2: (c["d"], c["KV"] * c["hd"]), 3: (c["H"] * c["hd"], c["d"]),
              4: (c["d"], c["ffn"]), 5: (c["d"], c["ffn"]), 6: (c["ffn"], c["d"])}
    for layer in range(c["L"]):
        for kind, shp in shapes.items():
            gm.set_f32(layer * 16 + kind, oracle.synth_normal(7, layer * 16 + kind, shp))
        gm.set_f32(0x50000000 + layer, np.ones(c["d"], np.float32))
        gm.set_f32(0x52000000 + layer, np.ones(c["d"], np.float32))
    gm.set_f32(0x10000000, oracle.synth_normal(7, 0x10000000, (c["V"], c["d"])))
    gm.set_f32(T_LMHEAD, oracle.synth_normal(7, T_LMHEAD, (c["d"], c["V"])))
    gm.set_f32(0x40000000, np.ones(c["d"], np.float32))
    with pytest.raises(nn.RuaiError, match="must be even and divide"):
        gm.quantize_int4(5)
    gm2 = nn.Llama(dev, gc)
    gm2.load_synthetic(7, 4, 16)
    om = oracle.Model(oc, seed=7, bits=4, group=16)
    ids = np.array([[3, 1, 4, 1, 5, 9]], np.int32)
    want = om.forward_cached(ids, all_positions=True)
    close(want, gm2.forward_cached(ids, all_positions=True), "synthetic")


# ---- the benchmark configurations --------------------------------------------------------

def greedy_parity(om, gm, prompt, n_new, min_same=32):
    ids_o, trace = om.generate(prompt, n_new, trace=True)
    ids_g = gm.generate(prompt, n_new)
    same = 0
    for a, b in zip(ids_o[prompt.size:], ids_g[prompt.size:]):
        if a != b:
            break
        same += 1
    if same < n_new:
        row = np.sort(trace[same])[::-1]
        msg = f"first divergence at generated token {same}; checker top-2 margin there {row[0] - row[1]:.3e}"
    else:
        msg = ""
    assert same >= min(min_same, n_new), msg
    return same, trace


def test_config1_gpt2_small_int8_greedy(dev):
    """GPT-2-small-shaped int8: 12 layers, d 768, 12 heads, vocab 50257, ctx 1024; prompt 16, 32 greedy tokens."""
    om, gm = build(dev, gpt2_cfg(50257, 1024, 768, 12, 12), 0, 8)
    prompt = oracle.synth_tokens(0, 0x20000000, 16, 50257)
    same, trace = greedy_parity(om, gm, prompt, 32)
    assert same == 32
    # logits of the prompt's last position and of a decode step
    gm.cache_clear()
    got = gm.forward_cached(prompt[None, :])
    close(trace[0:1], got, "prompt logits")


@pytest.mark.parametrize("bits", [8, 4])
def test_config2_3_smollm2_shaped(dev, bits):
    """SmolLM2-135M-shaped Llama (30 layers, d 576, 9/3 heads, ffn 1536, vocab 49152, tied), int8 and int4 g32."""
    om, gm = build(dev, llama_cfg(49152, 576, 1536, 30, 9, 3, 64, 2048, tied=True), 0, bits, 32)
    prompt = oracle.synth_tokens(0, 0x20000000, 64, 49152)
    same, trace = greedy_parity(om, gm, prompt, 40)
    gm.cache_clear()
    close(trace[0:1], gm.forward_cached(prompt[None, :]), "prompt logits")
    # batch 16: sixteen different prompts, forward_cached([B, 1]) steps with per-row argmax
    B, T = 16, 8
    prompts = np.stack([oracle.synth_tokens(0, 0x20000000 + b, T, 49152) for b in range(B)])
    om.cache_clear()
    gm.cache_clear()
    lo = om.forward_cached(prompts)
    close(lo, gm.forward_cached(prompts), "batch-16 prefill")
    nxt = np.array([oracle.argmax(r) for r in lo], np.int32)
    ids_dev = nn.Tensor.from_numpy(dev, nxt)
    for step in range(3):
        lo = om.forward_cached(nxt[:, None])
        want_next = np.array([oracle.argmax(r) for r in lo], np.int32)
        got_next = gm.decode_step(B, ids_dev.ptr if step == 0 else None)
        assert got_next.tolist() == want_next.tolist(), f"batched greedy step {step}"
        nxt = want_next
    assert gm.step_launches() > 0


@pytest.mark.parametrize("name,cfg", [
    ("tinyllama-1.1b-shaped, 2 of 22 layers", dict(V=32000, d=2048, ffn=5632, L=2, H=32, KV=4, hd=64, max_pos=2048)),
    ("llama-3-8b-shaped, 2 of 32 layers", dict(V=128256, d=4096, ffn=14336, L=2, H=32, KV=8, hd=128, max_pos=2048, theta=500000.0)),
])
@pytest.mark.parametrize("bits", [8, 4])
def test_config4_5_full_width_layer_reduced(dev, name, cfg, bits):
    """Full layer widths, vocabulary and head geometry of configs 4 and 5 with the layer count cut to 2 so the
    CPU checker finishes in seconds: prompt 12, then 6 greedy tokens and their logits."""
    om, gm = build(dev, llama_cfg(**cfg), 0, bits, 32)
    prompt = oracle.synth_tokens(0, 0x20000000, 12, cfg["V"])
    same, trace = greedy_parity(om, gm, prompt, 6, min_same=6)
    gm.cache_clear()
    close(trace[0:1], gm.forward_cached(prompt[None, :]), name)


# ---- the benchmark models at FULL depth, against tokens and logits the checker produced for them ----------------

FULL = {
    "tinyllama-1.1b": dict(V=32000, d=2048, ffn=5632, L=22, H=32, KV=4, hd=64, max_pos=2048, theta=10000.0),
    "llama3-8b": dict(V=128256, d=4096, ffn=14336, L=32, H=32, KV=8, hd=128, max_pos=2048, theta=500000.0),
}


@pytest.mark.parametrize("persistent", [False, True])
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("name", ["tinyllama-1.1b", "llama3-8b"])
def test_full_depth_greedy_tokens_and_logits(dev, greedy_golden, name, bits, persistent):
    """All 22 / 32 layers, prompt 16, 32 greedy tokens: identical ids, and the logits of every step within max-abs 1e-2
    and 1e-3 of the row's largest magnitude, on both implementations of the single-token step (chain of launches,
    persistent kernel).  The expected values come from tests/golden/make_greedy_golden.py (the CPU checker run on the
    full model); the top-2 margins stored there show every pick is decisive (>= 7e-3)."""
    key = f"{name}-int{bits}"
    ids, margin = greedy_golden[key + "/ids"], greedy_golden[key + "/margin"]
    want, absmax = greedy_golden[key + "/logits"], greedy_golden[key + "/absmax"]
    _, gc = llama_cfg(**FULL[name])
    gm = nn.Llama(dev, gc)
    gm.load_synthetic(0, bits, 32)
    gm.use_persistent_step(persistent)
    assert gm.uses_persistent_step(1) == persistent
    prompt = oracle.synth_tokens(0, 0x20000000, 16, FULL[name]["V"])
    assert prompt.tolist() == ids[:16].tolist()
    got = gm.generate(prompt, 32)
    assert got.tolist() == ids.tolist(), f"first difference at {int(np.argmax(got != ids)) - 16}; margins {margin[:4]}"
    # teacher-forced logits of every step (single-token steps after the prompt)
    gm.cache_clear()
    rows = [gm.forward_cached(prompt[None, :])[0]]
    for t in ids[16:-1]:
        rows.append(gm.forward_cached(np.array([[t]], np.int32))[0])
    got_l = np.stack(rows)[:, ::61]
    err = np.abs(got_l - want).max(axis=1)
    assert (err <= TOL_ABS).all() and (err <= TOL_REL * absmax).all(), (err.max(), absmax.min())


@pytest.mark.slow
@pytest.mark.parametrize("name,B,cfg", [
    ("tinyllama-1.1b-shaped, batch 64", 64, dict(V=32000, d=2048, ffn=5632, L=2, H=32, KV=4, hd=64, max_pos=2048)),
    ("llama-3-8b-shaped, batch 128", 128, dict(V=128256, d=4096, ffn=14336, L=2, H=32, KV=8, hd=128, max_pos=2048, theta=500000.0)),
])
def test_large_batch_decode_steps(dev, name, B, cfg):
    """Batched decode at the benchmark's large batches (the tensor-core GEMM inside the decode loop): B prompts of 3
    tokens, then two greedy steps through decode_step; ids and logits against the checker.  Full widths, 2 layers."""
    om, gm = build(dev, llama_cfg(**cfg), 0, 4, 32)
    prompts = np.stack([oracle.synth_tokens(0, 0x20000000 + b, 3, cfg["V"]) for b in range(B)])
    lo = om.forward_cached(prompts)
    close(lo, gm.forward_cached(prompts), name + " prefill")
    nxt = np.array([oracle.argmax(r) for r in lo], np.int32)
    ids_dev = nn.Tensor.from_numpy(dev, nxt)
    for step in range(2):
        # both models are fed the checker's ids, so that a near-tie in one step does not send them down different paths
        lo = om.forward_cached(nxt[:, None])
        want_next = np.array([oracle.argmax(r) for r in lo], np.int32)
        got_next = gm.decode_step(B, ids_dev.ptr)
        srt = np.sort(lo, axis=1)
        decisive = (srt[:, -1] - srt[:, -2]) > 1e-4
        assert (got_next[decisive] == want_next[decisive]).all(), f"{name}: step {step}"
        assert gm.cache_len() == om.cache_len() == 3 + step + 1
        nxt = want_next
        ids_dev = nn.Tensor.from_numpy(dev, nxt)
    # the logits of one more step, all B rows
    close(om.forward_cached(nxt[:, None]), gm.forward_cached(nxt[:, None]), name + " step logits")


# ---- sampling on the device (generation.rs:15-73) ----

@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.8, 40, 1.0), (0.7, 0, 0.9), (1.3, 50, 0.95), (1.0, 1, 1.0), (1.0, 0, 0.01), (0.0, 0, 1.0)])
def test_device_sampler_matches_checker(dev, temperature, top_k, top_p):
    """The same draws from the same seed on rows of logits with a wide and with a narrow spread, vocabulary sizes that
    are not multiples of the warp.  A draw that the checker reports as decided by less than 2e-6 of probability mass
    (the two round exp differently, about 1e-7 relative) may fall either way and is not compared."""
    rng = np.random.default_rng(7)
    for V, spread in [(4, 1.0), (1000, 3.0), (32003, 1.0), (128256, 6.0)]:
        logits = (rng.standard_normal(V) * spread).astype(np.float32)
        logits[V // 3] = logits[V // 2]  # a tie
        t = nn.Tensor.from_numpy(dev, logits)
        so, sg = oracle.Sampler(temperature, top_k, top_p, 123), nn.Sampler(temperature, top_k, top_p, 123)
        compared = 0
        for _ in range(12):
            want, got = so.sample(logits), sg.sample(t)
            assert so.state.value == sg.state.value
            if so.margin > 2e-6:
                assert want == got, (V, want, got, so.margin)
                compared += 1
        assert compared >= 6, (V, compared)


def test_device_sampler_reference_cases(dev):
    """tests/inference.rs:186-208 on the device sampler."""
    logits = np.array([1.0, 3.0, 2.0, -1.0], np.float32)
    t = nn.Tensor.from_numpy(dev, logits)
    assert nn.Sampler(0.0).sample(t) == 1
    assert nn.Sampler(1.0, 1, 1.0, 7).sample(t) == 1
    assert nn.Sampler(1.0, 0, 0.01, 7).sample(t) == 1
    s = nn.Sampler(1.0, 2, 1.0, 3)
    assert all(s.sample(t) in (1, 2) for _ in range(200))
    s = nn.Sampler(1.0, 0, 1.0, 11)
    counts = np.zeros(4)
    for _ in range(4000):
        counts[s.sample(t)] += 1
    p = np.exp(logits) / np.exp(logits).sum()
    assert np.abs(counts / 4000.0 - p).max() < 0.03, counts


@pytest.mark.parametrize("persistent", [False, True])
def test_sampled_generation_matches_checker(dev, persistent):
    """generate with Sampler::new(0.9, 20, 0.95, seed): the same tokens as the checker up to the first draw that the
    checker reports as decided by less than 1e-4 of probability mass (the logits of the two differ by their tolerance)."""
    cfg = dict(V=331, d=256, ffn=704, L=3, H=8, KV=2, hd=32, max_pos=256)
    oc = oracle.LlamaConfig(cfg["V"], cfg["d"], cfg["ffn"], cfg["L"], cfg["H"], cfg["KV"], cfg["hd"], cfg["max_pos"], 1e-5, 10000.0, 0)
    gc = nn.LlamaConfig(cfg["V"], cfg["d"], cfg["ffn"], cfg["L"], cfg["H"], cfg["KV"], cfg["hd"], cfg["max_pos"], 1e-5, 10000.0, 0)
    om = oracle.Model(oc, seed=5, bits=8, group=32)
    gm = nn.Llama(dev, gc)
    gm.load_synthetic(5, 8, 32)
    gm.use_persistent_step(persistent)
    prompt = oracle.synth_tokens(0, 0x20000000, 7, cfg["V"])
    agree = 0
    for seed in (1, 2, 3):
        want, margins = om.generate_sampled(prompt, 24, 0.9, 20, 0.95, seed)
        got = gm.generate_sampled(prompt, 24, 0.9, 20, 0.95, seed)
        safe = int(np.argmax(margins < 1e-4)) if (margins < 1e-4).any() else 24
        assert got[:7 + safe].tolist() == want[:7 + safe].tolist(), (seed, safe)
        agree += safe
    assert agree >= 24


def test_failed_cache_growth_leaves_the_model_usable(dev):
    """A cache the device cannot hold (one allocation of terabytes, refused by the driver at once: nothing is consumed)
    fails with an error that says the cache was dropped; the model then answers as after cache_clear."""
    cfg = dict(V=331, d=256, ffn=704, L=3, H=8, KV=2, hd=32, max_pos=256)
    om, gm = build(dev, llama_cfg(**cfg), 2, 8, 32)
    prompt = oracle.synth_tokens(0, 0x20000000, 9, cfg["V"])[None, :]
    close(om.forward_cached(prompt), gm.forward_cached(prompt), "before")
    gm.cache_clear()
    om.cache_clear()
    with pytest.raises(nn.RuaiError, match="cache was dropped"):
        gm.cache_reserve(1 << 26, 256)
    assert gm.cache_len() == 0
    close(om.forward_cached(prompt), gm.forward_cached(prompt), "after the failed growth")
    tok = np.array([[7]], np.int32)
    close(om.forward_cached(tok), gm.forward_cached(tok), "a step after it")
