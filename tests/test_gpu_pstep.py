"""GPU parity of the persistent decode kernel (one cooperative launch per token) and of its GEMV data path.

`ruai_matmul_q_stream` runs one quantized Linear through the same ring / tensor-core / fixed-point-accumulator
path the decode step uses, so the arithmetic is checked here against the CPU checker at the reference's own
GPU-vs-CPU tolerance (tests/devices.rs:31-40), on shapes that exercise column and k tails, a weight whose k
exceeds the digit window, several rounds per CTA, and both row counts.  The model-level tests compare the
persistent step with the checker and with the per-launch path of the same library.
"""
import os

import numpy as np
import pytest

import oracle
from ruai_b200 import nn

pytestmark = pytest.mark.gpu

TOL_ABS, TOL_REL = 1e-2, 1e-3


@pytest.fixture(scope="module")
def dev():
    assert nn.Device.is_available(), "these tests need a CUDA device"
    return nn.Device.cuda(0)


def same(cpu, got, tol=1e-4):
    cpu, got = np.asarray(cpu, np.float64), np.asarray(got, np.float64)
    assert cpu.shape == got.shape
    bad = ~((np.abs(cpu - got) <= tol * (1 + np.abs(cpu))) | (cpu == got))
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ; worst {np.abs(cpu - got).max()} (scale {np.abs(cpu).max()})"


def make_weight(dev, bits, k, n, seed):
    rng = np.random.default_rng(seed)
    if bits == 8:
        q = rng.integers(-127, 128, (k, n), dtype=np.int8)
        s = (rng.random(n, dtype=np.float32) + 0.5) * 1e-3
        return q, s, nn.QWeight.int8(dev, q, s)
    q = rng.integers(-128, 128, (k // 2, n), dtype=np.int8)
    s = (rng.random((k // 32, n), dtype=np.float32) + 0.5) * 1e-2
    return q, s, nn.QWeight.int4(dev, q, s, 32)


def ref_matmul(bits, x, q, s):
    return oracle.matmul_int8(x, q, s) if bits == 8 else oracle.matmul_int4(x, q, s)


SHAPES = [
    (64, 300),       # column tail, fewer units than CTAs
    (96, 70),        # one partial tile
    (576, 576),
    (1536, 576),
    (4096, 4096),    # o_proj of the 8B shape
    (4096, 6144),    # q/k/v of the 8B shape
    (14336, 4096),   # down_proj: k beyond the digit window (int4: 448 groups)
    (512, 20000),    # many tiles per CTA: runs of whole tiles and the accumulator rotation
]


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("k,n", SHAPES)
@pytest.mark.parametrize("bits", [4, 8])
def test_stream_matmul_matches_checker(dev, bits, k, n, m):
    q, s, w = make_weight(dev, bits, k, n, k * 31 + n + bits)
    x = oracle.synth_normal(3, k + n + m, (m, k), 1.0)
    want = ref_matmul(bits, x, q, s)
    got = nn.matmul_q_stream(nn.Tensor.from_numpy(dev, x), w).numpy()
    same(want, got)
    # the accumulator is left clean and the sums do not depend on arrival order: identical bits again, and inside a
    # launch that repeats the product
    again = nn.matmul_q_stream(nn.Tensor.from_numpy(dev, x), w, repeat=3).numpy()
    assert np.array_equal(got, again)


def test_stream_matmul_k_tail_int8(dev):
    """k = 100: the last 32-row block of the int8 layout is partly padding."""
    q, s, w = make_weight(dev, 8, 100, 200, 5)
    x = oracle.synth_normal(3, 77, (2, 100), 1.0)
    same(oracle.matmul_int8(x, q, s), nn.matmul_q_stream(nn.Tensor.from_numpy(dev, x), w).numpy())


@pytest.mark.parametrize("bits,k,n", [(4, 16384, 12800), (8, 6400, 15360)])
def test_stream_matmul_several_rounds(dev, bits, k, n):
    """More than 128 units of a k beyond the window per CTA: the digits are rewritten round by round."""
    q, s, w = make_weight(dev, bits, k, n, 11)
    x = oracle.synth_normal(3, 9, (2, k), 1.0)
    same(ref_matmul(bits, x, q, s), nn.matmul_q_stream(nn.Tensor.from_numpy(dev, x), w).numpy())


@pytest.mark.parametrize("bits", [4, 8])
def test_stream_matmul_value_ranges(dev, bits):
    """Rows of very different magnitude, a group of zeros, one huge element: block fixed point keeps f32-grade accuracy."""
    k, n = 1024, 384
    q, s, w = make_weight(dev, bits, k, n, 21)
    x = oracle.synth_normal(3, 5, (2, k), 1.0)
    x[0] *= 1e-6
    x[1, 32:64] = 0.0
    x[1, 100] = 3.0e4
    want = ref_matmul(bits, x, q, s)
    got = nn.matmul_q_stream(nn.Tensor.from_numpy(dev, x), w).numpy()
    for r in range(2):  # tolerance relative to each row's own scale
        sc = np.abs(want[r]).max()
        assert np.abs(want[r] - got[r]).max() <= 2e-5 * sc, (r, np.abs(want[r] - got[r]).max(), sc)


@pytest.mark.parametrize("bits", [4, 8])
def test_stream_matmul_non_finite_rows_stay_non_finite(dev, bits):
    """A NaN or Inf activation must not come out as a plausible finite number (cpu.rs:897-927 propagates it)."""
    k, n = 256, 256
    q, s, w = make_weight(dev, bits, k, n, 22)
    x = oracle.synth_normal(3, 6, (2, k), 1.0)
    x[0, 7] = np.nan
    got = nn.matmul_q_stream(nn.Tensor.from_numpy(dev, x), w).numpy()
    assert not np.isfinite(got[0]).any()
    same(ref_matmul(bits, x[1:], q, s), got[1:])
    x[0, 7] = np.inf
    got = nn.matmul_q_stream(nn.Tensor.from_numpy(dev, x), w).numpy()
    assert not np.isfinite(got[0]).any()
    same(ref_matmul(bits, x[1:], q, s), got[1:])


def test_bounded_wait_runs_out_and_the_context_survives(dev):
    """Failure injected on the host: the launch is told to expect arrivals that never come, the grid barrier's
    bounded wait runs out, the call reports RUAI_ERR_TIMEOUT, and the next call on the same context is correct."""
    q, s, w = make_weight(dev, 4, 576, 576, 1)
    x = oracle.synth_normal(3, 1, (1, 576), 1.0)
    xt = nn.Tensor.from_numpy(dev, x)
    want = oracle.matmul_int4(x, q, s)
    same(want, nn.matmul_q_stream(xt, w).numpy())
    dev.set_wait_limit(4000)
    dev.inject_barrier_skew(1)
    try:
        with pytest.raises(nn.RuaiError, match="bounded wait") as e:
            nn.matmul_q_stream(xt, w)
            dev.synchronize()
        assert e.value.code == 4  # RUAI_ERR_TIMEOUT
    finally:
        dev.set_wait_limit(0)
    same(want, nn.matmul_q_stream(xt, w).numpy())
    dev.synchronize()


@pytest.mark.parametrize("bits", [4, 8])
def test_copy_that_never_completes_runs_the_stage_wait_out(dev, bits):
    """The same for a shared-memory barrier: the first bulk copy is announced larger than it is (on the host), the
    barrier it signals never completes, the consumers' bounded wait for that stage runs out, the kernel leaves in
    order (tensor memory freed, no copy in flight), RUAI_ERR_TIMEOUT is reported and the next call is correct."""
    q, s, w = make_weight(dev, bits, 576, 576, 2)
    x = oracle.synth_normal(3, 2, (1, 576), 1.0)
    xt = nn.Tensor.from_numpy(dev, x)
    want = ref_matmul(bits, x, q, s)
    same(want, nn.matmul_q_stream(xt, w).numpy())
    dev.set_wait_limit(4000)
    dev.inject_copy_shortfall(16)
    try:
        with pytest.raises(nn.RuaiError, match="bounded wait") as e:
            nn.matmul_q_stream(xt, w)
            dev.synchronize()
        assert e.value.code == 4  # RUAI_ERR_TIMEOUT
    finally:
        dev.set_wait_limit(0)
    same(want, nn.matmul_q_stream(xt, w).numpy())
    dev.synchronize()


# ---- the whole step -----------------------------------------------------------------------------------------

def close(want, got, what=""):
    want, got = np.asarray(want, np.float64), np.asarray(got, np.float64)
    assert want.shape == got.shape
    err = np.abs(want - got).max()
    assert err <= TOL_ABS and err <= TOL_REL * max(np.abs(want).max(), 1e-6), f"{what}: max-abs {err}, scale {np.abs(want).max()}"
    return err


def llama_cfgs(V, d, ffn, L, H, KV, hd, max_pos, theta=10000.0, tied=False):
    return (oracle.LlamaConfig(V, d, ffn, L, H, KV, hd, max_pos, 1e-5, theta, int(tied)),
            nn.LlamaConfig(V, d, ffn, L, H, KV, hd, max_pos, 1e-5, theta, int(tied)))


def build_pair(dev, cfgs, seed, bits, persistent=True):
    oc, gc = cfgs
    om = oracle.Model(oc, seed=seed, bits=bits, group=32)
    gm = nn.Llama(dev, gc)
    gm.load_synthetic(seed, bits, 32)
    gm.use_persistent_step(persistent)
    assert gm.uses_persistent_step(1) == persistent
    return om, gm


SMALL = dict(V=331, d=256, ffn=704, L=3, H=8, KV=2, hd=32, max_pos=256)


@pytest.mark.parametrize("B", [1, 2])
@pytest.mark.parametrize("bits", [4, 8])
def test_persistent_step_matches_checker_and_launch_chain(dev, bits, B):
    """Single-token steps from an empty cache (the first has no cached key at all), then after a prefill: logits of
    the persistent step against the checker and against the per-launch path of this library."""
    om, gp = build_pair(dev, llama_cfgs(**SMALL), 3, bits, persistent=True)
    _, gl = build_pair(dev, llama_cfgs(**SMALL), 3, bits, persistent=False)
    assert gp.forward_cached(np.zeros((B, 1), np.int32)) is not None and gp.step_launches() == 1
    gp.cache_clear()
    rng = np.random.default_rng(bits + B)
    tok = rng.integers(0, SMALL["V"], (B, 1)).astype(np.int32)
    for step in range(40):
        want = om.forward_cached(tok)
        got = gp.forward_cached(tok)
        chain = gl.forward_cached(tok)
        close(want, got, f"step {step}")
        close(chain, got, f"step {step} vs launch chain")
        tok = np.array([[oracle.argmax(r)] for r in want], np.int32)
    for m in (om, gp, gl):
        m.cache_clear()
    prompt = rng.integers(0, SMALL["V"], (B, 37)).astype(np.int32)
    close(om.forward_cached(prompt), gp.forward_cached(prompt), "prefill")
    gl.forward_cached(prompt)
    tok = rng.integers(0, SMALL["V"], (B, 1)).astype(np.int32)
    for step in range(30):
        want, got = om.forward_cached(tok), gp.forward_cached(tok)
        close(want, got, f"after prefill, step {step}")
        tok = np.array([[oracle.argmax(r)] for r in want], np.int32)


@pytest.mark.parametrize("H,KV,hd", [(4, 2, 96), (8, 8, 24), (8, 1, 40), (9, 3, 64)])
def test_persistent_step_attention_geometries(dev, H, KV, hd):
    """1, 2, 3 and 8 query heads per KV head, head dimensions that are not powers of two, 70 cached keys plus steps."""
    cfg = dict(V=53, d=H * hd, ffn=64 * 3, L=2, H=H, KV=KV, hd=hd, max_pos=256)
    if cfg["d"] % 32:
        pytest.skip("the persistent step needs a hidden size that is a multiple of 32")
    om, gm = build_pair(dev, llama_cfgs(**cfg), 11, 8)
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, cfg["V"], (2, 70)).astype(np.int32)
    close(om.forward_cached(prompt), gm.forward_cached(prompt), "prefill")
    tok = rng.integers(0, cfg["V"], (2, 1)).astype(np.int32)
    for step in range(40):
        want, got = om.forward_cached(tok), gm.forward_cached(tok)
        assert gm.step_launches() == 1
        close(want, got, f"step {step}")
        tok = np.argmax(want, axis=1).astype(np.int32).reshape(2, 1)


@pytest.mark.parametrize("persistent", [True, False])
def test_greedy_tokens_and_device_argmax_ties(dev, persistent):
    """Greedy generation through either implementation of the step equals the checker's; with two identical head columns
    the device pick (the persistent kernel's pick phase; the chain's fused pick of the head GEMV) takes the larger index
    (generation.rs:6-8, the last maximum)."""
    oc, gc = llama_cfgs(**SMALL)
    om, gm = build_pair(dev, (oc, gc), 4, 4, persistent=persistent)
    prompt = oracle.synth_tokens(0, 0x20000000, 9, SMALL["V"])
    assert gm.generate(prompt, 40).tolist() == om.generate(prompt, 40).tolist()
    # a model whose lm_head is zero except for two identical columns: the largest logit is always shared by several
    # columns (17 and 300, or every other column), and the pick must be the last of them
    c = SMALL
    gm2 = nn.Llama(dev, gc)
    shapes = {0: (c["d"], c["H"] * c["hd"]), 1: (c["d"], c["KV"] * c["hd"]), 2: (c["d"], c["KV"] * c["hd"]), 3: (c["H"] * c["hd"], c["d"]),
              4: (c["d"], c["ffn"]), 5: (c["d"], c["ffn"]), 6: (c["ffn"], c["d"])}
    for layer in range(c["L"]):
        for kind, shp in shapes.items():
            gm2.set_f32(layer * 16 + kind, oracle.synth_normal(7, layer * 16 + kind, shp))
        gm2.set_f32(0x50000000 + layer, np.ones(c["d"], np.float32))
        gm2.set_f32(0x52000000 + layer, np.ones(c["d"], np.float32))
    emb = oracle.synth_normal(7, 0x10000000, (c["V"], c["d"]))
    gm2.set_f32(0x10000000, emb)
    head = np.zeros((c["d"], c["V"]), np.float32)
    head[:, 17] = head[:, 300] = oracle.synth_normal(7, 99, (c["d"],))
    gm2.set_f32(0x10000001, head)
    gm2.set_f32(0x40000000, np.ones(c["d"], np.float32))
    gm2.quantize_int8()
    gm2.use_persistent_step(persistent)
    logits = gm2.forward_cached(np.array([[5]], np.int32))
    assert logits[0, 17] == logits[0, 300]
    best = float(logits.max())
    ties = np.flatnonzero(logits[0] == best)
    assert len(ties) >= 2
    ids = nn.Tensor.from_numpy(dev, np.array([5], np.int32))
    gm2.cache_clear()
    nxt = gm2.decode_step(1, ids.ptr)
    assert nxt[0] == ties[-1], (nxt, ties)
    # several sequences at once (the chain's separate argmax kernel; the persistent pick for two rows)
    for B in (2,) if persistent else (2, 5):
        gm2.cache_clear()
        idsB = nn.Tensor.from_numpy(dev, np.full(B, 5, np.int32))
        assert gm2.decode_step(B, idsB.ptr).tolist() == [int(ties[-1])] * B


@pytest.mark.parametrize("persistent", [True, False])
def test_cache_clear_then_decode_step_with_a_new_batch(dev, persistent):
    """cache_clear() followed directly by decode_step() with another batch size must start at position 0 of fresh
    buffers (the host's position is the authority), not at the device's stale position; on both step paths."""
    om, gm = build_pair(dev, llama_cfgs(**SMALL), 6, 8, persistent=persistent)
    gm.forward_cached(np.array([[1, 2, 3, 4, 5, 6, 7]], np.int32))
    gm.cache_clear()
    om.cache_clear()
    ids = np.array([3, 9], np.int32)
    ids_dev = nn.Tensor.from_numpy(dev, ids)
    nxt = gm.decode_step(2, ids_dev.ptr)
    want = om.forward_cached(ids[:, None])
    assert nxt.tolist() == [oracle.argmax(r) for r in want]
    assert gm.cache_len() == 1
    # switching the path in mid-sequence keeps the position
    gm.use_persistent_step(not persistent)
    nxt2 = gm.decode_step(2, None)
    want2 = om.forward_cached(np.array([[oracle.argmax(r)] for r in want], np.int32))
    assert nxt2.tolist() == [oracle.argmax(r) for r in want2]
    assert gm.cache_len() == 2
