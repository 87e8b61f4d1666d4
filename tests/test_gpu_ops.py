"""GPU parity of the op-level C ABI (quantizer, repack, dequant, quantized matmul) against the CPU checker."""
import numpy as np
import pytest

import oracle
from ruai_b200 import nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert nn.Device.is_available(), "these tests need a CUDA device"
    return nn.Device.cuda(0)


def same(cpu, got, tol):
    """tests/devices.rs:31-40."""
    cpu, got = np.asarray(cpu, np.float64), np.asarray(got, np.float64)
    assert cpu.shape == got.shape
    bad = ~((np.abs(cpu - got) <= tol * (1 + np.abs(cpu))) | (cpu == got))
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ; worst {np.abs(cpu - got).max()}"


def bf16_round(a):
    """f32 -> bf16 (round to nearest even) as raw uint16, and the widened value."""
    b = np.ascontiguousarray(a, np.float32).view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return r, (r.astype(np.uint32) << 16).view(np.float32)


def bf16_widen(r):
    return (np.asarray(r, np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---- quantizer: bit exact with the checker (and so with layers.rs:112-165) ------------

@pytest.mark.parametrize("k,n", [(48, 17), (576, 192), (768, 2304), (4096, 1024)])
def test_quantize_int8_bit_exact(dev, k, n):
    w = oracle.synth_normal(7, k * 131 + n, (k, n))
    if n > 3:
        w[:, 3] = 0.0
    q, s = nn.quantize_int8_device(dev, w)
    qo, so = oracle.quantize_int8(w)
    assert np.array_equal(s, so) and np.array_equal(q, qo)


@pytest.mark.parametrize("k,n,g", [(8, 3, 4), (64, 20, 32), (576, 1536, 32), (4096, 512, 32), (64, 48, 16)])
def test_quantize_int4_bit_exact(dev, k, n, g):
    w = oracle.synth_normal(8, k * 131 + n, (k, n))
    w[:g, 0] = 0.0
    q, s = nn.quantize_int4_device(dev, w, g)
    qo, so = oracle.quantize_int4(w, g)
    assert np.array_equal(s, so) and np.array_equal(q, qo)


def test_quantizer_golden(dev, golden):
    q, s = nn.quantize_int8_device(dev, golden["q8_w"])
    assert np.array_equal(q, golden["q8_q"]) and np.array_equal(s, golden["q8_scale"])
    for tag in ("qa", "qb"):
        q, s = nn.quantize_int4_device(dev, golden[f"{tag}_w"], int(golden[f"{tag}_g"]))
        assert np.array_equal(q, golden[f"{tag}_packed"]) and np.array_equal(s, golden[f"{tag}_scale"])


def test_int4_group_must_divide_the_input_width(dev):
    """tests/quant.rs:136-140 through the C ABI."""
    with pytest.raises(ValueError, match="must be even and divide"):
        nn.quantize_int4_device(dev, np.zeros((30, 4), np.float32), 16)
    q = np.zeros((15, 4), np.int8)
    with pytest.raises(nn.RuaiError, match="must be even and divide"):
        nn.QWeight.int4(dev, q, np.zeros((2, 4), np.float32), 16)


# ---- repack round trip: bit exact -------------------------------------------------------

@pytest.mark.parametrize("k,n", [(64, 300), (33, 70), (32, 48), (576, 576), (4096, 1024), (1, 1)])
def test_repack_int8_round_trip(dev, k, n):
    rng = np.random.default_rng(k * 7 + n)
    q = rng.integers(-128, 128, (k, n), dtype=np.int8)
    s = rng.random(n, dtype=np.float32)
    w = nn.QWeight.int8(dev, q, s)
    q2, s2 = w.unpack()
    assert np.array_equal(q, q2) and np.array_equal(s, s2)


@pytest.mark.parametrize("k,n,g", [(64, 300, 32), (32, 70, 8), (64, 48, 16), (576, 1536, 32), (4096, 256, 32), (2, 1, 2)])
def test_repack_int4_round_trip_and_dequant(dev, k, n, g):
    rng = np.random.default_rng(k * 7 + n)
    q = rng.integers(-128, 128, (k // 2, n), dtype=np.int8)
    s = rng.random((k // g, n), dtype=np.float32)
    w = nn.QWeight.int4(dev, q, s, g)
    q2, s2 = w.unpack()
    assert np.array_equal(q, q2) and np.array_equal(s, s2)
    assert np.array_equal(w.dequant(), oracle.dequant_int4(q, s, g))  # tol 0, tests/devices.rs:491


# ---- quantized matmul: the reference's own GPU-vs-CPU cases (tests/devices.rs:444-502) ----

def run_matmul(dev, x, w, dtype, bias=None):
    if dtype == "f32":
        xt, xf = nn.Tensor.from_numpy(dev, x.astype(np.float32)), x.astype(np.float32)
    elif dtype == "f16":
        xh = x.astype(np.float16)
        xt, xf = nn.Tensor.from_numpy(dev, xh), xh.astype(np.float32)
    else:
        raw, xf = bf16_round(x)
        xt = nn.Tensor.from_numpy(dev, raw, rdtype=nn.BF16)
    bt = None if bias is None else nn.Tensor.from_numpy(dev, bias)
    y = nn._matmul_q(xt, w, bt).numpy()
    if dtype == "bf16":
        y = bf16_widen(y)
    return xf, y.astype(np.float32)


TOL = {"f32": 1e-4, "f16": 6e-3, "bf16": 3e-2}  # devices.rs: 1e-4, half_tol * 3


def round_to(y, dtype):
    if dtype == "f16":
        return y.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_round(y)[1]
    return y


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("idx", [0, 1, 2])
def test_int8_matmul_reference_cases(dev, golden, idx, dtype):
    q, s = golden[f"i8_{idx}_q"], golden[f"i8_{idx}_s"]
    xf, y = run_matmul(dev, golden[f"i8_{idx}_x"], nn.QWeight.int8(dev, q, s), dtype)
    same(round_to(oracle.matmul_int8(xf, q, s), dtype), y, TOL[dtype])
    if dtype == "f32":
        same(golden[f"i8_{idx}_y"], y, 1e-4)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("idx", [0, 1, 2])
def test_int4_matmul_reference_cases(dev, golden, idx, dtype):
    q, s, g = golden[f"i4_{idx}_q"], golden[f"i4_{idx}_s"], int(golden[f"i4_{idx}_g"])
    xf, y = run_matmul(dev, golden[f"i4_{idx}_x"], nn.QWeight.int4(dev, q, s, g), dtype)
    same(round_to(oracle.matmul_int4(xf, q, s), dtype), y, TOL[dtype])
    if dtype == "f32":
        same(golden[f"i4_{idx}_y"], y, 1e-4)


def test_int4_identity_reads_the_weights_back(dev, golden):
    """tests/quant.rs:55-57 on the device."""
    for tag in ("qa", "qb"):
        w, g = golden[f"{tag}_w"], int(golden[f"{tag}_g"])
        lin = nn.Linear(dev, w)
        lin.quantize_int4(g)
        assert sorted(lin.state_dict()) == ["weight_int4", "weight_int4_scale"]
        assert lin.dims() == w.shape
        got = lin.forward(nn.Tensor.from_numpy(dev, np.eye(w.shape[0], dtype=np.float32))).numpy()
        assert np.abs(got - golden[f"{tag}_want"]).max() < 1e-6


# ---- the microbenchmark grid: M in {1,4,16,64,512}, K=N in {576,1536,4096}, + [1,2048]@[2048,2048] ----

GRID = [(m, kn, kn) for kn in (576, 1536, 4096) for m in (1, 4, 16, 64)] + [(512, 576, 576), (512, 1536, 1536), (1, 2048, 2048),
        (3, 4096, 14336 // 4), (2, 14336 // 4, 4096), (16, 768, 2304), (7, 1000, 130)]


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,k,n", GRID)
def test_matmul_grid_f32(dev, m, k, n, bits):
    if bits == 4 and k % 32:
        k = (k // 32) * 32
    x = oracle.synth_normal(11, 0x30000000 + m * 31 + k, (m, k), 1.0)
    x[:, ::7] = 0.0  # the CPU path skips zero activations (cpu.rs:909, 1052)
    w = oracle.synth_normal(11, k * 65537 + n, (k, n))
    if bits == 8:
        q, s = oracle.quantize_int8(w)
        qw, want = nn.QWeight.int8(dev, q, s), oracle.matmul_int8(x, q, s)
    else:
        q, s = oracle.quantize_int4(w, 32)
        qw, want = nn.QWeight.int4(dev, q, s, 32), oracle.matmul_int4(x, q, s)
    bias = oracle.synth_normal(11, 99, (n,))
    _, y = run_matmul(dev, x, qw, "f32", bias)
    same(want + bias, y, 1e-4)
    q2, s2 = qw.unpack()
    assert np.array_equal(q2, q) and np.array_equal(s2, s)


# the Llama-3-8B widths (hidden 4096, q/k/v 6144, MLP 14336) at prefill-sized row counts, ragged and full tiles
WIDE = [(17, 4096, 14336), (64, 4096, 6144), (128, 14336, 4096), (512, 4096, 4096), (17, 4096, 28672), (64, 4096, 28672), (512, 14336, 4096)]


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,k,n", WIDE)
def test_matmul_grid_8b_widths(dev, m, k, n, bits):
    x = oracle.synth_normal(13, 0x31000000 + m, (m, k), 1.0)
    w = oracle.synth_normal(13, k * 65537 + n, (k, n))
    if bits == 8:
        q, s = oracle.quantize_int8(w)
        qw, want = nn.QWeight.int8(dev, q, s), oracle.matmul_int8(x, q, s)
    else:
        q, s = oracle.quantize_int4(w, 32)
        qw, want = nn.QWeight.int4(dev, q, s, 32), oracle.matmul_int4(x, q, s)
    _, y = run_matmul(dev, x, qw, "f32")
    # Quantized-Linear outputs: max-abs 1e-2 and 1e-3 relative to the output's scale.  (The rows-by-the-hundred GEMM
    # carries the activations as two bf16 pieces, 16 significant bits; over k = 14336 a handful of the 524288 outputs
    # miss the 1e-4 * (1 + |y|) of tests/devices.rs by up to 4e-4, which the smaller shapes above all meet.)
    err = np.abs(want.astype(np.float64) - y).max()
    assert err <= 1e-2 and err <= 1e-3 * np.abs(want).max(), (err, np.abs(want).max())
    loose = ~(np.abs(want - y) <= 1e-4 * (1 + np.abs(want)))
    assert loose.mean() <= 1e-4, f"{loose.sum()} of {loose.size} outputs beyond the tests/devices.rs tolerance"


# 5..16 rows: the 16-row tile (weights streamed once).  Shapes chosen so that k splits over 1, 2, 4 and 8 CTAs, the last
# stage and the last column tile are ragged, and k is not a multiple of the group.
ROWS16 = [(9, 64, 48), (12, 96, 130), (16, 4096, 512), (13, 4096, 6144), (16, 14336, 4096), (10, 4096, 28672), (16, 1000, 130), (11, 1536, 1536),
          (5, 4096, 4096), (8, 14336, 4096), (6, 96, 70), (4, 14336, 4096),
          # 4M weights and more (what the 16-row kernel takes) with ragged edges: a last column tile of 76 / 4 / 2 columns, an
          # odd number of groups, a last stage of one group, k that is no multiple of 32 (int8), 8 splits of a long k
          (16, 4128, 1100), (9, 4000, 1100), (12, 8192, 516), (7, 2080, 2052), (16, 4096, 1026), (13, 1000, 4400)]


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,k,n", ROWS16)
def test_matmul_five_to_sixteen_rows(dev, m, k, n, bits):
    if bits == 4 and k % 32:
        k = (k // 32) * 32
    x = oracle.synth_normal(17, 0x32000000 + m * 31 + k, (m, k), 1.0)
    x[:, ::5] = 0.0
    w = oracle.synth_normal(17, k * 65537 + n, (k, n))
    if bits == 8:
        q, s = oracle.quantize_int8(w)
        qw, want = nn.QWeight.int8(dev, q, s), oracle.matmul_int8(x, q, s)
    else:
        q, s = oracle.quantize_int4(w, 32)
        qw, want = nn.QWeight.int4(dev, q, s, 32), oracle.matmul_int4(x, q, s)
    bias = oracle.synth_normal(17, 98, (n,))
    _, y = run_matmul(dev, x, qw, "f32", bias)
    want = want + bias
    # the activations ride as two bf16 pieces (16 significant bits): the stated tolerance of quantized-Linear outputs,
    # and all but a sliver inside the 1e-4 of tests/devices.rs
    err = np.abs(want.astype(np.float64) - y).max()
    assert err <= 1e-2 and err <= 1e-3 * np.abs(want).max(), (err, np.abs(want).max())
    loose = ~(np.abs(want - y) <= 1e-4 * (1 + np.abs(want)))
    assert loose.mean() <= 1e-4, f"{loose.sum()} of {loose.size} outputs beyond the tests/devices.rs tolerance"
    for dtype in ("f16", "bf16"):
        xf, yh = run_matmul(dev, x, qw, dtype, bias)
        ref = oracle.matmul_int8(xf, q, s) if bits == 8 else oracle.matmul_int4(xf, q, s)
        same(round_to(ref + bias, dtype), yh, TOL[dtype])


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m", [1, 3, 9])
def test_fixed_split_counts_give_the_same_product(dev, bits, m):
    """ruai_ctx_force_splits: the product does not depend on how many CTAs share k beyond the order of a few f32 additions
    (more splits than stages of k leave some CTAs of the cluster without work)."""
    k, n = 2048, 2304
    x = oracle.synth_normal(19, m, (m, k), 1.0)
    w = oracle.synth_normal(19, 2, (k, n))
    if bits == 8:
        q, s = oracle.quantize_int8(w)
        qw, want = nn.QWeight.int8(dev, q, s), oracle.matmul_int8(x, q, s)
    else:
        q, s = oracle.quantize_int4(w, 32)
        qw, want = nn.QWeight.int4(dev, q, s, 32), oracle.matmul_int4(x, q, s)
    try:
        for splits in (0, 1, 2, 4, 8):
            dev.force_splits(splits)
            _, y = run_matmul(dev, x, qw, "f32")
            same(want, y, 1e-4 if m < 5 else 3e-4)
        with pytest.raises(Exception):
            dev.force_splits(9)
    finally:
        dev.force_splits(0)


@pytest.mark.slow
@pytest.mark.parametrize("m", [17, 64])
def test_matmul_head_width_int8(dev, m):
    """The 8B head [4096 -> 128256], int8 as the reference keeps it, at more than 16 rows (the GEMM path)."""
    k, n = 4096, 128256
    x = oracle.synth_normal(15, m, (m, k), 1.0)
    q, s = oracle.quantize_int8(oracle.synth_normal(15, 3, (k, n)))
    want = oracle.matmul_int8(x, q, s)
    _, y = run_matmul(dev, x, nn.QWeight.int8(dev, q, s), "f32")
    err = np.abs(want.astype(np.float64) - y).max()
    assert err <= 1e-2 and err <= 1e-3 * np.abs(want).max(), (err, np.abs(want).max())


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m", [1, 2, 5, 16, 40])
def test_matmul_non_finite_activations_propagate(dev, bits, m):
    """A NaN or an infinity in a row of x makes that row of the product non-finite, as f32 arithmetic on the CPU does
    (cpu.rs:1002-1029, 1035-1067); the other rows are unaffected."""
    k, n = 4096, 1024
    x = oracle.synth_normal(14, m, (m, k), 1.0)
    w = oracle.synth_normal(14, 2, (k, n))
    if bits == 8:
        q, s = oracle.quantize_int8(w)
        qw, f = nn.QWeight.int8(dev, q, s), oracle.matmul_int8
    else:
        q, s = oracle.quantize_int4(w, 32)
        qw, f = nn.QWeight.int4(dev, q, s, 32), oracle.matmul_int4
    want = f(x, q, s)
    for bad in (np.nan, np.inf, -np.inf):
        xb = x.copy()
        xb[0, 1234] = bad
        _, y = run_matmul(dev, xb, qw, "f32")
        assert not np.isfinite(y[0]).any(), bad
        if m > 1:  # (five rows and more: activations as two bf16 pieces, see test_matmul_five_to_sixteen_rows)
            same(want[1:], y[1:], 1e-4 if m < 5 else 3e-4)


@pytest.mark.parametrize("bits", [8, 4])
def test_matmul_bf16_activations(dev, bits):
    m, k, n = 16, 1536, 1536
    x = oracle.synth_normal(12, 1, (m, k), 1.0)
    w = oracle.synth_normal(12, 2, (k, n))
    if bits == 8:
        q, s = oracle.quantize_int8(w)
        qw, f = nn.QWeight.int8(dev, q, s), oracle.matmul_int8
    else:
        q, s = oracle.quantize_int4(w, 32)
        qw, f = nn.QWeight.int4(dev, q, s, 32), oracle.matmul_int4
    xf, y = run_matmul(dev, x, qw, "bf16")
    same(bf16_round(f(xf, q, s))[1], y, 3e-2)


def test_linearity_and_determinism(dev):
    """Size-independent properties at a full-size shape: y(a*x1 + x2) = a*y(x1) + y(x2); repeat calls are bit identical."""
    k, n = 4096, 14336
    w = oracle.synth_normal(13, 5, (k, n))
    lin = nn.Linear(dev, w)
    lin.quantize_int4(32)
    x1 = oracle.synth_normal(13, 6, (1, k), 1.0)
    x2 = oracle.synth_normal(13, 7, (1, k), 1.0)
    y1 = lin.forward(nn.Tensor.from_numpy(dev, x1)).numpy()
    y2 = lin.forward(nn.Tensor.from_numpy(dev, x2)).numpy()
    y3 = lin.forward(nn.Tensor.from_numpy(dev, 2.0 * x1 + x2)).numpy()
    assert np.abs(y3 - (2.0 * y1 + y2)).max() < 1e-3 * np.abs(y3).max()
    again = lin.forward(nn.Tensor.from_numpy(dev, x1)).numpy()
    assert np.array_equal(again, y1)
    q, s = lin.int4
    same(oracle.matmul_int4(x1, q, s), y1, 1e-4)


# ---- training-side ops on the packed weights: input gradient and LoRA forward (layers.rs:169-190, ops.rs:705-734) ----

def _qw(dev, bits, k, n, seed, group=32):
    w = oracle.synth_normal(seed, k * 65537 + n, (k, n))
    if bits == 8:
        q, s = oracle.quantize_int8(w)
        return q, s, nn.QWeight.int8(dev, q, s)
    q, s = oracle.quantize_int4(w, group)
    return q, s, nn.QWeight.int4(dev, q, s, group)


@pytest.mark.parametrize("bits,group", [(8, 32), (4, 32), (4, 16)])
@pytest.mark.parametrize("m,k,n", [(1, 64, 48), (3, 576, 1536), (5, 4096, 1024), (2, 96, 130)])
def test_grad_input_matches_checker_and_is_the_adjoint(dev, m, k, n, bits, group):
    q, s, qw = _qw(dev, bits, k, n, 21, group)
    g = oracle.synth_normal(21, 7, (m, n), 1.0)
    want = oracle.matmul_q_grad_input(bits, g, q, s, group)
    got = nn.matmul_q_grad_input(nn.Tensor.from_numpy(dev, g), qw).numpy()
    same(want, got, 1e-4)
    # adjoint identity with the forward op of this library: <g, x @ W> == <g @ W^T, x>
    x = oracle.synth_normal(21, 8, (m, k), 1.0)
    y = nn._matmul_q(nn.Tensor.from_numpy(dev, x), qw).numpy().astype(np.float64)
    lhs, rhs = float((g * y).sum()), float((got.astype(np.float64) * x).sum())
    assert abs(lhs - rhs) <= 2e-4 * max(abs(lhs), np.abs(g).sum() * 1e-3)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,k,n,rank", [(1, 64, 48, 4), (4, 576, 1536, 8), (2, 4096, 1024, 16), (3, 96, 130, 3)])
def test_lora_forward_matches_checker(dev, m, k, n, rank, bits):
    q, s, qw = _qw(dev, bits, k, n, 22)
    x = oracle.synth_normal(22, 1, (m, k), 1.0)
    a = oracle.synth_normal(22, 2, (k, rank), 1.0 / np.sqrt(k))
    b = oracle.synth_normal(22, 3, (rank, n), 0.05)
    bias = oracle.synth_normal(22, 4, (n,))
    scale = 16.0 / rank
    T = lambda v: nn.Tensor.from_numpy(dev, v)
    for bb in (None, bias):
        want = oracle.linear_lora_forward(bits, x, q, s, a, b, scale, bb)
        got = nn.linear_lora_forward(T(x), qw, T(a), T(b), scale, None if bb is None else T(bb)).numpy()
        same(want, got, 1e-4)
    # B = 0 (a fresh adapter, layers.rs:93): the output is the base layer's
    zero = np.zeros((rank, n), np.float32)
    got = nn.linear_lora_forward(T(x), qw, T(a), T(zero), scale).numpy()
    assert np.array_equal(got, nn._matmul_q(T(x), qw).numpy())
