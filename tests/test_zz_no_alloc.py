"""GPU test of ruai_matmul_q_static, the quantized matmul that allocates nothing.

It is for hosts that cannot let the library call cudaMalloc while serving (their framework already
owns the device memory, or they cannot afford the synchronisation an allocation implies).  The
entry point keeps its split-K scratch in a fixed array inside the library, so the test calls it
twice in a row on the same stream (the second call meets the first call's leftovers in that array)
and checks both results against ruai_matmul_q.  Runs last so that a failure here cannot hide others.
"""
import ctypes as C

import numpy as np
import pytest

import oracle
from ruai_b200 import nn

pytestmark = pytest.mark.gpu


def same(want, got, tol=1e-4):
    want, got = np.asarray(want, np.float64), np.asarray(got, np.float64)
    bad = ~((np.abs(want - got) <= tol * (1 + np.abs(want))) | (want == got))
    assert not bad.any(), f"{bad.sum()} of {bad.size} differ; worst {np.abs(want - got).max()}"


@pytest.mark.parametrize("bits", [4, 8])
def test_static_scratch_matmul_matches_the_allocating_one_twice_in_a_row(bits):
    assert nn.Device.is_available(), "this test needs a CUDA device"
    dev = nn.Device.cuda(0)
    k, n, m = 2048, 1536, 3  # small n: the work is split along k, so the scratch is really used
    w = oracle.synth_normal(21, 1, (k, n))
    if bits == 8:
        q, s = oracle.quantize_int8(w)
        qw = nn.QWeight.int8(dev, q, s)
    else:
        q, s = oracle.quantize_int4(w, 32)
        qw = nn.QWeight.int4(dev, q, s, 32)
    bias = nn.Tensor.from_numpy(dev, oracle.synth_normal(21, 2, (n,)))
    xs = [nn.Tensor.from_numpy(dev, oracle.synth_normal(21, 3 + i, (m, k), 1.0)) for i in range(2)]
    wants = [nn._matmul_q(x, qw, bias).numpy() for x in xs]
    outs = [nn.Tensor(dev, (m, n), np.float32, nn.F32) for _ in xs]
    for x, out in zip(xs, outs):  # two calls back to back, no synchronisation in between
        dev.check(dev.L.ruai_matmul_q_static(dev.ctx, nn.F32, x.ptr, qw.h, bias.ptr, out.ptr, m))
    dev.synchronize()
    for want, out in zip(wants, outs):
        same(want, out.numpy())
    # and the checker agrees with both
    f = oracle.matmul_int8 if bits == 8 else oracle.matmul_int4
    same(f(xs[1].numpy(), q, s) + bias.numpy(), outs[1].numpy())


def test_static_scratch_matmul_rejects_what_does_not_fit():
    dev = nn.Device.cuda(0)
    k, n, m = 1024, 8448, 64  # 4 splits x 64 rows x 8448 columns of f32 partials exceed the fixed 8 MiB
    rng = np.random.default_rng(0)
    qw = nn.QWeight.int8(dev, rng.integers(-127, 128, (k, n), dtype=np.int8), np.ones(n, np.float32))
    x = nn.Tensor(dev, (m, k), np.float32, nn.F32)
    out = nn.Tensor(dev, (m, n), np.float32, nn.F32)
    with pytest.raises(nn.RuaiError, match="fixed scratch holds"):
        dev.check(dev.L.ruai_matmul_q_static(dev.ctx, nn.F32, x.ptr, qw.h, None, out.ptr, m))
