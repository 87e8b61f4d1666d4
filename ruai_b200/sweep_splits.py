"""Compares the split-k cost model of the tensor-core GEMVs with every fixed split, shape by shape.

    python -m ruai_b200.sweep_splits [rows ...]          (default rows: 1 4; needs a B200)

Per shape and row count: `ruai_matmul_q` timed with CUDA events over copies of the weight that together exceed the L2
(so every launch streams from HBM), six rounds, once with the library's choice and once each with 1, 2, 4 and 8 splits
fixed through `ruai_ctx_force_splits`.  Prints microseconds per launch and the ratio choice / best.  The int8 kernel
only lets the count be raised above its own choice, so its fixed columns mostly repeat the choice.
"""
import sys

import numpy as np

from . import nn

SHAPES = [(576, 576), (576, 1536), (576, 3072), (1536, 576), (768, 768), (768, 2304), (768, 3072), (3072, 768), (2048, 2048), (2048, 2560),
          (2048, 11264), (5632, 2048), (4096, 4096), (4096, 6144), (4096, 28672), (14336, 4096), (1024, 4096), (8192, 1024), (4096, 1000)]


def main(rows):
    dev = nn.Device.cuda(0)
    rng = np.random.default_rng(0)

    def make(k, n, bits):
        if bits == 4:
            q = rng.integers(-128, 128, (k // 2, n), dtype=np.int8)
            return nn.QWeight.int4(dev, q, np.ones((k // 32, n), np.float32), 32), k * n // 2 + k * n // 8
        q = rng.integers(-127, 128, (k, n), dtype=np.int8)
        return nn.QWeight.int8(dev, q, np.ones(n, np.float32)), k * n + 4 * n

    print("bits rows k n | choice us | fixed 1 2 4 8 us | choice / best")
    worst = {}
    for bits in (4, 8):
        for m in rows:
            for k, n in SHAPES:
                w0, nbytes = make(k, n, bits)
                copies = max(2, min(24, int(300e6 // nbytes) + 1))
                ws = [w0] + [make(k, n, bits)[0] for _ in range(copies - 1)]
                x = nn.Tensor.from_numpy(dev, rng.standard_normal((m, k)).astype(np.float32))
                out = nn.Tensor(dev, (m, n), np.float32, nn.F32)

                def timed(splits):
                    dev.force_splits(splits)
                    for w in ws:
                        dev.check(dev.L.ruai_matmul_q(dev.ctx, nn.F32, x.ptr, w.h, None, out.ptr, m))
                    dev.synchronize()
                    dev.timer_start()
                    for _ in range(6):
                        for w in ws:
                            dev.check(dev.L.ruai_matmul_q(dev.ctx, nn.F32, x.ptr, w.h, None, out.ptr, m))
                    return 1000 * dev.timer_stop_ms() / (6 * len(ws))

                choice = timed(0)
                fixed = [timed(f) for f in (1, 2, 4, 8)]
                dev.force_splits(0)
                ratio = choice / min(fixed)
                worst[(bits, m)] = max(worst.get((bits, m), 0.0), ratio)
                print(f"int{bits} {m:2d} {k:5d} {n:5d} | {choice:6.2f} | " + " ".join(f"{f:6.2f}" for f in fixed) + f" | {ratio:.2f}", flush=True)
                for w in ws:
                    w.free()
    print("worst choice / best per (bits, rows):", {k: round(v, 2) for k, v in worst.items()})


if __name__ == "__main__":
    main([int(a) for a in sys.argv[1:]] or [1, 4])
