"""Generates tests/golden/quant_golden.npz.

The reference (Rust) cannot be run where this repository is built, so these
vectors do not come from running it.  They restate, in float64 numpy and
independently of oracle/ and of the CUDA library, the closed-form definitions
that the reference's own tests use as their expected values:

  * tests/quant.rs:39-53   int4: s = max|w| / 7 per (group, column),
                           w_hat = round(w / s).clamp(-8, 7) * s
  * tests/devices.rs:451-452  int8 pattern q[i] = (i*37 % 255) - 127,
                              s[j] = 0.001 + j*1e-5, shapes (1,64,300) (5,33,70) (40,32,48)
  * tests/devices.rs:486-487  int4 pattern q[i] = (i*73 % 256) as i8,
                              s[j] = 0.01 + (j % 13)*1e-3, shapes (1,64,300,32) (5,32,70,8) (40,64,48,16)
  * tests/llama.rs:34-43   rms_norm known values

Inputs x are drawn from numpy's PCG64 with a fixed seed and stored alongside
the expected outputs.  Run:  python tests/golden/make_golden.py
"""
import os

import numpy as np


def round_half_away(x64):
    return np.sign(x64) * np.floor(np.abs(x64) + 0.5)


def int4_value(q_bytes, l, j):
    # backend/mod.rs:98-102
    b = int(q_bytes[l // 2, j]) & 0xFF
    v = (b >> 4) if (l % 2 == 1) else (b & 0xF)
    return v - 16 if v >= 8 else v


def main():
    rng = np.random.Generator(np.random.PCG64(20240607))
    out = {}
    # --- int8 synthetic pattern, tests/devices.rs:444-463 ---
    for idx, (m, k, n) in enumerate([(1, 64, 300), (5, 33, 70), (40, 32, 48)]):
        q = np.array([((i * 37 % 255) - 127) for i in range(k * n)], dtype=np.int8).reshape(k, n)
        s = np.array([np.float32(0.001) + np.float32(j) * np.float32(1e-5) for j in range(n)], dtype=np.float32)
        x = rng.standard_normal((m, k)).astype(np.float32)
        y = (x.astype(np.float64) @ q.astype(np.float64)) * s.astype(np.float64)
        out[f"i8_{idx}_x"], out[f"i8_{idx}_q"], out[f"i8_{idx}_s"], out[f"i8_{idx}_y"] = x, q, s, y
    # --- int4 synthetic pattern, tests/devices.rs:479-500 ---
    for idx, (m, k, n, g) in enumerate([(1, 64, 300, 32), (5, 32, 70, 8), (40, 64, 48, 16)]):
        q = np.array([(i * 73 % 256) for i in range(k // 2 * n)], dtype=np.uint8).astype(np.int8).reshape(k // 2, n)
        s = np.array([np.float32(0.01) + np.float32(j % 13) * np.float32(1e-3) for j in range(k // g * n)],
                     dtype=np.float32).reshape(k // g, n)
        x = rng.standard_normal((m, k)).astype(np.float32)
        vals = np.array([[int4_value(q, l, j) for j in range(n)] for l in range(k)], dtype=np.float64)
        # dequant is exact in f32: a 4-bit integer times an f32 scale, rounded once
        w = (vals.astype(np.float32) * np.repeat(s, g, axis=0)).astype(np.float32)
        y = x.astype(np.float64) @ (vals * np.repeat(s, g, axis=0).astype(np.float64))
        out[f"i4_{idx}_x"], out[f"i4_{idx}_q"], out[f"i4_{idx}_s"] = x, q, s
        out[f"i4_{idx}_w"], out[f"i4_{idx}_y"], out[f"i4_{idx}_g"] = w, y, np.int32(g)
    # --- int4 quantizer definition, tests/quant.rs:29-53 (k=8, n=3, group=4) and a group-32 case ---
    for tag, (k, n, g) in {"qa": (8, 3, 4), "qb": (64, 20, 32)}.items():
        w = (rng.standard_normal((k, n)) * 0.35).astype(np.float32)
        if tag == "qb":
            w[:32, 5] = 0.0  # an all-zero group: scale must be 1.0 (layers.rs:154)
        want = np.zeros((k, n), np.float32)
        scales = np.zeros((k // g, n), np.float32)
        vals = np.zeros((k, n), np.int8)
        for j in range(n):
            for gi in range(k // g):
                rows = slice(gi * g, (gi + 1) * g)
                mx = np.float32(np.max(np.abs(w[rows, j])))
                s = np.float32(mx / np.float32(7.0)) if mx > 0 else np.float32(1.0)
                scales[gi, j] = s
                r = round_half_away((w[rows, j] / s).astype(np.float32).astype(np.float64))
                r = np.clip(r, -8, 7)
                vals[rows, j] = r.astype(np.int8)
                want[rows, j] = (r.astype(np.float32) * s).astype(np.float32)
        packed = ((vals[0::2].astype(np.uint8) & 0xF) | ((vals[1::2].astype(np.uint8) & 0xF) << 4)).astype(np.int8)
        out[f"{tag}_w"], out[f"{tag}_want"], out[f"{tag}_scale"], out[f"{tag}_packed"], out[f"{tag}_g"] = \
            w, want, scales, packed, np.int32(g)
    # --- int8 quantizer definition, layers.rs:112-129 ---
    k, n = 48, 17
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    w[:, 3] = 0.0
    mx = np.max(np.abs(w), axis=0).astype(np.float32)
    s = np.where(mx > 0, (mx / np.float32(127.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    r = round_half_away((w / s[None, :]).astype(np.float32).astype(np.float64))
    out["q8_w"], out["q8_scale"], out["q8_q"] = w, s, np.clip(r, -127, 127).astype(np.int8)
    # --- rms_norm known values, tests/llama.rs:34-43 ---
    x = np.array([[1., 2., 3., 4.], [-2., 0., 2., 0.]], np.float32)
    wn = np.array([1., 2., 1., 0.5], np.float32)
    r0, r1 = np.sqrt(np.float32(30.0) / np.float32(4.0)), np.sqrt(np.float32(2.0))
    out["rms_x"], out["rms_w"] = x, wn
    out["rms_want"] = np.array([[1. / r0, 4. / r0, 3. / r0, 2. / r0], [-2. / r1, 0., 2. / r1, 0.]], np.float32)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
