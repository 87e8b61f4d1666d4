"""Generates tests/golden/greedy_golden.npz: greedy tokens and logit samples of the FULL-DEPTH benchmark models.

Run on a CPU host:  python tests/golden/make_greedy_golden.py
For every (model shape, weight bits) below the CPU checker (oracle/, the restatement of the reference's CPU path)
builds the full model from the seeded synthetic weights, runs the prompt and 32 greedy tokens
(generation.rs:83-113) and stores: the ids, the top-2 margin of every step (so a reader can see how decisive
each pick is) and every 61st logit of every step.  The GPU tests and `bench.py` compare against this file, so
the full-depth check costs no CPU time where the GPU is.  Takes about 15 minutes on 8 cores.
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

SHAPES = {
    "tinyllama-1.1b": dict(V=32000, d=2048, ffn=5632, L=22, H=32, KV=4, hd=64, max_pos=2048, theta=10000.0),
    "llama3-8b": dict(V=128256, d=4096, ffn=14336, L=32, H=32, KV=8, hd=128, max_pos=2048, theta=500000.0),
}
PROMPT, NEW, STRIDE = 16, 32, 61


def main():
    out = {}
    for name, c in SHAPES.items():
        for bits in (4, 8):
            t0 = time.time()
            cfg = oracle.LlamaConfig(c["V"], c["d"], c["ffn"], c["L"], c["H"], c["KV"], c["hd"], c["max_pos"], 1e-5, c["theta"], 0)
            m = oracle.Model(cfg, seed=0, bits=bits, group=32)
            prompt = oracle.synth_tokens(0, 0x20000000, PROMPT, c["V"])
            ids, trace = m.generate(prompt, NEW, trace=True)
            srt = np.sort(trace, axis=1)
            key = f"{name}-int{bits}"
            out[key + "/ids"] = ids.astype(np.int32)
            out[key + "/margin"] = (srt[:, -1] - srt[:, -2]).astype(np.float32)
            out[key + "/logits"] = trace[:, ::STRIDE].astype(np.float32)
            out[key + "/absmax"] = np.abs(trace).max(axis=1).astype(np.float32)
            m.close()
            print(key, "done in %.0f s; min margin %.3e" % (time.time() - t0, out[key + "/margin"].min()), flush=True)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "greedy_golden.npz"), **out)


if __name__ == "__main__":
    main()
