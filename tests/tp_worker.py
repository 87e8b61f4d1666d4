"""Child process of tests/test_gpu_tp.py: one tensor-parallel rank on its own GPU.

usage: python tests/tp_worker.py RANK WORLD DIR BITS
Builds the sharded model, exchanges the IPC handles through files in DIR, generates greedily and writes the ids.
"""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, d, bits = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], int(sys.argv[4])
    from ruai_b200 import nn
    dev = nn.Device.cuda(rank)
    cfg = nn.LlamaConfig(1024, 512, 1536, 3, 8, 4, 64, 256, 1e-5, 10000.0, 0)
    m = nn.Llama(dev, cfg, nn.TP(rank, world))
    m.load_synthetic(3, bits, 32)
    with open(os.path.join(d, f"h{rank}.tmp"), "wb") as f:
        f.write(m.tp_export())
    os.rename(os.path.join(d, f"h{rank}.tmp"), os.path.join(d, f"h{rank}"))
    handles = []
    for r in range(world):
        p = os.path.join(d, f"h{r}")
        t0 = time.time()
        while not os.path.exists(p):
            if time.time() - t0 > 120:
                raise SystemExit(f"rank {rank}: no handle from rank {r}")
            time.sleep(0.05)
        handles.append(open(p, "rb").read())
    m.tp_connect(handles)
    prompt = np.array([(i * 37 + 11) % 1024 for i in range(12)], np.int32)
    ids = m.generate(prompt, 24)
    # batched device-resident steps as well
    B = 4
    m.cache_clear()
    prompts = np.stack([(prompt + b) % 1024 for b in range(B)]).astype(np.int32)
    m.forward_cached(prompts, want_logits=False)
    steps = []
    first = nn.Tensor.from_numpy(dev, ids[12:12 + B].astype(np.int32))
    nxt = m.decode_step(B, first.ptr)
    steps.append(nxt.copy())
    for _ in range(3):
        nxt = m.decode_step(B, None)
        steps.append(nxt.copy())
    np.savez(os.path.join(d, f"out{rank}.npz"), ids=ids, steps=np.stack(steps))


if __name__ == "__main__":
    main()
