"""Child process of tests/test_gpu_tp.py: one tensor-parallel rank on its own GPU.

usage: python tests/tp_worker.py RANK WORLD DIR BITS
Builds the sharded model, exchanges the IPC handles through files in DIR, generates greedily and writes the ids.
"""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def barrier(d, rank, world, name):
    """All ranks have reached `name` (files in DIR)."""
    open(os.path.join(d, f"{name}.{rank}"), "w").close()
    t0 = time.time()
    while not all(os.path.exists(os.path.join(d, f"{name}.{r}")) for r in range(world)):
        if time.time() - t0 > 120:
            raise SystemExit(f"rank {rank}: barrier {name} timed out")
        time.sleep(0.02)


def main():
    rank, world, d, bits = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], int(sys.argv[4])
    scenario = sys.argv[5] if len(sys.argv) > 5 else "generate"
    from ruai_b200 import nn
    dev = nn.Device.cuda(rank)
    if scenario == "peer_skips_a_step":
        dev.set_wait_limit(250000)  # about 0.1 s per wait for a peer instead of half a second; before the first step
    cfg = nn.LlamaConfig(1024, 512, 1536, 3, 8, 4, 64, 256, 1e-5, 10000.0, 0)
    m = nn.Llama(dev, cfg, nn.TP(rank, world))
    if scenario == "argmax_tie":
        # a head that is zero except for two identical columns, one in each rank's half of the vocabulary
        import oracle
        V, dm, ffn, L, H, KV, hd = 1024, 512, 1536, 3, 8, 4, 64
        shapes = {0: (dm, H * hd), 1: (dm, KV * hd), 2: (dm, KV * hd), 3: (H * hd, dm), 4: (dm, ffn), 5: (dm, ffn), 6: (ffn, dm)}
        for layer in range(L):
            for kind, shp in shapes.items():
                m.set_f32(layer * 16 + kind, oracle.synth_normal(7, layer * 16 + kind, shp))
            m.set_f32(0x50000000 + layer, np.ones(dm, np.float32))
            m.set_f32(0x52000000 + layer, np.ones(dm, np.float32))
        m.set_f32(0x10000000, oracle.synth_normal(7, 0x10000000, (V, dm)))
        head = np.zeros((dm, V), np.float32)
        head[:, 17] = head[:, 900] = oracle.synth_normal(7, 99, (dm,))
        m.set_f32(0x10000001, head)
        m.set_f32(0x40000000, np.ones(dm, np.float32))
        m.quantize_int8()
    else:
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
    if scenario == "argmax_tie":
        picks = []
        for B in (1, 3):
            m.cache_clear()
            t = nn.Tensor.from_numpy(dev, np.full(B, 5, np.int32))
            picks.append(m.decode_step(B, t.ptr).tolist())
        np.savez(os.path.join(d, f"out{rank}.npz"), ids=np.array(sum(picks, []), np.int32), steps=np.zeros((1, 1), np.int32))
        return
    if scenario == "peer_skips_a_step":
        # Failure made on the host: rank 1 leaves out one step (between steps, nothing of its own in flight).  Rank 0's
        # waits for the peer run out, its call reports RUAI_ERR_TIMEOUT, nothing hangs.  Then both resynchronise.
        barrier(d, rank, world, "start")  # the ranks begin within the (shortened) wait of each other
        m.forward_cached(prompt[None, :], want_logits=False)
        tok = nn.Tensor.from_numpy(dev, np.array([5], np.int32))
        m.decode_step(1, tok.ptr)
        barrier(d, rank, world, "before")
        outcome = "ok"
        if rank == 0:
            try:
                m.decode_step(1, None)
            except nn.RuaiError as e:
                outcome = "timeout" if e.code == 4 and "timed out" in str(e) else f"other: {e}"
        barrier(d, rank, world, "after")
        m.tp_resync()
        barrier(d, rank, world, "resynced")
        m.cache_clear()
        ids = m.generate(prompt, 24)
        np.savez(os.path.join(d, f"out{rank}.npz"), ids=ids, steps=np.zeros((1, 1), np.int32), outcome=np.array(outcome))
        return
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
