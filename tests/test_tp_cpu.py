"""CPU tests (gloo, world_size 2) of the tensor-parallel plan: column-split q/k/v/gate/up/head, row-split o/down with
int4 groups kept whole, one sum exchange per row-split Linear, (value, index) exchange for the split argmax.
Each rank computes its shard with the CPU checker on slices of the full quantized buffers; the summed result must
equal the unsharded computation.  This is the arithmetic model.cu and tp.cu implement on the device."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, bits, out):
    sys.path.insert(0, ROOT)
    import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    d, ffn, V, g = 128, 256, 96, 32
    x = oracle.synth_normal(5, 1, (3, d), 1.0)
    w_up, w_down, w_head = oracle.synth_normal(5, 2, (d, ffn)), oracle.synth_normal(5, 3, (ffn, d)), oracle.synth_normal(5, 4, (d, V))
    quant = (lambda w: oracle.quantize_int8(w)) if bits == 8 else (lambda w: oracle.quantize_int4(w, g))
    mm = oracle.matmul_int8 if bits == 8 else oracle.matmul_int4
    (qu, su), (qd, sd) = quant(w_up), quant(w_down)
    fl = ffn // world
    cols = slice(rank * fl, (rank + 1) * fl)
    # column split: slice columns of q and of the scales
    h_local = mm(x, np.ascontiguousarray(qu[:, cols]), np.ascontiguousarray(su[..., cols]))
    # row split: rows of q; int8 scales replicated, int4 scale rows follow the groups
    if bits == 8:
        part = mm(h_local, np.ascontiguousarray(qd[cols, :]), sd)
    else:
        assert (rank * fl) % g == 0 and fl % g == 0
        part = mm(h_local, np.ascontiguousarray(qd[rank * fl // 2:(rank + 1) * fl // 2, :]), np.ascontiguousarray(sd[rank * fl // g:(rank + 1) * fl // g, :]))
    # sum exchange in rank order (what allreduce_push_kernel does)
    parts = [torch.zeros(part.shape, dtype=torch.float32) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(part))
    y = np.zeros_like(part)
    for p in parts:
        y = y + p.numpy()
    # vocabulary-parallel argmax with the last-maximum rule
    qh, sh = oracle.quantize_int8(w_head)
    Vl = V // world
    logits_local = oracle.matmul_int8(y, np.ascontiguousarray(qh[:, rank * Vl:(rank + 1) * Vl]), np.ascontiguousarray(sh[rank * Vl:(rank + 1) * Vl]))
    logits_local[:, -1] = logits_local[:, 0] = 7.0  # ties across and inside ranks
    mine = torch.tensor([[float(r[oracle.argmax(r)]), float(oracle.argmax(r) + rank * Vl)] for r in logits_local], dtype=torch.float64)
    allp = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(allp, mine)
    best = allp[0].clone()
    for p in allp[1:]:
        take = (p[:, 0] > best[:, 0]) | ((p[:, 0] == best[:, 0]) & (p[:, 1] > best[:, 1]))
        best[take] = p[take]
    if rank == 0:
        h_full = mm(x, qu, su)
        y_full = mm(h_full, qd, sd)
        logits = oracle.matmul_int8(y_full, qh, sh)
        np.savez(out, y=y, y_full=y_full, h_ok=np.allclose(h_full[:, cols], h_local, atol=0), idx=best[:, 1].numpy(), V=V, Vl=Vl)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("bits", [8, 4])
def test_sharded_linears_sum_to_the_unsharded_result(tmp_path, bits):
    world, port = 2, 29600 + bits + os.getpid() % 200
    out = str(tmp_path / "r0.npz")
    mp.spawn(_worker, args=(world, port, bits, out), nprocs=world, join=True)
    r = np.load(out)
    assert bool(r["h_ok"])  # a column shard is bit-identical to the same columns of the full result
    assert np.abs(r["y"] - r["y_full"]).max() <= 1e-4 * (1 + np.abs(r["y_full"]).max())
    # ties: every rank's slice has 7.0 at its first and last column; the global pick is the last column of the last rank
    assert r["idx"].tolist() == [int(r["V"]) - 1] * 3


# ---- the flag / parity protocol of the exchange, modelled on the host ------------------------------------------------

class _Rank:
    """What one rank's side of allreduce_push_kernel (tp.cu) does, step by step, on shared host arrays: slots and flags
    are double-buffered by the parity of a sequence number; a rank pushes its part into every peer's slot, releases
    the flag with the sequence number, and waits (bounded) for every peer's flag to reach the same number."""

    def __init__(self, rank, world, slots, flags, limit):
        self.rank, self.world, self.slots, self.flags, self.limit, self.seq = rank, world, slots, flags, limit, 0

    def exchange(self, part):
        import time
        seq = self.seq + 1
        par = seq & 1
        for p in range(self.world):
            if p != self.rank:
                self.slots[p][par][self.rank][:] = part
                self.flags[p][par][self.rank] = seq          # release after the data
        ok = True
        for p in range(self.world):
            if p == self.rank:
                continue
            t0 = time.time()
            while self.flags[self.rank][par][p] != seq:
                if time.time() - t0 > self.limit:
                    ok = False
                    break
                time.sleep(0.0005)
        self.seq = seq                                        # advances whether or not the wait ran out (as on the device)
        if not ok:
            return None
        total = np.zeros_like(part)
        for p in range(self.world):                           # rank order: identical bits everywhere
            total = total + (part if p == self.rank else self.slots[self.rank][par][p])
        return total

    def resync(self):
        self.seq = 0
        for par in range(2):
            self.flags[self.rank][par][:] = 0


def test_exchange_protocol_with_a_rank_that_never_posts():
    """Host model of the exchange: both ranks agree for several steps (the double buffering by parity holds when one
    rank runs a step ahead); a rank that leaves a step out makes the other's bounded wait run out (no result, no
    hang); the sequence numbers then disagree, so a later exchange fails as well until both sides resynchronise."""
    import threading
    world, n = 2, 64
    slots = [np.zeros((2, world, n), np.float32) for _ in range(world)]
    flags = [np.zeros((2, world), np.int64) for _ in range(world)]
    ranks = [_Rank(r, world, slots, flags, 0.2) for r in range(world)]
    parts = lambda step, r: np.full(n, 10.0 * step + r + 1, np.float32)

    def run(step, who):
        out = {}
        ts = [threading.Thread(target=lambda r=r: out.__setitem__(r, ranks[r].exchange(parts(step, r)))) for r in who]
        [t.start() for t in ts]
        [t.join() for t in ts]
        return out

    for step in range(5):
        out = run(step, (0, 1))
        want = parts(step, 0) + parts(step, 1)
        assert np.array_equal(out[0], want) and np.array_equal(out[1], want)
    out = run(5, (0,))                       # rank 1 leaves the step out
    assert out[0] is None                    # the wait ran out; nothing hung
    out = run(6, (0, 1))                     # sequence numbers differ by one now: rank 0 waits for 7, rank 1 posts 6
    assert out[0] is None
    # ... while rank 1 finds rank 0's flag of the step it missed and adds that step's stale part: after a time-out
    # anywhere, every rank has to stop and resynchronise (ruai_tp_resync) before the results mean anything again
    assert np.array_equal(out[1], parts(5, 0) + parts(6, 1))
    for r in ranks:
        r.resync()
    out = run(7, (0, 1))
    want = parts(7, 0) + parts(7, 1)
    assert np.array_equal(out[0], want) and np.array_equal(out[1], want)
