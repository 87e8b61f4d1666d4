"""Tensor-parallel parity on 2 GPUs (skipped on a single-GPU box): the sharded model generates the same
greedy tokens as the CPU checker, and every rank agrees.  Ranks are child processes, one GPU each."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

import oracle
from ruai_b200 import _lib

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("bits", [8, 4])
def test_two_rank_generate_matches_the_checker(bits):
    if _lib.load().ruai_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    with tempfile.TemporaryDirectory() as d:
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), str(world), d, str(bits)], env=env)
                 for r in range(world)]
        try:
            for p in procs:
                assert p.wait(timeout=300) == 0
        finally:
            for p in procs:
                if p.poll() is None:
                    p.kill()
        outs = [np.load(os.path.join(d, f"out{r}.npz")) for r in range(world)]
    assert np.array_equal(outs[0]["ids"], outs[1]["ids"]) and np.array_equal(outs[0]["steps"], outs[1]["steps"])
    cfg = oracle.LlamaConfig(1024, 512, 1536, 3, 8, 4, 64, 256, 1e-5, 10000.0, 0)
    om = oracle.Model(cfg, seed=3, bits=bits, group=32)
    prompt = np.array([(i * 37 + 11) % 1024 for i in range(12)], np.int32)
    want = om.generate(prompt, 24)
    assert outs[0]["ids"].tolist() == want.tolist()
    B = 4
    om.cache_clear()
    prompts = np.stack([(prompt + b) % 1024 for b in range(B)]).astype(np.int32)
    om.forward_cached(prompts)
    nxt = want[12:12 + B].astype(np.int32)
    for s in range(4):
        lo = om.forward_cached(nxt[:, None])
        nxt = np.array([oracle.argmax(r) for r in lo], np.int32)
        assert outs[0]["steps"][s].tolist() == nxt.tolist(), f"step {s}"


def test_a_rank_that_skips_a_step_times_the_peer_out_and_both_recover():
    """Failure detection without a GPU fault: rank 1 leaves out one decode step, rank 0's bounded waits for it run out
    and its call returns RUAI_ERR_TIMEOUT; after ruai_tp_resync on both ranks the sharded model generates the checker's
    tokens again.  Plain peer loads and stores only (no NCCL, no multicast); the waits are shortened through
    ruai_ctx_set_wait_limit."""
    if _lib.load().ruai_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world, bits = 2, 8
    with tempfile.TemporaryDirectory() as d:
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), str(world), d, str(bits), "peer_skips_a_step"], env=env)
                 for r in range(world)]
        try:
            for p in procs:
                assert p.wait(timeout=300) == 0
        finally:
            for p in procs:
                if p.poll() is None:
                    p.kill()
        outs = [np.load(os.path.join(d, f"out{r}.npz")) for r in range(world)]
    assert str(outs[0]["outcome"]) == "timeout", outs[0]["outcome"]
    assert str(outs[1]["outcome"]) == "ok"
    cfg = oracle.LlamaConfig(1024, 512, 1536, 3, 8, 4, 64, 256, 1e-5, 10000.0, 0)
    om = oracle.Model(cfg, seed=3, bits=bits, group=32)
    prompt = np.array([(i * 37 + 11) % 1024 for i in range(12)], np.int32)
    want = om.generate(prompt, 24)
    assert outs[0]["ids"].tolist() == want.tolist() and outs[1]["ids"].tolist() == want.tolist()


def test_vocabulary_parallel_argmax_tie_goes_to_the_larger_index():
    """Two identical head columns, one in each rank's half of the vocabulary (17 and 900): the exchanged pick is the
    last maximum globally (generation.rs:6-8), for one and for several sequences, on both ranks."""
    if _lib.load().ruai_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    with tempfile.TemporaryDirectory() as d:
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), str(world), d, "8", "argmax_tie"], env=env)
                 for r in range(world)]
        try:
            for p in procs:
                assert p.wait(timeout=300) == 0
        finally:
            for p in procs:
                if p.poll() is None:
                    p.kill()
        outs = [np.load(os.path.join(d, f"out{r}.npz")) for r in range(world)]
    for o in outs:
        # the largest logit is shared by the two columns, or (if negative) by all the zero columns: the last of them wins
        assert set(o["ids"].tolist()) <= {900, 1023} and len(set(o["ids"].tolist())) == 1, o["ids"]
    assert outs[0]["ids"].tolist() == outs[1]["ids"].tolist()
