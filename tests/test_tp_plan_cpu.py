"""The tensor-parallel shard plan on the CPU: slicing of packed words, and a two-rank gloo run in which each
rank computes its slices with the oracle's primitives, exchanges what the GPU path exchanges and must
reproduce the oracle's unsharded layers bit for bit."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from loom_b200.tp import ShardPlan, slice_cols, slice_rows
from refkit import np_pack, np_unpack

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_slices_of_packed_words():
    rng = np.random.default_rng(5)
    rows, cols = 24, 80
    q = rng.integers(-1, 2, (rows, cols)).astype(np.int8)
    words = np_pack(q, rows, cols)
    assert (np_unpack(slice_rows(words, rows, cols, 8, 16), 8, cols) == q[8:16]).all()
    assert (np_unpack(slice_cols(words, rows, cols, 32, 64), rows, 32) == q[:, 32:64]).all()
    assert (np_unpack(slice_cols(words, rows, cols, 64, 80), rows, 16) == q[:, 64:80]).all()
    with pytest.raises(ValueError):
        slice_cols(words, rows, cols, 8, 40)  # not on a word boundary
    with pytest.raises(ValueError):
        slice_rows(words, rows, cols, 16, 30)


def test_plan_bounds_and_errors():
    p = ShardPlan(4, 2, hidden=4096, heads=32, kv_heads=8, head_dim=128, inter=14336, vocab=128256)
    assert p.q_rows == (2048, 3072) and p.kv_rows == (512, 768) and p.inter_rows == (7168, 10752)
    assert p.vocab_rows == (64128, 96192)
    with pytest.raises(ValueError):
        ShardPlan(2, 0, hidden=2560, heads=20, kv_heads=5, head_dim=128, inter=6912, vocab=128256)  # 5 KV heads
    # a vocabulary that does not divide stays whole on every rank
    assert ShardPlan(8, 3, 8192, 64, 8, 128, 28672, 128257).vocab_rows == (0, 128257)


def test_block_slices_have_matching_shapes():
    rng = np.random.default_rng(9)
    H, heads, kvh, hd, I = 64, 4, 2, 16, 96
    qd, kvd = heads * hd, kvh * hd
    shapes = ((qd, H), (kvd, H), (kvd, H), (H, qd), (I, H), (I, H), (H, I))
    qs = [rng.integers(-1, 2, s).astype(np.int8) for s in shapes]
    words7 = [np_pack(q, *s) for q, s in zip(qs, shapes)]
    inner_a = rng.standard_normal(qd).astype(np.float32)
    inner_f = rng.standard_normal(40).astype(np.float32)  # shorter than the row: the tail counts as 1
    got_q, got_o = [], []
    for r in range(2):
        plan = ShardPlan(2, r, H, heads, kvh, hd, I, 100)
        slices, ia, fi = plan.shard_block(words7, inner_a, inner_f)
        assert [(s[1], s[2]) for s in slices] == [(qd // 2, H), (kvd // 2, H), (kvd // 2, H), (H, qd // 2), (I // 2, H),
                                                  (I // 2, H), (H, I // 2)]
        got_q.append(np_unpack(*slices[0]))
        got_o.append(np_unpack(*slices[3]))
        assert (ia == inner_a[r * qd // 2:(r + 1) * qd // 2]).all()
        if r == 0:
            assert (fi == inner_f).all()  # 40 of this rank's 48 entries
        else:
            assert fi is None
    assert (np.concatenate(got_q, 0) == qs[0]).all() and (np.concatenate(got_o, 1) == qs[3]).all()


@pytest.mark.parametrize("world", [2])
def test_sharded_layers_match_oracle_over_gloo(world):
    env = dict(os.environ)
    env.update(OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(HERE, "tp_cpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    for k in range(world):
        assert "rank %d ok" % k in r.stdout
