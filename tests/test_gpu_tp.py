"""Tensor parallelism on the GPU.  The one-GPU cases run the row-sharded path with a group of one (no exchange,
but the supplied-statistics prologue, the raw-accumulator epilogue and the finalize kernel); the multi-GPU case
needs at least two GPUs and runs one process per GPU against the unsharded CPU oracle."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from loom_b200 import cabi
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("rows,K,batch,with_inner", [(96, 256, 1, True), (2560, 6912, 1, False), (130, 1040, 8, True)])
def test_rowsharded_linear_group_of_one(rows, K, batch, with_inner):
    ctx = cabi.Context(0)
    ctx.tp_init(0, 1, bytes(128))
    assert ctx.tp_world == 1 and ctx.tp_rank == 0
    rng = np.random.default_rng(rows + K)
    words, scale = orc.pack_f32((rng.standard_normal(rows * K) * 0.05).astype(np.float32), rows, K)
    inner = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32) if with_inner else None
    bias = (0.01 * rng.standard_normal(rows)).astype(np.float32)
    x = rng.standard_normal((batch, K)).astype(np.float32)
    w = ctx.upload_ternary(words, rows, K, scale)
    d_x, d_b = ctx.to_device(x), ctx.to_device(bias)
    d_in = ctx.to_device(inner) if with_inner else None
    d_out = ctx.alloc(batch * rows * 4)
    ctx.tp_rowsharded_linear(w, batch, d_x, K, d_out, inner_w=d_in, inner_w_len=K if with_inner else 0, eps=0.0, bias=d_b)
    got = ctx.download(d_out, (batch, rows), np.float32)
    for t in range(batch):
        xq, amax = orc.quantize_f32(orc.inner_rmsnorm_f32(x[t], inner, 0.0))
        acc = orc.matvec_i32(words, rows, K, xq).astype(np.float64)
        want = (acc * float(np.float64(scale) * np.float64(amax) / 127.0) + bias.astype(np.float64)).astype(np.float32)
        assert np.array_equal(got[t], want)
    with pytest.raises(cabi.LoomB200Error):
        ctx.tp_rowsharded_linear(w, 9, d_x, K, d_out)  # more tokens than one pass carries
    with pytest.raises(cabi.LoomB200Error):
        ctx.tp_rowsharded_linear(w, 1, d_x, K - 16, d_out)  # whole vector narrower than the slice
    ctx.close()


def test_decoder_refuses_dimensions_that_do_not_divide():
    # a group of one accepts everything; the divisibility rule itself is covered on the CPU by the shard plan
    ctx = cabi.Context(0)
    dec = cabi.Decoder(ctx, 1, 64, 4, 1, 16, 96, 50, 1e-5, 10000.0)
    dec.close()
    ctx.close()


@pytest.mark.parametrize("mode", ["nograph", "graph", "peer", "peer3"])
def test_two_ranks_match_unsharded_oracle(mode):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ)
    env.update(OMP_NUM_THREADS="4", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(HERE, "tp_gpu_worker.py"), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
