"""One rank of the tensor-parallel GPU check.  Run by test_gpu_tp.py under torch.distributed.run (one process per
GPU), and called by bench.py on every rank before it times a multi-GPU run.  Every rank builds the same weights,
keeps only its slices on its GPU, and must end with the logits and greedy tokens of the CPU oracle's UNSHARDED
decoder.  A gloo (CPU) group carries the NCCL unique id and the mailbox handles."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from loom_b200 import cabi  # noqa: E402
from loom_b200.tp import ShardPlan, slice_cols  # noqa: E402
from oracle import oracle as orc  # noqa: E402


def share_unique_id(rank: int, group=None) -> bytes:
    t = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        t = torch.frombuffer(bytearray(cabi.Context.tp_unique_id()), dtype=torch.uint8).clone()
    dist.broadcast(t, 0, group=group)
    return bytes(t.numpy().tobytes())


def run_checks(mode: str, local: int, group=None):
    """The whole check on this rank: (failures, microseconds per sharded decode token).  `group` is a gloo group over
    all ranks (None = the default group, which must then be gloo).  Collective: every rank calls it."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ctx = cabi.Context(device=local)
    ctx.tp_init(rank, world, share_unique_id(rank, group))
    assert ctx.tp_rank == rank and ctx.tp_world == world
    if mode == "nograph":
        ctx.set_option("tp_graph", 0)
    if mode == "peer3":  # the three-launch form of a row-parallel projection (statistics kernel, GEMV, finalize kernel)
        ctx.set_option("tp_fused", 0)
    if mode in ("peer", "peer3"):  # exchange through peer mailboxes instead of NCCL: gather every rank's IPC handle
        mine = torch.frombuffer(bytearray(ctx.tp_peer_handle()), dtype=torch.uint8).clone()
        allh = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(allh, mine, group=group)
        ctx.tp_attach_peers(b"".join(bytes(t.numpy().tobytes()) for t in allh))
    failures = []

    # ---- the exact int32 sum ----
    n = 5000
    host = (np.arange(n, dtype=np.int32) * (rank + 1)) - 7
    buf = ctx.to_device(host)
    ctx.tp_allreduce_i32(buf, n)
    got = ctx.download(buf, (n,), np.int32)
    want = np.arange(n, dtype=np.int64) * (world * (world + 1) // 2) - 7 * world
    if not np.array_equal(got.astype(np.int64), want):
        failures.append("allreduce_i32 wrong")
    ctx.free(buf)

    # ---- a row-sharded linear with inner-norm weights, bias and residual ----
    rng = np.random.default_rng(77)
    for rows, K, batch in ((96, 256 * world, 3), (200, 512 * world, 1), (96, 256 * world, 8)):
        master = (rng.standard_normal(rows * K) * 0.05).astype(np.float32)
        words, scale = orc.pack_f32(master, rows, K)
        inner = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
        bias = (0.01 * rng.standard_normal(rows)).astype(np.float32)
        resid = rng.standard_normal((batch, rows)).astype(np.float32)
        x = rng.standard_normal((batch, K)).astype(np.float32)
        c0, c1 = rank * K // world, (rank + 1) * K // world
        w_l = ctx.upload_ternary(slice_cols(words, rows, K, c0, c1), rows, c1 - c0, scale)
        d_x = ctx.to_device(np.ascontiguousarray(x[:, c0:c1]))
        d_in, d_b, d_r = ctx.to_device(np.ascontiguousarray(inner[c0:c1])), ctx.to_device(bias), ctx.to_device(resid)
        d_out = ctx.alloc(batch * rows * 4)
        for rep in range(3):  # repeated: the mailbox halves and sequence numbers must keep working
            ctx.tp_rowsharded_linear(w_l, batch, d_x, K, d_out, inner_w=d_in, inner_w_len=c1 - c0, eps=1e-5, bias=d_b, residual=d_r)
        got = ctx.download(d_out, (batch, rows), np.float32)
        for t in range(batch):
            y = orc.inner_rmsnorm_f32(x[t], inner, 1e-5)
            xq, amax = orc.quantize_f32(y)
            acc = orc.matvec_i32(words, rows, K, xq).astype(np.float64)
            os_ = float(np.float64(scale) * np.float64(amax) / 127.0)
            want = (acc * os_ + bias.astype(np.float64)).astype(np.float32) + resid[t]
            if not np.array_equal(got[t], want):
                failures.append("row-sharded linear %dx%d batch %d token %d differs in %d of %d" % (rows, K, batch, t, int((got[t] != want).sum()), rows))

    # ---- the decoder: logits and greedy tokens of the unsharded oracle ----
    L, H, heads, kvh, hd, I, V, msl = 2, 512, 8, 8, 64, 1024, 512, 96  # 8 heads / 8 KV heads: any group of up to 8 ranks divides them
    eps, theta, act = 1e-5, 500000.0, cabi.ACT_SILU
    plan = ShardPlan(world, rank, H, heads, kvh, hd, I, V)
    odec = orc.Decoder(L, H, heads, kvh, hd, I, V, eps, theta, act, msl)
    gdec = cabi.Decoder(ctx, L, H, heads, kvh, hd, I, V, eps, theta, act, msl)
    shapes = ((heads * hd, H), (kvh * hd, H), (kvh * hd, H), (H, heads * hd), (I, H), (I, H), (H, I))
    blocks = []
    for b in range(L):
        masters = [(rng.standard_normal(r * c) * 0.02).astype(np.float32) for r, c in shapes]
        g1 = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        g2 = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        odec.set_block(b, *masters, g1=g1, g2=g2)
        packed = [orc.pack_f32(m, r, c) for m, (r, c) in zip(masters, shapes)]
        slices, _, _ = plan.shard_block([p[0] for p in packed])
        ws = [ctx.upload_ternary(sw, sr, sc, packed[i][1]) for i, (sw, sr, sc) in enumerate(slices)]
        gdec.set_block(b, ws, g1=g1, g2=g2)
        blocks.append((masters, ws, g1, g2))
    emb = (rng.standard_normal((V, H)) * 0.02).astype(np.float32)
    fg = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    emb_dev = ctx.to_device(emb)
    odec.set_embeddings(emb, fg)
    gdec.set_embeddings(emb_dev, fg)
    prompt = rng.integers(0, V, 13).astype(np.int32)
    elog = odec.forward(prompt)
    glog = gdec.forward(prompt)
    tol = 1e-5 * max(1.0, float(np.max(np.abs(elog))))
    if not np.max(np.abs(glog - elog)) <= tol:
        failures.append("prompt logits differ by %g" % float(np.max(np.abs(glog - elog))))
    nxt = np.array([orc.argmax(elog)], np.int32)
    e2, g2_ = odec.forward(nxt), gdec.forward(nxt)
    if not np.max(np.abs(g2_ - e2)) <= tol:
        failures.append("step logits differ by %g" % float(np.max(np.abs(g2_ - e2))))
    etok, _, _ = odec.generate(prompt, 20, threads=4, attn_threads=2)
    gtok, m = gdec.generate(prompt, 20)
    if not (gtok == etok).all():
        failures.append("greedy tokens differ: %s vs %s" % (gtok.tolist(), etok.tolist()))
    # a prompt long enough for the token-block path (tcgen05 GEMMs; row-parallel projections all-reduce their int32 sums)
    long_prompt = rng.integers(0, V, 45).astype(np.int32)
    el, gl = odec.forward(long_prompt), gdec.forward(long_prompt)
    if not np.max(np.abs(gl - el)) <= tol:
        failures.append("token-block prompt logits differ by %g" % float(np.max(np.abs(gl - el))))
    nxt = np.array([orc.argmax(el)], np.int32)
    el, gl = odec.forward(nxt), gdec.forward(nxt)
    if not np.max(np.abs(gl - el)) <= tol:
        failures.append("step after the token-block prompt: logits differ by %g" % float(np.max(np.abs(gl - el))))
    # every rank must hold the same logits bit for bit
    mine = torch.from_numpy(gdec.forward(prompt).view(np.int32).astype(np.int64))
    lo, hi = mine.clone(), mine.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
    if not torch.equal(lo, hi):
        failures.append("ranks disagree on the logits")
    ctx.sync()
    gdec.close()

    # ---- independent sequences on the sharded decoder (peer exchange only: the sharded head's tail exchanges the
    #      (maximum, index) pairs of the vocabulary slices): every sequence against an oracle decoder of its own ----
    if mode in ("peer", "peer3"):
        B = 3
        bdec = cabi.Decoder(ctx, L, H, heads, kvh, hd, I, V, eps, theta, act, msl)
        bdec.set_batch(B)
        odecs = [orc.Decoder(L, H, heads, kvh, hd, I, V, eps, theta, act, msl) for _ in range(B)]
        for b, (masters, ws, g1, g2) in enumerate(blocks):
            bdec.set_block(b, ws, g1=g1, g2=g2)
            for od in odecs:
                od.set_block(b, *masters, g1=g1, g2=g2)
        bdec.set_embeddings(emb_dev, fg)
        elogs = []
        for i, od in enumerate(odecs):
            od.set_embeddings(emb, fg)
            pr = rng.integers(0, V, 5 + 4 * i).astype(np.int32)
            bdec.select(i)
            gl = bdec.forward(pr)
            el = od.forward(pr)
            if not np.max(np.abs(gl - el)) <= tol:
                failures.append("batch: prompt logits of sequence %d differ by %g" % (i, float(np.max(np.abs(gl - el)))))
            elogs.append(el)
        toks = rng.integers(0, V, B).astype(np.int32)
        glogs = bdec.step_batch(toks)
        for i, od in enumerate(odecs):
            elogs[i] = od.forward(toks[i:i + 1])
            if not np.max(np.abs(glogs[i] - elogs[i])) <= tol:
                failures.append("batch: step logits of sequence %d differ by %g" % (i, float(np.max(np.abs(glogs[i] - elogs[i])))))
        bdec.continue_batch(5)
        got = bdec.generated_tokens_batch(5)
        for i, od in enumerate(odecs):
            want, lg = [], elogs[i]
            for _ in range(5):
                t = orc.argmax(lg)
                want.append(t)
                lg = od.forward(np.array([t], np.int32))
            if got[i].tolist() != want:
                failures.append("batch: greedy tokens of sequence %d: %s vs %s" % (i, got[i].tolist(), want))
        ctx.sync()
        bdec.close()
    dist.barrier(group=group)  # nobody leaves while a peer may still be inside a collective
    ctx.tp_finalize()
    ctx.close()
    return failures, 1e6 * m.decode_device_seconds / max(1, m.generated_tokens)


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    local = int(os.environ.get("LOCAL_RANK", rank))
    mode = sys.argv[1] if len(sys.argv) > 1 else "graph"
    failures, us = run_checks(mode, local)
    dist.destroy_process_group()
    if failures:
        print("rank %d FAILED: %s" % (rank, "; ".join(failures)), flush=True)
        sys.exit(1)
    print("rank %d ok (%.1f us/token sharded decode)" % (rank, us), flush=True)


if __name__ == "__main__":
    main()
