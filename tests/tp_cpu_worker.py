"""One rank of the CPU model of the tensor-parallel shard plan (run by test_tp_plan_cpu.py under
torch.distributed.run with the gloo backend).

Each rank holds the slices loom_b200.tp.ShardPlan gives it, computes its part with the CPU oracle's
primitives, exchanges exactly what the GPU path exchanges (float64 sum of squares, float32 absmax, int32
partial accumulators) and checks the result against the oracle's UNSHARDED layer, bit for bit.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from loom_b200.tp import ShardPlan, slice_cols, slice_rows  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from refkit import round_half_away  # noqa: E402


def allreduce(a: np.ndarray, op) -> np.ndarray:
    t = torch.from_numpy(np.ascontiguousarray(a))
    dist.all_reduce(t, op=op)
    return t.numpy()


def output_scale(scale, amax) -> float:
    s = float(np.float64(np.float32(scale)) * np.float64(np.float32(amax)) / 127.0)
    return 1.0 if s == 0 else s


def rowsharded_linear(x_l, is_f64, words_l, rows, cols_l, cols_global, scale, inner_w_l, eps, bias):
    """x_l: this rank's slice of one token's vector -> float32 [rows], identical on every rank."""
    v = x_l.astype(np.float64)
    ss = 0.0
    for t in v:  # sequential float64 sum like the reference's loop, per slice
        ss += t * t
    ss = float(allreduce(np.array([ss], np.float64), dist.ReduceOp.SUM)[0])
    sc = 1.0 / np.sqrt(ss / cols_global + eps)
    w = np.ones(v.size, np.float64)
    if inner_w_l is not None:
        w[:inner_w_l.size] = inner_w_l.astype(np.float64)
    if is_f64:
        y = v * (sc * w)
    else:
        y = ((v * sc) * w).astype(np.float32).astype(np.float64)
    amax = np.float32(np.max(np.abs(y))) if y.size else np.float32(0)
    amax = np.float32(allreduce(np.array([amax], np.float32), dist.ReduceOp.MAX)[0])
    if amax < np.float32(1e-5):
        amax = np.float32(1e-5)
    s = 127.0 / np.float64(amax)
    q = np.clip(round_half_away(y * s), -128, 127).astype(np.int8)
    acc = orc.matvec_i32(words_l, rows, cols_l, q)
    acc = allreduce(acc, dist.ReduceOp.SUM)
    out = acc.astype(np.float64) * output_scale(scale, amax)
    if bias is not None:
        out = out + bias.astype(np.float64)
    return out.astype(np.float32)


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    rng = np.random.default_rng(1234)  # the same stream on every rank
    H, heads, kvh, hd, I, V = 64, 4, 2, 16, 128, 128
    plan = ShardPlan(world, rank, H, heads, kvh, hd, I, V)
    failures = []

    # ---- a row-sharded linear on a float64 vector: the MHA output projection ----
    qd = heads * hd
    wo = (rng.standard_normal(H * qd) * 0.05).astype(np.float32)
    o_words, o_scale = orc.pack_f32(wo, H, qd)
    inner = (1 + 0.1 * rng.standard_normal(qd)).astype(np.float32)
    bias = (0.01 * rng.standard_normal(H)).astype(np.float32)
    attn = rng.standard_normal(qd) * 0.3
    q0, q1 = plan.q_rows
    got = rowsharded_linear(attn[q0:q1], True, slice_cols(o_words, H, qd, q0, q1), H, q1 - q0, qd, o_scale, inner[q0:q1],
                            1e-5, bias)
    y = orc.inner_rmsnorm_f64(attn, inner, 1e-5)
    xq, amax = orc.quantize_f64(y)
    acc = orc.matvec_i32(o_words, H, qd, xq)
    want = (acc.astype(np.float64) * output_scale(o_scale, amax) + bias.astype(np.float64)).astype(np.float32)
    if not np.array_equal(got, want):
        failures.append("f64 row-sharded linear differs in %d of %d" % (int((got != want).sum()), want.size))

    # ---- the SwiGLU layer: column-sharded gate/up, row-sharded down ----
    act = orc.ACT_SILU
    seq = 3
    masters = [(rng.standard_normal(I * H) * 0.05).astype(np.float32) for _ in range(3)]
    g_words, g_scale = orc.pack_f32(masters[0], I, H)
    u_words, u_scale = orc.pack_f32(masters[1], I, H)
    d_words, d_scale = orc.pack_f32(masters[2], H, I)
    ffn_inner = (1 + 0.1 * rng.standard_normal(I)).astype(np.float32)
    x = rng.standard_normal((seq, H)).astype(np.float32)
    G = orc.Matrix.from_words(g_words, I, H, g_scale)
    U = orc.Matrix.from_words(u_words, I, H, u_scale)
    D = orc.Matrix.from_words(d_words, H, I, d_scale)
    _, want = orc.swiglu_forward(G, U, D, x, act=act, inner_w=ffn_inner, eps=0.0)
    i0, i1 = plan.inter_rows
    g_l, u_l = slice_rows(g_words, I, H, i0, i1), slice_rows(u_words, I, H, i0, i1)
    d_l = slice_cols(d_words, H, I, i0, i1)
    for t in range(seq):
        xq, amax = orc.quantize_f32(x[t])
        # gate and up stay in float64 until the product is rounded to float32 (poly/swiglu.go:299-306)
        gv = orc.matvec_i32(g_l, i1 - i0, H, xq).astype(np.float64) * output_scale(g_scale, amax)
        uv = orc.matvec_i32(u_l, i1 - i0, H, xq).astype(np.float64) * output_scale(u_scale, amax)
        prod = np.array([orc.gate_product(float(a), float(b), act) for a, b in zip(gv, uv)], np.float32)
        got = rowsharded_linear(prod, False, d_l, H, i1 - i0, I, d_scale, ffn_inner[i0:i1], 1e-5, None)
        if not np.array_equal(got, want[t]):
            failures.append("swiglu token %d differs in %d of %d" % (t, int((got != want[t]).sum()), H))

    # ---- vocabulary slices of the tied head cover every row once ----
    v0, v1 = plan.vocab_rows
    cover = np.zeros(V, np.int32)
    cover[v0:v1] += 1
    cover = allreduce(cover, dist.ReduceOp.SUM)
    expect = 1 if V % world == 0 else world
    if not (cover == expect).all():
        failures.append("vocabulary slices do not tile the head")

    dist.barrier()
    dist.destroy_process_group()
    if failures:
        print("rank %d FAILED: %s" % (rank, "; ".join(failures)), flush=True)
        sys.exit(1)
    print("rank %d ok" % rank, flush=True)


if __name__ == "__main__":
    main()
