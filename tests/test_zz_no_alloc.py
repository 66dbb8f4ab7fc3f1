"""The allocation-free ternary linear against the regular entry point and the CPU oracle.

Some hosts of this library may not allocate device memory while they run inference (a fixed, already-spent
memory budget; a frame loop that promised "no allocation after load").  `loom_b200_ternary_linear_no_alloc`
serves them with its stream-K scratch in a fixed array inside the library.  It must give exactly the bits of
`loom_b200_ternary_linear` and of the oracle's integer matvec + float64 rescale, on repeated calls (the array
keeps the previous call's contents), alone in a fresh process or after every other test has used the library.
This file sorts last on purpose.
"""
import numpy as np
import pytest

import loom_b200
from loom_b200 import cabi
from oracle import oracle as orc
from refkit import np_pack

pytestmark = pytest.mark.gpu


def _oracle_linear(words, rows, cols, scale, xq, amax, bias, resid, relu):
    """float32(float64(acc) * outputScale + bias) -> ReLU -> + residual, as the CPU path computes it."""
    m = orc.Matrix.from_words(words, rows, cols, scale)
    out = np.empty((xq.shape[0], rows), np.float32)
    for n in range(xq.shape[0]):
        y = m.matvec(xq[n], amax[n])  # float64 [rows]
        if bias is not None:
            y = y + bias.astype(np.float64)
        f = y.astype(np.float32)
        if relu:
            f = np.maximum(f, np.float32(0))
        if resid is not None:
            f = (f + resid[n]).astype(np.float32)
        out[n] = f
    return out


def _case(ctx, rows, cols, batch, seed, with_bias_residual):
    rng = np.random.default_rng(seed)
    q_w = rng.integers(-1, 2, rows * cols).astype(np.int8)
    words = np_pack(q_w, rows, cols)
    w = ctx.upload_ternary(words, rows, cols, 0.0371)
    xq = rng.integers(-127, 128, (batch, cols)).astype(np.int8)
    amax = (rng.random(batch) * 4 + 0.1).astype(np.float32)
    bias = (rng.standard_normal(rows) * 0.1).astype(np.float32) if with_bias_residual else None
    resid = rng.standard_normal((batch, rows)).astype(np.float32) if with_bias_residual else None
    dq, da = ctx.to_device(xq), ctx.to_device(amax)
    db = ctx.to_device(bias) if bias is not None else None
    dr = ctx.to_device(resid) if resid is not None else None
    d_ref, d_new = ctx.alloc(batch * rows * 4), ctx.alloc(batch * rows * 4)
    ctx.ternary_linear(w, batch, dq, da, d_ref, bias=db, residual=dr, act=cabi.ACT_RELU)
    ref = ctx.download(d_ref, (batch, rows), np.uint32)
    expect = _oracle_linear(words, rows, cols, np.float32(0.0371), xq, amax, bias, resid, True)
    assert (ref == expect.view(np.uint32)).all(), "loom_b200_ternary_linear differs from the CPU oracle"
    for call in range(2):  # two calls in a row: the second starts from whatever the first left in the array
        ctx.zero(d_new, batch * rows * 4)
        ctx.ternary_linear_no_alloc(w, batch, dq, da, d_new, bias=db, residual=dr, act=cabi.ACT_RELU)
        got = ctx.download(d_new, (batch, rows), np.uint32)
        assert (got == ref).all(), "call %d differs from loom_b200_ternary_linear" % call
        assert (got == expect.view(np.uint32)).all(), "call %d differs from the CPU oracle" % call
    # the regular entry point still works afterwards (its own scratch was left alone)
    ctx.ternary_linear(w, batch, dq, da, d_ref, bias=db, residual=dr, act=cabi.ACT_RELU)
    assert (ctx.download(d_ref, (batch, rows), np.uint32) == ref).all()
    for p in (dq, da, db, dr, d_ref, d_new):
        if p:
            ctx.free(p)


def test_no_alloc_matches_regular_entry_point_and_oracle():
    ctx = loom_b200.Context(0)
    try:
        _case(ctx, 2560, 6912, 1, 1, False)   # every strip is shared between CTAs: the scratch carries all sums
        _case(ctx, 6912, 2560, 11, 2, True)   # two passes of tokens, bias + residual + activation
        _case(ctx, 40, 70, 2, 3, True)        # ragged rows and columns
        _case(ctx, 48, 28672, 8, 4, True)     # very wide input: five tokens per pass, like the regular entry point
    finally:
        ctx.close()


def test_no_alloc_allocates_nothing():
    """Free device memory is the same before and after repeated calls (after one warm-up call that resolves the
    array's address and raises the kernel's shared-memory limit)."""
    import torch

    ctx = loom_b200.Context(0)
    try:
        rows, cols, batch = 6912, 2560, 3
        rng = np.random.default_rng(5)
        w = ctx.upload_ternary(np_pack(rng.integers(-1, 2, rows * cols).astype(np.int8), rows, cols), rows, cols, 0.05)
        dq = ctx.to_device(rng.integers(-127, 128, (batch, cols)).astype(np.int8))
        da = ctx.to_device(np.ones(batch, np.float32))
        do = ctx.alloc(batch * rows * 4)
        ctx.ternary_linear_no_alloc(w, batch, dq, da, do)
        ctx.sync()
        free0, _ = torch.cuda.mem_get_info(0)
        for _ in range(5):
            ctx.ternary_linear_no_alloc(w, batch, dq, da, do)
        ctx.sync()
        free1, _ = torch.cuda.mem_get_info(0)
        assert free1 == free0, "device memory changed by %d bytes across no_alloc calls" % (free0 - free1)
        for p in (dq, da, do):
            ctx.free(p)
    finally:
        ctx.close()


def test_no_alloc_rejects_shapes_beyond_its_scratch():
    ctx = loom_b200.Context(0)
    try:
        rows, cols = 70000, 16  # more than 65,536 rows
        words = np.full((rows, 1), 0x55555555, np.uint32)
        w = ctx.upload_ternary(words, rows, cols, 1.0)
        dq, da, do = ctx.to_device(np.zeros((1, cols), np.int8)), ctx.to_device(np.ones(1, np.float32)), ctx.alloc(rows * 4)
        with pytest.raises(loom_b200.LoomB200Error) as ei:
            ctx.ternary_linear_no_alloc(w, 1, dq, da, do)
        assert ei.value.code == -3 and "loom_b200_ternary_linear" in str(ei.value)
        ctx.ternary_linear(w, 1, dq, da, do)  # the regular entry point takes it
        ctx.sync()
    finally:
        ctx.close()
