"""GPU parity of the tcgen05 (kind::i8) prefill GEMM against the CPU oracle: int32 accumulators and float32
outputs must be bit-exact, like the per-token path (config "batched prefill": M = 512, 2560 -> 6912 and back)."""
import numpy as np
import pytest

import loom_b200
from loom_b200 import cabi
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=[(1, 1), (1, 0), (0, 0)], ids=["cached-codes-persistent", "cached-codes-one-shot", "expand-in-kernel"])
def ctx(request):
    # the ways the weights reach the tensor core: pre-expanded int8 codes (built on a matrix's first GEMM) read by the
    # persistent kernel with two accumulator buffers or by the one-shot kernel, and 2-bit tiles expanded inside the kernel
    c = loom_b200.Context(0)
    c.set_option("gemm_cache", request.param[0])
    c.set_option("gemm_stream", request.param[1])
    yield c
    c.close()


def run_case(ctx, rows, cols, tokens, seed, bias=False, residual=False, act=cabi.ACT_LINEAR):
    rng = np.random.default_rng(seed)
    m = orc.Matrix.from_f32((rng.standard_normal(rows * cols) * 0.02).astype(np.float32), rows, cols)
    w = ctx.upload_ternary(m.words, rows, cols, m.scale)
    x = rng.standard_normal((tokens, cols)).astype(np.float32)
    b = (rng.standard_normal(rows) * 0.1).astype(np.float32) if bias else None
    r = rng.standard_normal((tokens, rows)).astype(np.float32) if residual else None
    dx = ctx.to_device(x)
    db = ctx.to_device(b) if bias else None
    dr = ctx.to_device(r) if residual else None
    dout, dacc, damax = ctx.alloc(tokens * rows * 4), ctx.alloc(tokens * rows * 4), ctx.alloc(tokens * 4)
    ctx.ternary_gemm(w, tokens, dx, out=dout, bias=db, residual=dr, act=act, acc_out=dacc, amax_out=damax)
    out = ctx.download(dout, (tokens, rows), np.float32)
    acc = ctx.download(dacc, (tokens, rows), np.int32)
    amax = ctx.download(damax, (tokens,), np.float32)
    xq, eamax = orc.quantize_rows_f32(x)
    assert (amax == eamax).all()
    eacc = np.stack([m.acc_i32(xq[t]) for t in range(tokens)]) if tokens * rows * cols < 3e8 else None
    if eacc is not None:
        assert (acc == eacc).all()
    else:  # full-size: exact integer product with numpy (int64) instead of the scalar oracle loop
        from refkit import np_unpack
        wmat = np_unpack(m.words, rows, cols).astype(np.int32)
        eacc = (xq.astype(np.int32) @ wmat.T).astype(np.int32)
        assert (acc == eacc).all()
    os_ = np.float64(m.scale) * amax.astype(np.float64) / 127.0
    y = eacc.astype(np.float64) * os_[:, None]
    if bias:
        y = y + b.astype(np.float64)[None, :]
    f = y.astype(np.float32)
    f = orc.activate_f32(f, act) if act not in (cabi.ACT_LINEAR,) and f.size < 200000 else (np.maximum(f, 0) if act == cabi.ACT_RELU else f)
    if residual:
        f = (f + r).astype(np.float32)
    assert (out.view(np.uint32) == f.view(np.uint32)).all()
    for p in (dx, db, dr, dout, dacc, damax):
        if p:
            ctx.free(p)


def test_gemm_single_tile(ctx):
    run_case(ctx, 128, 128, 128, 1)


@pytest.mark.parametrize("rows,cols,tokens", [(256, 512, 128), (128, 1024, 37), (200, 300, 70), (33, 65, 5), (1000, 700, 300)])
def test_gemm_ragged_shapes(ctx, rows, cols, tokens):
    run_case(ctx, rows, cols, tokens, rows + tokens, bias=True, residual=True, act=cabi.ACT_RELU)


@pytest.mark.parametrize("rows,cols,tokens", [(2560, 6912, 64), (512, 8192, 20), (100, 4096, 130)])
def test_gemm_split_k(ctx, rows, cols, tokens):
    # few output tiles and a long K: several CTAs share a tile and hand their int32 partial sums over through atomics;
    # the result must be the same bits, and a second run must find the scratch clean again
    run_case(ctx, rows, cols, tokens, 3 * rows + tokens, bias=True, residual=True, act=cabi.ACT_RELU2)
    run_case(ctx, rows, cols, tokens, 5 * rows + tokens, bias=False, residual=False)
    ctx.set_option("gemm_splitk", 0)
    try:
        run_case(ctx, rows, cols, tokens, 7 * rows + tokens, bias=True, residual=False)
    finally:
        ctx.set_option("gemm_splitk", 1)


@pytest.mark.parametrize("rows,cols", [(6912, 2560), (2560, 6912)])
def test_gemm_prefill_config(ctx, rows, cols):
    run_case(ctx, rows, cols, 512, 7, bias=False, residual=True)


def test_i8_micro_peak_is_plausible(ctx):
    # the denominator of the GEMM's tensor roofline: dense int8 on tcgen05 with nothing but MMAs in flight.  The B200's
    # nominal figure is 4,500 TOP/s; anything below 1,000 or above 6,000 means the measurement, not the GPU, is off
    tops = ctx.i8_peak_tops(5000)
    assert 1000.0 < tops < 6000.0, tops
