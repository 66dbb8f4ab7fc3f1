"""GPU parity tests of the kernel-level C ABI against the CPU oracle (bit-exact bar).

Shapes follow the reference's own sweeps (poly/tests/bitnet_packed_test.go:19-21, bitnet_cpu_test.go) plus
the benchmark shapes 2560x6912 / 6912x2560 (poly/tests/bitnet_matvec_bench_test.go:40-43).
"""
import numpy as np
import pytest

import loom_b200
from loom_b200 import cabi
from oracle import oracle as orc
from refkit import deterministic_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = loom_b200.Context(0)
    yield c
    c.close()


def gpu_linear(ctx, w, x_q, amax, batch, bias=None, residual=None, act=cabi.ACT_LINEAR):
    dq = ctx.to_device(x_q)
    da = ctx.to_device(amax)
    dout = ctx.alloc(batch * w.rows * 4)
    dacc = ctx.alloc(batch * w.rows * 4)
    db = ctx.to_device(bias) if bias is not None else None
    dr = ctx.to_device(residual) if residual is not None else None
    ctx.ternary_linear(w, batch, dq, da, dout, bias=db, residual=dr, act=act, acc_out=dacc)
    out = ctx.download(dout, (batch, w.rows), np.float32)
    acc = ctx.download(dacc, (batch, w.rows), np.int32)
    for p in (dq, da, dout, dacc, db, dr):
        if p:
            ctx.free(p)
    return out, acc


def oracle_linear(m, x_q, amax, bias=None, residual=None, act=orc.ACT_LINEAR):
    outs, accs = [], []
    for b in range(x_q.shape[0]):
        y = m.matvec(x_q[b], amax[b])
        if bias is not None:
            y = y + bias.astype(np.float64)
        f = y.astype(np.float32)
        f = orc.activate_f32(f, act)
        if residual is not None:
            f = (f + residual[b]).astype(np.float32)
        outs.append(f)
        accs.append(m.acc_i32(x_q[b]))
    return np.stack(outs), np.stack(accs)


SWEEP = [(40, 70), (8, 64), (33, 65), (16, 128), (64, 2560), (128, 6912), (7, 191), (3, 17), (1, 1), (17, 129)]


@pytest.mark.parametrize("rows,cols", SWEEP)
def test_retile_round_trip(ctx, rows, cols):
    words, scale = orc.pack_f32(deterministic_weights(rows * cols), rows, cols)
    w = ctx.upload_ternary(words, rows, cols, scale)
    assert (w.rows, w.cols, w.row_words) == (rows, cols, (cols + 15) // 16)
    assert w.scale == scale
    assert (w.words() == words).all()


@pytest.mark.parametrize("rows,cols", SWEEP + [(6912, 2560)])
def test_device_ternarizer_matches_oracle(ctx, rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    master = (rng.standard_normal(rows * cols) * 0.02).astype(np.float32)
    if rows * cols < 10000:
        master = deterministic_weights(rows * cols)
    words, scale = orc.pack_f32(master, rows, cols)
    d = ctx.to_device(master)
    w = ctx.pack_ternary_f32(d, rows, cols)
    ctx.free(d)
    assert w.scale == scale
    assert (w.words() == words).all()


def test_device_ternarizer_already_ternary_rule(ctx):
    master = np.array([-1, 0, 1, 1, 0, -1, 0, 0] * 4, np.float32)
    words, scale = orc.pack_f32(master, 2, 16)
    d = ctx.to_device(master)
    w = ctx.pack_ternary_f32(d, 2, 16)
    ctx.free(d)
    assert scale == np.float32(1.0) and w.scale == scale and (w.words() == words).all()


@pytest.mark.parametrize("batch,n", [(1, 2560), (3, 6912), (2, 17), (5, 191), (1, 1), (4, 4096)])
def test_quantize_matches_oracle(ctx, batch, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal((batch, n)).astype(np.float32)
    x[0, 0] = 0.0
    if batch > 1:
        x[1] = 0.0  # all-zero row: amax floor 1e-5
    dx, dq, da = ctx.to_device(x), ctx.alloc(batch * n), ctx.alloc(batch * 4)
    ctx.quantize_activation(batch, n, dx, dq, da)
    q = ctx.download(dq, (batch, n), np.int8)
    a = ctx.download(da, (batch,), np.float32)
    oq, oa = orc.quantize_rows_f32(x)
    assert (a == oa).all() and (q == oq).all()
    # float64 twin
    x64 = x.astype(np.float64) * 1.0000001
    dx64 = ctx.to_device(x64)
    ctx.quantize_activation_f64(batch, n, dx64, dq, da)
    q = ctx.download(dq, (batch, n), np.int8)
    a = ctx.download(da, (batch,), np.float32)
    for b in range(batch):
        eq, ea = orc.quantize_f64(x64[b])
        assert ea == a[b] and (eq == q[b]).all()
    for p in (dx, dq, da, dx64):
        ctx.free(p)


def test_quantize_ties_round_away(ctx):
    x = np.array([[127.0, 0.5, -0.5, 1.5, -1.5, 2.5, -127.0, 0.0]], np.float32)
    dx, dq, da = ctx.to_device(x), ctx.alloc(8), ctx.alloc(4)
    ctx.quantize_activation(1, 8, dx, dq, da)
    q = ctx.download(dq, (8,), np.int8)
    assert q.tolist() == [127, 1, -1, 2, -2, 3, -127, 0]
    for p in (dx, dq, da):
        ctx.free(p)


@pytest.mark.parametrize("variant,part", [(0, 1), (0, 2), (1, 1), (1, 2)])
@pytest.mark.parametrize("rows,cols", SWEEP)
def test_linear_reference_sweep_bit_exact(ctx, rows, cols, variant, part):
    # the reference's SIMD-vs-scalar sweep, batch 2, difference must be exactly 0
    ctx.set_option("gemv_variant", variant)
    ctx.set_option("gemv_partition", part)
    m = orc.Matrix.from_f32(deterministic_weights(rows * cols), rows, cols)
    x = deterministic_weights(2 * cols).reshape(2, cols)
    xq, amax = orc.quantize_rows_f32(x)
    w = ctx.upload_ternary(m.words, rows, cols, m.scale)
    out, acc = gpu_linear(ctx, w, xq, amax, 2)
    eo, ea = oracle_linear(m, xq, amax)
    ctx.set_option("gemv_variant", 0)
    ctx.set_option("gemv_partition", 0)
    assert (acc == ea).all()
    assert (out.view(np.uint32) == eo.view(np.uint32)).all()


@pytest.mark.parametrize("variant", [0, 1, 2, 3])
@pytest.mark.parametrize("rows,cols,batch", [(6912, 2560, 1), (2560, 6912, 1), (6912, 2560, 5), (2560, 6912, 19),
                                             (3840, 2560, 8), (1000, 300, 3)])
def test_linear_benchmark_shapes_bit_exact(ctx, rows, cols, batch, variant):
    ctx.set_option("gemv_variant", variant & 1)
    ctx.set_option("gemv_partition", 1 + (variant >> 1))
    rng = np.random.default_rng(rows + cols + batch)
    master = (rng.standard_normal(rows * cols) * 0.02).astype(np.float32)
    m = orc.Matrix.from_f32(master, rows, cols)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    xq, amax = orc.quantize_rows_f32(x)
    bias = (rng.standard_normal(rows) * 0.1).astype(np.float32)
    resid = rng.standard_normal((batch, rows)).astype(np.float32)
    w = ctx.upload_ternary(m.words, rows, cols, m.scale)
    for kw in (dict(), dict(bias=bias), dict(bias=bias, residual=resid), dict(act=cabi.ACT_RELU2),
               dict(act=cabi.ACT_RELU, residual=resid)):
        out, acc = gpu_linear(ctx, w, xq, amax, batch, **kw)
        eo, ea = oracle_linear(m, xq, amax, **kw)
        assert (acc == ea).all()
        assert (out.view(np.uint32) == eo.view(np.uint32)).all(), kw
    ctx.set_option("gemv_variant", 0)
    ctx.set_option("gemv_partition", 0)


def test_linear_extreme_activations(ctx):
    # every activation at -128/127 and every weight +-1: the largest accumulators the path can see
    rows, cols = 32, 6912
    q = np.ones((rows, cols), np.int8)
    q[1::2] = -1
    words = orc.pack_native(q, rows, cols)
    m = orc.Matrix.from_words(words, rows, cols, 0.75)
    xq = np.full((2, cols), 127, np.int8)
    xq[1] = -128
    amax = np.array([3.0, 5.0], np.float32)
    w = ctx.upload_ternary(words, rows, cols, 0.75)
    out, acc = gpu_linear(ctx, w, xq, amax, 2)
    eo, ea = oracle_linear(m, xq, amax)
    assert (acc == ea).all() and abs(int(acc[1, 0])) == 128 * cols
    assert (out.view(np.uint32) == eo.view(np.uint32)).all()


def test_linear_repeat_is_stable(ctx):
    # the fix-up scratch must be clean after every launch
    rows, cols = 2560, 6912
    rng = np.random.default_rng(5)
    m = orc.Matrix.from_f32((rng.standard_normal(rows * cols) * 0.02).astype(np.float32), rows, cols)
    xq, amax = orc.quantize_rows_f32(rng.standard_normal((1, cols)).astype(np.float32))
    w = ctx.upload_ternary(m.words, rows, cols, m.scale)
    first, _ = gpu_linear(ctx, w, xq, amax, 1)
    for grid in (1, 2, 3):
        ctx.set_option("gemv_ctas_per_sm", grid)
        for part in (1, 2, 0):
            ctx.set_option("gemv_partition", part)
            for pdl in (0, 1):
                ctx.set_option("pdl", pdl)
                again, _ = gpu_linear(ctx, w, xq, amax, 1)
                assert (again.view(np.uint32) == first.view(np.uint32)).all()
    ctx.set_option("gemv_ctas_per_sm", 2)
    ctx.set_option("pdl", 1)


def test_microsoft_layout_upload(ctx):
    # TestMicrosoftOfflinePackedBitNetRowsDecode through the GPU path
    packed = np.array([0b10100001, 0b00011000, 0b10010000, 0b00001010], np.uint8)
    w = ctx.upload_microsoft_u8(packed, 8, 2, 0.5)
    assert (w.words() == orc.pack_microsoft_u8(packed, 8, 2)).all()
    out, _ = gpu_linear(ctx, w, np.array([[2, -3]], np.int8), np.array([127.0], np.float32), 1)
    assert np.max(np.abs(out[0] - np.array([1.5, -2.5, -2.5, -2.5, 1, 1.5, 2.5, 2.5]))) <= 1e-6


def entity_blob(words, rows, cols, offset, scale, row_words=None):
    """encodeEntityBitNetTernaryBlob (poly/entity_bitnet.go:38-55): 24-byte little-endian header + words."""
    import struct
    words = np.ascontiguousarray(words, dtype="<u4").ravel()
    rw = (cols + 15) // 16 if row_words is None else row_words
    return struct.pack("<IIIfII", rows, cols, offset, float(scale), rw, words.size) + words.tobytes()


def test_entity_blob_upload(ctx):
    # the round trip the reference pins in TestEntityBitNetTernaryBlobRoundTrip (poly/tests/entity_test.go:331-348),
    # here blob -> device: words, shape, scale and slab offset survive, and the matrix computes
    rng = np.random.default_rng(11)
    rows, cols = 24, 70
    words, scale = orc.pack_f32((rng.standard_normal(rows * cols) * 0.05).astype(np.float32), rows, cols)
    w, off = ctx.upload_entity_blob(entity_blob(words, rows, cols, 1792, scale))
    assert off == 1792 and (w.words() == words).all() and w.scale == scale
    xq, amax = orc.quantize_f32(rng.standard_normal(cols).astype(np.float32))
    out, _ = gpu_linear(ctx, w, xq[None, :], np.array([amax], np.float32), 1)
    want = (orc.matvec_i32(words, rows, cols, xq).astype(np.float64) * (np.float64(scale) * np.float64(amax) / 127.0)).astype(np.float32)
    assert (out[0] == want).all()
    # rowWords = 0 in the header means ceil(cols/16)
    w2, _ = ctx.upload_entity_blob(entity_blob(words, rows, cols, 0, scale, row_words=0))
    assert (w2.words() == words).all()
    blob = entity_blob(words, rows, cols, 0, scale)
    for bad in (blob[:10], blob[:-4], b""):
        with pytest.raises(cabi.LoomB200Error):
            ctx.upload_entity_blob(bad)


@pytest.mark.parametrize("act", [cabi.ACT_SILU, cabi.ACT_RELU2])
def test_gate_product(ctx, act):
    rng = np.random.default_rng(3)
    g = rng.standard_normal((3, 6912)).astype(np.float32)
    u = rng.standard_normal((3, 6912)).astype(np.float32)
    dg, du, do = ctx.to_device(g), ctx.to_device(u), ctx.alloc(g.nbytes)
    ctx.gate_product(3, 6912, act, dg, du, do)
    out = ctx.download(do, g.shape, np.float32)
    exp = np.array([orc.gate_product(float(a), float(b), act) for a, b in zip(g.ravel(), u.ravel())]).astype(
        np.float32).reshape(g.shape)
    if act == cabi.ACT_RELU2:
        assert (out == exp).all()
    else:  # exp() differs between libm implementations in the last bit of the double
        assert np.max(np.abs(out - exp) / np.maximum(np.abs(exp), 1e-30)) <= 1e-6
        assert (out == exp).mean() > 0.999
    for p in (dg, du, do):
        ctx.free(p)


def test_inner_rmsnorm(ctx):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((2, 6912)).astype(np.float32)
    wt = rng.standard_normal(100).astype(np.float32)
    dx, dw = ctx.to_device(x), ctx.to_device(wt)
    ctx.inner_rmsnorm(2, 6912, dx, dw, 100, 0.0)
    out = ctx.download(dx, x.shape, np.float32)
    exp = np.stack([orc.inner_rmsnorm_f32(x[b], wt, 0.0) for b in range(2)])
    # the sum of squares is a parallel float64 tree here, sequential in the reference
    assert np.max(np.abs(out - exp) / np.maximum(np.abs(exp), 1e-30)) <= 1e-6
    assert (out == exp).mean() > 0.999
    ctx.free(dx)
    ctx.free(dw)


def test_error_reporting(ctx):
    L = cabi.lib()
    assert L.loom_b200_quantize_activation(ctx.h, 1, 0, None, None, None) == -1
    assert b"bad shape" in L.loom_b200_last_error(ctx.h)
    import ctypes as C
    h = C.c_void_p()
    words = np.zeros(4, np.uint32)
    assert L.loom_b200_upload_ternary(ctx.h, words.ctypes.data, 2, 17, 1, 1.0, C.byref(h)) == -1  # row_words wrong
    assert L.loom_b200_upload_microsoft_u8(ctx.h, words.ctypes.data, 6, 2, 1.0, C.byref(h)) == -1  # rows % 4
    assert L.loom_b200_ctx_set_option(ctx.h, b"nope", 1) == -1
    n0 = ctx.launch_count
    assert n0 > 0


def test_bounded_wait_reports_timeout_and_context_survives(ctx):
    # failure detection without a fault: a device-side wait on a flag nothing sets gives up after its poll limit, the
    # status word comes back through sync as LOOM_B200_ERR_TIMEOUT, and the context keeps working afterwards
    with pytest.raises(cabi.LoomB200Error) as err:
        ctx.selftest_wait_timeout(200000)
    assert err.value.code == cabi.ERR_TIMEOUT and "bounded device-side wait" in str(err.value)
    ctx.sync()  # the condition was cleared
    rng = np.random.default_rng(1)
    words, scale = orc.pack_f32((rng.standard_normal(32 * 64) * 0.05).astype(np.float32), 32, 64)
    w = ctx.upload_ternary(words, 32, 64, scale)
    xq, amax = orc.quantize_f32(rng.standard_normal(64).astype(np.float32))
    _, acc = gpu_linear(ctx, w, xq[None, :], np.array([amax], np.float32), 1)
    assert (acc[0] == orc.matvec_i32(words, 32, 64, xq)).all()
