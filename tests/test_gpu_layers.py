"""GPU parity tests of the layer-level and decoder-level C ABI against the CPU oracle.

Integer parts (int8 activations, int32 accumulators) are bit-exact by construction; what these tests add is
the float32/float64 glue: layer outputs must match the oracle within max relative error 1e-6 (the parallel
float64 reductions and the device libm's exp/sin/cos differ from the sequential CPU loops only far below
float32 resolution), and greedy token streams must be identical.
"""
import numpy as np
import pytest

import loom_b200
from loom_b200 import cabi
from oracle import oracle as orc
from refkit import deterministic_weights, split_mha_slab, split_swiglu_slab

pytestmark = pytest.mark.gpu

REL = 1e-6  # the tolerance the task states for float32 layer outputs


@pytest.fixture(scope="module")
def ctx():
    c = loom_b200.Context(0)
    yield c
    c.close()


def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-6)))


def pair(ctx, master, rows, cols):
    m = orc.Matrix.from_f32(master, rows, cols)
    w = ctx.upload_ternary(m.words, rows, cols, m.scale)
    return m, w


@pytest.mark.parametrize("rows,cols,batch,act", [(40, 70, 2, cabi.ACT_LINEAR), (6912, 2560, 1, cabi.ACT_LINEAR),
                                                 (128, 6912, 11, cabi.ACT_RELU2), (33, 65, 3, cabi.ACT_SILU),
                                                 (16, 128, 2, cabi.ACT_GELU), (7, 191, 2, cabi.ACT_LEAKY_RELU),
                                                 (48, 8192, 3, cabi.ACT_LINEAR), (96, 28672, 7, cabi.ACT_RELU2)])
def test_dense_forward(ctx, rows, cols, batch, act):
    rng = np.random.default_rng(rows + cols)
    m, w = pair(ctx, (rng.standard_normal(rows * cols) * 0.02).astype(np.float32), rows, cols)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    pre, post = cabi.dense_forward(ctx, w, act, x)
    epre, epost = orc.dense_forward(m, act, x)
    assert (pre.view(np.uint32) == epre.view(np.uint32)).all()  # quantize + matvec + rescale: bit-exact
    if act in (cabi.ACT_LINEAR, cabi.ACT_RELU2, cabi.ACT_LEAKY_RELU, cabi.ACT_RELU):
        assert (post.view(np.uint32) == epost.view(np.uint32)).all()
    else:
        assert rel_err(post, epost) <= REL


def test_dense_reference_fixture(ctx):
    # TestPackedTernaryDenseMatchesDequantizedPath (poly/tests/bitnet_cpu_test.go:184-214) through the GPU
    m, w = pair(ctx, deterministic_weights(15), 3, 5)
    x = np.array([0.1, -0.2, 0.3, -0.4, 0.5, 0.6, -0.7, 0.8, -0.9, 1.0], np.float32).reshape(2, 5)
    _, post = cabi.dense_forward(ctx, w, cabi.ACT_LINEAR, x)
    _, epost = orc.dense_forward(m, orc.ACT_LINEAR, x)
    assert (post == epost).all()


@pytest.mark.parametrize("H,I,seq,act,bias,inner", [(4, 6, 2, cabi.ACT_SILU, True, False),
                                                    (2560, 6912, 1, cabi.ACT_SILU, False, False),
                                                    (2560, 6912, 3, cabi.ACT_RELU2, False, True),
                                                    (128, 200, 9, cabi.ACT_SILU, True, True),
                                                    (128, 8192, 3, cabi.ACT_RELU2, True, True),
                                                    (8192, 256, 2, cabi.ACT_SILU, False, False)])
def test_swiglu_forward(ctx, H, I, seq, act, bias, inner):
    rng = np.random.default_rng(H + I)
    if H == 4:  # TestPackedTernarySwiGLUProducesFiniteOutput fixture, poly/tests/bitnet_cpu_test.go:388-409
        g = split_swiglu_slab(deterministic_weights(88), 4, 6)
        x = np.array([0.1, -0.2, 0.3, -0.4, 0.2, -0.1, 0.4, -0.3], np.float32).reshape(2, 4)
    else:
        g = dict(wg=(rng.standard_normal(H * I) * 0.02).astype(np.float32),
                 wu=(rng.standard_normal(H * I) * 0.02).astype(np.float32),
                 wd=(rng.standard_normal(H * I) * 0.02).astype(np.float32),
                 bg=(rng.standard_normal(I) * 0.05).astype(np.float32), bu=(rng.standard_normal(I) * 0.05).astype(np.float32),
                 bd=(rng.standard_normal(H) * 0.05).astype(np.float32))
        x = rng.standard_normal((seq, H)).astype(np.float32)
    mg, wg = pair(ctx, g["wg"], I, H)
    mu, wu = pair(ctx, g["wu"], I, H)
    md, wd = pair(ctx, g["wd"], H, I)
    kw = dict(act=act)
    if bias:
        kw.update(bias_gate=g["bg"], bias_up=g["bu"], bias_down=g["bd"])
    if inner:
        kw.update(inner_w=(1.0 + 0.1 * rng.standard_normal(I)).astype(np.float32), eps=1e-6)
    pre, post = cabi.swiglu_forward(ctx, wg, wu, wd, x, **kw)
    epre, epost = orc.swiglu_forward(mg, mu, md, x, **kw)
    assert np.isfinite(post).all()
    assert rel_err(pre, epre) <= REL
    assert rel_err(post, epost) <= REL
    if act == cabi.ACT_RELU2:
        assert (post == epost).mean() > 0.99  # no libm in this path: only the reduction order can differ


def build_mha(ctx, rng, D, heads, kvh, hd, msl, theta, eps, biases=False, norms=False):
    qd, kvd = heads * hd, kvh * hd
    ws = {k: (rng.standard_normal(r * c) * 0.05).astype(np.float32) for k, r, c in
          (("wq", qd, D), ("wk", kvd, D), ("wv", kvd, D), ("wo", D, qd))}
    kw = {}
    if biases:
        kw.update(bq=(rng.standard_normal(qd) * 0.1).astype(np.float32), bk=(rng.standard_normal(kvd) * 0.1).astype(np.float32),
                  bv=(rng.standard_normal(kvd) * 0.1).astype(np.float32), bo=(rng.standard_normal(D) * 0.1).astype(np.float32))
    if norms:
        kw.update(q_norm=(1 + 0.1 * rng.standard_normal(hd)).astype(np.float32),
                  k_norm=(1 + 0.1 * rng.standard_normal(kvh * hd)).astype(np.float32),
                  inner_w=(1 + 0.1 * rng.standard_normal(qd)).astype(np.float32))
    om, gw = [], []
    for k, r, c in (("wq", qd, D), ("wk", kvd, D), ("wv", kvd, D), ("wo", D, qd)):
        m, w = pair(ctx, ws[k], r, c)
        om.append(m)
        gw.append(w)
    o = orc.MHA(D, heads, kvh, hd, msl, theta, eps, *om, **kw)
    g = cabi.MHA(ctx, D, heads, kvh, hd, msl, theta, eps, *gw, **kw)
    return o, g


def test_mha_reference_fixture(ctx):
    # TestPackedTernaryMHAProducesFiniteOutput fixture, poly/tests/bitnet_cpu_test.go:364-386: d_model 4, two heads of
    # dimension 2 (below the tiled kernels' vector width: the plain attention kernel computes it)
    s = split_mha_slab(deterministic_weights(80), 4, 2, 2, 2)
    om, gw = [], []
    for k in ("wq", "wk", "wv", "wo"):
        m, w = pair(ctx, s[k], 4, 4)
        om.append(m)
        gw.append(w)
    kw = dict(bq=s["bq"], bk=s["bk"], bv=s["bv"], bo=s["bo"])
    o = orc.MHA(4, 2, 2, 2, 8, 0.0, 0.0, *om, **kw)
    g = cabi.MHA(ctx, 4, 2, 2, 2, 8, 0.0, 0.0, *gw, **kw)
    x = np.array([0.1, -0.2, 0.3, -0.4, 0.2, -0.1, 0.4, -0.3], np.float32).reshape(2, 4)
    epre, epost = o.forward(x)
    pre, post = g.forward(x)
    assert np.isfinite(post).all()
    assert rel_err(pre, epre) <= REL and rel_err(post, epost) <= REL
    x1 = np.array([[0.05, 0.15, -0.25, 0.35]], np.float32)
    _, ep = o.forward(x1)
    _, gp = g.forward(x1)
    assert g.kv_offset == 3 and rel_err(gp, ep) <= REL
    g.close()


@pytest.mark.parametrize("D,heads,kvh,hd,seq,biases,norms", [(64, 4, 2, 16, 5, True, True), (256, 2, 1, 128, 12, False, False),
                                                             (2560, 20, 5, 128, 3, False, False)])
def test_mha_forward_prefill_then_decode(ctx, D, heads, kvh, hd, seq, biases, norms):
    rng = np.random.default_rng(D + seq)
    o, g = build_mha(ctx, rng, D, heads, kvh, hd, 64, 500000.0, 1e-5, biases, norms)
    x = rng.standard_normal((seq, D)).astype(np.float32)
    epre, epost = o.forward(x)
    pre, post = g.forward(x)
    assert g.kv_offset == o.kv_offset == seq
    assert rel_err(pre, epre) <= REL and rel_err(post, epost) <= REL
    ek, ev = o.cache()
    k, v = g.cache()
    assert rel_err(k[:seq], ek[:seq]) <= REL
    assert (v[:seq].view(np.uint32) == ev[:seq].view(np.uint32)).all()  # V rows: pure ternary linear, bit-exact
    for step in range(3):  # incremental decode keeps the ring
        x1 = rng.standard_normal((1, D)).astype(np.float32)
        _, ep = o.forward(x1)
        _, gp = g.forward(x1)
        assert rel_err(gp, ep) <= REL
    assert g.kv_offset == seq + 3
    # a multi-token call restarts the ring (mhaPrepareKVForForward)
    _, ep = o.forward(x[:2])
    _, gp = g.forward(x[:2])
    assert g.kv_offset == 2 and rel_err(gp, ep) <= REL
    g.close()


def test_mha_multi_batch_shares_one_ring(ctx):
    rng = np.random.default_rng(9)
    o, g = build_mha(ctx, rng, 64, 4, 4, 16, 32, 10000.0, 0.0)
    x = rng.standard_normal((2, 3, 64)).astype(np.float32)
    _, ep = o.forward(x)
    _, gp = g.forward(x)
    assert g.kv_offset == 6 and rel_err(gp, ep) <= REL
    with pytest.raises(loom_b200.LoomB200Error):  # beyond MaxSeqLen the reference's ring wraps silently: refused here
        g.forward(rng.standard_normal((40, 64)).astype(np.float32))
    g.close()


def make_decoder(ctx, rng, L, H, heads, kvh, hd, I, V, eps, theta, act, msl):
    import torch
    odec = orc.Decoder(L, H, heads, kvh, hd, I, V, eps, theta, act, msl)
    gdec = cabi.Decoder(ctx, L, H, heads, kvh, hd, I, V, eps, theta, act, msl)
    emb = (rng.standard_normal((V, H)) * 0.02).astype(np.float32)
    shapes = ((heads * hd, H), (kvh * hd, H), (kvh * hd, H), (H, heads * hd), (I, H), (I, H), (H, I))
    for b in range(L):
        masters = [(rng.standard_normal(r * c) * 0.02).astype(np.float32) for r, c in shapes]
        g1 = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        g2 = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        odec.set_block(b, *masters, g1=g1, g2=g2)
        ws = []
        for (r, c), mst in zip(shapes, masters):
            d = ctx.to_device(mst)
            ws.append(ctx.pack_ternary_f32(d, r, c))  # the device-side ternarizer, as the bench uses it
            ctx.free(d)
        gdec.set_block(b, ws, g1=g1, g2=g2)
    fg = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    odec.set_embeddings(emb, fg)
    emb_dev = ctx.to_device(emb)
    gdec.set_embeddings(emb_dev, fg)
    return odec, gdec


@pytest.mark.parametrize("L,H,heads,kvh,hd,I,V,act", [(2, 64, 4, 2, 16, 96, 101, cabi.ACT_SILU),
                                                      (3, 256, 2, 1, 128, 384, 500, cabi.ACT_RELU2)])
def test_decoder_logits_and_greedy_tokens(ctx, L, H, heads, kvh, hd, I, V, act):
    rng = np.random.default_rng(L * 100 + H)
    odec, gdec = make_decoder(ctx, rng, L, H, heads, kvh, hd, I, V, 1e-5, 500000.0, act, 128)
    prompt = rng.integers(0, V, 19).astype(np.int32)
    elog = odec.forward(prompt)
    glog = gdec.forward(prompt)
    assert gdec.kv_offset == 19
    assert np.max(np.abs(glog - elog)) <= 1e-5 * max(1.0, float(np.max(np.abs(elog))))
    assert int(np.argmax(glog)) == orc.argmax(elog)
    # one incremental step through the recorded frame
    nxt = np.array([orc.argmax(elog)], np.int32)
    e2 = odec.forward(nxt)
    g2 = gdec.forward(nxt)
    assert np.max(np.abs(g2 - e2)) <= 1e-5 * max(1.0, float(np.max(np.abs(e2))))
    # greedy generation: identical token streams
    etok, _, _ = odec.generate(prompt, 24, threads=4, attn_threads=4)
    gtok, m = gdec.generate(prompt, 24)
    assert (gtok == etok).all()
    assert m.generated_tokens == 24 and m.decode_device_seconds > 0
    # and again from a one-token prompt (fresh sequence, replayed frame)
    etok, _, _ = odec.generate(prompt[:1], 8)
    gtok, _ = gdec.generate(prompt[:1], 8)
    assert (gtok == etok).all()
    gdec.close()


def test_decoder_with_wide_rows(ctx):
    # hidden and heads*head_dim of 8192 columns: the block norms and the attention inner norm take the stand-alone
    # normalise-and-quantize launch instead of the prologue fused into the GEMV
    L, H, heads, kvh, hd, I, V = 1, 8192, 64, 8, 128, 512, 64
    rng = np.random.default_rng(8192)
    odec, gdec = make_decoder(ctx, rng, L, H, heads, kvh, hd, I, V, 1e-5, 500000.0, cabi.ACT_SILU, 32)
    prompt = rng.integers(0, V, 11).astype(np.int32)
    elog = odec.forward(prompt, threads=4)
    glog = gdec.forward(prompt)
    assert np.max(np.abs(glog - elog)) <= 1e-5 * max(1.0, float(np.max(np.abs(elog))))
    etok, _, _ = odec.generate(prompt, 6, threads=4, attn_threads=4)
    gtok, _ = gdec.generate(prompt, 6)
    assert (gtok == etok).all()
    gdec.close()


@pytest.mark.parametrize("n_prompt,H,heads,kvh,hd", [(32, 256, 4, 2, 64), (70, 256, 4, 2, 64), (150, 256, 4, 2, 64),
                                                      (97, 256, 2, 2, 128), (130, 512, 8, 1, 64), (45, 96, 3, 1, 32)])
def test_decoder_prompt_blocks_on_tensor_cores(ctx, n_prompt, H, heads, kvh, hd):
    # prompts of 32+ tokens run every projection as a token-block GEMM (tcgen05); the logits, the KV rings and the
    # greedy continuation must be those of the oracle, and of the eight-token GEMV path
    # (3 heads over 1 KV head does not divide 64 query rows: that shape keeps the per-token attention kernel)
    L, I, V = 2, 384, 300
    rng = np.random.default_rng(n_prompt)
    odec, gdec = make_decoder(ctx, rng, L, H, heads, kvh, hd, I, V, 1e-5, 500000.0, cabi.ACT_SILU, 256)
    prompt = rng.integers(0, V, n_prompt).astype(np.int32)
    elog = odec.forward(prompt, threads=4)
    glog = gdec.forward(prompt)
    tol = 1e-5 * max(1.0, float(np.max(np.abs(elog))))
    assert np.max(np.abs(glog - elog)) <= tol
    k_gemm, v_gemm = gdec.cache(L - 1)
    ctx.set_option("prefill_gemm", 0)
    try:
        slog = gdec.forward(prompt)
        k_gemv, v_gemv = gdec.cache(L - 1)
    finally:
        ctx.set_option("prefill_gemm", 1)
    assert np.max(np.abs(glog - slog)) <= tol
    # without the pre-expanded codes: tiles expanded in the kernel, gate and up as two GEMMs plus the gate-product kernel;
    # the arithmetic is the same, so the logits are the same bits
    ctx.set_option("gemm_cache", 0)
    try:
        xlog = gdec.forward(prompt)
    finally:
        ctx.set_option("gemm_cache", 1)
    assert (xlog.view(np.uint32) == glog.view(np.uint32)).all()
    assert np.allclose(k_gemm[:n_prompt], k_gemv[:n_prompt], rtol=1e-5, atol=1e-6)
    assert np.allclose(v_gemm[:n_prompt], v_gemv[:n_prompt], rtol=1e-5, atol=1e-6)
    etok, _, _ = odec.generate(prompt, 12, threads=4, attn_threads=4)
    gtok, _ = gdec.generate(prompt, 12)
    assert (gtok == etok).all()
    gdec.close()


def test_decoder_with_untied_ternary_lm_head(ctx):
    # with an untied head and exact dtypes the reference runs the LM head through the packed-ternary matvec
    # (poly/transformer.go:721-755): logits bit-exact up to the final norm's float64 reduction order, tokens identical
    L, H, heads, kvh, hd, I, V = 2, 256, 4, 2, 64, 384, 1000
    rng = np.random.default_rng(721)
    odec, gdec = make_decoder(ctx, rng, L, H, heads, kvh, hd, I, V, 1e-5, 500000.0, cabi.ACT_SILU, 128)
    head_master = (rng.standard_normal(V * H) * 0.02).astype(np.float32)
    om = orc.Matrix.from_f32(head_master, V, H)
    gw = ctx.upload_ternary(om.words, V, H, om.scale)
    odec.set_lm_head_ternary(om)
    gdec.set_lm_head_ternary(gw)
    prompt = rng.integers(0, V, 11).astype(np.int32)
    elog = odec.forward(prompt)
    glog = gdec.forward(prompt)
    assert np.max(np.abs(glog - elog)) <= 1e-5 * max(1.0, float(np.max(np.abs(elog))))
    assert (glog == elog).mean() > 0.99
    etok, _, _ = odec.generate(prompt, 12)
    gtok, _ = gdec.generate(prompt, 12)
    assert (gtok == etok).all()
    # a 40-token prompt: the token-block path ends in the same head
    prompt = rng.integers(0, V, 40).astype(np.int32)
    etok, _, _ = odec.generate(prompt, 6, threads=4)
    gtok, _ = gdec.generate(prompt, 6)
    assert (gtok == etok).all()
    gdec.close()
