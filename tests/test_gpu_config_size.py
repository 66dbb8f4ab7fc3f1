"""Decoder parity at the benchmark's own widths (BitNet-b1.58-2B shape: hidden 2560, 20 query / 5 KV heads x 128,
FFN 6912, vocabulary 128256), two blocks deep, against the CPU oracle:

  * a 160-token prompt through the token-block path (tcgen05 GEMMs + block attention): logits, then the residual
    stream of every block with the oracle's own block input fed in (teacher forcing), so that an error inside a block
    cannot hide behind, or be blamed on, a difference inherited from the block before;
  * one-token steps through the recorded decode frame at context > 1000 (KV rings restored from the same seeded
    rows on both sides; 14-way split attention): logits and 16 greedy tokens.

Bars: logits within 1e-5 * max|logit|; block outputs (which include the float32 residual additions, so single
elements can cancel to almost nothing) within 1e-6 of the row's largest magnitude on every element and bit-identical
on more than 99.9 % of them; tokens identical.
"""
import numpy as np
import pytest

import loom_b200
from loom_b200 import cabi
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

L, H, HEADS, KVH, HD, I, V = 2, 2560, 20, 5, 128, 6912, 128256
EPS, THETA, MSL = 1e-5, 500000.0, 2048
SHAPES = ((HEADS * HD, H), (KVH * HD, H), (KVH * HD, H), (H, HEADS * HD), (I, H), (I, H), (H, I))
THREADS = min(16, orc.host_threads())


def row_err(a, b):
    """max over rows of max|a - b| / max|b| (error relative to the row's largest magnitude)."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.max(np.abs(a - b), axis=1) / np.maximum(np.max(np.abs(b), axis=1), 1e-30)))


@pytest.fixture(scope="module")
def model():
    ctx = loom_b200.Context(0)
    rng = np.random.default_rng(2560)
    odec = orc.Decoder(L, H, HEADS, KVH, HD, I, V, EPS, THETA, orc.ACT_SILU, MSL)
    gdec = cabi.Decoder(ctx, L, H, HEADS, KVH, HD, I, V, EPS, THETA, cabi.ACT_SILU, MSL)
    blocks = []
    for b in range(L):
        masters = [(rng.standard_normal(r * c) * 0.02).astype(np.float32) for r, c in SHAPES]
        g1 = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        g2 = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        odec.set_block(b, *masters, g1=g1, g2=g2)
        ws = []
        for (r, c), mst in zip(SHAPES, masters):
            d = ctx.to_device(mst)
            ws.append(ctx.pack_ternary_f32(d, r, c))
            ctx.free(d)
        gdec.set_block(b, ws, g1=g1, g2=g2)
        blocks.append((ws, g1, g2))
    emb = (rng.standard_normal((V, H)) * 0.02).astype(np.float32)
    fg = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    odec.set_embeddings(emb, fg)
    emb_dev = ctx.to_device(emb)
    gdec.set_embeddings(emb_dev, fg)
    yield dict(ctx=ctx, odec=odec, gdec=gdec, blocks=blocks, emb=emb, rng=rng)
    gdec.close()
    ctx.close()


def test_prompt_on_tensor_cores_and_teacher_forced_blocks(model):
    ctx, odec, gdec, rng = model["ctx"], model["odec"], model["gdec"], model["rng"]
    n = 160
    prompt = rng.integers(0, V, n).astype(np.int32)
    elog, taps = odec.forward_taps(prompt, simd=1, threads=THREADS, attn_threads=THREADS)
    glog = gdec.forward(prompt)
    assert gdec.kv_offset == n
    assert np.max(np.abs(glog - elog)) <= 1e-5 * max(1.0, float(np.max(np.abs(elog))))
    assert int(np.argmax(glog)) == orc.argmax(elog)
    resid = gdec.last_residual(n)
    assert resid.shape == (n, H) and row_err(resid, taps[L - 1]) <= 1e-5  # two blocks deep: inherited differences allowed
    # teacher forcing: block b alone, fed the oracle's input of block b as an embedding table of n rows
    block_in = [model["emb"][prompt]] + [taps[b] for b in range(L - 1)]
    for b in range(L):
        ws, g1, g2 = model["blocks"][b]
        one = cabi.Decoder(ctx, 1, H, HEADS, KVH, HD, I, n, EPS, THETA, cabi.ACT_SILU, 256)
        one.set_block(0, ws, g1=g1, g2=g2)
        tab = ctx.to_device(np.ascontiguousarray(block_in[b], np.float32))
        one.set_embeddings(tab)
        one.forward(np.arange(n, dtype=np.int32), want_logits=False)
        out = one.last_residual(n)
        assert row_err(out, taps[b]) <= 1e-6, "block %d output differs from the oracle's" % b
        assert (out.view(np.uint32) == taps[b].view(np.uint32)).mean() > 0.999, "block %d: too few identical elements" % b
        one.close()
        ctx.free(tab)
    # greedy continuation after the prompt: identical tokens
    etok, _, _ = odec.generate(prompt, 4, simd=1, threads=THREADS, attn_threads=THREADS)
    gtok, _ = gdec.generate(prompt, 4)
    assert (gtok == etok).all()


def test_decode_frame_at_long_context(model):
    ctx, odec, gdec = model["ctx"], model["odec"], model["gdec"]
    rng = np.random.default_rng(1024)
    ctx_len, kvd = 1024, KVH * HD
    odec.reset()
    gdec.reset()
    for b in range(L):
        k = rng.standard_normal((ctx_len, kvd)).astype(np.float32)
        v = rng.standard_normal((ctx_len, kvd)).astype(np.float32)
        odec.set_kv(b, ctx_len, k, v)
        gdec.upload_cache(b, ctx_len, k, v)
    assert gdec.kv_offset == ctx_len
    tok = int(rng.integers(0, V))
    etoks, gtoks = [], []
    for step in range(16):
        elog = odec.forward(np.array([tok], np.int32), simd=1, threads=THREADS, attn_threads=THREADS)
        glog = gdec.forward(np.array([tok], np.int32))
        assert np.max(np.abs(glog - elog)) <= 1e-5 * max(1.0, float(np.max(np.abs(elog)))), "step %d" % step
        et, gt = orc.argmax(elog), int(np.argmax(glog))
        etoks.append(et)
        gtoks.append(gt)
        assert et == gt, "step %d: greedy token %d vs oracle %d" % (step, gt, et)
        tok = et
    assert gdec.kv_offset == ctx_len + 16
    # the device-resident greedy loop (argmax on the device, no host round trip) continues like the oracle
    elog = odec.forward(np.array([tok], np.int32), simd=1, threads=THREADS, attn_threads=THREADS)
    gdec.forward(np.array([tok], np.int32), want_logits=False)
    gdec.continue_greedy(6)
    ctx.sync()
    more = []
    for _ in range(6):
        t = orc.argmax(elog)
        more.append(t)
        elog = odec.forward(np.array([t], np.int32), simd=1, threads=THREADS, attn_threads=THREADS)
    got = gdec.generated_tokens(6)
    assert got.tolist() == more
