"""Independent sequences on one decoder (`loom_b200_decoder_set_batch` / `select` / `step_batch` / `continue_batch`).

The reference shares one KV ring across a batch (poly/mha.go:258-270), so serving several sequences at once is an
extension whose contract is stated through the oracle: every sequence must behave like a CPU decoder of its own that is
fed the same tokens.  The tests prefill every sequence with a prompt of its own length (single-sequence calls on the
selected sequence), then step all of them together: logits within 1e-5 * max|logit| of the per-sequence oracle, greedy
tokens identical.
"""
import numpy as np
import pytest

import loom_b200
from loom_b200 import cabi
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
THREADS = min(16, orc.host_threads())


def build(ctx, rng, B, L, H, heads, kvh, hd, I, V, msl, act=cabi.ACT_SILU):
    """One GPU decoder with B sequences and B oracle decoders that share the same packed weights."""
    shapes = ((heads * hd, H), (kvh * hd, H), (kvh * hd, H), (H, heads * hd), (I, H), (I, H), (H, I))
    gdec = cabi.Decoder(ctx, L, H, heads, kvh, hd, I, V, 1e-5, 500000.0, act, msl)
    gdec.set_batch(B)
    odecs = [orc.Decoder(L, H, heads, kvh, hd, I, V, 1e-5, 500000.0, act, msl) for _ in range(B)]
    for b in range(L):
        g1 = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        g2 = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        packed = [orc.pack_f32((rng.standard_normal(r * c) * 0.02).astype(np.float32), r, c) for r, c in shapes]
        for od in odecs:
            od.set_block_packed(b, [p[0] for p in packed], [p[1] for p in packed], g1=g1, g2=g2)
        ws = [ctx.upload_ternary(p[0], r, c, p[1]) for p, (r, c) in zip(packed, shapes)]
        gdec.set_block(b, ws, g1=g1, g2=g2)
    emb = (rng.standard_normal((V, H)) * 0.02).astype(np.float32)
    fg = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    for od in odecs:
        od.set_embeddings(emb, fg)
    gdec.set_embeddings(ctx.to_device(emb), fg)
    return gdec, odecs


def run_case(ctx, rng, B, dims, prompt_lens, steps, greedy_steps):
    gdec, odecs = build(ctx, rng, B, *dims)
    try:
        _run_case(gdec, odecs, rng, B, dims, prompt_lens, steps, greedy_steps)
    finally:
        gdec.close()  # before the context goes away


def _run_case(gdec, odecs, rng, B, dims, prompt_lens, steps, greedy_steps):
    V = dims[6]
    elogs = []
    for i in range(B):  # prompts of different lengths, one sequence at a time
        prompt = rng.integers(0, V, prompt_lens[i]).astype(np.int32)
        gdec.select(i)
        glog = gdec.forward(prompt)
        elog = odecs[i].forward(prompt, threads=THREADS)
        assert gdec.kv_offset == prompt_lens[i]
        assert np.max(np.abs(glog - elog)) <= 1e-5 * max(1.0, float(np.max(np.abs(elog)))), "prompt of sequence %d" % i
        elogs.append(elog)
    # teacher-forced steps: the same (arbitrary) token for a sequence on both sides
    for s in range(steps):
        toks = rng.integers(0, V, B).astype(np.int32)
        glogs = gdec.step_batch(toks)
        for i in range(B):
            elogs[i] = odecs[i].forward(toks[i:i + 1], threads=THREADS)
            assert np.max(np.abs(glogs[i] - elogs[i])) <= 1e-5 * max(1.0, float(np.max(np.abs(elogs[i])))), "step %d sequence %d" % (s, i)
            assert int(np.argmax(glogs[i])) == orc.argmax(elogs[i])
    for i in range(B):
        gdec.select(i)
        assert gdec.kv_offset == prompt_lens[i] + steps
    # greedy continuation of all sequences on the device
    gdec.continue_batch(greedy_steps)
    got = gdec.generated_tokens_batch(greedy_steps)
    for i in range(B):
        want = []
        logits = elogs[i]
        for _ in range(greedy_steps):
            t = orc.argmax(logits)
            want.append(t)
            logits = odecs[i].forward(np.array([t], np.int32), threads=THREADS)
        assert got[i].tolist() == want, "greedy tokens of sequence %d" % i


def test_three_sequences_small():
    ctx = loom_b200.Context(0)
    try:
        rng = np.random.default_rng(3)
        run_case(ctx, rng, 3, (2, 256, 4, 2, 64, 384, 300, 96), [9, 1, 40], 3, 6)
        # eleven sequences: two passes of the projections (eight + three), three passes of the head
        run_case(ctx, rng, 11, (1, 128, 2, 1, 64, 256, 200, 64), [3 + (i % 5) for i in range(11)], 2, 4)
    finally:
        ctx.close()


def test_sixteen_sequences_at_8b_widths():
    # Llama-3-8B-shaped widths (hidden 4096, 32 query / 8 KV heads x 128, FFN 14336, vocabulary 128256), one block
    ctx = loom_b200.Context(0)
    try:
        rng = np.random.default_rng(16)
        run_case(ctx, rng, 16, (1, 4096, 32, 8, 128, 14336, 128256, 64), [4 + (i % 7) for i in range(16)], 1, 2)
    finally:
        ctx.close()


def test_batch_calls_refuse_what_they_cannot_do():
    ctx = loom_b200.Context(0)
    try:
        rng = np.random.default_rng(5)
        gdec, _ = build(ctx, rng, 2, 1, 64, 4, 2, 16, 96, 50, 32)
        try:
            with pytest.raises(loom_b200.LoomB200Error):  # no prompts yet
                gdec.step_batch(np.array([1, 2], np.int32))
            with pytest.raises(loom_b200.LoomB200Error):
                gdec.select(2)
            with pytest.raises(loom_b200.LoomB200Error):  # after set_block
                gdec.set_batch(3)
        finally:
            gdec.close()
    finally:
        ctx.close()
