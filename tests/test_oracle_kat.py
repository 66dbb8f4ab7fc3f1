"""Pins the CPU oracle against the reference's own known-answer tests and fixtures.

Each test names the reference test it replays (paths relative to the openfluke/loom project).
The expected numbers are the ones written in those Go tests; nothing here needs a GPU.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from refkit import (deterministic_weights, np_matvec, np_pack, np_quantize, np_ternarize, np_ternary_scale,
                    np_unpack, split_mha_slab, split_swiglu_slab)


def test_absmean_quantizer_kat():
    # TestBitNetTernaryQuantizerUsesAbsMean, poly/tests/bitnet_cpu_test.go:134-153
    q, scale = orc.morph_ternary(np.array([-0.2, -0.8, 0.1, 0.8], np.float32))
    assert abs(float(scale) - 0.475) <= 1e-6
    assert q.tolist() == [0, -1, 0, 1]


def test_native_ternary_unit_scale():
    # TestBitNetNativeTernaryUsesUnitScale, poly/tests/bitnet_cpu_test.go:155-182: a master that is
    # already {-1,0,1} packs with scale 1 and keeps its values.
    w = np.array([-0.2, -0.8, 0.1, 0.8, 0.4, -0.3, 0.0, 0.9], np.float32)
    q, _ = orc.morph_ternary(w)
    native = q.astype(np.float32)
    words, scale = orc.pack_f32(native, 2, 4)
    assert scale == np.float32(1.0)
    assert (np_unpack(words, 2, 4).ravel() == q).all()


def test_microsoft_offline_decode_kat():
    # TestMicrosoftOfflinePackedBitNetRowsDecode, poly/tests/bitnet_cpu_test.go:334-362
    packed = np.array([0b10100001, 0b00011000, 0b10010000, 0b00001010], np.float32)
    words = orc.pack_microsoft_f32slots(packed, 8, 2)
    m = orc.Matrix.from_words(words, 8, 2, 1.0)
    m.set_scale(0.5)
    got = m.matvec(np.array([2, -3], np.int8), 127.0)
    want = [1.5, -2.5, -2.5, -2.5, 1, 1.5, 2.5, 2.5]
    assert np.max(np.abs(got - np.array(want))) <= 1e-6
    # and with the SIMD byte-code path
    got2 = m.matvec(np.array([2, -3], np.int8), 127.0, simd=1)
    assert (got2 == got).all()


def test_microsoft_bytes_match_float_slots():
    # TestSetMicrosoftBitNetPackedMatrixBytesMatchesFloatU8Slots, poly/tests/bitnet_cpu_test.go:284-315
    rows, cols = 8, 4
    b = np.array([(i * 17) & 0xFF for i in range((rows // 4) * cols)], np.uint8)
    wa = orc.pack_microsoft_u8(b, rows, cols)
    wb = orc.pack_microsoft_f32slots(b.astype(np.float32), rows, cols)
    assert (wa == wb).all()
    # code 3 is not a ternary code: the loader maps it to 1 (= weight 0)
    w = np_unpack(wa, rows, cols)
    assert set(np.unique(w)).issubset({-1, 0, 1})


def test_offline_packed_without_master():
    # TestGetBitNetTernaryMatrixFindsOfflinePackedWithoutMasterSlab, poly/tests/bitnet_cpu_test.go:317-332
    words = orc.pack_microsoft_f32slots(np.array([0x01, 0x10], np.float32), 4, 2)
    m = orc.Matrix.from_words(words, 4, 2, 1.0)
    assert (m.rows, m.cols) == (4, 2)


def test_tail_columns_kat():
    # TestBitNetTernaryKernelHandlesTailColumns, poly/tests/bitnet_cpu_test.go:216-247
    rows, cols = 3, 17
    w = deterministic_weights(rows * cols)
    m = orc.Matrix.from_f32(w, rows, cols)
    assert m.row_words == 2  # poly/tests/bitnet_cpu_test.go:270-272
    x = deterministic_weights(cols)
    xq, amax = orc.quantize_f32(x)
    got = m.matvec(xq, amax)
    os_ = float(np.float64(m.scale) * np.float64(amax) / 127.0)
    for r in range(rows):
        s = 0
        for c in range(cols):
            q = orc.lib().orc_quant_value(float(w[r * cols + c]), float(m.scale))
            s += int(xq[c]) * q
        assert abs(got[r] - s * os_) <= 1e-6
    # padding bits of the last word are zero
    assert (m.words[:, 1] >> np.uint32(2)).max() == 0


def test_packed_dense_matches_dequantized_path():
    # TestPackedTernaryDenseMatchesDequantizedPath, poly/tests/bitnet_cpu_test.go:184-214
    w = deterministic_weights(15)
    scale = np_ternary_scale(w)
    deq = np_ternarize(w, scale).astype(np.float32) * scale
    x = np.array([0.1, -0.2, 0.3, -0.4, 0.5, 0.6, -0.7, 0.8, -0.9, 1.0], np.float32).reshape(2, 5)
    ref = x.astype(np.float64) @ deq.reshape(3, 5).astype(np.float64).T
    m = orc.Matrix.from_f32(w, 3, 5)
    _, post = orc.dense_forward(m, orc.ACT_LINEAR, x)
    assert np.max(np.abs(post - ref)) <= 5e-3


@pytest.mark.parametrize("rows,cols", [(40, 70), (8, 64), (33, 65), (16, 128), (64, 2560), (128, 6912), (7, 191)])
def test_simd_matches_scalar_exactly(rows, cols):
    # TestBitNetTernaryDenseSimdMatchesScalar, poly/tests/bitnet_simd_test.go:13-45 and the shape sweep of
    # TestBitNetPackedMatVecMatchesScalar, poly/tests/bitnet_packed_test.go:15-52: the difference must be 0.
    w = deterministic_weights(rows * cols)
    x = deterministic_weights(2 * cols).reshape(2, cols)
    m = orc.Matrix.from_f32(w, rows, cols)
    _, a = orc.dense_forward(m, orc.ACT_LINEAR, x, simd=0)
    _, b = orc.dense_forward(m, orc.ACT_LINEAR, x, simd=1)
    _, c = orc.dense_forward(m, orc.ACT_LINEAR, x, simd=1, threads=4)
    assert (a == b).all() and (a == c).all()


def test_code_row_dot_kernel_sweep():
    # TestBitNetTernaryKernelMatchesGo, poly/simd/bitnet_ternary_test.go:11-36 (200 trials per width;
    # 25 here keep the CPU suite short, same widths, same value ranges)
    rng = np.random.default_rng(42)
    L = orc.lib()
    import ctypes as C
    for n in (32, 64, 96, 512, 1536, 4096):
        for _ in range(25):
            codes = rng.integers(0, 3, n).astype(np.uint8)
            acts = rng.integers(-128, 128, n).astype(np.int8)
            cp = codes.ctypes.data_as(C.POINTER(C.c_uint8))
            ap = acts.ctypes.data_as(C.POINTER(C.c_int8))
            want = int(codes.astype(np.int64) @ acts.astype(np.int64))
            assert L.orc_code_row_dot_scalar(cp, ap, n) == want
            assert L.orc_code_row_dot_avx2(cp, ap, n) == want


def test_mha_and_swiglu_finite_on_reference_fixtures():
    # TestPackedTernaryMHAProducesFiniteOutput / ...SwiGLU..., poly/tests/bitnet_cpu_test.go:364-409.
    # Same slabs (biases included, taken from the fixture tail), same inputs.
    x = np.array([0.1, -0.2, 0.3, -0.4, 0.2, -0.1, 0.4, -0.3], np.float32).reshape(2, 4)
    s = split_mha_slab(deterministic_weights(80), 4, 2, 2, 2)
    mats = [orc.Matrix.from_f32(s[k], r, c) for k, r, c in (("wq", 4, 4), ("wk", 4, 4), ("wv", 4, 4), ("wo", 4, 4))]
    mha = orc.MHA(4, 2, 2, 2, 8, 0.0, 0.0, *mats, bq=s["bq"], bk=s["bk"], bv=s["bv"], bo=s["bo"])
    _, post = mha.forward(x)
    assert post.shape == (2, 4) and np.isfinite(post).all()
    assert mha.kv_offset == 2

    g = split_swiglu_slab(deterministic_weights(88), 4, 6)
    gate, up, down = (orc.Matrix.from_f32(g["wg"], 6, 4), orc.Matrix.from_f32(g["wu"], 6, 4),
                      orc.Matrix.from_f32(g["wd"], 4, 6))
    _, post = orc.swiglu_forward(gate, up, down, x, act=orc.ACT_SILU, bias_gate=g["bg"], bias_up=g["bu"],
                                 bias_down=g["bd"])
    assert post.shape == (2, 4) and np.isfinite(post).all()


# ---- the oracle against an independent numpy recomputation ---------------------------------


@pytest.mark.parametrize("rows,cols,seed", [(3, 17, 0), (16, 128, 1), (33, 65, 2), (128, 2560, 3), (7, 191, 4)])
def test_oracle_matches_numpy_recomputation(rows, cols, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(rows * cols) * 0.02).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    scale = np_ternary_scale(w)
    q = np_ternarize(w, scale)
    words = np_pack(q, rows, cols)
    ow, os_ = orc.pack_f32(w, rows, cols)
    assert os_ == scale
    assert (ow == words).all()
    xq, amax = np_quantize(x)
    oq, oamax = orc.quantize_f32(x)
    assert oamax == amax and (oq == xq).all()
    acc, y = np_matvec(words, rows, cols, scale, xq, amax)
    m = orc.Matrix.from_words(ow, rows, cols, os_)
    assert (m.acc_i32(xq) == acc).all()
    for simd in (0, 1):
        assert (m.matvec(xq, amax, simd=simd, threads=3) == y).all()


def test_quantize_edge_cases():
    # all-zero row: amax floors at 1e-5 (float32), every q is 0
    q, amax = orc.quantize_f32(np.zeros(8, np.float32))
    assert amax == np.float32(1e-5) and not q.any()
    # exact .5 ties round away from zero: x*127/amax = 0.5 when x = amax/254
    x = np.array([127.0, 0.5, -0.5, 1.5, -1.5, 2.5], np.float32)
    q, amax = orc.quantize_f32(x)
    assert amax == np.float32(127.0)
    assert q.tolist() == [127, 1, -1, 2, -2, 3]
    # the float64 twin used before the O projection
    q2, amax2 = orc.quantize_f64(x.astype(np.float64))
    assert amax2 == amax and (q2 == q).all()
    # -amax maps to -127, never -128
    q, _ = orc.quantize_f32(np.array([-3.0, 3.0], np.float32))
    assert q.tolist() == [-127, 127]


def test_zero_matrix_and_zero_scale_rule():
    # all-zero master: absmean 0 -> scale 1, every code is 1 (weight 0) -- and a zero master is "already ternary"
    words, scale = orc.pack_f32(np.zeros(32, np.float32), 2, 16)
    assert scale == np.float32(1.0)
    assert (np_unpack(words, 2, 16) == 0).all()


def test_gate_product_and_activations():
    assert orc.gate_product(-2.0, 3.0, orc.ACT_RELU2) == 0.0
    assert orc.gate_product(2.0, 3.0, orc.ACT_RELU2) == 12.0
    g, u = 0.7, -1.3
    assert orc.gate_product(g, u, orc.ACT_SILU) == (g * (1.0 / (1.0 + np.exp(-g)))) * u
    v = np.array([-1.5, 0.0, 2.0], np.float32)
    assert orc.activate_f32(v, orc.ACT_RELU).tolist() == [0.0, 0.0, 2.0]
    assert orc.activate_f32(v, orc.ACT_RELU2).tolist() == [0.0, 0.0, 4.0]
    assert orc.activate_f32(v, orc.ACT_LINEAR).tolist() == v.tolist()


def test_inner_norm_defaults():
    x = np.array([1.0, -2.0, 3.0, 0.5], np.float32)
    n0 = orc.inner_rmsnorm_f32(x, None, 0.0)  # eps <= 0 -> 1e-5
    n1 = orc.inner_rmsnorm_f32(x, None, 1e-5)
    assert (n0 == n1).all()
    sc = 1.0 / np.sqrt(np.sum(x.astype(np.float64) ** 2) / 4 + 1e-5)
    assert (n0 == (x.astype(np.float64) * sc).astype(np.float32)).all()
    # weights shorter than the row: the rest use 1.0 (poly/bitnet_cpu.go:906-911)
    nw = orc.inner_rmsnorm_f32(x, np.array([2.0], np.float32), 1e-5)
    assert nw[0] == np.float32(np.float64(x[0]) * sc * 2.0) and (nw[1:] == n0[1:]).all()


def test_decoder_tiny_prefill_equals_incremental():
    # A tiny HF-style decoder like newTinyHFTransformer (poly/tests/pipeline_forward_test.go:9-39):
    # feeding the prompt at once or token by token must give the same last-token logits (the KV ring
    # keeps state across incremental steps), and generation must be deterministic.
    rng = np.random.default_rng(7)
    L, H, heads, kvh, hd, I, V = 2, 8, 2, 1, 4, 16, 32
    dec = orc.Decoder(L, H, heads, kvh, hd, I, V, 1e-5, 10000.0, orc.ACT_SILU, 64)
    emb = (rng.standard_normal((V, H)) * 0.5).astype(np.float32)
    for b in range(L):
        ws = [(rng.standard_normal(r * c) * 0.02).astype(np.float32)
              for r, c in ((heads * hd, H), (kvh * hd, H), (kvh * hd, H), (H, heads * hd), (I, H), (I, H), (H, I))]
        dec.set_block(b, *ws)
    dec.set_embeddings(emb)
    prompt = rng.integers(0, V, 5).astype(np.int32)
    dec.reset()
    full = dec.forward(prompt)
    dec.reset()
    dec.forward(prompt[:1])
    for t in prompt[1:]:
        inc = dec.forward(np.array([t], np.int32))
    assert np.allclose(full, inc, rtol=1e-6, atol=1e-7)
    a, _, _ = dec.generate(prompt, 6)
    b, _, _ = dec.generate(prompt, 6, simd=1, threads=2, attn_threads=2)
    assert (a == b).all()


def test_summation_order_of_the_norm_statistics_is_bounded():
    # The reference adds the squares of a row one after the other in float64 (poly/bitnet_cpu.go:893-913); the GPU
    # kernels add them as trees of partial sums.  What that can change: the sum by some tens of units in its last place, the
    # normalised float32 values in their last bit on a few elements, and an int8 code by one where a value sits on a
    # rounding boundary.  The bound is shown here on the CPU: oracle (sequential) against a pairwise recomputation.
    rng = np.random.default_rng(893)
    flips = total = 0
    for K in (2560, 6912):
        for _ in range(8):
            x = rng.standard_normal(K).astype(np.float32)
            w = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
            y_seq = orc.inner_rmsnorm_f32(x, w, 1e-5)  # the oracle: sequential sum
            xd = x.astype(np.float64)
            sq = xd * xd
            ss_seq = 0.0
            for v in sq:
                ss_seq += v
            ss_tree = float(np.sum(sq.reshape(-1, 256).sum(axis=1)))  # partial sums of 256, then their sum
            assert abs(ss_tree - ss_seq) <= 4 * np.sqrt(K) * np.spacing(ss_seq)  # random-walk growth of the sequential sum's rounding
            sc = 1.0 / np.sqrt(ss_tree / K + 1e-5)
            y_tree = ((xd * sc).astype(np.float64) * w.astype(np.float64)).astype(np.float32)
            assert np.max(np.abs(y_tree.astype(np.float64) - y_seq.astype(np.float64))) <= 2 * np.max(np.spacing(np.abs(y_seq)))
            q_seq, a_seq = orc.quantize_f32(y_seq)
            q_tree, a_tree = orc.quantize_f32(y_tree)
            d = np.abs(q_seq.astype(np.int32) - q_tree.astype(np.int32))
            assert d.max() <= 1
            flips += int((d != 0).sum())
            total += K
    assert flips <= total // 1000  # a code moves only where a value sits within an ulp of a rounding boundary
