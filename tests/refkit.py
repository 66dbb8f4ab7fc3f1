"""Fixtures and independent numpy recomputations shared by the tests.

`deterministic_weights` is the input generator of the reference's own BitNet tests
(poly/tests/bitnet_cpu_test.go:10-20); the numpy functions recompute the integer parts of the
path independently of the C++ oracle so that the two can be checked against each other.
"""
import numpy as np


def deterministic_weights(n: int) -> np.ndarray:
    i = np.arange(n)
    v = ((i % 11) - 5).astype(np.float32) * np.float32(0.13)
    v = np.where(i % 7 == 0, v * np.float32(-0.5), v).astype(np.float32)
    return v


def round_half_away(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float64)
    return np.sign(x) * np.floor(np.abs(x) + 0.5)


def np_ternary_scale(w: np.ndarray) -> np.float32:
    w = np.asarray(w, dtype=np.float32).ravel()
    if w.size == 0:
        return np.float32(1.0)
    acc = 0.0
    for v in w.astype(np.float64):  # sequential fp64 sum, index order
        acc += abs(v)
    s = np.float32(acc / w.size)
    return np.float32(1.0) if s == 0 else s


def np_ternarize(w: np.ndarray, scale: np.float32) -> np.ndarray:
    w = np.asarray(w, dtype=np.float32)
    ratio = (w / np.float32(scale)).astype(np.float32)  # float32 division
    return np.clip(round_half_away(ratio), -1, 1).astype(np.int8)


def np_pack(q: np.ndarray, rows: int, cols: int) -> np.ndarray:
    q = np.asarray(q, dtype=np.int8).reshape(rows, cols)
    rw = (cols + 15) // 16
    words = np.zeros((rows, rw), dtype=np.uint32)
    code = (q.astype(np.int32) + 1).astype(np.uint32)
    for c in range(cols):
        words[:, c // 16] |= code[:, c] << np.uint32(2 * (c % 16))
    return words


def np_unpack(words: np.ndarray, rows: int, cols: int) -> np.ndarray:
    words = np.asarray(words, dtype=np.uint32).reshape(rows, -1)
    c = np.arange(cols)
    codes = (words[:, c // 16] >> (2 * (c % 16)).astype(np.uint32)) & np.uint32(3)
    return codes.astype(np.int32) - 1


def np_quantize(x: np.ndarray):
    x = np.asarray(x)
    amax = np.float32(np.max(np.abs(x.astype(np.float64))).astype(np.float32)) if x.size else np.float32(0)
    if amax < np.float32(1e-5):
        amax = np.float32(1e-5)
    s = 127.0 / np.float64(amax)
    q = np.clip(round_half_away(x.astype(np.float64) * s), -128, 127).astype(np.int8)
    return q, amax


def np_matvec(words, rows, cols, scale, xq, amax):
    w = np_unpack(words, rows, cols)
    acc = (w.astype(np.int64) @ np.asarray(xq, dtype=np.int64)[:cols]).astype(np.int32)
    os_ = np.float64(np.float32(scale)) * np.float64(np.float32(amax)) / 127.0
    if os_ == 0:
        os_ = 1.0
    return acc, acc.astype(np.float64) * os_


def split_mha_slab(master, d_model, heads, kv_heads, head_dim):
    """Slab offsets of an MHA WeightStore (poly/bitnet_cpu.go:453-458, poly/mha.go:233-240)."""
    qd, kvd = heads * head_dim, kv_heads * head_dim
    o = 0
    out = {}
    for name, n in (("wq", qd * d_model), ("wk", kvd * d_model), ("wv", kvd * d_model), ("wo", d_model * qd),
                    ("bq", qd), ("bk", kvd), ("bv", kvd), ("bo", d_model)):
        out[name] = np.asarray(master[o:o + n], dtype=np.float32)
        o += n
    return out


def split_swiglu_slab(master, hidden, inter):
    """Slab offsets of a SwiGLU WeightStore (poly/swiglu.go:275-280)."""
    w = hidden * inter
    o = 0
    out = {}
    for name, n in (("wg", w), ("wu", w), ("wd", w), ("bg", inter), ("bu", inter), ("bd", hidden)):
        out[name] = np.asarray(master[o:o + n], dtype=np.float32)
        o += n
    return out
