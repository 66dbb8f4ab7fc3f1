"""ctypes binding of the CPU oracle (oracle/loom_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline legs.  Nothing in the product package imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libloom_oracle.so")

ACT_RELU, ACT_SILU, ACT_GELU, ACT_TANH, ACT_SIGMOID, ACT_LEAKY_RELU, ACT_RELU2, ACT_LINEAR = 0, 1, 2, 3, 4, 5, 6, -1


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (g++ only; no GPU needed)."""
    src = [os.path.join(_HERE, f) for f in ("loom_oracle.cpp", "loom_oracle.h", "Makefile")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src
    )
    if stale:
        env = dict(os.environ)
        env.pop("CXX", None)
        env.pop("CXXFLAGS", None)
        subprocess.run(["make", "-C", _HERE, "CXX=g++"], check=True, env=env, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _declare(_lib)
    return _lib


_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_i8p = C.POINTER(C.c_int8)
_u8p = C.POINTER(C.c_uint8)
_i32p = C.POINTER(C.c_int32)
_u32p = C.POINTER(C.c_uint32)
_vp = C.c_void_p


def _declare(L):
    L.orc_ternary_scale.restype = C.c_float
    L.orc_ternary_scale.argtypes = [_f32p, C.c_size_t]
    L.orc_quant_value.restype = C.c_int
    L.orc_quant_value.argtypes = [C.c_float, C.c_float]
    L.orc_row_words.restype = C.c_int
    L.orc_row_words.argtypes = [C.c_int]
    L.orc_pack_f32.restype = C.c_int
    L.orc_pack_f32.argtypes = [_f32p, C.c_int, C.c_int, _u32p, _f32p]
    L.orc_morph_ternary.restype = C.c_float
    L.orc_morph_ternary.argtypes = [_f32p, C.c_size_t, _i8p]
    L.orc_pack_native.restype = C.c_int
    L.orc_pack_native.argtypes = [_i8p, C.c_int, C.c_int, _u32p]
    L.orc_pack_microsoft_u8.restype = C.c_int
    L.orc_pack_microsoft_u8.argtypes = [_u8p, C.c_int, C.c_int, _u32p]
    L.orc_pack_microsoft_f32slots.restype = C.c_int
    L.orc_pack_microsoft_f32slots.argtypes = [_f32p, C.c_int, C.c_int, _u32p]
    L.orc_quantize_f32.restype = C.c_float
    L.orc_quantize_f32.argtypes = [_f32p, C.c_int, _i8p]
    L.orc_quantize_f64.restype = C.c_float
    L.orc_quantize_f64.argtypes = [_f64p, C.c_int, _i8p]
    L.orc_matvec_i32.restype = None
    L.orc_matvec_i32.argtypes = [_u32p, C.c_int, C.c_int, _i8p, _i32p]
    L.orc_code_row_dot_scalar.restype = C.c_int32
    L.orc_code_row_dot_scalar.argtypes = [_u8p, _i8p, C.c_int]
    L.orc_code_row_dot_avx2.restype = C.c_int32
    L.orc_code_row_dot_avx2.argtypes = [_u8p, _i8p, C.c_int]
    L.orc_has_avx2.restype = C.c_int
    L.orc_gate_product.restype = C.c_double
    L.orc_gate_product.argtypes = [C.c_double, C.c_double, C.c_int]
    L.orc_activate_f32.restype = C.c_float
    L.orc_activate_f32.argtypes = [C.c_float, C.c_int]
    L.orc_inner_rmsnorm_f32.restype = None
    L.orc_inner_rmsnorm_f32.argtypes = [_f32p, C.c_int, _f32p, C.c_int, C.c_double]
    L.orc_inner_rmsnorm_f64.restype = None
    L.orc_inner_rmsnorm_f64.argtypes = [_f64p, C.c_int, _f32p, C.c_int, C.c_double]
    L.orc_block_rmsnorm.restype = None
    L.orc_block_rmsnorm.argtypes = [_f32p, C.c_int, C.c_int, _f32p, C.c_double, _f32p, _f32p]
    L.orc_matrix_from_words.restype = _vp
    L.orc_matrix_from_words.argtypes = [_u32p, C.c_int, C.c_int, C.c_float]
    L.orc_matrix_from_f32.restype = _vp
    L.orc_matrix_from_f32.argtypes = [_f32p, C.c_int, C.c_int]
    L.orc_matrix_free.restype = None
    L.orc_matrix_free.argtypes = [_vp]
    for n in ("rows", "cols", "row_words"):
        f = getattr(L, "orc_matrix_" + n)
        f.restype = C.c_int
        f.argtypes = [_vp]
    L.orc_matrix_scale.restype = C.c_float
    L.orc_matrix_scale.argtypes = [_vp]
    L.orc_matrix_set_scale.restype = None
    L.orc_matrix_set_scale.argtypes = [_vp, C.c_float]
    L.orc_matrix_words.restype = _u32p
    L.orc_matrix_words.argtypes = [_vp]
    L.orc_matrix_matvec.restype = C.c_int
    L.orc_matrix_matvec.argtypes = [_vp, _i8p, C.c_float, _f64p, C.c_int, C.c_int]
    L.orc_dense_forward.restype = C.c_int
    L.orc_dense_forward.argtypes = [_vp, C.c_int, _f32p, C.c_int, _f32p, _f32p, C.c_int, C.c_int]
    L.orc_swiglu_forward.restype = C.c_int
    L.orc_swiglu_forward.argtypes = [_vp, _vp, _vp, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_double, C.c_int,
                                     _f32p, C.c_int, _f32p, _f32p, _i8p, _f32p, _f32p, _i8p, _f32p, C.c_int, C.c_int]
    L.orc_mha_create.restype = _vp
    L.orc_mha_create.argtypes = [C.c_int] * 5 + [C.c_double, C.c_double] + [_vp] * 4 + [_f32p] * 4 + [
        _f32p, C.c_int, _f32p, C.c_int, _f32p, C.c_int]
    L.orc_mha_free.restype = None
    L.orc_mha_free.argtypes = [_vp]
    L.orc_mha_reset.restype = None
    L.orc_mha_reset.argtypes = [_vp]
    L.orc_mha_kv_offset.restype = C.c_int
    L.orc_mha_kv_offset.argtypes = [_vp]
    L.orc_mha_cache_k.restype = _f32p
    L.orc_mha_cache_k.argtypes = [_vp]
    L.orc_mha_cache_v.restype = _f32p
    L.orc_mha_cache_v.argtypes = [_vp]
    L.orc_mha_forward.restype = C.c_int
    L.orc_mha_forward.argtypes = [_vp, _f32p, C.c_int, C.c_int, _f32p, _f32p, _f64p, _f64p, C.c_int, C.c_int, C.c_int]
    L.orc_decoder_create.restype = _vp
    L.orc_decoder_create.argtypes = [C.c_int] * 7 + [C.c_double, C.c_double, C.c_int, C.c_int]
    L.orc_decoder_free.restype = None
    L.orc_decoder_free.argtypes = [_vp]
    L.orc_decoder_set_block.restype = C.c_int
    L.orc_decoder_set_block.argtypes = [_vp, C.c_int] + [_f32p] * 9
    L.orc_decoder_set_block_packed.restype = C.c_int
    L.orc_decoder_set_block_packed.argtypes = [_vp, C.c_int, _f32p, _f32p, C.POINTER(_u32p), _f32p]
    L.orc_decoder_set_embeddings.restype = C.c_int
    L.orc_decoder_set_embeddings.argtypes = [_vp, _f32p, _f32p]
    L.orc_decoder_set_lm_head_ternary.restype = C.c_int
    L.orc_decoder_set_lm_head_ternary.argtypes = [_vp, _vp]
    L.orc_decoder_set_kv.restype = C.c_int
    L.orc_decoder_set_kv.argtypes = [_vp, C.c_int, C.c_int, _f32p, _f32p]
    L.orc_decoder_reset.restype = None
    L.orc_decoder_reset.argtypes = [_vp]
    L.orc_decoder_forward.restype = C.c_int
    L.orc_decoder_forward.argtypes = [_vp, _i32p, C.c_int, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
    L.orc_decoder_forward_taps.restype = C.c_int
    L.orc_decoder_forward_taps.argtypes = [_vp, _i32p, C.c_int, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
    L.orc_decoder_generate.restype = C.c_int
    L.orc_decoder_generate.argtypes = [_vp, _i32p, C.c_int, C.c_int, _i32p, _f64p, _f64p, C.c_int, C.c_int, C.c_int]
    L.orc_argmax.restype = C.c_int
    L.orc_argmax.argtypes = [_f32p, C.c_int]
    L.orc_lm_head.restype = None
    L.orc_lm_head.argtypes = [_f32p, _f32p, C.c_int, C.c_int, _f32p, C.c_int]


def _p(a, ty):
    return None if a is None else a.ctypes.data_as(ty)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


def host_threads() -> int:
    return os.cpu_count() or 1


# ---- thin numpy wrappers ----------------------------------------------------------------


def row_words(cols: int) -> int:
    return (cols + 15) // 16


def ternary_scale(w) -> np.float32:
    w = _c(w, np.float32).ravel()
    return np.float32(lib().orc_ternary_scale(_p(w, _f32p), w.size))


def pack_f32(w, rows: int, cols: int):
    w = _c(w, np.float32).ravel()
    assert w.size >= rows * cols
    words = np.zeros(rows * row_words(cols), dtype=np.uint32)
    sc = C.c_float(0)
    rc = lib().orc_pack_f32(_p(w, _f32p), rows, cols, _p(words, _u32p), C.byref(sc))
    assert rc == 0
    return words.reshape(rows, row_words(cols)), np.float32(sc.value)


def morph_ternary(w):
    w = _c(w, np.float32).ravel()
    q = np.zeros(w.size, dtype=np.int8)
    s = lib().orc_morph_ternary(_p(w, _f32p), w.size, _p(q, _i8p))
    return q, np.float32(s)


def pack_native(q, rows: int, cols: int):
    q = _c(q, np.int8).ravel()
    words = np.zeros(rows * row_words(cols), dtype=np.uint32)
    assert lib().orc_pack_native(_p(q, _i8p), rows, cols, _p(words, _u32p)) == 0
    return words.reshape(rows, row_words(cols))


def pack_microsoft_u8(packed, rows: int, cols: int):
    packed = _c(packed, np.uint8).ravel()
    words = np.zeros(rows * row_words(cols), dtype=np.uint32)
    assert lib().orc_pack_microsoft_u8(_p(packed, _u8p), rows, cols, _p(words, _u32p)) == 0
    return words.reshape(rows, row_words(cols))


def pack_microsoft_f32slots(packed, rows: int, cols: int):
    packed = _c(packed, np.float32).ravel()
    words = np.zeros(rows * row_words(cols), dtype=np.uint32)
    assert lib().orc_pack_microsoft_f32slots(_p(packed, _f32p), rows, cols, _p(words, _u32p)) == 0
    return words.reshape(rows, row_words(cols))


def quantize_f32(x):
    x = _c(x, np.float32).ravel()
    q = np.zeros(x.size, dtype=np.int8)
    amax = lib().orc_quantize_f32(_p(x, _f32p), x.size, _p(q, _i8p))
    return q, np.float32(amax)


def quantize_f64(x):
    x = _c(x, np.float64).ravel()
    q = np.zeros(x.size, dtype=np.int8)
    amax = lib().orc_quantize_f64(_p(x, _f64p), x.size, _p(q, _i8p))
    return q, np.float32(amax)


def quantize_rows_f32(x):
    x = _c(x, np.float32)
    q = np.zeros(x.shape, dtype=np.int8)
    amax = np.zeros(x.shape[0], dtype=np.float32)
    for i in range(x.shape[0]):
        q[i], amax[i] = quantize_f32(x[i])
    return q, amax


def matvec_i32(words, rows: int, cols: int, xq):
    words = _c(words, np.uint32).ravel()
    xq = _c(xq, np.int8).ravel()
    acc = np.zeros(rows, dtype=np.int32)
    lib().orc_matvec_i32(_p(words, _u32p), rows, cols, _p(xq, _i8p), _p(acc, _i32p))
    return acc


def gate_product(g: float, u: float, act: int) -> float:
    return lib().orc_gate_product(g, u, act)


def activate_f32(v, act: int):
    v = _c(v, np.float32)
    out = np.empty_like(v)
    flat, o = v.ravel(), out.ravel()
    L = lib()
    for i in range(flat.size):
        o[i] = L.orc_activate_f32(float(flat[i]), act)
    return out


def inner_rmsnorm_f32(x, weight=None, eps: float = 0.0):
    x = np.array(x, dtype=np.float32, copy=True).ravel()
    w = _c(weight, np.float32)
    lib().orc_inner_rmsnorm_f32(_p(x, _f32p), x.size, _p(w, _f32p), 0 if w is None else w.size, eps)
    return x


def inner_rmsnorm_f64(x, weight=None, eps: float = 0.0):
    x = np.array(x, dtype=np.float64, copy=True).ravel()
    w = _c(weight, np.float32)
    lib().orc_inner_rmsnorm_f64(_p(x, _f64p), x.size, _p(w, _f32p), 0 if w is None else w.size, eps)
    return x


def block_rmsnorm(x, gain=None, eps: float = 0.0):
    x = _c(x, np.float32)
    rows, n = x.shape
    g = _c(gain, np.float32)
    out = np.empty_like(x)
    lib().orc_block_rmsnorm(_p(x, _f32p), rows, n, _p(g, _f32p), eps, _p(out, _f32p), None)
    return out


def lm_head(hidden, head, threads: int = 1):
    hidden = _c(hidden, np.float32).ravel()
    head = _c(head, np.float32)
    vocab, hs = head.shape
    logits = np.empty(vocab, dtype=np.float32)
    lib().orc_lm_head(_p(hidden, _f32p), _p(head, _f32p), vocab, hs, _p(logits, _f32p), threads)
    return logits


def argmax(logits) -> int:
    logits = _c(logits, np.float32).ravel()
    return lib().orc_argmax(_p(logits, _f32p), logits.size)


class Matrix:
    """BitNetTernaryMatrix stand-in (poly/bitnet_cpu.go:16-43)."""

    def __init__(self, handle):
        assert handle
        self.h = handle
        L = lib()
        self.rows = L.orc_matrix_rows(handle)
        self.cols = L.orc_matrix_cols(handle)
        self.row_words = L.orc_matrix_row_words(handle)

    @classmethod
    def from_f32(cls, w, rows, cols):
        w = _c(w, np.float32).ravel()
        assert w.size >= rows * cols
        return cls(lib().orc_matrix_from_f32(_p(w, _f32p), rows, cols))

    @classmethod
    def from_words(cls, words, rows, cols, scale):
        words = _c(words, np.uint32).ravel()
        assert words.size >= rows * row_words(cols)
        return cls(lib().orc_matrix_from_words(_p(words, _u32p), rows, cols, float(scale)))

    @property
    def scale(self) -> np.float32:
        return np.float32(lib().orc_matrix_scale(self.h))

    def set_scale(self, s):
        lib().orc_matrix_set_scale(self.h, float(s))

    @property
    def words(self):
        n = self.rows * self.row_words
        return np.ctypeslib.as_array(lib().orc_matrix_words(self.h), shape=(n,)).copy().reshape(self.rows, self.row_words)

    def matvec(self, xq, amax, simd=0, threads=1):
        xq = _c(xq, np.int8).ravel()
        assert xq.size >= self.cols
        out = np.empty(self.rows, dtype=np.float64)
        rc = lib().orc_matrix_matvec(self.h, _p(xq, _i8p), float(amax), _p(out, _f64p), simd, threads)
        assert rc == 0
        return out

    def acc_i32(self, xq):
        return matvec_i32(self.words, self.rows, self.cols, xq)

    def __del__(self):
        try:
            if self.h:
                lib().orc_matrix_free(self.h)
                self.h = None
        except Exception:
            pass


def dense_forward(m: Matrix, act: int, x, simd=0, threads=1):
    x = _c(x, np.float32)
    batch = x.shape[0]
    pre = np.empty((batch, m.rows), dtype=np.float32)
    post = np.empty((batch, m.rows), dtype=np.float32)
    rc = lib().orc_dense_forward(m.h, act, _p(x, _f32p), batch, _p(pre, _f32p), _p(post, _f32p), simd, threads)
    assert rc == 0
    return pre, post


def swiglu_forward(gate: Matrix, up: Matrix, down: Matrix, x, act=ACT_SILU, bias_gate=None, bias_up=None,
                   bias_down=None, inner_w=None, eps=0.0, simd=0, threads=1, taps=False):
    x = _c(x, np.float32)
    seq, H = x.shape
    I = gate.rows
    pre = np.empty((seq, I), dtype=np.float32)
    post = np.empty((seq, H), dtype=np.float32)
    bg, bu, bd, iw = (_c(a, np.float32) for a in (bias_gate, bias_up, bias_down, inner_w))
    t = {}
    if taps:
        t = dict(q_in=np.empty((seq, H), np.int8), amax_in=np.empty(seq, np.float32),
                 raw_prod=np.empty((seq, I), np.float32), q_pre=np.empty((seq, I), np.int8),
                 amax_pre=np.empty(seq, np.float32))
    rc = lib().orc_swiglu_forward(gate.h, up.h, down.h, _p(bg, _f32p), _p(bu, _f32p), _p(bd, _f32p), _p(iw, _f32p),
                                  0 if iw is None else iw.size, eps, act, _p(x, _f32p), seq, _p(pre, _f32p),
                                  _p(post, _f32p), _p(t.get("q_in"), _i8p), _p(t.get("amax_in"), _f32p),
                                  _p(t.get("raw_prod"), _f32p), _p(t.get("q_pre"), _i8p), _p(t.get("amax_pre"), _f32p),
                                  simd, threads)
    assert rc == 0
    return (pre, post, t) if taps else (pre, post)


class MHA:
    """The MHA layer with its ring KV cache (poly/mha.go:204-371)."""

    def __init__(self, d_model, heads, kv_heads, head_dim, max_seq_len, theta, eps, wq, wk, wv, wo, bq=None, bk=None,
                 bv=None, bo=None, q_norm=None, k_norm=None, inner_w=None):
        self.mats = (wq, wk, wv, wo)  # keep alive
        self.d_model, self.heads, self.kv_heads, self.head_dim = d_model, heads, kv_heads or heads, head_dim
        self.msl = max_seq_len or 512
        a = [_c(v, np.float32) for v in (bq, bk, bv, bo, q_norm, k_norm, inner_w)]
        self.h = lib().orc_mha_create(d_model, heads, kv_heads, head_dim, max_seq_len, theta, eps, wq.h, wk.h, wv.h,
                                      wo.h, _p(a[0], _f32p), _p(a[1], _f32p), _p(a[2], _f32p), _p(a[3], _f32p),
                                      _p(a[4], _f32p), 0 if a[4] is None else a[4].size, _p(a[5], _f32p),
                                      0 if a[5] is None else a[5].size, _p(a[6], _f32p),
                                      0 if a[6] is None else a[6].size)
        assert self.h

    def reset(self):
        lib().orc_mha_reset(self.h)

    @property
    def kv_offset(self):
        return lib().orc_mha_kv_offset(self.h)

    def cache(self):
        kvd = self.kv_heads * self.head_dim
        k = np.ctypeslib.as_array(lib().orc_mha_cache_k(self.h), shape=(self.msl, kvd)).copy()
        v = np.ctypeslib.as_array(lib().orc_mha_cache_v(self.h), shape=(self.msl, kvd)).copy()
        return k, v

    def forward(self, x, simd=0, threads=1, attn_threads=1, taps=False):
        x = _c(x, np.float32)
        if x.ndim == 2:
            batch, seq = 1, x.shape[0]
        else:
            batch, seq = x.shape[0], x.shape[1]
        pre = np.empty((batch * seq, self.d_model), np.float32)
        post = np.empty((batch * seq, self.d_model), np.float32)
        qd = self.heads * self.head_dim
        qt = np.empty((batch * seq, qd), np.float64) if taps else None
        at = np.empty((batch * seq, qd), np.float64) if taps else None
        rc = lib().orc_mha_forward(self.h, _p(x, _f32p), batch, seq, _p(pre, _f32p), _p(post, _f32p), _p(qt, _f64p),
                                   _p(at, _f64p), simd, threads, attn_threads)
        assert rc == 0
        return (pre, post, qt, at) if taps else (pre, post)

    def __del__(self):
        try:
            if self.h:
                lib().orc_mha_free(self.h)
                self.h = None
        except Exception:
            pass


class Decoder:
    """InitHFDecoderBlocks + Transformer restated (poly/hf_decoder.go:20-68, poly/transformer.go)."""

    def __init__(self, layers, hidden, heads, kv_heads, head_dim, inter, vocab, eps, theta, act=ACT_SILU,
                 max_seq_len=2048):
        self.dims = dict(layers=layers, hidden=hidden, heads=heads, kv_heads=kv_heads, head_dim=head_dim, inter=inter,
                         vocab=vocab)
        self.h = lib().orc_decoder_create(layers, hidden, heads, kv_heads, head_dim, inter, vocab, eps, theta, act,
                                          max_seq_len)
        self._keep = []
        self.max_seq_len = max_seq_len

    def set_block(self, b, wq, wk, wv, wo, wg, wu, wd, g1=None, g2=None):
        a = [_c(v, np.float32) for v in (g1, wq, wk, wv, wo, g2, wg, wu, wd)]
        rc = lib().orc_decoder_set_block(self.h, b, *[_p(v, _f32p) for v in a])
        assert rc == 0

    def set_block_packed(self, b, words7, scales7, g1=None, g2=None):
        ws = [_c(w, np.uint32).ravel() for w in words7]
        arr = (_u32p * 7)(*[_p(w, _u32p) for w in ws])
        sc = _c(scales7, np.float32)
        g1, g2 = _c(g1, np.float32), _c(g2, np.float32)
        rc = lib().orc_decoder_set_block_packed(self.h, b, _p(g1, _f32p), _p(g2, _f32p), arr, _p(sc, _f32p))
        assert rc == 0

    def set_embeddings(self, emb, final_gain=None):
        emb = _c(emb, np.float32)
        fg = _c(final_gain, np.float32)
        self._keep.append(emb)
        assert lib().orc_decoder_set_embeddings(self.h, _p(emb, _f32p), _p(fg, _f32p)) == 0

    def set_lm_head_ternary(self, head: "Matrix"):
        """Untied LM head as a packed ternary matrix [vocab, hidden] (poly/transformer.go:721-755)."""
        self._keep.append(head)
        assert lib().orc_decoder_set_lm_head_ternary(self.h, head.h) == 0

    def set_kv(self, block, kv_offset, k, v):
        """Restores a block's KV rings: rows [0, kv_offset) of k and v ([rows, kv_heads * head_dim]); rows the caller
        does not give are zero (the C side copies the whole ring of max_seq_len rows)."""
        kvd = self.dims["kv_heads"] * self.dims["head_dim"]
        full = []
        for a in (k, v):
            a = np.asarray(a, np.float32).reshape(-1, kvd)
            assert kv_offset <= a.shape[0] <= self.max_seq_len
            ring = np.zeros((self.max_seq_len, kvd), np.float32)
            ring[:a.shape[0]] = a
            full.append(ring)
        k, v = full
        assert lib().orc_decoder_set_kv(self.h, block, kv_offset, _p(k, _f32p), _p(v, _f32p)) == 0

    def reset(self):
        lib().orc_decoder_reset(self.h)

    def forward(self, tokens, simd=0, threads=1, attn_threads=1, want_hidden=False):
        tokens = _c(tokens, np.int32).ravel()
        logits = np.empty(self.dims["vocab"], np.float32)
        hidden = np.empty((tokens.size, self.dims["hidden"]), np.float32) if want_hidden else None
        rc = lib().orc_decoder_forward(self.h, _p(tokens, _i32p), tokens.size, _p(hidden, _f32p), _p(logits, _f32p),
                                       simd, threads, attn_threads)
        assert rc == 0
        return (logits, hidden) if want_hidden else logits

    def forward_taps(self, tokens, simd=0, threads=1, attn_threads=1):
        """forward() that also returns the residual stream after every block: (logits, [layers, n, hidden])."""
        tokens = _c(tokens, np.int32).ravel()
        logits = np.empty(self.dims["vocab"], np.float32)
        taps = np.empty((self.dims["layers"], tokens.size, self.dims["hidden"]), np.float32)
        rc = lib().orc_decoder_forward_taps(self.h, _p(tokens, _i32p), tokens.size, None, _p(logits, _f32p),
                                            _p(taps, _f32p), simd, threads, attn_threads)
        assert rc == 0
        return logits, taps

    def generate(self, prompt, max_new, simd=0, threads=1, attn_threads=1):
        prompt = _c(prompt, np.int32).ravel()
        out = np.zeros(max_new, np.int32)
        tp, td = C.c_double(0), C.c_double(0)
        rc = lib().orc_decoder_generate(self.h, _p(prompt, _i32p), prompt.size, max_new, _p(out, _i32p), C.byref(tp),
                                        C.byref(td), simd, threads, attn_threads)
        assert rc == 0
        return out, tp.value, td.value

    def __del__(self):
        try:
            if self.h:
                lib().orc_decoder_free(self.h)
                self.h = None
        except Exception:
            pass
