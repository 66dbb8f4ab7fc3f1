"""ctypes binding of libloom_b200.so: one Python method per C-ABI entry point.

Device buffers are torch CUDA tensors or raw integer device addresses; nothing here computes.
If the shared library is missing the import of `lib()` raises: there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))

ACT_RELU, ACT_SILU, ACT_GELU, ACT_TANH, ACT_SIGMOID, ACT_LEAKY_RELU, ACT_RELU2, ACT_LINEAR = 0, 1, 2, 3, 4, 5, 6, -1


ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_NO_DEVICE, ERR_TIMEOUT, ERR_COMM = -1, -2, -3, -4, -5, -6


class LoomB200Error(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("loom_b200 error %d: %s" % (code, msg))
        self.code = code


def lib_path() -> str:
    return os.path.join(_PKG, "lib", "libloom_b200.so")


_lib = None

_vp = C.c_void_p
_i = C.c_int
_f = C.c_float
_d = C.c_double
_sz = C.c_size_t

# name -> (restype, argtypes); kept in one table so that the symbol-export test can walk it
SIGNATURES = {
    "loom_b200_api_version": (_i, []),
    "loom_b200_device_count": (_i, []),
    "loom_b200_last_error": (C.c_char_p, [_vp]),
    "loom_b200_ctx_create": (_i, [_i, _vp, C.POINTER(_vp)]),
    "loom_b200_ctx_destroy": (None, [_vp]),
    "loom_b200_sync": (_i, [_vp]),
    "loom_b200_selftest_wait_timeout": (_i, [_vp, C.c_uint]),
    "loom_b200_selftest_i8_peak": (_i, [_vp, _i, C.POINTER(_d)]),
    "loom_b200_ctx_stream": (_vp, [_vp]),
    "loom_b200_graph_begin": (_i, [_vp]),
    "loom_b200_graph_end": (_i, [_vp, C.POINTER(_vp)]),
    "loom_b200_graph_launch": (_i, [_vp, _vp]),
    "loom_b200_graph_free": (None, [_vp, _vp]),
    "loom_b200_launch_count": (C.c_uint64, [_vp]),
    "loom_b200_trace_read": (_i, [_vp, _vp, _i]),
    "loom_b200_trace_label": (C.c_char_p, [_vp, _i]),
    "loom_b200_ctx_set_option": (_i, [_vp, C.c_char_p, _i]),
    "loom_b200_buffer_alloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "loom_b200_buffer_free": (_i, [_vp, _vp]),
    "loom_b200_buffer_upload": (_i, [_vp, _vp, _vp, _sz]),
    "loom_b200_buffer_download": (_i, [_vp, _vp, _vp, _sz]),
    "loom_b200_buffer_zero": (_i, [_vp, _vp, _sz]),
    "loom_b200_upload_ternary": (_i, [_vp, _vp, _i, _i, _i, _f, C.POINTER(_vp)]),
    "loom_b200_pack_ternary_f32": (_i, [_vp, _vp, _i, _i, C.POINTER(_vp)]),
    "loom_b200_upload_microsoft_u8": (_i, [_vp, _vp, _i, _i, _f, C.POINTER(_vp)]),
    "loom_b200_upload_entity_blob": (_i, [_vp, _vp, _sz, C.POINTER(_i), C.POINTER(_vp)]),
    "loom_b200_weight_info": (_i, [_vp, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_f)]),
    "loom_b200_weight_set_scale": (_i, [_vp, _f]),
    "loom_b200_weight_download_words": (_i, [_vp, _vp, _vp]),
    "loom_b200_weight_free": (None, [_vp, _vp]),
    "loom_b200_quantize_activation": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "loom_b200_quantize_activation_f64": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "loom_b200_ternary_linear": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp]),
    "loom_b200_ternary_gemm": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp]),
    "loom_b200_ternary_linear_no_alloc": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp]),
    "loom_b200_gate_product": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "loom_b200_inner_rmsnorm": (_i, [_vp, _i, _i, _vp, _vp, _i, _d]),
    "loom_b200_dense_forward": (_i, [_vp, _vp, _i, _vp, _i, _vp, _vp]),
    "loom_b200_swiglu_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _d, _i, _vp, _i, _vp, _vp]),
    "loom_b200_mha_create": (_i, [_vp, _i, _i, _i, _i, _i, _d, _d, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i,
                                   _vp, _i, _vp, _i, C.POINTER(_vp)]),
    "loom_b200_mha_destroy": (None, [_vp]),
    "loom_b200_mha_reset": (_i, [_vp]),
    "loom_b200_mha_kv_offset": (_i, [_vp]),
    "loom_b200_mha_forward": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "loom_b200_mha_download_cache": (_i, [_vp, _vp, _vp]),
    "loom_b200_decoder_create": (_i, [_vp, _vp, C.POINTER(_vp)]),
    "loom_b200_decoder_destroy": (None, [_vp]),
    "loom_b200_decoder_set_block": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i]),
    "loom_b200_decoder_set_embeddings": (_i, [_vp, _vp, _vp]),
    "loom_b200_decoder_set_lm_head_ternary": (_i, [_vp, _vp]),
    "loom_b200_decoder_reset": (_i, [_vp]),
    "loom_b200_decoder_kv_offset": (_i, [_vp]),
    "loom_b200_decoder_forward": (_i, [_vp, _vp, _i, _vp]),
    "loom_b200_decoder_last_hidden": (_i, [_vp, _vp]),
    "loom_b200_decoder_continue": (_i, [_vp, _i]),
    "loom_b200_decoder_download_cache": (_i, [_vp, _i, _vp, _vp]),
    "loom_b200_decoder_generate": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "loom_b200_decoder_upload_cache": (_i, [_vp, _i, _i, _vp, _vp]),
    "loom_b200_decoder_read_tokens": (_i, [_vp, _vp, _i]),
    "loom_b200_decoder_set_kv_offset": (_i, [_vp, _i]),
    "loom_b200_decoder_set_batch": (_i, [_vp, _i]),
    "loom_b200_decoder_batch": (_i, [_vp]),
    "loom_b200_decoder_select": (_i, [_vp, _i]),
    "loom_b200_decoder_step_batch": (_i, [_vp, _vp, _vp]),
    "loom_b200_decoder_continue_batch": (_i, [_vp, _i]),
    "loom_b200_decoder_read_tokens_batch": (_i, [_vp, _vp, _i]),
    "loom_b200_decoder_step_launches": (_i, [_vp]),
    "loom_b200_decoder_linears_frame": (_i, [_vp]),
    "loom_b200_decoder_last_residual": (_i, [_vp, _vp, _i, C.POINTER(_i)]),
    "loom_b200_tp_unique_id": (_i, [_vp]),
    "loom_b200_tp_init": (_i, [_vp, _i, _i, _vp]),
    "loom_b200_tp_peer_handle": (_i, [_vp, _vp]),
    "loom_b200_tp_attach_peers": (_i, [_vp, _vp]),
    "loom_b200_tp_finalize": (None, [_vp]),
    "loom_b200_tp_rank": (_i, [_vp]),
    "loom_b200_tp_world": (_i, [_vp]),
    "loom_b200_tp_allreduce_i32": (_i, [_vp, _vp, _sz]),
    "loom_b200_tp_rowsharded_linear": (_i, [_vp, _vp, _i, _vp, _i, _vp, _i, _d, _vp, _vp, _vp]),
}


class DecoderDims(C.Structure):
    _fields_ = [("num_layers", _i), ("hidden", _i), ("num_heads", _i), ("num_kv_heads", _i), ("head_dim", _i),
                ("intermediate", _i), ("vocab", _i), ("rms_eps", _d), ("rope_theta", _d), ("activation", _i),
                ("max_seq_len", _i)]


class GenMetrics(C.Structure):
    _fields_ = [("prefill_seconds", _d), ("decode_seconds", _d), ("decode_device_seconds", _d), ("prefill_tokens", _i),
                ("generated_tokens", _i), ("launches_per_token", _d)]


def lib() -> C.CDLL:
    """Loads the CUDA library.  Raises if it has not been built: nothing runs without it."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise LoomB200Error(-4, "%s is missing: build it with `python -m loom_b200.build` "
                                "(there is no CPU fallback)" % path)
        L = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _ptr(x):
    """Device or host address of a torch tensor / numpy array / int / None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if isinstance(x, np.ndarray):
        assert x.flags["C_CONTIGUOUS"]
        return x.ctypes.data
    if hasattr(x, "data_ptr"):
        assert x.is_contiguous()
        return x.data_ptr()
    raise TypeError(type(x))


class Weight:
    """A packed ternary matrix resident in HBM (GPUWeights[key] + GPUScaleValues[key])."""

    def __init__(self, ctx: "Context", handle):
        self.ctx, self.h = ctx, handle
        r, c, rw, s = _i(), _i(), _i(), _f()
        ctx._check(lib().loom_b200_weight_info(handle, C.byref(r), C.byref(c), C.byref(rw), C.byref(s)))
        self.rows, self.cols, self.row_words = r.value, c.value, rw.value

    @property
    def scale(self) -> np.float32:
        s = _f()
        lib().loom_b200_weight_info(self.h, None, None, None, C.byref(s))
        return np.float32(s.value)

    def set_scale(self, s: float):
        self.ctx._check(lib().loom_b200_weight_set_scale(self.h, float(s)))

    def words(self) -> np.ndarray:
        out = np.zeros((self.rows, self.row_words), np.uint32)
        self.ctx._check(lib().loom_b200_weight_download_words(self.ctx.h, self.h, out.ctypes.data))
        return out

    def free(self):
        if self.h:
            lib().loom_b200_weight_free(self.ctx.h, self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Context:
    """Stands in for *poly.WGPUContext on this path."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self.h = None
        h = _vp()
        rc = lib().loom_b200_ctx_create(device, stream, C.byref(h))
        if rc != 0:
            raise LoomB200Error(rc, (lib().loom_b200_last_error(None) or b"").decode())
        self.h = h
        self.device = device

    def _check(self, rc: int):
        if rc != 0:
            raise LoomB200Error(rc, (lib().loom_b200_last_error(self.h) or b"").decode())

    def close(self):
        if self.h:
            lib().loom_b200_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        self._check(lib().loom_b200_sync(self.h))

    def i8_peak_tops(self, iters: int = 20000) -> float:
        """Dense int8 TOP/s of back-to-back tcgen05 kind::i8 MMAs on operands resident in shared memory."""
        t = _d(0.0)
        self._check(lib().loom_b200_selftest_i8_peak(self.h, iters, C.byref(t)))
        return t.value

    def selftest_wait_timeout(self, polls: int = 100000):
        """Makes a bounded device-side wait run out; raises LoomB200Error(LOOM_B200_ERR_TIMEOUT)."""
        self._check(lib().loom_b200_selftest_wait_timeout(self.h, polls))

    def graph_begin(self):
        self._check(lib().loom_b200_graph_begin(self.h))

    def graph_end(self):
        g = _vp()
        self._check(lib().loom_b200_graph_end(self.h, C.byref(g)))
        return g

    def graph_launch(self, g):
        self._check(lib().loom_b200_graph_launch(self.h, g))

    def graph_free(self, g):
        lib().loom_b200_graph_free(self.h, g)

    def trace_read(self, ctas: int) -> np.ndarray:
        out = np.zeros((ctas, 8), np.uint64)
        self._check(lib().loom_b200_trace_read(self.h, out.ctypes.data, ctas))
        return out

    def trace_label(self, row: int) -> str:
        return (lib().loom_b200_trace_label(self.h, row) or b"").decode()

    def set_option(self, key: str, value: int):
        self._check(lib().loom_b200_ctx_set_option(self.h, key.encode(), int(value)))

    @property
    def stream(self) -> int:
        return lib().loom_b200_ctx_stream(self.h) or 0

    @property
    def launch_count(self) -> int:
        return int(lib().loom_b200_launch_count(self.h))

    # ---- buffers -----------------------------------------------------------------------------
    def alloc(self, nbytes: int) -> int:
        p = _vp()
        self._check(lib().loom_b200_buffer_alloc(self.h, nbytes, C.byref(p)))
        return p.value

    def free(self, dptr: int):
        self._check(lib().loom_b200_buffer_free(self.h, dptr))

    def upload(self, dst, src: np.ndarray):
        src = np.ascontiguousarray(src)
        self._check(lib().loom_b200_buffer_upload(self.h, _ptr(dst), src.ctypes.data, src.nbytes))

    def download(self, src, shape, dtype) -> np.ndarray:
        out = np.empty(shape, dtype)
        self._check(lib().loom_b200_buffer_download(self.h, out.ctypes.data, _ptr(src), out.nbytes))
        return out

    def zero(self, dst, nbytes: int):
        self._check(lib().loom_b200_buffer_zero(self.h, _ptr(dst), nbytes))

    def to_device(self, arr: np.ndarray) -> int:
        arr = np.ascontiguousarray(arr)
        p = self.alloc(arr.nbytes)
        self.upload(p, arr)
        return p

    # ---- weights --------------------------------------------------------------------------------
    def upload_ternary(self, words: np.ndarray, rows: int, cols: int, scale: float) -> Weight:
        words = np.ascontiguousarray(words, np.uint32)
        h = _vp()
        self._check(lib().loom_b200_upload_ternary(self.h, words.ctypes.data, rows, cols, (cols + 15) // 16,
                                                   float(scale), C.byref(h)))
        return Weight(self, h)

    def pack_ternary_f32(self, master_dev, rows: int, cols: int) -> Weight:
        h = _vp()
        self._check(lib().loom_b200_pack_ternary_f32(self.h, _ptr(master_dev), rows, cols, C.byref(h)))
        return Weight(self, h)

    def upload_entity_blob(self, blob: bytes):
        """A BITNET_TERNARY blob of an .entity checkpoint -> (Weight, slab offset)."""
        h, off = _vp(), _i(0)
        self._check(lib().loom_b200_upload_entity_blob(self.h, C.c_char_p(blob), len(blob), C.byref(off), C.byref(h)))
        return Weight(self, h), off.value

    def upload_microsoft_u8(self, packed: np.ndarray, rows: int, cols: int, scale: float) -> Weight:
        packed = np.ascontiguousarray(packed, np.uint8)
        h = _vp()
        self._check(lib().loom_b200_upload_microsoft_u8(self.h, packed.ctypes.data, rows, cols, float(scale),
                                                        C.byref(h)))
        return Weight(self, h)

    # ---- kernel dispatch ---------------------------------------------------------------------------
    def quantize_activation(self, batch, n, x, q, amax):
        self._check(lib().loom_b200_quantize_activation(self.h, batch, n, _ptr(x), _ptr(q), _ptr(amax)))

    def quantize_activation_f64(self, batch, n, x, q, amax):
        self._check(lib().loom_b200_quantize_activation_f64(self.h, batch, n, _ptr(x), _ptr(q), _ptr(amax)))

    def ternary_linear(self, w: Weight, batch, q, amax, out, bias=None, residual=None, act=ACT_LINEAR, acc_out=None):
        self._check(lib().loom_b200_ternary_linear(self.h, w.h, batch, _ptr(q), _ptr(amax), _ptr(bias),
                                                   _ptr(residual), act, _ptr(out), _ptr(acc_out)))

    def ternary_linear_no_alloc(self, w: Weight, batch, q, amax, out, bias=None, residual=None, act=ACT_LINEAR):
        """The ternary linear with its scratch in the library's built-in array: allocates nothing."""
        self._check(lib().loom_b200_ternary_linear_no_alloc(self.h, w.h, batch, _ptr(q), _ptr(amax), _ptr(bias),
                                                            _ptr(residual), act, _ptr(out)))

    def ternary_gemm(self, w: Weight, tokens, x, out=None, bias=None, residual=None, act=ACT_LINEAR, acc_out=None, amax_out=None):
        self._check(lib().loom_b200_ternary_gemm(self.h, w.h, tokens, _ptr(x), _ptr(bias), _ptr(residual), act, _ptr(out),
                                                 _ptr(acc_out), _ptr(amax_out)))

    # ---- tensor parallelism: one process per GPU, one context per process ----
    @staticmethod
    def tp_unique_id() -> bytes:
        """128 bytes that rank 0 creates and hands to every rank (any transport: a file, a store, a broadcast)."""
        buf = C.create_string_buffer(128)
        rc = lib().loom_b200_tp_unique_id(buf)
        if rc != 0:
            raise LoomB200Error(rc, (lib().loom_b200_last_error(None) or b"").decode())
        return buf.raw

    def tp_init(self, rank: int, world: int, unique_id: bytes):
        assert len(unique_id) == 128
        self._check(lib().loom_b200_tp_init(self.h, rank, world, C.c_char_p(unique_id)))

    def tp_peer_handle(self) -> bytes:
        """This rank's mailbox as a 64-byte CUDA IPC handle; gather all ranks' handles in rank order for tp_attach_peers."""
        buf = C.create_string_buffer(64)
        self._check(lib().loom_b200_tp_peer_handle(self.h, buf))
        return buf.raw

    def tp_attach_peers(self, handles: bytes):
        assert len(handles) % 64 == 0
        self._check(lib().loom_b200_tp_attach_peers(self.h, C.c_char_p(handles)))

    def tp_finalize(self):
        lib().loom_b200_tp_finalize(self.h)

    @property
    def tp_rank(self) -> int:
        return lib().loom_b200_tp_rank(self.h)

    @property
    def tp_world(self) -> int:
        return lib().loom_b200_tp_world(self.h)

    def tp_allreduce_i32(self, buf, n: int):
        self._check(lib().loom_b200_tp_allreduce_i32(self.h, _ptr(buf), n))

    def tp_rowsharded_linear(self, w: Weight, batch, x_local, cols_global, out, inner_w=None, inner_w_len=0, eps=0.0,
                             bias=None, residual=None):
        self._check(lib().loom_b200_tp_rowsharded_linear(self.h, w.h, batch, _ptr(x_local), cols_global, _ptr(inner_w),
                                                         inner_w_len, eps, _ptr(bias), _ptr(residual), _ptr(out)))

    def gate_product(self, batch, hidden, act, gate, up, out):
        self._check(lib().loom_b200_gate_product(self.h, batch, hidden, act, _ptr(gate), _ptr(up), _ptr(out)))

    def inner_rmsnorm(self, batch, n, x, weight=None, weight_len=0, eps=0.0):
        self._check(lib().loom_b200_inner_rmsnorm(self.h, batch, n, _ptr(x), _ptr(weight), weight_len, eps))


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, np.float32)


def _hp(a):
    return None if a is None else a.ctypes.data


def dense_forward(ctx: Context, w: Weight, act: int, x: np.ndarray):
    """DenseForwardPackedTernaryCPU stand-in: host in, host (pre, post) out."""
    x = _f32(x)
    batch = x.shape[0]
    pre = np.empty((batch, w.rows), np.float32)
    post = np.empty((batch, w.rows), np.float32)
    ctx._check(lib().loom_b200_dense_forward(ctx.h, w.h, act, x.ctypes.data, batch, pre.ctypes.data, post.ctypes.data))
    return pre, post


def swiglu_forward(ctx: Context, gate: Weight, up: Weight, down: Weight, x: np.ndarray, act=ACT_SILU, bias_gate=None,
                   bias_up=None, bias_down=None, inner_w=None, eps=0.0):
    """SwiGLUForwardPackedTernaryCPU stand-in."""
    x = _f32(x)
    seq = x.shape[0]
    pre = np.empty((seq, gate.rows), np.float32)
    post = np.empty((seq, gate.cols), np.float32)
    bg, bu, bd, iw = _f32(bias_gate), _f32(bias_up), _f32(bias_down), _f32(inner_w)
    ctx._check(lib().loom_b200_swiglu_forward(ctx.h, gate.h, up.h, down.h, _hp(bg), _hp(bu), _hp(bd), _hp(iw),
                                              0 if iw is None else iw.size, eps, act, x.ctypes.data, seq,
                                              pre.ctypes.data, post.ctypes.data))
    return pre, post


class MHA:
    """The MHA layer with its KV ring on the device (MHAForwardPackedTernaryCPU stand-in)."""

    def __init__(self, ctx: Context, d_model, heads, kv_heads, head_dim, max_seq_len, theta, eps, wq, wk, wv, wo,
                 bq=None, bk=None, bv=None, bo=None, q_norm=None, k_norm=None, inner_w=None):
        self.ctx, self.h = ctx, None
        self.weights = (wq, wk, wv, wo)
        self.d_model, self.heads, self.kv_heads, self.head_dim = d_model, heads, kv_heads or heads, head_dim
        self.msl = max_seq_len or 512
        a = [_f32(v) for v in (bq, bk, bv, bo, q_norm, k_norm, inner_w)]
        h = _vp()
        ctx._check(lib().loom_b200_mha_create(ctx.h, d_model, heads, kv_heads, head_dim, max_seq_len, theta, eps, wq.h,
                                              wk.h, wv.h, wo.h, _hp(a[0]), _hp(a[1]), _hp(a[2]), _hp(a[3]), _hp(a[4]),
                                              0 if a[4] is None else a[4].size, _hp(a[5]),
                                              0 if a[5] is None else a[5].size, _hp(a[6]),
                                              0 if a[6] is None else a[6].size, C.byref(h)))
        self.h = h

    def reset(self):
        self.ctx._check(lib().loom_b200_mha_reset(self.h))

    @property
    def kv_offset(self):
        return lib().loom_b200_mha_kv_offset(self.h)

    def forward(self, x):
        x = _f32(x)
        batch, seq = (1, x.shape[0]) if x.ndim == 2 else (x.shape[0], x.shape[1])
        pre = np.empty((batch * seq, self.d_model), np.float32)
        post = np.empty((batch * seq, self.d_model), np.float32)
        self.ctx._check(lib().loom_b200_mha_forward(self.h, x.ctypes.data, batch, seq, pre.ctypes.data, post.ctypes.data))
        return pre, post

    def cache(self):
        kvd = self.kv_heads * self.head_dim
        k = np.empty((self.msl, kvd), np.float32)
        v = np.empty((self.msl, kvd), np.float32)
        self.ctx._check(lib().loom_b200_mha_download_cache(self.h, k.ctypes.data, v.ctypes.data))
        return k, v

    def close(self):
        if self.h:
            lib().loom_b200_mha_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Decoder:
    """The ternary decoder stack on the device (InitHFDecoderBlocks + Transformer stand-in)."""

    def __init__(self, ctx: Context, layers, hidden, heads, kv_heads, head_dim, inter, vocab, eps, theta,
                 act=ACT_SILU, max_seq_len=2048):
        self.ctx, self.h = ctx, None
        self.dims = DecoderDims(layers, hidden, heads, kv_heads, head_dim, inter, vocab, eps, theta, act, max_seq_len)
        h = _vp()
        ctx._check(lib().loom_b200_decoder_create(ctx.h, C.byref(self.dims), C.byref(h)))
        self.h = h
        self._keep = []

    def set_block(self, b, weights7, g1=None, g2=None, attn_inner=None, ffn_inner=None):
        assert len(weights7) == 7
        self._keep.append(list(weights7))
        arr = (_vp * 7)(*[w.h for w in weights7])
        g1, g2, ai, fi = _f32(g1), _f32(g2), _f32(attn_inner), _f32(ffn_inner)
        self.ctx._check(lib().loom_b200_decoder_set_block(self.h, b, _hp(g1), _hp(g2), C.cast(arr, _vp), _hp(ai),
                                                          0 if ai is None else ai.size, _hp(fi),
                                                          0 if fi is None else fi.size))

    def set_embeddings(self, emb_dev, final_gain=None):
        self._keep.append(emb_dev)
        fg = _f32(final_gain)
        self.ctx._check(lib().loom_b200_decoder_set_embeddings(self.h, _ptr(emb_dev), _hp(fg)))

    def set_lm_head_ternary(self, head: "Weight"):
        """Untied LM head as a packed ternary matrix [vocab, hidden] (None = back to the tied fp32 head)."""
        self._keep.append(head)
        self.ctx._check(lib().loom_b200_decoder_set_lm_head_ternary(self.h, head.h if head is not None else None))

    def reset(self):
        self.ctx._check(lib().loom_b200_decoder_reset(self.h))

    @property
    def kv_offset(self):
        return lib().loom_b200_decoder_kv_offset(self.h)

    def forward(self, tokens, want_logits=True):
        tokens = np.ascontiguousarray(tokens, np.int32).ravel()
        logits = np.empty(self.dims.vocab, np.float32) if want_logits else None
        self.ctx._check(lib().loom_b200_decoder_forward(self.h, tokens.ctypes.data, tokens.size, _hp(logits)))
        return logits

    def last_hidden(self):
        out = np.empty(self.dims.hidden, np.float32)
        self.ctx._check(lib().loom_b200_decoder_last_hidden(self.h, out.ctypes.data))
        return out

    def continue_greedy(self, steps: int):
        """`steps` more greedy tokens on the device; returns without waiting."""
        self.ctx._check(lib().loom_b200_decoder_continue(self.h, steps))

    def cache(self, block: int):
        kvd = self.dims.num_kv_heads * self.dims.head_dim // max(1, self.ctx.tp_world)  # this rank's KV heads
        k = np.empty((self.dims.max_seq_len, kvd), np.float32)
        v = np.empty((self.dims.max_seq_len, kvd), np.float32)
        self.ctx._check(lib().loom_b200_decoder_download_cache(self.h, block, k.ctypes.data, v.ctypes.data))
        return k, v

    # ---- independent sequences ----
    def set_batch(self, batch: int):
        """`batch` independent sequences (one KV ring each); before the first set_block."""
        self.ctx._check(lib().loom_b200_decoder_set_batch(self.h, batch))

    @property
    def batch(self) -> int:
        return lib().loom_b200_decoder_batch(self.h)

    def select(self, seq: int):
        """The sequence the single-sequence calls (forward, kv_offset, cache, ...) act on."""
        self.ctx._check(lib().loom_b200_decoder_select(self.h, seq))

    def step_batch(self, tokens=None, want_logits=True):
        """One token per sequence (None = greedy continuation); logits [batch, vocab]."""
        t = None if tokens is None else np.ascontiguousarray(tokens, np.int32).ravel()
        logits = np.empty((self.batch, self.dims.vocab), np.float32) if want_logits else None
        self.ctx._check(lib().loom_b200_decoder_step_batch(self.h, _hp(t), _hp(logits)))
        return logits

    def continue_batch(self, steps: int):
        self.ctx._check(lib().loom_b200_decoder_continue_batch(self.h, steps))

    def generated_tokens_batch(self, n: int) -> np.ndarray:
        out = np.zeros((self.batch, n), np.int32)
        self.ctx._check(lib().loom_b200_decoder_read_tokens_batch(self.h, out.ctypes.data, n))
        return out

    def set_kv_offset(self, kv_offset: int):
        """Cuts the sequence back to its first kv_offset positions."""
        self.ctx._check(lib().loom_b200_decoder_set_kv_offset(self.h, kv_offset))

    def launches_per_token(self) -> int:
        return int(lib().loom_b200_decoder_step_launches(self.h))

    def linears_frame(self):
        """Enqueues the ternary projections of one decode step as the step runs them (no attention, no head)."""
        self.ctx._check(lib().loom_b200_decoder_linears_frame(self.h))

    def generated_tokens(self, n: int) -> np.ndarray:
        """The last n tokens sampled by the device-resident greedy loop (waits for the device)."""
        out = np.zeros(n, np.int32)
        self.ctx._check(lib().loom_b200_decoder_read_tokens(self.h, out.ctypes.data, n))
        return out

    def upload_cache(self, block: int, kv_offset: int, k, v):
        """Installs positions 0..kv_offset-1 of a block's KV ring from host rows [kv_offset, kv_dim]."""
        k, v = _f32(k), _f32(v)
        self.ctx._check(lib().loom_b200_decoder_upload_cache(self.h, block, kv_offset, k.ctypes.data, v.ctypes.data))

    def last_residual(self, max_rows: int):
        """Residual stream after the last block (before the final norm) for the tokens of the last pass."""
        out = np.empty((max_rows, self.dims.hidden), np.float32)
        n = _i(0)
        self.ctx._check(lib().loom_b200_decoder_last_residual(self.h, out.ctypes.data, max_rows, C.byref(n)))
        return out[:n.value]

    def generate(self, prompt, max_new):
        prompt = np.ascontiguousarray(prompt, np.int32).ravel()
        out = np.zeros(max(max_new, 1), np.int32)
        m = GenMetrics()
        self.ctx._check(lib().loom_b200_decoder_generate(self.h, prompt.ctypes.data, prompt.size, max_new,
                                                         out.ctypes.data, C.byref(m)))
        return out[:max_new], m

    def close(self):
        if self.h:
            lib().loom_b200_decoder_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
