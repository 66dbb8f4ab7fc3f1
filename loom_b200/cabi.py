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
    "loom_b200_ctx_stream": (_vp, [_vp]),
    "loom_b200_graph_begin": (_i, [_vp]),
    "loom_b200_graph_end": (_i, [_vp, C.POINTER(_vp)]),
    "loom_b200_graph_launch": (_i, [_vp, _vp]),
    "loom_b200_graph_free": (None, [_vp, _vp]),
    "loom_b200_launch_count": (C.c_uint64, [_vp]),
    "loom_b200_ctx_set_option": (_i, [_vp, C.c_char_p, _i]),
    "loom_b200_buffer_alloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "loom_b200_buffer_free": (_i, [_vp, _vp]),
    "loom_b200_buffer_upload": (_i, [_vp, _vp, _vp, _sz]),
    "loom_b200_buffer_download": (_i, [_vp, _vp, _vp, _sz]),
    "loom_b200_buffer_zero": (_i, [_vp, _vp, _sz]),
    "loom_b200_upload_ternary": (_i, [_vp, _vp, _i, _i, _i, _f, C.POINTER(_vp)]),
    "loom_b200_pack_ternary_f32": (_i, [_vp, _vp, _i, _i, C.POINTER(_vp)]),
    "loom_b200_upload_microsoft_u8": (_i, [_vp, _vp, _i, _i, _f, C.POINTER(_vp)]),
    "loom_b200_weight_info": (_i, [_vp, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_f)]),
    "loom_b200_weight_set_scale": (_i, [_vp, _f]),
    "loom_b200_weight_download_words": (_i, [_vp, _vp, _vp]),
    "loom_b200_weight_free": (None, [_vp, _vp]),
    "loom_b200_quantize_activation": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "loom_b200_quantize_activation_f64": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "loom_b200_ternary_linear": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp]),
    "loom_b200_gate_product": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "loom_b200_inner_rmsnorm": (_i, [_vp, _i, _i, _vp, _vp, _i, _d]),
}


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

    def gate_product(self, batch, hidden, act, gate, up, out):
        self._check(lib().loom_b200_gate_product(self.h, batch, hidden, act, _ptr(gate), _ptr(up), _ptr(out)))

    def inner_rmsnorm(self, batch, n, x, weight=None, weight_len=0, eps=0.0):
        self._check(lib().loom_b200_inner_rmsnorm(self.h, batch, n, _ptr(x), _ptr(weight), weight_len, eps))
