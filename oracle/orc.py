"""TEST INFRASTRUCTURE — ctypes access to the C++ CPU oracle (oracle/rwkv7_cpu.cpp).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liborc_rwkv7.so")
_lib = None


def build(force=False):
    src = os.path.join(_HERE, "rwkv7_cpu.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        vp, c = ctypes.c_void_p, ctypes
        L.orc_last_error.restype = c.c_char_p
        L.orc_model_load.restype = vp
        L.orc_model_load.argtypes = [c.c_char_p]
        L.orc_model_free.argtypes = [vp]
        L.orc_model_info.argtypes = [vp, c.POINTER(c.c_int64)]
        L.orc_state_new.restype = vp
        L.orc_state_new.argtypes = [vp]
        L.orc_state_free.argtypes = [vp]
        L.orc_state_reset.argtypes = [vp, vp]
        L.orc_state_len.restype = c.c_int64
        L.orc_state_len.argtypes = [vp]
        L.orc_state_export.argtypes = [vp, vp]
        L.orc_state_import.argtypes = [vp, vp]
        L.orc_forward.argtypes = [vp, vp, vp, c.c_int64, vp, vp]
        L.orc_dequant_int8.argtypes = [vp, vp, c.c_int64, c.c_int64, vp]
        L.orc_mean_hidden.argtypes = [vp, vp, vp, c.c_int64, vp]
        L.orc_wkv7.argtypes = [c.c_int64, c.c_int64] + [vp] * 15
        L.orc_argmax.restype = c.c_uint32
        L.orc_argmax.argtypes = [vp, c.c_int64]
        L.orc_sample.restype = c.c_uint32
        L.orc_sample.argtypes = [vp, c.c_int64, vp, vp]
        L.orc_u01.restype = c.c_float
        L.orc_u01.argtypes = [c.c_uint32]
        L.orc_set_threads.argtypes = [c.c_int]
        L.orc_max_threads.restype = c.c_int
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def set_threads(n):
    lib().orc_set_threads(int(n))


def max_threads():
    return int(lib().orc_max_threads())


def dequant_int8(idx_u8, sz_u32):
    m, k = idx_u8.shape
    idx = np.ascontiguousarray(idx_u8, dtype=np.uint8)
    sz = np.ascontiguousarray(sz_u32, dtype=np.uint32)
    out = np.empty((m, k), dtype=np.float32)
    lib().orc_dequant_int8(_p(idx), _p(sz), m, k, _p(out))
    return out


def wkv7(r, k, v, w, a, g, k_k, k_a, r_k, lnx_w, lnx_b, state, vgate=None, vfirst=None):
    """The WKV-7 step of one layer for one session: rows [T, H*64], parameters [H*64], state [H, 64, 64].  Returns (y, new state)."""
    rr = np.ascontiguousarray(r, dtype=np.float32)
    T, C = rr.shape
    rows = [np.ascontiguousarray(x, dtype=np.float32).reshape(T, C) for x in (k, v, w, a, g)]
    opt = [None if x is None else np.ascontiguousarray(x, dtype=np.float32).reshape(T, C) for x in (vgate, vfirst)]
    par = [np.ascontiguousarray(x, dtype=np.float32).reshape(C) for x in (k_k, k_a, r_k, lnx_w, lnx_b)]
    st = np.array(state, dtype=np.float32, order="C").reshape(C // 64, 64, 64)
    y = np.empty((T, C), dtype=np.float32)
    lib().orc_wkv7(C // 64, T, _p(rr), *[_p(x) for x in rows], *[None if x is None else _p(x) for x in opt], *[_p(x) for x in par], _p(st), _p(y))
    return y, st


def argmax(logits):
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    return int(lib().orc_argmax(_p(lg), lg.size))


def pack_sampler(temperature=1.0, top_k=0, top_p=1.0, seed=0, repetition_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0,
                 hist_len=0):
    """The 8-word sampler row of the reference (src/backend_cuda.rs:5025-5034)."""
    row = np.zeros(8, dtype=np.float32)
    u = row.view(np.uint32)
    row[0] = temperature
    u[1] = top_k
    row[2] = top_p
    u[3] = seed & 0xFFFFFFFF
    row[4], row[5], row[6] = repetition_penalty, frequency_penalty, presence_penalty
    u[7] = hist_len
    return row


def sample(logits, history=(), **params):
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    hist = np.ascontiguousarray(np.asarray(history, dtype=np.uint32))
    row = pack_sampler(hist_len=hist.size, **params)
    return int(lib().orc_sample(_p(lg), lg.size, _p(row), _p(hist) if hist.size else None))


class OracleModel:
    """Model::from_safetensors + init_state + forward of the reference's CPU path (src/model.rs)."""

    def __init__(self, path):
        self._h = lib().orc_model_load(os.fsencode(path))
        if not self._h:
            raise RuntimeError(lib().orc_last_error().decode())
        info = (ctypes.c_int64 * 10)()
        lib().orc_model_info(self._h, info)
        (self.n_layer, self.n_embd, self.vocab, self.head_size, self.n_head, self.ffn_hidden, self.w_mid, self.a_mid, self.v_mid,
         self.g_mid) = [int(v) for v in info]
        self._s = lib().orc_state_new(self._h)
        self.state_len = int(lib().orc_state_len(self._h))

    def close(self):
        if self._h:
            lib().orc_state_free(self._s)
            lib().orc_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def reset(self):
        lib().orc_state_reset(self._h, self._s)

    def forward(self, tokens, full=False):
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        last = np.empty(self.vocab, dtype=np.float32)
        allp = np.empty((toks.size, self.vocab), dtype=np.float32) if full else None
        rc = lib().orc_forward(self._h, self._s, _p(toks), toks.size, _p(last), _p(allp) if full else None)
        if rc:
            raise RuntimeError(lib().orc_last_error().decode())
        return allp if full else last

    def mean_hidden(self, tokens):
        """From a zero state: mean over the tokens of the last layer's residual stream (the router feature)."""
        toks = np.ascontiguousarray(tokens, dtype=np.uint32)
        self.reset()
        out = np.empty(self.n_embd, dtype=np.float32)
        if lib().orc_mean_hidden(self._h, self._s, _p(toks), toks.size, _p(out)):
            raise RuntimeError(lib().orc_last_error().decode())
        return out

    def state_back(self):
        out = np.empty(self.state_len, dtype=np.float32)
        lib().orc_state_export(self._s, _p(out))
        return out

    def state_load(self, data):
        d = np.ascontiguousarray(data, dtype=np.float32)
        if d.size != self.state_len:
            raise ValueError(f"state length {d.size} != {self.state_len}")
        lib().orc_state_import(self._s, _p(d))
