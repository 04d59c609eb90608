"""B200-native RWKV-7 forward step behind the reference's library API.

This Python layer is a thin ctypes mirror of the C ABI in `include/rsv_b200.h`, with the names of the
reference's Rust API (`ModelBuilder`, `Bundle`, `State`, `SamplerParams`, `RnnInput`/`RnnOption`;
src/gpu_model.rs:3685-3913).  All computation happens in `librsv_b200.so` (hand-written sm_100a CUDA);
there is no CPU path here: loading a model without the native library or without a B200 raises.
"""
import ctypes as _c
import json as _json
import os as _os

import numpy as _np

_PKG = _os.path.dirname(_os.path.abspath(__file__))
LIB_CUDA = _os.path.join(_PKG, "librsv_b200.so")
LIB_SYNTH = _os.path.join(_PKG, "librsv_synth.so")

__all__ = ["ModelBuilder", "Bundle", "State", "Scheduler", "SamplerParams", "RnnInput", "RnnOption", "ModelInfo", "RsvError", "write_synthetic", "SHAPES",
           "quantize_int8", "op_dequant_int8", "op_linear", "op_wkv7", "op_argmax", "op_sample", "native", "ABI_SYMBOLS"]


class RsvError(RuntimeError):
    """An error string returned through the C ABI (the reference's `Box<dyn Error>`)."""


# Every symbol include/rsv_b200.h declares.
ABI_SYMBOLS = [
    "rsv_last_error", "rsv_model_load", "rsv_model_free", "rsv_model_info_get", "rsv_model_weight_bytes", "rsv_state_new", "rsv_state_free",
    "rsv_state_batch", "rsv_state_len", "rsv_state_back", "rsv_state_load", "rsv_state_slot_back", "rsv_state_slot_load", "rsv_state_reset",
    "rsv_state_save", "rsv_state_restore", "rsv_state_slot_save", "rsv_state_slot_restore", "rsv_state_slot_copy",
    "rsv_infer_tokens", "rsv_infer_seq", "rsv_infer_chunked", "rsv_infer_full", "rsv_infer_argmax", "rsv_infer_argmax_selfloop",
    "rsv_infer_sample", "rsv_infer_sample_selfloop", "rsv_prefill_batch", "rsv_prefill_batch_mean_hidden", "rsv_sample_selfloop_submit", "rsv_sample_selfloop_collect",
    "rsv_prof_enable", "rsv_prof_clear", "rsv_prof_dump", "rsv_launch_count", "rsv_timer_start", "rsv_timer_stop", "rsv_synchronize",
    "rsv_sched_new", "rsv_sched_free", "rsv_sched_submit", "rsv_sched_step", "rsv_sched_poll", "rsv_sched_result", "rsv_sched_sync",
    "rsv_sched_stats", "rsv_quantize_int8", "rsv_op_dequant_int8", "rsv_op_linear", "rsv_op_wkv7", "rsv_op_argmax", "rsv_op_sample", "rsv_op_sample_static",
]


class _ModelInfoC(_c.Structure):
    _fields_ = [("version", _c.c_int32)] + [(n, _c.c_int64) for n in
                                             ("num_layer", "num_emb", "num_hidden", "num_vocab", "num_head", "head_size", "ffn_hidden", "w_mid",
                                              "a_mid", "v_mid", "g_mid")]


class SamplerParams(_c.Structure):
    """SamplerParams (src/gpu_model.rs:3883-3913); defaults as its `Default` impl."""
    _fields_ = [("temperature", _c.c_float), ("top_k", _c.c_uint32), ("top_p", _c.c_float), ("seed", _c.c_uint32),
                ("repetition_penalty", _c.c_float), ("frequency_penalty", _c.c_float), ("presence_penalty", _c.c_float)]

    def __init__(self, temperature=1.0, top_k=0, top_p=1.0, seed=0, repetition_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0):
        super().__init__(temperature, top_k, top_p, seed, repetition_penalty, frequency_penalty, presence_penalty)


_native = None


def native():
    """Loads librsv_b200.so (raises if it has not been built) and declares the C signatures."""
    global _native
    if _native is None:
        if not _os.path.exists(LIB_CUDA):
            raise RsvError(f"{LIB_CUDA} is missing: build it with `python -m rwkv_rsv_b200.build` (there is no fallback path)")
        L = _c.CDLL(LIB_CUDA)
        vp, i64, u32, pp = _c.c_void_p, _c.c_int64, _c.c_uint32, _c.POINTER(_c.c_void_p)
        L.rsv_last_error.restype = _c.c_char_p
        L.rsv_model_load.argtypes = [_c.c_char_p, _c.c_int, pp]
        L.rsv_model_free.argtypes = [vp]
        L.rsv_model_free.restype = None
        L.rsv_model_info_get.argtypes = [vp, _c.POINTER(_ModelInfoC)]
        L.rsv_model_weight_bytes.argtypes = [vp]
        L.rsv_model_weight_bytes.restype = i64
        L.rsv_state_new.argtypes = [vp, i64, pp]
        L.rsv_state_free.argtypes = [vp]
        L.rsv_state_free.restype = None
        L.rsv_state_batch.argtypes = [vp]
        L.rsv_state_batch.restype = i64
        L.rsv_state_len.argtypes = [vp]
        L.rsv_state_len.restype = i64
        L.rsv_state_back.argtypes = [vp, vp, i64]
        L.rsv_state_load.argtypes = [vp, vp, i64]
        L.rsv_state_slot_back.argtypes = [vp, i64, vp, i64]
        L.rsv_state_slot_load.argtypes = [vp, i64, vp, i64]
        L.rsv_state_reset.argtypes = [vp]
        L.rsv_state_save.argtypes = [vp, _c.c_char_p]
        L.rsv_state_restore.argtypes = [vp, _c.c_char_p]
        L.rsv_state_slot_save.argtypes = [vp, i64, _c.c_char_p]
        L.rsv_state_slot_restore.argtypes = [vp, i64, _c.c_char_p]
        L.rsv_state_slot_copy.argtypes = [vp, i64, vp, i64]
        for f in ("rsv_infer_tokens", "rsv_infer_seq", "rsv_infer_full", "rsv_infer_argmax"):
            getattr(L, f).argtypes = [vp, vp, vp, i64, vp]
        L.rsv_infer_chunked.argtypes = [vp, vp, vp, i64, i64, vp]
        L.rsv_infer_argmax_selfloop.argtypes = [vp, vp, u32, i64, vp]
        L.rsv_infer_sample.argtypes = [vp, vp, vp, i64, _c.POINTER(SamplerParams), vp, i64, vp]
        L.rsv_infer_sample_selfloop.argtypes = [vp, vp, u32, i64, _c.POINTER(SamplerParams), vp]
        L.rsv_prefill_batch.argtypes = [vp, vp, vp, vp, i64, i64, vp]
        L.rsv_prefill_batch_mean_hidden.argtypes = [vp, vp, vp, vp, i64, i64, vp]
        L.rsv_sample_selfloop_submit.argtypes = [vp, vp, vp, i64, i64, _c.POINTER(SamplerParams), pp]
        L.rsv_sample_selfloop_collect.argtypes = [vp, vp, i64]
        L.rsv_prof_enable.argtypes = [vp, _c.c_int]
        L.rsv_prof_clear.argtypes = [vp]
        L.rsv_prof_dump.argtypes = [vp, _c.c_char_p, i64]
        L.rsv_launch_count.argtypes = [vp]
        L.rsv_launch_count.restype = i64
        L.rsv_timer_start.argtypes = [vp]
        L.rsv_timer_stop.argtypes = [vp, _c.POINTER(_c.c_float)]
        L.rsv_synchronize.argtypes = [vp]
        L.rsv_sched_new.argtypes = [vp, i64, i64, i64, i64, pp]
        L.rsv_sched_free.argtypes = [vp]
        L.rsv_sched_free.restype = None
        L.rsv_sched_submit.argtypes = [vp, vp, i64, i64, _c.POINTER(SamplerParams), _c.POINTER(i64)]
        L.rsv_sched_step.argtypes = [vp, _c.POINTER(i64), _c.POINTER(i64)]
        L.rsv_sched_poll.argtypes = [vp, vp, i64, _c.POINTER(i64)]
        L.rsv_sched_result.argtypes = [vp, i64, vp, i64, _c.POINTER(i64)]
        L.rsv_sched_sync.argtypes = [vp]
        L.rsv_sched_stats.argtypes = [vp, _c.POINTER(i64), _c.POINTER(i64)]
        L.rsv_op_dequant_int8.argtypes = [_c.c_int, vp, vp, i64, i64, vp]
        L.rsv_quantize_int8.argtypes = [_c.c_int, vp, i64, i64, vp, vp]
        L.rsv_op_argmax.argtypes = [_c.c_int, vp, i64, i64, vp]
        L.rsv_op_linear.argtypes = [_c.c_int, _c.c_int, _c.c_int, vp, vp, i64, i64, vp, i64, vp]
        L.rsv_op_wkv7.argtypes = [_c.c_int, _c.c_int, i64, i64, i64] + [vp] * 15
        L.rsv_op_sample.argtypes = [_c.c_int, vp, i64, i64, vp, vp, i64, vp]
        L.rsv_op_sample_static.argtypes = [_c.c_int, vp, vp, i64, i64, vp, vp, i64, vp]
        _native = L
    return _native


def _check(rc):
    if rc != 0:
        raise RsvError(native().rsv_last_error().decode(errors="replace"))


def _ptr(a):
    return a.ctypes.data_as(_c.c_void_p)


def _tokens(t):
    return _np.ascontiguousarray(_np.asarray(t, dtype=_np.uint32).reshape(-1))


class ModelInfo:
    """ModelInfo (src/gpu_model.rs:75-99)."""

    def __init__(self, c):
        self.version = "V7" if c.version == 7 else str(c.version)
        for n, _t in _ModelInfoC._fields_[1:]:
            setattr(self, n, int(getattr(c, n)))

    def __repr__(self):
        return "ModelInfo(" + ", ".join(f"{k}={v}" for k, v in self.__dict__.items()) + ")"


class RnnOption:
    """RnnOption (src/gpu_model.rs:3846-3853)."""
    Last = "Last"
    Full = "Full"


class RnnInput:
    """RnnInput (src/gpu_model.rs:3857-3876)."""

    def __init__(self, tokens, chunk_size=0, option=RnnOption.Last):
        self.tokens, self.chunk_size, self.option = list(tokens), chunk_size, option


class Model:
    """GpuModel: weights in HBM plus work buffers (src/gpu_model.rs:401-546)."""

    def __init__(self, path, device=0):
        h = _c.c_void_p()
        _check(native().rsv_model_load(_os.fsencode(path), int(device), _c.byref(h)))
        self._h = h
        c = _ModelInfoC()
        _check(native().rsv_model_info_get(self._h, _c.byref(c)))
        self._info = ModelInfo(c)

    def info(self):
        return self._info

    def weight_bytes(self):
        return int(native().rsv_model_weight_bytes(self._h))

    def create_state(self):
        return State(self, 1)

    def create_batch_state(self, batch):
        return State(self, batch)

    def close(self):
        if getattr(self, "_h", None):
            native().rsv_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- batch API (src/gpu_model.rs:868-1011, 1639-1802) ----
    def forward_seq_batch(self, state, tokens_batch):
        """Prefills slot b with tokens_batch[b]; returns each slot's last token (the decode seed)."""
        batch = len(tokens_batch)
        if batch == 0:
            raise RsvError("forward_seq_batch: empty batch")
        t_pad = max(1, max(len(t) for t in tokens_batch))
        flat = _np.zeros((batch, t_pad), dtype=_np.uint32)
        lens = _np.zeros(batch, dtype=_np.uint32)
        for b, t in enumerate(tokens_batch):
            flat[b, :len(t)] = t
            lens[b] = len(t)
        seeds = _np.zeros(batch, dtype=_np.uint32)
        _check(native().rsv_prefill_batch(self._h, state._h, _ptr(flat), _ptr(lens), batch, t_pad, _ptr(seeds)))
        return seeds

    def forward_seq_batch_mean_hidden(self, state, tokens_batch, pad_to=None):
        """Resets the state, prefills slot b with tokens_batch[b] and returns [batch, n_embd]: per slot the mean over its tokens of the
        last layer's residual stream (src/gpu_model.rs:1013-1036).  `pad_to` fixes the row pitch of the token matrix (rows past a
        prompt's length are never read)."""
        batch = len(tokens_batch)
        if batch == 0:
            raise RsvError("forward_seq_batch: empty batch")
        t_pad = max(1, max(len(t) for t in tokens_batch), int(pad_to or 0))
        flat = _np.zeros((batch, t_pad), dtype=_np.uint32)
        lens = _np.zeros(batch, dtype=_np.uint32)
        for b, t in enumerate(tokens_batch):
            flat[b, :len(t)] = t
            lens[b] = len(t)
        out = _np.empty((batch, self.info().num_emb), dtype=_np.float32)
        _check(native().rsv_prefill_batch_mean_hidden(self._h, state._h, _ptr(flat), _ptr(lens), batch, t_pad, _ptr(out)))
        return out

    def submit_sample_selfloop_batch(self, state, seeds, n, sp):
        seeds = _tokens(seeds)
        t = _c.c_void_p()
        _check(native().rsv_sample_selfloop_submit(self._h, state._h, _ptr(seeds), seeds.size, int(n), _c.byref(sp) if sp is not None else None,
                                                   _c.byref(t)))
        return (t, seeds.size, int(n))

    def collect_sample_selfloop_batch(self, ticket):
        t, batch, n = ticket
        out = _np.zeros((batch, n), dtype=_np.uint32)
        _check(native().rsv_sample_selfloop_collect(t, _ptr(out), out.size))
        return out

    # ---- diagnostics ----
    def prof_enable(self, on=True):
        _check(native().rsv_prof_enable(self._h, 1 if on else 0))

    def clear_kernel_prof(self):
        _check(native().rsv_prof_clear(self._h))

    def kernel_prof(self):
        buf = _c.create_string_buffer(1 << 16)
        _check(native().rsv_prof_dump(self._h, buf, len(buf)))
        return _json.loads(buf.value.decode())

    def launch_count(self):
        return int(native().rsv_launch_count(self._h))

    def timer_start(self):
        _check(native().rsv_timer_start(self._h))

    def timer_stop(self):
        ms = _c.c_float()
        _check(native().rsv_timer_stop(self._h, _c.byref(ms)))
        return float(ms.value)

    def synchronize(self):
        _check(native().rsv_synchronize(self._h))


class State:
    """State (src/gpu_model.rs:3920-4105)."""

    def __init__(self, model, batch=1):
        h = _c.c_void_p()
        _check(native().rsv_state_new(model._h, int(batch), _c.byref(h)))
        self._h, self._model = h, model

    def batch(self):
        return int(native().rsv_state_batch(self._h))

    def __len__(self):
        return int(native().rsv_state_len(self._h))

    def back(self):
        out = _np.empty(len(self), dtype=_np.float32)
        _check(native().rsv_state_back(self._h, _ptr(out), out.size))
        return out

    def load(self, data):
        d = _np.ascontiguousarray(data, dtype=_np.float32).reshape(-1)
        _check(native().rsv_state_load(self._h, _ptr(d), d.size))

    def slot_back(self, slot):
        out = _np.empty(len(self) // self.batch(), dtype=_np.float32)
        _check(native().rsv_state_slot_back(self._h, int(slot), _ptr(out), out.size))
        return out

    def slot_load(self, slot, data):
        d = _np.ascontiguousarray(data, dtype=_np.float32).reshape(-1)
        _check(native().rsv_state_slot_load(self._h, int(slot), _ptr(d), d.size))

    def save(self, path):
        """The whole state as a raw f32 file (the file of examples/state_persist.rs:38-47)."""
        _check(native().rsv_state_save(self._h, _os.fsencode(path)))

    def restore(self, path):
        _check(native().rsv_state_restore(self._h, _os.fsencode(path)))

    def slot_save(self, slot, path):
        _check(native().rsv_state_slot_save(self._h, int(slot), _os.fsencode(path)))

    def slot_restore(self, slot, path):
        _check(native().rsv_state_slot_restore(self._h, int(slot), _os.fsencode(path)))

    def slot_copy_from(self, slot, src, src_slot):
        """Session migration: slot `src_slot` of state `src` (any model handle of the same shape, any GPU) -> slot `slot` here."""
        _check(native().rsv_state_slot_copy(self._h, int(slot), src._h, int(src_slot)))

    def reset(self):
        _check(native().rsv_state_reset(self._h))

    def close(self):
        if getattr(self, "_h", None):
            native().rsv_state_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Bundle:
    """Bundle {model, state} (src/gpu_model.rs:3708-3843)."""

    def __init__(self, model):
        self.model = model
        self.state = model.create_state()

    def info(self):
        return self.model.info()

    def _logits(self):
        return _np.empty(self.model.info().num_vocab, dtype=_np.float32)

    def infer_tokens(self, tokens):
        t, out = _tokens(tokens), self._logits()
        _check(native().rsv_infer_tokens(self.model._h, self.state._h, _ptr(t), t.size, _ptr(out)))
        return out

    def infer_seq(self, tokens):
        t, out = _tokens(tokens), self._logits()
        _check(native().rsv_infer_seq(self.model._h, self.state._h, _ptr(t), t.size, _ptr(out)))
        return out

    def infer(self, inp):
        t = _tokens(inp.tokens)
        if inp.option == RnnOption.Full:
            out = _np.empty((t.size, self.model.info().num_vocab), dtype=_np.float32)
            _check(native().rsv_infer_full(self.model._h, self.state._h, _ptr(t), t.size, _ptr(out)))
            return out.reshape(-1)
        out = self._logits()
        _check(native().rsv_infer_chunked(self.model._h, self.state._h, _ptr(t), t.size, max(int(inp.chunk_size), 1), _ptr(out)))
        return out

    def infer_chunked(self, tokens, chunk_size):
        return self.infer(RnnInput(tokens, chunk_size, RnnOption.Last))

    def infer_argmax(self, tokens):
        t, out = _tokens(tokens), _np.zeros(1, dtype=_np.uint32)
        _check(native().rsv_infer_argmax(self.model._h, self.state._h, _ptr(t), t.size, _ptr(out)))
        return int(out[0])

    def infer_argmax_selfloop(self, seed, n):
        out = _np.zeros(int(n), dtype=_np.uint32)
        _check(native().rsv_infer_argmax_selfloop(self.model._h, self.state._h, int(seed), int(n), _ptr(out)))
        return out

    def infer_sample(self, tokens, sp, history=()):
        t, out = _tokens(tokens), _np.zeros(1, dtype=_np.uint32)
        h = _tokens(history)
        _check(native().rsv_infer_sample(self.model._h, self.state._h, _ptr(t), t.size, _c.byref(sp), _ptr(h) if h.size else None, h.size, _ptr(out)))
        return int(out[0])

    def infer_sample_selfloop(self, seed, n, sp):
        out = _np.zeros(int(n), dtype=_np.uint32)
        _check(native().rsv_infer_sample_selfloop(self.model._h, self.state._h, int(seed), int(n), _c.byref(sp), _ptr(out)))
        return out

    def state_back(self):
        return self.state.back()

    def state_load(self, data):
        self.state.load(data)

    def reset(self):
        self.state.reset()

    def clear_kernel_prof(self):
        self.model.clear_kernel_prof()

    def dump_kernel_prof(self):
        for k, v in sorted(self.model.kernel_prof().items(), key=lambda kv: -kv[1]["ms"]):
            print(f"{k:24s} {v['launches']:8d} launches {v['ms']:10.3f} ms")


class Scheduler:
    """Continuous batching over one model (rsv_sched_*): submit sessions at any time, call step() repeatedly."""

    def __init__(self, model, max_slots, chunk=512, max_rows=None, max_new_cap=4096):
        h = _c.c_void_p()
        max_rows = max_rows if max_rows is not None else max(max_slots, chunk) + max_slots
        _check(native().rsv_sched_new(model._h, int(max_slots), int(chunk), int(max_rows), int(max_new_cap), _c.byref(h)))
        self._h, self._model, self._cap = h, model, int(max_new_cap)

    def submit(self, prompt, max_new, sp=None):
        t = _tokens(prompt)
        rid = _c.c_int64()
        _check(native().rsv_sched_submit(self._h, _ptr(t), t.size, int(max_new), _c.byref(sp) if sp is not None else None, _c.byref(rid)))
        return int(rid.value)

    def step(self):
        """Queues one packed step; returns (rows in the step, sessions not yet finished)."""
        rows, active = _c.c_int64(), _c.c_int64()
        _check(native().rsv_sched_step(self._h, _c.byref(rows), _c.byref(active)))
        return int(rows.value), int(active.value)

    def poll(self):
        ids = _np.zeros(1024, dtype=_np.int64)
        n = _c.c_int64()
        _check(native().rsv_sched_poll(self._h, _ptr(ids), ids.size, _c.byref(n)))
        return [int(i) for i in ids[:n.value]]

    def result(self, rid):
        out = _np.zeros(self._cap, dtype=_np.uint32)
        n = _c.c_int64()
        _check(native().rsv_sched_result(self._h, int(rid), _ptr(out), out.size, _c.byref(n)))
        return out[:n.value].copy()

    def sync(self):
        _check(native().rsv_sched_sync(self._h))

    def stats(self):
        a, b = _c.c_int64(), _c.c_int64()
        _check(native().rsv_sched_stats(self._h, _c.byref(a), _c.byref(b)))
        return {"steps": int(a.value), "rows": int(b.value)}

    def run_until_done(self):
        """Steps until every submitted session has finished; returns {id: tokens}."""
        done = {}
        while True:
            rows, active = self.step()
            for rid in self.poll():
                done[rid] = self.result(rid)
            if active == 0:
                break
            if rows == 0:
                self.sync()
        for rid in self.poll():
            done[rid] = self.result(rid)
        return done

    def close(self):
        if getattr(self, "_h", None):
            native().rsv_sched_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ModelBuilder:
    """ModelBuilder::new(path).build() (src/gpu_model.rs:3685-3703)."""

    def __init__(self, path, device=0):
        self.path, self.device = path, device

    def build(self):
        return Bundle(Model(self.path, self.device))


# ---- operator-level entry points (kernel parity tests) ----
def quantize_int8(w, device=0):
    """The reference's per-group (128) asymmetric int8 quantiser (tools/quantize_any4.py:241-300): float [M,K] -> (idx u8 [M,K], sz u32 [M,K/128])."""
    ww = _np.ascontiguousarray(w, dtype=_np.float32)
    m, k = ww.shape
    idx, sz = _np.empty((m, k), dtype=_np.uint8), _np.empty((m, k // 128), dtype=_np.uint32)
    _check(native().rsv_quantize_int8(device, _ptr(ww), m, k, _ptr(idx), _ptr(sz)))
    return idx, sz


def op_dequant_int8(idx_u8, sz_u32, device=0):
    idx = _np.ascontiguousarray(idx_u8, dtype=_np.uint8)
    sz = _np.ascontiguousarray(sz_u32, dtype=_np.uint32)
    m, k = idx.shape
    out = _np.empty((m, k), dtype=_np.float32)
    _check(native().rsv_op_dequant_int8(device, _ptr(idx), _ptr(sz), m, k, _ptr(out)))
    return out


def op_linear(x, w, sz=None, path=0, device=0):
    """y = x @ W^T.  w: float16 [M,K], or uint8 [M,K] with sz uint32 [M,K/128] (the int8 container).  path 0 SIMT, 1 tensor core."""
    xx = _np.ascontiguousarray(_np.atleast_2d(x), dtype=_np.float32)
    if sz is None:
        ww, wtype, szp = _np.ascontiguousarray(w, dtype=_np.float16), 0, None
    else:
        ww, wtype = _np.ascontiguousarray(w, dtype=_np.uint8), 1
        szz = _np.ascontiguousarray(sz, dtype=_np.uint32)
        szp = _ptr(szz)
    m, k = ww.shape
    y = _np.empty((xx.shape[0], m), dtype=_np.float32)
    _check(native().rsv_op_linear(device, int(path), wtype, _ptr(ww), szp, m, k, _ptr(xx), xx.shape[0], _ptr(y)))
    return y


def op_wkv7(r, k, v, w, a, g, k_k, k_a, r_k, lnx_w, lnx_b, state, vgate=None, vfirst=None, variant=0, device=0):
    """The WKV-7 step of one layer: inputs [nseg, T, H*64], parameters [H*64], state [nseg, H, 64, 64].  Returns (y, new state)."""
    rr = _np.ascontiguousarray(r, dtype=_np.float32)
    nseg, T, C = rr.shape
    H = C // 64
    rows = [_np.ascontiguousarray(x, dtype=_np.float32).reshape(nseg, T, C) for x in (k, v, w, a, g)]
    opt = [None if x is None else _np.ascontiguousarray(x, dtype=_np.float32).reshape(nseg, T, C) for x in (vgate, vfirst)]
    par = [_np.ascontiguousarray(x, dtype=_np.float32).reshape(C) for x in (k_k, k_a, r_k, lnx_w, lnx_b)]
    st = _np.array(state, dtype=_np.float32, order="C").reshape(nseg, H, 64, 64)
    y = _np.empty((nseg, T, C), dtype=_np.float32)
    _check(native().rsv_op_wkv7(device, int(variant), nseg, T, H, _ptr(rr), *[_ptr(x) for x in rows], *[None if x is None else _ptr(x) for x in opt],
                                *[_ptr(x) for x in par], _ptr(st), _ptr(y)))
    return y, st


def op_argmax(logits, device=0):
    lg = _np.ascontiguousarray(_np.atleast_2d(logits), dtype=_np.float32)
    out = _np.zeros(lg.shape[0], dtype=_np.uint32)
    _check(native().rsv_op_argmax(device, _ptr(lg), lg.shape[0], lg.shape[1], _ptr(out)))
    return out


def op_sample(logits, sampler_rows, hist=None, device=0):
    lg = _np.ascontiguousarray(_np.atleast_2d(logits), dtype=_np.float32)
    rows = _np.ascontiguousarray(_np.atleast_2d(sampler_rows), dtype=_np.float32)
    out = _np.zeros(lg.shape[0], dtype=_np.uint32)
    if hist is not None:
        h = _np.ascontiguousarray(_np.atleast_2d(hist), dtype=_np.uint32)
        _check(native().rsv_op_sample(device, _ptr(lg), lg.shape[0], lg.shape[1], _ptr(rows), _ptr(h), h.shape[1], _ptr(out)))
    else:
        _check(native().rsv_op_sample(device, _ptr(lg), lg.shape[0], lg.shape[1], _ptr(rows), None, 0, _ptr(out)))
    return out


# ---- synthetic checkpoints (csrc/synth.cpp) ----
class _SynthShape(_c.Structure):
    _fields_ = [(n, _c.c_int32) for n in "n_layer n_embd n_head head_size ffn_hidden vocab w_mid a_mid v_mid g_mid".split()]


# The benchmark shapes: tiny (4 layers, C=512), RWKV-7 3B and 7B.
SHAPES = {
    "tiny": dict(n_layer=4, n_embd=512, n_head=8, head_size=64, ffn_hidden=2048, vocab=4096, w_mid=32, a_mid=32, v_mid=16, g_mid=64),
    "3b": dict(n_layer=32, n_embd=2560, n_head=40, head_size=64, ffn_hidden=10240, vocab=65536, w_mid=96, a_mid=96, v_mid=64, g_mid=320),
    "7b": dict(n_layer=32, n_embd=4096, n_head=64, head_size=64, ffn_hidden=16384, vocab=65536, w_mid=128, a_mid=128, v_mid=96, g_mid=480),
}


def write_synthetic(path, shape="tiny", seed=0, quant=0, lowrank_transposed=False, quant_head=False, threads=None, **overrides):
    """Writes a seeded random-init RWKV-7 checkpoint.  quant: 0 fp16, 1 int8 symmetric per output row (in the
    reference's container), 2 int8 per group of 128 (the reference quantiser's rule)."""
    if not _os.path.exists(LIB_SYNTH):
        from . import build as _b
        _b.build_synth()
    L = _c.CDLL(LIB_SYNTH)
    L.rsv_synth_write.argtypes = [_c.c_char_p, _c.POINTER(_SynthShape), _c.c_uint64, _c.c_int, _c.c_int]
    L.rsv_synth_last_error.restype = _c.c_char_p
    L.rsv_synth_set_threads.argtypes = [_c.c_int]
    L.rsv_synth_set_threads(int(threads) if threads else (_os.cpu_count() or 1))
    d = dict(SHAPES[shape]) if isinstance(shape, str) else dict(shape)
    d.update(overrides)
    sh = _SynthShape(**d)
    flags = (1 if lowrank_transposed else 0) | (2 if quant_head else 0)
    if L.rsv_synth_write(_os.fsencode(path), _c.byref(sh), int(seed), int(quant), flags) != 0:
        raise RsvError(L.rsv_synth_last_error().decode())
    return path
