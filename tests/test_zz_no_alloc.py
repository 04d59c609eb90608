"""The allocation-free sampling entry point (rsv_op_sample_static), checked against rsv_op_sample.

It exists for callers that may not allocate device memory while sampling (arena/pool disciplines that ban
cudaMalloc on the hot path, latency-critical loops, plugins that only borrow buffers from their host): the
caller passes device pointers and the kernel's work area is a static device array inside the library.
This file sorts last on purpose, so a run that stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest

import orc
import rwkv_rsv_b200 as rsv

pytestmark = pytest.mark.gpu


def _static_sample(logits, srows, hist=None):
    import torch
    dev = torch.device("cuda", 0)
    lg = torch.from_numpy(np.ascontiguousarray(logits, dtype=np.float32)).to(dev)
    sr = torch.from_numpy(np.ascontiguousarray(srows, dtype=np.float32)).to(dev)
    out = torch.full((lg.shape[0],), -1, dtype=torch.int32, device=dev)
    hp, stride = None, 0
    if hist is not None:
        h = torch.from_numpy(np.ascontiguousarray(hist, dtype=np.uint32).view(np.int32)).to(dev)
        hp, stride = ctypes.c_void_p(h.data_ptr()), h.shape[1]
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream(dev)
    rc = rsv.native().rsv_op_sample_static(0, ctypes.c_void_p(stream.cuda_stream), ctypes.c_void_p(lg.data_ptr()), lg.shape[0], lg.shape[1],
                                           ctypes.c_void_p(sr.data_ptr()), hp, stride, ctypes.c_void_p(out.data_ptr()))
    if rc != 0:
        raise rsv.RsvError(rsv.native().rsv_last_error().decode())
    stream.synchronize()
    return out.cpu().numpy().view(np.uint32)


def test_static_sampler_matches_allocating_entry_point_twice():
    rng = np.random.default_rng(31)
    # call 1: penalties on (the histogram part of the work area is used), small vocabulary
    rows, V = 12, 4096
    logits = (rng.standard_normal((rows, V)) * 2).astype(np.float32)
    hist = rng.integers(0, V, size=(rows, 16)).astype(np.uint32)
    srows = np.stack([orc.pack_sampler(seed=77 + r, top_p=0.9, temperature=0.8, repetition_penalty=1.2, frequency_penalty=0.3, hist_len=16)
                      for r in range(rows)])
    want1 = rsv.op_sample(logits, srows, hist)
    got1 = _static_sample(logits, srows, hist)
    assert np.array_equal(got1, want1)
    # call 2, straight after, different shape and parameters: nothing stale may leak from call 1
    rows2, V2 = 16, 65536
    logits2 = rng.standard_normal((rows2, V2)).astype(np.float32)
    srows2 = np.stack([orc.pack_sampler(seed=5 + r, top_k=100, top_p=0.95) for r in range(rows2)])
    want2 = rsv.op_sample(logits2, srows2)
    got2 = _static_sample(logits2, srows2)
    assert np.array_equal(got2, want2)
    # and the first call repeated gives the first answer again
    assert np.array_equal(_static_sample(logits, srows, hist), want1)


def test_static_sampler_rejects_oversize_requests():
    rows, V = 17, 65536      # 17 * 65536 > 1,048,576
    with pytest.raises(rsv.RsvError, match="exceeds the static work area"):
        _static_sample(np.zeros((rows, V), dtype=np.float32), np.stack([orc.pack_sampler() for _ in range(rows)]))
