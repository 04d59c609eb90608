"""GPU parity at the benchmark's full size: the RWKV-7 3B shape with int8 weights (benchmark config 2), seeded synthetic
weights, against the fp32 CPU oracle and through size-independent properties (state round trip, batch == single,
chunked == token by token).  The checkpoint is the one `bench.py` times (same directory and file name, written once).

The oracle runs a few tokens per second at this size, so the oracle comparisons use a short prompt and a short stream; the
properties need no oracle.
"""
import os

import numpy as np
import pytest

import orc
import rwkv_rsv_b200 as rsv

pytestmark = pytest.mark.gpu
RMSE_TOL = 1e-3  # logits within an RMSE of 1e-3 of the fp32 CPU path


def rmse(a, b):
    return float(np.sqrt(np.mean((np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64)) ** 2)))


@pytest.fixture(scope="module")
def path_3b():
    d = os.environ.get("RSV_BENCH_DIR", "/tmp/rsv_bench")
    path = os.path.join(d, "rwkv7_3b_int8_seed0.st")
    if not os.path.exists(path):
        os.makedirs(d, exist_ok=True)
        tmp = path + f".tmp{os.getpid()}"
        rsv.write_synthetic(tmp, "3b", seed=0, quant=1)
        os.replace(tmp, path)
    return path


@pytest.fixture(scope="module")
def bundle_3b(path_3b):
    return rsv.ModelBuilder(path_3b).build()


def test_3b_prefill_logits_and_decode_stream_match_oracle(bundle_3b, path_3b):
    b = bundle_3b
    V = b.info().num_vocab
    prompt = np.random.default_rng(5).integers(0, V, size=6).astype(np.uint32)
    n = 6
    o = orc.OracleModel(path_3b)
    try:
        want = o.forward(prompt)
        stream_o, tok = [], int(prompt[-1])
        for _ in range(n):  # self-loop convention: the seed (= last prompt token) is fed again
            tok = orc.argmax(o.forward([tok]))
            stream_o.append(tok)
        state_o = o.state_back()
    finally:
        o.close()
    b.reset()
    lg = b.infer_seq(prompt)  # 6 rows: the tensor-core linear path
    assert rmse(lg, want) <= RMSE_TOL and rmse(lg, want) <= 1e-3 * float(want.std())
    assert int(lg.argmax()) == int(want.argmax())
    stream_g = b.infer_argmax_selfloop(int(prompt[-1]), n)  # the persistent decode kernel
    assert list(stream_g) == stream_o
    sg = b.state_back()
    assert sg.shape == state_o.shape
    assert np.abs(sg - state_o).max() <= 1e-4 * max(1.0, float(np.abs(state_o).max()))


def test_3b_state_round_trip_bit_exact_and_deterministic(bundle_3b):
    b = bundle_3b
    V = b.info().num_vocab
    prompt = np.random.default_rng(6).integers(0, V, size=40).astype(np.uint32)
    b.reset()
    b.infer_seq(prompt)
    s0 = b.state_back()
    first = b.infer_argmax_selfloop(int(prompt[-1]), 16)
    b.reset()
    b.state_load(s0)
    assert np.array_equal(b.state_back(), s0)  # bit-exact round trip
    again = b.infer_argmax_selfloop(int(prompt[-1]), 16)
    assert list(first) == list(again)


def test_3b_chunked_prefill_equals_token_by_token(bundle_3b):
    # 600 tokens: a 512-token chunk and a ragged 88-token chunk (the prefill WKV kernel with a head over two CTAs, full and
    # partial ring groups) against one token per step (the persistent decode kernel)
    b = bundle_3b
    V = b.info().num_vocab
    toks = np.random.default_rng(7).integers(0, V, size=600).astype(np.uint32)
    b.reset()
    lg_chunk = b.infer_chunked(toks, 512)
    s_chunk = b.state_back()
    b.reset()
    lg_tok = b.infer_tokens(toks)
    s_tok = b.state_back()
    assert rmse(lg_chunk, lg_tok) <= RMSE_TOL and int(lg_chunk.argmax()) == int(lg_tok.argmax())
    assert np.abs(s_chunk - s_tok).max() <= 1e-3 * max(1.0, float(np.abs(s_tok).max()))


def test_3b_batch_equals_single(bundle_3b):
    # 8 ragged sessions through the batched path (tensor-core linears, CUDA-graph self-loop) against each session alone
    b = bundle_3b
    m = b.model
    V = b.info().num_vocab
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, V, size=k).astype(np.uint32) for k in (3, 19, 1, 40, 7, 12, 28, 5)]
    B, n = len(prompts), 8
    st = m.create_batch_state(B)
    try:
        seeds = m.forward_seq_batch(st, prompts)
        out = m.collect_sample_selfloop_batch(m.submit_sample_selfloop_batch(st, seeds, n, None))
        for i in (0, 3, 7):
            b.reset()
            b.infer_seq(prompts[i])
            assert list(b.infer_argmax_selfloop(int(prompts[i][-1]), n)) == list(out[i]), i
            assert np.abs(st.slot_back(i) - b.state_back()).max() <= 1e-4, i
    finally:
        st.close()
