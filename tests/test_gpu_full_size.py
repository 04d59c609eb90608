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


# ---- benchmark config 2 at length: 512-token prefill, then a long free-running arg-max stream ----------------------------
def _stream_vs_oracle(b, path, prompt, n):
    """Free-running arg-max streams of the GPU self-loop and of the oracle after the same prompt.  Returns both streams, the
    oracle's top-2 logit gap at every position and, if they differ, the teacher-forced Top-1 agreement over the oracle's tokens
    (the reference's own way of judging a fork, src/main.rs:378-446, 1056-1085)."""
    o = orc.OracleModel(path)
    try:
        o.forward(prompt)
        stream_o, gaps, tok = [], [], int(prompt[-1])
        for _ in range(n):  # self-loop convention: the seed (= last prompt token) is fed again
            lg = o.forward([tok])
            top2 = np.partition(lg, -2)[-2:]
            gaps.append(float(top2[1] - top2[0]))
            tok = int(orc.argmax(lg))
            stream_o.append(tok)
    finally:
        o.close()
    b.reset()
    b.infer_chunked(prompt, 512)
    stream_g = [int(t) for t in b.infer_argmax_selfloop(int(prompt[-1]), n)]
    forced = None
    if stream_g != stream_o:
        b.reset()
        b.infer_chunked(prompt, 512)
        fed = np.asarray([int(prompt[-1])] + stream_o[:-1], dtype=np.uint32)
        full = b.infer(rsv.RnnInput(fed, 0, rsv.RnnOption.Full)).reshape(len(fed), -1)
        forced = float(np.mean(full.argmax(1) == np.asarray(stream_o)))
    return stream_g, stream_o, gaps, forced


def _assert_identical_stream(stream_g, stream_o, gaps, forced):
    if stream_g == stream_o:
        return
    p = next(i for i, (x, y) in enumerate(zip(stream_g, stream_o)) if x != y)
    raise AssertionError(f"arg-max streams fork at position {p} of {len(stream_o)}: GPU {stream_g[p]}, oracle {stream_o[p]}; the oracle's top-2 logit gap "
                         f"there is {gaps[p]:.3e} (smallest gap over the stream {min(gaps):.3e}); teacher-forced Top-1 agreement over the oracle's tokens "
                         f"{forced:.4f}")


def test_3b_config2_prefill_512_then_256_token_stream(bundle_3b, path_3b):
    # 512-token prompt through the chunked prefill path (tcgen05 linears, sequence WKV kernel), then 256 tokens from the
    # single-launch decode kernel, against the fp32 CPU oracle (about four minutes of oracle time on 16 cores)
    prompt = np.random.default_rng(1).integers(0, bundle_3b.info().num_vocab, size=512).astype(np.uint32)
    _assert_identical_stream(*_stream_vs_oracle(bundle_3b, path_3b, prompt, 256))


@pytest.mark.skipif(not os.environ.get("RSV_SLOW"), reason="the full 1000-token stream of benchmark config 2 needs about eight minutes of oracle time: set RSV_SLOW=1")
def test_3b_config2_prefill_512_then_1000_token_stream(bundle_3b, path_3b):
    prompt = np.random.default_rng(1).integers(0, bundle_3b.info().num_vocab, size=512).astype(np.uint32)
    _assert_identical_stream(*_stream_vs_oracle(bundle_3b, path_3b, prompt, 1000))


# ---- the same shape with fp16 weights (benchmark config 3 names both) -----------------------------------------------------
def _checkpoint(shape, quant_name):
    d = os.environ.get("RSV_BENCH_DIR", "/tmp/rsv_bench")
    path = os.path.join(d, f"rwkv7_{shape}_{quant_name}_seed0.st")
    if not os.path.exists(path):
        os.makedirs(d, exist_ok=True)
        tmp = path + f".tmp{os.getpid()}"
        rsv.write_synthetic(tmp, shape, seed=0, quant={"fp16": 0, "int8": 1, "int8g": 2}[quant_name])
        os.replace(tmp, path)
    return path


def _short_parity(path, n_prompt, n_stream, chunk_tokens):
    """Prefill logits, a short arg-max stream and the state against the oracle; then chunked prefill == token by token."""
    b = rsv.ModelBuilder(path).build()
    try:
        V = b.info().num_vocab
        prompt = np.random.default_rng(5).integers(0, V, size=n_prompt).astype(np.uint32)
        o = orc.OracleModel(path)
        try:
            want = o.forward(prompt)
            stream_o, tok = [], int(prompt[-1])
            for _ in range(n_stream):
                tok = int(orc.argmax(o.forward([tok])))
                stream_o.append(tok)
            state_o = o.state_back()
        finally:
            o.close()
        b.reset()
        lg = b.infer_seq(prompt)
        assert rmse(lg, want) <= RMSE_TOL and rmse(lg, want) <= 1e-3 * float(want.std())
        assert int(lg.argmax()) == int(want.argmax())
        assert [int(t) for t in b.infer_argmax_selfloop(int(prompt[-1]), n_stream)] == stream_o
        sg = b.state_back()
        assert np.abs(sg - state_o).max() <= 1e-4 * max(1.0, float(np.abs(state_o).max()))
        # size-independent property at this shape: a long prompt in chunks equals the same prompt token by token
        toks = np.random.default_rng(7).integers(0, V, size=chunk_tokens + 40).astype(np.uint32)
        b.reset()
        lg_chunk = b.infer_chunked(toks, chunk_tokens)
        s_chunk = b.state_back()
        b.reset()
        lg_tok = b.infer_tokens(toks)
        s_tok = b.state_back()
        assert rmse(lg_chunk, lg_tok) <= RMSE_TOL and int(lg_chunk.argmax()) == int(lg_tok.argmax())
        assert np.abs(s_chunk - s_tok).max() <= 1e-3 * max(1.0, float(np.abs(s_tok).max()))
    finally:
        b.state.close()
        b.model.close()


def test_3b_fp16_matches_oracle():
    # fp16 weights at the 3B shape: the fp16 tensor-core linears (prefill) and the fp16 rows of the decode kernel
    _short_parity(_checkpoint("3b", "fp16"), n_prompt=6, n_stream=32, chunk_tokens=512)


def test_7b_int8_matches_oracle():
    # benchmark config 5's model: C = 4096, 64 heads, FFN 16384 (wider LayerNorm rows, more pieces per row, more tiles per SM),
    # prefill chunk 1024
    _short_parity(_checkpoint("7b", "int8"), n_prompt=6, n_stream=6, chunk_tokens=1024)


def test_3b_per_group_int8_matches_oracle():
    # the reference's own container (one scale and zero per row and group of 128 weights) at the 3B shape: the one-launch decode
    # kernel rescales every group inside its multiply loop; prefill runs on the weight-streaming SIMT kernel
    _short_parity(_checkpoint("3b", "int8g"), n_prompt=6, n_stream=16, chunk_tokens=64)
