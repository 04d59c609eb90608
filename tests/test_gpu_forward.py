"""GPU parity of the forward step against the CPU oracle, through the reference-shaped API
(ModelBuilder / Bundle / State), which calls the C ABI.

Tolerances: int8 dequant and state round-trip bit-exact, arg-max token streams identical, logits within an RMSE of
1e-3 of the fp32 CPU path.
"""
import os

import numpy as np
import pytest

import orc
import rwkv_rsv_b200 as rsv
from conftest import GOLDEN, config1_tokens

pytestmark = pytest.mark.gpu
RMSE_TOL = 1e-3


def rmse(a, b):
    return float(np.sqrt(np.mean((np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64)) ** 2)))


@pytest.fixture(scope="module")
def bundles(tiny_paths):
    return {k: rsv.ModelBuilder(p).build() for k, p in tiny_paths.items()}


@pytest.fixture(scope="module")
def oracles(tiny_paths):
    return {k: orc.OracleModel(p) for k, p in tiny_paths.items()}


def test_model_info(bundles):
    i = bundles["fp16"].info()
    assert (i.version, i.num_layer, i.num_emb, i.num_hidden, i.num_vocab, i.num_head, i.head_size, i.ffn_hidden) == ("V7", 4, 512, 512, 4096, 8, 64, 2048)
    assert (i.w_mid, i.a_mid, i.v_mid, i.g_mid) == (32, 32, 16, 64)
    assert bundles["int8"].model.weight_bytes() < bundles["fp16"].model.weight_bytes()


@pytest.mark.parametrize("name", ["fp16", "int8", "int8g"])
def test_decode_logits_and_state_vs_oracle_and_golden(bundles, oracles, name):
    b, o = bundles[name], oracles[name]
    toks = config1_tokens()
    b.reset()
    o.reset()
    lg = b.infer_tokens(toks)
    want = o.forward(toks)
    g = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
    assert np.array_equal(want, g["logits"])
    assert rmse(lg, want) <= RMSE_TOL and rmse(lg, want) <= 1e-3 * float(want.std())
    assert int(lg.argmax()) == int(want.argmax())
    sg, so = b.state_back(), o.state_back()
    assert sg.shape == so.shape
    assert np.abs(sg - so).max() <= 1e-4 * max(1.0, float(np.abs(so).max()))


@pytest.mark.parametrize("name", ["fp16", "int8", "int8g"])
def test_argmax_stream_identical_config1(bundles, name):
    # benchmark config 1: 128 prompt tokens, then 64 arg-max tokens from the GPU self-loop
    b = bundles[name]
    g = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
    b.reset()
    b.infer_seq(g["tokens"])
    stream = b.infer_argmax_selfloop(int(g["tokens"][-1]), 64)
    assert list(stream) == list(g["stream"]), f"first divergence at {int(np.argmax(stream != g['stream']))}, oracle top-2 gaps {g['top2_gap'][:8]}"


def test_teacher_forced_top1_agreement(bundles, oracles):
    # the reference's own check (src/main.rs:378-446): per-position arg-max with the oracle's tokens forced
    b, o = bundles["int8"], oracles["int8"]
    toks = config1_tokens()[:48]
    b.reset()
    o.reset()
    full = b.infer(rsv.RnnInput(toks, 0, rsv.RnnOption.Full)).reshape(len(toks), -1)
    want = o.forward(toks, full=True)
    assert np.array_equal(full.argmax(1), want.argmax(1))
    assert rmse(full, want) <= RMSE_TOL


@pytest.mark.parametrize("name", ["fp16", "int8g"])
def test_seq_chunked_and_token_paths_agree(bundles, oracles, name):
    b, o = bundles[name], oracles[name]
    toks = config1_tokens()[:77]
    o.reset()
    want = o.forward(toks)
    outs = {}
    b.reset()
    outs["tokens"] = b.infer_tokens(toks)
    s_tok = b.state_back()
    b.reset()
    outs["seq"] = b.infer_seq(toks)
    s_seq = b.state_back()
    b.reset()
    outs["chunk16"] = b.infer_chunked(toks, 16)
    b.reset()
    outs["chunk1"] = b.infer_chunked(toks, 1)
    b.reset()
    b.infer_seq(toks[:30])
    outs["split"] = b.infer_tokens(toks[30:])
    for k, v in outs.items():
        assert rmse(v, want) <= RMSE_TOL, k
        assert int(v.argmax()) == int(want.argmax()), k
    assert np.abs(s_tok - s_seq).max() <= 1e-4


@pytest.mark.parametrize("name", ["int8", "fp16"])
def test_long_prompt_single_chunk(bundles, oracles, name):
    # 700 rows in one step: the large-row variants of the LayerNorm / operand-preparation kernels and many N tiles per GEMM
    b, o = bundles[name], oracles[name]
    toks = np.random.default_rng(7).integers(0, 4096, size=700).astype(np.uint32)
    o.reset()
    want = o.forward(toks)
    b.reset()
    got = b.infer_seq(toks)
    assert rmse(got, want) <= RMSE_TOL and int(got.argmax()) == int(want.argmax())
    so, sg = o.state_back(), b.state_back()
    assert np.abs(sg - so).max() <= 1e-4 * max(1.0, float(np.abs(so).max()))
    # the same prompt in chunks of 256 reaches the same state
    b.reset()
    b.infer_chunked(toks, 256)
    assert np.abs(b.state_back() - sg).max() <= 1e-4 * max(1.0, float(np.abs(sg).max()))


def test_state_roundtrip_bit_exact_and_reset(bundles):
    # examples/state_persist.rs:54-67: back -> load -> back must give max_diff == 0
    b = bundles["int8"]
    toks = config1_tokens()
    b.reset()
    b.infer_seq(toks[:40])
    s = b.state_back()
    cont = b.infer_tokens(toks[40:48])
    s_after = b.state_back()
    b.reset()
    z = b.state_back()
    assert not z.any()
    b.state_load(s)
    assert np.array_equal(b.state_back().view(np.uint32), s.view(np.uint32))
    again = b.infer_tokens(toks[40:48])
    assert np.array_equal(again.view(np.uint32), cont.view(np.uint32))        # deterministic kernels: same bits
    assert np.array_equal(b.state_back().view(np.uint32), s_after.view(np.uint32))
    with pytest.raises(rsv.RsvError, match="length"):
        b.state_load(s[:-1])


def test_argmax_and_sample_entry_points(bundles, oracles):
    b, o = bundles["fp16"], oracles["fp16"]
    toks = config1_tokens()[:20]
    b.reset()
    o.reset()
    want = o.forward(toks)
    assert b.infer_argmax(toks) == int(want.argmax())
    b.reset()
    sp = rsv.SamplerParams(temperature=0.8, top_k=0, top_p=0.9, seed=1234)
    hist = [1, 2, 3]
    got = b.infer_sample(toks, sp, hist)
    assert got == orc.sample(want, history=hist, temperature=0.8, top_p=0.9, seed=1234)
    # top_k = 1 is arg-max whatever the seed
    b.reset()
    assert b.infer_sample(toks, rsv.SamplerParams(top_k=1, seed=99)) == int(want.argmax())


def test_sample_selfloop_follows_oracle(bundles, oracles):
    # round r: RNG seed = seed_token + r, history = the r tokens generated so far (src/gpu_model.rs:790-810)
    b, o = bundles["int8"], oracles["int8"]
    toks = config1_tokens()[:32]
    sp = rsv.SamplerParams(temperature=1.0, top_p=0.9, repetition_penalty=1.1)
    b.reset()
    o.reset()
    b.infer_seq(toks)
    o.forward(toks)
    seed, n = int(toks[-1]), 24
    got = b.infer_sample_selfloop(seed, n, sp)
    tok, want = seed, []
    for r in range(n):
        lg = o.forward([tok])
        tok = orc.sample(lg, history=want, temperature=1.0, top_p=0.9, repetition_penalty=1.1, seed=(seed + r) & 0xFFFFFFFF)
        want.append(tok)
    assert list(got) == want


def test_batch_equals_single(bundles, tiny_paths):
    # batch == single equivalence, the reference's gemv_variant_mb / rkv_stage1_batch / sample_batch tests
    # (src/backend_cuda.rs:7919, 8074, 8195) at the level of whole sessions
    b = bundles["int8"]
    m = b.model
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, 4096, size=n).astype(np.uint32) for n in (5, 17, 1, 64, 33)]
    B, n = len(prompts), 12
    singles, states = [], []
    for p in prompts:
        b.reset()
        b.infer_seq(p)
        singles.append(b.infer_argmax_selfloop(int(p[-1]), n))
        states.append(b.state_back())
    st = m.create_batch_state(B)
    seeds = m.forward_seq_batch(st, prompts)
    assert list(seeds) == [int(p[-1]) for p in prompts]
    out = m.collect_sample_selfloop_batch(m.submit_sample_selfloop_batch(st, seeds, n, None))
    for i in range(B):
        assert list(out[i]) == list(singles[i]), i
        assert np.abs(st.slot_back(i) - states[i]).max() <= 1e-4
    # slot_load / slot_back round trip and whole-state layout = slots concatenated
    whole = st.back()
    per = len(whole) // B
    assert np.array_equal(whole[2 * per:3 * per], st.slot_back(2))
    st.slot_load(1, states[3])
    assert np.array_equal(st.slot_back(1), states[3])
    with pytest.raises(rsv.RsvError, match="slot"):
        st.slot_back(B)
    # sampling in a batch: slot b uses seeds[b] + round as its RNG seed, like the single-session loop
    sp = rsv.SamplerParams(top_p=0.9)
    st2 = m.create_batch_state(2)
    m.forward_seq_batch(st2, prompts[:2])
    got = m.collect_sample_selfloop_batch(m.submit_sample_selfloop_batch(st2, [int(prompts[0][-1]), int(prompts[1][-1])], 8, sp))
    for i in range(2):
        b.reset()
        b.infer_seq(prompts[i])
        assert list(b.infer_sample_selfloop(int(prompts[i][-1]), 8, sp)) == list(got[i])


def test_many_sessions_equal_single(bundles):
    # 96 sessions x 8 heads = 768 (head, segment) pairs: the ragged prefill (segments of 1-8 tokens: full and partial ring groups)
    # runs wkv7_seq_kernel<4> (a head per CTA), the decode steps the row-per-lane kernel for large batches; the single-session
    # runs they are compared with use wkv7_seq_kernel<2> (a head over two CTAs) and the persistent decode kernel
    b = bundles["int8"]
    m = b.model
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, 4096, size=int(n)).astype(np.uint32) for n in rng.integers(1, 9, size=96)]
    B, n = len(prompts), 5
    st = m.create_batch_state(B)
    seeds = m.forward_seq_batch(st, prompts)
    out = m.collect_sample_selfloop_batch(m.submit_sample_selfloop_batch(st, seeds, n, None))
    for i in (0, 1, 17, 40, 63, 95):
        b.reset()
        b.infer_seq(prompts[i])
        assert list(b.infer_argmax_selfloop(int(prompts[i][-1]), n)) == list(out[i]), i
        assert np.abs(st.slot_back(i) - b.state_back()).max() <= 1e-4, i


def test_error_paths(bundles, tiny_paths):
    b = bundles["fp16"]
    with pytest.raises(rsv.RsvError, match="vocab"):
        b.infer_tokens([5, 4096])
    with pytest.raises(rsv.RsvError, match="empty"):
        b.infer_tokens([])
    st = b.model.create_batch_state(3)
    with pytest.raises(rsv.RsvError, match="batch"):
        b.model.submit_sample_selfloop_batch(st, [1, 2], 4, None)
    with pytest.raises(rsv.RsvError):
        rsv.ModelBuilder(tiny_paths["fp16"] + ".missing").build()
    b.reset()
    assert b.infer_tokens([7]).shape == (4096,)       # the handle is still usable after errors


def test_lowrank_transposed_and_quantised_head_checkpoints(model_dir, bundles):
    # the loader accepts both low-rank orientations (src/model.rs:564-581) and an int8 head
    # (tools/quantize_any4.py:696-712)
    p = rsv.write_synthetic(os.path.join(model_dir, "tiny_t.st"), "tiny", seed=0, quant=2, lowrank_transposed=True, quant_head=True)
    b, o = rsv.ModelBuilder(p).build(), orc.OracleModel(p)
    toks = config1_tokens()[:24]
    lg, want = b.infer_seq(toks), o.forward(toks)
    assert rmse(lg, want) <= RMSE_TOL and int(lg.argmax()) == int(want.argmax())


def test_kernel_profile_and_launch_count(bundles):
    b = bundles["fp16"]
    b.reset()
    b.clear_kernel_prof()
    b.model.prof_enable(True)
    b.infer_tokens([1, 2, 3])
    b.model.prof_enable(False)
    prof = b.model.kernel_prof()
    assert prof["wkv7"]["launches"] == 3 * 4 and prof["linear_head"]["launches"] == 1
    assert b.model.launch_count() == sum(v["launches"] for v in prof.values())


def test_batch_mean_hidden_matches_cpu_path(bundles, oracles):
    # forward_seq_batch_mean_hidden (src/gpu_model.rs:1013-1036): per slot the token mean of the last layer's residual stream,
    # from a zero state whatever the state held before; ragged lengths, one prompt longer than a packed step
    m, o = bundles["int8"].model, oracles["int8"]
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, m.info().num_vocab, size=k).astype(np.uint32) for k in (1, 7, 40, 1300)]
    st = m.create_batch_state(len(prompts))
    try:
        m.forward_seq_batch(st, [p[:5] for p in prompts])  # something to reset
        feat = m.forward_seq_batch_mean_hidden(st, prompts, pad_to=1536)
        assert feat.shape == (4, m.info().num_emb)
        for b, p in enumerate(prompts):
            want = o.mean_hidden(p)
            assert np.abs(feat[b] - want).max() <= 1e-4 * max(1.0, float(np.abs(want).max())), b
            assert np.abs(st.slot_back(b) - o.state_back()).max() <= 1e-4 * max(1.0, float(np.abs(o.state_back()).max())), b
        again = m.forward_seq_batch_mean_hidden(st, prompts)  # deterministic, and independent of the row pitch
        assert np.array_equal(again, feat)
    finally:
        st.close()
        o.reset()


def test_states_of_different_batch_sizes_one_after_the_other(bundles):
    # The one-launch decode kernels keep per-layer state pointers in a device table; a new state may reuse the freed
    # state's addresses with another slot count (other per-layer strides), so the table has to follow the state, not its address.
    b = bundles["int8"]
    m = b.model
    rng = np.random.default_rng(31)
    prompts = [rng.integers(0, m.info().num_vocab, size=k).astype(np.uint32) for k in (9, 3, 17, 5)]
    want = []
    for p in prompts:
        b.reset()
        b.infer_seq(p)
        want.append(list(b.infer_argmax_selfloop(int(p[-1]), 12)))
    for batch in (4, 1, 2, 3, 4):  # allocate, decode, free - the allocator hands the same blocks out again
        st = m.create_batch_state(batch)
        try:
            seeds = m.forward_seq_batch(st, prompts[:batch])
            out = m.collect_sample_selfloop_batch(m.submit_sample_selfloop_batch(st, seeds, 12, None))
            for i in range(batch):
                assert list(out[i]) == want[i], (batch, i)
        finally:
            st.close()


def test_malformed_checkpoints_are_refused_by_the_loader(tiny_paths, tmp_path):
    import json
    import struct

    def rewrite(dst, edit):
        raw = open(tiny_paths["fp16"], "rb").read()
        n = struct.unpack("<Q", raw[:8])[0]
        hdr = json.loads(raw[8:8 + n])
        edit(hdr)
        out = json.dumps(hdr, separators=(",", ":")).encode()
        out += b" " * ((8 - len(out) % 8) % 8)
        open(dst, "wb").write(struct.pack("<Q", len(out)) + out + raw[8 + n:])
        return str(dst)

    def grow(hdr):  # a shape that claims twice the elements its byte range holds
        hdr["ln_out.weight"]["shape"] = [hdr["ln_out.weight"]["shape"][0] * 2]
    with pytest.raises(rsv.RsvError, match="bytes but its shape"):
        rsv.Model(rewrite(tmp_path / "grow.st", grow))

    def negative(hdr):
        hdr["emb.weight"]["shape"] = [-4096, -512]
    with pytest.raises(rsv.RsvError):
        rsv.Model(rewrite(tmp_path / "neg.st", negative))

    def past_the_end(hdr):
        a, e = hdr["head.weight"]["data_offsets"]
        hdr["head.weight"]["data_offsets"] = [a, e + (1 << 30)]
    with pytest.raises(rsv.RsvError):
        rsv.Model(rewrite(tmp_path / "range.st", past_the_end))
    open(tmp_path / "short.st", "wb").write(open(tiny_paths["fp16"], "rb").read()[:1000])
    with pytest.raises(rsv.RsvError):
        rsv.Model(str(tmp_path / "short.st"))
    assert rsv.Model(tiny_paths["fp16"]).info().num_layer == 4  # the library still loads a good file afterwards


def test_text_level_driver(bundles, tiny_paths, tmp_path, capsys):
    # examples/generate.rs:20-113 as a library function and a command: text -> tokens -> prefill -> self-loop -> text
    import json

    from rwkv_rsv_b200 import generate as gen
    from rwkv_rsv_b200.tokenizer import Tokenizer
    vocab = {str(i + 1): [i] for i in range(256)}
    vocab.update({"300": "the ", "301": "tower", "302": " tow"})
    vocab.update({str(i): [128 + (i >> 8), i & 255] for i in range(303, 4096)})  # every id the tiny model can emit decodes
    vf = tmp_path / "vocab.json"
    vf.write_text(json.dumps(vocab))
    tk = Tokenizer(vf.read_text())
    prompt = tk.encode("the tower")
    assert prompt == [300, 301]
    b = bundles["int8"]
    b.reset()
    out, _ = gen.generate(b, prompt, 12, mode="argmax")
    b.reset()
    b.infer_tokens(prompt)
    assert out == [int(t) for t in b.infer_argmax_selfloop(prompt[-1], 12)]
    b.reset()
    s1, _ = gen.generate(b, prompt, 12)
    b.reset()
    s2, _ = gen.generate(b, prompt, 12)
    assert s1 == s2 and len(s1) == 12  # seeded sampling is reproducible
    assert gen.main(["--model", tiny_paths["int8"], "--vocab", str(vf), "--prompt", "the tower", "--tokens", "5", "--mode", "argmax"]) == 0
    printed = capsys.readouterr().out.splitlines()
    assert json.loads(printed[0])[:2] == prompt and len(json.loads(printed[0])) == 7
    with pytest.raises(SystemExit):
        gen.main(["--model", tiny_paths["int8"], "--prompt", "x"])


def test_first_use_of_the_small_batch_kernel_on_recycled_memory(bundles, tiny_paths):
    # The one-launch kernels allocate their counters and scratch on first use; the allocator may hand them memory another buffer
    # has just left full of other bits, and zeroing it has to be ordered before the first launch on the model's own stream.
    b = bundles["int8"]
    rng = np.random.default_rng(41)
    prompts = [rng.integers(0, 4096, size=k).astype(np.uint32) for k in (11, 4, 23)]
    want = []
    for p in prompts:
        b.reset()
        b.infer_seq(p)
        want.append(list(b.infer_argmax_selfloop(int(p[-1]), 10)))
    m = rsv.Model(tiny_paths["int8"])  # a fresh handle: nothing built yet
    try:
        big = m.create_batch_state(96)
        big.load(np.full(len(big), -3.0e38, dtype=np.float32))  # 50 MB of non-zero bits ...
        big.close()                                             # ... back to the allocator
        st = m.create_batch_state(3)
        seeds = m.forward_seq_batch(st, prompts)
        out = m.collect_sample_selfloop_batch(m.submit_sample_selfloop_batch(st, seeds, 10, None))  # first launch of the 2-4 session kernel
        for i in range(3):
            assert list(out[i]) == want[i], i
        st.close()
    finally:
        m.close()
