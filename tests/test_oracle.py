"""CPU tests of the oracle (oracle/rwkv7_cpu.cpp): the reference's own known-answer vectors, the
independent numpy restatement, and the committed golden fixtures."""
import os
import zlib

import numpy as np
import pytest

import orc
from conftest import GOLDEN, config1_tokens


def f16bits(x):
    return int(np.float16(x).view(np.uint16))


def test_int8_byte_unpack_and_scale_zero():
    # src/model.rs:839-861: idx[0]=0x00005123, scale 0.5, zero 1.0
    idx = np.zeros(32, dtype=np.uint32)
    idx[0] = 0x00005123
    sz = np.full((1, 1), (f16bits(1.0) << 16) | f16bits(0.5), dtype=np.uint32)
    w = orc.dequant_int8(idx.view(np.uint8).reshape(1, 128), sz)[0]
    assert w[0] == 0.5 * 35.0 + 1.0
    assert w[1] == 0.5 * 81.0 + 1.0
    assert w[2] == 1.0 and w[3] == 1.0
    assert np.all(w[4:] == 1.0)


def test_int8_constant_group_exact_rebuild():
    # src/model.rs:863-876: scale 0 -> exactly zero
    idx = np.zeros((1, 128), dtype=np.uint8)
    sz = np.full((1, 1), f16bits(-2.5) << 16, dtype=np.uint32)
    assert np.all(orc.dequant_int8(idx, sz) == -2.5)


def test_int8_precision_meets_target():
    # src/model.rs:878-918 with a seeded 12-uniform pseudo-gaussian (the reference uses fastrand seed 42;
    # the thresholds cos >= 0.999 and rel <= 2 % are what the test pins)
    rng = np.random.default_rng(42)
    m, k = 32, 2560
    w = (rng.random((m, k, 12), dtype=np.float32) - 0.5).sum(-1).astype(np.float32)
    wr = w.reshape(m, k // 128, 128)
    mn, mx = wr.min(-1), wr.max(-1)
    sc = (mx - mn) / 255.0
    inv = np.where(sc <= 0, 1.0, 1.0 / np.where(sc <= 0, 1.0, sc))
    q = np.clip(np.floor((wr - mn[..., None]) * inv[..., None] + 0.5), 0, 255).astype(np.uint8)  # f32::round = half away from zero
    sz = (np.float16(mn).view(np.uint16).astype(np.uint32) << 16) | np.float16(sc).view(np.uint16).astype(np.uint32)
    w_hat = orc.dequant_int8(q.reshape(m, k), sz)
    cos = float((w_hat * w).sum() / np.sqrt((w_hat ** 2).sum() * (w ** 2).sum()))
    rel = float(np.sqrt(((w_hat - w) ** 2).sum() / (w ** 2).sum()))
    assert cos >= 0.999 and rel <= 0.02


def test_dequant_matches_numpy_formula():
    rng = np.random.default_rng(5)
    idx = rng.integers(0, 256, size=(7, 384), dtype=np.uint8)
    sz = rng.integers(0, 2 ** 32, size=(7, 3), dtype=np.uint64).astype(np.uint32) & np.uint32(0x7BFF7BFF)  # finite fp16 halves
    from rwkv7_numpy import dequant_int8
    assert np.array_equal(orc.dequant_int8(idx, sz), dequant_int8(idx, sz))


def test_argmax_unique_and_tie():
    # src/backend_cuda.rs:9276-9322
    logits = np.sin(np.arange(65536, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    best = max(range(65536), key=lambda i: (logits[i], -i))
    assert orc.argmax(logits) == best
    l2 = np.zeros(1024, dtype=np.float32)
    l2[0] = l2[999] = 5.0
    assert orc.argmax(l2) == 0


def test_sampler_degenerate_cases():
    # src/backend_cuda.rs:9327-9396
    n = 4096
    logits = np.zeros(n, dtype=np.float32)
    logits[5] = 100.0
    for seed in (1, 42, 0xDEADBEEF):
        assert orc.sample(logits, seed=seed) == 5
    l2 = np.ones(n, dtype=np.float32)
    l2[7] = 2.0
    assert orc.sample(l2, temperature=0.5, top_k=1, seed=7) == 7
    l3 = np.full(n, -100.0, dtype=np.float32)
    l3[0] = l3[1] = 5.0
    assert orc.sample(l3, history=[0] * 6, seed=99, frequency_penalty=1.0) == 1


def test_u01_matches_integer_mix():
    # src/backend_cuda.rs:3691-3698 restated with Python integers
    def u01(s):
        s = (s + 0x9E3779B9) & 0xFFFFFFFF
        z = s
        z = ((z ^ (z >> 16)) * 0x85EBCA6B) & 0xFFFFFFFF
        z = ((z ^ (z >> 13)) * 0xC2B2AE35) & 0xFFFFFFFF
        z ^= z >> 16
        return np.float32(z) / np.float32(4294967296.0)
    for s in (0, 1, 12345, 0xFFFFFFFF, 0xDEADBEEF):
        assert np.float32(orc.lib().orc_u01(s)) == u01(s)


def test_sampler_top_p_semantics():
    # general path: probabilities picked from the largest down until the running sum reaches top_p;
    # everything >= the last pick is kept; draw walks the vocabulary in index order
    p = np.array([0.5, 0.3, 0.2], dtype=np.float32)
    logits = np.log(p)
    picks = {orc.sample(logits, top_p=0.75, seed=s) for s in range(200)}
    assert picks == {0, 1}           # 0.5 + 0.3 >= 0.75 -> cutoff 0.3 -> token 2 dropped
    picks = {orc.sample(logits, top_p=0.4, seed=s) for s in range(50)}
    assert picks == {0}
    picks = {orc.sample(logits, top_k=2, seed=s) for s in range(200)}
    assert picks == {0, 1}


@pytest.mark.parametrize("name", ["fp16", "int8", "int8g"])
def test_oracle_matches_numpy_restatement(tiny_paths, name):
    from rwkv7_numpy import Rwkv7Numpy
    toks = config1_tokens()[:12]
    m = orc.OracleModel(tiny_paths[name])
    lg = m.forward(toks)
    ref = Rwkv7Numpy(tiny_paths[name], np.float64)
    st = ref.new_state()
    lr = ref.forward(st, toks)
    assert np.sqrt(np.mean((lg - lr) ** 2)) < 2e-6
    sb = m.state_back()
    C, H, N, L = m.n_embd, m.n_head, m.head_size, m.n_layer
    off = 0
    for i in range(L):
        assert np.abs(sb[off:off + C] - st[i]["tmix_x"]).max() < 1e-5
        off += C
        assert np.abs(sb[off:off + H * N * N] - st[i]["S"].reshape(-1)).max() < 1e-5
        off += H * N * N
        assert np.abs(sb[off:off + C] - st[i]["cmix_x"]).max() < 1e-5
        off += C


@pytest.mark.parametrize("name", ["fp16", "int8", "int8g"])
def test_golden_fixture_reproduced(tiny_paths, name):
    g = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
    assert zlib.crc32(open(tiny_paths[name], "rb").read()) == int(g["file_crc32"]), "synthetic generator drifted"
    assert np.array_equal(g["tokens"], config1_tokens())
    m = orc.OracleModel(tiny_paths[name])
    lg = m.forward(g["tokens"])
    assert np.array_equal(lg, g["logits"])
    st = m.state_back()
    assert zlib.crc32(st.tobytes()) == int(g["state_crc32"])
    tok, stream = int(g["tokens"][-1]), []
    for _ in range(8):
        tok = orc.argmax(m.forward([tok]))
        stream.append(tok)
    assert stream == list(g["stream"][:8])


def test_oracle_thread_count_does_not_change_bits(tiny_paths):
    toks = config1_tokens()[:6]
    m = orc.OracleModel(tiny_paths["int8"])
    orc.set_threads(1)
    a = m.forward(toks)
    m.reset()
    orc.set_threads(max(2, orc.max_threads()))
    b = m.forward(toks)
    assert np.array_equal(a, b)


def test_oracle_state_roundtrip_and_reset(tiny_paths):
    toks = config1_tokens()
    m = orc.OracleModel(tiny_paths["fp16"])
    m.forward(toks[:10])
    s = m.state_back()
    a = m.forward(toks[10:14])
    m.reset()
    assert not m.state_back()[:-m.n_embd].any()
    m.state_load(s)
    assert np.array_equal(m.forward(toks[10:14]), a)
    with pytest.raises(ValueError):
        m.state_load(s[:-1])


def test_oracle_rejects_bad_token(tiny_paths):
    m = orc.OracleModel(tiny_paths["fp16"])
    with pytest.raises(RuntimeError):
        m.forward([4096])


def _rewrite_header(src, dst, edit):
    """Copies a safetensors file with its JSON header passed through `edit` (the data bytes stay as they are)."""
    import json
    import struct
    raw = open(src, "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + n])
    edit(hdr)
    out = json.dumps(hdr, separators=(",", ":")).encode()
    out += b" " * ((8 - len(out) % 8) % 8)
    open(dst, "wb").write(struct.pack("<Q", len(out)) + out + raw[8 + n:])
    return dst


def test_parser_rejects_a_shape_larger_than_its_data(tiny_paths, tmp_path):
    # A header whose shape claims more elements than the byte range holds must be refused (the reference's safetensors
    # crate refuses it too): readers copy shape-many elements.  The product library uses the same parser.
    def grow(hdr):
        hdr["ln_out.weight"]["shape"] = [hdr["ln_out.weight"]["shape"][0] * 2]
    bad = _rewrite_header(tiny_paths["fp16"], str(tmp_path / "bad_shape.st"), grow)
    with pytest.raises(RuntimeError, match="bytes but its shape"):
        orc.OracleModel(bad)

    def negative(hdr):
        hdr["emb.weight"]["shape"] = [-4096, -512]
    bad2 = _rewrite_header(tiny_paths["fp16"], str(tmp_path / "bad_neg.st"), negative)
    with pytest.raises(RuntimeError):
        orc.OracleModel(bad2)


def test_wkv7_step_matches_an_independent_float64_statement():
    # the op-level restatement (orc_wkv7) against the matrix form of the same recurrence written with einsum in float64
    rng = np.random.default_rng(12)
    H, T, N = 3, 5, 64
    C = H * N
    f = lambda *s: rng.standard_normal(s)
    sig = lambda z: 1.0 / (1.0 + np.exp(-z))
    r, k, v, g = f(T, C), f(T, C), f(T, C), f(T, C)
    w, a = np.exp(-np.exp(-0.5) * sig(f(T, C))), sig(f(T, C))
    vgate, vfirst = sig(f(T, C)), f(T, C)
    k_k, k_a, r_k = rng.uniform(0.5, 1.5, C), rng.uniform(0, 1, C), 0.02 * f(C)
    lnx_w, lnx_b = 1 + 0.02 * f(C), 0.02 * f(C)
    S0 = 0.1 * f(H, N, N)
    for gate in (False, True):
        S, ys = S0.copy(), []
        for t in range(T):
            vt = (v[t] + vgate[t] * (vfirst[t] - v[t])) if gate else v[t]
            kk = (k[t] * k_k).reshape(H, N)
            kk = kk / np.maximum(np.sqrt((kk * kk).sum(1, keepdims=True)), 1e-12)
            kt = (k[t] + k_a * (k[t] * a[t] - k[t])).reshape(H, N)
            b = -kk * a[t].reshape(H, N)
            sa = np.einsum("hij,hj->hi", S, kk)
            S = S * w[t].reshape(H, 1, N) + sa[:, :, None] * b[:, None, :] + vt.reshape(H, N)[:, :, None] * kt[:, None, :]
            y = np.einsum("hij,hj->hi", S, r[t].reshape(H, N))
            m = y.mean(1, keepdims=True)
            y = ((y - m) / np.sqrt(((y - m) ** 2).mean(1, keepdims=True) + 64e-5)).reshape(-1) * lnx_w + lnx_b
            y = y + ((r[t].reshape(H, N) * kt * r_k.reshape(H, N)).sum(1, keepdims=True) * vt.reshape(H, N)).reshape(-1)
            ys.append(y * g[t])
        got_y, got_s = orc.wkv7(r, k, v, w, a, g, k_k, k_a, r_k, lnx_w, lnx_b, S0, vgate=vgate if gate else None, vfirst=vfirst if gate else None)
        assert np.abs(got_y - np.stack(ys)).max() < 2e-5 * max(1.0, float(np.abs(np.stack(ys)).max()))
        assert np.abs(got_s - S).max() < 2e-5 * max(1.0, float(np.abs(S).max()))


def test_mean_hidden_matches_numpy_restatement(tiny_paths):
    from rwkv7_numpy import Rwkv7Numpy
    toks = config1_tokens()[:9]
    m = orc.OracleModel(tiny_paths["int8"])
    got = m.mean_hidden(toks)
    ref = Rwkv7Numpy(tiny_paths["int8"], np.float64)
    st = ref.new_state()
    acc = np.zeros(ref.C)
    for t in toks:
        ref.forward_token(st, int(t))
        acc += ref.last_hidden
    want = acc / len(toks)
    assert got.shape == want.shape and np.abs(got - want).max() < 1e-5 * max(1.0, float(np.abs(want).max()))
    # it starts from a zero state whatever the oracle held before, and leaves the prompt's state behind
    m.forward([1, 2, 3])
    assert np.array_equal(m.mean_hidden(toks), got)
    m.close()
