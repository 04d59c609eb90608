"""GPU parity of the stand-alone operators, called through the C ABI (host buffers in and out)."""
import numpy as np
import pytest

import orc
import rwkv_rsv_b200 as rsv

pytestmark = pytest.mark.gpu


def f16bits(x):
    return int(np.float16(x).view(np.uint16))


def test_dequant_known_answers():
    idx = np.zeros(32, dtype=np.uint32)
    idx[0] = 0x00005123
    sz = np.full((1, 1), (f16bits(1.0) << 16) | f16bits(0.5), dtype=np.uint32)
    w = rsv.op_dequant_int8(idx.view(np.uint8).reshape(1, 128), sz)[0]
    assert w[0] == 18.5 and w[1] == 41.5 and np.all(w[2:] == 1.0)
    sz = np.full((1, 1), f16bits(-2.5) << 16, dtype=np.uint32)
    assert np.all(rsv.op_dequant_int8(np.zeros((1, 128), dtype=np.uint8), sz) == -2.5)


def test_dequant_bit_exact_vs_oracle():
    rng = np.random.default_rng(11)
    for m, k in ((3, 128), (32, 2560), (257, 1024)):
        idx = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
        sz = rng.integers(0, 2 ** 32, size=(m, k // 128), dtype=np.uint64).astype(np.uint32) & np.uint32(0x7BFF7BFF)
        got, want = rsv.op_dequant_int8(idx, sz), orc.dequant_int8(idx, sz)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_argmax_unique_tie_and_batch():
    logits = np.sin(np.arange(65536, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    assert int(rsv.op_argmax(logits)[0]) == orc.argmax(logits)
    l2 = np.zeros(1024, dtype=np.float32)
    l2[0] = l2[999] = 5.0
    assert int(rsv.op_argmax(l2)[0]) == 0
    rng = np.random.default_rng(3)
    lg = rng.standard_normal((37, 4099)).astype(np.float32)
    lg[5, 100] = lg[5, 4000] = 9.0          # a tie inside one row
    got = rsv.op_argmax(lg)
    assert [int(t) for t in got] == [orc.argmax(r) for r in lg]
    assert int(rsv.op_argmax(np.array([3.0], dtype=np.float32))[0]) == 0


def test_sampler_degenerate_cases():
    n = 4096
    logits = np.zeros(n, dtype=np.float32)
    logits[5] = 100.0
    for seed in (1, 42, 0xDEADBEEF):
        assert int(rsv.op_sample(logits, orc.pack_sampler(seed=seed))[0]) == 5
    l2 = np.ones(n, dtype=np.float32)
    l2[7] = 2.0
    assert int(rsv.op_sample(l2, orc.pack_sampler(temperature=0.5, top_k=1, seed=7))[0]) == 7
    l3 = np.full(n, -100.0, dtype=np.float32)
    l3[0] = l3[1] = 5.0
    hist = np.zeros((1, 6), dtype=np.uint32)
    assert int(rsv.op_sample(l3, orc.pack_sampler(seed=99, frequency_penalty=1.0, hist_len=6), hist)[0]) == 1


@pytest.mark.parametrize("params", [
    dict(), dict(top_p=0.9), dict(top_k=40), dict(top_k=200, top_p=0.8, temperature=0.7), dict(temperature=1.5, top_p=0.5),
    dict(top_k=5, temperature=0.0), dict(top_p=0.9, repetition_penalty=1.3, presence_penalty=0.4, frequency_penalty=0.2),
])
def test_sampler_matches_oracle_on_random_logits(params):
    rng = np.random.default_rng(17)
    rows, V = 24, 4096
    logits = (rng.standard_normal((rows, V)) * 2.0).astype(np.float32)
    hist = rng.integers(0, V, size=(rows, 20)).astype(np.uint32)
    use_hist = "repetition_penalty" in params
    srows = np.stack([orc.pack_sampler(seed=1000 + r, hist_len=20 if use_hist else 0, **params) for r in range(rows)])
    got = rsv.op_sample(logits, srows, hist if use_hist else None)
    want = [orc.sample(logits[r], history=hist[r] if use_hist else (), seed=1000 + r, **params) for r in range(rows)]
    # the draw compares a running fp32 sum with u; the two implementations group that sum differently,
    # so allow a rare boundary disagreement but nothing systematic
    agree = sum(int(g) == w for g, w in zip(got, want))
    assert agree >= rows - 1, (list(got), want)


def test_sampler_large_vocab_top_p_cap():
    # flat-ish distribution over 65536 tokens: top_p 0.9 is never reached within the 512 picks the
    # reference allows, so the kept set is the 512 most probable tokens
    rng = np.random.default_rng(23)
    logits = rng.standard_normal((4, 65536)).astype(np.float32)
    srows = np.stack([orc.pack_sampler(seed=s, top_p=0.9) for s in (5, 6, 7, 8)])
    got = rsv.op_sample(logits, srows)
    want = [orc.sample(logits[r], seed=5 + r, top_p=0.9) for r in range(4)]
    assert [int(g) for g in got] == want
    for r in range(4):
        assert logits[r, int(got[r])] >= np.sort(logits[r])[-512]


def _int8_container(rng, m, k, per_row):
    idx = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
    scale = (rng.random((m, 1 if per_row else k // 128)) * 0.01 + 0.001).astype(np.float16)
    zero = (-128.0 * scale.astype(np.float32)).astype(np.float16) if per_row else (rng.standard_normal(scale.shape) * 0.05).astype(np.float16)
    sz = (zero.view(np.uint16).astype(np.uint32) << 16) | scale.view(np.uint16).astype(np.uint32)
    if per_row:
        sz = np.repeat(sz, k // 128, axis=1)
    return idx, np.ascontiguousarray(sz)


def _ref_linear(x, w64):
    return x.astype(np.float64) @ w64.T


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("shape", [(128, 128, 1), (256, 512, 3), (2560, 2560, 1), (512, 2048, 8), (1024, 512, 70), (384, 256, 300)])
def test_linear_int8_vs_float64(path, shape):
    # fp16/int8 GEMV / GEMM unit tests of the reference (src/backend_cuda.rs:8880-9066) with fp32-accurate bounds
    m, k, r = shape
    rng = np.random.default_rng(m * 7 + k + r)
    idx, sz = _int8_container(rng, m, k, per_row=True)
    x = rng.standard_normal((r, k)).astype(np.float32)
    x[0, :5] = [0.0, 1e-6, -3.0, 7.5, -1e-3]
    want = _ref_linear(x, orc.dequant_int8(idx, sz).astype(np.float64))
    got = rsv.op_linear(x, idx, sz, path=path)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-5 * scale, (path, shape, float(np.abs(got - want).max()), float(scale))


def test_linear_int8_per_group_container_simt():
    rng = np.random.default_rng(9)
    idx, sz = _int8_container(rng, 256, 512, per_row=False)
    x = rng.standard_normal((5, 512)).astype(np.float32)
    want = _ref_linear(x, orc.dequant_int8(idx, sz).astype(np.float64))
    got = rsv.op_linear(x, idx, sz, path=0)
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
    with pytest.raises(rsv.RsvError, match="tensor-core path"):
        rsv.op_linear(x, idx, sz, path=1)


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("shape", [(128, 64, 1), (96, 512, 4), (512, 96, 9), (4096, 512, 2), (320, 2560, 33), (2560, 16, 6)])
def test_linear_fp16_vs_float64(path, shape):
    m, k, r = shape
    rng = np.random.default_rng(m + k * 3 + r)
    w = (rng.standard_normal((m, k)) * 0.02).astype(np.float16)
    x = rng.standard_normal((r, k)).astype(np.float32)
    want = _ref_linear(x, w.astype(np.float64))
    got = rsv.op_linear(x, w, None, path=path)
    assert np.abs(got - want).max() <= 2e-5 * max(np.abs(want).max(), 1e-3), (path, shape, float(np.abs(got - want).max()))


def test_linear_tc_is_schedule_independent_and_exact_in_integers():
    # the int8 tensor-core path accumulates exactly: integer-valued activations give the exact integer result
    rng = np.random.default_rng(2)
    m, k = 256, 1024
    idx = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
    one, mz = np.float16(1.0).view(np.uint16), np.float16(-128.0).view(np.uint16)
    sz = np.full((m, k // 128), (int(mz) << 16) | int(one), dtype=np.uint32)
    x = rng.integers(-64, 65, size=(3, k)).astype(np.float32)
    want = x.astype(np.int64) @ (idx.astype(np.int64) - 128).T
    got = rsv.op_linear(x, idx, sz, path=1)
    assert np.array_equal(got.astype(np.int64), want)


# ---- the WKV-7 step of one layer, each of its kernels on its own --------------------------------------------------------------
def _wkv_case(nseg, T, H, seed, gate):
    """Seeded inputs with the forward step's value ranges: decay in (e^-0.61, 1), a and the gates in (0, 1), a state with history."""
    rng = np.random.default_rng(seed)
    C = H * 64
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    sig = lambda x: (1.0 / (1.0 + np.exp(-x))).astype(np.float32)
    d = dict(r=f(nseg, T, C), k=f(nseg, T, C), v=f(nseg, T, C), w=np.exp(-np.exp(-0.5) * sig(f(nseg, T, C) * 2 - 2)).astype(np.float32),
             a=sig(f(nseg, T, C)), g=f(nseg, T, C), k_k=rng.uniform(0.5, 1.5, C).astype(np.float32), k_a=rng.uniform(0, 1, C).astype(np.float32),
             r_k=(0.02 * f(C)), lnx_w=(1 + 0.02 * f(C)), lnx_b=(0.02 * f(C)), state=0.1 * f(nseg, H, 64, 64))
    if gate:
        d["vgate"], d["vfirst"] = sig(f(nseg, T, C)), f(nseg, T, C)
    return d


def _wkv_oracle(d):
    nseg = d["r"].shape[0]
    ys, ss = [], []
    per_seg = ("r", "k", "v", "w", "a", "g", "vgate", "vfirst", "state")
    for s in range(nseg):
        y, st = orc.wkv7(**{k: (v[s] if k in per_seg else v) for k, v in d.items()})
        ys.append(y)
        ss.append(st)
    return np.stack(ys), np.stack(ss)


# variant 1 token kernel, 2 row-per-lane kernel (TMA-staged states), 3 / 4 sequence kernel with a head over two CTAs / in one CTA
@pytest.mark.parametrize("variant,nseg,T,H,gate", [
    (1, 1, 1, 8, False), (1, 5, 1, 40, True), (1, 3, 7, 8, True),
    (2, 1, 1, 8, True), (2, 37, 1, 40, True), (2, 100, 1, 8, False), (2, 3, 5, 8, True),
    (3, 1, 1, 8, True), (3, 1, 33, 8, False), (3, 2, 200, 8, True), (3, 1, 64, 40, True),
    (4, 1, 1, 8, True), (4, 6, 50, 8, True), (4, 2, 129, 40, False),
    (0, 1, 1, 40, True), (0, 1, 96, 40, True), (0, 30, 1, 40, True),
])
def test_wkv7_kernels_match_cpu_step(variant, nseg, T, H, gate):
    d = _wkv_case(nseg, T, H, seed=100 * variant + nseg + T, gate=gate)
    y_want, s_want = _wkv_oracle(d)
    y, s = rsv.op_wkv7(variant=variant, **d)
    # same fp32 operations in a different summation order (lanes split the 64-long dot products): a few ulps per token, relative to
    # the vector's scale; the reference's own kernel tests allow 1e-4 / 1e-3 (src/backend_cuda.rs:8549-8669)
    assert np.abs(s - s_want).max() <= 2e-5 * max(1.0, float(np.abs(s_want).max()))
    assert np.abs(y - y_want).max() <= 1e-4 * max(1.0, float(np.abs(y_want).max()))


def test_wkv7_kernels_agree_with_each_other_and_reject_bad_arguments():
    d = _wkv_case(4, 1, 8, seed=9, gate=True)
    outs = [rsv.op_wkv7(variant=v, **d) for v in (1, 2, 3, 4)]
    for y, s in outs[1:]:
        assert np.abs(y - outs[0][0]).max() <= 1e-4 and np.abs(s - outs[0][1]).max() <= 2e-5
    with pytest.raises(rsv.RsvError, match="variant"):
        rsv.op_wkv7(variant=9, **d)
    bad = dict(d)
    bad.pop("vfirst")
    with pytest.raises(rsv.RsvError, match="come together"):
        rsv.op_wkv7(**bad)


# ---- the offline int8 quantiser (tools/quantize_any4.py:241-300) ---------------------------------------------------------------
def _quantize_numpy(w, group=128):
    """quantize_int8_matrix restated with numpy, fp32 throughout like the tool."""
    m, k = w.shape
    wr = w.reshape(m, k // group, group)
    wmin, wmax = wr.min(axis=2), wr.max(axis=2)
    span = wmax - wmin
    flat = span == 0
    scale = (np.where(flat, np.float32(1.0), span) / np.float32(255.0)).astype(np.float32)
    q = np.clip(np.round((wr - wmin[..., None]) / scale[..., None]), 0, 255).astype(np.uint8).reshape(m, k)
    scale[flat] = 0.0
    s16 = scale.astype(np.float16).view(np.uint16).astype(np.uint32)
    z16 = wmin.astype(np.float16).view(np.uint16).astype(np.uint32)
    return q, ((z16 << 16) | s16).astype(np.uint32)


def test_quantize_int8_bit_exact_and_meets_the_precision_target():
    rng = np.random.default_rng(42)
    w = (0.02 * rng.standard_normal((32, 2560))).astype(np.float32)  # the shape of the reference's precision test (src/model.rs:878-918)
    w[3, 128:256] = 0.125                                            # a constant group
    w[5, :128] = np.linspace(-1, 1, 128, dtype=np.float32)           # exact ties of the rounding
    idx, sz = rsv.quantize_int8(w)
    qi, qs = _quantize_numpy(w)
    assert np.array_equal(idx, qi) and np.array_equal(sz, qs)
    assert np.all(idx[3, 128:256] == 0) and (sz[3, 1] & 0xFFFF) == 0 and (sz[3, 1] >> 16) == f16bits(0.125)
    back = rsv.op_dequant_int8(idx, sz)
    assert np.array_equal(back, orc.dequant_int8(idx, sz))
    assert np.all(back[3, 128:256] == 0.125)
    cos = float((w * back).sum() / (np.linalg.norm(w) * np.linalg.norm(back)))
    rel = float(np.linalg.norm(back - w) / np.linalg.norm(w))
    assert cos >= 0.999 and rel <= 0.02  # the reference's thresholds
    with pytest.raises(rsv.RsvError, match="multiple of 128"):
        rsv.quantize_int8(np.zeros((2, 100), dtype=np.float32))


def test_quantized_matrix_runs_through_the_linear_kernel():
    rng = np.random.default_rng(4)
    w = (0.02 * rng.standard_normal((256, 512))).astype(np.float32)
    x = rng.standard_normal((3, 512)).astype(np.float32)
    idx, sz = rsv.quantize_int8(w)
    want = x @ orc.dequant_int8(idx, sz).T
    y = rsv.op_linear(x, idx, sz, path=0)
    assert np.abs(y - want).max() <= 1e-4 * max(1.0, float(np.abs(want).max()))
    # per-group scales run on the weight-streaming kernel only: the tensor-core kernel takes one (scale, zero) per row and says so
    with pytest.raises(rsv.RsvError, match="one scale/zero per row"):
        rsv.op_linear(x, idx, sz, path=1)
