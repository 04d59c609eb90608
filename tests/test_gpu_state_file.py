"""State files and session migration: the wire format is the f32 array of State::back as raw bytes (the file the reference's
examples/state_persist.rs:38-67 writes and checks with max_diff == 0), so everything here is bit-exact."""
import os

import numpy as np
import pytest

import orc
import rwkv_rsv_b200 as rsv
from conftest import config1_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bundle(tiny_paths):
    return rsv.ModelBuilder(tiny_paths["int8"]).build()


def test_file_is_the_raw_state_and_round_trips(bundle, tmp_path):
    b = bundle
    b.reset()
    b.infer_tokens(config1_tokens()[:40])
    s0 = b.state_back()
    f = tmp_path / "state.bin"
    b.state.save(f)
    assert f.read_bytes() == s0.tobytes()  # no header: what std::fs::write(bytemuck::cast_slice(&state)) produces
    assert not os.path.exists(str(f) + ".part")
    first = list(b.infer_argmax_selfloop(7, 12))
    b.reset()
    assert not b.state_back().any()
    b.state.restore(f)
    assert np.array_equal(b.state_back(), s0)  # max_diff == 0
    assert list(b.infer_argmax_selfloop(7, 12)) == first


def test_file_of_the_wrong_size_is_refused_and_the_state_kept(bundle, tmp_path):
    b = bundle
    b.reset()
    b.infer_tokens([3, 1, 4, 1, 5])
    s0 = b.state_back()
    for n in (s0.size - 1, s0.size + 1, 0):
        f = tmp_path / f"bad{n}.bin"
        np.zeros(n, dtype=np.float32).tofile(f)
        with pytest.raises(rsv.RsvError, match="length mismatch"):
            b.state.restore(f)
    with pytest.raises(rsv.RsvError, match="cannot open"):
        b.state.restore(tmp_path / "missing.bin")
    with pytest.raises(rsv.RsvError, match="cannot create"):
        b.state.save(tmp_path / "no_such_dir" / "s.bin")
    assert np.array_equal(b.state_back(), s0)


def test_state_written_by_the_cpu_path_continues_on_the_gpu(bundle, tiny_paths, tmp_path):
    # the file crosses implementations: the oracle's state after a prompt, loaded here, continues with the oracle's tokens
    o = orc.OracleModel(tiny_paths["int8"])
    try:
        toks = config1_tokens()[:32]
        o.forward(toks)
        f = tmp_path / "cpu_state.bin"
        np.asarray(o.state_back(), dtype="<f4").tofile(f)
        want, tok = [], int(toks[-1])
        for _ in range(16):
            tok = int(orc.argmax(o.forward([tok])))
            want.append(tok)
    finally:
        o.close()
    bundle.reset()
    bundle.state.restore(f)
    assert list(bundle.infer_argmax_selfloop(int(toks[-1]), 16)) == want


def test_slot_files_and_batched_states(bundle, tmp_path):
    m = bundle.model
    st = m.create_batch_state(4)
    try:
        rng = np.random.default_rng(3)
        prompts = [rng.integers(0, m.info().num_vocab, size=k).astype(np.uint32) for k in (5, 17, 2, 9)]
        m.forward_seq_batch(st, prompts)
        whole = st.back()
        st.save(tmp_path / "all.bin")
        assert (tmp_path / "all.bin").read_bytes() == whole.tobytes()
        per = whole.size // 4
        st.slot_save(2, tmp_path / "slot2.bin")
        assert (tmp_path / "slot2.bin").read_bytes() == whole[2 * per:3 * per].tobytes()
        # a slot file is a batch-1 state file: the session continues in a Bundle
        bundle.reset()
        bundle.state.restore(tmp_path / "slot2.bin")
        assert np.array_equal(bundle.state_back(), st.slot_back(2))
        st.slot_restore(0, tmp_path / "slot2.bin")
        assert np.array_equal(st.slot_back(0), st.slot_back(2))
        assert np.array_equal(st.slot_back(1), whole[per:2 * per])  # the neighbours are untouched
        with pytest.raises(rsv.RsvError, match="length mismatch"):
            st.slot_restore(1, tmp_path / "all.bin")
        with pytest.raises(rsv.RsvError, match="slot >= batch"):
            st.slot_save(4, tmp_path / "x.bin")
    finally:
        st.close()


def _migrate_and_continue(path, dev_a, dev_b):
    """A session prefilled in slot 2 of a batch-4 state of one model handle moves to slot 0 of a batch-2 state of another
    handle and decodes on; the tokens equal those of the session that stayed."""
    a, b = rsv.Model(path, device=dev_a), rsv.Model(path, device=dev_b)
    sa, sb = a.create_batch_state(4), b.create_batch_state(2)
    try:
        rng = np.random.default_rng(11)
        prompts = [rng.integers(0, a.info().num_vocab, size=k).astype(np.uint32) for k in (4, 30, 12, 7)]
        seeds = a.forward_seq_batch(sa, prompts)
        sb.slot_copy_from(0, sa, 2)
        assert np.array_equal(sb.slot_back(0), sa.slot_back(2))  # bit for bit
        assert not sb.slot_back(1).any()
        stay = a.collect_sample_selfloop_batch(a.submit_sample_selfloop_batch(sa, seeds, 10, None))
        moved = b.collect_sample_selfloop_batch(b.submit_sample_selfloop_batch(sb, [seeds[2], 0], 10, None))
        assert list(moved[0]) == list(stay[2])
        with pytest.raises(rsv.RsvError, match="slot >= batch"):
            sb.slot_copy_from(2, sa, 0)
    finally:
        sa.close()
        sb.close()
        a.close()
        b.close()


def test_session_moves_between_two_model_handles(tiny_paths):
    _migrate_and_continue(tiny_paths["int8"], 0, 0)


def test_session_moves_between_two_gpus(tiny_paths):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _migrate_and_continue(tiny_paths["int8"], 0, 1)
