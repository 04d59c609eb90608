"""The greedy longest-match tokenizer (src/tokenizer.rs) against a brute-force restatement on a seeded synthetic vocabulary
(the reference has no tokenizer tests and its vocabulary file is not in the repository)."""
import json

import numpy as np
import pytest

from rwkv_rsv_b200.tokenizer import Tokenizer, TokenizerError


def _vocab(seed=0, extra=400):
    rng = np.random.default_rng(seed)
    toks = {i + 1: [i] for i in range(256)}  # every single byte, as byte arrays (ids start at 1: id 0 stays empty)
    seen = {bytes([i]) for i in range(256)}
    tid = 257
    alphabet = b"abcde \n\xe4\xbd\xa0\xe5\xa5\xbd"
    while len(toks) < 256 + extra:
        b = bytes(rng.choice(list(alphabet), size=int(rng.integers(2, 9))).tolist())
        if b in seen:
            continue
        seen.add(b)
        try:
            toks[tid] = b.decode("utf-8")  # stored as a string where it is valid UTF-8 ...
        except UnicodeDecodeError:
            toks[tid] = list(b)            # ... and as a byte array otherwise
        tid += 1
    return toks


def _brute_force(table, data):
    out, pos = [], 0
    by_len = sorted(table.items(), key=lambda kv: -len(kv[0]))
    while pos < len(data):
        for b, tid in by_len:
            if data.startswith(b, pos):
                out.append(tid)
                pos += len(b)
                break
        else:
            raise AssertionError("no match")
    return out


def test_longest_match_and_round_trip():
    v = _vocab()
    tk = Tokenizer(json.dumps({str(k): x for k, x in v.items()}))
    table = {(x.encode() if isinstance(x, str) else bytes(x)): k for k, x in v.items()}
    rng = np.random.default_rng(1)
    alphabet = list(b"abcde \n\xe4\xbd\xa0\xe5\xa5\xbdXYZ\x00\xff")
    for n in (0, 1, 2, 3, 17, 400, 5000):
        data = bytes(rng.choice(alphabet, size=n).tolist())
        ids = tk.encode(data)
        assert ids == _brute_force(table, data)
        assert tk.decode(ids) == data
    assert tk.encode("abc 你好") == tk.encode("abc 你好".encode("utf-8"))
    assert len(tk) == max(v) + 1


def test_prefers_the_longest_token_even_when_a_shorter_one_matches_first():
    tk = Tokenizer(json.dumps({"1": "a", "2": "b", "3": "ab", "4": "abab", "5": "c", "6": "aba"}))
    assert tk.encode("ababc") == [4, 5]
    assert tk.encode("abac") == [6, 5]
    assert tk.encode("abb") == [3, 2]
    assert tk.encode("a") == [1]  # a single trailing byte only ever matches a one-byte token


def test_errors():
    tk = Tokenizer(json.dumps({"1": "a", "2": "ab"}))
    with pytest.raises(TokenizerError, match="no matching token"):
        tk.encode("abz")
    with pytest.raises(TokenizerError, match="out of range token: 3"):
        tk.decode([1, 3])
    assert tk.decode([0]) == b""  # an id inside the table that the file does not define decodes to nothing
    for bad in ("not json", "[1, 2]", json.dumps({"x": "a"}), json.dumps({"1": [300]})):
        with pytest.raises(TokenizerError, match="failed to parse vocabulary"):
            Tokenizer(bad)


def test_text_driver_refuses_a_prompt_without_a_vocabulary_before_touching_the_gpu():
    # examples/generate.rs:49 "PROMPT requires VOCAB_JSON": the check comes before the model is loaded, so it runs anywhere
    from rwkv_rsv_b200 import generate as gen
    with pytest.raises(SystemExit):
        gen.main(["--model", "no_such_model.st", "--prompt", "hello"])
