"""RWKV "world" tokenizer: greedy longest-match over a byte vocabulary (src/tokenizer.rs).

The vocabulary is the JSON map of the reference, `{token id: string | [byte, ...]}` (e.g. rwkv_vocab_v20230424.json; the file is
not shipped here).  Host-side text handling only: nothing of this runs on the GPU, it turns a prompt into the `u32` token list the
forward step takes and the generated tokens back into bytes (examples/generate.rs:33-57, 102-110).
"""
import json


class TokenizerError(ValueError):
    """TokenizerError (src/tokenizer.rs:9-17)."""


class Tokenizer:
    def __init__(self, vocab_json):
        """`vocab_json`: the text of the vocabulary file (Tokenizer::new, src/tokenizer.rs:34-87)."""
        try:
            raw = json.loads(vocab_json)
            items = sorted((int(k), v) for k, v in raw.items())
        except (ValueError, AttributeError, TypeError) as e:
            raise TokenizerError(f"failed to parse vocabulary: {e}") from None
        self._to_id = {}
        self._to_bytes = [b""] * ((items[-1][0] + 1) if items else 1)
        # candidate token lengths per pair of leading bytes, longest first; every pair may also match a one-byte token
        lengths = {}
        for tid, pat in items:
            if tid < 0 or tid > 0xFFFFFFFF:
                raise TokenizerError(f"failed to parse vocabulary: token id {tid} does not fit u32")
            try:
                b = pat.encode("utf-8") if isinstance(pat, str) else bytes(pat)
            except (ValueError, TypeError) as e:
                raise TokenizerError(f"failed to parse vocabulary: token {tid}: {e}") from None
            if len(b) >= 2:
                lengths.setdefault(b[:2], {1}).add(len(b))
            self._to_id[b] = tid
            self._to_bytes[tid] = b
        self._lengths = {k: sorted(v, reverse=True) for k, v in lengths.items()}

    def __len__(self):
        return len(self._to_bytes)

    def encode(self, data):
        """bytes (or str, taken as UTF-8) -> token ids; at every position the longest token that matches (encode_into,
        src/tokenizer.rs:101-131).  Raises when no token matches."""
        if isinstance(data, str):
            data = data.encode("utf-8")
        data = bytes(data)
        out, pos, n = [], 0, len(data)
        one = (1,)
        while pos < n:
            cand = self._lengths.get(data[pos:pos + 2], one) if n - pos >= 2 else one
            for ln in cand:
                if ln > n - pos:
                    continue
                tid = self._to_id.get(data[pos:pos + ln])
                if tid is not None:
                    out.append(tid)
                    pos += ln
                    break
            else:
                raise TokenizerError("no matching token found")
        return out

    def decode(self, tokens):
        """token ids -> bytes (decode_into, src/tokenizer.rs:133-142); an id past the vocabulary raises."""
        parts = []
        for t in tokens:
            t = int(t)
            if t < 0 or t >= len(self._to_bytes):
                raise TokenizerError(f"out of range token: {t}")
            parts.append(self._to_bytes[t])
        return b"".join(parts)
