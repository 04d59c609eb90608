"""Regenerates tests/golden/*.npz.

The Rust reference cannot be built in this image, so these vectors come from the C++ CPU oracle
(oracle/rwkv7_cpu.cpp, cross-checked against oracle/rwkv7_numpy.py) on the seeded synthetic tiny model of
benchmark config 1.  They pin (a) the synthetic generator + oracle against drift and (b) the GPU path.
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys
import tempfile
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [ROOT, os.path.join(ROOT, "oracle")]
import orc  # noqa: E402
import rwkv_rsv_b200 as rsv  # noqa: E402

N_PROMPT, N_DECODE = 128, 64


def main():
    tokens = np.random.default_rng(0).integers(0, 4096, size=N_PROMPT).astype(np.uint32)
    with tempfile.TemporaryDirectory() as d:
        for name, q in (("fp16", 0), ("int8", 1), ("int8g", 2)):
            path = rsv.write_synthetic(os.path.join(d, f"{name}.st"), "tiny", seed=0, quant=q)
            crc = zlib.crc32(open(path, "rb").read())
            m = orc.OracleModel(path)
            logits = m.forward(tokens)
            state = m.state_back()
            # free-running arg-max stream, self-loop convention: the seed (= last prompt token) is fed again
            stream, tok = [], int(tokens[-1])
            gaps = []
            for _ in range(N_DECODE):
                lg = m.forward([tok])
                tok = orc.argmax(lg)
                top2 = np.partition(lg, -2)[-2:]
                gaps.append(float(top2[1] - top2[0]))
                stream.append(tok)
            np.savez_compressed(os.path.join(ROOT, "tests", "golden", f"tiny_{name}.npz"), tokens=tokens, file_crc32=np.uint32(crc),
                                logits=logits, state_crc32=np.uint32(zlib.crc32(state.tobytes())), state_head=state[:64],
                                stream=np.asarray(stream, dtype=np.uint32), top2_gap=np.asarray(gaps, dtype=np.float32))
            print(name, "crc", crc, "argmax", int(logits.argmax()), "min top-2 gap", min(gaps))


if __name__ == "__main__":
    main()
