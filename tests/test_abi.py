"""CPU tests of the boundary: the native library builds, loads, exports every declared symbol, and the
product path refuses to run without a GPU (no CPU fallback)."""
import os
import re

import numpy as np
import pytest

import rwkv_rsv_b200 as rsv
from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "rsv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rsv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = rsv.native()
    syms = declared_symbols()
    assert len(syms) >= 30
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/rsv_b200.h but not exported"
    assert sorted(rsv.ABI_SYMBOLS) == syms


def test_cpp_mirror_header_compiles_and_links(tmp_path):
    # include/rsv_bundle.hpp (the C++ mirror of ModelBuilder / Bundle / State) instantiates every wrapper against the C header,
    # links against the shared library, and a program using it fails loudly on a box without a GPU
    import shutil
    import subprocess
    if not shutil.which("g++"):
        pytest.skip("no g++")
    src = tmp_path / "use_bundle.cpp"
    src.write_text(r"""
#include <cstdio>
#include "rsv_bundle.hpp"
int main(int argc, char** argv) {
    try {
        rsv::Bundle b = rsv::ModelBuilder(argc > 1 ? argv[1] : "missing.st").build();
        std::vector<float> lg = b.infer_tokens({1, 2, 3});
        std::vector<uint32_t> out = b.infer_argmax_selfloop(3, 4);
        b.state.save("s.bin");
        b.state.restore("s.bin");
        b.state_load(b.state_back());
        rsv::SamplerParams sp;
        b.infer_sample_selfloop(3, 2, sp);
        std::printf("%zu %zu\n", lg.size(), out.size());
    } catch (const rsv::Error& e) {
        std::printf("rsv::Error: %s\n", e.what());
        return 3;
    }
    return 0;
}
""")
    exe = tmp_path / "use_bundle"
    libdir = os.path.dirname(rsv.LIB_CUDA)
    cmd = ["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe), "-L", libdir,
           "-l:" + os.path.basename(rsv.LIB_CUDA), "-Wl,-rpath," + libdir]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    import torch
    if not torch.cuda.is_available():
        run = subprocess.run([str(exe)], capture_output=True, text=True, cwd=tmp_path)
        assert run.returncode == 3 and "rsv::Error" in run.stdout, (run.returncode, run.stdout, run.stderr)


def test_header_cites_reference_for_each_entry_point():
    text = open(os.path.join(ROOT, "include", "rsv_b200.h")).read()
    assert text.count("src/gpu_model.rs") >= 20


def test_synthetic_generator_is_deterministic_and_seeded(model_dir):
    a = rsv.write_synthetic(os.path.join(model_dir, "a.st"), "tiny", seed=7, quant=1, n_layer=1, vocab=256)
    b = rsv.write_synthetic(os.path.join(model_dir, "b.st"), "tiny", seed=7, quant=1, n_layer=1, vocab=256)
    c = rsv.write_synthetic(os.path.join(model_dir, "c.st"), "tiny", seed=8, quant=1, n_layer=1, vocab=256)
    assert open(a, "rb").read() == open(b, "rb").read()
    assert open(a, "rb").read() != open(c, "rb").read()


def test_synthetic_int8_container(model_dir):
    from safetensors.numpy import load_file
    f = load_file(rsv.write_synthetic(os.path.join(model_dir, "f.st"), "tiny", seed=1, quant=0, n_layer=2))
    q = load_file(rsv.write_synthetic(os.path.join(model_dir, "q.st"), "tiny", seed=1, quant=1, n_layer=2))
    assert "head.weight" in q and "emb.weight" in q            # head and embedding stay fp16
    assert "blocks.1.att.key.weight" not in q                  # exactly one of the two forms per matrix
    w = f["blocks.1.ffn.value.weight"].astype(np.float32)
    idx, sz = q["blocks.1.ffn.value.weight.int8_idx"], q["blocks.1.ffn.value.weight.int8_sz"]
    assert idx.dtype == np.uint8 and idx.shape == w.shape and sz.shape == (w.shape[0], w.shape[1] // 128)
    scale = (sz & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32)
    zero = (sz >> 16).astype(np.uint16).view(np.float16).astype(np.float32)
    assert np.array_equal(zero, -128.0 * scale)                # symmetric form: zero = -128*scale exactly
    assert np.all(sz == sz[:, :1])                             # one scale per output row
    deq = np.repeat(scale, 128, 1) * idx.astype(np.float32) + np.repeat(zero, 128, 1)
    assert np.array_equal(deq, np.repeat(scale, 128, 1) * (idx.astype(np.float32) - 128.0))
    assert np.abs(deq - w).max() <= 0.5 * scale.max() * 1.001
    assert idx.min() >= 1                                      # q_s8 in [-127, 127]
    # shapes carry the hyper-parameters (src/model.rs:281-315)
    assert f["blocks.0.att.r_k"].shape == (8, 64) and f["blocks.0.att.w1"].shape == (512, 32) and f["blocks.0.att.v2"].shape == (16, 512)
    assert "blocks.0.att.v0" in f and "blocks.0.att.v1" in f   # loaded for layer 0 too (src/model.rs:594-602)


def test_no_cpu_fallback(tiny_paths):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(rsv.RsvError, match="no CUDA device"):
        rsv.ModelBuilder(tiny_paths["fp16"]).build()
    with pytest.raises(rsv.RsvError, match="no CUDA device"):
        rsv.op_argmax(np.zeros(8, dtype=np.float32))


def test_missing_file_and_bad_header_are_reported(tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("load errors other than 'no device' need a GPU")
    with pytest.raises(rsv.RsvError):
        rsv.ModelBuilder(str(tmp_path / "nope.st")).build()
