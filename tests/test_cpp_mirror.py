"""The header-only C++ mirror (``include/rllama_b200.hpp``) compiles against the C header and its
host-side classes (Tokenizer, TokenSampler, ModelParams, DataSource) work without a GPU."""
import os
import shutil
import subprocess

import pytest

from rllama_b200.build import HERE, LIB

ROOT = os.path.dirname(HERE)

PROGRAM = r'''
#include <cstdio>
#include "rllama_b200.hpp"
int main(int argc, char** argv) {
    using namespace rllama;
    try {
        Tokenizer tk = Tokenizer::load(argv[1]);
        std::vector<int32_t> ids = tk.tokenize_to_ids("kalo miren");
        std::printf("ids");
        for (int32_t t : ids) std::printf(" %d", t);
        std::printf("\n%s %d\n", tk.id_to_str(1).c_str(), tk.str_to_id("no such piece"));
        TokenSampler s;
        std::printf("%.1f %.1f %d %.1f\n", s.get_temperature(), s.get_top_p(), s.get_top_k(), s.get_repetition_penalty());
        s.temperature(1.0f).top_k(1).repetition_penalty(1.0f).seed(3);
        std::vector<float> logits = {0.5f, 3.0f, -1.0f, 2.5f};
        auto r = s.sample(logits, {1, 2});
        std::printf("%d %.3f\n", r.first, r.second);
        ModelParams p = ModelParams::from_json(argv[2]);
        std::printf("%d %d %d %ld\n", p.dim, p.n_heads, p.n_layers, p.vocab_size);
        DataSource ds = DataSource::from_inferred_source(argv[3]);
        std::printf("antitranspose %d\n", ds.need_to_do_antitranspose() ? 1 : 0);
        try {
            Cuda cuda;  // on a CPU box this is the "no device" error, on a GPU box it succeeds
            DataSettings settings;
            settings.cl = &cuda;
            settings = settings.force_f16();
            std::printf("device ok\n");
        } catch (const Error& e) {
            std::printf("no device: status %d\n", e.status);
        }
        try {
            Tokenizer::load("/nonexistent/tokenizer.model");
            return 2;
        } catch (const Error& e) {
            std::printf("error %d\n", e.status);
        }
    } catch (const Error& e) {
        std::fprintf(stderr, "unexpected: %s\n", e.what());
        return 1;
    }
    return 0;
}
'''


def test_cpp_mirror_compiles_and_runs(tmp_path):
    pytest.importorskip("torch")
    cxx = shutil.which(os.environ.get("CXX", "g++"))
    if cxx is None:
        pytest.skip("no C++ compiler")
    from checkpoint import write_llama_checkpoint
    from helpers import cfg_variant
    from rllama_b200 import Tokenizer
    from test_tokenizer_sampler import train_model

    model, _ = train_model()
    tok = tmp_path / "tokenizer.model"
    tok.write_bytes(model)
    cfg = cfg_variant("tiny", dim=256, n_heads=4, n_layers=1, ffn=352, vocab=304, max_seq_len=16)
    write_llama_checkpoint(str(tmp_path / "ckpt"), cfg)
    src = tmp_path / "mirror.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "mirror"
    cuda_lib = "/usr/local/cuda/lib64"
    r = subprocess.run([cxx, "-std=c++17", "-Wall", "-Werror", "-I" + os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                        "-L" + HERE, "-lrllama_b200", "-Wl,-rpath," + HERE, "-Wl,-rpath," + cuda_lib], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe), str(tok), str(tmp_path / "ckpt" / "params.json"), str(tmp_path / "ckpt")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr + r.stdout
    lines = r.stdout.splitlines()
    want_ids = Tokenizer.load(tok).tokenize_to_ids("kalo miren")
    assert lines[0] == "ids " + " ".join(str(t) for t in want_ids)
    assert lines[1] == "<s> -1"
    assert lines[2] == "0.2 1.0 1 0.8"
    assert lines[3] == "1 1.000"
    assert lines[4] == "256 4 1 -1"
    assert lines[5] == "antitranspose 0"
    assert lines[6] in ("device ok", "no device: status 3")
    assert lines[7].startswith("error ")
