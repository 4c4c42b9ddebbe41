"""The command-line program ``rllama_b200/bin/rllama-b200`` (``rllama_b200/cli/rllama_cli.cpp``): flag
handling without a GPU; on a GPU the whole chain tokenizer -> checkpoint loader -> prefill -> decode
loop -> sampler -> text against the same chain driven from Python."""
import os
import re
import subprocess

import numpy as np
import pytest

from rllama_b200.build import CLI

ANSI = re.compile(r"\x1b\[[0-9;]*m")


def run_cli(args, env_extra=None, stdin=None):
    env = dict(os.environ)
    for k in ("CLICOLOR", "CLICOLOR_FORCE", "NO_COLOR"):
        env.pop(k, None)
    env.update(env_extra or {})
    return subprocess.run([CLI] + args, capture_output=True, text=True, env=env, input=stdin, timeout=300)


def test_cli_flag_errors_need_no_device():
    assert os.path.exists(CLI), "the command-line program is built by rllama_b200.build"
    r = run_cli([])
    assert r.returncode == 2 and "--model-path <MODEL_PATH>" in r.stderr and "--param-path <PARAM_PATH>" in r.stderr
    r = run_cli(["--model-path", "m", "--tokenizer-path", "t"])
    assert r.returncode == 2 and "--param-path <PARAM_PATH>" in r.stderr and "--model-path <MODEL_PATH>" not in r.stderr.split("Usage")[0]
    base = ["--model-path", "m", "--tokenizer-path=t", "--param-path", "p"]
    r = run_cli(base + ["--no-such-flag"])
    assert r.returncode == 2 and "unexpected argument '--no-such-flag'" in r.stderr
    r = run_cli(base + ["--top-k", "many"])
    assert r.returncode == 2 and "invalid value 'many' for '--top-k'" in r.stderr
    r = run_cli(base + ["--temperature"])
    assert r.returncode == 2 and "a value is required" in r.stderr
    # a build of the reference without its server feature refuses the flag the same way
    r = run_cli(base + ["--inference-server", "--inference-server-port", "8080"])
    assert r.returncode == 1 and "Inference server is not enabled in this build." in r.stderr
    assert run_cli(["--help"]).returncode == 0


@pytest.mark.gpu
def test_cli_generates_the_same_text_as_the_python_chain(tmp_path, cuda_ctx):
    torch = pytest.importorskip("torch")
    from checkpoint import write_llama_checkpoint
    from helpers import cfg_variant
    from rllama_b200 import DataSettings, DataSource, ModelParams, Tokenizer, Transformer
    from test_tokenizer_sampler import train_model

    model_bytes, _ = train_model(byte_fallback=True, vocab=400)
    tok_path = tmp_path / "tokenizer.model"
    tok_path.write_bytes(model_bytes)
    cfg = cfg_variant("tiny", dim=256, n_heads=4, n_layers=2, ffn=352, vocab=400, max_seq_len=40)
    ckpt = tmp_path / "ckpt"
    os.makedirs(ckpt)
    write_llama_checkpoint(str(ckpt), cfg)
    prompt = "kalo miren tas\nvu shi"
    max_seq = 24

    # the same chain from Python: tokenizer, loader, forward, arg-max (top_k 1), text
    tk = Tokenizer.load(tok_path)
    p = ModelParams.from_json(os.path.join(str(ckpt), "params.json"))
    model = Transformer.from_unpickled(p.dim, p.n_layers, p.n_heads, max_seq, p.norm_eps, DataSettings(cl=cuda_ctx).force_f16(),
                                       DataSource.from_llama_source(ckpt))
    toks = tk.tokenize_to_ids(prompt)
    caches = model.make_caches()
    text, prev, stop = "", 0, False
    while len(toks) < max_seq and not stop:
        logits = model.forward(toks[prev:], prev, caches)
        nxt = int(np.argmax(logits))
        toks.append(nxt)
        piece = tk.id_to_str(nxt)
        if nxt != 1:
            text += "\n" if piece == "<0x0A>" else piece.replace("▁", " ")
        stop = piece == "</s>"
        prev = len(toks) - 1

    args = ["--model-path", str(ckpt), "--tokenizer-path", str(tok_path), "--param-path", os.path.join(str(ckpt), "params.json"),
            "--prompt", prompt, "--max-seq-len", str(max_seq), "--top-k", "1", "--f16"]
    # piped output is quiet, as with the reference: prompt + generated text + newline and nothing else
    r = run_cli(args)
    assert r.returncode == 0, r.stderr
    assert r.stdout == prompt + text + "\n"
    # colour forced: banner, parameters, coloured text and the timing lines
    r = run_cli(args, {"CLICOLOR_FORCE": "1"})
    assert r.returncode == 0, r.stderr
    out = ANSI.sub("", r.stdout)
    for line in (" dim: 256", " n_heads: 4", " n_layers: 2", " norm_eps: 0.000001", " vocab_size: -1", "Max sequence length: 24",
                 "Temperature: 1", "Top P: 1", "Top K: 1", "Repetition penalty: 1", "All is loaded. Starting inference.",
                 "Using prompt: " + prompt.split("\n")[0]):
        assert line in out, line
    assert (prompt + text + "\n") in out
    assert "\x1b[38;2;128;128;255m" in r.stdout  # the prompt's colour
    m1 = re.search(r"Time taken to generate first token: (\d+)ms\n", out)
    m2 = re.search(r"Time taken per token \(excluding first token\): (\d+)ms\n", out)
    assert m1 and m2 and out.rstrip().endswith(m2.group(0).rstrip())
    # sampling with a seed repeats; without top-k 1 the text may differ from the arg-max text but has the same length rule
    sargs = [a for a in args if a not in ("--top-k", "1")] + ["--temperature", "0.8", "--seed", "7"]
    a, b = run_cli(sargs), run_cli(sargs)
    assert a.returncode == 0 and a.stdout == b.stdout and a.stdout.startswith(prompt)
    # no prompt at all
    r = run_cli([x for x in args if x not in ("--prompt", prompt)])
    assert r.returncode == 1 and "Please provide either a prompt or a prompt file." in r.stderr
    # prompt from a file; a missing checkpoint
    pf = tmp_path / "prompt.txt"
    pf.write_text(prompt)
    r = run_cli([x for x in args if x not in ("--prompt", prompt)] + ["--prompt-file", str(pf)])
    assert r.returncode == 0 and r.stdout == prompt + text + "\n"
    r = run_cli(["--model-path", str(tmp_path / "nowhere")] + args[2:])
    assert r.returncode == 1 and r.stderr.startswith("Error: ")
