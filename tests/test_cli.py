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
    r = run_cli(base + ["--inference-server-port", "99999"])
    assert r.returncode == 2 and "--inference-server-port" in r.stderr
    # nothing to load at these paths (and no device on a CPU box): an error, not a crash
    r = run_cli(base + ["--inference-server", "--inference-server-port", "8080"])
    assert r.returncode == 1 and r.stderr.startswith("Error: ")
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
    # interactive mode (src/rllama_main.rs:824-838, :886-893): the system prompt, then a line from stdin wrapped in
    # prefix / postfix and fed token by token, generation until the sequence is full; a second read at end of input
    # yields an empty line
    iargs = [x for x in args if x not in ("--prompt", prompt)] + ["--start-interactive", "--interactive-system-prompt", "kalo miren",
                                                                  "--interactive-prompt-prefix", " ", "--interactive-prompt-postfix", " vu",
                                                                  "--interactive-stop", "zéñu"]
    r = run_cli(iargs, stdin="ren tas\n")
    assert r.returncode == 0, r.stderr
    assert r.stdout.startswith("kalo miren") and " ren tas vu" in r.stdout
    sys_toks = tk.tokenize_to_ids("kalo miren")
    user_toks = tk.tokenize_to_ids(" ren tas vu")[1:]
    assert len(sys_toks) + len(user_toks) < max_seq
    r2 = run_cli(iargs, {"CLICOLOR_FORCE": "1"}, stdin="ren tas\n")
    out2 = ANSI.sub("", r2.stdout)
    assert 'Interactive mode stop token sequences: ["zéñu"]' in out2 and "System prompt:\n  kalo miren" in out2
    assert "Interactive prompt prefix:  \nInteractive prompt postfix:  vu" in out2
    r = run_cli(iargs + ["--prompt", "x"], stdin="")
    assert r.returncode == 1 and "Cannot start interactive mode with a prompt." in r.stderr


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _post(port, path, body, method="POST"):
    import http.client
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
    c.request(method, path, body=body, headers={"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode("utf-8")
    c.close()
    return r.status, data


def _start_server(args, port):
    import time
    import socket
    env = dict(os.environ)
    proc = subprocess.Popen([CLI] + args + ["--inference-server", "--inference-server-port", str(port)], env=env,
                            stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    deadline = time.time() + 120
    while time.time() < deadline:
        if proc.poll() is not None:
            raise AssertionError("server exited: " + proc.stderr.read())
        try:
            with socket.create_connection(("127.0.0.1", port), timeout=1):
                return proc
        except OSError:
            time.sleep(0.2)
    proc.kill()
    raise AssertionError("server did not start listening")


@pytest.mark.gpu
def test_inference_server_streams_json_lines(tmp_path, cuda_ctx):
    """POST <api path>: chunked JSON lines, the reference's defaults, checks and status codes
    (src/rllama_main.rs:388-712), greedy tokens equal to the Python chain's."""
    import json
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
    prompt = "kalo miren tas"
    max_seq = 32
    tk = Tokenizer.load(tok_path)
    p = ModelParams.from_json(os.path.join(str(ckpt), "params.json"))
    model = Transformer.from_unpickled(p.dim, p.n_layers, p.n_heads, max_seq, p.norm_eps, DataSettings(cl=cuda_ctx).force_f16(),
                                       DataSource.from_llama_source(ckpt))
    toks = tk.tokenize_to_ids(prompt)
    n_prompt = len(toks)
    caches = model.make_caches()
    want, prev, first_logits = [], 0, None
    for _ in range(6):
        logits = model.forward(toks[prev:], prev, caches)
        if first_logits is None:
            first_logits = logits.copy()
        prev = len(toks)
        toks.append(int(np.argmax(logits)))
        want.append(tk.id_to_str(toks[-1]))

    args = ["--model-path", str(ckpt), "--tokenizer-path", str(tok_path), "--param-path", os.path.join(str(ckpt), "params.json"),
            "--max-seq-len", str(max_seq), "--f16", "--inference-server-prompt-cache-size", "4"]
    port = _free_port()
    proc = _start_server(args, port)
    try:
        path = "/rllama/v1/inference"
        status, body = _post(port, path, json.dumps({"prompt": prompt, "top_k": 1, "max_new_tokens": 6}))
        assert status == 200
        lines = [json.loads(l) for l in body.splitlines()]
        assert [list(l.keys())[0] for l in lines] == want
        assert all(list(l.values())[0] == {"p": 1.0} or list(l.values())[0] == {"p": 1.0, "is_end_token": True} for l in lines)
        # the same request again (served from the cache repository, which holds 4 sequences at most) and with a trailing slash
        status, body2 = _post(port, path + "/", json.dumps({"prompt": prompt, "top_k": 1, "max_new_tokens": 6, "ignored": [1, {"a": None}]}))
        assert status == 200 and body2 == body
        # defaults: 20 new tokens, bounded by the sequence length
        status, body3 = _post(port, path, json.dumps({"prompt": prompt}))
        assert status == 200 and 1 <= len(body3.splitlines()) <= 20
        status, body4 = _post(port, path, json.dumps({"prompt": prompt, "top_k": 1, "max_seq_len": n_prompt + 2, "max_new_tokens": 10}))
        assert status == 200 and body4.splitlines() == body.splitlines()[:2]
        status, body5 = _post(port, path, json.dumps({"prompt": prompt, "top_k": 1, "max_seq_len": 10 ** 6, "max_new_tokens": 1000}))
        assert status == 200 and len(body5.splitlines()) == max_seq - n_prompt
        # every piece with its logit
        status, body6 = _post(port, path, json.dumps({"prompt": prompt, "no_token_sampling": True, "max_new_tokens": 1}))
        assert status == 200
        allp = json.loads(body6.splitlines()[0])
        assert len(allp) == 400 and list(allp.keys()) == sorted(allp.keys(), key=lambda s: s.encode("utf-8"))
        for i in (0, 1, 2, 13, 57, 399):
            assert abs(allp[tk.id_to_str(i)]["p"] - float(first_logits[i])) <= 1e-6 * max(1.0, abs(float(first_logits[i])))
        assert allp["</s>"].get("is_end_token") is True and "is_end_token" not in allp["<s>"]
        # several requests at once: each has its own caches, the device work is serialised inside the library
        import threading
        results = [None] * 4
        def post(i):
            results[i] = _post(port, path, json.dumps({"prompt": prompt, "top_k": 1, "max_new_tokens": 6}))
        threads = [threading.Thread(target=post, args=(i,)) for i in range(4)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert all(r == (200, body) for r in results)
        # the reference's refusals
        for bad, text in (("{not json", "Invalid JSON."), (json.dumps({"top_k": 3}), "Invalid JSON."), (json.dumps({"prompt": 5}), "Invalid JSON."),
                          (json.dumps({"prompt": "x", "top_k": -1}), "Invalid JSON."), (json.dumps({"prompt": "x", "top_k": 1.5}), "Invalid JSON."),
                          (json.dumps({"prompt": "x", "top_k": 0}), "Top-k must be greater than 0."),
                          ('{"prompt": "x", "prompt": "y"}', "Invalid JSON.")):
            status, msg = _post(port, path, bad)
            assert (status, msg) == (400, text), bad
        assert _post(port, "/elsewhere", "{}")[0] == 404
        assert _post(port, path, None, method="GET")[0] == 404
        assert proc.poll() is None
    finally:
        proc.kill()
        proc.wait()
    # --inference-server-exit-after-one-query: one answer, then the process ends with status 0
    port = _free_port()
    proc = _start_server(args + ["--inference-server-exit-after-one-query", "--inference-server-api-path", "/v1"], port)
    try:
        status, body7 = _post(port, "/v1", json.dumps({"prompt": prompt, "top_k": 1, "max_new_tokens": 6}))
        assert status == 200 and body7 == body
        assert proc.wait(timeout=60) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
            proc.wait()


SERVER_UNIT = r'''
#include <cstdio>
#include "inference_server.hpp"
int main() {
    using namespace server;
    const float vals[] = {1.0f, 0.5f, 0.1f, 1e-7f, 1.5e-7f, 123456.0f, 3.0e20f, 0.00001f, 0.000012f, -2.5f, 16777216.0f, 0.0f, 0.33333334f};
    for (float v : vals) std::printf("%s\n", json_f32(v).c_str());
    std::printf("%s\n", json_f32(0.0f / 0.0f).c_str());
    std::printf("%s\n", json_string("a\"b\\c\n\t\x01\xc3\xa9").c_str());
    const char* bodies[] = {
        "{\"prompt\":\"a\\u00e9\\n\\ud83d\\ude00\",\"top_k\":3,\"temperature\":0.5,\"x\":{\"y\":[1,2,{\"z\":null}]}}",
        " { \"prompt\" : \"p\" , \"max_seq_len\" : 7, \"max_new_tokens\":0, \"no_token_sampling\":true, \"stop_at_end_token\":false, \"top_p\":1e-1, \"repetition_penalty\": 2 } ",
        "{\"prompt\":\"p\",\"temperature\":null,\"top_k\":null}",
        "{\"top_k\":3}", "{\"prompt\":5}", "{\"prompt\":\"x\",\"top_k\":-1}", "{\"prompt\":\"x\",\"top_k\":1.5}", "{\"prompt\":\"x\",\"top_k\":\"3\"}",
        "{\"prompt\":\"x\",\"no_token_sampling\":1}", "{\"prompt\":\"x\",\"prompt\":\"y\"}", "{\"prompt\":\"x\"} trailing", "[1]", "{\"prompt\":\"x\",}",
        "{\"prompt\":\"bad \\q escape\"}", "{\"prompt\":\"\\ud83d\"}", ""};
    for (const char* b : bodies) {
        InferenceRequest r;
        const bool ok = parse_request(b, &r);
        if (!ok) { std::printf("invalid\n"); continue; }
        std::printf("ok prompt=%s t=%g k=%llu p=%g rp=%g msl=%d:%llu mnt=%llu nts=%d stop=%d\n", json_string(r.prompt).c_str(), r.temperature,
                    (unsigned long long)r.top_k, r.top_p, r.repetition_penalty, (int)r.has_max_seq_len, (unsigned long long)r.max_seq_len,
                    (unsigned long long)r.max_new_tokens, (int)r.no_token_sampling, (int)r.stop_at_end_token);
    }
    return 0;
}
'''


def test_server_request_parsing_and_json_output(tmp_path):
    """The server's JSON reader and serde_json-style writers, compiled on their own (no device)."""
    import shutil
    from rllama_b200.build import HERE
    cxx = shutil.which(os.environ.get("CXX", "g++"))
    if cxx is None:
        pytest.skip("no C++ compiler")
    src = tmp_path / "unit.cpp"
    src.write_text(SERVER_UNIT)
    exe = tmp_path / "unit"
    r = subprocess.run([cxx, "-std=c++17", "-Wall", "-I" + os.path.join(HERE, "cli"), str(src), "-o", str(exe), "-L" + HERE, "-lrllama_b200",
                        "-Wl,-rpath," + HERE, "-Wl,-rpath,/usr/local/cuda/lib64", "-pthread"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = subprocess.run([str(exe)], capture_output=True, text=True).stdout.splitlines()
    assert out[:14] == ["1.0", "0.5", "0.1", "1e-7", "1.5e-7", "123456.0", "3e20", "0.00001", "0.000012", "-2.5", "16777216.0", "0.0",
                        "0.33333334", "null"]
    assert out[14] == '"a\\"b\\\\c\\n\\t\\u0001é"'
    assert out[15] == 'ok prompt="aé\\n😀" t=0.5 k=3 p=1 rp=1 msl=0:0 mnt=20 nts=0 stop=1'
    assert out[16] == 'ok prompt="p" t=1 k=20 p=0.1 rp=2 msl=1:7 mnt=0 nts=1 stop=0'
    assert out[17] == 'ok prompt="p" t=1 k=20 p=1 rp=1 msl=0:0 mnt=20 nts=0 stop=1'
    assert out[18:] == ["invalid"] * 13
