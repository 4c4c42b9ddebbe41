"""Regenerates the golden vectors in this directory from the CPU oracle.

    python tests/golden/make_golden.py

The reference itself holds no golden logits or token transcripts and cannot be built
where these were made (no Rust toolchain), so the vectors pin the ORACLE (the C++
restatement of rllama's CPU forward), not the Rust binary: they catch drift of the oracle
and give the GPU tests a fixed target that does not depend on the host CPU.

Protocol (the benchmark configuration's own): seeded N(0, 0.02) f16-representable weights,
gains 1.0, a 16-token random prompt, prefill at position 0, then greedy decode steps.
Stored per case: the greedy token sequence, and full logits of the prefill and of two
decode steps.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402
from rllama_b200 import synthetic as S  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (config overrides, force_f16, decode steps, steps whose logits are stored)
    "tiny_f32": (dict(), False, 64, (0, 1, 64)),
    "tiny_f16": (dict(), True, 64, (0, 1, 64)),
}


def run_case(name):
    over, f16, steps, keep = CASES[name]
    cfg = dict(S.CONFIGS["tiny"])
    cfg.update(over)
    m = O.OracleTransformer(cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"], cfg["norm_eps"],
                            cfg["max_seq_len"], f16, nthreads=4)
    S.load_into(m, cfg)
    prompt = S.synth_tokens(cfg["prompt"], cfg["vocab"])
    caches = m.make_caches()
    logits = m.forward(prompt, 0, caches)
    out = {"prompt": prompt}
    tokens = []
    margins = []
    if 0 in keep:
        out["logits_step0"] = logits
    for i in range(1, steps + 1):
        top2 = np.partition(logits, -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
        tok = int(np.argmax(logits))
        tokens.append(tok)
        logits = m.forward([tok], cfg["prompt"] + i - 1, caches)
        if i in keep:
            out["logits_step%d" % i] = logits
    out["tokens"] = np.asarray(tokens, dtype=np.int32)
    out["top2_margin"] = np.asarray(margins, dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "golden_%s.npz" % name), **out)
    print(name, "tokens", tokens[:8], "... min top-2 margin %.3g" % min(margins))


if __name__ == "__main__":
    for case in CASES:
        run_case(case)
