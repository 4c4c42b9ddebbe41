"""Shared builders for the parity tests: the same synthetic checkpoint goes into the CUDA
model (through the C ABI) and into the CPU oracle."""
import numpy as np

from rllama_b200 import synthetic as S


def cfg_variant(base="tiny", **over):
    cfg = dict(S.CONFIGS[base])
    cfg.update(over)
    return cfg


def build_pair(cfg, f16, cuda_ctx=None, oracle_threads=0, with_oracle=True, with_gpu=True, seed=1234):
    gpu = orc = None
    if with_gpu:
        from rllama_b200 import DataSettings, Transformer
        ds = DataSettings(cl=cuda_ctx)
        if f16:
            ds = ds.force_f16()
        gpu = Transformer(cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"], cfg["max_seq_len"],
                          cfg["norm_eps"], ds)
    if with_oracle:
        from oracle import oracle as O
        orc = O.OracleTransformer(cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"], cfg["norm_eps"],
                                  cfg["max_seq_len"], f16, nthreads=oracle_threads)
    for kind, layer in S.tensor_list(cfg):
        t = S.synth_tensor(kind, layer, cfg, seed)
        if gpu is not None:
            gpu.set_tensor(kind, layer, t)
        if orc is not None:
            orc.set_tensor(kind, layer, t)
    if gpu is not None:
        gpu.finalize()
    return gpu, orc


def rel_err(got, want):
    """max |delta| / max |want|: the f32 parity measure (bound 1e-4)."""
    return float(np.abs(got - want).max() / np.abs(want).max())


def top2_margin(logits):
    top2 = np.partition(logits, -2)[-2:]
    return float(top2[1] - top2[0])
