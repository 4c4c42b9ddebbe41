"""Writes synthetic checkpoints in the layout rllama reads (README "unzip the .pth" step):
``<model>/consolidated.NN/data.pkl`` + ``<model>/consolidated.NN/data/<key>`` + ``params.json``.
The pickle is produced by the real ``torch.save`` (protocol 2) and unzipped, so the loader is
tested against what PyTorch actually emits."""
import io
import json
import os
import pickle
import zipfile

import numpy as np

from rllama_b200 import sharding
from rllama_b200 import synthetic as S

NAMES = {
    "tok_embeddings": "tok_embeddings.weight", "norm": "norm.weight", "output": "output.weight",
    "wq": "layers.{l}.attention.wq.weight", "wk": "layers.{l}.attention.wk.weight", "wv": "layers.{l}.attention.wv.weight",
    "wo": "layers.{l}.attention.wo.weight", "w1": "layers.{l}.feed_forward.w1.weight", "w2": "layers.{l}.feed_forward.w2.weight",
    "w3": "layers.{l}.feed_forward.w3.weight", "attention_norm": "layers.{l}.attention_norm.weight",
    "ffn_norm": "layers.{l}.ffn_norm.weight",
}
COL_SPLIT = ("wo", "w2", "tok_embeddings")  # concatenated along columns by the reference
REPLICATED = ("attention_norm", "ffn_norm", "norm")


def write_llama_checkpoint(path, cfg, seed=1234, n_shards=1):
    import torch
    os.makedirs(path, exist_ok=True)
    full = {}
    for kind, layer in S.tensor_list(cfg):
        full[(kind, layer)] = S.synth_tensor(kind, layer, cfg, seed).astype(np.float16)
    for shard in range(n_shards):
        state = {}
        for (kind, layer), t in full.items():
            name = NAMES[kind].format(l=layer)
            if kind in REPLICATED:
                piece = t.reshape(-1)  # gains are 1-D in Meta's files
            elif kind in COL_SPLIT:
                n = t.shape[1] // n_shards
                piece = t[:, shard * n:(shard + 1) * n]
            else:
                n = t.shape[0] // n_shards
                piece = t[shard * n:(shard + 1) * n]
            state[name] = torch.from_numpy(np.ascontiguousarray(piece)).clone()
        buf = io.BytesIO()
        torch.save(state, buf)
        out = os.path.join(path, "consolidated.%02d" % shard)
        os.makedirs(os.path.join(out, "data"), exist_ok=True)
        with zipfile.ZipFile(io.BytesIO(buf.getvalue())) as z:
            for info in z.infolist():
                rel = info.filename.split("/", 1)[1] if "/" in info.filename else info.filename
                if rel == "data.pkl" or rel.startswith("data/"):
                    with open(os.path.join(out, rel), "wb") as f:
                        f.write(z.read(info))
    with open(os.path.join(path, "params.json"), "w") as f:
        json.dump({"dim": cfg["dim"], "multiple_of": 256, "n_heads": cfg["n_heads"], "n_layers": cfg["n_layers"],
                   "norm_eps": cfg["norm_eps"], "vocab_size": -1}, f)
    return full


def python_unpickle(path):
    """Independent reading of data.pkl with Python's own pickle VM: name -> (storage key, shape, offset)."""
    class Stub:
        def __init__(self, *a):
            self.a = a

    class U(pickle.Unpickler):
        def find_class(self, module, name):
            if (module, name) == ("torch._utils", "_rebuild_tensor_v2"):
                return lambda storage, offset, shape, stride, *rest: (storage[2], tuple(shape), offset, tuple(stride))
            if (module, name) == ("collections", "OrderedDict"):
                import collections
                return collections.OrderedDict
            return type(name, (), {"__module__": module})

        def persistent_load(self, pid):
            return pid

    with open(path, "rb") as f:
        return U(f).load()


HF_NAMES = {
    "tok_embeddings": "model.embed_tokens.weight", "norm": "model.norm.weight", "output": "lm_head.weight",
    "wq": "model.layers.{l}.self_attn.q_proj.weight", "wk": "model.layers.{l}.self_attn.k_proj.weight",
    "wv": "model.layers.{l}.self_attn.v_proj.weight", "wo": "model.layers.{l}.self_attn.o_proj.weight",
    "w1": "model.layers.{l}.mlp.gate_proj.weight", "w2": "model.layers.{l}.mlp.down_proj.weight",
    "w3": "model.layers.{l}.mlp.up_proj.weight", "attention_norm": "model.layers.{l}.input_layernorm.weight",
    "ffn_norm": "model.layers.{l}.post_attention_layernorm.weight",
}


def hf_permute(w, n_heads):
    """What HuggingFace's conversion does to wq / wk: per head, the interleaved rotary pairs
    [hd/2][2] become [2][hd/2] (all even components first)."""
    rows, cols = w.shape
    hd = rows // n_heads
    return np.ascontiguousarray(w.reshape(n_heads, hd // 2, 2, cols).transpose(0, 2, 1, 3).reshape(rows, cols))


def write_hf_checkpoint(path, cfg, seed=1234, n_files=2, deflate=False, zip64=False):
    """A HuggingFace-style directory (config.json, pytorch_model.bin.index.json, *.bin torch.save
    archives) holding the same synthetic weights as write_llama_checkpoint, with HuggingFace's tensor
    names and its q/k row permutation. Returns {hf name: float16 array as stored}."""
    import torch
    os.makedirs(path, exist_ok=True)
    stored = {}
    for kind, layer in S.tensor_list(cfg):
        t = S.synth_tensor(kind, layer, cfg, seed).astype(np.float16)
        if kind in ("wq", "wk"):
            t = hf_permute(t, cfg["n_heads"])
        if kind in REPLICATED:
            t = t.reshape(-1)
        stored[HF_NAMES[kind].format(l=layer)] = t
    names = list(stored)
    weight_map = {}
    for i in range(n_files):
        fname = "pytorch_model-%05d-of-%05d.bin" % (i + 1, n_files)
        part = {n: torch.from_numpy(np.ascontiguousarray(stored[n])).clone() for n in names[i::n_files]}
        for n in part:
            weight_map[n] = fname
        buf = io.BytesIO()
        torch.save(part, buf)
        raw = buf.getvalue()
        if deflate:  # the same members, compressed (the reference reads these through the zip crate)
            out = io.BytesIO()
            with zipfile.ZipFile(io.BytesIO(raw)) as zin, zipfile.ZipFile(out, "w", zipfile.ZIP_DEFLATED) as zout:
                for info in zin.infolist():
                    if zip64:  # zip64 extra fields in the local header and the central directory
                        with zout.open(info.filename, "w", force_zip64=True) as dst:
                            dst.write(zin.read(info))
                    else:
                        zout.writestr(info.filename, zin.read(info))
            raw = out.getvalue()
        with open(os.path.join(path, fname), "wb") as f:
            f.write(raw)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump({"vocab_size": cfg["vocab"], "hidden_size": cfg["dim"], "intermediate_size": cfg["ffn"],
                   "num_hidden_layers": cfg["n_layers"], "num_attention_heads": cfg["n_heads"],
                   "max_position_embeddings": cfg["max_seq_len"], "rms_norm_eps": cfg["norm_eps"], "architectures": ["LlamaForCausalLM"],
                   "bos_token_id": 1, "eos_token_id": 2, "torch_dtype": "float16"}, f)
    with open(os.path.join(path, "pytorch_model.bin.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": int(sum(v.nbytes for v in stored.values()))}, "weight_map": weight_map}, f)
    return stored
