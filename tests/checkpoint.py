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
