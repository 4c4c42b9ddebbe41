"""The checkpoint loader (pickle reader + LLaMA data source + params.json), against checkpoints
written by the real torch.save and against Python's own pickle VM. The reading half needs no GPU;
constructing a model from a checkpoint is checked against the direct set_tensor path on the GPU."""
import os

import numpy as np
import pytest

from rllama_b200 import DataSource, ModelParams, RllamaError
from rllama_b200 import synthetic as S
from rllama_b200.data_source import COLS, FIRST, ROWS
from checkpoint import HF_NAMES, NAMES, hf_permute, python_unpickle, write_hf_checkpoint, write_llama_checkpoint
from helpers import cfg_variant

torch = pytest.importorskip("torch")


def small():
    return cfg_variant("tiny", dim=256, n_heads=4, n_layers=2, ffn=352, vocab=304, max_seq_len=24)


@pytest.mark.parametrize("n_shards", [1, 2])
def test_data_source_reads_what_torch_writes(tmp_path, n_shards):
    cfg = small()
    full = write_llama_checkpoint(str(tmp_path), cfg, n_shards=n_shards)
    ds = DataSource.from_llama_source(tmp_path)
    assert ds.shards() == n_shards
    direction = {"wo": COLS, "w2": COLS, "tok_embeddings": COLS, "attention_norm": FIRST, "ffn_norm": FIRST, "norm": FIRST}
    for (kind, layer), want in full.items():
        name = NAMES[kind].format(l=layer)
        got = ds.tensor(name, direction.get(kind, ROWS))
        assert got.shape == want.shape
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16)), name
    # the pickle reader agrees with Python's own pickle VM on every record
    ref = python_unpickle(os.path.join(str(tmp_path), "consolidated.00", "data.pkl"))
    for name, (key, shape, offset, stride) in ref.items():
        d = FIRST if len(shape) == 1 else ROWS
        rows, cols = ds.tensor_shape(name, FIRST)  # first shard only = this shard's own shape
        assert (rows, cols) == ((1, shape[0]) if len(shape) == 1 else tuple(shape))
    p = ModelParams.from_json(os.path.join(str(tmp_path), "params.json"))
    assert (p.dim, p.n_heads, p.n_layers, p.vocab_size) == (cfg["dim"], cfg["n_heads"], cfg["n_layers"], -1)
    assert abs(p.norm_eps - cfg["norm_eps"]) < 1e-12


def test_loader_errors(tmp_path):
    with pytest.raises(RllamaError):
        DataSource.from_llama_source(tmp_path / "nothing_here")
    cfg = small()
    write_llama_checkpoint(str(tmp_path), cfg)
    ds = DataSource.from_llama_source(tmp_path)
    with pytest.raises(RllamaError):  # UnpicklingError::MissingField
        ds.tensor("layers.9.attention.wq.weight")
    # only torch.HalfStorage loads (src/unpickler.rs:186-191)
    import io, zipfile
    buf = io.BytesIO()
    torch.save({"x.weight": torch.zeros(4, 8, dtype=torch.float32)}, buf)
    out = tmp_path / "f32" / "consolidated.00"
    os.makedirs(out / "data")
    with zipfile.ZipFile(io.BytesIO(buf.getvalue())) as z:
        for info in z.infolist():
            rel = info.filename.split("/", 1)[1]
            if rel == "data.pkl" or rel.startswith("data/"):
                open(out / rel, "wb").write(z.read(info))
    ds32 = DataSource.from_llama_source(tmp_path / "f32")
    with pytest.raises(RllamaError):
        ds32.tensor("x.weight")
    # truncated storage file
    key = os.listdir(tmp_path / "consolidated.00" / "data")[0]
    with open(tmp_path / "consolidated.00" / "data" / key, "r+b") as f:
        f.truncate(10)
    bad = [n for n in [NAMES[k].format(l=l) for k, l in S.tensor_list(cfg)]]
    with pytest.raises(RllamaError):
        for n in bad:
            ds.tensor(n, COLS if (".wo." in n or ".w2." in n or n.startswith("tok_")) else (FIRST if "norm" in n else ROWS))
    # not a pickle
    os.makedirs(tmp_path / "junk" / "consolidated.00")
    open(tmp_path / "junk" / "consolidated.00" / "data.pkl", "wb").write(b"hello")
    with pytest.raises(RllamaError):
        DataSource.from_llama_source(tmp_path / "junk")


@pytest.mark.parametrize("deflate,zip64", [(False, False), (True, False), (True, True)])
def test_huggingface_source_reads_archives_in_place(tmp_path, deflate, zip64):
    """DataSource::from_vicuna_source / from_inferred_source and the q/k anti-transpose."""
    from rllama_b200.data_source import huggingface_llama_model_antitranspose
    cfg = small()
    stored = write_hf_checkpoint(str(tmp_path / "hf"), cfg, n_files=2, deflate=deflate, zip64=zip64)
    ds = DataSource.from_inferred_source(tmp_path / "hf")
    assert ds.need_to_do_antitranspose() and ds.shards() == 1
    for name, want in stored.items():
        got = ds.tensor(name, FIRST if want.ndim == 1 else ROWS)
        assert np.array_equal(got.view(np.uint16).reshape(-1), want.view(np.uint16).reshape(-1)), name
    # the permutation HuggingFace applies is undone exactly (src/tensor.rs:841-909)
    meta = S.synth_tensor("wq", 1, cfg, 1234).astype(np.float16)
    hf = stored[HF_NAMES["wq"].format(l=1)]
    assert not np.array_equal(hf, meta)
    back = huggingface_llama_model_antitranspose(hf, cfg["n_heads"])
    assert np.array_equal(back.view(np.uint16), meta.view(np.uint16))
    rows, cols = meta.shape
    hd = rows // cfg["n_heads"]
    literal = hf.reshape(cfg["n_heads"], 2, hd // 2, cols).transpose(0, 2, 1, 3).reshape(rows, cols)  # the reference's doc comment
    assert np.array_equal(back, literal)
    with pytest.raises(RllamaError):
        huggingface_llama_model_antitranspose(meta[:6], 4)
    # Meta's layout is still recognised by its params.json; anything else is unknown
    write_llama_checkpoint(str(tmp_path / "meta"), cfg)
    assert not DataSource.from_inferred_source(tmp_path / "meta").need_to_do_antitranspose()
    os.makedirs(tmp_path / "empty")
    with pytest.raises(RllamaError, match="Unknown source"):
        DataSource.from_inferred_source(tmp_path / "empty")
    # config.json must carry every field of the reference's struct; a corrupt archive is refused
    import json
    cfgp = tmp_path / "hf" / "config.json"
    full = json.loads(cfgp.read_text())
    del full["torch_dtype"]
    cfgp.write_text(json.dumps(full))
    with pytest.raises(RllamaError, match="torch_dtype"):
        DataSource.from_vicuna_source(tmp_path / "hf")
    full["torch_dtype"] = "float16"
    cfgp.write_text(json.dumps(full))
    (tmp_path / "hf" / "zzz.bin").write_bytes(b"PK\x03\x04 not really a zip")
    with pytest.raises(RllamaError):
        DataSource.from_vicuna_source(tmp_path / "hf")


@pytest.mark.gpu
def test_huggingface_checkpoint_gives_the_same_model(tmp_path, cuda_ctx):
    from rllama_b200 import DataSettings, Transformer
    cfg = small()
    write_llama_checkpoint(str(tmp_path / "meta"), cfg)
    write_hf_checkpoint(str(tmp_path / "hf"), cfg, n_files=3, deflate=True)
    p = ModelParams.from_json(os.path.join(str(tmp_path / "hf"), "config.json"))  # serde aliases: hidden_size, ...
    assert (p.dim, p.n_heads, p.n_layers, p.vocab_size) == (cfg["dim"], cfg["n_heads"], cfg["n_layers"], cfg["vocab"])
    ds = DataSettings(cl=cuda_ctx).force_f16()
    a = Transformer.from_unpickled(p.dim, p.n_layers, p.n_heads, cfg["max_seq_len"], p.norm_eps, ds, DataSource.from_inferred_source(tmp_path / "hf"))
    b = Transformer.from_unpickled(p.dim, p.n_layers, p.n_heads, cfg["max_seq_len"], p.norm_eps, ds, DataSource.from_inferred_source(tmp_path / "meta"))
    toks = S.synth_tokens(9, cfg["vocab"])
    assert np.array_equal(a.forward(toks, 0, a.make_caches()), b.forward(toks, 0, b.make_caches()))


@pytest.mark.gpu
@pytest.mark.parametrize("n_shards,f16", [(1, False), (2, True)])
def test_from_unpickled_equals_set_tensor_path(tmp_path, cuda_ctx, n_shards, f16):
    from rllama_b200 import DataSettings, Transformer
    from helpers import build_pair
    cfg = small()
    write_llama_checkpoint(str(tmp_path), cfg, n_shards=n_shards)
    p = ModelParams.from_json(os.path.join(str(tmp_path), "params.json"))
    ds = DataSettings(cl=cuda_ctx)
    if f16:
        ds = ds.force_f16()
    loaded = Transformer.from_unpickled(p.dim, p.n_layers, p.n_heads, cfg["max_seq_len"], p.norm_eps, ds,
                                        DataSource.from_llama_source(tmp_path))
    assert (loaded.vocab_size, loaded.ffn_dim) == (cfg["vocab"], cfg["ffn"])
    direct, _ = build_pair(cfg, f16, cuda_ctx, with_oracle=False)
    toks = S.synth_tokens(7, cfg["vocab"])
    a = loaded.forward(toks, 0, loaded.make_caches())
    b = direct.forward(toks, 0, direct.make_caches())
    assert np.array_equal(a, b)
