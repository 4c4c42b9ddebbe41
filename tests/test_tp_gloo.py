"""Tensor-parallel plan on CPU: two `gloo` ranks shard a small model along the axes the
library uses (rows of wq/wk/wv/w1/w3/output, columns of wo/w2), all-reduce after `wo` and
`w2`, all-gather the vocabulary shards, and must reproduce the unsharded float64 forward.
Also exercises the rendezvous plumbing `bench.py` uses to hand the communicator id around."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _sharded_forward(rank, world, cfg, weights, tokens, start_pos, caches, dist, torch):
    from rllama_b200 import sharding
    d, H = cfg["dim"], cfg["n_heads"]
    hd = d // H
    h0, hc = sharding.head_span(H, world, rank)

    def sl(kind, layer):
        w = weights[(kind, layer)].astype(np.float64)
        (r0, r1), (c0, c1) = sharding.tensor_slice(kind, w.shape, H, hd, world, rank)
        return w[r0:r1, c0:c1]

    def allreduce(x):
        t = torch.from_numpy(np.ascontiguousarray(x))
        dist.all_reduce(t)
        return t.numpy()

    def norm(x, g):
        return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + cfg["norm_eps"]) * g

    inv = 1.0 / (10000.0 ** (np.arange(0, hd, 2, dtype=np.float64) / hd))
    n = len(tokens)
    T = start_pos + n
    ang = np.outer(np.arange(start_pos, T, dtype=np.float64), inv)
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]

    def rope(x):
        out = np.empty_like(x)
        out[..., 0::2] = x[..., 0::2] * cos - x[..., 1::2] * sin
        out[..., 1::2] = x[..., 0::2] * sin + x[..., 1::2] * cos
        return out

    x = weights[("tok_embeddings", 0)].astype(np.float64)[tokens]
    for l in range(cfg["n_layers"]):
        a = norm(x, weights[("attention_norm", l)].astype(np.float64).reshape(-1))
        q = rope((a @ sl("wq", l).T).reshape(n, hc, hd))
        k = rope((a @ sl("wk", l).T).reshape(n, hc, hd))
        v = (a @ sl("wv", l).T).reshape(n, hc, hd)
        caches["k"][l][start_pos:T] = k
        caches["v"][l][start_pos:T] = v
        K, V = caches["k"][l][:T], caches["v"][l][:T]
        s = np.einsum("ihd,thd->hit", q, K) / np.sqrt(hd)
        mask = np.arange(T)[None, :] > (np.arange(n)[:, None] + start_pos)
        s = np.where(mask[None], -np.inf, s)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        p /= p.sum(axis=-1, keepdims=True)
        o = np.einsum("hit,thd->ihd", p, V).reshape(n, hc * hd)
        x = x + allreduce(o @ sl("wo", l).T)          # exchange step 1
        f = norm(x, weights[("ffn_norm", l)].astype(np.float64).reshape(-1))
        g1 = f @ sl("w1", l).T
        g = g1 / (1.0 + np.exp(-g1)) * (f @ sl("w3", l).T)
        x = x + allreduce(g @ sl("w2", l).T)          # exchange step 2
    x = norm(x, weights[("norm", 0)].astype(np.float64).reshape(-1))
    local = x[-1] @ sl("output", 0).T
    parts = [torch.zeros(local.shape[0], dtype=torch.float64) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(local)))
    return np.concatenate([t.numpy() for t in parts])


def _worker(rank, world, port, heads, result_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    from oracle.llama_f64 import F64Transformer
    from rllama_b200 import sharding, synthetic as S

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = dict(S.CONFIGS["tiny"])
        cfg.update(dim=64 * heads // 2 if heads == 3 else 256, n_heads=heads, n_layers=2, ffn=128 * world, vocab=96 * world, max_seq_len=16)
        weights = {(k, l): S.synth_tensor(k, l, cfg) for k, l in S.tensor_list(cfg)}
        # the communicator id travels as bench.py sends it: rank 0 creates, everyone receives
        ids = [bytes(range(128)) if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        assert ids[0] == bytes(range(128))
        h0, hc = sharding.head_span(heads, world, rank)
        hd = cfg["dim"] // heads
        caches = {"k": [np.zeros((16, hc, hd)) for _ in range(2)], "v": [np.zeros((16, hc, hd)) for _ in range(2)]}
        toks = S.synth_tokens(6, cfg["vocab"])
        outs = [_sharded_forward(rank, world, cfg, weights, toks, 0, caches, dist, torch)]
        for i in range(2):
            outs.append(_sharded_forward(rank, world, cfg, weights, np.array([int(np.argmax(outs[-1]))]), 6 + i, caches, dist, torch))
        if rank == 0:
            ref = F64Transformer(cfg["dim"], cfg["n_layers"], heads, cfg["norm_eps"], 16)
            for (k, l), w in weights.items():
                ref.set_tensor(k, l, w)
            rc = ref.make_caches()
            want = [ref.forward(toks, 0, rc)]
            for i in range(2):
                want.append(ref.forward([int(np.argmax(want[-1]))], 6 + i, rc))
            err = max(float(np.abs(a - b).max() / np.abs(b).max()) for a, b in zip(outs, want))
            with open(result_path, "w") as f:
                f.write(repr(err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("heads", [4, 3])  # 3 heads over 2 ranks: the uneven split (2 + 1)
def test_two_rank_sharded_forward_matches_unsharded(tmp_path, heads):
    import torch.multiprocessing as mp
    port = _free_port()
    result = str(tmp_path / "err.txt")
    mp.spawn(_worker, args=(2, port, heads, result), nprocs=2, join=True)
    err = float(open(result).read())
    assert err < 1e-10, err
