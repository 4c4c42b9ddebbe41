"""Tensor-parallel shard arithmetic (host side), the same rules the library applies in
``rlb_model_set_tensor``: heads and FFN columns are split along the axes on which rllama
concatenates Meta's model-parallel checkpoint shards -- rows for wq, wk, wv, w1, w3 and
output, columns for wo and w2 (``src/transformer.rs:489-506``, ``:594-617``, ``:302-307``).
"""


def head_span(n_heads, tp_size, rank):
    """(first head, head count) of ``rank``; an uneven remainder goes to the lowest ranks."""
    base, rem = divmod(n_heads, tp_size)
    return rank * base + min(rank, rem), base + (1 if rank < rem else 0)


def tensor_slice(kind, shape, n_heads, head_dim, tp_size, rank):
    """((row0, row1), (col0, col1)) that ``rank`` keeps of a whole checkpoint tensor."""
    rows, cols = shape
    h0, hc = head_span(n_heads, tp_size, rank)
    if kind in ("wq", "wk", "wv"):
        return (h0 * head_dim, (h0 + hc) * head_dim), (0, cols)
    if kind == "wo":
        return (0, rows), (h0 * head_dim, (h0 + hc) * head_dim)
    if kind in ("w1", "w3", "output"):
        n = rows // tp_size
        return (rank * n, (rank + 1) * n), (0, cols)
    if kind == "w2":
        n = cols // tp_size
        return (0, rows), (rank * n, (rank + 1) * n)
    return (0, rows), (0, cols)  # embeddings and gains are replicated
