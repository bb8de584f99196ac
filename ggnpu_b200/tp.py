"""Tensor-parallel sharding of a GGUF tensor set (host side, numpy only).

The reference drives one device (no DP/TP/EP code at all); this is the Megatron-style split the
B200 path uses for models that shard naturally, one process per GPU:

* column parallel (split the weight ROWS, i.e. the output features): attn_q / attn_k / attn_v by
  head, ffn_gate / ffn_up by FFN row, their biases with them.  GGUF rows are independent block
  runs, so a shard is a contiguous byte range.
* row parallel (split K, the input features): attn_output (K = this rank's heads) and ffn_down
  (K = this rank's FFN rows).  Every row's block run is cut at a block boundary, so the K range
  must be a whole number of quant blocks (256 for K-quants, 32 for Q4_0 / Q8_0 ...).
  The partial products are summed over ranks (all-reduce) by the library.
* vocabulary parallel logits: rows [r V / n, (r+1) V / n) of the output matrix (of token_embd when
  the embeddings are tied); the library gathers the slices.
* replicated: token_embd (row gather), norms, rope_freqs.

`shard_tensors` returns the tensor dict of one rank in the form ggnpu_b200.backend.Model takes.
"""
from __future__ import annotations

import dataclasses

import numpy as np

from . import gguf_types as S

COLUMN = ("attn_q.weight", "attn_k.weight", "attn_v.weight", "ffn_gate.weight", "ffn_up.weight",
          "attn_q.bias", "attn_k.bias", "attn_v.bias")
ROW = ("attn_output.weight", "ffn_down.weight")


def check_divisible(cfg, size: int, types: dict | None = None) -> None:
    """Raise ValueError unless the model splits evenly over `size` ranks."""
    if size < 1:
        raise ValueError("group size must be positive")
    for what, v in (("n_head", cfg.n_head), ("n_kv", cfg.n_kv), ("ffn", cfg.ffn), ("vocab", cfg.vocab)):
        if v % size:
            raise ValueError(f"{what} = {v} is not divisible by the tensor-parallel size {size}")


def shard_config(cfg, size: int):
    """The per-rank model description: heads and FFN rows divided, everything else as is."""
    check_divisible(cfg, size)
    return dataclasses.replace(cfg, n_head=cfg.n_head // size, n_kv=cfg.n_kv // size, ffn=cfg.ffn // size)


def slice_rows(tid: int, raw: np.ndarray, n: int, k: int, rank: int, size: int) -> np.ndarray:
    """Rows [rank n / size, (rank + 1) n / size) of an [n][k] tensor of type `tid` (raw GGUF bytes)."""
    if n % size:
        raise ValueError(f"{n} rows do not split over {size} ranks")
    rb = S.row_bytes(tid, k)
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(n, rb)
    nl = n // size
    return np.ascontiguousarray(raw[rank * nl:(rank + 1) * nl]).reshape(-1)


def slice_k(tid: int, raw: np.ndarray, n: int, k: int, rank: int, size: int) -> np.ndarray:
    """Columns [rank k / size, (rank + 1) k / size) of every row: whole quant blocks only."""
    be, bb = S.BLOCK[tid]
    if k % size or (k // size) % be:
        raise ValueError(f"K = {k} does not split over {size} ranks in whole blocks of {be}")
    nb_l = (k // size) // be
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(n, k // be, bb)
    return np.ascontiguousarray(raw[:, rank * nb_l:(rank + 1) * nb_l]).reshape(-1)


def shard_tensors(cfg, tensors: dict, rank: int, size: int) -> dict:
    """One rank's tensors.  `tensors`: name -> (type id, dims with dims[0] = K, raw bytes)."""
    check_divisible(cfg, size)
    if not 0 <= rank < size:
        raise ValueError("rank out of range")
    if size == 1:
        return dict(tensors)
    out = {}
    for name, (tid, dims, raw) in tensors.items():
        leaf = name.split(".", 2)[2] if name.startswith("blk.") else name
        if len(dims) == 2:
            k, n = dims[0], dims[1]
        else:
            k, n = 1, dims[0]
        if leaf in COLUMN:
            if len(dims) == 2:
                out[name] = (tid, (k, n // size), slice_rows(tid, raw, n, k, rank, size))
            else:                                   # bias vector: n F32 values
                v = np.ascontiguousarray(raw).view(np.uint8).reshape(n, -1)
                nl = n // size
                out[name] = (tid, (nl,), np.ascontiguousarray(v[rank * nl:(rank + 1) * nl]).reshape(-1))
        elif leaf in ROW:
            out[name] = (tid, (k // size, n), slice_k(tid, raw, n, k, rank, size))
        elif name == "output.weight":
            out[name] = (tid, (k, n // size), slice_rows(tid, raw, n, k, rank, size))
        else:
            out[name] = (tid, dims, raw)
    if "output.weight" not in tensors:              # tied embeddings: the logits slice comes from token_embd
        tid, dims, raw = tensors["token_embd.weight"]
        out["output.weight"] = (tid, (dims[0], dims[1] // size), slice_rows(tid, raw, dims[1], dims[0], rank, size))
    return out
