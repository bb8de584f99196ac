"""Host side of the tensor-parallel path on CPU: the sharding rules of ggnpu_b200/tp.py, checked with
two gloo ranks against the CPU oracle's exact matmul (dequant_tensor_row + sequential dot,
src/cli/main.cpp:1379-1388).  Column-parallel shards reproduce their rows bit for bit; row-parallel
partial products sum (all-reduce) to the full product up to fp32 summation order."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ggnpu_b200.testing import synth as S
from ggnpu_b200 import tp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank(rank, size, port, q):
    try:
        sys.path.insert(0, ROOT)
        from oracle.binding import Oracle
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=size)
        oracle = Oracle()
        cfg = S.tiny_config(seed=31, n_head=8, n_kv=2, ffn=1024)
        synth = S.build_model(cfg)                       # same seed on every rank: the full model
        mine = tp.shard_tensors(cfg, synth.tensors, rank, size)
        lcfg = tp.shard_config(cfg, size)
        assert (lcfg.n_head, lcfg.n_kv, lcfg.ffn) == (cfg.n_head // size, cfg.n_kv // size, cfg.ffn // size)
        x = np.random.default_rng(5).standard_normal((3, cfg.hidden)).astype(np.float32)

        def full(name):
            t, dims, raw = synth.tensors[name]
            return oracle.matmul_exact(np.ascontiguousarray(x[:, :dims[0]]) if dims[0] <= x.shape[1] else None, raw, t, dims[1], dims[0])

        # column parallel: concatenated shard outputs == full output, bit for bit
        for leaf in ("attn_q.weight", "attn_k.weight", "ffn_gate.weight"):
            name = f"blk.0.{leaf}"
            t, dims, raw = mine[name]
            part = torch.from_numpy(oracle.matmul_exact(x, raw, t, dims[1], dims[0]))
            parts = [torch.empty_like(part) for _ in range(size)]
            dist.all_gather(parts, part)
            assert np.array_equal(torch.cat(parts, dim=1).numpy(), full(name)), name
        # row parallel: this rank's K range of the input against its K range of every row, summed over ranks
        for leaf, kfull in (("attn_output.weight", cfg.n_head * cfg.head_dim), ("ffn_down.weight", cfg.ffn)):
            name = f"blk.0.{leaf}"
            a = np.random.default_rng(6).standard_normal((3, kfull)).astype(np.float32)
            t, dims, raw = mine[name]
            kl = dims[0]
            assert kl == kfull // size
            part = torch.from_numpy(oracle.matmul_exact(np.ascontiguousarray(a[:, rank * kl:(rank + 1) * kl]), raw, t, dims[1], kl))
            dist.all_reduce(part)
            tf, df, rf = synth.tensors[name]
            want = oracle.matmul_exact(a, rf, tf, df[1], df[0])
            rel = np.linalg.norm(part.numpy() - want) / np.linalg.norm(want)
            assert rel <= 1e-6, (name, rel)
        # vocabulary-parallel logits slice (tied embeddings: cut from token_embd)
        t, dims, raw = mine["output.weight"]
        assert dims[1] == cfg.vocab // size
        h = np.random.default_rng(7).standard_normal((1, cfg.hidden)).astype(np.float32)
        part = torch.from_numpy(oracle.matmul_exact(h, raw, t, dims[1], dims[0]))
        parts = [torch.empty_like(part) for _ in range(size)]
        dist.all_gather(parts, part)
        te = synth.tensors["token_embd.weight"]
        assert np.array_equal(torch.cat(parts, dim=1).numpy(), oracle.matmul_exact(h, te[2], te[0], te[1][1], te[1][0]))
        # replicated tensors are untouched
        assert mine["blk.0.attn_norm.weight"][2] is synth.tensors["blk.0.attn_norm.weight"][2]
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # report to the parent instead of dying silently
        import traceback
        q.put((rank, traceback.format_exc()))


def test_two_gloo_ranks_shards_recombine_to_the_full_model():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 500
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert all(msg == "ok" for _, msg in results), results


def test_shard_rules_and_errors():
    cfg = S.tiny_config(seed=3, n_head=8, n_kv=2, ffn=1024)
    with pytest.raises(ValueError):
        tp.check_divisible(cfg, 3)
    with pytest.raises(ValueError):
        tp.shard_config(cfg, 4)                      # n_kv = 2 does not split four ways
    # K ranges must be whole blocks
    raw = S.quantize(torch.randn(8, 512) * 0.02, S.Q4_K).numpy()
    with pytest.raises(ValueError):
        tp.slice_k(S.Q4_K, raw, 8, 512, 0, 4)        # 128 columns per rank < one 256-block
    got = tp.slice_k(S.Q4_K, raw, 8, 512, 1, 2)
    rb = S.row_bytes(S.Q4_K, 512)
    assert np.array_equal(got.reshape(8, -1), raw.reshape(8, rb)[:, rb // 2:])
    rows = tp.slice_rows(S.Q4_K, raw, 8, 512, 1, 4)
    assert np.array_equal(rows, raw.reshape(8, rb)[2:4].reshape(-1))
    one = tp.shard_tensors(cfg, {"output_norm.weight": (S.F32, (cfg.hidden,), np.ones(cfg.hidden, np.float32))}, 0, 1)
    assert list(one) == ["output_norm.weight"]
