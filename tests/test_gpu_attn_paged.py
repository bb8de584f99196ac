"""Paged grouped-query attention (device pointers, bf16 KV pages, split over the context) vs the CPU
oracle's flash_attn (src/backends/cpu_ref/cpu_ref.cpp:223-280) on the same bf16-rounded K/V expanded
per query head the way the reference's caller does (src/cli/main.cpp:3364-3383)."""
import numpy as np
import pytest
import torch

from ggnpu_b200.backend import Status

pytestmark = pytest.mark.gpu


def make_case(n_head, n_kv, hd, page, n_pages, seed):
    g = torch.Generator().manual_seed(seed)
    ctx = page * n_pages
    k = torch.randn(ctx, n_kv, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(ctx, n_kv, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(n_head, hd, generator=g)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)        # a shuffled block table

    def paged(x):
        pages = x.reshape(n_pages, page, n_kv, hd).permute(0, 2, 1, 3).contiguous()   # [logical page][kv][slot][hd]
        phys = torch.empty_like(pages)
        phys[perm.long()] = pages
        return phys

    return q, k, v, paged(k), paged(v), perm


def expanded(x, n_head, n_kv, upto):
    grp = n_head // n_kv
    xf = x[:upto].float().numpy()                                        # [ctx][kv][hd]
    return np.ascontiguousarray(np.stack([xf[:, h // grp, :] for h in range(n_head)]))


@pytest.mark.parametrize("shape", [(32, 8, 64, 64, 8), (12, 2, 128, 64, 5), (16, 2, 256, 16, 40), (4, 4, 64, 32, 3)])
def test_paged_attention_matches_oracle(backend, oracle, shape):
    n_head, n_kv, hd, page, n_pages = shape
    q, k, v, kp, vp, table = make_case(*shape, seed=sum(shape))
    dev = torch.device("cuda:0")
    dq, dk, dv, dt = q.to(dev), kp.to(dev), vp.to(dev), table.to(dev)
    out = torch.empty(n_head, hd, device=dev)
    ctx = page * n_pages
    for pos in (0, page - 1, page, ctx // 2 + 3, ctx - 1):
        torch.cuda.synchronize()
        st = backend.attn_paged_device(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dt.data_ptr(), out.data_ptr(),
                                       n_head, n_kv, hd, page, n_pages, pos)
        assert st == Status.OK, backend.last_error_message()
        backend.sync()
        want = oracle.flash_attn(q.numpy(), expanded(k, n_head, n_kv, pos + 1), expanded(v, n_head, n_kv, pos + 1), -1)
        assert np.allclose(out.cpu().numpy(), want, rtol=2e-5, atol=2e-6), (shape, pos)


@pytest.mark.parametrize("shape", [(32, 8, 64, 64, 8), (12, 2, 128, 64, 5), (8, 2, 64, 16, 12)])
def test_prefill_attention_matches_oracle(backend, oracle, shape):
    """A chunk of query tokens, causal: every token against the oracle's single-query flash_attn.
    page 64 with head_dim 64 / 128 runs the tensor-core kernel (Q and the softmax weights rounded to
    bf16: rel-L2 <= 5e-3, max-abs <= 2e-2 of the largest output); page 16 runs the per-token kernel
    (fp32 queries: 2e-5)."""
    n_head, n_kv, hd, page, n_pages = shape
    _, k, v, kp, vp, table = make_case(*shape, seed=sum(shape) + 1)
    dev = torch.device("cuda:0")
    dk, dv, dt = kp.to(dev), vp.to(dev), table.to(dev)
    ctx = page * n_pages
    tensor_path = page == 64
    for pos0, n_tok in ((0, 70), (page + 5, 100), (ctx - 130, 130), (3, 32)):
        g = torch.Generator().manual_seed(pos0 + n_tok)
        q = torch.randn(n_tok, n_head, hd, generator=g)
        dq = q.to(dev)
        out = torch.full((n_tok, n_head, hd), float("nan"), device=dev)
        torch.cuda.synchronize()
        st = backend.attn_prefill_device(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dt.data_ptr(), out.data_ptr(),
                                         n_head, n_kv, hd, page, n_pages, pos0, n_tok)
        assert st == Status.OK, backend.last_error_message()
        backend.sync()
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        for t in (0, 1, n_tok // 2, n_tok - 2, n_tok - 1):
            upto = pos0 + t + 1
            want = oracle.flash_attn(q[t].numpy(), expanded(k, n_head, n_kv, upto), expanded(v, n_head, n_kv, upto), -1)
            if tensor_path:
                err = got[t] - want
                assert np.linalg.norm(err) <= 5e-3 * np.linalg.norm(want), (shape, pos0, t, np.linalg.norm(err) / np.linalg.norm(want))
                assert np.abs(err).max() <= 2e-2 * np.abs(want).max()
            else:
                assert np.allclose(got[t], want, rtol=2e-5, atol=2e-6), (shape, pos0, t)


def test_gated_attention_head_256(backend, oracle):
    """qwen35 full-attention layer core (src/cli/main.cpp:3054-3060, 3098): the q projection holds per head
    [query(256) | gate(256)]; the query halves feed the paged attention (16 Q / 2 KV heads of 256), the output is
    multiplied by sigmoid(gate).  vs the oracle's flash_attn on the gathered query times the same gate."""
    n_head, n_kv, hd, page, n_pages = 16, 2, 256, 64, 4
    _, k, v, kp, vp, table = make_case(n_head, n_kv, hd, page, n_pages, seed=99)
    g = torch.Generator().manual_seed(5)
    qg = torch.randn(n_head, 2 * hd, generator=g)
    dev = torch.device("cuda:0")
    dqg, dk, dv, dt = qg.to(dev), kp.to(dev), vp.to(dev), table.to(dev)
    dq = torch.full((n_head, hd), float("nan"), device=dev)
    out = torch.empty(n_head, hd, device=dev)
    pos = 150
    torch.cuda.synchronize()
    assert backend.qgate_split_device(dqg.data_ptr(), dq.data_ptr(), n_head, hd) == Status.OK
    assert backend.attn_paged_device(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dt.data_ptr(), out.data_ptr(),
                                     n_head, n_kv, hd, page, n_pages, pos) == Status.OK, backend.last_error_message()
    assert backend.attn_gate_device(out.data_ptr(), dqg.data_ptr(), n_head, hd) == Status.OK
    backend.sync()
    q = qg[:, :hd].contiguous().numpy()
    gate = qg[:, hd:].numpy().astype(np.float32)
    assert np.array_equal(dq.cpu().numpy(), q)
    want = oracle.flash_attn(q, expanded(k, n_head, n_kv, pos + 1), expanded(v, n_head, n_kv, pos + 1), -1)
    want = want * (np.float32(1.0) / (np.float32(1.0) + np.exp(-gate)))
    assert np.allclose(out.cpu().numpy(), want, rtol=3e-5, atol=3e-6)
    assert backend.attn_gate_device(0, dqg.data_ptr(), n_head, hd) == Status.INVALID_PARAM


def test_paged_attention_argument_errors(backend):
    dev = torch.device("cuda:0")
    t = torch.zeros(64, device=dev)
    it = torch.zeros(4, device=dev, dtype=torch.int32)
    ok = dict(n_head=4, n_kv=2, head_dim=64, page=16, n_pages=4, pos=3)
    bad = [dict(ok, pos=64), dict(ok, pos=-1), dict(ok, n_head=3), dict(ok, head_dim=96), dict(ok, n_head=32, n_kv=2)]
    for kw in bad:
        st = backend.attn_paged_device(t.data_ptr(), t.data_ptr(), t.data_ptr(), it.data_ptr(), t.data_ptr(), **kw)
        assert st == Status.INVALID_PARAM
    assert backend.attn_paged_device(0, t.data_ptr(), t.data_ptr(), it.data_ptr(), t.data_ptr(), **ok) == Status.INVALID_PARAM
