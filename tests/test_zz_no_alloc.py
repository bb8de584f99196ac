"""ggb_attn_paged_static -- paged attention for callers that must not trigger a device allocation
(a process that handed all GPU memory to its own pool, a serving loop that cannot take the stall of
a cudaMalloc).  Its scratch is a fixed array inside the library, shared by all calls.

Checked through the C ABI against ggb_attn_paged_device (same kernels, handle-owned scratch) on two
calls in a row -- the second call finds the first call's leftovers in the shared array -- with the
tolerance the other attention tests use, and against the CPU oracle.  Collected last on purpose."""
import numpy as np
import pytest
import torch

from ggnpu_b200.backend import Status
from test_gpu_attn_paged import expanded, make_case

pytestmark = pytest.mark.gpu


def test_static_scratch_attention_equals_allocating_entry_point(backend, oracle):
    shape = (32, 8, 64, 64, 8)                      # the Llama-3.2-1B attention shape, 512-token cache
    n_head, n_kv, hd, page, n_pages = shape
    q, k, v, kp, vp, table = make_case(*shape, seed=99)
    dev = torch.device("cuda:0")
    dq, dk, dv, dt = q.to(dev), kp.to(dev), vp.to(dev), table.to(dev)
    ref_out = torch.empty(n_head, hd, device=dev)
    out = torch.full((n_head, hd), float("nan"), device=dev)
    # two calls in a row at different positions: more splits first, fewer second, so stale partials
    # from call one sit in the shared array while call two runs
    for pos in (page * n_pages - 1, page + 5):
        torch.cuda.synchronize()
        args = (dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dt.data_ptr())
        dims = (n_head, n_kv, hd, page, n_pages, pos)
        assert backend.attn_paged_device(*args, ref_out.data_ptr(), *dims) == Status.OK
        assert backend.attn_paged_static(*args, out.data_ptr(), *dims) == Status.OK, backend.last_error_message()
        backend.sync()
        got, want = out.cpu().numpy(), ref_out.cpu().numpy()
        assert np.allclose(got, want, rtol=2e-5, atol=2e-6)
        cpu = oracle.flash_attn(q.numpy(), expanded(k, n_head, n_kv, pos + 1), expanded(v, n_head, n_kv, pos + 1), -1)
        assert np.allclose(got, cpu, rtol=2e-5, atol=2e-6)


def test_static_scratch_rejects_oversize_requests(backend):
    dev = torch.device("cuda:0")
    t = torch.zeros(16, device=dev)
    it = torch.zeros(64, device=dev, dtype=torch.int32)
    # 128 query heads exceed the built-in buffer's 64
    st = backend.attn_paged_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), it.data_ptr(), t.data_ptr(), 128, 16, 64, 16, 64, 0)
    assert st == Status.INVALID_PARAM
    assert "built-in scratch" in backend.last_error_message()


def test_static_scratch_entry_point_allocates_no_device_memory(oracle):
    """The property the entry point exists for.  On a handle of its own, which never ran the allocating
    entry point (so no scratch buffer of the handle exists that a regression could quietly borrow), the
    first call does the one-time set-up (symbol address, kernel image); across the next two calls the
    device's free memory, as the driver reports it, must not move by a byte."""
    from ggnpu_b200.backend import CudaBackend
    shape = (32, 8, 64, 64, 8)
    n_head, n_kv, hd, page, n_pages = shape
    q, k, v, kp, vp, table = make_case(*shape, seed=7)
    dev = torch.device("cuda:0")
    dq, dk, dv, dt = q.to(dev), kp.to(dev), vp.to(dev), table.to(dev)
    out = torch.full((n_head, hd), float("nan"), device=dev)
    fresh = CudaBackend(0)
    try:
        args = (dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dt.data_ptr(), out.data_ptr())
        assert fresh.attn_paged_static(*args, n_head, n_kv, hd, page, n_pages, 17) == Status.OK      # set-up call
        fresh.sync()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(0)
        for pos in (page * n_pages - 1, 3):
            assert fresh.attn_paged_static(*args, n_head, n_kv, hd, page, n_pages, pos) == Status.OK, fresh.last_error_message()
            fresh.sync()
        free_after, _ = torch.cuda.mem_get_info(0)
        assert free_after == free_before, (free_before, free_after)
        cpu = oracle.flash_attn(q.numpy(), expanded(k, n_head, n_kv, 4), expanded(v, n_head, n_kv, 4), -1)
        assert np.allclose(out.cpu().numpy(), cpu, rtol=2e-5, atol=2e-6)
    finally:
        fresh.close()
