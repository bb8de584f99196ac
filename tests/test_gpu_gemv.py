"""Dequant-fused quantised matmul (decode GEMV path, M <= 16) through Backend::mul_mat_q vs the exact
CPU matmul (dequant_tensor_row + sequential fp32 dot, src/cli/main.cpp:1379-1388).

Tolerance: the GPU sums in a different order and factors the block scales out of the inner sum, so
results agree to fp32 summation error: rel-L2 <= 1e-5 and max-abs <= 1e-4 * max|ref|."""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from ggnpu_b200.testing import synth as S
from ggnpu_b200.backend import Status

pytestmark = pytest.mark.gpu

REL_L2, MAX_REL = 1e-5, 1e-4
BENCH_TYPES = [S.Q4_0, S.Q8_0, S.Q4_K, S.Q6_K, S.IQ4_XS]
OTHER_TYPES = [S.Q4_1, S.Q2_K, S.Q3_K, S.Q5_K, S.IQ4_NL, S.BF16, S.F16]


def make(t, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    return S.quantize(torch.randn(N, K, generator=g) * 0.02, t).numpy()


def check(backend, oracle, t, N, K, M, seed=7, sample_rows=None):
    raw = make(t, N, K, seed)
    A = np.random.default_rng(seed).standard_normal((M, K)).astype(np.float32)
    C = np.full((M, N), np.nan, np.float32)
    assert backend.mul_mat_q(A, raw, C, M, N, K, t) == Status.OK, backend.last_error_message()
    if sample_rows is None:
        want = oracle.matmul_exact(A, raw, t, N, K)
        got = C
    else:
        rows = np.unique(np.concatenate([np.arange(8), np.arange(N - 8, N), np.random.default_rng(1).integers(0, N, sample_rows)]))
        rb = S.row_bytes(t, K)
        sub = np.ascontiguousarray(raw.reshape(N, rb)[rows])
        want = oracle.matmul_exact(A, sub, t, len(rows), K)
        got = C[:, rows]
        assert np.isfinite(C).all()
    assert rel_l2(got, want) <= REL_L2, (S.TYPE_NAMES[t], N, K, M, rel_l2(got, want))
    assert np.abs(got - want).max() <= MAX_REL * np.abs(want).max()


@pytest.mark.parametrize("t", BENCH_TYPES + OTHER_TYPES)
@pytest.mark.parametrize("M", [1, 2, 3, 16])
def test_small_shapes_all_formats(backend, oracle, t, M):
    check(backend, oracle, t, 67, 1024, M)          # N not a multiple of the row group
    check(backend, oracle, t, 256, 256, M)          # one super-block per row


@pytest.mark.parametrize("t", BENCH_TYPES)
@pytest.mark.parametrize("shape", [(2048, 2048), (8192, 2048), (2048, 8192), (8960, 1536)])
def test_benchmark_shapes(backend, oracle, t, shape):
    """The four microbenchmark weight shapes at M = 1 and 16, checked on sampled rows (the exact
    CPU matmul over whole matrices would take minutes)."""
    N, K = shape
    for M in (1, 16):
        check(backend, oracle, t, N, K, M, sample_rows=48)


@pytest.mark.parametrize("t", [S.Q4_K, S.Q6_K])
def test_cpu_backend_matmul_also_within_tolerance(backend, oracle, vectors, t):
    """The CPU backend's own K-quant matmul (per-block partial sums, cpu_ref.cpp:87-117) differs
    from the exact path only in summation order; both sit inside the tolerance."""
    A, W = vectors["mm_A"], vectors[f"mm_W_{t}"]
    C = np.empty((3, 24), np.float32)
    assert backend.mul_mat_q(A, W, C, 3, 24, 512, t) == Status.OK
    assert rel_l2(C, vectors[f"mm_exact_{t}"]) <= REL_L2
    assert rel_l2(C, vectors[f"mm_cpuref_{t}"]) <= REL_L2


def test_linearity_at_full_size(backend):
    """Size-independent property on a full benchmark matrix: W(a x + b y) == a W x + b W y."""
    N, K, t = 8192, 2048, S.Q4_K
    raw = make(t, N, K, 21)
    rng = np.random.default_rng(4)
    x, y = rng.standard_normal((1, K)).astype(np.float32), rng.standard_normal((1, K)).astype(np.float32)
    outs = []
    for v in (x, y, (2.0 * x - 3.0 * y).astype(np.float32)):
        C = np.empty((1, N), np.float32)
        assert backend.mul_mat_q(v, raw, C, 1, N, K, t) == Status.OK
        outs.append(C)
    assert rel_l2(outs[2], 2.0 * outs[0] - 3.0 * outs[1]) < 5e-6


def test_strided_rows_and_weight_cache(backend, oracle):
    """lda/ldc wider than K/N are honoured (the NPU backend honours them, amd_xdna.cpp:637,894), and
    a second call with the same weight pointer reuses the packed HBM copy."""
    t, N, K, M = S.Q4_K, 40, 512, 3
    raw = make(t, N, K, 3)
    Abuf = np.random.default_rng(0).standard_normal((M, K + 64)).astype(np.float32)
    Cbuf = np.zeros((M, N + 8), np.float32)
    before = backend.launch_count()
    assert backend.mul_mat_q(Abuf, raw, Cbuf, M, N, K, t, lda=K + 64, ldc=N + 8) == Status.OK
    first = backend.launch_count() - before
    want = oracle.matmul_exact(np.ascontiguousarray(Abuf[:, :K]), raw, t, N, K)
    assert rel_l2(Cbuf[:, :N], want) <= REL_L2 and np.all(Cbuf[:, N:] == 0)
    before = backend.launch_count()
    assert backend.mul_mat_q(Abuf, raw, Cbuf, M, N, K, t, lda=K + 64, ldc=N + 8) == Status.OK
    assert backend.launch_count() - before < first      # no re-pack kernels the second time


def test_fused_epilogues_device_path(backend, oracle):
    """Device-pointer GEMV with the fused pieces of the layer graph: RMSNorm prologue
    (cpu_ref.cpp:139-156), bias (main.cpp:3274-3284), residual (main.cpp:3423-3431) and the SwiGLU
    pair (main.cpp:3449-3479)."""
    t, N, K = S.Q4_K, 96, 512
    wg, wu = make(t, N, K, 1), make(t, N, K, 2)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, K)).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    resid = rng.standard_normal((2, N)).astype(np.float32)
    dev = torch.device("cuda:0")
    dx, dg = torch.from_numpy(x).to(dev), torch.from_numpy(gamma).to(dev)
    db, dr = torch.from_numpy(bias).to(dev), torch.from_numpy(resid).to(dev)
    dy = torch.empty((2, N), device=dev, dtype=torch.float32)
    hg, hu = backend.upload_weight(t, wg, N, K), backend.upload_weight(t, wu, N, K)
    xn = np.stack([oracle.rms_norm(r, 1e-5, gamma) for r in x])
    g_ref, u_ref = oracle.matmul_exact(xn, wg, t, N, K), oracle.matmul_exact(xn, wu, t, N, K)

    def run(fn):
        torch.cuda.synchronize()
        fn()
        backend.sync()
        return dy.cpu().numpy()

    got = run(lambda: backend.gemv_device(hg, dx.data_ptr(), 2, K, dy.data_ptr(), N, 1, db.data_ptr(), dg.data_ptr(), 1e-5))
    assert rel_l2(got, g_ref + bias) <= REL_L2
    got = run(lambda: backend.gemv_device(hg, dx.data_ptr(), 2, K, dy.data_ptr(), N, 2, dr.data_ptr(), dg.data_ptr(), 1e-5))
    assert rel_l2(got, g_ref + resid) <= REL_L2
    got = run(lambda: backend.gemv_swiglu_device(hg, hu, dx.data_ptr(), 2, K, dy.data_ptr(), N, dg.data_ptr(), 1e-5))
    want = np.stack([oracle.silu(r) for r in g_ref]) * u_ref
    assert rel_l2(got, want) <= 2e-5
    backend.free_weight(hg)
    backend.free_weight(hu)


@pytest.mark.parametrize("t", [S.Q8_0, S.Q4_0, S.IQ4_XS], ids=lambda t: S.TYPE_NAMES[t])
@pytest.mark.parametrize("K", [8960, 8448, 9216])
def test_m1_k_slightly_over_one_unit_per_lane(backend, oracle, t, K):
    """K = 8960 (the Qwen2.5-1.5B down projection) has 280 units of 32 values: one per lane of the eight warps plus 24 that
    the warps take in turn, one row each; 8448 leaves 8 such units, 9216 exactly 32.  M = 1 and the rows path (M = 5)."""
    check(backend, oracle, t, 264, K, 1, seed=K)
    check(backend, oracle, t, 264, K, 5, seed=K + 1, sample_rows=40)


@pytest.mark.parametrize("t", [S.Q8_0, S.Q4_0, S.IQ4_NL, S.IQ4_XS], ids=lambda t: S.TYPE_NAMES[t])
@pytest.mark.parametrize("M", [3, 5, 8, 11, 16])
def test_stream_formats_on_tensor_cores(backend, oracle, t, M):
    """Q8_0 / Q4_0 / IQ4_NL / IQ4_XS at 3..16 rows: int8 MMAs fed by ldmatrix from the stream layout (padded rows in shared
    memory).  Few row groups (teams of warps share one), many row groups, K of one 256-run (IQ4_XS then takes the general
    path: its headers are fetched in pairs), K cut into slices (8192 at 16 rows)."""
    check(backend, oracle, t, 64, 1024, M, seed=M)
    check(backend, oracle, t, 4096, 256, M, seed=M + 1, sample_rows=40)
    check(backend, oracle, t, 256, 1536, M, seed=M + 4, sample_rows=40)
    check(backend, oracle, t, 1024, 2048, M, seed=M + 2, sample_rows=40)
    check(backend, oracle, t, 512, 8192, M, seed=M + 3, sample_rows=40)


@pytest.mark.parametrize("t", [S.Q4_K, S.Q6_K])
@pytest.mark.parametrize("M", [3, 5, 6, 8, 9, 13, 16])
def test_rows_kernel_every_chunk_size(backend, oracle, t, M):
    """3..16 activation rows in one pass over the weights (2, 3 or 6 column groups of the int8 tensor-core operand):
    every group-count boundary, a row-group count that leaves some CTAs idle and one that gives every warp its own
    groups, K with one and with several super-blocks."""
    check(backend, oracle, t, 67, 1024, M, seed=M)            # N not a multiple of 16, few row groups: teams of 8 warps
    check(backend, oracle, t, 4096, 256, M, seed=M + 1, sample_rows=40)     # many row groups per CTA, one super-block per row
    check(backend, oracle, t, 1024, 2048, M, seed=M + 2, sample_rows=40)


@pytest.mark.parametrize("K", [2048, 4096, 5632, 8192, 14336])
def test_rows_kernel_k_slices(backend, oracle, K):
    """Shared memory holds the limb planes of 16 rows over 2048 values of K: a longer K is cut into slices along the grid
    (2, 3 with a shorter last slice, 4 and 7 here), whose partial sums a second kernel adds; M = 11 fits longer slices."""
    for t in (S.Q4_K, S.Q6_K):
        check(backend, oracle, t, 512, K, 16, seed=K, sample_rows=40)
        check(backend, oracle, t, 512, K, 11, seed=K + 1, sample_rows=40)


@pytest.mark.parametrize("t", [S.Q4_K, S.Q8_0, S.IQ4_XS], ids=lambda t: S.TYPE_NAMES[t])
@pytest.mark.parametrize("K", [1024, 5632])
def test_rows_kernel_fused_epilogues(backend, oracle, K, t):
    """RMSNorm prologue, bias, residual (in place) and the SwiGLU pair at M = 7 and 16 on device pointers.  Q4_K (tensor-
    core layout): K = 5632 is cut into three slices (8, 8 and 6 super-blocks).  Q8_0 / IQ4_XS (stream layout): the
    multi-row kernel takes the 16 rows in two chunks at K = 5632."""
    N = 208
    wg, wu = make(t, N, K, 1), make(t, N, K, 2)
    dev = torch.device("cuda:0")
    hg, hu = backend.upload_weight(t, wg, N, K), backend.upload_weight(t, wu, N, K)
    for M in (7, 16):
        rng = np.random.default_rng(M)
        x = rng.standard_normal((M, K)).astype(np.float32)
        gamma = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
        bias = rng.standard_normal(N).astype(np.float32)
        resid = rng.standard_normal((M, N)).astype(np.float32)
        dx, dg, db = torch.from_numpy(x).to(dev), torch.from_numpy(gamma).to(dev), torch.from_numpy(bias).to(dev)
        dy = torch.empty((M, N), device=dev, dtype=torch.float32)
        xn = np.stack([oracle.rms_norm(r, 1e-5, gamma) for r in x])
        g_ref, u_ref = oracle.matmul_exact(xn, wg, t, N, K), oracle.matmul_exact(xn, wu, t, N, K)

        def run(fn):
            torch.cuda.synchronize()
            fn()
            backend.sync()
            return dy.cpu().numpy()

        got = run(lambda: backend.gemv_device(hg, dx.data_ptr(), M, K, dy.data_ptr(), N, 1, db.data_ptr(), dg.data_ptr(), 1e-5))
        assert rel_l2(got, g_ref + bias) <= REL_L2
        dy.copy_(torch.from_numpy(resid))
        got = run(lambda: backend.gemv_device(hg, dx.data_ptr(), M, K, dy.data_ptr(), N, 2, dy.data_ptr(), dg.data_ptr(), 1e-5))
        assert rel_l2(got, g_ref + resid) <= REL_L2
        got = run(lambda: backend.gemv_swiglu_device(hg, hu, dx.data_ptr(), M, K, dy.data_ptr(), N, dg.data_ptr(), 1e-5))
        want = np.stack([oracle.silu(r) for r in g_ref]) * u_ref
        assert rel_l2(got, want) <= 2e-5
        got = run(lambda: backend.gemv_device(hg, dx.data_ptr(), M, K, dy.data_ptr(), N, 0, None, None, 0.0))
        assert rel_l2(got, oracle.matmul_exact(x, wg, t, N, K)) <= REL_L2
    backend.free_weight(hg)
    backend.free_weight(hu)
