"""Prefill GEMM on the tcgen05 tensor cores (M >= 17 through Backend::mul_mat_q and the device-pointer
entry points) vs the CPU oracle.

Operands are fp16 (weights dequantised to fp16, activations rounded to fp16 once), sums fp32.  Bars:
  * "fp16 model", tight: formats filled by the exact decoder (and Q8_0, Q4_0, IQ4_NL, whose fast fillers
    multiply an integer by the block's fp16 scale and round once) equal the oracle's dequantised rows with the SAME two roundings applied (float64 accumulation)
    up to summation order: rel-L2 <= 1e-5, max-abs <= 2e-5 * max|ref|.  This pins tile layout,
    swizzle, K permutation, descriptors and the epilogue.
  * "fp16 model", loose: the fast Q4_K / Q6_K / IQ4_XS fillers round the sub-block scale (and min term)
    to fp16 before the multiply: rel-L2 <= 1.5e-3 against the same model.
  * "reference": against the exact fp32 matmul of the reference's CPU path (dequant_tensor_row +
    sequential dot, src/cli/main.cpp:1379-1388): rel-L2 <= 2e-3."""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from ggnpu_b200.testing import synth as S
from ggnpu_b200.backend import Status

pytestmark = pytest.mark.gpu

TYPES = [S.Q4_K, S.Q6_K, S.Q8_0, S.Q4_0, S.IQ4_XS, S.Q5_K, S.Q2_K, S.Q3_K, S.Q4_1, S.IQ4_NL, S.F16, S.BF16]


def f16(a):
    return np.ascontiguousarray(a, dtype=np.float32).astype(np.float16).astype(np.float64)


LOOSE_TYPES = (S.Q4_K, S.Q6_K, S.IQ4_XS)      # fast fillers that round the scales to fp16


def make(t, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    return S.quantize(torch.randn(N, K, generator=g) * 0.02, t).numpy()


def dequant(oracle, t, raw, N, K):
    return np.stack([oracle.dequant_row(t, raw, r, K) for r in range(N)])


def check_model(got, A, Wd, t):
    want = f16(A) @ f16(Wd).T
    assert np.isfinite(got).all()
    if t in LOOSE_TYPES:
        assert rel_l2(got, want) <= 1.5e-3, rel_l2(got, want)
    else:
        assert rel_l2(got, want) <= 1e-5, rel_l2(got, want)
        assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()


@pytest.mark.parametrize("t", TYPES)
def test_all_formats_fp16_model_and_reference(backend, oracle, t):
    N, K, M = 200, 512, 100            # N not a multiple of the 128-row tile, M not a multiple of 64
    raw = make(t, N, K, 3)
    A = np.random.default_rng(3).standard_normal((M, K)).astype(np.float32)
    C = np.full((M, N), np.nan, np.float32)
    before = backend.launch_count()
    assert backend.mul_mat_q(A, raw, C, M, N, K, t) == Status.OK, backend.last_error_message()
    assert backend.launch_count() > before
    check_model(C, A, dequant(oracle, t, raw, N, K), t)
    assert rel_l2(C, oracle.matmul_exact(A, raw, t, N, K)) <= 2e-3


@pytest.mark.parametrize("M", [17, 24, 32, 64, 257, 600])
@pytest.mark.parametrize("t", [S.Q4_K, S.Q6_K])
def test_token_tiles(backend, oracle, t, M):
    """The smallest M that takes this path, a partly filled tile, exactly one tile, one tile + 1 row,
    several tiles; K with several 64-steps per stage parity."""
    N, K = 256, 1024
    raw = make(t, N, K, 5)
    A = np.random.default_rng(M).standard_normal((M, K)).astype(np.float32)
    C = np.full((M, N), np.nan, np.float32)
    assert backend.mul_mat_q(A, raw, C, M, N, K, t) == Status.OK, backend.last_error_message()
    check_model(C, A, dequant(oracle, t, raw, N, K), t)


def test_k_of_one_and_two_steps(backend, oracle):
    """K = 256 with a 32-wide format has four 64-steps; K = 64 (one step, no stage reuse) and K = 128."""
    for K in (64, 128, 256):
        t, N, M = S.Q8_0, 130, 40
        raw = make(t, N, K, K)
        A = np.random.default_rng(K).standard_normal((M, K)).astype(np.float32)
        C = np.full((M, N), np.nan, np.float32)
        assert backend.mul_mat_q(A, raw, C, M, N, K, t) == Status.OK, backend.last_error_message()
        check_model(C, A, dequant(oracle, t, raw, N, K), t)


def test_benchmark_shapes_sampled_rows(backend, oracle):
    """Llama-3.2-1B projection shapes at a 256-token chunk (one weight tile per CTA) and at 1024 tokens
    (two weight tiles per CTA), Qwen2.5-1.5B's Q8_0 FFN shape; a sample of weight rows is checked."""
    for (N, K), t, M in (((8192, 2048), S.Q4_K, 256), ((2048, 8192), S.Q6_K, 256), ((2048, 2048), S.Q4_K, 256),
                         ((8192, 2048), S.Q4_K, 1024), ((8192, 2048), S.Q6_K, 1024), ((8960, 1536), S.Q8_0, 1000)):
        raw = make(t, N, K, 9)
        A = np.random.default_rng(9).standard_normal((M, K)).astype(np.float32)
        C = np.full((M, N), np.nan, np.float32)
        assert backend.mul_mat_q(A, raw, C, M, N, K, t) == Status.OK, backend.last_error_message()
        assert np.isfinite(C).all()
        rows = np.unique(np.concatenate([np.arange(4), np.arange(N - 4, N), np.random.default_rng(1).integers(0, N, 40)]))
        rb = S.row_bytes(t, K)
        sub = np.ascontiguousarray(raw.reshape(N, rb)[rows])
        check_model(C[:, rows], A, dequant(oracle, t, sub, len(rows), K), t)


ROW_FILL_TYPES = [S.Q8_0, S.Q4_0, S.IQ4_NL, S.IQ4_XS]


@pytest.mark.parametrize("t", ROW_FILL_TYPES, ids=lambda t: S.TYPE_NAMES[t])
def test_row_fillers_tiles_split_k_and_pair(backend, oracle, t):
    """The formats whose weight tiles are filled one (row, 32-block) per thread: a ragged N with split-K
    (K = 2048 over two output tiles), a grid large enough for two weight tiles per CTA (sampled rows), and the
    SwiGLU pair (gate and up tiles side by side in one CTA)."""
    N, K, M = 130, 2048, 70
    raw = make(t, N, K, 11)
    A = np.random.default_rng(11).standard_normal((M, K)).astype(np.float32)
    C = np.full((M, N), np.nan, np.float32)
    assert backend.mul_mat_q(A, raw, C, M, N, K, t) == Status.OK, backend.last_error_message()
    check_model(C, A, dequant(oracle, t, raw, N, K), t)

    N, K, M = 8192, 512, 1024
    raw = make(t, N, K, 12)
    A = np.random.default_rng(12).standard_normal((M, K)).astype(np.float32)
    C = np.full((M, N), np.nan, np.float32)
    assert backend.mul_mat_q(A, raw, C, M, N, K, t) == Status.OK, backend.last_error_message()
    assert np.isfinite(C).all()
    rows = np.unique(np.concatenate([np.arange(4), np.arange(N - 4, N), np.random.default_rng(2).integers(0, N, 40)]))
    sub = np.ascontiguousarray(raw.reshape(N, S.row_bytes(t, K))[rows])
    check_model(C[:, rows], A, dequant(oracle, t, sub, len(rows), K), t)

    N, K, M = 200, 512, 40
    wg, wu = make(t, N, K, 13), make(t, N, K, 14)
    x = np.random.default_rng(13).standard_normal((M, K)).astype(np.float32)
    dev = torch.device("cuda:0")
    dx = torch.from_numpy(x).to(dev)
    dy = torch.empty((M, N), device=dev, dtype=torch.float32)
    hg, hu = backend.upload_weight(t, wg, N, K), backend.upload_weight(t, wu, N, K)
    torch.cuda.synchronize()
    backend.gemv_swiglu_device(hg, hu, dx.data_ptr(), M, K, dy.data_ptr(), N, None, 0.0)
    backend.sync()
    g_ref, u_ref = f16(x) @ f16(dequant(oracle, t, wg, N, K)).T, f16(x) @ f16(dequant(oracle, t, wu, N, K)).T
    assert rel_l2(dy.cpu().numpy(), g_ref / (1.0 + np.exp(-g_ref)) * u_ref) <= (3e-3 if t in LOOSE_TYPES else 2e-5)
    backend.free_weight(hg)
    backend.free_weight(hu)


MICRO_SHAPES = [(2048, 2048), (8192, 2048), (2048, 8192), (8960, 1536)]
MICRO_TYPES = [S.Q4_0, S.Q8_0, S.Q4_K, S.Q6_K, S.IQ4_XS]


@pytest.mark.parametrize("t", MICRO_TYPES, ids=lambda t: S.TYPE_NAMES[t])
@pytest.mark.parametrize("shape", MICRO_SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
def test_microbench_grid_m512(backend, oracle, shape, t):
    """The quantised-matmul microbenchmark grid at M = 512: every one of the four weight shapes in every one
    of the five formats through Backend::mul_mat_q.  A sample of weight rows (first, last and 40 random ones)
    is checked against the fp16-operand model and against the reference's exact fp32 matmul (src/cli/main.cpp:
    1379-1388) within the tensor-core tolerance; every output must be finite."""
    N, K = shape
    M = 512
    if K % S.BLOCK[t][0]:
        pytest.skip("K is not a whole number of blocks of this format")
    raw = make(t, N, K, 31)
    A = np.random.default_rng(7).standard_normal((M, K)).astype(np.float32)
    C = np.full((M, N), np.nan, np.float32)
    assert backend.mul_mat_q(A, raw, C, M, N, K, t) == Status.OK, backend.last_error_message()
    assert np.isfinite(C).all()
    rows = np.unique(np.concatenate([np.arange(4), np.arange(N - 4, N), np.random.default_rng(1).integers(0, N, 40)]))
    sub = np.ascontiguousarray(raw.reshape(N, S.row_bytes(t, K))[rows])
    check_model(C[:, rows], A, dequant(oracle, t, sub, len(rows), K), t)
    assert rel_l2(C[:8, rows], oracle.matmul_exact(A[:8], sub, t, len(rows), K)) <= 2e-3


@pytest.mark.parametrize("K", [512, 2048])
def test_fused_epilogues(backend, oracle, K):
    """RMSNorm prologue, bias, residual (aliasing y) and the SwiGLU pair at M = 70 on device pointers.
    K = 2048 with so few output tiles runs split-K: partial sums, then the epilogue in the reduce kernel."""
    t, N, M = S.Q4_K, 192, 70
    wg, wu = make(t, N, K, 1), make(t, N, K, 2)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((M, K)).astype(np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    resid = rng.standard_normal((M, N)).astype(np.float32)
    dev = torch.device("cuda:0")
    dx, dg, db = torch.from_numpy(x).to(dev), torch.from_numpy(gamma).to(dev), torch.from_numpy(bias).to(dev)
    dy = torch.empty((M, N), device=dev, dtype=torch.float32)
    hg, hu = backend.upload_weight(t, wg, N, K), backend.upload_weight(t, wu, N, K)
    # the kernel normalises in fp32 (x * inv * gamma) and then rounds to fp16
    inv = 1.0 / np.sqrt((x.astype(np.float32) ** 2).sum(1, dtype=np.float32) / np.float32(K) + np.float32(1e-5))
    xn = (x * inv[:, None].astype(np.float32) * gamma).astype(np.float32)
    Wg, Wu = dequant(oracle, t, wg, N, K), dequant(oracle, t, wu, N, K)
    g_ref, u_ref = f16(xn) @ f16(Wg).T, f16(xn) @ f16(Wu).T

    def run(fn):
        torch.cuda.synchronize()
        fn()
        backend.sync()
        return dy.cpu().numpy()

    got = run(lambda: backend.gemv_device(hg, dx.data_ptr(), M, K, dy.data_ptr(), N, 1, db.data_ptr(), dg.data_ptr(), 1e-5))
    assert rel_l2(got, g_ref + bias) <= 1.5e-3
    dy.copy_(torch.from_numpy(resid))
    got = run(lambda: backend.gemv_device(hg, dx.data_ptr(), M, K, dy.data_ptr(), N, 2, dy.data_ptr(), dg.data_ptr(), 1e-5))
    assert rel_l2(got, g_ref + resid) <= 1.5e-3
    got = run(lambda: backend.gemv_swiglu_device(hg, hu, dx.data_ptr(), M, K, dy.data_ptr(), N, dg.data_ptr(), 1e-5))
    want = g_ref / (1.0 + np.exp(-g_ref)) * u_ref
    assert rel_l2(got, want) <= 2e-3
    # against the reference's exact arithmetic
    xo = np.stack([oracle.rms_norm(r, 1e-5, gamma) for r in x])
    ge, ue = oracle.matmul_exact(xo, wg, t, N, K), oracle.matmul_exact(xo, wu, t, N, K)
    assert rel_l2(got, np.stack([oracle.silu(r) for r in ge]) * ue) <= 3e-3
    backend.free_weight(hg)
    backend.free_weight(hu)
