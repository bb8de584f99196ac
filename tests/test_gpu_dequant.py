"""CUDA block decode vs the CPU oracle: bit-exact, every format, through the C ABI
(ggb_dequant_rows packs the bytes into the HBM layout first, so the re-layout is covered too)."""
import numpy as np
import pytest

from conftest import bits
from ggnpu_b200.testing import synth as S

pytestmark = pytest.mark.gpu

ALL_TYPES = S.QUANT_TYPES + [S.F16, S.BF16, S.F32]


@pytest.mark.parametrize("t", ALL_TYPES)
def test_random_blocks_bit_exact(backend, oracle, t):
    be, bb = S.BLOCK[t]
    n_blocks = 4096 if be > 1 else 4096 * 32
    K = be * 8 if be > 1 else 256
    raw = S.random_blocks(t, n_blocks, seed=1000 + t)
    N = n_blocks * be // K
    got = backend.dequant_rows(t, raw, N, K)
    want = oracle.dequant_blocks(t, raw).reshape(N, K)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("t", S.QUANT_TYPES)
def test_reference_vectors_bit_exact(backend, vectors, t):
    raw = vectors[f"dq_in_{t}"]
    be, _ = S.BLOCK[t]
    got = backend.dequant_rows(t, raw, raw.shape[0], be)
    assert np.array_equal(bits(got.reshape(-1)), bits(vectors[f"dq_out_{t}"]))


def test_golden_blocks_of_the_reference_tests(backend):
    # tests/test_quant.cpp:209-288
    b = np.zeros(144, dtype=np.uint8)
    b[0:2] = np.array([0.5], np.float16).view(np.uint8)
    b[2:4] = np.array([0.25], np.float16).view(np.uint8)
    b[4:8], b[8:12], b[16] = 2, 1, 0x31
    y = backend.dequant_rows(S.Q4_K, b, 1, 256)[0]
    assert y[0] == 0.75 and y[1] == -0.25 and y[32] == 2.75
    b = np.zeros(210, dtype=np.uint8)
    b[208:210] = np.array([0.25], np.float16).view(np.uint8)
    b[192], b[196], b[0] = 4, 2, 0x21
    y = backend.dequant_rows(S.Q6_K, b, 1, 256)[0]
    assert y[0] == -31.0 and y[64] == -15.0 and y[1] == -32.0


@pytest.mark.parametrize("t", [S.Q4_K, S.Q6_K, S.Q8_0, S.IQ4_XS])
def test_row_ranges_and_ragged_shapes(backend, oracle, t):
    """Row windows (first, middle, last, empty) of a matrix whose row count is not a multiple of
    anything convenient: the role of dequant_tensor_row (src/cli/main.cpp:36-261)."""
    import torch
    be, _ = S.BLOCK[t]
    K, N = be * 3 if be == 256 else 32 * 7, 37
    raw = S.quantize(torch.randn(N, K, generator=torch.Generator().manual_seed(t)) * 0.02, t).numpy()
    full = oracle.dequant_blocks(t, raw).reshape(N, K)
    for r0, n in [(0, 1), (17, 5), (36, 1), (0, N), (5, 0)]:
        got = backend.dequant_rows(t, raw, N, K, r0, n)
        assert got.shape == (n, K)
        assert np.array_equal(bits(got), bits(full[r0:r0 + n]))


def test_large_matrix_round_trip(backend, oracle):
    """A full-size benchmark matrix (8192 x 2048 Q4_K, 9.4 MB) decoded on the GPU; checked through a
    checksum of per-row checksums plus sampled rows against the oracle."""
    import torch
    N, K = 8192, 2048
    raw = S.quantize(torch.randn(N, K, generator=torch.Generator().manual_seed(5)) * 0.02, S.Q4_K).numpy()
    got = backend.dequant_rows(S.Q4_K, raw, N, K)
    for r in (0, 1, 4095, 8191):
        assert np.array_equal(bits(got[r]), bits(oracle.dequant_row(S.Q4_K, raw, r, K)))
    want = oracle.dequant_blocks(S.Q4_K, raw).reshape(N, K)
    assert np.array_equal(bits(got).sum(axis=1, dtype=np.uint64), bits(want).sum(axis=1, dtype=np.uint64))


def test_invalid_arguments(backend):
    from ggnpu_b200.backend import BackendError, Status
    raw = np.zeros(144, dtype=np.uint8)
    with pytest.raises(BackendError) as e:
        backend.dequant_rows(S.Q4_K, raw, 1, 200)        # K not a multiple of 256
    assert e.value.status == Status.INVALID_PARAM
    with pytest.raises(BackendError):
        backend.dequant_rows(99, raw, 1, 256)            # unknown type
    with pytest.raises(BackendError):
        backend.dequant_rows(S.Q4_K, raw, 1, 256, 1, 1)  # row window out of range
    assert backend.last_error() == Status.INVALID_PARAM
