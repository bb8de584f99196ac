"""Grid-coded GGUF formats (IQ2_XXS / IQ2_XS / IQ2_S / IQ3_XXS / IQ3_S / IQ1_S / IQ1_M,
src/quant/iquants.cpp:37-203): the C restatement against the committed outputs of the reference's
decoders, against the reference compiled here (where its tree is present) and against the decode of
the gguf package; the CUDA path (block decode bit-exact, matmul at M = 1, 3 and 40) against the
restatement.  No quantiser exists for these formats here: inputs are random block bytes with finite
scales, which reach every bit pattern of the packed fields."""
import numpy as np
import pytest

from conftest import bits, rel_l2
from ggnpu_b200.testing import synth as S
from ggnpu_b200.backend import Status

GGUF_NAMES = {S.IQ2_XXS: "IQ2_XXS", S.IQ2_XS: "IQ2_XS", S.IQ2_S: "IQ2_S", S.IQ3_XXS: "IQ3_XXS", S.IQ3_S: "IQ3_S",
              S.IQ1_S: "IQ1_S", S.IQ1_M: "IQ1_M"}


@pytest.fixture(autouse=True)
def _needs_codebooks(oracle):
    # the codebooks are generated at build time from the gguf package; a build without it leaves these formats out
    if oracle.lib.ggo_block_elems(S.IQ2_XXS) == 0:
        pytest.skip("library built without the grid-coded formats (gguf package absent at build time)")


def test_block_geometry(oracle):
    # include/ggnpu/quant/iquants.h:40-46, tests/test_quant.cpp:294-317
    want = {S.IQ2_XXS: 66, S.IQ2_XS: 74, S.IQ2_S: 82, S.IQ3_XXS: 98, S.IQ3_S: 110, S.IQ1_S: 50, S.IQ1_M: 56}
    for t, bb in want.items():
        assert oracle.lib.ggo_block_elems(t) == 256 and oracle.lib.ggo_block_bytes(t) == bb
        assert S.BLOCK[t] == (256, bb)


@pytest.mark.parametrize("t", S.GRID_TYPES)
def test_oracle_matches_reference_vectors(oracle, grid_vectors, t):
    v = grid_vectors
    assert np.array_equal(bits(oracle.dequant_blocks(t, v[f"dq_in_{t}"])), bits(v[f"dq_out_{t}"]))
    got = oracle.matmul_exact(v["mm_A"], v[f"mm_W_{t}"], t, 8, 512)
    assert np.array_equal(bits(got), bits(v[f"mm_exact_{t}"]))


@pytest.mark.parametrize("t", S.GRID_TYPES)
def test_oracle_matches_compiled_reference(oracle, ref, t):
    raw = S.random_blocks(t, 4096, seed=500 + t)
    assert np.array_equal(bits(oracle.dequant_blocks(t, raw)), bits(ref.dequant_blocks(t, raw)))


@pytest.mark.parametrize("t", S.GRID_TYPES)
def test_oracle_matches_gguf_package(oracle, t):
    gguf = pytest.importorskip("gguf")
    raw = S.random_blocks(t, 4096, seed=600 + t)
    want = gguf.quants.dequantize(raw.reshape(-1), getattr(gguf.GGMLQuantizationType, GGUF_NAMES[t])).astype(np.float32)
    assert np.array_equal(bits(oracle.dequant_blocks(t, raw)).reshape(-1), bits(want).reshape(-1))


@pytest.mark.gpu
@pytest.mark.parametrize("t", S.GRID_TYPES)
def test_cuda_block_decode_bit_exact(backend, oracle, grid_vectors, t):
    raw = S.random_blocks(t, 4096, seed=1000 + t)
    got = backend.dequant_rows(t, raw, 512, 2048)
    assert np.array_equal(bits(got), bits(oracle.dequant_blocks(t, raw).reshape(512, 2048)))
    raw = grid_vectors[f"dq_in_{t}"]
    got = backend.dequant_rows(t, raw, raw.shape[0], 256)
    assert np.array_equal(bits(got.reshape(-1)), bits(grid_vectors[f"dq_out_{t}"]).reshape(-1))
    # a row window of a ragged matrix (the role of dequant_tensor_row, src/cli/main.cpp:36-261)
    N, K = 37, 768
    raw = S.random_blocks(t, N * 3, seed=t)
    full = oracle.dequant_blocks(t, raw).reshape(N, K)
    assert np.array_equal(bits(backend.dequant_rows(t, raw, N, K, 17, 5)), bits(full[17:22]))


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 3, 40])
@pytest.mark.parametrize("t", S.GRID_TYPES)
def test_cuda_matmul(backend, oracle, t, M):
    """mul_mat_q (Backend::mul_mat_q, include/ggnpu/backend.h:117-125) with a grid-coded weight.
    M = 1, 3: fp32 GEMV, summation order only (rel-L2 <= 1e-5).  M = 40: tcgen05 GEMM with fp16
    operands, rel-L2 <= 2e-3 against the exact fp32 product."""
    N, K = 136, 1024
    raw = S.random_blocks(t, N * K // 256, seed=2000 + t)
    # random scale bytes span the whole fp16 range; weights of a model's size keep the fp16 operands
    # of the tensor-core path finite
    rng = np.random.default_rng(t)
    raw = S.set_grid_block_scales(raw, t, rng.uniform(5e-4, 4e-3, raw.shape[0]) * rng.choice([-1.0, 1.0], raw.shape[0]))
    W = oracle.dequant_blocks(t, raw).reshape(N, K)
    assert np.isfinite(W).all() and np.abs(W).max() < 8.0
    A = np.random.default_rng(M).standard_normal((M, K)).astype(np.float32)
    C = np.full((M, N), np.nan, np.float32)
    before = backend.launch_count()
    assert backend.mul_mat_q(A, raw, C, M, N, K, t) == Status.OK, backend.last_error_message()
    assert backend.launch_count() > before
    want = oracle.matmul_exact(A, raw, t, N, K)
    assert np.isfinite(C).all()
    assert rel_l2(C, want) <= (1e-5 if M < 32 else 2e-3), rel_l2(C, want)


@pytest.mark.gpu
def test_cuda_gather_rows_of_a_grid_coded_embedding(backend, oracle):
    """The embedding lookup (dequant_tensor_row on token rows) on an IQ3_S table."""
    t, N, K = S.IQ3_S, 64, 512
    raw = S.random_blocks(t, N * 2, seed=7)
    full = oracle.dequant_blocks(t, raw).reshape(N, K)
    for r0 in (0, 31, 63):
        assert np.array_equal(bits(backend.dequant_rows(t, raw, N, K, r0, 1)), bits(full[r0:r0 + 1]))
