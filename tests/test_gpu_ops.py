"""The small Backend operators through the C ABI vs the CPU oracle, with the seeds and shapes of the
reference's own op-level harness (bench-layer, src/cli/main.cpp:1439-2063) and its unit-test known
answers (tests/test_arch.cpp:95-347)."""
import numpy as np
import pytest

from conftest import bits, rel_l2
from ggnpu_b200.backend import Status

pytestmark = pytest.mark.gpu

# fp32 tolerances: parallel reductions reorder sums; device expf/tanhf/powf/sinf/cosf differ from
# glibc's by a few ulp.
RTOL, ATOL = 2e-6, 1e-6


def mt19937_uniform(n, seed=42):
    # the reference seeds std::mt19937(42) and draws U(-0.5, 0.5) (main.cpp:1470-1475)
    return (np.random.RandomState(seed).random_sample(n) - 0.5).astype(np.float32)


def test_rms_norm(backend, oracle, vectors):
    x = np.array([3.0, 4.0], np.float32)
    y = np.zeros(2, np.float32)
    assert backend.rms_norm(x, y, 2, 1e-5) == Status.OK
    assert abs(y[0] - 0.8485) < 1e-3 and abs(y[1] - 1.1314) < 1e-3
    for n in (2048, 1536, 4096, 100):
        x = mt19937_uniform(n)
        w = (1.0 + 0.1 * np.random.default_rng(n).standard_normal(n)).astype(np.float32)
        y = np.empty(n, np.float32)
        assert backend.rms_norm(x, y, n, 1e-5, w) == Status.OK
        assert np.allclose(y, oracle.rms_norm(x, 1e-5, w), rtol=RTOL, atol=ATOL)
    y = np.empty(2048, np.float32)
    backend.rms_norm(vectors["rms_x"], y, 2048, 1e-5, vectors["rms_w"])
    assert np.allclose(y, vectors["rms_y"], rtol=RTOL, atol=ATOL)
    x = mt19937_uniform(512)
    want = oracle.rms_norm(x, 1e-6)
    assert backend.rms_norm(x, x, 512, 1e-6) == Status.OK          # in place
    assert np.allclose(x, want, rtol=RTOL, atol=ATOL)


def test_silu_gelu_softmax(backend, oracle, vectors):
    x = np.array([0.0, 1.0, -1.0], np.float32)
    y = np.empty(3, np.float32)
    assert backend.silu(x, y, 3) == Status.OK
    assert abs(y[0]) < 1e-3 and abs(y[1] - 0.7311) < 1e-3 and abs(y[2] + 0.2689) < 1e-3
    x = np.concatenate([mt19937_uniform(8192) * 20, np.array([-90.0, 90.0, 0.0], np.float32)])
    y = np.empty_like(x)
    assert backend.silu(x, y, x.size) == Status.OK
    assert np.allclose(y, oracle.silu(x), rtol=RTOL, atol=1e-7)
    assert backend.gelu(x, y, x.size) == Status.OK
    assert np.allclose(y, oracle.gelu(x), rtol=1e-5, atol=1e-6)
    g = x.copy()
    assert backend.gelu(g, g, g.size) == Status.OK                 # the reference calls gelu in place
    assert np.array_equal(bits(g), bits(y))
    sm = vectors["softmax_x"]
    out = np.empty_like(sm)
    assert backend.softmax(sm, out, sm.shape[0], sm.shape[1]) == Status.OK
    assert np.allclose(out, vectors["softmax_y"], rtol=1e-6, atol=1e-8)
    assert np.allclose(out.sum(axis=1), 1.0, atol=1e-6)
    big = np.random.default_rng(0).standard_normal((3, 5000)).astype(np.float32) * 10
    out = np.empty_like(big)
    assert backend.softmax(big, out, 3, 5000) == Status.OK
    assert np.allclose(out, oracle.softmax(big), rtol=1e-5, atol=1e-9)


def test_flash_attn_contract(backend, oracle, vectors):
    Q = np.array([[1.0, 0.0]], np.float32)
    K = np.array([[[1.0, 0.0], [0.0, 1.0]]], np.float32)
    out = np.zeros((1, 2), np.float32)
    assert backend.flash_attn(Q, K, K.copy(), out, 1, 2, 2) == Status.OK
    assert abs(out[0, 0] - 0.670) < 1e-2 and abs(out[0, 1] - 0.330) < 1e-2
    v = vectors
    out = np.empty_like(v["attn_q"])
    assert backend.flash_attn(v["attn_q"], v["attn_k"], v["attn_v"], out, 4, 64, 40, -1) == Status.OK
    assert np.allclose(out, v["attn_full"], rtol=1e-5, atol=1e-6)
    assert backend.flash_attn(v["attn_q"], v["attn_k"], v["attn_v"], out, 4, 64, 40, 17) == Status.OK
    assert np.allclose(out, v["attn_causal17"], rtol=1e-5, atol=1e-6)
    # bench-layer shapes: 1 head ctx 1, and 4 heads ctx 40 causal (main.cpp:1627-1689), plus long context
    rng = np.random.default_rng(1)
    for nh, hd, ctx, qp in [(1, 64, 1, -1), (4, 64, 40, 39), (32, 64, 700, 650), (12, 128, 2111, -1), (2, 256, 33, 0)]:
        Q = rng.standard_normal((nh, hd)).astype(np.float32)
        K = rng.standard_normal((nh, ctx, hd)).astype(np.float32)
        V = rng.standard_normal((nh, ctx, hd)).astype(np.float32)
        out = np.empty_like(Q)
        assert backend.flash_attn(Q, K, V, out, nh, hd, ctx, qp) == Status.OK
        assert np.allclose(out, oracle.flash_attn(Q, K, V, qp), rtol=2e-5, atol=2e-6)


def test_rope_variants(backend, oracle, vectors):
    # Backend::rope without tables: the CPU backend's formula (cpu_ref.cpp:158-174), offset 5
    x = vectors["rope_x"].copy()
    assert backend.rope(x, 64, 5, 1.0, 10000.0, 64) == Status.OK
    assert np.allclose(x, vectors["rope_y"], rtol=1e-5, atol=2e-6)
    # with the host-built tables (RopeCache) the rotation is exact arithmetic on table values
    cos, sin = vectors["rope_tab_cos"], vectors["rope_tab_sin"]
    rng = np.random.default_rng(2)
    for neox in (False, True):
        for heads, hd, rot in [(10, 64, 64), (2, 256, 64)]:      # batched 10 heads (main.cpp:1692-1761); partial
            x = rng.standard_normal((heads, hd)).astype(np.float32)
            want = oracle.rope_apply(x, heads, hd, rot, cos[5, :rot // 2], sin[5, :rot // 2], neox)
            got = x.copy()
            assert backend.rope_batched(got, heads, hd, 5, 1.0, 500000.0, rot, cos[5, :rot // 2].copy(), sin[5, :rot // 2].copy(), neox) == Status.OK
            assert np.allclose(got, want, rtol=1e-6, atol=1e-7)


def test_f32_matmul_and_bf16_entry(backend, oracle):
    # A = B = 1 -> C == K (src/cli/main.cpp:809-825, 1060-1090), including M = 1 and 16
    for M, N, K in [(1, 256, 256), (16, 256, 512), (256, 256, 256), (33, 70, 129)]:
        A, B = np.ones((M, K), np.float32), np.ones((K, N), np.float32)
        C = np.zeros((M, N), np.float32)
        assert backend.mul_mat_q(A, B, C, M, N, K, 0) == Status.OK
        assert np.all(C == K)
    rng = np.random.default_rng(3)
    A = rng.standard_normal((40, 300)).astype(np.float32)
    B = rng.standard_normal((300, 50)).astype(np.float32)
    C = np.empty((40, 50), np.float32)
    assert backend.matmul_bf16(A, B, C, 40, 50, 300) == Status.OK
    # the reference gates its bf16 GEMM at rel 0.03 (main.cpp:1622); this path computes in fp32
    assert rel_l2(C, oracle.matmul_f32_kn(A, B)) < 1e-5


def test_invalid_params_return_status(backend):
    # tests/test_arch.cpp:192-221: null pointers / non-positive sizes -> INVALID_PARAM, nothing thrown
    x = np.zeros(4, np.float32)
    assert backend.rms_norm(None, None, 0, 1e-5) == Status.INVALID_PARAM
    assert backend.rms_norm(x, x, 0, 1e-5) == Status.INVALID_PARAM
    assert backend.silu(None, x, 4) == Status.INVALID_PARAM
    assert backend.gelu(x, None, 4) == Status.INVALID_PARAM
    assert backend.softmax(x, x, 0, 4) == Status.INVALID_PARAM
    assert backend.flash_attn(None, x, x, x, 1, 4, 1) == Status.INVALID_PARAM
    assert backend.mul_mat_q(None, x, x, 1, 1, 4, 0) == Status.INVALID_PARAM
    assert backend.mul_mat_q(x, x, x, 1, 1, 4, 77) == Status.INVALID_PARAM
    assert backend.rope(None, 4, 0, 1.0, 10000.0, 4) == Status.INVALID_PARAM
    assert backend.last_error() == Status.INVALID_PARAM
    assert backend.name() == "cuda_b200" and backend.is_available()
    y = np.empty(4, np.float32)
    assert backend.silu(x, y, 4) == Status.OK          # the handle stays usable after errors
