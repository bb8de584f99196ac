"""Gated DeltaNet step (conv + SiLU with rolling state, L2-normed q / k, gated delta-rule recurrence,
gated RMS norm) on device pointers vs the CPU oracle's restatement of src/cli/main.cpp:2925-3023, over
several consecutive tokens so that both states are carried.

Tolerance: sums run in another order (row groups / block reductions): output and states rel-L2 <= 2e-5."""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from ggnpu_b200.backend import Status

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(2, 4, 64, 4), (16, 32, 128, 4), (3, 6, 128, 2)])     # (n_khead, n_vhead, sk, conv_k); the middle one is qwen35moe's
def test_deltanet_steps_match_oracle(backend, oracle, shape):
    nK, nV, sk, ck = shape
    cd = 2 * nK * sk + nV * sk
    rng = np.random.default_rng(sum(shape))
    conv_w = (0.3 * rng.standard_normal((cd, ck))).astype(np.float32)
    ssm_a = (-np.exp(0.5 * rng.standard_normal(nV))).astype(np.float32)
    dt_bias = rng.standard_normal(nV).astype(np.float32)
    ssm_norm = (1 + 0.1 * rng.standard_normal(sk)).astype(np.float32)
    cs = np.zeros((ck - 1, cd), np.float32)
    S = np.zeros((nV, sk, sk), np.float32)
    dev = torch.device("cuda:0")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev)
    d_conv_w, d_a, d_dt, d_norm, d_cs, d_S = t(conv_w), t(ssm_a), t(dt_bias), t(ssm_norm), t(cs), t(S)
    d_out = torch.empty(nV * sk, device=dev)
    for step in range(5):
        mixed = rng.standard_normal(cd).astype(np.float32)
        z = rng.standard_normal(nV * sk).astype(np.float32)
        araw = (rng.standard_normal(nV) + (25.0 if step == 3 else 0.0)).astype(np.float32)       # step 3: the softplus(a > 20) branch
        braw = rng.standard_normal(nV).astype(np.float32)
        want = oracle.deltanet_step(mixed, z, araw, braw, conv_w, ssm_a, dt_bias, ssm_norm, cs, S, nK, nV, sk, ck, 1e-6)
        dm, dz, da, db = t(mixed), t(z), t(araw), t(braw)
        torch.cuda.synchronize()
        st = backend.deltanet_step_device(mixed=dm.data_ptr(), zgate=dz.data_ptr(), araw=da.data_ptr(), braw=db.data_ptr(),
                                          conv_w=d_conv_w.data_ptr(), ssm_a=d_a.data_ptr(), dt_bias=d_dt.data_ptr(),
                                          ssm_norm=d_norm.data_ptr(), conv_state=d_cs.data_ptr(), rec_state=d_S.data_ptr(),
                                          out=d_out.data_ptr(), n_khead=nK, n_vhead=nV, sk=sk, conv_k=ck, rms_eps=1e-6)
        assert st == Status.OK, backend.last_error_message()
        backend.sync()
        assert rel_l2(d_out.cpu().numpy(), want) <= 2e-5, (shape, step, rel_l2(d_out.cpu().numpy(), want))
        assert np.array_equal(d_cs.cpu().numpy(), cs)                       # the rolled conv inputs are copies
        assert rel_l2(d_S.cpu().numpy(), S) <= 2e-5


def test_deltanet_argument_errors(backend):
    z = torch.zeros(16, device="cuda:0").data_ptr()
    ok = dict(mixed=z, zgate=z, araw=z, braw=z, conv_w=z, ssm_a=z, dt_bias=z, ssm_norm=z, conv_state=z, rec_state=z, out=z,
              n_khead=1, n_vhead=1, sk=64, conv_k=4, rms_eps=1e-6)
    assert backend.deltanet_step_device(**dict(ok, sk=96)) == Status.INVALID_PARAM
    assert backend.deltanet_step_device(**dict(ok, out=None)) == Status.INVALID_PARAM
    assert backend.deltanet_step_device(**dict(ok, conv_k=0)) == Status.INVALID_PARAM
