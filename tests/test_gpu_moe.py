"""Mixture-of-experts FFN (router, top-k, routed SwiGLU experts, sigmoid-gated shared expert) on device
pointers vs the CPU oracle's restatement of src/cli/main.cpp:3110-3193.

The chosen expert ids must match exactly (random logits: no near ties); weights to 1e-6; the output
to the GEMV tolerance (fp32 summation order / int8-limb activations): rel-L2 <= 2e-5."""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from ggnpu_b200.testing import synth as S
from ggnpu_b200.backend import Status

pytestmark = pytest.mark.gpu


def q(shape, t, seed, scale=0.05):
    g = torch.Generator().manual_seed(seed)
    return S.quantize(torch.randn(*shape, generator=g) * scale, t).numpy()


CASES = [
    # hidden, eff, n_expert, top_k, gate/up type, down type, shared eff (0: none), shared-gate vector
    (256, 256, 8, 2, S.Q4_K, S.Q6_K, 0, False),
    (512, 256, 64, 8, S.Q4_K, S.Q6_K, 512, True),
    (2048, 512, 32, 8, S.Q4_K, S.Q6_K, 512, True),     # the qwen35moe expert shapes (32 of its 256 experts)
    (256, 512, 256, 8, S.Q6_K, S.Q4_K, 256, False),    # 256 experts through the router; shared expert without a gate
]


@pytest.mark.parametrize("case", CASES)
def test_moe_ffn_matches_oracle(backend, oracle, case):
    H, eff, nE, k, tgu, td, eff_sh, with_gate = case
    ge, ue, de = q((nE * eff, H), tgu, 1), q((nE * eff, H), tgu, 2), q((nE * H, eff), td, 3)
    rng = np.random.default_rng(sum(case[:4]))
    router = (0.05 * rng.standard_normal((nE, H))).astype(np.float32)       # logits O(1), as a trained router's
    x = rng.standard_normal(H).astype(np.float32)
    resid = rng.standard_normal(H).astype(np.float32)
    shared = None
    sgi = None
    if eff_sh:
        sg, su, sd = q((eff_sh, H), tgu, 4), q((eff_sh, H), tgu, 5), q((H, eff_sh), td, 6)
        shared = (sg, su, tgu, sd, td, eff_sh)
        sgi = (0.05 * rng.standard_normal(H)).astype(np.float32) if with_gate else None
    want, ids, w = oracle.moe_ffn(x, router, k, eff, ge, ue, tgu, de, td, shared=shared, sh_gate_inp=sgi)

    dev = torch.device("cuda:0")
    up = backend.upload_weight
    hg, hu, hd = up(tgu, ge, nE * eff, H), up(tgu, ue, nE * eff, H), up(td, de, nE * H, eff)
    hs = [up(tgu, sg, eff_sh, H), up(tgu, su, eff_sh, H), up(td, sd, H, eff_sh)] if eff_sh else [None, None, None]
    dx, dr, drt = torch.from_numpy(x).to(dev), torch.from_numpy(resid).to(dev), torch.from_numpy(router).to(dev)
    dgi = torch.from_numpy(sgi).to(dev) if sgi is not None else None
    dy = torch.full((H,), float("nan"), device=dev)
    dsel = torch.full((k,), -1, device=dev, dtype=torch.int32)
    dw = torch.zeros(k + 1, device=dev)
    torch.cuda.synchronize()
    for with_resid in (False, True):
        st = backend.moe_ffn_device(x=dx.data_ptr(), resid=dr.data_ptr() if with_resid else None, y=dy.data_ptr(), router=drt.data_ptr(),
                                    gate_exps=hg, up_exps=hu, down_exps=hd, sh_gate=hs[0], sh_up=hs[1], sh_down=hs[2],
                                    sh_gate_inp=dgi.data_ptr() if dgi is not None else None, hidden=H, eff=eff, eff_sh=eff_sh,
                                    n_expert=nE, top_k=k, sel_out=dsel.data_ptr(), w_out=dw.data_ptr())
        assert st == Status.OK, backend.last_error_message()
        backend.sync()
        assert np.array_equal(dsel.cpu().numpy(), ids), (dsel.cpu().numpy(), ids)
        got_w = dw.cpu().numpy()
        assert np.allclose(got_w[:k], w[:k], rtol=2e-5, atol=1e-7)       # exp() of logits summed in another order
        if eff_sh:
            assert abs(got_w[k] - w[k]) <= 1e-6
        ref = want + (resid if with_resid else 0.0)
        assert rel_l2(dy.cpu().numpy(), ref) <= 2e-5, (case, with_resid, rel_l2(dy.cpu().numpy(), ref))
    for hw in (hg, hu, hd, *hs):
        if hw is not None:
            backend.free_weight(hw)


def test_moe_argument_errors(backend):
    dev = torch.device("cuda:0")
    t = torch.zeros(256, device=dev)
    w = backend.upload_weight(S.Q4_K, q((512, 256), S.Q4_K, 9), 512, 256)
    d = backend.upload_weight(S.Q4_K, q((512, 256), S.Q4_K, 9), 512, 256)
    base = dict(x=t.data_ptr(), resid=None, y=t.data_ptr(), router=t.data_ptr(), gate_exps=w, up_exps=w, down_exps=d, sh_gate=None,
                sh_up=None, sh_down=None, sh_gate_inp=None, hidden=256, eff=256, eff_sh=0, n_expert=2, top_k=1, sel_out=None, w_out=None)
    assert backend.moe_ffn_device(**dict(base, top_k=3)) == Status.INVALID_PARAM          # more than n_expert
    assert backend.moe_ffn_device(**dict(base, n_expert=3)) == Status.INVALID_PARAM       # tensors do not hold 3 experts
    assert backend.moe_ffn_device(**dict(base, x=None)) == Status.INVALID_PARAM
    assert backend.moe_ffn_device(**dict(base, hidden=128)) == Status.INVALID_PARAM
    backend.free_weight(w)
    backend.free_weight(d)


def test_moe_nan_input_returns_normally(backend):
    """An x that holds a NaN makes every router logit NaN, so no expert wins a comparison.  The call must
    still return OK with valid expert ids (the NaN travels through the weights into y) and leave the
    device usable, as the argmax path does (src/cli/main.cpp:3128-3135 has no guard either; it sorts NaNs
    into some order and carries on)."""
    H, eff, nE, k = 256, 256, 8, 2
    ge, ue, de = q((nE * eff, H), S.Q4_K, 1), q((nE * eff, H), S.Q4_K, 2), q((nE * H, eff), S.Q6_K, 3)
    dev = torch.device("cuda:0")
    hg, hu, hd = (backend.upload_weight(S.Q4_K, ge, nE * eff, H), backend.upload_weight(S.Q4_K, ue, nE * eff, H),
                  backend.upload_weight(S.Q6_K, de, nE * H, eff))
    x = torch.randn(H, device=dev)
    x[7] = float("nan")
    router = torch.randn(nE, H, device=dev) * 0.05
    y = torch.zeros(H, device=dev)
    dsel = torch.full((k,), -7, device=dev, dtype=torch.int32)
    dw = torch.zeros(k + 1, device=dev)
    st = backend.moe_ffn_device(x=x.data_ptr(), resid=None, y=y.data_ptr(), router=router.data_ptr(), gate_exps=hg, up_exps=hu,
                                down_exps=hd, sh_gate=None, sh_up=None, sh_down=None, sh_gate_inp=None, hidden=H, eff=eff, eff_sh=0,
                                n_expert=nE, top_k=k, sel_out=dsel.data_ptr(), w_out=dw.data_ptr())
    assert st == Status.OK, backend.last_error_message()
    backend.sync()
    ids = dsel.cpu().numpy()
    assert ((ids >= 0) & (ids < nE)).all() and len(set(ids.tolist())) == k, ids
    # the device still works afterwards
    x2 = torch.randn(H, device=dev)
    st = backend.moe_ffn_device(x=x2.data_ptr(), resid=None, y=y.data_ptr(), router=router.data_ptr(), gate_exps=hg, up_exps=hu,
                                down_exps=hd, sh_gate=None, sh_up=None, sh_down=None, sh_gate_inp=None, hidden=H, eff=eff, eff_sh=0,
                                n_expert=nE, top_k=k, sel_out=dsel.data_ptr(), w_out=dw.data_ptr())
    assert st == Status.OK
    backend.sync()
    assert torch.isfinite(y).all()
    for hw in (hg, hu, hd):
        backend.free_weight(hw)
