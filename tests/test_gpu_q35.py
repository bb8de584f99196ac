"""The device-resident qwen35moe decoder (Gated DeltaNet layers, gated full-attention layer, mixture-of-experts
FFN; src/cli/main.cpp:2859-3232) against the CPU oracle's restatement of that forward -- which is itself held to
the unmodified reference CLI on the same synthetic models (tests/test_oracle_pins.py) -- and against the CLI's
recorded top-10 logits and greedy stream directly (tests/golden/ref_cli.npz).

Tolerances as for the generic model: logits max-abs <= 0.15 and <= 2 % of the oracle's logit range (bf16 KV
cache, reordered fp32 sums, int8-limb activations), greedy tokens equal wherever the oracle's top-1 margin
exceeds twice the measured error; the recurrent state to 1e-4 relative (5e-3 behind a bf16-KV attention layer)."""
import numpy as np
import pytest

from conftest import rel_l2
from ggnpu_b200.testing import synth as S

pytestmark = pytest.mark.gpu

CASES = {"qwen35moe": dict(), "qwen35moe_sk128": dict(sk=128, seed=77)}


def logits_ok(got, want):
    err = np.abs(got - want).max()
    rng = want.max() - want.min()
    assert err <= 0.15 and err <= 0.02 * rng, (err, rng)
    return err


@pytest.mark.parametrize("name", list(CASES))
def test_q35_prefill_decode_match_oracle_and_reference_cli(backend, oracle, cli_vectors, name):
    from ggnpu_b200.backend import Q35Model
    from oracle.binding import OracleQ35Model
    cfg = S.tiny_q35_config(**CASES[name])
    synth = S.build_q35_model(cfg)
    om = OracleQ35Model(oracle, synth)
    gm = Q35Model(backend, cfg, synth.tensors)
    ids = cli_vectors[f"{name}_prompt"]
    want = om.feed(ids)
    got, nxt = gm.prefill(ids, 0)
    err = logits_ok(got, want)
    # the reference CLI's own numbers
    top_ids, top_l = cli_vectors[f"{name}_top_ids"], cli_vectors[f"{name}_top_logits"]
    assert np.abs(got[top_ids] - top_l).max() <= 0.02 * (want.max() - want.min())
    if top_l[0] - top_l[1] > 2 * err:
        assert nxt == top_ids[0]
    # recurrent state of the first DeltaNet layer after the prompt
    assert rel_l2(gm.rec_state(0), om.rec_state(0)) <= 1e-4
    greedy = list(cli_vectors[f"{name}_greedy"])
    tok, pos = oracle.argmax_first(want), len(ids)
    assert tok == greedy[0]
    for step in range(len(greedy) - 1):
        want = om.forward(tok, pos)
        got, nxt = gm.decode(tok, pos)
        err = logits_ok(got, want)
        assert nxt == int(np.argmax(got))
        srt = np.sort(want)
        nt = oracle.argmax_first(want)
        assert nt == greedy[step + 1]
        if srt[-1] - srt[-2] > 2 * err:
            assert nxt == nt
        tok, pos = nt, pos + 1
    assert gm.decode_bytes(pos) > 0
    gm.close()


def test_q35_longer_sequence_and_device_feedback(backend, oracle):
    """40 tokens through a model with two attention layers (the KV cache crosses no page but the attention
    splits see growing contexts), states carried across all of them; then the device-feedback loop must produce
    the ids that stepping from the host produces, and a reset must reproduce the first run."""
    from ggnpu_b200.backend import Q35Model
    from oracle.binding import OracleQ35Model
    cfg = S.tiny_q35_config(n_layer=8, seed=9, ctx=128, top_k=3)
    synth = S.build_q35_model(cfg)
    om = OracleQ35Model(oracle, synth)
    gm = Q35Model(backend, cfg, synth.tensors)
    ids = np.random.default_rng(5).integers(0, cfg.vocab, 40).astype(np.int32)
    want = om.feed(ids)
    got, first = gm.prefill(ids, 0)
    logits_ok(got, want)
    # layer 0 sees only the embedding; layer 6 sits behind an attention layer whose KV cache is bf16 (2^-9 per element)
    assert rel_l2(gm.rec_state(0), om.rec_state(0)) <= 1e-4
    assert rel_l2(gm.rec_state(6), om.rec_state(6)) <= 5e-3
    host, tok = [], first
    for i in range(8):
        _, tok = gm.decode(tok, 40 + i)
        host.append(tok)
    gm.reset()
    got2, first2 = gm.prefill(ids, 0)
    assert first2 == first and np.array_equal(got2, got)          # same kernels, same order: bit-identical
    dev = gm.generate(first, 40, 8)
    assert list(dev) == host
    gm.close()


def test_q35_argument_errors(backend):
    from ggnpu_b200.backend import BackendError, Q35Model, Status
    cfg = S.tiny_q35_config(n_layer=4, seed=2)
    synth = S.build_q35_model(cfg)
    missing = dict(synth.tensors)
    del missing["blk.0.ssm_out.weight"]
    with pytest.raises(BackendError) as e:
        Q35Model(backend, cfg, missing)
    assert e.value.status == Status.INVALID_PARAM
    gm = Q35Model(backend, cfg, synth.tensors)
    with pytest.raises(BackendError):
        gm.decode(cfg.vocab, 0)
    with pytest.raises(BackendError):
        gm.prefill(np.zeros(cfg.ctx + 1, np.int32), 0)
    gm.close()
