"""The lfm2 branch (src/cli/main.cpp:2145-2167, 2680-2856) in the device-resident graph: gated short-convolution
layers (in_proj -> per-channel causal convolution with a carried state -> out_proj) around GQA attention layers with
per-head QK-norm, final norm from token_embd_norm, tied output.

Checked against the CPU oracle's restatement of the branch, which tests/test_oracle_pins.py holds to the unmodified
reference CLI's output on the same synthetic models, and against that output directly (tests/golden/ref_cli.npz).
Tolerances as tests/test_gpu_model.py: logits max-abs <= 0.15 and <= 2 % of the oracle's logit range (bf16 KV cache,
reordered sums); greedy tokens agree wherever the oracle's top-1 / top-2 margin exceeds twice the measured error.

Two rotations are covered: what the branch asks its backend for (split-half pairs at lfm2.rope.freq_base), and what the
reference's CPU backend does with that request (adjacent pairs at base 10000, cpu_ref.cpp:158-174), which is what the
CLI's recorded output contains."""
import numpy as np
import pytest

from ggnpu_b200.testing import synth as S

pytestmark = pytest.mark.gpu

CPU_ROPE = dict(rope_neox=0, rope_base=10000.0)


def logits_ok(got, want):
    err = np.abs(got - want).max()
    rng = want.max() - want.min()
    assert err <= 0.15 and err <= 0.02 * rng, (err, rng)
    return err


@pytest.mark.parametrize("name", list(S.LFM2_CASES))
@pytest.mark.parametrize("cpu_rope", [True, False])
def test_prefill_then_decode_matches_oracle(backend, oracle, name, cpu_rope):
    from ggnpu_b200.backend import Model
    from oracle.binding import OracleModel
    cfg = S.tiny_config(**S.LFM2_CASES[name])
    synth = S.build_model(cfg)
    om = OracleModel(oracle, synth, cpu_rope=cpu_rope)
    gm = Model(backend, cfg, synth.tensors, **(CPU_ROPE if cpu_rope else {}))
    ids = np.random.default_rng(42).integers(0, cfg.vocab, 9).astype(np.int32)
    want = om.forward(ids, 0)
    got, nxt = gm.prefill(ids, 0)                       # the rows of the chunk walk the convolution in order
    err = logits_ok(got, want)
    tok, pos = oracle.argmax_first(want), len(ids)
    srt = np.sort(want)
    if srt[-1] - srt[-2] > 2 * err:
        assert nxt == tok
    for _ in range(6):                                  # teacher-forced single-token steps (the captured graph)
        want = om.forward([tok], pos)
        got, nxt = gm.decode(tok, pos)
        err = logits_ok(got, want)
        t2 = oracle.argmax_first(want)
        srt = np.sort(want)
        if srt[-1] - srt[-2] > 2 * err:
            assert nxt == t2
        tok, pos = t2, pos + 1
    # a second sequence on the same objects: a call at position 0 starts from zero convolution states,
    # and token-by-token prompt processing (as the reference runs this branch) equals the chunk
    om.reset()
    ids2 = np.random.default_rng(7).integers(0, cfg.vocab, 5).astype(np.int32)
    want = om.forward(ids2, 0)
    for i, t in enumerate(ids2):
        got, _ = gm.decode(int(t), i)
    logits_ok(got, want)
    got_chunk, _ = gm.prefill(ids2, 0)
    logits_ok(got_chunk, want)
    assert np.abs(got_chunk - got).max() <= 5e-3
    gm.close()
    om.close()


@pytest.mark.parametrize("name", list(S.LFM2_CASES))
def test_long_prompt_chunk_on_the_tensor_core_gemm(backend, oracle, name):
    """40 prompt rows: in_proj / out_proj run the tcgen05 GEMM and the convolution walks 40 rows in one launch; a
    continuation of the prompt in a second call (position > 0) carries the state on."""
    from ggnpu_b200.backend import Model
    from oracle.binding import OracleModel
    cfg = S.tiny_config(**S.LFM2_CASES[name])
    synth = S.build_model(cfg)
    om = OracleModel(oracle, synth, cpu_rope=False)
    gm = Model(backend, cfg, synth.tensors)
    ids = np.random.default_rng(9).integers(0, cfg.vocab, 52).astype(np.int32)
    want = om.forward(ids[:40], 0)
    got, _ = gm.prefill(ids[:40], 0)
    logits_ok(got, want)
    want = om.forward(ids[40:], 40)
    got, _ = gm.prefill(ids[40:], 40)
    logits_ok(got, want)
    gm.close()
    om.close()


@pytest.mark.parametrize("name", list(S.LFM2_CASES))
def test_reference_cli_output(backend, cli_vectors, name):
    """The unmodified reference CLI's recorded top-10 logits after the prompt and its greedy continuation."""
    from ggnpu_b200.backend import Model
    cfg = S.tiny_config(**S.LFM2_CASES[name])
    synth = S.build_model(cfg)
    gm = Model(backend, cfg, synth.tensors, **CPU_ROPE)
    ids = cli_vectors[f"{name}_prompt"]
    logits, nxt = gm.prefill(ids, 0)
    top_ids, top_l = cli_vectors[f"{name}_top_ids"], cli_vectors[f"{name}_top_logits"]
    err = np.abs(logits[top_ids] - top_l).max()
    assert err <= 0.02 * (logits.max() - logits.min())
    if top_l[0] - top_l[1] > 2 * err:
        assert nxt == top_ids[0]
    # device-resident greedy loop against the CLI's stream, fed with the CLI's own first token
    greedy = cli_vectors[f"{name}_greedy"]
    dev = gm.generate(int(greedy[0]), len(ids), len(greedy) - 1)
    host, tok = [], int(greedy[0])
    gm.prefill(ids, 0)
    for i in range(len(greedy) - 1):
        lg, tok = gm.decode(tok, len(ids) + i)
        host.append(tok)
    assert list(dev) == host                            # graph replays with device feedback == host-stepped decode
    # where this model's margins are wide the stream is the CLI's
    if list(dev) != list(greedy[1:]):
        gm.prefill(ids, 0)
        tok = int(greedy[0])
        for i in range(len(greedy) - 1):
            lg, nx = gm.decode(tok, len(ids) + i)
            srt = np.sort(lg)
            assert nx == greedy[i + 1] or srt[-1] - srt[-2] <= 2 * max(err, 1e-3), (i, nx, greedy[i + 1])
            tok = int(greedy[i + 1])
    gm.close()


def test_sampled_generation_and_refusals(backend):
    """Temperature sampling runs on the same graph; what cannot work with a state inside the model is refused."""
    from ggnpu_b200.backend import Model
    cfg = S.tiny_config(**S.LFM2_CASES["lfm2"])
    synth = S.build_model(cfg)
    gm = Model(backend, cfg, synth.tensors)
    ids = np.random.default_rng(3).integers(0, cfg.vocab, 6).astype(np.int32)
    _, first = gm.prefill(ids, 0)
    a, seed_a = gm.generate_sampled(first, len(ids), 8, temp=0.9, seed=5)
    gm.prefill(ids, 0)
    b, seed_b = gm.generate_sampled(first, len(ids), 8, temp=0.9, seed=5)
    assert list(a) == list(b) and seed_a == seed_b      # same seed, same state: same stream
    hist = np.concatenate([ids, [first]]).astype(np.int32)
    with pytest.raises(Exception):
        gm.generate_spec(hist, len(ids), 4)             # a rejected draft cannot leave a recurrent state again
    _, nxt = gm.decode(int(first), len(ids))            # the handle stays usable after the refusal
    assert 0 <= nxt < cfg.vocab
    gm.close()
    with pytest.raises(Exception):
        Model(backend, cfg, synth.tensors, n_seq=2)     # one sequence only
    # a layer with both kinds of tensors, or with half of one, is refused
    bad = dict(synth.tensors)
    bad["blk.0.attn_q.weight"] = synth.tensors["blk.2.attn_q.weight"]
    with pytest.raises(Exception):
        Model(backend, cfg, bad)
