"""The drop-in check: the UNMODIFIED reference CLI (its own main(), loader, tokenizer, layer loop),
linked against ggnpu_b200/host/cuda_backend.cpp + libggb200.so instead of the NPU backend, generates
the same greedy stream as the CPU oracle.  The binary is built by `make -C oracle dropin` where the
reference tree is present and travels prebuilt (oracle/_ref/ggnpu_cuda_dropin)."""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT
from ggnpu_b200.testing import synth as S

pytestmark = pytest.mark.gpu

DROPIN = os.path.join(ROOT, "oracle", "_ref", "ggnpu_cuda_dropin")


@pytest.mark.parametrize("case", ["llama", "qwen2", "lfm2", "lfm2_q8"])
def test_unmodified_cli_on_cuda_backend(oracle, tmp_path, case):
    if not os.path.exists(DROPIN):
        pytest.skip("oracle/_ref/ggnpu_cuda_dropin not built (needs the reference tree at build time)")
    from oracle.binding import OracleModel
    # lfm2 (src/cli/main.cpp:2680-2856): the CLI's own branch drives rms_norm, rope_batched (split-half pairs at the model's
    # base, which this backend honours as the NPU backend does), mul_mat_q, flash_attn and silu of the C ABI
    kw = {"llama": dict(seed=11), "qwen2": dict(arch="qwen2", qkv_bias=True, wtype=S.Q8_0, wtype_alt=S.Q8_0, seed=12, rope_base=1e6, tied=False),
          **S.LFM2_CASES}[case]
    cfg = S.tiny_config(**kw)
    synth = S.build_model(cfg)
    path = str(tmp_path / "m.gguf")
    synth.write(path)
    ids = np.random.default_rng(42).integers(0, cfg.vocab, 7)
    n_gen = 6
    env = {k: v for k, v in os.environ.items() if not k.startswith("GGNPU_")}     # no CPU-matmul switches
    r = subprocess.run([DROPIN, "-m", path, "-p", S.prompt_text(ids), "-c", str(cfg.ctx), "--no-cache", "-n", str(n_gen),
                        "--temp", "0", "-v"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "Backend: cuda_b200" in r.stdout + r.stderr
    # generated code points appear after the "Generating:" marker
    tail = r.stdout.split("Generating:")[-1]
    got = S.text_ids(tail)[:n_gen]
    assert len(got) == n_gen, r.stdout[-1500:]
    # teacher-forced comparison with the oracle along the CLI's own stream
    om = OracleModel(oracle, synth, cpu_rope=False)      # lfm2: the rotation the branch asks its backend for
    logits = om.forward(ids, 0)
    pos = len(ids)
    for tok in got:
        srt = np.sort(logits)
        if srt[-1] - srt[-2] > 1e-3:        # fp32 summation-order differences are ~1e-6 on O(1) logits
            assert tok == oracle.argmax_first(logits)
        logits = om.forward([tok], pos)
        pos += 1


@pytest.mark.parametrize("kw", [dict(), dict(sk=128, seed=77)], ids=["sk64", "sk128"])
def test_unmodified_cli_qwen35moe_on_cuda_backend(oracle, tmp_path, kw):
    """The CLI's own qwen35moe branch (Gated DeltaNet layers, gated full attention, MoE FFN: src/cli/main.cpp:2859-3232)
    with every matmul, norm, attention and activation it hands to its backend served by the C ABI."""
    if not os.path.exists(DROPIN):
        pytest.skip("oracle/_ref/ggnpu_cuda_dropin not built (needs the reference tree at build time)")
    from oracle.binding import OracleQ35Model
    cfg = S.tiny_q35_config(**kw)
    synth = S.build_q35_model(cfg)
    path = str(tmp_path / "q35.gguf")
    synth.write(path)
    ids = np.random.default_rng(42).integers(0, cfg.vocab, 7)
    n_gen = 6
    env = {k: v for k, v in os.environ.items() if not k.startswith("GGNPU_")}
    r = subprocess.run([DROPIN, "-m", path, "-p", S.prompt_text(ids), "-c", str(cfg.ctx), "--no-cache", "-n", str(n_gen),
                        "--temp", "0", "-v"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "Backend: cuda_b200" in r.stdout + r.stderr
    got = S.text_ids(r.stdout.split("Generating:")[-1])[:n_gen]
    assert len(got) == n_gen, r.stdout[-1500:]
    om = OracleQ35Model(oracle, synth)
    for i, t in enumerate(ids):
        logits = om.forward(int(t), i)
    pos = len(ids)
    for tok in got:
        srt = np.sort(logits)
        if srt[-1] - srt[-2] > 1e-3:
            assert tok == oracle.argmax_first(logits)
        logits = om.forward(tok, pos)
        pos += 1
