"""Regenerate tests/golden/*.npz from the reference's own compiled code.

Run where the reference tree is available:

    make -C oracle ref REF=/path/to/ggnpu && python tests/golden/make_golden.py [--cli-only | --grid-only | --cli-cases a,b]

Every array stored here is an INPUT (seeded random bytes / floats) or an OUTPUT of
the reference's functions on that input (oracle/_ref/libggnpu_ref.so, built from
the unmodified reference sources).  Tests then hold the C restatement and the
CUDA path to these outputs on machines where the reference tree is absent.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from ggnpu_b200.testing import synth as S  # noqa: E402
from oracle.binding import Ref, run_ref_cli  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = Ref()
    out = {}
    # 1. block decoders: 24 random blocks per format + 8 blocks from the quantiser
    for t in S.QUANT_TYPES:
        be, bb = S.BLOCK[t]
        blk = S.random_blocks(t, 24, seed=100 + t)
        import torch
        g = torch.Generator().manual_seed(200 + t)
        x = torch.randn(2, 4 * be if be == 256 else 32 * 4, generator=g) * 0.02
        qb = S.quantize(x, t).numpy().reshape(-1, bb)
        allb = np.concatenate([blk, qb])
        out[f"dq_in_{t}"] = allb
        out[f"dq_out_{t}"] = ref.dequant_blocks(t, allb)
    # fp16 / bf16 scalar conversions over every 16-bit pattern (finite or not)
    h = np.arange(65536, dtype=np.uint32)
    out["f16_all"] = np.array([ref.lib.ref_f16_to_f32(int(v)) for v in h], dtype=np.float32).view(np.uint32)
    out["kq_f16_all"] = np.array([ref.lib.ref_kquant_fp16_to_f32(int(v)) for v in h], dtype=np.float32).view(np.uint32)
    rng = np.random.default_rng(5)
    fl = rng.standard_normal(4096).astype(np.float32) * np.float32(10.0) ** rng.integers(-6, 6, 4096).astype(np.float32)
    out["bf16_in"] = fl
    out["bf16_out"] = np.array([ref.lib.ref_f32_to_bf16(float(v)) for v in fl], dtype=np.uint16)
    # 2. operators of the CPU backend
    x = (rng.random(2048).astype(np.float32) - 0.5)
    w = (1.0 + 0.1 * rng.standard_normal(2048)).astype(np.float32)
    out["rms_x"], out["rms_w"] = x, w
    out["rms_y"] = ref.rms_norm(x, 1e-5, w)[1]
    out["silu_y"] = ref.silu(x)[1]
    out["gelu_y"] = ref.gelu(x)[1]
    sm = rng.standard_normal((4, 40)).astype(np.float32)
    out["softmax_x"], out["softmax_y"] = sm, ref.softmax(sm)[1]
    Q = rng.standard_normal((4, 64)).astype(np.float32)
    K = rng.standard_normal((4, 40, 64)).astype(np.float32)
    V = rng.standard_normal((4, 40, 64)).astype(np.float32)
    out["attn_q"], out["attn_k"], out["attn_v"] = Q, K, V
    out["attn_full"] = ref.flash_attn(Q, K, V, -1)[1]
    out["attn_causal17"] = ref.flash_attn(Q, K, V, 17)[1]
    r = rng.standard_normal(64).astype(np.float32)
    out["rope_x"] = r
    out["rope_y"] = ref.rope(r, 64, 5, 1.0, 10000.0, 64)[1]
    c, s = ref.rope_table(48, 64, 1.0, 500000.0)
    out["rope_tab_cos"], out["rope_tab_sin"] = c, s
    ff = (1.0 + rng.random(32)).astype(np.float32)
    c2, s2 = ref.rope_table(16, 64, 1.0, 1e6, ff)
    out["rope_ff"], out["rope_tab_cos_ff"], out["rope_tab_sin_ff"] = ff, c2, s2
    # 3. matmul: the exact path for every format, and the CPU backend's K-quant path
    A = rng.standard_normal((3, 512)).astype(np.float32)
    out["mm_A"] = A
    for t in S.QUANT_TYPES + [S.BF16, S.F16]:
        import torch
        g = torch.Generator().manual_seed(300 + t)
        wq = S.quantize(torch.randn(24, 512, generator=g) * 0.02, t).numpy()
        out[f"mm_W_{t}"] = wq
        out[f"mm_exact_{t}"] = ref.matmul_exact(A, wq, t, 24, 512)
        if t in (S.Q4_K, S.Q6_K):
            out[f"mm_cpuref_{t}"] = ref.mul_mat_q(A, wq, t, 24, 512)[1]
    np.savez_compressed(os.path.join(HERE, "ref_vectors.npz"), **out)

    print("wrote", os.path.join(HERE, "ref_vectors.npz"))


def cli_cases():
    """name -> (config, builder, prompt length, greedy tokens).  The same table drives the tests."""
    return {
        "llama": (S.tiny_config(seed=11), S.build_model, 7, 6),
        "qwen2": (S.tiny_config(arch="qwen2", qkv_bias=True, wtype=S.Q8_0, wtype_alt=S.Q8_0, seed=12, rope_base=1e6, tied=False),
                  S.build_model, 7, 6),
        # the full Llama-3.2-1B shape (16 layers, hidden 2048, vocab 128256, Q4_K / Q6_K, tied embeddings)
        "llama1b": (S.LLAMA_1B, S.build_model, 8, 4),
        # qwen35moe: 3 Gated DeltaNet layers + 1 gated full-attention layer, 8 experts top-2 + shared expert
        "qwen35moe": (S.tiny_q35_config(), S.build_q35_model, 7, 6),
        "qwen35moe_sk128": (S.tiny_q35_config(sk=128, seed=77), S.build_q35_model, 9, 6),
        # lfm2: gated short-convolution layers around GQA attention layers with per-head QK-norm; tied output,
        # final norm stored as token_embd_norm
        "lfm2": (S.tiny_config(**S.LFM2_CASES["lfm2"]), S.build_model, 7, 6),
        "lfm2_q8": (S.tiny_config(**S.LFM2_CASES["lfm2_q8"]), S.build_model, 9, 6),
    }


# temperature-sampled streams: name -> [(temp, seed)]
SAMPLED_CASES = {"llama": [(0.8, 42), (1.5, 7)], "qwen2": [(0.7, 123456789012)]}
N_SAMPLED = 12


def cli_vectors(only=None):
    """End to end: the unmodified reference CLI (exact fp32 matmul path) on seeded synthetic models:
    top-10 logits after the prompt and the greedy continuation -> ref_cli.npz.  only: names of the cases to
    (re)generate; the other cases keep the arrays the file already holds."""
    e2e = {}
    if only:
        with np.load(os.path.join(HERE, "ref_cli.npz")) as old:
            e2e = {k: old[k] for k in old.files}
    for name, (cfg, builder, n_prompt, n_gen) in cli_cases().items():
        if only and name not in only:
            continue
        m = builder(cfg)
        path = f"/tmp/ggb_golden_{name}.gguf"
        m.write(path)
        ids = np.random.default_rng(42).integers(0, cfg.vocab, n_prompt)
        r1 = run_ref_cli(path, S.prompt_text(ids), 0, ctx=cfg.ctx, bench_logits=True)
        top = []
        for line in (r1.stdout + r1.stderr).splitlines():
            line = line.strip()
            if line.startswith("top") and "id=" in line:
                tid = int(line.split("id=")[1].split()[0])
                lg = float(line.split("logit=")[1].split()[0])
                top.append((tid, lg))
        assert len(top) == 10, (r1.stdout, r1.stderr)
        r2 = run_ref_cli(path, S.prompt_text(ids), n_gen, ctx=cfg.ctx)
        gen = S.text_ids(r2.stdout)
        assert len(gen) == n_gen, (r2.stdout, r2.stderr)
        e2e[f"{name}_prompt"] = ids.astype(np.int32)
        e2e[f"{name}_top_ids"] = np.array([t for t, _ in top], dtype=np.int32)
        e2e[f"{name}_top_logits"] = np.array([v for _, v in top], dtype=np.float32)
        e2e[f"{name}_greedy"] = np.array(gen, dtype=np.int32)
        if name in SAMPLED_CASES:
            # temperature sampling (sample_token, src/cli/main.cpp:839-864): the stream the CLI prints for a seed
            for temp, seed in SAMPLED_CASES[name]:
                r3 = run_ref_cli(path, S.prompt_text(ids), N_SAMPLED, ctx=cfg.ctx, temp=temp, seed=seed)
                smp = S.text_ids(r3.stdout)
                assert len(smp) == N_SAMPLED, (r3.stdout, r3.stderr)
                e2e[f"{name}_sampled_t{temp}_s{seed}"] = np.array(smp, dtype=np.int32)
                print(name, "sampled", temp, seed, smp)
        os.remove(path)
        print(name, "top-1", top[0], "greedy", gen)
    np.savez_compressed(os.path.join(HERE, "ref_cli.npz"), **e2e)
    print("wrote", os.path.join(HERE, "ref_cli.npz"))


def grid_vectors(ref=None):
    """Grid-coded formats (IQ1 / IQ2 / IQ3): outputs of the reference's block decoders
    (src/quant/iquants.cpp:37-203) and of its exact matmul on random block bytes -> ref_grid_vectors.npz.
    There is no quantiser for these formats here, so random bytes (finite scales) stand in for weights."""
    ref = ref or Ref()
    out = {}
    A = np.random.default_rng(21).standard_normal((3, 512)).astype(np.float32)
    out["mm_A"] = A
    for t in S.GRID_TYPES:
        blk = S.random_blocks(t, 32, seed=100 + t)
        out[f"dq_in_{t}"] = blk
        out[f"dq_out_{t}"] = ref.dequant_blocks(t, blk)
        w = S.random_blocks(t, 8 * 2, seed=300 + t)               # 8 rows x 512
        out[f"mm_W_{t}"] = w
        out[f"mm_exact_{t}"] = ref.matmul_exact(A, w, t, 8, 512)
    np.savez_compressed(os.path.join(HERE, "ref_grid_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "ref_grid_vectors.npz"))


if __name__ == "__main__":
    if "--grid-only" in sys.argv:
        grid_vectors()
    elif "--cli-only" in sys.argv:
        cli_vectors()
    elif "--cli-cases" in sys.argv:                      # --cli-cases lfm2,lfm2_q8: only these, the rest kept
        cli_vectors(only=sys.argv[sys.argv.index("--cli-cases") + 1].split(","))
    else:
        main()
        cli_vectors()
        grid_vectors()
