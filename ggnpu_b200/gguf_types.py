"""GGUF tensor type ids, block geometry and model descriptions shared by the host-side code (backend.py, tp.py) and
by the test fixtures (ggnpu_b200/testing)."""
from __future__ import annotations

from dataclasses import dataclass

# ggml type ids (include/ggnpu/tensor.h:11-42)
F32, F16, Q4_0, Q4_1, Q8_0 = 0, 1, 2, 3, 8
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 10, 11, 12, 13, 14
IQ4_NL, IQ4_XS, BF16 = 20, 23, 30
# grid-coded formats: decoded everywhere, never produced by quantize() (tests use random block bytes)
IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ3_S, IQ2_S, IQ1_M = 16, 17, 18, 19, 21, 22, 29
GRID_TYPES = [IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S, IQ1_S, IQ1_M]

TYPE_NAMES = {F32: "F32", F16: "F16", Q4_0: "Q4_0", Q4_1: "Q4_1", Q8_0: "Q8_0", Q2_K: "Q2_K", Q3_K: "Q3_K",
              Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", IQ4_NL: "IQ4_NL", IQ4_XS: "IQ4_XS", BF16: "BF16",
              IQ2_XXS: "IQ2_XXS", IQ2_XS: "IQ2_XS", IQ2_S: "IQ2_S", IQ3_XXS: "IQ3_XXS", IQ3_S: "IQ3_S",
              IQ1_S: "IQ1_S", IQ1_M: "IQ1_M"}
TYPE_IDS = {v: k for k, v in TYPE_NAMES.items()}
# (elements per block, bytes per block): src/gguf/tensor.cpp:18-38
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), Q8_0: (32, 34),
         Q2_K: (256, 84), Q3_K: (256, 110), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210),
         IQ4_NL: (32, 18), IQ4_XS: (256, 136),
         # include/ggnpu/quant/iquants.h:40-46
         IQ2_XXS: (256, 66), IQ2_XS: (256, 74), IQ2_S: (256, 82), IQ3_XXS: (256, 98), IQ3_S: (256, 110),
         IQ1_S: (256, 50), IQ1_M: (256, 56)}
QUANT_TYPES = [Q4_0, Q4_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ4_XS]
IQ4_CODEBOOK = [-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113]


def row_bytes(type_id: int, k: int) -> int:
    be, bb = BLOCK[type_id]
    return (k + be - 1) // be * bb


@dataclass
class ModelConfig:
    arch: str = "llama"
    n_layer: int = 16
    hidden: int = 2048
    n_head: int = 32
    n_kv: int = 8
    head_dim: int = 64
    ffn: int = 8192
    vocab: int = 128256
    ctx: int = 2048
    rms_eps: float = 1e-5
    rope_base: float = 500000.0
    qkv_bias: bool = False
    tied: bool = True
    wtype: int = Q4_K            # every matrix ...
    wtype_alt: int = Q6_K        # ... except attn_v and ffn_down ("Q4_K_M-style")
    out_type: int | None = None  # output.weight type when not tied
    norm_jitter: float = 0.1     # norm gammas = 1 + jitter*N(0,1)
    seed: int = 1234
    qk_norm: bool = False        # per-head attn_q_norm / attn_k_norm (qwen3, lfm2)
    # lfm2 (src/cli/main.cpp:2145-2167): layers listed here carry shortconv.* instead of attn_*; taps = shortconv.l_cache
    conv_layers: tuple = ()
    d_conv: int = 3


# The benchmark shapes (model dims only; weights are random-init).
LLAMA_1B = ModelConfig()
QWEN25_1P5B = ModelConfig(arch="qwen2", n_layer=28, hidden=1536, n_head=12, n_kv=2, head_dim=128, ffn=8960,
                          vocab=151936, rope_base=1e6, qkv_bias=True, tied=True, wtype=Q8_0, wtype_alt=Q8_0,
                          rms_eps=1e-6)
# an lfm2 shape of about 1.2 B parameters: 10 gated short-convolution layers (3 taps) around 6 GQA attention layers
LFM2_1P2B = ModelConfig(arch="lfm2", n_layer=16, hidden=2048, n_head=32, n_kv=8, head_dim=64, ffn=8192, vocab=65536,
                        rope_base=1e6, qk_norm=True, conv_layers=(0, 1, 3, 4, 6, 7, 9, 11, 13, 15), d_conv=3)
LLAMA_8B = ModelConfig(n_layer=32, hidden=4096, n_head=32, n_kv=8, head_dim=128, ffn=14336, vocab=128256,
                       tied=False, out_type=Q6_K)


@dataclass
class Qwen35MoeConfig:
    """qwen35moe: Gated DeltaNet layers with a gated full-attention layer every `attn_every` layers, MoE FFN in
    every layer (metadata keys and tensor names as src/cli/main.cpp:2181-2218, 2894-3193 reads them)."""
    arch: str = "qwen35moe"
    n_layer: int = 40
    hidden: int = 2048
    n_head: int = 16            # full-attention query heads
    n_kv: int = 2
    head_dim: int = 256         # attention.key_length
    rope_dim: int = 64          # rope.dimension_count: rotated leading dims of each head
    rope_base: float = 1e7
    conv_k: int = 4
    sk: int = 128               # ssm.state_size: DeltaNet head size (keys and values)
    n_vhead: int = 32           # ssm.inner_size / sk
    n_khead: int = 16           # ssm.group_count
    n_expert: int = 256
    top_k: int = 8
    eff: int = 512              # expert_feed_forward_length (routed and shared experts)
    attn_every: int = 4         # layers L with (L + 1) % attn_every == 0 are full attention
    vocab: int = 248320
    ctx: int = 2048
    rms_eps: float = 1e-6
    tied: bool = True
    wtype: int = Q4_K
    wtype_alt: int = Q6_K       # attention output and expert down projections
    norm_jitter: float = 0.1
    seed: int = 4321

    @property
    def ffn(self) -> int:       # the loader wants feed_forward_length; the MoE path never uses it
        return self.eff

    def is_ssm(self, layer: int) -> bool:
        return (layer + 1) % self.attn_every != 0


QWEN35MOE = Qwen35MoeConfig()
