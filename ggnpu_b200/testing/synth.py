"""Test and benchmark fixtures, not part of the product path.  Synthetic inputs for the ggnpu operator path: GGUF block quantisers, a GGUF
file writer and seeded random-init models of the benchmark shapes.

The reference (ggnpu) only *decodes* GGUF blocks; it has no float->block
quantiser.  These are simple round-to-nearest quantisers whose only contract is
that they emit valid blocks of each format (layouts as decoded by
include/ggnpu/quant/kquant.h:66-202, src/quant/q4_0.cpp:18-26,
src/quant/q4_1.cpp:20-29, src/quant/q8_0.cpp:19-25, src/quant/iq4_nl.cpp:24-31,
src/quant/iq4_xs.cpp:21-39).  All of them are vectorised torch code that runs on
CPU or CUDA; the block bytes they produce are what both the CUDA path and the
CPU checkers consume, so the quantiser itself is never part of a parity claim.
"""
from __future__ import annotations

import struct
import zlib
from dataclasses import dataclass, field

import numpy as np
import torch

from ..gguf_types import *  # noqa: F401,F403  (type ids, BLOCK, row_bytes, ModelConfig, Qwen35MoeConfig, the benchmark shapes)
from ..gguf_types import BLOCK, ModelConfig, Qwen35MoeConfig, row_bytes  # noqa: F401


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """[...]-shaped float -> [..., 2] uint8 (little-endian fp16)."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def _f16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).to(torch.float32)


def _safe_inv(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x != 0, 1.0 / x, torch.zeros_like(x))


def _nib(lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    return (lo.to(torch.uint8) | (hi.to(torch.uint8) << 4)).to(torch.uint8)


def _pack_k4_scales(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """8 six-bit scales + 8 six-bit mins -> 12 bytes (include/ggnpu/quant/kquant.h:56-64)."""
    sc = sc.to(torch.int32)
    mn = mn.to(torch.int32)
    b0 = sc[..., :4] | ((sc[..., 4:] >> 4) << 6)
    b1 = mn[..., :4] | ((mn[..., 4:] >> 4) << 6)
    b2 = (sc[..., 4:] & 15) | ((mn[..., 4:] & 15) << 4)
    return torch.cat([b0, b1, b2], dim=-1).to(torch.uint8)


def quantize(x: torch.Tensor, type_id: int) -> torch.Tensor:
    """x: float32 [N, K] (K a multiple of the block length) -> uint8 [N, row_bytes]."""
    assert x.dim() == 2
    n, k = x.shape
    be, bb = BLOCK[type_id]
    assert k % be == 0, f"K={k} is not a multiple of the {TYPE_NAMES[type_id]} block length {be}"
    x = x.to(torch.float32)
    if type_id == F32:
        return x.contiguous().view(torch.uint8).reshape(n, k * 4)
    if type_id == F16:
        return x.to(torch.float16).contiguous().view(torch.uint8).reshape(n, k * 2)
    if type_id == BF16:
        return x.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(n, k * 2)
    nb = k // be
    xb = x.reshape(n, nb, be)
    if type_id == Q8_0:
        d = _f16_round(xb.abs().amax(-1) / 127.0)
        q = torch.clamp(torch.round(xb * _safe_inv(d)[..., None]), -127, 127).to(torch.int8)
        out = torch.cat([_f16_bytes(d), q.view(torch.uint8)], dim=-1)
    elif type_id == Q4_0:
        d = _f16_round(xb.abs().amax(-1) / 7.0)
        q = torch.clamp(torch.round(xb * _safe_inv(d)[..., None]) + 8, 0, 15)
        out = torch.cat([_f16_bytes(d), _nib(q[..., :16], q[..., 16:])], dim=-1)
    elif type_id == Q4_1:
        mn = _f16_round(xb.amin(-1))
        d = _f16_round((xb.amax(-1) - mn) / 15.0)
        q = torch.clamp(torch.round((xb - mn[..., None]) * _safe_inv(d)[..., None]), 0, 15)
        out = torch.cat([_f16_bytes(d), _f16_bytes(mn), _nib(q[..., :16], q[..., 16:])], dim=-1)
    elif type_id == IQ4_NL:
        d = _f16_round(xb.abs().amax(-1) / 127.0)
        cb = torch.tensor(IQ4_CODEBOOK, dtype=torch.float32, device=x.device)
        idx = ((xb * _safe_inv(d)[..., None])[..., None] - cb).abs().argmin(-1)
        out = torch.cat([_f16_bytes(d), _nib(idx[..., :16], idx[..., 16:])], dim=-1)
    elif type_id == IQ4_XS:
        sub = xb.reshape(n, nb, 8, 32)
        s_amax = sub.abs().amax(-1) / 127.0                       # ideal per-32 scale
        d = _f16_round(s_amax.amax(-1) / 31.0)
        ls = torch.clamp(torch.round(s_amax * _safe_inv(d)[..., None]), 1, 31).to(torch.int32)   # ls-32 in [-31,31]
        dl = d[..., None] * ls
        cb = torch.tensor(IQ4_CODEBOOK, dtype=torch.float32, device=x.device)
        idx = ((sub * _safe_inv(dl)[..., None])[..., None] - cb).abs().argmin(-1)                # [n,nb,8,32]
        st = ls + 32
        sl = ((st[..., 0::2] & 15) | ((st[..., 1::2] & 15) << 4)).to(torch.uint8)                # [n,nb,4]
        shifts = torch.arange(8, device=x.device, dtype=torch.int32) * 2
        sh = ((st >> 4) << shifts).sum(-1).to(torch.int32)
        shb = torch.stack([sh & 255, sh >> 8], dim=-1).to(torch.uint8)
        qs = _nib(idx[..., :16], idx[..., 16:]).reshape(n, nb, 128)
        out = torch.cat([_f16_bytes(d), shb, sl, qs], dim=-1)
    elif type_id in (Q4_K, Q5_K):
        levels = 15.0 if type_id == Q4_K else 31.0
        sub = xb.reshape(n, nb, 8, 32)
        smin = torch.clamp(-sub.amin(-1), min=0.0)
        sscale = (sub.amax(-1) + smin) / levels
        d = _f16_round(sscale.amax(-1) / 63.0)
        dmin = _f16_round(smin.amax(-1) / 63.0)
        sc = torch.clamp(torch.round(sscale * _safe_inv(d)[..., None]), 0, 63)
        mn = torch.clamp(torch.round(smin * _safe_inv(dmin)[..., None]), 0, 63)
        eff = d[..., None] * sc
        q = torch.clamp(torch.round((sub + (dmin[..., None] * mn)[..., None]) * _safe_inv(eff)[..., None]), 0, levels)
        q = q.to(torch.int32).reshape(n, nb, 4, 2, 32)                 # group g, low/high nibble half, l
        ql = _nib(q[..., 0, :] & 15, q[..., 1, :] & 15).reshape(n, nb, 128)
        head = torch.cat([_f16_bytes(d), _f16_bytes(dmin), _pack_k4_scales(sc, mn)], dim=-1)
        if type_id == Q4_K:
            out = torch.cat([head, ql], dim=-1)
        else:
            g = torch.arange(4, device=x.device, dtype=torch.int32)
            bits = ((q[..., 0, :] >> 4) << (2 * g)[:, None]) | ((q[..., 1, :] >> 4) << (2 * g + 1)[:, None])
            qh = bits.sum(-2).to(torch.uint8)                          # [n,nb,32]
            out = torch.cat([head, qh, ql], dim=-1)
    elif type_id == Q6_K:
        sub = xb.reshape(n, nb, 16, 16)
        sscale = sub.abs().amax(-1) / 31.0
        d = _f16_round(sscale.amax(-1) / 127.0)
        sc = torch.clamp(torch.round(sscale * _safe_inv(d)[..., None]), 0, 127)
        eff = d[..., None] * sc
        q = torch.clamp(torch.round(sub * _safe_inv(eff)[..., None]) + 32, 0, 63).to(torch.int32)
        q = q.reshape(n, nb, 2, 4, 32)                                 # half, quarter (q1..q4), l
        q1, q2, q3, q4 = q[..., 0, :], q[..., 1, :], q[..., 2, :], q[..., 3, :]
        ql = torch.cat([_nib(q1 & 15, q3 & 15), _nib(q2 & 15, q4 & 15)], dim=-1).reshape(n, nb, 128)
        qh = ((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)).to(torch.uint8).reshape(n, nb, 64)
        out = torch.cat([ql, qh, sc.to(torch.int8).view(torch.uint8), _f16_bytes(d)], dim=-1)
    elif type_id == Q2_K:
        sub = xb.reshape(n, nb, 16, 16)
        smin = torch.clamp(-sub.amin(-1), min=0.0)
        sscale = (sub.amax(-1) + smin) / 3.0
        d = _f16_round(sscale.amax(-1) / 15.0)
        dmin = _f16_round(smin.amax(-1) / 15.0)
        sc = torch.clamp(torch.round(sscale * _safe_inv(d)[..., None]), 0, 15).to(torch.int32)
        mn = torch.clamp(torch.round(smin * _safe_inv(dmin)[..., None]), 0, 15).to(torch.int32)
        eff = d[..., None] * sc
        q = torch.clamp(torch.round((sub + (dmin[..., None] * mn)[..., None]) * _safe_inv(eff)[..., None]), 0, 3)
        q = q.to(torch.int32).reshape(n, nb, 2, 4, 2, 16)              # half, j(shift), odd, l
        j = torch.arange(4, device=x.device, dtype=torch.int32)
        qs = (q << (2 * j)[:, None, None]).sum(-3).to(torch.uint8).reshape(n, nb, 64)   # [half][odd][l]
        scales = (sc | (mn << 4)).to(torch.uint8)
        out = torch.cat([scales, qs, _f16_bytes(d), _f16_bytes(dmin)], dim=-1)
    elif type_id == Q3_K:
        sub = xb.reshape(n, nb, 16, 16)
        sscale = sub.abs().amax(-1) / 4.0
        d = _f16_round(sscale.amax(-1) / 31.0)
        sc = torch.clamp(torch.round(sscale * _safe_inv(d)[..., None]), 0, 31).to(torch.int32)   # stored +32
        eff = d[..., None] * sc
        q = torch.clamp(torch.round(sub * _safe_inv(eff)[..., None]), -4, 3).to(torch.int32)
        hbit = (q >= 0).to(torch.int32)
        q2 = torch.where(q >= 0, q, q + 4).reshape(n, nb, 2, 4, 2, 16)
        hbit = hbit.reshape(n, nb, 2, 4, 2, 16)
        j = torch.arange(4, device=x.device, dtype=torch.int32)
        qs = (q2 << (2 * j)[:, None, None]).sum(-3).to(torch.uint8).reshape(n, nb, 64)
        half = torch.arange(2, device=x.device, dtype=torch.int32)
        bitpos = (4 * half)[:, None] + j[None, :]                                       # [2,4]
        hm = (hbit << bitpos[:, :, None, None]).sum((-4, -3)).to(torch.uint8).reshape(n, nb, 32)   # [odd][l]
        st = sc + 32
        lo = ((st[..., :8] & 15) | ((st[..., 8:] & 15) << 4)).to(torch.uint8)
        hi4 = (st >> 4).reshape(n, nb, 4, 4)                                            # [sb>>2][sb&3]
        sh = torch.arange(4, device=x.device, dtype=torch.int32) * 2
        hi = (hi4 << sh[:, None]).sum(-2).to(torch.uint8)
        out = torch.cat([hm, qs, lo, hi, _f16_bytes(d)], dim=-1)
    else:
        raise ValueError(f"no quantiser for type {type_id}")
    out = out.reshape(n, nb * bb).contiguous()
    assert out.dtype == torch.uint8
    return out


def random_blocks(type_id: int, n_blocks: int, seed: int) -> np.ndarray:
    """Uniform random block bytes with every fp16 field forced finite: exercises
    all bit patterns of the packed fields, which quantiser output does not."""
    be, bb = BLOCK[type_id]
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(n_blocks, bb), dtype=np.uint8)
    f16_at = {Q4_0: [0], Q4_1: [0, 2], Q8_0: [0], Q2_K: [80, 82], Q3_K: [108], Q4_K: [0, 2], Q5_K: [0, 2],
              Q6_K: [208], IQ4_NL: [0], IQ4_XS: [0], F16: [0], BF16: [], F32: [],
              IQ2_XXS: [0], IQ2_XS: [0], IQ2_S: [0], IQ3_XXS: [0], IQ3_S: [0], IQ1_S: [0], IQ1_M: []}[type_id]
    for off in f16_at:
        hi = raw[:, off + 1]
        inf_nan = (hi & 0x7C) == 0x7C
        raw[:, off + 1] = np.where(inf_nan, hi & 0xBF, hi)      # clear one exponent bit
    if type_id == IQ1_M:
        # the fp16 scale is spread over the top nibbles of the four scale words (bytes 49, 51, 53, 55);
        # its exponent's top bits sit in byte 55: clear one so that the scale is finite
        raw[:, 55] &= 0xBF
    if type_id == F32:
        f = rng.standard_normal(n_blocks).astype(np.float32)
        raw = f.view(np.uint8).reshape(n_blocks, 4).copy()
    if type_id == BF16:
        hi = raw[:, 1]
        raw[:, 1] = np.where((hi & 0x7F) == 0x7F, hi & 0xBF, hi)
    return raw


def set_grid_block_scales(raw: np.ndarray, type_id: int, d: np.ndarray) -> np.ndarray:
    """Overwrites the fp16 block scale of grid-coded blocks ([n_blocks][block bytes]) with d (one value
    per block), leaving every other field as it is: random bytes then give weights of a chosen size."""
    bits16 = np.asarray(d, dtype=np.float16).view(np.uint16).astype(np.uint16)
    out = raw.copy()
    if type_id == IQ1_M:
        # the scale's four nibbles are the top nibbles of the four 16-bit scale words (src/quant/iquants.cpp:183-184)
        for i in range(4):
            nib = ((bits16 >> (4 * i)) & 15).astype(np.uint8)
            out[:, 49 + 2 * i] = (out[:, 49 + 2 * i] & 0x0F) | (nib << 4)
    else:
        out[:, 0] = (bits16 & 0xFF).astype(np.uint8)
        out[:, 1] = (bits16 >> 8).astype(np.uint8)
    return out


# ---------------------------------------------------------------------------
# GGUF v3 writer (only what the reference loader reads: src/gguf/gguf.cpp:108-398)
# ---------------------------------------------------------------------------
_GGUF_U32, _GGUF_F32, _GGUF_BOOL, _GGUF_STR, _GGUF_ARR, _GGUF_U64 = 4, 6, 7, 8, 9, 10


def _gstr(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _gval(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I?", _GGUF_BOOL, v)
    if isinstance(v, int):
        return struct.pack("<II", _GGUF_U32, v)
    if isinstance(v, float):
        return struct.pack("<If", _GGUF_F32, v)
    if isinstance(v, str):
        return struct.pack("<I", _GGUF_STR) + _gstr(v)
    if isinstance(v, (list, tuple)):
        if len(v) and isinstance(v[0], str):
            return struct.pack("<IIQ", _GGUF_ARR, _GGUF_STR, len(v)) + b"".join(_gstr(s) for s in v)
        return struct.pack("<IIQ", _GGUF_ARR, _GGUF_F32, len(v)) + np.asarray(v, dtype="<f4").tobytes()
    raise TypeError(type(v))


def write_gguf(path: str, kv: dict, tensors: list[tuple[str, int, list[int], np.ndarray]]) -> None:
    """tensors: (name, ggml type id, dims with dims[0]=K innermost, raw uint8 bytes)."""
    align = 32
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv))
    body = b"".join(_gstr(k) + _gval(v) for k, v in kv.items())
    infos, off = [], 0
    for name, tid, dims, data in tensors:
        infos.append(_gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
                     + struct.pack("<IQ", tid, off))
        off += (data.nbytes + align - 1) // align * align
    meta = head + body + b"".join(infos)
    pad = (-len(meta)) % align
    with open(path, "wb") as f:
        f.write(meta + b"\0" * pad)
        for _, _, _, data in tensors:
            f.write(memoryview(np.ascontiguousarray(data)).cast("B"))
            f.write(b"\0" * ((-data.nbytes) % align))


# ---------------------------------------------------------------------------
# Seeded random-init models
# ---------------------------------------------------------------------------
def tiny_config(**kw) -> ModelConfig:
    base = dict(n_layer=2, hidden=256, n_head=4, n_kv=2, head_dim=64, ffn=512, vocab=320, ctx=64)
    base.update(kw)
    return ModelConfig(**base)


# lfm2 test models (keyword arguments of tiny_config): gated short-convolution layers around GQA attention layers with
# per-head QK-norm; tied output, final norm stored as token_embd_norm
LFM2_CASES = {
    "lfm2": dict(arch="lfm2", n_layer=4, conv_layers=(0, 1, 3), qk_norm=True, rope_base=1e6, seed=33),
    "lfm2_q8": dict(arch="lfm2", n_layer=3, conv_layers=(0, 2), d_conv=4, qk_norm=True, rope_base=1e6, wtype=Q8_0, wtype_alt=Q8_0, seed=22),
}


@dataclass
class SynthModel:
    cfg: ModelConfig
    # name -> (type id, dims [K, N] or [n], uint8 numpy bytes)
    tensors: dict = field(default_factory=dict)

    def add(self, name, tid, dims, data):
        self.tensors[name] = (tid, list(dims), data)

    def kv(self) -> dict:
        c, a = self.cfg, self.cfg.arch
        kv = {
            "general.architecture": a,
            f"{a}.context_length": c.ctx, f"{a}.embedding_length": c.hidden, f"{a}.block_count": c.n_layer,
            f"{a}.feed_forward_length": c.ffn, f"{a}.attention.head_count": c.n_head,
            f"{a}.attention.head_count_kv": c.n_kv, f"{a}.attention.layer_norm_rms_epsilon": float(c.rms_eps),
            f"{a}.rope.freq_base": float(c.rope_base), f"{a}.rope.dimension_count": c.head_dim,
            # one unique code point per id so a prompt string maps 1:1 to token ids
            "tokenizer.ggml.model": "llama",
            "tokenizer.ggml.tokens": [chr(0x10000 + i) for i in range(c.vocab)],
            "tokenizer.ggml.scores": [0.0] * c.vocab,
            "tokenizer.ggml.add_space_prefix": False,
        }
        if a == "lfm2":
            kv["lfm2.shortconv.l_cache"] = c.d_conv
        return kv

    def write(self, path: str) -> None:
        write_gguf(path, self.kv(), [(n, t, d, b) for n, (t, d, b) in self.tensors.items()])

    def weight_bytes(self) -> int:
        return sum(b.nbytes for _, _, b in self.tensors.values())


def _name_seed(base: int, name: str) -> int:
    return (base ^ zlib.crc32(name.encode())) & 0x7FFFFFFF


def build_model(cfg: ModelConfig, device: str = "cpu") -> SynthModel:
    """Random-init N(0, 0.02) weights, one generator per tensor name, quantised
    with the quantisers above.  The same (cfg, device) always yields the same bytes."""
    m = SynthModel(cfg)
    dev = torch.device(device)

    def mat(name, n, k, tid):
        g = torch.Generator(device=dev)
        g.manual_seed(_name_seed(cfg.seed, name))
        rows_per = max(1, (64 << 20) // max(k, 1))
        parts = []
        for r0 in range(0, n, rows_per):
            w = torch.randn(min(rows_per, n - r0), k, generator=g, device=dev, dtype=torch.float32) * 0.02
            parts.append(quantize(w, tid).cpu())
        m.add(name, tid, [k, n], torch.cat(parts).numpy())

    def vec(name, n, kind):
        g = torch.Generator(device="cpu")
        g.manual_seed(_name_seed(cfg.seed, name))
        r = torch.randn(n, generator=g, dtype=torch.float32)
        v = 1.0 + cfg.norm_jitter * r if kind == "norm" else 0.02 * r
        m.add(name, F32, [n], v.numpy().view(np.uint8).copy())

    qd, kvd = cfg.n_head * cfg.head_dim, cfg.n_kv * cfg.head_dim
    lfm2 = cfg.arch == "lfm2"
    mat("token_embd.weight", cfg.vocab, cfg.hidden, cfg.wtype)
    vec("token_embd_norm.weight" if lfm2 else "output_norm.weight", cfg.hidden, "norm")   # lfm2's final norm (src/cli/main.cpp:2853-2855)
    if not cfg.tied:
        mat("output.weight", cfg.vocab, cfg.hidden, cfg.out_type if cfg.out_type is not None else cfg.wtype)
    for l in range(cfg.n_layer):
        p = f"blk.{l}."
        vec(p + "attn_norm.weight", cfg.hidden, "norm")
        vec(p + "ffn_norm.weight", cfg.hidden, "norm")
        if lfm2 and l in cfg.conv_layers:
            # gated short convolution (src/cli/main.cpp:2693-2732): in_proj -> [B | C | x], F32 conv {d_conv, hidden}
            mat(p + "shortconv.in_proj.weight", 3 * cfg.hidden, cfg.hidden, cfg.wtype)
            mat(p + "shortconv.out_proj.weight", cfg.hidden, cfg.hidden, cfg.wtype_alt)
            g = torch.Generator(device="cpu")
            g.manual_seed(_name_seed(cfg.seed, p + "shortconv.conv.weight"))
            cw = (torch.randn(cfg.hidden, cfg.d_conv, generator=g, dtype=torch.float32) * 0.5).contiguous()
            m.add(p + "shortconv.conv.weight", F32, [cfg.d_conv, cfg.hidden], cw.numpy().view(np.uint8).reshape(-1).copy())
        else:
            mat(p + "attn_q.weight", qd, cfg.hidden, cfg.wtype)
            mat(p + "attn_k.weight", kvd, cfg.hidden, cfg.wtype)
            mat(p + "attn_v.weight", kvd, cfg.hidden, cfg.wtype_alt)
            mat(p + "attn_output.weight", cfg.hidden, qd, cfg.wtype)
            if cfg.qk_norm:
                vec(p + "attn_q_norm.weight", cfg.head_dim, "norm")
                vec(p + "attn_k_norm.weight", cfg.head_dim, "norm")
        mat(p + "ffn_gate.weight", cfg.ffn, cfg.hidden, cfg.wtype)
        mat(p + "ffn_up.weight", cfg.ffn, cfg.hidden, cfg.wtype)
        mat(p + "ffn_down.weight", cfg.hidden, cfg.ffn, cfg.wtype_alt)
        if cfg.qkv_bias:
            vec(p + "attn_q.bias", qd, "bias")
            vec(p + "attn_k.bias", kvd, "bias")
            vec(p + "attn_v.bias", kvd, "bias")
    return m


def tiny_q35_config(**kw) -> Qwen35MoeConfig:
    base = dict(n_layer=4, hidden=256, n_head=2, n_kv=1, head_dim=256, rope_dim=64, sk=64, n_vhead=4, n_khead=2,
                n_expert=8, top_k=2, eff=256, vocab=320, ctx=64)
    base.update(kw)
    return Qwen35MoeConfig(**base)


def q35_kv(cfg: Qwen35MoeConfig) -> dict:
    a = cfg.arch
    return {
        "general.architecture": a,
        f"{a}.context_length": cfg.ctx, f"{a}.embedding_length": cfg.hidden, f"{a}.block_count": cfg.n_layer,
        f"{a}.feed_forward_length": cfg.ffn, f"{a}.attention.head_count": cfg.n_head,
        f"{a}.attention.head_count_kv": cfg.n_kv, f"{a}.attention.layer_norm_rms_epsilon": float(cfg.rms_eps),
        f"{a}.rope.freq_base": float(cfg.rope_base), f"{a}.rope.dimension_count": cfg.rope_dim,
        f"{a}.attention.key_length": cfg.head_dim, f"{a}.ssm.conv_kernel": cfg.conv_k, f"{a}.ssm.state_size": cfg.sk,
        f"{a}.ssm.inner_size": cfg.n_vhead * cfg.sk, f"{a}.ssm.group_count": cfg.n_khead,
        f"{a}.expert_count": cfg.n_expert, f"{a}.expert_used_count": cfg.top_k,
        f"{a}.expert_feed_forward_length": cfg.eff, f"{a}.nextn_predict_layers": 0,
        "tokenizer.ggml.model": "llama",
        "tokenizer.ggml.tokens": [chr(0x10000 + i) for i in range(cfg.vocab)],
        "tokenizer.ggml.scores": [0.0] * cfg.vocab,
        "tokenizer.ggml.add_space_prefix": False,
    }


def build_q35_model(cfg: Qwen35MoeConfig, device: str = "cpu") -> SynthModel:
    """Random-init qwen35moe tensors: matrices N(0, 0.02) quantised (Q4_K; Q6_K for attention output and expert
    down), F32 router / alpha / beta / conv / decay vectors, norm gammas 1 + jitter N(0,1)."""
    m = SynthModel(cfg)
    m.kv = lambda: q35_kv(cfg)
    dev = torch.device(device)

    def randn(name, *shape, scale=1.0):
        g = torch.Generator(device=dev)
        g.manual_seed(_name_seed(cfg.seed, name))
        return torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * scale

    def mat(name, n, k, tid, n_exp=0):
        rows = n * max(n_exp, 1)
        rows_per = max(1, (64 << 20) // max(k, 1))
        g = torch.Generator(device=dev)
        g.manual_seed(_name_seed(cfg.seed, name))
        parts = []
        for r0 in range(0, rows, rows_per):
            w = torch.randn(min(rows_per, rows - r0), k, generator=g, device=dev, dtype=torch.float32) * 0.02
            parts.append(quantize(w, tid).cpu())
        m.add(name, tid, [k, n, n_exp] if n_exp else [k, n], torch.cat(parts).numpy())

    def f32(name, dims, t):
        m.add(name, F32, list(dims), t.cpu().contiguous().numpy().view(np.uint8).copy())

    def norm(name, n):
        f32(name, [n], 1.0 + cfg.norm_jitter * randn(name, n))

    H, sk = cfg.hidden, cfg.sk
    key_dim, value_dim = cfg.n_khead * sk, cfg.n_vhead * sk
    conv_dim = 2 * key_dim + value_dim
    qdim, kvdim = cfg.n_head * cfg.head_dim, cfg.n_kv * cfg.head_dim
    mat("token_embd.weight", cfg.vocab, H, cfg.wtype)
    norm("output_norm.weight", H)
    if not cfg.tied:
        mat("output.weight", cfg.vocab, H, cfg.wtype_alt)
    for l in range(cfg.n_layer):
        p = f"blk.{l}."
        norm(p + "attn_norm.weight", H)
        norm(p + "post_attention_norm.weight", H)
        if cfg.is_ssm(l):
            mat(p + "attn_qkv.weight", conv_dim, H, cfg.wtype)
            mat(p + "attn_gate.weight", value_dim, H, cfg.wtype)
            f32(p + "ssm_alpha.weight", [H, cfg.n_vhead], randn(p + "ssm_alpha.weight", cfg.n_vhead, H, scale=0.05))
            f32(p + "ssm_beta.weight", [H, cfg.n_vhead], randn(p + "ssm_beta.weight", cfg.n_vhead, H, scale=0.05))
            # conv taps: [channel][tap], newest tap last (main.cpp:2927-2935)
            f32(p + "ssm_conv1d.weight", [cfg.conv_k, conv_dim], randn(p + "ssm_conv1d.weight", conv_dim, cfg.conv_k, scale=0.5))
            f32(p + "ssm_a", [cfg.n_vhead], -torch.exp(randn(p + "ssm_a", cfg.n_vhead, scale=0.5)))   # stored as -exp(A_log)
            f32(p + "ssm_dt.bias", [cfg.n_vhead], randn(p + "ssm_dt.bias", cfg.n_vhead, scale=0.5))
            norm(p + "ssm_norm.weight", sk)
            mat(p + "ssm_out.weight", H, value_dim, cfg.wtype)
        else:
            mat(p + "attn_q.weight", 2 * qdim, H, cfg.wtype)
            mat(p + "attn_k.weight", kvdim, H, cfg.wtype)
            mat(p + "attn_v.weight", kvdim, H, cfg.wtype)
            mat(p + "attn_output.weight", H, qdim, cfg.wtype_alt)
            norm(p + "attn_q_norm.weight", cfg.head_dim)
            norm(p + "attn_k_norm.weight", cfg.head_dim)
        f32(p + "ffn_gate_inp.weight", [H, cfg.n_expert], randn(p + "ffn_gate_inp.weight", cfg.n_expert, H, scale=0.05))
        mat(p + "ffn_gate_exps.weight", cfg.eff, H, cfg.wtype, cfg.n_expert)
        mat(p + "ffn_up_exps.weight", cfg.eff, H, cfg.wtype, cfg.n_expert)
        mat(p + "ffn_down_exps.weight", H, cfg.eff, cfg.wtype_alt, cfg.n_expert)
        mat(p + "ffn_gate_shexp.weight", cfg.eff, H, cfg.wtype)
        mat(p + "ffn_up_shexp.weight", cfg.eff, H, cfg.wtype)
        mat(p + "ffn_down_shexp.weight", H, cfg.eff, cfg.wtype_alt)
        f32(p + "ffn_gate_inp_shexp.weight", [H], randn(p + "ffn_gate_inp_shexp.weight", H, scale=0.05))
    return m


def prompt_text(ids) -> str:
    """Token ids -> the prompt string the code-point tokenizer maps back to them."""
    return "".join(chr(0x10000 + int(i)) for i in ids)


def text_ids(s: str) -> list[int]:
    return [ord(ch) - 0x10000 for ch in s if ord(ch) >= 0x10000]
