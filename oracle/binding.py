"""ctypes bindings for the two CPU checkers.  TEST INFRASTRUCTURE ONLY: import
this from tests/, from the smoke check and from the benchmark's CPU-baseline
leg; never from the product package.

  Oracle  -- libggb_oracle.so, the C restatement in ggb_oracle.c
  Ref     -- _ref/libggnpu_ref.so, the reference's own sources behind ref_shim.cpp
             (present only where `make -C oracle ref` could see the reference tree,
             or where the prebuilt file travelled with the checkout)
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libggb_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libggnpu_ref.so")
REF_CLI = os.path.join(HERE, "_ref", "ggnpu_cpu_oracle")

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)


def _fp(a):
    return a.ctypes.data_as(_f32p) if a is not None else None


def _bp(a):
    return a.ctypes.data_as(_u8p) if a is not None else None


def build_oracle() -> str:
    # the codebooks of the grid-coded formats are generated (from the gguf package) next to the CUDA objects
    inc = os.path.join(HERE, "..", "ggnpu_b200", "build", "ggb_iq_grids.inc")
    try:
        from ggnpu_b200.iq_tables import write_include
        write_include(inc)
    except Exception:
        pass
    deps = [os.path.join(HERE, "ggb_oracle.c")] + ([inc] if os.path.exists(inc) else [])
    if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < max(os.path.getmtime(d) for d in deps):
        subprocess.check_call(["make", "-s", "-C", HERE, "oracle"])
    return ORACLE_SO


def reference_root() -> str | None:
    """Where the reference tree lies: $GGNPU_REFERENCE, else a `reference` directory next to this
    checkout.  None when neither holds the reference's CLI sources."""
    for cand in (os.environ.get("GGNPU_REFERENCE"), os.path.join(HERE, "..", "..", "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src", "cli")):
            return os.path.abspath(cand)
    return None


def build_ref(ref_root: str | None = None) -> str | None:
    """Build oracle/_ref from the reference tree when it is present; otherwise
    use a prebuilt copy if there is one."""
    ref_root = ref_root or reference_root()
    if ref_root:
        subprocess.check_call(["make", "-s", "-j8", "-C", HERE, "ref", f"REF={ref_root}"])
        # the unmodified reference CLI linked against the CUDA backend (the drop-in check)
        if os.path.exists(os.path.join(HERE, "..", "ggnpu_b200", "libggb200.so")):
            subprocess.check_call(["make", "-s", "-j8", "-C", HERE, "dropin", f"REF={ref_root}"])
    return REF_SO if os.path.exists(REF_SO) else None


class Oracle:
    """The C restatement.  Array arguments are numpy; outputs are new arrays."""

    def __init__(self):
        self.lib = L = C.CDLL(build_oracle())
        L.ggo_f16_to_f32.restype = C.c_float
        L.ggo_f16_to_f32.argtypes = [C.c_uint16]
        L.ggo_bf16_to_f32.restype = C.c_float
        L.ggo_bf16_to_f32.argtypes = [C.c_uint16]
        L.ggo_f32_to_bf16.restype = C.c_uint16
        L.ggo_f32_to_bf16.argtypes = [C.c_float]
        L.ggo_dequant_blocks.argtypes = [C.c_uint32, _u8p, C.c_int64, _f32p]
        L.ggo_dequant_row.argtypes = [C.c_uint32, _u8p, C.c_int64, C.c_int, _f32p]
        L.ggo_matmul_exact.argtypes = [_f32p, C.c_int, C.c_int, _u8p, C.c_uint32, C.c_int, C.c_int, _f32p, C.c_int]
        L.ggo_moe_ffn.argtypes = [_f32p, C.c_int, _f32p, C.c_int, C.c_int, C.c_int, _u8p, _u8p, C.c_uint32, _u8p, C.c_uint32,
                                  _u8p, _u8p, C.c_uint32, _u8p, C.c_uint32, C.c_int, _f32p, _f32p, C.c_void_p, _f32p]
        L.ggo_deltanet_step.argtypes = [_f32p] * 11 + [C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        L.ggo_matmul_cpu_ref_k.argtypes = [_f32p, C.c_int, _u8p, C.c_uint32, C.c_int, C.c_int, _f32p]
        L.ggo_matmul_f32_kn.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.ggo_rms_norm.argtypes = [_f32p, _f32p, C.c_int, C.c_float, _f32p]
        L.ggo_rms_norm_head_f64.argtypes = [_f32p, C.c_int, C.c_float, _f32p]
        L.ggo_silu.argtypes = [_f32p, _f32p, C.c_int]
        L.ggo_gelu.argtypes = [_f32p, _f32p, C.c_int]
        L.ggo_softmax.argtypes = [_f32p, _f32p, C.c_int, C.c_int]
        L.ggo_flash_attn.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int64, C.c_int64]
        L.ggo_rope_cpu_ref.argtypes = [_f32p, C.c_int, C.c_int64, C.c_float, C.c_int64]
        L.ggo_rope_table.argtypes = [C.c_int64, C.c_int, C.c_float, C.c_float, _f32p, C.c_int, _f32p, _f32p]
        L.ggo_rope_apply.argtypes = [_f32p, _f32p, C.c_int, C.c_int, C.c_int, _f32p, _f32p, C.c_int]
        L.ggo_argmax_first.argtypes = [_f32p, C.c_int]
        L.ggo_sample_token.argtypes = [_f32p, C.c_int, C.c_float, C.POINTER(C.c_uint64)]
        L.ggo_model_new.restype = C.c_void_p
        L.ggo_model_new.argtypes = [C.c_int] * 8 + [C.c_float] * 3 + [C.c_int]
        L.ggo_model_free.argtypes = [C.c_void_p]
        L.ggo_model_set_globals.argtypes = [C.c_void_p, _u8p, C.c_uint32, _u8p, C.c_uint32, _f32p, _f32p, C.c_int]
        L.ggo_model_set_weight.argtypes = [C.c_void_p, C.c_int, C.c_int, _u8p, C.c_uint32]
        L.ggo_model_set_vec.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p]
        L.ggo_model_set_lfm2.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.ggo_model_reset_conv.argtypes = [C.c_void_p]
        L.ggo_forward.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_int, _f32p, _f32p]
        L.ggo_model_kv.restype = _f32p
        L.ggo_model_kv.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.ggo_block_elems.argtypes = [C.c_uint32]
        L.ggo_block_bytes.argtypes = [C.c_uint32]
        L.ggo_q35_new.restype = C.c_void_p
        L.ggo_q35_new.argtypes = [C.c_int] * 15 + [C.c_float] * 2
        L.ggo_q35_free.argtypes = [C.c_void_p]
        L.ggo_q35_set_globals.argtypes = [C.c_void_p, _u8p, C.c_uint32, _u8p, C.c_uint32, _f32p]
        L.ggo_q35_set_kind.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.ggo_q35_set_weight.argtypes = [C.c_void_p, C.c_int, C.c_int, _u8p, C.c_uint32]
        L.ggo_q35_set_vec.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p]
        L.ggo_q35_rope_table.argtypes = [C.c_int64, C.c_int, C.c_float, _f32p, _f32p]
        L.ggo_q35_forward.argtypes = [C.c_void_p, C.c_int32, C.c_int, _f32p, _f32p]
        L.ggo_q35_kv.restype = _f32p
        L.ggo_q35_kv.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.ggo_q35_rec_state.restype = _f32p
        L.ggo_q35_rec_state.argtypes = [C.c_void_p, C.c_int]

    def block_geom(self, t):
        return self.lib.ggo_block_elems(t), self.lib.ggo_block_bytes(t)

    def dequant_blocks(self, t, data: np.ndarray) -> np.ndarray:
        be, bb = self.block_geom(t)
        data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
        nb = data.size // bb
        out = np.empty(nb * be, dtype=np.float32)
        assert self.lib.ggo_dequant_blocks(t, _bp(data), nb, _fp(out)) == 0
        return out

    def dequant_row(self, t, data, row, K):
        data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
        out = np.empty(K, dtype=np.float32)
        assert self.lib.ggo_dequant_row(t, _bp(data), row, K, _fp(out)) == 0
        return out

    def matmul_exact(self, A, W, t, N, K):
        A = np.ascontiguousarray(A, dtype=np.float32).reshape(-1, K)
        W = np.ascontiguousarray(W, dtype=np.uint8).reshape(-1)
        out = np.empty((A.shape[0], N), dtype=np.float32)
        assert self.lib.ggo_matmul_exact(_fp(A), A.shape[0], K, _bp(W), t, N, K, _fp(out), N) == 0
        return out

    def matmul_cpu_ref_k(self, A, W, t, N, K):
        A = np.ascontiguousarray(A, dtype=np.float32).reshape(-1, K)
        W = np.ascontiguousarray(W, dtype=np.uint8).reshape(-1)
        out = np.empty((A.shape[0], N), dtype=np.float32)
        assert self.lib.ggo_matmul_cpu_ref_k(_fp(A), A.shape[0], _bp(W), t, N, K, _fp(out)) == 0
        return out

    def matmul_f32_kn(self, A, B):
        A = np.ascontiguousarray(A, dtype=np.float32)
        B = np.ascontiguousarray(B, dtype=np.float32)
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, N), dtype=np.float32)
        self.lib.ggo_matmul_f32_kn(_fp(A), _fp(B), _fp(out), M, N, K)
        return out

    def rms_norm(self, x, eps, w=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        w = None if w is None else np.ascontiguousarray(w, dtype=np.float32)
        self.lib.ggo_rms_norm(_fp(x), _fp(y), x.size, eps, _fp(w))
        return y

    def rms_norm_head_f64(self, x, eps, w):
        v = np.array(x, dtype=np.float32, copy=True)
        w = np.ascontiguousarray(w, dtype=np.float32)
        self.lib.ggo_rms_norm_head_f64(_fp(v), v.size, eps, _fp(w))
        return v

    def _unary(self, fn, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        fn(_fp(x), _fp(y), x.size)
        return y

    def silu(self, x):
        return self._unary(self.lib.ggo_silu, x)

    def gelu(self, x):
        return self._unary(self.lib.ggo_gelu, x)

    def softmax(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        self.lib.ggo_softmax(_fp(x), _fp(y), x.shape[0], x.shape[1])
        return y

    def flash_attn(self, Q, K, V, qpos=-1):
        Q = np.ascontiguousarray(Q, dtype=np.float32)
        K = np.ascontiguousarray(K, dtype=np.float32)
        V = np.ascontiguousarray(V, dtype=np.float32)
        nh, hd = Q.shape
        ctx = K.shape[1]
        out = np.empty_like(Q)
        assert self.lib.ggo_flash_attn(_fp(Q), _fp(K), _fp(V), _fp(out), nh, hd, ctx, qpos) == 0
        return out

    def moe_ffn(self, x, router, top_k, eff, gate_exps, up_exps, type_gu, down_exps, type_d,
                shared=None, sh_gate_inp=None):
        """MoE FFN of one token (src/cli/main.cpp:3110-3193).  shared = (gate, up, type_gu, down, type_d, eff_sh) or None.
        Returns (moe_out[hidden], chosen ids[top_k], weights[top_k (+1 with a shared expert)])."""
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        router = np.ascontiguousarray(router, dtype=np.float32)
        n_expert, hidden = router.shape
        out = np.empty(hidden, np.float32)
        ids = np.empty(top_k, np.int32)
        w = np.zeros(top_k + 1, np.float32)
        u8 = lambda a: np.ascontiguousarray(a, dtype=np.uint8).reshape(-1)
        ge, ue, de = u8(gate_exps), u8(up_exps), u8(down_exps)
        if shared is not None:
            sg, su, stgu, sd, std, eff_sh = shared
            sg, su, sd = u8(sg), u8(su), u8(sd)
            sgp, sup, sdp = _bp(sg), _bp(su), _bp(sd)
        else:
            sgp = sup = sdp = None
            stgu = std = eff_sh = 0
        gi = np.ascontiguousarray(sh_gate_inp, dtype=np.float32) if sh_gate_inp is not None else None
        rc = self.lib.ggo_moe_ffn(_fp(x), hidden, _fp(router), n_expert, top_k, eff, _bp(ge), _bp(ue), type_gu, _bp(de), type_d,
                                  sgp, sup, stgu, sdp, std, eff_sh, _fp(gi) if gi is not None else None, _fp(out),
                                  ids.ctypes.data_as(C.c_void_p), _fp(w))
        assert rc == 0
        return out, ids, (w if shared is not None else w[:top_k])

    def deltanet_step(self, mixed, zgate, araw, braw, conv_w, ssm_a, dt_bias, ssm_norm, conv_state, rec_state,
                      n_khead, n_vhead, sk, conv_k, rms_eps):
        """One token of a Gated DeltaNet layer (src/cli/main.cpp:2925-3023); conv_state and rec_state (float32,
        C-contiguous) are updated in place.  Returns out[n_vhead * sk]."""
        f = lambda a: np.ascontiguousarray(a, dtype=np.float32)
        assert conv_state.dtype == np.float32 and conv_state.flags.c_contiguous and rec_state.dtype == np.float32 and rec_state.flags.c_contiguous
        out = np.empty(n_vhead * sk, np.float32)
        args = [f(mixed), f(zgate), f(araw), f(braw), f(conv_w), f(ssm_a), f(dt_bias), f(ssm_norm)]
        rc = self.lib.ggo_deltanet_step(*[_fp(a) for a in args], _fp(conv_state), _fp(rec_state), _fp(out),
                                        n_khead, n_vhead, sk, conv_k, rms_eps)
        assert rc == 0
        return out

    def rope_cpu_ref(self, x, n_dims, offset, freq_scale, rope_dims):
        v = np.array(x, dtype=np.float32, copy=True)
        self.lib.ggo_rope_cpu_ref(_fp(v), n_dims, offset, freq_scale, rope_dims)
        return v

    def rope_table(self, max_pos, n_dims, scale, base, ff=None):
        c = np.empty((max_pos, n_dims // 2), dtype=np.float32)
        s = np.empty_like(c)
        ff = None if ff is None else np.ascontiguousarray(ff, dtype=np.float32)
        self.lib.ggo_rope_table(max_pos, n_dims, scale, base, _fp(ff), 0 if ff is None else ff.size, _fp(c), _fp(s))
        return c, s

    def rope_apply(self, x, n_heads, head_dim, rot_dims, cos_row, sin_row, neox=False):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty_like(x)
        cos_row = np.ascontiguousarray(cos_row, dtype=np.float32)
        sin_row = np.ascontiguousarray(sin_row, dtype=np.float32)
        self.lib.ggo_rope_apply(_fp(out), _fp(x), n_heads, head_dim, rot_dims, _fp(cos_row), _fp(sin_row), int(neox))
        return out

    def argmax_first(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        return self.lib.ggo_argmax_first(_fp(x), x.size)

    def sample_token(self, x, temp, seed):
        """sample_token (src/cli/main.cpp:827-864): (token, advanced seed)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        sd = C.c_uint64(int(seed))
        tok = self.lib.ggo_sample_token(_fp(x), x.size, float(temp), C.byref(sd))
        return tok, sd.value


_W_SLOTS = {"attn_q": 0, "attn_k": 1, "attn_v": 2, "attn_output": 3, "ffn_gate": 4, "ffn_up": 5, "ffn_down": 6,
            "shortconv.in_proj": 7, "shortconv.out_proj": 8}
_V_SLOTS = {"attn_norm.weight": 0, "ffn_norm.weight": 1, "attn_q.bias": 2, "attn_k.bias": 3, "attn_v.bias": 4,
            "attn_q_norm.weight": 5, "attn_k_norm.weight": 6, "shortconv.conv.weight": 7}


class OracleModel:
    """The generic-architecture forward of the reference CLI, restated
    (ggo_forward), over the tensors of a ggnpu_b200.testing.synth.SynthModel."""

    def __init__(self, oracle: Oracle, synth, cpu_rope: bool = True):
        """lfm2 models: cpu_rope=True rotates as the reference CLI does on its CPU backend (adjacent pairs, base
        10000); False as the branch asks its backend to (split-half pairs, the model's base)."""
        self.o, self.cfg = oracle, synth.cfg
        c = synth.cfg
        L = oracle.lib
        self._keep = []
        lfm2 = c.arch == "lfm2"
        self.h = L.ggo_model_new(c.n_layer, c.hidden, c.n_head, c.n_kv, c.head_dim, c.ffn, c.vocab, c.ctx,
                                 c.rms_eps, float(np.float32(c.rope_base)), 1.0, 1 if c.arch in ("qwen3", "lfm2") else 0)
        if lfm2:
            L.ggo_model_set_lfm2(self.h, c.d_conv, 1 if cpu_rope else 0)
        t = synth.tensors

        def raw(name):
            tid, _, b = t[name]
            b = np.ascontiguousarray(b).view(np.uint8).reshape(-1)
            self._keep.append(b)
            return b, tid

        def f32(name):
            b, _ = raw(name)
            return b.view(np.float32)

        emb, et = raw("token_embd.weight")
        out, ot = raw("output.weight") if "output.weight" in t else (None, 0)
        ff = f32("rope_freqs.weight") if "rope_freqs.weight" in t else None
        L.ggo_model_set_globals(self.h, _bp(emb), et, _bp(out), ot, _fp(f32("token_embd_norm.weight" if lfm2 else "output_norm.weight")), _fp(ff),
                                0 if ff is None else ff.size)
        for l in range(c.n_layer):
            for nm, slot in _W_SLOTS.items():
                if f"blk.{l}.{nm}.weight" not in t:        # lfm2: a layer has attention or the short convolution
                    continue
                b, tid = raw(f"blk.{l}.{nm}.weight")
                L.ggo_model_set_weight(self.h, l, slot, _bp(b), tid)
            for nm, slot in _V_SLOTS.items():
                key = f"blk.{l}.{nm}"
                if key in t:
                    L.ggo_model_set_vec(self.h, l, slot, _fp(f32(key)))

    def forward(self, tokens, pos, want_logits=True, want_hidden=False):
        c = self.cfg
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(c.vocab, dtype=np.float32) if want_logits else None
        hid = np.empty((toks.size, c.hidden), dtype=np.float32) if want_hidden else None
        rc = self.o.lib.ggo_forward(self.h, toks.ctypes.data_as(C.POINTER(C.c_int32)), toks.size, pos, _fp(logits), _fp(hid))
        assert rc == 0
        return (logits, hid) if want_hidden else logits

    def reset(self):
        """A new sequence (lfm2: the convolution states return to zero; the KV cache is overwritten by position)."""
        if self.cfg.arch == "lfm2":
            self.o.lib.ggo_model_reset_conv(self.h)

    def kv_row(self, layer, pos, want_v):
        c = self.cfg
        p = self.o.lib.ggo_model_kv(self.h, layer, pos, int(want_v))
        return np.ctypeslib.as_array(p, shape=(c.n_kv, c.head_dim)).copy()

    def close(self):
        if self.h:
            self.o.lib.ggo_model_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_Q35_W = {"attn_qkv": 0, "attn_gate": 1, "ssm_alpha": 2, "ssm_beta": 3, "ssm_out": 4, "attn_q": 5, "attn_k": 6, "attn_v": 7,
          "attn_output": 8, "ffn_gate_exps": 9, "ffn_up_exps": 10, "ffn_down_exps": 11, "ffn_gate_shexp": 12,
          "ffn_up_shexp": 13, "ffn_down_shexp": 14}
_Q35_V = {"attn_norm.weight": 0, "post_attention_norm.weight": 1, "ssm_conv1d.weight": 2, "ssm_a": 3, "ssm_dt.bias": 4,
          "ssm_norm.weight": 5, "attn_q_norm.weight": 6, "attn_k_norm.weight": 7, "ffn_gate_inp.weight": 8,
          "ffn_gate_inp_shexp.weight": 9}


class OracleQ35Model:
    """The qwen35moe forward of the reference CLI, restated (ggo_q35_forward), over the tensors of
    ggnpu_b200.testing.synth.build_q35_model.  One token per call, like the reference."""

    def __init__(self, oracle: Oracle, synth):
        self.o, self.cfg = oracle, synth.cfg
        c = synth.cfg
        L = oracle.lib
        self._keep = []
        self.h = L.ggo_q35_new(c.n_layer, c.hidden, c.n_head, c.n_kv, c.head_dim, c.rope_dim, c.conv_k, c.sk, c.n_vhead,
                               c.n_khead, c.n_expert, c.top_k, c.eff, c.vocab, c.ctx, c.rms_eps, float(np.float32(c.rope_base)))
        t = synth.tensors

        def raw(name):
            tid, _, b = t[name]
            b = np.ascontiguousarray(b).view(np.uint8).reshape(-1)
            self._keep.append(b)
            return b, tid

        emb, et = raw("token_embd.weight")
        out, ot = raw("output.weight") if "output.weight" in t else (None, 0)
        L.ggo_q35_set_globals(self.h, _bp(emb), et, _bp(out), ot, _fp(raw("output_norm.weight")[0].view(np.float32)))
        for l in range(c.n_layer):
            L.ggo_q35_set_kind(self.h, l, 1 if f"blk.{l}.ssm_conv1d.weight" in t else 0)
            for nm, slot in _Q35_W.items():
                key = f"blk.{l}.{nm}.weight"
                if key in t:
                    b, tid = raw(key)
                    L.ggo_q35_set_weight(self.h, l, slot, _bp(b), tid)
            for nm, slot in _Q35_V.items():
                key = f"blk.{l}.{nm}"
                if key in t:
                    L.ggo_q35_set_vec(self.h, l, slot, _fp(raw(key)[0].view(np.float32)))

    def forward(self, token, pos, want_hidden=False):
        c = self.cfg
        logits = np.empty(c.vocab, dtype=np.float32)
        hid = np.empty(c.hidden, dtype=np.float32) if want_hidden else None
        rc = self.o.lib.ggo_q35_forward(self.h, int(token), int(pos), _fp(logits), _fp(hid))
        assert rc == 0
        return (logits, hid) if want_hidden else logits

    def feed(self, tokens, pos0=0):
        """Run the tokens one by one from position pos0; returns the logits after the last."""
        out = None
        for i, tk in enumerate(tokens):
            out = self.forward(tk, pos0 + i)
        return out

    def reset(self):
        """A new sequence (lfm2: the convolution states return to zero; the KV cache is overwritten by position)."""
        if self.cfg.arch == "lfm2":
            self.o.lib.ggo_model_reset_conv(self.h)

    def kv_row(self, layer, pos, want_v):
        c = self.cfg
        p = self.o.lib.ggo_q35_kv(self.h, layer, pos, int(want_v))
        return np.ctypeslib.as_array(p, shape=(c.n_kv, c.head_dim)).copy()

    def rec_state(self, layer):
        c = self.cfg
        p = self.o.lib.ggo_q35_rec_state(self.h, layer)
        return np.ctypeslib.as_array(p, shape=(c.n_vhead, c.sk, c.sk)).copy()

    def close(self):
        if self.h:
            self.o.lib.ggo_q35_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Ref:
    """The reference's own compiled functions (oracle/_ref).  `Ref.available()`
    is False where neither the reference tree nor a prebuilt library exists."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self):
        self.lib = L = C.CDLL(REF_SO)
        L.ref_f16_to_f32.restype = C.c_float
        L.ref_f16_to_f32.argtypes = [C.c_uint16]
        L.ref_kquant_fp16_to_f32.restype = C.c_float
        L.ref_kquant_fp16_to_f32.argtypes = [C.c_uint16]
        L.ref_bf16_to_f32.restype = C.c_float
        L.ref_bf16_to_f32.argtypes = [C.c_uint16]
        L.ref_f32_to_bf16.restype = C.c_uint16
        L.ref_f32_to_bf16.argtypes = [C.c_float]
        L.ref_dequant_block.argtypes = [C.c_uint32, _u8p, _f32p]
        L.ref_dequant_tensor_row.argtypes = [C.c_uint32, _u8p, C.c_int, C.c_int, _f32p]
        L.ref_matmul_exact.argtypes = [_f32p, C.c_int, C.c_int, _u8p, C.c_uint32, C.c_int, C.c_int, _f32p, C.c_int]
        L.ref_rope_table.argtypes = [C.c_int64, C.c_int, C.c_float, C.c_float, _f32p, C.c_int, _f32p, _f32p]
        L.ref_mul_mat_q.argtypes = [_f32p, C.c_void_p, _f32p, C.c_int, C.c_int, C.c_int, C.c_uint32]
        L.ref_rms_norm.argtypes = [_f32p, _f32p, C.c_int, C.c_float, _f32p]
        L.ref_rope.argtypes = [_f32p, C.c_int, C.c_int64, C.c_float, C.c_float, C.c_int64]
        L.ref_softmax.argtypes = [_f32p, _f32p, C.c_int, C.c_int]
        L.ref_silu.argtypes = [_f32p, _f32p, C.c_int]
        L.ref_gelu.argtypes = [_f32p, _f32p, C.c_int]
        L.ref_flash_attn.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int64, C.c_int64]
        L.ref_argmax.argtypes = [_f32p, C.c_int]
        L.ref_block_elems.argtypes = [C.c_uint32]
        L.ref_block_bytes.argtypes = [C.c_uint32]

    def dequant_blocks(self, t, data):
        be, bb = self.lib.ref_block_elems(t), self.lib.ref_block_bytes(t)
        data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1, bb)
        out = np.empty((data.shape[0], be), dtype=np.float32)
        for i in range(data.shape[0]):
            assert self.lib.ref_dequant_block(t, _bp(data[i]), _fp(out[i])) == 0
        return out.reshape(-1)

    def dequant_row(self, t, data, row, K):
        data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
        out = np.empty(K, dtype=np.float32)
        self.lib.ref_dequant_tensor_row(t, _bp(data), row, K, _fp(out))
        return out

    def matmul_exact(self, A, W, t, N, K):
        A = np.ascontiguousarray(A, dtype=np.float32).reshape(-1, K)
        W = np.ascontiguousarray(W, dtype=np.uint8).reshape(-1)
        out = np.empty((A.shape[0], N), dtype=np.float32)
        self.lib.ref_matmul_exact(_fp(A), A.shape[0], K, _bp(W), t, N, K, _fp(out), N)
        return out

    def mul_mat_q(self, A, B, t, N, K):
        A = np.ascontiguousarray(A, dtype=np.float32).reshape(-1, K)
        B = np.ascontiguousarray(B)
        out = np.empty((A.shape[0], N), dtype=np.float32)
        st = self.lib.ref_mul_mat_q(_fp(A), B.ctypes.data_as(C.c_void_p), _fp(out), A.shape[0], N, K, t)
        return st, out

    def rope_table(self, max_pos, n_dims, scale, base, ff=None):
        c = np.empty((max_pos, n_dims // 2), dtype=np.float32)
        s = np.empty_like(c)
        ff = None if ff is None else np.ascontiguousarray(ff, dtype=np.float32)
        self.lib.ref_rope_table(max_pos, n_dims, scale, base, _fp(ff), 0 if ff is None else ff.size, _fp(c), _fp(s))
        return c, s

    def rms_norm(self, x, eps, w=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        w = None if w is None else np.ascontiguousarray(w, dtype=np.float32)
        st = self.lib.ref_rms_norm(_fp(x), _fp(y), x.size, eps, _fp(w))
        return st, y

    def rope(self, x, n_dims, offset, freq_scale, freq_base, rope_dims):
        v = np.array(x, dtype=np.float32, copy=True)
        st = self.lib.ref_rope(_fp(v), n_dims, offset, freq_scale, freq_base, rope_dims)
        return st, v

    def _unary(self, fn, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        st = fn(_fp(x), _fp(y), x.size)
        return st, y

    def silu(self, x):
        return self._unary(self.lib.ref_silu, x)

    def gelu(self, x):
        return self._unary(self.lib.ref_gelu, x)

    def softmax(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        st = self.lib.ref_softmax(_fp(x), _fp(y), x.shape[0], x.shape[1])
        return st, y

    def flash_attn(self, Q, K, V, qpos=-1):
        Q = np.ascontiguousarray(Q, dtype=np.float32)
        K = np.ascontiguousarray(K, dtype=np.float32)
        V = np.ascontiguousarray(V, dtype=np.float32)
        out = np.empty_like(Q)
        st = self.lib.ref_flash_attn(_fp(Q), _fp(K), _fp(V), _fp(out), Q.shape[0], Q.shape[1], K.shape[1], qpos)
        return st, out

    def argmax(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        return self.lib.ref_argmax(_fp(x), x.size)


def run_ref_cli(gguf_path: str, prompt: str, n_tokens: int, ctx: int = 2048, bench_logits: bool = False,
                exact: bool = True, timeout: float | None = None, extra_env: dict | None = None,
                temp: float = 0.0, seed: int | None = None):
    """Run the reference CLI on its CPU backend.  exact=True sets the two
    environment switches that select the exact fp32 matmul for every format."""
    env = dict(os.environ)
    if exact:
        env["GGNPU_FP32_MATMUL"] = "1"
        env["GGNPU_NO_PREFILL_BATCH"] = "1"
    env.update(extra_env or {})
    cmd = [REF_CLI]
    if bench_logits:
        cmd.append("bench-logits")
    cmd += ["-m", gguf_path, "-p", prompt, "-c", str(ctx), "--no-cache"]
    if not bench_logits:
        cmd += ["-n", str(n_tokens), "--temp", repr(float(temp)) if temp else "0", "--quiet"]
        if seed is not None:
            cmd += ["--seed", str(int(seed))]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
