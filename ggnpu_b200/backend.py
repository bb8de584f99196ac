"""Host-side mirror of ggnpu's Backend interface over the C ABI of libggb200.so.

`CudaBackend` has the reference's method names, argument meaning and status
codes (include/ggnpu/backend.h:113-160): mul_mat_q, rms_norm, rope,
rope_batched, matmul_bf16, softmax, silu, gelu, flash_attn, sync,
is_available, name, last_error.  Arrays are numpy (host memory), as the
reference's callers hold every activation in host memory.  `Model` wraps the
device-resident path (packed weights, paged KV, CUDA-graph decode).

There is no CPU fallback: if the library is missing or no B200 is usable the
constructors raise.
"""
from __future__ import annotations

import ctypes as C
import enum
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libggb200.so")


class Status(enum.IntEnum):
    """ggnpu::Status, include/ggnpu/backend.h:12-19."""
    OK = 0
    ERROR = 1
    NOT_FOUND = 2
    INVALID_PARAM = 3
    NPU_UNAVAILABLE = 4
    OUT_OF_MEMORY = 5


class MulMatParams(C.Structure):
    _fields_ = [("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
                ("lda", C.c_int), ("ldb", C.c_int), ("ldc", C.c_int), ("n_batches", C.c_int32), ("scales", C.c_void_p),
                ("n_weight_scales", C.c_int), ("B_type", C.c_uint32)]


class RmsNormParams(C.Structure):
    _fields_ = [("input", C.c_void_p), ("output", C.c_void_p), ("size", C.c_int), ("eps", C.c_float), ("weight", C.c_void_p)]


class RopeParams(C.Structure):
    _fields_ = [("data", C.c_void_p), ("n_dims", C.c_int), ("offset", C.c_int64), ("freq_scale", C.c_float),
                ("freq_base", C.c_float), ("rope_dims", C.c_int64), ("cos_table", C.c_void_p), ("sin_table", C.c_void_p),
                ("neox_split_half", C.c_uint8)]


class RopeBatchedParams(C.Structure):
    _fields_ = [("data", C.c_void_p), ("n_heads", C.c_int), ("n_dims", C.c_int), ("offset", C.c_int64),
                ("freq_scale", C.c_float), ("freq_base", C.c_float), ("rope_dims", C.c_int64), ("cos_table", C.c_void_p),
                ("sin_table", C.c_void_p), ("neox_split_half", C.c_uint8)]


class SoftmaxParams(C.Structure):
    _fields_ = [("input", C.c_void_p), ("output", C.c_void_p), ("rows", C.c_int), ("cols", C.c_int)]


class UnaryParams(C.Structure):
    _fields_ = [("input", C.c_void_p), ("output", C.c_void_p), ("size", C.c_int)]


class AttnParams(C.Structure):
    _fields_ = [("Q", C.c_void_p), ("K", C.c_void_p), ("V", C.c_void_p), ("output", C.c_void_p), ("batch_size", C.c_int),
                ("n_head", C.c_int), ("head_dim", C.c_int), ("ctx_len", C.c_int64), ("query_pos", C.c_int64),
                ("freq_factors", C.c_void_p)]


class AttnPagedParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("block_table", C.c_void_p),
                ("out", C.c_void_p), ("n_head", C.c_int), ("n_kv", C.c_int), ("head_dim", C.c_int), ("page", C.c_int),
                ("n_pages", C.c_int), ("pos", C.c_int)]


class MoeParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("resid", C.c_void_p), ("y", C.c_void_p), ("router", C.c_void_p),
                ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
                ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p), ("sh_gate_inp", C.c_void_p),
                ("hidden", C.c_int), ("eff", C.c_int), ("eff_sh", C.c_int), ("n_expert", C.c_int), ("top_k", C.c_int),
                ("sel_out", C.c_void_p), ("w_out", C.c_void_p), ("ep_first", C.c_int), ("ep_local", C.c_int),
                ("gamma", C.c_void_p), ("eps", C.c_float)]


class DeltaNetParams(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("mixed", "zgate", "araw", "braw", "conv_w", "ssm_a", "dt_bias", "ssm_norm",
                                           "conv_state", "rec_state", "out")] + \
               [("n_khead", C.c_int), ("n_vhead", C.c_int), ("sk", C.c_int), ("conv_k", C.c_int), ("rms_eps", C.c_float)]


class ModelDesc(C.Structure):
    _fields_ = [("n_layer", C.c_int), ("hidden", C.c_int), ("n_head", C.c_int), ("n_kv", C.c_int), ("head_dim", C.c_int),
                ("ffn", C.c_int), ("vocab", C.c_int), ("ctx", C.c_int), ("rms_eps", C.c_float), ("rope_base", C.c_float),
                ("rope_scale", C.c_float), ("rope_neox", C.c_int), ("kv_page", C.c_int), ("conv_taps", C.c_int)]


class Q35Desc(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layer", "hidden", "n_head", "n_kv", "head_dim", "rope_dim", "conv_k", "sk", "n_vhead",
                                        "n_khead", "n_expert", "top_k", "eff", "vocab", "ctx")] + \
               [("rms_eps", C.c_float), ("rope_base", C.c_float), ("kv_page", C.c_int)]


# every symbol include/ggb200.h declares
EXPORTS = [
    "ggb_create", "ggb_destroy", "ggb_mul_mat_q", "ggb_rms_norm", "ggb_rope", "ggb_rope_batched", "ggb_matmul_bf16",
    "ggb_softmax", "ggb_silu", "ggb_gelu", "ggb_flash_attn", "ggb_sync", "ggb_is_available", "ggb_name", "ggb_last_error",
    "ggb_last_error_message", "ggb_dequant_rows", "ggb_weight_upload", "ggb_weight_free", "ggb_weight_bytes",
    "ggb_gemv_device", "ggb_gemv_swiglu_device", "ggb_attn_paged_device", "ggb_attn_prefill_device", "ggb_attn_paged_static", "ggb_stream", "ggb_launch_count", "ggb_model_create", "ggb_model_destroy",
    "ggb_model_set_tensor", "ggb_model_finalize", "ggb_model_prefill", "ggb_model_decode", "ggb_model_generate",
    "ggb_model_read_kv", "ggb_model_decode_bytes", "ggb_model_generate_spec", "ggb_model_set_cache", "ggb_model_cache_stats", "ggb_weight_upload_cached",
    "ggb_sample", "ggb_sample_device", "ggb_model_generate_sampled", "ggb_model_set_sequences", "ggb_model_select_sequence", "ggb_model_decode_batch", "ggb_model_generate_batch",
    "ggb_pack_cache_key", "ggb_pack_file_write", "ggb_pack_file_read", "ggb_tp_unique_id", "ggb_tp_init", "ggb_tp_all_reduce_device", "ggb_tp_ipc_handle", "ggb_tp_attach_peers", "ggb_moe_ffn_device", "ggb_deltanet_step_device", "ggb_qgate_split_device", "ggb_attn_gate_device",
    "ggb_q35_create", "ggb_q35_destroy", "ggb_q35_set_tensor", "ggb_q35_finalize", "ggb_q35_reset", "ggb_q35_prefill", "ggb_q35_decode",
    "ggb_q35_generate", "ggb_q35_read_state", "ggb_q35_decode_bytes",
]

_lib = None


def load_library() -> C.CDLL:
    """dlopen libggb200.so and declare the signatures.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m ggnpu_b200.build` (there is no CPU fallback)")
    L = C.CDLL(LIB_PATH)
    vp, i32, i64, u32, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_uint32, C.c_float
    L.ggb_create.argtypes = [i32, C.POINTER(vp)]
    L.ggb_destroy.argtypes = [vp]
    L.ggb_destroy.restype = None
    for name, st in [("ggb_mul_mat_q", MulMatParams), ("ggb_rms_norm", RmsNormParams), ("ggb_rope", RopeParams),
                     ("ggb_rope_batched", RopeBatchedParams), ("ggb_softmax", SoftmaxParams), ("ggb_silu", UnaryParams),
                     ("ggb_gelu", UnaryParams), ("ggb_flash_attn", AttnParams)]:
        getattr(L, name).argtypes = [vp, C.POINTER(st)]
    L.ggb_matmul_bf16.argtypes = [vp, vp, vp, vp, i32, i32, i32]
    L.ggb_sync.argtypes = [vp]
    L.ggb_sync.restype = None
    L.ggb_is_available.argtypes = [vp]
    L.ggb_name.argtypes = [vp]
    L.ggb_name.restype = C.c_char_p
    L.ggb_last_error.argtypes = [vp]
    L.ggb_last_error_message.argtypes = [vp]
    L.ggb_last_error_message.restype = C.c_char_p
    L.ggb_dequant_rows.argtypes = [vp, u32, vp, i64, i32, i64, i64, vp]
    L.ggb_weight_upload.argtypes = [vp, u32, i64, i32, vp, C.POINTER(vp)]
    L.ggb_weight_free.argtypes = [vp, vp]
    L.ggb_weight_free.restype = None
    L.ggb_weight_bytes.argtypes = [vp]
    L.ggb_weight_bytes.restype = C.c_size_t
    L.ggb_gemv_device.argtypes = [vp, vp, vp, i32, i32, vp, i32, i32, vp, vp, f32]
    L.ggb_gemv_swiglu_device.argtypes = [vp, vp, vp, vp, i32, i32, vp, i32, vp, f32]
    L.ggb_attn_paged_device.argtypes = [vp, C.POINTER(AttnPagedParams)]
    L.ggb_attn_prefill_device.argtypes = [vp, C.POINTER(AttnPagedParams), i32]
    L.ggb_moe_ffn_device.argtypes = [vp, C.POINTER(MoeParams)]
    L.ggb_deltanet_step_device.argtypes = [vp, C.POINTER(DeltaNetParams)]
    L.ggb_qgate_split_device.argtypes = [vp, vp, vp, i32, i32]
    L.ggb_attn_gate_device.argtypes = [vp, vp, vp, i32, i32]
    L.ggb_tp_unique_id.argtypes = [vp]
    L.ggb_tp_init.argtypes = [vp, vp, i32, i32]
    L.ggb_tp_all_reduce_device.argtypes = [vp, vp, i64]
    L.ggb_tp_ipc_handle.argtypes = [vp, vp]
    L.ggb_tp_attach_peers.argtypes = [vp, vp]
    L.ggb_attn_paged_static.argtypes = [vp, C.POINTER(AttnPagedParams)]
    L.ggb_stream.argtypes = [vp]
    L.ggb_stream.restype = vp
    L.ggb_launch_count.argtypes = [vp]
    L.ggb_launch_count.restype = C.c_uint64
    L.ggb_model_create.argtypes = [vp, C.POINTER(ModelDesc), C.POINTER(vp)]
    L.ggb_model_destroy.argtypes = [vp]
    L.ggb_model_destroy.restype = None
    L.ggb_model_set_tensor.argtypes = [vp, i32, i32, u32, i64, i32, vp]
    L.ggb_model_finalize.argtypes = [vp]
    L.ggb_model_prefill.argtypes = [vp, vp, i32, i32, vp, C.POINTER(C.c_int32)]
    L.ggb_model_decode.argtypes = [vp, C.c_int32, i32, vp, C.POINTER(C.c_int32)]
    L.ggb_model_generate.argtypes = [vp, C.c_int32, i32, i32, vp]
    L.ggb_model_read_kv.argtypes = [vp, i32, i32, i32, vp]
    L.ggb_model_generate_spec.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp]
    L.ggb_model_set_sequences.argtypes = [vp, i32]
    L.ggb_sample.argtypes = [vp, vp, i32, f32, vp, vp]
    L.ggb_sample_device.argtypes = [vp, vp, i32, f32, vp, vp]
    L.ggb_model_generate_sampled.argtypes = [vp, i32, i32, i32, f32, vp, vp]
    L.ggb_model_select_sequence.argtypes = [vp, i32]
    L.ggb_model_decode_batch.argtypes = [vp, vp, vp, i32, vp, vp]
    L.ggb_model_generate_batch.argtypes = [vp, vp, vp, i32, i32, vp]
    L.ggb_model_set_cache.argtypes = [vp, C.c_char_p, C.c_char_p]
    L.ggb_model_cache_stats.argtypes = [vp, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.ggb_weight_upload_cached.argtypes = [vp, C.c_char_p, C.c_char_p, C.c_char_p, u32, i64, i32, vp, C.POINTER(vp), C.POINTER(C.c_int)]
    L.ggb_pack_cache_key.argtypes = [C.c_char_p, C.c_char_p, u32, C.c_uint64, C.c_char_p, i32]
    L.ggb_pack_file_write.argtypes = [C.c_char_p, u32, i64, i32, i32, i32, vp, C.c_uint64, vp, C.c_uint64]
    L.ggb_pack_file_read.argtypes = [C.c_char_p, u32, i64, i32, C.c_uint64, C.POINTER(C.c_int), C.POINTER(C.c_int), vp, vp, C.c_uint64,
                                     C.POINTER(C.c_uint64)]
    L.ggb_model_decode_bytes.argtypes = [vp, i32]
    L.ggb_model_decode_bytes.restype = C.c_uint64
    L.ggb_q35_create.argtypes = [vp, vp, C.POINTER(vp)]
    L.ggb_q35_destroy.argtypes = [vp]
    L.ggb_q35_destroy.restype = None
    L.ggb_q35_set_tensor.argtypes = [vp, i32, i32, u32, i64, i32, vp]
    L.ggb_q35_finalize.argtypes = [vp]
    L.ggb_q35_reset.argtypes = [vp]
    L.ggb_q35_prefill.argtypes = [vp, vp, i32, i32, vp, C.POINTER(C.c_int32)]
    L.ggb_q35_decode.argtypes = [vp, C.c_int32, i32, vp, C.POINTER(C.c_int32)]
    L.ggb_q35_generate.argtypes = [vp, C.c_int32, i32, i32, vp]
    L.ggb_q35_read_state.argtypes = [vp, i32, vp]
    L.ggb_q35_decode_bytes.argtypes = [vp, i32]
    L.ggb_q35_decode_bytes.restype = C.c_uint64
    _lib = L
    return L


def _ptr(a):
    return None if a is None else a.ctypes.data


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class BackendError(RuntimeError):
    def __init__(self, status: Status, message: str):
        super().__init__(f"{status.name}: {message}")
        self.status = status


class CudaBackend:
    """The reference's `Backend` (include/ggnpu/backend.h:113-160), CUDA-backed.

    Methods return a `Status`; outputs are written into the arrays passed in,
    exactly as the reference writes through the caller's pointers."""

    def __init__(self, device: int = 0):
        self.lib = load_library()
        h = C.c_void_p()
        st = Status(self.lib.ggb_create(device, C.byref(h)))
        if st != Status.OK:
            raise BackendError(st, f"ggb_create(device={device}) failed: no usable sm_100 GPU")
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            for m in list(getattr(self, "_models", ())):      # models hold pointers into the handle: they go first
                m.close()
            self.lib.ggb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- Backend interface ------------------------------------------------
    def mul_mat_q(self, A, B, C_out, M, N, K, B_type, lda=None, ldb=None, ldc=None) -> Status:
        p = MulMatParams(_ptr(A), _ptr(B), _ptr(C_out), M, N, K, K if lda is None else lda, K if ldb is None else ldb,
                         N if ldc is None else ldc, 1, None, 0, int(B_type))
        return Status(self.lib.ggb_mul_mat_q(self.h, C.byref(p)))

    def rms_norm(self, input, output, size, eps, weight=None) -> Status:
        p = RmsNormParams(_ptr(input), _ptr(output), size, eps, _ptr(weight))
        return Status(self.lib.ggb_rms_norm(self.h, C.byref(p)))

    def rope(self, data, n_dims, offset, freq_scale, freq_base, rope_dims, cos_table=None, sin_table=None,
             neox_split_half=False) -> Status:
        p = RopeParams(_ptr(data), n_dims, offset, freq_scale, freq_base, rope_dims, _ptr(cos_table), _ptr(sin_table),
                       int(neox_split_half))
        return Status(self.lib.ggb_rope(self.h, C.byref(p)))

    def rope_batched(self, data, n_heads, n_dims, offset, freq_scale, freq_base, rope_dims, cos_table=None, sin_table=None,
                     neox_split_half=False) -> Status:
        p = RopeBatchedParams(_ptr(data), n_heads, n_dims, offset, freq_scale, freq_base, rope_dims, _ptr(cos_table),
                              _ptr(sin_table), int(neox_split_half))
        return Status(self.lib.ggb_rope_batched(self.h, C.byref(p)))

    def matmul_bf16(self, A, B, C_out, M, N, K) -> Status:
        return Status(self.lib.ggb_matmul_bf16(self.h, _ptr(A), _ptr(B), _ptr(C_out), M, N, K))

    def softmax(self, input, output, rows, cols) -> Status:
        p = SoftmaxParams(_ptr(input), _ptr(output), rows, cols)
        return Status(self.lib.ggb_softmax(self.h, C.byref(p)))

    def silu(self, input, output, size) -> Status:
        p = UnaryParams(_ptr(input), _ptr(output), size)
        return Status(self.lib.ggb_silu(self.h, C.byref(p)))

    def gelu(self, input, output, size) -> Status:
        p = UnaryParams(_ptr(input), _ptr(output), size)
        return Status(self.lib.ggb_gelu(self.h, C.byref(p)))

    def flash_attn(self, Q, K, V, output, n_head, head_dim, ctx_len, query_pos=-1) -> Status:
        p = AttnParams(_ptr(Q), _ptr(K), _ptr(V), _ptr(output), 1, n_head, head_dim, ctx_len, query_pos, None)
        return Status(self.lib.ggb_flash_attn(self.h, C.byref(p)))

    def sample_token(self, logits, temp, seed):
        """sample_token of the reference CLI (src/cli/main.cpp:827-864) on host logits: (token, advanced seed)."""
        lg = _f32(logits).reshape(-1)
        sd, tok = C.c_uint64(int(seed)), C.c_int32()
        self.check(self.lib.ggb_sample(self.h, _ptr(lg), lg.size, float(temp), C.byref(sd), C.byref(tok)), "sample")
        return tok.value, sd.value

    def sync(self) -> None:
        self.lib.ggb_sync(self.h)

    def is_available(self) -> bool:
        return bool(self.lib.ggb_is_available(self.h))

    def name(self) -> str:
        return self.lib.ggb_name(self.h).decode()

    def last_error(self) -> Status:
        return Status(self.lib.ggb_last_error(self.h))

    def last_error_message(self) -> str:
        return self.lib.ggb_last_error_message(self.h).decode()

    # -- device-resident extras ---------------------------------------------
    def check(self, st, what=""):
        st = Status(st)
        if st != Status.OK:
            raise BackendError(st, f"{what}: {self.last_error_message()}")

    def dequant_rows(self, type_id, raw, N, K, row0=0, n_rows=None) -> np.ndarray:
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        n_rows = N - row0 if n_rows is None else n_rows
        out = np.empty((n_rows, K), dtype=np.float32)
        self.check(self.lib.ggb_dequant_rows(self.h, int(type_id), _ptr(raw), N, K, row0, n_rows, _ptr(out)), "dequant_rows")
        return out

    def upload_weight(self, type_id, raw, N, K):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        w = C.c_void_p()
        self.check(self.lib.ggb_weight_upload(self.h, int(type_id), N, K, _ptr(raw), C.byref(w)), "weight_upload")
        return w

    def free_weight(self, w):
        self.lib.ggb_weight_free(self.h, w)

    def gemv_device(self, w, d_x, M, lda, d_y, ldc, epilogue=0, d_extra=None, d_gamma=None, eps=0.0):
        self.check(self.lib.ggb_gemv_device(self.h, w, d_x, M, lda, d_y, ldc, epilogue, d_extra, d_gamma, eps), "gemv_device")

    def gemv_swiglu_device(self, wg, wu, d_x, M, lda, d_y, ldc, d_gamma=None, eps=0.0):
        self.check(self.lib.ggb_gemv_swiglu_device(self.h, wg, wu, d_x, M, lda, d_y, ldc, d_gamma, eps), "gemv_swiglu_device")

    def upload_weight_cached(self, cache_dir, model_id, tensor_name, type_id, raw, N, K):
        """upload_weight through the packed-weight disk cache; raw may be None (load from the cache only).
        Returns (weight handle, hit)."""
        w, hit = C.c_void_p(), C.c_int()
        if raw is not None:
            raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        self.check(self.lib.ggb_weight_upload_cached(self.h, cache_dir.encode(), model_id.encode(), tensor_name.encode(), int(type_id), N, K,
                                                     _ptr(raw), C.byref(w), C.byref(hit)), "weight_upload_cached")
        return w, bool(hit.value)

    def attn_paged_device(self, q, k_cache, v_cache, block_table, out, n_head, n_kv, head_dim, page, n_pages, pos) -> Status:
        """All pointer arguments are device addresses (ints)."""
        p = AttnPagedParams(q, k_cache, v_cache, block_table, out, n_head, n_kv, head_dim, page, n_pages, pos)
        return Status(self.lib.ggb_attn_paged_device(self.h, C.byref(p)))

    def attn_prefill_device(self, q, k_cache, v_cache, block_table, out, n_head, n_kv, head_dim, page, n_pages, pos, n_tok) -> Status:
        """Causal attention of n_tok query tokens starting at position pos (device pointers)."""
        p = AttnPagedParams(q, k_cache, v_cache, block_table, out, n_head, n_kv, head_dim, page, n_pages, pos)
        return Status(self.lib.ggb_attn_prefill_device(self.h, C.byref(p), n_tok))

    def attn_paged_static(self, q, k_cache, v_cache, block_table, out, n_head, n_kv, head_dim, page, n_pages, pos) -> Status:
        """attn_paged_device without any device allocation (fixed scratch inside the library)."""
        p = AttnPagedParams(q, k_cache, v_cache, block_table, out, n_head, n_kv, head_dim, page, n_pages, pos)
        return Status(self.lib.ggb_attn_paged_static(self.h, C.byref(p)))

    def moe_ffn_device(self, **kw) -> Status:
        """Mixture-of-experts FFN of one token; keyword arguments are the fields of ggb_moe_params (device pointers / weights)."""
        p = MoeParams(**{k: (v if v is not None else None) for k, v in kw.items()})
        return Status(self.lib.ggb_moe_ffn_device(self.h, C.byref(p)))

    def qgate_split_device(self, d_qg, d_q, n_head, head_dim) -> Status:
        return Status(self.lib.ggb_qgate_split_device(self.h, d_qg, d_q, n_head, head_dim))

    def attn_gate_device(self, d_out, d_qg, n_head, head_dim) -> Status:
        return Status(self.lib.ggb_attn_gate_device(self.h, d_out, d_qg, n_head, head_dim))

    def deltanet_step_device(self, **kw) -> Status:
        """One token of a Gated DeltaNet layer; keyword arguments are the fields of ggb_deltanet_params (device pointers)."""
        p = DeltaNetParams(**kw)
        return Status(self.lib.ggb_deltanet_step_device(self.h, C.byref(p)))

    # ---- tensor-parallel group (one process per GPU, NCCL underneath) ----
    tp_rank, tp_size = 0, 1

    def tp_unique_id(self) -> bytes:
        """Rank 0: the 128-byte id every rank passes to tp_init."""
        buf = C.create_string_buffer(128)
        self.check(self.lib.ggb_tp_unique_id(buf), "tp_unique_id")
        return buf.raw

    def tp_init(self, unique_id: bytes, rank: int, size: int) -> None:
        """Collective: returns when all `size` ranks have joined."""
        buf = C.create_string_buffer(bytes(unique_id), 128)
        self.check(self.lib.ggb_tp_init(self.h, buf, rank, size), "tp_init")
        self.tp_rank, self.tp_size = rank, size

    def tp_ipc_handle(self) -> bytes:
        """This rank's exchange region for the one-shot all-reduce, as a 64-byte CUDA IPC handle."""
        buf = C.create_string_buffer(64)
        self.check(self.lib.ggb_tp_ipc_handle(self.h, buf), "tp_ipc_handle")
        return buf.raw

    def tp_attach_peers(self, handles) -> None:
        """handles: the `size` IPC handles in rank order (every rank's tp_ipc_handle())."""
        blob = b"".join(bytes(x) for x in handles)
        assert len(blob) == 64 * self.tp_size
        self.check(self.lib.ggb_tp_attach_peers(self.h, C.create_string_buffer(blob, len(blob))), "tp_attach_peers")

    def tp_all_reduce_device(self, d_buf: int, count: int) -> Status:
        return Status(self.lib.ggb_tp_all_reduce_device(self.h, d_buf, count))

    def stream(self) -> int:
        return int(self.lib.ggb_stream(self.h) or 0)

    def launch_count(self) -> int:
        return int(self.lib.ggb_launch_count(self.h))


_SLOTS = {"token_embd.weight": 0, "output.weight": 1, "output_norm.weight": 2, "rope_freqs.weight": 3,
          "token_embd_norm.weight": 2}        # lfm2 keeps its final norm under this name (src/cli/main.cpp:2853-2855)
_LAYER_SLOTS = {"attn_norm.weight": 10, "attn_q.weight": 11, "attn_k.weight": 12, "attn_v.weight": 13,
                "attn_output.weight": 14, "ffn_norm.weight": 15, "ffn_gate.weight": 16, "ffn_up.weight": 17,
                "ffn_down.weight": 18, "attn_q.bias": 19, "attn_k.bias": 20, "attn_v.bias": 21, "attn_q_norm.weight": 22,
                "attn_k_norm.weight": 23,
                "shortconv.in_proj.weight": 24, "shortconv.out_proj.weight": 25, "shortconv.conv.weight": 26}


class Model:
    """A llama / qwen2 / qwen3 / lfm2-style decoder resident in HBM.

    `tensors` maps GGUF tensor names to (ggml type id, dims with dims[0]=K, raw bytes),
    the form ggnpu_b200.testing.synth.SynthModel.tensors has."""

    def __init__(self, backend: CudaBackend, cfg, tensors: dict, cache_dir: str | None = None, model_id: str = "", n_seq: int = 1,
                 rope_neox: int | None = None, rope_base: float | None = None):
        """rope_neox / rope_base override what the architecture implies (qwen3 and lfm2: split-half pairs at the model's
        base); rope_neox=0, rope_base=10000 on an lfm2 model is the rotation the reference CLI applies on its CPU backend."""
        self.b, self.cfg = backend, cfg
        L = backend.lib
        if backend.tp_size > 1:          # this process holds one shard; `cfg` and `tensors` describe the full model
            from . import tp
            tensors = tp.shard_tensors(cfg, tensors, backend.tp_rank, backend.tp_size)
            cfg = tp.shard_config(cfg, backend.tp_size)
        self.cfg_local = cfg
        neox = (1 if cfg.arch in ("qwen3", "lfm2") else 0) if rope_neox is None else int(rope_neox)
        base = cfg.rope_base if rope_base is None else rope_base
        desc = ModelDesc(cfg.n_layer, cfg.hidden, cfg.n_head, cfg.n_kv, cfg.head_dim, cfg.ffn, cfg.vocab, cfg.ctx,
                         cfg.rms_eps, float(np.float32(base)), 1.0, neox, 0, getattr(cfg, "d_conv", 0) if cfg.arch == "lfm2" else 0)
        m = C.c_void_p()
        backend.check(L.ggb_model_create(backend.h, C.byref(desc), C.byref(m)), "model_create")
        self.m = m
        if n_seq > 1:                    # KV streams for batched sequences
            backend.check(L.ggb_model_set_sequences(m, n_seq), "model_set_sequences")
        if cache_dir:                    # packed-weight disk cache for the matrices
            backend.check(L.ggb_model_set_cache(m, cache_dir.encode(), model_id.encode()), "model_set_cache")
        if not hasattr(backend, "_models"):
            import weakref
            backend._models = weakref.WeakSet()
        backend._models.add(self)
        for name, (tid, dims, raw) in tensors.items():
            raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
            if name in _SLOTS:
                slot, layer = _SLOTS[name], -1
            else:
                parts = name.split(".", 2)
                if parts[0] != "blk" or parts[2] not in _LAYER_SLOTS:
                    raise KeyError(f"tensor {name} has no slot in the generic graph")
                slot, layer = _LAYER_SLOTS[parts[2]], int(parts[1])
            n, k = (dims[1], dims[0]) if len(dims) == 2 else (dims[0], 1)
            if slot == 26:               # F32 {taps, hidden}: one vector of hidden x taps values
                n, k = dims[0] * dims[1], 1
            backend.check(L.ggb_model_set_tensor(m, slot, layer, int(tid), n, k, _ptr(raw)), f"set_tensor({name})")
        backend.check(L.ggb_model_finalize(m), "model_finalize")

    def prefill(self, tokens, pos0=0, want_logits=True):
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.cfg.vocab, dtype=np.float32) if want_logits else None
        nxt = C.c_int32()
        self.b.check(self.b.lib.ggb_model_prefill(self.m, _ptr(toks), toks.size, pos0, _ptr(logits), C.byref(nxt)), "prefill")
        return logits, nxt.value

    def decode(self, token, pos, want_logits=True, logits_out=None):
        logits = logits_out if logits_out is not None else (np.empty(self.cfg.vocab, dtype=np.float32) if want_logits else None)
        nxt = C.c_int32()
        self.b.check(self.b.lib.ggb_model_decode(self.m, int(token), int(pos), _ptr(logits), C.byref(nxt)), "decode")
        return logits, nxt.value

    def generate(self, first_token, pos0, n):
        out = np.empty(n, dtype=np.int32)
        self.b.check(self.b.lib.ggb_model_generate(self.m, int(first_token), int(pos0), n, _ptr(out)), "generate")
        return out

    def generate_spec(self, history, pos0, n, draft_k=8):
        """Greedy generation with prompt-lookup speculative decoding; history ends with the token to feed at pos0.
        Returns (tokens, stats dict)."""
        hist = np.ascontiguousarray(history, dtype=np.int32)
        out = np.empty(n, dtype=np.int32)
        st = np.zeros(4, dtype=np.int32)
        self.b.check(self.b.lib.ggb_model_generate_spec(self.m, _ptr(hist), hist.size, int(pos0), n, draft_k, _ptr(out), _ptr(st)), "generate_spec")
        return out[:st[3]], {"steps": int(st[0]), "drafted": int(st[1]), "accepted": int(st[2])}

    def generate_sampled(self, first_token, pos0, n, temp, seed):
        """n steps with the reference CLI's temperature sampling; returns (tokens, advanced seed)."""
        out = np.empty(n, dtype=np.int32)
        sd = C.c_uint64(int(seed))
        self.b.check(self.b.lib.ggb_model_generate_sampled(self.m, int(first_token), int(pos0), n, float(temp), C.byref(sd), _ptr(out)), "generate_sampled")
        return out, sd.value

    def select_sequence(self, seq):
        """The KV stream prefill / decode / read_kv work on (streams are reserved with n_seq at construction)."""
        self.b.check(self.b.lib.ggb_model_select_sequence(self.m, int(seq)), "select_sequence")

    def decode_batch(self, tokens, pos, want_logits=True):
        """One step of len(tokens) sequences: row r is sequence r's next token at position pos[r].
        Returns (logits [n_seq][vocab] or None, greedy next tokens)."""
        toks, p = np.ascontiguousarray(tokens, dtype=np.int32), np.ascontiguousarray(pos, dtype=np.int32)
        logits = np.empty((toks.size, self.cfg.vocab), dtype=np.float32) if want_logits else None
        nxt = np.empty(toks.size, dtype=np.int32)
        self.b.check(self.b.lib.ggb_model_decode_batch(self.m, _ptr(toks), _ptr(p), toks.size, _ptr(logits), _ptr(nxt)), "decode_batch")
        return logits, nxt

    def generate_batch(self, first_tokens, pos0, n):
        """n greedy steps of len(first_tokens) sequences with device-side feedback; returns ids [n][n_seq]."""
        toks, p = np.ascontiguousarray(first_tokens, dtype=np.int32), np.ascontiguousarray(pos0, dtype=np.int32)
        out = np.empty((n, toks.size), dtype=np.int32)
        self.b.check(self.b.lib.ggb_model_generate_batch(self.m, _ptr(toks), _ptr(p), toks.size, n, _ptr(out)), "generate_batch")
        return out

    def read_kv(self, layer, pos, want_v):
        out = np.empty((self.cfg_local.n_kv, self.cfg_local.head_dim), dtype=np.float32)
        self.b.check(self.b.lib.ggb_model_read_kv(self.m, layer, pos, int(want_v), _ptr(out)), "read_kv")
        return out

    def decode_bytes(self, pos) -> int:
        return int(self.b.lib.ggb_model_decode_bytes(self.m, pos))

    def cache_stats(self):
        """(matrices loaded from packed files, matrices packed and written) of the packed-weight disk cache."""
        h, mi = C.c_int(), C.c_int()
        self.b.lib.ggb_model_cache_stats(self.m, C.byref(h), C.byref(mi))
        return h.value, mi.value

    def close(self):
        if getattr(self, "m", None):
            if getattr(self.b, "h", None):                    # a destroyed handle took its models' memory with the context
                self.b.lib.ggb_model_destroy(self.m)
            self.m = None
            try:
                self.b._models.discard(self)
            except Exception:
                pass

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_Q35_SLOTS = {"token_embd.weight": 0, "output.weight": 1, "output_norm.weight": 2}
_Q35_LAYER_SLOTS = {
    "attn_norm.weight": 10, "post_attention_norm.weight": 11,
    "attn_qkv.weight": 20, "attn_gate.weight": 21, "ssm_alpha.weight": 22, "ssm_beta.weight": 23, "ssm_conv1d.weight": 24,
    "ssm_a": 25, "ssm_dt.bias": 26, "ssm_norm.weight": 27, "ssm_out.weight": 28,
    "attn_q.weight": 30, "attn_k.weight": 31, "attn_v.weight": 32, "attn_output.weight": 33, "attn_q_norm.weight": 34,
    "attn_k_norm.weight": 35,
    "ffn_gate_inp.weight": 40, "ffn_gate_exps.weight": 41, "ffn_up_exps.weight": 42, "ffn_down_exps.weight": 43,
    "ffn_gate_shexp.weight": 44, "ffn_up_shexp.weight": 45, "ffn_down_shexp.weight": 46, "ffn_gate_inp_shexp.weight": 47,
}
_Q35_EXPERT = ("ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight")


class Q35Model:
    """A qwen35moe decoder (Gated DeltaNet + gated full attention + mixture-of-experts FFN, the reference's
    src/cli/main.cpp:2859-3232) resident in HBM.  `tensors` as ggnpu_b200.testing.synth.build_q35_model makes them.
    On a backend that joined a group the model is expert parallel: this process keeps its slice of the
    experts (a contiguous range along the expert axis), everything else is replicated."""

    def __init__(self, backend: CudaBackend, cfg, tensors: dict):
        self.b, self.cfg = backend, cfg
        L = backend.lib
        desc = Q35Desc(cfg.n_layer, cfg.hidden, cfg.n_head, cfg.n_kv, cfg.head_dim, cfg.rope_dim, cfg.conv_k, cfg.sk, cfg.n_vhead,
                       cfg.n_khead, cfg.n_expert, cfg.top_k, cfg.eff, cfg.vocab, cfg.ctx, cfg.rms_eps,
                       float(np.float32(cfg.rope_base)), 0)
        m = C.c_void_p()
        backend.check(L.ggb_q35_create(backend.h, C.byref(desc), C.byref(m)), "q35_create")
        self.m = m
        if not hasattr(backend, "_models"):
            import weakref
            backend._models = weakref.WeakSet()
        backend._models.add(self)
        rank, size = backend.tp_rank, backend.tp_size
        for name, (tid, dims, raw) in tensors.items():
            raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
            if name in _Q35_SLOTS:
                slot, layer, key = _Q35_SLOTS[name], -1, name
            else:
                parts = name.split(".", 2)
                if parts[0] != "blk" or parts[2] not in _Q35_LAYER_SLOTS:
                    raise KeyError(f"tensor {name} has no slot in the qwen35moe graph")
                slot, layer, key = _Q35_LAYER_SLOTS[parts[2]], int(parts[1]), parts[2]
            if len(dims) == 3:                      # expert tensor [K, N, n_expert]: experts stacked along N
                k, n_exp = dims[0], dims[2]
                n = dims[1] * n_exp
                if size > 1 and key in _Q35_EXPERT:
                    per = raw.size // n_exp
                    nl = n_exp // size
                    raw = np.ascontiguousarray(raw[rank * nl * per:(rank + 1) * nl * per])
                    n = dims[1] * nl
            elif len(dims) == 2:
                n, k = dims[1], dims[0]
            else:
                n, k = dims[0], 1
            backend.check(L.ggb_q35_set_tensor(m, slot, layer, int(tid), n, k, _ptr(raw)), f"q35_set_tensor({name})")
        backend.check(L.ggb_q35_finalize(m), "q35_finalize")

    def reset(self):
        self.b.check(self.b.lib.ggb_q35_reset(self.m), "q35_reset")

    def prefill(self, tokens, pos0=0, want_logits=True):
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.cfg.vocab, dtype=np.float32) if want_logits else None
        nxt = C.c_int32()
        self.b.check(self.b.lib.ggb_q35_prefill(self.m, _ptr(toks), toks.size, pos0, _ptr(logits), C.byref(nxt)), "q35_prefill")
        return logits, nxt.value

    def decode(self, token, pos, want_logits=True):
        logits = np.empty(self.cfg.vocab, dtype=np.float32) if want_logits else None
        nxt = C.c_int32()
        self.b.check(self.b.lib.ggb_q35_decode(self.m, int(token), int(pos), _ptr(logits), C.byref(nxt)), "q35_decode")
        return logits, nxt.value

    def generate(self, first_token, pos0, n):
        out = np.empty(n, dtype=np.int32)
        self.b.check(self.b.lib.ggb_q35_generate(self.m, int(first_token), int(pos0), n, _ptr(out)), "q35_generate")
        return out

    def rec_state(self, layer):
        c = self.cfg
        out = np.empty((c.n_vhead, c.sk, c.sk), dtype=np.float32)
        self.b.check(self.b.lib.ggb_q35_read_state(self.m, layer, _ptr(out)), "q35_read_state")
        return out

    def decode_bytes(self, pos) -> int:
        return int(self.b.lib.ggb_q35_decode_bytes(self.m, pos))

    def close(self):
        if getattr(self, "m", None):
            if getattr(self.b, "h", None):
                self.b.lib.ggb_q35_destroy(self.m)
            self.m = None
            try:
                self.b._models.discard(self)
            except Exception:
                pass

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
