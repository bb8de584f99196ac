"""CPU-only checks of the host side: the C-ABI library builds, loads and exports every symbol
the header declares; the synthetic-model tooling produces decodable GGUF files."""
import os
import re
import struct

import numpy as np
import pytest

from conftest import ROOT, bits
from ggnpu_b200.testing import synth as S


def test_library_exports_every_declared_symbol():
    from ggnpu_b200.build import build
    from ggnpu_b200 import backend as B
    path = build()
    assert os.path.exists(path)
    hdr = open(os.path.join(ROOT, "include", "ggb200.h")).read()
    declared = set(re.findall(r"GGB_API\s+[\w\s\*]+?\b(ggb_\w+)\s*\(", hdr))
    assert declared, "no declarations found"
    lib = B.load_library()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in ggb200.h but not exported"
    assert declared == set(B.EXPORTS)


def test_struct_layouts_match_reference_field_order():
    # field order of include/ggnpu/backend.h:21-111
    from ggnpu_b200 import backend as B
    assert [f[0] for f in B.MulMatParams._fields_] == ["A", "B", "C", "M", "N", "K", "lda", "ldb", "ldc", "n_batches",
                                                        "scales", "n_weight_scales", "B_type"]
    assert [f[0] for f in B.AttnParams._fields_] == ["Q", "K", "V", "output", "batch_size", "n_head", "head_dim",
                                                      "ctx_len", "query_pos", "freq_factors"]
    assert [int(s) for s in B.Status] == [0, 1, 2, 3, 4, 5]


def test_no_gpu_means_unavailable_not_fallback():
    """Without a usable device the factory reports NPU_UNAVAILABLE (as create_amd_xdna_backend's
    caller sees is_available()==false); it never substitutes a CPU path."""
    import torch
    from ggnpu_b200 import backend as B
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(B.BackendError) as e:
        B.CudaBackend(0)
    assert e.value.status == B.Status.NPU_UNAVAILABLE


@pytest.mark.parametrize("t", S.QUANT_TYPES)
def test_quantiser_emits_valid_blocks(oracle, t):
    import torch
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4, 1024, generator=g) * 0.02
    raw = S.quantize(x, t).numpy()
    assert raw.shape == (4, S.row_bytes(t, 1024))
    y = oracle.dequant_blocks(t, raw).reshape(4, 1024)
    err = np.linalg.norm(y - x.numpy()) / np.linalg.norm(x.numpy())
    assert err < {S.Q2_K: 0.45, S.Q3_K: 0.25}.get(t, 0.12)


def test_gguf_writer_layout(tmp_path):
    cfg = S.tiny_config(n_layer=1, vocab=64)
    m = S.build_model(cfg)
    p = tmp_path / "t.gguf"
    m.write(str(p))
    blob = p.read_bytes()
    magic, ver, n_t, n_kv = struct.unpack_from("<IIQQ", blob, 0)
    assert magic == 0x46554747 and ver == 3 and n_t == len(m.tensors) and n_kv == len(m.kv())
    # tensor data is appended in order, 32-byte aligned; the last tensor's bytes end the file
    last = list(m.tensors.values())[-1][2]
    tail = blob[len(blob) - ((last.nbytes + 31) // 32 * 32):][:last.nbytes]
    assert tail == last.tobytes()


def test_reference_cli_reads_our_gguf(tmp_path):
    from oracle.binding import REF_CLI, run_ref_cli
    if not os.path.exists(REF_CLI):
        pytest.skip("reference CLI not built")
    cfg = S.tiny_config(n_layer=1, vocab=96, seed=3)
    m = S.build_model(cfg)
    p = tmp_path / "t.gguf"
    m.write(str(p))
    r = run_ref_cli(str(p), S.prompt_text([5, 9, 2]), 3, ctx=cfg.ctx, timeout=120)
    assert r.returncode == 0, r.stderr
    assert len(S.text_ids(r.stdout)) == 3


def test_pack_cache_key_and_file_round_trip(tmp_path):
    """The packed-weight disk cache's key and file format, without a GPU.  The key follows WeightCache::make_key
    (include/ggnpu/weight_cache.h:141-152): model fingerprint and tensor name hashed together, then type and data size, so
    the same tensor name in two model files gives two keys.  A file reads back exactly; a file for another shape, with
    another source fingerprint, truncated, or with trailing bytes is refused."""
    import ctypes as C
    from ggnpu_b200.backend import load_library
    L = load_library()
    buf = C.create_string_buffer(128)

    def key(mid, name, t, size):
        assert L.ggb_pack_cache_key(mid, name, t, size, buf, 128) == 0
        return buf.value.decode()

    k1 = key(b"/models/a.gguf:1000", b"blk.0.attn_q.weight", 12, 2359296)
    assert k1 == key(b"/models/a.gguf:1000", b"blk.0.attn_q.weight", 12, 2359296)
    assert k1 != key(b"/models/b.gguf:1000", b"blk.0.attn_q.weight", 12, 2359296)      # another model file
    assert k1 != key(b"/models/a.gguf:1000", b"blk.1.attn_q.weight", 12, 2359296)
    assert k1 != key(b"/models/a.gguf:1000", b"blk.0.attn_q.weight", 14, 2359296)
    assert k1.endswith("_t12_2359296") and k1.startswith("p1_")
    assert L.ggb_pack_cache_key(b"m", b"t", 12, 1, buf, 8) != 0                          # buffer too small

    blob = np.random.default_rng(0).integers(0, 256, 5000, dtype=np.uint8)
    off = (C.c_uint64 * 4)(0, 1024, 2**64 - 1, 2**64 - 1)
    path = str(tmp_path / "w.ggbpack").encode()
    assert L.ggb_pack_file_write(path, 12, 64, 512, 2, 1, off, 777, blob.ctypes.data, blob.size) == 0
    nb, layout, n = C.c_int(), C.c_int(), C.c_uint64()
    got_off = (C.c_uint64 * 4)()
    out = np.zeros(8192, np.uint8)
    args = (C.byref(nb), C.byref(layout), got_off, out.ctypes.data, out.size, C.byref(n))
    assert L.ggb_pack_file_read(path, 12, 64, 512, 777, *args) == 0
    assert (nb.value, layout.value, n.value) == (2, 1, 5000) and list(got_off) == list(off)
    assert np.array_equal(out[:5000], blob)
    assert L.ggb_pack_file_read(path, 12, 64, 512, 0, *args) == 0                        # fingerprint 0: not checked
    assert L.ggb_pack_file_read(path, 12, 64, 512, 778, *args) == 1                      # stale: other source bytes
    assert L.ggb_pack_file_read(path, 14, 64, 512, 777, *args) == 1                      # other type
    assert L.ggb_pack_file_read(path, 12, 65, 512, 777, *args) == 1                      # other shape
    assert L.ggb_pack_file_read(str(tmp_path / "none").encode(), 12, 64, 512, 777, *args) == 2   # NOT_FOUND
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[:-10])
    assert L.ggb_pack_file_read(path, 12, 64, 512, 777, *args) == 1                      # truncated
    open(path, "wb").write(raw + b"x")
    assert L.ggb_pack_file_read(path, 12, 64, 512, 777, *args) == 1                      # trailing bytes
    assert not [f for f in os.listdir(tmp_path) if ".tmp." in f]                        # written through a temporary name


def test_model_description_mirror_and_lfm2_tensor_names():
    """The ctypes mirror of ggb_model_desc has the header's fields in the header's order (the library reads it by
    offset), and every tensor an lfm2 model carries has a slot in the generic graph."""
    import re
    from ggnpu_b200 import backend as B
    hdr = open(os.path.join(ROOT, "include", "ggb200.h")).read()
    body = hdr[hdr.index("typedef struct ggb_model_desc {"):hdr.index("} ggb_model_desc;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for decl in body.split("{", 1)[1].split(";"):
        decl = decl.strip()
        if decl:
            names += [n.strip() for n in decl.split(None, 1)[1].split(",")]
    assert names == [f[0] for f in B.ModelDesc._fields_]
    cfg = S.tiny_config(**S.LFM2_CASES["lfm2"])
    m = S.build_model(cfg)
    conv = attn = 0
    for name in m.tensors:
        if name in B._SLOTS:
            continue
        blk, layer, rest = name.split(".", 2)
        assert blk == "blk" and rest in B._LAYER_SLOTS, name
        conv += rest == "shortconv.conv.weight"
        attn += rest == "attn_q.weight"
    assert conv == len(cfg.conv_layers) and attn == cfg.n_layer - conv
    assert m.kv()["lfm2.shortconv.l_cache"] == cfg.d_conv and "token_embd_norm.weight" in m.tensors
