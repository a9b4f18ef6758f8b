"""GGUF parser and weight loader (muser_b200/gguf.py) against the reference's own container tests
(crates/muser-engine/src/gguf/tests.rs, src/weights.rs:448-560), restated on byte strings built here."""
import io
import struct

import numpy as np
import pytest

from muser_b200 import gguf as G
from oracle import oracle as O


def header(n_tensors, n_kv, version=3):
    return struct.pack("<IIQQ", G.GGUF_MAGIC, version, n_tensors, n_kv)


def kv_string(key, value):
    k, v = key.encode(), value.encode()
    return struct.pack("<Q", len(k)) + k + struct.pack("<I", 8) + struct.pack("<Q", len(v)) + v


def test_parse_minimal_gguf():  # gguf/tests.rs:23-31
    g = G.GgufFile.parse(io.BytesIO(header(0, 1) + kv_string("general.architecture", "qwen2")))
    assert g.version == 3 and g.meta_str("general.architecture") == "qwen2" and g.tensors == []


def test_rejects_counts_that_cannot_fit_in_the_input():  # gguf/tests.rs:46-55
    with pytest.raises(G.GgufError) as e:
        G.GgufFile.parse(io.BytesIO(header(0, 10_000)))
    assert e.value.kind == "LimitExceeded"


def test_rejects_zero_alignment():  # gguf/tests.rs:57-72
    key = b"general.alignment"
    data = header(0, 1) + struct.pack("<Q", len(key)) + key + struct.pack("<II", 4, 0)
    with pytest.raises(G.GgufError) as e:
        G.GgufFile.parse(io.BytesIO(data))
    assert e.value.kind == "InvalidAlignment"


def test_rejects_duplicate_metadata_keys_and_tensor_names():  # gguf/tests.rs:74-113
    with pytest.raises(G.GgufError) as e:
        G.GgufFile.parse(io.BytesIO(header(0, 2) + kv_string("tokenizer.chat_template", "first") + kv_string("tokenizer.chat_template", "second")))
    assert e.value.kind == "DuplicateMetadataKey"
    data = header(2, 0)
    for offset in (0, 4):
        name = b"duplicate.weight"
        data += struct.pack("<Q", len(name)) + name + struct.pack("<IQIQ", 1, 1, 0, offset)
    data += b"\0" * ((len(data) + 31) // 32 * 32 + 8 - len(data))
    with pytest.raises(G.GgufError) as e:
        G.GgufFile.parse(io.BytesIO(data))
    assert e.value.kind == "DuplicateTensorName"


def test_bad_magic_version_type_and_out_of_bounds():
    with pytest.raises(G.GgufError) as e:
        G.GgufFile.parse(io.BytesIO(struct.pack("<IIQQ", 0x12345678, 3, 0, 0)))
    assert e.value.kind == "BadMagic"
    with pytest.raises(G.GgufError) as e:
        G.GgufFile.parse(io.BytesIO(header(0, 0, version=4)))
    assert e.value.kind == "UnsupportedVersion"
    name = b"t"
    one = header(1, 0) + struct.pack("<Q", 1) + name + struct.pack("<IQ", 1, 256)
    with pytest.raises(G.GgufError) as e:
        G.GgufFile.parse(io.BytesIO(one + struct.pack("<IQ", 999, 0)))
    assert e.value.kind == "UnsupportedType"
    with pytest.raises(G.GgufError) as e:  # a Q4_K block of 144 bytes that the file does not hold
        G.GgufFile.parse(io.BytesIO(one + struct.pack("<IQ", G.Q4_K, 0) + b"\0" * 64))
    assert e.value.kind == "TensorOutOfBounds"


def test_metadata_value_types_round_trip(tmp_path):
    meta = {"a.u8": (0, 7), "a.i8": (1, -7), "a.u16": (2, 65535), "a.i16": (3, -3), "a.u32": (4, 1 << 31), "a.i32": (5, -5),
            "a.f32": (6, 0.25), "a.bool": (7, True), "a.str": (8, "muse"), "a.arr": (9, (8, ["x", "yz"])),
            "a.nested": (9, (9, [(4, [1, 2]), (4, [3])])), "a.u64": (10, 1 << 40), "a.i64": (11, -(1 << 40)), "a.f64": (12, 1e-300)}
    p = tmp_path / "meta.gguf"
    G.write_gguf(p, {}, meta)
    g = G.GgufFile.parse_path(p)
    assert g.metadata["a.u32"] == (4, 1 << 31) and g.metadata["a.i64"][1] == -(1 << 40) and g.metadata["a.bool"][1] is True
    assert g.metadata["a.arr"][1] == ["x", "yz"] and g.metadata["a.nested"][1] == [[1, 2], [3]]
    assert g.meta_str("a.str") == "muse" and g.meta_u32("a.u32") == 1 << 31 and g.meta_str("a.u32") is None


# ---- the NVFP4 loader fixture of weights.rs:448-503: one 16-wide row with scale 1.0 (0x38) and scale2 0.25
PACKED = bytes([0x10, 0x32, 0x54, 0x76, 0x98, 0xba, 0xdc, 0xfe])


def nvfp4_fixture(tmp_path, include_scales=True, input_scale_inv=None, scale_byte=0x38, precision=None):
    tensors = {"matrix": (G.NVFP4_E2M1, [16, 1], PACKED)}
    if include_scales:
        tensors["matrix.nvfp4_scale"] = (G.F8_E4M3FN, [1, 1], bytes([scale_byte]))
        tensors["matrix.nvfp4_scale2"] = (G.F32, [1], struct.pack("<f", 0.25))
        if input_scale_inv is not None:
            tensors["matrix.nvfp4_input_scale_inv"] = (G.F32, [1], struct.pack("<f", input_scale_inv))
    meta = {}
    if precision or input_scale_inv is not None:
        meta["muser.activation_precision"] = (8, precision or "nvfp4")
    p = tmp_path / "fixture.gguf"
    G.write_gguf(p, tensors, meta)
    return p


def test_native_nvfp4_view_binds_companions_and_dequantizes_exactly(tmp_path):  # weights.rs:518-536
    w = G.MuseWeights.open(nvfp4_fixture(tmp_path))
    v = w.view("matrix")
    assert v.raw.shape == (1, 8) and bytes(v.block_scales.reshape(-1)) == b"\x38"
    assert np.float32(v.scale2).view(np.uint32) == np.float32(0.25).view(np.uint32) and v.input_scale_inv is None
    want = np.array([0.0, 0.125, 0.25, 0.375, 0.5, 0.75, 1.0, 1.5, -0.0, -0.125, -0.25, -0.375, -0.5, -0.75, -1.0, -1.5], dtype=np.float32)
    got = O.dequant_nvfp4(np.array(v.raw), np.array(v.block_scales), v.scale2)
    assert np.array_equal(got.reshape(-1).view(np.uint32), want.view(np.uint32))
    lay = w.layout("matrix")
    assert (lay.byte_len, lay.n_in, lay.n_out, lay.nvfp4_scale_len, lay.nvfp4_scale2) == (8, 16, 1, 1, 0.25)
    assert w.contains("matrix") and not w.contains("other")
    w.close()


def test_native_nvfp4_loader_fails_closed(tmp_path):  # weights.rs:538-560 and the checks of :215-289
    with pytest.raises(G.MuseConfigError) as e:
        G.MuseWeights.open(nvfp4_fixture(tmp_path, include_scales=False))
    assert e.value.kind == "MissingTensor" and e.value.detail == "matrix.nvfp4_scale"
    with pytest.raises(G.MuseConfigError) as e:  # an E4M3FN NaN code among the scales
        G.MuseWeights.open(nvfp4_fixture(tmp_path, scale_byte=0x7F))
    assert "NaN" in str(e.value)
    with pytest.raises(G.MuseConfigError) as e:  # a stored activation scale without the precision tag, and the reverse
        G.MuseWeights.open(nvfp4_fixture(tmp_path, input_scale_inv=12.0, precision="f16"))
    assert "activation_precision" in str(e.value)
    with pytest.raises(G.MuseConfigError):
        G.MuseWeights.open(nvfp4_fixture(tmp_path, precision="nvfp4"))
    with pytest.raises(G.MuseConfigError):
        G.MuseWeights.open(nvfp4_fixture(tmp_path, input_scale_inv=-1.0))
    w = G.MuseWeights.open(nvfp4_fixture(tmp_path, input_scale_inv=12.0))
    assert w.view("matrix").input_scale_inv == 12.0
    with pytest.raises(G.MuseConfigError) as e:
        w.view("absent")
    assert e.value.kind == "MissingTensor"
    w.close()


def test_kquant_views_are_zero_copy_slices_of_the_file(tmp_path):
    from tests import helpers as H
    q4, q6 = H.lcg_weights(O.Q4_K, 5, 2, seed=3), H.lcg_weights(O.Q6_K, 3, 1, seed=4)
    p = tmp_path / "k.gguf"
    G.write_gguf(p, {"blk.0.attn_q.weight": (G.Q4_K, [512, 5], q4), "blk.0.attn_v.weight": (G.Q6_K, [256, 3], q6),
                     "conv": (G.F32, [2, 2, 3, 4], np.arange(48, dtype=np.float32))}, {"general.architecture": (8, "muse")})
    w = G.MuseWeights.open(p)
    vq = w.view("blk.0.attn_q.weight")
    assert (vq.dtype, vq.n_in, vq.n_out) == (G.Q4_K, 512, 5) and np.array_equal(np.array(vq.raw).reshape(q4.shape), q4)
    assert np.array_equal(np.array(w.view("blk.0.attn_v.weight").raw).reshape(q6.shape), q6)
    assert np.array_equal(O.dequant_blocks(O.Q4_K, np.array(vq.raw).reshape(q4.shape)), O.dequant_blocks(O.Q4_K, q4))
    v2 = w.view_2d("conv", 12, 4)
    assert (v2.n_in, v2.n_out) == (12, 4)
    with pytest.raises(G.MuseConfigError):
        w.view_2d("conv", 5, 5)
    assert w.layout("blk.0.attn_q.weight").file_offset % 32 == 0
    w.close()
