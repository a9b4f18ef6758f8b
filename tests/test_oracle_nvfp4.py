"""Pins the oracle's NVFP4 functions to the reference.

Part 1 replays the known-answer tests of crates/muser-engine/src/quant/nvfp4.rs:381-543.
Part 2 compares with vectors produced by the reference's own Python code
(tests/golden/make_golden.py).
"""
import math
import struct

import numpy as np

from oracle import oracle as O


def bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def f16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return a.view(np.float16).astype(np.float32)


# ---- nvfp4.rs:385-391
def test_e2m1_lut_preserves_signed_zero_and_endpoints():
    assert bits(O.e2m1_to_f32(0)) == bits(0.0)
    assert bits(O.e2m1_to_f32(8)) == bits(-0.0)
    assert O.e2m1_to_f32(7) == 6.0 and O.e2m1_to_f32(15) == -6.0


# ---- nvfp4.rs:394-407
def test_e4m3fn_lut_matches_pinned_reference_cases():
    assert bits(O.e4m3fn_to_f32(0x00)) == bits(0.0)
    assert bits(O.e4m3fn_to_f32(0x80)) == bits(-0.0)
    assert O.e4m3fn_to_f32(0x01) == 1.0 / 512.0
    assert O.e4m3fn_to_f32(0x38) == 1.0
    assert O.e4m3fn_to_f32(0x7E) == 448.0
    assert math.isnan(O.e4m3fn_to_f32(0x7F)) and math.isnan(O.e4m3fn_to_f32(0xFF))
    for code in range(0x7F):
        assert O.e4m3fn_from_f32(O.e4m3fn_to_f32(code)) == code
    assert O.e4m3fn_from_f32(1000.0) == 0x7E
    assert O.e4m3fn_from_f32(-1000.0) == 0xFE


# ---- nvfp4.rs:410-428
def test_integer_encodings_are_exact_for_every_finite_code():
    for code in range(256):
        if code in (0x7F, 0xFF):
            continue
        assert float(O.e4m3fn_q9(code)) == O.e4m3fn_to_f32(code) * 512.0
    for code in range(16):
        assert float(O.e2m1_q1(code)) == O.e2m1_to_f32(code) * 2.0


# ---- nvfp4.rs:431-448
def test_e2m1_ties_follow_the_modelopt_contract():
    f32 = lambda v: float(np.float32(v))
    for value, code in [(0.25, 0), (0.250001, 1), (0.75, 2), (1.25, 2), (1.250001, 3), (1.75, 4), (2.5, 4),
                        (2.500001, 5), (3.5, 6), (5.0, 6), (5.000001, 7)]:
        assert O.e2m1_from_f32(f32(value)) == code
        assert O.e2m1_from_f32(f32(-value)) == code | 8


WEIGHT_GROUP = [0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]


# ---- nvfp4.rs:451-482
def test_w4a4_oracle_quantizes_f16_activation_groups_before_the_dot():
    x = np.asarray([np.float32(np.float32(i) - np.float32(7.5)) * np.float32(0.125) + np.float32(0.00001)
                    for i in range(16)], dtype=np.float32)
    isi = 43.75
    a_packed, a_scales = O.quantize_nvfp4_activation(x, isi)
    actual = O.dot_nvfp4_w4a4_f32(WEIGHT_GROUP, [0x38], 0.25, isi, x)
    codes = O.dequant_nvfp4(a_packed, a_scales, float(np.float32(1.0) / np.float32(isi)))
    fused = O.dot_nvfp4_block_fused_f32(WEIGHT_GROUP, [0x38], 0.25, codes)
    expected = O.f16_to_f32(O.f32_to_f16_rne(fused))
    assert bits(actual) == bits(expected)


# ---- nvfp4.rs:485-517
def test_a16_q8_oracle_uses_signed_first_max_and_pinned_integer_epilogue():
    x = np.zeros(256, dtype=np.float32)
    x[0], x[1] = 2.0, -2.0
    for i in range(2, 256):
        x[i] = np.float32(np.float16(np.float32(np.float32(i) - np.float32(128.0)) * np.float32(0.003)))
    d, qs = O.quantize_nvfp4_q8_block(x)
    assert bits(d) == bits(float(np.float32(-2.0) / np.float32(127.0)))
    assert qs[0] == -127 and qs[1] == 127
    packed = [0x62] * 128
    scales = [0x38] * 16
    scales[3], scales[11] = 0x30, 0xB8
    actual = O.dot_nvfp4_a16_q8_f32(packed, scales, 0.25, x)
    total = 0
    for g, s in enumerate(scales):
        dot = sum(O.e2m1_q1(0x02) * int(qs[g * 16 + p * 2]) + O.e2m1_q1(0x06) * int(qs[g * 16 + p * 2 + 1])
                  for p in range(8))
        total += dot * O.e4m3fn_q9(s)
    e = np.float32(total) * np.float32(1.0 / 1024.0)   # each product is a single rounding = fma(a, b, 0)
    e = np.float32(e * np.float32(d))
    e = np.float32(e * np.float32(0.25))
    expected = float(np.float32(np.float16(e)))
    assert bits(actual) == bits(expected)


# ---- nvfp4.rs:520-542
def test_block_dequant_and_dot_use_the_pinned_order():
    got = O.dequant_nvfp4(WEIGHT_GROUP, [0x38], 0.25)
    expected = np.asarray([0.0, .125, .25, .375, .5, .75, 1.0, 1.5, -0.0, -.125, -.25, -.375, -.5, -.75, -1.0, -1.5],
                          dtype=np.float32)
    assert got.view(np.uint32).tolist() == expected.view(np.uint32).tolist()
    x = np.asarray([v * 0.125 for v in range(1, 17)], dtype=np.float32)
    s = np.float32(0.0)
    for w, v in zip(expected, x):
        s = np.float32(s + np.float32(w * v))
    assert bits(O.dot_nvfp4_f32(WEIGHT_GROUP, [0x38], 0.25, x)) == bits(float(s))


# ---- vectors made by the reference's Python code -----------------------------------------

def test_weight_decode_matches_reference_python_codec(golden):
    got = O.dequant_nvfp4(golden["codec_packed"], golden["codec_scales"], float(golden["codec_scale2"]))
    assert np.array_equal(got.view(np.uint32), golden["codec_dequant"].view(np.uint32))
    for code in range(16):
        assert bits(O.e2m1_to_f32(code)) == bits(float(golden["codec_e2m1_table"][code]))
    for code in range(256):
        ref = float(golden["codec_e4m3_table"][code])
        assert (math.isnan(ref) and math.isnan(O.e4m3fn_to_f32(code))) or bits(O.e4m3fn_to_f32(code)) == bits(ref)


def unswizzle(swizzled: np.ndarray, rows: int, groups: int) -> np.ndarray:
    """Logical [rows][groups] view of the [rows/128][groups/4][32][4][4] scale layout
    (scripts/gx10/vllm/muser_vllm/exact_fp4_quant.py:149-162)."""
    rounded_groups = (groups + 3) // 4 * 4
    raw = swizzled.reshape(-1)
    r = np.arange(rows)[:, None]
    g = np.arange(groups)[None, :]
    off = (r // 128) * rounded_groups * 128 + (g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4
    return raw[off]


def test_activation_quantiser_matches_reference_fixture(golden):
    for tag in ("quant", "quant2"):
        x = f16_bits_to_f32(golden[f"{tag}_input_f16_bits"])
        packed, scales = O.quantize_nvfp4_activation(x, float(golden[f"{tag}_global_scale"]))
        assert np.array_equal(packed, golden[f"{tag}_packed"]), tag
        rows, groups = scales.shape
        assert np.array_equal(scales, unswizzle(golden[f"{tag}_scales_swizzled"], rows, groups)), tag


def test_a16_q8_lane_matches_reference_fixture(golden):
    x = f16_bits_to_f32(golden["a16_activation_f16_bits"])
    for t in range(x.shape[0]):
        d, qs = O.quantize_nvfp4_q8_block(x[t])
        assert np.array_equal(qs, golden["a16_q8_codes"][t])
        assert bits(d) == bits(float(golden["a16_q8_scales"][t]))
    w = O.TensorView(golden["a16_w_packed"], O.NVFP4, 256, 11, golden["a16_w_scales"], float(golden["a16_scale2"]), None)
    out = O.matmul(w, x)
    assert np.array_equal(out.astype(np.float16).view(np.uint16), golden["a16_expected_f16_bits"])
    assert np.array_equal(out, out.astype(np.float16).astype(np.float32))  # already on the f16 grid


def test_w4a4_lane_matches_reference_fixture(golden):
    x = f16_bits_to_f32(golden["w4a4_activation_f16_bits"])
    isi = float(golden["w4a4_act_global"])
    packed, scales = O.quantize_nvfp4_activation(x, isi)
    assert np.array_equal(packed, golden["w4a4_act_packed"])
    assert np.array_equal(scales, golden["w4a4_act_scales_logical"])
    w = O.TensorView(golden["w4a4_w_packed"], O.NVFP4, 128, 128, golden["w4a4_w_scales_logical"],
                     float(golden["w4a4_weight_scale2"]), isi)
    expected = golden["w4a4_expected_f16_bits"]
    for hoist in (True, False):
        out = O.matmul(w, x, threads=2, hoist_activation=hoist)
        assert np.array_equal(out.astype(np.float16).view(np.uint16), expected), hoist
    out, pre = O.matmul(w, x, return_pre_round=True)
    assert np.array_equal(pre.astype(np.float16).view(np.uint16), expected)
