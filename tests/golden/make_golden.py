#!/usr/bin/env python3
"""Generate tests/golden/nvfp4_reference_vectors.npz from the reference's own Python code.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

Everything that produces an EXPECTED value below is a function imported from
the reference tree (its NVFP4 decoder and the CPU halves of its GB10 fixture
scripts).  This script only builds inputs and calls them.  The resulting file
is small and committed, because the reference checkout is not present where
the GPU tests run.

Imported reference code:
  scripts/nvfp4_codec.py                           dequantize, E2M1, E4M3FN
  scripts/gx10/vllm/test_exact_fp4_quant.py        reference() (activation quantiser + swizzled scales)
  scripts/gx10/vllm/test_exact_fp4_a16_mm.py       quantize_q8k, e4m3_q9, unpack_q1, f32_mul, f32_add
  scripts/gx10/vllm/test_exact_fp4_mm.py           logical_scale_codes, e4m3_q9, unpack_q1
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of the reference project>")
    ref = Path(sys.argv[1])
    sys.path.insert(0, str(ref / "scripts"))
    sys.path.insert(0, str(ref / "scripts" / "gx10" / "vllm"))
    import nvfp4_codec
    import test_exact_fp4_a16_mm as a16
    import test_exact_fp4_mm as mm
    import test_exact_fp4_quant as quant

    out: dict[str, np.ndarray] = {}
    rng = np.random.default_rng(20260825)

    # 1. weight decode: scripts/nvfp4_codec.py dequantize()
    finite = np.asarray([c for c in range(256) if c not in (0x7F, 0xFF)], dtype=np.uint8)
    packed = rng.integers(0, 256, size=(9, 64), dtype=np.uint8)
    packed[0, :8] = [0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]
    scales = finite[rng.integers(0, finite.size, size=(9, 8))]
    scales[0, 0] = 0x38
    out["codec_packed"] = packed
    out["codec_scales"] = scales
    out["codec_scale2"] = np.float32(0.25)
    out["codec_dequant"] = nvfp4_codec.dequantize(packed, scales, 0.25)
    out["codec_e2m1_table"] = nvfp4_codec.E2M1.copy()
    out["codec_e4m3_table"] = nvfp4_codec.E4M3FN.copy()

    # 2. activation quantiser: test_exact_fp4_quant.py reference(); its own fixture first
    torch.manual_seed(0)
    fixture = torch.randn((5, 64), dtype=torch.float32).mul_(2.5).to(torch.float16)
    fixture[0, :16] = torch.tensor(
        [-0.0, 0.0, 0.25, -0.25, 0.75, -0.75, 1.25, -1.25, 1.75, -1.75, 2.5, -2.5, 3.5, -3.5, 5.0, -6.0],
        dtype=torch.float16,
    )
    global_scale = 43.75
    q_packed, q_scales = quant.reference(fixture, global_scale)
    out["quant_input_f16_bits"] = fixture.view(torch.uint16).numpy().copy()
    out["quant_global_scale"] = np.float32(global_scale)
    out["quant_packed"] = q_packed.numpy().copy()
    out["quant_scales_swizzled"] = q_scales.numpy().copy()

    # a second case that spans two 128-row tiles and a ragged group count
    torch.manual_seed(1)
    big = torch.randn((130, 96), dtype=torch.float32).mul_(1.7).to(torch.float16)
    big[3, 16:32] = 0.0
    big[129, :16] = 1000.0  # saturates the E4M3 scale
    big_scale = 61.5
    b_packed, b_scales = quant.reference(big, big_scale)
    out["quant2_input_f16_bits"] = big.view(torch.uint16).numpy().copy()
    out["quant2_global_scale"] = np.float32(big_scale)
    out["quant2_packed"] = b_packed.numpy().copy()
    out["quant2_scales_swizzled"] = b_scales.numpy().copy()

    # 3. weight-only x Q8_K lane: inputs and expectation exactly as test_exact_fp4_a16_mm.py main() builds them
    tokens, outputs, width = 7, 11, 256
    scale2 = np.float32(0.25)
    one_group = np.asarray([0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE], dtype=np.uint8)
    w_packed = np.empty((outputs, width // 2), dtype=np.uint8)
    w_scales = np.empty((outputs, width // 16), dtype=np.uint8)
    for row in range(outputs):
        w_packed[row] = np.tile(one_group, width // 16)
        for group in range(width // 16):
            w_scales[row, group] = finite[(row * 29 + group * 17) % finite.size]
    activation = np.empty((tokens, width), dtype=np.float32)
    for token in range(tokens):
        for element in range(width):
            activation[token, element] = np.float32(((token * 19 + element * 7 + 3) - 901.0) * 0.003125 + 0.00001)
        activation[token, 0] = 2.0
        activation[token, 1] = -2.0
    activation_f16 = activation.astype(np.float16)
    weights_q1 = a16.unpack_q1(w_packed)
    scales_q9 = a16.e4m3_q9(w_scales)
    expected = np.empty((tokens, outputs), dtype=np.float16)
    q8_codes = np.empty((tokens, width), dtype=np.int8)
    q8_scales = np.empty((tokens,), dtype=np.float32)
    for token in range(tokens):
        q8, q8_scale = a16.quantize_q8k(activation_f16[token])
        q8_codes[token], q8_scales[token] = q8, q8_scale
        for row in range(outputs):
            integer_total = np.int64(0)
            for group in range(width // 16):
                s = group * 16
                integer_total += np.dot(weights_q1[row, s:s + 16], q8[s:s + 16].astype(np.int64)) * scales_q9[row, group]
            c = a16.f32_mul(np.float32(integer_total), np.float32(1.0 / 1024.0))
            c = a16.f32_mul(c, q8_scale)
            c = a16.f32_mul(c, scale2)
            expected[token, row] = np.float16(a16.f32_add(np.float32(0.0), c))
    out["a16_w_packed"] = w_packed
    out["a16_w_scales"] = w_scales
    out["a16_scale2"] = scale2
    out["a16_activation_f16_bits"] = activation_f16.view(np.uint16)
    out["a16_q8_codes"] = q8_codes
    out["a16_q8_scales"] = q8_scales
    out["a16_expected_f16_bits"] = expected.view(np.uint16)

    # 4. W4A4 integer contraction: both operands quantised by reference(), contraction as test_exact_fp4_mm.py main()
    torch.manual_seed(170072)
    rows, n_out, k = 32, 128, 128
    act_global, w_global = 43.75, 37.25
    a = torch.randn((rows, k), dtype=torch.float16)
    b = torch.randn((n_out, k), dtype=torch.float16)
    a_packed, a_scale = quant.reference(a, act_global)
    b_packed, b_scale = quant.reference(b, w_global)
    weight_scale2 = np.float32(1.0) / np.float32(w_global)
    input_scale = np.float32(1.0) / np.float32(act_global)
    a_codes, b_codes = mm.unpack_q1(a_packed), mm.unpack_q1(b_packed)
    groups = k // 16
    a_logical = mm.logical_scale_codes(a_scale, rows, groups)
    b_logical = mm.logical_scale_codes(b_scale, n_out, groups)
    a_q9, b_q9 = mm.e4m3_q9(a_logical), mm.e4m3_q9(b_logical)
    exp = np.empty((rows, n_out), dtype=np.float16)
    for r in range(rows):
        for o in range(n_out):
            total = np.int64(0)
            for g in range(groups):
                total += np.dot(a_codes[r, g * 16:(g + 1) * 16], b_codes[o, g * 16:(g + 1) * 16]) * a_q9[r, g] * b_q9[o, g]
            s = np.multiply(np.float32(total), np.float32(1.0 / 1048576.0), dtype=np.float32)
            s = np.multiply(s, weight_scale2, dtype=np.float32)
            s = np.multiply(s, input_scale, dtype=np.float32)
            exp[r, o] = np.float16(s)
    out["w4a4_activation_f16_bits"] = a.view(torch.uint16).numpy().copy()
    out["w4a4_act_global"] = np.float32(act_global)
    out["w4a4_act_packed"] = a_packed.numpy().copy()
    out["w4a4_act_scales_logical"] = a_logical
    out["w4a4_w_packed"] = b_packed.numpy().copy()
    out["w4a4_w_scales_logical"] = b_logical
    out["w4a4_w_scales_swizzled"] = b_scale.numpy().copy()
    out["w4a4_weight_scale2"] = weight_scale2
    out["w4a4_expected_f16_bits"] = exp.view(np.uint16)

    dst = Path(__file__).resolve().parent / "nvfp4_reference_vectors.npz"
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} ({dst.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main()
