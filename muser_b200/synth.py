"""Seeded synthetic tensors for the quantized linear-layer path.

The reference ships no K-quant encoder and no NVFP4 weight encoder: weights
arrive pre-quantised in GGUF / compressed-tensors files and the engine only
decodes them (crates/muser-engine/src/quant/k_block.rs:12-49,
quant/k_block/q6.rs:283-325, quant/nvfp4.rs:240-255).  Parity is defined on the
produced BYTES, so any encoder that emits valid blocks serves.  The encoders
here are plain min/max (Q4_K) and abs-max (Q6_K) sub-block quantisers written
for this repository; NVFP4 weights use the reference's activation-quantiser
contract (quant/nvfp4.rs:173-238) with input_scale_inv = 448*6/amax(W).

Everything is torch tensor arithmetic so that the 141 M-weight projections of
the benchmark are encoded on the GPU in milliseconds; the same code runs on CPU
for the small test shapes.
"""
from __future__ import annotations

import torch

Q4_K, Q5_K, Q6_K, NVFP4 = 12, 13, 14, 1000
BLOCK_BYTES = {Q4_K: 144, Q5_K: 176, Q6_K: 210}

# One synthetic decoder layer (hidden 5120, 40 q / 8 kv heads x 128, SwiGLU FFN 27648) in the
# "Q4_K_M" mix: Q6_K for attn_v and ffn_down, Q4_K elsewhere.  name -> (n_in, n_out, k-quant dtype)
LAYER_PROJECTIONS = {
    "attn_q": (5120, 5120, Q4_K),
    "attn_k": (5120, 1024, Q4_K),
    "attn_v": (5120, 1024, Q6_K),
    "attn_o": (5120, 5120, Q4_K),
    "ffn_gate": (5120, 27648, Q4_K),
    "ffn_up": (5120, 27648, Q4_K),
    "ffn_down": (27648, 5120, Q6_K),
}


def _gen(seed: int, stream: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((seed << 20) + stream)
    return g


def normal_weights(n_out: int, n_in: int, seed: int = 0, stream: int = 0, device="cpu", std: float = 0.02) -> torch.Tensor:
    """f32 N(0, std) weight matrix [n_out][n_in]."""
    return torch.randn((n_out, n_in), generator=_gen(seed, stream, device), device=device, dtype=torch.float32) * std


def normal_activations(tokens: int, n_in: int, seed: int = 0, stream: int = 1000, device="cpu") -> torch.Tensor:
    """bf16 N(0, 1) activations, token-major [tokens][n_in]."""
    x = torch.randn((tokens, n_in), generator=_gen(seed, stream, device), device=device, dtype=torch.float32)
    return x.to(torch.bfloat16)


def _f16_bytes(v: torch.Tensor) -> torch.Tensor:
    """[...] f32 -> [..., 2] u8, little-endian IEEE half (round to nearest even)."""
    return v.to(torch.float16).view(torch.int16).to(torch.int32).bitwise_and(0xFFFF).unsqueeze(-1).bitwise_right_shift(
        torch.tensor([0, 8], device=v.device, dtype=torch.int32)).bitwise_and(0xFF).to(torch.uint8)


def _quantize_q45_k(w: torch.Tensor, bits: int) -> torch.Tensor:
    """Min/max encoder shared by Q4_K (bits = 4) and Q5_K (bits = 5): per 32-element sub-block a 6-bit scale and a
    6-bit min against the super-block's f16 d and dmin, `bits`-bit quants."""
    n_out, n_in = w.shape
    assert n_in % 256 == 0
    nb = n_in // 256
    qmax = float((1 << bits) - 1)
    v = w.reshape(n_out, nb, 8, 32)
    lo = v.amin(-1).clamp_max(0.0)
    hi = v.amax(-1).clamp_min(0.0)
    scale = (hi - lo) / qmax
    mn = -lo
    d = (scale.amax(-1) / 63.0).to(torch.float16)
    dmin = (mn.amax(-1) / 63.0).to(torch.float16)
    df, dminf = d.float().unsqueeze(-1), dmin.float().unsqueeze(-1)
    sc = torch.where(df > 0, (scale / df.clamp_min(1e-30)).round(), torch.zeros_like(scale)).clamp(0, 63)
    m = torch.where(dminf > 0, (mn / dminf.clamp_min(1e-30)).round(), torch.zeros_like(mn)).clamp(0, 63)
    step = (df * sc).unsqueeze(-1)
    q = torch.where(step > 0, ((v + (dminf * m).unsqueeze(-1)) / step.clamp_min(1e-30)).round(), torch.zeros_like(v))
    q = q.clamp(0, qmax).to(torch.uint8)
    sc, m = sc.to(torch.uint8), m.to(torch.uint8)
    scales = torch.empty((n_out, nb, 12), dtype=torch.uint8, device=w.device)
    scales[..., 0:4] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    scales[..., 4:8] = m[..., 0:4] | ((m[..., 4:8] >> 4) << 6)
    scales[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((m[..., 4:8] & 0x0F) << 4)
    qg = q.reshape(n_out, nb, 4, 2, 32)
    qs = ((qg[:, :, :, 0, :] & 15) | ((qg[:, :, :, 1, :] & 15) << 4)).reshape(n_out, nb, 128)
    parts = [_f16_bytes(d.float()), _f16_bytes(dmin.float()), scales]
    if bits == 5:  # qh[l]: bit 2g is the fifth bit of element 64g + l, bit 2g + 1 of element 64g + 32 + l
        qh = torch.zeros((n_out, nb, 32), dtype=torch.uint8, device=w.device)
        for g in range(4):
            qh |= ((qg[:, :, g, 0, :] >> 4) & 1) << (2 * g)
            qh |= ((qg[:, :, g, 1, :] >> 4) & 1) << (2 * g + 1)
        parts.append(qh)
    parts.append(qs)
    blocks = torch.cat(parts, dim=-1)
    assert blocks.shape[-1] == (144 if bits == 4 else 176)
    return blocks.reshape(n_out, nb * blocks.shape[-1]).contiguous()


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    """[n_out][n_in] f32 -> [n_out][n_in/256*144] u8 of Q4_K super-blocks.

    Block layout as decoded by quant/k_block.rs:16-48: d f16, dmin f16,
    12 bytes of packed 6-bit (scale, min) pairs, 128 bytes of nibbles where
    byte 32g+l holds element 64g+l (low) and 64g+32+l (high).
    """
    return _quantize_q45_k(w, 4)


def quantize_q5_k(w: torch.Tensor) -> torch.Tensor:
    """[n_out][n_in] f32 -> [n_out][n_in/256*176] u8 of Q5_K super-blocks (quant/k_block.rs:61-105): the Q4_K block
    with a 32-byte plane of fifth bits between the scales and the nibbles."""
    return _quantize_q45_k(w, 5)


def quantize_q6_k(w: torch.Tensor) -> torch.Tensor:
    """[n_out][n_in] f32 -> [n_out][n_in/256*210] u8 of Q6_K super-blocks.

    Block layout as decoded by quant/k_block/q6.rs:264-325: ql[128], qh[64],
    sc[16] int8, d f16; element 128h + 32c + l (c = 0..3) takes its low nibble
    from ql[64h + 32(c&1) + l] (upper half of the byte for c >= 2), its two
    high bits from bits 2c..2c+1 of qh[32h + l], and scale sc[8h + 2c + l/16].
    """
    n_out, n_in = w.shape
    assert n_in % 256 == 0
    nb = n_in // 256
    v = w.reshape(n_out, nb, 16, 16)
    amax_idx = v.abs().argmax(-1, keepdim=True)
    signed_max = v.gather(-1, amax_idx).squeeze(-1)
    scale = signed_max / -32.0
    d = (scale.abs().amax(-1) / 127.0).to(torch.float16)
    df = d.float().unsqueeze(-1)
    sc = torch.where(df > 0, (scale / df.clamp_min(1e-30)).round(), torch.zeros_like(scale)).clamp(-128, 127)
    step = (df * sc).unsqueeze(-1)
    q = torch.where(step != 0, (v / torch.where(step != 0, step, torch.ones_like(step))).round(), torch.zeros_like(v))
    q = (q.clamp(-32, 31) + 32).to(torch.uint8).reshape(n_out, nb, 2, 4, 32)  # [h][c][l]
    lo, hi2 = q & 0x0F, q >> 4
    ql = torch.empty((n_out, nb, 2, 64), dtype=torch.uint8, device=w.device)
    ql[..., 0:32] = lo[:, :, :, 0, :] | (lo[:, :, :, 2, :] << 4)
    ql[..., 32:64] = lo[:, :, :, 1, :] | (lo[:, :, :, 3, :] << 4)
    qh = hi2[:, :, :, 0, :] | (hi2[:, :, :, 1, :] << 2) | (hi2[:, :, :, 2, :] << 4) | (hi2[:, :, :, 3, :] << 6)
    # sub-block index within the super-block is 8h + 2c + l/16 == position in the [16][16] view
    sc_bytes = sc.to(torch.int8).view(torch.uint8)
    blocks = torch.cat([ql.reshape(n_out, nb, 128), qh.reshape(n_out, nb, 64), sc_bytes, _f16_bytes(d.float())], dim=-1)
    assert blocks.shape[-1] == 210
    return blocks.reshape(n_out, nb * 210).contiguous()


def quantize_nvfp4(x: torch.Tensor, input_scale_inv: float):
    """The reference's group-16 quantiser (quant/nvfp4.rs:173-238) as tensor ops.

    x [rows][K] (any float dtype) -> packed [rows][K/2] u8 (low nibble = even
    element) and E4M3FN scale codes [rows][K/16] u8, row-major.
    """
    rows, k = x.shape
    assert k % 16 == 0
    isi = torch.tensor(input_scale_inv, dtype=torch.float32, device=x.device)
    r = x.to(torch.float32).to(torch.float16).to(torch.float32).reshape(rows, k // 16, 16)
    amax = r.abs().amax(-1)
    target = (amax * torch.tensor(1.0 / 6.0, dtype=torch.float32, device=x.device) * isi).clamp_max(448.0)
    scale8 = target.to(torch.float8_e4m3fn)
    scale = scale8.to(torch.float32).unsqueeze(-1)
    mag = r.abs() * isi
    code = torch.zeros_like(mag, dtype=torch.uint8)
    for bound, inclusive in ((0.25, True), (0.75, False), (1.25, True), (1.75, False), (2.5, True), (3.5, False), (5.0, True)):
        edge = scale * bound
        code += (mag > edge).to(torch.uint8) if inclusive else (mag >= edge).to(torch.uint8)
    code = torch.where(scale == 0, torch.zeros_like(code), code)
    code |= (torch.signbit(r).to(torch.uint8) << 3)
    code = code.reshape(rows, k // 2, 2)
    packed = code[..., 0] | (code[..., 1] << 4)
    return packed.contiguous(), scale8.view(torch.uint8).contiguous()


def nvfp4_weight(w: torch.Tensor):
    """Quantise a weight matrix to NVFP4: returns (packed, scales, scale2)."""
    amax = float(w.abs().max())
    isi = float(torch.tensor(448.0 * 6.0, dtype=torch.float32) / torch.tensor(amax, dtype=torch.float32))
    packed, scales = quantize_nvfp4(w, isi)
    scale2 = float(torch.tensor(1.0, dtype=torch.float32) / torch.tensor(isi, dtype=torch.float32))
    return packed, scales, scale2


def activation_input_scale_inv(x: torch.Tensor) -> float:
    """Static per-tensor activation scale, the stored-scale contract of weights.rs:30-36."""
    amax = x.to(torch.float32).to(torch.float16).to(torch.float32).abs().max()
    return float(torch.tensor(448.0 * 6.0, dtype=torch.float32) / amax.cpu())


def quantize_kquant(w: torch.Tensor, dtype: int) -> torch.Tensor:
    return {Q4_K: quantize_q4_k, Q5_K: quantize_q5_k, Q6_K: quantize_q6_k}[dtype](w)
