"""Shared test helpers: the reference's deterministic fixture generators and an
independent numpy decoder for the K-quant block formats."""
import numpy as np

from oracle import oracle as O


def quant_rows(row_bytes: int, rows: int) -> np.ndarray:
    """Closed-form Q4_K rows of crates/muser-engine/src/metal.rs:1243-1263 (one block per row)."""
    out = np.zeros((rows, row_bytes), dtype=np.uint8)
    for row in range(rows):
        b = out[row]
        b[0:2] = [0x00, 0x38]  # d = 0.5
        b[2:4] = [0x00, 0x34]  # dmin = 0.25
        for i in range(12):
            b[4 + i] = (i * 13 + row * 7 + 3) & 0xFF
        for i in range(row_bytes - 16):
            b[16 + i] = (i * 37 + row * 11 + 9) & 0xFF
    return out


def q6_rows(rows: int) -> np.ndarray:
    """Closed-form Q6_K rows of crates/muser-engine/src/metal.rs:369-383."""
    out = np.zeros((rows, 210), dtype=np.uint8)
    for row in range(rows):
        b = out[row]
        for i in range(192):
            b[i] = (i * 31 + row * 13 + 7) & 0xFF
        for i in range(16):
            b[192 + i] = ((i * 11 + row * 5 + 3) & 0x3F) ^ 0x20
        b[208:210] = [0x00, 0x2C]  # d = 0.0625
    return out


def lcg_weights(dtype: int, rows: int, blocks: int, seed: int) -> np.ndarray:
    """LCG blocks with small finite scales, crates/muser-engine/src/metal/encode/multicol.rs:292-319."""
    stride = O.BLOCK_BYTES[dtype]
    state = seed | 1
    mask = (1 << 64) - 1

    def nxt():
        nonlocal state
        state = (state * 6364136223846793005 + 1442695040888963407) & mask
        return (state >> 33) & 0xFFFFFFFF

    out = np.zeros(rows * blocks * stride, dtype=np.uint8)
    for b in range(rows * blocks):
        blk = out[b * stride:(b + 1) * stride]
        for i in range(stride):
            blk[i] = nxt() & 0xFF
        d = np.float32(0.002) + np.float32(nxt() % 128) * np.float32(0.0005)
        dmin = np.float32(0.001) + np.float32(nxt() % 128) * np.float32(0.0003)
        dh = O.f32_to_f16_trunc(float(d))
        mh = O.f32_to_f16_trunc(float(dmin))
        if dtype == O.Q6_K:
            blk[208:210] = [dh & 0xFF, dh >> 8]
        else:
            blk[0:2] = [dh & 0xFF, dh >> 8]
            blk[2:4] = [mh & 0xFF, mh >> 8]
    return out.reshape(rows, blocks * stride)


def lcg_activations(count: int, seed: int) -> np.ndarray:
    """crates/muser-engine/src/metal/encode/multicol.rs:321-331"""
    state = seed | 1
    mask = (1 << 64) - 1
    out = np.empty(count, dtype=np.float32)
    for i in range(count):
        state = (state * 6364136223846793005 + 1442695040888963407) & mask
        out[i] = (np.float32(state >> 33) / np.float32(1 << 31) - np.float32(0.5)) * np.float32(2.0)
    return out


def numpy_dequant_q4_k(blocks: np.ndarray) -> np.ndarray:
    """Independent decoder written from the block-format description (not from the oracle)."""
    b = blocks.reshape(-1, 144)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)[:, 0]
    s = b[:, 4:16].astype(np.uint32)
    sc = np.empty((b.shape[0], 8), dtype=np.uint32)
    mn = np.empty((b.shape[0], 8), dtype=np.uint32)
    sc[:, 0:4] = s[:, 0:4] & 63
    mn[:, 0:4] = s[:, 4:8] & 63
    sc[:, 4:8] = (s[:, 8:12] & 15) | ((s[:, 0:4] >> 6) << 4)
    mn[:, 4:8] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    qs = b[:, 16:144].reshape(-1, 4, 32)
    q = np.stack([qs & 15, qs >> 4], axis=2).reshape(-1, 8, 32).astype(np.float32)
    step = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    off = (dmin[:, None] * mn.astype(np.float32)).astype(np.float32)
    return ((step[:, :, None] * q).astype(np.float32) - off[:, :, None]).astype(np.float32).reshape(-1)


def numpy_dequant_q6_k(blocks: np.ndarray) -> np.ndarray:
    b = blocks.reshape(-1, 210)
    n = b.shape[0]
    ql = b[:, 0:128].reshape(n, 2, 2, 32).astype(np.int32)   # [h][c&1][l]
    qh = b[:, 128:192].reshape(n, 2, 32).astype(np.int32)
    sc = b[:, 192:208].copy().view(np.int8).astype(np.float32).reshape(n, 2, 4, 2)  # [h][c][l/16]
    d = b[:, 208:210].copy().view(np.float16).astype(np.float32)[:, 0]
    out = np.empty((n, 2, 4, 32), dtype=np.float32)
    for c in range(4):
        nib = (ql[:, :, c & 1, :] >> (4 * (c >> 1))) & 15
        q = (nib | (((qh >> (2 * c)) & 3) << 4)) - 32
        s = (d[:, None, None] * np.repeat(sc[:, :, c, :], 16, axis=-1)).astype(np.float32)
        out[:, :, c, :] = (s * q.astype(np.float32)).astype(np.float32)
    return out.reshape(-1)


def rel_l2(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
