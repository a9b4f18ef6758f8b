"""K-quant half of the oracle.

The reference holds no CPU-only known-answer test for dot_q4_k_f32 / dot_q6_k_f32
(quant/k_block.rs and quant/k_block/q6.rs have no #[cfg(test)]), so these tests pin the oracle
themselves: dequantisation against an independent numpy decoder on the reference's own fixture
generators, the dot products against an f64 dot of the dequantised row, and SHA-256 digests of
the results recorded below so that a later change of the oracle is caught.
"""
import hashlib

import numpy as np
import pytest
import torch

from muser_b200 import synth
from oracle import oracle as O
from tests import helpers as H


@pytest.mark.parametrize("dtype,gen", [(O.Q4_K, lambda: H.quant_rows(144, 64)), (O.Q6_K, lambda: H.q6_rows(64))])
def test_dequant_matches_independent_decoder_on_closed_form_rows(dtype, gen):
    rows = gen()
    got = O.dequant_blocks(dtype, rows)
    ref = (H.numpy_dequant_q4_k if dtype == O.Q4_K else H.numpy_dequant_q6_k)(rows)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q6_K])
def test_dequant_matches_independent_decoder_on_lcg_blocks(dtype):
    rows = H.lcg_weights(dtype, 13, 2, seed=0x5EED + dtype)
    got = O.dequant_blocks(dtype, rows)
    ref = (H.numpy_dequant_q4_k if dtype == O.Q4_K else H.numpy_dequant_q6_k)(rows)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


GOLDEN_DIGESTS = {
    # sha256 over the little-endian f32 bytes of [dequant | dots] for the LCG fixture below
    O.Q4_K: "abc407724b360b32e20cf71fbc6a4402ffae6ae92020077b0fc0a49db3a01afe",
    O.Q6_K: "cd5efc719ebbf5fc9ba85b3cf93395c2db8a124615fea249d8cdb306c0001d8d",
}


@pytest.mark.parametrize("dtype", [O.Q4_K, O.Q6_K])
def test_dot_matches_f64_dot_of_dequantised_row_and_recorded_digest(dtype):
    n_in, n_out = 512, 13  # the shape of metal/encode/multicol.rs:357-358
    rows = H.lcg_weights(dtype, n_out, n_in // 256, seed=0xC0FFEE + dtype)
    x = H.lcg_activations(n_in, seed=0xBEEF)
    deq = O.dequant_blocks(dtype, rows).reshape(n_out, n_in)
    dots = np.asarray([O.dot_kquant(dtype, rows[r], x) for r in range(n_out)], dtype=np.float32)
    exact = deq.astype(np.float64) @ x.astype(np.float64)
    scale = np.abs(deq.astype(np.float64)) @ np.abs(x.astype(np.float64))
    assert np.all(np.abs(dots - exact) <= 2e-6 * scale)
    if dtype == O.Q4_K:
        llama = np.asarray([O.dot_kquant(dtype, rows[r], x, llama_order=True) for r in range(n_out)])
        assert np.all(np.abs(llama - exact) <= 2e-5 * scale)
    digest = hashlib.sha256(deq.tobytes() + dots.tobytes()).hexdigest()
    assert digest == GOLDEN_DIGESTS[dtype], digest


def test_matmul_is_token_major_and_thread_count_invariant():
    n_in, n_out, tokens = 512, 37, 3
    rows = H.lcg_weights(O.Q4_K, n_out, 2, seed=7)
    x = H.lcg_activations(tokens * n_in, seed=9).reshape(tokens, n_in)
    w = O.TensorView(rows, O.Q4_K, n_in, n_out)
    a = O.matmul(w, x, threads=1)
    b = O.matmul(w, x, threads=5)
    assert a.shape == (tokens, n_out) and np.array_equal(a, b)
    assert a[2, 11] == np.float32(O.dot_kquant(O.Q4_K, rows[11], x[2]))


@pytest.mark.parametrize("dtype,max_rel", [(synth.Q4_K, 0.08), (synth.Q6_K, 0.02)])
def test_synthetic_encoders_emit_valid_blocks(dtype, max_rel):
    w = synth.normal_weights(8, 1024, seed=0, stream=3)
    blocks = synth.quantize_kquant(w, dtype).numpy()
    assert blocks.shape == (8, 1024 // 256 * synth.BLOCK_BYTES[dtype])
    deq = O.dequant_blocks(dtype, blocks).reshape(8, 1024)
    assert np.all(np.isfinite(deq))
    assert H.rel_l2(deq, w.numpy()) < max_rel


def test_synthetic_nvfp4_quantiser_is_bit_identical_to_oracle():
    x = synth.normal_activations(5, 256, seed=0).float()
    x[1, 16:32] = 0.0
    x[2, 0] = 3000.0
    isi = synth.activation_input_scale_inv(x)
    packed, scales = synth.quantize_nvfp4(x, isi)
    op, os_ = O.quantize_nvfp4_activation(x.numpy(), isi)
    assert np.array_equal(packed.numpy(), op) and np.array_equal(scales.numpy(), os_)
    w = synth.normal_weights(16, 128, seed=0, stream=5)
    wp, ws, scale2 = synth.nvfp4_weight(w)
    deq = O.dequant_nvfp4(wp.numpy(), ws.numpy(), scale2)
    assert H.rel_l2(deq, w.numpy()) < 0.12
    assert not np.any((ws.numpy() & 0x7F) == 0x7F)


def test_rms_norm_and_silu_follow_reference_formulas():
    x = np.asarray([[1.0, -2.0, 3.0, 0.5]], dtype=np.float32)
    w = np.asarray([0.5, 1.0, 2.0, 1.5], dtype=np.float32)
    ss = np.float32(0.0)
    for v in x[0]:
        ss = np.float32(ss + np.float32(v * v))
    scale = np.float32(1.0) / np.sqrt(np.float32(ss / np.float32(4.0) + np.float32(1e-6)))
    want = (x[0] * scale).astype(np.float32) * w
    assert np.array_equal(O.rms_norm_mul(x, 1e-6, w)[0], want)
    g = np.asarray([0.3, -1.2], dtype=np.float32)
    u = np.asarray([2.0, 0.5], dtype=np.float32)
    got = O.silu_mul(g, u)
    assert np.allclose(got, g / (1 + np.exp(-g)) * u, rtol=1e-6)


def test_matmul_rows_and_logit_tail_follow_the_reference():
    """weights.rs:425-449 (`matmul_rows` is `matmul` over the listed rows, same dot_row) and reference.rs:559-570."""
    rng = np.random.default_rng(3)
    for dtype in (O.Q4_K, O.Q6_K):
        raw = H.lcg_weights(dtype, 21, 2, seed=5 + dtype)
        w = O.TensorView(raw, dtype, 512, 21)
        x = rng.standard_normal((3, 512)).astype(np.float32)
        rows = [20, 0, 7, 7]
        assert np.array_equal(O.matmul_rows(w, x, rows), O.matmul(w, x)[:, rows])
        with pytest.raises(ValueError):
            O.matmul_rows(w, x, [21])
    logits = np.array([0.0, 1.0, -2.5, 90.0, -1e4], dtype=np.float32)
    scaled = O.logit_tail(logits, 0.5, 0.0)
    assert np.array_equal(scaled, logits * np.float32(0.5))
    capped = O.logit_tail(logits, 0.5, 30.0)
    want = 30.0 * np.tanh(logits.astype(np.float64) * 0.5 / 30.0)
    assert np.allclose(capped, want, rtol=1e-6, atol=1e-6) and np.all(np.abs(capped) <= 30.0)
