"""The CPU restatement against the reference's own compiled C functions (oracle/_ref/libh3_ref.so)
on fresh seeded inputs, larger than the committed vectors.  Skipped where that library is absent."""
import numpy as np
import pytest


@pytest.mark.parametrize("seed", [1, 2])
def test_linear_chain_bit_exact(oracle, ref, seed):
    rng = np.random.default_rng(seed)
    m, k, n = 33, 512, 48
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    x[rng.random((m, k)) < 0.001] *= 20
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    for gs in (0, 256):
        xr_o, xr_r = oracle.convrot(x, gs), ref.convrot(x, gs)
        assert np.array_equal(xr_o, xr_r)
        (q_o, s_o), (q_r, s_r) = oracle.quantize_act_int8(xr_o), ref.quantize_act_int8(xr_r)
        assert np.array_equal(q_o, q_r) and np.array_equal(s_o, s_r)
        wq, ws = ref.quantize_act_int8(w)
        assert np.array_equal(oracle.gemm_i8_dequant(q_o, wq, s_o, ws), ref.gemm_i8_dequant(q_r, wq, s_r, ws))
    assert np.array_equal(oracle.gemm_f32(x, w), ref.gemm_f32(x, w))


@pytest.mark.parametrize("gs", [2, 8, 64, 256])
def test_sylvester_rotation_bit_exact(oracle, ref, gs):
    """The Walsh-Hadamard form of ConvRot that H3_CONVROT_SYLVESTER=1 selects (h3_w4a8_dequant.c:241-284)."""
    rng = np.random.default_rng(40 + gs)
    x = rng.normal(0, 1, (19, 512)).astype(np.float32)
    assert np.array_equal(oracle.fwht(x, gs), ref.fwht(x, gs))
    # it is the product with the Sylvester matrix, an orthogonal map
    assert np.allclose(np.linalg.norm(oracle.fwht(x, gs), axis=1), np.linalg.norm(x, axis=1), rtol=1e-5)


def test_w4a8_decode_random(oracle, ref):
    rng = np.random.default_rng(3)
    n, k = 64, 256
    packed = rng.integers(-128, 128, (n, k // 2), dtype=np.int8)
    codebook = rng.normal(0, 60, 16).astype(np.float32)
    s_rel = rng.integers(0, 0x7F, (n, k // 16), dtype=np.uint8)
    assert np.array_equal(oracle.w4a8_dequant_to_int8(packed, codebook, s_rel), ref.w4a8_dequant_to_int8(packed, codebook, s_rel))


def test_attention_pieces(oracle, ref):
    rng = np.random.default_rng(4)
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    for (t, h, w) in ((4, 32, 32), (2, 60, 108)):
        po, pr = oracle.fill_video_pos(512, t, h, w), ref.fill_video_pos(512, t, h, w)
        assert all(np.array_equal(a, b) for a, b in zip(po, pr))
    pt, ph, pw = (a[:80] for a in po)
    co, so = oracle.rope_tables(inv_freq, pt, ph, pw, 0.5)
    cr, sr = ref.rope_tables(inv_freq, pt, ph, pw, 0.5)
    assert np.array_equal(co, cr) and np.array_equal(so, sr)
    heads, hd = 3, 128
    qkv = rng.normal(0, 1, (80, 3 * heads * hd)).astype(np.float32)
    qn, kn = rng.normal(1, 0.1, hd).astype(np.float32), rng.normal(1, 0.1, hd).astype(np.float32)
    qo = oracle.qkv_rope(qkv, qn, kn, co, so, heads, hd, 48)
    qr = ref.qkv_rope(qkv, qn, kn, cr, sr, heads, hd, 48)
    assert all(np.array_equal(a, b) for a, b in zip(qo, qr))
    assert np.array_equal(oracle.sdpa(*qo), ref.sdpa(*qr))


def test_rect_sdpa_reduces_to_reference_on_square(oracle, ref):
    """The rectangular form used for cross-attention is the reference loop with the key count
    decoupled; with Lq == Lk and equal strides it must give the reference's bits."""
    rng = np.random.default_rng(5)
    q, k, v = (rng.normal(0, 1, (19, 2, 32)).astype(np.float32) for _ in range(3))
    assert np.array_equal(oracle.sdpa(q, k, v), ref.sdpa(q, k, v))
    # every query row of a rectangular call equals the square call restricted to those keys
    out = oracle.sdpa(q[:5], k, v)
    assert np.array_equal(out, ref.sdpa(q, k, v)[:5])


def test_checksum(oracle, ref):
    x = np.random.default_rng(6).normal(0, 1, 1000).astype(np.float32)
    assert oracle.checksum_f32(x) == ref.checksum_f32(x)


def test_dense_and_euler_step_bit_exact(oracle, ref):
    """Patch-embedding / final-head linear and the Euler update: the restatement against the reference's
    own functions (h3_dit_w4a8_dense_f32, h3_dit_w4a8_euler_step_f32), including the rejected sigma pairs."""
    rng = np.random.default_rng(90)
    for m, n, k, with_bias in ((37, 64, 96, True), (5, 96, 3072, True), (9, 32, 40, False)):
        x = rng.normal(0, 1, (m, k)).astype(np.float32)
        w = rng.normal(0, 0.05, (n, k)).astype(np.float32)
        b = rng.normal(0, 0.1, n).astype(np.float32) if with_bias else None
        assert np.array_equal(oracle.dense(x, w, b), ref.dense(x, w, b))
    s = rng.normal(0, 1, 1000).astype(np.float32)
    v = rng.normal(0, 1, 1000).astype(np.float32)
    assert np.array_equal(oracle.euler_step(s, v, 0.75, 0.5), ref.euler_step(s, v, 0.75, 0.5))
    for sigma, nxt in ((0.5, 0.5), (0.25, 0.5), (0.5, -0.1), (float("nan"), 0.1), (float("inf"), 0.1)):
        assert oracle.euler_step(s, v, sigma, nxt) is None and ref.euler_step(s, v, sigma, nxt) is None
