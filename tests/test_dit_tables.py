"""Host-side step tables of the library (RoPE positions, cos/sin tables, time-table row): plain C inside
libh3_b200.so, no GPU needed.  Checked bit for bit against vectors the reference produced
(tests/golden/step_tables.npz) and, where the reference-built checker exists, against it live."""
import ctypes as C

import numpy as np
import pytest

import h3c_b200


def test_tables_match_reference_vectors(golden, oracle):
    g = golden("step_tables")
    inv = g["inv_freq"]
    text_len = int(g["text_len"][0])
    for i, grid in enumerate(g["grids"]):
        t, h, w = (int(v) for v in grid)
        pt, ph, pw = h3c_b200.fill_video_pos(text_len, t, 2 * h, 2 * w)
        cos, sin = h3c_b200.rope_tables(inv, pt, ph, pw, 1.0)
        sums = [oracle.checksum_f32(x) for x in (pt, ph, pw, cos, sin)]
        assert sums == [int(v) for v in g[f"sum_{i}"]], f"grid {grid}"
        assert np.array_equal(cos[:4], g[f"cos_head_{i}"]) and np.array_equal(cos[-4:], g[f"cos_tail_{i}"])
        assert np.array_equal(sin[:4], g[f"sin_head_{i}"]) and np.array_equal(sin[-4:], g[f"sin_tail_{i}"])
        cos2, sin2 = h3c_b200.video_rope_tables(inv, text_len, (t, h, w), 1.0, pad_rows=20)
        assert np.array_equal(cos2[:-20], cos) and np.array_equal(sin2[:-20], sin)
        assert (cos2[-20:] == 1).all() and (sin2[-20:] == 0).all()


def test_t_row_and_span_match_reference_vectors(golden):
    g = golden("step_tables")
    got = [[h3c_b200.t_row_from_sigma(float(s), r) for r in (0, 1, 2, 1025)] for s in g["sigma"]]
    assert np.array_equal(np.array(got, np.uint64), g["t_rows"])
    assert h3c_b200.t_row_from_sigma(float("nan"), 1025) == 1024     # non-finite counts as sigma 0
    span = h3c_b200.load().h3_dit_w4a8_video_span_sum
    assert np.array_equal(np.array([span(t) for t in range(len(g["span_sum"]))], np.float32), g["span_sum"])


def test_bad_arguments_are_refused():
    buf = np.zeros(64, np.float32)
    with pytest.raises(h3c_b200.H3Error):      # odd latent height
        h3c_b200.call("h3_dit_w4a8_fill_metal_video_pos", 0, 1, 3, 4, buf.ctypes.data, buf.ctypes.data, buf.ctypes.data)
    with pytest.raises(h3c_b200.H3Error):      # spatial scale must be positive
        h3c_b200.call("h3_dit_w4a8_rope_tables_f32", buf.ctypes.data, 1, buf.ctypes.data, buf.ctypes.data,
                      buf.ctypes.data, C.c_float(0.0), buf.ctypes.data, buf.ctypes.data)


def test_tables_match_live_reference(ref):
    inv = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    for text_len, (t, h, w), scale in [(0, (1, 1, 1), 1.0), (77, (5, 3, 7), 0.5), (512, (7, 18, 10), 2.0)]:
        a = h3c_b200.fill_video_pos(text_len, t, 2 * h, 2 * w)
        b = ref.fill_video_pos(text_len, t, 2 * h, 2 * w)
        assert all(np.array_equal(x, y) for x, y in zip(a, b))
        got, want = h3c_b200.rope_tables(inv, *a, scale), ref.rope_tables(inv, *b, scale)
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
