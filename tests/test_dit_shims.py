"""The Metal twin's DiT signatures (h3_dit.h:94-140) as exported by libh3_b200.so: the host conversions and the
reuse schedule against the known answers of the reference's own tests (tests/test_h3.c:122-141, 351-375, read as
text), and, where the reference-built checker exists, against its CUDA-side twins live.  No GPU needed."""
import ctypes as C

import numpy as np
import pytest

import h3c_b200
from h3c_b200.lib import load


def ptr(a):
    return a.ctypes.data


def test_reuse_schedule_known_answers():
    L = load()
    sel = np.zeros(50, np.uint8)
    assert L.h3_dit_reuse_schedule(20, 3, ptr(sel), 50) == 8
    assert list(np.flatnonzero(sel[:20])) == [0, 3, 6, 9, 12, 15, 18, 19]
    assert L.h3_dit_reuse_schedule(20, 2, ptr(sel), 50) == 11
    assert all(sel[s] == (s % 2 == 0 or s == 19) for s in range(20))
    assert L.h3_dit_reuse_schedule(50, 3, ptr(sel), 50) == 18
    assert all(sel[s] == (s % 3 == 0 or s == 49) for s in range(50))
    assert L.h3_dit_reuse_schedule(20, 1, ptr(sel), 50) == 20
    assert L.h3_dit_reuse_schedule(20, 3, ptr(sel), 19) == -1
    assert L.h3_dit_reuse_schedule(20, 33, ptr(sel), 50) == -1 and L.h3_dit_reuse_schedule(0, 3, ptr(sel), 50) == -1


def test_row_conversions_known_answers():
    L = load()
    c, t, h, w = 3, 2, 4, 6
    n = c * t * h * w
    latent = np.arange(n, dtype=np.float32)
    rows, back = np.empty(n, np.float32), np.empty(n, np.float32)
    assert L.h3_dit_patchify_video(ptr(latent), c, t, h, w, ptr(rows), n) == 1
    assert list(rows[:12]) == [0, 1, 6, 7, 48, 49, 54, 55, 96, 97, 102, 103]
    assert L.h3_dit_unpatchify_video(ptr(rows), c, t, h, w, ptr(back), n) == 1
    assert np.array_equal(latent, back)
    assert L.h3_dit_patchify_video(ptr(latent), c, t, h, w, ptr(rows), n - 1) == 0
    assert L.h3_dit_patchify_video(ptr(latent), c, t, 3, w, ptr(rows), c * t * 3 * w) == 0      # odd height
    ac, at = 4, 3
    audio = np.arange(ac * 2 * at, dtype=np.float32)
    packed, unpacked = np.empty_like(audio), np.empty_like(audio)
    assert L.h3_dit_pack_audio(ptr(audio), ac, at, ptr(packed), audio.size) == 1
    assert list(packed) == [0, 6, 12, 18, 1, 7, 13, 19, 2, 8, 14, 20, 3, 9, 15, 21, 4, 10, 16, 22, 5, 11, 17, 23]
    assert L.h3_dit_unpack_audio(ptr(packed), ac, at, ptr(unpacked), audio.size) == 1
    assert np.array_equal(audio, unpacked)
    assert L.h3_dit_pack_audio(ptr(audio), ac, at, ptr(packed), audio.size + 1) == 0


def test_entry_points_bound_to_the_metal_object_say_so():
    with pytest.raises(h3c_b200.H3Error, match="Metal path: unavailable on this box"):
        h3c_b200.call("h3_dit_forward", None, 0, None, None, None, None)
    with pytest.raises(h3c_b200.H3Error, match="Metal path: unavailable on this box"):
        h3c_b200.call("h3_dit_denoise_euler", None, None, None, 1, None, None)
    assert load().h3_dit_video_elements(None) == 0 and load().h3_dit_audio_elements(None) == 0


def test_against_the_reference_cuda_side_twins(ref):
    """h3_dit_w4a8_reuse_schedule and h3_dit_w4a8_pack_audio_latent (32 channels) are the reference's copies of
    the same arithmetic on its CUDA side."""
    L = load()
    for steps, interval in [(20, 3), (50, 7), (7, 32), (1, 1), (33, 2)]:
        a, b = np.zeros(steps, np.uint8), np.zeros(steps, np.uint8)
        assert L.h3_dit_reuse_schedule(steps, interval, ptr(a), steps) == \
            ref.lib.h3_dit_w4a8_reuse_schedule(steps, interval, C.c_void_p(ptr(b)), C.c_size_t(steps))
        assert np.array_equal(a, b)
    at = 11
    audio = np.random.default_rng(0).normal(0, 1, 32 * 2 * at).astype(np.float32)
    mine, theirs = np.empty_like(audio), np.empty_like(audio)
    assert L.h3_dit_pack_audio(ptr(audio), 32, at, ptr(mine), audio.size) == 1
    err = C.create_string_buffer(256)
    assert ref.lib.h3_dit_w4a8_pack_audio_latent(C.c_void_p(ptr(audio)), at, C.c_void_p(ptr(theirs)), err, C.c_size_t(256)) == 1
    assert np.array_equal(mine, theirs)
