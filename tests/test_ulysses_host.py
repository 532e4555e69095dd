"""Host model of the sequence<->head all-to-all, following the reference's own host test
(tests/test_h3_ulysses.c:22-236): integer-valued fill, exact comparison, U=2 and U=8."""
import numpy as np
import pytest


def fill(rank, seq_local, heads, hd):
    i = np.arange(seq_local * 3 * heads * hd, dtype=np.float32).reshape(seq_local, 3, heads, hd)
    return i + 1 + rank * 100000


@pytest.mark.parametrize("u,seq_local,heads,hd", [(2, 32, 56, 8), (8, 8, 56, 8), (4, 5, 24, 16), (1, 7, 24, 8)])
@pytest.mark.parametrize("dtype", [np.float32, np.uint16])
def test_a2a_permutation(oracle, u, seq_local, heads, hd, dtype):
    hl = heads // u
    local = [fill(r, seq_local, heads, hd).astype(dtype) for r in range(u)]
    gathered = oracle.ulysses_a2a_qkv(local, heads, hd)
    for r in range(u):
        for src in range(u):
            want = local[src][:, :, r * hl:(r + 1) * hl, :]
            got = gathered[r][src * seq_local:(src + 1) * seq_local]
            assert np.array_equal(got, want)
    # attention-out direction: send the Q slice back; every rank recovers its own Q rows for all heads
    back = oracle.ulysses_a2a_attn([np.ascontiguousarray(g[:, 0]) for g in gathered], heads, hd)
    for r in range(u):
        assert np.array_equal(back[r], local[r][:, 0])


def test_pad_and_local_rows(oracle):
    L = oracle.lib
    assert L.ho_ulysses_pad_seq(50220, 64) == 50240
    assert [L.ho_ulysses_local_rows(50240, u, 0) for u in (2, 4, 8)] == [25120, 12560, 6280]
    assert L.ho_ulysses_local_rows(16000, 2, 1) == 8000 and L.ho_ulysses_local_rows(16000, 8, 0) == 2000
    assert L.ho_ulysses_validate(24, 64, 1, 8, 1) == 1 and L.ho_ulysses_validate(24, 64, 1, 16, 1) == 0


@pytest.mark.parametrize("u,seq_local,heads,hd", [(2, 32, 8, 8), (8, 8, 24, 8), (4, 5, 24, 16)])
def test_direct_store_addresses_equal_the_exchange(oracle, u, seq_local, heads, hd):
    """The exchange-free path stores (row, head) slices straight into the destination rank's buffers.
    Its address arithmetic (GEMM epilogue: peer = h / hl, row = rank*seq_local + s, head = h % hl; attention
    epilogue: owner = row / seq_local, row % seq_local, head = rank*hl + h), mirrored here in numpy, must place
    every value where the reference's all-to-all places it."""
    hl = heads // u
    local = [fill(r, seq_local, heads, hd) for r in range(u)]
    want = oracle.ulysses_a2a_qkv(local, heads, hd)           # per rank [u*seq_local, 3, hl, hd]
    got = [np.zeros((3, u * seq_local, hl, hd), np.float32) for _ in range(u)]   # separate Q, K, V buffers
    for rank in range(u):
        for s in range(seq_local):
            for which in range(3):
                for h in range(heads):
                    peer = h // hl
                    got[peer][which, rank * seq_local + s, h - peer * hl] = local[rank][s, which, h]
    for r in range(u):
        assert np.array_equal(np.moveaxis(got[r], 0, 1), want[r])
    # attention output: rank r holds rows of the whole sequence for its hl heads
    att = [np.ascontiguousarray(w[:, 0]) for w in want]       # [u*seq_local, hl, hd] on every rank
    back_want = oracle.ulysses_a2a_attn(att, heads, hd)        # per rank [seq_local, heads, hd]
    back = [np.zeros((seq_local, heads, hd), np.float32) for _ in range(u)]
    for rank in range(u):
        for row in range(u * seq_local):
            owner = row // seq_local
            back[owner][row - owner * seq_local, rank * hl:(rank + 1) * hl] = att[rank][row]
    for r in range(u):
        assert np.array_equal(back[r], back_want[r])
