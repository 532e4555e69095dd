"""Parity at the benchmark's full sizes.  The CUDA path runs the whole shape; the CPU oracle checks sampled
rows (every column of each sampled row), so the CPU side stays bounded.  Rows always include the first and the
last row tile; at M = 50,220 they include 50,176 ... 50,219, the clipped last 256-row pair tile.

Integer accumulators: bit-exact.  Float epilogues: the tolerance written beside each check."""
import numpy as np
import pytest

from tests.conftest import rel_l2

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

SHAPES_KN = [(3072, 9216), (3072, 3072), (3072, 12288), (12288, 3072)]


@pytest.fixture(scope="module")
def cuda():
    import h3c_b200
    c = h3c_b200.Cuda(0)
    yield c
    c.check()
    c.close()


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.detach().float().cpu().numpy() if t.dtype in (torch.bfloat16, torch.float16) else t.detach().cpu().numpy()


def sample_rows(rng, m, extra=24):
    """First / last rows of the first tiles, the whole tail of the last pair tile, and random rows."""
    tail = np.arange((m - 1) // 256 * 256, m) if m % 256 else np.arange(m - 8, m)
    rows = np.concatenate([[0, 127, 128, 255, 256], tail[:: max(1, len(tail) // 12)], [m - 1], rng.integers(0, m, extra)])
    return np.unique(rows)


def device_codes(m, k, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return torch.randint(-127, 128, (m, k), dtype=torch.int8, device="cuda", generator=g)


def exact_i32(x_rows, w_i8):
    """int8 x int8 -> int32 sums through float64 BLAS (every partial sum is below 2^53, so it is exact)."""
    return (x_rows.astype(np.float64) @ w_i8.astype(np.float64).T).astype(np.int64)


@pytest.fixture(scope="module")
def weights(cuda):
    rng = np.random.default_rng(700)
    out = {}
    for k, n in SHAPES_KN:
        w_i8 = rng.integers(-127, 128, (n, k), dtype=np.int8)
        s = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
        out[(k, n)] = (cuda.weight_from_i8(w_i8, s), w_i8, s)
    return out


@pytest.mark.parametrize("m", [24576, 50220])
@pytest.mark.parametrize("k,n", SHAPES_KN)
def test_gemm_int32_exact_at_benchmark_sizes(cuda, weights, m, k, n):
    rng = np.random.default_rng(m + k + n)
    w, w_i8, _ = weights[(k, n)]
    x = device_codes(m, k, seed=m + 3 * k + n)
    ones = torch.ones(m, dtype=torch.float32, device="cuda")
    acc = cuda.gemm_i8(w, x, ones, out_dtype=torch.int32)
    cuda.check()
    rows = sample_rows(rng, m)
    idx = torch.from_numpy(rows).cuda()
    want = exact_i32(host(x[idx]), w_i8)
    assert np.array_equal(host(acc[idx]).astype(np.int64), want)
    del acc
    torch.cuda.empty_cache()


def test_block_epilogues_at_50220_rows(cuda, oracle, weights):
    """The three epilogues of the benchmark's block at M = 50,220: gate + residual -> bf16, tanh-GELU -> bf16,
    QKV + QK-norm + RoPE -> bf16 Q/K/V."""
    import h3c_b200
    m, slots = 50220, 6
    rng = np.random.default_rng(50220)
    rows = sample_rows(rng, m, extra=12)
    idx = torch.from_numpy(rows).cuda()
    scales = torch.from_numpy(rng.uniform(0.01, 0.05, m).astype(np.float32)).cuda()
    a_rows = host(scales[idx])

    # gate + residual, bf16 stream (K = N = 3072)
    w, w_i8, s = weights[(3072, 3072)]
    x = device_codes(m, 3072, seed=1)
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    res = torch.randn((m, 3072), device="cuda", generator=g).to(torch.bfloat16)
    mod = rng.normal(0, 0.5, (1, slots, 3072)).astype(np.float32)
    y = cuda.gemm_i8(w, x, scales, kind=h3c_b200.EPI_GATE, out_dtype=torch.bfloat16, residual=res, modulation=dev(mod),
                     row_map=torch.zeros(m, dtype=torch.int32, device="cuda"), slots=slots, gate_slot=2)
    cuda.check()
    acc = exact_i32(host(x[idx]), w_i8).astype(np.int32)
    want = oracle.bf16_round(oracle.dequant_gate(acc, a_rows, s, host(res[idx]), mod, np.zeros(len(rows), np.uint32),
                                                 slots, 2))
    assert np.array_equal(host(y[idx]), want)            # same operation order, one rounding: identical bits
    del y, res

    # tanh-GELU, bf16 (K = 3072, N = 12288): the device uses tanh.approx for 16-bit outputs
    w, w_i8, s = weights[(3072, 12288)]
    y = cuda.gemm_i8(w, x, scales, kind=h3c_b200.EPI_GELU, out_dtype=torch.bfloat16)
    cuda.check()
    acc = exact_i32(host(x[idx]), w_i8).astype(np.int32)
    assert rel_l2(host(y[idx]), oracle.dequant_gelu(acc, a_rows, s)) < 3e-3   # bf16 rounding + tanh.approx
    del y

    # QKV + QK-norm + RoPE (K = 3072, N = 9216), tables of the 31 x 30 x 54 grid from the library's host code
    w, w_i8, s = weights[(3072, 9216)]
    heads, hd = 24, 128
    inv_freq = (1.0 / (10000.0 ** (np.arange(16) / 16.0))).astype(np.float32)
    cos, sin = h3c_b200.video_rope_tables(inv_freq, 512, (31, 30, 54))
    qn, kn = rng.normal(1, 0.1, hd).astype(np.float32), rng.normal(1, 0.1, hd).astype(np.float32)
    q, kk, v = cuda.gemm_i8_qkv_rope(w, x, scales, dev(qn), dev(kn), dev(cos), dev(sin), 48, round_qkv=True)
    cuda.check()
    acc = exact_i32(host(x[idx]), w_i8).astype(np.int32)
    # y = a[m] * s[n] * acc evaluated left to right in f32 (h3_w4a8_dequant.c:692-710), then one bf16 rounding
    qkv = oracle.bf16_round((a_rows[:, None] * s[None, :]).astype(np.float32) * acc.astype(np.float32))
    qo, ko, vo = oracle.qkv_rope(qkv, qn, kn, cos[rows], sin[rows], heads, hd, 48)
    assert rel_l2(host(q[idx]), qo) < 3e-3 and rel_l2(host(kk[idx]), ko) < 3e-3
    assert rel_l2(host(v[idx]), vo) < 3e-3


# the third shape has more 256-row bands (79) than the device has CTA pairs: two groups of the grouped tile order
@pytest.mark.parametrize("m,n,k", [(6144, 9216, 3072), (6144, 3072, 12288), (20030, 768, 256)])
def test_gemm_nvfp4_at_benchmark_sizes(cuda, oracle, m, n, k):
    rng = np.random.default_rng(n + k)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    x[rng.random((m, k)) < 0.001] *= 20
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    w4, sfw = oracle.quantize_nvfp4(w, rule=1)
    x4, sfx = cuda.quantize_act_nvfp4(dev(x))
    y = cuda.gemm_fp4(dev(w4), dev(sfw), x4, sfx, alpha=0.5)
    cuda.check()
    rows = sample_rows(rng, m, extra=28)
    assert len(rows) >= 32
    xd = oracle.dequant_nvfp4(host(x4), host(sfx))[:m]          # [m, k] f32: code x block scale
    wd = oracle.dequant_nvfp4(w4, sfw)[:n]
    want = 0.5 * (xd[rows].astype(np.float64) @ wd.astype(np.float64).T)
    assert rel_l2(host(y)[rows], want) < 1e-5


@pytest.mark.parametrize("lq,lk", [(24576, 24576), (50220, 50220), (50220, 512)])
def test_sdpa_at_benchmark_sizes(cuda, oracle, lq, lk):
    """Self-attention at 24,576 and 50,220 tokens and the 50,220 x 512 cross shape, 2 of the 24 heads."""
    rng = np.random.default_rng(lq + lk)
    heads, hd = 2, 128
    g = torch.Generator(device="cuda")
    g.manual_seed(lq * 3 + lk)
    q, k, v = (torch.randn((n, heads, hd), device="cuda", generator=g).to(torch.bfloat16) for n in (lq, lk, lk))
    out = cuda.sdpa_bf16(q, k, v)
    cuda.check()
    rows = np.unique(np.concatenate([[0, 127, 128, 255, 256, lq - 1, lq - 2, (lq - 1) // 256 * 256], rng.integers(0, lq, 8)]))
    assert len(rows) >= 12
    idx = torch.from_numpy(rows).cuda()
    want = oracle.sdpa(host(q[idx]), host(k), host(v))
    assert rel_l2(host(out[idx]), want) < 4e-3
