"""The exact form of the benchmark's weight format (symmetric int4, one f16 scale per 128 input channels): the
weight stays packed on the device, the codes are expanded in registers into the int8 tile of tcgen05.mma, and every
128-K group's int32 sums are scaled in f32 -- against the definition written out in numpy, bit for bit."""
import numpy as np
import pytest

from tests.test_w4g_reexpression import unpack_q

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def cuda():
    import h3c_b200
    c = h3c_b200.Cuda(0)
    yield c
    c.check()
    c.close()


def exact_product(xq, xs, packed, scales_bits, group=128):
    """y = a * sum_g s[n,g] * int32 partial sum of group g: f32 multiply, f32 add, in group order."""
    m, k = xq.shape
    n = packed.shape[0]
    q = unpack_q(packed)
    s = scales_bits.view(np.float16).astype(np.float32)
    part = np.einsum("mgk,ngk->mng", xq.reshape(m, k // group, group).astype(np.int64),
                     q.reshape(n, k // group, group).astype(np.int64)).astype(np.int32)
    y = np.zeros((m, n), np.float32)
    for g in range(k // group):
        y += s[None, :, g] * part[:, :, g].astype(np.float32)
    return y * xs[:, None]


@pytest.mark.parametrize("m,n,k", [(96, 384, 3072), (257, 192, 1024), (1, 128, 128), (130, 260, 256), (64, 136, 12288)])
def test_exact_group_product_bit_for_bit(cuda, oracle, m, n, k):
    rng = np.random.default_rng(m + n + k)
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    packed, scales = oracle.w4g128_encode(w, 128)
    scales = np.ascontiguousarray(scales).view(np.uint16)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    x[rng.random((m, k)) < 0.001] *= 20
    xq, xs = oracle.quantize_act_int8(x)
    h = cuda.w4g_exact_weight(packed, scales)
    y = cuda.gemm_w4g_exact(h, n, torch.from_numpy(xq).cuda(), torch.from_numpy(xs).cuda())
    cuda.check()
    want = exact_product(xq, xs, packed, scales)
    assert np.array_equal(y.cpu().numpy(), want)
    if n % 8 == 0:
        yb = cuda.gemm_w4g_exact(h, n, torch.from_numpy(xq).cuda(), torch.from_numpy(xs).cuda(), out_dtype=torch.bfloat16)
        assert np.array_equal(yb.float().cpu().numpy(), torch.from_numpy(want).to(torch.bfloat16).float().numpy())
    cuda.w4g_exact_weight_free(h)


def test_extreme_codes_and_scales(cuda):
    """Codes -8 and 7 everywhere with activations +-127: the largest group sums the format allows (x 16 inside the
    kernel) stay inside int32, and the scale 1/16 trick is exact for the smallest and largest f16 scales."""
    m, n, k = 128, 128, 256
    q = np.where(np.arange(n * k).reshape(n, k) % 3 == 0, -8, 7).astype(np.int8)
    packed = ((q[:, 0::2] & 0xF) | ((q[:, 1::2] & 0xF) << 4)).astype(np.uint8)
    scales = np.empty((n, k // 128), np.float16)
    scales[:, 0], scales[:, 1] = np.float16(6e-8), np.float16(65504.0)
    xq = np.where(np.arange(m * k).reshape(m, k) % 2 == 0, 127, -127).astype(np.int8)
    xs = np.full(m, 2.0 ** -20, np.float32)
    h = cuda.w4g_exact_weight(packed, scales.view(np.uint16))
    y = cuda.gemm_w4g_exact(h, n, torch.from_numpy(xq).cuda(), torch.from_numpy(xs).cuda())
    cuda.check()
    assert np.array_equal(y.cpu().numpy(), exact_product(xq, xs, packed, scales.view(np.uint16)))
    cuda.w4g_exact_weight_free(h)
