// NVFP4 (E2M1 values, one UE4M3 scale per 16 elements, 128x4-blocked scale layout) activation
// quantisation.  Rounding is the reference's software rule (h3_gpu_cuda.cu:4468-4614), not the
// hardware cvt: E2M1 by a threshold table with ties going up in magnitude, scale = amax / 6
// converted with frexpf + lroundf and clamped to at least byte 1.
#include "h3b_internal.h"
#include "h3b_nvfp4.cuh"

namespace h3b {

// One thread per 16-element block; rows in [m, ceil128(m)) only clear their scale bytes.
__global__ void k_quant_nvfp4(const float *x, size_t m, size_t m_pad, size_t k, uint8_t *packed, uint8_t *sf) {
    const size_t nc = k / 16, ncb = k / 64;
    const size_t total = m_pad * nc;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / nc, blk = i - row * nc;
        if (row >= m) {
            sf[sf_offset(row, blk, ncb)] = 0;
            continue;
        }
        const float4 *src = reinterpret_cast<const float4 *>(x + row * k + blk * 16);
        float v[16];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float4 t = src[j];
            v[4 * j] = t.x; v[4 * j + 1] = t.y; v[4 * j + 2] = t.z; v[4 * j + 3] = t.w;
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(v[j]));
        float scale = amax > 0.0f ? amax / 6.0f : 1.0f;
        uint8_t sb = f32_to_ue4m3(scale);
        if (sb == 0) sb = 1;
        scale = ue4m3_to_f32(sb);
        const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
        sf[sf_offset(row, blk, ncb)] = sb;
        uint32_t lo = 0, hi = 0;   // high nibble = even k (the reference's byte order)
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            lo |= ((e2m1_nibble(__fmul_rn(v[j], inv)) << 4) | e2m1_nibble(__fmul_rn(v[j + 1], inv))) << (4 * j);
            hi |= ((e2m1_nibble(__fmul_rn(v[8 + j], inv)) << 4) | e2m1_nibble(__fmul_rn(v[9 + j], inv))) << (4 * j);
        }
        *reinterpret_cast<uint2 *>(packed + row * (k / 2) + blk * 8) = make_uint2(lo, hi);
    }
}

}  // namespace h3b

using namespace h3b;

extern "C" {

size_t h3_cuda_nvfp4_sf_bytes(size_t rows, size_t k) {
    if (rows == 0 || k == 0 || (k & 63u)) return 0;
    return ((rows + 127u) / 128u) * (k / 64u) * 512u;
}

int h3_cuda_quantize_act_nvfp4_dev(h3_cuda *cuda, const float *d_x, size_t m, size_t k, uint8_t *d_x_fp4,
                                   uint8_t *d_sf, char *error, size_t error_size) {
    if (!cuda || !d_x || !d_x_fp4 || !d_sf || !m || !k) return fail(error, error_size, "invalid quantize_act_nvfp4 arguments");
    if (k % 64) return fail(error, error_size, "quantize_act_nvfp4: K=%zu must be a multiple of 64", k);
    if ((reinterpret_cast<uintptr_t>(d_x) & 15) || (reinterpret_cast<uintptr_t>(d_x_fp4) & 7))
        return fail(error, error_size, "quantize_act_nvfp4: misaligned buffers");
    const size_t m_pad = (m + 127) / 128 * 128;
    const size_t total = m_pad * (k / 16);
    size_t grid = ceil_div(total, 256);
    if (grid > (size_t)cuda->sm_count * 32) grid = (size_t)cuda->sm_count * 32;
    k_quant_nvfp4<<<(unsigned)grid, 256, 0, cuda->op_stream>>>(d_x, m, m_pad, k, d_x_fp4, d_sf);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_quant_nvfp4 launch");
    return 1;
}

}  // extern "C"
