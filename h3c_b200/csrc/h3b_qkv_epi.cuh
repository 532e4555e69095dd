// QK-norm and split-half RoPE on one head (128 values) that a thread of a GEMM epilogue holds in registers: shared by
// the int8 and the NVFP4 GEMM, arithmetic and order of the stand-alone kernel k_qkv_rope so that a chain that runs
// them in an epilogue and one that runs them stand-alone give the same bits.
#pragma once
#include <cuda_runtime.h>

namespace h3b {

// split-half RoPE: dimension d pairs with d + RH (h3_dit_w4a8.c:2850-2883), cos/sin rows of RH floats
template <int RH>
__device__ __forceinline__ void rope_split_half(float (&v)[128], const float *cr, const float *sr) {
#pragma unroll
    for (int d4 = 0; d4 < RH / 4; d4++) {
        const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cr) + d4);
        const float4 s4 = __ldg(reinterpret_cast<const float4 *>(sr) + d4);
        const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int d = d4 * 4 + e;
            const float lo = v[d], hi = v[d + RH];
            v[d] = __fsub_rn(__fmul_rn(lo, cc[e]), __fmul_rn(hi, sn[e]));
            v[d + RH] = __fadd_rn(__fmul_rn(hi, cc[e]), __fmul_rn(lo, sn[e]));
        }
    }
}

// v <- v * rsqrt(mean(v^2) + eps) * w (h3_dit_w4a8.c:2836-2849).  Sum of squares: sixteen partial sums of eight
// consecutive values each, then a pairwise tree, the order of the stand-alone kernel's sixteen lanes and xor butterfly.
__device__ __forceinline__ void qk_norm_head(float (&v)[128], const float *w, float eps) {
    float part[16];
#pragma unroll
    for (int l = 0; l < 16; l++) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) t = __fmaf_rn(v[8 * l + i], v[8 * l + i], t);
        part[l] = t;
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1)
#pragma unroll
        for (int l = 0; l < o; l++) part[l] = __fadd_rn(part[l], part[l + o]);
    const float inv = 1.0f / sqrtf(part[0] / 128.0f + eps);
#pragma unroll
    for (int c4 = 0; c4 < 32; c4++) {
        const float4 n4 = __ldg(reinterpret_cast<const float4 *>(w) + c4);
        v[4 * c4] = __fmul_rn(__fmul_rn(v[4 * c4], inv), n4.x);
        v[4 * c4 + 1] = __fmul_rn(__fmul_rn(v[4 * c4 + 1], inv), n4.y);
        v[4 * c4 + 2] = __fmul_rn(__fmul_rn(v[4 * c4 + 2], inv), n4.z);
        v[4 * c4 + 3] = __fmul_rn(__fmul_rn(v[4 * c4 + 3], inv), n4.w);
    }
}

}  // namespace h3b
