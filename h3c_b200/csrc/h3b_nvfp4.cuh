// The reference's software rounding rule for NVFP4 (E2M1 values, one UE4M3 scale per 16 elements) and the byte
// position of a scale in the 128 x 4 tile layout (h3_gpu_cuda.cu:4468-4552), shared by the stand-alone quantiser
// and the row kernel that quantises in its last stage.
#pragma once
#include <stdint.h>

namespace h3b {

// The reference's encoder (h3_gpu_cuda.cu:4498-4513: frexpf, lroundf, ldexpf) on the bits of the float: for a
// normal v = 1.f x 2^e the biased field is E = e + 7 and the mantissa lroundf(0.f x 8) = (f23 + 2^19) >> 20 (half
// away from zero = half up for a positive value); E <= 0 is the subnormal range of the format, lroundf(v x 2^9).
// Same byte as the library-call form for each of the 2,139,095,040 positive finite floats (checked exhaustively on
// the host); the quantiser tests compare whole tensors of scale bytes with the CPU restatement of the reference.
__device__ __forceinline__ uint8_t f32_to_ue4m3(float v) {
    if (!(v > 0.0f)) return 0;
    const uint32_t bits = __float_as_uint(v);
    int E = (int)(bits >> 23) - 127 + 7;
    if ((bits >> 23) == 0) E = -200;   // f32 subnormal: far below the format
    if (E <= 0) {
        // half up by adding the predecessor of one half (adding 0.5 itself would round 0.49999997 up to 1)
        const int m = __float2int_rz(__fadd_rn(__fmul_rn(v, 512.0f), 0.49999997f));
        return (uint8_t)(m > 7 ? 7 : m);
    }
    if (E >= 15) return 0x7E;
    uint32_t m = ((bits & 0x7fffffu) + (1u << 19)) >> 20;
    if (m == 8) {
        E++;
        m = 0;
        if (E >= 15) return 0x7E;
    }
    return (uint8_t)((E << 3) | (int)m);
}

__device__ __forceinline__ float ue4m3_to_f32(uint8_t b) {   // h3_gpu_cuda.cu:4515-4520
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    if (e == 0) return __fmul_rn((float)m, 0.001953125f);                 // m / 8 x 2^-6
    if (e == 15 && m == 7) return __int_as_float(0x7fc00000);
    return __uint_as_float(((e + 120u) << 23) | (m << 20));               // (1 + m / 8) x 2^(e - 7)
}

__device__ __forceinline__ uint32_t e2m1_nibble(float q) {   // h3_gpu_cuda.cu:4468-4496
    const float a = fabsf(q);
    uint32_t mag = (a >= 0.25f) + (a >= 0.75f) + (a >= 1.25f) + (a >= 1.75f) + (a >= 2.5f) + (a >= 3.5f) + (a >= 5.0f);
    return ((q < 0.0f && mag != 0) ? 8u : 0u) | mag;
}

// byte offset of the scale of (row, 16-block) in the 128x4-blocked layout (h3_gpu_cuda.cu:4534-4552)
__device__ __forceinline__ size_t sf_offset(size_t row, size_t blk, size_t ncb) {
    const size_t r128 = row & 127u;
    return ((row >> 7) * ncb + (blk >> 2)) * 512u + 16u * (r128 & 31u) + 4u * (r128 >> 5) + (blk & 3u);
}


// 16 values held four per lane by four consecutive lanes (`mask` = the lanes taking part): scale byte of the block
// and this lane's four codes, packed high nibble = even k (the reference's byte order), as the two bytes that
// follow each other in the packed row.
__device__ __forceinline__ uint16_t nvfp4_quad(float4 v, unsigned mask, uint8_t *scale_byte) {
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 2));
    float scale = amax > 0.0f ? amax / 6.0f : 1.0f;
    uint8_t sb = f32_to_ue4m3(scale);
    if (sb == 0) sb = 1;
    scale = ue4m3_to_f32(sb);
    const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
    *scale_byte = sb;
    const uint32_t b0 = (e2m1_nibble(__fmul_rn(v.x, inv)) << 4) | e2m1_nibble(__fmul_rn(v.y, inv));
    const uint32_t b1 = (e2m1_nibble(__fmul_rn(v.z, inv)) << 4) | e2m1_nibble(__fmul_rn(v.w, inv));
    return (uint16_t)(b0 | (b1 << 8));
}

}  // namespace h3b
