// HBM-bound row-wise kernels of the DiT block: gate / RMSNorm / adaLN modulate /
// ConvRot / per-row INT8 quantisation fused in one launch, plus the elementwise
// gate, SwiGLU, GELU, cast and QK-norm+RoPE kernels.
//
// Arithmetic follows the reference's CPU functions operation by operation
// (explicit __fmul_rn / __fadd_rn so the compiler does not contract them into
// FMAs); only the order of the row reductions differs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "h3b_internal.h"
#include "h3b_nvfp4.cuh"

namespace h3b {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// value as it reads back after being stored in T
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f<T>(from_f<T>(v)); }

// V consecutive elements as one or two aligned vector accesses (4, 8, 16 or 32 bytes in total)
template <typename T, int V>
__device__ __forceinline__ void load_vec(const T *p, float (&out)[V]) {
    constexpr int BYTES = sizeof(T) * V;
    if constexpr (V == 1) {
        out[0] = to_f<T>(p[0]);
    } else if constexpr (BYTES == 32) {
        uint4 raw[2];
        raw[0] = reinterpret_cast<const uint4 *>(p)[0];
        raw[1] = reinterpret_cast<const uint4 *>(p)[1];
        const T *e = reinterpret_cast<const T *>(raw);
#pragma unroll
        for (int i = 0; i < V; i++) out[i] = to_f<T>(e[i]);
    } else {
        static_assert(BYTES == 16 || BYTES == 8 || BYTES == 4, "unsupported vector width");
        using VT = typename std::conditional<BYTES == 16, uint4, typename std::conditional<BYTES == 8, uint2, uint32_t>::type>::type;
        VT raw = *reinterpret_cast<const VT *>(p);
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < V; i++) out[i] = to_f<T>(e[i]);
    }
}
template <typename T, int V>
__device__ __forceinline__ void store_vec(T *p, const float (&in)[V]) {
    constexpr int BYTES = sizeof(T) * V;
    if constexpr (V == 1) {
        p[0] = from_f<T>(in[0]);
    } else if constexpr (BYTES == 32) {
        uint4 raw[2];
        T *e = reinterpret_cast<T *>(raw);
#pragma unroll
        for (int i = 0; i < V; i++) e[i] = from_f<T>(in[i]);
        reinterpret_cast<uint4 *>(p)[0] = raw[0];
        reinterpret_cast<uint4 *>(p)[1] = raw[1];
    } else {
        static_assert(BYTES == 16 || BYTES == 8 || BYTES == 4, "unsupported vector width");
        using VT = typename std::conditional<BYTES == 16, uint4, typename std::conditional<BYTES == 8, uint2, uint32_t>::type>::type;
        VT raw;
        T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
        for (int i = 0; i < V; i++) e[i] = from_f<T>(in[i]);
        *reinterpret_cast<VT *>(p) = raw;
    }
}

// V f32 values through the read-only path (one 16-byte load when V == 4); `fill` where the pointer is null
template <int V>
__device__ __forceinline__ void load_vec_ro(const float *p, float (&out)[V], float fill) {
    if (!p) {
#pragma unroll
        for (int i = 0; i < V; i++) out[i] = fill;
    } else if constexpr (V == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
        out[0] = t.x; out[1] = t.y; out[2] = t.z; out[3] = t.w;
    } else {
#pragma unroll
        for (int i = 0; i < V; i++) out[i] = __ldg(p + i);
    }
}

__device__ __forceinline__ float block_sum(float v, float *red) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += red[i];
    return t;
}
__device__ __forceinline__ float block_max(float v, float *red) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < (int)(blockDim.x >> 5); i++) t = fmaxf(t, red[i]);
    return t;
}

__device__ __forceinline__ int8_t quant_code(float v, float inv) {
    float q = roundf(__fmul_rn(v, inv));   // half away from zero, as the reference
    q = fminf(fmaxf(q, -127.0f), 127.0f);
    return (int8_t)(int)q;
}

struct NormParams {
    const void *x, *branch;
    const float *norm_w, *mod;
    const uint32_t *row_map;
    unsigned width, slots, gate_slot, shift_slot, scale_slot;
    float eps;
    int identity, gs;
    int sylvester;       // ConvRot by the Walsh-Hadamard matrix (radix-2 butterflies) instead of the regular one
    void *gated, *normed;
    float *rot;
    int8_t *q;
    float *scales;
    uint8_t *fp4, *sf;   // NVFP4 codes [rows, width/2] and scale bytes (128 x 4 tile layout) of the final row values
};

// V = elements per vector access (4 when width % 4 == 0 and all pointers are
// 16-byte aligned, else 1).  Dynamic shared memory: width floats.
template <typename T, int V>
__global__ void __launch_bounds__(256) k_norm(NormParams p) {
    extern __shared__ float row[];
    __shared__ float red[8];
    const size_t r = blockIdx.x;
    const unsigned W = p.width;
    const size_t mrow = p.row_map ? p.row_map[r] : r;
    const float *mod = p.mod ? p.mod + mrow * p.slots * W : nullptr;
    const T *x = reinterpret_cast<const T *>(p.x) + r * W;
    const T *br = p.branch ? reinterpret_cast<const T *>(p.branch) + r * W : nullptr;
    T *gated = p.gated ? reinterpret_cast<T *>(p.gated) + r * W : nullptr;
    T *normed = p.normed ? reinterpret_cast<T *>(p.normed) + r * W : nullptr;

    // Rotate-and-quantise of plain rows (the reference's quantised linear on f32 activations): the warp-resident
    // rotation below reads the row straight from global memory, nothing is staged and nothing is reduced first.
    const bool direct = V == 4 && p.identity && !br && p.gs > 0 && !p.sylvester && (W & 255u) == 0;

    // ---- stage the row (optionally residual + branch * gate), sum of squares
    float ss = 0.0f;
    for (unsigned c = threadIdx.x * V; c < W && !direct; c += blockDim.x * V) {
        float v[V];
        load_vec<T, V>(x + c, v);
        if (br) {
            float b[V];
            load_vec<T, V>(br + c, b);
#pragma unroll
            for (int i = 0; i < V; i++) {
                float g = mod ? mod[p.gate_slot * W + c + i] : 1.0f;
                v[i] = round_to<T>(__fadd_rn(v[i], __fmul_rn(b[i], g)));
            }
            if (gated) store_vec<T, V>(gated + c, v);
        }
#pragma unroll
        for (int i = 0; i < V; i++) {
            row[c + i] = v[i];
            ss = __fadd_rn(ss, __fmul_rn(v[i], v[i]));
        }
    }
    float amax = 0.0f;
    if (!p.identity) {
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)W + p.eps);
        for (unsigned c = threadIdx.x * V; c < W; c += blockDim.x * V) {
            // the weight and modulation values of the V columns are fetched first, as vectors through the read-only
            // path: scalar loads between the shared-memory stores below are not reordered by the compiler and
            // each exposed a round trip to L2
            float wv[V], sc[V], sh[V];
            load_vec_ro<V>(p.norm_w ? p.norm_w + c : nullptr, wv, 1.0f);
            load_vec_ro<V>(mod ? mod + p.scale_slot * W + c : nullptr, sc, 0.0f);
            load_vec_ro<V>(mod ? mod + p.shift_slot * W + c : nullptr, sh, 0.0f);
            float y[V];
#pragma unroll
            for (int i = 0; i < V; i++) {
                float n = __fmul_rn(__fmul_rn(row[c + i], inv), wv[i]);
                if (mod) n = __fadd_rn(__fmul_rn(n, __fadd_rn(1.0f, sc[i])), sh[i]);
                y[i] = round_to<T>(n);
                row[c + i] = y[i];
                amax = fmaxf(amax, fabsf(y[i]));
            }
            if (normed) store_vec<T, V>(normed + c, y);
        }
    } else if (p.gs == 0) {   // (with a rotation the maximum is taken after it)
        // same element ownership as the staging loop, so no barrier is needed here
        for (unsigned c = threadIdx.x * V; c < W; c += blockDim.x * V)
#pragma unroll
            for (int i = 0; i < V; i++) amax = fmaxf(amax, fabsf(row[c + i]));
    }

    bool fp4_done = false;
    // ---- ConvRot: y = x * H per group, H = kron-power of the 4x4 regular Hadamard / sqrt(gs).
    // H is symmetric, so this is a radix-4 butterfly network with strides 1, 4, 16, 64.
    if (p.gs > 0 && p.sylvester) {
        // H3_CONVROT_SYLVESTER=1: the reference's in-place radix-2 transform, butterfly for butterfly, then one
        // multiplication by 1/sqrt(gs) (h3_w4a8_dequant.c:241-258): bit-identical to it
        for (int h = 1, sh = 0; h < p.gs; h <<= 1, sh++) {
            __syncthreads();
            for (unsigned b = threadIdx.x; b < W / 2; b += blockDim.x) {
                const unsigned lo = b & (unsigned)(h - 1), base = (((b >> sh) << sh) << 1) + lo;
                const float u = row[base], v = row[base + h];
                row[base] = __fadd_rn(u, v);
                row[base + h] = __fsub_rn(u, v);
            }
        }
        __syncthreads();
        const float norm = 1.0f / sqrtf((float)p.gs);
        amax = 0.0f;
        for (unsigned c = threadIdx.x; c < W; c += blockDim.x) {
            const float v = __fmul_rn(row[c], norm);
            row[c] = v;
            amax = fmaxf(amax, fabsf(v));
            if (p.rot) p.rot[r * W + c] = v;
        }
    } else if (p.gs > 0 && (W & 255u) == 0) {
        // Warp-resident form (every width of the block path is a multiple of 256): a warp takes 256 consecutive
        // elements, lane l holding [4l, 4l+4) and [128+4l, 128+4l+4), so that the stride-1 butterfly is inside a lane,
        // strides 4 and 16 are lane exchanges (xor 1,2,3 and 4,8,12) and stride 64 pairs the two halves of lanes
        // l and l^16.  Of a butterfly's four inputs a0..a3 (by position) the sum (a0+a1)+(a2+a3) is symmetric under
        // the exchanges used, and output k is sum - 2 a(3-k), which for every lane is "sum - 2 x the value three
        // strides away": the same arithmetic as the shared-memory network below, value for value, without its
        // barriers and index arithmetic.  Scaling, the row maximum, the f32 output and the NVFP4 codes follow while
        // the values are still in registers.
        if (!direct) __syncthreads();   // the row is complete in shared memory
        const float norm = 1.0f / sqrtf((float)p.gs);   // exact: gs is a power of four
        const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
        auto lane_bfly = [](float x, int d) {
            const float x1 = __shfl_xor_sync(0xffffffffu, x, d), x2 = __shfl_xor_sync(0xffffffffu, x, 2 * d),
                        x3 = __shfl_xor_sync(0xffffffffu, x, 3 * d);
            const float sum = (x + x1) + (x2 + x3);
            return sum - 2.0f * x3;
        };
        amax = 0.0f;
        for (unsigned g = warp; g < W / 256; g += nw) {
            float *grp = row + g * 256;
            float a[4], b[4];
            if (direct) {
                if constexpr (V == 4) {
                    load_vec<T, 4>(x + g * 256 + 4 * lane, a);
                    load_vec<T, 4>(x + g * 256 + 128 + 4 * lane, b);
                }
            } else {
                const float4 lo4 = *reinterpret_cast<const float4 *>(grp + 4 * lane);
                const float4 hi4 = *reinterpret_cast<const float4 *>(grp + 128 + 4 * lane);
                a[0] = lo4.x; a[1] = lo4.y; a[2] = lo4.z; a[3] = lo4.w;
                b[0] = hi4.x; b[1] = hi4.y; b[2] = hi4.z; b[3] = hi4.w;
            }
            {   // stride 1
                float sa = (a[0] + a[1]) + (a[2] + a[3]), sb = (b[0] + b[1]) + (b[2] + b[3]);
                const float t0 = sa - 2.0f * a[3], t1 = sa - 2.0f * a[2], t2 = sa - 2.0f * a[1], t3 = sa - 2.0f * a[0];
                a[0] = t0; a[1] = t1; a[2] = t2; a[3] = t3;
                const float u0 = sb - 2.0f * b[3], u1 = sb - 2.0f * b[2], u2 = sb - 2.0f * b[1], u3 = sb - 2.0f * b[0];
                b[0] = u0; b[1] = u1; b[2] = u2; b[3] = u3;
            }
            if (p.gs >= 16) {
#pragma unroll
                for (int i = 0; i < 4; i++) { a[i] = lane_bfly(a[i], 1); b[i] = lane_bfly(b[i], 1); }
            }
            if (p.gs >= 64) {
#pragma unroll
                for (int i = 0; i < 4; i++) { a[i] = lane_bfly(a[i], 4); b[i] = lane_bfly(b[i], 4); }
            }
            if (p.gs >= 256) {   // positions: first half of lanes < 16, first half of lanes >= 16, second halves likewise
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float pa = __shfl_xor_sync(0xffffffffu, a[i], 16), pb = __shfl_xor_sync(0xffffffffu, b[i], 16);
                    const float sum = (a[i] + pa) + (b[i] + pb);
                    a[i] = sum - 2.0f * pb;
                    b[i] = sum - 2.0f * pa;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a[i] = a[i] * norm;
                b[i] = b[i] * norm;
                amax = fmaxf(amax, fmaxf(fabsf(a[i]), fabsf(b[i])));
            }
            const float4 ra = make_float4(a[0], a[1], a[2], a[3]), rb = make_float4(b[0], b[1], b[2], b[3]);
            *reinterpret_cast<float4 *>(grp + 4 * lane) = ra;
            *reinterpret_cast<float4 *>(grp + 128 + 4 * lane) = rb;
            const unsigned c0 = g * 256 + 4 * lane, c1 = c0 + 128;
            if (p.rot) {
                float *ro = p.rot + r * W;
                if ((reinterpret_cast<uintptr_t>(p.rot) & 15) == 0) {
                    *reinterpret_cast<float4 *>(ro + c0) = ra;
                    *reinterpret_cast<float4 *>(ro + c1) = rb;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        ro[c0 + i] = a[i];
                        ro[c1 + i] = b[i];
                    }
                }
            }
            if (p.fp4) {   // four lanes = one 16-element block, in both halves
                uint8_t s0, s1;
                uint8_t *dst = p.fp4 + r * (size_t)(W / 2);
                *reinterpret_cast<uint16_t *>(dst + c0 / 2) = nvfp4_quad(ra, 0xffffffffu, &s0);
                *reinterpret_cast<uint16_t *>(dst + c1 / 2) = nvfp4_quad(rb, 0xffffffffu, &s1);
                if ((lane & 3) == 0) {
                    p.sf[sf_offset(r, c0 / 16, W / 64)] = s0;
                    p.sf[sf_offset(r, c1 / 16, W / 64)] = s1;
                }
            }
        }
        fp4_done = p.fp4 != nullptr;
    } else if (p.gs > 0) {
        for (int stride = 1, sh = 0; stride < p.gs; stride <<= 2, sh += 2) {
            __syncthreads();
            for (unsigned b = threadIdx.x; b < W / 4; b += blockDim.x) {
                // stride is a power of two: shifts and masks (a division by a run-time value costs some thirty
                // instructions, and this loop runs once per four elements and stage)
                const unsigned lo = b & (unsigned)(stride - 1), hi = b >> sh;
                unsigned base = ((hi << sh) << 2) + lo;
                float a0 = row[base], a1 = row[base + stride], a2 = row[base + 2 * stride], a3 = row[base + 3 * stride];
                float s = (a0 + a1) + (a2 + a3);
                row[base] = s - 2.0f * a3;
                row[base + stride] = s - 2.0f * a2;
                row[base + 2 * stride] = s - 2.0f * a1;
                row[base + 3 * stride] = s - 2.0f * a0;
            }
        }
        __syncthreads();
        const float norm = 1.0f / sqrtf((float)p.gs);   // exact: gs is a power of four
        amax = 0.0f;
        for (unsigned c = threadIdx.x; c < W; c += blockDim.x) {
            float v = row[c] * norm;
            row[c] = v;
            amax = fmaxf(amax, fabsf(v));
            if (p.rot) p.rot[r * W + c] = v;
        }
    }

    // ---- NVFP4 quantisation of the final row values (width % 16 == 0): four lanes per 16-element block
    if (p.fp4 && !fp4_done) {
        __syncthreads();   // the row is complete in shared memory, whichever stage wrote it last
        uint8_t *dst = p.fp4 + r * (size_t)(W / 2);
        for (unsigned base = 0; base < W; base += blockDim.x * 4) {
            const unsigned c = base + threadIdx.x * 4;
            const bool on = c < W;
            const unsigned mask = __ballot_sync(0xffffffffu, on);
            if (on) {
                uint8_t sb;
                const uint16_t codes = nvfp4_quad(*reinterpret_cast<const float4 *>(row + c), mask, &sb);
                *reinterpret_cast<uint16_t *>(dst + c / 2) = codes;
                if ((threadIdx.x & 3) == 0) p.sf[sf_offset(r, c / 16, W / 64)] = sb;
            }
        }
    }

    // ---- per-row INT8 quantisation
    if (p.q) {
        amax = block_max(amax, red);
        const float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
        const float inv = 1.0f / scale;
        if (threadIdx.x == 0) p.scales[r] = scale;
        int8_t *q = p.q + r * W;
        if constexpr (V == 4) {
            for (unsigned c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
                char4 o;
                o.x = quant_code(row[c], inv);
                o.y = quant_code(row[c + 1], inv);
                o.z = quant_code(row[c + 2], inv);
                o.w = quant_code(row[c + 3], inv);
                *reinterpret_cast<char4 *>(q + c) = o;
            }
        } else {
            for (unsigned c = threadIdx.x; c < W; c += blockDim.x) q[c] = quant_code(row[c], inv);
        }
    }
}

// Register-resident variant for 16-bit rows whose width is THREADS * NV * 8: each thread keeps
// NV 16-byte vectors (8 elements each) of the row, so the row is read from HBM once and never
// staged in shared memory.  Same arithmetic, same order per element as k_norm; the row
// reductions combine per-thread partials (fixed order), so results are deterministic.
template <typename T, int NV, int THREADS>
__global__ void __launch_bounds__(THREADS) k_norm_reg(NormParams p) {
    __shared__ float red[THREADS / 32];
    const size_t r = blockIdx.x;
    const unsigned W = p.width;
    const size_t mrow = p.row_map ? p.row_map[r] : r;
    const float *mod = p.mod ? p.mod + mrow * p.slots * W : nullptr;
    const T *x = reinterpret_cast<const T *>(p.x) + r * W;
    const T *br = p.branch ? reinterpret_cast<const T *>(p.branch) + r * W : nullptr;
    T *gated = p.gated ? reinterpret_cast<T *>(p.gated) + r * W : nullptr;
    T *normed = p.normed ? reinterpret_cast<T *>(p.normed) + r * W : nullptr;
    float v[NV][8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const unsigned c = (j * THREADS + threadIdx.x) * 8;
        load_vec<T, 8>(x + c, v[j]);
        if (br) {
            float b[8];
            load_vec<T, 8>(br + c, b);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float g = mod ? mod[p.gate_slot * W + c + i] : 1.0f;
                v[j][i] = round_to<T>(__fadd_rn(v[j][i], __fmul_rn(b[i], g)));
            }
            if (gated) store_vec<T, 8>(gated + c, v[j]);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) ss = __fadd_rn(ss, __fmul_rn(v[j][i], v[j][i]));
    }
    float amax = 0.0f;
    if (!p.identity) {
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)W + p.eps);
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const unsigned c = (j * THREADS + threadIdx.x) * 8;
            float w[8], sc[8], sh[8];
            if (p.norm_w) {
                load_vec<float, 4>(p.norm_w + c, reinterpret_cast<float(&)[4]>(w[0]));
                load_vec<float, 4>(p.norm_w + c + 4, reinterpret_cast<float(&)[4]>(w[4]));
            }
            if (mod) {
                load_vec<float, 4>(mod + p.scale_slot * W + c, reinterpret_cast<float(&)[4]>(sc[0]));
                load_vec<float, 4>(mod + p.scale_slot * W + c + 4, reinterpret_cast<float(&)[4]>(sc[4]));
                load_vec<float, 4>(mod + p.shift_slot * W + c, reinterpret_cast<float(&)[4]>(sh[0]));
                load_vec<float, 4>(mod + p.shift_slot * W + c + 4, reinterpret_cast<float(&)[4]>(sh[4]));
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float n = __fmul_rn(__fmul_rn(v[j][i], inv), p.norm_w ? w[i] : 1.0f);
                if (mod) n = __fadd_rn(__fmul_rn(n, __fadd_rn(1.0f, sc[i])), sh[i]);
                v[j][i] = round_to<T>(n);
                amax = fmaxf(amax, fabsf(v[j][i]));
            }
            if (normed) store_vec<T, 8>(normed + c, v[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < NV; j++)
#pragma unroll
            for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[j][i]));
    }
    if (p.q) {
        amax = block_max(amax, red);
        const float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
        const float inv = 1.0f / scale;
        if (threadIdx.x == 0) p.scales[r] = scale;
        int8_t *q = p.q + r * W;
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const unsigned c = (j * THREADS + threadIdx.x) * 8;
            union { int8_t b[8]; uint2 u; } o;
#pragma unroll
            for (int i = 0; i < 8; i++) o.b[i] = quant_code(v[j][i], inv);
            *reinterpret_cast<uint2 *>(q + c) = o.u;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Streaming row kernel for the block's hot cases (16-bit rows, no branch / ConvRot): RMSNorm and/or
// adaLN modulate -> round to the stream type -> per-row INT8 quantisation, or quantisation alone.
// Persistent CTAs walk the rows with a stride of the grid; the norm weight and the row's modulation
// vectors stay in registers while consecutive rows map to the same modulation row (the usual case: one
// conditioning vector for all video tokens), the next row is fetched while the current one is reduced,
// and the per-element work is trimmed to about ten instructions (two-wide f32 arithmetic, one block
// barrier per reduction).  Element arithmetic is the reference's, operation by operation; only the
// row-sum order differs.

__device__ __forceinline__ void mul2(float &d0, float &d1, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void add2f(float &d0, float &d1, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void fma2f(float &d0, float &d1, float a0, float a1, float b0, float b1) {   // d += a * b
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 rd, {%0, %1};\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rd;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two 16-bit stream values of one 32-bit word as floats
template <typename T> __device__ __forceinline__ void unpack2(uint32_t w, float &lo, float &hi);
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float &lo, float &hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack2<__half>(uint32_t w, float &lo, float &hi) {
    float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
    lo = f.x; hi = f.y;
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
// roundf(y) for |y| < 2^22 as an integer: truncation of y + copysign(pred(0.5), y).  Adding the
// predecessor of one half instead of one half keeps 0.49999997 from rounding up to 1 in the addition;
// checked against floor(|y| + 0.5) for every float in [0, 128].
__device__ __forceinline__ int round_half_away(float y) {
    const float h = __uint_as_float((__float_as_uint(y) & 0x80000000u) | 0x3effffffu);
    return __float2int_rz(__fadd_rn(y, h));
}
// four codes -> one word, saturating to int8 (byte 0 = a)
__device__ __forceinline__ uint32_t pack_codes(int a, int b, int c, int d) {
    uint32_t hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
    return out;
}

template <typename T, int NV, int THREADS, bool NORM>
__global__ void __launch_bounds__(THREADS) k_rowq(NormParams p, unsigned rows) {
    constexpr int NW = THREADS / 32;
    __shared__ float red_ss[NW];
    __shared__ float red_mx[2][NW];
    const unsigned W = p.width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T *xbase = reinterpret_cast<const T *>(p.x);
    unsigned r = blockIdx.x;
    if (r >= rows) return;

    float w[NORM ? NV : 1][8], sc1[NORM ? NV : 1][8], sh[NORM ? NV : 1][8];   // norm weight, 1 + scale, shift
    size_t cached_mrow = ~(size_t)0;
    if (NORM) {
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const unsigned c = (j * THREADS + threadIdx.x) * 8;
#pragma unroll
            for (int i = 0; i < 8; i++) w[j][i] = 1.0f;
            if (p.norm_w) {
                load_vec<float, 4>(p.norm_w + c, reinterpret_cast<float(&)[4]>(w[j][0]));
                load_vec<float, 4>(p.norm_w + c + 4, reinterpret_cast<float(&)[4]>(w[j][4]));
            }
        }
    }
    uint4 cur[NV], nxt[NV];
#pragma unroll
    for (int j = 0; j < NV; j++)
        cur[j] = *reinterpret_cast<const uint4 *>(xbase + (size_t)r * W + (j * THREADS + threadIdx.x) * 8);
    unsigned par = 0;
    while (true) {
        const unsigned rn = r + gridDim.x;
        if (rn < rows) {
#pragma unroll
            for (int j = 0; j < NV; j++)
                nxt[j] = *reinterpret_cast<const uint4 *>(xbase + (size_t)rn * W + (j * THREADS + threadIdx.x) * 8);
        }
        float v[NV][8];
#pragma unroll
        for (int j = 0; j < NV; j++) {
            const uint32_t *u = reinterpret_cast<const uint32_t *>(&cur[j]);
#pragma unroll
            for (int i = 0; i < 4; i++) unpack2<T>(u[i], v[j][2 * i], v[j][2 * i + 1]);
        }
        float amax = 0.0f;
        if (NORM) {
            const size_t mrow = p.mod ? (p.row_map ? p.row_map[r] : (size_t)r) : 0;
            if (p.mod && mrow != cached_mrow) {
                const float *mod = p.mod + mrow * p.slots * W;
#pragma unroll
                for (int j = 0; j < NV; j++) {
                    const unsigned c = (j * THREADS + threadIdx.x) * 8;
                    load_vec<float, 4>(mod + p.scale_slot * W + c, reinterpret_cast<float(&)[4]>(sc1[j][0]));
                    load_vec<float, 4>(mod + p.scale_slot * W + c + 4, reinterpret_cast<float(&)[4]>(sc1[j][4]));
                    load_vec<float, 4>(mod + p.shift_slot * W + c, reinterpret_cast<float(&)[4]>(sh[j][0]));
                    load_vec<float, 4>(mod + p.shift_slot * W + c + 4, reinterpret_cast<float(&)[4]>(sh[j][4]));
#pragma unroll
                    for (int i = 0; i < 8; i++) sc1[j][i] = __fadd_rn(1.0f, sc1[j][i]);
                }
                cached_mrow = mrow;
            }
            float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
            for (int j = 0; j < NV; j++)
#pragma unroll
                for (int i = 0; i < 8; i += 2) fma2f(s0, s1, v[j][i], v[j][i + 1], v[j][i], v[j][i + 1]);
            float ss = s0 + s1;
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red_ss[warp] = ss;
            __syncthreads();
            ss = 0.0f;
#pragma unroll
            for (int i = 0; i < NW; i++) ss += red_ss[i];
            const float inv = 1.0f / sqrtf(ss / (float)W + p.eps);
            T *normed = p.normed ? reinterpret_cast<T *>(p.normed) + (size_t)r * W : nullptr;
#pragma unroll
            for (int j = 0; j < NV; j++) {
                uint32_t packed[4];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    float n0, n1;
                    mul2(n0, n1, v[j][i], v[j][i + 1], inv, inv);
                    mul2(n0, n1, n0, n1, w[j][i], w[j][i + 1]);
                    if (p.mod) {
                        mul2(n0, n1, n0, n1, sc1[j][i], sc1[j][i + 1]);
                        add2f(n0, n1, n0, n1, sh[j][i], sh[j][i + 1]);
                    }
                    packed[i >> 1] = pack2<T>(n0, n1);
                    unpack2<T>(packed[i >> 1], v[j][i], v[j][i + 1]);
                    amax = max3f(amax, fabsf(v[j][i]), fabsf(v[j][i + 1]));
                }
                if (normed)
                    *reinterpret_cast<uint4 *>(normed + (j * THREADS + threadIdx.x) * 8) =
                        make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < NV; j++)
#pragma unroll
                for (int i = 0; i < 8; i += 2) amax = max3f(amax, fabsf(v[j][i]), fabsf(v[j][i + 1]));
        }
        if (p.q) {
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0) red_mx[par][warp] = amax;
            __syncthreads();
            amax = 0.0f;
#pragma unroll
            for (int i = 0; i < NW; i++) amax = fmaxf(amax, red_mx[par][i]);
            par ^= 1;
            const float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
            const float inv = 1.0f / scale;
            if (threadIdx.x == 0) p.scales[r] = scale;
            int8_t *q = p.q + (size_t)r * W;
#pragma unroll
            for (int j = 0; j < NV; j++) {
                float y[8];
#pragma unroll
                for (int i = 0; i < 8; i += 2) mul2(y[i], y[i + 1], v[j][i], v[j][i + 1], inv, inv);
                uint2 o;
                o.x = pack_codes(round_half_away(y[0]), round_half_away(y[1]), round_half_away(y[2]), round_half_away(y[3]));
                o.y = pack_codes(round_half_away(y[4]), round_half_away(y[5]), round_half_away(y[6]), round_half_away(y[7]));
                *reinterpret_cast<uint2 *>(q + (j * THREADS + threadIdx.x) * 8) = o;
            }
        }
        if (rn >= rows) break;
#pragma unroll
        for (int j = 0; j < NV; j++) cur[j] = nxt[j];
        r = rn;
    }
}

template <typename T, int NV, int THREADS, bool NORM>
static int rowq_launch_k(h3_cuda *cuda, const NormParams &p, size_t rows, char *error, size_t error_size) {
    auto kern = k_rowq<T, NV, THREADS, NORM>;
    static int per_sm[64];   // resident CTAs per SM of this kernel, asked once per device
    const int dev = cuda->device & 63;
    if (per_sm[dev] == 0) {
        int n = 0;
        H3B_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, THREADS, 0), "k_rowq occupancy");
        per_sm[dev] = n > 0 ? n : 1;
    }
    size_t grid = (size_t)cuda->sm_count * per_sm[dev];
    if (grid > rows) grid = rows;
    ProfScope prof(cuda, PROF_ROWS);
    kern<<<(unsigned)grid, THREADS, 0, cuda->op_stream>>>(p, (unsigned)rows);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_rowq launch");
    return 1;
}
// Streaming kernel when the shape allows it; returns -1 when it does not apply.
template <typename T>
static int rowq_dispatch(h3_cuda *cuda, const NormParams &p, size_t rows, char *error, size_t error_size) {
    if constexpr (sizeof(T) != 2) {
        return -1;
    } else {
    if (p.gs != 0 || p.rot || p.branch || p.gated || p.fp4) return -1;
    auto al16 = [](const void *q_) { return !q_ || (reinterpret_cast<uintptr_t>(q_) & 15) == 0; };
    if (!al16(p.x) || !al16(p.normed) || !al16(p.norm_w) || !al16(p.mod) || (p.q && (reinterpret_cast<uintptr_t>(p.q) & 7)))
        return -1;
    // Quantisation alone is latency-bound: many threads with one vector each.  With a norm, the two block
    // reductions per row cost as many instructions as eight elements' arithmetic, so each thread takes
    // three or four vectors and the CTA has few warps.
    if (!p.identity) {
        switch (p.width) {
        case 1024: return rowq_launch_k<T, 1, 128, true>(cuda, p, rows, error, error_size);
        case 2048: return rowq_launch_k<T, 2, 128, true>(cuda, p, rows, error, error_size);
        case 3072: return rowq_launch_k<T, 3, 128, true>(cuda, p, rows, error, error_size);
        case 4096: return rowq_launch_k<T, 4, 128, true>(cuda, p, rows, error, error_size);
        case 6144: return rowq_launch_k<T, 3, 256, true>(cuda, p, rows, error, error_size);
        case 8192: return rowq_launch_k<T, 4, 256, true>(cuda, p, rows, error, error_size);
        case 12288: return rowq_launch_k<T, 3, 512, true>(cuda, p, rows, error, error_size);
        }
        return -1;
    }
    switch (p.width) {
    case 1024: return rowq_launch_k<T, 1, 128, false>(cuda, p, rows, error, error_size);
    case 2048: return rowq_launch_k<T, 1, 256, false>(cuda, p, rows, error, error_size);
    case 3072: return rowq_launch_k<T, 1, 384, false>(cuda, p, rows, error, error_size);
    case 4096: return rowq_launch_k<T, 1, 512, false>(cuda, p, rows, error, error_size);
    case 6144: return rowq_launch_k<T, 2, 384, false>(cuda, p, rows, error, error_size);
    case 8192: return rowq_launch_k<T, 2, 512, false>(cuda, p, rows, error, error_size);
    case 12288: return rowq_launch_k<T, 3, 512, false>(cuda, p, rows, error, error_size);
    case 16384: return rowq_launch_k<T, 4, 512, false>(cuda, p, rows, error, error_size);
    }
    return -1;
    }
}

template <typename T, int NV, int THREADS>
static int norm_reg_launch(h3_cuda *cuda, const NormParams &p, size_t rows, char *error, size_t error_size) {
    ProfScope prof(cuda, PROF_ROWS);
    k_norm_reg<T, NV, THREADS><<<(unsigned)rows, THREADS, 0, cuda->op_stream>>>(p);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_norm_reg launch");
    return 1;
}

// Picks the register-resident kernel when the shape allows it; returns -1 when it does not apply.
template <typename T>
static int norm_reg_dispatch(h3_cuda *cuda, const NormParams &p, size_t rows, char *error, size_t error_size) {
    if (sizeof(T) != 2 || p.gs != 0 || p.rot || p.fp4 || p.width % 1024) return -1;
    auto al16 = [](const void *q_) { return !q_ || (reinterpret_cast<uintptr_t>(q_) & 15) == 0; };
    if (!al16(p.x) || !al16(p.branch) || !al16(p.gated) || !al16(p.normed) || !al16(p.norm_w) || !al16(p.mod) ||
        (p.q && (reinterpret_cast<uintptr_t>(p.q) & 7)))
        return -1;
    switch (p.width) {
    case 1024: return norm_reg_launch<T, 1, 128>(cuda, p, rows, error, error_size);
    case 2048: return norm_reg_launch<T, 2, 128>(cuda, p, rows, error, error_size);
    case 3072: return norm_reg_launch<T, 3, 128>(cuda, p, rows, error, error_size);
    case 4096: return norm_reg_launch<T, 4, 128>(cuda, p, rows, error, error_size);
    case 6144: return norm_reg_launch<T, 3, 256>(cuda, p, rows, error, error_size);
    case 8192: return norm_reg_launch<T, 4, 256>(cuda, p, rows, error, error_size);
    case 12288: return norm_reg_launch<T, 6, 256>(cuda, p, rows, error, error_size);
    case 16384: return norm_reg_launch<T, 4, 512>(cuda, p, rows, error, error_size);
    }
    return -1;
}

template <typename T>
static int norm_dispatch(h3_cuda *cuda, const NormParams &p, size_t rows, bool vec, char *error, size_t error_size) {
    if (sizeof(T) == 2) {
        int rc = rowq_dispatch<T>(cuda, p, rows, error, error_size);
        if (rc >= 0) return rc;
        rc = norm_reg_dispatch<T>(cuda, p, rows, error, error_size);
        if (rc >= 0) return rc;
    }
    size_t smem = (size_t)p.width * sizeof(float);
    if (smem > 200 * 1024) return fail(error, error_size, "row width %u too large for the row kernel", p.width);
    auto kv = k_norm<T, 4>;
    auto ks = k_norm<T, 1>;
    if (smem > 40 * 1024) {   // the kernel also has a few static shared words
        H3B_CUDA_OK(cudaFuncSetAttribute(kv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "smem attr");
        H3B_CUDA_OK(cudaFuncSetAttribute(ks, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "smem attr");
    }
    ProfScope prof(cuda, PROF_ROWS);
    if (vec) kv<<<(unsigned)rows, 256, smem, cuda->op_stream>>>(p);
    else ks<<<(unsigned)rows, 256, smem, cuda->op_stream>>>(p);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_norm launch");
    return 1;
}

int launch_norm(h3_cuda *cuda, const h3b_norm_args *a, char *error, size_t error_size) {
    if (!cuda || !a || !a->d_x || !a->rows || !a->width) return fail(error, error_size, "norm: invalid arguments");
    if (a->d_q && !a->d_scales) return fail(error, error_size, "norm: d_q without d_scales");
    if (a->d_modulation && a->slots == 0) return fail(error, error_size, "norm: slots must be > 0");
    // the reference's switch, read per call: Walsh-Hadamard groups of any power of two up to 256
    const int sylvester = a->convrot_gs > 0 && strcmp(h3_plugin_value("H3_CONVROT_SYLVESTER"), "1") == 0;
    if (sylvester) {
        if (a->convrot_gs < 2 || a->convrot_gs > 256 || (a->convrot_gs & (a->convrot_gs - 1)))
            return fail(error, error_size, "invalid fwht groupsize=%d K=%zu", a->convrot_gs, a->width);
    } else if (a->convrot_gs != 0 && a->convrot_gs != 4 && a->convrot_gs != 16 && a->convrot_gs != 64 &&
               a->convrot_gs != 256)
        return fail(error, error_size, "norm: ConvRot group size %d unsupported (0, 4, 16, 64, 256)", a->convrot_gs);
    if (a->convrot_gs && a->width % (size_t)a->convrot_gs)
        return fail(error, error_size, "K=%zu not divisible by convrot_groupsize=%d", a->width, a->convrot_gs);
    if (a->rows > 0x7fffffffu) return fail(error, error_size, "norm: too many rows");
    NormParams p;
    p.x = a->d_x; p.branch = a->d_branch; p.norm_w = a->d_norm_w; p.mod = a->d_modulation;
    p.row_map = a->d_row_map; p.width = (unsigned)a->width; p.slots = (unsigned)a->slots;
    p.gate_slot = (unsigned)a->gate_slot; p.shift_slot = (unsigned)a->shift_slot;
    p.scale_slot = (unsigned)a->scale_slot; p.eps = a->epsilon; p.identity = a->identity;
    p.sylvester = sylvester;
    p.gs = a->convrot_gs; p.gated = a->d_gated; p.normed = a->d_normed; p.rot = a->d_rot; p.q = a->d_q;
    p.scales = a->d_scales; p.fp4 = a->d_fp4; p.sf = a->d_sf;
    if (a->d_fp4) {
        if (!a->d_sf) return fail(error, error_size, "norm: d_fp4 without d_sf");
        if (a->width % 64) return fail(error, error_size, "norm: NVFP4 output needs a width that is a multiple of 64");
        if (reinterpret_cast<uintptr_t>(a->d_fp4) & 1) return fail(error, error_size, "norm: misaligned d_fp4");
        // scale bytes of the pad rows [rows, ceil128(rows)) are zero (h3_gpu_cuda.cu:4590-4596): they sit inside the
        // last 128-row tile, which is cleared before the kernel writes the bytes of its real rows
        if (a->rows % 128) {
            const size_t tile = (a->width / 64) * 512;
            H3B_CUDA_OK(cudaMemsetAsync(a->d_sf + (a->rows / 128) * tile, 0, tile, cuda->op_stream), "norm: clearing pad scales");
        }
    }
    // vector path: 4 elements per access (16 bytes of f32, 8 bytes of 16-bit types, 4 codes)
    const uintptr_t amask = 4 * dtype_bytes(a->dtype) - 1;
    auto al = [&](const void *q_, uintptr_t mask) { return !q_ || (reinterpret_cast<uintptr_t>(q_) & mask) == 0; };
    bool vec = a->width % 4 == 0 && al(a->d_x, amask) && al(a->d_branch, amask) && al(a->d_gated, amask) &&
               al(a->d_normed, amask) && al(a->d_q, 3) && al(a->d_norm_w, 15) && al(a->d_modulation, 15);
    switch (a->dtype) {
    case H3B_F32: return norm_dispatch<float>(cuda, p, a->rows, vec, error, error_size);
    case H3B_BF16: return norm_dispatch<__nv_bfloat16>(cuda, p, a->rows, vec, error, error_size);
    case H3B_F16: return norm_dispatch<__half>(cuda, p, a->rows, vec, error, error_size);
    }
    return fail(error, error_size, "norm: unsupported dtype %d", a->dtype);
}

int launch_quant(h3_cuda *cuda, const void *x, int dtype, size_t m, size_t k, int8_t *q, float *scales, char *error,
                 size_t error_size) {
    h3b_norm_args a = {};
    a.d_x = x; a.rows = m; a.width = k; a.dtype = dtype; a.identity = 1; a.d_q = q; a.d_scales = scales;
    return launch_norm(cuda, &a, error, error_size);
}

int launch_convrot(h3_cuda *cuda, const float *x, size_t m, size_t k, int gs, float *y, char *error,
                   size_t error_size) {
    if (gs <= 0) {
        if (x != y) H3B_CUDA_OK(cudaMemcpyAsync(y, x, m * k * sizeof(float), cudaMemcpyDeviceToDevice, cuda->op_stream), "convrot copy");
        return 1;
    }
    h3b_norm_args a = {};
    a.d_x = x; a.rows = m; a.width = k; a.dtype = H3B_F32; a.identity = 1; a.convrot_gs = gs; a.d_rot = y;
    return launch_norm(cuda, &a, error, error_size);
}

// ------------------------------------------------------------- elementwise

template <typename T>
__global__ void k_gate(const T *res, const T *br, const float *mod, const uint32_t *row_map, size_t rows,
                       unsigned width, unsigned slots, unsigned gate_slot, T *out) {
    size_t n = rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        size_t r = i / width;
        unsigned c = (unsigned)(i - r * width);
        size_t mrow = row_map ? row_map[r] : r;
        float g = mod[(mrow * slots + gate_slot) * width + c];
        out[i] = from_f<T>(__fadd_rn(to_f<T>(res[i]), __fmul_rn(to_f<T>(br[i]), g)));
    }
}

template <typename T>
__global__ void k_swiglu(const T *fused, size_t rows, unsigned width, T *out) {
    size_t n = rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        size_t r = i / width;
        unsigned c = (unsigned)(i - r * width);
        float g = to_f<T>(fused[r * 2 * width + c]), u = to_f<T>(fused[r * 2 * width + width + c]);
        out[i] = from_f<T>(__fmul_rn(g / __fadd_rn(1.0f, expf(-g)), u));
    }
}

__device__ __forceinline__ float gelu_tanh_f(float v) {
    float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    if (inner <= -10.0f) return 0.0f;
    if (inner >= 10.0f) return v;
    return 0.5f * v * (1.0f + tanhf(inner));
}

template <typename T>
__global__ void k_gelu(const T *in, T *out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f<T>(gelu_tanh_f(to_f<T>(in[i])));
}

template <typename TI, typename TO>
__global__ void k_cast(const TI *in, TO *out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f<TO>(to_f<TI>(in[i]));
}

// modulation[o] = b[o] + sum_i W[o,i] * t[i]; one warp per output (h3_dit_w4a8.c:2256-2261)
__global__ void k_adaln_project(const float *w, const float *b, size_t out_dim, unsigned in_dim, const float *t,
                                float *out) {
    const size_t o = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (o >= out_dim) return;
    const unsigned lane = threadIdx.x & 31;
    float acc = 0.0f;
    for (unsigned i = lane; i < in_dim; i += 32) acc = fmaf(w[o * in_dim + i], t[i], acc);
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) out[o] = b[o] + acc;
}

static unsigned ew_grid(h3_cuda *cuda, size_t n) {
    size_t g = ceil_div(n, 256);
    size_t cap = (size_t)cuda->sm_count * 16;
    return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

int launch_gate(h3_cuda *cuda, const void *res, const void *branch, const float *mod, const uint32_t *row_map,
                size_t rows, size_t width, size_t slots, size_t gate_slot, void *out, int dtype, char *error,
                size_t error_size) {
    if (!res || !branch || !mod || !out || !width || !slots) return fail(error, error_size, "gate: invalid arguments");
    unsigned g = ew_grid(cuda, rows * width);
    if (dtype == H3B_F32)
        k_gate<float><<<g, 256, 0, cuda->op_stream>>>((const float *)res, (const float *)branch, mod, row_map, rows,
                                                      (unsigned)width, (unsigned)slots, (unsigned)gate_slot, (float *)out);
    else if (dtype == H3B_BF16)
        k_gate<__nv_bfloat16><<<g, 256, 0, cuda->op_stream>>>((const __nv_bfloat16 *)res, (const __nv_bfloat16 *)branch,
                                                              mod, row_map, rows, (unsigned)width, (unsigned)slots,
                                                              (unsigned)gate_slot, (__nv_bfloat16 *)out);
    else
        return fail(error, error_size, "gate: unsupported dtype %d", dtype);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_gate launch");
    return 1;
}

int launch_swiglu(h3_cuda *cuda, const void *fused, size_t rows, size_t width, void *out, int dtype, char *error,
                  size_t error_size) {
    if (!fused || !out || !width) return fail(error, error_size, "swiglu: invalid arguments");
    unsigned g = ew_grid(cuda, rows * width);
    if (dtype == H3B_F32)
        k_swiglu<float><<<g, 256, 0, cuda->op_stream>>>((const float *)fused, rows, (unsigned)width, (float *)out);
    else if (dtype == H3B_BF16)
        k_swiglu<__nv_bfloat16><<<g, 256, 0, cuda->op_stream>>>((const __nv_bfloat16 *)fused, rows, (unsigned)width,
                                                                (__nv_bfloat16 *)out);
    else
        return fail(error, error_size, "swiglu: unsupported dtype %d", dtype);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_swiglu launch");
    return 1;
}

// ---------------------------------------------------------- QK-norm + RoPE
//
// LANES = head_dim / EPL threads per (row, head); each owns EPL consecutive dimensions
// (16-byte loads for 16-bit inputs with EPL = 8).  Split-half pairing (d, d + rope_half)
// lives rope_half / EPL lanes apart; consecutive pairing (2d, 2d+1) lives inside one lane.
template <typename TI, typename TO, int EPL, int LANES>
__global__ void __launch_bounds__(256) k_qkv_rope(const TI *qkv, const float *q_norm, const float *k_norm,
                                                  const float *cosT, const float *sinT, size_t seq, unsigned heads,
                                                  unsigned rope_half, float eps, int grouped, int split_half, TO *q,
                                                  TO *k, TO *v) {
    constexpr unsigned HD = EPL * LANES;
    const unsigned lane = threadIdx.x % LANES;
    size_t item = (size_t)blockIdx.x * (blockDim.x / LANES) + threadIdx.x / LANES;
    // surplus groups of the last CTA redo the last item (identical values) so that every lane of a
    // warp takes part in the shuffles below
    if (item >= seq * heads) item = seq * heads - 1;
    const size_t row = item / heads;
    const unsigned head = (unsigned)(item - row * heads);
    const size_t inner = (size_t)heads * HD;
    const TI *base = qkv + row * inner * 3;
    const TI *qb = grouped ? base + (size_t)head * HD * 3 : base + (size_t)head * HD;
    const TI *kb = grouped ? qb + HD : qb + inner;
    const TI *vb = grouped ? kb + HD : qb + 2 * inner;
    const unsigned d0 = lane * EPL;
    float qv[EPL], kv[EPL], vv[EPL];
    load_vec<TI, EPL>(qb + d0, qv);
    load_vec<TI, EPL>(kb + d0, kv);
    load_vec<TI, EPL>(vb + d0, vv);
    float qs = 0.0f, ks = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; i++) {   // the QKV GEMM epilogue repeats this order exactly
        qs = __fmaf_rn(qv[i], qv[i], qs);
        ks = __fmaf_rn(kv[i], kv[i], ks);
    }
    for (int o = LANES / 2; o > 0; o >>= 1) {
        qs = __fadd_rn(qs, __shfl_xor_sync(0xffffffffu, qs, o));
        ks = __fadd_rn(ks, __shfl_xor_sync(0xffffffffu, ks, o));
    }
    const float qi = 1.0f / sqrtf(qs / (float)HD + eps), ki = 1.0f / sqrtf(ks / (float)HD + eps);
#pragma unroll
    for (int i = 0; i < EPL; i++) {
        qv[i] = __fmul_rn(__fmul_rn(qv[i], qi), q_norm[d0 + i]);
        kv[i] = __fmul_rn(__fmul_rn(kv[i], ki), k_norm[d0 + i]);
    }
    if (rope_half) {
        const float *cr = cosT + row * rope_half, *sr = sinT + row * rope_half;
        if (split_half) {
            const int lane_off = (int)(rope_half / EPL);
            float qo[EPL], ko[EPL];
#pragma unroll
            for (int i = 0; i < EPL; i++) {
                // partner values: from lane + off for the low half, lane - off for the high half
                float q_up = __shfl_down_sync(0xffffffffu, qv[i], lane_off, LANES);
                float q_dn = __shfl_up_sync(0xffffffffu, qv[i], lane_off, LANES);
                float k_up = __shfl_down_sync(0xffffffffu, kv[i], lane_off, LANES);
                float k_dn = __shfl_up_sync(0xffffffffu, kv[i], lane_off, LANES);
                unsigned d = d0 + i;
                if (d < rope_half) {
                    float c = cr[d], s = sr[d];
                    qo[i] = __fsub_rn(__fmul_rn(qv[i], c), __fmul_rn(q_up, s));
                    ko[i] = __fsub_rn(__fmul_rn(kv[i], c), __fmul_rn(k_up, s));
                } else if (d < 2 * rope_half) {
                    float c = cr[d - rope_half], s = sr[d - rope_half];
                    qo[i] = __fadd_rn(__fmul_rn(qv[i], c), __fmul_rn(q_dn, s));
                    ko[i] = __fadd_rn(__fmul_rn(kv[i], c), __fmul_rn(k_dn, s));
                } else {
                    qo[i] = qv[i];
                    ko[i] = kv[i];
                }
            }
#pragma unroll
            for (int i = 0; i < EPL; i++) {
                qv[i] = qo[i];
                kv[i] = ko[i];
            }
        } else if constexpr (EPL >= 2) {
#pragma unroll
            for (int i = 0; i < EPL; i += 2) {
                unsigned pair = (d0 + i) >> 1;
                if (pair < rope_half) {
                    float c = cr[pair], s = sr[pair];
                    float q0 = qv[i], q1 = qv[i + 1], k0 = kv[i], k1 = kv[i + 1];
                    qv[i] = __fsub_rn(__fmul_rn(q0, c), __fmul_rn(q1, s));
                    qv[i + 1] = __fadd_rn(__fmul_rn(q0, s), __fmul_rn(q1, c));
                    kv[i] = __fsub_rn(__fmul_rn(k0, c), __fmul_rn(k1, s));
                    kv[i + 1] = __fadd_rn(__fmul_rn(k0, s), __fmul_rn(k1, c));
                }
            }
        }
    }
    const size_t o = (row * heads + head) * HD + d0;
    store_vec<TO, EPL>(q + o, qv);
    store_vec<TO, EPL>(k + o, kv);
    store_vec<TO, EPL>(v + o, vv);
}

template <typename TI, typename TO>
static int qkv_rope_dispatch(h3_cuda *cuda, const void *qkv, const float *qn, const float *kn, const float *c,
                             const float *s, size_t seq, size_t heads, size_t hd, size_t rope_half, float eps,
                             int grouped, int split_half, void *q, void *k, void *v, char *error, size_t error_size) {
    size_t items = seq * heads;
    unsigned grid = (unsigned)ceil_div(items, 16);   // 16 lanes per item, 256 threads
    ProfScope prof(cuda, PROF_ROPE);
#define H3B_ROPE(EPL)                                                                                              \
    k_qkv_rope<TI, TO, EPL, 16><<<grid, 256, 0, cuda->op_stream>>>((const TI *)qkv, qn, kn, c, s, seq, (unsigned)heads, \
                                                                   (unsigned)rope_half, eps, grouped, split_half,  \
                                                                   (TO *)q, (TO *)k, (TO *)v)
    if (hd == 128) H3B_ROPE(8);
    else if (hd == 64) H3B_ROPE(4);
    else return fail(error, error_size, "qkv_rope: head_dim %zu unsupported (64 or 128)", hd);
#undef H3B_ROPE
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_qkv_rope launch");
    return 1;
}

}  // namespace h3b

using namespace h3b;

extern "C" {

int h3b_norm_dev(h3_cuda *cuda, const h3b_norm_args *args, char *error, size_t error_size) {
    return launch_norm(cuda, args, error, error_size);
}

int h3b_quantize_act_int8_dev(h3_cuda *cuda, const void *d_x, int dtype, size_t m, size_t k, int8_t *d_q,
                              float *d_scales, char *error, size_t error_size) {
    if (!cuda || !d_x || !d_q || !d_scales || !m || !k)
        return fail(error, error_size, "invalid quantize_act_int8 arguments");
    return launch_quant(cuda, d_x, dtype, m, k, d_q, d_scales, error, error_size);
}

int h3_cuda_convrot_act_f32_dd(h3_cuda *cuda, const float *d_x, size_t m, size_t k, int convrot_groupsize,
                               float *d_y, char *error, size_t error_size) {
    if (!cuda || !d_x || !d_y || !m || !k) return fail(error, error_size, "invalid convrot_act arguments");
    if (d_x == d_y && convrot_groupsize > 0) return fail(error, error_size, "convrot_act: d_x and d_y must not alias");
    return launch_convrot(cuda, d_x, m, k, convrot_groupsize, d_y, error, error_size);
}

int h3_cuda_adaln_f32_dev(h3_cuda *cuda, const float *d_x, const float *d_norm_w, const float *d_modulation,
                          const uint32_t *d_row_map, size_t rows, size_t width, size_t slots, size_t shift_slot,
                          size_t scale_slot, float epsilon, float *d_out, double *op_ms, char *error,
                          size_t error_size) {
    if (!cuda || !d_x || !d_norm_w || !d_modulation || !d_out || !width || !slots)
        return fail(error, error_size, "invalid adaln arguments");
    h3b_norm_args a = {};
    a.d_x = d_x; a.d_norm_w = d_norm_w; a.d_modulation = d_modulation; a.d_row_map = d_row_map; a.rows = rows;
    a.width = width; a.slots = slots; a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = epsilon;
    a.dtype = H3B_F32; a.d_normed = d_out;
    Timer t(cuda, op_ms);
    int ok = launch_norm(cuda, &a, error, error_size);
    t.stop();
    return ok;
}

int h3_cuda_rms_norm_f32_dev(h3_cuda *cuda, const float *d_x, const float *d_w, size_t rows, size_t width,
                             float eps, float *d_out, char *error, size_t error_size) {
    if (!cuda || !d_x || !d_w || !d_out || !width) return fail(error, error_size, "invalid rms_norm arguments");
    h3b_norm_args a = {};
    a.d_x = d_x; a.d_norm_w = d_w; a.rows = rows; a.width = width; a.epsilon = eps; a.dtype = H3B_F32;
    a.d_normed = d_out;
    return launch_norm(cuda, &a, error, error_size);
}

int h3_cuda_gate_adaln_f32_dev(h3_cuda *cuda, const float *d_residual, const float *d_branch, const float *d_norm_w,
                               const float *d_modulation, const uint32_t *d_row_map, size_t rows, size_t width,
                               size_t slots, size_t gate_slot, size_t shift_slot, size_t scale_slot, float epsilon,
                               float *d_gated, float *d_normed, double *op_ms, char *error, size_t error_size) {
    if (!cuda || !d_residual || !d_branch || !d_norm_w || !d_modulation || !d_gated || !d_normed || !width || !slots)
        return fail(error, error_size, "invalid gate_adaln arguments");
    h3b_norm_args a = {};
    a.d_x = d_residual; a.d_branch = d_branch; a.d_norm_w = d_norm_w; a.d_modulation = d_modulation;
    a.d_row_map = d_row_map; a.rows = rows; a.width = width; a.slots = slots; a.gate_slot = gate_slot;
    a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = epsilon; a.dtype = H3B_F32;
    a.d_gated = d_gated; a.d_normed = d_normed;
    Timer t(cuda, op_ms);
    int ok = launch_norm(cuda, &a, error, error_size);
    t.stop();
    return ok;
}

int h3_cuda_gate_f32_dev(h3_cuda *cuda, const float *d_residual, const float *d_branch, const float *d_modulation,
                         const uint32_t *d_row_map, size_t rows, size_t width, size_t slots, size_t gate_slot,
                         float *d_out, double *op_ms, char *error, size_t error_size) {
    if (!cuda) return fail(error, error_size, "gate: NULL handle");
    Timer t(cuda, op_ms);
    int ok = launch_gate(cuda, d_residual, d_branch, d_modulation, d_row_map, rows, width, slots, gate_slot, d_out,
                         H3B_F32, error, error_size);
    t.stop();
    return ok;
}

int h3_cuda_swiglu_f32_dev(h3_cuda *cuda, const float *d_fused, size_t rows, size_t width, float *d_out,
                           double *op_ms, char *error, size_t error_size) {
    if (!cuda) return fail(error, error_size, "swiglu: NULL handle");
    Timer t(cuda, op_ms);
    int ok = launch_swiglu(cuda, d_fused, rows, width, d_out, H3B_F32, error, error_size);
    t.stop();
    return ok;
}

int h3b_qkv_rope_dev(h3_cuda *cuda, const void *d_qkv, int in_dtype, const float *d_q_norm, const float *d_k_norm,
                     const float *d_rope_cos, const float *d_rope_sin, size_t seq, size_t heads, size_t head_dim,
                     size_t rope_half, float epsilon, int grouped, int split_half, void *d_query, void *d_key,
                     void *d_value, int out_dtype, char *error, size_t error_size) {
    if (!cuda || !d_qkv || !d_q_norm || !d_k_norm || !d_query || !d_key || !d_value || !seq || !heads || !head_dim ||
        (rope_half > 0 && (!d_rope_cos || !d_rope_sin)))
        return fail(error, error_size, "invalid qkv_rope args");
    if (rope_half * 2 > head_dim) return fail(error, error_size, "rope_half too large for head_dim");
    if ((reinterpret_cast<uintptr_t>(d_qkv) | reinterpret_cast<uintptr_t>(d_query) | reinterpret_cast<uintptr_t>(d_key) |
         reinterpret_cast<uintptr_t>(d_value)) & 15)
        return fail(error, error_size, "qkv_rope: tensors must be 16-byte aligned");
    if (split_half && rope_half % (head_dim / 16))
        return fail(error, error_size, "qkv_rope: rope_half must be a multiple of head_dim/16");
#define H3B_QR(TI, TO)                                                                                             \
    return qkv_rope_dispatch<TI, TO>(cuda, d_qkv, d_q_norm, d_k_norm, d_rope_cos, d_rope_sin, seq, heads, head_dim, \
                                     rope_half, epsilon, grouped, split_half, d_query, d_key, d_value, error,      \
                                     error_size)
    if (in_dtype == H3B_F32 && out_dtype == H3B_F32) H3B_QR(float, float);
    if (in_dtype == H3B_F32 && out_dtype == H3B_BF16) H3B_QR(float, __nv_bfloat16);
    if (in_dtype == H3B_BF16 && out_dtype == H3B_BF16) H3B_QR(__nv_bfloat16, __nv_bfloat16);
    if (in_dtype == H3B_BF16 && out_dtype == H3B_F32) H3B_QR(__nv_bfloat16, float);
    if (in_dtype == H3B_F32 && out_dtype == H3B_F16) H3B_QR(float, __half);
    if (in_dtype == H3B_F16 && out_dtype == H3B_F16) H3B_QR(__half, __half);
#undef H3B_QR
    return fail(error, error_size, "qkv_rope: unsupported dtype pair %d -> %d", in_dtype, out_dtype);
}

int h3_cuda_qkv_rope_f32_dev_layout(h3_cuda *cuda, const float *d_qkv, const float *d_q_norm, const float *d_k_norm,
                                    const float *d_rope_cos, const float *d_rope_sin, size_t seq, size_t heads,
                                    size_t head_dim, size_t rope_half, float epsilon, int grouped, int split_half,
                                    float *d_query, float *d_key, float *d_value, double *op_ms, char *error,
                                    size_t error_size) {
    if (!cuda) return fail(error, error_size, "qkv_rope: NULL handle");
    Timer t(cuda, op_ms);
    int ok = h3b_qkv_rope_dev(cuda, d_qkv, H3B_F32, d_q_norm, d_k_norm, d_rope_cos, d_rope_sin, seq, heads, head_dim,
                              rope_half, epsilon, grouped, split_half, d_query, d_key, d_value, H3B_F32, error,
                              error_size);
    t.stop();
    return ok;
}

int h3_cuda_qkv_rope_f32_dev(h3_cuda *cuda, const float *d_qkv, const float *d_q_norm, const float *d_k_norm,
                             const float *d_rope_cos, const float *d_rope_sin, size_t seq, size_t heads,
                             size_t head_dim, size_t rope_half, float epsilon, float *d_query, float *d_key,
                             float *d_value, double *op_ms, char *error, size_t error_size) {
    // reference default: contiguous [Q|K|V] thirds, split-half pairing (h3_dit_w4a8.c:239-253)
    return h3_cuda_qkv_rope_f32_dev_layout(cuda, d_qkv, d_q_norm, d_k_norm, d_rope_cos, d_rope_sin, seq, heads,
                                           head_dim, rope_half, epsilon, 0, 1, d_query, d_key, d_value, op_ms, error,
                                           error_size);
}

int h3b_cast_dev(h3_cuda *cuda, const void *d_in, int in_dtype, void *d_out, int out_dtype, size_t n, char *error,
                 size_t error_size) {
    if (!cuda || !d_in || !d_out) return fail(error, error_size, "cast: invalid arguments");
    if (n == 0) return 1;
    unsigned g = ew_grid(cuda, n);
#define H3B_CAST(TI, TO) k_cast<TI, TO><<<g, 256, 0, cuda->op_stream>>>((const TI *)d_in, (TO *)d_out, n)
    if (in_dtype == H3B_F32 && out_dtype == H3B_BF16) H3B_CAST(float, __nv_bfloat16);
    else if (in_dtype == H3B_BF16 && out_dtype == H3B_F32) H3B_CAST(__nv_bfloat16, float);
    else if (in_dtype == H3B_F32 && out_dtype == H3B_F16) H3B_CAST(float, __half);
    else if (in_dtype == H3B_F16 && out_dtype == H3B_F32) H3B_CAST(__half, float);
    else return fail(error, error_size, "cast: unsupported dtype pair %d -> %d", in_dtype, out_dtype);
#undef H3B_CAST
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_cast launch");
    return 1;
}

int h3_cuda_f32_to_f16_dev(h3_cuda *cuda, const float *d_in, void *d_out_half, size_t n, char *error,
                           size_t error_size) {
    return h3b_cast_dev(cuda, d_in, H3B_F32, d_out_half, H3B_F16, n, error, error_size);
}
int h3_cuda_f16_to_f32_dev(h3_cuda *cuda, const void *d_in_half, float *d_out, size_t n, char *error,
                           size_t error_size) {
    return h3b_cast_dev(cuda, d_in_half, H3B_F16, d_out, H3B_F32, n, error, error_size);
}

int h3b_adaln_project_dev(h3_cuda *cuda, const float *d_w, const float *d_b, size_t out_dim, size_t in_dim,
                          const float *d_t_feat, float *d_out, char *error, size_t error_size) {
    if (!cuda || !d_w || !d_b || !d_t_feat || !d_out || !out_dim || !in_dim)
        return fail(error, error_size, "invalid adaln_project args");
    ProfScope prof(cuda, PROF_OTHER);
    k_adaln_project<<<(unsigned)ceil_div(out_dim, 8), 256, 0, cuda->op_stream>>>(d_w, d_b, out_dim, (unsigned)in_dim,
                                                                                 d_t_feat, d_out);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_adaln_project launch");
    return 1;
}

int h3b_gelu_tanh_dev(h3_cuda *cuda, const void *d_in, void *d_out, int dtype, size_t n, char *error,
                      size_t error_size) {
    if (!cuda || !d_in || !d_out) return fail(error, error_size, "gelu: invalid arguments");
    unsigned g = ew_grid(cuda, n);
    if (dtype == H3B_F32) k_gelu<float><<<g, 256, 0, cuda->op_stream>>>((const float *)d_in, (float *)d_out, n);
    else if (dtype == H3B_BF16)
        k_gelu<__nv_bfloat16><<<g, 256, 0, cuda->op_stream>>>((const __nv_bfloat16 *)d_in, (__nv_bfloat16 *)d_out, n);
    else return fail(error, error_size, "gelu: unsupported dtype %d", dtype);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_gelu launch");
    return 1;
}

}  // extern "C"
