// Exact linear on symmetric int4 weights with one f16 scale per 128 input channels:
//     y[m,n] = a[m] * sum_g s[n,g] * (sum_{k in group g} x_i8[m,k] * q[n,k]),   q in [-8, 7]
// int32 partial sums per 128-K group, each scaled in f32 and added in group order -- the definition of the
// format, bit for bit.  (The default path of the library decodes such a weight once to resident int8 with one
// scale per output channel and runs the plain int8 GEMM; this kernel is the selectable exact form.)
//
// The weight stays packed in HBM, two codes per byte (half the bytes of the int8 form).  One CTA per 128 x 128
// output tile, persistent over tiles; per 128-K group:
//   warp 0       TMA: the 128 x 128 int8 activation tile (128-byte swizzle) and the 128 x 64 bytes of packed codes
//   warps 2-5    unpack: four lanes per weight row read its 64 packed bytes from shared memory, expand them in
//                registers and write the 128-byte row of the int8 tile that tcgen05.mma reads (same swizzle, no bank
//                conflicts on either side).  A code is put into the HIGH nibble of its byte, i.e. the tile holds
//                16 q: two logic operations and two byte permutes per eight codes instead of a sign extension; the
//                factor 16 is divided out of the scale, which is exact in binary floating point.
//   warp 1       MMA: four tcgen05.mma kind::i8 (128 x 128 x 32) into one of two accumulators, overwriting it
//   warps 6-13   drain: the group's int32 sums leave tensor memory (64 columns per thread), are converted, multiplied
//                by the group's scales and added to the thread's f32 totals; after the last group the totals are
//                multiplied by the row's activation scale and stored.
// The drain (one conversion, one multiplication and one addition per output and group, on the CUDA cores) takes 2.4
// times as long as the MMAs of a group, so this form runs at 0.27 of the rate of the plain int8 GEMM on the
// re-expressed weight (813-884 against 3000-3160 TOPS at the benchmark's shapes).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "h3b_internal.h"
#include "h3b_ptx.cuh"

namespace h3b {

namespace w4g {
constexpr int BM = 128, BN = 128, GROUP = 128, STAGES = 5;
// per stage: activations 16 KiB | expanded weights 16 KiB | packed weights 8 KiB
constexpr int A_BYTES = BM * GROUP, B_BYTES = BN * GROUP, P_BYTES = BN * GROUP / 2, STAGE_BYTES = A_BYTES + B_BYTES + P_BYTES;
// scales of a group's 128 columns: a ring two slots deeper than the stages (a slot is read by the drain after the
// MMAs of its group have completed, i.e. after its stage may already have been handed back to the TMA warp)
constexpr int SC_SLOTS = STAGES + 2, SC_BYTES = BN * 4;
constexpr int THREADS = 14 * 32;
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (size_t)SC_SLOTS * SC_BYTES + 256;
}  // namespace w4g

struct W4gParams {
    CUtensorMap tmap_x;         // int8 [M, K], box {128 bytes, 128 rows}, 128-byte swizzle
    CUtensorMap tmap_w;         // packed codes [N, K/2] bytes (low nibble = even k), box {64 bytes, 128 rows}, no swizzle
    const float *scales_t;      // [K/128, n_pad]: f16 scale / 16, as f32; n_pad = N rounded up to 128, zeros beyond N
    int n_pad;
    const float *act_scales;    // [M]
    void *y;                    // [M, N] f32 or bf16
    int M, N, K, groups, m_tiles, n_tiles, out_bf16;
    int *status;
};

// Exact conversion of an integer of magnitude below 2^22 (a group sum is at most 128 * 127 * 8 * 16 = 2,080,768) with
// one integer and one floating-point addition instead of a conversion instruction: 1.5 * 2^23 + i is representable.
__device__ __forceinline__ float small_int_to_float(uint32_t i) {
    return __fsub_rn(__uint_as_float(0x4B400000u + i), 12582912.0f);
}

__global__ void __launch_bounds__(w4g::THREADS, 1) k_gemm_w4g(const __grid_constant__ W4gParams p) {
    using namespace w4g;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float *sc_ring = reinterpret_cast<float *>(smem + (size_t)STAGES * STAGE_BYTES);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)STAGES * STAGE_BYTES + (size_t)SC_SLOTS * SC_BYTES);
    uint64_t *a_full = bars, *b_full = bars + STAGES, *empty = bars + 2 * STAGES, *acc_full = bars + 3 * STAGES,
             *acc_empty = bars + 3 * STAGES + 2, *sc_full = bars + 3 * STAGES + 4;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * STAGES + 4 + SC_SLOTS);
    volatile int *abort_word = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&a_full[s], 1);
            mbar_init(&b_full[s], 4);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);
        }
        for (int i = 0; i < SC_SLOTS; i++) mbar_init(&sc_full[i], 1);
        *abort_word = 0;
        mbar_fence_init();
        tma_prefetch_desc(&p.tmap_x);
        tma_prefetch_desc(&p.tmap_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 256);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // every role walks the same sequence of (tile, group) pairs; gi counts them
    if (warp == 0) {
        if (lane == 0) {
            uint32_t gi = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_word; tile += gridDim.x) {
                const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
                for (int g = 0; g < p.groups; g++, gi++) {
                    const int s = gi % STAGES;
                    // the stage is free once the MMAs that read its two int8 tiles have completed; the unpack warps
                    // had finished with its packed codes before those MMAs were issued
                    if (!mbar_wait(&empty[s], ((gi / STAGES) & 1) ^ 1, abort_word, p.status, H3B_ST_TIMEOUT_EMPTY)) break;
                    mbar_expect_tx(&a_full[s], A_BYTES + P_BYTES);
                    tma_load_2d(smem + (size_t)s * STAGE_BYTES, &p.tmap_x, &a_full[s], g * GROUP, mt * BM);
                    tma_load_2d(smem + (size_t)s * STAGE_BYTES + A_BYTES + B_BYTES, &p.tmap_w, &a_full[s], g * (GROUP / 2),
                                nt * BN);   // rows past N arrive as zeros
                    // Scale slot gi % SC_SLOTS was last read by the drain of group gi - SC_SLOTS.  That drain released
                    // its accumulator only after its last read; the MMAs of group gi - SC_SLOTS + 2 = gi - STAGES waited
                    // for that release, and this thread has just seen them complete (empty[s]): the slot is free.
                    const int slot = gi % SC_SLOTS;
                    mbar_expect_tx(&sc_full[slot], SC_BYTES);
                    bulk_load(sc_ring + slot * BN, p.scales_t + (size_t)g * p.n_pad + (size_t)nt * BN, SC_BYTES, &sc_full[slot]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        constexpr uint32_t idesc = umma_idesc(2 /*s32*/, 1 /*s8*/, 1 /*s8*/, BM, BN, 0, 0);
        uint32_t gi = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !*abort_word; tile += gridDim.x) {
            for (int g = 0; g < p.groups; g++, gi++) {
                const int s = gi % STAGES, buf = gi & 1;
                const uint32_t ph = (gi / STAGES) & 1;
                if (!mbar_wait(&acc_empty[buf], ((gi >> 1) & 1) ^ 1, abort_word, p.status, H3B_ST_TIMEOUT_TMEM_EMPTY) ||
                    !mbar_wait(&a_full[s], ph, abort_word, p.status, H3B_ST_TIMEOUT_FULL) ||
                    !mbar_wait(&b_full[s], ph, abort_word, p.status, H3B_ST_TIMEOUT_FULL))
                    break;
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int j = 0; j < GROUP / 32; j++)
                        umma_i8_ss(tmem_base + (uint32_t)buf * BN, umma_desc_k_sw128(a_addr + j * 32),
                                   umma_desc_k_sw128(b_addr + j * 32), idesc, (uint32_t)(j != 0));
                    tc_commit(&empty[s]);
                    tc_commit(&acc_full[buf]);
                }
                __syncwarp();
            }
        }
        __syncwarp();
    } else if (warp < 6) {
        // ---- unpack: four lanes per weight row (a 16-byte piece of its 64 packed bytes each), 32 rows per pass
        const int t = threadIdx.x - 64;
        const int piece = t & 3;
        uint32_t gi = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !*abort_word; tile += gridDim.x) {
            for (int g = 0; g < p.groups; g++, gi++) {
                const int s = gi % STAGES;
                if (!mbar_wait(&a_full[s], (gi / STAGES) & 1, abort_word, p.status, H3B_ST_TIMEOUT_FULL)) break;
                uint8_t *b_tile = smem + (size_t)s * STAGE_BYTES + A_BYTES;
                const uint8_t *pk = b_tile + B_BYTES;
#pragma unroll
                for (int pass = 0; pass < 4; pass++) {
                    const int r = pass * 32 + (t >> 2);
                    // 16 packed bytes = 32 codes = two 16-byte chunks (2 piece, 2 piece + 1) of the int8 row
                    const uint4 raw = *reinterpret_cast<const uint4 *>(pk + r * (GROUP / 2) + piece * 16);
                    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
                    uint32_t o[8];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t lo = (w[i] << 4) & 0xF0F0F0F0u, hi = w[i] & 0xF0F0F0F0u;   // even k, odd k: 16 q per byte
                        o[2 * i] = __byte_perm(lo, hi, 0x5140);       // k0 k1 k2 k3 of the word
                        o[2 * i + 1] = __byte_perm(lo, hi, 0x7362);   // k4 .. k7
                    }
                    uint8_t *row = b_tile + (size_t)r * GROUP;
                    *reinterpret_cast<uint4 *>(row + (((2 * piece) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4 *>(row + (((2 * piece + 1) ^ (r & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                }
                fence_proxy_async_smem();   // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&b_full[s]);
            }
        }
    } else {
        // ---- drain: lane quarter q of the accumulator rows, column half h
        const int q = warp & 3, h = (warp - 6) >> 2;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        uint32_t gi = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !*abort_word; tile += gridDim.x) {
            const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
            const int col0 = nt * BN + h * 64;
            float f[64];
#pragma unroll
            for (int c = 0; c < 64; c++) f[c] = 0.0f;
            bool ok = true;
            for (int g = 0; g < p.groups; g++, gi++) {
                const int buf = gi & 1;
                ok = mbar_wait(&acc_full[buf], (gi >> 1) & 1, abort_word, p.status, H3B_ST_TIMEOUT_TMEM_FULL);
                if (!ok) break;
                tc_fence_after();
                const uint32_t t_addr = tmem_base + lane_base + (uint32_t)buf * BN + (uint32_t)h * 64;
                const int slot = gi % SC_SLOTS;
                ok = mbar_wait(&sc_full[slot], (gi / SC_SLOTS) & 1, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
                if (!ok) break;
                const float *sg = sc_ring + slot * BN + h * 64;   // the same address in every lane: broadcast reads
                // two passes of 32 columns: 64 totals and 32 sums live at a time (14 warps leave 128 registers a thread)
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t acc[32];
                    tmem_ld_32x32b_x32(t_addr + half * 32, acc);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        const int cc = half * 32 + c;
                        const float4 s4 = *reinterpret_cast<const float4 *>(sg + cc);
                        f[cc] = __fadd_rn(f[cc], __fmul_rn(s4.x, small_int_to_float(acc[c])));
                        f[cc + 1] = __fadd_rn(f[cc + 1], __fmul_rn(s4.y, small_int_to_float(acc[c + 1])));
                        f[cc + 2] = __fadd_rn(f[cc + 2], __fmul_rn(s4.z, small_int_to_float(acc[c + 2])));
                        f[cc + 3] = __fadd_rn(f[cc + 3], __fmul_rn(s4.w, small_int_to_float(acc[c + 3])));
                    }
                }
                // released only now, after the last read of the scale slot: see the TMA warp
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
            }
            if (!ok) break;
            const int row = mt * BM + q * 32 + lane;
            if (row < p.M) {
                const float a = __ldg(p.act_scales + row);
                if (p.out_bf16) {
                    __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(p.y) + (size_t)row * p.N + col0;
#pragma unroll
                    for (int c = 0; c < 64; c += 8) {
                        if (col0 + c + 7 < p.N) {
                            uint4 v;
                            __nv_bfloat162 *hh = reinterpret_cast<__nv_bfloat162 *>(&v);
#pragma unroll
                            for (int e = 0; e < 4; e++)
                                hh[e] = __floats2bfloat162_rn(__fmul_rn(f[c + 2 * e], a), __fmul_rn(f[c + 2 * e + 1], a));
                            *reinterpret_cast<uint4 *>(dst + c) = v;
                        } else {
                            for (int e = 0; e < 8; e++)
                                if (col0 + c + e < p.N) dst[c + e] = __float2bfloat16_rn(__fmul_rn(f[c + e], a));
                        }
                    }
                } else {
                    float *dst = reinterpret_cast<float *>(p.y) + (size_t)row * p.N + col0;
#pragma unroll
                    for (int c = 0; c < 64; c += 4) {
                        if (col0 + c + 3 < p.N) {
                            *reinterpret_cast<float4 *>(dst + c) = make_float4(__fmul_rn(f[c], a), __fmul_rn(f[c + 1], a),
                                                                              __fmul_rn(f[c + 2], a), __fmul_rn(f[c + 3], a));
                        } else {
                            for (int e = 0; e < 4; e++)
                                if (col0 + c + e < p.N) dst[c + e] = __fmul_rn(f[c + e], a);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 256);
    }
}

}  // namespace h3b

struct h3b_w4g_exact_weight {
    h3_cuda *cuda;
    int device;
    size_t n, k;
    uint8_t *d_packed;
    float *d_scales_t;
};

using namespace h3b;

extern "C" {

int h3b_w4g_exact_weight_create(h3_cuda *cuda, const uint8_t *packed_host, const uint16_t *scales_f16_host, size_t n, size_t k,
                          h3b_w4g_exact_weight **out, char *error, size_t error_size) {
    if (out) *out = NULL;
    if (!cuda || !packed_host || !scales_f16_host || !out || !n || !k)
        return fail(error, error_size, "w4g_weight_create: invalid arguments");
    if (k % 128) return fail(error, error_size, "w4g_weight_create: K=%zu must be a multiple of the group size 128", k);
    if (n % 4) return fail(error, error_size, "w4g_weight_create: N=%zu must be a multiple of 4", n);
    const size_t groups = k / 128, n_pad = (n + 127) / 128 * 128;
    h3b_w4g_exact_weight *w = (h3b_w4g_exact_weight *)calloc(1, sizeof(*w));
    float *st = (float *)calloc(groups * n_pad, sizeof(float));
    if (!w || !st) {
        free(w);
        free(st);
        return fail(error, error_size, "w4g_weight_create: out of host memory");
    }
    // [n, groups] f16 -> [groups, n_pad] f32, divided by the 16 that the unpacked codes carry; zeros past n
    for (size_t r = 0; r < n; r++)
        for (size_t g = 0; g < groups; g++) {
            __half_raw hr;
            hr.x = scales_f16_host[r * groups + g];
            st[g * n_pad + r] = __half2float(__half(hr)) * 0.0625f;
        }
    w->cuda = cuda; w->device = cuda->device; w->n = n; w->k = k;
    cudaError_t e = cudaMalloc((void **)&w->d_packed, n * k / 2);
    if (e == cudaSuccess) e = cudaMalloc((void **)&w->d_scales_t, groups * n_pad * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpy(w->d_packed, packed_host, n * k / 2, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(w->d_scales_t, st, groups * n_pad * sizeof(float), cudaMemcpyHostToDevice);
    free(st);
    if (e != cudaSuccess) {
        if (w->d_packed) cudaFree(w->d_packed);
        if (w->d_scales_t) cudaFree(w->d_scales_t);
        free(w);
        return cuda_fail(e, "w4g_weight_create", error, error_size);
    }
    *out = w;
    return 1;
}

void h3b_w4g_exact_weight_free(h3b_w4g_exact_weight *w) {
    if (!w) return;
    if (w->d_packed) cudaFree(w->d_packed);
    if (w->d_scales_t) cudaFree(w->d_scales_t);
    free(w);
}

int h3b_gemm_w4g_exact_dev(h3_cuda *cuda, const h3b_w4g_exact_weight *weight, const int8_t *d_x_i8, const float *d_act_scales,
                           size_t m, void *d_y, int out_dtype, char *error, size_t error_size) {
    using namespace w4g;
    if (!cuda || !weight || !d_x_i8 || !d_act_scales || !d_y || !m) return fail(error, error_size, "gemm_w4g: invalid arguments");
    if (weight->device != cuda->device) return fail(error, error_size, "gemm_w4g: the weight lives on another device");
    if (out_dtype != H3B_F32 && out_dtype != H3B_BF16) return fail(error, error_size, "gemm_w4g: output must be f32 or bf16");
    if (((uintptr_t)d_x_i8 | (uintptr_t)d_y) & 15) return fail(error, error_size, "gemm_w4g: buffers must be 16-byte aligned");
    if (m > 0x7fffff00u || weight->n > 0x7fffff00u) return fail(error, error_size, "gemm_w4g: shape too large");
    if (out_dtype == H3B_BF16 && weight->n % 8) return fail(error, error_size, "gemm_w4g: bf16 output needs N %% 8 == 0");
    W4gParams p;
    memset(&p, 0, sizeof(p));
    int rc = h3b_encode_tmap_2d(&p.tmap_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d_x_i8, weight->k, m, weight->k, GROUP, BM,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == 0)
        rc = h3b_encode_tmap_2d(&p.tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, weight->d_packed, weight->k / 2, weight->n,
                                weight->k / 2, GROUP / 2, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != 0) return fail(error, error_size, "gemm_w4g: cuTensorMapEncodeTiled failed (%d)", rc);
    p.scales_t = weight->d_scales_t; p.act_scales = d_act_scales; p.y = d_y;
    p.n_pad = (int)((weight->n + 127) / 128 * 128);
    p.M = (int)m; p.N = (int)weight->n; p.K = (int)weight->k; p.groups = (int)(weight->k / 128);
    p.m_tiles = (int)ceil_div(m, (size_t)BM); p.n_tiles = (int)ceil_div(weight->n, (size_t)BN);
    p.out_bf16 = out_dtype == H3B_BF16; p.status = cuda->d_status;
    H3B_CUDA_OK(cudaFuncSetAttribute(k_gemm_w4g, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES),
                "gemm_w4g smem attribute");
    const int tiles = p.m_tiles * p.n_tiles;
    const int grid = tiles < cuda->sm_count ? tiles : cuda->sm_count;
    ProfScope prof(cuda, PROF_GEMM);
    k_gemm_w4g<<<grid, THREADS, SMEM_BYTES, cuda->op_stream>>>(p);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_gemm_w4g launch");
    return 1;
}

}  // extern "C"
