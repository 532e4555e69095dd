// INT8 x INT8 -> INT32 GEMM on the 5th-generation tensor cores (tcgen05, kind::i8)
// with the DiT epilogues fused:  Y = epi( a[m] * s[n] * sum_k X[m,k] W[n,k] ).
//
// Persistent kernel, one CTA per SM, K in 128-byte blocks.  Two tile shapes:
//   CTAS = 2   a pair of CTAs (cluster of two SMs) computes a 256 x 256 tile with cta_group::2 MMAs:
//              each CTA loads its own 128 rows of A and HALF of the B tile (32 KiB per stage instead
//              of 48), which lowers the L2 -> shared-memory traffic per MMA by a third; six stages
//   CTAS = 1   one CTA computes a 128 x 256 tile (four stages); used when M <= 128
//   warp 0     TMA producer: A (activation codes) and B (weight) tiles into the
//              shared-memory ring, 128-byte swizzle
//   warp 1     MMA issuer (of the even CTA of a pair): four K=32 tcgen05.mma per stage into one of
//              two 256-column TMEM accumulators; tcgen05.commit frees the stage in both CTAs
//   warps 2-9  epilogue: tcgen05.ld the finished accumulator (one output row and half of the
//              tile's columns per thread), scale, apply gate+residual / SwiGLU / tanh-GELU,
//              store.  Runs while the MMA warp fills the other accumulator.  The QKV epilogue applies
//              QK-norm and split-half RoPE to whole heads in registers and can scatter the head slices
//              to per-rank (peer) buffers through a shared-memory transpose.
// Accumulators are exact int32, so the integer part is bit-identical to
// h3_w4a8_gemm_i8_dequant_f32 (h3_w4a8_dequant.c:692); the float part follows the
// reference's operation order (a * s) * (float)acc and h3_dit_fused_epi.h:87-141.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <math.h>
#include <stdlib.h>

#include "h3b_internal.h"
#include "h3b_ptx.cuh"
#include "h3b_gemm_plan.h"
#include "h3b_qkv_epi.cuh"

namespace h3b {

namespace gemm {
constexpr int BM = 128;          // rows of X per tile
constexpr int BN = 256;          // rows of W per tile (TMEM columns per accumulator)
constexpr int BK = 128;          // int8 elements (= bytes) of K per stage
constexpr int A_BYTES = BM * BK;             // 16 KiB
constexpr int THREADS = 320;
constexpr int TMEM_COLS = 512;
constexpr int SPLITK_CNT_BYTES = 1024;   // two counters per slot ahead of the slots' sums
constexpr int GROUP_M_MIN = 8;   // rasterisation: at least 8 row bands share the weight tiles in L2
// internal epilogue id: QKV + QK-norm + RoPE whose rows go to (peer) buffers selected by head group; the rows
// are first transposed through shared memory so that every store instruction writes whole 256-byte head
// slices (a thread-per-row store pattern reached 0.18 TB/s over NVLink)
constexpr int EPI_QKV_ROPE_SCATTER = 5;
constexpr int STG_ROW = 256 + 16;                 // staged bf16 head slice + pad against bank conflicts
constexpr int STG_WARP = 32 * STG_ROW;            // per epilogue warp
constexpr int OUT_WARP = 32 * 128;                // TMA-store staging per epilogue warp
constexpr int TAB_GROUP = 4 * 32 * 128;           // cos and sin rows of one 32-row group: four boxes of 32 x 128 bytes
constexpr int BAR_BYTES = 512;                    // barriers, TMEM slot, abort word
template <int CTAS, int EPI = 0> struct Shape {
    static constexpr bool STAGED = EPI == EPI_QKV_ROPE_SCATTER;
    // QKV + RoPE epilogue of a pair: cos / sin rows arrive by TMA (16 KiB per 32-row group) and Q, K, V leave by
    // TMA stores, which takes two stages of the ring
    static constexpr bool QTMA = EPI == H3B_EPI_QKV_ROPE && CTAS == 2;
    static constexpr int STAGES = STAGED ? (CTAS == 2 ? 4 : 3) : QTMA ? 4 : CTAS == 2 ? 6 : 4;
    static constexpr int B_BYTES = BN * BK / CTAS;          // B rows held by one CTA: 32 KiB or 16 KiB
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // per CTA
    static constexpr int TILE_M = BM * CTAS;
    // Every other epilogue leaves through TMA stores: each of the eight epilogue warps owns 32 rows x 128 bytes
    // of shared memory (128-byte swizzle), placed between the operand ring and the barriers.
    static constexpr bool TSTORE = EPI != EPI_QKV_ROPE_SCATTER && EPI != H3B_EPI_QKV_ROPE;
    static constexpr int OUT_BYTES = (TSTORE || QTMA) ? 8 * OUT_WARP : 0;
    static constexpr int TAB_BYTES = QTMA ? 4 * TAB_GROUP : 0;
    static constexpr size_t SMEM_BYTES = 1024 /*alignment slack*/ + (size_t)STAGES * STAGE_BYTES + OUT_BYTES + TAB_BYTES +
                                         BAR_BYTES + (STAGED ? 8 * (size_t)STG_WARP : 0);
};
}  // namespace gemm

struct GemmParams {
    CUtensorMap tmap_a;   // X codes  [M, K] int8, box 128 (k) x 128 (m)
    CUtensorMap tmap_b;   // W        [N, K] int8, box 128 (k) x 128 (n)
    CUtensorMap tmap_y;   // Y        [M, n_out], box 128 bytes x 32 rows, 128-byte swizzle
    CUtensorMap tmap_res; // residual of the gate epilogue, same geometry
    CUtensorMap tmap_yk, tmap_yv;     // QKV + RoPE by TMA: K and V outputs [M, heads * 128] bf16 (Q is tmap_y)
    CUtensorMap tmap_cos, tmap_sin;   // QKV + RoPE by TMA: tables [M, rope_half] f32, box 32 floats x 32 rows
    int M, N, K;          // N = rows of W
    int n_out;            // columns of Y (N, or N/2 for SwiGLU)
    int m_tiles, n_tiles, k_blocks;
    int group_m;   // row bands per rasterisation group
    // Work items: items [0, tail_first) are whole tiles; with split_s > 1 the last tiles_total - tail_first tiles are cut
    // into split_s slices of K each (item = tail_first + slot * split_s + slice), all of them in the last wave.
    int items_total, tail_first, split_s;
    int32_t *sk_acc;        // [slot][slice - 1][256 columns][256 rows] sums of the slices 1..
    unsigned *sk_cnt;       // [slot][2]: slices' warps that have stored their sums; owner warps that have folded them
                            // (zero between launches)
    int swiglu;
    const float *act_scale;   // [M]
    const float *s_channel;   // [N]
    void *y;
    const void *residual;     // gate: [M, n_out] in the output type
    const float *mod;         // gate: [mod_rows, slots, n_out] or NULL
    const uint32_t *row_map;  // gate: [M] or NULL
    int slots, gate_slot;
    const float *lora;        // optional [M, N] f32 delta added to the dequantised value
    int *status;
    // QKV + QK-norm + RoPE epilogue
    void *y_k, *y_v;
    const float *q_norm, *k_norm, *cosT, *sinT;
    int rope_half, heads, round_qkv;
    float eps;
    // optional scatter of the QKV+RoPE outputs by head group (sequence parallelism): head h of row r goes to
    // sc_{q,k,v}[h / sc_hl] (possibly another GPU's memory) at row sc_row0 + r, head h % sc_hl; 0 = off
    int sc_hl, sc_row0;
    void *sc_q[8], *sc_k[8], *sc_v[8];
};

__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int group_m, int &mt, int &nt) {
    const int per_group = group_m * n_tiles;
    const int g = tile / per_group;
    const int first_m = g * group_m;
    const int gm = min(group_m, m_tiles - first_m);
    const int local = tile - g * per_group;
    mt = first_m + local % gm;
    nt = local / gm;
}

typedef h3b_gemm_item GemmItem;
__device__ __forceinline__ GemmItem gemm_item(const GemmParams &p, int item) {
    return h3b_gemm_get_item(p.tail_first, p.split_s, p.k_blocks, item);
}

__device__ __forceinline__ float gelu_tanh_dev(float v) {   // h3_vision_cuda.c:365-371
    float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    if (inner <= -10.0f) return 0.0f;
    if (inner >= 10.0f) return v;
    return 0.5f * v * (1.0f + tanhf(inner));
}

// tanh-GELU with the hardware tanh approximation (relative error about 2^-11), used when the result
// is stored in a 16-bit type whose own rounding step (2^-9 for bf16) is coarser than that error.
__device__ __forceinline__ float gelu_tanh_fast(float v) {
    float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v), t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(inner));
    return 0.5f * v * (1.0f + t);
}

// The same with the cos / sin rows of the warp's 32 rows in shared memory, as TMA left them: per table two
// boxes of 32 rows x 128 bytes (dimensions 0-31 and 32-63) under the 128-byte swizzle; sin follows cos.
template <int RH>
__device__ __forceinline__ void rope_split_half_smem(float (&v)[128], const uint8_t *tab, int lane) {
#pragma unroll
    for (int d4 = 0; d4 < RH / 4; d4++) {
        const uint32_t off = (uint32_t)(d4 >> 3) * 4096u + (uint32_t)lane * 128u + (uint32_t)(((d4 & 7) ^ (lane & 7)) << 4);
        const float4 c4 = *reinterpret_cast<const float4 *>(tab + off);
        const float4 s4 = *reinterpret_cast<const float4 *>(tab + 8192 + off);
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

// The same for a warp that owns a staging buffer of 32 rows x STG_ROW bytes: the tables of the warp's 32 rows
// come in by coalesced loads, 32 dimensions at a time (cos in the first 128 bytes of a row, sin in the next),
// and every thread then reads its own row from shared memory.  Called by the whole warp.
template <int RH, int ROW_BYTES>
__device__ __forceinline__ void rope_split_half_staged(float (&v)[128], const float *cosT, const float *sinT, int row_first,
                                                       int rows, uint8_t *stg, int lane) {
#pragma unroll
    for (int ph = 0; ph < 2; ph++) {
        constexpr int FULL = 32;
        const int nd = (RH - FULL * ph) < FULL ? (RH - FULL * ph) : FULL;   // dimensions of this pass
        const int u = lane & 7;
#pragma unroll 2
        for (int rr = 0; rr < 8; rr++) {
            const int r = rr * 4 + (lane >> 3);
            if (u < nd / 4 && row_first + r < rows) {
                const size_t at = (size_t)(row_first + r) * RH + FULL * ph + u * 4;
                *reinterpret_cast<float4 *>(stg + r * ROW_BYTES + u * 16) = __ldg(reinterpret_cast<const float4 *>(cosT + at));
                *reinterpret_cast<float4 *>(stg + r * ROW_BYTES + 128 + u * 16) = __ldg(reinterpret_cast<const float4 *>(sinT + at));
            }
        }
        __syncwarp();
#pragma unroll
        for (int d4 = 0; d4 < FULL / 4; d4++) {
            if (d4 < nd / 4) {
                const float4 c4 = *reinterpret_cast<const float4 *>(stg + lane * ROW_BYTES + d4 * 16);
                const float4 s4 = *reinterpret_cast<const float4 *>(stg + lane * ROW_BYTES + 128 + d4 * 16);
                const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int d = FULL * ph + d4 * 4 + e;
                    const float lo = v[d], hi = v[d + RH];
                    v[d] = __fsub_rn(__fmul_rn(lo, cc[e]), __fmul_rn(hi, sn[e]));
                    v[d + RH] = __fadd_rn(__fmul_rn(hi, cc[e]), __fmul_rn(lo, sn[e]));
                }
            }
        }
        __syncwarp();
    }
}

template <typename T> struct OutTraits;
template <> struct OutTraits<float> {
    static constexpr int VEC = 4;
    __device__ static void store(float *p, const float *v) { *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]); }
    __device__ static void load(const float *p, float *v) {
        float4 t = *reinterpret_cast<const float4 *>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
};
template <> struct OutTraits<__nv_bfloat16> {
    static constexpr int VEC = 8;
    __device__ static void store(__nv_bfloat16 *p, const float *v) {
        uint4 raw;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = raw;
    }
    __device__ static void load(const __nv_bfloat16 *p, float *v) {
        uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
};
template <> struct OutTraits<__half> {
    static constexpr int VEC = 8;
    __device__ static void store(__half *p, const float *v) {
        uint4 raw;
        __half2 *h = reinterpret_cast<__half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = raw;
    }
    __device__ static void load(const __half *p, float *v) {
        uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 f = __half22float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
};
template <> struct OutTraits<int32_t> {
    static constexpr int VEC = 4;
    __device__ static void store(int32_t *p, const float *v) { (void)p; (void)v; }
    __device__ static void load(const int32_t *p, float *v) { (void)p; (void)v; }
};

template <int EPI, typename OutT, int CTAS>
__global__ void __launch_bounds__(gemm::THREADS, 1) k_gemm_i8(const __grid_constant__ GemmParams p) {
    using namespace gemm;
    constexpr int STAGES = Shape<CTAS, EPI>::STAGES, STAGE_BYTES = Shape<CTAS, EPI>::STAGE_BYTES,
                  B_BYTES = Shape<CTAS, EPI>::B_BYTES, TILE_M = Shape<CTAS, EPI>::TILE_M;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: required by the 128-byte swizzle pattern of TMA and the MMA descriptors
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr bool TSTORE = Shape<CTAS, EPI>::TSTORE;
    uint8_t *out_stage = smem + (size_t)STAGES * STAGE_BYTES;
    constexpr bool QTMA = Shape<CTAS, EPI>::QTMA;
    uint8_t *tab_stage = out_stage + Shape<CTAS, EPI>::OUT_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(tab_stage + Shape<CTAS, EPI>::TAB_BYTES);
    uint64_t *full = bars, *empty = bars + STAGES, *tmem_full = bars + 2 * STAGES, *tmem_empty = bars + 2 * STAGES + 2;
    uint64_t *res_bar = bars + 2 * STAGES + 4;   // one per epilogue warp (residual tiles of the gate epilogue)
    uint64_t *tab_full = bars + 2 * STAGES + 12, *tab_empty = bars + 2 * STAGES + 16;   // per 32-row group
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 20);
    volatile int *abort_word = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // A pair walks the tile list together; cta_rank selects this CTA's rows of A, half of B and rows of Y.
    const int cta_rank = CTAS == 2 ? (int)cluster_ctarank() : 0;
    const int first_tile = CTAS == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int tile_step = CTAS == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 8 * CTAS);   // one arrival per epilogue warp of every CTA of the pair
        }
        for (int w = 0; w < 8; w++) mbar_init(&res_bar[w], 1);
        for (int g = 0; g < 4; g++) {
            mbar_init(&tab_full[g], 1);
            mbar_init(&tab_empty[g], 2);   // the two warps that share the rows
        }
        *abort_word = 0;
        mbar_fence_init();
        tma_prefetch_desc(&p.tmap_a);
        tma_prefetch_desc(&p.tmap_b);
        if (TSTORE || QTMA) tma_prefetch_desc(&p.tmap_y);
    }
    if (warp == 1) {
        if (CTAS == 2) {
            tmem_alloc_pair(tmem_slot, TMEM_COLS);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, TMEM_COLS);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    if (CTAS == 2) cluster_sync_all();   // the peer's barriers must exist before anything signals them
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------- TMA producer
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (int item = first_tile; item < p.items_total; item += tile_step) {
                const GemmItem w = gemm_item(p, item);
                int mt, nt;
                tile_coords(w.tile, p.m_tiles, p.n_tiles, p.group_m, mt, nt);
                const int m0 = mt * TILE_M + cta_rank * BM;
                const int n0 = p.swiglu ? nt * (BN / 2) : nt * BN;
                const int n1 = p.swiglu ? p.N / 2 + n0 : n0 + BN / 2;
                for (int kb = w.kb0; kb < w.kb1; kb++) {
                    if (!mbar_wait(&empty[s], ph ^ 1, abort_word, p.status, H3B_ST_TIMEOUT_EMPTY)) break;
                    uint8_t *a_dst = smem + (size_t)s * STAGE_BYTES;
                    uint8_t *b_dst = a_dst + A_BYTES;
                    if (CTAS == 2) {
                        // Both CTAs' loads are counted on the even CTA's barrier, which expects the bytes of
                        // both.  A stage is refilled only after the MMAs that read it have completed, i.e.
                        // after that barrier has moved on to the phase these loads belong to.
                        const uint32_t bar = mapa_shared(smem_u32(&full[s]), 0);
                        if (cta_rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
                        tma_load_2d_pair(a_dst, &p.tmap_a, bar, kb * BK, m0);
                        tma_load_2d_pair(b_dst, &p.tmap_b, bar, kb * BK, cta_rank == 0 ? n0 : n1);
                    } else {
                        mbar_expect_tx(&full[s], STAGE_BYTES);
                        tma_load_2d(a_dst, &p.tmap_a, &full[s], kb * BK, m0);
                        tma_load_2d(b_dst, &p.tmap_b, &full[s], kb * BK, n0);
                        tma_load_2d(b_dst + B_BYTES / 2, &p.tmap_b, &full[s], kb * BK, n1);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (*abort_word) break;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer
        // The whole warp walks the loop, converged (descriptor arithmetic stays in uniform registers);
        // one elected lane issues each tcgen05 instruction.
        if (cta_rank == 0) {
            constexpr uint32_t idesc = umma_idesc(2 /*s32*/, 1 /*s8*/, 1 /*s8*/, TILE_M, BN, 0, 0);
            int s = 0;
            uint32_t ph = 0;
            int it = 0;
            for (int item = first_tile; item < p.items_total; item += tile_step, it++) {
                const GemmItem w = gemm_item(p, item);
                const int buf = it & 1;
                if (!mbar_wait(&tmem_empty[buf], ((it >> 1) & 1) ^ 1, abort_word, p.status, H3B_ST_TIMEOUT_TMEM_EMPTY))
                    break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
                for (int kb = w.kb0; kb < w.kb1; kb++) {
                    if (!mbar_wait(&full[s], ph, abort_word, p.status, H3B_ST_TIMEOUT_FULL)) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint64_t a_desc = umma_desc_k_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_k_sw128(a_addr + A_BYTES);
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < BK / 32; k++) {
                            if (CTAS == 2)
                                umma_i8_ss_pair(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc,
                                                (uint32_t)(kb != w.kb0 || k != 0));
                            else
                                umma_i8_ss(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)(k * 2), idesc,
                                           (uint32_t)(kb != w.kb0 || k != 0));
                        }
                        // the stage is free (in both CTAs) once these MMAs have read it
                        if (CTAS == 2) tc_commit_pair(&empty[s], 3);
                        else tc_commit(&empty[s]);
                    }
                    __syncwarp();
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (*abort_word) break;
                if (elect_one()) {
                    if (CTAS == 2) tc_commit_pair(&tmem_full[buf], 3);
                    else tc_commit(&tmem_full[buf]);
                }
            }
        }
        __syncwarp();
    } else {
        // ----------------------------------------------------------- epilogue
        // Eight warps: warp w reads TMEM lane quarter w % 4 (rows) and half (w - 2) / 4 of the tile's
        // columns, 32 columns at a time.  Two warps per scheduler hide each other's load latency.
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        OutT *y = reinterpret_cast<OutT *>(p.y);
        (void)y;
        constexpr int VEC = OutTraits<OutT>::VEC;
        constexpr int CHUNKS = (EPI == H3B_EPI_SWIGLU) ? (BN / 2) / 64 : BN / 64;   // per warp
        uint8_t *ostg = out_stage + (size_t)(warp - 2) * OUT_WARP;
        uint64_t *rbar = &res_bar[warp - 2];
        uint32_t res_phase = 0;
        int tab_it = 0;   // tiles of this CTA that used the cos / sin buffer so far
        int it = 0;
        for (int item = first_tile; item < p.items_total; item += tile_step, it++) {
            const GemmItem w = gemm_item(p, item);
            int mt, nt;
            tile_coords(w.tile, p.m_tiles, p.n_tiles, p.group_m, mt, nt);
            const int buf = it & 1;
            const int row0 = mt * TILE_M + cta_rank * BM + q * 32;
            const int row = row0 + lane;
            const bool row_ok = row < p.M;
            const int c0 = (EPI == H3B_EPI_SWIGLU) ? nt * (BN / 2) : nt * BN;   // first output column
            const float a = row_ok ? p.act_scale[row] : 0.0f;
            const float *gate = nullptr;
            if (EPI == H3B_EPI_GATE && p.mod && row_ok) {
                const size_t mrow = p.row_map ? p.row_map[row] : (size_t)row;
                gate = p.mod + (mrow * p.slots + p.gate_slot) * (size_t)p.n_out;
            }
            // QKV + RoPE by TMA: does a head of this tile rotate?  Both warps of a row group see the same answer.
            bool tile_rope = false;
            uint8_t *tab = tab_stage + (size_t)q * TAB_GROUP;
            if constexpr (QTMA) {
                const int g0 = c0 >> 7;
                // (a slice of a split tile that only adds its sums never rotates anything)
                tile_rope = p.rope_half != 0 && w.slice == 0 && (g0 / p.heads < 2 || (c0 + 128 < p.N && (g0 + 1) / p.heads < 2));
                if (tile_rope && half == 0 && lane == 0 &&
                    mbar_wait(&tab_empty[q], (tab_it & 1) ^ 1, abort_word, p.status, H3B_ST_TIMEOUT_EMPTY)) {
                    mbar_expect_tx(&tab_full[q], TAB_GROUP);
                    tma_load_2d(tab, &p.tmap_cos, &tab_full[q], 0, row0);
                    tma_load_2d(tab + 4096, &p.tmap_cos, &tab_full[q], 32, row0);
                    tma_load_2d(tab + 8192, &p.tmap_sin, &tab_full[q], 0, row0);
                    tma_load_2d(tab + 12288, &p.tmap_sin, &tab_full[q], 32, row0);
                }
                __syncwarp();
            }
            bool ok = mbar_wait(&tmem_full[buf], (it >> 1) & 1, abort_word, p.status, H3B_ST_TIMEOUT_TMEM_FULL);
            tc_fence_after();
            const uint32_t t_addr = tmem_base + lane_base + (uint32_t)buf * BN;
            if (w.parts > 1) {
                // A tail tile cut along K.  Slices 1.. store their int32 sums to their own region of the tile's slot in
                // global memory and are done; slice 0 waits for them, adds the regions to its accumulator in tensor
                // memory (integer sums: exact in any order), and then runs the epilogue below as for a whole tile.
                // Each warp touches exactly the columns its epilogue reads, so no other warp's fold is ever needed.
                // Regions are [column][row]: a warp's 32 rows of one column are one 128-byte line.  (Adding into
                // one region with red.global took 17 us per tile whatever the slice count: an SM retires about one
                // 32-bit reduction per clock.)
                constexpr unsigned WARPS = 8 * CTAS;
                constexpr size_t REGION = (size_t)TILE_M * BN;
                int32_t *slot_acc = p.sk_acc + (size_t)w.slot * (p.split_s - 1) * REGION + cta_rank * BM + q * 32 + lane;
                unsigned *cnt = p.sk_cnt + 2 * w.slot;
                if (w.slice != 0) {
                    if (ok) {
                        int32_t *mine = slot_acc + (size_t)(w.slice - 1) * REGION;
#pragma unroll 1
                        for (int j = 0; j < 4; j++) {
                            const int col = (EPI == H3B_EPI_SWIGLU) ? (j >> 1) * (BN / 2) + half * 64 + (j & 1) * 32 : half * 128 + j * 32;
                            uint32_t r[32];
                            tmem_ld_32x32b_x32(t_addr + col, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int v = 0; v < 32; v++) __stcg(mine + (size_t)(col + v) * TILE_M, (int32_t)r[v]);
                        }
                        __threadfence();
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (CTAS == 2) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[buf]), 0));
                        else mbar_arrive(&tmem_empty[buf]);
                        if (ok) atomicAdd(cnt, 1u);
                    }
                    if (*abort_word) break;
                    continue;
                }
                if (ok && lane == 0) {
                    const unsigned want = (unsigned)(w.parts - 1) * WARPS;
                    const long long start = clock64();
                    unsigned seen;
                    while (true) {
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(cnt) : "memory");
                        if (seen >= want || *abort_word) break;
                        if (clock64() - start > H3B_WAIT_CYCLES) {
                            *abort_word = H3B_ST_TIMEOUT_OTHER;
                            if (p.status) atomicCAS(p.status, 0, H3B_ST_TIMEOUT_OTHER);
                            break;
                        }
                        __nanosleep(100);
                    }
                    ok = seen >= want;
                }
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                if (ok) {
#pragma unroll 1
                    for (int j = 0; j < 4; j++) {
                        const int col = (EPI == H3B_EPI_SWIGLU) ? (j >> 1) * (BN / 2) + half * 64 + (j & 1) * 32 : half * 128 + j * 32;
                        uint32_t r[32];
                        tmem_ld_32x32b_x32(t_addr + col, r);
                        tmem_ld_wait();
                        // three regions' loads are in flight together (96 per thread) before the first add needs one
                        const int32_t *theirs = slot_acc + (size_t)col * TILE_M;
                        int sl = 0;
#pragma unroll 1
                        for (; sl + 3 <= w.parts - 1; sl += 3) {
                            int32_t t0[32], t1[32], t2[32];
#pragma unroll
                            for (int v = 0; v < 32; v++) {
                                t0[v] = __ldcg(theirs + (size_t)sl * REGION + (size_t)v * TILE_M);
                                t1[v] = __ldcg(theirs + (size_t)(sl + 1) * REGION + (size_t)v * TILE_M);
                                t2[v] = __ldcg(theirs + (size_t)(sl + 2) * REGION + (size_t)v * TILE_M);
                            }
#pragma unroll
                            for (int v = 0; v < 32; v++) r[v] += (uint32_t)(t0[v] + t1[v] + t2[v]);
                        }
#pragma unroll 1
                        for (; sl < w.parts - 1; sl++) {
#pragma unroll
                            for (int v = 0; v < 32; v++) r[v] += (uint32_t)__ldcg(theirs + (size_t)sl * REGION + (size_t)v * TILE_M);
                        }
                        tmem_st_32x32b_x32(t_addr + col, r);
                    }
                    tmem_st_wait();
                    __syncwarp();
                    // the last of the owner's warps leaves the counters at zero for the next launch
                    if (lane == 0 && atomicAdd(cnt + 1, 1u) == WARPS - 1) {
                        cnt[0] = 0;
                        cnt[1] = 0;
                    }
                }
            }
            if constexpr (EPI == H3B_EPI_QKV_ROPE || EPI == EPI_QKV_ROPE_SCATTER) {
                // This warp's 128 columns are exactly one head of Q, K or V; the thread holds its row of it.
                const int col = c0 + half * 128;
                if (ok && col < p.N && (!QTMA || row0 < p.M)) {
                    const int g = col >> 7, which = g / p.heads, head = g - which * p.heads;
                    uint32_t r[128];
#pragma unroll
                    for (int ch = 0; ch < 4; ch++)
                        tmem_ld_32x32b_x32(t_addr + half * 128 + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[ch * 32]));
                    tmem_ld_wait();
                    float v[128];
#pragma unroll
                    for (int c4 = 0; c4 < 32; c4++) {
                        const float4 s4 = __ldg(reinterpret_cast<const float4 *>(p.s_channel + col) + c4);
                        const float sc[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            float val = __fmul_rn(__fmul_rn(a, sc[e]), (float)(int32_t)r[4 * c4 + e]);
                            if (p.round_qkv) val = __bfloat162float(__float2bfloat16_rn(val));
                            v[4 * c4 + e] = val;
                        }
                    }
                    // by TMA and in the scatter form every lane computes; rows past M are not stored
                    if (row_ok || QTMA || EPI == EPI_QKV_ROPE_SCATTER) {
                        if (which < 2) {
                            // Sum of squares in the order of the stand-alone kernel (k_qkv_rope: sixteen lanes
                            // with eight consecutive values each, then an xor butterfly), so that a chain
                            // that runs QK-norm here and one that runs it there give the same bits.
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
                            const float ss = part[0];
                            const float inv = 1.0f / sqrtf(ss / 128.0f + p.eps);
                            const float *nw = which == 0 ? p.q_norm : p.k_norm;
#pragma unroll
                            for (int c4 = 0; c4 < 32; c4++) {
                                const float4 n4 = __ldg(reinterpret_cast<const float4 *>(nw) + c4);
                                v[4 * c4] = __fmul_rn(__fmul_rn(v[4 * c4], inv), n4.x);
                                v[4 * c4 + 1] = __fmul_rn(__fmul_rn(v[4 * c4 + 1], inv), n4.y);
                                v[4 * c4 + 2] = __fmul_rn(__fmul_rn(v[4 * c4 + 2], inv), n4.z);
                                v[4 * c4 + 3] = __fmul_rn(__fmul_rn(v[4 * c4 + 3], inv), n4.w);
                            }
                            if constexpr (QTMA) {
                                if (p.rope_half) {
                                    if (!mbar_wait(&tab_full[q], tab_it & 1, abort_word, p.status, H3B_ST_TIMEOUT_FULL)) break;
                                    if (p.rope_half == 48) rope_split_half_smem<48>(v, tab, lane);
                                    else rope_split_half_smem<64>(v, tab, lane);
                                }
                            } else if constexpr (EPI == EPI_QKV_ROPE_SCATTER) {
                                uint8_t *tstg = reinterpret_cast<uint8_t *>(bars) + BAR_BYTES + (size_t)(warp - 2) * STG_WARP;
                                if (p.rope_half == 48) rope_split_half_staged<48, STG_ROW>(v, p.cosT, p.sinT, row0, p.M, tstg, lane);
                                else if (p.rope_half == 64) rope_split_half_staged<64, STG_ROW>(v, p.cosT, p.sinT, row0, p.M, tstg, lane);
                            } else {
                                if (p.rope_half == 48)
                                    rope_split_half<48>(v, p.cosT + (size_t)row * 48, p.sinT + (size_t)row * 48);
                                else if (p.rope_half == 64)
                                    rope_split_half<64>(v, p.cosT + (size_t)row * 64, p.sinT + (size_t)row * 64);
                            }
                        }
                        if constexpr (QTMA) {
                            const CUtensorMap *om = which == 0 ? &p.tmap_y : which == 1 ? &p.tmap_yk : &p.tmap_yv;
#pragma unroll
                            for (int gi = 0; gi < 2; gi++) {   // the head in two groups of 64 dimensions
                                if (lane == 0) tma_store_wait_read<0>();
                                __syncwarp();
#pragma unroll
                                for (int u = 0; u < 8; u++)
                                    OutTraits<__nv_bfloat16>::store(
                                        reinterpret_cast<__nv_bfloat16 *>(ostg + lane * 128 + ((u ^ (lane & 7)) << 4)),
                                        &v[gi * 64 + u * 8]);
                                fence_proxy_async_smem();
                                __syncwarp();
                                if (lane == 0) {
                                    tma_store_2d(om, ostg, head * 128 + gi * 64, row0);
                                    tma_store_commit();
                                }
                            }
                        } else if constexpr (EPI == H3B_EPI_QKV_ROPE) {
                            __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(which == 0 ? p.y : which == 1 ? p.y_k : p.y_v) +
                                                 ((size_t)row * p.heads + head) * 128;
#pragma unroll
                            for (int d = 0; d < 128; d += 8) OutTraits<__nv_bfloat16>::store(dst + d, &v[d]);
                        }
                    }
                    if constexpr (EPI == EPI_QKV_ROPE_SCATTER) {
                        // lane = row: park the head slices of the warp's 32 rows in shared memory, then let sixteen
                        // lanes write one 256-byte slice each, two rows per store instruction
                        uint8_t *stg = reinterpret_cast<uint8_t *>(bars) + BAR_BYTES + (size_t)(warp - 2) * STG_WARP;
#pragma unroll
                        for (int d = 0; d < 128; d += 8)
                            OutTraits<__nv_bfloat16>::store(reinterpret_cast<__nv_bfloat16 *>(stg + lane * STG_ROW) + d, &v[d]);
                        __syncwarp();
                        const int peer = head / p.sc_hl;
                        uint8_t *base = reinterpret_cast<uint8_t *>(which == 0 ? p.sc_q[peer] : which == 1 ? p.sc_k[peer] : p.sc_v[peer]);
                        const int row_first = mt * TILE_M + cta_rank * BM + q * 32;   // row of lane 0
                        const size_t row_pitch = (size_t)p.sc_hl * 256;
                        uint8_t *dst0 = base + ((size_t)(p.sc_row0 + row_first) * p.sc_hl + (head - peer * p.sc_hl)) * 256;
                        const int sub = lane >> 4, chunk = lane & 15;
#pragma unroll
                        for (int k2 = 0; k2 < 16; k2++) {
                            const int rr = 2 * k2 + sub;
                            if (row_first + rr < p.M)
                                *reinterpret_cast<uint4 *>(dst0 + (size_t)rr * row_pitch + chunk * 16) =
                                    *reinterpret_cast<const uint4 *>(stg + rr * STG_ROW + chunk * 16);
                        }
                        __syncwarp();
                    }
                }
            } else
            if (ok && row0 < p.M) {
                // 128 bytes of every row form one staged group: two 32-column chunks of a 16-bit type, one of a
                // 32-bit type.  A thread that stored its own row straight to global memory made each store touch
                // 32 lines: 32 passes of the load/store unit per instruction, behind which the mbarrier polls
                // and the TMA and MMA issues of the other warps queued (13,000 cycles per tile of bf16, 29,000
                // with the residual reads of the gate).
                constexpr int PER = sizeof(OutT) == 2 ? 2 : 1;   // chunks per group
                constexpr int UPC = 32 / VEC;                    // 16-byte units per chunk
#pragma unroll 1
                for (int i = 0; i < CHUNKS; i++) {
                    const int ch = half * CHUNKS + i;
                    const int col = c0 + ch * 32;
                    if (col >= p.n_out) break;   // uniform across the warp
                    const int sub = i & (PER - 1);
                    const int gcol = col - sub * 32;
                    if (sub == 0) {
                        if (lane == 0) tma_store_wait_read<0>();   // the previous group has left the buffer
                        __syncwarp();
                        if (EPI == H3B_EPI_GATE && lane == 0) {
                            mbar_expect_tx(rbar, OUT_WARP);
                            tma_load_2d(ostg, &p.tmap_res, rbar, gcol, row0);
                        }
                    }
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(t_addr + ch * 32, r);
                    uint32_t r2[32];
                    if (EPI == H3B_EPI_SWIGLU) tmem_ld_32x32b_x32(t_addr + BN / 2 + ch * 32, r2);
                    const bool full = col + 32 <= p.n_out;
                    // column scales (and gate) of the chunk: the same addresses for every lane, fetched as
                    // vectors while the TMEM load is in flight
                    float sc[32], sc2[32], gt[32];
                    if (full) {
#pragma unroll
                        for (int v = 0; v < 8; v++) {
                            const float4 t4 = __ldg(reinterpret_cast<const float4 *>(p.s_channel + col) + v);
                            sc[4 * v] = t4.x; sc[4 * v + 1] = t4.y; sc[4 * v + 2] = t4.z; sc[4 * v + 3] = t4.w;
                        }
                        if (EPI == H3B_EPI_SWIGLU) {
#pragma unroll
                            for (int v = 0; v < 8; v++) {
                                const float4 t4 = __ldg(reinterpret_cast<const float4 *>(p.s_channel + p.n_out + col) + v);
                                sc2[4 * v] = t4.x; sc2[4 * v + 1] = t4.y; sc2[4 * v + 2] = t4.z; sc2[4 * v + 3] = t4.w;
                            }
                        }
                        if (EPI == H3B_EPI_GATE) {
                            if (gate) {
#pragma unroll
                                for (int v = 0; v < 8; v++) {
                                    const float4 t4 = __ldg(reinterpret_cast<const float4 *>(gate + col) + v);
                                    gt[4 * v] = t4.x; gt[4 * v + 1] = t4.y; gt[4 * v + 2] = t4.z; gt[4 * v + 3] = t4.w;
                                }
                            } else {
#pragma unroll
                                for (int v = 0; v < 32; v++) gt[v] = 1.0f;
                            }
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < 32; v++) {
                            const bool in = col + v < p.n_out;
                            sc[v] = in ? __ldg(p.s_channel + col + v) : 0.0f;
                            if (EPI == H3B_EPI_SWIGLU) sc2[v] = in ? __ldg(p.s_channel + p.n_out + col + v) : 0.0f;
                            if (EPI == H3B_EPI_GATE) gt[v] = (in && gate) ? __ldg(gate + col + v) : 1.0f;
                        }
                    }
                    tmem_ld_wait();
                    if (EPI == H3B_EPI_GATE && sub == 0) {
                        ok = mbar_wait(rbar, res_phase, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
                        res_phase ^= 1;
                        if (!ok) break;
                    }
                    const bool lora_on = p.lora && row_ok;
#pragma unroll
                    for (int v = 0; v < 32; v += VEC) {
                        // rows past M and columns past n_out are clipped by the store
                        uint8_t *cell = ostg + lane * 128 + (((sub * UPC + v / VEC) ^ (lane & 7)) << 4);
                        if constexpr (std::is_same<OutT, int32_t>::value) {
                            *reinterpret_cast<uint4 *>(cell) = make_uint4(r[v], r[v + 1], r[v + 2], r[v + 3]);
                        } else {
                            float out[VEC], resv[VEC];
                            if (EPI == H3B_EPI_GATE) OutTraits<OutT>::load(reinterpret_cast<const OutT *>(cell), resv);
#pragma unroll
                            for (int e = 0; e < VEC; e++) {
                                float val = __fmul_rn(__fmul_rn(a, sc[v + e]), (float)(int32_t)r[v + e]);
                                if (lora_on && col + v + e < p.n_out)
                                    val = __fadd_rn(val, __ldg(p.lora + (size_t)row * p.N + col + v + e));
                                if (EPI == H3B_EPI_GATE) {
                                    val = __fadd_rn(resv[e], __fmul_rn(val, gt[v + e]));
                                } else if (EPI == H3B_EPI_GELU) {
                                    val = sizeof(OutT) == 2 ? gelu_tanh_fast(val) : gelu_tanh_dev(val);
                                } else if (EPI == H3B_EPI_SWIGLU) {
                                    float u = __fmul_rn(__fmul_rn(a, sc2[v + e]), (float)(int32_t)r2[v + e]);
                                    if (lora_on && col + v + e < p.n_out)
                                        u = __fadd_rn(u, __ldg(p.lora + (size_t)row * p.N + p.n_out + col + v + e));
                                    // 16-bit outputs: hardware exponential and reciprocal (2 ulp, far below the output's
                                    // rounding); f32 outputs keep the IEEE forms the CPU path uses
                                    val = sizeof(OutT) == 2 ? __fmul_rn(__fdividef(val, __fadd_rn(1.0f, __expf(-val))), u)
                                                            : __fmul_rn(val / __fadd_rn(1.0f, expf(-val)), u);
                                }
                                out[e] = val;
                            }
                            OutTraits<OutT>::store(reinterpret_cast<OutT *>(cell), out);
                        }
                    }
                    if (sub == PER - 1 || col + 32 >= p.n_out) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&p.tmap_y, ostg, gcol, row0);
                            tma_store_commit();
                        }
                    }
                }
            }
            if constexpr (QTMA) {
                // Give the cos / sin buffer back.  A warp that did not rotate (a V head, rows past M) still waits
                // for the tables first, so that it cannot run a tile ahead and arrive twice in one phase.
                if (tile_rope) {
                    const bool seen = mbar_wait(&tab_full[q], tab_it & 1, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
                    __syncwarp();
                    if (seen && lane == 0) mbar_arrive(&tab_empty[q]);
                    tab_it++;
                }
            }
            // hand the accumulator back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CTAS == 2) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[buf]), 0));
                else mbar_arrive(&tmem_empty[buf]);
            }
            if (*abort_word) break;
        }
        if (TSTORE && lane == 0) tma_store_wait<0>();
    }

    tc_fence_before();
    // A pair leaves together: neither CTA may exit while the other can still signal its barriers,
    // read its shared memory or write its tensor memory.
    if (CTAS == 2) cluster_sync_all();
    else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if (CTAS == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int EPI, typename OutT>
static int gemm_launch_t(h3_cuda *cuda, GemmParams &p, char *error, size_t error_size) {
    using namespace gemm;
    // CTA pairs whenever there is more than one 128-row band (H3B_GEMM_PAIRS=0 keeps single CTAs)
    if constexpr (Shape<1, EPI>::TSTORE) {
        const CUtensorMapDataType dt = std::is_same<OutT, float>::value           ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                       : std::is_same<OutT, int32_t>::value       ? CU_TENSOR_MAP_DATA_TYPE_INT32
                                       : std::is_same<OutT, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        const uint32_t box = 128 / sizeof(OutT);
        int rc = h3b_encode_tmap_2d(&p.tmap_y, dt, sizeof(OutT), p.y, (uint64_t)p.n_out, (uint64_t)p.M,
                                    (uint64_t)p.n_out * sizeof(OutT), box, 32, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc == 0 && EPI == H3B_EPI_GATE)
            rc = h3b_encode_tmap_2d(&p.tmap_res, dt, sizeof(OutT), p.residual, (uint64_t)p.n_out, (uint64_t)p.M,
                                    (uint64_t)p.n_out * sizeof(OutT), box, 32, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != 0) return fail(error, error_size, "gemm_i8: cuTensorMapEncodeTiled(Y) failed (%d)", rc);
    }
    if constexpr (EPI == H3B_EPI_QKV_ROPE) {
        const uint64_t width = (uint64_t)p.heads * 128;
        void *outs[3] = {p.y, p.y_k, p.y_v};
        CUtensorMap *maps[3] = {&p.tmap_y, &p.tmap_yk, &p.tmap_yv};
        int rc = 0;
        for (int i = 0; i < 3 && rc == 0; i++)
            rc = h3b_encode_tmap_2d(maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, outs[i], width, (uint64_t)p.M, width * 2, 64, 32,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc == 0 && p.rope_half) {
            rc = h3b_encode_tmap_2d(&p.tmap_cos, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.cosT, (uint64_t)p.rope_half, (uint64_t)p.M,
                                    (uint64_t)p.rope_half * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc == 0)
                rc = h3b_encode_tmap_2d(&p.tmap_sin, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.sinT, (uint64_t)p.rope_half,
                                        (uint64_t)p.M, (uint64_t)p.rope_half * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
        }
        if (rc != 0) return fail(error, error_size, "gemm_i8: cuTensorMapEncodeTiled(QKV outputs, RoPE tables) failed (%d)", rc);
    }
    static const bool pairs_allowed = h3_plugin_enabled("H3B_GEMM_PAIRS") != 0;
    if (pairs_allowed && p.M > BM) {
        auto kern = k_gemm_i8<EPI, OutT, 2>;
        constexpr size_t smem = Shape<2, EPI>::SMEM_BYTES;
        // co-resident pairs on this device (an SM without a free neighbour cannot host half a pair);
        // asked once per kernel and device
        static int max_pairs[64];
        const int dev = cuda->device & 63;
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = cuda->op_stream;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        if (max_pairs[dev] == 0) {
            H3B_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "gemm smem attribute");
            cfg.gridDim = dim3((unsigned)(cuda->sm_count & ~1));
            int n = 0;
            H3B_CUDA_OK(cudaOccupancyMaxActiveClusters(&n, kern, &cfg), "gemm cluster occupancy");
            if (n < 1) return fail(error, error_size, "gemm_i8: no CTA pair fits on this device");
            max_pairs[dev] = n;
        }
        p.m_tiles = (p.M + Shape<2, EPI>::TILE_M - 1) / Shape<2, EPI>::TILE_M;
        const int tiles = p.m_tiles * p.n_tiles;
        const int n_pairs = tiles < max_pairs[dev] ? tiles : max_pairs[dev];
        cfg.gridDim = dim3((unsigned)(2 * n_pairs));
        // A last wave that fills at most half of the pairs can be cut along K: its `rem` tiles become rem * S slices, one
        // per pair; slices 1.. store their int32 sums to global memory, slice 0 adds them to its accumulator and runs the
        // epilogue.  Storing, signalling, the fold and its extra pass through tensor memory cost about 10 us plus 2 us
        // per region read; a k-block of MMAs saved is 0.39 us.  S minimises T/S + 2 (S - 1) for a tile of T us, and the
        // tail is cut only where the estimate gains 8 us or more.  In the sharded step that is the K = 12288 projection
        // (6,280 rows x 3,072 columns: 300 tiles on 74 pairs are 4 waves and 4 tiles): 172.2 -> 165.2 us with three or
        // four slices, 320.3 -> 313.4 at 12,560 rows, 616.5 -> 607.7 at 25,110; forced on the K = 3072 projections it
        // loses 6 us.  H3B_GEMM_SPLITK=0 keeps whole tiles, a value of 2 or more forces that many slices.  The slot
        // memory belongs to the handle: one GEMM at a time per handle, as the op stream orders them.
        // (never inside a stream capture: a graph would keep the slots' address beyond h3_cuda_release_heavy_workspace)
        h3b_gemm_plan plan = h3b_gemm_make_plan(tiles, n_pairs, p.k_blocks,
                                                cuda->graph_capture ? 0 : atoi(h3_plugin_value("H3B_GEMM_SPLITK")));
        if (plan.split_s > 1) {
            const size_t need = SPLITK_CNT_BYTES + (size_t)max_pairs[dev] * Shape<2, EPI>::TILE_M * BN * sizeof(int32_t);
            if (cuda->splitk_bytes < need && !cuda->graph_capture) {
                if (cuda->splitk) cudaFree(cuda->splitk);
                cuda->splitk = nullptr; cuda->splitk_bytes = 0;
                H3B_CUDA_OK(cudaMalloc(&cuda->splitk, need), "cudaMalloc(split-K slots)");
                cuda->splitk_bytes = need;
                H3B_CUDA_OK(cudaMemsetAsync(cuda->splitk, 0, need, cuda->op_stream), "cudaMemsetAsync(split-K slots)");
            }
            if (cuda->splitk_bytes < need) plan = h3b_gemm_make_plan(tiles, n_pairs, p.k_blocks, 0);   // no slots: whole tiles
        }
        p.items_total = plan.items_total; p.tail_first = plan.tail_first; p.split_s = plan.split_s;
        if (plan.split_s > 1) {
            p.sk_cnt = reinterpret_cast<unsigned *>(cuda->splitk);
            p.sk_acc = reinterpret_cast<int32_t *>(reinterpret_cast<uint8_t *>(cuda->splitk) + SPLITK_CNT_BYTES);
        }
        ProfScope prof(cuda, PROF_GEMM);
        H3B_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p), "k_gemm_i8 pair launch");
        cuda->launches++;
        return 1;
    }
    auto kern = k_gemm_i8<EPI, OutT, 1>;
    H3B_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Shape<1, EPI>::SMEM_BYTES),
                "gemm smem attribute");
    int tiles = p.m_tiles * p.n_tiles;
    int grid = tiles < cuda->sm_count ? tiles : cuda->sm_count;
    p.items_total = tiles; p.tail_first = tiles; p.split_s = 1;
    ProfScope prof(cuda, PROF_GEMM);
    kern<<<grid, THREADS, Shape<1, EPI>::SMEM_BYTES, cuda->op_stream>>>(p);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_gemm_i8 launch");
    return 1;
}

template <int EPI>
static int gemm_launch_e(h3_cuda *cuda, GemmParams &p, int out_dtype, char *error, size_t error_size) {
    switch (out_dtype) {
    case H3B_F32: return gemm_launch_t<EPI, float>(cuda, p, error, error_size);
    case H3B_BF16: return gemm_launch_t<EPI, __nv_bfloat16>(cuda, p, error, error_size);
    case H3B_F16: return gemm_launch_t<EPI, __half>(cuda, p, error, error_size);
    }
    return fail(error, error_size, "gemm: unsupported output dtype %d", out_dtype);
}

int launch_gemm_i8(h3_cuda *cuda, const h3_cuda_w4a8_weight *w, const int8_t *x, const float *a, size_t m, void *y,
                   const h3b_gemm_epi *epi, char *error, size_t error_size) {
    using namespace gemm;
    const h3b_ulysses_direct *sc = (epi && epi->kind == H3B_EPI_QKV_ROPE) ? epi->scatter : nullptr;
    if (!cuda || !w || !x || !a || (!y && !sc) || !epi || m == 0) return fail(error, error_size, "gemm_i8: invalid arguments");
    if (!w->tmap_ok) return fail(error, error_size, "gemm_i8: weight has no tensor map (K %% 16 != 0?)");
    if (w->device != cuda->device) return fail(error, error_size, "gemm_i8: weight lives on device %d, handle on %d", w->device, cuda->device);
    const size_t N = w->n, K = w->k;
    if (K % 16 || (reinterpret_cast<uintptr_t>(x) & 15))
        return fail(error, error_size, "gemm_i8: K must be a multiple of 16 and X 16-byte aligned (K=%zu)", K);
    if (m > 0x7fffff00u || N > 0x7fffff00u) return fail(error, error_size, "gemm_i8: shape too large");
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.swiglu = epi->kind == H3B_EPI_SWIGLU;
    if (p.swiglu && (N % 2)) return fail(error, error_size, "gemm_i8: SwiGLU needs an even N");
    p.M = (int)m; p.N = (int)N; p.K = (int)K;
    p.n_out = p.swiglu ? (int)(N / 2) : (int)N;
    if (p.n_out % 8) return fail(error, error_size, "gemm_i8: output width %d must be a multiple of 8", p.n_out);
    if (reinterpret_cast<uintptr_t>(y) & 15) return fail(error, error_size, "gemm_i8: Y must be 16-byte aligned");
    p.m_tiles = (int)ceil_div(m, BM);
    // Rasterisation group: as many 256-row bands of X as keep about 32 MB in flight, so that a sweep over the column
    // tiles finds them in L2 (K = 4096: 32 bands, K = 16384: 8).  Measured at 50,220 rows: +5 % on the 16384-wide
    // GELU linear and +3 % on the QKV projection against a fixed 8; larger groups lose again.
    p.group_m = (int)((32u << 20) / (256 * K));
    p.group_m = p.group_m < GROUP_M_MIN ? GROUP_M_MIN : p.group_m > 64 ? 64 : p.group_m;
    p.n_tiles = p.swiglu ? (int)ceil_div((size_t)p.n_out, BN / 2) : (int)ceil_div(N, BN);
    p.k_blocks = (int)ceil_div(K, BK);
    p.act_scale = a; p.s_channel = w->d_s; p.y = y;
    p.residual = epi->d_residual; p.mod = epi->d_modulation; p.row_map = epi->d_row_map;
    p.slots = (int)epi->slots; p.gate_slot = (int)epi->gate_slot;
    p.lora = epi->d_lora;
    if (epi->d_lora) {
        if (epi->kind == H3B_EPI_QKV_ROPE || epi->out_dtype == H3B_I32)
            return fail(error, error_size, "gemm_i8: a LoRA delta goes with the plain, gate, swiglu or gelu epilogue");
        if (reinterpret_cast<uintptr_t>(epi->d_lora) & 3) return fail(error, error_size, "gemm_i8: LoRA delta must be 4-byte aligned");
        if (epi->lora_ready)
            H3B_CUDA_OK(cudaStreamWaitEvent(cuda->op_stream, (cudaEvent_t)epi->lora_ready, 0), "wait for the LoRA delta");
    }
    p.status = cuda->d_status;
    p.tmap_b = w->tmap_b;
    int rc = h3b_encode_tmap_2d(&p.tmap_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x, K, m, K, BK, BM,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return fail(error, error_size, "gemm_i8: cuTensorMapEncodeTiled(A) failed (%d)", rc);
    if (epi->kind == H3B_EPI_GATE) {
        if (!epi->d_residual) return fail(error, error_size, "gemm_i8: gate epilogue needs a residual");
        if (epi->d_modulation && epi->slots == 0) return fail(error, error_size, "gemm_i8: gate epilogue needs slots > 0");
        if (reinterpret_cast<uintptr_t>(epi->d_residual) & 15) return fail(error, error_size, "gemm_i8: residual must be 16-byte aligned");
    }
    if (epi->kind == H3B_EPI_QKV_ROPE) {
        if (epi->out_dtype != H3B_BF16) return fail(error, error_size, "gemm_i8: the QKV+RoPE epilogue writes bf16");
        if (N % 384) return fail(error, error_size, "gemm_i8: QKV+RoPE needs N = 3 * heads * 128 (N=%zu)", N);
        if ((!sc && (!epi->d_key || !epi->d_value)) || !epi->d_q_norm || !epi->d_k_norm)
            return fail(error, error_size, "gemm_i8: QKV+RoPE needs key/value outputs and q/k norm weights");
        if (sc) {
            if (sc->ulysses < 1 || sc->ulysses > 8 || sc->rank < 0 || sc->rank >= sc->ulysses || sc->head_dim != 128 ||
                sc->heads * 384 != N || sc->heads % (size_t)sc->ulysses || m > sc->seq_local)
                return fail(error, error_size, "gemm_i8: scatter geometry does not match (N=%zu, m=%zu)", N, m);
            p.sc_hl = (int)(sc->heads / (size_t)sc->ulysses);
            p.sc_row0 = (int)((size_t)sc->rank * sc->seq_local);
            for (int r = 0; r < sc->ulysses; r++) {
                if (!sc->peer_q[r] || !sc->peer_k[r] || !sc->peer_v[r])
                    return fail(error, error_size, "gemm_i8: scatter buffer of rank %d is not mapped", r);
                p.sc_q[r] = sc->peer_q[r]; p.sc_k[r] = sc->peer_k[r]; p.sc_v[r] = sc->peer_v[r];
            }
        }
        if (epi->rope_half != 0 && epi->rope_half != 48 && epi->rope_half != 64)
            return fail(error, error_size, "gemm_i8: QKV+RoPE supports rope_half 0, 48 or 64 (got %zu)", epi->rope_half);
        if (epi->rope_half && (!epi->d_rope_cos || !epi->d_rope_sin)) return fail(error, error_size, "gemm_i8: rope tables missing");
        if (((uintptr_t)epi->d_key | (uintptr_t)epi->d_value | (uintptr_t)epi->d_q_norm | (uintptr_t)epi->d_k_norm |
             (uintptr_t)epi->d_rope_cos | (uintptr_t)epi->d_rope_sin) & 15)
            return fail(error, error_size, "gemm_i8: QKV+RoPE tensors must be 16-byte aligned");
        p.y_k = epi->d_key; p.y_v = epi->d_value; p.q_norm = epi->d_q_norm; p.k_norm = epi->d_k_norm;
        p.cosT = epi->d_rope_cos; p.sinT = epi->d_rope_sin; p.rope_half = (int)epi->rope_half;
        p.heads = (int)(N / 384); p.eps = epi->epsilon; p.round_qkv = epi->round_qkv;
        if (sc) return gemm_launch_t<gemm::EPI_QKV_ROPE_SCATTER, __nv_bfloat16>(cuda, p, error, error_size);
        return gemm_launch_t<H3B_EPI_QKV_ROPE, __nv_bfloat16>(cuda, p, error, error_size);
    }
    switch (epi->kind) {
    case H3B_EPI_PLAIN:
        if (epi->out_dtype == H3B_I32) return gemm_launch_t<H3B_EPI_PLAIN, int32_t>(cuda, p, error, error_size);
        return gemm_launch_e<H3B_EPI_PLAIN>(cuda, p, epi->out_dtype, error, error_size);
    case H3B_EPI_GATE: return gemm_launch_e<H3B_EPI_GATE>(cuda, p, epi->out_dtype, error, error_size);
    case H3B_EPI_SWIGLU: return gemm_launch_e<H3B_EPI_SWIGLU>(cuda, p, epi->out_dtype, error, error_size);
    case H3B_EPI_GELU: return gemm_launch_e<H3B_EPI_GELU>(cuda, p, epi->out_dtype, error, error_size);
    }
    return fail(error, error_size, "gemm_i8: unknown epilogue kind %d", epi->kind);
}

}  // namespace h3b
