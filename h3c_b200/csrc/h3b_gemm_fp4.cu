// NVFP4 block-scaled GEMM on tcgen05 (kind::mxf4nvf4, one UE4M3 scale per 16 E2M1 values):
//   Y[m,n] = alpha * sum_k  (x4[m,k] * sfx[m,k/16]) * (w4[n,k] * sfw[n,k/16])
// replacing the reference's cuBLASLt call + bf16 round trip + separate dequant epilogue
// (h3_gpu_cuda.cu:5696-5932 h3_cuda_lt_gemm_fp4_bf16, :6351 h3_cuda_fp4_gemm_run, :757-808).
//
// Operands are the reference's tensors unchanged: packed E2M1 [rows, K/2] with the high nibble
// holding the even k (the tensor core assumes the opposite order, but X and W are swapped the
// same way inside every byte, so each product pairs the right elements and every 16-block keeps
// its scale), and UE4M3 scales in the 128x4 blocked layout (h3_gpu_cuda.cu:4534), which is the
// layout tcgen05.cp moves into tensor memory as it is: one 512-byte block = 128 rows x 64 k.
//
// Two kernels.  N >= 256 runs k_gemm_nvfp4_wide (tile 128 x 256, or 256 x 256 over a CTA pair when M > 128; described
// at its definition below); narrower outputs run k_gemm_nvfp4:
// Persistent kernel, tile 128 x 128, 256 k (128 packed bytes) per stage.  A 128x128x64 fp4 MMA executes in
// 64 cycles, while one stage costs its issuing warp a barrier poll (about 100 cycles), eight tcgen05.cp
// scale copies, four MMAs and a commit: a single issuer kept the pipe a third busy.  So the CTA runs TWO
// independent pipelines, each with its own TMA warp, issuing warp, three-stage ring, accumulator and
// scale-factor columns; pipeline p takes the CTA's tiles number p, p+2, p+4, ... and the epilogue drains
// the two accumulators alternately, so a tile's epilogue still overlaps the other pipeline's mainloop.
//   warps 0, 10  TMA of pipeline 0 / 1: X and W tiles (128-byte swizzle) + four scale blocks each (bulk copies)
//   warps 1, 11  issuers: per stage tcgen05.cp the eight scale blocks into TMEM, then four 128x128x64
//                block-scaled MMAs into the pipeline's 128-column accumulator
//   warps 2-9    epilogue (one row, 64 columns per thread): alpha, optional gate + residual, store
#include <cuda_bf16.h>
#include <stdlib.h>

#include "h3b_internal.h"
#include "h3b_ptx.cuh"
#include "h3b_qkv_epi.cuh"

namespace h3b {

namespace fp4 {
constexpr int BM = 128, BN = 128;
constexpr int BK_BYTES = 128;                 // 256 four-bit values of K per stage
constexpr int PIPES = 2;
constexpr int STAGES = 3;                     // per pipeline
constexpr int A_BYTES = BM * BK_BYTES;        // 16 KiB
constexpr int B_BYTES = BN * BK_BYTES;        // 16 KiB
constexpr int SF_BYTES = 4 * 512;             // four 128x64 scale blocks per operand and stage
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + 2 * SF_BYTES;
constexpr int THREADS = 384;
constexpr int TMEM_COLS = 512;
constexpr uint32_t ACC_COL = 0;               // two accumulators of 128 columns, one per pipeline
constexpr uint32_t SF_COL = 256;              // per pipeline 64 columns: two parities of 16 SFA + 16 SFB columns
constexpr size_t SMEM_BYTES = 1024 + (size_t)PIPES * STAGES * STAGE_BYTES + 256;
}  // namespace fp4

struct Fp4Params {
    CUtensorMap tmap_x;   // [M, K/2] bytes, box 128 x 128
    CUtensorMap tmap_w;   // [N, K/2] bytes, box 128 x 128
    CUtensorMap tmap_y;   // wide form: [M, N] outputs, box 128 bytes x 32 rows, 128-byte swizzle
    CUtensorMap tmap_res; // wide form, gate epilogue: the residual, same geometry
    CUtensorMap tmap_sfx; // pair form: scale tiles of X as [tiles, 128] words, box of four tiles
    CUtensorMap tmap_sfw; // pair form: scale tiles of W, same geometry
    CUtensorMap tmap_yk, tmap_yv;   // QKV epilogue: K and V outputs [M, heads * 128] bf16 (Q is tmap_y)
    const float *q_norm, *k_norm, *cosT, *sinT;   // QKV epilogue: QK-norm weights [128], RoPE tables [M, rope_half]
    int rope_half, heads;
    float eps;
    const uint8_t *sf_x, *sf_w;
    int M, N, K;
    int m_tiles, n_tiles, k_blocks;
    int sf_tiles_per_rowblock;   // K / 64
    int group_m;                 // wide form: row bands per rasterisation group
    float alpha;
    int gate;                    // 0 plain, 1 y = residual + alpha * acc * gate
    int out_bf16;                // 0 f32, 1 bf16
    void *y;
    const void *residual;
    const float *mod;
    const uint32_t *row_map;
    int slots, gate_slot;
    int *status;
};


// Shared-memory descriptor of one 512-byte scale block, read as 32 rows of 16 bytes (rows 16 bytes
// apart, 8-row groups 128 bytes apart, no swizzle); tcgen05.cp broadcasts it to the four lane quarters.
__device__ __forceinline__ uint64_t sf_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffff) >> 4);
    d |= (uint64_t)(128 >> 4) << 32;   // stride between 8-row groups
    d |= (uint64_t)1 << 46;
    return d;
}
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_nvfp4_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}

// CTA-pair forms: one instruction, issued by the even CTA, runs in both CTAs of the pair, each on its own shared and
// tensor memory at the same offsets.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_nvfp4_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}

// block-scaled instruction descriptor: E2M1 x E2M1, UE4M3 scales, K = 64 per instruction
__host__ __device__ constexpr uint32_t fp4_idesc(uint32_t m, uint32_t n) {
    return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (0u << 23) | ((m >> 4) << 24);
}

template <bool GATE, bool OUT_BF16>
__global__ void __launch_bounds__(fp4::THREADS, 1) k_gemm_nvfp4(const __grid_constant__ Fp4Params p) {
    using namespace fp4;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int NST = PIPES * STAGES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)NST * STAGE_BYTES);
    uint64_t *full = bars, *empty = bars + NST, *tmem_full = bars + 2 * NST, *tmem_empty = bars + 2 * NST + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * NST + 4);
    volatile int *abort_word = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 8);
        }
        *abort_word = 0;
        mbar_fence_init();
        tma_prefetch_desc(&p.tmap_x);
        tma_prefetch_desc(&p.tmap_w);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 || warp == 10) {
        const int pipe = warp == 0 ? 0 : 1;
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            uint64_t *full = bars + pipe * STAGES, *empty = bars + NST + pipe * STAGES;   // this pipeline's ring
            uint8_t *ring = smem + (size_t)pipe * STAGES * STAGE_BYTES;
            for (int tile = blockIdx.x + pipe * gridDim.x; tile < total_tiles; tile += 2 * gridDim.x) {
                const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(&empty[s], ph ^ 1, abort_word, p.status, H3B_ST_TIMEOUT_EMPTY)) break;
                    uint8_t *a_dst = ring + (size_t)s * STAGE_BYTES;
                    uint8_t *b_dst = a_dst + A_BYTES, *sfa_dst = b_dst + B_BYTES, *sfb_dst = sfa_dst + SF_BYTES;
                    // scale blocks of this stage: k tiles [4 kb, 4 kb + 4) of the row block, clipped at K / 64
                    const int kt0 = kb * 4;
                    const int nkt = min(4, p.sf_tiles_per_rowblock - kt0);
                    const uint32_t sf_bytes = (uint32_t)nkt * 512;
                    mbar_expect_tx(&full[s], A_BYTES + B_BYTES + 2 * sf_bytes);
                    tma_load_2d(a_dst, &p.tmap_x, &full[s], kb * BK_BYTES, mt * BM);
                    tma_load_2d(b_dst, &p.tmap_w, &full[s], kb * BK_BYTES, nt * BN);
                    bulk_load(sfa_dst, p.sf_x + ((size_t)mt * p.sf_tiles_per_rowblock + kt0) * 512, sf_bytes, &full[s]);
                    bulk_load(sfb_dst, p.sf_w + ((size_t)nt * p.sf_tiles_per_rowblock + kt0) * 512, sf_bytes, &full[s]);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (*abort_word) break;
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 11) {
        // whole warp converged (uniform descriptor arithmetic); one elected lane issues
        {
            constexpr uint32_t idesc = fp4_idesc(BM, BN);
            const int pipe = warp == 1 ? 0 : 1, buf = pipe;
            uint64_t *full = bars + pipe * STAGES, *empty = bars + NST + pipe * STAGES;
            uint8_t *ring = smem + (size_t)pipe * STAGES * STAGE_BYTES;
            int s = 0, it = 0, sfbuf = 0;   // it: tiles of this pipeline so far
            uint32_t ph = 0;
            for (int tile = blockIdx.x + pipe * gridDim.x; tile < total_tiles; tile += 2 * gridDim.x, it++) {
                if (!mbar_wait(&tmem_empty[buf], (it & 1) ^ 1, abort_word, p.status, H3B_ST_TIMEOUT_TMEM_EMPTY))
                    break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + ACC_COL + (uint32_t)buf * BN;
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(&full[s], ph, abort_word, p.status, H3B_ST_TIMEOUT_FULL)) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(ring + (size_t)s * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_BYTES, sfa_addr = b_addr + B_BYTES, sfb_addr = sfa_addr + SF_BYTES;
                    const int nkt = min(4, p.sf_tiles_per_rowblock - kb * 4);   // MMAs (64 k each) with data
                    const uint32_t sf_t = tmem_base + SF_COL + (uint32_t)pipe * 64 + (uint32_t)sfbuf * 32;
                    if (elect_one()) {
                        for (int j = 0; j < nkt; j++) {   // copies of MMA j + 1 run while MMA j executes
                            tmem_cp_32x128b_warpx4(sf_t + j * 4, sf_desc(sfa_addr + j * 512));
                            tmem_cp_32x128b_warpx4(sf_t + 16 + j * 4, sf_desc(sfb_addr + j * 512));
                            umma_nvfp4_ss(d_tmem, umma_desc_k_sw128(a_addr + j * 32), umma_desc_k_sw128(b_addr + j * 32),
                                          idesc, sf_t + j * 4, sf_t + 16 + j * 4, (uint32_t)((kb | j) != 0));
                        }
                        tc_commit(&empty[s]);
                    }
                    __syncwarp();
                    sfbuf ^= 1;
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (*abort_word) break;
                if (elect_one()) tc_commit(&tmem_full[buf]);
                __syncwarp();
            }
        }
        __syncwarp();
    } else {
        const int q = warp & 3, half = (warp - 2) >> 2;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        int it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, it++) {
            const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
            const int buf = it & 1;
            const int row = mt * BM + q * 32 + lane;
            const bool row_ok = row < p.M;
            const float *gate = nullptr;
            if (GATE && p.mod && row_ok) {
                const size_t mrow = p.row_map ? p.row_map[row] : (size_t)row;
                gate = p.mod + (mrow * p.slots + p.gate_slot) * (size_t)p.N;
            }
            bool ok = mbar_wait(&tmem_full[buf], (it >> 1) & 1, abort_word, p.status, H3B_ST_TIMEOUT_TMEM_FULL);
            tc_fence_after();
            const uint32_t t_addr = tmem_base + lane_base + ACC_COL + (uint32_t)buf * BN;
            if (ok) {
                // this warp's 64 columns in one TMEM round trip
                const int col0 = nt * BN + half * 64;
                uint32_t r[64];
                tmem_ld_32x32b_x32(t_addr + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                tmem_ld_32x32b_x32(t_addr + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int v = 0; v < 64; v += 8) {
                        const int col = col0 + v;
                        if (col >= p.N) break;
                        float out[8];
#pragma unroll
                        for (int e = 0; e < 8; e++) out[e] = __fmul_rn(p.alpha, __uint_as_float(r[v + e]));
                        if (GATE) {
                            float resv[8], g[8];
                            const size_t idx = (size_t)row * p.N + col;
                            if (OUT_BF16) {
                                const uint4 raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(p.residual) + idx);
                                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                                for (int e = 0; e < 4; e++) {
                                    const float2 f = __bfloat1622float2(h[e]);
                                    resv[2 * e] = f.x; resv[2 * e + 1] = f.y;
                                }
                            } else {
                                const float4 r0 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.residual) + idx);
                                const float4 r1 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.residual) + idx + 4);
                                resv[0] = r0.x; resv[1] = r0.y; resv[2] = r0.z; resv[3] = r0.w;
                                resv[4] = r1.x; resv[5] = r1.y; resv[6] = r1.z; resv[7] = r1.w;
                            }
                            if (gate) {
                                const float4 g0 = __ldg(reinterpret_cast<const float4 *>(gate + col));
                                const float4 g1 = __ldg(reinterpret_cast<const float4 *>(gate + col + 4));
                                g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; e++) g[e] = 1.0f;
                            }
#pragma unroll
                            for (int e = 0; e < 8; e++) out[e] = __fadd_rn(resv[e], __fmul_rn(out[e], g[e]));
                        }
                        if (OUT_BF16) {
                            uint4 raw;
                            __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
                            for (int e = 0; e < 4; e++) h[e] = __floats2bfloat162_rn(out[2 * e], out[2 * e + 1]);
                            *reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(p.y) + (size_t)row * p.N + col) = raw;
                        } else {
                            float *dst = reinterpret_cast<float *>(p.y) + (size_t)row * p.N + col;
                            *reinterpret_cast<float4 *>(dst) = make_float4(out[0], out[1], out[2], out[3]);
                            *reinterpret_cast<float4 *>(dst + 4) = make_float4(out[4], out[5], out[6], out[7]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
            if (*abort_word) break;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// Wide form, tile 128 x 256 with N = 256 instructions.  A 128x128 tile reads 128 B/clk of operands from shared
// memory while TMA writes 128 B/clk into it, twice what shared memory moves: 50 % is its ceiling.  At 128x256 the
// two streams are 96 B/clk each.  Two 256-column accumulators would leave no tensor memory for the scale
// factors, so there is ONE accumulator; the epilogue pulls its 128 columns per warp into registers and hands
// the accumulator back before it converts and stores, which keeps the hole between two tiles short.
// Scale factors of B: the two 128-row blocks of the tile sit in eight consecutive TMEM columns per MMA
// (block 0 in columns 0-3, block 1 in columns 4-7).
// Outputs leave through shared memory and TMA stores, 32 rows x 128 bytes per warp and copy.  A thread that
// stores its own row straight to global memory makes every store instruction touch 32 lines; the load/store
// unit then spends 32 passes per instruction, 4096 cycles per tile, and the mbarrier polls and TMA / MMA
// issues of the other warps queue behind them: measured as a fixed 41 us per 113 MB of bf16 output on top
// of a mainloop that by itself runs at 5900 TFLOP/s.  The gate epilogue fetches the residual the same way.
namespace fp4w {
constexpr int BM = 128, BN = 256, BK_BYTES = 128, STAGES = 3;
constexpr int A_BYTES = BM * BK_BYTES, B_BYTES = BN * BK_BYTES;   // 16 KiB, 32 KiB
constexpr int OUT_STAGE_BYTES = 32 * 128;                         // per epilogue warp: 32 rows of 128 bytes
constexpr int SFA_BYTES = 4 * 512, SFB_BYTES = 8 * 512;            // per stage: 4 MMAs x (1 | 2) blocks
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
constexpr int THREADS = 320;
constexpr uint32_t SF_COL = 256;                                    // per stage 16 SFA + 32 SFB columns
constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + 8 * OUT_STAGE_BYTES + 256;
// CTA pair: tile 256 x 256 over two CTAs.  Each CTA holds its own 128 rows of X and their scales, HALF of the tile's
// weight rows, and the scales of all 256 weight rows (its half of the accumulator spans all 256 columns).
constexpr int PAIR_STAGES = 5;
constexpr int PAIR_STAGE_BYTES = A_BYTES + B_BYTES / 2 + SFA_BYTES + SFB_BYTES;
constexpr size_t PAIR_SMEM_BYTES = 1024 + (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 8 * OUT_STAGE_BYTES + 256;
static_assert(SF_COL + PAIR_STAGES * 48 <= 512, "scale columns of every stage must fit tensor memory");
}  // namespace fp4w

// Tile order: row bands in groups that hold about 32 MB of X (64 bands of 256 rows at K = 4096); inside a group the
// band index runs fastest.  A sweep over the column tiles then finds the group's bands in L2: a tall X (50,220 rows
// x 2 KiB = 103 MB at K = 4096) comes from HBM once, not once per column tile.
__device__ __forceinline__ void wide_tile_coords(int tile, int m_tiles, int n_tiles, int group, int &mt, int &nt) {
    const int per_group = group * n_tiles;
    const int g = tile / per_group;
    const int first_m = g * group;
    const int gm = min(group, m_tiles - first_m);
    const int local = tile - g * per_group;
    mt = first_m + local % gm;
    nt = local / gm;
}

// MODE 3: the QKV projection with QK-norm and split-half RoPE: a warp's 128 columns are one head of Q, K or V, the
// thread holds its row of it; Q, K, V leave as bf16 [M, heads, 128] (h3_dit_w4a8_qkv_rope_f32, h3_dit_w4a8.c:2805-2890,
// on the f32 accumulators; the [M, 3 heads 128] intermediate is never written).
// MODE 0: y = alpha acc; 1: y = residual + alpha acc gate; 2: SwiGLU, y[:, c] = silu(alpha acc[:, c]) * alpha acc[:, N/2 + c]
// in f32 straight from the accumulator (the reference's chain h3_cutlass_nvfp4_fc1_f32_run -> swiglu, h3_dit_nvfp4_chain.cu:
// 201-277, 322-435, as one kernel).  For SwiGLU the tile's first 128 weight rows are gate rows nt*128.., the second
// 128 the matching up rows N/2 + nt*128.., so gate and up of an output column sit 128 accumulator columns apart.
//
// PAIR: two CTAs of a cluster share a 256 x 256 tile (instruction M = 256 over both).  Per MMA clock each CTA then
// reads 16 KiB of X and 16 KiB of W instead of 16 + 32, and a tile hand-over covers twice the work.  Every load of
// both CTAs completes on the even CTA's barrier; that CTA issues the scale copies and MMAs for both.
template <int MODE, bool OUT_BF16, bool PAIR>
__global__ void __launch_bounds__(fp4w::THREADS, 1) k_gemm_nvfp4_wide(const __grid_constant__ Fp4Params p) {
    using namespace fp4w;
    constexpr bool GATE = MODE == 1, SWIGLU = MODE == 2, QKV = MODE == 3;
    static_assert(!QKV || OUT_BF16, "the QKV epilogue writes bf16");
    constexpr int STAGES = PAIR ? fp4w::PAIR_STAGES : fp4w::STAGES;
    constexpr int B_BYTES = PAIR ? fp4w::B_BYTES / 2 : fp4w::B_BYTES;
    constexpr int STAGE_BYTES = PAIR ? fp4w::PAIR_STAGE_BYTES : fp4w::STAGE_BYTES;
    constexpr int TILE_M = PAIR ? 2 * BM : BM;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *out_stage = smem + (size_t)STAGES * STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(out_stage + 8 * OUT_STAGE_BYTES);
    uint64_t *full = bars, *empty = bars + STAGES, *tmem_full = bars + 2 * STAGES, *tmem_empty = bars + 2 * STAGES + 1;
    uint64_t *res_bar = bars + 2 * STAGES + 2;   // one per epilogue warp
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 10);
    volatile int *abort_word = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int n_blocks = (p.N + 127) / 128;   // scale row blocks of W
    const int cta_rank = PAIR ? (int)cluster_ctarank() : 0;
    const int first_tile = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, PAIR ? 16 : 8);   // one arrival per epilogue warp of every CTA of the pair
        for (int w = 0; w < 8; w++) mbar_init(&res_bar[w], 1);
        *abort_word = 0;
        mbar_fence_init();
        tma_prefetch_desc(&p.tmap_x);
        tma_prefetch_desc(&p.tmap_w);
        tma_prefetch_desc(&p.tmap_y);
        if (PAIR) {
            tma_prefetch_desc(&p.tmap_sfx);
            tma_prefetch_desc(&p.tmap_sfw);
        }
        if (QKV) {
            tma_prefetch_desc(&p.tmap_yk);
            tma_prefetch_desc(&p.tmap_yv);
        }
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(tmem_slot, 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 512);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    if (PAIR) cluster_sync_all();   // the peer's barriers must exist before anything signals them
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (int tile = first_tile; tile < total_tiles; tile += tile_step) {
                int mt, nt;
                wide_tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, mt, nt);
                // weight rows of the tile's two halves and their scale row blocks
                const int n0 = SWIGLU ? nt * 128 : nt * BN, n1 = SWIGLU ? p.N / 2 + nt * 128 : nt * BN + 128;
                const int nb0 = n0 / 128, nb1 = min(n1 / 128, n_blocks - 1);   // a missing second block repeats the first
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(&empty[s], ph ^ 1, abort_word, p.status, H3B_ST_TIMEOUT_EMPTY)) break;
                    uint8_t *a_dst = smem + (size_t)s * STAGE_BYTES;
                    uint8_t *b_dst = a_dst + A_BYTES, *sfa_dst = b_dst + B_BYTES, *sfb_dst = sfa_dst + SFA_BYTES;
                    const int kt0 = kb * 4;
                    const int nkt = min(4, p.sf_tiles_per_rowblock - kt0);
                    const uint32_t sf_bytes = (uint32_t)nkt * 512;
                    if (PAIR) {
                        // the scale boxes are always four tiles long: past the last tile of a row block they bring
                        // tiles nobody reads (or zeros past the end of the array)
                        const uint32_t bar = mapa_shared(smem_u32(&full[s]), 0);
                        if (cta_rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
                        tma_load_2d_pair(a_dst, &p.tmap_x, bar, kb * BK_BYTES, mt * TILE_M + cta_rank * BM);
                        tma_load_2d_pair(b_dst, &p.tmap_w, bar, kb * BK_BYTES, cta_rank == 0 ? n0 : n1);
                        tma_load_2d_pair(sfa_dst, &p.tmap_sfx, bar, 0, (mt * 2 + cta_rank) * p.sf_tiles_per_rowblock + kt0);
                        tma_load_2d_pair(sfb_dst, &p.tmap_sfw, bar, 0, nb0 * p.sf_tiles_per_rowblock + kt0);
                        tma_load_2d_pair(sfb_dst + 4 * 512, &p.tmap_sfw, bar, 0, nb1 * p.sf_tiles_per_rowblock + kt0);
                        if (++s == STAGES) { s = 0; ph ^= 1; }
                        continue;
                    }
                    mbar_expect_tx(&full[s], A_BYTES + B_BYTES + 3 * sf_bytes);
                    tma_load_2d(a_dst, &p.tmap_x, &full[s], kb * BK_BYTES, mt * BM);
                    tma_load_2d(b_dst, &p.tmap_w, &full[s], kb * BK_BYTES, n0);
                    tma_load_2d(b_dst + B_BYTES / 2, &p.tmap_w, &full[s], kb * BK_BYTES, n1);
                    bulk_load(sfa_dst, p.sf_x + ((size_t)mt * p.sf_tiles_per_rowblock + kt0) * 512, sf_bytes, &full[s]);
                    bulk_load(sfb_dst, p.sf_w + ((size_t)nb0 * p.sf_tiles_per_rowblock + kt0) * 512, sf_bytes, &full[s]);
                    bulk_load(sfb_dst + 4 * 512, p.sf_w + ((size_t)nb1 * p.sf_tiles_per_rowblock + kt0) * 512, sf_bytes, &full[s]);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (*abort_word) break;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        constexpr uint32_t idesc = fp4_idesc(TILE_M, BN);
        int s = 0, it = 0;
        uint32_t ph = 0;
        for (int tile = cta_rank == 0 ? first_tile : total_tiles; tile < total_tiles; tile += tile_step, it++) {
            if (!mbar_wait(tmem_empty, (it & 1) ^ 1, abort_word, p.status, H3B_ST_TIMEOUT_TMEM_EMPTY)) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base;
            for (int kb = 0; kb < p.k_blocks; kb++) {
                if (!mbar_wait(&full[s], ph, abort_word, p.status, H3B_ST_TIMEOUT_FULL)) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES, sfa_addr = b_addr + B_BYTES, sfb_addr = sfa_addr + SFA_BYTES;
                const int nkt = min(4, p.sf_tiles_per_rowblock - kb * 4);
                const uint32_t sfa_t = tmem_base + SF_COL + (uint32_t)s * 48, sfb_t = sfa_t + 16;
                // The scale copies of MMA j + 1 follow MMA j in the queue and run while it executes.  All twelve
                // copies of a stage ahead of its four MMAs cost 6 % (the pipe waits for the whole run of copies),
                // two stages' copies ahead of eight MMAs 15 %.
                if (elect_one()) {
                    if (PAIR) {
                        for (int j = 0; j < nkt; j++) {
                            tmem_cp_32x128b_warpx4_pair(sfa_t + j * 4, sf_desc(sfa_addr + j * 512));
                            tmem_cp_32x128b_warpx4_pair(sfb_t + j * 8, sf_desc(sfb_addr + j * 512));
                            tmem_cp_32x128b_warpx4_pair(sfb_t + j * 8 + 4, sf_desc(sfb_addr + (4 + j) * 512));
                            umma_nvfp4_ss_pair(d_tmem, umma_desc_k_sw128(a_addr + j * 32), umma_desc_k_sw128(b_addr + j * 32),
                                               idesc, sfa_t + j * 4, sfb_t + j * 8, (uint32_t)((kb | j) != 0));
                        }
                        tc_commit_pair(&empty[s], 3);   // the stage is free in both CTAs once these have read it
                    } else {
                        for (int j = 0; j < nkt; j++) {
                            tmem_cp_32x128b_warpx4(sfa_t + j * 4, sf_desc(sfa_addr + j * 512));
                            tmem_cp_32x128b_warpx4(sfb_t + j * 8, sf_desc(sfb_addr + j * 512));
                            tmem_cp_32x128b_warpx4(sfb_t + j * 8 + 4, sf_desc(sfb_addr + (4 + j) * 512));
                            umma_nvfp4_ss(d_tmem, umma_desc_k_sw128(a_addr + j * 32), umma_desc_k_sw128(b_addr + j * 32), idesc,
                                          sfa_t + j * 4, sfb_t + j * 8, (uint32_t)((kb | j) != 0));
                        }
                        tc_commit(&empty[s]);
                    }
                }
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            if (*abort_word) break;
            if (elect_one()) {
                if (PAIR) tc_commit_pair(tmem_full, 3);
                else tc_commit(tmem_full);
            }
            __syncwarp();
        }
        __syncwarp();
    } else {
        const int q = warp & 3, half = (warp - 2) >> 2;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        constexpr int CH_COLS = OUT_BF16 ? 64 : 32;   // 128 bytes of a row per copy
        constexpr int OUT_COLS = SWIGLU ? 64 : 128;   // output columns per thread
        constexpr int NCH = OUT_COLS / CH_COLS;
        constexpr int UNIT = OUT_BF16 ? 8 : 4;        // values per 16-byte unit
        uint8_t *stg = out_stage + (size_t)(warp - 2) * OUT_STAGE_BYTES;
        uint64_t *rbar = &res_bar[warp - 2];
        uint32_t res_phase = 0;
        int it = 0;
        for (int tile = first_tile; tile < total_tiles; tile += tile_step, it++) {
            int mt, nt;
            wide_tile_coords(tile, p.m_tiles, p.n_tiles, p.group_m, mt, nt);
            const int row0 = mt * TILE_M + cta_rank * BM + q * 32;
            const float *gate = nullptr;
            if (GATE && p.mod) {
                const int row = min(row0 + lane, p.M - 1);   // rows past M are clipped by the store
                const size_t mrow = p.row_map ? p.row_map[row] : (size_t)row;
                gate = p.mod + (mrow * p.slots + p.gate_slot) * (size_t)p.N;
            }
            bool ok = mbar_wait(tmem_full, it & 1, abort_word, p.status, H3B_ST_TIMEOUT_TMEM_FULL);
            tc_fence_after();
            // plain / gate: 128 accumulator columns per thread; SwiGLU: 64 gate columns in r[0..63] and the 64 up
            // columns 128 further on in r[64..127]
            const uint32_t t_addr = tmem_base + lane_base + (uint32_t)half * (SWIGLU ? 64 : 128);
            uint32_t r[128];
            if (ok) {
#pragma unroll
                for (int ch = 0; ch < 4; ch++)
                    tmem_ld_32x32b_x32(t_addr + (SWIGLU ? (ch >> 1) * 128 + (ch & 1) * 32 : ch * 32),
                                       *reinterpret_cast<uint32_t(*)[32]>(&r[ch * 32]));
                tmem_ld_wait();
            }
            // the values are in registers: the accumulator can take the next tile
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR && cta_rank != 0) mbar_arrive_cluster(mapa_shared(smem_u32(tmem_empty), 0));
                else mbar_arrive(tmem_empty);
            }
            const int col0 = SWIGLU ? nt * 128 + half * 64 : nt * BN + half * 128;
            const int n_out = SWIGLU ? p.N / 2 : p.N;
            float(&hv)[128] = reinterpret_cast<float(&)[128]>(r);   // QKV: the finished head, in the accumulator's registers
            int which = 0, head = 0;
            if (QKV && ok && row0 < p.M && col0 < p.N) {
#pragma unroll
                for (int i = 0; i < 128; i++) hv[i] = __fmul_rn(p.alpha, __uint_as_float(r[i]));
                const int g = col0 >> 7;
                which = g / p.heads;
                head = g - which * p.heads;
                if constexpr (QKV) {
                    if (which < 2) {
                        qk_norm_head(hv, which == 0 ? p.q_norm : p.k_norm, p.eps);
                        const size_t trow = (size_t)min(row0 + lane, p.M - 1);   // rows past M are clipped by the store
                        if (p.rope_half == 48) rope_split_half<48>(hv, p.cosT + trow * 48, p.sinT + trow * 48);
                        else if (p.rope_half == 64) rope_split_half<64>(hv, p.cosT + trow * 64, p.sinT + trow * 64);
                    }
                }
            }
            if (ok && row0 < p.M) {
#pragma unroll
                for (int ch = 0; ch < NCH; ch++) {
                    const int col = col0 + ch * CH_COLS;
                    if (col >= n_out) break;
                    if (lane == 0) tma_store_wait_read<0>();   // the previous copy has left the buffer
                    __syncwarp();
                    if (GATE) {
                        if (lane == 0) {
                            mbar_expect_tx(rbar, OUT_STAGE_BYTES);
                            tma_load_2d(stg, &p.tmap_res, rbar, col, row0);
                        }
                        ok = mbar_wait(rbar, res_phase, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
                        res_phase ^= 1;
                        if (!ok) break;
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        uint4 *cell = reinterpret_cast<uint4 *>(stg + lane * 128 + ((u ^ (lane & 7)) << 4));
                        const int v = ch * CH_COLS + u * UNIT;
                        float out[UNIT];
#pragma unroll
                        for (int e = 0; e < UNIT; e++) {
                            out[e] = QKV ? hv[v + e] : __fmul_rn(p.alpha, __uint_as_float(r[v + e]));
                            if (SWIGLU) {
                                const float u_ = __fmul_rn(p.alpha, __uint_as_float(r[64 + v + e]));
                                // hardware exponential and reciprocal (about 2 ulp): the IEEE division and expf expand to
                                // some forty instructions per element, 64 elements per thread
                                out[e] = __fmul_rn(__fdividef(out[e], __fadd_rn(1.0f, __expf(-out[e]))), u_);
                            }
                        }
                        if (GATE) {
                            float resv[UNIT], g[UNIT];
                            const uint4 raw = *cell;
                            if (OUT_BF16) {
                                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                                for (int e = 0; e < UNIT / 2; e++) {
                                    const float2 f = __bfloat1622float2(h[e]);
                                    resv[2 * e] = f.x; resv[2 * e + 1] = f.y;
                                }
                            } else {
                                resv[0] = __uint_as_float(raw.x); resv[1] = __uint_as_float(raw.y);
                                resv[2] = __uint_as_float(raw.z); resv[3] = __uint_as_float(raw.w);
                            }
                            const int gc = min(col + u * UNIT, p.N - UNIT);   // columns past N are clipped by the store
#pragma unroll
                            for (int e = 0; e < UNIT; e += 4) {
                                float4 gv = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
                                if (gate) gv = __ldg(reinterpret_cast<const float4 *>(gate + gc + e));
                                g[e] = gv.x; g[e + 1] = gv.y; g[e + 2] = gv.z; g[e + 3] = gv.w;
                            }
#pragma unroll
                            for (int e = 0; e < UNIT; e++) out[e] = __fadd_rn(resv[e], __fmul_rn(out[e], g[e]));
                        }
                        uint4 pack;
                        if (OUT_BF16) {
                            __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pack);
#pragma unroll
                            for (int e = 0; e < UNIT / 2; e++) h[e] = __floats2bfloat162_rn(out[2 * e], out[2 * e + 1]);
                        } else {
                            pack = make_uint4(__float_as_uint(out[0]), __float_as_uint(out[1]), __float_as_uint(out[2]),
                                              __float_as_uint(out[3]));
                        }
                        *cell = pack;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (QKV)
                            tma_store_2d(which == 0 ? &p.tmap_y : which == 1 ? &p.tmap_yk : &p.tmap_yv, stg,
                                         head * 128 + ch * CH_COLS, row0);
                        else tma_store_2d(&p.tmap_y, stg, col, row0);
                        tma_store_commit();
                    }
                }
            }
            if (*abort_word) break;
        }
        if (lane == 0) tma_store_wait<0>();
    }

    tc_fence_before();
    // A pair leaves together: neither CTA may exit while the other can still signal its barriers, read its shared
    // memory or write its tensor memory.
    if (PAIR) cluster_sync_all();
    else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem_base, 512);
        else tmem_dealloc(tmem_base, 512);
    }
}

int launch_gemm_nvfp4(h3_cuda *cuda, const uint8_t *w_fp4, const uint8_t *sf_w, const uint8_t *x_fp4, const uint8_t *sf_x,
                      size_t m, size_t n, size_t k, float alpha, void *y, int out_dtype, int gate, const void *residual,
                      const float *mod, const uint32_t *row_map, size_t slots, size_t gate_slot, char *error,
                      size_t error_size, const Fp4QkvArgs *qkv) {
    using namespace fp4;
    if (!cuda || !w_fp4 || !sf_w || !x_fp4 || !sf_x || !y || !m || !n || !k)
        return fail(error, error_size, "gemm_fp4: invalid arguments");
    if (k % 64) return fail(error, error_size, "gemm_fp4: K=%zu must be a multiple of 64", k);
    if (n % 8) return fail(error, error_size, "gemm_fp4: N=%zu must be a multiple of 8", n);
    if (out_dtype != H3B_F32 && out_dtype != H3B_BF16) return fail(error, error_size, "gemm_fp4: output must be f32 or bf16");
    if (((uintptr_t)w_fp4 | (uintptr_t)x_fp4 | (uintptr_t)sf_w | (uintptr_t)sf_x | (uintptr_t)y) & 15)
        return fail(error, error_size, "gemm_fp4: buffers must be 16-byte aligned");
    if (gate == 1 && !residual) return fail(error, error_size, "gemm_fp4: gate epilogue needs a residual");
    if (gate == 3) {
        if (!qkv || !qkv->k || !qkv->v || !qkv->q_norm || !qkv->k_norm || !qkv->heads || n != 3 * qkv->heads * 128 ||
            out_dtype != H3B_BF16 || n < 256 || !h3_plugin_enabled("H3B_FP4_WIDE"))
            return fail(error, error_size, "gemm_fp4: the QKV epilogue needs N = 3 x heads x 128, bf16 outputs and the 128 x 256 tile form");
        if (qkv->rope_half != 0 && qkv->rope_half != 48 && qkv->rope_half != 64)
            return fail(error, error_size, "gemm_fp4: the QKV epilogue rotates 48 or 64 dimension pairs (or none)");
        if (qkv->rope_half && (!qkv->cosT || !qkv->sinT)) return fail(error, error_size, "gemm_fp4: RoPE tables missing");
        if (((uintptr_t)qkv->k | (uintptr_t)qkv->v | (uintptr_t)qkv->q_norm | (uintptr_t)qkv->k_norm | (uintptr_t)qkv->cosT |
             (uintptr_t)qkv->sinT) & 15)
            return fail(error, error_size, "gemm_fp4: QKV outputs, norm weights and tables must be 16-byte aligned");
    }
    if (gate == 2 && (n % 256 || !h3_plugin_enabled("H3B_FP4_WIDE")))
        return fail(error, error_size, "gemm_fp4: the fused SwiGLU epilogue needs N %% 256 == 0 and the 128 x 256 tile form");
    if (m > 0x7fffff00u || n > 0x7fffff00u) return fail(error, error_size, "gemm_fp4: shape too large");
    Fp4Params p;
    memset(&p, 0, sizeof(p));
    int rc = h3b_encode_tmap_2d(&p.tmap_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x_fp4, k / 2, m, k / 2, BK_BYTES, BM,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == 0)
        rc = h3b_encode_tmap_2d(&p.tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_fp4, k / 2, n, k / 2, BK_BYTES, BN,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return fail(error, error_size, "gemm_fp4: cuTensorMapEncodeTiled failed (%d)", rc);
    p.sf_x = sf_x; p.sf_w = sf_w; p.M = (int)m; p.N = (int)n; p.K = (int)k;
    p.m_tiles = (int)ceil_div(m, BM); p.n_tiles = (int)ceil_div(n, BN); p.k_blocks = (int)ceil_div(k / 2, BK_BYTES);
    p.sf_tiles_per_rowblock = (int)(k / 64);
    p.alpha = alpha; p.gate = gate; p.out_bf16 = out_dtype == H3B_BF16; p.y = y; p.residual = residual; p.mod = mod;
    p.row_map = row_map; p.slots = (int)slots; p.gate_slot = (int)gate_slot; p.status = cuda->d_status;
    if (gate == 1 && (((uintptr_t)residual | (uintptr_t)mod) & 15)) return fail(error, error_size, "gemm_fp4: residual and modulation must be 16-byte aligned");
    // 128 x 256 tiles whenever N has two column blocks; H3B_FP4_WIDE=0 keeps the 128 x 128 form (A/B timing)
    static const bool wide_on = h3_plugin_enabled("H3B_FP4_WIDE") != 0;
    if (wide_on && n >= 256) {
        int rc2 = h3b_encode_tmap_2d(&p.tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_fp4, k / 2, n, k / 2, BK_BYTES, 128,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc2 != 0) return fail(error, error_size, "gemm_fp4: cuTensorMapEncodeTiled failed (%d)", rc2);
        p.group_m = (int)((32u << 20) / (256 * (k / 2)));
        p.group_m = p.group_m < 8 ? 8 : p.group_m > 74 ? 74 : p.group_m;
        p.n_tiles = (int)ceil_div(n, (size_t)fp4w::BN);   // SwiGLU: N/2 output columns, 128 per tile: the same count
        const bool bf = out_dtype == H3B_BF16;
        const CUtensorMapDataType odt = bf ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
        const size_t osz = bf ? 2 : 4, n_y = gate == 2 ? n / 2 : gate == 3 ? n / 3 : n;
        rc2 = h3b_encode_tmap_2d(&p.tmap_y, odt, osz, y, n_y, m, n_y * osz, (uint32_t)(128 / osz), 32, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc2 == 0 && gate == 3) {
            rc2 = h3b_encode_tmap_2d(&p.tmap_yk, odt, osz, qkv->k, n_y, m, n_y * osz, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc2 == 0)
                rc2 = h3b_encode_tmap_2d(&p.tmap_yv, odt, osz, qkv->v, n_y, m, n_y * osz, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B);
            p.q_norm = qkv->q_norm; p.k_norm = qkv->k_norm; p.cosT = qkv->cosT; p.sinT = qkv->sinT;
            p.rope_half = qkv->rope_half; p.heads = (int)qkv->heads; p.eps = qkv->eps;
        }
        if (rc2 == 0 && gate == 1)
            rc2 = h3b_encode_tmap_2d(&p.tmap_res, odt, osz, residual, n, m, n * osz, (uint32_t)(128 / osz), 32,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc2 != 0) return fail(error, error_size, "gemm_fp4: cuTensorMapEncodeTiled (outputs) failed (%d)", rc2);
        // CTA pairs whenever there is more than one 128-row band (H3B_FP4_PAIRS=0 keeps single CTAs)
        if (m > 128 && h3_plugin_enabled("H3B_FP4_PAIRS")) {
            const uint64_t tiles_x = (uint64_t)ceil_div(m, 128) * (k / 64), tiles_wt = (uint64_t)ceil_div(n, 128) * (k / 64);
            rc2 = h3b_encode_tmap_2d(&p.tmap_sfx, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sf_x, 128, tiles_x, 512, 128, 4,
                                     CU_TENSOR_MAP_SWIZZLE_NONE);
            if (rc2 == 0)
                rc2 = h3b_encode_tmap_2d(&p.tmap_sfw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sf_w, 128, tiles_wt, 512, 128, 4,
                                         CU_TENSOR_MAP_SWIZZLE_NONE);
            if (rc2 != 0) return fail(error, error_size, "gemm_fp4: cuTensorMapEncodeTiled (scales) failed (%d)", rc2);
            auto kp = gate == 3   ? k_gemm_nvfp4_wide<3, true, true>
                      : gate == 2 ? (p.out_bf16 ? k_gemm_nvfp4_wide<2, true, true> : k_gemm_nvfp4_wide<2, false, true>)
                      : gate == 1 ? (p.out_bf16 ? k_gemm_nvfp4_wide<1, true, true> : k_gemm_nvfp4_wide<1, false, true>)
                                  : (p.out_bf16 ? k_gemm_nvfp4_wide<0, true, true> : k_gemm_nvfp4_wide<0, false, true>);
            H3B_CUDA_OK(cudaFuncSetAttribute(kp, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp4w::PAIR_SMEM_BYTES),
                        "gemm_fp4 smem attribute");
            cudaLaunchConfig_t cfg;
            memset(&cfg, 0, sizeof(cfg));
            cudaLaunchAttribute attr;
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
            cfg.blockDim = dim3(fp4w::THREADS);
            cfg.dynamicSmemBytes = fp4w::PAIR_SMEM_BYTES;
            cfg.stream = cuda->op_stream;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            // co-resident pairs on this device, asked once per kernel form and device
            static int max_pairs[8][64];
            const int dev = cuda->device & 63, form = gate * 2 + (p.out_bf16 ? 1 : 0);
            if (max_pairs[form][dev] == 0) {
                cfg.gridDim = dim3((unsigned)(cuda->sm_count & ~1));
                int np = 0;
                H3B_CUDA_OK(cudaOccupancyMaxActiveClusters(&np, kp, &cfg), "gemm_fp4 cluster occupancy");
                if (np < 1) return fail(error, error_size, "gemm_fp4: no CTA pair fits on this device");
                max_pairs[form][dev] = np;
            }
            p.m_tiles = (int)ceil_div(m, (size_t)256);
            const int tiles_p = p.m_tiles * p.n_tiles;
            const int n_pairs = tiles_p < max_pairs[form][dev] ? tiles_p : max_pairs[form][dev];
            cfg.gridDim = dim3((unsigned)(2 * n_pairs));
            ProfScope prof(cuda, PROF_GEMM);
            H3B_CUDA_OK(cudaLaunchKernelEx(&cfg, kp, p), "k_gemm_nvfp4_wide pair launch");
            cuda->launches++;
            return 1;
        }
        auto kw = gate == 3   ? k_gemm_nvfp4_wide<3, true, false>
                  : gate == 2 ? (p.out_bf16 ? k_gemm_nvfp4_wide<2, true, false> : k_gemm_nvfp4_wide<2, false, false>)
                  : gate == 1 ? (p.out_bf16 ? k_gemm_nvfp4_wide<1, true, false> : k_gemm_nvfp4_wide<1, false, false>)
                              : (p.out_bf16 ? k_gemm_nvfp4_wide<0, true, false> : k_gemm_nvfp4_wide<0, false, false>);
        H3B_CUDA_OK(cudaFuncSetAttribute(kw, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fp4w::SMEM_BYTES),
                    "gemm_fp4 smem attribute");
        const int tiles_w = p.m_tiles * p.n_tiles;
        const int grid_w = tiles_w < cuda->sm_count ? tiles_w : cuda->sm_count;
        ProfScope prof(cuda, PROF_GEMM);
        kw<<<grid_w, fp4w::THREADS, fp4w::SMEM_BYTES, cuda->op_stream>>>(p);
        cuda->launches++;
        H3B_CUDA_OK(cudaGetLastError(), "k_gemm_nvfp4_wide launch");
        return 1;
    }
    auto kern = gate ? (p.out_bf16 ? k_gemm_nvfp4<true, true> : k_gemm_nvfp4<true, false>)
                     : (p.out_bf16 ? k_gemm_nvfp4<false, true> : k_gemm_nvfp4<false, false>);
    H3B_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES),
                "gemm_fp4 smem attribute");
    int tiles = p.m_tiles * p.n_tiles;
    int grid = tiles < cuda->sm_count ? tiles : cuda->sm_count;
    ProfScope prof(cuda, PROF_GEMM);
    kern<<<grid, THREADS, SMEM_BYTES, cuda->op_stream>>>(p);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_gemm_nvfp4 launch");
    return 1;
}

// bf16 accumulators [m, 2w] * scale -> SwiGLU -> f32 [m, w] (h3_gpu_cuda.cu:757-808 fp4 swiglu epilogue)
__global__ void k_fp4_swiglu(const __nv_bfloat16 *acc, float scale, size_t rows, unsigned width, float *out) {
    const size_t n = rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width;
        const unsigned c = (unsigned)(i - r * width);
        const float g = __fmul_rn(scale, __bfloat162float(acc[r * 2 * width + c]));
        const float u = __fmul_rn(scale, __bfloat162float(acc[r * 2 * width + width + c]));
        out[i] = __fmul_rn(g / __fadd_rn(1.0f, expf(-g)), u);
    }
}

}  // namespace h3b

struct h3_cuda_nvfp4_weight {
    h3_cuda *cuda;
    int device;
    size_t n, k;
    uint8_t *d_packed, *d_sf;
    float scale2;
};

using namespace h3b;

extern "C" {

size_t h3_cuda_nvfp4_gemm_scratch_bytes(size_t m, size_t n, size_t k) {
    const size_t m_pad = (m + 127) / 128 * 128;
    return m_pad * k / 2 + h3_cuda_nvfp4_sf_bytes(m, k) + m_pad * n * 2;
}

int h3_cuda_nvfp4_weight_create(h3_cuda *cuda, const uint8_t *packed_host, const uint8_t *sf_swizzled_host, float scale2,
                                size_t n, size_t k, h3_cuda_nvfp4_weight **out, double *h2d_ms, char *error,
                                size_t error_size) {
    if (out) *out = NULL;
    if (!cuda || !packed_host || !sf_swizzled_host || !out || !n || !k || (k % 64))
        return fail(error, error_size, "invalid nvfp4_weight_create arguments");
    h3_cuda_nvfp4_weight *w = (h3_cuda_nvfp4_weight *)calloc(1, sizeof(*w));
    if (!w) return fail(error, error_size, "nvfp4_weight_create: out of memory");
    w->cuda = cuda; w->device = cuda->device; w->n = n; w->k = k; w->scale2 = scale2;
    const size_t sfb = h3_cuda_nvfp4_sf_bytes(n, k);
    cudaSetDevice(cuda->device);
    if (cudaMalloc((void **)&w->d_packed, n * k / 2) != cudaSuccess || cudaMalloc((void **)&w->d_sf, sfb) != cudaSuccess) {
        cudaError_t e = cudaGetLastError();
        if (w->d_packed) cudaFree(w->d_packed);
        free(w);
        return cuda_fail(e, "nvfp4_weight_create: device allocation", error, error_size);
    }
    Timer t(cuda, h2d_ms);
    cudaMemcpyAsync(w->d_packed, packed_host, n * k / 2, cudaMemcpyHostToDevice, cuda->op_stream);
    cudaMemcpyAsync(w->d_sf, sf_swizzled_host, sfb, cudaMemcpyHostToDevice, cuda->op_stream);
    t.stop();
    cudaError_t e = cudaStreamSynchronize(cuda->op_stream);
    if (e != cudaSuccess) {
        cudaFree(w->d_packed);
        cudaFree(w->d_sf);
        free(w);
        return cuda_fail(e, "nvfp4_weight_create: upload", error, error_size);   // the caller keeps its buffers
    }
    // On success the two host buffers belong to the library (h3_gpu_cuda.h:437-444): the copies have completed, so
    // they are released here; the reference's loaders malloc them and never free them after a successful call.
    free(const_cast<uint8_t *>(packed_host));
    free(const_cast<uint8_t *>(sf_swizzled_host));
    *out = w;
    return 1;
}

int h3_cuda_nvfp4_weight_ensure_ready(h3_cuda_nvfp4_weight *w, char *error, size_t error_size) {
    if (!w) return fail(error, error_size, "nvfp4_weight_ensure_ready: NULL weight");
    return 1;   // uploads complete inside create
}

void h3_cuda_nvfp4_weight_free(h3_cuda *cuda, h3_cuda_nvfp4_weight *w) {
    (void)cuda;
    if (!w) return;
    cudaSetDevice(w->device);
    if (w->d_packed) cudaFree(w->d_packed);
    if (w->d_sf) cudaFree(w->d_sf);
    free(w);
}

const uint8_t *h3_cuda_nvfp4_weight_packed(const h3_cuda_nvfp4_weight *w) { return w ? w->d_packed : NULL; }
const uint8_t *h3_cuda_nvfp4_weight_sf(const h3_cuda_nvfp4_weight *w) { return w ? w->d_sf : NULL; }
float h3_cuda_nvfp4_weight_scale2(const h3_cuda_nvfp4_weight *w) { return w ? w->scale2 : 0.0f; }
size_t h3_cuda_nvfp4_weight_n(const h3_cuda_nvfp4_weight *w) { return w ? w->n : 0; }
size_t h3_cuda_nvfp4_weight_k(const h3_cuda_nvfp4_weight *w) { return w ? w->k : 0; }

int h3_cuda_gemm_fp4_bs_dev(h3_cuda *cuda, const uint8_t *d_w_fp4, const uint8_t *d_sf_w, const uint8_t *d_x_fp4,
                            const uint8_t *d_sf_x, size_t m, size_t n, size_t k, void *d_y_bf16, double *gemm_ms,
                            char *error, size_t error_size) {
    if (!cuda) return fail(error, error_size, "gemm_fp4_bs: NULL handle");
    Timer t(cuda, gemm_ms);
    int ok = launch_gemm_nvfp4(cuda, d_w_fp4, d_sf_w, d_x_fp4, d_sf_x, m, n, k, 1.0f, d_y_bf16, H3B_BF16, 0, NULL, NULL,
                               NULL, 0, 0, error, error_size);
    t.stop();
    return ok;
}

/* Addition: general form (alpha, f32 or bf16 output, optional gate + residual). */
int h3b_gemm_fp4_dev(h3_cuda *cuda, const uint8_t *d_w_fp4, const uint8_t *d_sf_w, const uint8_t *d_x_fp4,
                     const uint8_t *d_sf_x, size_t m, size_t n, size_t k, float alpha, void *d_y, int out_dtype,
                     char *error, size_t error_size) {
    return launch_gemm_nvfp4(cuda, d_w_fp4, d_sf_w, d_x_fp4, d_sf_x, m, n, k, alpha, d_y, out_dtype, 0, NULL, NULL, NULL, 0,
                             0, error, error_size);
}

int h3b_gemm_fp4_swiglu_dev(h3_cuda *cuda, const uint8_t *d_w_fp4, const uint8_t *d_sf_w, const uint8_t *d_x_fp4,
                            const uint8_t *d_sf_x, size_t m, size_t n, size_t k, float alpha, void *d_y, int out_dtype,
                            char *error, size_t error_size) {
    return launch_gemm_nvfp4(cuda, d_w_fp4, d_sf_w, d_x_fp4, d_sf_x, m, n, k, alpha, d_y, out_dtype, 2, NULL, NULL, NULL, 0,
                             0, error, error_size);
}

int h3b_gemm_fp4_w_preq_dev(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const uint8_t *d_x_fp4,
                            const uint8_t *d_sf_x, size_t m, float act_scale, int epi, const void *d_residual,
                            const float *d_modulation, const uint32_t *d_row_map, size_t slots, size_t gate_slot,
                            void *d_y, int out_dtype, char *error, size_t error_size) {
    if (!cuda || !weight || !d_x_fp4 || !d_sf_x || !d_y || !m || epi < 0 || epi > 2)
        return fail(error, error_size, "gemm_fp4_w_preq: invalid arguments");
    if (epi == 2 && (!d_residual || !d_modulation || !slots)) return fail(error, error_size, "gemm_fp4_w_preq: gate epilogue needs residual and modulation");
    return launch_gemm_nvfp4(cuda, weight->d_packed, weight->d_sf, d_x_fp4, d_sf_x, m, weight->n, weight->k,
                             weight->scale2 * act_scale, d_y, out_dtype, epi == 2 ? 1 : epi == 1 ? 2 : 0,
                             epi == 2 ? d_residual : NULL, epi == 2 ? d_modulation : NULL, epi == 2 ? d_row_map : NULL,
                             epi == 2 ? slots : 0, epi == 2 ? gate_slot : 0, error, error_size);
}

int h3b_gemm_fp4_w_preq_qkv_rope_dev(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const uint8_t *d_x_fp4,
                                     const uint8_t *d_sf_x, size_t m, float act_scale, const float *d_q_norm,
                                     const float *d_k_norm, const float *d_cos, const float *d_sin, size_t rope_half,
                                     size_t heads, float epsilon, void *d_q, void *d_k, void *d_v, char *error,
                                     size_t error_size) {
    if (!cuda || !weight || !d_x_fp4 || !d_sf_x || !d_q || !m) return fail(error, error_size, "gemm_fp4_w_preq_qkv_rope: invalid arguments");
    Fp4QkvArgs a;
    a.k = d_k; a.v = d_v; a.q_norm = d_q_norm; a.k_norm = d_k_norm; a.cosT = d_cos; a.sinT = d_sin;
    a.rope_half = (int)rope_half; a.heads = heads; a.eps = epsilon;
    return launch_gemm_nvfp4(cuda, weight->d_packed, weight->d_sf, d_x_fp4, d_sf_x, m, weight->n, weight->k,
                             weight->scale2 * act_scale, d_q, H3B_BF16, 3, NULL, NULL, NULL, 0, 0, error, error_size, &a);
}

// activation quantisation into the scratch area; returns pointers into it
static int fp4_prepare(h3_cuda *cuda, const h3_cuda_nvfp4_weight *w, const float *d_x, size_t m, uint8_t *scratch,
                       uint8_t **x4, uint8_t **sfx, uint8_t **acc, double *prep_ms, char *error, size_t error_size) {
    if (!cuda || !w || !d_x || !m) return fail(error, error_size, "gemm_fp4_w_act: invalid arguments");
    const size_t k = w->k, m_pad = (m + 127) / 128 * 128;
    if (!scratch) {
        if (!grow(cuda, &cuda->act_rot, &cuda->act_rot_bytes, h3_cuda_nvfp4_gemm_scratch_bytes(m, w->n, k), error, error_size))
            return 0;
        scratch = (uint8_t *)cuda->act_rot;
    }
    *x4 = scratch;
    *sfx = scratch + m_pad * k / 2;
    *acc = *sfx + h3_cuda_nvfp4_sf_bytes(m, k);
    Timer t(cuda, prep_ms);
    int ok = h3_cuda_quantize_act_nvfp4_dev(cuda, d_x, m, k, *x4, *sfx, error, error_size);
    t.stop();
    return ok;
}

int h3_cuda_gemm_fp4_w_act_dev(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const float *d_x, float act_scale,
                               size_t m, float *d_y_f32, uint8_t *scratch, double *prep_ms, double *gemm_ms, char *error,
                               size_t error_size, const char *tag) {
    uint8_t *x4, *sfx, *acc;
    (void)tag;
    if (!d_y_f32) return fail(error, error_size, "gemm_fp4_w_act: NULL output");
    if (!fp4_prepare(cuda, weight, d_x, m, scratch, &x4, &sfx, &acc, prep_ms, error, error_size)) return 0;
    Timer t(cuda, gemm_ms);
    int ok = launch_gemm_nvfp4(cuda, weight->d_packed, weight->d_sf, x4, sfx, m, weight->n, weight->k,
                               weight->scale2 * act_scale, d_y_f32, H3B_F32, 0, NULL, NULL, NULL, 0, 0, error, error_size);
    t.stop();
    return ok;
}

int h3_cuda_gemm_fp4_w_act_dev_gate(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const float *d_x, float act_scale,
                                    size_t m, const float *d_residual, const float *d_modulation,
                                    const uint32_t *d_row_map, size_t slots, size_t gate_slot, const float *d_lora,
                                    float *d_y_f32, uint8_t *scratch, double *prep_ms, double *gemm_ms, char *error,
                                    size_t error_size, const char *tag) {
    uint8_t *x4, *sfx, *acc;
    (void)tag;
    if (d_lora) return fail(error, error_size, "gemm_fp4_w_act_gate: LoRA deltas are not supported by this library");
    if (!d_y_f32 || !d_residual || !d_modulation || !slots) return fail(error, error_size, "gemm_fp4_w_act_gate: invalid arguments");
    if (!fp4_prepare(cuda, weight, d_x, m, scratch, &x4, &sfx, &acc, prep_ms, error, error_size)) return 0;
    Timer t(cuda, gemm_ms);
    int ok = launch_gemm_nvfp4(cuda, weight->d_packed, weight->d_sf, x4, sfx, m, weight->n, weight->k,
                               weight->scale2 * act_scale, d_y_f32, H3B_F32, 1, d_residual, d_modulation, d_row_map, slots,
                               gate_slot, error, error_size);
    t.stop();
    return ok;
}

int h3_cuda_gemm_fp4_w_act_dev_swiglu(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const float *d_x,
                                      float act_scale, size_t m, const float *d_lora, float *d_y_f32, uint8_t *scratch,
                                      double *prep_ms, double *gemm_ms, char *error, size_t error_size, const char *tag) {
    uint8_t *x4, *sfx, *acc;
    (void)tag;
    if (d_lora) return fail(error, error_size, "gemm_fp4_w_act_swiglu: LoRA deltas are not supported by this library");
    if (!d_y_f32 || (weight && (weight->n % 2))) return fail(error, error_size, "gemm_fp4_w_act_swiglu: invalid arguments");
    if (!fp4_prepare(cuda, weight, d_x, m, scratch, &x4, &sfx, &acc, prep_ms, error, error_size)) return 0;
    Timer t(cuda, gemm_ms);
    int ok;
    if (weight->n % 256 == 0 && h3_plugin_enabled("H3B_FP4_WIDE")) {
        // SwiGLU in the GEMM epilogue, on the f32 accumulators
        ok = launch_gemm_nvfp4(cuda, weight->d_packed, weight->d_sf, x4, sfx, m, weight->n, weight->k,
                               weight->scale2 * act_scale, d_y_f32, H3B_F32, 2, NULL, NULL, NULL, 0, 0, error, error_size);
    } else {
        // odd widths: block-scaled GEMM to bf16 accumulators in the scratch area (as the reference does,
        // h3_gpu_cuda.cu:757-808), then the SwiGLU kernel
        ok = launch_gemm_nvfp4(cuda, weight->d_packed, weight->d_sf, x4, sfx, m, weight->n, weight->k, 1.0f, acc, H3B_BF16, 0,
                               NULL, NULL, NULL, 0, 0, error, error_size);
        if (ok) {
            const size_t width = weight->n / 2, total = m * width;
            size_t grid = ceil_div(total, 256);
            if (grid > (size_t)cuda->sm_count * 16) grid = (size_t)cuda->sm_count * 16;
            k_fp4_swiglu<<<(unsigned)grid, 256, 0, cuda->op_stream>>>((const __nv_bfloat16 *)acc, weight->scale2 * act_scale, m,
                                                                     (unsigned)width, d_y_f32);
            cuda->launches++;
            if (cudaGetLastError() != cudaSuccess) ok = fail(error, error_size, "k_fp4_swiglu launch failed");
        }
    }
    t.stop();
    return ok;
}

}  // extern "C"
