// Flash-style attention for head_dim 128 on tcgen05: softmax(Q K^T * scale) V, bf16
// operands, f32 scores / accumulation, non-causal, separate query and key counts
// (self-attention and the rectangular cross-attention).  Same math as the
// reference's h3_dit_w4a8_sdpa_f32 (h3_dit_w4a8.c:3073-3116) evaluated tile by tile
// with a running maximum.
//
// One CTA per (256 queries = two 128-row tiles A and B, head); 320 threads:
//   warp 0      TMA: both Q tiles once, then K and V tiles of 128 keys, two-deep rings
//   warp 1      MMA issuer.  Per key tile and per query tile: S = Q K^T (128x128x128) into the
//               tile's TMEM score buffer, then O += P V (128x128x128) with P read from TMEM.
//               The two query tiles are interleaved so that the tensor core works on one
//               while the other is in its softmax.
//   warps 2-5   softmax of tile A, warps 6-9 softmax of tile B: one query row per thread.
//               The 128 scores of the row are read from TMEM into registers once; maximum,
//               exponentials and row sum are computed there and P (bf16 pairs) is written back
//               to TMEM over the score columns, handed to the MMA warp in two halves of 64 keys.
//               The accumulator is rescaled only when the running maximum grew by more than 2^8;
//               the final division by the row sum undoes the stale scale.  At the end the rows go
//               through the CTA's (then free) tile memory so that each store instruction writes
//               whole 256-byte head slices, to this GPU's output or, under sequence parallelism,
//               to the mapped buffer of the rank that owns the row.
// TMEM (512 columns): S_A 0..127, S_B 128..255 (P overlays the first 64 columns of each),
// O_A 256..383, O_B 384..511.
//
// Measured and rejected forms (B200 under its 1000 W limit, where a long run of this kernel is power-bound at
// about 1.5 GHz, so extra instructions or operand traffic cost more than the pipeline bubbles they remove):
//   - scores of the next key tile issued as two 64-key halves, the half that P does not overlay early: an
//     M = 128, N = 64 product re-reads the whole Q operand from shared memory for half the work, -15 %;
//   - two softmax threads per row (16 softmax warps, row maxima and sums exchanged through shared memory): equal
//     without FMA-pipe exponentials, -10 % with them;
//   - exponent offset taken from the previous key tile so that the row maximum leaves the path score ->
//     probability: -6 %;
//   - packed f16 exponentials (ex2.approx.f16x2) in the f16 form: -10 %.
// The CTA-pair form further down (k_attn_pair: cta_group::2 MMAs, K and V tiles split over two SMs, three K/V stages)
// is kept selectable (H3B_ATTN_EMU = 212 / 213).  It measures the same as this kernel (1273 / 1282 against 1296 / 1299
// TFLOP/s at 6,144 / 24,576 keys, 1183 against 1191 sustained): halving the B-operand reads and the K/V traffic per SM
// changes nothing, so shared-memory bandwidth is not what holds the score products back.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <stdlib.h>

#include <algorithm>
#include <type_traits>

#include "h3b_internal.h"
#include "h3b_ptx.cuh"

namespace h3b {

namespace attn {
constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int SLAB = BQ * 64 * 2;        // 128 rows x 64 bf16: one 128-byte-swizzled slab (16 KiB)
constexpr int TILE = 2 * SLAB;           // 128 x 128 bf16 tile (32 KiB)
constexpr int THREADS = 320;
constexpr int TMEM_COLS = 512;
constexpr uint32_t S_COL = 0, O_COL = 256;   // + 128 * tile
// shared memory: Q_A Q_B | K0 K1 | V0 V1 | barriers
constexpr size_t SMEM_BYTES = 1024 + 6 * (size_t)TILE + 256;
}  // namespace attn

struct AttnParams {
    CUtensorMap tmap_q, tmap_k, tmap_v;   // 3-D {d, head, row}, box {64, 1, 128}
    void *out;                            // 16-bit elements of the kernel's type
    size_t o_stride, o_head_stride;       // elements between output rows / between heads of a row
    int lq, lk, heads;
    float scale_log2;                     // scale * log2(e)
    int *status;
    // optional scatter of the output rows by owner (sequence parallelism): row r goes to
    // sc_out[r / sc_rows] (possibly another GPU's memory) at row r % sc_rows, head sc_head0 + head of
    // sc_heads; sc_rows == 0 = off
    int sc_rows, sc_heads, sc_head0;
    void *sc_out[8];
};

// The two 16-bit operand types: bf16 (the benchmark's residual-stream type) and f16 (what the reference's
// own f16 attention entry points stage in: three more mantissa bits in Q, K, V and in the probabilities).
template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
    static constexpr uint32_t FMT = 1;   // tcgen05 kind::f16 operand format code
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
};
template <> struct Elem<__half> {
    static constexpr uint32_t FMT = 0;
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x for two values on the FMA pipe instead of the special-function unit (which is the unit the softmax
// saturates: 16 results per clock and SM against 128 FMA lanes).  x is clamped to >= -127, split into
// floor and fraction by adding 1.5 * 2^23 with round-down (the floor lands in the low mantissa bits), the
// fraction goes through a degree-3 minimax polynomial (relative error 8.6e-5, far below the rounding of the
// probabilities to 16 bits) and the floor is added to the exponent field.  Packed two-wide f32 instructions.
__device__ __forceinline__ void ex2_emu2(float &p0, float &p1, float x0, float x1) {
    x0 = fmaxf(x0, -127.0f);
    x1 = fmaxf(x1, -127.0f);
    uint32_t r0, r1, q0, q1;
    asm("{\n\t.reg .b64 x, m, r, b, f, p, c;\n\t"
        "mov.b64 x, {%4, %5};\n\t"
        "mov.b64 m, {%6, %6};\n\t"
        "add.rm.ftz.f32x2 r, x, m;\n\t"
        "sub.rn.ftz.f32x2 b, r, m;\n\t"
        "sub.rn.ftz.f32x2 f, x, b;\n\t"
        "mov.b64 p, {%7, %7};\n\t"
        "mov.b64 c, {%8, %8};\n\t"
        "fma.rn.ftz.f32x2 p, p, f, c;\n\t"
        "mov.b64 c, {%9, %9};\n\t"
        "fma.rn.ftz.f32x2 p, p, f, c;\n\t"
        "mov.b64 c, {%10, %10};\n\t"
        "fma.rn.ftz.f32x2 p, p, f, c;\n\t"
        "mov.b64 {%0, %1}, r;\n\t"
        "mov.b64 {%2, %3}, p;\n\t}"
        : "=r"(r0), "=r"(r1), "=r"(q0), "=r"(q1)
        : "f"(x0), "f"(x1), "f"(12582912.0f), "f"(0.07706703990697861f), "f"(0.22764499485492706f),
          "f"(0.6951167583465576f), "f"(1.0f));
    p0 = __uint_as_float(q0 + (r0 << 23));
    p1 = __uint_as_float(q1 + (r1 << 23));
}

// max of three (one instruction on sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two-wide f32 FMA / add: one issue slot for two independent IEEE operations
__device__ __forceinline__ void fma2(float &d0, float &d1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float &d0, float &d1, float a0, float a1) {
    asm("{\n\t.reg .b64 ra, rd;\n\t"
        "mov.b64 rd, {%0, %1};\n\tmov.b64 ra, {%2, %3};\n\t"
        "add.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1)
        : "f"(a0), "f"(a1));
}

// The softmax role of one warp (see the head of the file): warps 2-5 serve the CTA's first query tile, 6-9 its
// second.  row0 = first query row of the CTA's first tile, tile_stride = rows between its two tiles.  PAIR: the CTA is
// one of a pair whose MMAs the CTA of cluster rank 0 issues, so "P is ready" is signalled on THAT CTA's barriers.
template <typename T, uint32_t EMU, bool PAIR>
__device__ __forceinline__ void softmax_role(const AttnParams &p, uint8_t *smem, uint32_t tmem_base, uint64_t *s_full,
                                             uint64_t *p_full, uint64_t *o_done, volatile int *abort_word, int warp,
                                             int lane, int n_kv, int n_tiles, int row0, int tile_stride, int head,
                                             uint32_t rank) {
    using namespace attn;
    // ------------------------------------------------------------ softmax
    const int t = (warp - 2) >> 2;                     // query tile of this warp group (warps 2-5: A, 6-9: B)
    const int q = warp & 3;                            // TMEM lane quarter of this warp
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base + S_COL + 128u * t;
    const uint32_t o_addr = tmem_base + lane_base + O_COL + 128u * t;
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = t < n_tiles;
    for (int j = 0; j < n_kv && ok; j++) {
        const int valid = min(BKV, p.lk - j * BKV);    // keys of this tile that exist
        ok = mbar_wait(&s_full[t], j & 1, abort_word, p.status, H3B_ST_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        // all 128 scores of the row in registers (one TMEM round trip)
        uint32_t sv[BKV];
#pragma unroll
        for (int ch = 0; ch < BKV / 32; ch++)
            tmem_ld_32x32b_x32(s_addr + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[ch * 32]));
        tmem_ld_wait();
        if (valid != BKV) {
#pragma unroll
            for (int i = 0; i < BKV; i++)
                if (i >= valid) sv[i] = 0xff800000u;   // -inf: exp2 gives 0
        }
        // eight independent chains of three-input maxima (eight dependent steps instead of sixteen)
        float mxc[8];
#pragma unroll
        for (int c = 0; c < 8; c++) mxc[c] = -INFINITY;
#pragma unroll
        for (int i = 0; i < BKV; i += 16)
#pragma unroll
            for (int c = 0; c < 8; c++)
                mxc[c] = max3(mxc[c], __uint_as_float(sv[i + 2 * c]), __uint_as_float(sv[i + 2 * c + 1]));
        const float mx = fmaxf(max3(mxc[0], mxc[1], mxc[2]), fmaxf(max3(mxc[3], mxc[4], mxc[5]), fmaxf(mxc[6], mxc[7])));
        const float m_new = fmaxf(m_run, mx * p.scale_log2);
        const bool grow_me = (m_new - m_run) > 8.0f;   // also true on the first tile (m_run = -inf)
        if (__any_sync(0xffffffffu, grow_me)) {
            float alpha = 1.0f;
            if (grow_me) {
                alpha = ex2_approx(m_run - m_new);     // 0 on the first tile
                m_run = m_new;
                l_run *= alpha;
            }
            // The score buffer of tile j became full only after the P V product of tile j-1 had
            // completed (same issuing thread, in order), so the accumulator is at rest here.
            if (j > 0) {
#pragma unroll 1
                for (int ch = 0; ch < HD / 16; ch++) {
                    uint32_t o[16];
                    tmem_ld_32x32b_x16(o_addr + ch * 16, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_32x32b_x16(o_addr + ch * 16, o);
                }
            }
        }
        // probabilities -> bf16 pairs -> TMEM, over the score columns (already in registers)
        float l0 = 0.0f, l1 = 0.0f, l2 = 0.0f, l3 = 0.0f;
        const float neg_m = -m_run;
        // 32 probabilities of chunk `ch` -> 16 packed words
        auto chunk = [&](int ch, uint32_t (&packed)[16]) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                float x0, x1, x2, x3;
                fma2(x0, x1, __uint_as_float(sv[ch * 32 + i]), __uint_as_float(sv[ch * 32 + i + 1]), p.scale_log2, neg_m);
                fma2(x2, x3, __uint_as_float(sv[ch * 32 + i + 2]), __uint_as_float(sv[ch * 32 + i + 3]), p.scale_log2, neg_m);
                float p0, p1, p2, p3;
                if ((EMU >> (i >> 2)) & 1u) {
                    ex2_emu2(p0, p1, x0, x1);
                    ex2_emu2(p2, p3, x2, x3);
                } else {
                    p0 = ex2_approx(x0); p1 = ex2_approx(x1); p2 = ex2_approx(x2); p3 = ex2_approx(x3);
                }
                add2(l0, l1, p0, p1);
                add2(l2, l3, p2, p3);
                packed[i >> 1] = Elem<T>::pack(p0, p1);
                packed[(i >> 1) + 1] = Elem<T>::pack(p2, p3);
            }
        };
        // a half (64 keys) of P is in tensor memory: hand it to the MMA warp
        auto hand_over = [&](int half) {
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
            if (PAIR && rank != 0) mbar_arrive_cluster(mapa_shared(smem_u32(&p_full[2 * t + half]), 0));   // the issuing CTA's barrier
            else mbar_arrive(&p_full[2 * t + half]);
        }
        };
        // The stores of the first half are waited for only after the exponentials of the third chunk have
        // been computed: the store latency hides behind arithmetic instead of stalling the warp twice per step.
        uint32_t pk[16];
        chunk(0, pk);
        tmem_st_32x32b_x16(s_addr, pk);
        chunk(1, pk);
        tmem_st_32x32b_x16(s_addr + 16, pk);
        chunk(2, pk);
        hand_over(0);
        tmem_st_32x32b_x16(s_addr + 32, pk);
        chunk(3, pk);
        tmem_st_32x32b_x16(s_addr + 48, pk);
        hand_over(1);
        const float l_add = (l0 + l1) + (l2 + l3);
        l_run += l_add;
    }
    // ---- final: O / l -> bf16 -> global
    if (t < n_tiles) {
        if (ok) ok = mbar_wait(o_done, 0, abort_word, p.status, H3B_ST_TIMEOUT_OTHER);
        tc_fence_after();
        const float inv_l = 1.0f / l_run;
        // All MMAs and loads of the CTA are done: its tile memory is free.  Lane = row here; the rows of
        // the warp are parked in shared memory and written out sixteen lanes per 256-byte head slice,
        // two rows per store instruction (whole slices matter when the owner of a row is another GPU).
        constexpr int STG_ROW = 256 + 16;
        uint8_t *stg = smem + (size_t)(warp - 2) * 32 * STG_ROW;
#pragma unroll 1
        for (int ch = 0; ch < HD / 32; ch++) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(o_addr + ch * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                uint4 raw;
                uint32_t *h = reinterpret_cast<uint32_t *>(&raw);
#pragma unroll
                for (int u = 0; u < 4; u++)
                    h[u] = Elem<T>::pack(__uint_as_float(o[i + 2 * u]) * inv_l, __uint_as_float(o[i + 2 * u + 1]) * inv_l);
                *reinterpret_cast<uint4 *>(stg + lane * STG_ROW + (ch * 32 + i) * 2) = raw;
            }
        }
        __syncwarp();
        const int row_first = row0 + t * tile_stride + q * 32;   // row of lane 0
        const int sub = lane >> 4, chunk = lane & 15;
#pragma unroll
        for (int k2 = 0; k2 < 16; k2++) {
            const int rr = 2 * k2 + sub, row = row_first + rr;
            if (ok && row < p.lq) {
                T *dst;
                if (p.sc_rows) {
                    const int owner = row / p.sc_rows;
                    dst = reinterpret_cast<T *>(p.sc_out[owner < 8 ? owner : 0]) +
                          ((size_t)(row - owner * p.sc_rows) * p.sc_heads + p.sc_head0 + head) * HD;
                } else {
                    dst = reinterpret_cast<T *>(p.out) + (size_t)row * p.o_stride + (size_t)head * p.o_head_stride;
                }
                *reinterpret_cast<uint4 *>(dst + chunk * 8) = *reinterpret_cast<const uint4 *>(stg + rr * STG_ROW + chunk * 16);
            }
        }
    }

}

// EMU: bit q set = the q-th group of four probabilities of every 32 is computed by ex2_emu2 instead of ex2.approx
template <typename T, uint32_t EMU>
__global__ void __launch_bounds__(attn::THREADS, 1) k_attn(const __grid_constant__ AttnParams p) {
    using namespace attn;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sK = smem + 2 * TILE, *sV = smem + 4 * TILE;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + 6 * TILE);
    uint64_t *q_full = bars, *k_full = bars + 1, *v_full = bars + 3, *k_empty = bars + 5, *v_empty = bars + 7,
             *s_full = bars + 9, *p_full = bars + 11 /* [tile][half] */, *o_done = bars + 15;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 16);
    volatile int *abort_word = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * (2 * BQ), head = blockIdx.y;
    const int n_kv = (p.lk + BKV - 1) / BKV;
    // the second query tile may lie entirely beyond lq: it is then skipped by every role
    const int n_tiles = (q0 + BQ < p.lq) ? 2 : 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[2 * i], 4);
            mbar_init(&p_full[2 * i + 1], 4);
        }
        mbar_init(o_done, 1);
        *abort_word = 0;
        mbar_fence_init();
        tma_prefetch_desc(&p.tmap_q);
        tma_prefetch_desc(&p.tmap_k);
        tma_prefetch_desc(&p.tmap_v);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, n_tiles * TILE);
            for (int t = 0; t < n_tiles; t++) {
                tma_load_3d(sQ + t * TILE, &p.tmap_q, q_full, 0, head, q0 + t * BQ);
                tma_load_3d(sQ + t * TILE + SLAB, &p.tmap_q, q_full, 64, head, q0 + t * BQ);
            }
            for (int j = 0; j < n_kv; j++) {
                const int st = j & 1;
                const uint32_t ph = ((j >> 1) & 1) ^ 1;
                if (!mbar_wait(&k_empty[st], ph, abort_word, p.status, H3B_ST_TIMEOUT_EMPTY)) break;
                mbar_expect_tx(&k_full[st], TILE);
                tma_load_3d(sK + st * TILE, &p.tmap_k, &k_full[st], 0, head, j * BKV);
                tma_load_3d(sK + st * TILE + SLAB, &p.tmap_k, &k_full[st], 64, head, j * BKV);
                if (!mbar_wait(&v_empty[st], ph, abort_word, p.status, H3B_ST_TIMEOUT_EMPTY)) break;
                mbar_expect_tx(&v_full[st], TILE);
                tma_load_3d(sV + st * TILE, &p.tmap_v, &v_full[st], 0, head, j * BKV);
                tma_load_3d(sV + st * TILE + SLAB, &p.tmap_v, &v_full[st], 64, head, j * BKV);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp walks the loop, converged, so that descriptor arithmetic stays in uniform
        // registers; one elected lane issues each tcgen05 instruction.  (With a single active lane the
        // operands cross from vector to uniform registers per instruction, which cost about 85 cycles per
        // MMA against the 64 the MMA itself takes.)  The issuing thread is held back by the tensor pipe's
        // queue while its MMAs run, so whatever it does between two blocks happens with the pipe idle:
        // the K/V stage barriers of the NEXT iteration are therefore polled right after a block has been
        // issued (while the queue drains), and the loop is unrolled by two so that every shared-memory
        // descriptor is a loop-invariant value.
        // (One issuer per tile was tried: their MMAs interleave in the pipe, both tiles finish late, and the
        // kernel ran 30 % slower.)
        {
            // S = Q K^T : both operands K-major in shared memory (d contiguous).
            // O += P V  : P from TMEM (row = lane, two bf16 keys per 32-bit column); V as stored
            //             ([key][d], d contiguous) is the N-major form of the B operand.
            // EMU bit 31: one lane is elected once for the whole kernel and issues every tcgen05 instruction (the
            // commits must come from the thread that issued the MMAs they track); otherwise elect.sync runs in
            // front of every instruction
            const bool fixed_leader = elect_one();
            auto leader = [&]() -> bool { return (EMU >> 31) ? fixed_leader : elect_one(); };
            constexpr uint32_t idesc_s = umma_idesc(1, Elem<T>::FMT, Elem<T>::FMT, BQ, BKV, 0, 0);
            constexpr uint32_t idesc_o = umma_idesc(1, Elem<T>::FMT, Elem<T>::FMT, BQ, HD, 0, 1);
            const uint32_t q_base = smem_u32(sQ), k_base = smem_u32(sK), v_base = smem_u32(sV);
            // shared-memory descriptors as 32-bit halves (see umma_f16_ss_lh): one addition per operand and MMA
            constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, 128-byte swizzle
            const uint32_t q_lo0 = ((q_base & 0x3ffffu) >> 4) | (1u << 16), q_lo1 = q_lo0 + (TILE >> 4);
            const uint32_t k_lo0 = ((k_base & 0x3ffffu) >> 4) | (1u << 16);
            const uint32_t v_lo0 = ((v_base & 0x3ffffu) >> 4) | ((uint32_t)((SLAB >> 4) & 0x3fff) << 16);   // LBO = slab
            auto issue_s = [&](int t, int stage) {   // scores of tile t against the K tile in `stage`
                const uint32_t qa = t ? q_lo1 : q_lo0, kb = k_lo0 + (uint32_t)stage * (TILE >> 4);
                const uint32_t d_tmem = tmem_base + S_COL + 128u * t;
#pragma unroll
                for (int k = 0; k < HD / 16; k++) {
                    const uint32_t c = (uint32_t)(k >> 2) * (SLAB >> 4) + (uint32_t)(k & 3) * 2;   // (slab, 32 bytes) >> 4
                    if (leader()) umma_f16_ss_lh(d_tmem, qa + c, kb + c, DESC_HI, idesc_s, (uint32_t)(k != 0));
                }
                if (leader()) tc_commit(&s_full[t]);
            };
            auto issue_pv = [&](int t, int stage, int half, bool first) {
                const uint32_t vb = v_lo0 + (uint32_t)stage * (TILE >> 4);
#pragma unroll
                for (int k = half * (BKV / 32); k < (half + 1) * (BKV / 32); k++)
                    if (leader())
                        umma_f16_ts_lh(tmem_base + O_COL + 128u * t, tmem_base + S_COL + 128u * t + (uint32_t)k * 8,
                                       vb + (uint32_t)k * (2048 >> 4), DESC_HI, idesc_o, (uint32_t)(!first || k != 0));
            };
            bool ok = mbar_wait(q_full, 0, abort_word, p.status, H3B_ST_TIMEOUT_FULL) &&
                      mbar_wait(&k_full[0], 0, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
            if (ok) {
                tc_fence_after();
                for (int t = 0; t < n_tiles; t++) issue_s(t, 0);
                if (leader()) tc_commit(&k_empty[0]);
                ok = mbar_wait(&v_full[0], 0, abort_word, p.status, H3B_ST_TIMEOUT_FULL) &&
                     (n_kv < 2 || mbar_wait(&k_full[1], 0, abort_word, p.status, H3B_ST_TIMEOUT_FULL));
            }
            // one iteration with the K/V stage index as a compile-time constant
            auto step = [&](int j, auto stage_c) {
                constexpr int st = decltype(stage_c)::value, nx = st ^ 1;
                const bool more = j + 1 < n_kv;
                for (int t = 0; t < n_tiles && ok; t++) {
                    // P of this tile arrives in TMEM in two halves of 64 keys (all its scores are in the
                    // softmax threads' registers by then); the product over the first half runs while the
                    // second half is still being exponentiated
                    ok = mbar_wait(&p_full[2 * t], j & 1, abort_word, p.status, H3B_ST_TIMEOUT_OTHER);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(t, st, 0, j == 0);
                    ok = mbar_wait(&p_full[2 * t + 1], j & 1, abort_word, p.status, H3B_ST_TIMEOUT_OTHER);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(t, st, 1, false);
                    if (t == n_tiles - 1 && leader()) tc_commit(&v_empty[st]);
                    if (more) {
                        issue_s(t, nx);   // overwrites the tile's scores / P, in order after the P V product
                        if (t == n_tiles - 1 && leader()) tc_commit(&k_empty[nx]);
                    }
                }
                // stages of the next iteration: V(j+1) in stage nx, K(j+2) in stage st
                if (ok && more) {
                    ok = mbar_wait(&v_full[nx], ((j + 1) >> 1) & 1, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
                    if (ok && j + 2 < n_kv)
                        ok = mbar_wait(&k_full[st], ((j + 2) >> 1) & 1, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
                    tc_fence_after();
                }
            };
            for (int j = 0; ok && j < n_kv; j += 2) {
                step(j, std::integral_constant<int, 0>{});
                if (ok && j + 1 < n_kv) step(j + 1, std::integral_constant<int, 1>{});
            }
            if (leader()) tc_commit(o_done);
        }
        __syncwarp();
    } else {
        softmax_role<T, EMU, false>(p, smem, tmem_base, s_full, p_full, o_done, abort_word, warp, lane, n_kv, n_tiles, q0, BQ,
                                    head, 0);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// CTA-pair form.  A cluster of two CTAs serves 512 queries of one head: its two query tiles are 256 rows each, CTA r
// of the pair holds rows [128 r, 128 r + 128) of both, and every MMA is a cta_group::2 instruction of M = 256 issued
// by the CTA of rank 0.  The B operands are split along N: each CTA loads and holds HALF of every K tile (64 of its
// 128 keys) and HALF of every V tile (64 of its 128 columns), so per SM the shared-memory reads of B, the TMA writes
// and the L2 traffic of K and V are halved; the 64 KB that frees hold a third K/V stage.  Softmax and epilogue are
// the single-CTA kernel's, per CTA; "P is ready" is signalled on the issuing CTA's barriers, commits are multicast
// to both CTAs.  No TMA load is multicast: each CTA loads its own halves into its own shared memory.
namespace attnp {
constexpr int STAGES = 3;
constexpr int KH = 64 * 128 * 2, KSLAB = 64 * 64 * 2;   // K half: 64 keys x 128 d as two 64-row slabs (8 KiB each)
constexpr int VH = 128 * 64 * 2;                         // V half: 128 keys x 64 d, one slab (16 KiB)
// shared memory: Q_A Q_B | K halves | V halves | barriers
constexpr size_t SMEM_BYTES = 1024 + 2 * (size_t)attn::TILE + (size_t)STAGES * (KH + VH) + 256;
}  // namespace attnp

template <typename T, uint32_t EMU>
__global__ void __launch_bounds__(attn::THREADS, 1) k_attn_pair(const __grid_constant__ AttnParams p) {
    using namespace attn;
    using namespace attnp;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sK = smem + 2 * TILE, *sV = sK + STAGES * KH;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sV + STAGES * VH);
    uint64_t *q_full = bars, *k_full = bars + 1, *v_full = k_full + STAGES, *k_empty = v_full + STAGES,
             *v_empty = k_empty + STAGES, *s_full = v_empty + STAGES, *p_full = s_full + 2 /* [tile][half] */,
             *o_done = p_full + 4;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_done + 1);
    volatile int *abort_word = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int q0_pair = (int)(blockIdx.x >> 1) * (4 * BQ), head = blockIdx.y;
    const int row0 = q0_pair + (int)rank * BQ;          // this CTA's rows of the pair's first tile
    const int n_kv = (p.lk + BKV - 1) / BKV;
    const int n_tiles = (q0_pair + 2 * BQ < p.lq) ? 2 : 1;   // the same for both CTAs of the pair

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < STAGES; i++) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[2 * i], 8);       // four softmax warps of each CTA
            mbar_init(&p_full[2 * i + 1], 8);
        }
        mbar_init(o_done, 1);
        *abort_word = 0;
        mbar_fence_init();
        tma_prefetch_desc(&p.tmap_q);
        tma_prefetch_desc(&p.tmap_k);
        tma_prefetch_desc(&p.tmap_v);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // completion of both CTAs' loads is counted on the barriers of rank 0, which alone waits for them
            const uint32_t qf = mapa_shared(smem_u32(q_full), 0);
            if (rank == 0) mbar_expect_tx(q_full, 2 * n_tiles * TILE);
            for (int t = 0; t < n_tiles; t++) {
                tma_load_3d_pair(sQ + t * TILE, &p.tmap_q, qf, 0, head, row0 + t * 2 * BQ);
                tma_load_3d_pair(sQ + t * TILE + SLAB, &p.tmap_q, qf, 64, head, row0 + t * 2 * BQ);
            }
            for (int j = 0; j < n_kv; j++) {
                const int st = j % STAGES;
                const uint32_t ph = ((j / STAGES) & 1) ^ 1;
                if (!mbar_wait(&k_empty[st], ph, abort_word, p.status, H3B_ST_TIMEOUT_EMPTY)) break;
                const uint32_t kf = mapa_shared(smem_u32(&k_full[st]), 0);
                if (rank == 0) mbar_expect_tx(&k_full[st], 2 * KH);
                tma_load_3d_pair(sK + st * KH, &p.tmap_k, kf, 0, head, j * BKV + (int)rank * 64);
                tma_load_3d_pair(sK + st * KH + KSLAB, &p.tmap_k, kf, 64, head, j * BKV + (int)rank * 64);
                if (!mbar_wait(&v_empty[st], ph, abort_word, p.status, H3B_ST_TIMEOUT_EMPTY)) break;
                const uint32_t vf = mapa_shared(smem_u32(&v_full[st]), 0);
                if (rank == 0) mbar_expect_tx(&v_full[st], 2 * VH);
                tma_load_3d_pair(sV + st * VH, &p.tmap_v, vf, (int)rank * 64, head, j * BKV);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (rank == 0) {
            // ---- MMA issuer of the pair: the whole warp walks the loop, one lane elected once issues
            const bool lead = elect_one();
            constexpr uint32_t idesc_s = umma_idesc(1, Elem<T>::FMT, Elem<T>::FMT, 2 * BQ, BKV, 0, 0);
            constexpr uint32_t idesc_o = umma_idesc(1, Elem<T>::FMT, Elem<T>::FMT, 2 * BQ, HD, 0, 1);
            const uint32_t q_base = smem_u32(sQ), k_base = smem_u32(sK), v_base = smem_u32(sV);
            auto issue_s = [&](int t, int stage) {
                const uint32_t q_addr = q_base + t * TILE, k_addr = k_base + stage * KH;
                const uint32_t d_tmem = tmem_base + S_COL + 128u * t;
#pragma unroll
                for (int k = 0; k < HD / 16; k++) {
                    const uint32_t qo = (uint32_t)(k >> 2) * SLAB + (uint32_t)(k & 3) * 32;
                    const uint32_t ko = (uint32_t)(k >> 2) * KSLAB + (uint32_t)(k & 3) * 32;
                    if (lead)
                        umma_f16_ss_pair(d_tmem, umma_desc_k_sw128(q_addr + qo), umma_desc_k_sw128(k_addr + ko), idesc_s,
                                         (uint32_t)(k != 0));
                }
                if (lead) tc_commit_pair(&s_full[t], 3);
            };
            auto issue_pv = [&](int t, int stage, int half, bool first) {
                const uint32_t v_addr = v_base + stage * VH;
#pragma unroll
                for (int k = half * (BKV / 32); k < (half + 1) * (BKV / 32); k++)
                    if (lead)
                        umma_f16_ts_pair(tmem_base + O_COL + 128u * t, tmem_base + S_COL + 128u * t + (uint32_t)k * 8,
                                         umma_desc_mn_sw128(v_addr + (uint32_t)k * 2048, SLAB, 1024), idesc_o,
                                         (uint32_t)(!first || k != 0));
            };
            bool ok = mbar_wait(q_full, 0, abort_word, p.status, H3B_ST_TIMEOUT_FULL) &&
                      mbar_wait(&k_full[0], 0, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
            if (ok) {
                tc_fence_after();
                for (int t = 0; t < n_tiles; t++) issue_s(t, 0);
                if (lead) tc_commit_pair(&k_empty[0], 3);
                ok = mbar_wait(&v_full[0], 0, abort_word, p.status, H3B_ST_TIMEOUT_FULL) &&
                     (n_kv < 2 || mbar_wait(&k_full[1 % STAGES], 0, abort_word, p.status, H3B_ST_TIMEOUT_FULL));
            }
            // one iteration with the K/V stage index as a compile-time constant: V(j) in stage st, K(j+1) in nx
            auto step = [&](int j, auto stage_c) {
                constexpr int st = decltype(stage_c)::value, nx = (st + 1) % STAGES, n2 = (st + 2) % STAGES;
                const bool more = j + 1 < n_kv;
                for (int t = 0; t < n_tiles && ok; t++) {
                    ok = mbar_wait(&p_full[2 * t], j & 1, abort_word, p.status, H3B_ST_TIMEOUT_OTHER);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(t, st, 0, j == 0);
                    ok = mbar_wait(&p_full[2 * t + 1], j & 1, abort_word, p.status, H3B_ST_TIMEOUT_OTHER);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(t, st, 1, false);
                    if (t == n_tiles - 1 && lead) tc_commit_pair(&v_empty[st], 3);
                    if (more) {
                        issue_s(t, nx);
                        if (t == n_tiles - 1 && lead) tc_commit_pair(&k_empty[nx], 3);
                    }
                }
                if (ok && more) {
                    ok = mbar_wait(&v_full[nx], ((j + 1) / STAGES) & 1, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
                    if (ok && j + 2 < n_kv)
                        ok = mbar_wait(&k_full[n2], ((j + 2) / STAGES) & 1, abort_word, p.status, H3B_ST_TIMEOUT_FULL);
                    tc_fence_after();
                }
            };
            for (int j = 0; ok && j < n_kv; j += 3) {
                step(j, std::integral_constant<int, 0>{});
                if (ok && j + 1 < n_kv) step(j + 1, std::integral_constant<int, 1>{});
                if (ok && j + 2 < n_kv) step(j + 2, std::integral_constant<int, 2>{});
            }
            if (lead) tc_commit_pair(o_done, 3);
        }
        __syncwarp();
    } else {
        softmax_role<T, EMU, true>(p, smem, tmem_base, s_full, p_full, o_done, abort_word, warp, lane, n_kv, n_tiles, row0,
                                   2 * BQ, head, rank);
    }

    // a pair leaves together: neither CTA may exit while the other can still signal its barriers or read its tiles
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

static int make_map(CUtensorMap *map, const void *base, size_t stride_elems, size_t head_stride_elems, size_t rows,
                    size_t heads, int f16, char *error, size_t error_size, const char *what, uint32_t box_rows = 128) {
    int rc = h3b_encode_tmap_3d(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base,
                                attn::HD, heads, rows,
                                head_stride_elems * 2, stride_elems * 2, 64, 1, box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return fail(error, error_size, "sdpa: cuTensorMapEncodeTiled(%s) failed (%d)", what, rc);
    return 1;
}

// distances between heads of one row, in elements (0 = heads are contiguous, head_dim apart)
struct HeadStrides {
    size_t q = 0, k = 0, v = 0, o = 0;
};
static int launch_sdpa_impl(h3_cuda *cuda, const void *q, size_t qs, const void *k, size_t ks, const void *v, size_t vs,
                            size_t lq, size_t lk, size_t heads, size_t hd, float scale, void *out, size_t os,
                            const h3b_ulysses_direct *sc, int f16, char *error, size_t error_size,
                            HeadStrides hs = HeadStrides());

int launch_sdpa_bf16(h3_cuda *cuda, const void *q, size_t qs, const void *k, size_t ks, const void *v, size_t vs,
                     size_t lq, size_t lk, size_t heads, size_t hd, float scale, void *out, size_t os, char *error,
                     size_t error_size) {
    return launch_sdpa_impl(cuda, q, qs, k, ks, v, vs, lq, lk, heads, hd, scale, out, os, nullptr, 0, error, error_size);
}
int launch_sdpa_f16(h3_cuda *cuda, const void *q, size_t qs, const void *k, size_t ks, const void *v, size_t vs,
                    size_t lq, size_t lk, size_t heads, size_t hd, float scale, void *out, size_t os, char *error,
                    size_t error_size) {
    return launch_sdpa_impl(cuda, q, qs, k, ks, v, vs, lq, lk, heads, hd, scale, out, os, nullptr, 1, error, error_size);
}

static int launch_sdpa_impl(h3_cuda *cuda, const void *q, size_t qs, const void *k, size_t ks, const void *v, size_t vs,
                            size_t lq, size_t lk, size_t heads, size_t hd, float scale, void *out, size_t os,
                            const h3b_ulysses_direct *sc, int f16, char *error, size_t error_size, HeadStrides hs) {
    if (!cuda || !q || !k || !v || !out || !lq || !lk || !heads) return fail(error, error_size, "invalid sdpa args");
    if (hd != attn::HD) return fail(error, error_size, "sdpa: head_dim %zu unsupported (128 only)", hd);
    if ((qs % 8) || (ks % 8) || (vs % 8) || (os % 8) || ((uintptr_t)q & 15) || ((uintptr_t)k & 15) ||
        ((uintptr_t)v & 15) || ((uintptr_t)out & 15))
        return fail(error, error_size, "sdpa: pointers must be 16-byte aligned and row strides multiples of 8 elements");
    const bool packed = !hs.q && !hs.k && !hs.v && !hs.o;
    if (packed && (qs < heads * hd || ks < heads * hd || vs < heads * hd || os < heads * hd))
        return fail(error, error_size, "sdpa: row stride smaller than heads*head_dim");
    if (!hs.q) hs.q = hd;
    if (!hs.k) hs.k = hd;
    if (!hs.v) hs.v = hd;
    if (!hs.o) hs.o = hd;
    if ((hs.q | hs.k | hs.v | hs.o) % 8) return fail(error, error_size, "sdpa: head strides must be multiples of 8 elements");
    if (lq > 0x7fffff00u || lk > 0x7fffff00u || heads > 65535) return fail(error, error_size, "sdpa: shape too large");
    if (!(scale > 0.0f)) return fail(error, error_size, "sdpa: scale must be positive");
    // H3B_ATTN_EMU = 212 / 213: the CTA-pair form of the kernel (two / three eighths of the exponentials on the FMA pipe)
    static const int emu = atoi(h3_plugin_value("H3B_ATTN_EMU"));
    const bool pair = emu == 212 || emu == 213;
    AttnParams p;
    memset(&p, 0, sizeof(p));
    if (!make_map(&p.tmap_q, q, qs, hs.q, lq, heads, f16, error, error_size, "Q") ||
        !make_map(&p.tmap_k, k, ks, hs.k, lk, heads, f16, error, error_size, "K", pair ? 64 : 128) ||
        !make_map(&p.tmap_v, v, vs, hs.v, lk, heads, f16, error, error_size, "V"))
        return 0;
    p.out = out; p.o_stride = os; p.o_head_stride = hs.o; p.lq = (int)lq; p.lk = (int)lk; p.heads = (int)heads;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = cuda->d_status;
    if (sc) {
        // lq rows of the gathered sequence, each owned by rank row / seq_local
        if (lq > (size_t)sc->ulysses * sc->seq_local) return fail(error, error_size, "sdpa scatter: more rows than the ranks own");
        p.sc_rows = (int)sc->seq_local; p.sc_heads = (int)sc->heads;
        p.sc_head0 = (int)((size_t)sc->rank * (sc->heads / (size_t)sc->ulysses));
        for (int r = 0; r < sc->ulysses; r++) {
            if (!sc->peer_att[r]) return fail(error, error_size, "sdpa scatter: buffer of rank %d is not mapped", r);
            p.sc_out[r] = sc->peer_att[r];
        }
    }
    // Variant of the kernel (H3B_ATTN_EMU): 12 (default) = one lane elected once issues every tcgen05 instruction and
    // two eighths of the exponentials run on the FMA pipe; 13 = three eighths; 10 = none; 0 = none, and a lane is
    // elected in front of every instruction.
    constexpr uint32_t LEAD = 0x80000000u;
    if (pair) {
        void (*kp)(const AttnParams) = f16 ? k_attn_pair<__half, 0x11> : (emu == 213 ? k_attn_pair<__nv_bfloat16, 0x49>
                                                                                      : k_attn_pair<__nv_bfloat16, 0x11>);
        H3B_CUDA_OK(cudaFuncSetAttribute(kp, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attnp::SMEM_BYTES),
                    "sdpa smem attribute");
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.gridDim = dim3((unsigned)(2 * ceil_div(lq, 4 * attn::BQ)), (unsigned)heads);
        cfg.blockDim = dim3(attn::THREADS);
        cfg.dynamicSmemBytes = attnp::SMEM_BYTES;
        cfg.stream = cuda->op_stream;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        ProfScope prof(cuda, PROF_ATTN);
        H3B_CUDA_OK(cudaLaunchKernelEx(&cfg, kp, p), "k_attn_pair launch");
        cuda->launches++;
        return 1;
    }
    void (*kernel)(const AttnParams) = nullptr;
    if (f16) {
        kernel = k_attn<__half, LEAD | 0x11>;
        if (emu == 0) kernel = k_attn<__half, 0>;
    } else {
        kernel = k_attn<__nv_bfloat16, LEAD | 0x11>;
        if (emu == 0) kernel = k_attn<__nv_bfloat16, 0>;
        else if (emu == 10) kernel = k_attn<__nv_bfloat16, LEAD>;
        else if (emu == 13) kernel = k_attn<__nv_bfloat16, LEAD | 0x49>;
    }
    H3B_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn::SMEM_BYTES),
                "sdpa smem attribute");
    dim3 grid((unsigned)ceil_div(lq, 2 * attn::BQ), (unsigned)heads);
    ProfScope prof(cuda, PROF_ATTN);
    kernel<<<grid, attn::THREADS, attn::SMEM_BYTES, cuda->op_stream>>>(p);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_attn launch");
    return 1;
}

}  // namespace h3b

using namespace h3b;

static const char *g_last_backend = "none";

extern "C" {

int h3b_sdpa_bf16_dev(h3_cuda *cuda, const void *d_q, size_t q_stride, const void *d_k, size_t k_stride,
                      const void *d_v, size_t v_stride, size_t lq, size_t lk, size_t heads, size_t head_dim,
                      float scale, void *d_out, size_t o_stride, char *error, size_t error_size) {
    int ok = launch_sdpa_bf16(cuda, d_q, q_stride, d_k, k_stride, d_v, v_stride, lq, lk, heads, head_dim, scale, d_out,
                              o_stride, error, error_size);
    if (ok) g_last_backend = "tcgen05_flash_bf16";
    return ok;
}

// General form: bf16 or f16 tensors, explicit row AND head strides for every tensor (elements).  With head
// strides of lq * 128 / lk * 128 and row strides of 128 this is the [heads, rows, 128] layout of the reference's
// attention plugins.
int h3b_sdpa_strided_dev(h3_cuda *cuda, int dtype, const void *d_q, size_t q_row_stride, size_t q_head_stride,
                         const void *d_k, size_t k_row_stride, size_t k_head_stride, const void *d_v, size_t v_row_stride,
                         size_t v_head_stride, size_t lq, size_t lk, size_t heads, size_t head_dim, float scale, void *d_out,
                         size_t o_row_stride, size_t o_head_stride, char *error, size_t error_size) {
    if (dtype != H3B_BF16 && dtype != H3B_F16) return fail(error, error_size, "sdpa: dtype must be bf16 or f16");
    if (!q_head_stride || !k_head_stride || !v_head_stride || !o_head_stride)
        return fail(error, error_size, "sdpa: head strides must be given");
    HeadStrides hs;
    hs.q = q_head_stride; hs.k = k_head_stride; hs.v = v_head_stride; hs.o = o_head_stride;
    int ok = launch_sdpa_impl(cuda, d_q, q_row_stride, d_k, k_row_stride, d_v, v_row_stride, lq, lk, heads, head_dim, scale,
                              d_out, o_row_stride, nullptr, dtype == H3B_F16, error, error_size, hs);
    if (ok) g_last_backend = dtype == H3B_F16 ? "tcgen05_flash_f16" : "tcgen05_flash_bf16";
    return ok;
}

int h3b_sdpa_bf16_scatter_dev(h3_cuda *cuda, const h3b_ulysses_direct *sc, size_t seq_real, float scale, char *error,
                              size_t error_size) {
    if (!cuda || !sc || !seq_real) return fail(error, error_size, "sdpa scatter: invalid arguments");
    if (sc->ulysses < 1 || sc->ulysses > 8 || sc->rank < 0 || sc->rank >= sc->ulysses || sc->head_dim != 128 ||
        !sc->heads || sc->heads % (size_t)sc->ulysses || !sc->q || !sc->k || !sc->v)
        return fail(error, error_size, "sdpa scatter: bad geometry");
    const size_t hl = sc->heads / (size_t)sc->ulysses, il = hl * sc->head_dim;
    // `out` of the plain form is only checked for alignment: rows are stored through the scatter table
    int ok = launch_sdpa_impl(cuda, sc->q, il, sc->k, il, sc->v, il, seq_real, seq_real, hl, sc->head_dim, scale, sc->att,
                              sc->heads * sc->head_dim, sc, 0, error, error_size);
    if (ok) g_last_backend = "tcgen05_flash_bf16";
    return ok;
}

const char *h3_cuda_sdpa_backend_name(void) { return "tcgen05_flash"; }
const char *h3_cuda_sdpa_last_backend_name(void) { return g_last_backend; }

// ---- the reference's f16 attention entry points --------------------------------------------------------------
// F32 tensors in and out; Q, K, V and the result are staged as f16 like the reference's default path
// (h3_gpu_cuda.cu:12084-12220), the attention runs on the f16 form of the kernel above.

// layout of the handle's staging area for `n` elements per tensor: Q | K | V | O (f16)
static int stage4(h3_cuda *cuda, size_t n, __half **q, __half **k, __half **v, __half **o, char *error, size_t error_size) {
    if (!grow(cuda, &cuda->attn, &cuda->attn_bytes, 4 * n * sizeof(__half), error, error_size)) return 0;
    *q = (__half *)cuda->attn;
    *k = *q + n;
    *v = *k + n;
    *o = *v + n;
    return 1;
}

int h3_cuda_sdpa_f16_dev_ex(h3_cuda *cuda, const float *d_query, const float *d_key, const float *d_value,
                            size_t seq, size_t heads, size_t head_dim, float scale, int attn_window, float *d_out,
                            double *sdpa_ms, char *backend_out, size_t backend_out_size, char *error,
                            size_t error_size) {
    if (!cuda || !d_query || !d_key || !d_value || !d_out || !seq || !heads || !head_dim)
        return fail(error, error_size, "invalid sdpa args");
    if (attn_window != 0) return fail(error, error_size, "sdpa: windowed attention (attn_window=%d) is not supported", attn_window);
    const size_t n = seq * heads * head_dim, row = heads * head_dim;
    __half *q, *k, *v, *o;
    if (!stage4(cuda, n, &q, &k, &v, &o, error, error_size)) return 0;
    Timer t(cuda, sdpa_ms);
    int ok = h3b_cast_dev(cuda, d_query, H3B_F32, q, H3B_F16, n, error, error_size) &&
             h3b_cast_dev(cuda, d_key, H3B_F32, k, H3B_F16, n, error, error_size) &&
             h3b_cast_dev(cuda, d_value, H3B_F32, v, H3B_F16, n, error, error_size) &&
             launch_sdpa_f16(cuda, q, row, k, row, v, row, seq, seq, heads, head_dim, scale, o, row, error, error_size) &&
             h3b_cast_dev(cuda, o, H3B_F16, d_out, H3B_F32, n, error, error_size);
    t.stop();
    if (ok) g_last_backend = "tcgen05_flash_f16";
    if (backend_out && backend_out_size) snprintf(backend_out, backend_out_size, "tcgen05_flash_f16");
    return ok;
}

int h3_cuda_sdpa_f16_dev(h3_cuda *cuda, const float *d_query, const float *d_key, const float *d_value, size_t seq,
                         size_t heads, size_t head_dim, float scale, float *d_out, double *sdpa_ms, char *error,
                         size_t error_size) {
    return h3_cuda_sdpa_f16_dev_ex(cuda, d_query, d_key, d_value, seq, heads, head_dim, scale, 0, d_out, sdpa_ms, NULL,
                                   0, error, error_size);
}

// The reference's f32 name runs an FP32 flash kernel; here it runs the f16 tensor-core kernel (f32 softmax and
// accumulation, 11-bit operands): results agree with an f32 evaluation to about 5e-4 relative L2, not to f32 rounding.
int h3_cuda_sdpa_f32_dev(h3_cuda *cuda, const float *d_query, const float *d_key, const float *d_value, size_t seq,
                         size_t heads, size_t head_dim, float scale, float *d_out, double *sdpa_ms, char *error,
                         size_t error_size) {
    return h3_cuda_sdpa_f16_dev_ex(cuda, d_query, d_key, d_value, seq, heads, head_dim, scale, 0, d_out, sdpa_ms, NULL,
                                   0, error, error_size);
}

// Host tensors in and out (h3_gpu_cuda.h:562, :573, :610).
static int sdpa_host(h3_cuda *cuda, const float *query, const float *key, const float *value, size_t seq, size_t heads,
                     size_t head_dim, float scale, int attn_window, float *out, double *sdpa_ms, char *backend_out,
                     size_t backend_out_size, char *error, size_t error_size) {
    if (!cuda || !query || !key || !value || !out || !seq || !heads || !head_dim) return fail(error, error_size, "invalid sdpa args");
    const size_t bytes = seq * heads * head_dim * sizeof(float);
    float *d[4] = {NULL, NULL, NULL, NULL};
    int ok = 1;
    for (int i = 0; i < 4 && ok; i++)
        if (cudaMalloc((void **)&d[i], bytes) != cudaSuccess) ok = fail(error, error_size, "sdpa: device staging failed");
    const float *src[3] = {query, key, value};
    for (int i = 0; i < 3 && ok; i++)
        if (cudaMemcpyAsync(d[i], src[i], bytes, cudaMemcpyHostToDevice, cuda->op_stream) != cudaSuccess)
            ok = fail(error, error_size, "sdpa: upload failed");
    ok = ok && h3_cuda_sdpa_f16_dev_ex(cuda, d[0], d[1], d[2], seq, heads, head_dim, scale, attn_window, d[3], sdpa_ms, backend_out,
                                       backend_out_size, error, error_size);
    if (ok && (cudaMemcpyAsync(out, d[3], bytes, cudaMemcpyDeviceToHost, cuda->op_stream) != cudaSuccess ||
               cudaStreamSynchronize(cuda->op_stream) != cudaSuccess))
        ok = fail(error, error_size, "sdpa: download failed");
    cudaStreamSynchronize(cuda->op_stream);
    for (int i = 0; i < 4; i++)
        if (d[i]) cudaFree(d[i]);
    return ok;
}
int h3_cuda_sdpa_f16_ex(h3_cuda *cuda, const float *query, const float *key, const float *value, size_t seq, size_t heads,
                        size_t head_dim, float scale, int attn_window, float *out, double *sdpa_ms, char *backend_out,
                        size_t backend_out_size, char *error, size_t error_size) {
    return sdpa_host(cuda, query, key, value, seq, heads, head_dim, scale, attn_window, out, sdpa_ms, backend_out,
                     backend_out_size, error, error_size);
}
int h3_cuda_sdpa_f16(h3_cuda *cuda, const float *query, const float *key, const float *value, size_t seq, size_t heads,
                     size_t head_dim, float scale, float *out, double *sdpa_ms, char *error, size_t error_size) {
    return sdpa_host(cuda, query, key, value, seq, heads, head_dim, scale, 0, out, sdpa_ms, NULL, 0, error, error_size);
}
int h3_cuda_sdpa_f32(h3_cuda *cuda, const float *query, const float *key, const float *value, size_t seq, size_t heads,
                     size_t head_dim, float scale, float *out, double *sdpa_ms, char *error, size_t error_size) {
    return sdpa_host(cuda, query, key, value, seq, heads, head_dim, scale, 0, out, sdpa_ms, NULL, 0, error, error_size);
}

// ---- extra keys / values for the next QK-norm + RoPE + attention call (h3_gpu_cuda.h:815-819): a history of
// post-RoPE f16 K / V rows [hist_n, heads, head_dim] appended to the current ones (queries stay `seq` long), and a
// gather of chosen current K / V rows into caller buffers.  Process-wide, like the reference's.
static const void *g_kvcat_k, *g_kvcat_v;
static size_t g_kvcat_n;
static void *g_kvsave_k, *g_kvsave_v;
static const uint32_t *g_kvsave_idx;
static size_t g_kvsave_n;

void h3_cuda_sdpa_bind_kvcat(const void *d_k_hist, const void *d_v_hist, size_t hist_n) {
    g_kvcat_k = d_k_hist;
    g_kvcat_v = d_v_hist;
    g_kvcat_n = hist_n;
}
void h3_cuda_sdpa_bind_kvsave(void *d_k_save, void *d_v_save, const uint32_t *d_idx, size_t save_n) {
    g_kvsave_k = d_k_save;
    g_kvsave_v = d_v_save;
    g_kvsave_idx = d_idx;
    g_kvsave_n = save_n;
}
void h3_cuda_sdpa_clear_kvext(void) {
    g_kvcat_k = g_kvcat_v = NULL;
    g_kvcat_n = 0;
    g_kvsave_k = g_kvsave_v = NULL;
    g_kvsave_idx = NULL;
    g_kvsave_n = 0;
}

}  // extern "C"

namespace h3b {
// dst row r = src row idx[r]; rows are `row` f16 elements (a multiple of 8), moved 16 bytes per thread
__global__ void k_gather_rows_f16(const __half *src, __half *dst, const uint32_t *idx, size_t n_idx, size_t row) {
    const size_t vec = row / 8, total = n_idx * vec;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / vec, c = i - r * vec;
        reinterpret_cast<uint4 *>(dst + r * row)[c] = reinterpret_cast<const uint4 *>(src + (size_t)idx[r] * row)[c];
    }
}
}  // namespace h3b

extern "C" {

// common tail of the four QK-norm + RoPE + attention entry points: q/k/v are f16 [seq, heads, 128] in the staging area
static int rope_sdpa_tail(h3_cuda *cuda, __half *q, __half *k, __half *v, __half *o, size_t seq, size_t heads, size_t head_dim,
                          float scale, float *d_attn_out, double *sdpa_ms, char *backend_out, size_t backend_out_size,
                          char *error, size_t error_size) {
    const size_t row = heads * head_dim, n = seq * row;
    if (g_kvsave_n && g_kvsave_idx && g_kvsave_k && g_kvsave_v) {
        const unsigned grid = (unsigned)std::min<size_t>(ceil_div(g_kvsave_n * row / 8, 256), (size_t)cuda->sm_count * 8);
        k_gather_rows_f16<<<grid ? grid : 1, 256, 0, cuda->op_stream>>>(k, (__half *)g_kvsave_k, g_kvsave_idx, g_kvsave_n, row);
        k_gather_rows_f16<<<grid ? grid : 1, 256, 0, cuda->op_stream>>>(v, (__half *)g_kvsave_v, g_kvsave_idx, g_kvsave_n, row);
        cuda->launches += 2;
        H3B_CUDA_OK(cudaGetLastError(), "kvsave gather");
    }
    Timer t(cuda, sdpa_ms);
    int ok;
    if (g_kvcat_n > 0 && g_kvcat_k && g_kvcat_v) {
        // keys / values = [current | history] in one contiguous buffer, queries unchanged: rectangular attention
        const size_t lk = seq + g_kvcat_n;
        if (!grow(cuda, &cuda->kvx, &cuda->kvx_bytes, 2 * lk * row * sizeof(__half), error, error_size)) return 0;
        __half *kc = (__half *)cuda->kvx, *vc = kc + lk * row;
        cudaStream_t st = cuda->op_stream;
        H3B_CUDA_OK(cudaMemcpyAsync(kc, k, n * sizeof(__half), cudaMemcpyDeviceToDevice, st), "kvcat K");
        H3B_CUDA_OK(cudaMemcpyAsync(kc + n, g_kvcat_k, g_kvcat_n * row * sizeof(__half), cudaMemcpyDeviceToDevice, st), "kvcat K history");
        H3B_CUDA_OK(cudaMemcpyAsync(vc, v, n * sizeof(__half), cudaMemcpyDeviceToDevice, st), "kvcat V");
        H3B_CUDA_OK(cudaMemcpyAsync(vc + n, g_kvcat_v, g_kvcat_n * row * sizeof(__half), cudaMemcpyDeviceToDevice, st), "kvcat V history");
        ok = launch_sdpa_f16(cuda, q, row, kc, row, vc, row, seq, lk, heads, head_dim, scale, o, row, error, error_size);
    } else {
        ok = launch_sdpa_f16(cuda, q, row, k, row, v, row, seq, seq, heads, head_dim, scale, o, row, error, error_size);
    }
    ok = ok && h3b_cast_dev(cuda, o, H3B_F16, d_attn_out, H3B_F32, n, error, error_size);
    t.stop();
    if (ok) g_last_backend = "tcgen05_flash_f16";
    if (backend_out && backend_out_size) snprintf(backend_out, backend_out_size, "tcgen05_flash_f16");
    return ok;
}

static int rope_sdpa(h3_cuda *cuda, const void *d_qkv, int in_dtype, const float *d_q_norm, const float *d_k_norm,
                     const float *d_rope_cos, const float *d_rope_sin, size_t seq, size_t heads, size_t head_dim,
                     size_t rope_half, float epsilon, float scale, int attn_window, int grouped, int split_half,
                     float *d_attn_out, double *rope_ms, double *sdpa_ms, char *backend_out, size_t backend_out_size,
                     char *error, size_t error_size) {
    if (rope_ms) *rope_ms = 0.0;
    if (sdpa_ms) *sdpa_ms = 0.0;
    if (!cuda || !d_qkv || !d_attn_out || !seq || !heads || !head_dim) return fail(error, error_size, "invalid qkv_rope_sdpa args");
    if (attn_window != 0) return fail(error, error_size, "sdpa: windowed attention (attn_window=%d) is not supported", attn_window);
    const size_t n = seq * heads * head_dim;
    __half *q, *k, *v, *o;
    if (!stage4(cuda, n, &q, &k, &v, &o, error, error_size)) return 0;
    Timer tr(cuda, rope_ms);
    if (!h3b_qkv_rope_dev(cuda, d_qkv, in_dtype, d_q_norm, d_k_norm, d_rope_cos, d_rope_sin, seq, heads, head_dim, rope_half,
                          epsilon, grouped, split_half, q, k, v, H3B_F16, error, error_size))
        return 0;
    tr.stop();
    return rope_sdpa_tail(cuda, q, k, v, o, seq, heads, head_dim, scale, d_attn_out, sdpa_ms, backend_out, backend_out_size,
                          error, error_size);
}

// layout defaults of the reference (h3_gpu_cuda.cu:54-69): contiguous [Q|K|V] thirds unless H3_DIT_QKV_GROUPED=1,
// split-half RoPE pairing unless H3_DIT_ROPE_HALF_OFFSET=1 or H3_DIT_ROPE_SPLIT_HALF=0
static int default_grouped(void) { return strcmp(h3_plugin_value("H3_DIT_QKV_GROUPED"), "1") == 0; }
static int default_split_half(void) {
    return !(strcmp(h3_plugin_value("H3_DIT_ROPE_HALF_OFFSET"), "1") == 0 || strcmp(h3_plugin_value("H3_DIT_ROPE_SPLIT_HALF"), "0") == 0);
}

int h3_cuda_qkv_rope_sdpa_f16_dev_layout(h3_cuda *cuda, const float *d_qkv, const float *d_q_norm, const float *d_k_norm,
                                         const float *d_rope_cos, const float *d_rope_sin, size_t seq, size_t heads,
                                         size_t head_dim, size_t rope_half, float epsilon, float scale, int attn_window,
                                         int grouped, int split_half, float *d_attn_out, double *rope_ms, double *sdpa_ms,
                                         char *backend_out, size_t backend_out_size, char *error, size_t error_size) {
    return rope_sdpa(cuda, d_qkv, H3B_F32, d_q_norm, d_k_norm, d_rope_cos, d_rope_sin, seq, heads, head_dim, rope_half, epsilon,
                     scale, attn_window, grouped, split_half, d_attn_out, rope_ms, sdpa_ms, backend_out, backend_out_size, error,
                     error_size);
}
int h3_cuda_qkv_rope_sdpa_f16_dev(h3_cuda *cuda, const float *d_qkv, const float *d_q_norm, const float *d_k_norm,
                                  const float *d_rope_cos, const float *d_rope_sin, size_t seq, size_t heads,
                                  size_t head_dim, size_t rope_half, float epsilon, float scale, int attn_window,
                                  float *d_attn_out, double *rope_ms, double *sdpa_ms, char *backend_out,
                                  size_t backend_out_size, char *error, size_t error_size) {
    return rope_sdpa(cuda, d_qkv, H3B_F32, d_q_norm, d_k_norm, d_rope_cos, d_rope_sin, seq, heads, head_dim, rope_half, epsilon,
                     scale, attn_window, default_grouped(), default_split_half(), d_attn_out, rope_ms, sdpa_ms, backend_out,
                     backend_out_size, error, error_size);
}
// the same with the QKV projection already stored as f16 (h3_gpu_cuda.h:779-793)
int h3_cuda_qkv_rope_sdpa_f16_dev_layout_f16qkv(h3_cuda *cuda, const void *d_qkv_half, const float *d_q_norm,
                                                const float *d_k_norm, const float *d_rope_cos, const float *d_rope_sin,
                                                size_t seq, size_t heads, size_t head_dim, size_t rope_half, float epsilon,
                                                float scale, int attn_window, int grouped, int split_half, float *d_attn_out,
                                                double *rope_ms, double *sdpa_ms, char *backend_out, size_t backend_out_size,
                                                char *error, size_t error_size) {
    return rope_sdpa(cuda, d_qkv_half, H3B_F16, d_q_norm, d_k_norm, d_rope_cos, d_rope_sin, seq, heads, head_dim, rope_half,
                     epsilon, scale, attn_window, grouped, split_half, d_attn_out, rope_ms, sdpa_ms, backend_out, backend_out_size,
                     error, error_size);
}
int h3_cuda_qkv_rope_sdpa_f16_dev_f16qkv(h3_cuda *cuda, const void *d_qkv_half, const float *d_q_norm, const float *d_k_norm,
                                         const float *d_rope_cos, const float *d_rope_sin, size_t seq, size_t heads,
                                         size_t head_dim, size_t rope_half, float epsilon, float scale, int attn_window,
                                         float *d_attn_out, double *rope_ms, double *sdpa_ms, char *backend_out,
                                         size_t backend_out_size, char *error, size_t error_size) {
    return rope_sdpa(cuda, d_qkv_half, H3B_F16, d_q_norm, d_k_norm, d_rope_cos, d_rope_sin, seq, heads, head_dim, rope_half,
                     epsilon, scale, attn_window, default_grouped(), default_split_half(), d_attn_out, rope_ms, sdpa_ms,
                     backend_out, backend_out_size, error, error_size);
}

}  // extern "C"
