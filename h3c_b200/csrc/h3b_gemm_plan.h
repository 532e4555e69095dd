/* Work decomposition of the persistent int8 GEMM over CTA pairs: whole tiles, and the tiles of a short last wave cut
 * along K.  Plain C, shared by the kernel, its launcher and the tests (no GPU needed to evaluate it). */
#ifndef H3B_GEMM_PLAN_H
#define H3B_GEMM_PLAN_H

#include <math.h>

#if defined(__CUDACC__)
#define H3B_PLAN_FN __host__ __device__ static inline
#else
#define H3B_PLAN_FN static inline
#endif

typedef struct h3b_gemm_plan {
    int items_total;   /* work items; pair p takes items p, p + pairs, p + 2 pairs, ... */
    int tail_first;    /* items [0, tail_first) are whole tiles (item = tile); a multiple of `pairs` when split_s > 1 */
    int split_s;       /* slices per tail tile (1: every item is a whole tile) */
} h3b_gemm_plan;

typedef struct h3b_gemm_item {
    int tile, kb0, kb1;   /* k-blocks [kb0, kb1) of tile `tile` */
    int slice, slot;      /* slice 0 owns the tile's epilogue; slot = index of the tail tile */
    int parts;            /* slices of this tile (1 for a whole tile) */
} h3b_gemm_item;

/* mode 0: never cut; 1: cut where the estimate below gains 8 us or more; n >= 2: n slices wherever a cut is possible.
 * A cut is possible when there is more than one wave and the last one fills at most half of the pairs; the slices of
 * all tail tiles then fit into that one wave (rem * split <= pairs), every slice has at least two k-blocks, and there
 * are at most 16 of them.  Estimate: a tile of T = 0.39 us x k_blocks; cutting it in S saves T - T/S and costs about
 * 2 us per region the owning pair reads, on top of a fixed part that the 8 us threshold covers. */
H3B_PLAN_FN h3b_gemm_plan h3b_gemm_make_plan(int tiles, int pairs, int k_blocks, int mode) {
    h3b_gemm_plan pl;
    int rem, split;
    pl.items_total = tiles; pl.tail_first = tiles; pl.split_s = 1;
    if (pairs <= 0 || tiles <= pairs || mode <= 0) return pl;
    rem = tiles % pairs;
    if (rem == 0 || 2 * rem > pairs) return pl;
    split = mode;
    if (mode == 1) {
        const double t_tile = 0.39 * k_blocks, fold = 2.0;
        split = (int)(sqrt(t_tile / fold) + 0.5);
        if (split >= 2 && t_tile - t_tile / split - fold * (split - 1) < 8.0) split = 1;
    }
    if (split > pairs / rem) split = pairs / rem;
    if (split > k_blocks / 2) split = k_blocks / 2;
    if (split > 16) split = 16;
    if (split < 2) return pl;
    pl.split_s = split;
    pl.tail_first = tiles - rem;
    pl.items_total = pl.tail_first + rem * split;
    return pl;
}

H3B_PLAN_FN h3b_gemm_item h3b_gemm_get_item(int tail_first, int split_s, int k_blocks, int item) {
    h3b_gemm_item w;
    if (item < tail_first) {
        w.tile = item; w.kb0 = 0; w.kb1 = k_blocks; w.slice = 0; w.slot = 0; w.parts = 1;
    } else {
        const int idx = item - tail_first;
        w.slot = idx / split_s;
        w.slice = idx - w.slot * split_s;
        w.tile = tail_first + w.slot;
        w.parts = split_s;
        w.kb0 = (int)((long long)w.slice * k_blocks / split_s);
        w.kb1 = (int)((long long)(w.slice + 1) * k_blocks / split_s);
    }
    return w;
}

#endif
