/* DiT block and block-chain host code, plain C on top of the C ABI of this library.
 *
 * One block is a fixed sequence of kernel launches on the handle's stream; nothing
 * synchronises inside.  Two block shapes are supported:
 *   H3B_BLOCK_REFERENCE   the reference's block (h3_dit_w4a8.c:3597-3830 device phases):
 *                         adaLN -> QKV -> QK-norm/RoPE -> SDPA -> out (+gate, residual)
 *                         -> adaLN -> fc1 (SwiGLU) -> fc2 (+gate, residual)
 *   H3B_BLOCK_CROSS_GELU  the benchmark's block: the same self-attention part, then
 *                         rms_norm -> cross-attention to the text tokens (+residual),
 *                         then adaLN -> up (tanh-GELU) -> down (+gate, residual)
 * Activations are kept in the configured stream type (f32 like the reference's CUDA
 * path, or bf16); every quantised linear is "norm/rotate/quantise rows -> int8 GEMM
 * with fused epilogue".
 */
#include <cuda_runtime_api.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/h3_b200.h"
#include "../../include/h3b_plugin.h"

typedef struct {
    const h3_cuda_w4a8_weight *lin[H3B_LIN_COUNT];
    const h3_cuda_nvfp4_weight *fp4[4];                  /* NVFP4 form of QKV / OUT / FC1 / FC2; NULL = the INT8 weight */
    float *norm1, *norm2, *q_norm, *k_norm, *norm_cross; /* device */
    float *adaln_w, *adaln_b;                            /* device */
    float *modulation;                                   /* device [mod_rows, 6, dim] */
} h3b_block;

struct h3b_dit {
    h3_cuda *cuda;
    h3b_dit_config cfg;
    h3b_block *blocks;
    /* workspace (device) */
    size_t cap_seq, cap_text;
    void *xa, *xb;          /* block-internal residuals x1 / x2, stream dtype [seq, dim] */
    void *io;               /* chain input/output of the host-buffer entry point, stream dtype [seq, dim] */
    void *qkv;              /* [seq, 3*inner] stream dtype */
    void *wide;             /* [seq, ffn] stream dtype (FFN activation) */
    void *q, *k, *v, *att;  /* bf16 [seq, inner] each */
    void *cq;               /* bf16 [seq, inner] cross-attention queries */
    void *ckv;              /* bf16 [text, 2*inner] */
    float *rotf;            /* f32 [seq, max(dim, ffn, inner)]: activations of an NVFP4 linear (only when one is set) */
    uint8_t *x4, *sfx;      /* NVFP4 codes [seq, max/2] and scale bytes of those activations (same condition) */
    int any_fp4;
    int8_t *q8;             /* [seq, max(dim, ffn, inner)] activation codes */
    float *s8;              /* [seq] activation scales */
    int8_t *tq8;            /* [text, dim] */
    float *ts8;             /* [text] */
    /* staging for the host-buffer entry point */
    float *st_x;            /* f32 [seq, dim] */
    float *st_text;         /* f32 [text, dim] */
    void *text_dev;         /* stream-dtype copy of the text tokens */
    uint32_t *st_map;
    float *st_cos, *st_sin, *st_t;
    h3_ulysses_cfg *uly;    /* attached per-rank communicator, or NULL */
    h3_cuda_w4a8_weight **owned;   /* weights created by the checkpoint loaders, freed with the context */
    size_t n_owned, cap_owned;
    h3_cuda_nvfp4_weight **owned_fp4;
    size_t n_owned_fp4, cap_owned_fp4;
    /* the chain captured as one CUDA graph (h3b_dit_layers_forward_graph_dev) and what it was captured for */
    cudaGraph_t graph;
    cudaGraphExec_t graph_exec;
    struct {
        unsigned first, n;
        const void *x, *text;
        void *y;
        const uint32_t *row_map;
        const float *cos, *sin;
        size_t seq, text_seq;
    } graph_key;
};

static int fail(char *error, size_t error_size, const char *fmt, ...) {
    if (error && error_size) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(error, error_size, fmt, ap);
        va_end(ap);
    }
    return 0;
}

static size_t elem(const h3b_dit *d) { return d->cfg.stream_dtype == H3B_F32 ? 4 : 2; }
static size_t inner(const h3b_dit *d) { return d->cfg.heads * d->cfg.head_dim; }

static int dmalloc(void **p, size_t bytes, char *error, size_t error_size) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess) return fail(error, error_size, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
    return 1;
}

static int upload(float **dst, const float *src, size_t count, char *error, size_t error_size) {
    cudaError_t e;
    if (!src) return 1;
    if (!*dst && !dmalloc((void **)dst, count * sizeof(float), error, error_size)) return 0;
    e = cudaMemcpy(*dst, src, count * sizeof(float), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(error, error_size, "cudaMemcpy(H2D): %s", cudaGetErrorString(e));
    return 1;
}

h3b_dit *h3b_dit_create(h3_cuda *cuda, const h3b_dit_config *cfg, char *error, size_t error_size) {
    h3b_dit *d;
    if (!cuda || !cfg) {
        fail(error, error_size, "h3b_dit_create: invalid arguments");
        return NULL;
    }
    if (cfg->kind != H3B_BLOCK_REFERENCE && cfg->kind != H3B_BLOCK_CROSS_GELU) {
        fail(error, error_size, "h3b_dit_create: unknown block kind %d", cfg->kind);
        return NULL;
    }
    if (cfg->stream_dtype != H3B_F32 && cfg->stream_dtype != H3B_BF16) {
        fail(error, error_size, "h3b_dit_create: stream dtype must be f32 or bf16");
        return NULL;
    }
    if (!cfg->dim || !cfg->heads || cfg->head_dim != 128 || !cfg->ffn || !cfg->n_blocks || !cfg->mod_rows ||
        cfg->rope_half * 2 > cfg->head_dim) {
        fail(error, error_size, "h3b_dit_create: bad geometry (head_dim must be 128)");
        return NULL;
    }
    if (cfg->kind == H3B_BLOCK_CROSS_GELU && cfg->heads * cfg->head_dim != cfg->dim) {
        fail(error, error_size, "h3b_dit_create: cross block needs heads*head_dim == dim");
        return NULL;
    }
    d = (h3b_dit *)calloc(1, sizeof(*d));
    if (!d) {
        fail(error, error_size, "h3b_dit_create: out of memory");
        return NULL;
    }
    d->cuda = cuda;
    d->cfg = *cfg;
    d->blocks = (h3b_block *)calloc(cfg->n_blocks, sizeof(h3b_block));
    if (!d->blocks) {
        free(d);
        fail(error, error_size, "h3b_dit_create: out of memory");
        return NULL;
    }
    return d;
}

static void drop_graph(h3b_dit *d) {
    if (d->graph_exec) cudaGraphExecDestroy(d->graph_exec);
    if (d->graph) cudaGraphDestroy(d->graph);
    d->graph_exec = NULL;
    d->graph = NULL;
}

/* The workspace is two groups of buffers that grow independently and never shrink: those sized by the token
 * count (cq, the cross-attention queries, included) and those sized by the text length. */
static void free_group(void ***p, size_t n) {
    size_t i;
    for (i = 0; i < n; i++) {
        if (*p[i]) cudaFree(*p[i]);
        *p[i] = NULL;
    }
}
static void free_seq_ws(h3b_dit *d) {
    void **p[] = {&d->xa, &d->xb, &d->io, &d->qkv, &d->wide, &d->q, &d->k, &d->v, &d->att, &d->cq, (void **)&d->q8,
                  (void **)&d->rotf, (void **)&d->x4, (void **)&d->sfx, (void **)&d->s8, (void **)&d->st_x, (void **)&d->st_map, (void **)&d->st_cos, (void **)&d->st_sin,
                  (void **)&d->st_t};
    drop_graph(d);   /* a captured chain points into the workspace */
    free_group(p, sizeof(p) / sizeof(p[0]));
    d->cap_seq = 0;
}
static void free_text_ws(h3b_dit *d) {
    void **p[] = {&d->ckv, (void **)&d->tq8, (void **)&d->ts8, (void **)&d->st_text, &d->text_dev};
    drop_graph(d);
    free_group(p, sizeof(p) / sizeof(p[0]));
    d->cap_text = 0;
}
static void free_ws(h3b_dit *d) {
    free_seq_ws(d);
    free_text_ws(d);
}

void h3b_dit_free(h3b_dit *d) {
    size_t b;
    if (!d) return;
    cudaDeviceSynchronize();
    free_ws(d);
    for (b = 0; b < d->cfg.n_blocks; b++) {
        h3b_block *k = &d->blocks[b];
        float *p[] = {k->norm1, k->norm2, k->q_norm, k->k_norm, k->norm_cross, k->adaln_w, k->adaln_b, k->modulation};
        size_t i;
        for (i = 0; i < sizeof(p) / sizeof(p[0]); i++)
            if (p[i]) cudaFree(p[i]);
    }
    for (b = 0; b < d->n_owned; b++) h3_cuda_w4a8_weight_free(d->owned[b]);
    free(d->owned);
    for (b = 0; b < d->n_owned_fp4; b++) h3_cuda_nvfp4_weight_free(d->cuda, d->owned_fp4[b]);
    free(d->owned_fp4);
    free(d->blocks);
    free(d);
}

int h3b_dit_set_linear(h3b_dit *d, unsigned block, int which, const h3_cuda_w4a8_weight *w, char *error,
                       size_t error_size) {
    size_t n, k, D, I, F;
    if (!d || !w || block >= d->cfg.n_blocks || which < 0 || which >= H3B_LIN_COUNT)
        return fail(error, error_size, "h3b_dit_set_linear: invalid arguments");
    n = h3_cuda_w4a8_weight_n(w);
    k = h3_cuda_w4a8_weight_k(w);
    D = d->cfg.dim; I = inner(d); F = d->cfg.ffn;
    {
        const int swiglu = d->cfg.kind == H3B_BLOCK_REFERENCE;
        const size_t want_n[H3B_LIN_COUNT] = {3 * I, D, swiglu ? 2 * F : F, D, I, 2 * I, D};
        const size_t want_k[H3B_LIN_COUNT] = {D, I, D, F, D, D, I};
        if (n != want_n[which] || k != want_k[which])
            return fail(error, error_size, "h3b_dit_set_linear: linear %d is [%zu,%zu], expected [%zu,%zu]", which, n, k,
                        want_n[which], want_k[which]);
    }
    if (d->blocks[block].lin[which] != w) drop_graph(d);   /* a captured chain holds the old weight's pointers */
    d->blocks[block].lin[which] = w;
    return 1;
}

/* Per-linear choice between the INT8 and the NVFP4 form of a weight, as the reference's nvfp4_gemm_dispatch makes it
 * (h3_dit_w4a8.c:3519-3590, call sites :3623-3641): a linear with an NVFP4 weight set runs
 * ConvRot -> NVFP4 activation quantisation -> block-scaled GEMM with the plain (QKV), SwiGLU (FC1) or gate (OUT, FC2)
 * epilogue on f32 activations; the others keep their INT8 weight.  w == NULL returns the linear to INT8. */
int h3b_dit_set_linear_nvfp4(h3b_dit *d, unsigned block, int which, const h3_cuda_nvfp4_weight *w, char *error,
                             size_t error_size) {
    size_t D, I, F;
    if (!d || block >= d->cfg.n_blocks || which < H3B_LIN_QKV || which > H3B_LIN_FC2)
        return fail(error, error_size, "h3b_dit_set_linear_nvfp4: invalid arguments");
    if (d->cfg.kind != H3B_BLOCK_REFERENCE || d->cfg.stream_dtype != H3B_F32)
        return fail(error, error_size, "h3b_dit_set_linear_nvfp4: NVFP4 linears go with the reference block on an f32 stream");
    D = d->cfg.dim; I = inner(d); F = d->cfg.ffn;
    if (w) {
        const size_t want_n[4] = {3 * I, D, 2 * F, D}, want_k[4] = {D, I, D, F};
        const size_t n = h3_cuda_nvfp4_weight_n(w), k = h3_cuda_nvfp4_weight_k(w);
        if (n != want_n[which] || k != want_k[which])
            return fail(error, error_size, "h3b_dit_set_linear_nvfp4: linear %d is [%zu,%zu], expected [%zu,%zu]", which, n, k,
                        want_n[which], want_k[which]);
        if (!d->any_fp4) {
            d->any_fp4 = 1;
            if (d->cap_seq) free_seq_ws(d);   /* the next reserve adds the f32 activation buffer */
        }
    }
    if (d->blocks[block].fp4[which] != w) drop_graph(d);
    d->blocks[block].fp4[which] = w;
    return 1;
}

int h3b_dit_set_block_aux(h3b_dit *d, unsigned block, const float *norm1, const float *norm2, const float *q_norm,
                          const float *k_norm, const float *norm_cross, char *error, size_t error_size) {
    h3b_block *b;
    if (!d || block >= d->cfg.n_blocks || !norm1 || !norm2 || !q_norm || !k_norm)
        return fail(error, error_size, "h3b_dit_set_block_aux: invalid arguments");
    b = &d->blocks[block];
    return upload(&b->norm1, norm1, d->cfg.dim, error, error_size) &&
           upload(&b->norm2, norm2, d->cfg.dim, error, error_size) &&
           upload(&b->q_norm, q_norm, d->cfg.head_dim, error, error_size) &&
           upload(&b->k_norm, k_norm, d->cfg.head_dim, error, error_size) &&
           upload(&b->norm_cross, norm_cross, d->cfg.dim, error, error_size);
}

static size_t mod_elems(const h3b_dit *d) { return d->cfg.mod_rows * 6 * d->cfg.dim; }

int h3b_dit_set_adaln(h3b_dit *d, unsigned block, const float *w, const float *b, char *error, size_t error_size) {
    h3b_block *k;
    if (!d || block >= d->cfg.n_blocks || !w || !b || !d->cfg.t_dim)
        return fail(error, error_size, "h3b_dit_set_adaln: invalid arguments");
    k = &d->blocks[block];
    if (!k->modulation && !dmalloc((void **)&k->modulation, mod_elems(d) * sizeof(float), error, error_size)) return 0;
    return upload(&k->adaln_w, w, mod_elems(d) * d->cfg.t_dim, error, error_size) &&
           upload(&k->adaln_b, b, mod_elems(d), error, error_size);
}

/* ---- INT8-ConvRot checkpoint block -> context (names of h3_dit_int8.h:37-40 and h3_dit_w4a8.c:2056-2117) */
static const float *ckpt_f32(const h3b_ckpt *c, const char *name, size_t count, char *error, size_t error_size) {
    h3b_ckpt_tensor t;
    if (!h3b_ckpt_find(c, name, &t)) {
        fail(error, error_size, "checkpoint: tensor %s missing", name);
        return NULL;
    }
    if (strcmp(t.dtype, "F32") != 0 || t.bytes != count * sizeof(float)) {
        fail(error, error_size, "checkpoint: %s is %s with %zu bytes, expected F32 x %zu", name, t.dtype, t.bytes, count);
        return NULL;
    }
    return (const float *)t.data;
}

/* The four linears of a block under the reference's names, their slots and shapes [n, k]. */
static const char *const ckpt_suffix[4] = {"attn.qkv_proj", "attn.out_proj", "mlp.fc1", "mlp.fc2"};
static const int ckpt_slot[4] = {H3B_LIN_QKV, H3B_LIN_OUT, H3B_LIN_FC1, H3B_LIN_FC2};
static void ckpt_linear_shapes(const h3b_dit *d, size_t n[4], size_t k[4]) {
    const size_t D = d->cfg.dim, I = inner(d), F = d->cfg.ffn;
    n[0] = 3 * I; k[0] = D;
    n[1] = D;     k[1] = I;
    n[2] = 2 * F; k[2] = D;
    n[3] = D;     k[3] = F;
}

/* Keeps a weight the loader created until the context is freed; on failure the weight is freed here. */
static int own_weight(h3b_dit *d, h3_cuda_w4a8_weight *obj, char *error, size_t error_size) {
    if (d->n_owned == d->cap_owned) {
        size_t ncap = d->cap_owned ? 2 * d->cap_owned : 16;
        h3_cuda_w4a8_weight **no = (h3_cuda_w4a8_weight **)realloc(d->owned, ncap * sizeof(*no));
        if (!no) {
            h3_cuda_w4a8_weight_free(obj);
            return fail(error, error_size, "checkpoint loader: out of host memory");
        }
        d->owned = no;
        d->cap_owned = ncap;
    }
    d->owned[d->n_owned++] = obj;
    return 1;
}

/* Norm weights, QK-norm weights and (optional) adaLN projection of a block: the same names in all three checkpoint
 * formats (h3_dit_w4a8.c:2056-2104). */
static int load_block_aux_from_ckpt(h3b_dit *d, const h3b_ckpt *ckpt, unsigned src_block, unsigned dst_block, char *error,
                                    size_t error_size) {
    char name[256];
    const float *n1, *n2, *qn, *kn, *aw, *ab;
    const size_t D = d->cfg.dim, mod = d->cfg.mod_rows * 6 * D;
    snprintf(name, sizeof(name), "blocks.%u.norm1.weight", src_block);
    if (!(n1 = ckpt_f32(ckpt, name, D, error, error_size))) return 0;
    snprintf(name, sizeof(name), "blocks.%u.norm2.weight", src_block);
    if (!(n2 = ckpt_f32(ckpt, name, D, error, error_size))) return 0;
    snprintf(name, sizeof(name), "blocks.%u.attn.q_norm.weight", src_block);
    if (!(qn = ckpt_f32(ckpt, name, d->cfg.head_dim, error, error_size))) return 0;
    snprintf(name, sizeof(name), "blocks.%u.attn.k_norm.weight", src_block);
    if (!(kn = ckpt_f32(ckpt, name, d->cfg.head_dim, error, error_size))) return 0;
    if (!h3b_dit_set_block_aux(d, dst_block, n1, n2, qn, kn, NULL, error, error_size)) return 0;
    snprintf(name, sizeof(name), "blocks.%u.adaln_proj.linear.weight", src_block);
    if (h3b_ckpt_find(ckpt, name, NULL)) {   /* optional: a caller may supply the modulation itself */
        if (!(aw = ckpt_f32(ckpt, name, mod * d->cfg.t_dim, error, error_size))) return 0;
        snprintf(name, sizeof(name), "blocks.%u.adaln_proj.linear.bias", src_block);
        if (!(ab = ckpt_f32(ckpt, name, mod, error, error_size))) return 0;
        if (!h3b_dit_set_adaln(d, dst_block, aw, ab, error, error_size)) return 0;
    }
    return 1;
}

int h3b_dit_load_int8_convrot_block(h3b_dit *d, const h3b_ckpt *ckpt, unsigned src_block, unsigned dst_block,
                                    char *error, size_t error_size) {
    char name[256];
    size_t want_n[4], want_k[4];
    int l;
    if (!d || !ckpt || dst_block >= d->cfg.n_blocks) return fail(error, error_size, "load_int8_convrot_block: invalid arguments");
    if (d->cfg.kind != H3B_BLOCK_REFERENCE)
        return fail(error, error_size, "load_int8_convrot_block: the INT8-ConvRot checkpoint holds the reference block");
    ckpt_linear_shapes(d, want_n, want_k);
    for (l = 0; l < 4; l++) {
        h3b_ckpt_tensor w, s;
        h3_cuda_w4a8_weight *obj = NULL;
        snprintf(name, sizeof(name), "blocks.%u.%s.weight", src_block, ckpt_suffix[l]);
        if (!h3b_ckpt_find(ckpt, name, &w)) return fail(error, error_size, "checkpoint: tensor %s missing", name);
        if (strcmp(w.dtype, "I8") != 0 || w.rank != 2 || w.shape[0] != want_n[l] || w.shape[1] != want_k[l])
            return fail(error, error_size, "checkpoint: %s is %s rank %d [%zu, %zu], expected I8 [%zu, %zu]", name, w.dtype,
                        w.rank, w.shape[0], w.rank > 1 ? w.shape[1] : 0, want_n[l], want_k[l]);
        snprintf(name, sizeof(name), "blocks.%u.%s.weight_scale", src_block, ckpt_suffix[l]);
        if (!h3b_ckpt_find(ckpt, name, &s)) return fail(error, error_size, "checkpoint: tensor %s missing", name);
        if (strcmp(s.dtype, "F32") != 0 || s.bytes != want_n[l] * sizeof(float))
            return fail(error, error_size, "checkpoint: %s must be F32 with one scale per output row", name);
        /* the mapping is borrowed for the upload only: it has completed when ensure_ready returns, so the caller may
         * close the checkpoint right after this call */
        if (!h3_cuda_w4a8_weight_create_from_i8(d->cuda, (int8_t *)(uintptr_t)w.data, want_n[l], want_k[l],
                                                (float *)(uintptr_t)s.data, &obj, NULL, 1, error, error_size))
            return 0;
        if (!h3_cuda_w4a8_weight_ensure_ready(obj, error, error_size)) {
            h3_cuda_w4a8_weight_free(obj);
            return 0;
        }
        if (!own_weight(d, obj, error, error_size)) return 0;
        if (!h3b_dit_set_linear(d, dst_block, ckpt_slot[l], obj, error, error_size)) return 0;
    }
    return load_block_aux_from_ckpt(d, ckpt, src_block, dst_block, error, error_size);
}

/* The reference's W4A8 checkpoint (h3_w4a8.c:75-115): per linear `weight` I8 [n, k/2] (two codes per byte, low
 * nibble = even k), `weight_codebook` F32[16], `weight_s_rel` F8_E4M3 [n, k/16], `weight_s_channel` F32[n].  Decoded
 * on the device to the resident INT8 form by the reference's own rule (h3_w4a8_dequant.c:65-118). */
int h3b_dit_load_w4a8_block(h3b_dit *d, const h3b_ckpt *ckpt, unsigned src_block, unsigned dst_block, char *error,
                            size_t error_size) {
    char name[256];
    size_t want_n[4], want_k[4];
    int l;
    if (!d || !ckpt || dst_block >= d->cfg.n_blocks) return fail(error, error_size, "load_w4a8_block: invalid arguments");
    if (d->cfg.kind != H3B_BLOCK_REFERENCE)
        return fail(error, error_size, "load_w4a8_block: the W4A8 checkpoint holds the reference block");
    ckpt_linear_shapes(d, want_n, want_k);
    for (l = 0; l < 4; l++) {
        const size_t n = want_n[l], k = want_k[l];
        h3b_ckpt_tensor w, cb, sr, sc;
        h3_cuda_w4a8_weight *obj = NULL;
        if (k % 16) return fail(error, error_size, "load_w4a8_block: K = %zu is not a multiple of the 16-wide scale group", k);
        snprintf(name, sizeof(name), "blocks.%u.%s.weight", src_block, ckpt_suffix[l]);
        if (!h3b_ckpt_find(ckpt, name, &w)) return fail(error, error_size, "checkpoint: tensor %s missing", name);
        if (strcmp(w.dtype, "I8") != 0 || w.rank != 2 || w.shape[0] != n || w.shape[1] != k / 2)
            return fail(error, error_size, "checkpoint: %s is %s rank %d [%zu, %zu], expected packed I8 [%zu, %zu]", name,
                        w.dtype, w.rank, w.shape[0], w.rank > 1 ? w.shape[1] : 0, n, k / 2);
        snprintf(name, sizeof(name), "blocks.%u.%s.weight_codebook", src_block, ckpt_suffix[l]);
        if (!h3b_ckpt_find(ckpt, name, &cb)) return fail(error, error_size, "checkpoint: tensor %s missing", name);
        if (strcmp(cb.dtype, "F32") != 0 || cb.rank != 1 || cb.shape[0] != 16)
            return fail(error, error_size, "checkpoint: %s must be F32[16]", name);
        snprintf(name, sizeof(name), "blocks.%u.%s.weight_s_rel", src_block, ckpt_suffix[l]);
        if (!h3b_ckpt_find(ckpt, name, &sr)) return fail(error, error_size, "checkpoint: tensor %s missing", name);
        if (strcmp(sr.dtype, "F8_E4M3") != 0 || sr.bytes != n * (k / 16))
            return fail(error, error_size, "checkpoint: %s must be F8_E4M3 [%zu, %zu]", name, n, k / 16);
        snprintf(name, sizeof(name), "blocks.%u.%s.weight_s_channel", src_block, ckpt_suffix[l]);
        if (!h3b_ckpt_find(ckpt, name, &sc)) return fail(error, error_size, "checkpoint: tensor %s missing", name);
        if (strcmp(sc.dtype, "F32") != 0 || sc.bytes != n * sizeof(float))
            return fail(error, error_size, "checkpoint: %s must be F32 with one scale per output row", name);
        /* the constructor copies from the mapping and returns with the decode queued behind the copies */
        if (!h3_cuda_w4a8_weight_create(d->cuda, (const int8_t *)w.data, n, k / 2, (const float *)cb.data,
                                        (const uint8_t *)sr.data, (const float *)sc.data, 16, &obj, NULL, NULL, error,
                                        error_size))
            return 0;
        if (!h3_cuda_w4a8_weight_ensure_ready(obj, error, error_size)) {
            h3_cuda_w4a8_weight_free(obj);
            return 0;
        }
        if (!own_weight(d, obj, error, error_size)) return 0;
        if (!h3b_dit_set_linear(d, dst_block, ckpt_slot[l], obj, error, error_size)) return 0;
    }
    return load_block_aux_from_ckpt(d, ckpt, src_block, dst_block, error, error_size);
}

static void *heap_copy(const void *src, size_t bytes) {
    void *p = malloc(bytes ? bytes : 1);
    if (p) memcpy(p, src, bytes);
    return p;
}

/* The reference's NVFP4 sidecar (h3_dit_w4a8.c:3158-3274): per linear `weight_fp4` U8 [n, k/2], `weight_sf` U8 (the
 * 128x4-blocked UE4M3 scales, h3_cuda_nvfp4_sf_bytes(n, k) bytes) and an optional F32 scalar `weight_scale2` (1 when
 * absent).  `linears` is a mask of the linears to take from the sidecar (bit 0 QKV, 1 OUT, 2 FC1, 3 FC2: the
 * reference's per-linear NVFP4 / INT8 choice); a linear that is absent from the file is an error if its bit is set.
 * Norms and the adaLN projection are not part of a sidecar: load them from the checkpoint it accompanies. */
int h3b_dit_load_nvfp4_block(h3b_dit *d, const h3b_ckpt *sidecar, unsigned src_block, unsigned dst_block, unsigned linears,
                             char *error, size_t error_size) {
    char name[256];
    size_t want_n[4], want_k[4];
    int l;
    if (!d || !sidecar || dst_block >= d->cfg.n_blocks || !(linears & 15u))
        return fail(error, error_size, "load_nvfp4_block: invalid arguments");
    ckpt_linear_shapes(d, want_n, want_k);
    for (l = 0; l < 4; l++) {
        const size_t n = want_n[l], k = want_k[l], w_bytes = n * (k / 2), sf_bytes = h3_cuda_nvfp4_sf_bytes(n, k);
        h3b_ckpt_tensor w, sf, s2;
        h3_cuda_nvfp4_weight *obj = NULL;
        uint8_t *codes, *scales;
        float scale2 = 1.0f;
        if (!(linears & (1u << l))) continue;
        snprintf(name, sizeof(name), "blocks.%u.%s.weight_fp4", src_block, ckpt_suffix[l]);
        if (!h3b_ckpt_find(sidecar, name, &w)) return fail(error, error_size, "nvfp4 sidecar: tensor %s missing", name);
        if (w.bytes != w_bytes) return fail(error, error_size, "nvfp4 sidecar %s size mismatch: %zu bytes, expected %zu", name, w.bytes, w_bytes);
        snprintf(name, sizeof(name), "blocks.%u.%s.weight_sf", src_block, ckpt_suffix[l]);
        if (!h3b_ckpt_find(sidecar, name, &sf)) return fail(error, error_size, "nvfp4 sidecar: tensor %s missing", name);
        if (sf.bytes != sf_bytes) return fail(error, error_size, "nvfp4 sidecar %s size mismatch: %zu bytes, expected %zu", name, sf.bytes, sf_bytes);
        snprintf(name, sizeof(name), "blocks.%u.%s.weight_scale2", src_block, ckpt_suffix[l]);
        if (h3b_ckpt_find(sidecar, name, &s2)) {
            if (strcmp(s2.dtype, "F32") != 0 || s2.bytes != sizeof(float))
                return fail(error, error_size, "nvfp4 sidecar: %s must be one F32", name);
            memcpy(&scale2, s2.data, sizeof(float));
        }
        /* the constructor owns its two host buffers once it has succeeded (h3_gpu_cuda.h:437-444): it gets heap copies
         * of the mapped tensors, which are ours again only if it fails */
        codes = (uint8_t *)heap_copy(w.data, w_bytes);
        scales = (uint8_t *)heap_copy(sf.data, sf_bytes);
        if (!codes || !scales ||
            !h3_cuda_nvfp4_weight_create(d->cuda, codes, scales, scale2, n, k, &obj, NULL, error, error_size)) {
            const int oom = !codes || !scales;
            free(codes);
            free(scales);
            return oom ? fail(error, error_size, "load_nvfp4_block: out of host memory") : 0;
        }
        if (d->n_owned_fp4 == d->cap_owned_fp4) {
            size_t ncap = d->cap_owned_fp4 ? 2 * d->cap_owned_fp4 : 16;
            h3_cuda_nvfp4_weight **no = (h3_cuda_nvfp4_weight **)realloc(d->owned_fp4, ncap * sizeof(*no));
            if (!no) {
                h3_cuda_nvfp4_weight_free(d->cuda, obj);
                return fail(error, error_size, "load_nvfp4_block: out of host memory");
            }
            d->owned_fp4 = no;
            d->cap_owned_fp4 = ncap;
        }
        d->owned_fp4[d->n_owned_fp4++] = obj;
        if (!h3b_dit_set_linear_nvfp4(d, dst_block, ckpt_slot[l], obj, error, error_size)) return 0;
    }
    return 1;
}

int h3b_dit_project_modulation(h3b_dit *d, const float *d_t_feat, char *error, size_t error_size) {
    size_t b;
    if (!d || !d_t_feat) return fail(error, error_size, "h3b_dit_project_modulation: invalid arguments");
    for (b = 0; b < d->cfg.n_blocks; b++) {
        h3b_block *k = &d->blocks[b];
        if (!k->adaln_w) return fail(error, error_size, "block %zu has no adaLN projection", b);
        if (!h3b_adaln_project_dev(d->cuda, k->adaln_w, k->adaln_b, mod_elems(d), d->cfg.t_dim, d_t_feat, k->modulation,
                                   error, error_size))
            return 0;
    }
    return 1;
}

const float *h3b_dit_modulation(h3b_dit *d, unsigned block) {
    if (!d || block >= d->cfg.n_blocks) return NULL;
    return d->blocks[block].modulation;
}

int h3b_dit_reserve(h3b_dit *d, size_t seq, size_t text_seq, char *error, size_t error_size) {
    size_t D, I, F, widest, es, table_rows;
    const int cross = d && d->cfg.kind == H3B_BLOCK_CROSS_GELU;
    int grow_seq, grow_text;
    if (!d || !seq) return fail(error, error_size, "h3b_dit_reserve: invalid arguments");
    grow_seq = seq > d->cap_seq;
    grow_text = cross && (text_seq > d->cap_text || !d->ckv);
    if (!grow_seq && !grow_text) return 1;
    if (h3_cuda_graph_capture(d->cuda)) return fail(error, error_size, "workspace growth is forbidden during graph capture");
    cudaStreamSynchronize((cudaStream_t)h3_cuda_op_stream(d->cuda));
    D = d->cfg.dim; I = inner(d); F = d->cfg.ffn; es = elem(d);
    if (grow_seq) {
        /* only the group that is too small is released and allocated again, at the size asked for */
        free_seq_ws(d);
        table_rows = seq * (size_t)((d->uly && d->uly->comm) ? d->uly->ulysses : 1);
        widest = D > F ? D : F;
        if (I > widest) widest = I;
        if (!dmalloc(&d->xa, seq * D * es, error, error_size) || !dmalloc(&d->xb, seq * D * es, error, error_size) ||
            !dmalloc(&d->io, seq * D * es, error, error_size) ||
            !dmalloc(&d->qkv, seq * 3 * I * es, error, error_size) || !dmalloc(&d->wide, seq * F * es, error, error_size) ||
            !dmalloc(&d->q, seq * I * 2, error, error_size) || !dmalloc(&d->k, seq * I * 2, error, error_size) ||
            !dmalloc(&d->v, seq * I * 2, error, error_size) || !dmalloc(&d->att, seq * I * 2, error, error_size) ||
            !dmalloc((void **)&d->q8, seq * widest, error, error_size) ||
            !dmalloc((void **)&d->s8, seq * sizeof(float), error, error_size) ||
            !dmalloc((void **)&d->st_x, seq * D * sizeof(float), error, error_size) ||
            !dmalloc((void **)&d->st_map, seq * sizeof(uint32_t), error, error_size) ||
            !dmalloc((void **)&d->st_cos, table_rows * (d->cfg.rope_half ? d->cfg.rope_half : 1) * sizeof(float), error, error_size) ||
            !dmalloc((void **)&d->st_sin, table_rows * (d->cfg.rope_half ? d->cfg.rope_half : 1) * sizeof(float), error, error_size) ||
            !dmalloc((void **)&d->st_t, (d->cfg.t_dim ? d->cfg.t_dim : 1) * sizeof(float), error, error_size) ||
            (cross && !dmalloc(&d->cq, seq * I * 2, error, error_size)) ||
            (d->any_fp4 && (!dmalloc((void **)&d->rotf, seq * widest * sizeof(float), error, error_size) ||
                            !dmalloc((void **)&d->x4, seq * widest / 2, error, error_size) ||
                            !dmalloc((void **)&d->sfx, ((seq + 127) / 128) * ((widest + 63) / 64) * 512, error, error_size)))) {
            free_seq_ws(d);   /* a half-built group must not pass for capacity */
            return 0;
        }
        d->cap_seq = seq;
    }
    if (grow_text) {
        size_t t = text_seq ? text_seq : 1;
        free_text_ws(d);
        if (!dmalloc(&d->ckv, t * 2 * I * 2, error, error_size) || !dmalloc((void **)&d->tq8, t * D, error, error_size) ||
            !dmalloc((void **)&d->ts8, t * sizeof(float), error, error_size) ||
            !dmalloc((void **)&d->st_text, t * D * sizeof(float), error, error_size) ||
            !dmalloc(&d->text_dev, t * D * es, error, error_size)) {
            free_text_ws(d);
            return 0;
        }
        d->cap_text = text_seq;
    }
    return 1;
}

int h3b_dit_launches_per_block(const h3b_dit *d) {
    if (!d) return 0;
    /* the QKV projection carries the QK-norm and RoPE in its epilogue */
    return d->cfg.kind == H3B_BLOCK_REFERENCE ? 9 : 16;
}

/* rows -> (gate) -> norm -> (modulate) -> (rotate) -> int8 codes in d->q8 / d->s8 */
static int norm_quant(h3b_dit *d, const void *x, int dtype, size_t rows, size_t width, const float *norm_w,
                      const float *mod, const uint32_t *row_map, size_t shift_slot, size_t scale_slot, int identity,
                      int8_t *q, float *s, char *error, size_t error_size) {
    h3b_norm_args a;
    memset(&a, 0, sizeof(a));
    a.d_x = x; a.d_norm_w = norm_w; a.d_modulation = mod; a.d_row_map = row_map; a.rows = rows; a.width = width;
    a.slots = 6; a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = d->cfg.eps; a.dtype = dtype;
    a.identity = identity; a.convrot_gs = d->cfg.convrot_gs; a.d_q = q; a.d_scales = s;
    return h3b_norm_dev(d->cuda, &a, error, error_size);
}

static int gemm(h3b_dit *d, const h3_cuda_w4a8_weight *w, const int8_t *q, const float *s, size_t m, void *y, int kind,
                int out_dtype, const void *residual, const float *mod, const uint32_t *row_map, size_t gate_slot,
                char *error, size_t error_size) {
    h3b_gemm_epi e;
    memset(&e, 0, sizeof(e));
    e.kind = kind; e.out_dtype = out_dtype; e.d_residual = residual; e.d_modulation = mod; e.d_row_map = row_map;
    e.slots = 6; e.gate_slot = gate_slot;
    return h3b_gemm_i8_dev(d->cuda, w, q, s, m, y, &e, error, error_size);
}

/* One NVFP4 linear of the reference block: rows of `x` (dtype `dt`) -> optional RMSNorm + modulation -> ConvRot -> f32
 * in d->rotf -> the reference-named f32 entry point with the epilogue `epi` (0 plain, 1 SwiGLU, 2 gate). */
static int fp4_linear(h3b_dit *d, const h3_cuda_nvfp4_weight *w, const void *x, int dt, size_t rows, size_t width,
                      const float *norm_w, const float *mod, const uint32_t *row_map, size_t shift_slot,
                      size_t scale_slot, int identity, int epi, const float *residual, size_t gate_slot, float *y,
                      char *error, size_t error_size) {
    const float *x_use;
    if (!d->rotf) return fail(error, error_size, "NVFP4 linear: workspace not reserved");
    if (width % 64 == 0 && (epi != 1 || (h3_cuda_nvfp4_weight_n(w) % 256 == 0 && h3_plugin_enabled("H3B_FP4_WIDE")))) {
        /* one pass over the rows: (RMSNorm, modulation,) ConvRot and the NVFP4 quantisation in the row kernel, then the
         * block-scaled GEMM on the codes */
        h3b_norm_args a;
        memset(&a, 0, sizeof(a));
        a.d_x = x; a.d_norm_w = norm_w; a.d_modulation = identity ? NULL : mod; a.d_row_map = row_map; a.rows = rows;
        a.width = width; a.slots = 6; a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = d->cfg.eps;
        a.dtype = dt; a.identity = identity; a.convrot_gs = d->cfg.convrot_gs; a.d_fp4 = d->x4; a.d_sf = d->sfx;
        if (!h3b_norm_dev(d->cuda, &a, error, error_size)) return 0;
        return h3b_gemm_fp4_w_preq_dev(d->cuda, w, d->x4, d->sfx, rows, 1.0f, epi, residual, mod, row_map, 6, gate_slot, y,
                                       H3B_F32, error, error_size);
    }
    if (d->cfg.convrot_gs > 0 || !identity) {
        h3b_norm_args a;
        memset(&a, 0, sizeof(a));
        a.d_x = x; a.d_norm_w = norm_w; a.d_modulation = mod; a.d_row_map = row_map; a.rows = rows; a.width = width;
        a.slots = 6; a.shift_slot = shift_slot; a.scale_slot = scale_slot; a.epsilon = d->cfg.eps; a.dtype = dt;
        a.identity = identity; a.convrot_gs = d->cfg.convrot_gs;
        if (d->cfg.convrot_gs > 0) a.d_rot = d->rotf;
        else if (dt == H3B_F32) a.d_normed = d->rotf;
        else return fail(error, error_size, "NVFP4 linear: normalised rows without ConvRot need an f32 input");
        if (!h3b_norm_dev(d->cuda, &a, error, error_size)) return 0;
        x_use = d->rotf;
    } else if (dt == H3B_F32) {
        x_use = (const float *)x;
    } else {
        if (!h3b_cast_dev(d->cuda, x, dt, d->rotf, H3B_F32, rows * width, error, error_size)) return 0;
        x_use = d->rotf;
    }
    if (epi == 1)
        return h3_cuda_gemm_fp4_w_act_dev_swiglu(d->cuda, w, x_use, 1.0f, rows, NULL, y, NULL, NULL, NULL, error, error_size,
                                                 NULL);
    if (epi == 2)
        return h3_cuda_gemm_fp4_w_act_dev_gate(d->cuda, w, x_use, 1.0f, rows, residual, mod, row_map, 6, gate_slot, NULL, y,
                                               NULL, NULL, NULL, error, error_size, NULL);
    return h3_cuda_gemm_fp4_w_act_dev(d->cuda, w, x_use, 1.0f, rows, y, NULL, NULL, NULL, error, error_size, NULL);
}

static int block_forward(h3b_dit *d, unsigned block, const void *d_x, size_t seq, size_t seq_real,
                         const float *d_modulation, const uint32_t *d_row_map, const float *d_cos, const float *d_sin,
                         const void *d_text, size_t text_seq, void *d_y, char *error, size_t error_size) {
    const h3b_block *b;
    const float *mod;
    size_t D, I, F;
    int dt, i;
    float scale;
    const void *att_src;   /* bf16 [seq, inner] attention output that feeds the out projection */
    if (!d || block >= d->cfg.n_blocks || !d_x || !d_y || !seq)
        return fail(error, error_size, "block forward: invalid arguments");
    b = &d->blocks[block];
    mod = d_modulation ? d_modulation : b->modulation;
    if (!mod) return fail(error, error_size, "block %u: no modulation given or projected", block);
    if (!b->norm1) return fail(error, error_size, "block %u: aux tensors not set", block);
    for (i = 0; i < (d->cfg.kind == H3B_BLOCK_CROSS_GELU ? H3B_LIN_COUNT : 4); i++)
        if (!b->lin[i] && !(i < 4 && b->fp4[i])) return fail(error, error_size, "block %u: linear %d not set", block, i);
    if (d->cfg.rope_half && (!d_cos || !d_sin)) return fail(error, error_size, "block %u: rope tables missing", block);
    if (d->cfg.kind == H3B_BLOCK_CROSS_GELU && (!d_text || !text_seq))
        return fail(error, error_size, "block %u: text tokens missing", block);
    if (!h3b_dit_reserve(d, seq, text_seq, error, error_size)) return 0;
    D = d->cfg.dim; I = inner(d); F = d->cfg.ffn; dt = d->cfg.stream_dtype;
    scale = 1.0f / 11.313708498984761f; /* 1/sqrt(128) */
    att_src = d->att;

    /* ---- self-attention: adaLN(0,1) -> QKV -> QK-norm + RoPE -> SDPA -> out * gate(2) + x */
    if (!b->fp4[H3B_LIN_QKV] &&
        !norm_quant(d, d_x, dt, seq, D, b->norm1, mod, d_row_map, 0, 1, 0, d->q8, d->s8, error, error_size))
        return 0;
    if (!d->uly || !d->uly->comm) {
        /* QKV projection with the QK-norm and RoPE applied in the GEMM epilogue: Q, K, V leave the kernel
         * as bf16 [seq, heads, 128]; the [seq, 3*inner] intermediate is never written */
        if (b->fp4[H3B_LIN_QKV] && D % 64 == 0 && d->cfg.head_dim == 128 && dt == H3B_F32 &&
            (d->cfg.rope_half == 0 || d->cfg.rope_half == 48 || d->cfg.rope_half == 64) && 3 * I >= 256 &&
            h3_plugin_enabled("H3B_FP4_WIDE") && h3_plugin_enabled("H3B_FP4_QKV_ROPE")) {
            /* the same for an NVFP4 projection: adaLN, ConvRot and the NVFP4 quantisation in the row kernel, QK-norm and
             * RoPE on the f32 accumulators in the GEMM epilogue (H3B_FP4_QKV_ROPE=0 keeps the two stand-alone steps) */
            h3b_norm_args a;
            memset(&a, 0, sizeof(a));
            a.d_x = d_x; a.d_norm_w = b->norm1; a.d_modulation = mod; a.d_row_map = d_row_map; a.rows = seq; a.width = D;
            a.slots = 6; a.shift_slot = 0; a.scale_slot = 1; a.epsilon = d->cfg.eps; a.dtype = dt;
            a.convrot_gs = d->cfg.convrot_gs; a.d_fp4 = d->x4; a.d_sf = d->sfx;
            if (!h3b_norm_dev(d->cuda, &a, error, error_size) ||
                !h3b_gemm_fp4_w_preq_qkv_rope_dev(d->cuda, b->fp4[H3B_LIN_QKV], d->x4, d->sfx, seq, 1.0f, b->q_norm, b->k_norm,
                                                  d_cos, d_sin, d->cfg.rope_half, d->cfg.heads, d->cfg.eps, d->q, d->k, d->v,
                                                  error, error_size))
                return 0;
        } else if (b->fp4[H3B_LIN_QKV]) {
            if (!fp4_linear(d, b->fp4[H3B_LIN_QKV], d_x, dt, seq, D, b->norm1, mod, d_row_map, 0, 1, 0, 0, NULL, 0,
                            (float *)d->qkv, error, error_size) ||
                !h3b_qkv_rope_dev(d->cuda, d->qkv, dt, b->q_norm, b->k_norm, d_cos, d_sin, seq, d->cfg.heads,
                                  d->cfg.head_dim, d->cfg.rope_half, d->cfg.eps, 0, 1, d->q, d->k, d->v, H3B_BF16, error,
                                  error_size))
                return 0;
        } else if (d->cfg.rope_half == 0 || d->cfg.rope_half == 48 || d->cfg.rope_half == 64) {
            h3b_gemm_epi e;
            memset(&e, 0, sizeof(e));
            e.kind = H3B_EPI_QKV_ROPE; e.out_dtype = H3B_BF16; e.d_key = d->k; e.d_value = d->v;
            e.d_q_norm = b->q_norm; e.d_k_norm = b->k_norm; e.d_rope_cos = d_cos; e.d_rope_sin = d_sin;
            e.rope_half = d->cfg.rope_half; e.epsilon = d->cfg.eps; e.round_qkv = dt != H3B_F32;
            if (!h3b_gemm_i8_dev(d->cuda, b->lin[H3B_LIN_QKV], d->q8, d->s8, seq, d->q, &e, error, error_size)) return 0;
        } else {
            if (!gemm(d, b->lin[H3B_LIN_QKV], d->q8, d->s8, seq, d->qkv, H3B_EPI_PLAIN, dt, NULL, NULL, NULL, 0, error,
                      error_size))
                return 0;
            if (!h3b_qkv_rope_dev(d->cuda, d->qkv, dt, b->q_norm, b->k_norm, d_cos, d_sin, seq, d->cfg.heads,
                                  d->cfg.head_dim, d->cfg.rope_half, d->cfg.eps, 0, 1, d->q, d->k, d->v, H3B_BF16, error,
                                  error_size))
                return 0;
        }
        if (!h3b_sdpa_bf16_dev(d->cuda, d->q, I, d->k, I, d->v, I, seq, seq, d->cfg.heads, d->cfg.head_dim, scale,
                               d->att, I, error, error_size))
            return 0;
    } else {
        /* Ulysses: rows are this rank's slice.  Exchange sequence for heads, attend over the whole
         * (real) sequence with heads/U heads, exchange back.  Both exchanges run in place. */
        const size_t U = (size_t)d->uly->ulysses, hl = d->cfg.heads / U, seq_pad = seq * U, Il = hl * d->cfg.head_dim;
        const size_t es = dt == H3B_F32 ? 4 : 2;
        const h3b_ulysses_direct *dir = h3b_ulysses_direct_get(d->uly);
        if (dir && dir->seq_local == seq && dir->heads == d->cfg.heads && dir->head_dim == d->cfg.head_dim &&
            d->cfg.head_dim == 128 && dt != H3B_F32 && !b->fp4[H3B_LIN_QKV] &&
            (d->cfg.rope_half == 0 || d->cfg.rope_half == 48 || d->cfg.rope_half == 64)) {
            /* Exchange-free form: the QKV epilogue (QK-norm and RoPE included: both are per row and head) stores
             * every head slice into the gathered buffer of the rank that attends that head, the attention
             * epilogue stores every output row into the buffer of the rank that owns the row.  A barrier
             * after each makes the stores of all ranks visible before they are read; it also keeps a rank
             * from overwriting a buffer that a slower rank still reads. */
            h3b_gemm_epi e;
            const size_t off = (size_t)dir->rank * seq * d->cfg.rope_half;   /* this rank's rows of the tables */
            memset(&e, 0, sizeof(e));
            e.kind = H3B_EPI_QKV_ROPE; e.out_dtype = H3B_BF16; e.scatter = dir;
            e.d_q_norm = b->q_norm; e.d_k_norm = b->k_norm;
            e.d_rope_cos = d->cfg.rope_half ? d_cos + off : NULL; e.d_rope_sin = d->cfg.rope_half ? d_sin + off : NULL;
            e.rope_half = d->cfg.rope_half; e.epsilon = d->cfg.eps; e.round_qkv = 1;
            if (!h3b_gemm_i8_dev(d->cuda, b->lin[H3B_LIN_QKV], d->q8, d->s8, seq, NULL, &e, error, error_size)) return 0;
            if (!h3b_ulysses_barrier(d->uly, error, error_size)) return 0;
            if (!h3b_sdpa_bf16_scatter_dev(d->cuda, dir, seq_real, scale, error, error_size)) return 0;
            if (!h3b_ulysses_barrier(d->uly, error, error_size)) return 0;
            att_src = dir->att;
            goto attention_done;
        }
        if (b->fp4[H3B_LIN_QKV]) {
            if (!fp4_linear(d, b->fp4[H3B_LIN_QKV], d_x, dt, seq, D, b->norm1, mod, d_row_map, 0, 1, 0, 0, NULL, 0,
                            (float *)d->qkv, error, error_size))
                return 0;
        } else if (!gemm(d, b->lin[H3B_LIN_QKV], d->q8, d->s8, seq, d->qkv, H3B_EPI_PLAIN, dt, NULL, NULL, NULL, 0, error,
                         error_size))
            return 0;
        if (!h3_ulysses_a2a_qkv(d->uly, d->qkv, d->qkv, seq, d->cfg.heads, d->cfg.head_dim, (int)es, error, error_size))
            return 0;
        if (!h3b_qkv_rope_dev(d->cuda, d->qkv, dt, b->q_norm, b->k_norm, d_cos, d_sin, seq_pad, hl, d->cfg.head_dim,
                              d->cfg.rope_half, d->cfg.eps, 0, 1, d->q, d->k, d->v, H3B_BF16, error, error_size))
            return 0;
        if (!h3b_sdpa_bf16_dev(d->cuda, d->q, Il, d->k, Il, d->v, Il, seq_real, seq_real, hl, d->cfg.head_dim, scale,
                               d->att, Il, error, error_size))
            return 0;
        if (seq_pad > seq_real &&
            cudaMemsetAsync((char *)d->att + seq_real * Il * 2, 0, (seq_pad - seq_real) * Il * 2,
                            (cudaStream_t)h3_cuda_op_stream(d->cuda)) != cudaSuccess)
            return fail(error, error_size, "block %u: clearing pad rows failed", block);
        if (!h3_ulysses_a2a_attn_out(d->uly, d->att, d->att, seq, d->cfg.heads, d->cfg.head_dim, 2, error, error_size))
            return 0;
    }
attention_done:
    /* x1 -> xa */
    if (b->fp4[H3B_LIN_OUT]) {
        if (!fp4_linear(d, b->fp4[H3B_LIN_OUT], att_src, H3B_BF16, seq, I, NULL, mod, d_row_map, 0, 0, 1, 2, (const float *)d_x,
                        2, (float *)d->xa, error, error_size))
            return 0;
    } else if (!norm_quant(d, att_src, H3B_BF16, seq, I, NULL, NULL, NULL, 0, 0, 1, d->q8, d->s8, error, error_size) ||
               !gemm(d, b->lin[H3B_LIN_OUT], d->q8, d->s8, seq, d->xa, H3B_EPI_GATE, dt, d_x, mod, d_row_map, 2, error,
                     error_size))
        return 0;

    if (d->cfg.kind == H3B_BLOCK_REFERENCE) {
        /* ---- MLP: adaLN(3,4) -> fc1 + SwiGLU -> fc2 * gate(5) + x1 */
        if (b->fp4[H3B_LIN_FC1]) {
            if (!fp4_linear(d, b->fp4[H3B_LIN_FC1], d->xa, dt, seq, D, b->norm2, mod, d_row_map, 3, 4, 0, 1, NULL, 0,
                            (float *)d->wide, error, error_size))
                return 0;
        } else if (!norm_quant(d, d->xa, dt, seq, D, b->norm2, mod, d_row_map, 3, 4, 0, d->q8, d->s8, error, error_size) ||
                   !gemm(d, b->lin[H3B_LIN_FC1], d->q8, d->s8, seq, d->wide, H3B_EPI_SWIGLU, dt, NULL, NULL, NULL, 0, error,
                         error_size))
            return 0;
        if (b->fp4[H3B_LIN_FC2])
            return fp4_linear(d, b->fp4[H3B_LIN_FC2], d->wide, dt, seq, F, NULL, mod, d_row_map, 0, 0, 1, 2,
                              (const float *)d->xa, 5, (float *)d_y, error, error_size);
        if (!norm_quant(d, d->wide, dt, seq, F, NULL, NULL, NULL, 0, 0, 1, d->q8, d->s8, error, error_size)) return 0;
        return gemm(d, b->lin[H3B_LIN_FC2], d->q8, d->s8, seq, d_y, H3B_EPI_GATE, dt, d->xa, mod, d_row_map, 5, error,
                    error_size);
    }

    /* ---- cross-attention: rms_norm -> q proj; text -> kv proj; SDPA(lq=seq, lk=text) -> out + x1 (no gate) */
    if (!norm_quant(d, d->xa, dt, seq, D, b->norm_cross, NULL, NULL, 0, 0, 0, d->q8, d->s8, error, error_size)) return 0;
    if (!gemm(d, b->lin[H3B_LIN_CROSS_Q], d->q8, d->s8, seq, d->cq, H3B_EPI_PLAIN, H3B_BF16, NULL, NULL, NULL, 0, error,
              error_size))
        return 0;
    if (!norm_quant(d, d_text, dt, text_seq, D, NULL, NULL, NULL, 0, 0, 1, d->tq8, d->ts8, error, error_size)) return 0;
    if (!gemm(d, b->lin[H3B_LIN_CROSS_KV], d->tq8, d->ts8, text_seq, d->ckv, H3B_EPI_PLAIN, H3B_BF16, NULL, NULL, NULL, 0,
              error, error_size))
        return 0;
    if (!h3b_sdpa_bf16_dev(d->cuda, d->cq, I, d->ckv, 2 * I, (const char *)d->ckv + I * 2, 2 * I, seq, text_seq,
                           d->cfg.heads, d->cfg.head_dim, scale, d->att, I, error, error_size))
        return 0;
    if (!norm_quant(d, d->att, H3B_BF16, seq, I, NULL, NULL, NULL, 0, 0, 1, d->q8, d->s8, error, error_size)) return 0;
    /* x2 -> xb */
    if (!gemm(d, b->lin[H3B_LIN_CROSS_OUT], d->q8, d->s8, seq, d->xb, H3B_EPI_GATE, dt, d->xa, NULL, NULL, 0, error,
              error_size))
        return 0;

    /* ---- FFN: adaLN(3,4) -> up + tanh-GELU -> down * gate(5) + x2 */
    if (!norm_quant(d, d->xb, dt, seq, D, b->norm2, mod, d_row_map, 3, 4, 0, d->q8, d->s8, error, error_size)) return 0;
    if (!gemm(d, b->lin[H3B_LIN_FC1], d->q8, d->s8, seq, d->wide, H3B_EPI_GELU, dt, NULL, NULL, NULL, 0, error, error_size))
        return 0;
    if (!norm_quant(d, d->wide, dt, seq, F, NULL, NULL, NULL, 0, 0, 1, d->q8, d->s8, error, error_size)) return 0;
    return gemm(d, b->lin[H3B_LIN_FC2], d->q8, d->s8, seq, d_y, H3B_EPI_GATE, dt, d->xb, mod, d_row_map, 5, error,
                error_size);
}

int h3b_dit_block_forward_dev(h3b_dit *d, unsigned block, const void *d_x, size_t seq, const float *d_modulation,
                              const uint32_t *d_row_map, const float *d_cos, const float *d_sin, const void *d_text,
                              size_t text_seq, void *d_y, char *error, size_t error_size) {
    if (d && d->uly && d->uly->comm)
        return fail(error, error_size, "block_forward_dev: a Ulysses communicator is attached; use the ulysses chain");
    return block_forward(d, block, d_x, seq, seq, d_modulation, d_row_map, d_cos, d_sin, d_text, text_seq, d_y, error,
                         error_size);
}

int h3b_dit_set_ulysses(h3b_dit *d, h3_ulysses_cfg *cfg, char *error, size_t error_size) {
    if (!d) return fail(error, error_size, "h3b_dit_set_ulysses: NULL context");
    if (cfg && cfg->comm) {
        if (!h3_ulysses_validate((int)d->cfg.heads, H3_ULYSSES_PACKED_ALIGN, 1, cfg->ulysses, 1, error, error_size)) return 0;
        if (!h3_ulysses_comm_set_compute(cfg, cfg->rank, h3_cuda_op_stream(d->cuda), error, error_size)) return 0;
    }
    if (d->uly != cfg) {
        /* staging tables are sized for the gathered sequence: start from an empty workspace */
        cudaStreamSynchronize((cudaStream_t)h3_cuda_op_stream(d->cuda));
        free_ws(d);
    }
    d->uly = cfg;
    return 1;
}

int h3b_dit_layers_forward_ulysses_dev(h3b_dit *d, unsigned first, unsigned n, const void *d_x, size_t seq_local,
                                       size_t seq_real, const uint32_t *d_row_map, const float *d_cos_full,
                                       const float *d_sin_full, const void *d_text, size_t text_seq, void *d_y,
                                       char *error, size_t error_size) {
    unsigned i;
    const void *cur = d_x;
    if (!d || !n || first + n > d->cfg.n_blocks) return fail(error, error_size, "layers_forward_ulysses: bad block range");
    if (!d->uly || !d->uly->comm) return fail(error, error_size, "layers_forward_ulysses: no communicator attached");
    if (!seq_real || seq_real > seq_local * (size_t)d->uly->ulysses)
        return fail(error, error_size, "layers_forward_ulysses: seq_real must be in (0, U*seq_local]");
    for (i = 0; i < n; i++) {
        if (!block_forward(d, first + i, cur, seq_local, seq_real, NULL, d_row_map, d_cos_full, d_sin_full, d_text,
                           text_seq, d_y, error, error_size))
            return 0;
        cur = d_y;
    }
    return 1;
}

int h3b_dit_layers_forward_dev(h3b_dit *d, unsigned first, unsigned n, const void *d_x, size_t seq,
                               const uint32_t *d_row_map, const float *d_cos, const float *d_sin, const void *d_text,
                               size_t text_seq, void *d_y, char *error, size_t error_size) {
    unsigned i;
    const void *cur = d_x;
    if (!d || !n || first + n > d->cfg.n_blocks) return fail(error, error_size, "layers_forward: bad block range");
    /* every block writes its result to d_y; inside a block the input is last read by the
     * out-projection epilogue, before anything is written to d_y, so in-place chaining is safe */
    if (d->uly && d->uly->comm) return fail(error, error_size, "layers_forward: a Ulysses communicator is attached");
    for (i = 0; i < n; i++) {
        if (!block_forward(d, first + i, cur, seq, seq, NULL, d_row_map, d_cos, d_sin, d_text, text_seq, d_y, error,
                           error_size))
            return 0;
        cur = d_y;
    }
    return 1;
}

/* The block chain as ONE CUDA graph launch (the reference captures its step the same way,
 * h3_dit_w4a8.c:4390 run_all_blocks_device under H3_DIT_W4A8_CUDA_GRAPH).  The first call for a set of arguments
 * runs the chain once eagerly (every kernel gets loaded, the workspace gets its size), then captures the same
 * launches on the handle's stream and instantiates the graph; later calls with the SAME arguments only replay it.
 * Different arguments re-capture.  The chain reads the projected modulation through pointers that stay fixed, so
 * h3b_dit_project_modulation between replays is honoured. */
int h3b_dit_layers_forward_graph_dev(h3b_dit *d, unsigned first, unsigned n, const void *d_x, size_t seq,
                                     const uint32_t *d_row_map, const float *d_cos, const float *d_sin, const void *d_text,
                                     size_t text_seq, void *d_y, char *error, size_t error_size) {
    cudaStream_t st;
    cudaError_t e;
    int ok;
    if (!d || !n || first + n > d->cfg.n_blocks) return fail(error, error_size, "layers_forward_graph: bad block range");
    if (d->uly && d->uly->comm) return fail(error, error_size, "layers_forward_graph: a Ulysses communicator is attached");
    st = (cudaStream_t)h3_cuda_op_stream(d->cuda);
    if (!st) return fail(error, error_size, "layers_forward_graph: set an op stream first (the legacy default stream cannot be captured)");
    if (d->graph_exec && d->graph_key.first == first && d->graph_key.n == n && d->graph_key.x == d_x && d->graph_key.seq == seq &&
        d->graph_key.row_map == d_row_map && d->graph_key.cos == d_cos && d->graph_key.sin == d_sin &&
        d->graph_key.text == d_text && d->graph_key.text_seq == text_seq && d->graph_key.y == d_y) {
        e = cudaGraphLaunch(d->graph_exec, st);
        if (e != cudaSuccess) return fail(error, error_size, "cudaGraphLaunch: %s", cudaGetErrorString(e));
        return 1;
    }
    drop_graph(d);
    /* eager pass: loads the kernels, sizes the workspace, produces this call's result */
    if (!h3b_dit_layers_forward_dev(d, first, n, d_x, seq, d_row_map, d_cos, d_sin, d_text, text_seq, d_y, error, error_size)) return 0;
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(error, error_size, "layers_forward_graph: %s", cudaGetErrorString(e));
    e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) return fail(error, error_size, "cudaStreamBeginCapture: %s", cudaGetErrorString(e));
    h3_cuda_set_graph_capture(d->cuda, 1);   /* growth of scratch and event timing are off while capturing */
    ok = h3b_dit_layers_forward_dev(d, first, n, d_x, seq, d_row_map, d_cos, d_sin, d_text, text_seq, d_y, error, error_size);
    h3_cuda_set_graph_capture(d->cuda, 0);
    e = cudaStreamEndCapture(st, &d->graph);
    if (!ok || e != cudaSuccess || !d->graph) {
        drop_graph(d);
        if (ok) fail(error, error_size, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
        return 0;
    }
    e = cudaGraphInstantiate(&d->graph_exec, d->graph, 0);
    if (e != cudaSuccess) {
        drop_graph(d);
        return fail(error, error_size, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
    d->graph_key.first = first; d->graph_key.n = n; d->graph_key.x = d_x; d->graph_key.seq = seq;
    d->graph_key.row_map = d_row_map; d->graph_key.cos = d_cos; d->graph_key.sin = d_sin; d->graph_key.text = d_text;
    d->graph_key.text_seq = text_seq; d->graph_key.y = d_y;
    return 1;
}

/* Kernel nodes of the captured chain (0 when nothing is captured). */
size_t h3b_dit_graph_nodes(const h3b_dit *d) {
    size_t nodes = 0;
    if (!d || !d->graph || cudaGraphGetNodes(d->graph, NULL, &nodes) != cudaSuccess) return 0;
    return nodes;
}

static int layers_forward_host(h3b_dit *d, unsigned first, unsigned n, const float *t_feat, const float *x, size_t seq,
                               size_t seq_real, const uint32_t *row_map, const float *rope_cos, const float *rope_sin,
                               const float *text, size_t text_seq, float *y, char *error, size_t error_size) {
    cudaStream_t st;
    size_t D, rh, table_rows;
    const int uly = seq_real != 0;
    void *dx;
    const void *dtext = NULL;
    cudaError_t e;
    if (!d || !x || !y || !seq || !t_feat) return fail(error, error_size, "layers_forward_f32: invalid arguments");
    if (uly && (!d->uly || !d->uly->comm)) return fail(error, error_size, "layers_forward_ulysses_f32: no communicator attached");
    if (!h3b_dit_reserve(d, seq, text_seq, error, error_size)) return 0;
    table_rows = uly ? seq * (size_t)d->uly->ulysses : seq;
    st = (cudaStream_t)h3_cuda_op_stream(d->cuda);
    D = d->cfg.dim; rh = d->cfg.rope_half;
    /* every staging copy is checked: a failed copy would otherwise run the chain on stale inputs */
#define H3B_STAGE(call, what)                                                                              \
    do {                                                                                                   \
        e = (call);                                                                                        \
        if (e != cudaSuccess) return fail(error, error_size, "layers_forward_f32: %s: %s", what, cudaGetErrorString(e)); \
    } while (0)
    H3B_STAGE(cudaMemcpyAsync(d->st_x, x, seq * D * sizeof(float), cudaMemcpyHostToDevice, st), "H2D(x)");
    H3B_STAGE(cudaMemcpyAsync(d->st_t, t_feat, d->cfg.t_dim * sizeof(float), cudaMemcpyHostToDevice, st), "H2D(t_feat)");
    if (row_map) H3B_STAGE(cudaMemcpyAsync(d->st_map, row_map, seq * sizeof(uint32_t), cudaMemcpyHostToDevice, st), "H2D(row_map)");
    else H3B_STAGE(cudaMemsetAsync(d->st_map, 0, seq * sizeof(uint32_t), st), "memset(row_map)");
    if (rh) {
        if (!rope_cos || !rope_sin) return fail(error, error_size, "layers_forward_f32: rope tables missing");
        H3B_STAGE(cudaMemcpyAsync(d->st_cos, rope_cos, table_rows * rh * sizeof(float), cudaMemcpyHostToDevice, st), "H2D(rope_cos)");
        H3B_STAGE(cudaMemcpyAsync(d->st_sin, rope_sin, table_rows * rh * sizeof(float), cudaMemcpyHostToDevice, st), "H2D(rope_sin)");
    }
    if (d->cfg.kind == H3B_BLOCK_CROSS_GELU) {
        if (!text || !text_seq) return fail(error, error_size, "layers_forward_f32: text tokens missing");
        H3B_STAGE(cudaMemcpyAsync(d->st_text, text, text_seq * D * sizeof(float), cudaMemcpyHostToDevice, st), "H2D(text)");
#undef H3B_STAGE
        if (d->cfg.stream_dtype == H3B_F32) {
            dtext = d->st_text;
        } else {
            if (!h3b_cast_dev(d->cuda, d->st_text, H3B_F32, d->text_dev, d->cfg.stream_dtype, text_seq * D, error, error_size))
                return 0;
            dtext = d->text_dev;
        }
    }
    if (!h3b_dit_project_modulation(d, d->st_t, error, error_size)) return 0;
    if (d->cfg.stream_dtype == H3B_F32) {
        dx = d->st_x;
    } else {
        if (!h3b_cast_dev(d->cuda, d->st_x, H3B_F32, d->io, d->cfg.stream_dtype, seq * D, error, error_size)) return 0;
        dx = d->io;
    }
    if (uly) {
        if (!h3b_dit_layers_forward_ulysses_dev(d, first, n, dx, seq, seq_real, d->st_map, d->st_cos, d->st_sin, dtext,
                                                text_seq, dx, error, error_size))
            return 0;
    } else if (!h3b_dit_layers_forward_dev(d, first, n, dx, seq, d->st_map, d->st_cos, d->st_sin, dtext, text_seq, dx,
                                           error, error_size)) {
        return 0;
    }
    if (d->cfg.stream_dtype != H3B_F32) {
        if (!h3b_cast_dev(d->cuda, dx, d->cfg.stream_dtype, d->st_x, H3B_F32, seq * D, error, error_size)) return 0;
        dx = d->st_x;
    }
    e = cudaMemcpyAsync(y, dx, seq * D * sizeof(float), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(error, error_size, "layers_forward_f32 download: %s", cudaGetErrorString(e));
    return h3b_cuda_check(d->cuda, NULL, error, error_size);
}

int h3b_dit_layers_forward_f32(h3b_dit *d, unsigned first, unsigned n, const float *t_feat, const float *x, size_t seq,
                               const uint32_t *row_map, const float *rope_cos, const float *rope_sin, const float *text,
                               size_t text_seq, float *y, char *error, size_t error_size) {
    return layers_forward_host(d, first, n, t_feat, x, seq, 0, row_map, rope_cos, rope_sin, text, text_seq, y, error,
                               error_size);
}

int h3b_dit_layers_forward_ulysses_f32(h3b_dit *d, unsigned first, unsigned n, const float *t_feat, const float *x_local,
                                       size_t seq_local, size_t seq_real, const uint32_t *row_map,
                                       const float *rope_cos_full, const float *rope_sin_full, const float *text,
                                       size_t text_seq, float *y_local, char *error, size_t error_size) {
    if (!seq_real) return fail(error, error_size, "layers_forward_ulysses_f32: seq_real must be > 0");
    return layers_forward_host(d, first, n, t_feat, x_local, seq_local, seq_real, row_map, rope_cos_full, rope_sin_full,
                               text, text_seq, y_local, error, error_size);
}
