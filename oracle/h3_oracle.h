/* CPU restatement of h3.c's DiT denoiser block path.  TEST INFRASTRUCTURE ONLY.
 *
 * Only the test-suite, the smoke check and the benchmark's cpu_baseline leg may
 * load this library; the product library (libh3_b200.so) never links, loads or
 * calls anything declared here and has no CPU fallback.
 *
 * Every function names the reference function it restates (path inside the
 * h3.c tree, with line).  Parity of this file against the reference itself is
 * pinned by tests/test_oracle_vs_ref.py (which loads a library compiled from
 * the reference's own sources) and by the committed vectors in tests/golden/.
 *
 * Conventions: row-major, float32 unless stated, `ho_` prefix, return 1 = ok /
 * 0 = bad arguments (same as the reference, h3_w4a8_dequant.c:9-15).
 */
#ifndef H3_ORACLE_H
#define H3_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar formats ---- */
float ho_f8e4m3fn_to_f32(uint8_t bits);            /* h3_w4a8_dequant.c:17 */
uint8_t ho_f32_to_ue4m3(float v);                  /* h3_gpu_cuda.cu:4498 */
float ho_ue4m3_to_f32(uint8_t b);                  /* h3_gpu_cuda.cu:4515 */
uint8_t ho_e2m1_nibble(float q);                   /* h3_gpu_cuda.cu:4468-4496 */
float ho_e2m1_to_f32(uint8_t nibble);
float ho_bf16_round(float x);                      /* RNE to bfloat16, back to f32 */
uint16_t ho_f32_to_bf16_bits(float x);
float ho_bf16_bits_to_f32(uint16_t b);
float ho_f16_round(float x);                       /* RNE to IEEE half, back to f32 */

/* ---- W4A8 weights ---- */
/* "asym_w4a8_int8" (reference checkpoint format), h3_w4a8_dequant.c:65 */
int ho_w4a8_dequant_to_int8(const int8_t *packed, size_t n, size_t k_half,
                            const float *codebook16, const uint8_t *s_rel_f8,
                            int group_size, int8_t *int8_out);
/* Symmetric int4, groups of `group` along K with f16 scales (the benchmark's
 * weight format; no reference code exists for it).  Encoder: per group
 * s = absmax/7 rounded to f16 (0 -> 1), q = clamp(rint(w/s), -8, 7); nibble
 * = q & 0xF, low nibble = even k.  Decoder re-expresses w = s*q as resident
 * int8 + per-channel f32 scale exactly like the reference treats its own
 * format (decode once, then int8 x int8): s_ch[n] = max_k|s*q|/127 (0 -> 1),
 * w_i8 = clamp(roundf((s*q) * (1/s_ch[n])), -127, 127). */
int ho_w4g128_encode(const float *w, size_t n, size_t k, int group,
                     uint8_t *packed, uint16_t *scales_f16);
int ho_w4g128_decode_to_int8(const uint8_t *packed, const uint16_t *scales_f16,
                             size_t n, size_t k, int group, int8_t *w_i8,
                             float *s_channel);
/* Plain per-channel symmetric int8 weight quantiser used to make synthetic
 * INT8-ConvRot style weights ([N,K] int8 + weight_scale[N], h3_dit_int8.h:26). */
int ho_quantize_weight_int8(const float *w, size_t n, size_t k, int8_t *w_i8,
                            float *s_channel);

/* ---- ConvRot ---- */
int ho_hadamard_normalized(int size, float *h);    /* h3_w4a8_dequant.c:139 */
int ho_convrot_act_f32(const float *x, size_t m, size_t k, int gs, float *y); /* :286,:367 */
int ho_fwht_act_f32(const float *x, size_t m, size_t k, int gs, float *y);    /* :241-284 (H3_CONVROT_SYLVESTER=1) */

/* ---- INT8 activation quant + GEMM ---- */
int ho_quantize_act_int8(const float *x, size_t m, size_t k, int8_t *q,
                         float *scales);           /* h3_w4a8_dequant.c:671 */
void ho_gemm_i8_i32(const int8_t *x, const int8_t *w, size_t m, size_t n,
                    size_t k, int32_t *acc);       /* h3_w4a8_dequant.c:703 */
void ho_gemm_i8_dequant_f32(const int8_t *x, const int8_t *w, const float *a,
                            const float *s, size_t m, size_t n, size_t k,
                            float *y);             /* h3_w4a8_dequant.c:692 */
void ho_gemm_f32(const float *x, const float *w, size_t m, size_t n, size_t k,
                 float *y);                        /* h3_w4a8_dequant.c:515 */

/* ---- epilogues (h3_dit_fused_epi.h:87,116) ---- */
void ho_dequant_swiglu_f32(const int32_t *acc, const float *a, const float *s,
                           size_t rows, size_t width, const float *lora,
                           float *out);
void ho_dequant_gate_f32(const int32_t *acc, const float *a, const float *s,
                         const float *residual, const float *modulation,
                         const uint32_t *row_map, size_t rows, size_t width,
                         size_t slots, size_t gate_slot, const float *lora,
                         float *out);
/* tanh-GELU (formula as h3_vision_cuda.c:365-371): 0.5 v (1 + tanh(c (v + 0.044715 v^3))) */
float ho_gelu_tanh(float v);
void ho_dequant_gelu_f32(const int32_t *acc, const float *a, const float *s,
                         size_t rows, size_t width, float *out);

/* ---- row-wise ops (h3_dit_w4a8.c:2747, 2761, 2787; h3_dit_fused_epi.h:51) ---- */
void ho_rms_norm_f32(const float *x, const float *w, size_t rows, size_t width,
                     float eps, float *out);
void ho_adaln_f32(const float *x, const float *norm_w, const float *modulation,
                  const uint32_t *row_map, size_t rows, size_t width,
                  size_t slots, size_t shift_slot, size_t scale_slot, float eps,
                  float *out);
void ho_gate_f32(const float *residual, const float *branch,
                 const float *modulation, const uint32_t *row_map, size_t rows,
                 size_t width, size_t slots, size_t gate_slot, float *out);
void ho_gate_adaln_f32(const float *residual, const float *branch,
                       const float *norm_w, const float *modulation,
                       const uint32_t *row_map, size_t rows, size_t width,
                       size_t slots, size_t gate_slot, size_t shift_slot,
                       size_t scale_slot, float eps, float *gated, float *normed);
void ho_swiglu_f32(const float *fused, size_t rows, size_t width, float *out);

/* ---- QK-norm + RoPE, attention (h3_dit_w4a8.c:2805, 3073) ---- */
/* layout: 0 contiguous [Q|K|V] thirds (default), 1 grouped per head.
 * rope_mode: 1 split-half (pair d with d+rope_half; default), 0 consecutive pairs. */
int ho_qkv_rope_f32(const float *qkv, const float *q_norm, const float *k_norm,
                    const float *rope_cos, const float *rope_sin, size_t seq,
                    size_t heads, size_t head_dim, size_t rope_half, float eps,
                    int grouped, int split_half, float *q, float *k, float *v);
/* q [lq,heads,d] (row stride given in floats), k/v [lk,heads,d]; out [lq,heads*d]. */
int ho_sdpa_rect_f32(const float *q, size_t q_stride, const float *k,
                     size_t k_stride, const float *v, size_t v_stride, size_t lq,
                     size_t lk, size_t heads, size_t head_dim, float scale,
                     float *out);
int ho_sdpa_f32(const float *q, const float *k, const float *v, size_t seq,
                size_t heads, size_t head_dim, float scale, float *out);

/* ---- positions / RoPE tables / modulation (h3_dit_w4a8.c:2412, 2496, 2236) ---- */
int ho_rope_tables_f32(const float *inv_freq, size_t freqs, size_t seq,
                       const float *pos_t, const float *pos_h, const float *pos_w,
                       float spatial_scale, float *cos_out, float *sin_out);
int ho_fill_video_pos(size_t text_len, int latent_t, int latent_h, int latent_w,
                      float *pos_t, float *pos_h, float *pos_w);
void ho_adaln_project_f32(const float *w, const float *b, size_t out_dim,
                          size_t in_dim, const float *t_feat, float *mod);

/* ---- either side of the chain: dense f32 linear and Euler update (h3_dit_w4a8.c:5298, 8822) ---- */
void ho_dense_f32(const float *x, const float *w, const float *bias, size_t m, size_t n, size_t k,
                  float *y);
int ho_euler_step_f32(float *sample, const float *velocity, size_t count, float sigma,
                      float sigma_next);

/* ---- NVFP4 (h3_gpu_cuda.cu:4455-4614, 5940; tools/quant_dit_nvfp4.py:65) ---- */
size_t ho_nvfp4_sf_bytes(size_t rows, size_t k);
size_t ho_nvfp4_sf_offset(size_t row, size_t block16, size_t k);
/* x [m,k] -> packed [m,k/2] (high nibble = even k) + swizzled UE4M3 SF sized for
 * ceil128(m) rows (pad rows get SF 0). */
int ho_quantize_nvfp4(const float *x, size_t m, size_t k, uint8_t *packed,
                      uint8_t *sf);
/* rule 0 = CUDA activation kernel (same as ho_quantize_nvfp4); rule 1 = the Python
 * weight quantiser tools/quant_dit_nvfp4.py:65 (division, sign kept on zero). */
int ho_quantize_nvfp4_rule(const float *x, size_t m, size_t k, int rule,
                           uint8_t *packed, uint8_t *sf);
int ho_dequant_nvfp4(const uint8_t *packed, const uint8_t *sf, size_t m, size_t k,
                     float *x);
/* y = scale2 * sum_k dq(x)[m,k] dq(w)[n,k]; f32 accumulation per 16-block in
 * ascending k. */
int ho_gemm_nvfp4_f32(const uint8_t *x_fp4, const uint8_t *x_sf,
                      const uint8_t *w_fp4, const uint8_t *w_sf, float scale2,
                      size_t m, size_t n, size_t k, float *y);

/* ---- Ulysses (h3_ulysses.c:12-56, h3_ulysses_comm.cu:256-344) ---- */
int ho_ulysses_validate(int heads, int packed_align, int tp, int ulysses, int ring);
size_t ho_ulysses_pad_seq(size_t seq, int align);
size_t ho_ulysses_local_rows(size_t seq_pad, int ulysses, int rank);
/* elem = bytes per element; buffers are byte pointers. */
void ho_ulysses_pack_qkv(const void *in, void *out, size_t seq_local, size_t heads,
                         size_t head_dim, int u, size_t elem);
void ho_ulysses_unpack_qkv(const void *in, void *out, size_t seq_local,
                           size_t heads, size_t head_dim, int u, size_t elem);
void ho_ulysses_pack_attn(const void *in, void *out, size_t seq_local,
                          size_t heads, size_t head_dim, int u, size_t elem);
void ho_ulysses_unpack_attn(const void *in, void *out, size_t seq_local,
                            size_t heads, size_t head_dim, int u, size_t elem);
/* Whole exchange among u simulated ranks: in[r] -> out[r] (arrays of u pointers). */
void ho_ulysses_a2a_qkv_sim(const void *const *in, void *const *out,
                            size_t seq_local, size_t heads, size_t head_dim,
                            int u, size_t elem);
void ho_ulysses_a2a_attn_sim(const void *const *in, void *const *out,
                             size_t seq_local, size_t heads, size_t head_dim,
                             int u, size_t elem);

/* ---- whole blocks ---- */
typedef struct ho_linear {
    /* exactly one of w_f32 / w_i8 is used, chosen by ho_block_cfg.quantised */
    const float *w_f32;     /* [n,k] */
    const int8_t *w_i8;     /* [n,k] resident int8 */
    const float *s_channel; /* [n] */
    size_t n, k;
} ho_linear;

typedef struct ho_block_cfg {
    size_t dim, heads, head_dim, ffn, rope_half;
    float eps;
    int quantised;   /* 0: f32 weights, f32 GEMM; 1: int8 act quant + int8 GEMM */
    int bf16_stream; /* 1: round every stored tensor to bf16 (device dataflow) */
    int convrot_gs;  /* 0 or 256 (reference-geometry block only) */
} ho_block_cfg;

/* Benchmark block: adaLN -> QKV -> QK-norm+3D RoPE -> self-attn -> out·gate + x
 * -> rms_norm -> cross-attn(text) + residual -> adaLN -> up -> tanh-GELU -> down·gate
 * + residual.  Every op is one of the reference functions above. */
typedef struct ho_block_b {
    ho_linear qkv, o, cq, ckv, co, up, down;
    const float *norm1, *norm_c, *norm2, *q_norm, *k_norm; /* [dim],[dim],[dim],[hd],[hd] */
    const float *modulation; /* [6, dim] */
} ho_block_b;

int ho_block_b_forward(const ho_block_cfg *cfg, const ho_block_b *blk,
                       const float *x, size_t m, const float *text, size_t t,
                       const float *rope_cos, const float *rope_sin, float *y);

/* Reference-geometry block (h3_dit_w4a8.c:4798-4974, tools/h3_dit_w4a8_block_probe.c:360):
 * adaLN -> qkv -> qknorm/rope -> sdpa -> out + gate(2) -> adaLN(3,4) -> fc1 ->
 * SwiGLU -> fc2 + gate(5); modulation [mod_rows, 6, dim] with row_map. */
typedef struct ho_block_r {
    ho_linear qkv, out, fc1, fc2;
    const float *norm1, *norm2, *q_norm, *k_norm;
    const float *modulation;
    const uint32_t *row_map;
} ho_block_r;

int ho_block_r_forward(const ho_block_cfg *cfg, const ho_block_r *blk,
                       const float *x, size_t m, const float *rope_cos,
                       const float *rope_sin, float *y);

/* FNV-1a 64 over raw bytes. */
uint64_t ho_fnv1a64(const void *data, size_t bytes);
/* word-wise form the reference uses on f32 outputs (h3_dit_w4a8.c:8911) */
uint64_t ho_checksum_f32(const float *x, size_t n);

/* Number of worker threads the row-parallel loops may use (default 1). */
void ho_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
