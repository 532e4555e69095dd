/* CPU restatement of h3.c's DiT denoiser block path.  TEST INFRASTRUCTURE ONLY:
 * see h3_oracle.h for who may load it.  Each function follows the reference
 * function cited beside it (paths are inside the h3.c tree). */
#define _GNU_SOURCE
#include "h3_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ threads */

static int g_threads = 1;

void ho_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }

typedef void (*ho_range_fn)(size_t lo, size_t hi, void *ctx);
typedef struct {
    ho_range_fn fn;
    void *ctx;
    size_t lo, hi;
} ho_job;

static void *ho_job_main(void *p) {
    ho_job *j = (ho_job *)p;
    j->fn(j->lo, j->hi, j->ctx);
    return NULL;
}

/* Static split of [0,n) over the worker threads; the reference's own loops are
 * serial, and every loop split here is over independent rows. */
static void ho_parallel_for(size_t n, ho_range_fn fn, void *ctx) {
    int t = g_threads, i;
    pthread_t tid[256];
    ho_job job[256];
    if ((size_t)t > n) t = (int)n;
    if (t <= 1) {
        fn(0, n, ctx);
        return;
    }
    for (i = 0; i < t; i++) {
        job[i].fn = fn;
        job[i].ctx = ctx;
        job[i].lo = n * (size_t)i / (size_t)t;
        job[i].hi = n * (size_t)(i + 1) / (size_t)t;
        pthread_create(&tid[i], NULL, ho_job_main, &job[i]);
    }
    for (i = 0; i < t; i++) pthread_join(tid[i], NULL);
}

/* ------------------------------------------------------------ scalar formats */

/* h3_w4a8_dequant.c:17-39 */
float ho_f8e4m3fn_to_f32(uint8_t bits) {
    int sign = bits >> 7, e = (bits >> 3) & 15, m = bits & 7;
    float v;
    if (e == 15 && m == 7) return sign ? -NAN : NAN;
    if (e == 0)
        v = m ? ldexpf((float)m, -9) : 0.0f;
    else
        v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return sign ? -v : v;
}

/* h3_gpu_cuda.cu:4498-4513 */
uint8_t ho_f32_to_ue4m3(float v) {
    int e, m, E;
    float f;
    if (!(v > 0.0f)) return 0;
    f = frexpf(v, &e);
    E = e + 6;
    if (E <= 0) {
        m = (int)lroundf(ldexpf(v, 6) * 8.0f);
        return (uint8_t)(m > 7 ? 7 : m);
    }
    if (E >= 15) return 0x7E;
    m = (int)lroundf((f * 2.0f - 1.0f) * 8.0f);
    if (m == 8) {
        E++;
        m = 0;
        if (E >= 15) return 0x7E;
    }
    return (uint8_t)((E << 3) | m);
}

/* h3_gpu_cuda.cu:4515-4520 */
float ho_ue4m3_to_f32(uint8_t b) {
    int e = (b >> 3) & 15, m = b & 7;
    if (e == 0) return ldexpf((float)m / 8.0f, -6);
    if (e == 15 && m == 7) return NAN;
    return ldexpf(1.0f + (float)m / 8.0f, e - 7);
}

/* h3_gpu_cuda.cu:4468-4496: threshold table, ties go up in magnitude. */
uint8_t ho_e2m1_nibble(float q) {
    static const float thr[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    float a = fabsf(q);
    uint8_t mag = 0;
    while (mag < 7 && !(a < thr[mag])) mag++;
    /* the reference takes the sign of the rounded value: -0.1 -> +0 */
    return (uint8_t)(((q < 0.0f && mag != 0) ? 8 : 0) | mag);
}

float ho_e2m1_to_f32(uint8_t nib) {
    static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float v = mag[nib & 7];
    return (nib & 8) ? -v : v;
}

uint16_t ho_f32_to_bf16_bits(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float ho_bf16_bits_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

float ho_bf16_round(float x) { return ho_bf16_bits_to_f32(ho_f32_to_bf16_bits(x)); }

static uint16_t f32_to_f16_bits(float x) {
    uint32_t u, sign, mant;
    int32_t e;
    memcpy(&u, &x, 4);
    sign = (u >> 16) & 0x8000u;
    e = (int32_t)((u >> 23) & 0xff) - 127 + 15;
    mant = u & 0x7fffffu;
    if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (mant ? 0x200u : 0));
    if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        uint32_t shift, half, rem, q;
        if (e < -10) return (uint16_t)sign;
        mant |= 0x800000u;
        shift = (uint32_t)(14 - e);
        q = mant >> shift;
        rem = mant & ((1u << shift) - 1u);
        half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    {
        uint32_t q = ((uint32_t)e << 10) | (mant >> 13);
        uint32_t rem = mant & 0x1fffu;
        if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
}

static float f16_bits_to_f32(uint16_t h) {
    int sign = h >> 15, e = (h >> 10) & 31, m = h & 1023;
    float v;
    if (e == 31) v = m ? NAN : INFINITY;
    else if (e == 0) v = ldexpf((float)m, -24);
    else v = ldexpf(1.0f + (float)m / 1024.0f, e - 15);
    return sign ? -v : v;
}

float ho_f16_round(float x) { return f16_bits_to_f32(f32_to_f16_bits(x)); }

/* ------------------------------------------------------------------ weights */

/* h3_w4a8_dequant.c:41-118: low nibble -> even k; codebook[idx] * e4m3 scale,
 * roundf (half away from zero), clamp +-127. */
int ho_w4a8_dequant_to_int8(const int8_t *packed, size_t n, size_t k_half,
                            const float *codebook16, const uint8_t *s_rel_f8,
                            int group_size, int8_t *out) {
    size_t k = k_half * 2, groups, r, c;
    if (!packed || !codebook16 || !s_rel_f8 || !out) return 0;
    if (group_size < 4 || (group_size % 16 != 0 && 16 % group_size != 0)) return 0;
    if (k % (size_t)group_size) return 0;
    groups = k / (size_t)group_size;
    for (r = 0; r < n; r++)
        for (c = 0; c < k; c++) {
            unsigned byte = (uint8_t)packed[r * k_half + c / 2];
            unsigned idx = (c & 1) ? (byte >> 4) : (byte & 15u);
            float s = ho_f8e4m3fn_to_f32(s_rel_f8[r * groups + c / (size_t)group_size]);
            float v = roundf(codebook16[idx] * s);
            if (v > 127.0f) v = 127.0f;
            if (v < -127.0f) v = -127.0f;
            out[r * k + c] = (int8_t)v;
        }
    return 1;
}

int ho_w4g128_encode(const float *w, size_t n, size_t k, int group,
                     uint8_t *packed, uint16_t *scales) {
    size_t groups, r, g, c;
    if (!w || !packed || !scales || group < 2 || (group & 1) || k % (size_t)group) return 0;
    groups = k / (size_t)group;
    for (r = 0; r < n; r++)
        for (g = 0; g < groups; g++) {
            const float *src = w + r * k + g * (size_t)group;
            float amax = 0.0f, s;
            uint16_t sb;
            for (c = 0; c < (size_t)group; c++)
                if (fabsf(src[c]) > amax) amax = fabsf(src[c]);
            sb = f32_to_f16_bits(amax > 0.0f ? amax / 7.0f : 1.0f);
            if ((sb & 0x7fffu) == 0) sb = 0x0001; /* never a zero scale */
            s = f16_bits_to_f32(sb);
            scales[r * groups + g] = sb;
            for (c = 0; c < (size_t)group; c++) {
                float q = rintf(src[c] / s);
                int qi;
                size_t col = g * (size_t)group + c;
                uint8_t *dst = packed + r * (k / 2) + col / 2;
                if (q > 7.0f) q = 7.0f;
                if (q < -8.0f) q = -8.0f;
                qi = (int)q & 15;
                if (col & 1) *dst = (uint8_t)((*dst & 0x0f) | (qi << 4));
                else *dst = (uint8_t)((*dst & 0xf0) | qi);
            }
        }
    return 1;
}

int ho_w4g128_decode_to_int8(const uint8_t *packed, const uint16_t *scales,
                             size_t n, size_t k, int group, int8_t *w_i8,
                             float *s_channel) {
    size_t groups, r, c;
    if (!packed || !scales || !w_i8 || !s_channel || group < 2 || k % (size_t)group) return 0;
    groups = k / (size_t)group;
    for (r = 0; r < n; r++) {
        float amax = 0.0f, sc, inv;
        for (c = 0; c < k; c++) {
            unsigned byte = packed[r * (k / 2) + c / 2];
            int q = (int)((c & 1) ? (byte >> 4) : (byte & 15u));
            float v;
            if (q > 7) q -= 16;
            v = fabsf(f16_bits_to_f32(scales[r * groups + c / (size_t)group]) * (float)q);
            if (v > amax) amax = v;
        }
        sc = amax > 0.0f ? amax / 127.0f : 1.0f;
        inv = 1.0f / sc;
        s_channel[r] = sc;
        for (c = 0; c < k; c++) {
            unsigned byte = packed[r * (k / 2) + c / 2];
            int q = (int)((c & 1) ? (byte >> 4) : (byte & 15u));
            float v;
            if (q > 7) q -= 16;
            v = roundf(f16_bits_to_f32(scales[r * groups + c / (size_t)group]) * (float)q * inv);
            if (v > 127.0f) v = 127.0f;
            if (v < -127.0f) v = -127.0f;
            w_i8[r * k + c] = (int8_t)v;
        }
    }
    return 1;
}

int ho_quantize_weight_int8(const float *w, size_t n, size_t k, int8_t *w_i8,
                            float *s_channel) {
    if (!w || !w_i8 || !s_channel) return 0;
    return ho_quantize_act_int8(w, n, k, w_i8, s_channel);
}

/* ------------------------------------------------------------------ ConvRot */

/* h3_w4a8_dequant.c:139-195: H4 kron-powers, scaled by 1/sqrt(size). */
int ho_hadamard_normalized(int size, float *h) {
    static const float h4[16] = {1, 1, 1, -1, 1, 1, -1, 1, 1, -1, 1, 1, -1, 1, 1, 1};
    int t = size, i, j;
    float inv;
    if (size < 4 || !h) return 0;
    while (t % 4 == 0) t /= 4;
    if (t != 1) return 0;
    for (i = 0; i < size; i++)
        for (j = 0; j < size; j++) {
            /* entry = product over base-4 digits of h4[digit_i][digit_j] */
            float v = 1.0f;
            int a = i, b = j, s = size;
            while (s > 1) {
                v *= h4[(a & 3) * 4 + (b & 3)];
                a >>= 2;
                b >>= 2;
                s >>= 2;
            }
            h[i * size + j] = v;
        }
    inv = 1.0f / sqrtf((float)size);
    for (i = 0; i < size * size; i++) h[i] *= inv;
    return 1;
}

typedef struct {
    const float *x;
    float *y;
    const float *h;
    size_t k, gs;
} convrot_ctx;

/* h3_w4a8_dequant.c:339-352: out[j] += x[i] * H[i][j], i ascending, zero
 * entries skipped (there are none), so each output is a 256-term f32 sum in
 * ascending i. */
static void convrot_rows(size_t lo, size_t hi, void *p) {
    convrot_ctx *c = (convrot_ctx *)p;
    size_t r, g, i, j;
    for (r = lo; r < hi; r++)
        for (g = 0; g < c->k / c->gs; g++) {
            const float *src = c->x + r * c->k + g * c->gs;
            float *dst = c->y + r * c->k + g * c->gs;
            for (j = 0; j < c->gs; j++) dst[j] = 0.0f;
            for (i = 0; i < c->gs; i++)
                for (j = 0; j < c->gs; j++) dst[j] += src[i] * c->h[i * c->gs + j];
        }
}

int ho_convrot_act_f32(const float *x, size_t m, size_t k, int gs, float *y) {
    convrot_ctx c;
    float *h;
    if (!x || !y || m == 0 || k == 0) return 0;
    if (gs <= 0) {
        if (x != y) memcpy(y, x, m * k * sizeof(float));
        return 1;
    }
    if (gs < 4 || k % (size_t)gs) return 0;
    h = (float *)malloc((size_t)gs * (size_t)gs * sizeof(float));
    if (!h || !ho_hadamard_normalized(gs, h)) {
        free(h);
        return 0;
    }
    c.x = x; c.y = y; c.h = h; c.k = k; c.gs = (size_t)gs;
    ho_parallel_for(m, convrot_rows, &c);
    free(h);
    return 1;
}

/* Walsh-Hadamard rotation of every `gs` group of a row by in-place radix-2 butterflies, then one multiplication by
 * 1/sqrt(gs): what H3_CONVROT_SYLVESTER=1 selects instead of the regular-Hadamard product
 * (h3_w4a8_dequant.c:241-284, switch at :371-375). */
int ho_fwht_act_f32(const float *x, size_t m, size_t k, int gs, float *y) {
    size_t row, g;
    if (!x || !y || m == 0 || k == 0) return 0;
    if (gs < 2 || (gs & (gs - 1)) || k % (size_t)gs) return 0;
    if (x != y) memcpy(y, x, m * k * sizeof(float));
    for (row = 0; row < m; row++)
        for (g = 0; g < k / (size_t)gs; g++) {
            float *a = y + row * k + g * (size_t)gs;
            const float scale = 1.0f / sqrtf((float)gs);
            int h, i, j;
            for (h = 1; h < gs; h *= 2)
                for (i = 0; i < gs; i += 2 * h)
                    for (j = i; j < i + h; j++) {
                        const float u = a[j], v = a[j + h];
                        a[j] = u + v;
                        a[j + h] = u - v;
                    }
            for (h = 0; h < gs; h++) a[h] *= scale;
        }
    return 1;
}

/* ------------------------------------------------ activation quant and GEMMs */

/* h3_w4a8_dequant.c:671-688 */
int ho_quantize_act_int8(const float *x, size_t m, size_t k, int8_t *q, float *scales) {
    size_t r, c;
    if (!x || !q || !scales || m == 0 || k == 0) return 0;
    for (r = 0; r < m; r++) {
        const float *src = x + r * k;
        float amax = 0.0f, scale, inv;
        for (c = 0; c < k; c++) {
            float a = fabsf(src[c]);
            if (a > amax) amax = a;
        }
        scale = amax > 0.0f ? amax / 127.0f : 1.0f;
        scales[r] = scale;
        inv = 1.0f / scale;
        for (c = 0; c < k; c++) {
            float v = roundf(src[c] * inv);
            if (v > 127.0f) v = 127.0f;
            if (v < -127.0f) v = -127.0f;
            q[r * k + c] = (int8_t)v;
        }
    }
    return 1;
}

typedef struct {
    const int8_t *x, *w;
    const float *a, *s;
    size_t n, k;
    int32_t *acc;
    float *y;
} gemm_i8_ctx;

static void gemm_i8_rows(size_t lo, size_t hi, void *p) {
    gemm_i8_ctx *c = (gemm_i8_ctx *)p;
    size_t i, j, t;
    for (i = lo; i < hi; i++)
        for (j = 0; j < c->n; j++) {
            const int8_t *xi = c->x + i * c->k, *wj = c->w + j * c->k;
            int32_t acc = 0;
            for (t = 0; t < c->k; t++) acc += (int32_t)xi[t] * (int32_t)wj[t];
            if (c->acc) c->acc[i * c->n + j] = acc;
            if (c->y) c->y[i * c->n + j] = c->a[i] * c->s[j] * (float)acc;
        }
}

void ho_gemm_i8_i32(const int8_t *x, const int8_t *w, size_t m, size_t n, size_t k,
                    int32_t *acc) {
    gemm_i8_ctx c = {x, w, NULL, NULL, n, k, acc, NULL};
    ho_parallel_for(m, gemm_i8_rows, &c);
}

/* h3_w4a8_dequant.c:692-710: y = a[m] * s[n] * (float)acc, evaluated left to right. */
void ho_gemm_i8_dequant_f32(const int8_t *x, const int8_t *w, const float *a,
                            const float *s, size_t m, size_t n, size_t k, float *y) {
    gemm_i8_ctx c = {x, w, a, s, n, k, NULL, y};
    ho_parallel_for(m, gemm_i8_rows, &c);
}

typedef struct {
    const float *x, *w;
    size_t n, k;
    float *y;
} gemm_f32_ctx;

static void gemm_f32_rows(size_t lo, size_t hi, void *p) {
    gemm_f32_ctx *c = (gemm_f32_ctx *)p;
    size_t i, j, t;
    for (i = lo; i < hi; i++)
        for (j = 0; j < c->n; j++) {
            const float *xi = c->x + i * c->k, *wj = c->w + j * c->k;
            float acc = 0.0f;
            for (t = 0; t < c->k; t++) acc += xi[t] * wj[t];
            c->y[i * c->n + j] = acc;
        }
}

/* h3_w4a8_dequant.c:515-529 */
void ho_gemm_f32(const float *x, const float *w, size_t m, size_t n, size_t k, float *y) {
    gemm_f32_ctx c = {x, w, n, k, y};
    ho_parallel_for(m, gemm_f32_rows, &c);
}

/* ---------------------------------------------------------------- epilogues */

/* h3_dit_fused_epi.h:87-110 */
void ho_dequant_swiglu_f32(const int32_t *acc, const float *a, const float *s,
                           size_t rows, size_t width, const float *lora, float *out) {
    size_t r, c, n = width * 2;
    for (r = 0; r < rows; r++)
        for (c = 0; c < width; c++) {
            float g = a[r] * s[c] * (float)acc[r * n + c];
            float u = a[r] * s[width + c] * (float)acc[r * n + width + c];
            if (lora) {
                g += lora[r * n + c];
                u += lora[r * n + width + c];
            }
            out[r * width + c] = (g / (1.0f + expf(-g))) * u;
        }
}

/* h3_dit_fused_epi.h:116-141 */
void ho_dequant_gate_f32(const int32_t *acc, const float *a, const float *s,
                         const float *residual, const float *modulation,
                         const uint32_t *row_map, size_t rows, size_t width,
                         size_t slots, size_t gate_slot, const float *lora, float *out) {
    size_t r, c;
    for (r = 0; r < rows; r++) {
        size_t mrow = row_map ? row_map[r] : r;
        const float *gate = modulation + mrow * slots * width + gate_slot * width;
        for (c = 0; c < width; c++) {
            float br = a[r] * s[c] * (float)acc[r * width + c];
            if (lora) br += lora[r * width + c];
            out[r * width + c] = residual[r * width + c] + br * gate[c];
        }
    }
}

/* h3_vision_cuda.c:365-371 */
float ho_gelu_tanh(float v) {
    float inner = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    if (inner <= -10.0f) return 0.0f;
    if (inner >= 10.0f) return v;
    return 0.5f * v * (1.0f + tanhf(inner));
}

void ho_dequant_gelu_f32(const int32_t *acc, const float *a, const float *s,
                         size_t rows, size_t width, float *out) {
    size_t r, c;
    for (r = 0; r < rows; r++)
        for (c = 0; c < width; c++)
            out[r * width + c] = ho_gelu_tanh(a[r] * s[c] * (float)acc[r * width + c]);
}

/* ------------------------------------------------------------- row-wise ops */

/* h3_dit_w4a8.c:2747-2759 */
void ho_rms_norm_f32(const float *x, const float *w, size_t rows, size_t width,
                     float eps, float *out) {
    size_t r, c;
    for (r = 0; r < rows; r++) {
        const float *xr = x + r * width;
        float sum = 0.0f, inv;
        for (c = 0; c < width; c++) sum += xr[c] * xr[c];
        inv = 1.0f / sqrtf(sum / (float)width + eps);
        for (c = 0; c < width; c++) out[r * width + c] = xr[c] * inv * w[c];
    }
}

/* h3_dit_w4a8.c:2761-2785 */
void ho_adaln_f32(const float *x, const float *norm_w, const float *modulation,
                  const uint32_t *row_map, size_t rows, size_t width, size_t slots,
                  size_t shift_slot, size_t scale_slot, float eps, float *out) {
    size_t r, c;
    for (r = 0; r < rows; r++) {
        const float *xr = x + r * width;
        size_t mrow = row_map ? row_map[r] : r;
        const float *base = modulation + mrow * slots * width;
        const float *shift = base + shift_slot * width, *scale = base + scale_slot * width;
        float sum = 0.0f, inv;
        for (c = 0; c < width; c++) sum += xr[c] * xr[c];
        inv = 1.0f / sqrtf(sum / (float)width + eps);
        for (c = 0; c < width; c++) {
            float nrm = xr[c] * inv * norm_w[c];
            out[r * width + c] = nrm * (1.0f + scale[c]) + shift[c];
        }
    }
}

/* h3_dit_w4a8.c:2787-2803 */
void ho_gate_f32(const float *residual, const float *branch, const float *modulation,
                 const uint32_t *row_map, size_t rows, size_t width, size_t slots,
                 size_t gate_slot, float *out) {
    size_t r, c;
    for (r = 0; r < rows; r++) {
        size_t mrow = row_map ? row_map[r] : r;
        const float *gate = modulation + mrow * slots * width + gate_slot * width;
        for (c = 0; c < width; c++)
            out[r * width + c] = residual[r * width + c] + branch[r * width + c] * gate[c];
    }
}

/* h3_dit_fused_epi.h:51-83 */
void ho_gate_adaln_f32(const float *residual, const float *branch, const float *norm_w,
                       const float *modulation, const uint32_t *row_map, size_t rows,
                       size_t width, size_t slots, size_t gate_slot, size_t shift_slot,
                       size_t scale_slot, float eps, float *gated, float *normed) {
    ho_gate_f32(residual, branch, modulation, row_map, rows, width, slots, gate_slot, gated);
    ho_adaln_f32(gated, norm_w, modulation, row_map, rows, width, slots, shift_slot,
                 scale_slot, eps, normed);
}

/* h3_dit_w4a8.c:1976-1989 */
void ho_swiglu_f32(const float *fused, size_t rows, size_t width, float *out) {
    size_t r, c;
    for (r = 0; r < rows; r++)
        for (c = 0; c < width; c++) {
            float g = fused[r * 2 * width + c], u = fused[r * 2 * width + width + c];
            out[r * width + c] = (g / (1.0f + expf(-g))) * u;
        }
}

/* ------------------------------------------------- QK-norm + RoPE, attention */

/* h3_dit_w4a8.c:2805-2920 */
int ho_qkv_rope_f32(const float *qkv, const float *q_norm, const float *k_norm,
                    const float *rope_cos, const float *rope_sin, size_t seq,
                    size_t heads, size_t head_dim, size_t rope_half, float eps,
                    int grouped, int split_half, float *q, float *k, float *v) {
    size_t row, head, d, inner = heads * head_dim;
    if (!qkv || !q_norm || !k_norm || !q || !k || !v || !seq || !heads || !head_dim) return 0;
    if (rope_half && (!rope_cos || !rope_sin)) return 0;
    if (rope_half * 2 > head_dim) return 0;
    for (row = 0; row < seq; row++) {
        const float *qr = qkv + row * inner * 3;
        const float *cr = rope_half ? rope_cos + row * rope_half : NULL;
        const float *sr = rope_half ? rope_sin + row * rope_half : NULL;
        for (head = 0; head < heads; head++) {
            const float *qb = grouped ? qr + head * head_dim * 3 : qr + head * head_dim;
            const float *kb = grouped ? qb + head_dim : qb + inner;
            const float *vb = grouped ? kb + head_dim : qb + inner * 2;
            float *qo = q + (row * heads + head) * head_dim;
            float *ko = k + (row * heads + head) * head_dim;
            float *vo = v + (row * heads + head) * head_dim;
            float qs = 0.0f, ks = 0.0f, qi, ki;
            for (d = 0; d < head_dim; d++) {
                qs += qb[d] * qb[d];
                ks += kb[d] * kb[d];
                vo[d] = vb[d];
            }
            qi = 1.0f / sqrtf(qs / (float)head_dim + eps);
            ki = 1.0f / sqrtf(ks / (float)head_dim + eps);
            if (split_half && rope_half) {
                for (d = 0; d < head_dim; d++) {
                    float q0 = qb[d] * qi * q_norm[d], k0 = kb[d] * ki * k_norm[d];
                    if (d < rope_half) {
                        size_t p = d + rope_half;
                        float q1 = qb[p] * qi * q_norm[p], k1 = kb[p] * ki * k_norm[p];
                        q0 = q0 * cr[d] - q1 * sr[d];
                        k0 = k0 * cr[d] - k1 * sr[d];
                    } else if (d < rope_half * 2) {
                        size_t p = d - rope_half;
                        float q1 = qb[p] * qi * q_norm[p], k1 = kb[p] * ki * k_norm[p];
                        q0 = q0 * cr[p] + q1 * sr[p];
                        k0 = k0 * cr[p] + k1 * sr[p];
                    }
                    qo[d] = q0;
                    ko[d] = k0;
                }
            } else {
                for (d = 0; d < head_dim; d++) {
                    qo[d] = qb[d] * qi * q_norm[d];
                    ko[d] = kb[d] * ki * k_norm[d];
                }
                for (d = 0; d < rope_half; d++) {
                    size_t i0 = d * 2, i1 = i0 + 1;
                    float c = cr[d], s = sr[d];
                    float q0 = qo[i0], q1 = qo[i1], k0 = ko[i0], k1 = ko[i1];
                    qo[i0] = q0 * c - q1 * s;
                    qo[i1] = q0 * s + q1 * c;
                    ko[i0] = k0 * c - k1 * s;
                    ko[i1] = k0 * s + k1 * c;
                }
            }
        }
    }
    return 1;
}

typedef struct {
    const float *q, *k, *v;
    size_t qs, ks, vs, lk, heads, hd;
    float scale;
    float *out;
} sdpa_ctx;

/* h3_dit_w4a8.c:3089-3112, with the key count decoupled from the query count */
static void sdpa_rows(size_t lo, size_t hi, void *p) {
    sdpa_ctx *c = (sdpa_ctx *)p;
    float *scores = (float *)malloc(c->lk * sizeof(float));
    size_t qi, h, ki, d;
    if (!scores) return;
    for (qi = lo; qi < hi; qi++)
        for (h = 0; h < c->heads; h++) {
            const float *q = c->q + qi * c->qs + h * c->hd;
            float *o = c->out + (qi * c->heads + h) * c->hd;
            float mx = -INFINITY, sum = 0.0f;
            for (ki = 0; ki < c->lk; ki++) {
                const float *k = c->k + ki * c->ks + h * c->hd;
                float dot = 0.0f;
                for (d = 0; d < c->hd; d++) dot += q[d] * k[d];
                scores[ki] = dot * c->scale;
                if (scores[ki] > mx) mx = scores[ki];
            }
            for (ki = 0; ki < c->lk; ki++) {
                scores[ki] = expf(scores[ki] - mx);
                sum += scores[ki];
            }
            for (d = 0; d < c->hd; d++) o[d] = 0.0f;
            for (ki = 0; ki < c->lk; ki++) {
                const float *v = c->v + ki * c->vs + h * c->hd;
                float w = scores[ki] / sum;
                for (d = 0; d < c->hd; d++) o[d] += w * v[d];
            }
        }
    free(scores);
}

int ho_sdpa_rect_f32(const float *q, size_t q_stride, const float *k, size_t k_stride,
                     const float *v, size_t v_stride, size_t lq, size_t lk,
                     size_t heads, size_t head_dim, float scale, float *out) {
    sdpa_ctx c = {q, k, v, q_stride, k_stride, v_stride, lk, heads, head_dim, scale, out};
    if (!q || !k || !v || !out || !lq || !lk || !heads || !head_dim) return 0;
    ho_parallel_for(lq, sdpa_rows, &c);
    return 1;
}

int ho_sdpa_f32(const float *q, const float *k, const float *v, size_t seq, size_t heads,
                size_t head_dim, float scale, float *out) {
    size_t st = heads * head_dim;
    return ho_sdpa_rect_f32(q, st, k, st, v, st, seq, seq, heads, head_dim, scale, out);
}

/* ------------------------------------------- positions, tables, modulation */

/* h3_dit_w4a8.c:2451-2468 */
int ho_rope_tables_f32(const float *inv_freq, size_t freqs, size_t seq,
                       const float *pos_t, const float *pos_h, const float *pos_w,
                       float spatial_scale, float *cos_out, float *sin_out) {
    size_t row, axis, f;
    if (!inv_freq || !pos_t || !pos_h || !pos_w || !cos_out || !sin_out || !seq) return 0;
    if (!isfinite(spatial_scale) || spatial_scale <= 0.0f) return 0;
    for (row = 0; row < seq; row++) {
        float axes[3];
        axes[0] = pos_t[row];
        axes[1] = pos_h[row] * spatial_scale;
        axes[2] = pos_w[row] * spatial_scale;
        for (axis = 0; axis < 3; axis++)
            for (f = 0; f < freqs; f++) {
                size_t idx = row * 3 * freqs + axis * freqs + f;
                float angle = axes[axis] * inv_freq[f];
                cos_out[idx] = cosf(angle);
                sin_out[idx] = sinf(angle);
            }
    }
    return 1;
}

/* h3_dit_w4a8.c:2477-2531 */
int ho_fill_video_pos(size_t text_len, int latent_t, int latent_h, int latent_w,
                      float *pos_t, float *pos_h, float *pos_w) {
    static const int per_token[5] = {1, 4, 4, 4, 4};
    int nh, nw, t, y, x;
    size_t idx = 0;
    float area, rh, rw, sh, sw, bh, bw, time;
    if (!pos_t || !pos_h || !pos_w || latent_t < 1 || latent_h < 2 || latent_w < 2 ||
        (latent_h % 2) || (latent_w % 2))
        return 0;
    nh = latent_h / 2;
    nw = latent_w / 2;
    area = sqrtf((float)latent_h * (float)latent_w);
    rh = (float)latent_h / area;
    rw = (float)latent_w / area;
    sh = rh / (float)nh;
    sw = rw / (float)nw;
    bh = (1.0f - rh) * 0.5f;
    bw = (1.0f - rw) * 0.5f;
    time = (float)text_len;
    for (t = 0; t < latent_t; t++) {
        for (y = 0; y < nh; y++) {
            float hh = ((float)y * sh + bh) * 32.0f;
            for (x = 0; x < nw; x++, idx++) {
                pos_t[idx] = time;
                pos_h[idx] = hh;
                pos_w[idx] = ((float)x * sw + bw) * 32.0f;
            }
        }
        time += (5.0f / 3.0f) * (float)per_token[t % 5];
    }
    return 1;
}

/* h3_dit_w4a8.c:2256-2261 (no SiLU on the time feature by default) */
void ho_adaln_project_f32(const float *w, const float *b, size_t out_dim, size_t in_dim,
                          const float *t_feat, float *mod) {
    size_t o, i;
    for (o = 0; o < out_dim; o++) {
        float sum = b[o];
        for (i = 0; i < in_dim; i++) sum += w[o * in_dim + i] * t_feat[i];
        mod[o] = sum;
    }
}

/* h3_dit_w4a8.c:5298-5318: y = x W^T + b, the bias is the first term of the sum */
void ho_dense_f32(const float *x, const float *w, const float *bias, size_t m, size_t n, size_t k, float *y) {
    size_t r, o, i;
    for (r = 0; r < m; r++)
        for (o = 0; o < n; o++) {
            float sum = bias ? bias[o] : 0.0f;
            for (i = 0; i < k; i++) sum += x[r * k + i] * w[o * k + i];
            y[r * n + o] = sum;
        }
}

/* h3_dit_w4a8.c:8822-8839: returns 0 for a sigma pair the reference rejects */
int ho_euler_step_f32(float *sample, const float *velocity, size_t count, float sigma, float sigma_next) {
    size_t i;
    float delta;
    if (!sample || !velocity || count == 0) return 0;
    if (!isfinite(sigma) || !isfinite(sigma_next) || !(sigma > sigma_next) || sigma_next < 0.0f) return 0;
    delta = sigma - sigma_next;
    for (i = 0; i < count; i++) sample[i] += delta * velocity[i];
    return 1;
}

/* -------------------------------------------------------------------- NVFP4 */

/* tests/test_h3_nvfp4_sf_bytes.c:8-14, h3_gpu_cuda.cu:5940-5948 */
size_t ho_nvfp4_sf_bytes(size_t rows, size_t k) {
    if (rows == 0 || k == 0 || (k & 63u)) return 0;
    return ((rows + 127u) / 128u) * (k / 64u) * 512u;
}

/* h3_gpu_cuda.cu:4534-4537, 4552, 4596-4600 */
size_t ho_nvfp4_sf_offset(size_t row, size_t block16, size_t k) {
    size_t ncb = k / 64u, r128 = row & 127u;
    return ((row >> 7) * ncb + (block16 >> 2)) * 512u + 16u * (r128 & 31u) + 4u * (r128 >> 5) +
           (block16 & 3u);
}

/* rule 0: the CUDA activation kernel, h3_gpu_cuda.cu:4539-4614 (multiply by 1/scale;
 * a negative value that rounds to zero gets sign 0).  rule 1: the Python weight
 * quantiser, tools/quant_dit_nvfp4.py:65-107 (divide by scale; sign bit taken from
 * the unrounded value, so a small negative gives the "negative zero" nibble 0x8). */
int ho_quantize_nvfp4_rule(const float *x, size_t m, size_t k, int rule, uint8_t *packed,
                           uint8_t *sf) {
    size_t r, g, e, nc = k / 16;
    if (!x || !packed || !sf || !m || !k || (k & 63u)) return 0;
    memset(sf, 0, ho_nvfp4_sf_bytes(m, k));
    for (r = 0; r < m; r++)
        for (g = 0; g < nc; g++) {
            const float *src = x + r * k + g * 16;
            float amax = 0.0f, scale, inv;
            uint8_t sb, nib[16];
            for (e = 0; e < 16; e++) amax = fmaxf(amax, fabsf(src[e]));
            scale = amax > 0.0f ? amax / 6.0f : 1.0f;
            sb = ho_f32_to_ue4m3(scale);
            if (sb == 0) sb = 1;
            scale = ho_ue4m3_to_f32(sb);
            inv = scale > 0.0f ? 1.0f / scale : 0.0f;
            sf[ho_nvfp4_sf_offset(r, g, k)] = sb;
            for (e = 0; e < 16; e++) {
                if (rule == 0) {
                    nib[e] = ho_e2m1_nibble(src[e] * inv);
                } else {
                    float q = src[e] / scale;
                    nib[e] = (uint8_t)((ho_e2m1_nibble(q) & 7u) | (q < 0.0f ? 8u : 0u));
                }
            }
            for (e = 0; e < 16; e += 2)
                packed[r * (k / 2) + (g * 16 + e) / 2] = (uint8_t)((nib[e] << 4) | nib[e + 1]);
        }
    return 1;
}

int ho_quantize_nvfp4(const float *x, size_t m, size_t k, uint8_t *packed, uint8_t *sf) {
    return ho_quantize_nvfp4_rule(x, m, k, 0, packed, sf);
}

/* h3_nvfp4.c:322-400 (hi nibble first), scale from the swizzled table */
int ho_dequant_nvfp4(const uint8_t *packed, const uint8_t *sf, size_t m, size_t k, float *x) {
    size_t r, c;
    if (!packed || !sf || !x || (k & 63u)) return 0;
    for (r = 0; r < m; r++)
        for (c = 0; c < k; c++) {
            uint8_t byte = packed[r * (k / 2) + c / 2];
            uint8_t nib = (c & 1) ? (byte & 15u) : (byte >> 4);
            x[r * k + c] = ho_e2m1_to_f32(nib) * ho_ue4m3_to_f32(sf[ho_nvfp4_sf_offset(r, c / 16, k)]);
        }
    return 1;
}

typedef struct {
    const float *x, *w;
    size_t n, k;
    float scale2;
    float *y;
} fp4_ctx;

static void fp4_rows(size_t lo, size_t hi, void *p) {
    fp4_ctx *c = (fp4_ctx *)p;
    size_t i, j, t;
    for (i = lo; i < hi; i++)
        for (j = 0; j < c->n; j++) {
            double acc = 0.0; /* products are exact in f32; the sum is kept wide */
            for (t = 0; t < c->k; t++) acc += (double)(c->x[i * c->k + t] * c->w[j * c->k + t]);
            c->y[i * c->n + j] = c->scale2 * (float)acc;
        }
}

int ho_gemm_nvfp4_f32(const uint8_t *x_fp4, const uint8_t *x_sf, const uint8_t *w_fp4,
                      const uint8_t *w_sf, float scale2, size_t m, size_t n, size_t k, float *y) {
    float *xd = (float *)malloc(m * k * sizeof(float));
    float *wd = (float *)malloc(n * k * sizeof(float));
    int ok = xd && wd && ho_dequant_nvfp4(x_fp4, x_sf, m, k, xd) && ho_dequant_nvfp4(w_fp4, w_sf, n, k, wd);
    if (ok) {
        fp4_ctx c = {xd, wd, n, k, scale2, y};
        ho_parallel_for(m, fp4_rows, &c);
    }
    free(xd);
    free(wd);
    return ok;
}

/* ------------------------------------------------------------------ Ulysses */

/* h3_ulysses.c:12-37 */
int ho_ulysses_validate(int heads, int packed_align, int tp, int ulysses, int ring) {
    if (tp < 1 || ulysses < 1 || ring < 1 || heads < 1 || packed_align < 1) return 0;
    if (ulysses != 1 && ulysses != 2 && ulysses != 4 && ulysses != 8) return 0;
    if (heads % tp) return 0;
    if ((heads / tp) % ulysses) return 0;
    if (packed_align % (ulysses * ring)) return 0;
    return 1;
}

/* h3_ulysses.c:39-45 */
size_t ho_ulysses_pad_seq(size_t seq, int align) {
    size_t a = (size_t)align;
    return align < 1 ? seq : (seq + a - 1) / a * a;
}

/* h3_ulysses.c:47-56 */
size_t ho_ulysses_local_rows(size_t seq_pad, int ulysses, int rank) {
    size_t u = (size_t)ulysses;
    if (ulysses < 1) return seq_pad;
    if (rank < 0 || (size_t)rank >= u) return 0;
    return seq_pad / u + ((size_t)rank < seq_pad % u ? 1u : 0u);
}

/* h3_ulysses_comm.cu:256-279: in[s][q][h][d] -> out[peer][s][q][h%hl][d] */
void ho_ulysses_pack_qkv(const void *in, void *out, size_t seq_local, size_t heads,
                         size_t head_dim, int u, size_t elem) {
    size_t hl = heads / (size_t)u, s, q, h, row = head_dim * elem;
    for (s = 0; s < seq_local; s++)
        for (q = 0; q < 3; q++)
            for (h = 0; h < heads; h++) {
                size_t peer = h / hl;
                size_t src = ((s * 3 + q) * heads + h) * row;
                size_t dst = (((peer * seq_local + s) * 3 + q) * hl + (h - peer * hl)) * row;
                memcpy((char *)out + dst, (const char *)in + src, row);
            }
}

/* h3_ulysses_comm.cu:281-304: in[src][s][q][hl][d] -> out[src*seq_local+s][q][hl][d] */
void ho_ulysses_unpack_qkv(const void *in, void *out, size_t seq_local, size_t heads,
                           size_t head_dim, int u, size_t elem) {
    /* With destination rows ordered by source rank the unpacked buffer has the
     * same linear order as the received chunks. */
    size_t hl = heads / (size_t)u;
    memcpy(out, in, (size_t)u * seq_local * 3 * hl * head_dim * elem);
}

/* h3_ulysses_comm.cu:306-323: in[src*seq_local+s][hl][d] -> out[src][s][hl][d] */
void ho_ulysses_pack_attn(const void *in, void *out, size_t seq_local, size_t heads,
                          size_t head_dim, int u, size_t elem) {
    size_t hl = heads / (size_t)u;
    memcpy(out, in, (size_t)u * seq_local * hl * head_dim * elem);
}

/* h3_ulysses_comm.cu:325-344: in[peer][s][hl][d] -> out[s][peer*hl+hl'][d] */
void ho_ulysses_unpack_attn(const void *in, void *out, size_t seq_local, size_t heads,
                            size_t head_dim, int u, size_t elem) {
    size_t hl = heads / (size_t)u, peer, s, h, row = head_dim * elem;
    for (peer = 0; peer < (size_t)u; peer++)
        for (s = 0; s < seq_local; s++)
            for (h = 0; h < hl; h++)
                memcpy((char *)out + ((s * heads) + peer * hl + h) * row,
                       (const char *)in + (((peer * seq_local + s) * hl) + h) * row, row);
}

/* h3_ulysses_comm.cu:411-434: rank r's p-th packed chunk lands as rank p's r-th chunk */
static void a2a_exchange(char *const *pack, char *const *unp, int u, size_t chunk) {
    int r, p;
    for (r = 0; r < u; r++)
        for (p = 0; p < u; p++)
            memcpy(unp[p] + (size_t)r * chunk, pack[r] + (size_t)p * chunk, chunk);
}

void ho_ulysses_a2a_qkv_sim(const void *const *in, void *const *out, size_t seq_local,
                            size_t heads, size_t head_dim, int u, size_t elem) {
    size_t total = seq_local * 3 * heads * head_dim * elem, chunk = total / (size_t)u;
    char *pack[8], *unp[8];
    int r;
    for (r = 0; r < u; r++) {
        pack[r] = (char *)malloc(total);
        unp[r] = (char *)malloc(total);
        ho_ulysses_pack_qkv(in[r], pack[r], seq_local, heads, head_dim, u, elem);
    }
    a2a_exchange(pack, unp, u, chunk);
    for (r = 0; r < u; r++) {
        ho_ulysses_unpack_qkv(unp[r], out[r], seq_local, heads, head_dim, u, elem);
        free(pack[r]);
        free(unp[r]);
    }
}

void ho_ulysses_a2a_attn_sim(const void *const *in, void *const *out, size_t seq_local,
                             size_t heads, size_t head_dim, int u, size_t elem) {
    size_t total = seq_local * heads * head_dim * elem, chunk = total / (size_t)u;
    char *pack[8], *unp[8];
    int r;
    for (r = 0; r < u; r++) {
        pack[r] = (char *)malloc(total);
        unp[r] = (char *)malloc(total);
        ho_ulysses_pack_attn(in[r], pack[r], seq_local, heads, head_dim, u, elem);
    }
    a2a_exchange(pack, unp, u, chunk);
    for (r = 0; r < u; r++) {
        ho_ulysses_unpack_attn(unp[r], out[r], seq_local, heads, head_dim, u, elem);
        free(pack[r]);
        free(unp[r]);
    }
}

/* ------------------------------------------------------------- whole blocks */

static void round_bf16(float *x, size_t n) {
    size_t i;
    for (i = 0; i < n; i++) x[i] = ho_bf16_round(x[i]);
}

/* One linear: f32 GEMM, or (ConvRot ->) per-row int8 quant -> int8 GEMM with the
 * raw accumulator returned so the caller applies its epilogue
 * (tools/h3_dit_w4a8_block_probe.c:106-137). */
typedef struct {
    int32_t *acc; /* quantised */
    float *a;     /* quantised: per-row act scale */
    float *y;     /* f32 path: plain product */
} lin_out;

static int run_linear(const ho_block_cfg *cfg, const ho_linear *l, const float *x, size_t m,
                      lin_out *o) {
    memset(o, 0, sizeof(*o));
    if (!cfg->quantised) {
        o->y = (float *)malloc(m * l->n * sizeof(float));
        if (!o->y) return 0;
        ho_gemm_f32(x, l->w_f32, m, l->n, l->k, o->y);
        return 1;
    } else {
        float *rot = (float *)malloc(m * l->k * sizeof(float));
        int8_t *q = (int8_t *)malloc(m * l->k);
        int ok;
        o->acc = (int32_t *)malloc(m * l->n * sizeof(int32_t));
        o->a = (float *)malloc(m * sizeof(float));
        ok = rot && q && o->acc && o->a && ho_convrot_act_f32(x, m, l->k, cfg->convrot_gs, rot) &&
             ho_quantize_act_int8(rot, m, l->k, q, o->a);
        if (ok) ho_gemm_i8_i32(q, l->w_i8, m, l->n, l->k, o->acc);
        free(rot);
        free(q);
        return ok;
    }
}

static void lin_free(lin_out *o) {
    free(o->acc);
    free(o->a);
    free(o->y);
}

/* plain dequant of a linear result into y[m,n] */
static void lin_plain(const ho_block_cfg *cfg, const ho_linear *l, const lin_out *o, size_t m,
                      float *y) {
    size_t i, j;
    if (!cfg->quantised) {
        memcpy(y, o->y, m * l->n * sizeof(float));
        return;
    }
    for (i = 0; i < m; i++)
        for (j = 0; j < l->n; j++)
            y[i * l->n + j] = o->a[i] * l->s_channel[j] * (float)o->acc[i * l->n + j];
}

int ho_block_b_forward(const ho_block_cfg *cfg, const ho_block_b *b, const float *x, size_t m,
                       const float *text, size_t t, const float *rope_cos,
                       const float *rope_sin, float *y) {
    const size_t D = cfg->dim, H = cfg->heads, hd = cfg->head_dim, F = cfg->ffn;
    const float scale = 1.0f / sqrtf((float)hd);
    float *a = (float *)malloc(m * D * sizeof(float));
    float *qkv = (float *)malloc(m * 3 * D * sizeof(float));
    float *q = (float *)malloc(m * D * sizeof(float));
    float *k = (float *)malloc(m * D * sizeof(float));
    float *v = (float *)malloc(m * D * sizeof(float));
    float *att = (float *)malloc(m * D * sizeof(float));
    float *br = (float *)malloc(m * D * sizeof(float));
    float *x1 = (float *)malloc(m * D * sizeof(float));
    float *x2 = (float *)malloc(m * D * sizeof(float));
    float *ckv = (float *)malloc(t * 2 * D * sizeof(float));
    float *h = (float *)malloc(m * F * sizeof(float));
    uint32_t *zero_map = (uint32_t *)calloc(m, sizeof(uint32_t));
    lin_out lo;
    size_t i;
    int ok = 0, bf = cfg->bf16_stream;
    if (!a || !qkv || !q || !k || !v || !att || !br || !x1 || !x2 || !ckv || !h || !zero_map)
        goto done;

    /* self-attention branch */
    ho_adaln_f32(x, b->norm1, b->modulation, zero_map, m, D, 6, 0, 1, cfg->eps, a);
    if (bf) round_bf16(a, m * D);
    if (!run_linear(cfg, &b->qkv, a, m, &lo)) goto done;
    lin_plain(cfg, &b->qkv, &lo, m, qkv);
    lin_free(&lo);
    if (bf) round_bf16(qkv, m * 3 * D);
    if (!ho_qkv_rope_f32(qkv, b->q_norm, b->k_norm, rope_cos, rope_sin, m, H, hd, cfg->rope_half,
                         cfg->eps, 0, 1, q, k, v))
        goto done;
    if (bf) {
        round_bf16(q, m * D);
        round_bf16(k, m * D);
    }
    if (!ho_sdpa_f32(q, k, v, m, H, hd, scale, att)) goto done;
    if (bf) round_bf16(att, m * D);
    if (!run_linear(cfg, &b->o, att, m, &lo)) goto done;
    lin_plain(cfg, &b->o, &lo, m, br);
    lin_free(&lo);
    ho_gate_f32(x, br, b->modulation, zero_map, m, D, 6, 2, x1);
    if (bf) round_bf16(x1, m * D);

    /* cross-attention branch: no RoPE, no QK-norm, no gate */
    ho_rms_norm_f32(x1, b->norm_c, m, D, cfg->eps, a);
    if (bf) round_bf16(a, m * D);
    if (!run_linear(cfg, &b->cq, a, m, &lo)) goto done;
    lin_plain(cfg, &b->cq, &lo, m, q);
    lin_free(&lo);
    if (bf) round_bf16(q, m * D);
    if (!run_linear(cfg, &b->ckv, text, t, &lo)) goto done;
    lin_plain(cfg, &b->ckv, &lo, t, ckv);
    lin_free(&lo);
    if (bf) round_bf16(ckv, t * 2 * D);
    if (!ho_sdpa_rect_f32(q, D, ckv, 2 * D, ckv + D, 2 * D, m, t, H, hd, scale, att)) goto done;
    if (bf) round_bf16(att, m * D);
    if (!run_linear(cfg, &b->co, att, m, &lo)) goto done;
    lin_plain(cfg, &b->co, &lo, m, br);
    lin_free(&lo);
    for (i = 0; i < m * D; i++) x2[i] = x1[i] + br[i];
    if (bf) round_bf16(x2, m * D);

    /* feed-forward branch */
    ho_adaln_f32(x2, b->norm2, b->modulation, zero_map, m, D, 6, 3, 4, cfg->eps, a);
    if (bf) round_bf16(a, m * D);
    if (!run_linear(cfg, &b->up, a, m, &lo)) goto done;
    lin_plain(cfg, &b->up, &lo, m, h);
    lin_free(&lo);
    for (i = 0; i < m * F; i++) h[i] = ho_gelu_tanh(h[i]);
    if (bf) round_bf16(h, m * F);
    if (!run_linear(cfg, &b->down, h, m, &lo)) goto done;
    lin_plain(cfg, &b->down, &lo, m, br);
    lin_free(&lo);
    ho_gate_f32(x2, br, b->modulation, zero_map, m, D, 6, 5, y);
    if (bf) round_bf16(y, m * D);
    ok = 1;
done:
    free(a); free(qkv); free(q); free(k); free(v); free(att); free(br); free(x1); free(x2);
    free(ckv); free(h); free(zero_map);
    return ok;
}

int ho_block_r_forward(const ho_block_cfg *cfg, const ho_block_r *b, const float *x, size_t m,
                       const float *rope_cos, const float *rope_sin, float *y) {
    const size_t D = cfg->dim, H = cfg->heads, hd = cfg->head_dim, F = cfg->ffn, I = H * hd;
    float *a = (float *)malloc(m * D * sizeof(float));
    float *qkv = (float *)malloc(m * 3 * I * sizeof(float));
    float *q = (float *)malloc(m * I * sizeof(float));
    float *k = (float *)malloc(m * I * sizeof(float));
    float *v = (float *)malloc(m * I * sizeof(float));
    float *att = (float *)malloc(m * I * sizeof(float));
    float *br = (float *)malloc(m * D * sizeof(float));
    float *x1 = (float *)malloc(m * D * sizeof(float));
    float *fc1 = (float *)malloc(m * 2 * F * sizeof(float));
    float *act = (float *)malloc(m * F * sizeof(float));
    lin_out lo;
    int ok = 0;
    if (!a || !qkv || !q || !k || !v || !att || !br || !x1 || !fc1 || !act) goto done;
    ho_adaln_f32(x, b->norm1, b->modulation, b->row_map, m, D, 6, 0, 1, cfg->eps, a);
    if (!run_linear(cfg, &b->qkv, a, m, &lo)) goto done;
    lin_plain(cfg, &b->qkv, &lo, m, qkv);
    lin_free(&lo);
    if (!ho_qkv_rope_f32(qkv, b->q_norm, b->k_norm, rope_cos, rope_sin, m, H, hd, cfg->rope_half,
                         cfg->eps, 0, 1, q, k, v))
        goto done;
    if (!ho_sdpa_f32(q, k, v, m, H, hd, 1.0f / sqrtf((float)hd), att)) goto done;
    if (!run_linear(cfg, &b->out, att, m, &lo)) goto done;
    lin_plain(cfg, &b->out, &lo, m, br);
    lin_free(&lo);
    ho_gate_f32(x, br, b->modulation, b->row_map, m, D, 6, 2, x1);
    ho_adaln_f32(x1, b->norm2, b->modulation, b->row_map, m, D, 6, 3, 4, cfg->eps, a);
    if (!run_linear(cfg, &b->fc1, a, m, &lo)) goto done;
    lin_plain(cfg, &b->fc1, &lo, m, fc1);
    lin_free(&lo);
    ho_swiglu_f32(fc1, m, F, act);
    if (!run_linear(cfg, &b->fc2, act, m, &lo)) goto done;
    lin_plain(cfg, &b->fc2, &lo, m, br);
    lin_free(&lo);
    ho_gate_f32(x1, br, b->modulation, b->row_map, m, D, 6, 5, y);
    ok = 1;
done:
    free(a); free(qkv); free(q); free(k); free(v); free(att); free(br); free(x1); free(fc1);
    free(act);
    return ok;
}

/* Byte-wise FNV-1a 64 for arbitrary buffers; ho_checksum_f32 below is the
 * word-wise form of h3_dit_w4a8.c:8911-8922. */
uint64_t ho_fnv1a64(const void *data, size_t bytes) {
    const uint8_t *p = (const uint8_t *)data;
    uint64_t h = 0xcbf29ce484222325ULL;
    size_t i;
    for (i = 0; i < bytes; i++) {
        h ^= p[i];
        h *= 0x100000001b3ULL;
    }
    return h;
}

uint64_t ho_checksum_f32(const float *x, size_t n) {
    uint64_t h = 0xcbf29ce484222325ULL;
    size_t i;
    if (!x) return 0;
    for (i = 0; i < n; i++) {
        uint32_t bits;
        memcpy(&bits, &x[i], 4);
        h ^= (uint64_t)bits;
        h *= 0x100000001b3ULL;
    }
    return h;
}
