/* Host-side tables of a denoiser step: RoPE positions of the video tokens, the cos/sin
 * tables built from them, and the row of the time-feature table a noise level selects.
 * Same names, signatures and arithmetic as the reference (h3_dit_w4a8.h:366, :382, :395,
 * :545), so a caller needs nothing but this library to prepare the inputs of the block
 * chain.  Plain C, single precision exactly where the reference uses it: the results are
 * bit-identical to the reference's functions.
 */
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/h3_b200.h"
#include "../../include/h3b_plugin.h"

enum { ROPE_FREQS = 16, ROPE_AXES = 3, ROPE_HALF = ROPE_FREQS * ROPE_AXES };

static int fail(char *error, size_t error_size, const char *fmt, ...) {
    if (error && error_size) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(error, error_size, fmt, ap);
        va_end(ap);
    }
    return 0;
}

/* Latent frame t advances the time coordinate by 5/3 * {1,4,4,4,4}[t % 5]
 * (h3_dit_w4a8.c:2472-2478). */
static float time_step_of_frame(int t) {
    static const int frames_per_token[5] = {1, 4, 4, 4, 4};
    const float rescale = 5.0f / 3.0f;
    return rescale * (float)frames_per_token[t % 5];
}

float h3_dit_w4a8_video_span_sum(int latent_t) {
    float sum = 0.0f;
    int t;
    for (t = 0; t < latent_t; t++) sum += time_step_of_frame(t);
    return sum;
}

int h3_dit_w4a8_fill_metal_video_pos(size_t text_len, int latent_t, int latent_h, int latent_w, float *pos_t,
                                     float *pos_h, float *pos_w, char *error, size_t error_size) {
    int grid_h, grid_w, t, y, x;
    float diag, share_h, share_w, step_h, step_w, origin_h, origin_w, now;
    size_t at = 0;
    if (!pos_t || !pos_h || !pos_w || latent_t < 1 || latent_h < 2 || latent_w < 2 || (latent_h & 1) || (latent_w & 1))
        return fail(error, error_size, "invalid fill_metal_video_pos args");
    /* token grid = latent / 2 per spatial axis; coordinates are centred in a unit square whose
     * sides are shared out by aspect ratio, then scaled by 32 */
    grid_h = latent_h / 2;
    grid_w = latent_w / 2;
    diag = sqrtf((float)latent_h * (float)latent_w);
    share_h = (float)latent_h / diag;
    share_w = (float)latent_w / diag;
    step_h = share_h / (float)grid_h;
    step_w = share_w / (float)grid_w;
    origin_h = (1.0f - share_h) * 0.5f;
    origin_w = (1.0f - share_w) * 0.5f;
    now = (float)text_len;
    for (t = 0; t < latent_t; t++) {
        for (y = 0; y < grid_h; y++) {
            const float ph = ((float)y * step_h + origin_h) * 32.0f;
            for (x = 0; x < grid_w; x++) {
                pos_t[at] = now;
                pos_h[at] = ph;
                pos_w[at] = ((float)x * step_w + origin_w) * 32.0f;
                at++;
            }
        }
        now += time_step_of_frame(t);
    }
    return 1;
}

int h3_dit_w4a8_rope_tables_f32(const float *inv_freq, size_t seq, const float *pos_t, const float *pos_h,
                                const float *pos_w, float spatial_scale, float *cos_out, float *sin_out, char *error,
                                size_t error_size) {
    size_t r;
    int a, f;
    if (!inv_freq || !pos_t || !pos_h || !pos_w || !cos_out || !sin_out || !seq)
        return fail(error, error_size, "invalid rope_tables args");
    if (!isfinite(spatial_scale) || spatial_scale <= 0.0f) return fail(error, error_size, "invalid spatial_scale");
    for (r = 0; r < seq; r++) {
        const float coord[ROPE_AXES] = {pos_t[r], pos_h[r] * spatial_scale, pos_w[r] * spatial_scale};
        float *c = cos_out + r * ROPE_HALF, *s = sin_out + r * ROPE_HALF;
        for (a = 0; a < ROPE_AXES; a++)
            for (f = 0; f < ROPE_FREQS; f++) {
                const float angle = coord[a] * inv_freq[f];
                c[a * ROPE_FREQS + f] = cosf(angle);
                s[a * ROPE_FREQS + f] = sinf(angle);
            }
    }
    return 1;
}

size_t h3_dit_w4a8_t_row_from_sigma(float sigma, size_t t_table_rows) {
    const int by_sigma = strcmp(h3_plugin_value("H3_DIT_T_ROW_BY_SIGMA"), "1") == 0;
    float t;
    size_t row;
    if (!t_table_rows) return 0;
    if (!isfinite(sigma) || sigma < 0.0f) sigma = 0.0f;
    if (sigma > 1.0f) sigma = 1.0f;
    /* the table is laid out over time = 1 - sigma; the switch restores the older sigma axis */
    t = by_sigma ? sigma : 1.0f - sigma;
    row = (size_t)llround((double)t * (double)(t_table_rows - 1));
    return row < t_table_rows ? row : t_table_rows - 1;
}

/* Addition: video positions and tables of a whole step in one call (text_len temporal offset, token grid
 * grid_t x grid_h x grid_w, i.e. latent dims grid_t x 2 grid_h x 2 grid_w), `pad_rows` extra rows of angle 0
 * at the end (cos 1, sin 0: rows a sequence-parallel run pads the sequence with).  cos_out / sin_out:
 * [(grid_t*grid_h*grid_w + pad_rows), 48]. */
int h3b_dit_video_rope_tables(const float *inv_freq16, size_t text_len, int grid_t, int grid_h, int grid_w,
                              float spatial_scale, size_t pad_rows, float *cos_out, float *sin_out, char *error,
                              size_t error_size) {
    size_t seq, i;
    float *pos;
    int ok;
    if (grid_t < 1 || grid_h < 1 || grid_w < 1) return fail(error, error_size, "video_rope_tables: bad grid");
    seq = (size_t)grid_t * (size_t)grid_h * (size_t)grid_w;
    pos = (float *)malloc(3 * seq * sizeof(float));
    if (!pos) return fail(error, error_size, "video_rope_tables: out of memory");
    ok = h3_dit_w4a8_fill_metal_video_pos(text_len, grid_t, 2 * grid_h, 2 * grid_w, pos, pos + seq, pos + 2 * seq, error,
                                          error_size) &&
         h3_dit_w4a8_rope_tables_f32(inv_freq16, seq, pos, pos + seq, pos + 2 * seq, spatial_scale, cos_out, sin_out,
                                     error, error_size);
    free(pos);
    if (!ok) return 0;
    for (i = seq * ROPE_HALF; i < (seq + pad_rows) * ROPE_HALF; i++) {
        cos_out[i] = 1.0f;
        sin_out[i] = 0.0f;
    }
    return 1;
}
