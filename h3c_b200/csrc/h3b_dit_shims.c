/* The Metal twin's DiT signatures (h3_dit.h:94-140), kept as thin shims.  The row-order conversions and the
 * velocity-reuse schedule are plain host arithmetic and are implemented (the reference pins them with known
 * answers in tests/test_h3.c:122-141, 351-375, restated in this repository's tests).  The entry points that
 * take an `h3_dit` object belong to the reference's Apple-GPU product: such an object cannot exist here, so
 * they fail with a message that says so.
 */
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/h3_b200.h"

static int shim_fail(char *error, size_t error_size, const char *what) {
    if (error && error_size) snprintf(error, error_size, "%s: Metal path: unavailable on this box", what);
    return 0;
}

/* ---- row-order conversions ------------------------------------------------------------------------------ */

/* element counts of a [channels, time, height, width] latent; 0 when the shape is unusable or overflows */
static size_t video_elements(int channels, int time, int height, int width) {
    size_t c, t, h, w;
    if (channels < 1 || time < 1 || height < 2 || width < 2 || (height & 1) || (width & 1)) return 0;
    c = (size_t)channels; t = (size_t)time; h = (size_t)height; w = (size_t)width;
    if (c > SIZE_MAX / t || c * t > SIZE_MAX / h || c * t * h > SIZE_MAX / w) return 0;
    return c * t * h * w;
}

/* Walks the patch order (frame, patch row, patch column, channel, 2 x 2 pixels) and calls back with the
 * latent index of every row element in turn. */
#define FOR_EACH_PATCH_ELEMENT(body)                                                                      \
    do {                                                                                                  \
        size_t at = 0;                                                                                    \
        int t, h, w, c, dh, dw;                                                                           \
        for (t = 0; t < time; t++)                                                                        \
            for (h = 0; h < height; h += 2)                                                               \
                for (w = 0; w < width; w += 2)                                                            \
                    for (c = 0; c < channels; c++)                                                        \
                        for (dh = 0; dh < 2; dh++)                                                        \
                            for (dw = 0; dw < 2; dw++) {                                                  \
                                const size_t li = (((size_t)c * (size_t)time + (size_t)t) * (size_t)height + \
                                                   (size_t)(h + dh)) * (size_t)width + (size_t)(w + dw);  \
                                body;                                                                     \
                                at++;                                                                     \
                            }                                                                             \
    } while (0)

int h3_dit_patchify_video(const float *latent, int channels, int time, int height, int width, float *rows,
                          size_t row_elements) {                                              /* h3_dit.h:131 */
    const size_t n = video_elements(channels, time, height, width);
    if (!latent || !rows || !n || row_elements != n) return 0;
    FOR_EACH_PATCH_ELEMENT(rows[at] = latent[li]);
    return 1;
}

int h3_dit_unpatchify_video(const float *rows, int channels, int time, int height, int width, float *latent,
                            size_t latent_elements) {                                         /* h3_dit.h:134 */
    const size_t n = video_elements(channels, time, height, width);
    if (!rows || !latent || !n || latent_elements != n) return 0;
    FOR_EACH_PATCH_ELEMENT(latent[li] = rows[at]);
    return 1;
}

/* audio latent [channels, 2 streams, time] <-> rows [stream, time, channels] */
static size_t audio_elements(int channels, int time) {
    if (channels < 1 || time < 1 || (size_t)channels > SIZE_MAX / (2 * (size_t)time)) return 0;
    return (size_t)channels * 2 * (size_t)time;
}

int h3_dit_pack_audio(const float *latent, int channels, int time, float *rows, size_t row_elements) {   /* :137 */
    const size_t n = audio_elements(channels, time);
    size_t at = 0;
    int s, t, c;
    if (!latent || !rows || !n || row_elements != n) return 0;
    for (s = 0; s < 2; s++)
        for (t = 0; t < time; t++)
            for (c = 0; c < channels; c++) rows[at++] = latent[((size_t)c * 2 + (size_t)s) * (size_t)time + (size_t)t];
    return 1;
}

int h3_dit_unpack_audio(const float *rows, int channels, int time, float *latent, size_t latent_elements) {   /* :139 */
    const size_t n = audio_elements(channels, time);
    size_t at = 0;
    int s, t, c;
    if (!rows || !latent || !n || latent_elements != n) return 0;
    for (s = 0; s < 2; s++)
        for (t = 0; t < time; t++)
            for (c = 0; c < channels; c++) latent[((size_t)c * 2 + (size_t)s) * (size_t)time + (size_t)t] = rows[at++];
    return 1;
}

/* Steps that run the transformer under velocity reuse: the first, the last and every reuse_interval-th; the
 * others extrapolate.  Returns how many were selected, -1 for bad arguments.  h3_dit.h:124 */
int h3_dit_reuse_schedule(int steps, int reuse_interval, uint8_t *selected, size_t selected_count) {
    int step, count = 0;
    if (steps < 1 || reuse_interval < 1 || reuse_interval > 32 || !selected || selected_count < (size_t)steps) return -1;
    for (step = 0; step < steps; step++) {
        selected[step] = (uint8_t)(step == 0 || step == steps - 1 || step % reuse_interval == 0);
        count += selected[step];
    }
    return count;
}

/* ---- entry points bound to the Apple-GPU transformer object ---------------------------------------------- */

int h3_dit_forward(h3_dit *dit, int step, const float *video_latent, const float *audio_latent, float *video_velocity,
                   float *audio_velocity, char *error, size_t error_size) {                  /* h3_dit.h:94 */
    (void)dit; (void)step; (void)video_latent; (void)audio_latent; (void)video_velocity; (void)audio_velocity;
    return shim_fail(error, error_size, "h3_dit_forward");
}

int h3_dit_denoise_euler(h3_dit *dit, float *video_latent, float *audio_latent, int reuse_interval,
                         h3_dit_progress progress, void *progress_opaque, char *error, size_t error_size) {   /* :106 */
    (void)dit; (void)video_latent; (void)audio_latent; (void)reuse_interval; (void)progress; (void)progress_opaque;
    return shim_fail(error, error_size, "h3_dit_denoise_euler");
}

size_t h3_dit_video_elements(const h3_dit *dit) { (void)dit; return 0; }   /* :88 */
size_t h3_dit_audio_elements(const h3_dit *dit) { (void)dit; return 0; }   /* :89 */
void h3_dit_free(h3_dit *dit) { (void)dit; }                               /* :77 */
