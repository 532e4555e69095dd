/* libh3_b200.so -- B200 (sm_100a) implementation of h3.c's DiT denoiser block path.
 *
 * C ABI only: plain pointers and sizes, no C++ or PyTorch types.  Entry points
 * named h3_cuda_* / h3_ulysses_* keep the reference's name, argument order and
 * meaning so a caller of the reference links against this library unchanged for
 * this path; each one cites the reference declaration it replaces (file:line in
 * the h3.c tree).  Entry points named h3b_* are additions (bf16 residual stream,
 * the benchmark's block with cross-attention, one-process-per-GPU Ulysses) and
 * say so.
 *
 * Conventions (as in the reference, h3_gpu_cuda.h / h3_ulysses.c:6-10):
 *   - return int: 1 = ok, 0 = failure; message written to `error` (may be NULL)
 *   - device pointers are raw; work is enqueued on h3_cuda_op_stream(cuda)
 *     (NULL = legacy default stream); no implicit synchronisation in quiet mode
 *   - `double *..._ms` outputs are optional; they are filled (with an event
 *     synchronise) only when non-NULL and quiet mode is off
 *   - one handle per device, one host thread per handle; handles are not
 *     thread-safe
 *   - there is no CPU fallback: every entry point fails if no sm_100 device or
 *     kernel is available.
 */
#ifndef H3_B200_H
#define H3_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ handle */

typedef struct {                    /* h3_gpu_cuda.h:13-23 (same layout) */
    int device_index;
    char name[256];
    int compute_major;
    int compute_minor;
    size_t total_memory_bytes;
    size_t free_memory_bytes;
    int multiprocessor_count;
    int driver_version;
    int runtime_version;
} h3_cuda_device_info;

typedef struct h3_cuda h3_cuda;     /* h3_gpu_cuda.h:25 */

h3_cuda *h3_cuda_create(int device_index, char *error, size_t error_size);     /* h3_gpu_cuda.h:28 */
void h3_cuda_free(h3_cuda *cuda);                                              /* :29 */
void h3_cuda_release_heavy_workspace(h3_cuda *cuda);                           /* :33 */
int h3_cuda_pregrow_dit_scratch(h3_cuda *cuda, size_t seq, size_t hidden, size_t heads,
                                size_t head_dim, size_t ffn, char *error,
                                size_t error_size);                            /* :40 */
int h3_cuda_pregrow_hadamard(h3_cuda *cuda, int gs, char *error, size_t error_size); /* :47 */
int h3_cuda_dit_scratch_pregrown(const h3_cuda *cuda);                         /* :53 */
int h3_cuda_bind_device(h3_cuda *cuda, char *error, size_t error_size);        /* :57 */
int h3_cuda_device_count(char *error, size_t error_size);                      /* :80 */
int h3_cuda_probe(int device_index, h3_cuda_device_info *info, char *error,
                  size_t error_size);                                          /* :81 */
int h3_cuda_get_info(const h3_cuda *cuda, h3_cuda_device_info *info);          /* :83 */
int h3_cuda_mem_info(h3_cuda *cuda, size_t *free_bytes, size_t *total_bytes, char *error,
                     size_t error_size);                                       /* :86 */
void h3_cuda_set_graph_capture(h3_cuda *cuda, int enabled);                    /* :209 */
int h3_cuda_graph_capture(const h3_cuda *cuda);                                /* :210 */
void h3_cuda_set_quiet(h3_cuda *cuda, int enabled);                            /* :212 */
int h3_cuda_quiet(const h3_cuda *cuda);                                        /* :213 */
int h3_cuda_set_op_stream(h3_cuda *cuda, void *stream, char *error, size_t error_size); /* :217 */
void *h3_cuda_op_stream(const h3_cuda *cuda);                                  /* :219 */
void *h3_cuda_stream(h3_cuda *cuda, int index);                                /* :227 */
int h3_cuda_stream_count(void);                                                /* :228 */
int h3_cuda_event_record_default(h3_cuda *cuda, void **out_event, char *error,
                                 size_t error_size);                           /* :231 */
int h3_cuda_event_record(void *stream, void *event, char *error, size_t error_size);      /* :234 */
int h3_cuda_stream_wait_event(void *stream, void *event, char *error, size_t error_size); /* :237 */
void h3_cuda_event_destroy(void *event);                                       /* :239 */
void *h3_cuda_host_alloc(size_t bytes, int *pinned_out);                       /* :318 */
void h3_cuda_host_free(void *p, int pinned);                                   /* :319 */

/* Addition.  Synchronises the op stream and returns the device status word:
 * 0 = every kernel launched through this handle ran to completion; non-zero =
 * a kernel gave up a bounded wait (code in h3b_ptx.cuh) and its output is
 * invalid.  Also reports sticky CUDA errors through `error`. */
int h3b_cuda_check(h3_cuda *cuda, int *status_out, char *error, size_t error_size);
/* Additions.  Per-launch device timing: between _begin and _end every kernel launch of the handle
 * is bracketed by an event pair; _end synchronises and sums milliseconds and launches per kernel
 * class (0 int8 GEMM, 1 attention, 2 row-wise norm/quant, 3 QK-norm+RoPE, 4 other) and returns the
 * number of classes filled. */
void h3b_cuda_profile_begin(h3_cuda *cuda);
int h3b_cuda_profile_end(h3_cuda *cuda, double *ms_by_class, int *launches_by_class, int n_classes);
/* Addition.  Kernel launches issued through this handle since the last call. */
unsigned long long h3b_cuda_launch_count(h3_cuda *cuda, int reset);

/* Additions: the switch registry (include/h3b_plugin.h, the counterpart of the reference's tools/h3_plugin.h)
 * as exported functions.  _value: the environment's value if set and not empty, else the registered default;
 * NULL for an unregistered name.  _enabled: that value is not one of "", "0", "false", "off", "no". */
size_t h3b_plugin_count(void);
int h3b_plugin_get(size_t index, const char **name, const char **status, const char **stage, const char **default_value);
const char *h3b_plugin_value(const char *name);
int h3b_plugin_enabled(const char *name);

/* ----------------------------------------------------------------- weights */

typedef struct h3_cuda_w4a8_weight h3_cuda_w4a8_weight;   /* h3_gpu_cuda.h:284 */

/* Packed W4A8 (+ codebook / e4m3 group scales / per-channel scale) -> resident
 * INT8 [N,K] + s_channel[N], decoded on the device.  h3_gpu_cuda.h:289-295 */
int h3_cuda_w4a8_weight_create(h3_cuda *cuda, const int8_t *packed_host, size_t n, size_t k_half,
                               const float *codebook16, const uint8_t *s_rel_f8,
                               const float *s_channel, int group_size,
                               h3_cuda_w4a8_weight **out, double *unpack_ms, double *h2d_ms,
                               char *error, size_t error_size);
/* Already-decoded INT8 [N,K] + weight_scale[N].  h3_gpu_cuda.h:304-308.  With
 * borrow_host=0 the library takes ownership of both host buffers (allocated
 * with malloc or h3_cuda_host_alloc) on success. */
int h3_cuda_w4a8_weight_create_from_i8(h3_cuda *cuda, int8_t *w_i8, size_t n, size_t k,
                                       float *s_channel, h3_cuda_w4a8_weight **out,
                                       double *h2d_ms, int borrow_host, char *error,
                                       size_t error_size);
int h3_cuda_w4a8_weight_upload_i8(h3_cuda_w4a8_weight *weight, int8_t *w_i8, size_t n, size_t k,
                                  float *s_channel, int borrow_host, char *error,
                                  size_t error_size);                          /* :312 */
int h3_cuda_w4a8_weight_ensure_ready(h3_cuda_w4a8_weight *weight, char *error,
                                     size_t error_size);                       /* :326 */
int h3_cuda_w4a8_weight_on_device(const h3_cuda_w4a8_weight *weight, int want_dev, char *error,
                                  size_t error_size);                          /* :330 */
void h3_cuda_w4a8_weight_free(h3_cuda_w4a8_weight *weight);                    /* :337 */
size_t h3_cuda_w4a8_weight_n(const h3_cuda_w4a8_weight *weight);               /* :339 */
size_t h3_cuda_w4a8_weight_k(const h3_cuda_w4a8_weight *weight);               /* :340 */
int h3_cuda_w4a8_weight_download_int8(const h3_cuda_w4a8_weight *weight, int8_t *host_out,
                                      char *error, size_t error_size);         /* :343 */
/* Addition: symmetric int4 in groups of `group` along K with f16 scales (the
 * benchmark's weight format): packed [N,K/2] (low nibble = even k, two's
 * complement), scales_f16 [N,K/group].  Decoded on the device to the same
 * resident INT8 + per-channel scale object: s_ch = max|s*q|/127,
 * w_i8 = clamp(roundf(s*q / s_ch)). */
int h3b_w4g_weight_create(h3_cuda *cuda, const uint8_t *packed_host, const uint16_t *scales_f16,
                          size_t n, size_t k, int group, h3_cuda_w4a8_weight **out,
                          char *error, size_t error_size);
/* Addition: the same weight format kept PACKED on the device and multiplied exactly as the format defines it,
 *   y[m,n] = a[m] * sum_g s[n,g] * (sum_{k in group g} x_i8[m,k] * q[n,k]),
 * int32 partial sums per 128-K group, each scaled in f32 (one multiplication, one addition, in group order): the codes
 * are expanded to int8 in registers on their way into the tile that tcgen05.mma reads.  Selectable next to the
 * resident-int8 form above, which is the faster one.  K % 128 == 0, N % 4 == 0 (N % 8 for bf16 output);
 * d_x_i8 [m, K] and d_act_scales [m] as produced by the activation quantiser; d_y [m, N] H3B_F32 or H3B_BF16. */
typedef struct h3b_w4g_exact_weight h3b_w4g_exact_weight;
int h3b_w4g_exact_weight_create(h3_cuda *cuda, const uint8_t *packed_host, const uint16_t *scales_f16_host, size_t n,
                                size_t k, h3b_w4g_exact_weight **out, char *error, size_t error_size);
void h3b_w4g_exact_weight_free(h3b_w4g_exact_weight *weight);
int h3b_gemm_w4g_exact_dev(h3_cuda *cuda, const h3b_w4g_exact_weight *weight, const int8_t *d_x_i8,
                           const float *d_act_scales, size_t m, void *d_y, int out_dtype, char *error,
                           size_t error_size);
/* Addition: device pointers of the resident tensors. */
const int8_t *h3b_w4a8_weight_data(const h3_cuda_w4a8_weight *weight);
const float *h3b_w4a8_weight_scales(const h3_cuda_w4a8_weight *weight);
int h3b_w4a8_weight_download_scales(const h3_cuda_w4a8_weight *weight, float *host_out, char *error,
                                    size_t error_size);

/* ------------------------------------------------------------------ linears */

/* h3_gpu_cuda.h:378-401, same layout */
typedef struct h3_cuda_dit_gemm_epi {
    int swiglu;
    int gate;
    const float *d_residual;
    const float *d_modulation;
    const uint32_t *d_row_map;
    const float *d_lora;
    void *lora_ready;
    size_t slots;
    size_t gate_slot;
    int requant_mode;
    int requant_gs;
    int8_t *d_rq_x;
    float *d_rq_act;
    float *d_rq_pre;
    size_t requant_rows;
    int y_f16;
} h3_cuda_dit_gemm_epi;

/* Host in / host out INT8 GEMM + dequant.  h3_gpu_cuda.h:274-280 */
int h3_cuda_gemm_i8_dequant_f32(h3_cuda *cuda, const int8_t *x_i8, const int8_t *w_i8,
                                const float *act_scales, int per_tensor_scale,
                                const float *s_channel, size_t m, size_t n, size_t k, float *y_f32,
                                double *gemm_ms, char *backend_out, size_t backend_out_size,
                                char *error, size_t error_size);
int h3_cuda_gemm_i8_dequant_f32_w(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight,
                                  const int8_t *x_i8, const float *act_scales, int per_tensor_scale,
                                  size_t m, float *y_f32, double *gemm_ms, char *backend_out,
                                  size_t backend_out_size, char *error, size_t error_size); /* :349 */
int h3_cuda_gemm_i8_dequant_f32_w_act(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight,
                                      const float *x_f32, int convrot_groupsize, size_t m,
                                      float *y_f32, double *prep_ms, double *gemm_ms,
                                      char *backend_out, size_t backend_out_size, char *error,
                                      size_t error_size);                      /* :360 */
int h3_cuda_gemm_i8_dequant_f32_w_act_dev(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight,
                                          const float *d_x_f32, int convrot_groupsize, size_t m,
                                          float *d_y_f32, double *prep_ms, double *gemm_ms,
                                          char *backend_out, size_t backend_out_size, char *error,
                                          size_t error_size);                  /* :368 */
int h3_cuda_gemm_i8_dequant_f32_w_act_dev_epi(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight,
                                              const float *d_x_f32, int convrot_groupsize, size_t m,
                                              float *d_y_f32, double *prep_ms, double *gemm_ms,
                                              char *backend_out, size_t backend_out_size,
                                              const h3_cuda_dit_gemm_epi *epi, char *error,
                                              size_t error_size);              /* :403 */
int h3_cuda_gemm_i8_dequant_f32_dev_pre_q(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight,
                                          const int8_t *d_x_i8, const float *d_act_in, size_t m,
                                          float *d_y_f32, double *prep_ms, double *gemm_ms,
                                          char *backend_out, size_t backend_out_size,
                                          const h3_cuda_dit_gemm_epi *epi, char *error,
                                          size_t error_size);                  /* :414 */
int h3_cuda_convrot_act_f32_dd(h3_cuda *cuda, const float *d_x, size_t m, size_t k,
                               int convrot_groupsize, float *d_y, char *error,
                               size_t error_size);                             /* :137 */

/* No counterpart in the reference.  Same result as h3_cuda_gemm_i8_dequant_f32_w_act_dev
 * (f32 activations in, ConvRot + per-row INT8 quantisation + INT8 GEMM inside, f32 out) for
 * callers that cannot allocate device memory: a host whose device memory is already fully
 * committed (resident weights up to the last byte), or one that cannot afford the device-wide
 * synchronisation cudaMalloc/cudaFree bring in the middle of its step loop, or one that runs the
 * handle where growth of library scratch is refused.  The INT8 codes and row scales go to a
 * fixed area compiled into the library (8 MiB + 64 KiB per GPU, held from library load to
 * process exit) instead of scratch grown on demand, so the call performs no cudaMalloc, cudaFree
 * or other allocating call.
 *   - limits: m <= h3b_linear_noalloc_max_rows() (16384) and m * K <= h3b_linear_noalloc_max_codes()
 *     (8 Mi); larger shapes are rejected with an error that names the limits
 *   - the handle's device must be the calling thread's current device (h3_cuda_bind_device) and the
 *     weight must live on it: both are checked on every call, before anything is enqueued, and a
 *     mismatch is an error; the current device is never changed by this call
 *   - the first call on each device looks up the area's device address; make that first call before
 *     starting any stream capture.  The per-device cache of that address is written without a lock:
 *     concurrent first calls store the same value
 *   - every call on a device shares the one area and leaves its codes behind; each call
 *     overwrites what it reads, so nothing needs clearing, but two calls whose kernels can run at
 *     the same time on one GPU (different streams, threads or handles) race on it: serialise them
 *   - the weight's upload must be complete (h3_cuda_w4a8_weight_ensure_ready). */
int h3b_gemm_i8_dequant_f32_w_act_dev_noalloc(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight,
                                              const float *d_x_f32, int convrot_groupsize, size_t m,
                                              float *d_y_f32, char *error, size_t error_size);
size_t h3b_linear_noalloc_max_codes(void);
size_t h3b_linear_noalloc_max_rows(void);

/* Additions: the general form every linear above is built on. */
enum {            /* element types of activations / outputs */
    H3B_F32 = 0,
    H3B_BF16 = 1,
    H3B_F16 = 2,
    H3B_I32 = 3   /* raw int32 accumulators (parity checks) */
};
enum {            /* epilogue kinds */
    H3B_EPI_PLAIN = 0,   /* y = a[m] s[n] acc                                         */
    H3B_EPI_GATE = 1,    /* y = residual + (a s acc) * gate[row_map[m]][slot][n]; gate NULL -> 1 */
    H3B_EPI_SWIGLU = 2,  /* y[m,c] = silu(g) * u, g = col c, u = col n/2 + c           */
    H3B_EPI_GELU = 3,    /* y = gelu_tanh(a s acc)                                     */
    H3B_EPI_QKV_ROPE = 4 /* QKV projection: columns are [Q | K | V] x heads x 128; per head apply the QK RMS-norm and
                            split-half RoPE of h3_dit_w4a8_qkv_rope_f32 (h3_dit_w4a8.c:2805) and write
                            Q / K / V [m, heads, 128] (d_y = Q, d_key, d_value), bf16 */
};
/* Addition (no counterpart in the reference): exchange-free Ulysses.  Every rank maps the gathered
 * Q / K / V buffers and the attention-row buffer of all ranks (CUDA IPC), so that the QKV GEMM epilogue
 * and the attention epilogue store each (row, head) slice straight into the memory of the rank that
 * needs it, over NVLink, instead of packing, exchanging through NCCL and unpacking.  Filled by
 * h3b_ulysses_direct_setup (below, with the other sequence-parallel calls). */
typedef struct h3b_ulysses_direct {
    int ulysses, rank;
    size_t seq_local, heads, head_dim;   /* heads = all heads; a rank attends heads / ulysses of them */
    void *q, *k, *v;   /* this rank's gathered Q, K, V: [ulysses*seq_local, heads/ulysses, head_dim] bf16 */
    void *att;         /* this rank's attention rows: [seq_local, heads, head_dim] bf16 */
    void *peer_q[8], *peer_k[8], *peer_v[8], *peer_att[8];   /* the same buffers of rank p, mapped here */
} h3b_ulysses_direct;

typedef struct h3b_gemm_epi {
    int kind;                    /* H3B_EPI_* */
    int out_dtype;               /* H3B_F32 / H3B_BF16 / H3B_F16 / H3B_I32 (plain only) */
    const void *d_residual;      /* gate: [m,n] in out_dtype */
    const float *d_modulation;   /* gate: [mod_rows, slots, n] or NULL */
    const uint32_t *d_row_map;   /* gate: [m] or NULL (identity) */
    size_t slots, gate_slot;
    /* H3B_EPI_QKV_ROPE only */
    void *d_key, *d_value;       /* with d_y = query */
    const float *d_q_norm, *d_k_norm;     /* [128] */
    const float *d_rope_cos, *d_rope_sin; /* [m, rope_half]; NULL with rope_half = 0 */
    size_t rope_half;            /* <= 64 */
    float epsilon;
    int round_qkv;               /* 1: round the projection to out_dtype before the norm (what a stored
                                    intermediate would have been) */
    /* H3B_EPI_QKV_ROPE, optional: row r, head h goes to scatter->peer_{q,k,v}[h / hl] at row
     * rank*seq_local + r, head h % hl (hl = heads / ulysses); d_y / d_key / d_value are then unused.
     * d_rope_cos / d_rope_sin are the rows of THIS rank ([m, rope_half]). */
    const h3b_ulysses_direct *scatter;
    /* Plain / gate / swiglu / gelu, optional: already-scaled LoRA delta [m, n] f32 added to the dequantised
     * value before the activation or gate (h3_dit_fused_epi.h:85-141: gate += lora[c], up += lora[w+c];
     * br += lora[c]).  lora_ready: a cudaEvent_t the launch waits for, or NULL. */
    const float *d_lora;
    void *lora_ready;
} h3b_gemm_epi;
/* Work decomposition of the persistent int8 GEMM (no GPU needed): `tiles` 256 x 256 tiles on `pairs` CTA pairs with
 * `k_blocks` 128-byte blocks of K each; mode as H3B_GEMM_SPLITK (0 whole tiles, 1 the library's estimate, n >= 2 forced).
 * Pair p runs items p, p + pairs, ...; item `item` covers k-blocks [kb0, kb1) of tile `tile`, slice 0 of a tile runs its
 * epilogue after adding the other slices' sums.  Returns 0 if `item` is past the last item and item outputs are asked. */
int h3b_gemm_i8_plan(size_t tiles, size_t pairs, size_t k_blocks, int mode, size_t item, int *items_total, int *tail_first,
                     int *split, int *tile, int *kb0, int *kb1, int *slice);
/* d_x_i8 [m,k] codes, d_act_scales [m]; d_y is [m,n] ([m,n/2] for swiglu). */
int h3b_gemm_i8_dev(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight, const int8_t *d_x_i8,
                    const float *d_act_scales, size_t m, void *d_y, const h3b_gemm_epi *epi,
                    char *error, size_t error_size);
/* Per-row absmax INT8 quantisation (reference rule, h3_w4a8_dequant.c:671):
 * d_x [m,k] in `dtype`; writes codes [m,k] and scales [m]. */
int h3b_quantize_act_int8_dev(h3_cuda *cuda, const void *d_x, int dtype, size_t m, size_t k,
                              int8_t *d_q, float *d_scales, char *error, size_t error_size);
/* One launch, one CTA per row:  (gate ->) RMSNorm * w (-> modulate) (-> round to dtype)
 * (-> ConvRot per group) (-> per-row INT8 quant).  Optional parts are switched off by NULL
 * pointers / zero values: d_branch (no gate stage), d_modulation (plain RMSNorm), identity=1
 * (no normalisation at all: quantise / rotate d_x as it is), convrot_gs=0 (no rotation).
 * Outputs that are NULL are not written. */
typedef struct h3b_norm_args {
    const void *d_x;             /* [rows,width] residual / input, `dtype` */
    const void *d_branch;        /* optional [rows,width], `dtype` */
    const float *d_norm_w;       /* [width] or NULL (ones) */
    const float *d_modulation;   /* [mod_rows, slots, width] or NULL */
    const uint32_t *d_row_map;   /* [rows] or NULL (identity) */
    size_t rows, width, slots, gate_slot, shift_slot, scale_slot;
    float epsilon;
    int dtype;                   /* H3B_F32 / H3B_BF16 / H3B_F16: type of x, branch, gated, normed */
    int identity;                /* 1: skip RMSNorm and modulation */
    int convrot_gs;              /* 0, 4, 16, 64 or 256: Hadamard group size applied before the quant */
    void *d_gated;               /* out: residual + branch*gate, `dtype` */
    void *d_normed;              /* out: normalised (and modulated) row, `dtype` */
    float *d_rot;                /* out: rotated row, f32 (h3_cuda_convrot_act_f32_dd) */
    int8_t *d_q;                 /* out: INT8 codes */
    float *d_scales;             /* out, with d_q: per-row scale */
    uint8_t *d_fp4;              /* out: NVFP4 codes of the final row values [rows, width/2] (width % 64 == 0) */
    uint8_t *d_sf;               /* out, with d_fp4: UE4M3 scales, layout and size of h3_cuda_nvfp4_sf_bytes */
} h3b_norm_args;
int h3b_norm_dev(h3_cuda *cuda, const h3b_norm_args *args, char *error, size_t error_size);

/* -------------------------------------------------------------- elementwise */

int h3_cuda_adaln_f32(h3_cuda *cuda, const float *x, const float *norm_w, const float *modulation,
                      const uint32_t *row_map, size_t rows, size_t width, size_t slots,
                      size_t mod_rows, size_t shift_slot, size_t scale_slot, float epsilon,
                      float *out, double *op_ms, char *error, size_t error_size);   /* :694 */
int h3_cuda_gate_f32(h3_cuda *cuda, const float *residual, const float *branch,
                     const float *modulation, const uint32_t *row_map, size_t rows, size_t width,
                     size_t slots, size_t mod_rows, size_t gate_slot, float *out, double *op_ms,
                     char *error, size_t error_size);                               /* :700 */
int h3_cuda_swiglu_f32(h3_cuda *cuda, const float *fused, size_t rows, size_t width, float *out,
                       double *op_ms, char *error, size_t error_size);              /* :705 */
int h3_cuda_qkv_rope_f32(h3_cuda *cuda, const float *qkv, const float *q_norm, const float *k_norm,
                         const float *rope_cos, const float *rope_sin, size_t seq, size_t heads,
                         size_t head_dim, size_t rope_half, float epsilon, float *query, float *key,
                         float *value, double *op_ms, char *error, size_t error_size); /* :708 */
int h3_cuda_adaln_f32_dev(h3_cuda *cuda, const float *d_x, const float *d_norm_w,
                          const float *d_modulation, const uint32_t *d_row_map, size_t rows,
                          size_t width, size_t slots, size_t shift_slot, size_t scale_slot,
                          float epsilon, float *d_out, double *op_ms, char *error,
                          size_t error_size);                                       /* :716 */
int h3_cuda_gate_f32_dev(h3_cuda *cuda, const float *d_residual, const float *d_branch,
                         const float *d_modulation, const uint32_t *d_row_map, size_t rows,
                         size_t width, size_t slots, size_t gate_slot, float *d_out, double *op_ms,
                         char *error, size_t error_size);                           /* :722 */
int h3_cuda_swiglu_f32_dev(h3_cuda *cuda, const float *d_fused, size_t rows, size_t width,
                           float *d_out, double *op_ms, char *error, size_t error_size); /* :727 */
int h3_cuda_gate_adaln_f32_dev(h3_cuda *cuda, const float *d_residual, const float *d_branch,
                               const float *d_norm_w, const float *d_modulation,
                               const uint32_t *d_row_map, size_t rows, size_t width, size_t slots,
                               size_t gate_slot, size_t shift_slot, size_t scale_slot, float epsilon,
                               float *d_gated, float *d_normed, double *op_ms, char *error,
                               size_t error_size);                                  /* :733 */
int h3_cuda_rms_norm_f32_dev(h3_cuda *cuda, const float *d_x, const float *d_w, size_t rows,
                             size_t width, float eps, float *d_out, char *error,
                             size_t error_size);                                    /* :242 */
int h3_cuda_qkv_rope_f32_dev(h3_cuda *cuda, const float *d_qkv, const float *d_q_norm,
                             const float *d_k_norm, const float *d_rope_cos,
                             const float *d_rope_sin, size_t seq, size_t heads, size_t head_dim,
                             size_t rope_half, float epsilon, float *d_query, float *d_key,
                             float *d_value, double *op_ms, char *error, size_t error_size); /* :748 */
int h3_cuda_qkv_rope_f32_dev_layout(h3_cuda *cuda, const float *d_qkv, const float *d_q_norm,
                                    const float *d_k_norm, const float *d_rope_cos,
                                    const float *d_rope_sin, size_t seq, size_t heads,
                                    size_t head_dim, size_t rope_half, float epsilon, int grouped,
                                    int split_half, float *d_query, float *d_key, float *d_value,
                                    double *op_ms, char *error, size_t error_size);  /* :755 */
int h3_cuda_f32_to_f16_dev(h3_cuda *cuda, const float *d_in, void *d_out_half, size_t n, char *error,
                           size_t error_size);                                      /* :196 */
int h3_cuda_f16_to_f32_dev(h3_cuda *cuda, const void *d_in_half, float *d_out, size_t n, char *error,
                           size_t error_size);                                      /* :198 */
/* Additions: typed variants (dtype = H3B_F32 / H3B_BF16 for in and out). */
int h3b_qkv_rope_dev(h3_cuda *cuda, const void *d_qkv, int in_dtype, const float *d_q_norm,
                     const float *d_k_norm, const float *d_rope_cos, const float *d_rope_sin,
                     size_t seq, size_t heads, size_t head_dim, size_t rope_half, float epsilon,
                     int grouped, int split_half, void *d_query, void *d_key, void *d_value,
                     int out_dtype, char *error, size_t error_size);
int h3b_cast_dev(h3_cuda *cuda, const void *d_in, int in_dtype, void *d_out, int out_dtype, size_t n,
                 char *error, size_t error_size);
/* out[o] = b[o] + sum_i W[o,i] t[i] on the device (adaLN modulation projection,
 * h3_dit_w4a8.c:2236 h3_dit_w4a8_adaln_project_f32 without the optional SiLU). */
int h3b_adaln_project_dev(h3_cuda *cuda, const float *d_w, const float *d_b, size_t out_dim,
                          size_t in_dim, const float *d_t_feat, float *d_out, char *error,
                          size_t error_size);
int h3b_gelu_tanh_dev(h3_cuda *cuda, const void *d_in, void *d_out, int dtype, size_t n, char *error,
                      size_t error_size);

/* ------------------------------------------- the step on either side of the chain */

/* d_y[m,n] = d_x[m,k] @ d_weight[n,k]^T, all f32 on the device (h3_gpu_cuda.h:120; the patch
 * embeddings and final heads call it through dense_f32_cuda_to_dev, h3_dit_w4a8.c:5370). */
int h3_cuda_gemm_f32_dd(h3_cuda *cuda, const float *d_x, const float *d_weight, size_t m, size_t n,
                        size_t k, float *d_y, double *gemm_ms, char *error, size_t error_size);
/* d_y = alpha * (d_x @ d_weight^T) + beta * d_y (h3_gpu_cuda.h:125, :130).  The LoRA delta of a linear is
 * t = x A^T (h3_cuda_gemm_f32_dd) followed by delta = scale * t B^T + beta * delta (this call), as
 * h3_dit_w4a8.c:1036-1050 issues them; the delta then enters the INT8 GEMM epilogue as d_lora.  The _tf32_
 * name computes in full f32 here. */
int h3_cuda_gemm_f32_dd_ex(h3_cuda *cuda, const float *d_x, const float *d_weight, size_t m, size_t n,
                           size_t k, float *d_y, float alpha, float beta, double *gemm_ms, char *error,
                           size_t error_size);
int h3_cuda_gemm_f32_dd_tf32_ex(h3_cuda *cuda, const float *d_x, const float *d_weight, size_t m,
                                size_t n, size_t k, float *d_y, float alpha, float beta, char *error,
                                size_t error_size);
/* d_y[r,c] += d_bias[c] (h3_gpu_cuda.h:263). */
int h3_cuda_bias_add_f32_dev(h3_cuda *cuda, float *d_y, const float *d_bias, size_t rows, size_t width,
                             char *error, size_t error_size);
/* The two calls above in one launch: y = x W^T + b (h3_dit_w4a8.c:5298 h3_dit_w4a8_dense_f32);
 * d_bias may be NULL.  Patch embedding: m = tokens, n = hidden, k = 96 (video) or 32 (audio). */
int h3b_dense_f32_dev(h3_cuda *cuda, const float *d_x, const float *d_weight, const float *d_bias,
                      size_t m, size_t n, size_t k, float *d_y, char *error, size_t error_size);
/* Final head (h3_dit_w4a8.c:5578 final_head_cuda): adaLN of every token with shift = d_modulation[0,:]
 * and scale = d_modulation[1,:] (one modulation row of two slots), then y = normed W^T + b with
 * W [out_dim, hidden].  d_scratch: h3b_final_head_scratch_bytes(seq, hidden) bytes, 16-byte aligned. */
size_t h3b_final_head_scratch_bytes(size_t seq, size_t hidden);
int h3b_final_head_f32_dev(h3_cuda *cuda, const float *d_x, const float *d_norm_w,
                           const float *d_modulation, size_t seq, size_t hidden, const float *d_weight,
                           const float *d_bias, size_t out_dim, float epsilon, void *d_scratch,
                           size_t scratch_bytes, float *d_y, char *error, size_t error_size);
/* sample += (sigma - sigma_next) * velocity on the device; refuses a pair that is not finite,
 * not decreasing or negative, like h3_dit_w4a8.c:8822 h3_dit_w4a8_euler_step_f32. */
int h3b_euler_step_f32_dev(h3_cuda *cuda, float *d_sample, const float *d_velocity, size_t count,
                           float sigma, float sigma_next, char *error, size_t error_size);

/* ---------------------------------------------------------------- attention */

/* F32 Q/K/V/out on the device, [seq, heads, head_dim]; computed in bf16 on the
 * tensor cores with f32 softmax and accumulation.  h3_gpu_cuda.h:566, 579 */
int h3_cuda_sdpa_f32_dev(h3_cuda *cuda, const float *d_query, const float *d_key,
                         const float *d_value, size_t seq, size_t heads, size_t head_dim, float scale,
                         float *d_out, double *sdpa_ms, char *error, size_t error_size);
int h3_cuda_sdpa_f16_dev(h3_cuda *cuda, const float *d_query, const float *d_key,
                         const float *d_value, size_t seq, size_t heads, size_t head_dim, float scale,
                         float *d_out, double *sdpa_ms, char *error, size_t error_size);
int h3_cuda_sdpa_f16_dev_ex(h3_cuda *cuda, const float *d_query, const float *d_key,
                            const float *d_value, size_t seq, size_t heads, size_t head_dim,
                            float scale, int attn_window, float *d_out, double *sdpa_ms,
                            char *backend_out, size_t backend_out_size, char *error,
                            size_t error_size);                                     /* :601 */
/* QK-norm + RoPE into 16-bit staging, then attention.  h3_gpu_cuda.h:771 */
int h3_cuda_qkv_rope_sdpa_f16_dev(h3_cuda *cuda, const float *d_qkv, const float *d_q_norm,
                                  const float *d_k_norm, const float *d_rope_cos,
                                  const float *d_rope_sin, size_t seq, size_t heads, size_t head_dim,
                                  size_t rope_half, float epsilon, float scale, int attn_window,
                                  float *d_attn_out, double *rope_ms, double *sdpa_ms,
                                  char *backend_out, size_t backend_out_size, char *error,
                                  size_t error_size);
const char *h3_cuda_sdpa_backend_name(void);                                        /* :643 */
const char *h3_cuda_sdpa_last_backend_name(void);                                   /* :680 */
/* Addition: bf16 attention with explicit row strides (elements) and separate
 * query / key counts (cross-attention).  q [lq, heads, 128] at q_stride per row,
 * k/v [lk, heads, 128]; out [lq, heads*128] bf16 at o_stride.  Non-causal. */
int h3b_sdpa_bf16_dev(h3_cuda *cuda, const void *d_q, size_t q_stride, const void *d_k,
                      size_t k_stride, const void *d_v, size_t v_stride, size_t lq, size_t lk,
                      size_t heads, size_t head_dim, float scale, void *d_out, size_t o_stride,
                      char *error, size_t error_size);
/* Addition: the general form.  dtype H3B_BF16 or H3B_F16 for all four tensors; row and head strides in elements
 * (multiples of 8); e.g. [heads, rows, 128] tensors have row stride 128 and head stride rows * 128. */
int h3b_sdpa_strided_dev(h3_cuda *cuda, int dtype, const void *d_q, size_t q_row_stride, size_t q_head_stride,
                         const void *d_k, size_t k_row_stride, size_t k_head_stride, const void *d_v, size_t v_row_stride,
                         size_t v_head_stride, size_t lq, size_t lk, size_t heads, size_t head_dim, float scale, void *d_out,
                         size_t o_row_stride, size_t o_head_stride, char *error, size_t error_size);
/* Addition: the same attention over this rank's heads/ulysses heads of the gathered sequence
 * (scatter->q, ->k, ->v, lq = lk = seq_real), each output row stored into scatter->peer_att of the
 * rank that owns the row, at head rank*hl + h. */
int h3b_sdpa_bf16_scatter_dev(h3_cuda *cuda, const h3b_ulysses_direct *scatter, size_t seq_real,
                              float scale, char *error, size_t error_size);

/* -------------------------------------------------------------------- NVFP4 */

typedef struct h3_cuda_nvfp4_weight h3_cuda_nvfp4_weight;                           /* :445 */
size_t h3_cuda_nvfp4_sf_bytes(size_t rows, size_t k);                               /* :450 */
int h3_cuda_quantize_act_nvfp4_dev(h3_cuda *cuda, const float *d_x, size_t m, size_t k,
                                   uint8_t *d_x_fp4, uint8_t *d_sf, char *error,
                                   size_t error_size);                              /* :433 */
/* Block-scaled FP4 GEMM: A = weights [n,k] packed E2M1, B = activations [m,k] packed E2M1, both with
 * 128x4-blocked UE4M3 scales; out bf16 [m,n].  K a multiple of 64.  h3_gpu_cuda.h:424 */
int h3_cuda_gemm_fp4_bs_dev(h3_cuda *cuda, const uint8_t *d_w_fp4, const uint8_t *d_sf_w,
                            const uint8_t *d_x_fp4, const uint8_t *d_sf_x, size_t m, size_t n, size_t k,
                            void *d_y_bf16, double *gemm_ms, char *error, size_t error_size);
/* On success the library owns both host buffers (malloc'ed by the caller; copied, then released with free()); on failure
 * the caller keeps them.  h3_gpu_cuda.h:437-444 */
int h3_cuda_nvfp4_weight_create(h3_cuda *cuda, const uint8_t *packed_host,
                                const uint8_t *sf_swizzled_host, float scale2, size_t n, size_t k,
                                h3_cuda_nvfp4_weight **out, double *h2d_ms, char *error,
                                size_t error_size);                                 /* :452 */
int h3_cuda_nvfp4_weight_ensure_ready(h3_cuda_nvfp4_weight *weight, char *error, size_t error_size); /* :457 */
void h3_cuda_nvfp4_weight_free(h3_cuda *cuda, h3_cuda_nvfp4_weight *w);             /* :459 */
const uint8_t *h3_cuda_nvfp4_weight_packed(const h3_cuda_nvfp4_weight *w);          /* :460 */
const uint8_t *h3_cuda_nvfp4_weight_sf(const h3_cuda_nvfp4_weight *w);              /* :461 */
float h3_cuda_nvfp4_weight_scale2(const h3_cuda_nvfp4_weight *w);                   /* :462 */
size_t h3_cuda_nvfp4_weight_n(const h3_cuda_nvfp4_weight *w);                       /* :463 */
size_t h3_cuda_nvfp4_weight_k(const h3_cuda_nvfp4_weight *w);                       /* :464 */
size_t h3_cuda_nvfp4_gemm_scratch_bytes(size_t m, size_t n, size_t k);              /* :468 */
/* f32 activations in: NVFP4 quantise + block-scaled GEMM + epilogue (scale2 * act_scale applied to the
 * f32 accumulator).  scratch NULL = library scratch.  d_lora must be NULL.  h3_gpu_cuda.h:480-504 */
int h3_cuda_gemm_fp4_w_act_dev(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const float *d_x,
                               float act_scale, size_t m, float *d_y_f32, uint8_t *scratch,
                               double *prep_ms, double *gemm_ms, char *error, size_t error_size,
                               const char *tag);
int h3_cuda_gemm_fp4_w_act_dev_swiglu(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const float *d_x,
                                      float act_scale, size_t m, const float *d_lora, float *d_y_f32,
                                      uint8_t *scratch, double *prep_ms, double *gemm_ms, char *error,
                                      size_t error_size, const char *tag);
int h3_cuda_gemm_fp4_w_act_dev_gate(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const float *d_x,
                                    float act_scale, size_t m, const float *d_residual,
                                    const float *d_modulation, const uint32_t *d_row_map, size_t slots,
                                    size_t gate_slot, const float *d_lora, float *d_y_f32,
                                    uint8_t *scratch, double *prep_ms, double *gemm_ms, char *error,
                                    size_t error_size, const char *tag);
/* Addition: block-scaled GEMM with a scalar alpha and f32 or bf16 output. */
int h3b_gemm_fp4_dev(h3_cuda *cuda, const uint8_t *d_w_fp4, const uint8_t *d_sf_w, const uint8_t *d_x_fp4,
                     const uint8_t *d_sf_x, size_t m, size_t n, size_t k, float alpha, void *d_y,
                     int out_dtype, char *error, size_t error_size);

/* Addition: the same GEMM with SwiGLU on the f32 accumulators in the epilogue: weight rows [0, n/2) are the gate,
 * [n/2, n) the up projection; d_y [m, n/2] = silu(alpha acc_gate) * (alpha acc_up).  n % 256 == 0.  This is the
 * reference's chain FC1 (h3_cutlass_nvfp4_fc1_f32_run) + SwiGLU (h3_dit_nvfp4_chain.cu:201-277) as one kernel. */
int h3b_gemm_fp4_swiglu_dev(h3_cuda *cuda, const uint8_t *d_w_fp4, const uint8_t *d_sf_w, const uint8_t *d_x_fp4,
                            const uint8_t *d_sf_x, size_t m, size_t n, size_t k, float alpha, void *d_y,
                            int out_dtype, char *error, size_t error_size);

/* Addition: NVFP4 weight object x activations that are ALREADY NVFP4 codes + scales (for instance written by
 * h3b_norm_dev's d_fp4 / d_sf outputs, which fuse RMSNorm, modulation, ConvRot and the quantisation into one pass
 * over the row): epi 0 plain, 1 SwiGLU on the f32 accumulators (N % 256 == 0), 2 gate + residual.  The accumulator
 * is scaled by weight scale2 * act_scale.  d_y H3B_F32 or H3B_BF16 (the residual has the same type). */
int h3b_gemm_fp4_w_preq_dev(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const uint8_t *d_x_fp4,
                            const uint8_t *d_sf_x, size_t m, float act_scale, int epi, const void *d_residual,
                            const float *d_modulation, const uint32_t *d_row_map, size_t slots, size_t gate_slot,
                            void *d_y, int out_dtype, char *error, size_t error_size);
/* The QKV projection on pre-quantised activations with QK-norm and split-half RoPE in the epilogue, on the f32
 * accumulators: Q, K, V bf16 [m, heads, 128]; N of the weight = 3 * heads * 128, rope_half 0, 48 or 64, tables
 * [m, rope_half] f32 (h3_dit_w4a8_qkv_rope_f32, h3_dit_w4a8.c:2805-2890, fused behind nvfp4_gemm_dispatch, :3519). */
int h3b_gemm_fp4_w_preq_qkv_rope_dev(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const uint8_t *d_x_fp4,
                                     const uint8_t *d_sf_x, size_t m, float act_scale, const float *d_q_norm,
                                     const float *d_k_norm, const float *d_cos, const float *d_sin, size_t rope_half,
                                     size_t heads, float epsilon, void *d_q, void *d_k, void *d_v, char *error,
                                     size_t error_size);

/* ------------------------------------------- the rest of the reference's operator surface
 * Everything below keeps the reference's name and signature (h3_gpu_cuda.h line cited per entry) so that the
 * reference's own DiT host (h3_dit_w4a8.c) links against this library without a change. */

/* housekeeping */
int h3_cuda_copy_stream_synchronize(h3_cuda *cuda, char *error, size_t error_size);                 /* :334 */
/* moves the f32 dense GEMMs (LoRA deltas) onto side stream 1 / back to the op stream */
int h3_cuda_cublas_use_side(h3_cuda *cuda, int on, char *error, size_t error_size);                  /* :220 */
void *h3_cuda_cublas_stream(const h3_cuda *cuda);                                                    /* :223 */
int h3_cuda_recreate_blas(h3_cuda *cuda, char *error, size_t error_size);                            /* :60 */
int h3_cuda_dit_scratch_rehome(h3_cuda *cuda, char *error, size_t error_size);                       /* :58 */
int h3_cuda_dit_scratch_check(h3_cuda *cuda, char *error, size_t error_size);                        /* :59 */
int h3_cuda_host_register(void *p, size_t bytes, char *error, size_t error_size);                    /* :321 */
void h3_cuda_host_unregister(void *p);                                                               /* :322 */

/* f32 GEMM y = x W^T with host x / host or device W (:91, :115), and with f16 weights + alpha/beta (:183) */
int h3_cuda_gemm_f32(h3_cuda *cuda, const float *x, const float *weight, size_t m, size_t n, size_t k, float *y,
                     double *gemm_ms, char *error, size_t error_size);
int h3_cuda_gemm_f32_dw(h3_cuda *cuda, const float *x, const float *d_weight, size_t m, size_t n, size_t k, float *y,
                        double *gemm_ms, char *error, size_t error_size);
int h3_cuda_gemm_f32in_f16w_f32out_dd_ex(h3_cuda *cuda, const float *d_x_f32, const void *d_w_h, size_t m, size_t n,
                                         size_t k, float *d_y_f32, float alpha, float beta, char *error,
                                         size_t error_size);

/* ConvRot on f16 activations (:149); ConvRot + per-row INT8 into library scratch for a following _dev_pre_q
 * GEMM (:143): *out_xi8 [ceil128(m), k], *out_scales [ceil128(m)], valid until the next call that grows it */
int h3_cuda_convrot_act_f16_dd(h3_cuda *cuda, const void *d_x_half, size_t m, size_t k, int convrot_groupsize,
                               void *d_y_half, char *error, size_t error_size);
int h3_cuda_epi_fuse_ink_prep_fc2(h3_cuda *cuda, const float *d_swiglu, size_t m, size_t k, int convrot_groupsize,
                                  int8_t **out_xi8, float **out_scales, char *error, size_t error_size);

/* NVFP4 FC1 -> SwiGLU -> requantise -> FC2 chain (:519-549).  _fc1_f32_run: block-scaled GEMM with the f32
 * accumulators written out [m, n]; _swiglu_requant: silu(acc_scale * gate (+lora)) * (acc_scale * up (+lora)) ->
 * E2M1 + UE4M3 scales in the layout of h3_cuda_quantize_act_nvfp4_dev; _pre_q: FC2 on those codes with the gate +
 * residual epilogue (d_bf16_scratch is not used, d_lora must be NULL). */
int h3_cutlass_nvfp4_fc1_f32_run(h3_cuda *cuda, const uint8_t *d_w_fp4, const uint8_t *d_sf_w, const uint8_t *d_x_fp4,
                                 const uint8_t *d_sf_x, size_t m, size_t n, size_t k, float *d_acc_f32, double *gemm_ms,
                                 char *error, size_t error_size);
int h3_nvfp4_swiglu_requant_dev(h3_cuda *cuda, const float *d_acc_f32, float acc_scale, const float *d_lora, size_t m,
                                size_t ffn, uint8_t *d_act_fp4, uint8_t *d_sf_act, char *error, size_t error_size);
size_t h3_cuda_nvfp4_chain_scratch_bytes(size_t m, size_t kdim, size_t ffn);
int h3_cuda_gemm_fp4_pre_q_dev(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const uint8_t *d_x_fp4,
                               const uint8_t *d_sf_x, size_t m, const float *d_residual, const float *d_modulation,
                               const uint32_t *d_row_map, size_t slots, size_t gate_slot, const float *d_lora,
                               float *d_y_f32, void *d_bf16_scratch, double *gemm_ms, char *error, size_t error_size,
                               const char *tag);
int h3_nvfp4_debug_nan_dev(void);                                                                    /* :554 */
void h3_nvfp4_debug_scan_dev(h3_cuda *cuda, const void *ptr, size_t n, const char *kind, const char *tag,
                             const char *stage);                                                     /* :555 */

/* attention: host-tensor forms (:562, :573, :610), explicit-layout and f16-QKV forms of QK-norm + RoPE +
 * attention (:779-801), history keys / values appended to the next such call and a gather of current K / V rows
 * (:815-819, f16 [rows, heads, head_dim]) */
int h3_cuda_sdpa_f32(h3_cuda *cuda, const float *query, const float *key, const float *value, size_t seq, size_t heads,
                     size_t head_dim, float scale, float *out, double *sdpa_ms, char *error, size_t error_size);
int h3_cuda_sdpa_f16(h3_cuda *cuda, const float *query, const float *key, const float *value, size_t seq, size_t heads,
                     size_t head_dim, float scale, float *out, double *sdpa_ms, char *error, size_t error_size);
int h3_cuda_sdpa_f16_ex(h3_cuda *cuda, const float *query, const float *key, const float *value, size_t seq, size_t heads,
                        size_t head_dim, float scale, int attn_window, float *out, double *sdpa_ms, char *backend_out,
                        size_t backend_out_size, char *error, size_t error_size);
int h3_cuda_qkv_rope_sdpa_f16_dev_layout(h3_cuda *cuda, const float *d_qkv, const float *d_q_norm, const float *d_k_norm,
                                         const float *d_rope_cos, const float *d_rope_sin, size_t seq, size_t heads,
                                         size_t head_dim, size_t rope_half, float epsilon, float scale, int attn_window,
                                         int grouped, int split_half, float *d_attn_out, double *rope_ms, double *sdpa_ms,
                                         char *backend_out, size_t backend_out_size, char *error, size_t error_size);
int h3_cuda_qkv_rope_sdpa_f16_dev_layout_f16qkv(h3_cuda *cuda, const void *d_qkv_half, const float *d_q_norm,
                                                const float *d_k_norm, const float *d_rope_cos, const float *d_rope_sin,
                                                size_t seq, size_t heads, size_t head_dim, size_t rope_half, float epsilon,
                                                float scale, int attn_window, int grouped, int split_half, float *d_attn_out,
                                                double *rope_ms, double *sdpa_ms, char *backend_out, size_t backend_out_size,
                                                char *error, size_t error_size);
int h3_cuda_qkv_rope_sdpa_f16_dev_f16qkv(h3_cuda *cuda, const void *d_qkv_half, const float *d_q_norm, const float *d_k_norm,
                                         const float *d_rope_cos, const float *d_rope_sin, size_t seq, size_t heads,
                                         size_t head_dim, size_t rope_half, float epsilon, float scale, int attn_window,
                                         float *d_attn_out, double *rope_ms, double *sdpa_ms, char *backend_out,
                                         size_t backend_out_size, char *error, size_t error_size);
void h3_cuda_sdpa_bind_kvcat(const void *d_k_hist, const void *d_v_hist, size_t hist_n);
void h3_cuda_sdpa_bind_kvsave(void *d_k_save, void *d_v_save, const uint32_t *d_idx, size_t save_n);
void h3_cuda_sdpa_clear_kvext(void);

/* token reduction (:827-858): pool pairs of rows, expand back with the delta against a baseline */
int h3_cuda_token_pool_f32(h3_cuda *cuda, const float *input, size_t full_rows, const uint32_t *pairs,
                           const uint32_t *baseline_idx, size_t reduced_rows, size_t baseline_rows, size_t width,
                           float *output, float **d_original_out, float **d_baseline_out, double *op_ms, char *error,
                           size_t error_size);
int h3_cuda_token_expand_f32(h3_cuda *cuda, const float *d_original, const float *reduced, const float *d_baseline,
                             const uint32_t *baseline_idx, const uint32_t *parents, size_t full_rows, size_t reduced_rows,
                             size_t baseline_rows, size_t width, uint32_t video_start, uint32_t video_rows,
                             float update_scale, float *output, double *op_ms, char *error, size_t error_size);
int h3_cuda_token_pool_f32_dev(h3_cuda *cuda, const float *d_input, size_t full_rows, const uint32_t *pairs,
                               const uint32_t *baseline_idx, size_t reduced_rows, size_t baseline_rows, size_t width,
                               float *d_output, float *d_original, float *d_baseline, double *op_ms, char *error,
                               size_t error_size);
int h3_cuda_token_expand_f32_dev(h3_cuda *cuda, const float *d_original, const float *d_reduced, const float *d_baseline,
                                 const uint32_t *baseline_idx, const uint32_t *parents, size_t full_rows,
                                 size_t reduced_rows, size_t baseline_rows, size_t width, uint32_t video_start,
                                 uint32_t video_rows, float update_scale, float *d_output, double *op_ms, char *error,
                                 size_t error_size);

/* optional features of the reference that this library does not have: switching them on is refused with
 * "... not supported by libh3_b200", everything else is a harmless success (:590-595, :653, :685, :689;
 * h3_nvfp4_cuda.h:26-44 for the text encoder's four) */
int h3_cuda_dist_attn_configure(h3_cuda *cuda, size_t seq, size_t video_start, size_t video_seq, int grid_t, int grid_h,
                                int grid_w, float scale, float temporal_weight, int enabled, char *error,
                                size_t error_size);
void h3_cuda_dist_attn_clear(void);
int h3_cuda_dist_attn_active(void);
void h3_cuda_sol_cute_set_step(int step);
void h3_cuda_sol_profile_add_unpack(double ms);
size_t h3_cuda_sage3_pool_bytes(void);
int h3_nvfp4_cuda_enabled(void);
void h3_nvfp4_cuda_cache_clear(void);
int h3_nvfp4_cuda_encode_text_layers(const void *store, float *hidden, size_t tokens, unsigned n_layers, char *error,
                                     size_t error_size);
int h3_nvfp4_cuda_gqa_causal(const float *q, const float *k, const float *v, size_t tokens, size_t q_heads, size_t kv_heads,
                             size_t head_dim, float *out, char *error, size_t error_size);

/* ---------------------------------------------------------- DiT block / chain */

/* Additions.  The reference's block-level entry points (h3_dit_w4a8.h:527
 * h3_dit_w4a8_block_forward_f32, :609 h3_dit_w4a8_layers_forward_f32) are bound
 * to its checkpoint store and fixed geometry; these take the geometry and the
 * weight objects explicitly and keep the same argument meaning otherwise
 * (x/y [seq, dim], modulation [mod_rows, 6, dim], row_map [seq], rope tables
 * [seq, rope_half]).  The host side is plain C (csrc/h3b_dit.c). */
enum {
    H3B_BLOCK_REFERENCE = 0, /* adaLN-QKV-RoPE-SDPA-out*gate | adaLN-fc1-SwiGLU-fc2*gate   (h3_dit_w4a8.c:4291) */
    H3B_BLOCK_CROSS_GELU = 1 /* + rms_norm / cross-attention(text) / residual, FFN with tanh-GELU            */
};
enum { /* linear slots of a block */
    H3B_LIN_QKV = 0, H3B_LIN_OUT = 1, H3B_LIN_FC1 = 2, H3B_LIN_FC2 = 3,
    H3B_LIN_CROSS_Q = 4, H3B_LIN_CROSS_KV = 5, H3B_LIN_CROSS_OUT = 6, H3B_LIN_COUNT = 7
};
typedef struct h3b_dit_config {
    int kind;          /* H3B_BLOCK_* */
    int stream_dtype;  /* H3B_F32 (reference CUDA path) or H3B_BF16 residual stream */
    int convrot_gs;    /* 0 or 256: activation rotation before every quantised linear */
    size_t dim, heads, head_dim, ffn, rope_half, n_blocks, mod_rows, t_dim;
    float eps;
} h3b_dit_config;
typedef struct h3b_dit h3b_dit;

h3b_dit *h3b_dit_create(h3_cuda *cuda, const h3b_dit_config *cfg, char *error, size_t error_size);
void h3b_dit_free(h3b_dit *dit);
/* The context borrows the weight object (the caller frees it after h3b_dit_free). */
int h3b_dit_set_linear(h3b_dit *dit, unsigned block, int which, const h3_cuda_w4a8_weight *weight,
                       char *error, size_t error_size);
/* Per-linear choice of the NVFP4 form of a weight (which = H3B_LIN_QKV, _OUT, _FC1 or _FC2), the decision the
 * reference's nvfp4_gemm_dispatch takes per linear (h3_dit_w4a8.c:3519-3590, call sites :3623-3641): the linear then
 * runs ConvRot -> NVFP4 activation quantisation -> block-scaled GEMM with the plain (QKV), SwiGLU (FC1) or
 * gate (OUT, FC2) epilogue.  Reference block on an f32 stream only.  weight == NULL returns the linear to its INT8
 * weight; a linear needs one of the two.  The weight object is borrowed. */
int h3b_dit_set_linear_nvfp4(h3b_dit *dit, unsigned block, int which, const h3_cuda_nvfp4_weight *weight,
                             char *error, size_t error_size);
/* ---- checkpoints: the safetensors container (the reference's reader: h3_safetensors.c; its INT8-ConvRot DiT store:
 * h3_dit_int8.c:120-206) -> device layouts.  The file is mapped read-only; a tensor is a view into the mapping. */
typedef struct h3b_ckpt h3b_ckpt;
typedef struct h3b_ckpt_tensor {
    const char *name;     /* owned by the checkpoint */
    char dtype[8];        /* "I8", "F32", "F16", "BF16", "U8", ... as written in the file */
    int rank;
    size_t shape[4];
    const void *data;
    size_t bytes;
} h3b_ckpt_tensor;
h3b_ckpt *h3b_ckpt_open(const char *path, char *error, size_t error_size);
void h3b_ckpt_close(h3b_ckpt *ckpt);
size_t h3b_ckpt_count(const h3b_ckpt *ckpt);
int h3b_ckpt_get(const h3b_ckpt *ckpt, size_t index, h3b_ckpt_tensor *out);
int h3b_ckpt_find(const h3b_ckpt *ckpt, const char *name, h3b_ckpt_tensor *out);
/* Block `src_block` of an INT8-ConvRot DiT checkpoint -> block `dst_block` of a reference-kind context: the four
 * linears blocks.N.{attn.qkv_proj, attn.out_proj, mlp.fc1, mlp.fc2}.weight (I8 [n, k]) + .weight_scale (F32 [n] or
 * [n, 1]) become resident INT8 weights owned by the context (names: h3_dit_int8.h:37-40, h3_dit_int8.c:173);
 * blocks.N.norm1/norm2.weight, blocks.N.attn.q_norm/k_norm.weight and blocks.N.adaln_proj.linear.weight/.bias (F32)
 * are uploaded as h3_dit_w4a8_load_block_aux_hdr reads them (h3_dit_w4a8.c:2056-2117). */
int h3b_dit_load_int8_convrot_block(h3b_dit *dit, const h3b_ckpt *ckpt, unsigned src_block, unsigned dst_block,
                                    char *error, size_t error_size);
/* The same for the reference's W4A8 checkpoint (h3_w4a8.c:75-115): per linear `weight` I8 [n, k/2] (two 4-bit codes per
 * byte), `weight_codebook` F32[16], `weight_s_rel` F8_E4M3 [n, k/16] and `weight_s_channel` F32[n], decoded on the
 * device by the reference's rule (h3_w4a8_dequant.c:65-118) into resident INT8 weights owned by the context; norms and
 * adaLN projection as above. */
int h3b_dit_load_w4a8_block(h3b_dit *dit, const h3b_ckpt *ckpt, unsigned src_block, unsigned dst_block, char *error,
                            size_t error_size);
/* The reference's NVFP4 sidecar (h3_dit_w4a8.c:3158-3274): per linear `weight_fp4` U8 [n, k/2], `weight_sf` (the
 * 128x4-blocked UE4M3 scales, h3_cuda_nvfp4_sf_bytes(n, k) bytes) and an optional F32 scalar `weight_scale2`.
 * `linears` is the mask of linears to take from it (bit 0 QKV, 1 OUT, 2 FC1, 3 FC2); they become NVFP4 weights owned
 * by the context and are selected as h3b_dit_set_linear_nvfp4 does.  A sidecar carries no norms: load the block from
 * the checkpoint it accompanies as well (first or afterwards). */
int h3b_dit_load_nvfp4_block(h3b_dit *dit, const h3b_ckpt *sidecar, unsigned src_block, unsigned dst_block,
                             unsigned linears, char *error, size_t error_size);
/* Host f32 vectors, copied to the device: norm1/norm2 [dim], q_norm/k_norm [head_dim],
 * norm_cross [dim] (cross block only, else NULL). */
int h3b_dit_set_block_aux(h3b_dit *dit, unsigned block, const float *norm1, const float *norm2,
                          const float *q_norm, const float *k_norm, const float *norm_cross,
                          char *error, size_t error_size);
/* adaLN projection of one block: W [mod_rows*6*dim, t_dim], b [mod_rows*6*dim] (host f32). */
int h3b_dit_set_adaln(h3b_dit *dit, unsigned block, const float *w, const float *b, char *error,
                      size_t error_size);
/* modulation[block] = W t_feat + b for every block, on the device (the reference does this on the
 * host per block and step, h3_dit_w4a8.c:2236).  d_t_feat: [t_dim] f32 on the device. */
int h3b_dit_project_modulation(h3b_dit *dit, const float *d_t_feat, char *error, size_t error_size);
/* Device pointer of the projected modulation of `block`: [mod_rows, 6, dim] f32. */
const float *h3b_dit_modulation(h3b_dit *dit, unsigned block);
/* Sizes the activation workspace for `seq` rows (+ `text_seq` text rows); afterwards the forward
 * calls allocate nothing for sequences up to that size. */
int h3b_dit_reserve(h3b_dit *dit, size_t seq, size_t text_seq, char *error, size_t error_size);
/* One block, device tensors in the stream dtype.  d_modulation NULL = the projected one.
 * d_text [text_seq, dim] (cross block only).  d_x and d_y may alias. */
int h3b_dit_block_forward_dev(h3b_dit *dit, unsigned block, const void *d_x, size_t seq,
                              const float *d_modulation, const uint32_t *d_row_map,
                              const float *d_rope_cos, const float *d_rope_sin, const void *d_text,
                              size_t text_seq, void *d_y, char *error, size_t error_size);
/* Blocks [first, first+n) chained on the device; uses the projected modulation. */
int h3b_dit_layers_forward_dev(h3b_dit *dit, unsigned first_block, unsigned n_blocks, const void *d_x,
                               size_t seq, const uint32_t *d_row_map, const float *d_rope_cos,
                               const float *d_rope_sin, const void *d_text, size_t text_seq, void *d_y,
                               char *error, size_t error_size);
/* The same chain as ONE CUDA graph launch (the reference's whole-step graph, h3_dit_w4a8.c:4390 under
 * H3_DIT_W4A8_CUDA_GRAPH).  The first call for a set of arguments runs the chain eagerly, then captures it on the
 * handle's op stream (which must be a real stream, not the legacy default one) and instantiates the graph; later
 * calls with the same arguments replay it; other arguments re-capture.  Not available with a communicator
 * attached.  _graph_nodes: nodes of the captured graph, 0 if none. */
int h3b_dit_layers_forward_graph_dev(h3b_dit *dit, unsigned first_block, unsigned n_blocks, const void *d_x,
                                     size_t seq, const uint32_t *d_row_map, const float *d_rope_cos,
                                     const float *d_rope_sin, const void *d_text, size_t text_seq, void *d_y,
                                     char *error, size_t error_size);
size_t h3b_dit_graph_nodes(const h3b_dit *dit);
/* Host f32 in / host f32 out, like h3_dit_w4a8_layers_forward_f32: uploads x (and text), the
 * time feature, row map and rope tables, runs the chain, downloads y.  row_map NULL = all zeros. */
int h3b_dit_layers_forward_f32(h3b_dit *dit, unsigned first_block, unsigned n_blocks,
                               const float *t_feat, const float *x, size_t seq,
                               const uint32_t *row_map, const float *rope_cos, const float *rope_sin,
                               const float *text, size_t text_seq, float *y, char *error,
                               size_t error_size);
/* Kernel launches one block forward issues (for launch accounting). */
int h3b_dit_launches_per_block(const h3b_dit *dit);

/* Host-side tables of a step, same names and arithmetic as the reference (bit-identical results).
 * Positions of the video tokens: latent dims (latent_t, latent_h, latent_w), token grid latent_h/2 x
 * latent_w/2 per frame, time starting at text_len.  h3_dit_w4a8.h:382, body h3_dit_w4a8.c:2496 */
int h3_dit_w4a8_fill_metal_video_pos(size_t text_len, int latent_t, int latent_h, int latent_w, float *pos_t,
                                     float *pos_h, float *pos_w, char *error, size_t error_size);
float h3_dit_w4a8_video_span_sum(int latent_t);                                     /* h3_dit_w4a8.h:395 */
/* cos/sin [seq, 48]: 3 axes (t, h*spatial_scale, w*spatial_scale) x 16 frequencies.
 * h3_dit_w4a8.h:366, body h3_dit_w4a8.c:2412 */
int h3_dit_w4a8_rope_tables_f32(const float *inv_freq, size_t seq, const float *pos_t, const float *pos_h,
                                const float *pos_w, float spatial_scale, float *cos_out, float *sin_out, char *error,
                                size_t error_size);
/* Row of the time-feature table for noise level sigma in [0,1] (indexed by 1 - sigma; the switch
 * H3_DIT_T_ROW_BY_SIGMA=1 indexes by sigma).  h3_dit_w4a8.h:545, body h3_dit_w4a8.c:5229 */
size_t h3_dit_w4a8_t_row_from_sigma(float sigma, size_t t_table_rows);
/* Addition: the two calls above for a token grid grid_t x grid_h x grid_w in one call, plus `pad_rows`
 * trailing rows of angle zero (cos 1, sin 0) for a sequence padded for sequence parallelism. */
int h3b_dit_video_rope_tables(const float *inv_freq16, size_t text_len, int grid_t, int grid_h, int grid_w,
                              float spatial_scale, size_t pad_rows, float *cos_out, float *sin_out, char *error,
                              size_t error_size);

/* ------------------------------------------------- Metal-twin signatures (h3_dit.h:94-140), thin shims
 * Row-order conversions and the reuse schedule are implemented (host arithmetic, int 1 = ok / 0 = bad
 * arguments; the schedule returns the number of selected steps or -1).  The calls that need the Apple-GPU
 * transformer object fail with "Metal path: unavailable on this box". */
typedef struct h3_dit h3_dit;                                                                 /* h3_dit.h:11 */
typedef void (*h3_dit_progress)(const char *phase, int completed, int total, void *opaque);   /* h3_dit.h:13 */
int h3_dit_patchify_video(const float *latent, int channels, int time, int height, int width, float *rows,
                          size_t row_elements);                                               /* :131 */
int h3_dit_unpatchify_video(const float *rows, int channels, int time, int height, int width, float *latent,
                            size_t latent_elements);                                          /* :134 */
int h3_dit_pack_audio(const float *latent, int channels, int time, float *rows, size_t row_elements);     /* :137 */
int h3_dit_unpack_audio(const float *rows, int channels, int time, float *latent, size_t latent_elements); /* :139 */
int h3_dit_reuse_schedule(int steps, int reuse_interval, uint8_t *selected, size_t selected_count);       /* :124 */
int h3_dit_forward(h3_dit *dit, int step, const float *video_latent, const float *audio_latent, float *video_velocity,
                   float *audio_velocity, char *error, size_t error_size);                    /* :94 */
int h3_dit_denoise_euler(h3_dit *dit, float *video_latent, float *audio_latent, int reuse_interval,
                         h3_dit_progress progress, void *progress_opaque, char *error, size_t error_size); /* :106 */
size_t h3_dit_video_elements(const h3_dit *dit);                                              /* :88 */
size_t h3_dit_audio_elements(const h3_dit *dit);                                              /* :89 */
void h3_dit_free(h3_dit *dit);                                                                /* :77 */

/* ------------------------------------------------------------------ Ulysses */

enum { H3_ULYSSES_PACKED_ALIGN = 64 };                                              /* h3_ulysses.h:10 */
typedef struct h3_ulysses_cfg {                                                     /* h3_ulysses.h:12-19 */
    int tp_size;
    int ulysses;
    int ring;
    int rank;
    int world_size;
    void *comm;
} h3_ulysses_cfg;
int h3_ulysses_validate(int heads, int packed_align, int tp, int ulysses, int ring, char *err,
                        size_t err_size);                                           /* h3_ulysses.h:21 */
size_t h3_ulysses_pad_seq(size_t seq, int align);                                   /* :23 */
size_t h3_ulysses_local_rows(size_t seq_pad, int ulysses, int rank);                /* :24 */

/* Communication (h3_ulysses_comm.h:13-33), same six calls.  dtype_bytes 2 or 4; buffers are device
 * pointers; d_in [seq_local, 3*heads*head_dim] -> d_out [seq_pad, 3*(heads/U)*head_dim] for QKV and
 * d_in [seq_pad, (heads/U)*head_dim] -> d_out [seq_local, heads*head_dim] for the attention output;
 * in and out may alias.  The exchange runs on the communicator's own stream, ordered after the rank's
 * compute stream (h3_ulysses_comm_set_compute) and before its later work; nothing blocks the host. */
int h3_ulysses_comm_init(h3_ulysses_cfg *cfg, const int *device_ids, int n_dev, char *err,
                         size_t err_size);                                          /* h3_ulysses_comm.h:13 */
void h3_ulysses_comm_destroy(h3_ulysses_cfg *cfg);                                  /* :15 */
int h3_ulysses_comm_bind(h3_ulysses_cfg *cfg, int rank, const void *d_in, void *d_out, char *err,
                         size_t err_size);                                          /* :18 */
int h3_ulysses_comm_set_compute(h3_ulysses_cfg *cfg, int rank, void *stream, char *err,
                                size_t err_size);                                   /* :22 */
int h3_ulysses_a2a_qkv(h3_ulysses_cfg *cfg, const void *d_in, void *d_out, size_t seq_local,
                       size_t heads, size_t head_dim, int dtype_bytes, char *err,
                       size_t err_size);                                            /* :26 */
int h3_ulysses_a2a_attn_out(h3_ulysses_cfg *cfg, const void *d_in, void *d_out, size_t seq_local,
                            size_t heads, size_t head_dim, int dtype_bytes, char *err,
                            size_t err_size);                                       /* :31 */
/* Additions for one process per GPU: rank 0 makes a 128-byte id, the caller distributes it (any
 * transport), every rank joins with it.  With world_size 1 no communicator is made. */
int h3b_ulysses_unique_id(void *out128, char *err, size_t err_size);
int h3b_ulysses_comm_init_rank(h3_ulysses_cfg *cfg, int rank, int world_size, const void *unique_id128,
                               int device, char *err, size_t err_size);
/* Additions, one process per GPU only.  _direct_setup allocates this rank's four buffers (zeroed),
 * exchanges their IPC handles through the communicator and maps the peers'; it is collective (every rank
 * calls it with the same sizes) and synchronises the device.  Once set up, the sequence-parallel chain
 * (h3b_dit_layers_forward_ulysses_*) of a context with matching geometry uses the direct stores and
 * two h3b_ulysses_barrier calls per block instead of the two exchanges.  _direct_get returns NULL when
 * nothing is set up or the path is switched off.  _barrier: all ranks, enqueued on the rank's compute stream;
 * work enqueued after it on any rank starts only when every rank's earlier work is done.  It is a one-warp
 * kernel that writes an epoch into a flag word in every peer's buffer and waits (bounded) for the peers'
 * words; H3B_ULYSSES_BARRIER=nccl in the environment at set-up time (the same on every rank) selects a
 * one-word NCCL all-reduce instead.  _check synchronises the compute stream and reports whether a barrier gave up waiting. */
int h3b_ulysses_direct_setup(h3_ulysses_cfg *cfg, size_t seq_local, size_t heads, size_t head_dim,
                             char *err, size_t err_size);
/* Addition: the set-up protocol of _direct_setup with its five steps supplied by the caller (the library's own
 * steps allocate, exchange IPC handles through NCCL, map, all-reduce the outcome, roll back).  Order: prepare
 * (local) -> gather (collective, ALWAYS reached, told whether prepare worked) -> map_peers (local, only when all
 * is well so far) -> agree (collective, ALWAYS reached: minimum of the ranks' outcomes) -> rollback on every
 * rank unless all agreed.  Every step returns 1 = ok / 0 = failed.  Exported so that the decision logic can be
 * exercised with stand-in steps on a CPU. */
typedef struct h3b_ulysses_setup_steps {
    void *ctx;
    int (*prepare)(void *ctx);
    int (*gather)(void *ctx, int have_handle);
    int (*map_peers)(void *ctx);
    int (*agree)(void *ctx, int ok, int *all_ok);
    void (*rollback)(void *ctx);
} h3b_ulysses_setup_steps;
int h3b_ulysses_setup_protocol(const h3b_ulysses_setup_steps *steps);
const h3b_ulysses_direct *h3b_ulysses_direct_get(const h3_ulysses_cfg *cfg);
/* Switches the use of a set-up direct path off (0) or back on (1); the mappings stay.  For launchers that
 * found the set-up failing on some rank and fall back to the exchange on all of them. */
void h3b_ulysses_direct_enable(h3_ulysses_cfg *cfg, int on);
int h3b_ulysses_barrier(h3_ulysses_cfg *cfg, char *err, size_t err_size);
int h3b_ulysses_check(h3_ulysses_cfg *cfg, int *status_out, char *err, size_t err_size);
/* Runs the flag-barrier kernel on the current device against a local stand-in for a second rank: once with
 * the peer's word already set (*status_arrived = 0) and once with a peer that never arrives, where the wait
 * ends after budget_cycles SM clocks (*status_absent = 6).  Needs no communicator and no second GPU. */
int h3b_ulysses_barrier_selftest(long long budget_cycles, int *status_arrived, int *status_absent, char *err,
                                 size_t err_size);
/* Host f32 rows of this rank in and out (see h3b_dit_layers_forward_f32); rope tables cover all
 * U*seq_local rows. */
int h3b_dit_layers_forward_ulysses_f32(h3b_dit *dit, unsigned first_block, unsigned n_blocks,
                                       const float *t_feat, const float *x_local, size_t seq_local,
                                       size_t seq_real, const uint32_t *row_map,
                                       const float *rope_cos_full, const float *rope_sin_full,
                                       const float *text, size_t text_seq, float *y_local, char *error,
                                       size_t error_size);
/* Attaches an initialised per-rank communicator to a block context (the reference's
 * h3_dit_w4a8_set_ulysses, h3_dit_w4a8.h:305, for one rank).  NULL detaches. */
int h3b_dit_set_ulysses(h3b_dit *dit, h3_ulysses_cfg *cfg, char *error, size_t error_size);
/* Sequence-parallel chain on this rank's rows (h3_dit_w4a8.c:6261 layers_forward_ulysses, one rank):
 * d_x / d_y [seq_local, dim]; rope tables for ALL seq_pad = U*seq_local rows; only the first
 * seq_real rows of the gathered sequence enter attention, pad rows of its output are zero. */
int h3b_dit_layers_forward_ulysses_dev(h3b_dit *dit, unsigned first_block, unsigned n_blocks,
                                       const void *d_x, size_t seq_local, size_t seq_real,
                                       const uint32_t *d_row_map, const float *d_rope_cos_full,
                                       const float *d_rope_sin_full, const void *d_text,
                                       size_t text_seq, void *d_y, char *error, size_t error_size);

#ifdef __cplusplus
}
#endif
#endif
