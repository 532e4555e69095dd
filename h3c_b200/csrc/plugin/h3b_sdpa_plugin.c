/* libh3_b200_sdpa.so -- this library's attention kernel behind the reference's dlopen'd attention-plugin ABI
 * (four C symbols looked up with dlsym: tools/h3_sage3_embed.c:94-200, typedefs h3_gpu_cuda.cu:7745-7752).
 * With H3_CUDA_SDPA_BACKEND=sage3 and H3_SAGE3_LIB pointing here, the UNMODIFIED reference runs its attention on
 * this kernel without relinking: the plugin owns four f16 buffers in [heads, seq, 128] layout, the reference
 * copies its Q / K / V in, calls fwd, and copies O out (h3_gpu_cuda.cu:7895-8050).
 *
 * init     allocates (or re-binds) the buffers of one (seq, heads, dim) shape and returns their device addresses;
 *          the first two integer arguments after `scale` are unused by the ABI
 * fwd      runs softmax(Q K^T * scale) V over the bound buffers on the legacy default stream, like the
 *          reference's own copies around the call
 * fwd_ex   the same, and reports five timings (only the kernel's is measured here)
 * warmup   makes the shape ready ahead of time (allocation and first launch)
 */
#include <cuda_runtime_api.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../../include/h3_b200.h"

enum { MAX_SHAPES = 8 };   /* the reference keeps a pool of eight shapes (H3_SAGE3_POOL) */

typedef struct {
    int seq, heads, dim, device;
    float scale;
    void *q, *k, *v, *o;
} shape_t;

static shape_t g_shapes[MAX_SHAPES];
static int g_n_shapes;
static shape_t *g_bound;
static h3_cuda *g_cuda[16];

static int fail(char *error, size_t error_size, const char *fmt, ...) {
    if (error && error_size) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(error, error_size, fmt, ap);
        va_end(ap);
    }
    return 0;
}

static h3_cuda *handle_for_current_device(char *error, size_t error_size) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) {
        fail(error, error_size, "h3_b200 sdpa plugin: no usable current device");
        return NULL;
    }
    if (!g_cuda[dev]) g_cuda[dev] = h3_cuda_create(dev, error, error_size);   /* op stream NULL = legacy default stream */
    return g_cuda[dev];
}

static shape_t *bind_shape(int seq, int heads, int dim, float scale, char *error, size_t error_size) {
    int dev = 0, i;
    size_t bytes;
    shape_t *s;
    if (seq <= 0 || heads <= 0 || dim != 128) {
        fail(error, error_size, "h3_b200 sdpa plugin: needs seq > 0, heads > 0, head_dim 128 (got %d, %d, %d)", seq, heads, dim);
        return NULL;
    }
    if (!(scale > 0.0f)) {
        fail(error, error_size, "h3_b200 sdpa plugin: scale must be positive");
        return NULL;
    }
    if (!handle_for_current_device(error, error_size)) return NULL;
    cudaGetDevice(&dev);
    for (i = 0; i < g_n_shapes; i++) {
        s = &g_shapes[i];
        if (s->seq == seq && s->heads == heads && s->dim == dim && s->device == dev) {
            s->scale = scale;
            return s;
        }
    }
    if (g_n_shapes == MAX_SHAPES) {
        fail(error, error_size, "h3_b200 sdpa plugin: more than %d shapes", MAX_SHAPES);
        return NULL;
    }
    s = &g_shapes[g_n_shapes];
    memset(s, 0, sizeof(*s));
    bytes = (size_t)seq * (size_t)heads * (size_t)dim * 2;
    if (cudaMalloc(&s->q, bytes) != cudaSuccess || cudaMalloc(&s->k, bytes) != cudaSuccess ||
        cudaMalloc(&s->v, bytes) != cudaSuccess || cudaMalloc(&s->o, bytes) != cudaSuccess) {
        if (s->q) cudaFree(s->q);
        if (s->k) cudaFree(s->k);
        if (s->v) cudaFree(s->v);
        fail(error, error_size, "h3_b200 sdpa plugin: cudaMalloc of %zu bytes x 4 failed", bytes);
        return NULL;
    }
    s->seq = seq; s->heads = heads; s->dim = dim; s->device = dev; s->scale = scale;
    g_n_shapes++;
    return s;
}

int h3_sage3_init(const char *root, int seq, int heads, int dim, float scale, int unused0, int unused1, void **q_ptr,
                  void **k_ptr, void **v_ptr, void **o_ptr, char *backend, size_t backend_n, char *error,
                  size_t error_size) {
    shape_t *s;
    (void)root; (void)unused0; (void)unused1;
    if (!q_ptr || !k_ptr || !v_ptr || !o_ptr) return fail(error, error_size, "h3_b200 sdpa plugin: init null ptrs");
    s = bind_shape(seq, heads, dim, scale, error, error_size);
    if (!s) return 0;
    g_bound = s;
    *q_ptr = s->q; *k_ptr = s->k; *v_ptr = s->v; *o_ptr = s->o;
    if (backend && backend_n) snprintf(backend, backend_n, "h3_b200_tcgen05_flash_f16");
    return 1;
}

int h3_sage3_fwd_ex(char *error, size_t error_size, double *prep_ms, double *kern_ms, double *copy_ms, double *compile_ms,
                    double *host_ms) {
    shape_t *s = g_bound;
    h3_cuda *cuda;
    cudaEvent_t e0 = NULL, e1 = NULL;
    size_t head_stride;
    int ok;
    if (prep_ms) *prep_ms = 0.0;
    if (kern_ms) *kern_ms = 0.0;
    if (copy_ms) *copy_ms = 0.0;
    if (compile_ms) *compile_ms = 0.0;
    if (host_ms) *host_ms = 0.0;
    if (!s) return fail(error, error_size, "h3_b200 sdpa plugin: not inited");
    if (cudaSetDevice(s->device) != cudaSuccess) return fail(error, error_size, "h3_b200 sdpa plugin: cudaSetDevice failed");
    cuda = handle_for_current_device(error, error_size);
    if (!cuda) return 0;
    if (kern_ms && cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess) cudaEventRecord(e0, 0);
    head_stride = (size_t)s->seq * (size_t)s->dim;   /* [heads, seq, dim]: rows dim apart, heads seq * dim apart */
    ok = h3b_sdpa_strided_dev(cuda, H3B_F16, s->q, (size_t)s->dim, head_stride, s->k, (size_t)s->dim, head_stride, s->v,
                              (size_t)s->dim, head_stride, (size_t)s->seq, (size_t)s->seq, (size_t)s->heads, (size_t)s->dim,
                              s->scale, s->o, (size_t)s->dim, head_stride, error, error_size);
    if (e0 && e1) {
        float ms = 0.0f;
        cudaEventRecord(e1, 0);
        cudaEventSynchronize(e1);
        if (cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) *kern_ms = (double)ms;
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    return ok;
}

int h3_sage3_fwd(char *error, size_t error_size) { return h3_sage3_fwd_ex(error, error_size, NULL, NULL, NULL, NULL, NULL); }

int h3_sage3_warmup(const char *root, int seq, int heads, int dim, float scale, int unused0, int unused1, char *error,
                    size_t error_size) {
    shape_t *keep = g_bound, *s;
    int ok;
    (void)root; (void)unused0; (void)unused1;
    s = bind_shape(seq, heads, dim, scale, error, error_size);
    if (!s) return 0;
    /* one launch on zeroed inputs: loads the kernel and sets its shared-memory attribute */
    cudaMemset(s->q, 0, (size_t)seq * heads * dim * 2);
    cudaMemset(s->k, 0, (size_t)seq * heads * dim * 2);
    cudaMemset(s->v, 0, (size_t)seq * heads * dim * 2);
    g_bound = s;
    ok = h3_sage3_fwd(error, error_size) && cudaDeviceSynchronize() == cudaSuccess;
    g_bound = keep ? keep : s;
    return ok;
}
