// Host-buffer forms of the DiT elementwise operators: stage through device memory, run the
// device kernels, copy the result back (the reference's h3_cuda_*_f32 without the _dev suffix).
#include "h3b_internal.h"

using namespace h3b;

namespace {
struct Staged {
    h3_cuda *cuda;
    void *bufs[12];
    int n = 0;
    explicit Staged(h3_cuda *c) : cuda(c) {}
    ~Staged() {
        cudaStreamSynchronize(cuda->op_stream);
        for (int i = 0; i < n; i++) cudaFree(bufs[i]);
    }
    // device copy of a host array (NULL stays NULL)
    template <typename T>
    T *up(const T *host, size_t count, bool *ok) {
        if (!host) return NULL;
        void *d = NULL;
        if (cudaMalloc(&d, count * sizeof(T) + 16) != cudaSuccess) { *ok = false; return NULL; }
        bufs[n++] = d;
        if (cudaMemcpyAsync(d, host, count * sizeof(T), cudaMemcpyHostToDevice, cuda->op_stream) != cudaSuccess) *ok = false;
        return (T *)d;
    }
    template <typename T>
    T *out(size_t count, bool *ok) {
        void *d = NULL;
        if (cudaMalloc(&d, count * sizeof(T) + 16) != cudaSuccess) { *ok = false; return NULL; }
        bufs[n++] = d;
        return (T *)d;
    }
    int down(void *host, const void *dev, size_t bytes, char *error, size_t error_size) {
        H3B_CUDA_OK(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, cuda->op_stream), "copy back");
        H3B_CUDA_OK(cudaStreamSynchronize(cuda->op_stream), "cudaStreamSynchronize");
        return 1;
    }
};
}  // namespace

extern "C" {

int h3_cuda_adaln_f32(h3_cuda *cuda, const float *x, const float *norm_w, const float *modulation,
                      const uint32_t *row_map, size_t rows, size_t width, size_t slots, size_t mod_rows,
                      size_t shift_slot, size_t scale_slot, float epsilon, float *out, double *op_ms, char *error,
                      size_t error_size) {
    if (!cuda || !x || !norm_w || !modulation || !out || !width || !slots || !mod_rows)
        return fail(error, error_size, "invalid adaln arguments");
    bool ok = true;
    Staged s(cuda);
    float *dx = s.up(x, rows * width, &ok), *dw = s.up(norm_w, width, &ok);
    float *dm = s.up(modulation, mod_rows * slots * width, &ok);
    uint32_t *dr = s.up(row_map, rows, &ok);
    float *dy = s.out<float>(rows * width, &ok);
    if (!ok) return fail(error, error_size, "adaln: device staging failed");
    return h3_cuda_adaln_f32_dev(cuda, dx, dw, dm, dr, rows, width, slots, shift_slot, scale_slot, epsilon, dy, op_ms,
                                 error, error_size) &&
           s.down(out, dy, rows * width * sizeof(float), error, error_size);
}

int h3_cuda_gate_f32(h3_cuda *cuda, const float *residual, const float *branch, const float *modulation,
                     const uint32_t *row_map, size_t rows, size_t width, size_t slots, size_t mod_rows,
                     size_t gate_slot, float *out, double *op_ms, char *error, size_t error_size) {
    if (!cuda || !residual || !branch || !modulation || !out || !width || !slots || !mod_rows)
        return fail(error, error_size, "invalid gate arguments");
    bool ok = true;
    Staged s(cuda);
    float *dr = s.up(residual, rows * width, &ok), *db = s.up(branch, rows * width, &ok);
    float *dm = s.up(modulation, mod_rows * slots * width, &ok);
    uint32_t *dmap = s.up(row_map, rows, &ok);
    float *dy = s.out<float>(rows * width, &ok);
    if (!ok) return fail(error, error_size, "gate: device staging failed");
    return h3_cuda_gate_f32_dev(cuda, dr, db, dm, dmap, rows, width, slots, gate_slot, dy, op_ms, error, error_size) &&
           s.down(out, dy, rows * width * sizeof(float), error, error_size);
}

int h3_cuda_swiglu_f32(h3_cuda *cuda, const float *fused, size_t rows, size_t width, float *out, double *op_ms,
                       char *error, size_t error_size) {
    if (!cuda || !fused || !out || !width) return fail(error, error_size, "invalid swiglu arguments");
    bool ok = true;
    Staged s(cuda);
    float *df = s.up(fused, rows * width * 2, &ok);
    float *dy = s.out<float>(rows * width, &ok);
    if (!ok) return fail(error, error_size, "swiglu: device staging failed");
    return h3_cuda_swiglu_f32_dev(cuda, df, rows, width, dy, op_ms, error, error_size) &&
           s.down(out, dy, rows * width * sizeof(float), error, error_size);
}

int h3_cuda_qkv_rope_f32(h3_cuda *cuda, const float *qkv, const float *q_norm, const float *k_norm,
                         const float *rope_cos, const float *rope_sin, size_t seq, size_t heads, size_t head_dim,
                         size_t rope_half, float epsilon, float *query, float *key, float *value, double *op_ms,
                         char *error, size_t error_size) {
    if (!cuda || !qkv || !q_norm || !k_norm || !query || !key || !value || !seq || !heads || !head_dim)
        return fail(error, error_size, "invalid qkv_rope args");
    const size_t inner = heads * head_dim;
    bool ok = true;
    Staged s(cuda);
    float *dq = s.up(qkv, seq * inner * 3, &ok), *dqn = s.up(q_norm, head_dim, &ok), *dkn = s.up(k_norm, head_dim, &ok);
    float *dc = s.up(rope_cos, seq * rope_half, &ok), *ds = s.up(rope_sin, seq * rope_half, &ok);
    float *oq = s.out<float>(seq * inner, &ok), *ok_ = s.out<float>(seq * inner, &ok), *ov = s.out<float>(seq * inner, &ok);
    if (!ok) return fail(error, error_size, "qkv_rope: device staging failed");
    return h3_cuda_qkv_rope_f32_dev(cuda, dq, dqn, dkn, dc, ds, seq, heads, head_dim, rope_half, epsilon, oq, ok_, ov,
                                    op_ms, error, error_size) &&
           s.down(query, oq, seq * inner * sizeof(float), error, error_size) &&
           s.down(key, ok_, seq * inner * sizeof(float), error, error_size) &&
           s.down(value, ov, seq * inner * sizeof(float), error, error_size);
}

}  // extern "C"
