// Internal declarations shared by the translation units of libh3_b200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/h3_b200.h"
#include "../../include/h3b_plugin.h"

struct h3_cuda {
    int device;
    cudaStream_t op_stream;      // NULL = legacy default stream
    cudaStream_t side[4];        // non-blocking side streams (weight uploads)
    int quiet;
    int graph_capture;
    int sm_count;
    int *d_status;               // device status word, see h3b_ptx.cuh
    h3_cuda_device_info info;
    cudaEvent_t ev0, ev1;
    unsigned long long launches;
    // library scratch, grown on demand (never while graph_capture is set)
    void *act_q;   size_t act_q_bytes;     // int8 activation codes
    void *act_s;   size_t act_s_bytes;     // per-row activation scales
    void *act_rot; size_t act_rot_bytes;   // ConvRot output (f32)
    void *attn;    size_t attn_bytes;      // 16-bit Q/K/V/O staging for the f32 attention entry points
    void *rq;      size_t rq_bytes;        // codes + scales handed out by h3_cuda_epi_fuse_ink_prep_fc2
    void *kvx;     size_t kvx_bytes;       // K/V with bound history appended (h3_cuda_sdpa_bind_kvcat)
    void *wtmp;    size_t wtmp_bytes;      // f32 copy of 16-bit weights (mixed-precision dense GEMM)
    void *splitk;  size_t splitk_bytes;    // int32 sums + counters of the int8 GEMM's split tail tiles (the counters are
                                           // zero between launches: the kernel that uses them resets them)
    int blas_side;                         // f32 GEMMs run on side[1] (h3_cuda_cublas_use_side)
    int pregrown;
    // optional per-launch timing (h3b_cuda_profile_begin / _end)
    int prof_on, prof_n, prof_cap;
    cudaEvent_t *prof_ev;        // 2 events per recorded launch
    int *prof_cls;
};

struct h3_cuda_w4a8_weight {
    h3_cuda *cuda;
    int device;
    size_t n, k;
    int8_t *d_w;        // [n,k] resident int8
    float *d_s;         // [n]
    CUtensorMap tmap_b;  // [n,k] int8, box 128 (k) x 128 (n), 128B swizzle
    int tmap_ok;
    cudaEvent_t ready;
    int pending;
    void *own_host_w;   // host staging owned until ensure_ready
    void *own_host_s;
};

namespace h3b {

int fail(char *error, size_t error_size, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what, char *error, size_t error_size);
#define H3B_CUDA_OK(call, what)                                              \
    do {                                                                     \
        cudaError_t e__ = (call);                                            \
        if (e__ != cudaSuccess) return h3b::cuda_fail(e__, what, error, error_size); \
    } while (0)

// grow a scratch slot of the handle to at least `bytes` (fails under graph capture)
int grow(h3_cuda *cuda, void **slot, size_t *have, size_t bytes, char *error, size_t error_size);

struct Timer {   // optional per-op timing, honouring quiet mode
    h3_cuda *cuda;
    double *ms;
    bool on;
    Timer(h3_cuda *c, double *out);
    void stop();
};

// kernel classes of the per-launch profile
enum { PROF_GEMM = 0, PROF_ATTN = 1, PROF_ROWS = 2, PROF_ROPE = 3, PROF_OTHER = 4, PROF_CLASSES = 5 };
// Brackets one kernel launch with an event pair while profiling is on.
struct ProfScope {
    h3_cuda *cuda;
    int slot;
    ProfScope(h3_cuda *c, int cls);
    ~ProfScope();
};

static inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }
static inline size_t dtype_bytes(int dt) { return dt == H3B_F32 || dt == H3B_I32 ? 4 : 2; }

// ---- kernels' host launchers (each returns 1/0 like the public API)
int launch_norm(h3_cuda *cuda, const h3b_norm_args *a, char *error, size_t error_size);
int launch_quant(h3_cuda *cuda, const void *x, int dtype, size_t m, size_t k, int8_t *q, float *scales,
                 char *error, size_t error_size);
int launch_gate(h3_cuda *cuda, const void *res, const void *branch, const float *mod, const uint32_t *row_map,
                size_t rows, size_t width, size_t slots, size_t gate_slot, void *out, int dtype, char *error,
                size_t error_size);
int launch_swiglu(h3_cuda *cuda, const void *fused, size_t rows, size_t width, void *out, int dtype, char *error,
                  size_t error_size);
int launch_convrot(h3_cuda *cuda, const float *x, size_t m, size_t k, int gs, float *y, char *error,
                   size_t error_size);
int launch_gemm_i8(h3_cuda *cuda, const h3_cuda_w4a8_weight *w, const int8_t *x, const float *a, size_t m,
                   void *y, const h3b_gemm_epi *epi, char *error, size_t error_size);
// gate: 0 plain, 1 residual + gate, 2 SwiGLU, 3 QKV with QK-norm and RoPE (y = Q, the rest in `qkv`)
struct Fp4QkvArgs {
    void *k, *v;
    const float *q_norm, *k_norm, *cosT, *sinT;
    int rope_half;
    size_t heads;
    float eps;
};
int launch_gemm_nvfp4(h3_cuda *cuda, const uint8_t *w_fp4, const uint8_t *sf_w, const uint8_t *x_fp4, const uint8_t *sf_x,
                      size_t m, size_t n, size_t k, float alpha, void *y, int out_dtype, int gate, const void *residual,
                      const float *mod, const uint32_t *row_map, size_t slots, size_t gate_slot, char *error,
                      size_t error_size, const Fp4QkvArgs *qkv = nullptr);
// stream the f32 dense GEMMs run on: the op stream, or side stream 1 while h3_cuda_cublas_use_side is on
static inline cudaStream_t dense_stream(const h3_cuda *c) { return c->blas_side ? c->side[1] : c->op_stream; }
int launch_sdpa_bf16(h3_cuda *cuda, const void *q, size_t qs, const void *k, size_t ks, const void *v, size_t vs,
                     size_t lq, size_t lk, size_t heads, size_t hd, float scale, void *out, size_t os,
                     char *error, size_t error_size);

int launch_sdpa_f16(h3_cuda *cuda, const void *q, size_t qs, const void *k, size_t ks, const void *v, size_t vs,
                    size_t lq, size_t lk, size_t heads, size_t hd, float scale, void *out, size_t os,
                    char *error, size_t error_size);

}  // namespace h3b
