// Weight objects (resident INT8 [N,K] + per-channel scale) and the quantised
// linear entry points built on the tcgen05 GEMM.
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "h3b_internal.h"
#include "h3b_gemm_plan.h"
#include "h3b_ptx.cuh"

namespace h3b {

// float8_e4m3fn -> f32 (h3_w4a8_dequant.c:17-39)
__device__ __forceinline__ float e4m3fn_to_f32(uint8_t bits) {
    const int sign = bits >> 7, e = (bits >> 3) & 15, m = bits & 7;
    float v;
    if (e == 15 && m == 7) v = __int_as_float(0x7fc00000);
    else if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return sign ? -v : v;
}

// Packed nibbles -> INT8, one thread per packed byte (two weights):
// w = clamp(roundf(codebook[nibble] * e4m3(s_rel[n, k / group])), +-127); low nibble = even k
// (h3_w4a8_dequant.c:65-118).
__global__ void k_w4a8_unpack(const uint8_t *packed, const float *codebook, const uint8_t *s_rel, size_t n,
                              size_t k_half, int group, int8_t *out) {
    __shared__ float cb[16];
    if (threadIdx.x < 16) cb[threadIdx.x] = codebook[threadIdx.x];
    __syncthreads();
    const size_t total = n * k_half, k = k_half * 2, groups = k / (size_t)group;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / k_half, cb2 = i - row * k_half;
        const unsigned byte = packed[i];
        char2 o;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const size_t col = cb2 * 2 + h;
            const float s = e4m3fn_to_f32(s_rel[row * groups + col / (size_t)group]);
            float v = roundf(__fmul_rn(cb[h ? (byte >> 4) : (byte & 15u)], s));
            v = fminf(fmaxf(v, -127.0f), 127.0f);
            if (h) o.y = (signed char)(int)v; else o.x = (signed char)(int)v;
        }
        *reinterpret_cast<char2 *>(out + row * k + cb2 * 2) = o;
    }
}

// Symmetric int4 (two's complement nibbles, f16 scale per `group` along K) -> resident INT8 with a
// per-channel scale: s_ch = max|s q| / 127, w = clamp(roundf((s q) * (1 / s_ch))).  One CTA per row.
__global__ void __launch_bounds__(256) k_w4g_decode(const uint8_t *packed, const __half *scales, size_t k,
                                                    int group, int8_t *out, float *s_channel) {
    __shared__ float red[8];
    const size_t row = blockIdx.x, groups = k / (size_t)group;
    const uint8_t *src = packed + row * (k / 2);
    float amax = 0.0f;
    for (size_t c = threadIdx.x; c < k; c += blockDim.x) {
        const unsigned byte = src[c >> 1];
        int q = (int)((c & 1) ? (byte >> 4) : (byte & 15u));
        if (q > 7) q -= 16;
        amax = fmaxf(amax, fabsf(__fmul_rn(__half2float(scales[row * groups + c / (size_t)group]), (float)q)));
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, red[i]);
    const float sc = amax > 0.0f ? amax / 127.0f : 1.0f;
    const float inv = 1.0f / sc;
    if (threadIdx.x == 0) s_channel[row] = sc;
    for (size_t c = threadIdx.x; c < k; c += blockDim.x) {
        const unsigned byte = src[c >> 1];
        int q = (int)((c & 1) ? (byte >> 4) : (byte & 15u));
        if (q > 7) q -= 16;
        float v = roundf(__fmul_rn(__fmul_rn(__half2float(scales[row * groups + c / (size_t)group]), (float)q), inv));
        v = fminf(fmaxf(v, -127.0f), 127.0f);
        out[row * k + c] = (int8_t)(int)v;
    }
}

static int weight_alloc(h3_cuda *cuda, size_t n, size_t k, h3_cuda_w4a8_weight **out, char *error,
                        size_t error_size) {
    if (!cuda || !out || !n || !k) return fail(error, error_size, "weight: invalid arguments");
    h3_cuda_w4a8_weight *w = (h3_cuda_w4a8_weight *)calloc(1, sizeof(*w));
    if (!w) return fail(error, error_size, "weight: out of host memory");
    w->cuda = cuda; w->device = cuda->device; w->n = n; w->k = k;
    cudaSetDevice(cuda->device);
    if (cudaMalloc((void **)&w->d_w, n * k) != cudaSuccess || cudaMalloc((void **)&w->d_s, n * sizeof(float)) != cudaSuccess ||
        cudaEventCreateWithFlags(&w->ready, cudaEventDisableTiming) != cudaSuccess) {
        cudaError_t e = cudaGetLastError();
        if (w->d_w) cudaFree(w->d_w);
        if (w->d_s) cudaFree(w->d_s);
        free(w);
        return cuda_fail(e, "weight: device allocation", error, error_size);
    }
    if (k % 16 == 0) {
        int rc = h3b_encode_tmap_2d(&w->tmap_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->d_w, k, n, k, 128, 128,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
        w->tmap_ok = rc == 0;
    }
    *out = w;
    return 1;
}

}  // namespace h3b

using namespace h3b;

extern "C" {

void h3_cuda_w4a8_weight_free(h3_cuda_w4a8_weight *w) {
    if (!w) return;
    cudaSetDevice(w->device);
    if (w->pending) cudaEventSynchronize(w->ready);
    if (w->own_host_w) free(w->own_host_w);
    if (w->own_host_s) free(w->own_host_s);
    if (w->ready) cudaEventDestroy(w->ready);
    if (w->d_w) cudaFree(w->d_w);
    if (w->d_s) cudaFree(w->d_s);
    free(w);
}

int h3_cuda_w4a8_weight_create(h3_cuda *cuda, const int8_t *packed_host, size_t n, size_t k_half,
                               const float *codebook16, const uint8_t *s_rel_f8, const float *s_channel,
                               int group_size, h3_cuda_w4a8_weight **out, double *unpack_ms, double *h2d_ms,
                               char *error, size_t error_size) {
    if (out) *out = NULL;
    if (!cuda || !packed_host || !codebook16 || !s_rel_f8 || !s_channel || !out || !n || !k_half)
        return fail(error, error_size, "invalid w4a8_weight_create arguments");
    if (group_size < 4 || (group_size % 16 != 0 && 16 % group_size != 0))
        return fail(error, error_size, "unsupported group_size=%d", group_size);
    const size_t k = k_half * 2;
    if (k % (size_t)group_size) return fail(error, error_size, "K=%zu not divisible by group_size=%d", k, group_size);
    const size_t groups = k / (size_t)group_size;
    h3_cuda_w4a8_weight *w = NULL;
    if (!weight_alloc(cuda, n, k, &w, error, error_size)) return 0;
    uint8_t *d_packed = NULL, *d_srel = NULL;
    float *d_cb = NULL;
    int ok = 0;
    cudaStream_t st = cuda->op_stream;
    do {
        if (cudaMalloc((void **)&d_packed, n * k_half) != cudaSuccess || cudaMalloc((void **)&d_srel, n * groups) != cudaSuccess ||
            cudaMalloc((void **)&d_cb, 16 * sizeof(float)) != cudaSuccess) {
            cuda_fail(cudaGetLastError(), "w4a8 staging allocation", error, error_size);
            break;
        }
        Timer th(cuda, h2d_ms);
        cudaError_t ec = cudaMemcpyAsync(d_packed, packed_host, n * k_half, cudaMemcpyHostToDevice, st);
        if (ec == cudaSuccess) ec = cudaMemcpyAsync(d_srel, s_rel_f8, n * groups, cudaMemcpyHostToDevice, st);
        if (ec == cudaSuccess) ec = cudaMemcpyAsync(d_cb, codebook16, 16 * sizeof(float), cudaMemcpyHostToDevice, st);
        if (ec == cudaSuccess) ec = cudaMemcpyAsync(w->d_s, s_channel, n * sizeof(float), cudaMemcpyHostToDevice, st);
        th.stop();
        if (ec != cudaSuccess) {
            cuda_fail(ec, "w4a8 weight H2D", error, error_size);
            break;
        }
        Timer tu(cuda, unpack_ms);
        size_t total = n * k_half;
        unsigned grid = (unsigned)(ceil_div(total, 256) > (size_t)cuda->sm_count * 32 ? (size_t)cuda->sm_count * 32
                                                                                       : ceil_div(total, 256));
        k_w4a8_unpack<<<grid, 256, 0, st>>>(d_packed, d_cb, d_srel, n, k_half, group_size, w->d_w);
        cuda->launches++;
        tu.stop();
        cudaError_t e = cudaStreamSynchronize(st);   // staging buffers and host pointers are released below
        if (e != cudaSuccess) {
            cuda_fail(e, "w4a8 unpack", error, error_size);
            break;
        }
        ok = 1;
    } while (0);
    if (d_packed) cudaFree(d_packed);
    if (d_srel) cudaFree(d_srel);
    if (d_cb) cudaFree(d_cb);
    if (!ok) {
        h3_cuda_w4a8_weight_free(w);
        return 0;
    }
    *out = w;
    return 1;
}

int h3b_w4g_weight_create(h3_cuda *cuda, const uint8_t *packed_host, const uint16_t *scales_f16, size_t n, size_t k,
                          int group, h3_cuda_w4a8_weight **out, char *error, size_t error_size) {
    if (out) *out = NULL;
    if (!cuda || !packed_host || !scales_f16 || !out || !n || !k || group < 2 || (k % (size_t)group) || (k & 1))
        return fail(error, error_size, "invalid w4g_weight_create arguments");
    h3_cuda_w4a8_weight *w = NULL;
    if (!weight_alloc(cuda, n, k, &w, error, error_size)) return 0;
    const size_t groups = k / (size_t)group;
    uint8_t *d_packed = NULL;
    __half *d_sc = NULL;
    int ok = 0;
    cudaStream_t st = cuda->op_stream;
    do {
        if (cudaMalloc((void **)&d_packed, n * k / 2) != cudaSuccess ||
            cudaMalloc((void **)&d_sc, n * groups * sizeof(__half)) != cudaSuccess) {
            cuda_fail(cudaGetLastError(), "w4g staging allocation", error, error_size);
            break;
        }
        cudaError_t ec = cudaMemcpyAsync(d_packed, packed_host, n * k / 2, cudaMemcpyHostToDevice, st);
        if (ec == cudaSuccess) ec = cudaMemcpyAsync(d_sc, scales_f16, n * groups * sizeof(__half), cudaMemcpyHostToDevice, st);
        if (ec != cudaSuccess) {
            cuda_fail(ec, "w4g weight H2D", error, error_size);
            break;
        }
        k_w4g_decode<<<(unsigned)n, 256, 0, st>>>(d_packed, d_sc, k, group, w->d_w, w->d_s);
        cuda->launches++;
        cudaError_t e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) {
            cuda_fail(e, "w4g decode", error, error_size);
            break;
        }
        ok = 1;
    } while (0);
    if (d_packed) cudaFree(d_packed);
    if (d_sc) cudaFree(d_sc);
    if (!ok) {
        h3_cuda_w4a8_weight_free(w);
        return 0;
    }
    *out = w;
    return 1;
}

int h3_cuda_w4a8_weight_upload_i8(h3_cuda_w4a8_weight *w, int8_t *w_i8, size_t n, size_t k, float *s_channel,
                                  int borrow_host, char *error, size_t error_size) {
    if (!w || !w_i8 || !s_channel) return fail(error, error_size, "invalid weight_upload_i8 arguments");
    if (w->n != n || w->k != k) return fail(error, error_size, "weight_upload_i8: shape mismatch (%zux%zu vs %zux%zu)", n, k, w->n, w->k);
    cudaSetDevice(w->device);
    if (w->pending && !h3_cuda_w4a8_weight_ensure_ready(w, error, error_size)) return 0;
    cudaStream_t st = w->cuda->side[0];
    H3B_CUDA_OK(cudaMemcpyAsync(w->d_w, w_i8, n * k, cudaMemcpyHostToDevice, st), "weight H2D");
    H3B_CUDA_OK(cudaMemcpyAsync(w->d_s, s_channel, n * sizeof(float), cudaMemcpyHostToDevice, st), "scale H2D");
    H3B_CUDA_OK(cudaEventRecord(w->ready, st), "cudaEventRecord");
    w->pending = 1;
    if (!borrow_host) {
        w->own_host_w = w_i8;
        w->own_host_s = s_channel;
    } else {
        // the caller may reuse its buffers at once
        H3B_CUDA_OK(cudaEventSynchronize(w->ready), "cudaEventSynchronize");
    }
    return 1;
}

int h3_cuda_w4a8_weight_create_from_i8(h3_cuda *cuda, int8_t *w_i8, size_t n, size_t k, float *s_channel,
                                       h3_cuda_w4a8_weight **out, double *h2d_ms, int borrow_host, char *error,
                                       size_t error_size) {
    if (out) *out = NULL;
    if (!cuda || !w_i8 || !s_channel || !out || !n || !k)
        return fail(error, error_size, "invalid w4a8_weight_create_from_i8 arguments");
    h3_cuda_w4a8_weight *w = NULL;
    if (!weight_alloc(cuda, n, k, &w, error, error_size)) return 0;
    if (h2d_ms) *h2d_ms = 0.0;
    if (!h3_cuda_w4a8_weight_upload_i8(w, w_i8, n, k, s_channel, borrow_host, error, error_size)) {
        w->own_host_w = w->own_host_s = NULL;   // on failure the caller keeps its buffers
        h3_cuda_w4a8_weight_free(w);
        return 0;
    }
    *out = w;
    return 1;
}

int h3_cuda_w4a8_weight_ensure_ready(h3_cuda_w4a8_weight *w, char *error, size_t error_size) {
    if (!w) return fail(error, error_size, "weight_ensure_ready: NULL weight");
    if (w->pending) {
        // make the upload visible to work enqueued later on the op stream, then drop host staging
        H3B_CUDA_OK(cudaStreamWaitEvent(w->cuda->op_stream, w->ready, 0), "cudaStreamWaitEvent");
        if (w->own_host_w || w->own_host_s) {
            H3B_CUDA_OK(cudaEventSynchronize(w->ready), "cudaEventSynchronize");
            free(w->own_host_w);
            free(w->own_host_s);
            w->own_host_w = w->own_host_s = NULL;
        }
        w->pending = 0;
    }
    return 1;
}

int h3_cuda_w4a8_weight_on_device(const h3_cuda_w4a8_weight *w, int want_dev, char *error, size_t error_size) {
    if (!w) return fail(error, error_size, "weight_on_device: NULL weight");
    if (w->device != want_dev) return fail(error, error_size, "weight lives on device %d, wanted %d", w->device, want_dev);
    return 1;
}

size_t h3_cuda_w4a8_weight_n(const h3_cuda_w4a8_weight *w) { return w ? w->n : 0; }
size_t h3_cuda_w4a8_weight_k(const h3_cuda_w4a8_weight *w) { return w ? w->k : 0; }
const int8_t *h3b_w4a8_weight_data(const h3_cuda_w4a8_weight *w) { return w ? w->d_w : NULL; }
const float *h3b_w4a8_weight_scales(const h3_cuda_w4a8_weight *w) { return w ? w->d_s : NULL; }

int h3_cuda_w4a8_weight_download_int8(const h3_cuda_w4a8_weight *w, int8_t *host_out, char *error,
                                      size_t error_size) {
    if (!w || !host_out) return fail(error, error_size, "invalid weight_download_int8 arguments");
    cudaSetDevice(w->device);
    if (w->pending) H3B_CUDA_OK(cudaEventSynchronize(w->ready), "cudaEventSynchronize");
    H3B_CUDA_OK(cudaStreamSynchronize(w->cuda->op_stream), "cudaStreamSynchronize");
    H3B_CUDA_OK(cudaMemcpy(host_out, w->d_w, w->n * w->k, cudaMemcpyDeviceToHost), "weight D2H");
    return 1;
}

int h3b_w4a8_weight_download_scales(const h3_cuda_w4a8_weight *w, float *host_out, char *error, size_t error_size) {
    if (!w || !host_out) return fail(error, error_size, "invalid weight_download_scales arguments");
    cudaSetDevice(w->device);
    if (w->pending) H3B_CUDA_OK(cudaEventSynchronize(w->ready), "cudaEventSynchronize");
    H3B_CUDA_OK(cudaStreamSynchronize(w->cuda->op_stream), "cudaStreamSynchronize");
    H3B_CUDA_OK(cudaMemcpy(host_out, w->d_s, w->n * sizeof(float), cudaMemcpyDeviceToHost), "scale D2H");
    return 1;
}

// ---------------------------------------------------------------- linears

int h3b_gemm_i8_plan(size_t tiles, size_t pairs, size_t k_blocks, int mode, size_t item, int *items_total, int *tail_first,
                     int *split, int *tile, int *kb0, int *kb1, int *slice) {
    if (tiles > 0x7fffffffu || pairs > 0x7fffffffu || k_blocks > 0x7fffffffu) return 0;
    const h3b_gemm_plan pl = h3b_gemm_make_plan((int)tiles, (int)pairs, (int)k_blocks, mode);
    if (items_total) *items_total = pl.items_total;
    if (tail_first) *tail_first = pl.tail_first;
    if (split) *split = pl.split_s;
    if (item >= (size_t)pl.items_total) return tile || kb0 || kb1 || slice ? 0 : 1;
    const h3b_gemm_item w = h3b_gemm_get_item(pl.tail_first, pl.split_s, (int)k_blocks, (int)item);
    if (tile) *tile = w.tile;
    if (kb0) *kb0 = w.kb0;
    if (kb1) *kb1 = w.kb1;
    if (slice) *slice = w.slice;
    return 1;
}

int h3b_gemm_i8_dev(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight, const int8_t *d_x_i8,
                    const float *d_act_scales, size_t m, void *d_y, const h3b_gemm_epi *epi, char *error,
                    size_t error_size) {
    if (weight && weight->pending &&
        !h3_cuda_w4a8_weight_ensure_ready(const_cast<h3_cuda_w4a8_weight *>(weight), error, error_size))
        return 0;
    return launch_gemm_i8(cuda, weight, d_x_i8, d_act_scales, m, d_y, epi, error, error_size);
}

static void backend_name(char *backend_out, size_t n) {
    if (backend_out && n) snprintf(backend_out, n, "tcgen05_i8");
}

// Translates the reference's epilogue struct (f32 tensors) into the general form.
static int map_epi(const h3_cuda_dit_gemm_epi *in, h3b_gemm_epi *out, char *error, size_t error_size) {
    memset(out, 0, sizeof(*out));
    out->kind = H3B_EPI_PLAIN;
    out->out_dtype = H3B_F32;
    if (!in) return 1;
    if (in->swiglu && in->gate) return fail(error, error_size, "gemm epilogue: swiglu and gate are mutually exclusive");
    out->d_lora = in->d_lora;
    out->lora_ready = in->d_lora ? in->lora_ready : NULL;
    // requant_mode 1 (SwiGLU output re-quantised per row for the next GEMM, the one mode the reference's host arms,
    // h3_dit_w4a8.c:4058, 4077) is served after the GEMM by the entry points below; the gate forms (2, 3) are not
    if (in->requant_mode < 0 || in->requant_mode > 1)
        return fail(error, error_size, "gemm epilogue: fused requant of the gate output (requant_mode=%d) is not supported",
                    in->requant_mode);
    if (in->requant_mode == 1) {
        if (!in->swiglu) return fail(error, error_size, "dit requant mode1 needs swiglu");
        if (in->y_f16) return fail(error, error_size, "dit gemm y_f16 incompatible with gate/requant");
    }
    if (in->swiglu) out->kind = H3B_EPI_SWIGLU;
    if (in->gate) {
        if (!in->d_residual || !in->d_modulation || !in->slots)
            return fail(error, error_size, "gemm epilogue: gate needs residual, modulation and slots");
        out->kind = H3B_EPI_GATE;
        out->d_residual = in->d_residual;
        out->d_modulation = in->d_modulation;
        out->d_row_map = in->d_row_map;
        out->slots = in->slots;
        out->gate_slot = in->gate_slot;
    } else if (in->y_f16) {
        out->out_dtype = H3B_F16;   // plain / swiglu only, as in the reference
    }
    return 1;
}

// requant_mode 1 (h3_gpu_cuda.cu:562-612, 5544-5570): the SwiGLU output d_y [m, n/2] is quantised per row (absmax / 127,
// round half away, no rotation) into library scratch, rows [m, ceil128(m)) zeroed, and the two pointers are handed
// back through the caller's struct, as the reference does.  The reference does it inside its row-wise dequant
// kernel; here the dequant lives in the tile-wise GEMM epilogue, so it is a second launch over rows that are still
// in L2.  requant_gs must equal the row width.
static int requant_swiglu_rows(h3_cuda *cuda, const h3_cuda_dit_gemm_epi *epi, const float *d_y, size_t m, size_t width,
                               bool own_scratch, char *error, size_t error_size) {
    if ((size_t)epi->requant_gs != width) return fail(error, error_size, "dit requant gs must equal act row width");
    int8_t *q;
    float *sc;
    size_t rows_out;
    if (own_scratch) {   // the f32-activation entry point: library scratch, pointers handed back (h3_gpu_cuda.cu:5544-5570)
        rows_out = (m + 127) / 128 * 128;
        const size_t act_off = (rows_out * width + 15) / 16 * 16;
        if (!grow(cuda, &cuda->rq, &cuda->rq_bytes, act_off + rows_out * sizeof(float), error, error_size)) return 0;
        q = (int8_t *)cuda->rq;
        sc = (float *)((char *)cuda->rq + act_off);
        h3_cuda_dit_gemm_epi *mut = const_cast<h3_cuda_dit_gemm_epi *>(epi);
        mut->d_rq_x = q;
        mut->d_rq_act = sc;
        mut->requant_rows = rows_out;
    } else {             // the pre-quantised entry point: the caller's buffers (h3_gpu_cuda.cu:5009-5012)
        if (!epi->d_rq_x || !epi->d_rq_act || epi->requant_rows < m) return fail(error, error_size, "dit gemm epi requant args");
        q = epi->d_rq_x;
        sc = epi->d_rq_act;
        rows_out = epi->requant_rows;
    }
    if (rows_out > m) {
        H3B_CUDA_OK(cudaMemsetAsync(q + m * width, 0, (rows_out - m) * width, cuda->op_stream), "requant pad rows");
        H3B_CUDA_OK(cudaMemsetAsync(sc + m, 0, (rows_out - m) * sizeof(float), cuda->op_stream), "requant pad scales");
    }
    return launch_quant(cuda, d_y, H3B_F32, m, width, q, sc, error, error_size);
}

int h3_cuda_gemm_i8_dequant_f32_dev_pre_q(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight, const int8_t *d_x_i8,
                                          const float *d_act_in, size_t m, float *d_y_f32, double *prep_ms,
                                          double *gemm_ms, char *backend_out, size_t backend_out_size,
                                          const h3_cuda_dit_gemm_epi *epi, char *error, size_t error_size) {
    h3b_gemm_epi e;
    if (!cuda || !weight || !d_x_i8 || !d_act_in || !d_y_f32 || !m)
        return fail(error, error_size, "invalid gemm_i8 pre_q arguments");
    if (!map_epi(epi, &e, error, error_size)) return 0;
    if (prep_ms) *prep_ms = 0.0;
    Timer t(cuda, gemm_ms);
    int ok = h3b_gemm_i8_dev(cuda, weight, d_x_i8, d_act_in, m, d_y_f32, &e, error, error_size);
    if (ok && epi && epi->requant_mode == 1)
        ok = requant_swiglu_rows(cuda, epi, d_y_f32, m, weight->n / 2, false, error, error_size);
    t.stop();
    backend_name(backend_out, backend_out_size);
    return ok;
}

int h3_cuda_gemm_i8_dequant_f32_w_act_dev_epi(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight, const float *d_x_f32,
                                              int convrot_groupsize, size_t m, float *d_y_f32, double *prep_ms,
                                              double *gemm_ms, char *backend_out, size_t backend_out_size,
                                              const h3_cuda_dit_gemm_epi *epi, char *error, size_t error_size) {
    h3b_gemm_epi e;
    if (!cuda || !weight || !d_x_f32 || !d_y_f32 || !m) return fail(error, error_size, "invalid gemm_i8 w_act arguments");
    if (!map_epi(epi, &e, error, error_size)) return 0;
    const size_t k = weight->k;
    if (!grow(cuda, &cuda->act_q, &cuda->act_q_bytes, m * k, error, error_size)) return 0;
    if (!grow(cuda, &cuda->act_s, &cuda->act_s_bytes, m * sizeof(float), error, error_size)) return 0;
    // ConvRot + per-row quant in one launch
    h3b_norm_args a;
    memset(&a, 0, sizeof(a));
    a.d_x = d_x_f32; a.rows = m; a.width = k; a.dtype = H3B_F32; a.identity = 1;
    a.convrot_gs = convrot_groupsize > 0 ? convrot_groupsize : 0;
    a.d_q = (int8_t *)cuda->act_q; a.d_scales = (float *)cuda->act_s;
    Timer tp(cuda, prep_ms);
    if (!launch_norm(cuda, &a, error, error_size)) return 0;
    tp.stop();
    Timer tg(cuda, gemm_ms);
    int ok = h3b_gemm_i8_dev(cuda, weight, (const int8_t *)cuda->act_q, (const float *)cuda->act_s, m, d_y_f32, &e,
                             error, error_size);
    if (ok && epi && epi->requant_mode == 1)
        ok = requant_swiglu_rows(cuda, epi, d_y_f32, m, weight->n / 2, true, error, error_size);
    tg.stop();
    backend_name(backend_out, backend_out_size);
    return ok;
}

int h3_cuda_gemm_i8_dequant_f32_w_act_dev(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight, const float *d_x_f32,
                                          int convrot_groupsize, size_t m, float *d_y_f32, double *prep_ms,
                                          double *gemm_ms, char *backend_out, size_t backend_out_size, char *error,
                                          size_t error_size) {
    return h3_cuda_gemm_i8_dequant_f32_w_act_dev_epi(cuda, weight, d_x_f32, convrot_groupsize, m, d_y_f32, prep_ms,
                                                     gemm_ms, backend_out, backend_out_size, NULL, error, error_size);
}

// ---- host-buffer forms: stage through device memory, run the device path, copy back

struct DevBuf {
    void *p = NULL;
    ~DevBuf() { if (p) cudaFree(p); }
    int alloc(size_t bytes, char *error, size_t error_size) {
        H3B_CUDA_OK(cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc(staging)");
        return 1;
    }
};

int h3_cuda_gemm_i8_dequant_f32_w(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight, const int8_t *x_i8,
                                  const float *act_scales, int per_tensor_scale, size_t m, float *y_f32,
                                  double *gemm_ms, char *backend_out, size_t backend_out_size, char *error,
                                  size_t error_size) {
    if (!cuda || !weight || !x_i8 || !act_scales || !y_f32 || !m) return fail(error, error_size, "invalid gemm_i8_w arguments");
    const size_t n = weight->n, k = weight->k;
    DevBuf dx, da, dy;
    if (!dx.alloc(m * k, error, error_size) || !da.alloc(m * sizeof(float), error, error_size) ||
        !dy.alloc(m * n * sizeof(float), error, error_size))
        return 0;
    float *tmp = NULL;
    const float *scales = act_scales;
    if (per_tensor_scale) {
        tmp = (float *)malloc(m * sizeof(float));
        if (!tmp) return fail(error, error_size, "gemm_i8_w: out of host memory");
        for (size_t i = 0; i < m; i++) tmp[i] = act_scales[0];
        scales = tmp;
    }
    cudaStream_t st = cuda->op_stream;
    {
        cudaError_t ec = cudaMemcpyAsync(dx.p, x_i8, m * k, cudaMemcpyHostToDevice, st);
        if (ec == cudaSuccess) ec = cudaMemcpyAsync(da.p, scales, m * sizeof(float), cudaMemcpyHostToDevice, st);
        if (ec != cudaSuccess) {
            free(tmp);
            return cuda_fail(ec, "gemm_i8_w: H2D", error, error_size);
        }
    }
    h3b_gemm_epi e;
    memset(&e, 0, sizeof(e));
    e.kind = H3B_EPI_PLAIN; e.out_dtype = H3B_F32;
    Timer t(cuda, gemm_ms);
    int ok = h3b_gemm_i8_dev(cuda, weight, (const int8_t *)dx.p, (const float *)da.p, m, dy.p, &e, error, error_size);
    t.stop();
    if (ok) {
        cudaError_t er = cudaMemcpyAsync(y_f32, dy.p, m * n * sizeof(float), cudaMemcpyDeviceToHost, st);
        if (er == cudaSuccess) er = cudaStreamSynchronize(st);
        if (er != cudaSuccess) ok = cuda_fail(er, "gemm_i8_w copy back", error, error_size);
        else ok = h3b_cuda_check(cuda, NULL, error, error_size);
    } else {
        cudaStreamSynchronize(st);
    }
    free(tmp);
    backend_name(backend_out, backend_out_size);
    return ok;
}

int h3_cuda_gemm_i8_dequant_f32(h3_cuda *cuda, const int8_t *x_i8, const int8_t *w_i8, const float *act_scales,
                                int per_tensor_scale, const float *s_channel, size_t m, size_t n, size_t k,
                                float *y_f32, double *gemm_ms, char *backend_out, size_t backend_out_size,
                                char *error, size_t error_size) {
    if (!cuda || !x_i8 || !w_i8 || !act_scales || !s_channel || !y_f32 || !m || !n || !k)
        return fail(error, error_size, "invalid gemm_i8 arguments");
    h3_cuda_w4a8_weight *w = NULL;
    if (!h3_cuda_w4a8_weight_create_from_i8(cuda, const_cast<int8_t *>(w_i8), n, k, const_cast<float *>(s_channel), &w,
                                            NULL, 1, error, error_size))
        return 0;
    int ok = h3_cuda_gemm_i8_dequant_f32_w(cuda, w, x_i8, act_scales, per_tensor_scale, m, y_f32, gemm_ms, backend_out,
                                           backend_out_size, error, error_size);
    h3_cuda_w4a8_weight_free(w);
    return ok;
}

int h3_cuda_gemm_i8_dequant_f32_w_act(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight, const float *x_f32,
                                      int convrot_groupsize, size_t m, float *y_f32, double *prep_ms,
                                      double *gemm_ms, char *backend_out, size_t backend_out_size, char *error,
                                      size_t error_size) {
    if (!cuda || !weight || !x_f32 || !y_f32 || !m) return fail(error, error_size, "invalid gemm_i8_w_act arguments");
    const size_t n = weight->n, k = weight->k;
    DevBuf dx, dy;
    if (!dx.alloc(m * k * sizeof(float), error, error_size) || !dy.alloc(m * n * sizeof(float), error, error_size))
        return 0;
    cudaStream_t st = cuda->op_stream;
    H3B_CUDA_OK(cudaMemcpyAsync(dx.p, x_f32, m * k * sizeof(float), cudaMemcpyHostToDevice, st), "gemm_i8_dequant_f32_w_act: H2D");
    int ok = h3_cuda_gemm_i8_dequant_f32_w_act_dev(cuda, weight, (const float *)dx.p, convrot_groupsize, m,
                                                   (float *)dy.p, prep_ms, gemm_ms, backend_out, backend_out_size,
                                                   error, error_size);
    if (ok) {
        cudaError_t er = cudaMemcpyAsync(y_f32, dy.p, m * n * sizeof(float), cudaMemcpyDeviceToHost, st);
        if (er == cudaSuccess) er = cudaStreamSynchronize(st);
        if (er != cudaSuccess) ok = cuda_fail(er, "gemm_i8_w_act copy back", error, error_size);
        else ok = h3b_cuda_check(cuda, NULL, error, error_size);
    } else {
        cudaStreamSynchronize(st);
    }
    return ok;
}

}  // extern "C"
