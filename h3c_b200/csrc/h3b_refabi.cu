// The rest of the reference's operator surface (h3_gpu_cuda.h) that its DiT host (h3_dit_w4a8.c) links
// against: host-buffer wrappers, the NVFP4 FC1 -> SwiGLU -> requantise -> FC2 chain, the ConvRot + requantise
// helper, token-reduction pool / expand, the mixed 16-bit-weight f32 GEMM, stream / scratch housekeeping calls.
// Optional features of the reference that have no meaning in this library (its cuBLAS handle management, its
// Python-backed attention plugins, distance attention) answer the way the reference's own stub files do:
// a harmless success where the call only tunes something, a clear "not supported by libh3_b200" otherwise.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "h3b_internal.h"
#include "h3b_nvfp4.cuh"

namespace h3b {

// NVFP4 rounding rules and scale layout: h3b_nvfp4.cuh

// FC1 accumulators [m, 2*ffn] f32 -> silu(gate) * up -> E2M1 codes + UE4M3 block scales of the FC2 input
// (h3_dit_nvfp4_chain.cu:201-277).  One thread per 16-element block; rows in [m, ceil128(m)) clear their scale
// bytes.  The scale bytes go to the 128x4-blocked positions h3_cuda_quantize_act_nvfp4_dev uses, which is the
// layout the FC2 GEMM of this library reads.
__global__ void k_swiglu_requant_nvfp4(const float *acc, float acc_scale, const float *lora, size_t m, size_t m_pad,
                                       size_t ffn, uint8_t *packed, uint8_t *sf) {
    const size_t nc = ffn / 16, ncb = ffn / 64, total = m_pad * nc;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / nc, blk = i - row * nc;
        if (row >= m) {
            sf[sf_offset(row, blk, ncb)] = 0;
            continue;
        }
        const float *g = acc + row * 2 * ffn + blk * 16, *u = g + ffn;
        const float *lg = lora ? lora + row * 2 * ffn + blk * 16 : nullptr;
        float v[16], amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
            const float4 g4 = *reinterpret_cast<const float4 *>(g + j), u4 = *reinterpret_cast<const float4 *>(u + j);
            const float gg[4] = {g4.x, g4.y, g4.z, g4.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
            for (int t = 0; t < 4; t++) {
                float gate = __fmul_rn(acc_scale, gg[t]), up = __fmul_rn(acc_scale, uu[t]);
                if (lg) {
                    gate = __fadd_rn(gate, lg[j + t]);
                    up = __fadd_rn(up, lg[ffn + j + t]);
                }
                v[j + t] = __fmul_rn(gate / __fadd_rn(1.0f, expf(-gate)), up);
                amax = fmaxf(amax, fabsf(v[j + t]));
            }
        }
        // unlike the activation quantiser the chain keeps a zero scale byte (no clamp to byte 1): a block of
        // zeros gets scale 1.0, a tiny block may underflow to scale 0 and then divides by zero like the reference
        const float scale_f = amax > 0.0f ? amax / 6.0f : 1.0f;
        const uint8_t sb = f32_to_ue4m3(scale_f);
        const float inv = 1.0f / ue4m3_to_f32(sb);
        sf[sf_offset(row, blk, ncb)] = sb;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            lo |= ((e2m1_nibble(__fmul_rn(v[j], inv)) << 4) | e2m1_nibble(__fmul_rn(v[j + 1], inv))) << (4 * j);
            hi |= ((e2m1_nibble(__fmul_rn(v[8 + j], inv)) << 4) | e2m1_nibble(__fmul_rn(v[9 + j], inv))) << (4 * j);
        }
        *reinterpret_cast<uint2 *>(packed + row * (ffn / 2) + blk * 8) = make_uint2(lo, hi);
    }
}

// ------------------------------------------------------------------ token reduction (h3_gpu_cuda.cu:12927-12981)

// One warp per reduced row: the row is the mean of the two source rows of its pair (or a copy when both
// indices agree); the source rows are kept in `original`, the pooled row also in `baseline[baseline_idx]`.
__global__ void k_token_pool(const float *in, const uint32_t *pairs, const uint32_t *baseline_idx, float *out,
                             float *original, float *baseline, size_t reduced_rows, size_t width) {
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const size_t n_warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t row = warp; row < reduced_rows; row += n_warps) {
        const uint32_t first = pairs[2 * row], second = pairs[2 * row + 1], bi = baseline_idx[row];
        const float *a = in + (size_t)first * width, *b = in + (size_t)second * width;
        for (size_t c = lane; c < width; c += 32) {
            const float x = a[c];
            float pooled = x;
            original[(size_t)first * width + c] = x;
            if (first != second) {
                const float y = b[c];
                original[(size_t)second * width + c] = y;
                pooled = __fmul_rn(0.5f, __fadd_rn(x, y));
            }
            out[row * width + c] = pooled;
            if (bi != 0xffffffffu && baseline) baseline[(size_t)bi * width + c] = pooled;
        }
    }
}

// One warp per full row: rows outside the video span, and rows whose parent has no baseline, take the reduced
// row; the others take original + update_scale * (reduced - baseline).
__global__ void k_token_expand(const float *original, const float *reduced, const float *baseline,
                               const uint32_t *baseline_idx, const uint32_t *parents, float *out, size_t full_rows,
                               size_t width, uint32_t video_start, uint32_t video_rows, float update_scale) {
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const size_t n_warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t row = warp; row < full_rows; row += n_warps) {
        const uint32_t parent = parents[row];
        const float *red = reduced + (size_t)parent * width;
        uint32_t bi = 0xffffffffu;
        const bool in_video = row >= video_start && row < (size_t)video_start + video_rows;
        if (in_video) bi = baseline_idx[parent];
        if (bi == 0xffffffffu) {
            for (size_t c = lane; c < width; c += 32) out[row * width + c] = red[c];
        } else {
            const float *orig = original + row * width, *base = baseline + (size_t)bi * width;
            for (size_t c = lane; c < width; c += 32)
                out[row * width + c] = __fadd_rn(orig[c], __fmul_rn(update_scale, __fsub_rn(red[c], base[c])));
        }
    }
}

__global__ void k_half_to_f32(const __half *in, float *out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __half2float(in[i]);
}

__global__ void k_count_nonfinite(const void *p, size_t n, int kind, unsigned long long *count) {
    unsigned long long bad = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v;
        if (kind == 0) v = reinterpret_cast<const float *>(p)[i];
        else if (kind == 1) v = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
        else v = __half2float(reinterpret_cast<const __half *>(p)[i]);
        bad += !isfinite(v);
    }
    if (bad) atomicAdd(count, bad);
}

static unsigned grid_for(const h3_cuda *cuda, size_t items, int threads, int per_sm) {
    const size_t want = ceil_div(items, (size_t)threads), cap = (size_t)cuda->sm_count * per_sm;
    const size_t g = want < cap ? want : cap;
    return (unsigned)(g ? g : 1);
}

static int unsupported(char *error, size_t error_size, const char *what) {
    return fail(error, error_size, "%s: not supported by libh3_b200", what);
}

}  // namespace h3b

using namespace h3b;

extern "C" {

// ------------------------------------------------------------------ streams, scratch, host memory

int h3_cuda_copy_stream_synchronize(h3_cuda *cuda, char *error, size_t error_size) {   // h3_gpu_cuda.h:334
    if (!cuda) return fail(error, error_size, "copy_stream_synchronize: NULL handle");
    // weight uploads run on side stream 0
    H3B_CUDA_OK(cudaStreamSynchronize(cuda->side[0]), "cudaStreamSynchronize(copy stream)");
    return 1;
}

// The reference moves its f32 (LoRA) GEMMs onto a second cuBLAS handle bound to side stream 1 so that they
// overlap the int8 GEMM; the same switch moves this library's f32 dense GEMMs onto that stream.
int h3_cuda_cublas_use_side(h3_cuda *cuda, int on, char *error, size_t error_size) {    // h3_gpu_cuda.h:220
    if (!cuda) return fail(error, error_size, "cublas_use_side: NULL handle");
    if (on && !cuda->side[1]) return fail(error, error_size, "cublas_use_side: no side stream");
    cuda->blas_side = on ? 1 : 0;
    return 1;
}
void *h3_cuda_cublas_stream(const h3_cuda *cuda) { return cuda ? (void *)dense_stream(cuda) : NULL; }   // :223

int h3_cuda_recreate_blas(h3_cuda *cuda, char *error, size_t error_size) {              // h3_gpu_cuda.h:60
    if (!cuda) return fail(error, error_size, "recreate_blas: NULL handle");
    return 1;   // no BLAS handle exists to rebuild
}

// Scratch of a handle is allocated with the handle's device current, so there is nothing to move; the check
// confirms that every live scratch buffer belongs to the handle's device.  h3_gpu_cuda.h:58-59
int h3_cuda_dit_scratch_check(h3_cuda *cuda, char *error, size_t error_size) {
    if (!cuda) return fail(error, error_size, "dit_scratch_check: NULL handle");
    void *bufs[] = {cuda->act_q, cuda->act_s, cuda->act_rot, cuda->attn, cuda->rq, cuda->kvx, cuda->wtmp};
    for (size_t i = 0; i < sizeof(bufs) / sizeof(bufs[0]); i++) {
        if (!bufs[i]) continue;
        cudaPointerAttributes attr;
        H3B_CUDA_OK(cudaPointerGetAttributes(&attr, bufs[i]), "cudaPointerGetAttributes(scratch)");
        if (attr.device != cuda->device)
            return fail(error, error_size, "dit_scratch_check: scratch %zu lives on device %d, handle on %d", i, attr.device,
                        cuda->device);
    }
    return 1;
}
int h3_cuda_dit_scratch_rehome(h3_cuda *cuda, char *error, size_t error_size) {
    if (!cuda) return fail(error, error_size, "dit_scratch_rehome: NULL handle");
    if (h3_cuda_dit_scratch_check(cuda, NULL, 0)) return 1;
    h3_cuda_release_heavy_workspace(cuda);   // regrown on the right device by the next call
    return h3_cuda_bind_device(cuda, error, error_size);
}

int h3_cuda_host_register(void *p, size_t bytes, char *error, size_t error_size) {      // h3_gpu_cuda.h:321
    if (!p || !bytes) return fail(error, error_size, "host_register: invalid arguments");
    H3B_CUDA_OK(cudaHostRegister(p, bytes, cudaHostRegisterDefault), "cudaHostRegister");
    return 1;
}
void h3_cuda_host_unregister(void *p) {
    if (p) cudaHostUnregister(p);
}

// ------------------------------------------------------------------ f32 GEMM with host operands

int h3_cuda_gemm_f32_dw(h3_cuda *cuda, const float *x, const float *d_weight, size_t m, size_t n, size_t k, float *y,
                        double *gemm_ms, char *error, size_t error_size) {             // h3_gpu_cuda.h:115
    if (!cuda || !x || !d_weight || !y || !m || !n || !k) return fail(error, error_size, "invalid gemm_f32_dw arguments");
    float *dx = NULL, *dy = NULL;
    cudaStream_t st = dense_stream(cuda);
    if (cudaMalloc((void **)&dx, m * k * sizeof(float)) != cudaSuccess ||
        cudaMalloc((void **)&dy, m * n * sizeof(float)) != cudaSuccess) {
        if (dx) cudaFree(dx);
        return cuda_fail(cudaGetLastError(), "gemm_f32_dw: device staging", error, error_size);
    }
    int ok = cudaMemcpyAsync(dx, x, m * k * sizeof(float), cudaMemcpyHostToDevice, st) == cudaSuccess;
    if (!ok) fail(error, error_size, "gemm_f32_dw: upload failed");
    ok = ok && h3_cuda_gemm_f32_dd(cuda, dx, d_weight, m, n, k, dy, gemm_ms, error, error_size);
    if (ok && (cudaMemcpyAsync(y, dy, m * n * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
               cudaStreamSynchronize(st) != cudaSuccess))
        ok = fail(error, error_size, "gemm_f32_dw: download failed");
    cudaStreamSynchronize(st);
    cudaFree(dx);
    cudaFree(dy);
    return ok;
}

int h3_cuda_gemm_f32(h3_cuda *cuda, const float *x, const float *weight, size_t m, size_t n, size_t k, float *y,
                     double *gemm_ms, char *error, size_t error_size) {                // h3_gpu_cuda.h:91
    if (!cuda || !x || !weight || !y || !m || !n || !k) return fail(error, error_size, "invalid gemm_f32 arguments");
    float *dw = NULL;
    H3B_CUDA_OK(cudaMalloc((void **)&dw, n * k * sizeof(float)), "gemm_f32: weight staging");
    int ok = cudaMemcpy(dw, weight, n * k * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess;
    if (!ok) fail(error, error_size, "gemm_f32: weight upload failed");
    ok = ok && h3_cuda_gemm_f32_dw(cuda, x, dw, m, n, k, y, gemm_ms, error, error_size);
    cudaFree(dw);
    return ok;
}

// f32 activations x 16-bit (f16) weights -> f32, y = alpha * x W^T + beta * y (the reference's LoRA option
// H3_DIT_LORA_F16; h3_gpu_cuda.h:183).  The weights are widened to f32 in scratch (exact) and the f32 kernel runs.
int h3_cuda_gemm_f32in_f16w_f32out_dd_ex(h3_cuda *cuda, const float *d_x_f32, const void *d_w_h, size_t m, size_t n,
                                         size_t k, float *d_y_f32, float alpha, float beta, char *error,
                                         size_t error_size) {
    if (!cuda || !d_x_f32 || !d_w_h || !d_y_f32 || !m || !n || !k)
        return fail(error, error_size, "invalid gemm_f32in_f16w arguments");
    if (!grow(cuda, &cuda->wtmp, &cuda->wtmp_bytes, n * k * sizeof(float), error, error_size)) return 0;
    k_half_to_f32<<<grid_for(cuda, n * k, 256, 8), 256, 0, dense_stream(cuda)>>>((const __half *)d_w_h, (float *)cuda->wtmp,
                                                                                n * k);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_half_to_f32 launch");
    return h3_cuda_gemm_f32_dd_ex(cuda, d_x_f32, (const float *)cuda->wtmp, m, n, k, d_y_f32, alpha, beta, NULL, error,
                                  error_size);
}

// ------------------------------------------------------------------ ConvRot + requantise helper

// Rotates the SwiGLU output per group and quantises it per row into library scratch; the caller hands the two
// pointers to h3_cuda_gemm_i8_dequant_f32_dev_pre_q.  h3_gpu_cuda.h:143, body h3_gpu_cuda.cu:4813
int h3_cuda_epi_fuse_ink_prep_fc2(h3_cuda *cuda, const float *d_swiglu, size_t m, size_t k, int convrot_groupsize,
                                  int8_t **out_xi8, float **out_scales, char *error, size_t error_size) {
    if (out_xi8) *out_xi8 = NULL;
    if (out_scales) *out_scales = NULL;
    if (!cuda || !d_swiglu || !out_xi8 || !out_scales || !m || !k || convrot_groupsize < 4)
        return fail(error, error_size, "invalid epi_fuse_ink_prep args");
    if (k % (size_t)convrot_groupsize) return fail(error, error_size, "K not divisible by convrot_gs");
    const size_t m_pad = (m + 127) / 128 * 128, act_off = (m_pad * k + 15) / 16 * 16;
    if (!grow(cuda, &cuda->rq, &cuda->rq_bytes, act_off + m_pad * sizeof(float), error, error_size)) return 0;
    int8_t *q = (int8_t *)cuda->rq;
    float *s = (float *)((char *)cuda->rq + act_off);
    if (m_pad > m) {   // rows of the padded tail read as zero codes, like the reference's kernel leaves them
        H3B_CUDA_OK(cudaMemsetAsync(q + m * k, 0, (m_pad - m) * k, cuda->op_stream), "ink_prep pad rows");
        H3B_CUDA_OK(cudaMemsetAsync(s + m, 0, (m_pad - m) * sizeof(float), cuda->op_stream), "ink_prep pad scales");
    }
    h3b_norm_args a;
    memset(&a, 0, sizeof(a));
    a.d_x = d_swiglu; a.rows = m; a.width = k; a.dtype = H3B_F32; a.identity = 1; a.convrot_gs = convrot_groupsize;
    a.d_q = q; a.d_scales = s;
    if (!launch_norm(cuda, &a, error, error_size)) return 0;
    *out_xi8 = q;
    *out_scales = s;
    return 1;
}

// The rotation on f16 activations (the reference's tensor-core form with f32 accumulation, h3_gpu_cuda.h:149):
// butterflies in f32 on the widened inputs, one rounding to f16 at the end.
int h3_cuda_convrot_act_f16_dd(h3_cuda *cuda, const void *d_x_half, size_t m, size_t k, int convrot_groupsize,
                               void *d_y_half, char *error, size_t error_size) {
    if (!cuda || !d_x_half || !d_y_half || !m || !k) return fail(error, error_size, "invalid convrot_act_f16 arguments");
    if (!grow(cuda, &cuda->act_rot, &cuda->act_rot_bytes, m * k * sizeof(float), error, error_size)) return 0;
    h3b_norm_args a;
    memset(&a, 0, sizeof(a));
    a.d_x = d_x_half; a.rows = m; a.width = k; a.dtype = H3B_F16; a.identity = 1; a.convrot_gs = convrot_groupsize;
    a.d_rot = (float *)cuda->act_rot;
    return launch_norm(cuda, &a, error, error_size) &&
           h3b_cast_dev(cuda, cuda->act_rot, H3B_F32, d_y_half, H3B_F16, m * k, error, error_size);
}

// ------------------------------------------------------------------ NVFP4 FC1 -> FC2 chain

// Block-scaled FP4 GEMM with f32 accumulators written out unrounded (the reference's CUTLASS sm_120a unit,
// h3_dit_nvfp4_chain.cu:322; here the same tcgen05 kernel as every other FP4 linear, f32 output).
int h3_cutlass_nvfp4_fc1_f32_run(h3_cuda *cuda, const uint8_t *d_w_fp4, const uint8_t *d_sf_w, const uint8_t *d_x_fp4,
                                 const uint8_t *d_sf_x, size_t m, size_t n, size_t k, float *d_acc_f32, double *gemm_ms,
                                 char *error, size_t error_size) {
    if (!cuda || !d_acc_f32) return fail(error, error_size, "nvfp4_fc1_f32: invalid arguments");
    Timer t(cuda, gemm_ms);
    const int ok = launch_gemm_nvfp4(cuda, d_w_fp4, d_sf_w, d_x_fp4, d_sf_x, m, n, k, 1.0f, d_acc_f32, H3B_F32, 0, NULL, NULL,
                                     NULL, 0, 0, error, error_size);
    t.stop();
    return ok;
}

int h3_nvfp4_swiglu_requant_dev(h3_cuda *cuda, const float *d_acc_f32, float acc_scale, const float *d_lora, size_t m,
                                size_t ffn, uint8_t *d_act_fp4, uint8_t *d_sf_act, char *error, size_t error_size) {
    if (!cuda || !d_acc_f32 || !d_act_fp4 || !d_sf_act || !m || !ffn || (ffn & 63))
        return fail(error, error_size, "swiglu_requant: invalid args (ffn%%64!=0)");
    if (((uintptr_t)d_acc_f32 & 15) || ((uintptr_t)d_act_fp4 & 7) || (d_lora && ((uintptr_t)d_lora & 3)))
        return fail(error, error_size, "swiglu_requant: misaligned buffers");
    const size_t m_pad = (m + 127) / 128 * 128;
    k_swiglu_requant_nvfp4<<<grid_for(cuda, m_pad * (ffn / 16), 256, 32), 256, 0, cuda->op_stream>>>(
        d_acc_f32, acc_scale, d_lora, m, m_pad, ffn, d_act_fp4, d_sf_act);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_swiglu_requant_nvfp4 launch");
    return 1;
}

// fc1 input codes + scales, fc1 f32 accumulators [m_pad, 2*ffn], fc2 input codes + scales.  h3_gpu_cuda.h:534
size_t h3_cuda_nvfp4_chain_scratch_bytes(size_t m, size_t kdim, size_t ffn) {
    const size_t m_pad = (m + 127) / 128 * 128;
    return m_pad * kdim / 2 + h3_cuda_nvfp4_sf_bytes(m_pad, kdim) + m_pad * 2 * ffn * sizeof(float) + m_pad * ffn / 2 +
           h3_cuda_nvfp4_sf_bytes(m_pad, ffn);
}

// FC2 on an activation that is already E2M1 + scales, with the gate + residual epilogue.  The bf16 scratch of
// the reference's two-step form is not needed (the epilogue reads the f32 accumulators in place).  :540
int h3_cuda_gemm_fp4_pre_q_dev(h3_cuda *cuda, const h3_cuda_nvfp4_weight *weight, const uint8_t *d_x_fp4,
                               const uint8_t *d_sf_x, size_t m, const float *d_residual, const float *d_modulation,
                               const uint32_t *d_row_map, size_t slots, size_t gate_slot, const float *d_lora,
                               float *d_y_f32, void *d_bf16_scratch, double *gemm_ms, char *error, size_t error_size,
                               const char *tag) {
    (void)d_bf16_scratch;
    (void)tag;
    if (!cuda || !weight || !d_x_fp4 || !d_sf_x || !d_y_f32 || !m) return fail(error, error_size, "gemm_fp4_pre_q: invalid arguments");
    if (d_lora) return unsupported(error, error_size, "gemm_fp4_pre_q with a LoRA delta");
    const int gate = d_residual != NULL;
    if (gate && (!d_modulation || !slots)) return fail(error, error_size, "gemm_fp4_pre_q: gate needs modulation and slots");
    Timer t(cuda, gemm_ms);
    const int ok = launch_gemm_nvfp4(cuda, h3_cuda_nvfp4_weight_packed(weight), h3_cuda_nvfp4_weight_sf(weight), d_x_fp4, d_sf_x,
                                     m, h3_cuda_nvfp4_weight_n(weight), h3_cuda_nvfp4_weight_k(weight),
                                     h3_cuda_nvfp4_weight_scale2(weight), d_y_f32, H3B_F32, gate, d_residual, d_modulation,
                                     d_row_map, slots, gate_slot, error, error_size);
    t.stop();
    return ok;
}

// H3_NVFP4_DEBUG_NAN=1 turns on a synchronous scan for non-finite values.  h3_gpu_cuda.h:554-557
int h3_nvfp4_debug_nan_dev(void) {
    return strcmp(h3_plugin_value("H3_NVFP4_DEBUG_NAN"), "1") == 0;
}
void h3_nvfp4_debug_scan_dev(h3_cuda *cuda, const void *ptr, size_t n, const char *kind, const char *tag, const char *stage) {
    if (!cuda || !ptr || !n || !h3_nvfp4_debug_nan_dev()) return;
    const int k = (kind && !strcmp(kind, "bf16")) ? 1 : (kind && !strcmp(kind, "f16")) ? 2 : 0;
    unsigned long long *d_count = NULL, bad = 0;
    if (cudaMalloc((void **)&d_count, sizeof(bad)) != cudaSuccess) return;
    cudaMemsetAsync(d_count, 0, sizeof(bad), cuda->op_stream);
    k_count_nonfinite<<<grid_for(cuda, n, 256, 8), 256, 0, cuda->op_stream>>>(ptr, n, k, d_count);
    cudaMemcpyAsync(&bad, d_count, sizeof(bad), cudaMemcpyDeviceToHost, cuda->op_stream);
    cudaStreamSynchronize(cuda->op_stream);
    cudaFree(d_count);
    if (bad) fprintf(stderr, "[nvfp4_dbg] %s %s: %llu of %zu values are not finite\n", tag ? tag : "?", stage ? stage : "?", bad, n);
}

// ------------------------------------------------------------------ token reduction

static int pool_dev(h3_cuda *cuda, const float *d_in, const uint32_t *pairs, const uint32_t *baseline_idx, size_t reduced_rows,
                    size_t width, float *d_out, float *d_original, float *d_baseline, double *op_ms, char *error,
                    size_t error_size) {
    uint32_t *d_idx = NULL;   // pairs then baseline indices
    H3B_CUDA_OK(cudaMalloc((void **)&d_idx, reduced_rows * 3 * sizeof(uint32_t)), "token_pool index staging");
    cudaStream_t st = cuda->op_stream;
    int ok = cudaMemcpyAsync(d_idx, pairs, reduced_rows * 2 * sizeof(uint32_t), cudaMemcpyHostToDevice, st) == cudaSuccess &&
             cudaMemcpyAsync(d_idx + 2 * reduced_rows, baseline_idx, reduced_rows * sizeof(uint32_t), cudaMemcpyHostToDevice,
                             st) == cudaSuccess;
    if (!ok) fail(error, error_size, "token_pool: index upload failed");
    if (ok) {
        Timer t(cuda, op_ms);
        k_token_pool<<<grid_for(cuda, reduced_rows * 32, 256, 8), 256, 0, st>>>(d_in, d_idx, d_idx + 2 * reduced_rows, d_out,
                                                                                d_original, d_baseline, reduced_rows, width);
        cuda->launches++;
        if (cudaGetLastError() != cudaSuccess) ok = fail(error, error_size, "token_pool kernel launch failed");
        t.stop();
    }
    cudaStreamSynchronize(st);   // the index tables are host memory of the caller and a temporary on the device
    cudaFree(d_idx);
    return ok;
}

int h3_cuda_token_pool_f32_dev(h3_cuda *cuda, const float *d_input, size_t full_rows, const uint32_t *pairs,
                               const uint32_t *baseline_idx, size_t reduced_rows, size_t baseline_rows, size_t width,
                               float *d_output, float *d_original, float *d_baseline, double *op_ms, char *error,
                               size_t error_size) {                                    // h3_gpu_cuda.h:845
    if (op_ms) *op_ms = 0.0;
    if (!cuda || !d_input || !pairs || !baseline_idx || !d_output || !d_original || !full_rows || !reduced_rows || !width)
        return fail(error, error_size, "invalid token_pool_dev args");
    if (baseline_rows && !d_baseline) return fail(error, error_size, "token_pool_dev missing baseline");
    return pool_dev(cuda, d_input, pairs, baseline_idx, reduced_rows, width, d_output, d_original, d_baseline, op_ms, error,
                    error_size);
}

static int expand_dev(h3_cuda *cuda, const float *d_original, const float *d_reduced, const float *d_baseline,
                      const uint32_t *baseline_idx, const uint32_t *parents, size_t full_rows, size_t reduced_rows, size_t width,
                      uint32_t video_start, uint32_t video_rows, float update_scale, float *d_output, double *op_ms, char *error,
                      size_t error_size) {
    uint32_t *d_idx = NULL;   // parents then baseline indices
    H3B_CUDA_OK(cudaMalloc((void **)&d_idx, (full_rows + reduced_rows) * sizeof(uint32_t)), "token_expand index staging");
    cudaStream_t st = cuda->op_stream;
    int ok = cudaMemcpyAsync(d_idx, parents, full_rows * sizeof(uint32_t), cudaMemcpyHostToDevice, st) == cudaSuccess &&
             cudaMemcpyAsync(d_idx + full_rows, baseline_idx, reduced_rows * sizeof(uint32_t), cudaMemcpyHostToDevice, st) ==
                 cudaSuccess;
    if (!ok) fail(error, error_size, "token_expand: index upload failed");
    if (ok) {
        Timer t(cuda, op_ms);
        k_token_expand<<<grid_for(cuda, full_rows * 32, 256, 8), 256, 0, st>>>(d_original, d_reduced, d_baseline, d_idx + full_rows,
                                                                               d_idx, d_output, full_rows, width, video_start,
                                                                               video_rows, update_scale);
        cuda->launches++;
        if (cudaGetLastError() != cudaSuccess) ok = fail(error, error_size, "token_expand kernel launch failed");
        t.stop();
    }
    cudaStreamSynchronize(st);
    cudaFree(d_idx);
    return ok;
}

int h3_cuda_token_expand_f32_dev(h3_cuda *cuda, const float *d_original, const float *d_reduced, const float *d_baseline,
                                 const uint32_t *baseline_idx, const uint32_t *parents, size_t full_rows,
                                 size_t reduced_rows, size_t baseline_rows, size_t width, uint32_t video_start,
                                 uint32_t video_rows, float update_scale, float *d_output, double *op_ms, char *error,
                                 size_t error_size) {                                  // h3_gpu_cuda.h:852
    if (op_ms) *op_ms = 0.0;
    if (!cuda || !d_original || !d_reduced || !baseline_idx || !parents || !d_output || !full_rows || !reduced_rows || !width)
        return fail(error, error_size, "invalid token_expand_dev args");
    if (baseline_rows && !d_baseline) return fail(error, error_size, "token_expand_dev missing baseline");
    return expand_dev(cuda, d_original, d_reduced, d_baseline, baseline_idx, parents, full_rows, reduced_rows, width,
                      video_start, video_rows, update_scale, d_output, op_ms, error, error_size);
}

// Host activations in / out; the original rows and the baseline stay on the device and are handed to the caller,
// who frees them with cudaFree after the matching expand.  h3_gpu_cuda.h:827
int h3_cuda_token_pool_f32(h3_cuda *cuda, const float *input, size_t full_rows, const uint32_t *pairs,
                           const uint32_t *baseline_idx, size_t reduced_rows, size_t baseline_rows, size_t width,
                           float *output, float **d_original_out, float **d_baseline_out, double *op_ms, char *error,
                           size_t error_size) {
    if (op_ms) *op_ms = 0.0;
    if (d_original_out) *d_original_out = NULL;
    if (d_baseline_out) *d_baseline_out = NULL;
    if (!cuda || !input || !pairs || !baseline_idx || !output || !d_original_out || !d_baseline_out || !full_rows ||
        !reduced_rows || !width)
        return fail(error, error_size, "invalid token_pool args");
    const size_t full_n = full_rows * width, red_n = reduced_rows * width;
    float *d_in = NULL, *d_out = NULL, *d_orig = NULL, *d_base = NULL;
    int ok = cudaMalloc((void **)&d_in, full_n * 4) == cudaSuccess && cudaMalloc((void **)&d_out, red_n * 4) == cudaSuccess &&
             cudaMalloc((void **)&d_orig, full_n * 4) == cudaSuccess &&
             (!baseline_rows || cudaMalloc((void **)&d_base, baseline_rows * width * 4) == cudaSuccess);
    if (!ok) fail(error, error_size, "token_pool OOM");
    if (ok && cudaMemcpyAsync(d_in, input, full_n * 4, cudaMemcpyHostToDevice, cuda->op_stream) != cudaSuccess)
        ok = fail(error, error_size, "token_pool H2D");
    ok = ok && pool_dev(cuda, d_in, pairs, baseline_idx, reduced_rows, width, d_out, d_orig, d_base, op_ms, error, error_size);
    if (ok && (cudaMemcpyAsync(output, d_out, red_n * 4, cudaMemcpyDeviceToHost, cuda->op_stream) != cudaSuccess ||
               cudaStreamSynchronize(cuda->op_stream) != cudaSuccess))
        ok = fail(error, error_size, "token_pool D2H");
    cudaStreamSynchronize(cuda->op_stream);
    if (d_in) cudaFree(d_in);
    if (d_out) cudaFree(d_out);
    if (ok) {
        *d_original_out = d_orig;
        *d_baseline_out = d_base;
    } else {
        if (d_orig) cudaFree(d_orig);
        if (d_base) cudaFree(d_base);
    }
    return ok;
}

int h3_cuda_token_expand_f32(h3_cuda *cuda, const float *d_original, const float *reduced, const float *d_baseline,
                             const uint32_t *baseline_idx, const uint32_t *parents, size_t full_rows, size_t reduced_rows,
                             size_t baseline_rows, size_t width, uint32_t video_start, uint32_t video_rows,
                             float update_scale, float *output, double *op_ms, char *error, size_t error_size) {   // :833
    if (op_ms) *op_ms = 0.0;
    if (!cuda || !d_original || !reduced || !baseline_idx || !parents || !output || !full_rows || !reduced_rows || !width)
        return fail(error, error_size, "invalid token_expand args");
    if (baseline_rows && !d_baseline) return fail(error, error_size, "token_expand missing baseline");
    const size_t full_n = full_rows * width, red_n = reduced_rows * width;
    float *d_red = NULL, *d_out = NULL;
    int ok = cudaMalloc((void **)&d_red, red_n * 4) == cudaSuccess && cudaMalloc((void **)&d_out, full_n * 4) == cudaSuccess;
    if (!ok) fail(error, error_size, "token_expand OOM");
    if (ok && cudaMemcpyAsync(d_red, reduced, red_n * 4, cudaMemcpyHostToDevice, cuda->op_stream) != cudaSuccess)
        ok = fail(error, error_size, "token_expand H2D");
    ok = ok && expand_dev(cuda, d_original, d_red, d_baseline, baseline_idx, parents, full_rows, reduced_rows, width, video_start,
                          video_rows, update_scale, d_out, op_ms, error, error_size);
    if (ok && (cudaMemcpyAsync(output, d_out, full_n * 4, cudaMemcpyDeviceToHost, cuda->op_stream) != cudaSuccess ||
               cudaStreamSynchronize(cuda->op_stream) != cudaSuccess))
        ok = fail(error, error_size, "token_expand D2H");
    cudaStreamSynchronize(cuda->op_stream);
    if (d_red) cudaFree(d_red);
    if (d_out) cudaFree(d_out);
    return ok;
}

// ------------------------------------------------------------------ optional features of the reference, absent here

// Distance attention (a Gaussian penalty on video-video scores, off by default in the reference): configuring it
// OFF succeeds, switching it ON is refused.  h3_gpu_cuda.h:590-595
int h3_cuda_dist_attn_configure(h3_cuda *cuda, size_t seq, size_t video_start, size_t video_seq, int grid_t, int grid_h,
                                int grid_w, float scale, float temporal_weight, int enabled, char *error,
                                size_t error_size) {
    (void)cuda; (void)seq; (void)video_start; (void)video_seq; (void)grid_t; (void)grid_h; (void)grid_w; (void)scale;
    (void)temporal_weight;
    if (enabled) return unsupported(error, error_size, "distance attention (H3_DIT_DIST_ATTN)");
    return 1;
}
void h3_cuda_dist_attn_clear(void) {}
int h3_cuda_dist_attn_active(void) { return 0; }

// Hooks of the reference's dlopen'd attention plugins and of its profiler: nothing to do.  :653, :685, :689
void h3_cuda_sol_cute_set_step(int step) { (void)step; }
void h3_cuda_sol_profile_add_unpack(double ms) { (void)ms; }
size_t h3_cuda_sage3_pool_bytes(void) { return 0; }

// The reference's NVFP4 text-encoder library (h3_nvfp4_cuda.h) is a different code path; its four entry points
// that the shared NVFP4 reader (h3_nvfp4.c) refers to report the feature as absent.
int h3_nvfp4_cuda_enabled(void) { return 0; }
void h3_nvfp4_cuda_cache_clear(void) {}
// "returns 0 when disabled / unavailable (caller uses the host path)", as the reference documents them
int h3_nvfp4_cuda_encode_text_layers(const void *store, float *hidden, size_t tokens, unsigned n_layers, char *error,
                                     size_t error_size) {
    (void)store; (void)hidden; (void)tokens; (void)n_layers;
    return unsupported(error, error_size, "the NVFP4 text encoder on the device");
}
int h3_nvfp4_cuda_gqa_causal(const float *q, const float *k, const float *v, size_t tokens, size_t q_heads, size_t kv_heads,
                             size_t head_dim, float *out, char *error, size_t error_size) {
    (void)q; (void)k; (void)v; (void)tokens; (void)q_heads; (void)kv_heads; (void)head_dim; (void)out;
    return unsupported(error, error_size, "causal grouped-query attention of the text encoder");
}

}  // extern "C"
