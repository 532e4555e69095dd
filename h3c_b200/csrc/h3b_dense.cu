// The step on either side of the block chain: f32 dense linears (patch embedding 96 -> D, final heads
// D -> 96 / 32), the final adaLN + head, and the Euler update of the sample.
//
// Reference: h3_dit_w4a8.c:5298 (h3_dit_w4a8_dense_f32: y = x W^T + b, f32), :5370 dense_f32_cuda_to_dev
// (device GEMM + bias add), :5578 final_head_cuda (adaLN with shift slot 0 / scale slot 1 of ONE modulation
// row for every token, then dense + bias), :8822 h3_dit_w4a8_euler_step_f32; device entry points
// h3_gpu_cuda.h:120 (h3_cuda_gemm_f32_dd) and :263 (h3_cuda_bias_add_f32_dev).
//
// These linears are small (K = 96 or N <= 96): 3.6 GFLOP at 6,144 tokens against 25 TFLOP of block GEMMs,
// and they compute in f32 like the reference, so they run on the FMA pipe, not on the tensor cores.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "h3b_internal.h"

namespace h3b {

namespace dense {
constexpr int BN = 64, BK = 16, PAD = 4;
}

// y[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n]); both operands row-major with k contiguous.
// BM x 64 tile per CTA (BM = 64 with 256 threads, or 32 with 128 where the taller tile would leave SMs idle),
// 16 k per step, a 4 x 4 block of outputs per thread; operands are transposed into shared memory so that a
// thread reads its four rows / columns as one float4, and the next step's global loads are in flight while
// the current step is multiplied.
template <int BM, bool VEC>
__global__ void __launch_bounds__(BM * 4) k_dense_f32(const float *__restrict__ x, const float *__restrict__ w,
                                                      const float *__restrict__ bias, size_t m, size_t n, size_t k,
                                                      float *y, float alpha, float beta) {
    using namespace dense;
    constexpr int THREADS = BM * 4;
    constexpr int WREP = BN * 4 / THREADS;   // rows of W each thread fetches per step (1 or 2)
    __shared__ __align__(16) float xs[BK][BM + PAD];
    __shared__ __align__(16) float ws[BK][BN + PAD];
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const size_t row0 = (size_t)blockIdx.y * BM, col0 = (size_t)blockIdx.x * BN;
    const int lr = t >> 2, lk = (t & 3) * 4;   // this thread's row and first k of the tile loads
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    auto fetch = [&](const float *base, size_t row, size_t rows, size_t kk, float (&v)[4]) {
        v[0] = v[1] = v[2] = v[3] = 0.0f;
        if (row >= rows) return;
        const float *src = base + row * k + kk;
        if (VEC && kk + 4 <= k) {
            const float4 q = __ldg(reinterpret_cast<const float4 *>(src));
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++)
                if (kk + i < k) v[i] = __ldg(src + i);
        }
    };
    float xv[4], wv[WREP][4];
    fetch(x, row0 + lr, m, lk, xv);
#pragma unroll
    for (int rep = 0; rep < WREP; rep++) fetch(w, col0 + lr + rep * (THREADS / 4), n, lk, wv[rep]);

    for (size_t k0 = 0; k0 < k; k0 += BK) {
        __syncthreads();   // the previous step's reads are done
#pragma unroll
        for (int i = 0; i < 4; i++) {
            xs[lk + i][lr] = xv[i];
#pragma unroll
            for (int rep = 0; rep < WREP; rep++) ws[lk + i][lr + rep * (THREADS / 4)] = wv[rep][i];
        }
        __syncthreads();
        if (k0 + BK < k) {
            fetch(x, row0 + lr, m, k0 + BK + lk, xv);
#pragma unroll
            for (int rep = 0; rep < WREP; rep++) fetch(w, col0 + lr + rep * (THREADS / 4), n, k0 + BK + lk, wv[rep]);
        }
#pragma unroll
        for (int kq = 0; kq < BK; kq++) {
            const float4 a = *reinterpret_cast<const float4 *>(&xs[kq][ty * 4]);
            const float4 b = *reinterpret_cast<const float4 *>(&ws[kq][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = __fmaf_rn(av[i], bv[j], acc[i][j]);
        }
    }
    const size_t c = col0 + tx * 4;
    float bv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (bias)
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (c + j < n) bv[j] = __ldg(bias + c + j);
    const bool wide = n % 4 == 0 && c + 4 <= n && !((uintptr_t)y & 15);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const size_t r = row0 + ty * 4 + i;
        if (r >= m) continue;
        float o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) o[j] = bias ? __fadd_rn(acc[i][j], bv[j]) : acc[i][j];
        if (alpha != 1.0f || beta != 0.0f) {   // y = alpha * (x W^T) + beta * y, the LoRA second product
#pragma unroll
            for (int j = 0; j < 4; j++) {
                o[j] = __fmul_rn(alpha, o[j]);
                if (beta != 0.0f && c + j < n) o[j] = __fmaf_rn(beta, y[r * n + c + j], o[j]);
            }
        }
        if (wide) {
            *reinterpret_cast<float4 *>(y + r * n + c) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (c + j < n) y[r * n + c + j] = o[j];
        }
    }
}

template <int BM>
static void dense_launch_t(h3_cuda *cuda, bool vec, const float *d_x, const float *d_w, const float *d_bias, size_t m, size_t n,
                           size_t k, float *d_y, float alpha, float beta) {
    const dim3 grid((unsigned)((n + dense::BN - 1) / dense::BN), (unsigned)((m + BM - 1) / BM));
    if (vec) k_dense_f32<BM, true><<<grid, BM * 4, 0, dense_stream(cuda)>>>(d_x, d_w, d_bias, m, n, k, d_y, alpha, beta);
    else k_dense_f32<BM, false><<<grid, BM * 4, 0, dense_stream(cuda)>>>(d_x, d_w, d_bias, m, n, k, d_y, alpha, beta);
}

static int launch_dense(h3_cuda *cuda, const float *d_x, const float *d_w, const float *d_bias, size_t m, size_t n, size_t k,
                        float *d_y, char *error, size_t error_size, float alpha = 1.0f, float beta = 0.0f) {
    using namespace dense;
    if (!cuda || !d_x || !d_w || !d_y || m == 0 || n == 0 || k == 0) return fail(error, error_size, "invalid dense_f32 arguments");
    if ((m + 31) / 32 > 65535) return fail(error, error_size, "dense_f32: more than %d rows", 65535 * 32);
    const bool vec = k % 4 == 0 && !(((uintptr_t)d_x | (uintptr_t)d_w) & 15);
    // the taller tile only where it still gives every SM several CTAs
    const size_t ctas64 = ((m + 63) / 64) * ((n + BN - 1) / BN);
    ProfScope prof(cuda, PROF_OTHER);
    if (ctas64 >= (size_t)cuda->sm_count * 4) dense_launch_t<64>(cuda, vec, d_x, d_w, d_bias, m, n, k, d_y, alpha, beta);
    else dense_launch_t<32>(cuda, vec, d_x, d_w, d_bias, m, n, k, d_y, alpha, beta);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_dense_f32 launch");
    return 1;
}

__global__ void k_bias_add_f32(float *y, const float *bias, size_t total, size_t width) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        y[i] = __fadd_rn(y[i], __ldg(bias + i % width));
}

// sample += (sigma - sigma_next) * velocity, product and sum rounded separately as in the reference's C loop
__global__ void k_euler_step_f32(float *sample, const float *velocity, size_t count, float delta) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        sample[i] = __fadd_rn(sample[i], __fmul_rn(delta, velocity[i]));
}

static unsigned stream_grid(h3_cuda *cuda, size_t items, int threads) {
    const size_t want = (items + threads - 1) / threads, cap = (size_t)cuda->sm_count * 8;
    return (unsigned)(want < cap ? want : cap);
}

}  // namespace h3b

using namespace h3b;

extern "C" {

int h3_cuda_gemm_f32_dd(h3_cuda *cuda, const float *d_x, const float *d_weight, size_t m, size_t n, size_t k, float *d_y,
                        double *gemm_ms, char *error, size_t error_size) {
    Timer t(cuda, gemm_ms);
    const int ok = launch_dense(cuda, d_x, d_weight, nullptr, m, n, k, d_y, error, error_size);
    t.stop();
    return ok;
}

int h3_cuda_gemm_f32_dd_ex(h3_cuda *cuda, const float *d_x, const float *d_weight, size_t m, size_t n, size_t k, float *d_y,
                           float alpha, float beta, double *gemm_ms, char *error, size_t error_size) {
    Timer t(cuda, gemm_ms);
    const int ok = launch_dense(cuda, d_x, d_weight, nullptr, m, n, k, d_y, error, error_size, alpha, beta);
    t.stop();
    return ok;
}

// The reference's TF32 form of the same product (CUBLAS_COMPUTE_32F_FAST_TF32, its LoRA option): computed
// in full f32 here, which is at least as accurate.
int h3_cuda_gemm_f32_dd_tf32_ex(h3_cuda *cuda, const float *d_x, const float *d_weight, size_t m, size_t n, size_t k,
                                float *d_y, float alpha, float beta, char *error, size_t error_size) {
    return launch_dense(cuda, d_x, d_weight, nullptr, m, n, k, d_y, error, error_size, alpha, beta);
}

int h3_cuda_bias_add_f32_dev(h3_cuda *cuda, float *d_y, const float *d_bias, size_t rows, size_t width, char *error,
                             size_t error_size) {
    if (!cuda || !d_y || !d_bias || rows == 0 || width == 0) return fail(error, error_size, "invalid bias_add arguments");
    ProfScope prof(cuda, PROF_OTHER);
    k_bias_add_f32<<<stream_grid(cuda, rows * width, 256), 256, 0, cuda->op_stream>>>(d_y, d_bias, rows * width, width);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_bias_add_f32 launch");
    return 1;
}

int h3b_dense_f32_dev(h3_cuda *cuda, const float *d_x, const float *d_weight, const float *d_bias, size_t m, size_t n,
                      size_t k, float *d_y, char *error, size_t error_size) {
    return launch_dense(cuda, d_x, d_weight, d_bias, m, n, k, d_y, error, error_size);
}

int h3b_final_head_f32_dev(h3_cuda *cuda, const float *d_x, const float *d_norm_w, const float *d_modulation, size_t seq,
                           size_t hidden, const float *d_weight, const float *d_bias, size_t out_dim, float epsilon,
                           void *d_scratch, size_t scratch_bytes, float *d_y, char *error, size_t error_size) {
    if (!cuda || !d_x || !d_norm_w || !d_modulation || !d_weight || !d_bias || !d_y || !d_scratch || seq == 0 || hidden == 0 ||
        out_dim == 0)
        return fail(error, error_size, "invalid final_head arguments");
    const size_t need = h3b_final_head_scratch_bytes(seq, hidden);
    if (scratch_bytes < need) return fail(error, error_size, "final_head: scratch of %zu bytes, %zu needed", scratch_bytes, need);
    if ((uintptr_t)d_scratch & 15) return fail(error, error_size, "final_head: scratch must be 16-byte aligned");
    float *d_normed = reinterpret_cast<float *>(d_scratch);
    uint32_t *d_map = reinterpret_cast<uint32_t *>(d_normed + seq * hidden);
    // every token reads modulation row 0 (two slots: shift, scale), as the reference's zero row map does
    H3B_CUDA_OK(cudaMemsetAsync(d_map, 0, seq * sizeof(uint32_t), cuda->op_stream), "final_head row map");
    if (!h3_cuda_adaln_f32_dev(cuda, d_x, d_norm_w, d_modulation, d_map, seq, hidden, 2, 0, 1, epsilon, d_normed, nullptr, error,
                               error_size))
        return 0;
    return launch_dense(cuda, d_normed, d_weight, d_bias, seq, out_dim, hidden, d_y, error, error_size);
}

size_t h3b_final_head_scratch_bytes(size_t seq, size_t hidden) { return seq * hidden * sizeof(float) + seq * sizeof(uint32_t); }

int h3b_euler_step_f32_dev(h3_cuda *cuda, float *d_sample, const float *d_velocity, size_t count, float sigma,
                           float sigma_next, char *error, size_t error_size) {
    if (!cuda || !d_sample || !d_velocity || count == 0) return fail(error, error_size, "invalid euler_step args");
    if (!isfinite(sigma) || !isfinite(sigma_next) || !(sigma > sigma_next) || sigma_next < 0.0f)
        return fail(error, error_size, "euler_step rejected sigma pair");
    ProfScope prof(cuda, PROF_OTHER);
    k_euler_step_f32<<<stream_grid(cuda, count, 256), 256, 0, cuda->op_stream>>>(d_sample, d_velocity, count, sigma - sigma_next);
    cuda->launches++;
    H3B_CUDA_OK(cudaGetLastError(), "k_euler_step_f32 launch");
    return 1;
}

}  // extern "C"
