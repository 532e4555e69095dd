// Tensor-pipe rate probe: every SM issues back-to-back tcgen05.mma on one resident shared-memory tile
// (no loads, no epilogue), which gives the sustained MMA rate of the part under its power limit for
// int8, bf16 and block-scaled fp4 -- the denominators the GEMM and attention kernels are measured against.
// Built into libh3_b200_probe.so, a helper of the bench, not into the product library.
#include "../h3b_internal.h"
#include "../h3b_ptx.cuh"

namespace h3b {

__device__ __forceinline__ void umma_nvfp4_probe(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}

// KIND 0: int8 128x256x32, 1: bf16 128x256x16, 2: nvfp4 128x256x64 (zero scales),
// 3: bf16 128x128x16, both operands K-major in shared memory (the attention score product),
// 4: bf16 128x128x16, A from tensor memory, B MN-major (the attention P V product),
// 5: nvfp4 128x128x64 (zero scales)
template <int KIND>
__global__ void __launch_bounds__(128, 1) k_umma_peak(int iters, int *status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    // pseudo-random operand bytes: all-zero data would toggle nothing and flatter the power-limited rate
    for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t *>(smem)[i] = (uint32_t)(i + blockIdx.x * 7919) * 2654435761u;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_word = 0;
        mbar_fence_init();
    }
    fence_proxy_async_smem();
    if (threadIdx.x < 32) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) {
        const uint32_t a_addr = smem_u32(smem), b_addr = a_addr + 16384;
        constexpr uint32_t idesc = KIND == 0   ? umma_idesc(2, 1, 1, 128, 256, 0, 0)
                                   : KIND == 1 ? umma_idesc(1, 1, 1, 128, 256, 0, 0)
                                   : KIND == 3 ? umma_idesc(1, 1, 1, 128, 128, 0, 0)
                                   : KIND == 4 ? umma_idesc(1, 1, 1, 128, 128, 0, 1)
                                   : KIND == 5 ? ((1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24))
                                               : ((1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24));
        for (int it = 0; it < iters; it++) {
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint64_t ad = umma_desc_k_sw128(a_addr + k * 32), bd = umma_desc_k_sw128(b_addr + k * 32);
                if (KIND == 0) umma_i8_ss(tmem_base, ad, bd, idesc, 1);
                else if (KIND == 1 || KIND == 3) umma_f16_ss(tmem_base, ad, bd, idesc, 1);
                else if (KIND == 4)
                    umma_f16_ts(tmem_base, tmem_base + 256 + k * 8, umma_desc_mn_sw128(b_addr + k * 2048, 16384, 1024),
                                idesc, 1);
                else umma_nvfp4_probe(tmem_base, ad, bd, idesc, tmem_base + 256, tmem_base + 272, 1);
            }
        }
        tc_commit(&bar);
        mbar_wait(&bar, 0, &abort_word, status, H3B_ST_TIMEOUT_OTHER);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace h3b

using namespace h3b;

extern "C" int h3b_umma_peak_dev(h3_cuda *cuda, int kind, int iters, double *tera_ops_per_s, char *error,
                                 size_t error_size) {
    if (!cuda || !tera_ops_per_s || iters <= 0 || kind < 0 || kind > 5)
        return fail(error, error_size, "umma_peak: invalid arguments");
    const size_t smem = 1024 + 16384 + 32768;
    cudaEvent_t e0 = cuda->ev0, e1 = cuda->ev1;
    const double ops_per_mma = kind == 5 ? 2.0 * 128 * 128 * 64 : kind >= 3 ? 2.0 * 128 * 128 * 16 : 2.0 * 128 * 256 * (kind == 0 ? 32 : kind == 1 ? 16 : 64);
    for (int rep = 0; rep < 2; rep++) {   // first launch warms up
        H3B_CUDA_OK(cudaEventRecord(e0, cuda->op_stream), "cudaEventRecord");
        if (kind == 0) {
            H3B_CUDA_OK(cudaFuncSetAttribute(k_umma_peak<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "attr");
            k_umma_peak<0><<<cuda->sm_count, 128, smem, cuda->op_stream>>>(iters, cuda->d_status);
        } else if (kind == 1) {
            H3B_CUDA_OK(cudaFuncSetAttribute(k_umma_peak<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "attr");
            k_umma_peak<1><<<cuda->sm_count, 128, smem, cuda->op_stream>>>(iters, cuda->d_status);
        } else if (kind == 3) {
            H3B_CUDA_OK(cudaFuncSetAttribute(k_umma_peak<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "attr");
            k_umma_peak<3><<<cuda->sm_count, 128, smem, cuda->op_stream>>>(iters, cuda->d_status);
        } else if (kind == 4) {
            H3B_CUDA_OK(cudaFuncSetAttribute(k_umma_peak<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "attr");
            k_umma_peak<4><<<cuda->sm_count, 128, smem, cuda->op_stream>>>(iters, cuda->d_status);
        } else if (kind == 5) {
            H3B_CUDA_OK(cudaFuncSetAttribute(k_umma_peak<5>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "attr");
            k_umma_peak<5><<<cuda->sm_count, 128, smem, cuda->op_stream>>>(iters, cuda->d_status);
        } else {
            H3B_CUDA_OK(cudaFuncSetAttribute(k_umma_peak<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "attr");
            k_umma_peak<2><<<cuda->sm_count, 128, smem, cuda->op_stream>>>(iters, cuda->d_status);
        }
        cuda->launches++;
        H3B_CUDA_OK(cudaGetLastError(), "k_umma_peak launch");
        H3B_CUDA_OK(cudaEventRecord(e1, cuda->op_stream), "cudaEventRecord");
        H3B_CUDA_OK(cudaEventSynchronize(e1), "cudaEventSynchronize");
    }
    float ms = 0.0f;
    H3B_CUDA_OK(cudaEventElapsedTime(&ms, e0, e1), "cudaEventElapsedTime");
    *tera_ops_per_s = ops_per_mma * 4.0 * iters * cuda->sm_count / (ms * 1e-3) / 1e12;
    return 1;
}
