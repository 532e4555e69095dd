// A quantised linear that allocates nothing.
//
// The ordinary device linear (h3_cuda_gemm_i8_dequant_f32_w_act_dev) needs scratch for the
// activation's INT8 codes and per-row scales and grows it with cudaMalloc on demand.  Some hosts
// cannot let it do that: a step loop that has already handed every free byte of device memory to
// resident weights, a caller that must not trigger the device-wide synchronisation an allocation
// or free implies in the middle of its own pipelining, or a caller running the handle in the mode
// where growing library scratch is refused.  For them this file keeps a fixed scratch area inside
// the library image itself: a file-scope __device__ array that every GPU loading the library
// carries until the process exits.
#include "h3b_internal.h"

namespace h3b {

// Limits of the no-allocation linear.
constexpr size_t NOALLOC_MAX_CODES = 8u << 20;   // m * k <= 8 Mi activation codes (8 MiB)
constexpr size_t NOALLOC_MAX_ROWS = 16384;       // m <= 16384 rows (64 KiB of scales)

// [ codes: NOALLOC_MAX_CODES bytes | scales: NOALLOC_MAX_ROWS floats ]
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_MAX_CODES + NOALLOC_MAX_ROWS * sizeof(float)];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not an address a kernel can
// use; the device address is looked up once per device and cached here.  The cache is written
// without a lock: every writer of a slot stores the same value (the address of the symbol on that
// device does not change), so racing first calls are harmless.
static void *g_noalloc_ptr[64];

// The handle's device must be the calling thread's current device: the kernels below are launched
// on the current device with the scratch address of cuda->device.  A mismatch is refused on every
// call rather than repaired, so that the caller's device binding is never changed behind its back
// (h3_cuda_bind_device is the call that binds).
static int noalloc_scratch(h3_cuda *cuda, void **out, char *error, size_t error_size) {
    const int dev = cuda->device;
    if (dev < 0 || dev >= 64) return fail(error, error_size, "no-alloc linear: device index %d out of range", dev);
    int cur = -1;
    H3B_CUDA_OK(cudaGetDevice(&cur), "cudaGetDevice");
    if (cur != dev)
        return fail(error, error_size,
                    "no-alloc linear: the handle belongs to device %d but device %d is current; call h3_cuda_bind_device first",
                    dev, cur);
    if (!g_noalloc_ptr[dev]) {
        void *p = NULL;
        H3B_CUDA_OK(cudaGetSymbolAddress(&p, g_noalloc_scratch), "cudaGetSymbolAddress(no-alloc scratch)");
        if (!p) return fail(error, error_size, "no-alloc linear: scratch symbol has no device address");
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return 1;
}

}  // namespace h3b

using namespace h3b;

extern "C" {

size_t h3b_linear_noalloc_max_codes(void) { return NOALLOC_MAX_CODES; }
size_t h3b_linear_noalloc_max_rows(void) { return NOALLOC_MAX_ROWS; }

int h3b_gemm_i8_dequant_f32_w_act_dev_noalloc(h3_cuda *cuda, const h3_cuda_w4a8_weight *weight,
                                              const float *d_x_f32, int convrot_groupsize, size_t m,
                                              float *d_y_f32, char *error, size_t error_size) {
    if (!cuda || !weight || !d_x_f32 || !d_y_f32 || !m)
        return fail(error, error_size, "no-alloc linear: invalid arguments");
    const size_t k = weight->k;
    if (m > NOALLOC_MAX_ROWS || m * k > NOALLOC_MAX_CODES)
        return fail(error, error_size,
                    "no-alloc linear: m=%zu, k=%zu exceeds the built-in scratch (at most %zu rows and %zu codes = m*k); "
                    "use h3_cuda_gemm_i8_dequant_f32_w_act_dev, which allocates",
                    m, k, NOALLOC_MAX_ROWS, NOALLOC_MAX_CODES);
    if (weight->pending) return fail(error, error_size, "no-alloc linear: weight upload still pending; call h3_cuda_w4a8_weight_ensure_ready first");
    if (weight->device != cuda->device)   // before anything is enqueued
        return fail(error, error_size, "no-alloc linear: the weight lives on device %d, the handle on device %d", weight->device,
                    cuda->device);
    void *base = NULL;
    if (!noalloc_scratch(cuda, &base, error, error_size)) return 0;
    int8_t *codes = reinterpret_cast<int8_t *>(base);
    float *scales = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(base) + NOALLOC_MAX_CODES);
    // The quantise kernel writes every code and scale of rows [0, m) before the GEMM reads them, and
    // the GEMM's tensor map ends at row m, so nothing in the scratch has to start at zero.
    h3b_norm_args a;
    memset(&a, 0, sizeof(a));
    a.d_x = d_x_f32; a.rows = m; a.width = k; a.dtype = H3B_F32; a.identity = 1;
    a.convrot_gs = convrot_groupsize > 0 ? convrot_groupsize : 0;
    a.d_q = codes; a.d_scales = scales;
    if (!launch_norm(cuda, &a, error, error_size)) return 0;
    h3b_gemm_epi e;
    memset(&e, 0, sizeof(e));
    e.kind = H3B_EPI_PLAIN; e.out_dtype = H3B_F32;
    return launch_gemm_i8(cuda, weight, codes, scales, m, d_y_f32, &e, error, error_size);
}

}  // extern "C"
