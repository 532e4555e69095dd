// Handle lifecycle, streams, events, scratch and tensor-map encoding.
#include <stdlib.h>
#include <string.h>

#include "h3b_internal.h"
#include "h3b_ptx.cuh"

namespace h3b {

int fail(char *error, size_t error_size, const char *fmt, ...) {
    if (error && error_size) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(error, error_size, fmt, ap);
        va_end(ap);
    }
    return 0;
}

int cuda_fail(cudaError_t e, const char *what, char *error, size_t error_size) {
    return fail(error, error_size, "%s: %s", what, cudaGetErrorString(e));
}

int grow(h3_cuda *cuda, void **slot, size_t *have, size_t bytes, char *error, size_t error_size) {
    if (*have >= bytes && *slot) return 1;
    if (cuda->graph_capture) return fail(error, error_size, "scratch growth is forbidden during graph capture");
    if (*slot) {
        // the previous buffer may still be in use by enqueued work
        cudaStreamSynchronize(cuda->op_stream);
        cudaFree(*slot);
        *slot = NULL;
        *have = 0;
    }
    H3B_CUDA_OK(cudaMalloc(slot, bytes), "cudaMalloc(scratch)");
    *have = bytes;
    return 1;
}

Timer::Timer(h3_cuda *c, double *out) : cuda(c), ms(out), on(out && !c->quiet && !c->graph_capture) {
    if (ms) *ms = 0.0;
    if (on) cudaEventRecord(cuda->ev0, cuda->op_stream);
}
void Timer::stop() {
    if (!on) return;
    float t = 0.0f;
    cudaEventRecord(cuda->ev1, cuda->op_stream);
    cudaEventSynchronize(cuda->ev1);
    cudaEventElapsedTime(&t, cuda->ev0, cuda->ev1);
    *ms = (double)t;
    on = false;
}

ProfScope::ProfScope(h3_cuda *c, int cls) : cuda(c), slot(-1) {
    if (!c->prof_on || c->graph_capture) return;
    if (c->prof_n == c->prof_cap) {
        int cap = c->prof_cap ? c->prof_cap * 2 : 1024;
        cudaEvent_t *ev = (cudaEvent_t *)realloc(c->prof_ev, sizeof(cudaEvent_t) * 2 * cap);
        int *cl = (int *)realloc(c->prof_cls, sizeof(int) * cap);
        if (!ev || !cl) return;
        c->prof_ev = ev;
        c->prof_cls = cl;
        for (int i = c->prof_cap; i < cap; i++) {
            cudaEventCreate(&ev[2 * i]);
            cudaEventCreate(&ev[2 * i + 1]);
        }
        c->prof_cap = cap;
    }
    slot = c->prof_n++;
    c->prof_cls[slot] = cls;
    cudaEventRecord(c->prof_ev[2 * slot], c->op_stream);
}
ProfScope::~ProfScope() {
    if (slot >= 0) cudaEventRecord(cuda->prof_ev[2 * slot + 1], cuda->op_stream);
}

// cuTensorMapEncodeTiled is reached through the runtime so that the library
// needs no link-time dependency on libcuda.
typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_fn get_encode() {
    static encode_fn fn = NULL;
    if (!fn) {
        void *p = NULL;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (encode_fn)p;
    }
    return fn;
}

int h3b_encode_tmap_2d(CUtensorMap *map, CUtensorMapDataType dtype, size_t elem_bytes, const void *base,
                       uint64_t inner, uint64_t outer, uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer,
                       CUtensorMapSwizzle swizzle) {
    encode_fn fn = get_encode();
    if (!fn) return -1;
    (void)elem_bytes;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return (int)fn(map, dtype, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

int h3b_encode_tmap_3d(CUtensorMap *map, CUtensorMapDataType dtype, size_t elem_bytes, const void *base,
                       uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1, uint64_t stride2, uint32_t b0,
                       uint32_t b1, uint32_t b2, CUtensorMapSwizzle swizzle) {
    encode_fn fn = get_encode();
    if (!fn) return -1;
    (void)elem_bytes;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1, stride2};
    cuuint32_t box[3] = {b0, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    return (int)fn(map, dtype, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

}  // namespace h3b

using namespace h3b;

static int fill_info(int dev, h3_cuda_device_info *info, char *error, size_t error_size) {
    cudaDeviceProp prop;
    H3B_CUDA_OK(cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties");
    memset(info, 0, sizeof(*info));
    info->device_index = dev;
    snprintf(info->name, sizeof(info->name), "%s", prop.name);
    info->compute_major = prop.major;
    info->compute_minor = prop.minor;
    info->total_memory_bytes = prop.totalGlobalMem;
    info->multiprocessor_count = prop.multiProcessorCount;
    cudaDriverGetVersion(&info->driver_version);
    cudaRuntimeGetVersion(&info->runtime_version);
    return 1;
}

extern "C" {

int h3_cuda_device_count(char *error, size_t error_size) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaGetDeviceCount", error, error_size);
        return 0;
    }
    return n;
}

int h3_cuda_probe(int device_index, h3_cuda_device_info *info, char *error, size_t error_size) {
    if (!info) return fail(error, error_size, "h3_cuda_probe: info is NULL");
    return fill_info(device_index < 0 ? 0 : device_index, info, error, error_size);
}

h3_cuda *h3_cuda_create(int device_index, char *error, size_t error_size) {
    int dev = device_index < 0 ? 0 : device_index;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        fail(error, error_size, "h3_cuda_create: no CUDA device (%s); this library has no CPU path",
             e == cudaSuccess ? "count 0" : cudaGetErrorString(e));
        return NULL;
    }
    if (dev >= n) {
        fail(error, error_size, "h3_cuda_create: device %d out of range (%d devices)", dev, n);
        return NULL;
    }
    h3_cuda *c = (h3_cuda *)calloc(1, sizeof(h3_cuda));
    if (!c) {
        fail(error, error_size, "h3_cuda_create: out of host memory");
        return NULL;
    }
    c->device = dev;
    if (cudaSetDevice(dev) != cudaSuccess || !fill_info(dev, &c->info, error, error_size)) {
        free(c);
        return NULL;
    }
    if (c->info.compute_major != 10) {
        fail(error, error_size,
             "h3_cuda_create: device %d is sm_%d%d; this library is built for sm_100a (B200) only", dev,
             c->info.compute_major, c->info.compute_minor);
        free(c);
        return NULL;
    }
    c->sm_count = c->info.multiprocessor_count;
    if (cudaMalloc((void **)&c->d_status, sizeof(int)) != cudaSuccess ||
        cudaMemset(c->d_status, 0, sizeof(int)) != cudaSuccess ||
        cudaEventCreate(&c->ev0) != cudaSuccess || cudaEventCreate(&c->ev1) != cudaSuccess) {
        fail(error, error_size, "h3_cuda_create: device set-up failed: %s", cudaGetErrorString(cudaGetLastError()));
        free(c);
        return NULL;
    }
    for (int i = 0; i < 4; i++) cudaStreamCreateWithFlags(&c->side[i], cudaStreamNonBlocking);
    return c;
}

void h3_cuda_release_heavy_workspace(h3_cuda *cuda) {
    if (!cuda) return;
    cudaSetDevice(cuda->device);
    cudaStreamSynchronize(cuda->op_stream);
    void **slots[] = {&cuda->act_q, &cuda->act_s, &cuda->act_rot, &cuda->attn, &cuda->rq, &cuda->kvx, &cuda->wtmp, &cuda->splitk};
    size_t *sizes[] = {&cuda->act_q_bytes, &cuda->act_s_bytes, &cuda->act_rot_bytes, &cuda->attn_bytes, &cuda->rq_bytes,
                       &cuda->kvx_bytes, &cuda->wtmp_bytes, &cuda->splitk_bytes};
    for (int i = 0; i < 8; i++) {
        if (*slots[i]) cudaFree(*slots[i]);
        *slots[i] = NULL;
        *sizes[i] = 0;
    }
    cuda->pregrown = 0;
}

void h3_cuda_free(h3_cuda *cuda) {
    if (!cuda) return;
    h3_cuda_release_heavy_workspace(cuda);
    for (int i = 0; i < 4; i++)
        if (cuda->side[i]) cudaStreamDestroy(cuda->side[i]);
    if (cuda->ev0) cudaEventDestroy(cuda->ev0);
    if (cuda->ev1) cudaEventDestroy(cuda->ev1);
    if (cuda->d_status) cudaFree(cuda->d_status);
    for (int i = 0; i < 2 * cuda->prof_cap; i++) cudaEventDestroy(cuda->prof_ev[i]);
    free(cuda->prof_ev);
    free(cuda->prof_cls);
    free(cuda);
}

int h3_cuda_pregrow_dit_scratch(h3_cuda *cuda, size_t seq, size_t hidden, size_t heads, size_t head_dim,
                                size_t ffn, char *error, size_t error_size) {
    if (!cuda || !seq || !hidden) return fail(error, error_size, "pregrow_dit_scratch: invalid arguments");
    size_t widest = hidden > ffn ? hidden : ffn;
    size_t inner = heads * head_dim;
    if (inner > widest) widest = inner;
    size_t rows = (seq + 127) / 128 * 128;
    if (!grow(cuda, &cuda->act_q, &cuda->act_q_bytes, rows * widest, error, error_size)) return 0;
    if (!grow(cuda, &cuda->act_s, &cuda->act_s_bytes, rows * sizeof(float), error, error_size)) return 0;
    if (!grow(cuda, &cuda->act_rot, &cuda->act_rot_bytes, rows * widest * sizeof(float), error, error_size))
        return 0;
    if (inner && !grow(cuda, &cuda->attn, &cuda->attn_bytes, rows * inner * 2 * 4, error, error_size)) return 0;
    cuda->pregrown = 1;
    return 1;
}

int h3_cuda_pregrow_hadamard(h3_cuda *cuda, int gs, char *error, size_t error_size) {
    // The rotation is computed by butterflies; there is no matrix to upload.
    if (!cuda) return fail(error, error_size, "pregrow_hadamard: NULL handle");
    if (gs != 0 && gs != 4 && gs != 16 && gs != 64 && gs != 256)
        return fail(error, error_size, "pregrow_hadamard: group size %d is not 0 or 4^p <= 256", gs);
    return 1;
}

int h3_cuda_dit_scratch_pregrown(const h3_cuda *cuda) { return cuda ? cuda->pregrown : 0; }

int h3_cuda_bind_device(h3_cuda *cuda, char *error, size_t error_size) {
    if (!cuda) return fail(error, error_size, "bind_device: NULL handle");
    H3B_CUDA_OK(cudaSetDevice(cuda->device), "cudaSetDevice");
    return 1;
}

int h3_cuda_get_info(const h3_cuda *cuda, h3_cuda_device_info *info) {
    if (!cuda || !info) return 0;
    *info = cuda->info;
    return 1;
}

int h3_cuda_mem_info(h3_cuda *cuda, size_t *free_bytes, size_t *total_bytes, char *error, size_t error_size) {
    size_t f = 0, t = 0;
    if (!cuda) return fail(error, error_size, "mem_info: NULL handle");
    H3B_CUDA_OK(cudaMemGetInfo(&f, &t), "cudaMemGetInfo");
    cuda->info.free_memory_bytes = f;
    cuda->info.total_memory_bytes = t;
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return 1;
}

void h3_cuda_set_graph_capture(h3_cuda *cuda, int enabled) {
    if (cuda) cuda->graph_capture = enabled ? 1 : 0;
}
int h3_cuda_graph_capture(const h3_cuda *cuda) { return cuda ? cuda->graph_capture : 0; }
void h3_cuda_set_quiet(h3_cuda *cuda, int enabled) {
    if (cuda) cuda->quiet = enabled ? 1 : 0;
}
int h3_cuda_quiet(const h3_cuda *cuda) { return cuda ? cuda->quiet : 0; }

int h3_cuda_set_op_stream(h3_cuda *cuda, void *stream, char *error, size_t error_size) {
    if (!cuda) return fail(error, error_size, "set_op_stream: NULL handle");
    cuda->op_stream = (cudaStream_t)stream;
    return 1;
}
void *h3_cuda_op_stream(const h3_cuda *cuda) { return cuda ? (void *)cuda->op_stream : NULL; }
void *h3_cuda_stream(h3_cuda *cuda, int index) {
    if (!cuda || index < 0 || index >= 4) return NULL;
    return (void *)cuda->side[index];
}
int h3_cuda_stream_count(void) { return 4; }

int h3_cuda_event_record_default(h3_cuda *cuda, void **out_event, char *error, size_t error_size) {
    cudaEvent_t ev;
    if (!cuda || !out_event) return fail(error, error_size, "event_record_default: invalid arguments");
    H3B_CUDA_OK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
    cudaError_t e = cudaEventRecord(ev, cuda->op_stream);
    if (e != cudaSuccess) {
        cudaEventDestroy(ev);
        return cuda_fail(e, "cudaEventRecord", error, error_size);
    }
    *out_event = (void *)ev;
    return 1;
}
int h3_cuda_event_record(void *stream, void *event, char *error, size_t error_size) {
    if (!event) return fail(error, error_size, "event_record: NULL event");
    H3B_CUDA_OK(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream), "cudaEventRecord");
    return 1;
}
int h3_cuda_stream_wait_event(void *stream, void *event, char *error, size_t error_size) {
    if (!event) return fail(error, error_size, "stream_wait_event: NULL event");
    H3B_CUDA_OK(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0), "cudaStreamWaitEvent");
    return 1;
}
void h3_cuda_event_destroy(void *event) {
    if (event) cudaEventDestroy((cudaEvent_t)event);
}

void *h3_cuda_host_alloc(size_t bytes, int *pinned_out) {
    void *p = NULL;
    if (cudaHostAlloc(&p, bytes, cudaHostAllocDefault) == cudaSuccess) {
        if (pinned_out) *pinned_out = 1;
        return p;
    }
    cudaGetLastError();
    if (pinned_out) *pinned_out = 0;
    return malloc(bytes);
}
void h3_cuda_host_free(void *p, int pinned) {
    if (!p) return;
    if (pinned) cudaFreeHost(p);
    else free(p);
}

int h3b_cuda_check(h3_cuda *cuda, int *status_out, char *error, size_t error_size) {
    int st = 0;
    if (!cuda) return fail(error, error_size, "h3b_cuda_check: NULL handle");
    H3B_CUDA_OK(cudaStreamSynchronize(cuda->op_stream), "cudaStreamSynchronize");
    H3B_CUDA_OK(cudaMemcpy(&st, cuda->d_status, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
    H3B_CUDA_OK(cudaGetLastError(), "sticky CUDA error");
    if (status_out) *status_out = st;
    if (st != 0) {
        cudaMemset(cuda->d_status, 0, sizeof(int));
        // a GEMM that gave up may have left the counters of its split tail tiles mid-count: start them over
        if (cuda->splitk) cudaMemset(cuda->splitk, 0, cuda->splitk_bytes < 1024 ? cuda->splitk_bytes : 1024);
        return fail(error, error_size, "a kernel gave up a bounded wait (status %d); its output is invalid", st);
    }
    return 1;
}

void h3b_cuda_profile_begin(h3_cuda *cuda) {
    if (!cuda) return;
    cuda->prof_n = 0;
    cuda->prof_on = 1;
}

int h3b_cuda_profile_end(h3_cuda *cuda, double *ms_by_class, int *launches_by_class, int n_classes) {
    if (!cuda || !ms_by_class || !launches_by_class) return 0;
    cuda->prof_on = 0;
    cudaStreamSynchronize(cuda->op_stream);
    for (int i = 0; i < n_classes; i++) {
        ms_by_class[i] = 0.0;
        launches_by_class[i] = 0;
    }
    for (int i = 0; i < cuda->prof_n; i++) {
        float t = 0.0f;
        int c = cuda->prof_cls[i];
        if (c < 0 || c >= n_classes) continue;
        if (cudaEventElapsedTime(&t, cuda->prof_ev[2 * i], cuda->prof_ev[2 * i + 1]) == cudaSuccess) {
            ms_by_class[c] += (double)t;
            launches_by_class[c]++;
        }
    }
    cuda->prof_n = 0;
    return n_classes < PROF_CLASSES ? n_classes : PROF_CLASSES;
}

unsigned long long h3b_cuda_launch_count(h3_cuda *cuda, int reset) {
    unsigned long long n;
    if (!cuda) return 0;
    n = cuda->launches;
    if (reset) cuda->launches = 0;
    return n;
}

}  // extern "C"
