// Ulysses sequence<->head all-to-all around self-attention (the reference's h3_ulysses_comm.cu,
// six-function API kept) over NCCL point-to-point groups on NVLink.
//
// Two ways to own ranks:
//   h3_ulysses_comm_init       one process drives every GPU (the reference's model,
//                              h3_ulysses_comm.cu:221 ncclCommInitAll)
//   h3b_ulysses_comm_init_rank one process per GPU: the caller distributes a 128-byte NCCL
//                              unique id (h3b_ulysses_unique_id) by its own means
// Index maps (h3_ulysses_comm.cu:256-344), hl = heads / U:
//   QKV:       in[s][q][h][d] -> pack[peer = h / hl][s][q][h % hl][d]; peer p's chunk lands as
//              out[(src * seq_local + s)][q][hl][d] on rank p -- the received chunks already are
//              the output layout, so they are received in place and no unpack kernel is needed
//   attn-out:  in[(src * seq_local + s)][hl][d] is already chunked by destination, sent as it is;
//              unpack[peer][s][hl][d] -> out[s][peer * hl + hl'][d]
// Exchange-free form (h3b_ulysses_direct_*, one process per GPU): every rank allocates one slab
// [gathered Q | K | V | attention rows], the ranks swap CUDA IPC handles through the communicator and
// map each other's slabs; the QKV GEMM epilogue and the attention epilogue then store across NVLink
// into the slab of the rank that needs each (row, head) slice, and a flag kernel on the compute stream
// (or a one-word all-reduce) is the barrier that makes the stores of all ranks visible (and keeps a fast
// rank from overwriting what a slow one still reads).  No pack, exchange or unpack remains on the critical path.
// NCCL is bound at run time (dlopen of libnccl.so.2) so the library loads where NCCL is absent;
// every entry point then fails with a message, like the reference's stub (h3_ulysses_comm_stub.c).
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include "h3b_internal.h"

namespace h3b {

struct NcclApi {
    void *handle;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)(void);
    ncclResult_t (*GroupEnd)(void);
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    const char *(*GetErrorString)(ncclResult_t);
};

static NcclApi *nccl_api(char *err, size_t err_size) {
    static NcclApi api;
    static int state = 0;   // 0 untried, 1 ok, -1 failed
    if (state == 0) {
        const char *names[] = {"libnccl.so.2", "libnccl.so"};
        for (int i = 0; i < 2 && !api.handle; i++) api.handle = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
        state = -1;
        if (api.handle) {
#define H3B_SYM(field, name) *(void **)(&api.field) = dlsym(api.handle, name)
            H3B_SYM(GetUniqueId, "ncclGetUniqueId");
            H3B_SYM(CommInitRank, "ncclCommInitRank");
            H3B_SYM(CommInitAll, "ncclCommInitAll");
            H3B_SYM(CommDestroy, "ncclCommDestroy");
            H3B_SYM(Send, "ncclSend");
            H3B_SYM(Recv, "ncclRecv");
            H3B_SYM(GroupStart, "ncclGroupStart");
            H3B_SYM(GroupEnd, "ncclGroupEnd");
            H3B_SYM(AllGather, "ncclAllGather");
            H3B_SYM(AllReduce, "ncclAllReduce");
            H3B_SYM(GetErrorString, "ncclGetErrorString");
#undef H3B_SYM
            if (api.GetUniqueId && api.CommInitRank && api.CommInitAll && api.CommDestroy && api.Send && api.Recv &&
                api.GroupStart && api.GroupEnd && api.AllGather && api.AllReduce)
                state = 1;
        }
    }
    if (state != 1) {
        fail(err, err_size, "ulysses comm: NCCL not available (libnccl.so.2 could not be loaded)");
        return NULL;
    }
    return &api;
}

enum { MAX_U = 8 };

struct CommState {
    int n_ranks;             // U
    int n_local;             // ranks owned by this process
    int local_rank[MAX_U];   // global rank of each owned slot
    int device[MAX_U];
    ncclComm_t comm[MAX_U];
    cudaStream_t stream[MAX_U];    // communication stream
    cudaStream_t compute[MAX_U];   // borrowed compute stream (NULL = legacy default)
    cudaEvent_t ev_compute[MAX_U], ev_comm[MAX_U];
    void *scratch[MAX_U];
    size_t scratch_bytes[MAX_U];
    const void *bound_in[MAX_U];
    void *bound_out[MAX_U];
    // direct stores (one owned rank only): this rank's slab [q | k | v | att], the peers' slabs as mapped
    // here through CUDA IPC, and the one-word buffers of the barrier
    h3b_ulysses_direct direct;
    int direct_ready, direct_off;
    void *slab;
    void *peer_slab[MAX_U];
    int *d_barrier;                // [0..1] words of the NCCL barrier, [2] epoch of the flag barrier, [3] its status
    uint32_t *peer_flags[MAX_U];   // rank r's arrival flags (one word per rank) at the end of its slab
    int flag_barrier;              // 1: barriers are the flag kernel, 0: the one-word all-reduce
};

static int slot_of(const CommState *st, int rank) {
    for (int i = 0; i < st->n_local; i++)
        if (st->local_rank[i] == rank) return i;
    return -1;
}

// in[s][q][h][d] -> out[peer][s][q][hl][d]; 16-byte vectors (head_dim * elem is a multiple of 16)
// Barrier of the exchange-free form: every rank writes the next epoch into its word of every peer's flag row
// and waits until its own row shows that epoch (or a later one: a rank that is already through may have moved
// on) from everybody.  One warp, lane r talks to rank r.  The earlier kernels of the stream have finished, so
// their stores into peer memory are ordered before the release store of the flag on the same NVLink path; the
// acquire load orders the reads of the kernels that follow.  The wait is bounded: after about two seconds the
// kernel records status 6 in `state[1]` and returns, and later barriers only signal until the status is read.
struct FlagBarrier {
    uint32_t *peer_flags[8];
    int *state;   // [0] epoch, [1] status
    int rank, world;
    long long budget;
};
__global__ void k_ulysses_flag_barrier(const __grid_constant__ FlagBarrier p) {
    __shared__ uint32_t epoch_s;
    if (threadIdx.x == 0) {
        epoch_s = (uint32_t)p.state[0] + 1u;
        p.state[0] = (int)epoch_s;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    __threadfence_system();
    const int r = (int)threadIdx.x;
    if (r >= p.world) return;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.peer_flags[r] + p.rank), "r"(epoch) : "memory");
    const uint32_t *mine = p.peer_flags[p.rank] + r;
    if (*(volatile int *)&p.state[1] != 0) return;   // an earlier barrier gave up: signal, but do not wait again
    const long long start = clock64();
    uint32_t spins = 0;
    while (true) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int32_t)(seen - epoch) >= 0) break;
        if ((++spins & 0xff) == 0 && clock64() - start > p.budget) {
            atomicCAS(&p.state[1], 0, 6);
            break;
        }
    }
}

__global__ void k_ulysses_pack_qkv(const uint4 *in, uint4 *out, size_t seq_local, unsigned heads, unsigned vec_per_head,
                                   unsigned u) {
    const unsigned hl = heads / u;
    const size_t n = seq_local * 3 * heads * vec_per_head;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned d = (unsigned)(i % vec_per_head);
        size_t t = i / vec_per_head;
        const unsigned h = (unsigned)(t % heads);
        t /= heads;
        const unsigned q = (unsigned)(t % 3);
        const size_t s = t / 3;
        const unsigned peer = h / hl;
        out[((((size_t)peer * seq_local + s) * 3 + q) * hl + (h - peer * hl)) * vec_per_head + d] = in[i];
    }
}

// in[peer][s][hl][d] -> out[s][peer * hl + hl'][d]
__global__ void k_ulysses_unpack_attn(const uint4 *in, uint4 *out, size_t seq_local, unsigned heads,
                                      unsigned vec_per_head, unsigned u) {
    const unsigned hl = heads / u;
    const size_t n = (size_t)u * seq_local * hl * vec_per_head;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned d = (unsigned)(i % vec_per_head);
        size_t t = i / vec_per_head;
        const unsigned h = (unsigned)(t % hl);
        t /= hl;
        const size_t s = t % seq_local;
        const unsigned peer = (unsigned)(t / seq_local);
        out[(s * heads + peer * hl + h) * vec_per_head + d] = in[i];
    }
}

static unsigned copy_grid(size_t n) {
    size_t g = (n + 255) / 256;
    return (unsigned)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

static int ensure_scratch(CommState *st, int slot, size_t bytes, char *err, size_t err_size) {
    if (st->scratch_bytes[slot] >= bytes) return 1;
    if (st->scratch[slot]) {
        cudaStreamSynchronize(st->stream[slot]);
        cudaFree(st->scratch[slot]);
        st->scratch[slot] = NULL;
        st->scratch_bytes[slot] = 0;
    }
    cudaError_t e = cudaMalloc(&st->scratch[slot], bytes);
    if (e != cudaSuccess) return cuda_fail(e, "ulysses a2a: scratch allocation", err, err_size);
    st->scratch_bytes[slot] = bytes;
    return 1;
}

static int finish_init(h3_ulysses_cfg *cfg, CommState *st, char *err, size_t err_size) {
    for (int i = 0; i < st->n_local; i++) {
        if (cudaSetDevice(st->device[i]) != cudaSuccess ||
            cudaStreamCreateWithFlags(&st->stream[i], cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&st->ev_compute[i], cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&st->ev_comm[i], cudaEventDisableTiming) != cudaSuccess)
            return fail(err, err_size, "ulysses comm: stream/event creation failed on device %d", st->device[i]);
    }
    cfg->comm = st;
    return 1;
}

// order: compute stream -> comm stream
static int wait_compute(CommState *st, int i, char *err, size_t err_size) {
    cudaError_t e = cudaEventRecord(st->ev_compute[i], st->compute[i]);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(st->stream[i], st->ev_compute[i], 0);
    if (e != cudaSuccess) return cuda_fail(e, "ulysses a2a: wait compute", err, err_size);
    return 1;
}
// order: comm stream -> compute stream
static int publish_comm(CommState *st, int i, char *err, size_t err_size) {
    cudaError_t e = cudaEventRecord(st->ev_comm[i], st->stream[i]);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(st->compute[i], st->ev_comm[i], 0);
    if (e != cudaSuccess) return cuda_fail(e, "ulysses a2a: publish", err, err_size);
    return 1;
}

// exchange: slot i sends send[i] + p*chunk to rank p and receives chunk p into recv[i] + p*chunk
static int exchange(CommState *st, NcclApi *api, const char *const *send, char *const *recv, size_t chunk_bytes,
                    char *err, size_t err_size) {
    ncclResult_t rc = api->GroupStart();
    if (rc != ncclSuccess) return fail(err, err_size, "ncclGroupStart: %s", api->GetErrorString ? api->GetErrorString(rc) : "error");
    for (int i = 0; i < st->n_local; i++)
        for (int p = 0; p < st->n_ranks; p++) {
            rc = api->Send(send[i] + (size_t)p * chunk_bytes, chunk_bytes, ncclInt8, p, st->comm[i], st->stream[i]);
            if (rc == ncclSuccess)
                rc = api->Recv(recv[i] + (size_t)p * chunk_bytes, chunk_bytes, ncclInt8, p, st->comm[i], st->stream[i]);
            if (rc != ncclSuccess) {
                api->GroupEnd();
                return fail(err, err_size, "nccl send/recv a2a failed: %s", api->GetErrorString ? api->GetErrorString(rc) : "error");
            }
        }
    rc = api->GroupEnd();
    if (rc != ncclSuccess) return fail(err, err_size, "ncclGroupEnd: %s", api->GetErrorString ? api->GetErrorString(rc) : "error");
    return 1;
}

static int check_geometry(const CommState *st, size_t seq_local, size_t heads, size_t head_dim, int dtype_bytes,
                          char *err, size_t err_size) {
    if (!seq_local || !heads || !head_dim) return fail(err, err_size, "ulysses a2a: zero dimension");
    if (dtype_bytes != 2 && dtype_bytes != 4) return fail(err, err_size, "ulysses a2a: dtype_bytes must be 2 or 4");
    if (heads % (size_t)st->n_ranks) return fail(err, err_size, "ulysses a2a: heads %% U != 0");
    if ((head_dim * (size_t)dtype_bytes) % 16) return fail(err, err_size, "ulysses a2a: head_dim * dtype_bytes must be a multiple of 16");
    return 1;
}

}  // namespace h3b

using namespace h3b;

extern "C" {

int h3b_ulysses_unique_id(void *out128, char *err, size_t err_size) {
    NcclApi *api = nccl_api(err, err_size);
    if (!api) return 0;
    if (!out128) return fail(err, err_size, "ulysses unique id: NULL buffer");
    ncclUniqueId id;
    ncclResult_t rc = api->GetUniqueId(&id);
    if (rc != ncclSuccess) return fail(err, err_size, "ncclGetUniqueId failed");
    memcpy(out128, &id, sizeof(id));
    return 1;
}

int h3b_ulysses_comm_init_rank(h3_ulysses_cfg *cfg, int rank, int world_size, const void *unique_id128, int device,
                               char *err, size_t err_size) {
    if (!cfg || !unique_id128) return fail(err, err_size, "ulysses init: invalid arguments");
    if (world_size != 1 && world_size != 2 && world_size != 4 && world_size != 8)
        return fail(err, err_size, "ulysses=%d illegal (legal {1,2,4,8}; packed align)", world_size);
    if (rank < 0 || rank >= world_size) return fail(err, err_size, "ulysses init: rank %d out of range", rank);
    cfg->comm = NULL;
    cfg->ulysses = world_size; cfg->world_size = world_size; cfg->rank = rank;
    if (!cfg->tp_size) cfg->tp_size = 1;
    if (!cfg->ring) cfg->ring = 1;
    if (world_size == 1) return 1;   // U = 1: no communicator, a2a calls are refused like the reference
    NcclApi *api = nccl_api(err, err_size);
    if (!api) return 0;
    CommState *st = (CommState *)calloc(1, sizeof(CommState));
    if (!st) return fail(err, err_size, "ulysses init: out of memory");
    st->n_ranks = world_size; st->n_local = 1; st->local_rank[0] = rank; st->device[0] = device;
    if (cudaSetDevice(device) != cudaSuccess) {
        free(st);
        return fail(err, err_size, "ulysses init: cudaSetDevice(%d) failed", device);
    }
    ncclUniqueId id;
    memcpy(&id, unique_id128, sizeof(id));
    ncclResult_t rc = api->CommInitRank(&st->comm[0], world_size, id, rank);
    if (rc != ncclSuccess) {
        free(st);
        return fail(err, err_size, "ncclCommInitRank failed: %s", api->GetErrorString ? api->GetErrorString(rc) : "error");
    }
    if (!finish_init(cfg, st, err, err_size)) {
        api->CommDestroy(st->comm[0]);
        free(st);
        cfg->comm = NULL;
        return 0;
    }
    return 1;
}

int h3_ulysses_comm_init(h3_ulysses_cfg *cfg, const int *device_ids, int n_dev, char *err, size_t err_size) {
    if (!cfg) return fail(err, err_size, "ulysses init: NULL cfg");
    cfg->comm = NULL;
    if (n_dev <= 1) return 1;   // U = 1 needs no communicator (h3_ulysses_comm_stub.c:16)
    if (!device_ids) return fail(err, err_size, "ulysses init: NULL device list");
    if (n_dev != 2 && n_dev != 4 && n_dev != 8) return fail(err, err_size, "ulysses=%d illegal (legal {1,2,4,8}; packed align)", n_dev);
    NcclApi *api = nccl_api(err, err_size);
    if (!api) return 0;
    CommState *st = (CommState *)calloc(1, sizeof(CommState));
    if (!st) return fail(err, err_size, "ulysses init: out of memory");
    st->n_ranks = n_dev; st->n_local = n_dev;
    for (int i = 0; i < n_dev; i++) {
        st->local_rank[i] = i;
        st->device[i] = device_ids[i];
    }
    ncclResult_t rc = api->CommInitAll(st->comm, n_dev, device_ids);
    if (rc != ncclSuccess) {
        free(st);
        return fail(err, err_size, "ncclCommInitAll failed: %s", api->GetErrorString ? api->GetErrorString(rc) : "error");
    }
    if (!finish_init(cfg, st, err, err_size)) {
        for (int i = 0; i < n_dev; i++) api->CommDestroy(st->comm[i]);
        free(st);
        cfg->comm = NULL;
        return 0;
    }
    cfg->ulysses = n_dev; cfg->world_size = n_dev;
    return 1;
}

void h3_ulysses_comm_destroy(h3_ulysses_cfg *cfg) {
    if (!cfg || !cfg->comm) return;
    CommState *st = (CommState *)cfg->comm;
    NcclApi *api = nccl_api(NULL, 0);
    for (int i = 0; i < st->n_local; i++) {
        cudaSetDevice(st->device[i]);
        if (st->stream[i]) cudaStreamSynchronize(st->stream[i]);
        if (st->scratch[i]) cudaFree(st->scratch[i]);
        if (i == 0) {
            cudaDeviceSynchronize();
            // Peers store into this rank's slab from their GEMM and attention epilogues.  Before the mappings go and
            // the slab is freed, all ranks meet in one more (bounded) barrier, so that nobody's kernels are still in
            // flight.  If the barrier gives up (a rank left early, or one of its own barriers ran out before), the
            // slab and the mappings are deliberately left alone until the process exits: freeing memory a peer may
            // still be writing would fault that peer's GPU.
            int quiesced = 1;
            if (st->direct_ready && st->n_local == 1 && st->d_barrier) {
                h3_ulysses_cfg tmp = *cfg;
                int status = 0;
                quiesced = st->flag_barrier && h3b_ulysses_barrier(&tmp, NULL, 0) && h3b_ulysses_check(&tmp, &status, NULL, 0) &&
                           status == 0;
                if (!st->flag_barrier) {   // the all-reduce barrier: NCCL's own time-out bounds it
                    quiesced = h3b_ulysses_barrier(&tmp, NULL, 0) && cudaStreamSynchronize(st->compute[0]) == cudaSuccess;
                }
            }
            if (quiesced) {
                for (int pr = 0; pr < st->n_ranks; pr++)
                    if (st->peer_slab[pr] && st->peer_slab[pr] != st->slab) cudaIpcCloseMemHandle(st->peer_slab[pr]);
                if (st->slab) cudaFree(st->slab);
                if (st->d_barrier) cudaFree(st->d_barrier);
            }
        }
        if (api && st->comm[i]) api->CommDestroy(st->comm[i]);
        if (st->ev_compute[i]) cudaEventDestroy(st->ev_compute[i]);
        if (st->ev_comm[i]) cudaEventDestroy(st->ev_comm[i]);
        if (st->stream[i]) cudaStreamDestroy(st->stream[i]);
    }
    free(st);
    cfg->comm = NULL;
}

int h3_ulysses_comm_bind(h3_ulysses_cfg *cfg, int rank, const void *d_in, void *d_out, char *err, size_t err_size) {
    if (!cfg || !cfg->comm) return fail(err, err_size, "ulysses bind: not inited");
    CommState *st = (CommState *)cfg->comm;
    int i = slot_of(st, rank);
    if (i < 0) return fail(err, err_size, "ulysses bind: bad rank");
    st->bound_in[i] = d_in;
    st->bound_out[i] = d_out;
    return 1;
}

int h3_ulysses_comm_set_compute(h3_ulysses_cfg *cfg, int rank, void *stream, char *err, size_t err_size) {
    if (!cfg || !cfg->comm) return fail(err, err_size, "ulysses set_compute: not inited");
    CommState *st = (CommState *)cfg->comm;
    int i = slot_of(st, rank);
    if (i < 0) return fail(err, err_size, "ulysses set_compute: bad rank");
    st->compute[i] = (cudaStream_t)stream;
    return 1;
}

// d_in / d_out: with one owned rank they may be passed directly; NULL (or several owned ranks)
// selects the buffers bound per rank.  In and out may alias.
int h3_ulysses_a2a_qkv(h3_ulysses_cfg *cfg, const void *d_in, void *d_out, size_t seq_local, size_t heads,
                       size_t head_dim, int dtype_bytes, char *err, size_t err_size) {
    if (!cfg || !cfg->comm) return fail(err, err_size, "ulysses a2a_qkv: not inited");
    CommState *st = (CommState *)cfg->comm;
    NcclApi *api = nccl_api(err, err_size);
    if (!api) return 0;
    if (!check_geometry(st, seq_local, heads, head_dim, dtype_bytes, err, err_size)) return 0;
    const size_t total = seq_local * 3 * heads * head_dim * (size_t)dtype_bytes;
    const size_t chunk = total / (size_t)st->n_ranks;
    const unsigned vec = (unsigned)(head_dim * (size_t)dtype_bytes / 16);
    const char *send[MAX_U];
    char *recv[MAX_U];
    for (int i = 0; i < st->n_local; i++) {
        const void *in = (st->n_local == 1 && d_in) ? d_in : st->bound_in[i];
        void *out = (st->n_local == 1 && d_out) ? d_out : st->bound_out[i];
        if (!in || !out) return fail(err, err_size, "ulysses a2a_qkv: rank %d has no buffers", st->local_rank[i]);
        if (cudaSetDevice(st->device[i]) != cudaSuccess) return fail(err, err_size, "ulysses a2a: set device");
        if (!ensure_scratch(st, i, total, err, err_size) || !wait_compute(st, i, err, err_size)) return 0;
        k_ulysses_pack_qkv<<<copy_grid(total / 16), 256, 0, st->stream[i]>>>((const uint4 *)in, (uint4 *)st->scratch[i],
                                                                            seq_local, (unsigned)heads, vec,
                                                                            (unsigned)st->n_ranks);
        if (cudaGetLastError() != cudaSuccess) return fail(err, err_size, "ulysses a2a_qkv: pack launch failed");
        send[i] = (const char *)st->scratch[i];
        recv[i] = (char *)out;
    }
    if (!exchange(st, api, send, recv, chunk, err, err_size)) return 0;
    for (int i = 0; i < st->n_local; i++) {
        if (cudaSetDevice(st->device[i]) != cudaSuccess) return fail(err, err_size, "ulysses a2a: set device");
        if (!publish_comm(st, i, err, err_size)) return 0;
    }
    return 1;
}

int h3_ulysses_a2a_attn_out(h3_ulysses_cfg *cfg, const void *d_in, void *d_out, size_t seq_local, size_t heads,
                            size_t head_dim, int dtype_bytes, char *err, size_t err_size) {
    if (!cfg || !cfg->comm) return fail(err, err_size, "ulysses a2a_attn_out: not inited");
    CommState *st = (CommState *)cfg->comm;
    NcclApi *api = nccl_api(err, err_size);
    if (!api) return 0;
    if (!check_geometry(st, seq_local, heads, head_dim, dtype_bytes, err, err_size)) return 0;
    const size_t total = seq_local * heads * head_dim * (size_t)dtype_bytes;
    const size_t chunk = total / (size_t)st->n_ranks;
    const unsigned vec = (unsigned)(head_dim * (size_t)dtype_bytes / 16);
    const char *send[MAX_U];
    char *recv[MAX_U];
    void *outs[MAX_U];
    for (int i = 0; i < st->n_local; i++) {
        const void *in = (st->n_local == 1 && d_in) ? d_in : st->bound_in[i];
        outs[i] = (st->n_local == 1 && d_out) ? d_out : st->bound_out[i];
        if (!in || !outs[i]) return fail(err, err_size, "ulysses a2a_attn_out: rank %d has no buffers", st->local_rank[i]);
        if (cudaSetDevice(st->device[i]) != cudaSuccess) return fail(err, err_size, "ulysses a2a: set device");
        if (!ensure_scratch(st, i, total, err, err_size) || !wait_compute(st, i, err, err_size)) return 0;
        send[i] = (const char *)in;
        recv[i] = (char *)st->scratch[i];
    }
    if (!exchange(st, api, send, recv, chunk, err, err_size)) return 0;
    for (int i = 0; i < st->n_local; i++) {
        if (cudaSetDevice(st->device[i]) != cudaSuccess) return fail(err, err_size, "ulysses a2a: set device");
        k_ulysses_unpack_attn<<<copy_grid(total / 16), 256, 0, st->stream[i]>>>((const uint4 *)st->scratch[i],
                                                                               (uint4 *)outs[i], seq_local,
                                                                               (unsigned)heads, vec,
                                                                               (unsigned)st->n_ranks);
        if (cudaGetLastError() != cudaSuccess) return fail(err, err_size, "ulysses a2a_attn_out: unpack launch failed");
        if (!publish_comm(st, i, err, err_size)) return 0;
    }
    return 1;
}

// ---------------------------------------------------------------- direct stores over peer memory

// The set-up protocol as a function of its steps, so that its decision logic can run on a CPU with stand-in
// steps (tests/test_ulysses_gloo.py drives it from two gloo ranks).  Both collectives are reached by EVERY rank
// whatever happened locally before them: a rank that bailed out early would leave its peers blocked inside a
// collective.  All ranks return the same value; on 0 every rank has rolled back.
int h3b_ulysses_setup_protocol(const h3b_ulysses_setup_steps *s) {
    if (!s || !s->prepare || !s->gather || !s->map_peers || !s->agree || !s->rollback) return 0;
    int ok = s->prepare(s->ctx) != 0;           // local: allocate the buffers, make the handle
    if (!s->gather(s->ctx, ok)) ok = 0;         // collective: exchange the handles (a rank without one still takes part)
    if (ok) ok = s->map_peers(s->ctx) != 0;     // local: map the peers' buffers
    int all_ok = 0;
    if (!s->agree(s->ctx, ok, &all_ok)) all_ok = 0;   // collective: minimum over the ranks
    if (!all_ok) {
        s->rollback(s->ctx);                    // local: close mappings, free buffers
        return 0;
    }
    return 1;
}

namespace {
struct DirectSetup {
    CommState *st;
    NcclApi *api;
    size_t part;
    char *d_handles;
    char *err;
    size_t err_size;
};

int ds_prepare(void *ctx) {
    DirectSetup *d = (DirectSetup *)ctx;
    CommState *st = d->st;
    const int U = st->n_ranks, rank = st->local_rank[0];
    // the exchange buffer and the barrier words come first: both collectives need them even when the slab fails
    cudaError_t e = cudaMalloc((void **)&d->d_handles, (size_t)U * sizeof(cudaIpcMemHandle_t));
    if (e == cudaSuccess) e = cudaMemset(d->d_handles, 0, (size_t)U * sizeof(cudaIpcMemHandle_t));
    if (e == cudaSuccess) e = cudaMalloc((void **)&st->d_barrier, 4 * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(st->d_barrier, 0, 4 * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&st->slab, 4 * d->part + 256);   // + one row of arrival flags
    if (e == cudaSuccess) e = cudaMemset(st->slab, 0, 4 * d->part + 256);
    cudaIpcMemHandle_t mine;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&mine, st->slab);
    if (e == cudaSuccess) e = cudaMemcpy(d->d_handles + (size_t)rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return cuda_fail(e, "ulysses direct: buffers / IPC handle", d->err, d->err_size);
    return 1;
}

int ds_gather(void *ctx, int have_handle) {
    DirectSetup *d = (DirectSetup *)ctx;
    CommState *st = d->st;
    (void)have_handle;   // a rank without a handle contributes the zeros its buffer was cleared to
    if (!d->d_handles) {
        // not even the exchange buffer exists: fall back to a scratch word so that the collective is still entered
        if (cudaMalloc((void **)&d->d_handles, (size_t)st->n_ranks * sizeof(cudaIpcMemHandle_t)) != cudaSuccess)
            return fail(d->err, d->err_size, "ulysses direct: no memory for the handle exchange");
        cudaMemset(d->d_handles, 0, (size_t)st->n_ranks * sizeof(cudaIpcMemHandle_t));
    }
    const size_t hb = sizeof(cudaIpcMemHandle_t);
    ncclResult_t rc = d->api->AllGather(d->d_handles + (size_t)st->local_rank[0] * hb, d->d_handles, hb, ncclInt8, st->comm[0],
                                        st->stream[0]);
    if (rc != ncclSuccess)
        return fail(d->err, d->err_size, "ulysses direct: ncclAllGather failed: %s",
                    d->api->GetErrorString ? d->api->GetErrorString(rc) : "error");
    if (cudaStreamSynchronize(st->stream[0]) != cudaSuccess) return fail(d->err, d->err_size, "ulysses direct: handle exchange");
    return 1;
}

int ds_map_peers(void *ctx) {
    DirectSetup *d = (DirectSetup *)ctx;
    CommState *st = d->st;
    const int U = st->n_ranks, rank = st->local_rank[0];
    cudaIpcMemHandle_t all[MAX_U];
    cudaError_t e = cudaMemcpy(all, d->d_handles, (size_t)U * sizeof(all[0]), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "ulysses direct: handle exchange", d->err, d->err_size);
    const cudaIpcMemHandle_t zero = {};
    int mapped = 1;
    for (int pr = 0; pr < U; pr++) {
        if (pr == rank) {
            st->peer_slab[pr] = st->slab;
            continue;
        }
        if (!memcmp(&all[pr], &zero, sizeof(zero))) {   // that rank could not allocate: nothing to map
            fail(d->err, d->err_size, "ulysses direct: rank %d has no buffer to share", pr);
            mapped = 0;
            continue;
        }
        e = cudaIpcOpenMemHandle(&st->peer_slab[pr], all[pr], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            st->peer_slab[pr] = NULL;
            cuda_fail(e, "ulysses direct: cudaIpcOpenMemHandle (no peer access between the GPUs?)", d->err, d->err_size);
            mapped = 0;
        }
    }
    return mapped;
}

int ds_agree(void *ctx, int ok, int *all_ok) {
    DirectSetup *d = (DirectSetup *)ctx;
    CommState *st = d->st;
    *all_ok = 0;
    // the reduction needs two device words; if even the barrier words could not be allocated, borrow the
    // front of the handle buffer (the exchange is over)
    int *words = st->d_barrier ? st->d_barrier : (int *)d->d_handles;
    if (!words) return fail(d->err, d->err_size, "ulysses direct: no device word for the agreement");
    if (cudaMemcpy(words, &ok, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) return 0;
    ncclResult_t rc = d->api->AllReduce(words, words + 1, 1, ncclInt32, ncclMin, st->comm[0], st->stream[0]);
    if (rc != ncclSuccess || cudaStreamSynchronize(st->stream[0]) != cudaSuccess) return 0;
    if (cudaMemcpy(all_ok, words + 1, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
    if (st->d_barrier) cudaMemset(st->d_barrier, 0, 2 * sizeof(int));
    if (ok && !*all_ok) fail(d->err, d->err_size, "ulysses direct: another rank could not set up its buffers");
    return 1;
}

void ds_rollback(void *ctx) {
    DirectSetup *d = (DirectSetup *)ctx;
    CommState *st = d->st;
    for (int pr = 0; pr < st->n_ranks; pr++) {
        if (st->peer_slab[pr] && st->peer_slab[pr] != st->slab) cudaIpcCloseMemHandle(st->peer_slab[pr]);
        st->peer_slab[pr] = NULL;
    }
    // no peer has written here: all ranks roll back together (the agreement above) before anyone stores
    if (st->slab) cudaFree(st->slab);
    if (st->d_barrier) cudaFree(st->d_barrier);
    st->slab = NULL;
    st->d_barrier = NULL;
}
}  // namespace

int h3b_ulysses_direct_setup(h3_ulysses_cfg *cfg, size_t seq_local, size_t heads, size_t head_dim, char *err,
                             size_t err_size) {
    if (!cfg || !cfg->comm) return fail(err, err_size, "ulysses direct: not inited");
    CommState *st = (CommState *)cfg->comm;
    NcclApi *api = nccl_api(err, err_size);
    if (!api) return 0;
    // argument errors are the same on every rank (all call with the same sizes), so returning here is collective
    if (st->n_local != 1) return fail(err, err_size, "ulysses direct: needs one process per GPU");
    if (st->direct_ready) return fail(err, err_size, "ulysses direct: already set up");
    if (!seq_local || !heads || !head_dim || heads % (size_t)st->n_ranks || (head_dim * 2) % 16)
        return fail(err, err_size, "ulysses direct: bad geometry (seq_local %zu, heads %zu, head_dim %zu, U %d)", seq_local,
                    heads, head_dim, st->n_ranks);
    const int U = st->n_ranks, rank = st->local_rank[0];
    // a failing cudaSetDevice is local: it is folded into `prepare` failing, the collectives below still run
    const int device_ok = cudaSetDevice(st->device[0]) == cudaSuccess;
    // the four buffers have the same size: U*seq_local rows of heads/U heads = seq_local rows of all heads
    DirectSetup ds = {st, api, (seq_local * heads * head_dim * 2 + 255) & ~(size_t)255, NULL, err, err_size};
    h3b_ulysses_setup_steps steps = {&ds, ds_prepare, ds_gather, ds_map_peers, ds_agree, ds_rollback};
    if (!device_ok) steps.prepare = [](void *c) { return fail(((DirectSetup *)c)->err, ((DirectSetup *)c)->err_size, "ulysses direct: set device"); };
    const int ok = h3b_ulysses_setup_protocol(&steps);
    if (ds.d_handles) cudaFree(ds.d_handles);
    if (!ok) return 0;
    const size_t part = ds.part;
    h3b_ulysses_direct *d = &st->direct;
    d->ulysses = U; d->rank = rank; d->seq_local = seq_local; d->heads = heads; d->head_dim = head_dim;
    for (int pr = 0; pr < U; pr++) {
        char *b = (char *)st->peer_slab[pr];
        d->peer_q[pr] = b; d->peer_k[pr] = b + part; d->peer_v[pr] = b + 2 * part; d->peer_att[pr] = b + 3 * part;
    }
    d->q = d->peer_q[rank]; d->k = d->peer_k[rank]; d->v = d->peer_v[rank]; d->att = d->peer_att[rank];
    for (int pr = 0; pr < U; pr++) st->peer_flags[pr] = (uint32_t *)((char *)st->peer_slab[pr] + 4 * part);
    st->direct_ready = 1;
    // nobody stores into a peer (data or flags) before every rank has mapped and zeroed its slab: this first
    // barrier is the all-reduce; later ones are the flag kernel unless H3B_ULYSSES_BARRIER=nccl
    st->flag_barrier = 0;
    if (!(h3b_ulysses_barrier(cfg, err, err_size) && cudaStreamSynchronize(st->compute[0]) == cudaSuccess)) return 0;
    st->flag_barrier = strcmp(h3_plugin_value("H3B_ULYSSES_BARRIER"), "nccl") != 0;
    return 1;
}

const h3b_ulysses_direct *h3b_ulysses_direct_get(const h3_ulysses_cfg *cfg) {
    if (!cfg || !cfg->comm) return NULL;
    const CommState *st = (const CommState *)cfg->comm;
    return (st->direct_ready && !st->direct_off) ? &st->direct : NULL;
}

void h3b_ulysses_direct_enable(h3_ulysses_cfg *cfg, int on) {
    if (cfg && cfg->comm) ((CommState *)cfg->comm)->direct_off = !on;
}

int h3b_ulysses_barrier(h3_ulysses_cfg *cfg, char *err, size_t err_size) {
    if (!cfg || !cfg->comm) return fail(err, err_size, "ulysses barrier: not inited");
    CommState *st = (CommState *)cfg->comm;
    NcclApi *api = nccl_api(err, err_size);
    if (!api) return 0;
    if (st->n_local != 1 || !st->d_barrier) return fail(err, err_size, "ulysses barrier: direct mode is not set up");
    if (st->flag_barrier) {
        FlagBarrier fb;
        memset(&fb, 0, sizeof(fb));
        for (int pr = 0; pr < st->n_ranks; pr++) fb.peer_flags[pr] = st->peer_flags[pr];
        fb.state = st->d_barrier + 2;
        fb.rank = st->local_rank[0];
        fb.world = st->n_ranks;
        fb.budget = 4000000000ll;   // about two seconds of SM clocks, as the waits of the GEMM and attention kernels
        k_ulysses_flag_barrier<<<1, 32, 0, st->compute[0]>>>(fb);
        if (cudaGetLastError() != cudaSuccess) return fail(err, err_size, "ulysses barrier: launch failed");
        return 1;
    }
    ncclResult_t rc = api->AllReduce(st->d_barrier, st->d_barrier + 1, 1, ncclInt32, ncclSum, st->comm[0], st->compute[0]);
    if (rc != ncclSuccess)
        return fail(err, err_size, "ulysses barrier: ncclAllReduce failed: %s", api->GetErrorString ? api->GetErrorString(rc) : "error");
    return 1;
}

int h3b_ulysses_barrier_selftest(long long budget_cycles, int *status_arrived, int *status_absent, char *err,
                                 size_t err_size) {
    // Two ranks' flag rows in one local buffer, this GPU playing rank 0.  First the peer's word is preset to the
    // epoch the kernel will use (the barrier passes: status 0), then it is left at zero (the wait runs out
    // after `budget_cycles` and the kernel returns with status 6).  Nothing faults and the context stays usable.
    if (budget_cycles <= 0 || budget_cycles > 2000000000ll || !status_arrived || !status_absent)
        return fail(err, err_size, "barrier selftest: budget must be in (0, 2e9] cycles");
    uint32_t *flags = NULL;
    int *state = NULL;
    cudaError_t e = cudaMalloc((void **)&flags, 64 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc((void **)&state, 2 * sizeof(int));
    int ok = 0;
    for (int pass = 0; pass < 2 && e == cudaSuccess; pass++) {
        uint32_t host_flags[64] = {0};
        if (pass == 0) host_flags[1] = 1;   // row of rank 0, word of rank 1: already at epoch 1
        e = cudaMemcpy(flags, host_flags, sizeof(host_flags), cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemset(state, 0, 2 * sizeof(int));
        if (e != cudaSuccess) break;
        FlagBarrier fb;
        memset(&fb, 0, sizeof(fb));
        fb.peer_flags[0] = flags;        // rank 0's row
        fb.peer_flags[1] = flags + 32;   // rank 1's row (only written)
        fb.state = state; fb.rank = 0; fb.world = 2; fb.budget = budget_cycles;
        k_ulysses_flag_barrier<<<1, 32>>>(fb);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        int st2[2] = {0, 0};
        if (e == cudaSuccess) e = cudaMemcpy(st2, state, sizeof(st2), cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) {
            *(pass == 0 ? status_arrived : status_absent) = st2[1];
            ok = pass == 1;
        }
    }
    if (flags) cudaFree(flags);
    if (state) cudaFree(state);
    if (e != cudaSuccess) return cuda_fail(e, "barrier selftest", err, err_size);
    return ok;
}

int h3b_ulysses_check(h3_ulysses_cfg *cfg, int *status_out, char *err, size_t err_size) {
    if (!cfg || !cfg->comm) return fail(err, err_size, "ulysses check: not inited");
    CommState *st = (CommState *)cfg->comm;
    if (status_out) *status_out = 0;
    if (st->n_local != 1 || !st->d_barrier) return 1;
    int status = 0;
    if (cudaStreamSynchronize(st->compute[0]) != cudaSuccess ||
        cudaMemcpy(&status, st->d_barrier + 3, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return fail(err, err_size, "ulysses check: CUDA error");
    if (status_out) *status_out = status;
    if (status != 0) {
        cudaMemset(st->d_barrier + 3, 0, sizeof(int));
        return fail(err, err_size, "a barrier between the ranks gave up waiting (status %d); results after it are invalid", status);
    }
    return 1;
}

}  // extern "C"
