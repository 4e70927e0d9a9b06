// The exchange step of the output-feature-split layer for callers of the C ABI: every GPU holds
// y[:, its column slice] and all of them need y[M, N].  Two forms: plain peer stores (each GPU writes its slice
// into every GPU's full-width output, mapped into this process by CUDA IPC, symmetric memory or peer access), and
// an NCCL all-gather followed by the local reordering of the gathered slices.  NCCL is looked up at run time
// (dlopen), so the library neither links against it nor needs it unless these entry points are called.  The
// reference has no multi-GPU code; this is the collective of the one configuration that needs an exchange.
#include <dlfcn.h>

#include <cstring>

#include <mutex>

#include "common.cuh"

namespace bitnet {

struct PeerPtrs {
    float *p[BITNET_MAX_PEERS];
};

// src [M, n_local] (row stride ld_src) -> dst[r] [M, n_local] at row stride ldy, for every peer r
__global__ void __launch_bounds__(256) peer_store_kernel(const float *__restrict__ src, size_t M, size_t n_local, size_t ld_src,
                                                         const PeerPtrs dst, int n_peers, size_t ldy, int vec)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (vec) {
        const size_t per_row = n_local / 4, total = M * per_row;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const size_t m = i / per_row, c = (i - m * per_row) * 4;
            const float4 v = *reinterpret_cast<const float4 *>(src + m * ld_src + c);
            for (int r = 0; r < n_peers; ++r) *reinterpret_cast<float4 *>(dst.p[r] + m * ldy + c) = v;
        }
    } else {
        const size_t total = M * n_local;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const size_t m = i / n_local, c = i - m * n_local;
            const float v = src[m * ld_src + c];
            for (int r = 0; r < n_peers; ++r) dst.p[r][m * ldy + c] = v;
        }
    }
}

// staging [g][M][n_local] (what ncclAllGather leaves) -> y [M][g * n_local]
__global__ void __launch_bounds__(256) gather_reorder_kernel(const float *__restrict__ staging, float *__restrict__ y, size_t M, size_t n_local,
                                                             int g, size_t ldy)
{
    const size_t total = (size_t)g * M * n_local;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / (M * n_local), rem = i - r * M * n_local;
        const size_t m = rem / n_local, c = rem - m * n_local;
        y[m * ldy + r * n_local + c] = staging[i];
    }
}

// ---- NCCL through dlopen ---------------------------------------------------------------------------------
struct NcclUid {
    char internal[128];
};
typedef int (*nccl_get_uid_fn)(NcclUid *);
typedef int (*nccl_init_rank_fn)(void **, int, NcclUid, int);
typedef int (*nccl_destroy_fn)(void *);
typedef int (*nccl_allgather_fn)(const void *, void *, size_t, int, void *, cudaStream_t);
typedef const char *(*nccl_error_fn)(int);

struct NcclApi {
    void *handle = nullptr;
    nccl_get_uid_fn get_uid = nullptr;
    nccl_init_rank_fn init_rank = nullptr;
    nccl_destroy_fn destroy = nullptr;
    nccl_allgather_fn allgather = nullptr;
    nccl_error_fn error_string = nullptr;
};

static bitnet_status_t nccl_api(const NcclApi **out)
{
    static std::mutex mu;
    static NcclApi api;
    std::lock_guard<std::mutex> lock(mu);
    if (!api.handle) {
        // the copy the process already uses, if any (a host framework may have loaded its own), else the system's
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "NCCL is not available: %s", dlerror());
        NcclApi a;
        a.handle = h;
        a.get_uid = reinterpret_cast<nccl_get_uid_fn>(dlsym(h, "ncclGetUniqueId"));
        a.init_rank = reinterpret_cast<nccl_init_rank_fn>(dlsym(h, "ncclCommInitRank"));
        a.destroy = reinterpret_cast<nccl_destroy_fn>(dlsym(h, "ncclCommDestroy"));
        a.allgather = reinterpret_cast<nccl_allgather_fn>(dlsym(h, "ncclAllGather"));
        a.error_string = reinterpret_cast<nccl_error_fn>(dlsym(h, "ncclGetErrorString"));
        if (!a.get_uid || !a.init_rank || !a.destroy || !a.allgather)
            return fail(BITNET_ERR_UNSUPPORTED_OPERATION, "the NCCL library lacks an expected symbol");
        api = a;
    }
    *out = &api;
    return BITNET_OK;
}

static bitnet_status_t nccl_check(const NcclApi *api, int rc, const char *what)
{
    if (rc == 0) return BITNET_OK;
    return fail(BITNET_ERR_CUDA_DRIVER, "%s: NCCL error %d (%s)", what, rc, api->error_string ? api->error_string(rc) : "?");
}

}  // namespace bitnet

using namespace bitnet;

extern "C" bitnet_status_t bitnet_allgather_output(const float *y_local_dev, size_t M, size_t n_local, size_t ld_local,
                                                   float *const *y_peers_dev, int32_t n_peers, size_t ldy, bitnet_stream_t stream)
{
    if (M == 0 || n_local == 0) return BITNET_OK;
    if (!y_local_dev || !y_peers_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_allgather_output: null buffer");
    if (n_peers < 1 || n_peers > BITNET_MAX_PEERS) return fail(BITNET_ERR_INVALID_CONFIG, "n_peers must be in 1..%d (got %d)", BITNET_MAX_PEERS, n_peers);
    if (ld_local < n_local || ldy < n_local) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "row strides %zu / %zu below the slice width %zu", ld_local, ldy, n_local);
    PeerPtrs dst = {};
    uintptr_t align = reinterpret_cast<uintptr_t>(y_local_dev);
    for (int r = 0; r < n_peers; ++r) {
        if (!y_peers_dev[r]) return fail(BITNET_ERR_NULL_POINTER, "y_peers_dev[%d] is null", r);
        dst.p[r] = y_peers_dev[r];
        align |= reinterpret_cast<uintptr_t>(y_peers_dev[r]);
    }
    const int vec = (align & 15) == 0 && n_local % 4 == 0 && ld_local % 4 == 0 && ldy % 4 == 0;
    const size_t work = vec ? M * n_local / 4 : M * n_local;
    size_t blocks = (work + 255) / 256;
    const size_t cap = (size_t)device_sm_count() * 4;
    if (blocks > cap) blocks = cap;
    peer_store_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(y_local_dev, M, n_local, ld_local, dst, n_peers, ldy, vec);
    return check_launch("peer_store_kernel");
}

extern "C" bitnet_status_t bitnet_nccl_unique_id(uint8_t *id_out)
{
    if (!id_out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_nccl_unique_id: null output");
    const NcclApi *api = nullptr;
    BITNET_TRY(nccl_api(&api));
    NcclUid uid;
    BITNET_TRY(nccl_check(api, api->get_uid(&uid), "ncclGetUniqueId"));
    memcpy(id_out, uid.internal, sizeof(uid.internal));
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_nccl_comm_create(const uint8_t *id, int32_t n_ranks, int32_t rank, void **comm_out)
{
    if (!id || !comm_out) return fail(BITNET_ERR_NULL_POINTER, "bitnet_nccl_comm_create: null argument");
    *comm_out = nullptr;
    if (n_ranks < 1 || rank < 0 || rank >= n_ranks) return fail(BITNET_ERR_INVALID_CONFIG, "rank %d of %d", rank, n_ranks);
    const NcclApi *api = nullptr;
    BITNET_TRY(nccl_api(&api));
    NcclUid uid;
    memcpy(uid.internal, id, sizeof(uid.internal));
    void *comm = nullptr;
    BITNET_TRY(nccl_check(api, api->init_rank(&comm, n_ranks, uid, rank), "ncclCommInitRank"));
    *comm_out = comm;
    return BITNET_OK;
}

extern "C" bitnet_status_t bitnet_nccl_comm_destroy(void *comm)
{
    if (!comm) return BITNET_OK;
    const NcclApi *api = nullptr;
    BITNET_TRY(nccl_api(&api));
    return nccl_check(api, api->destroy(comm), "ncclCommDestroy");
}

extern "C" bitnet_status_t bitnet_allgather_output_nccl(void *comm, const float *y_local_dev, size_t M, size_t n_local,
                                                        float *staging_dev, float *y_full_dev, int32_t n_ranks, size_t ldy,
                                                        bitnet_stream_t stream)
{
    if (M == 0 || n_local == 0) return BITNET_OK;
    if (!comm || !y_local_dev || !staging_dev || !y_full_dev) return fail(BITNET_ERR_NULL_POINTER, "bitnet_allgather_output_nccl: null argument");
    if (n_ranks < 1) return fail(BITNET_ERR_INVALID_CONFIG, "n_ranks must be positive");
    if (ldy < (size_t)n_ranks * n_local) return fail(BITNET_ERR_INCOMPATIBLE_SHAPES, "ldy %zu below the gathered width %zu", ldy, (size_t)n_ranks * n_local);
    const NcclApi *api = nullptr;
    BITNET_TRY(nccl_api(&api));
    const int nccl_float32 = 7;
    BITNET_TRY(nccl_check(api, api->allgather(y_local_dev, staging_dev, M * n_local, nccl_float32, comm, as_stream(stream)), "ncclAllGather"));
    const size_t total = (size_t)n_ranks * M * n_local;
    size_t blocks = (total + 255) / 256;
    const size_t cap = (size_t)device_sm_count() * 8;
    if (blocks > cap) blocks = cap;
    gather_reorder_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(staging_dev, y_full_dev, M, n_local, n_ranks, ldy);
    return check_launch("gather_reorder_kernel");
}
