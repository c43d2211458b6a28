// NCCL all-gather of the output slices of a column-parallel job, behind the C ABI.
//
// The reference has one GPU and no collective.  Column-parallel ranks (one process
// per GPU, every projection split by output rows) need the whole [M, N] on every
// rank before the next projection reads it as its K: ncclAllGather over NVLink on
// the context's stream is the plain way to get it, the baseline the kernels that
// store their slices straight into the peers' outputs are measured against, and
// the cross-check of their results.
//
// NCCL is looked up at run time (dlopen of libnccl.so.2) the first time a
// communicator is asked for: a process that never shards never needs it, and the
// library keeps linking against libcudart only.
#include "../../include/q4b200.h"
#include "q4b_kernels.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

using namespace q4b;

struct q4b_comm {
    ncclComm_t comm;
    uint32_t world, rank;
    int device;
};

namespace {

struct NcclApi {
    void *handle;
    ncclResult_t (*get_unique_id)(ncclUniqueId *);
    ncclResult_t (*comm_init_rank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*all_gather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*comm_destroy)(ncclComm_t);
    const char *(*get_error_string)(ncclResult_t);
};

NcclApi g_nccl;
std::mutex g_nccl_guard;

void comm_message(char *message, size_t capacity, const char *format, ...) {
    if (message == nullptr || capacity == 0) return;
    va_list list;
    va_start(list, format);
    vsnprintf(message, capacity, format, list);
    va_end(list);
}

// 0 when the five entry points are resolved
int load_nccl(char *error_message, size_t error_capacity) {
    std::lock_guard<std::mutex> lock(g_nccl_guard);
    if (g_nccl.handle != nullptr) return Q4B_OK;
    void *handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (handle == nullptr) handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (handle == nullptr) {
        comm_message(error_message, error_capacity, "libnccl.so.2 cannot be loaded: %s", dlerror());
        return Q4B_LOAD_FAILURE;
    }
    NcclApi api = {};
    api.handle = handle;
    api.get_unique_id = reinterpret_cast<decltype(api.get_unique_id)>(dlsym(handle, "ncclGetUniqueId"));
    api.comm_init_rank = reinterpret_cast<decltype(api.comm_init_rank)>(dlsym(handle, "ncclCommInitRank"));
    api.all_gather = reinterpret_cast<decltype(api.all_gather)>(dlsym(handle, "ncclAllGather"));
    api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(dlsym(handle, "ncclCommDestroy"));
    api.get_error_string = reinterpret_cast<decltype(api.get_error_string)>(dlsym(handle, "ncclGetErrorString"));
    if (api.get_unique_id == nullptr || api.comm_init_rank == nullptr || api.all_gather == nullptr ||
        api.comm_destroy == nullptr || api.get_error_string == nullptr) {
        dlclose(handle);
        comm_message(error_message, error_capacity, "libnccl.so.2 lacks an entry point this library needs");
        return Q4B_LOAD_FAILURE;
    }
    g_nccl = api;
    return Q4B_OK;
}

int nccl_failure(char *error_message, size_t error_capacity, const char *what, ncclResult_t result) {
    comm_message(error_message, error_capacity, "%s: %s", what, g_nccl.get_error_string(result));
    return Q4B_DEVICE_FAILURE;
}

// full[m][rank * n_local + c] = staging[rank][m][c]: NCCL delivers rank-major blocks, the next projection reads
// whole activation rows
__global__ void interleave_slices_kernel(const uint4 *staging, uint4 *full, uint32_t world, uint32_t m_rows,
                                         uint32_t row_vectors) {
    const size_t total = (size_t)world * m_rows * row_vectors;
    for (size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x; at < total; at += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = (uint32_t)(at % row_vectors);
        const uint32_t m = (uint32_t)((at / row_vectors) % m_rows);
        const uint32_t rank = (uint32_t)(at / ((size_t)row_vectors * m_rows));
        full[((size_t)m * world + rank) * row_vectors + c] = staging[at];
    }
}

// peers[r][m][c] = local[m][c] for a block of `m_rows` rows of `row_vectors` 16-byte pieces, rows `ld_vectors`
// apart: consecutive threads take consecutive pieces of one destination (whole 512-byte requests per warp on the
// link), the destinations rotate with the thread block so that every link is busy from the start
struct PushParams {
    const uint4 *local;
    uint4 *peers[kMaxPeers];
    uint32_t peer_count, m_rows, row_vectors, ld_vectors;
};
__global__ void __launch_bounds__(256) push_rows_kernel(const PushParams p) {
    const size_t per_peer = (size_t)p.m_rows * p.row_vectors;
    const size_t chunks = (per_peer + 255) / 256;  // 256 pieces = one thread block's turn on one destination
    for (size_t turn = blockIdx.x; turn < chunks * p.peer_count; turn += gridDim.x) {
        const uint32_t peer = (uint32_t)(turn % p.peer_count);
        const size_t at = (turn / p.peer_count) * 256 + threadIdx.x;
        if (at >= per_peer) continue;
        const size_t m = at / p.row_vectors, c = at % p.row_vectors;
        p.peers[peer][m * p.ld_vectors + c] = __ldcg(p.local + m * p.ld_vectors + c);
    }
}

}  // namespace

extern "C" {

int q4b_comm_unique_id(void *id_128_bytes, char *error_message, size_t error_capacity) {
    static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
    if (id_128_bytes == nullptr) {
        comm_message(error_message, error_capacity, "no buffer for the id");
        return Q4B_BAD_ARGUMENT;
    }
    int code = load_nccl(error_message, error_capacity);
    if (code != Q4B_OK) return code;
    ncclUniqueId id;
    ncclResult_t result = g_nccl.get_unique_id(&id);
    if (result != ncclSuccess) return nccl_failure(error_message, error_capacity, "ncclGetUniqueId", result);
    memcpy(id_128_bytes, &id, sizeof(id));
    return Q4B_OK;
}

int q4b_comm_create(q4b_context *context, uint32_t world, uint32_t rank, const void *id_128_bytes, q4b_comm **comm,
                    char *error_message, size_t error_capacity) {
    if (context == nullptr || comm == nullptr || id_128_bytes == nullptr || world == 0 || rank >= world) {
        comm_message(error_message, error_capacity, "context, id or output missing, or rank outside the world");
        return Q4B_BAD_ARGUMENT;
    }
    *comm = nullptr;
    int code = load_nccl(error_message, error_capacity);
    if (code != Q4B_OK) return code;
    const int device = context_device(context);
    cudaError_t status = cudaSetDevice(device);
    if (status != cudaSuccess) {
        comm_message(error_message, error_capacity, "cudaSetDevice: %s", cudaGetErrorString(status));
        return Q4B_DEVICE_FAILURE;
    }
    ncclUniqueId id;
    memcpy(&id, id_128_bytes, sizeof(id));
    q4b_comm *result = new (std::nothrow) q4b_comm();
    if (result == nullptr) return Q4B_DEVICE_FAILURE;
    ncclResult_t outcome = g_nccl.comm_init_rank(&result->comm, (int)world, id, (int)rank);
    if (outcome != ncclSuccess) {
        delete result;
        return nccl_failure(error_message, error_capacity, "ncclCommInitRank", outcome);
    }
    result->world = world;
    result->rank = rank;
    result->device = device;
    *comm = result;
    return Q4B_OK;
}

int q4b_all_gather(q4b_context *context, q4b_comm *comm, const void *slice, void *gathered, size_t bytes_per_rank,
                   char *error_message, size_t error_capacity) {
    if (context == nullptr || comm == nullptr || slice == nullptr || gathered == nullptr || bytes_per_rank == 0 ||
        comm->device != context_device(context)) {
        comm_message(error_message, error_capacity, "context, communicator or buffers missing, or on another device");
        return Q4B_BAD_ARGUMENT;
    }
    cudaSetDevice(comm->device);
    ncclResult_t result = g_nccl.all_gather(slice, gathered, bytes_per_rank, ncclUint8, comm->comm,
                                            static_cast<cudaStream_t>(q4b_context_stream(context)));
    if (result != ncclSuccess) return nccl_failure(error_message, error_capacity, "ncclAllGather", result);
    return Q4B_OK;
}

int q4b_all_gather_columns(q4b_context *context, q4b_comm *comm, const void *slice, void *full, uint32_t m_rows,
                           uint32_t slice_columns, uint32_t element_bytes, void *staging, char *error_message,
                           size_t error_capacity) {
    if (comm == nullptr || m_rows == 0 || slice_columns == 0 || (element_bytes != 2 && element_bytes != 4)) {
        comm_message(error_message, error_capacity, "communicator missing or shape invalid");
        return Q4B_BAD_ARGUMENT;
    }
    const size_t row_bytes = (size_t)slice_columns * element_bytes;
    if (m_rows == 1) {  // one activation row: rank-major IS the row
        return q4b_all_gather(context, comm, slice, full, row_bytes, error_message, error_capacity);
    }
    if (staging == nullptr || row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(full) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(staging) & 15u) != 0) {
        comm_message(error_message, error_capacity,
                     "M > 1 needs a staging buffer of world x M x slice bytes; slices of whole 16-byte pieces, "
                     "16-byte aligned buffers");
        return Q4B_BAD_ARGUMENT;
    }
    int code = q4b_all_gather(context, comm, slice, staging, row_bytes * m_rows, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    const uint32_t row_vectors = (uint32_t)(row_bytes / 16);
    const size_t total = (size_t)comm->world * m_rows * row_vectors;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184);
    interleave_slices_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(q4b_context_stream(context))>>>(
        static_cast<const uint4 *>(staging), static_cast<uint4 *>(full), comm->world, m_rows, row_vectors);
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) {
        comm_message(error_message, error_capacity, "slice interleave: %s", cudaGetErrorString(status));
        return Q4B_DEVICE_FAILURE;
    }
    context_count_launch(context);
    return Q4B_OK;
}

int q4b_push_rows(q4b_context *context, const void *local, void *const *peers, uint32_t peer_count, uint32_t m_rows,
                  uint32_t row_bytes, uint32_t ld_bytes, char *error_message, size_t error_capacity) {
    if (context == nullptr || local == nullptr || peers == nullptr || peer_count == 0 || peer_count > (uint32_t)kMaxPeers ||
        m_rows == 0 || row_bytes == 0 || row_bytes % 16 != 0 || ld_bytes % 16 != 0 || ld_bytes < row_bytes ||
        (reinterpret_cast<uintptr_t>(local) & 15u) != 0) {
        comm_message(error_message, error_capacity,
                     "1..%d peers; rows and row pitch in whole 16-byte pieces, 16-byte aligned blocks", kMaxPeers);
        return Q4B_BAD_ARGUMENT;
    }
    PushParams p = {};
    p.local = static_cast<const uint4 *>(local);
    for (uint32_t r = 0; r < peer_count; ++r) {
        if (peers[r] == nullptr || (reinterpret_cast<uintptr_t>(peers[r]) & 15u) != 0) {
            comm_message(error_message, error_capacity, "peer %u: no block, or not 16-byte aligned", r);
            return Q4B_BAD_ARGUMENT;
        }
        p.peers[r] = static_cast<uint4 *>(peers[r]);
    }
    p.peer_count = peer_count;
    p.m_rows = m_rows;
    p.row_vectors = row_bytes / 16;
    p.ld_vectors = ld_bytes / 16;
    const size_t turns = (((size_t)m_rows * p.row_vectors + 255) / 256) * peer_count;
    const unsigned blocks = (unsigned)(turns < 1184 ? turns : 1184);
    cudaSetDevice(context_device(context));
    push_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(q4b_context_stream(context))>>>(p);
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) {
        comm_message(error_message, error_capacity, "row push: %s", cudaGetErrorString(status));
        return Q4B_DEVICE_FAILURE;
    }
    context_count_launch(context);
    return Q4B_OK;
}

uint32_t q4b_comm_world(const q4b_comm *comm) { return comm != nullptr ? comm->world : 0; }
uint32_t q4b_comm_rank(const q4b_comm *comm) { return comm != nullptr ? comm->rank : 0; }

void q4b_comm_free(q4b_context *context, q4b_comm *comm) {
    if (comm == nullptr) return;
    if (context != nullptr) q4b_sync(context, nullptr, nullptr, 0);
    if (g_nccl.handle != nullptr) g_nccl.comm_destroy(comm->comm);
    delete comm;
}

}  // extern "C"
