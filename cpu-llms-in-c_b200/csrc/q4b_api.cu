// C ABI of libq4b200 (declared in include/q4b200.h): contexts, the weight-image
// loader, matmul dispatch, completion/timing and graph replay.  Host code only;
// the kernels live in q4b_pack.cu, q4b_decode.cu and q4b_gemm.cu.
#include "../../include/q4b200.h"
#include "q4b_kernels.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

using namespace q4b;

struct q4b_context {
    int device;
    int sm_count;
    int variant;
    cudaStream_t stream;
    cudaEvent_t timer_start, timer_stop;
    bool timer_armed;
    bool capturing;
    uint64_t launches;
    uint32_t *status_host;    // pinned, device-mapped: kernels store a code here when a wait expires
    uint32_t *status_device;  // the same word as the kernels see it
    float *scratch;           // partial-sum slots of split row blocks (grown on demand)
    size_t scratch_bytes;
    uint32_t *counters;       // arrival counters, zero between launches
    size_t counter_bytes;
    __half *x16;              // fp16 copy of fp32 activations for the tensor-core GEMM (grown on demand)
    size_t x16_bytes;
    void *push_y[kMaxSegments][kMaxPeers];  // q4b_context_push_outputs: consumed by the next tensor-core launch
    uint32_t push_peers;
    float *tc_workspace;      // partial tiles of the tensor-core GEMM when it splits tiles over CTAs
    size_t tc_workspace_bytes;
    uint32_t *tc_flags;
};

struct q4b_weight {
    WeightView view;
    uint64_t device_bytes;
    uint32_t rows_total;  // rows of the source matrix
    uint32_t row_begin;   // first source row held
    int device;
    bool borrowed;        // a row range of another weight: the tile stream is not this handle's to free
};

struct q4b_sequence {
    std::vector<DecodeJob> jobs;
    uint32_t m_rows, world, rank;
    int device;
    bool finalized;
    DecodeJob *device_jobs;
    uint32_t *done;        // [jobs][8] completion counters (kDoneStride words apart) + the epoch and exit words
    size_t done_words;
    uint32_t *peer_done[kMaxPeers];
    float *scratch;
    uint32_t *counters;
    unsigned long long *profile;  // optional phase clocks, [ctas][kProfileSlots]
    SequenceLaunch launch;
};

struct q4b_graph {
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    uint64_t launches;  // kernels recorded
};

namespace {

void set_error(char *message, size_t capacity, const char *format, ...) {
    if (message == nullptr || capacity == 0) return;
    va_list list;
    va_start(list, format);
    vsnprintf(message, capacity, format, list);
    va_end(list);
}

int device_failure(char *message, size_t capacity, const char *what, cudaError_t status) {
    set_error(message, capacity, "%s: %s", what, cudaGetErrorString(status));
    return Q4B_DEVICE_FAILURE;
}

#define Q4B_CUDA(call, what)                                                     \
    do {                                                                         \
        cudaError_t status_ = (call);                                            \
        if (status_ != cudaSuccess)                                              \
            return device_failure(error_message, error_capacity, what, status_); \
    } while (0)

bool valid_activation_dtype(int dtype) { return dtype == Q4B_F16 || dtype == Q4B_F32; }
// bf16 activations (the H3 projections) multiply weights rounded to bf16; outputs and residuals are then bf16 or
// fp32.  fp16 and fp32 activations keep fp16 or fp32 around them.
bool valid_dtype_pair(int x_dtype, int other_dtype) {
    if (x_dtype == Q4B_BF16) return other_dtype == Q4B_BF16 || other_dtype == Q4B_F32;
    return valid_activation_dtype(x_dtype) && valid_activation_dtype(other_dtype);
}
size_t dtype_bytes(int dtype) { return dtype == Q4B_F32 ? 4 : 2; }
bool aligned16(const void *pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0; }

int check_context(q4b_context *context, char *error_message, size_t error_capacity) {
    if (context == nullptr) {
        set_error(error_message, error_capacity, "context is NULL");
        return Q4B_BAD_ARGUMENT;
    }
    cudaError_t status = cudaSetDevice(context->device);
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "cudaSetDevice", status);
    return Q4B_OK;
}

uint64_t tile_stream_bytes(uint32_t row_count, uint32_t groups) {
    uint32_t row_tiles = ceil_div(row_count, kTileRows);
    uint32_t padded = ceil_div(row_tiles, kRowTilePad) * kRowTilePad;
    return (uint64_t)padded * groups * kTileBytes;
}

int validate_shape(uint32_t rows, uint32_t groups, uint32_t row_begin, uint32_t row_count,
                   char *error_message, size_t error_capacity) {
    if (rows == 0 || groups == 0 || row_count == 0 || row_begin >= rows ||
        row_count > rows - row_begin) {
        set_error(error_message, error_capacity,
                  "invalid weight shape: rows=%u groups_per_row=%u slice=[%u,+%u)", rows, groups,
                  row_begin, row_count);
        return Q4B_BAD_ARGUMENT;
    }
    if ((uint64_t)groups * kGroup > 0x7fffffffull) {
        set_error(error_message, error_capacity, "K = %llu is too large",
                  (unsigned long long)groups * kGroup);
        return Q4B_BAD_ARGUMENT;
    }
    return Q4B_OK;
}

// device planes -> tile stream in a fresh allocation
int build_weight(q4b_context *context, const uint8_t *device_quants, const void *device_meta,
                 const void *device_biases, int meta_dtype, uint32_t rows, uint32_t groups,
                 uint32_t row_begin, uint32_t row_count, q4b_weight **out, char *error_message,
                 size_t error_capacity) {
    uint64_t bytes = tile_stream_bytes(row_count, groups);
    uint8_t *tiles = nullptr;
    cudaError_t status = cudaMalloc(&tiles, bytes);
    if (status != cudaSuccess) {
        set_error(error_message, error_capacity, "cudaMalloc of %llu bytes for the weight image: %s",
                  (unsigned long long)bytes, cudaGetErrorString(status));
        return Q4B_LOAD_FAILURE;
    }
    status = launch_repack(device_quants, device_meta, device_biases, meta_dtype, groups, row_begin,
                           row_count, tiles, context->stream);
    ++context->launches;
    if (status == cudaSuccess) status = cudaStreamSynchronize(context->stream);
    if (status != cudaSuccess) {
        cudaFree(tiles);
        return device_failure(error_message, error_capacity, "repack", status);
    }
    q4b_weight *weight = new (std::nothrow) q4b_weight();
    if (weight == nullptr) {
        cudaFree(tiles);
        set_error(error_message, error_capacity, "out of host memory");
        return Q4B_LOAD_FAILURE;
    }
    weight->view.tiles = tiles;
    weight->view.rows = row_count;
    weight->view.groups = groups;
    weight->view.row_tiles = ceil_div(row_count, kTileRows);
    weight->device_bytes = bytes;
    weight->rows_total = rows;
    weight->row_begin = row_begin;
    weight->device = context->device;
    *out = weight;
    return Q4B_OK;
}

int upload_common(q4b_context *context, const void *quants, const void *meta, const void *biases,
                  int meta_dtype, uint32_t rows, uint32_t groups, uint32_t row_begin,
                  uint32_t row_count, q4b_weight **out, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (out == nullptr || quants == nullptr || meta == nullptr) {
        set_error(error_message, error_capacity, "NULL segment or output pointer");
        return Q4B_BAD_ARGUMENT;
    }
    *out = nullptr;
    code = validate_shape(rows, groups, row_begin, row_count, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (context->capturing) {
        set_error(error_message, error_capacity, "weights cannot be loaded while recording a graph");
        return Q4B_BAD_ARGUMENT;
    }
    // only the slice's bytes cross PCIe
    const size_t quant_bytes = (size_t)row_count * groups * 32;
    const size_t record_bytes = biases == nullptr ? 4 : 2;
    const size_t meta_bytes = (size_t)row_count * groups * record_bytes;
    const uint8_t *host_quants = static_cast<const uint8_t *>(quants) + (size_t)row_begin * groups * 32;
    const uint8_t *host_meta = static_cast<const uint8_t *>(meta) + (size_t)row_begin * groups * record_bytes;
    uint8_t *staging = nullptr;
    cudaError_t status = cudaMalloc(&staging, quant_bytes + 2 * meta_bytes + 64);
    if (status != cudaSuccess) {
        set_error(error_message, error_capacity, "cudaMalloc of upload staging: %s", cudaGetErrorString(status));
        return Q4B_LOAD_FAILURE;
    }
    uint8_t *device_quants = staging;
    uint8_t *device_meta = staging + ((quant_bytes + 15) & ~(size_t)15);
    uint8_t *device_biases = biases == nullptr ? nullptr : device_meta + ((meta_bytes + 15) & ~(size_t)15);
    status = cudaMemcpyAsync(device_quants, host_quants, quant_bytes, cudaMemcpyHostToDevice, context->stream);
    if (status == cudaSuccess)
        status = cudaMemcpyAsync(device_meta, host_meta, meta_bytes, cudaMemcpyHostToDevice, context->stream);
    if (status == cudaSuccess && biases != nullptr) {
        const uint8_t *host_biases = static_cast<const uint8_t *>(biases) + (size_t)row_begin * groups * 2;
        status = cudaMemcpyAsync(device_biases, host_biases, meta_bytes, cudaMemcpyHostToDevice, context->stream);
    }
    if (status != cudaSuccess) {
        cudaFree(staging);
        return device_failure(error_message, error_capacity, "upload copy", status);
    }
    code = build_weight(context, device_quants, device_meta, device_biases, meta_dtype, rows, groups,
                        0, row_count, out, error_message, error_capacity);
    cudaFree(staging);
    if (code == Q4B_OK) {
        (*out)->row_begin = row_begin;
    }
    return code;
}

int check_matmul_arguments(q4b_context *context, const q4b_weight *weight, const void *x, int x_dtype,
                           uint32_t m_rows, const void *y, int y_dtype, uint32_t ldy,
                           char *error_message, size_t error_capacity) {
    if (weight == nullptr || x == nullptr || y == nullptr) {
        set_error(error_message, error_capacity, "NULL weight, x or y");
        return Q4B_BAD_ARGUMENT;
    }
    if (weight->device != context->device) {
        set_error(error_message, error_capacity, "weight lives on device %d, context on %d",
                  weight->device, context->device);
        return Q4B_BAD_ARGUMENT;
    }
    if (m_rows == 0) {
        set_error(error_message, error_capacity, "batch_rows is 0");
        return Q4B_BAD_ARGUMENT;
    }
    if (!valid_dtype_pair(x_dtype, y_dtype)) {
        set_error(error_message, error_capacity,
                  "x and y must be fp16 or fp32, or x bf16 with y bf16 or fp32");
        return Q4B_BAD_ARGUMENT;
    }
    if (ldy < weight->view.rows) {
        set_error(error_message, error_capacity, "ldy=%u is smaller than the %u rows of the shard", ldy,
                  weight->view.rows);
        return Q4B_BAD_ARGUMENT;
    }
    if (!aligned16(x)) {
        set_error(error_message, error_capacity, "x must be 16-byte aligned");
        return Q4B_BAD_ARGUMENT;
    }
    return Q4B_OK;
}

// Grow the context's split-K scratch to what a launch needs.  Never during
// recording: an allocation cannot be captured, so the sequence must have run
// once (or q4b_reserve_scratch been called) before q4b_graph_begin.
struct ScratchNeed {
    size_t scratch_bytes, counter_bytes;
};
int ensure_scratch(q4b_context *context, const ScratchNeed &plan, char *error_message, size_t error_capacity) {
    if (plan.scratch_bytes <= context->scratch_bytes && plan.counter_bytes <= context->counter_bytes) return Q4B_OK;
    if (context->capturing) {
        set_error(error_message, error_capacity,
                  "the recorded sequence needs more scratch than the context holds; run it once before recording");
        return Q4B_BAD_ARGUMENT;
    }
    cudaError_t status = cudaStreamSynchronize(context->stream);
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "stream synchronize", status);
    if (plan.scratch_bytes > context->scratch_bytes) {
        cudaFree(context->scratch);
        context->scratch = nullptr;
        context->scratch_bytes = 0;
        const size_t bytes = plan.scratch_bytes + plan.scratch_bytes / 2;
        status = cudaMalloc(&context->scratch, bytes);
        if (status != cudaSuccess) return device_failure(error_message, error_capacity, "cudaMalloc of scratch", status);
        context->scratch_bytes = bytes;
    }
    if (plan.counter_bytes > context->counter_bytes) {
        cudaFree(context->counters);
        context->counters = nullptr;
        context->counter_bytes = 0;
        const size_t bytes = plan.counter_bytes * 2 + 1024;
        status = cudaMalloc(&context->counters, bytes);
        if (status == cudaSuccess) status = cudaMemset(context->counters, 0, bytes);
        if (status != cudaSuccess) return device_failure(error_message, error_capacity, "cudaMalloc of counters", status);
        context->counter_bytes = bytes;
    }
    return Q4B_OK;
}

// M above the small-M kernel's limit: the tcgen05 GEMM, one launch per matrix
int run_tensor_core(q4b_context *context, const ProjectionArgs &args, char *error_message, size_t error_capacity) {
    const size_t K = (size_t)args.w[0].groups * kGroup;
    const void *x = args.x;
    if (args.x_dtype == kF32) {
        const size_t bytes = (size_t)args.m_rows * K * sizeof(__half);
        if (bytes > context->x16_bytes) {
            if (context->capturing) {
                set_error(error_message, error_capacity,
                          "the recorded sequence needs a larger fp16 staging buffer; run it once before recording");
                return Q4B_BAD_ARGUMENT;
            }
            cudaError_t status = cudaStreamSynchronize(context->stream);
            if (status == cudaSuccess) {
                cudaFree(context->x16);
                context->x16 = nullptr;
                context->x16_bytes = 0;
                status = cudaMalloc(&context->x16, bytes);
            }
            if (status != cudaSuccess) return device_failure(error_message, error_capacity, "fp16 staging buffer", status);
            context->x16_bytes = bytes;
        }
        cudaError_t status = launch_convert_f32_to_f16(static_cast<const float *>(args.x), context->x16,
                                                       (size_t)args.m_rows * K, context->stream);
        if (!context->capturing) ++context->launches;
        if (status != cudaSuccess) return device_failure(error_message, error_capacity, "activation convert", status);
        x = context->x16;
    }
    if (context->tc_workspace == nullptr && !context->capturing) {
        // once per context: sm_count partial tiles of 128 x 256 floats and their flags
        const size_t bytes = (size_t)context->sm_count * 128 * 256 * sizeof(float);
        cudaError_t status = cudaMalloc(&context->tc_workspace, bytes);
        if (status == cudaSuccess) status = cudaMalloc(&context->tc_flags, (size_t)context->sm_count * sizeof(uint32_t));
        if (status == cudaSuccess) status = cudaMemset(context->tc_flags, 0, (size_t)context->sm_count * sizeof(uint32_t));
        if (status != cudaSuccess) return device_failure(error_message, error_capacity, "gemm workspace", status);
        context->tc_workspace_bytes = bytes;
    }
    TcGemmArgs gemm = {};
    gemm.peers = context->push_peers;
    for (int s = 0; s < kMaxSegments; ++s) {
        for (int r = 0; r < kMaxPeers; ++r) gemm.peer_y[s][r] = context->push_y[s][r];
    }
    context->push_peers = 0;
    gemm.workspace = context->tc_workspace;
    gemm.workspace_bytes = context->tc_workspace_bytes;
    gemm.flags = context->tc_flags;
    for (int s = 0; s < args.segments; ++s) {
        gemm.w[s] = args.w[s];
        gemm.y[s] = args.y[s];
        gemm.ldy[s] = args.ldy[s];
    }
    gemm.segments = args.segments;
    gemm.up = args.up;
    gemm.fused_silu = args.fused_silu;
    gemm.x = x;
    gemm.x_bf16 = args.x_dtype == kBF16;
    gemm.m_rows = args.m_rows;
    gemm.y_dtype = args.y_dtype;
    gemm.residual = args.residual;
    gemm.residual_dtype = args.residual_dtype;
    gemm.ld_residual = args.ld_residual;
    gemm.status = context->status_device;
    cudaError_t status = launch_tc_gemm(gemm, context->sm_count, context->stream);
    if (!context->capturing) ++context->launches;
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "tensor-core gemm launch", status);
    return Q4B_OK;
}

// One projection at any M: the decode kernel up to its row limit, the tensor-core GEMM above.
// With built_in_scratch the split-K scratch is the library's file-scope device
// array and nothing is allocated, grown or freed.
int run_projection(q4b_context *context, ProjectionArgs args, char *error_message, size_t error_capacity,
                   bool built_in_scratch = false) {
    const uint32_t limit = decode_max_m();
    const uint32_t total = args.m_rows;
    const size_t K = (size_t)args.w[0].groups * kGroup;
    // variant bit 15 keeps large M on the small-M kernel (row blocks of 16), for A/B runs
    if (total > limit && !built_in_scratch && ((context->variant >> 15) & 1) == 0 && args.w[0].kind == kQ4) {
        return run_tensor_core(context, args, error_message, error_capacity);
    }
    if (args.w[0].kind == kQ8) {
        // the affine-Q8 sibling exists as a GEMM only (as in the reference): the tensor-core kernel at every M
        if (built_in_scratch || args.fused_silu || args.segments != 1 || args.x_dtype == kBF16) {
            set_error(error_message, error_capacity,
                      "affine-Q8 weights: one matrix per call through q4b_matmul, fp16 or fp32 activations");
            return Q4B_BAD_ARGUMENT;
        }
        return run_tensor_core(context, args, error_message, error_capacity);
    }
    for (int s = 0; s < args.segments; ++s) {
        if (args.w[s].kind != kQ4 || (args.fused_silu && args.up.kind != kQ4)) {
            set_error(error_message, error_capacity, "affine-Q8 weights cannot share a call with Q4 weights");
            return Q4B_BAD_ARGUMENT;
        }
    }
    if (args.x_dtype == kBF16) {
        // the small-M kernel multiplies fp16 or integer digits; bf16 activations go to the tensor-core kernel at every M
        if (built_in_scratch) {
            set_error(error_message, error_capacity, "bf16 activations need q4b_matmul");
            return Q4B_BAD_ARGUMENT;
        }
        return run_tensor_core(context, args, error_message, error_capacity);
    }
    // q4b_context_push_outputs: this call's outputs also go into the peers' copies (consumed by this call)
    const uint32_t push_peers = built_in_scratch ? 0u : context->push_peers;
    context->push_peers = 0;
    for (uint32_t m0 = 0; m0 < total; m0 += limit) {
        const uint32_t m_rows = total - m0 < limit ? total - m0 : limit;
        DecodeJob job = {};
        for (int s = 0; s < args.segments; ++s) {
            job.tiles[s] = args.w[s].tiles;
            job.rows[s] = args.w[s].rows;
            job.ldy[s] = args.ldy[s];
            job.y[s][0] = static_cast<uint8_t *>(args.y[s]) + (size_t)m0 * args.ldy[s] * dtype_bytes(args.y_dtype);
        }
        uint32_t world = 1;
        for (uint32_t r = 0; r < push_peers; ++r) {  // the peers that were named, packed after the own copy
            bool named = false;
            for (int s = 0; s < args.segments; ++s) named = named || context->push_y[s][r] != nullptr;
            if (!named) continue;
            for (int s = 0; s < args.segments; ++s) {
                uint8_t *peer = static_cast<uint8_t *>(context->push_y[s][r]);
                job.y[s][world] = peer == nullptr ? nullptr
                                                  : peer + (size_t)m0 * args.ldy[s] * dtype_bytes(args.y_dtype);
            }
            if (++world == (uint32_t)kMaxPeers) break;
        }
        job.segments = (uint32_t)args.segments;
        job.groups = args.w[0].groups;
        if (args.fused_silu) {
            job.fused = 1;
            job.up_tiles = args.up.tiles;
        }
        job.x = static_cast<const uint8_t *>(args.x) + (size_t)m0 * K * dtype_bytes(args.x_dtype);
        job.x_dtype = args.x_dtype;
        job.y_dtype = args.y_dtype;
        job.residual_dtype = args.residual_dtype;
        job.ld_residual = args.ld_residual;
        if (args.residual != nullptr) {
            job.residual = static_cast<const uint8_t *>(args.residual) +
                           (size_t)m0 * args.ld_residual * dtype_bytes(args.residual_dtype);
        }
        DecodeGeometry geometry;
        cudaError_t status = decode_geometry(m_rows, context->variant, context->sm_count, false, &geometry);
        if (status != cudaSuccess) return device_failure(error_message, error_capacity, "decode geometry", status);
        ScratchNeed need = {};
        plan_decode_job(&job, m_rows, geometry, &need.scratch_bytes, &need.counter_bytes);
        float *scratch = nullptr;
        uint32_t *counters = nullptr;
        if (built_in_scratch) {
            size_t scratch_bytes = 0, counter_bytes = 0;
            status = decode_static_scratch(&scratch, &counters, &scratch_bytes, &counter_bytes);
            if (status != cudaSuccess) return device_failure(error_message, error_capacity, "built-in scratch", status);
            if (need.scratch_bytes > scratch_bytes || need.counter_bytes > counter_bytes) {
                set_error(error_message, error_capacity,
                          "this shape needs %zu bytes of scratch and %zu of counters; the built-in scratch holds "
                          "%zu and %zu -- use q4b_matmul, which allocates",
                          need.scratch_bytes, need.counter_bytes, scratch_bytes, counter_bytes);
                return Q4B_BAD_ARGUMENT;
            }
            // the array keeps whatever the previous call left: the counters must start at zero
            if (need.counter_bytes > 0) {
                status = cudaMemsetAsync(counters, 0, need.counter_bytes, context->stream);
                if (status != cudaSuccess) return device_failure(error_message, error_capacity, "counter reset", status);
            }
        } else {
            int code = ensure_scratch(context, need, error_message, error_capacity);
            if (code != Q4B_OK) return code;
            scratch = context->scratch;
            counters = context->counters;
        }
        status = launch_decode(job, m_rows, world, geometry, context->variant, scratch, counters,
                               context->status_device, context->stream);
        if (!context->capturing) ++context->launches;  // recorded launches count at replay
        if (status != cudaSuccess) return device_failure(error_message, error_capacity, "decode launch", status);
    }
    return Q4B_OK;
}

}  // namespace

namespace q4b {
int context_device(const q4b_context *context) { return context->device; }
void context_count_launch(q4b_context *context) {
    if (!context->capturing) ++context->launches;
}
}  // namespace q4b

extern "C" {

int q4b_device_count(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) return 0;
    return count;
}

q4b_context *q4b_context_open(int device, char *error_message, size_t error_capacity) {
    int count = 0;
    cudaError_t status = cudaGetDeviceCount(&count);
    if (status != cudaSuccess || count == 0) {
        set_error(error_message, error_capacity, "no CUDA device: %s (this library has no CPU path)",
                  status != cudaSuccess ? cudaGetErrorString(status) : "device count is 0");
        return nullptr;
    }
    if (device < 0 || device >= count) {
        set_error(error_message, error_capacity, "device %d out of range (0..%d)", device, count - 1);
        return nullptr;
    }
    cudaDeviceProp properties;
    status = cudaGetDeviceProperties(&properties, device);
    if (status != cudaSuccess) {
        set_error(error_message, error_capacity, "cudaGetDeviceProperties: %s", cudaGetErrorString(status));
        return nullptr;
    }
    if (properties.major != 10) {
        set_error(error_message, error_capacity,
                  "device %d is sm_%d%d; this library is built for sm_100a only", device,
                  properties.major, properties.minor);
        return nullptr;
    }
    q4b_context *context = new (std::nothrow) q4b_context();
    if (context == nullptr) {
        set_error(error_message, error_capacity, "out of host memory");
        return nullptr;
    }
    context->device = device;
    context->sm_count = properties.multiProcessorCount;
    const char *variant = getenv("Q4B_VARIANT");
    context->variant = variant != nullptr ? (int)strtol(variant, nullptr, 0) : 0;
    if ((status = cudaSetDevice(device)) != cudaSuccess ||
        (status = cudaStreamCreateWithFlags(&context->stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (status = cudaEventCreate(&context->timer_start)) != cudaSuccess ||
        (status = cudaEventCreate(&context->timer_stop)) != cudaSuccess ||
        (status = cudaHostAlloc(reinterpret_cast<void **>(&context->status_host), sizeof(uint32_t),
                                cudaHostAllocMapped)) != cudaSuccess ||
        (status = cudaHostGetDevicePointer(reinterpret_cast<void **>(&context->status_device),
                                           context->status_host, 0)) != cudaSuccess) {
        set_error(error_message, error_capacity, "context setup: %s", cudaGetErrorString(status));
        delete context;
        return nullptr;
    }
    *context->status_host = 0;
    return context;
}

void q4b_context_close(q4b_context *context) {
    if (context == nullptr) return;
    cudaSetDevice(context->device);
    cudaStreamSynchronize(context->stream);
    cudaEventDestroy(context->timer_start);
    cudaEventDestroy(context->timer_stop);
    cudaStreamDestroy(context->stream);
    cudaFreeHost(context->status_host);
    cudaFree(context->scratch);
    cudaFree(context->counters);
    cudaFree(context->tc_workspace);
    cudaFree(context->tc_flags);
    cudaFree(context->x16);
    delete context;
}

void *q4b_context_stream(q4b_context *context) { return context != nullptr ? context->stream : nullptr; }
void q4b_context_set_variant(q4b_context *context, int variant) {
    if (context != nullptr) context->variant = variant;
}
uint64_t q4b_context_launch_count(const q4b_context *context) {
    return context != nullptr ? context->launches : 0;
}

int q4b_alloc(q4b_context *context, size_t bytes, void **device_pointer, char *error_message,
              size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (device_pointer == nullptr) return Q4B_BAD_ARGUMENT;
    Q4B_CUDA(cudaMalloc(device_pointer, bytes > 0 ? bytes : 1), "cudaMalloc");
    return Q4B_OK;
}
int q4b_free(q4b_context *context, void *device_pointer) {
    if (context != nullptr) cudaSetDevice(context->device);
    return cudaFree(device_pointer) == cudaSuccess ? Q4B_OK : Q4B_DEVICE_FAILURE;
}
int q4b_alloc_host(q4b_context *context, size_t bytes, void **pinned_host_pointer, char *error_message,
                   size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (pinned_host_pointer == nullptr) return Q4B_BAD_ARGUMENT;
    Q4B_CUDA(cudaMallocHost(pinned_host_pointer, bytes > 0 ? bytes : 1), "cudaMallocHost");
    return Q4B_OK;
}
int q4b_free_host(q4b_context *context, void *pinned_host_pointer) {
    if (context != nullptr) cudaSetDevice(context->device);
    return cudaFreeHost(pinned_host_pointer) == cudaSuccess ? Q4B_OK : Q4B_DEVICE_FAILURE;
}
int q4b_copy_to_device(q4b_context *context, void *device_destination, const void *host_source,
                       size_t bytes, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    Q4B_CUDA(cudaMemcpyAsync(device_destination, host_source, bytes, cudaMemcpyHostToDevice, context->stream),
             "copy to device");
    return Q4B_OK;
}
int q4b_copy_to_host(q4b_context *context, void *host_destination, const void *device_source, size_t bytes,
                     char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    Q4B_CUDA(cudaMemcpyAsync(host_destination, device_source, bytes, cudaMemcpyDeviceToHost, context->stream),
             "copy to host");
    return Q4B_OK;
}

int q4b_copy_2d(q4b_context *context, void *destination, size_t destination_pitch, const void *source,
                size_t source_pitch, size_t row_bytes, size_t rows, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    Q4B_CUDA(cudaMemcpy2DAsync(destination, destination_pitch, source, source_pitch, row_bytes, rows,
                               cudaMemcpyDeviceToDevice, context->stream),
             "strided copy");
    return Q4B_OK;
}

int q4b_weight_upload(q4b_context *context, const void *quants, const void *meta, uint32_t rows,
                      uint32_t groups_per_row, uint32_t row_begin, uint32_t row_count,
                      q4b_weight **weight, char *error_message, size_t error_capacity) {
    return upload_common(context, quants, meta, nullptr, Q4B_F16, rows, groups_per_row, row_begin,
                         row_count, weight, error_message, error_capacity);
}

uint64_t q4b_planes_narrowed(const void *scales, const void *biases, int meta_dtype, uint64_t values_per_plane) {
    if (meta_dtype != Q4B_BF16 || scales == nullptr || biases == nullptr) return 0;  // fp16 planes are taken as they are
    uint64_t changed = 0;
    for (int plane = 0; plane < 2; ++plane) {
        const uint16_t *values = static_cast<const uint16_t *>(plane == 0 ? scales : biases);
        for (uint64_t i = 0; i < values_per_plane; ++i) {
            const uint32_t bits = (uint32_t)values[i] << 16;
            float value;
            memcpy(&value, &bits, sizeof(value));
            const float back = __half2float(__float2half_rn(value));
            if (!(back == value) && value == value) ++changed;  // NaN stays NaN: not counted
        }
    }
    return changed;
}

int q4b_weight_upload_planes(q4b_context *context, const void *quants, const void *scales,
                             const void *biases, int meta_dtype, uint32_t rows, uint32_t groups_per_row,
                             uint32_t row_begin, uint32_t row_count, q4b_weight **weight,
                             char *error_message, size_t error_capacity) {
    if (biases == nullptr || (meta_dtype != Q4B_F16 && meta_dtype != Q4B_BF16)) {
        set_error(error_message, error_capacity, "scale/bias planes must be fp16 or bf16 and non-NULL");
        return Q4B_BAD_ARGUMENT;
    }
    return upload_common(context, quants, scales, biases, meta_dtype, rows, groups_per_row, row_begin,
                         row_count, weight, error_message, error_capacity);
}

int q4b_weight_upload_q8(q4b_context *context, const void *quants, const void *scales_bf16, const void *biases_bf16,
                         uint32_t rows, uint32_t groups_per_row, uint32_t row_begin, uint32_t row_count,
                         q4b_weight **weight, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (weight == nullptr || quants == nullptr || scales_bf16 == nullptr || biases_bf16 == nullptr) {
        set_error(error_message, error_capacity, "NULL plane or output pointer");
        return Q4B_BAD_ARGUMENT;
    }
    *weight = nullptr;
    code = validate_shape(rows, groups_per_row, row_begin, row_count, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (context->capturing) {
        set_error(error_message, error_capacity, "weights cannot be loaded while recording a graph");
        return Q4B_BAD_ARGUMENT;
    }
    const size_t blocks = (size_t)row_count * groups_per_row;  // (row, group) cells of the slice
    const size_t quant_bytes = blocks * kGroup, plane_bytes = blocks * 2;
    const uint64_t stream_bytes = (uint64_t)ceil_div(row_count, kQ8Rows) * groups_per_row * kQ8TileBytes;
    uint8_t *staging = nullptr, *tiles = nullptr;
    cudaError_t status = cudaMalloc(&staging, quant_bytes + 2 * plane_bytes + 64);
    if (status == cudaSuccess) status = cudaMalloc(&tiles, stream_bytes);
    if (status != cudaSuccess) {
        cudaFree(staging);
        set_error(error_message, error_capacity, "cudaMalloc of the Q8 weight image: %s", cudaGetErrorString(status));
        return Q4B_LOAD_FAILURE;
    }
    uint8_t *device_quants = staging;
    uint8_t *device_scales = staging + ((quant_bytes + 15) & ~(size_t)15);
    uint8_t *device_biases = device_scales + ((plane_bytes + 15) & ~(size_t)15);
    const size_t first = (size_t)row_begin * groups_per_row;  // only the slice's bytes cross PCIe
    status = cudaMemcpyAsync(device_quants, static_cast<const uint8_t *>(quants) + first * kGroup, quant_bytes,
                             cudaMemcpyHostToDevice, context->stream);
    if (status == cudaSuccess)
        status = cudaMemcpyAsync(device_scales, static_cast<const uint8_t *>(scales_bf16) + first * 2, plane_bytes,
                                 cudaMemcpyHostToDevice, context->stream);
    if (status == cudaSuccess)
        status = cudaMemcpyAsync(device_biases, static_cast<const uint8_t *>(biases_bf16) + first * 2, plane_bytes,
                                 cudaMemcpyHostToDevice, context->stream);
    if (status == cudaSuccess)
        status = launch_repack_q8(device_quants, reinterpret_cast<const uint16_t *>(device_scales),
                                  reinterpret_cast<const uint16_t *>(device_biases), groups_per_row, 0, row_count, tiles,
                                  context->stream);
    ++context->launches;
    if (status == cudaSuccess) status = cudaStreamSynchronize(context->stream);
    cudaFree(staging);
    if (status != cudaSuccess) {
        cudaFree(tiles);
        return device_failure(error_message, error_capacity, "Q8 repack", status);
    }
    q4b_weight *result = new (std::nothrow) q4b_weight();
    if (result == nullptr) {
        cudaFree(tiles);
        return Q4B_LOAD_FAILURE;
    }
    result->view.tiles = tiles;
    result->view.rows = row_count;
    result->view.groups = groups_per_row;
    result->view.row_tiles = ceil_div(row_count, kTileRows);
    result->view.kind = kQ8;
    result->device_bytes = stream_bytes;
    result->rows_total = rows;
    result->row_begin = row_begin;
    result->device = context->device;
    *weight = result;
    return Q4B_OK;
}

int q4b_weight_from_device(q4b_context *context, const void *device_quants, const void *device_meta,
                           uint32_t rows, uint32_t groups_per_row, uint32_t row_begin, uint32_t row_count,
                           q4b_weight **weight, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (weight == nullptr || device_quants == nullptr || device_meta == nullptr) {
        set_error(error_message, error_capacity, "NULL segment or output pointer");
        return Q4B_BAD_ARGUMENT;
    }
    *weight = nullptr;
    code = validate_shape(rows, groups_per_row, row_begin, row_count, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (!aligned16(device_quants) || (reinterpret_cast<uintptr_t>(device_meta) & 3u) != 0) {
        set_error(error_message, error_capacity, "device segments must be 16-byte (quants) / 4-byte (meta) aligned");
        return Q4B_BAD_ARGUMENT;
    }
    return build_weight(context, static_cast<const uint8_t *>(device_quants), device_meta, nullptr, Q4B_F16,
                        rows, groups_per_row, row_begin, row_count, weight, error_message, error_capacity);
}

int q4b_weight_synth(q4b_context *context, uint64_t seed, uint32_t projection, uint32_t rows,
                     uint32_t groups_per_row, uint32_t row_begin, uint32_t row_count, q4b_weight **weight,
                     char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (weight == nullptr) return Q4B_BAD_ARGUMENT;
    *weight = nullptr;
    code = validate_shape(rows, groups_per_row, row_begin, row_count, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    // generate only the slice, in the reference image layout, then load it
    const uint64_t words = (uint64_t)row_count * groups_per_row * 8;
    const uint64_t groups = (uint64_t)row_count * groups_per_row;
    uint8_t *staging = nullptr;
    cudaError_t status = cudaMalloc(&staging, words * 4 + groups * 4);
    if (status != cudaSuccess) {
        set_error(error_message, error_capacity, "cudaMalloc of synthesis staging: %s", cudaGetErrorString(status));
        return Q4B_LOAD_FAILURE;
    }
    uint32_t *device_words = reinterpret_cast<uint32_t *>(staging);
    __half *device_meta = reinterpret_cast<__half *>(staging + words * 4);
    status = launch_synth_codes(seed, 1 + 2ull * projection, device_words,
                                (uint64_t)row_begin * groups_per_row * 8, words, context->stream);
    if (status == cudaSuccess)
        status = launch_synth_meta(seed, 2 + 2ull * projection, device_meta,
                                   (uint64_t)row_begin * groups_per_row, groups, context->stream);
    context->launches += 2;
    if (status != cudaSuccess) {
        cudaFree(staging);
        return device_failure(error_message, error_capacity, "synthesis", status);
    }
    code = build_weight(context, staging, device_meta, nullptr, Q4B_F16, rows, groups_per_row, 0, row_count,
                        weight, error_message, error_capacity);
    cudaFree(staging);
    if (code == Q4B_OK) (*weight)->row_begin = row_begin;
    return code;
}

int q4b_synth_x(q4b_context *context, uint64_t seed, uint64_t stream_id, void *device_x_f16, uint64_t begin,
                uint64_t count, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (device_x_f16 == nullptr) return Q4B_BAD_ARGUMENT;
    Q4B_CUDA(launch_synth_x(seed, stream_id, static_cast<__half *>(device_x_f16), begin, count, context->stream),
             "synthesis of x");
    ++context->launches;
    return Q4B_OK;
}

void q4b_weight_free(q4b_context *context, q4b_weight *weight) {
    if (weight == nullptr) return;
    if (context != nullptr) {
        cudaSetDevice(context->device);
        cudaStreamSynchronize(context->stream);
    }
    if (!weight->borrowed) cudaFree(const_cast<uint8_t *>(weight->view.tiles));
    delete weight;
}

int q4b_weight_rows(const q4b_weight *weight, uint32_t row_begin, uint32_t row_count, q4b_weight **rows,
                    char *error_message, size_t error_capacity) {
    if (weight == nullptr || rows == nullptr || row_count == 0 || row_begin % 128 != 0 || weight->view.kind != kQ4 ||
        row_begin >= weight->view.rows || row_count > weight->view.rows - row_begin) {
        set_error(error_message, error_capacity,
                  "a row range starts at a multiple of 128 rows and lies inside the weight");
        return Q4B_BAD_ARGUMENT;
    }
    q4b_weight *result = new (std::nothrow) q4b_weight(*weight);
    if (result == nullptr) return Q4B_LOAD_FAILURE;
    result->view.tiles = weight->view.tiles + (size_t)(row_begin / 64) * weight->view.groups * kUnitBytes;
    result->view.rows = row_count;
    result->view.row_tiles = ceil_div(row_count, kTileRows);
    result->row_begin = weight->row_begin + row_begin;
    result->device_bytes = 0;
    result->borrowed = true;
    *rows = result;
    return Q4B_OK;
}

int q4b_matmul_rows(q4b_context *context, const q4b_weight *weight, const uint32_t *row_ids, uint32_t count,
                    const void *x, int x_dtype, uint32_t m_rows, void *y, int y_dtype, uint32_t ldy,
                    char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (weight == nullptr || row_ids == nullptr || x == nullptr || y == nullptr || weight->device != context->device ||
        weight->view.kind != kQ4 || m_rows == 0 || m_rows > 16 || ldy < count || !valid_activation_dtype(x_dtype) ||
        !valid_activation_dtype(y_dtype) || !aligned16(x)) {
        set_error(error_message, error_capacity,
                  "weight, row list, x or y missing; 1..16 activation rows, fp16 or fp32, ldy >= count, x 16-byte aligned");
        return Q4B_BAD_ARGUMENT;
    }
    cudaError_t status = launch_matmul_rows(weight->view, row_ids, count, weight->row_begin, x, x_dtype, m_rows, y,
                                            y_dtype, ldy, context->stream);
    if (!context->capturing) ++context->launches;
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "listed-rows matmul", status);
    return Q4B_OK;
}

int q4b_weight_info(const q4b_weight *weight, uint32_t *rows, uint32_t *groups_per_row,
                    uint64_t *device_bytes) {
    if (weight == nullptr) return Q4B_BAD_ARGUMENT;
    if (rows != nullptr) *rows = weight->view.rows;
    if (groups_per_row != nullptr) *groups_per_row = weight->view.groups;
    if (device_bytes != nullptr) *device_bytes = weight->device_bytes;
    return Q4B_OK;
}

int q4b_context_push_outputs(q4b_context *context, uint32_t world, void *const *peer_y, int count) {
    if (context == nullptr) return Q4B_BAD_ARGUMENT;
    context->push_peers = 0;
    if (peer_y == nullptr || world == 0 || world > (uint32_t)kMaxPeers || count < 1 || count > kMaxSegments) {
        return Q4B_BAD_ARGUMENT;
    }
    for (int s = 0; s < kMaxSegments; ++s) {
        for (uint32_t r = 0; r < (uint32_t)kMaxPeers; ++r) {
            context->push_y[s][r] = s < count && r < world ? peer_y[(size_t)s * world + r] : nullptr;
        }
    }
    context->push_peers = world;
    return Q4B_OK;
}

struct q4b_barrier {
    uint32_t *counter;                 // own arrivals, device memory, counts up for ever
    uint32_t *counters[kMaxPeers];     // every rank's (own included)
    uint32_t world, rank;
    int device;
};

int q4b_barrier_create(q4b_context *context, uint32_t world, uint32_t rank, q4b_barrier **barrier,
                       char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (barrier == nullptr || world == 0 || world > (uint32_t)kMaxPeers || rank >= world) {
        set_error(error_message, error_capacity, "a barrier joins 1..%d ranks", kMaxPeers);
        return Q4B_BAD_ARGUMENT;
    }
    q4b_barrier *result = new (std::nothrow) q4b_barrier();
    if (result == nullptr) return Q4B_DEVICE_FAILURE;
    cudaError_t status = cudaMalloc(&result->counter, 256);
    if (status == cudaSuccess) status = cudaMemset(result->counter, 0, 256);
    if (status != cudaSuccess) {
        delete result;
        return device_failure(error_message, error_capacity, "barrier counter", status);
    }
    result->world = world;
    result->rank = rank;
    result->device = context->device;
    result->counters[rank] = result->counter;
    *barrier = result;
    return Q4B_OK;
}

void *q4b_barrier_counter(q4b_barrier *barrier) { return barrier != nullptr ? barrier->counter : nullptr; }

int q4b_barrier_set_peer(q4b_barrier *barrier, uint32_t peer_rank, void *peer_counter) {
    if (barrier == nullptr || peer_rank >= barrier->world || peer_counter == nullptr) return Q4B_BAD_ARGUMENT;
    barrier->counters[peer_rank] = static_cast<uint32_t *>(peer_counter);
    return Q4B_OK;
}

int q4b_barrier_queue(q4b_context *context, q4b_barrier *barrier, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (barrier == nullptr || barrier->device != context->device) {
        set_error(error_message, error_capacity, "no barrier, or another device's");
        return Q4B_BAD_ARGUMENT;
    }
    for (uint32_t r = 0; r < barrier->world; ++r) {
        if (barrier->counters[r] == nullptr) {
            set_error(error_message, error_capacity, "rank %u's counter is not set", r);
            return Q4B_BAD_ARGUMENT;
        }
    }
    // the number of the round lives in device memory (the second 128 bytes of the own counter's allocation), so a
    // recorded barrier counts on at every replay
    Q4B_CUDA(launch_rank_barrier(barrier->counters, barrier->world, barrier->rank, barrier->counter + 32,
                                 context->status_device, context->stream),
             "rank barrier");
    if (!context->capturing) ++context->launches;
    return Q4B_OK;
}

void q4b_barrier_free(q4b_context *context, q4b_barrier *barrier) {
    if (barrier == nullptr) return;
    if (context != nullptr) {
        cudaSetDevice(context->device);
        cudaStreamSynchronize(context->stream);
    }
    cudaFree(barrier->counter);
    delete barrier;
}

int q4b_embedding_lookup(q4b_context *context, const q4b_weight *embedding, const uint32_t *rows, uint32_t count,
                         void *out, int out_dtype, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (embedding == nullptr || rows == nullptr || out == nullptr || !valid_activation_dtype(out_dtype) ||
        embedding->device != context->device || !aligned16(out) || embedding->view.kind != kQ4) {
        set_error(error_message, error_capacity, "embedding, row list or output missing, or not fp16/fp32 16-byte aligned");
        return Q4B_BAD_ARGUMENT;
    }
    cudaError_t status = launch_lookup_rows(embedding->view, rows, count, embedding->row_begin, out, out_dtype,
                                            context->stream);
    if (!context->capturing) ++context->launches;
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "embedding lookup", status);
    return Q4B_OK;
}

int q4b_rmsnorm(q4b_context *context, const void *input, int input_dtype, const float *weight, void *output_f16,
                uint32_t hidden, uint32_t batch_rows, float epsilon, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (input == nullptr || weight == nullptr || output_f16 == nullptr || hidden == 0 || batch_rows == 0 ||
        !valid_activation_dtype(input_dtype) || !(epsilon >= 0.0f)) {
        set_error(error_message, error_capacity,
                  "input (fp16 or fp32), weight, output, hidden, batch_rows or epsilon missing or invalid");
        return Q4B_BAD_ARGUMENT;
    }
    cudaError_t status = launch_rmsnorm(input, input_dtype, weight, output_f16, hidden, batch_rows, epsilon,
                                        context->stream);
    if (!context->capturing) ++context->launches;
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "rms norm", status);
    return Q4B_OK;
}

int q4b_weight_unpack(q4b_context *context, const q4b_weight *weight, uint8_t *codes, float *w32,
                      uint16_t *w16, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (weight == nullptr) {
        set_error(error_message, error_capacity, "weight is NULL");
        return Q4B_BAD_ARGUMENT;
    }
    const size_t elements = (size_t)weight->view.rows * weight->view.groups * kGroup;
    uint8_t *device_codes = nullptr;
    float *device_w32 = nullptr;
    __half *device_w16 = nullptr;
    cudaError_t status = cudaSuccess;
    if (codes != nullptr) status = cudaMalloc(&device_codes, elements);
    if (status == cudaSuccess && w32 != nullptr) status = cudaMalloc(&device_w32, elements * 4);
    if (status == cudaSuccess && w16 != nullptr) status = cudaMalloc(&device_w16, elements * 2);
    if (status == cudaSuccess) {
        status = weight->view.kind == kQ8
                     ? launch_unpack_q8(weight->view, device_codes, device_w32, device_w16, context->stream)
                     : launch_unpack(weight->view, device_codes, device_w32, device_w16, context->stream);
        ++context->launches;
    }
    if (status == cudaSuccess && codes != nullptr)
        status = cudaMemcpyAsync(codes, device_codes, elements, cudaMemcpyDeviceToHost, context->stream);
    if (status == cudaSuccess && w32 != nullptr)
        status = cudaMemcpyAsync(w32, device_w32, elements * 4, cudaMemcpyDeviceToHost, context->stream);
    if (status == cudaSuccess && w16 != nullptr)
        status = cudaMemcpyAsync(w16, device_w16, elements * 2, cudaMemcpyDeviceToHost, context->stream);
    if (status == cudaSuccess) status = cudaStreamSynchronize(context->stream);
    cudaFree(device_codes);
    cudaFree(device_w32);
    cudaFree(device_w16);
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "unpack", status);
    return Q4B_OK;
}

int q4b_matmul(q4b_context *context, const q4b_weight *weight, const void *x, int x_dtype, uint32_t m_rows,
               void *y, int y_dtype, uint32_t ldy, const void *residual, int residual_dtype,
               uint32_t ld_residual, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    code = check_matmul_arguments(context, weight, x, x_dtype, m_rows, y, y_dtype, ldy, error_message,
                                  error_capacity);
    if (code != Q4B_OK) return code;
    if (residual != nullptr && (!valid_dtype_pair(x_dtype, residual_dtype) || ld_residual < weight->view.rows)) {
        set_error(error_message, error_capacity,
                  "residual must be fp16 or fp32 (bf16 or fp32 beside bf16 activations) with ld >= rows");
        return Q4B_BAD_ARGUMENT;
    }
    ProjectionArgs args = {};
    args.w[0] = weight->view;
    args.y[0] = y;
    args.ldy[0] = ldy;
    args.segments = 1;
    args.x = x;
    args.x_dtype = x_dtype;
    args.m_rows = m_rows;
    args.y_dtype = y_dtype;
    args.residual = residual;
    args.residual_dtype = residual != nullptr ? residual_dtype : (int)kNone;
    args.ld_residual = ld_residual;
    return run_projection(context, args, error_message, error_capacity);
}

int q4b_matmul_no_alloc(q4b_context *context, const q4b_weight *weight, const void *x, int x_dtype,
                        uint32_t m_rows, void *y, int y_dtype, uint32_t ldy, char *error_message,
                        size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    code = check_matmul_arguments(context, weight, x, x_dtype, m_rows, y, y_dtype, ldy, error_message,
                                  error_capacity);
    if (code != Q4B_OK) return code;
    ProjectionArgs args = {};
    args.w[0] = weight->view;
    args.y[0] = y;
    args.ldy[0] = ldy;
    args.segments = 1;
    args.x = x;
    args.x_dtype = x_dtype;
    args.m_rows = m_rows;
    args.y_dtype = y_dtype;
    args.residual_dtype = kNone;
    return run_projection(context, args, error_message, error_capacity, true);
}

int q4b_matmul_group(q4b_context *context, const q4b_weight *const *weights, int count, const void *x,
                     int x_dtype, uint32_t m_rows, void *const *y, int y_dtype, const uint32_t *ldy,
                     char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (weights == nullptr || y == nullptr || ldy == nullptr || count < 1 || count > kMaxSegments) {
        set_error(error_message, error_capacity, "a group holds 1..%d matrices", kMaxSegments);
        return Q4B_BAD_ARGUMENT;
    }
    ProjectionArgs args = {};
    for (int s = 0; s < count; ++s) {
        code = check_matmul_arguments(context, weights[s], x, x_dtype, m_rows, y[s], y_dtype, ldy[s],
                                      error_message, error_capacity);
        if (code != Q4B_OK) return code;
        if (weights[s]->view.groups != weights[0]->view.groups) {
            set_error(error_message, error_capacity, "matrices of a group must share K");
            return Q4B_BAD_ARGUMENT;
        }
        args.w[s] = weights[s]->view;
        args.y[s] = y[s];
        args.ldy[s] = ldy[s];
    }
    args.segments = count;
    args.x = x;
    args.x_dtype = x_dtype;
    args.m_rows = m_rows;
    args.y_dtype = y_dtype;
    args.residual_dtype = kNone;
    return run_projection(context, args, error_message, error_capacity);
}

int q4b_gate_up_silu(q4b_context *context, const q4b_weight *gate, const q4b_weight *up, const void *x,
                     int x_dtype, uint32_t m_rows, void *y, int y_dtype, uint32_t ldy, char *error_message,
                     size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    code = check_matmul_arguments(context, gate, x, x_dtype, m_rows, y, y_dtype, ldy, error_message,
                                  error_capacity);
    if (code != Q4B_OK) return code;
    if (up == nullptr || up->device != gate->device || up->view.rows != gate->view.rows ||
        up->view.groups != gate->view.groups) {
        set_error(error_message, error_capacity, "gate and up must have the same shape and device");
        return Q4B_BAD_ARGUMENT;
    }
    ProjectionArgs args = {};
    args.w[0] = gate->view;
    args.up = up->view;
    args.fused_silu = 1;
    args.y[0] = y;
    args.ldy[0] = ldy;
    args.segments = 1;
    args.x = x;
    args.x_dtype = x_dtype;
    args.m_rows = m_rows;
    args.y_dtype = y_dtype;
    args.residual_dtype = kNone;
    return run_projection(context, args, error_message, error_capacity);
}

static int host_call(q4b_context *context, const q4b_weight *gate, const q4b_weight *up, const void *x_host,
                     int x_dtype, uint32_t m_rows, void *y_host, int y_dtype, double *gpu_ms,
                     char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (gate == nullptr || x_host == nullptr || y_host == nullptr || m_rows == 0 ||
        !valid_dtype_pair(x_dtype, y_dtype)) {
        set_error(error_message, error_capacity, "invalid projection");
        return Q4B_BAD_ARGUMENT;
    }
    const size_t K = (size_t)gate->view.groups * kGroup, N = gate->view.rows;
    const size_t x_bytes = (size_t)m_rows * K * dtype_bytes(x_dtype);
    const size_t y_bytes = (size_t)m_rows * N * dtype_bytes(y_dtype);
    uint8_t *device = nullptr;
    const size_t x_padded = (x_bytes + 255) & ~(size_t)255;
    Q4B_CUDA(cudaMalloc(&device, x_padded + y_bytes), "cudaMalloc of call buffers");
    cudaError_t status = cudaMemcpyAsync(device, x_host, x_bytes, cudaMemcpyHostToDevice, context->stream);
    cudaEvent_t start = nullptr, stop = nullptr;
    if (status == cudaSuccess) status = cudaEventCreate(&start);
    if (status == cudaSuccess) status = cudaEventCreate(&stop);
    if (status == cudaSuccess) status = cudaEventRecord(start, context->stream);
    if (status == cudaSuccess) {
        if (up != nullptr) {
            code = q4b_gate_up_silu(context, gate, up, device, x_dtype, m_rows, device + x_padded, y_dtype,
                                    (uint32_t)N, error_message, error_capacity);
        } else {
            code = q4b_matmul(context, gate, device, x_dtype, m_rows, device + x_padded, y_dtype, (uint32_t)N,
                              nullptr, Q4B_NONE, 0, error_message, error_capacity);
        }
    }
    if (status == cudaSuccess && code == Q4B_OK) status = cudaEventRecord(stop, context->stream);
    if (status == cudaSuccess && code == Q4B_OK)
        status = cudaMemcpyAsync(y_host, device + x_padded, y_bytes, cudaMemcpyDeviceToHost, context->stream);
    if (status == cudaSuccess && code == Q4B_OK) status = cudaStreamSynchronize(context->stream);
    if (status == cudaSuccess && code == Q4B_OK && gpu_ms != nullptr) {
        float ms = 0.0f;
        status = cudaEventElapsedTime(&ms, start, stop);
        *gpu_ms = ms;
    }
    if (start != nullptr) cudaEventDestroy(start);
    if (stop != nullptr) cudaEventDestroy(stop);
    cudaFree(device);
    if (code != Q4B_OK) return code;
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "projection", status);
    return Q4B_OK;
}

int q4b_matmul_host(q4b_context *context, const q4b_weight *weight, const void *x_host, int x_dtype,
                    uint32_t m_rows, void *y_host, int y_dtype, double *gpu_ms, char *error_message,
                    size_t error_capacity) {
    return host_call(context, weight, nullptr, x_host, x_dtype, m_rows, y_host, y_dtype, gpu_ms,
                     error_message, error_capacity);
}

int q4b_gate_up_silu_host(q4b_context *context, const q4b_weight *gate, const q4b_weight *up,
                          const void *x_host, int x_dtype, uint32_t m_rows, void *y_host, int y_dtype,
                          double *gpu_ms, char *error_message, size_t error_capacity) {
    if (up == nullptr) {
        set_error(error_message, error_capacity, "invalid projection");
        return Q4B_BAD_ARGUMENT;
    }
    return host_call(context, gate, up, x_host, x_dtype, m_rows, y_host, y_dtype, gpu_ms, error_message,
                     error_capacity);
}

int q4b_probe_read(q4b_context *context, int mode, size_t bytes, int ctas_per_sm, uint32_t stages,
                   uint32_t stage_bytes, int iterations, double *gigabytes_per_second, char *error_message,
                   size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (gigabytes_per_second == nullptr || bytes < (1u << 20) || iterations < 1 || ctas_per_sm < 1 || mode < 0 ||
        mode > 2 || context->capturing) {
        set_error(error_message, error_capacity, "invalid probe arguments");
        return Q4B_BAD_ARGUMENT;
    }
    if (mode != 0 && stage_bytes != 0) bytes -= bytes % ((size_t)stage_bytes);
    uint8_t *buffer = nullptr;
    Q4B_CUDA(cudaMalloc(&buffer, bytes + 4), "cudaMalloc of the probe buffer");
    cudaError_t status = cudaMemsetAsync(buffer, 0x5a, bytes + 4, context->stream);
    uint32_t *sink = reinterpret_cast<uint32_t *>(buffer + bytes);
    const int ctas = context->sm_count * ctas_per_sm;
    if (status == cudaSuccess) status = launch_probe(mode, buffer, bytes, ctas, stages, stage_bytes, sink, context->stream);
    if (status == cudaSuccess) status = cudaEventRecord(context->timer_start, context->stream);
    for (int i = 0; i < iterations && status == cudaSuccess; ++i) {
        status = launch_probe(mode, buffer, bytes, ctas, stages, stage_bytes, sink, context->stream);
    }
    context->launches += iterations + 1;
    if (status == cudaSuccess) status = cudaEventRecord(context->timer_stop, context->stream);
    if (status == cudaSuccess) status = cudaStreamSynchronize(context->stream);
    float ms = 0.0f;
    if (status == cudaSuccess) status = cudaEventElapsedTime(&ms, context->timer_start, context->timer_stop);
    cudaFree(buffer);
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "probe", status);
    *gigabytes_per_second = (double)bytes * iterations / (ms * 1e-3) / 1e9;
    return Q4B_OK;
}

int q4b_probe_signal(q4b_context *context, void *own_words, void *peer_words, uint32_t payload_bytes,
                     uint32_t rounds, uint32_t rounds_before, int initiator, int mode,
                     double *microseconds_per_round_trip, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (own_words == nullptr || peer_words == nullptr || microseconds_per_round_trip == nullptr || rounds == 0 ||
        payload_bytes > (1u << 20) || payload_bytes % 4 != 0 || mode < 0 || mode > 7 || context->capturing) {
        set_error(error_message, error_capacity, "invalid signal probe arguments");
        return Q4B_BAD_ARGUMENT;
    }
    // word 0: the flag; word 1: the status; the payload from byte 256 on
    uint32_t *own = static_cast<uint32_t *>(own_words), *peer = static_cast<uint32_t *>(peer_words);
    cudaError_t status = cudaMemsetAsync(own + 1, 0, 4, context->stream);
    if (status == cudaSuccess) status = cudaEventRecord(context->timer_start, context->stream);
    if (status == cudaSuccess) {
        status = launch_probe_signal(own, peer, peer + 64, payload_bytes / 4, rounds, rounds_before, initiator, mode, own + 1,
                                     context->stream);
    }
    context->launches += 1;
    if (status == cudaSuccess) status = cudaEventRecord(context->timer_stop, context->stream);
    if (status == cudaSuccess) status = cudaStreamSynchronize(context->stream);
    float ms = 0.0f;
    if (status == cudaSuccess) status = cudaEventElapsedTime(&ms, context->timer_start, context->timer_stop);
    uint32_t gave_up = 0;
    if (status == cudaSuccess) status = cudaMemcpy(&gave_up, own + 1, 4, cudaMemcpyDeviceToHost);
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "signal probe", status);
    if (gave_up != 0) {
        set_error(error_message, error_capacity, "the peer did not answer in round %u", gave_up);
        return Q4B_DEVICE_FAILURE;
    }
    *microseconds_per_round_trip = (double)ms * 1e3 / rounds;
    return Q4B_OK;
}

/* ---------------------------------------------------------------- sequences */
int q4b_sequence_create(q4b_context *context, uint32_t m_rows, uint32_t world, uint32_t rank,
                        q4b_sequence **sequence, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (sequence == nullptr || m_rows == 0 || m_rows > 16 || world == 0 || world > (uint32_t)kMaxPeers || rank >= world) {
        set_error(error_message, error_capacity, "a sequence takes 1..16 activation rows and 1..%d ranks", kMaxPeers);
        return Q4B_BAD_ARGUMENT;
    }
    q4b_sequence *result = new (std::nothrow) q4b_sequence();
    if (result == nullptr) return Q4B_DEVICE_FAILURE;
    result->m_rows = m_rows;
    result->world = world;
    result->rank = rank;
    result->device = context->device;
    *sequence = result;
    return Q4B_OK;
}

static int sequence_add(q4b_sequence *sequence, const q4b_weight *const *weights, int count, const q4b_weight *up,
                        const void *x, int x_dtype, void *const *y, const uint32_t *ldy, int y_dtype,
                        const void *residual, int residual_dtype, uint32_t ld_residual, char *error_message,
                        size_t error_capacity) {
    if (sequence == nullptr || sequence->finalized || weights == nullptr || y == nullptr || ldy == nullptr ||
        x == nullptr || count < 1 || count > kMaxSegments || !valid_activation_dtype(y_dtype) ||
        !valid_activation_dtype(x_dtype) || !aligned16(x)) {
        set_error(error_message, error_capacity,
                  "invalid job (1..%d matrices, 16-byte aligned fp16 or fp32 x, fp16 or fp32 y)", kMaxSegments);
        return Q4B_BAD_ARGUMENT;
    }
    DecodeJob job = {};
    for (int s = 0; s < count; ++s) {
        if (weights[s] == nullptr || y[s] == nullptr || weights[s]->device != sequence->device ||
            weights[s]->view.groups != weights[0]->view.groups || ldy[s] < weights[s]->view.rows ||
            weights[s]->view.kind != kQ4) {
            set_error(error_message, error_capacity,
                      "matrices of a job must be Q4, live on the context's device, share K and fit ldy");
            return Q4B_BAD_ARGUMENT;
        }
        job.tiles[s] = weights[s]->view.tiles;
        job.rows[s] = weights[s]->view.rows;
        job.ldy[s] = ldy[s];
        job.y[s][sequence->rank] = y[s];
    }
    if (up != nullptr) {
        if (count != 1 || up->view.rows != weights[0]->view.rows || up->view.groups != weights[0]->view.groups ||
            up->view.kind != kQ4) {
            set_error(error_message, error_capacity, "gate and up must be Q4 matrices of the same shape");
            return Q4B_BAD_ARGUMENT;
        }
        job.up_tiles = up->view.tiles;
        job.fused = 1;
    }
    if (residual != nullptr && (!valid_activation_dtype(residual_dtype) || ld_residual < weights[0]->view.rows)) {
        set_error(error_message, error_capacity, "residual must be fp16 or fp32 with ld >= rows");
        return Q4B_BAD_ARGUMENT;
    }
    job.x = x;
    job.x_dtype = x_dtype;
    job.residual = residual;
    job.residual_dtype = residual != nullptr ? residual_dtype : (int)kNone;
    job.ld_residual = ld_residual;
    job.groups = weights[0]->view.groups;
    job.segments = (uint32_t)count;
    job.y_dtype = y_dtype;
    sequence->jobs.push_back(job);
    return Q4B_OK;
}

int q4b_sequence_add_matmul(q4b_sequence *sequence, const q4b_weight *const *weights, int count, const void *x,
                            void *const *y, const uint32_t *ldy, int y_dtype, char *error_message,
                            size_t error_capacity) {
    return sequence_add(sequence, weights, count, nullptr, x, Q4B_F16, y, ldy, y_dtype, nullptr, Q4B_NONE, 0,
                        error_message, error_capacity);
}

int q4b_sequence_add_projection(q4b_sequence *sequence, const q4b_weight *weight, const void *x, int x_dtype, void *y,
                                int y_dtype, uint32_t ldy, const void *residual, int residual_dtype,
                                uint32_t ld_residual, char *error_message, size_t error_capacity) {
    return sequence_add(sequence, &weight, 1, nullptr, x, x_dtype, &y, &ldy, y_dtype, residual, residual_dtype,
                        ld_residual, error_message, error_capacity);
}

int q4b_sequence_add_gate_up(q4b_sequence *sequence, const q4b_weight *gate, const q4b_weight *up, const void *x,
                             void *y, uint32_t ldy, int y_dtype, char *error_message, size_t error_capacity) {
    if (up == nullptr) {
        set_error(error_message, error_capacity, "up is NULL");
        return Q4B_BAD_ARGUMENT;
    }
    return sequence_add(sequence, &gate, 1, up, x, Q4B_F16, &y, &ldy, y_dtype, nullptr, Q4B_NONE, 0, error_message,
                        error_capacity);
}

int q4b_sequence_set_peer_output(q4b_sequence *sequence, uint32_t job, uint32_t segment, uint32_t peer_rank,
                                 void *peer_y) {
    if (sequence == nullptr || sequence->finalized || job >= sequence->jobs.size() || segment >= kMaxSegments ||
        peer_rank >= sequence->world) {
        return Q4B_BAD_ARGUMENT;
    }
    sequence->jobs[job].y[segment][peer_rank] = peer_y;
    return Q4B_OK;
}

int q4b_sequence_set_job_blocks(q4b_sequence *sequence, uint32_t job, uint32_t blocks_on_all_ranks) {
    if (sequence == nullptr || sequence->finalized || job >= sequence->jobs.size() || blocks_on_all_ranks == 0) {
        return Q4B_BAD_ARGUMENT;
    }
    sequence->jobs[job].expected_blocks = blocks_on_all_ranks;
    return Q4B_OK;
}

int q4b_sequence_finalize(q4b_context *context, q4b_sequence *sequence, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (sequence == nullptr || sequence->finalized || sequence->jobs.empty() || context->capturing) {
        set_error(error_message, error_capacity, "nothing to finalize");
        return Q4B_BAD_ARGUMENT;
    }
    SequenceLaunch &launch = sequence->launch;
    Q4B_CUDA(decode_geometry(sequence->m_rows, context->variant, context->sm_count, true, &launch.geometry),
             "sequence geometry");
    size_t scratch_bytes = 0, counter_bytes = 0;
    for (DecodeJob &job : sequence->jobs) {
        size_t s = 0, c = 0;
        plan_decode_job(&job, sequence->m_rows, launch.geometry, &s, &c);
        if (s > scratch_bytes) scratch_bytes = s;
        if (c > counter_bytes) counter_bytes = c;
        uint32_t own = 0;
        for (uint32_t q = 0; q < job.segments; ++q) own += ceil_div(job.rows[q], 64);
        if (job.expected_blocks == 0) job.expected_blocks = own * sequence->world;
        if (job.expected_blocks < own) {
            set_error(error_message, error_capacity, "a job's block count over all ranks is below this rank's own");
            return Q4B_BAD_ARGUMENT;
        }
    }
    const size_t job_bytes = sequence->jobs.size() * sizeof(DecodeJob);
    // completion counters, then one line for the epoch word and one for the exit count
    sequence->done_words = (sequence->jobs.size() * 8 + 2) * kDoneStride;
    cudaError_t status = cudaMalloc(&sequence->device_jobs, job_bytes);
    if (status == cudaSuccess) status = cudaMalloc(&sequence->done, sequence->done_words * sizeof(uint32_t));
    if (status == cudaSuccess) status = cudaMalloc(&sequence->scratch, scratch_bytes + 256);
    if (status == cudaSuccess) status = cudaMalloc(&sequence->counters, counter_bytes + 256);
    if (status == cudaSuccess) status = cudaMemcpy(sequence->device_jobs, sequence->jobs.data(), job_bytes, cudaMemcpyHostToDevice);
    if (status == cudaSuccess) status = cudaMemset(sequence->done, 0, sequence->done_words * sizeof(uint32_t));
    if (status == cudaSuccess) status = cudaMemset(sequence->counters, 0, counter_bytes + 256);
    if (status != cudaSuccess) return device_failure(error_message, error_capacity, "sequence buffers", status);
    sequence->peer_done[sequence->rank] = sequence->done;
    launch.jobs = sequence->device_jobs;
    launch.job_count = (uint32_t)sequence->jobs.size();
    launch.m_rows = sequence->m_rows;
    launch.world = sequence->world;
    launch.done = sequence->done;
    launch.epoch = sequence->done + sequence->jobs.size() * 8 * kDoneStride;
    launch.exit_count = launch.epoch + kDoneStride;
    launch.scratch = sequence->scratch;
    launch.counters = sequence->counters;
    launch.status = context->status_device;
    sequence->finalized = true;
    return Q4B_OK;
}

void *q4b_sequence_done_counters(q4b_sequence *sequence) {
    return sequence != nullptr && sequence->finalized ? sequence->done : nullptr;
}

int q4b_sequence_set_peer_counters(q4b_sequence *sequence, uint32_t peer_rank, void *peer_counters) {
    if (sequence == nullptr || !sequence->finalized || peer_rank >= sequence->world || peer_counters == nullptr) {
        return Q4B_BAD_ARGUMENT;
    }
    sequence->peer_done[peer_rank] = static_cast<uint32_t *>(peer_counters);
    return Q4B_OK;
}

int q4b_sequence_launch(q4b_context *context, q4b_sequence *sequence, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (sequence == nullptr || !sequence->finalized) {
        set_error(error_message, error_capacity, "the sequence is not finalized");
        return Q4B_BAD_ARGUMENT;
    }
    for (uint32_t r = 0; r < sequence->world; ++r) {
        if (sequence->peer_done[r] == nullptr) {
            set_error(error_message, error_capacity, "rank %u's completion counters are not set", r);
            return Q4B_BAD_ARGUMENT;
        }
        sequence->launch.peer_done[r] = sequence->peer_done[r];
    }
    Q4B_CUDA(launch_sequence(sequence->launch, context->stream), "sequence launch");
    if (!context->capturing) ++context->launches;
    return Q4B_OK;
}

int q4b_sequence_profile(q4b_context *context, q4b_sequence *sequence, uint64_t *clocks, uint32_t capacity,
                         uint32_t *thread_blocks, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (sequence == nullptr || !sequence->finalized || context->capturing) {
        set_error(error_message, error_capacity, "the sequence is not finalized, or a graph is being recorded");
        return Q4B_BAD_ARGUMENT;
    }
    const uint32_t ctas = sequence->launch.geometry.ctas;
    const size_t bytes = (size_t)ctas * kProfileSlots * sizeof(unsigned long long);
    if (thread_blocks != nullptr) *thread_blocks = ctas;
    Q4B_CUDA(cudaStreamSynchronize(context->stream), "stream synchronize");
    if (sequence->profile == nullptr) {  // first call: switch the clocks on
        Q4B_CUDA(cudaMalloc(&sequence->profile, bytes), "cudaMalloc of the profile");
        Q4B_CUDA(cudaMemset(sequence->profile, 0, bytes), "profile reset");
        sequence->launch.profile = sequence->profile;
        return Q4B_OK;
    }
    if (clocks != nullptr) {
        if (capacity < ctas * kProfileSlots) {
            set_error(error_message, error_capacity, "the buffer holds %u values, the profile has %u", capacity,
                      ctas * kProfileSlots);
            return Q4B_BAD_ARGUMENT;
        }
        Q4B_CUDA(cudaMemcpy(clocks, sequence->profile, bytes, cudaMemcpyDeviceToHost), "profile read");
    }
    Q4B_CUDA(cudaMemset(sequence->profile, 0, bytes), "profile reset");
    return Q4B_OK;
}

void q4b_sequence_free(q4b_context *context, q4b_sequence *sequence) {
    if (sequence == nullptr) return;
    if (context != nullptr) {
        cudaSetDevice(context->device);
        cudaStreamSynchronize(context->stream);
    }
    cudaFree(sequence->profile);
    cudaFree(sequence->device_jobs);
    cudaFree(sequence->done);
    cudaFree(sequence->scratch);
    cudaFree(sequence->counters);
    delete sequence;
}

/* ----------------------------------------------------- memory shared by ranks */
int q4b_ipc_export(q4b_context *context, void *device_pointer, void *handle_64_bytes, char *error_message,
                   size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (device_pointer == nullptr || handle_64_bytes == nullptr) return Q4B_BAD_ARGUMENT;
    cudaIpcMemHandle_t handle;
    Q4B_CUDA(cudaIpcGetMemHandle(&handle, device_pointer), "cudaIpcGetMemHandle");
    memcpy(handle_64_bytes, &handle, sizeof(handle));
    return Q4B_OK;
}

int q4b_ipc_open(q4b_context *context, const void *handle_64_bytes, void **peer_pointer, char *error_message,
                 size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (handle_64_bytes == nullptr || peer_pointer == nullptr) return Q4B_BAD_ARGUMENT;
    cudaIpcMemHandle_t handle;
    memcpy(&handle, handle_64_bytes, sizeof(handle));
    Q4B_CUDA(cudaIpcOpenMemHandle(peer_pointer, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    return Q4B_OK;
}

int q4b_ipc_close(q4b_context *context, void *peer_pointer) {
    if (context != nullptr) cudaSetDevice(context->device);
    return cudaIpcCloseMemHandle(peer_pointer) == cudaSuccess ? Q4B_OK : Q4B_DEVICE_FAILURE;
}

int q4b_timer_start(q4b_context *context, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    Q4B_CUDA(cudaEventRecord(context->timer_start, context->stream), "timer start");
    context->timer_armed = true;
    return Q4B_OK;
}

int q4b_sync(q4b_context *context, double *device_ms, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (device_ms != nullptr && context->timer_armed) {
        Q4B_CUDA(cudaEventRecord(context->timer_stop, context->stream), "timer stop");
    }
    Q4B_CUDA(cudaStreamSynchronize(context->stream), "stream synchronize");
    Q4B_CUDA(cudaGetLastError(), "asynchronous error");
    if (*context->status_host != 0) {
        const uint32_t code = *context->status_host;
        *context->status_host = 0;
        if (context->counters != nullptr) cudaMemset(context->counters, 0, context->counter_bytes);
        set_error(error_message, error_capacity,
                  "a device-side wait expired (code 0x%x); results of the queued work are invalid", code);
        return Q4B_DEVICE_FAILURE;
    }
    if (device_ms != nullptr) {
        *device_ms = 0.0;
        if (context->timer_armed) {
            float ms = 0.0f;
            Q4B_CUDA(cudaEventElapsedTime(&ms, context->timer_start, context->timer_stop), "timer read");
            *device_ms = ms;
        }
    }
    return Q4B_OK;
}

int q4b_graph_begin(q4b_context *context, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (context->capturing) {
        set_error(error_message, error_capacity, "already recording");
        return Q4B_BAD_ARGUMENT;
    }
    Q4B_CUDA(cudaStreamBeginCapture(context->stream, cudaStreamCaptureModeThreadLocal), "begin capture");
    context->capturing = true;
    return Q4B_OK;
}

int q4b_graph_end(q4b_context *context, q4b_graph **graph, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (!context->capturing || graph == nullptr) {
        set_error(error_message, error_capacity, "not recording");
        return Q4B_BAD_ARGUMENT;
    }
    context->capturing = false;
    cudaGraph_t captured = nullptr;
    Q4B_CUDA(cudaStreamEndCapture(context->stream, &captured), "end capture");
    cudaGraphExec_t exec = nullptr;
    cudaError_t status = cudaGraphInstantiate(&exec, captured, 0);
    if (status != cudaSuccess) {
        cudaGraphDestroy(captured);
        return device_failure(error_message, error_capacity, "graph instantiate", status);
    }
    size_t nodes = 0;
    cudaGraphGetNodes(captured, nullptr, &nodes);
    q4b_graph *result = new (std::nothrow) q4b_graph();
    if (result == nullptr) {
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(captured);
        set_error(error_message, error_capacity, "out of host memory");
        return Q4B_DEVICE_FAILURE;
    }
    result->graph = captured;
    result->exec = exec;
    result->launches = nodes;
    *graph = result;
    return Q4B_OK;
}

int q4b_graph_launch(q4b_context *context, q4b_graph *graph, char *error_message, size_t error_capacity) {
    int code = check_context(context, error_message, error_capacity);
    if (code != Q4B_OK) return code;
    if (graph == nullptr) return Q4B_BAD_ARGUMENT;
    Q4B_CUDA(cudaGraphLaunch(graph->exec, context->stream), "graph launch");
    context->launches += graph->launches;
    return Q4B_OK;
}

void q4b_graph_free(q4b_graph *graph) {
    if (graph == nullptr) return;
    cudaGraphExecDestroy(graph->exec);
    cudaGraphDestroy(graph->graph);
    delete graph;
}

}  // extern "C"
