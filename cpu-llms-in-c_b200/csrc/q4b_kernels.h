// Host-side launchers of the CUDA kernels (internal to the library).
#pragma once
#include "q4b_common.cuh"

struct q4b_context;

namespace q4b {

// cudaFuncSetAttribute applies to one device: the launchers remember what they set per device, so that a
// process with contexts on several GPUs configures each of them.  Returns -1 for a device beyond the table
// (the caller then sets the attribute on every launch).
constexpr int kMaxDevices = 64;
inline int device_slot() {
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return -1;
    return device;
}

// ---- q4b_pack.cu ----
// raw image planes (device) -> tile stream.  rows_total/groups describe the
// source matrix; rows [row_begin, row_begin+row_count) are packed.  meta is
// interleaved fp16 {scale,bias} when biases == nullptr, else `meta` is the
// scale plane and `biases` the bias plane (fp16 or bf16 by meta_dtype).
cudaError_t launch_repack(const uint8_t *quants, const void *meta, const void *biases,
                          int meta_dtype, uint32_t groups, uint32_t row_begin,
                          uint32_t row_count, uint8_t *tiles, cudaStream_t stream);
// tile stream -> codes u8 [rows][K], w32 [rows][K], w16 [rows][K] (any may be null)
cudaError_t launch_unpack(WeightView w, uint8_t *codes, float *w32, __half *w16,
                          cudaStream_t stream);
// affine Q8 planes (device): codes [N][G][64] bytes, bf16 scales / biases [N][G] -> the Q8 stream; and back
cudaError_t launch_repack_q8(const uint8_t *quants, const uint16_t *scales, const uint16_t *biases, uint32_t groups,
                             uint32_t row_begin, uint32_t row_count, uint8_t *tiles, cudaStream_t stream);
cudaError_t launch_unpack_q8(WeightView w, uint8_t *codes, float *w32, __half *w16, cudaStream_t stream);
// rows[i] (device, numbered in the whole matrix; row_base = first row this shard holds) dequantised into
// out[i][K] fp16 or fp32; rows the shard does not hold give zeros
cudaError_t launch_lookup_rows(WeightView w, const uint32_t *rows, uint32_t count, uint32_t row_base, void *out,
                               int out_dtype, cudaStream_t stream);
// y[m][slot] = sum_k w(ids[slot], k) x[m][k] for the listed rows (device ids, numbered in the whole matrix) that
// this shard holds; m_rows <= 16
cudaError_t launch_matmul_rows(WeightView w, const uint32_t *ids, uint32_t count, uint32_t row_base, const void *x,
                               int x_dtype, uint32_t m_rows, void *y, int y_dtype, uint32_t ldy, cudaStream_t stream);
// output[b][i] = half(input[b][i] * inv_rms(b) * weight[i]), input fp16 or fp32 [batch][hidden], one block per row
cudaError_t launch_rmsnorm(const void *input, int input_dtype, const float *weight, void *output, uint32_t hidden,
                           uint32_t batch, float epsilon, cudaStream_t stream);
cudaError_t launch_synth_codes(uint64_t seed, uint64_t stream_id, uint32_t *words,
                               uint64_t word_begin, uint64_t word_count, cudaStream_t stream);
cudaError_t launch_synth_meta(uint64_t seed, uint64_t stream_id, __half *meta,
                              uint64_t group_begin, uint64_t group_count, cudaStream_t stream);
cudaError_t launch_synth_x(uint64_t seed, uint64_t stream_id, __half *x, uint64_t begin,
                           uint64_t count, cudaStream_t stream);

// ---- q4b_decode.cu: decode GEMV / small-M GEMM, one projection per launch or a whole pass in one launch ----
constexpr int kMaxSegments = 4;
constexpr int kMaxPeers = 8;
constexpr uint32_t kDoneStride = 32;  // words between the completion sub-counters of a sequence (one L2 line each)

// One projection as the decode kernel reads it (a kernel argument for a single launch, a row of the job table
// in device memory for a sequence): up to kMaxSegments matrices that share x (same K), or a fused gate/up
// pair (segment 0 = gate) with the SiLU-gate epilogue.
struct DecodeJob {
    const uint8_t *tiles[kMaxSegments];
    const uint8_t *up_tiles;           // fused gate/up: the second matrix
    void *y[kMaxSegments][kMaxPeers];  // where segment s goes on rank r (own rank included), column offset applied;
                                       // a single launch uses rank 0 only
    const void *x;                     // [M][K] fp16 or fp32
    const void *residual;              // [M][ld_residual] or null; added to segment 0 only
    uint32_t rows[kMaxSegments];
    uint32_t ldy[kMaxSegments];
    uint32_t pair_begin[kMaxSegments + 1];  // prefix sums of pair blocks (128 rows; 64 gate + 64 up rows when fused)
    uint32_t groups, segments, fused;
    int x_dtype, y_dtype, residual_dtype;
    uint32_t ld_residual;
    uint32_t parts, units;             // K parts per pair block; units = pair blocks x parts
    uint32_t expected_blocks;          // 64-row blocks all ranks publish for this job per launch (sequences)
};
// what depends on M, the variant and the device only
struct DecodeGeometry {
    int mode;            // 0 integer form (M <= 4), 1 fp16 form M <= 8, 2 fp16 form M <= 16
    uint32_t ctas;       // CTAs that are resident at once (the grid of a sequence; the limit of a single launch)
    uint32_t plan_ctas;  // the grid the K split is planned for (two CTAs per SM)
    uint32_t threads;
    uint32_t max_parts;  // 0: no limit on the K parts of a pair block
    uint32_t stages;     // stages of the weight ring (3 when two CTAs then still share an SM, else 2)
    size_t smem_bytes;
    uint32_t cluster_room[9];  // [k]: clusters of k CTAs of this form the device holds at once (k = 2..8; 0 = none)
    uint32_t plan_room[9];     // the same for the integer form at M = 1: what the K split is planned around
};
struct SequenceLaunch {
    const DecodeJob *jobs;     // device
    uint32_t job_count, m_rows, world;
    DecodeGeometry geometry;
    uint32_t *epoch;           // device word, zeroed once: launches completed
    uint32_t *exit_count;      // device word, zero between launches
    uint32_t *done;            // device, [job_count][8] x kDoneStride words, zeroed once; counts up across launches
    uint32_t *peer_done[kMaxPeers];
    float *scratch;
    uint32_t *counters;
    uint32_t *status;
    unsigned long long *profile;  // null, or device [ctas][kProfileSlots]: SM clocks by phase, added up per launch
};
constexpr int kProfileSlots = 6;  // dependency wait, entries, weight wait, tiles, finish, total
// a projection as the entry points of the C ABI describe it, before it is routed to a kernel by M
struct ProjectionArgs {
    // up to kMaxSegments matrices that share x (same K); fused gate/up uses
    // segment 0 = gate, `up` = the second matrix, one output
    WeightView w[kMaxSegments];
    void *y[kMaxSegments];
    uint32_t ldy[kMaxSegments];
    int segments;
    WeightView up;       // valid when fused_silu
    int fused_silu;
    const void *x;       // [M][K]
    int x_dtype;         // kF16 / kF32 / kBF16
    uint32_t m_rows;
    int y_dtype;
    const void *residual;  // [M][ld_residual] or null (segment 0 only)
    int residual_dtype;
    uint32_t ld_residual;
};
uint32_t decode_max_m();
// variant: 0 = default; other values select alternatives for A/B measurements (see q4b_decode.cu)
cudaError_t decode_geometry(uint32_t m_rows, int variant, int sm_count, bool sequence, DecodeGeometry *geometry);
// fills pair_begin, parts and units of `job`; returns the split-K scratch it needs (0 when K is not split)
void plan_decode_job(DecodeJob *job, uint32_t m_rows, const DecodeGeometry &geometry, size_t *scratch_bytes,
                     size_t *counter_bytes);
cudaError_t launch_decode(const DecodeJob &job, uint32_t m_rows, uint32_t world, const DecodeGeometry &geometry, int variant,
                          float *scratch, uint32_t *counters, uint32_t *status, cudaStream_t stream);
cudaError_t launch_sequence(const SequenceLaunch &launch, cudaStream_t stream);
// device addresses and sizes of the library's built-in (never allocated) scratch on the current device
cudaError_t decode_static_scratch(float **scratch, uint32_t **counters, size_t *scratch_bytes,
                                  size_t *counter_bytes);

// ---- q4b_gemm.cu: tcgen05 prefill GEMM ----
struct TcGemmArgs {
    WeightView w[kMaxSegments];  // matrices that share x (same K), one launch
    void *y[kMaxSegments];       // [M][ldy]
    uint32_t ldy[kMaxSegments];
    int segments;
    WeightView up;        // valid when fused_silu (single segment)
    int fused_silu;
    const void *x;        // [M][K] fp16 (bf16 when x_bf16), 16-byte aligned
    int x_bf16;           // bf16 activations against weights rounded to bf16
    uint32_t m_rows;
    int y_dtype;
    const void *residual; // [M][ld_residual] or null
    int residual_dtype;
    uint32_t ld_residual;
    uint32_t *status;
    // column-parallel ranks: where the same output block lives in the other ranks' memory (entries may be null)
    void *peer_y[kMaxSegments][kMaxPeers];
    uint32_t peers;
    // optional, for splitting tiles over CTAs when there are few: sm_count x 128 x 256 floats and sm_count
    // zero-initialised flags (left zero by every launch)
    float *workspace;
    size_t workspace_bytes;
    uint32_t *flags;
};
cudaError_t launch_tc_gemm(const TcGemmArgs &args, int sm_count, cudaStream_t stream);
cudaError_t launch_convert_f32_to_f16(const float *in, __half *out, size_t count, cudaStream_t stream);
// One thread: after the launches before it are complete, a system-scope fence, 1 added to every rank's counter,
// and a bounded wait until the own counter shows world x (the round, counted in *round) arrivals; a wait that
// expires stores a code in *status.  A programmatic dependent of its predecessor, and its successor of it.
cudaError_t launch_rank_barrier(uint32_t *const *counters, uint32_t world, uint32_t rank, uint32_t *round,
                                uint32_t *status, cudaStream_t stream);

// ---- q4b_api.cu: what the other host files need to know of a context ----
int context_device(const q4b_context *context);
void context_count_launch(q4b_context *context);  // one more kernel of this library queued (not while recording)

// ---- q4b_probe.cu ----
cudaError_t launch_probe_signal(uint32_t *own_flag, uint32_t *peer_flag, uint32_t *peer_payload, uint32_t payload_words,
                                uint32_t rounds, uint32_t base, int initiator, int mode, uint32_t *status,
                                cudaStream_t stream);
cudaError_t launch_probe(int mode, const uint8_t *data, size_t bytes, int ctas, uint32_t stages, uint32_t stage_bytes,
                         uint32_t *sink, cudaStream_t stream);

}  // namespace q4b
