// Host-side launchers of the CUDA kernels (internal to the library).
#pragma once
#include "q4b_common.cuh"

namespace q4b {

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
// rows[i] (device, numbered in the whole matrix; row_base = first row this shard holds) dequantised into
// out[i][K] fp16 or fp32; rows the shard does not hold give zeros
cudaError_t launch_lookup_rows(WeightView w, const uint32_t *rows, uint32_t count, uint32_t row_base, void *out,
                               int out_dtype, cudaStream_t stream);
// output[b][i] = half(input[b][i] * inv_rms(b) * weight[i]), input fp16 or fp32 [batch][hidden], one block per row
cudaError_t launch_rmsnorm(const void *input, int input_dtype, const float *weight, void *output, uint32_t hidden,
                           uint32_t batch, float epsilon, cudaStream_t stream);
cudaError_t launch_synth_codes(uint64_t seed, uint64_t stream_id, uint32_t *words,
                               uint64_t word_begin, uint64_t word_count, cudaStream_t stream);
cudaError_t launch_synth_meta(uint64_t seed, uint64_t stream_id, __half *meta,
                              uint64_t group_begin, uint64_t group_count, cudaStream_t stream);
cudaError_t launch_synth_x(uint64_t seed, uint64_t stream_id, __half *x, uint64_t begin,
                           uint64_t count, cudaStream_t stream);

// ---- q4b_gemv.cu ----
constexpr int kMaxSegments = 4;
constexpr int kMaxPeers = 8;
struct GemvArgs {
    // up to kMaxSegments matrices that share x (same K); fused gate/up uses
    // segment 0 = gate, `up` = the second matrix, one output
    WeightView w[kMaxSegments];
    void *y[kMaxSegments];
    uint32_t ldy[kMaxSegments];
    int segments;
    WeightView up;       // valid when fused_silu
    int fused_silu;
    const void *x;       // [M][K]
    int x_dtype;         // kF16 / kF32
    uint32_t m_rows;
    int y_dtype;         // kF16 / kF32
    const void *residual;  // [M][ld_residual] or null (segment 0 only)
    int residual_dtype;
    uint32_t ld_residual;
    uint32_t *status;      // device-visible word that receives a code when a wait expires
    float *scratch;        // global partial-sum slots (plan.scratch_bytes)
    uint32_t *counters;    // zero-initialised, self-resetting (plan.counter_bytes)
};
// launch geometry and the scratch a launch needs, derived from the shapes alone
struct GemvPlan {
    uint32_t ctas, threads, stages, stage_units, total_units, blocks;
    uint32_t local_blocks, slots, parts;
    size_t smem_bytes, scratch_bytes, counter_bytes;
};
// variant: 0 = default; other values select alternatives for A/B measurements
cudaError_t plan_gemv(const GemvArgs &args, int variant, int sm_count, GemvPlan *plan);
cudaError_t launch_gemv(const GemvArgs &args, const GemvPlan &plan, int variant, cudaStream_t stream);
uint32_t gemv_max_m();
// device addresses and sizes of the library's built-in (never allocated) scratch on the current device
cudaError_t gemv_static_scratch(float **scratch, uint32_t **counters, size_t *scratch_bytes,
                                size_t *counter_bytes);

// ---- q4b_decode.cu: job sequences in one persistent launch ----
// One projection (a group of matrices sharing x, or a fused gate/up pair) as the
// sequence kernel reads it from device memory.
struct DecodeJob {
    const uint8_t *tiles[kMaxSegments];
    const uint8_t *up_tiles;
    void *y[kMaxSegments][kMaxPeers];  // where segment s goes on rank r (own rank included), column offset applied
    const void *x;                     // [M][K] fp16
    uint32_t rows[kMaxSegments];
    uint32_t ldy[kMaxSegments];
    uint32_t block_begin[kMaxSegments + 1];
    uint32_t groups, segments, fused, y_dtype;
    uint32_t total_units, units_per_cta, units_extra, parts, active_ctas, slots, local_blocks;
    uint32_t expected_blocks;  // row blocks all ranks publish for this job per launch (0: blocks * world)
};
struct SequenceLaunch {
    const DecodeJob *jobs;     // device
    uint32_t job_count, m_rows, stages, ctas, max_local_blocks;
    uint32_t world, rank, epoch;
    uint32_t *done;            // device, [job_count], zeroed once; counts up across launches
    uint32_t *peer_done[kMaxPeers];
    float *scratch;
    uint32_t *counters;
    uint32_t *status;
    size_t smem_bytes;
};
// fills the partition fields of `job` for a grid of `ctas`; returns scratch needs
void plan_decode_job(DecodeJob *job, uint32_t m_rows, uint32_t ctas, size_t *scratch_bytes, size_t *counter_bytes);
// grid size and shared memory of the sequence kernel on the current device
cudaError_t sequence_geometry(uint32_t m_rows, int sm_count, uint32_t stages, uint32_t max_local_blocks,
                              uint32_t *ctas, size_t *smem_bytes);
cudaError_t launch_sequence(const SequenceLaunch &launch, cudaStream_t stream);

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
// One thread: system-scope fence, add 1 to every rank's counter, wait (bounded) until the own counter shows
// `expected` arrivals; a wait that expires stores a code in *status.
cudaError_t launch_rank_barrier(uint32_t *const *counters, uint32_t world, uint32_t rank, uint32_t expected,
                                uint32_t *status, cudaStream_t stream);

// ---- q4b_probe.cu ----
cudaError_t launch_probe(int mode, const uint8_t *data, size_t bytes, int ctas, uint32_t stages, uint32_t stage_bytes,
                         uint32_t *sink, cudaStream_t stream);

}  // namespace q4b
