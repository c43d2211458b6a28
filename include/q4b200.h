/*
 * libq4b200 -- affine-Q4 matmul for NVIDIA B200 (sm_100a), C ABI.
 *
 * Drop-in device side of llm-in-c's Q4 hot path: w = scale*q + bias, uint4 codes
 * packed 8 per uint32 along K, one fp16 {scale, bias} record per 64-column group
 * (the reference's packed-image segments, models/qwen3.8-27b/targets/apple-m3-pro/
 * qwen38_m3_image.h:26-94, qwen38_q4.metal:10-37).  The library has no Python or
 * PyTorch dependency; it links only the CUDA runtime.
 *
 * Conventions follow the reference runtime (qwen38_m3_decode.h:20-25):
 *   - every call returns int: 0 ok, 1 bad argument or state, 2 device failure,
 *     3 image / load failure; on failure a NUL-terminated message is written to
 *     the caller's buffer (which may be NULL / 0);
 *   - handles are opaque; the library owns device memory, the caller owns host
 *     memory (host pointers passed to an upload may be freed on return);
 *   - one stream per context, one thread per context at a time; work is queued
 *     asynchronously on the context's stream unless the call is named *_host or
 *     documented as synchronous.
 */
#ifndef Q4B200_H
#define Q4B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct q4b_context q4b_context;
typedef struct q4b_weight q4b_weight;
typedef struct q4b_graph q4b_graph;
typedef struct q4b_sequence q4b_sequence;

enum { Q4B_OK = 0, Q4B_BAD_ARGUMENT = 1, Q4B_DEVICE_FAILURE = 2, Q4B_LOAD_FAILURE = 3 };
enum { Q4B_F16 = 0, Q4B_F32 = 1, Q4B_BF16 = 2, Q4B_NONE = -1 };

/* ---- context: replaces qwen38_m3_model_open / _close for this path
 * (qwen38_m3_decode.h:27-49, qwen38_m3_decode.m:1487).  NULL + message on
 * failure.  Fails loudly when no sm_100 device is present: there is no CPU
 * fallback. */
q4b_context *q4b_context_open(int device, char *error_message, size_t error_capacity);
void q4b_context_close(q4b_context *context);
int q4b_device_count(void);
/* cudaStream_t of the context, for callers that queue their own work */
void *q4b_context_stream(q4b_context *context);
/* Selects a kernel variant for A/B measurements (0 = library heuristics); the
 * counterpart of QWEN38_PREFILL_MMA / QWEN38_VERIFY_MMA (qwen38_m3_decode.m:
 * 1547-1555, :2757).  The environment variable Q4B_VARIANT sets the default. */
void q4b_context_set_variant(q4b_context *context, int variant);
/* number of kernels this context has launched since it was opened */
uint64_t q4b_context_launch_count(const q4b_context *context);

/* ---- plain device memory, for hosts without another CUDA allocator ---- */
int q4b_alloc(q4b_context *context, size_t bytes, void **device_pointer,
              char *error_message, size_t error_capacity);
int q4b_free(q4b_context *context, void *device_pointer);
int q4b_alloc_host(q4b_context *context, size_t bytes, void **pinned_host_pointer,
                   char *error_message, size_t error_capacity);
int q4b_free_host(q4b_context *context, void *pinned_host_pointer);
/* asynchronous on the context stream */
int q4b_copy_to_device(q4b_context *context, void *device_destination, const void *host_source,
                       size_t bytes, char *error_message, size_t error_capacity);
int q4b_copy_to_host(q4b_context *context, void *host_destination, const void *device_source,
                     size_t bytes, char *error_message, size_t error_capacity);
/* device to device, `rows` rows of `row_bytes` bytes with the given pitches (cudaMemcpy2DAsync on the stream) */
int q4b_copy_2d(q4b_context *context, void *destination, size_t destination_pitch, const void *source,
                size_t source_pitch, size_t row_bytes, size_t rows, char *error_message, size_t error_capacity);

/* ---- weight-image loader: replaces mapped_buffer / load_*_layer
 * (qwen38_m3_decode.m:398-407, :500-625).  Takes the two image segments of one
 * matrix exactly as the reference packer wrote them (quants = MLX U32 [rows,
 * K/8] bytes, PACK qwen38_m3_pack.c:395-418; meta = [rows, K/64] {fp16 scale,
 * fp16 bias}, :420-446), repacks rows [row_begin, row_begin+row_count) -- the
 * N-slice this GPU owns -- into the device tile stream and uploads them.
 * Synchronous.  Rejects K % 64 != 0, NULL segments and empty slices. */
int q4b_weight_upload(q4b_context *context, const void *quants, const void *meta,
                      uint32_t rows, uint32_t groups_per_row, uint32_t row_begin,
                      uint32_t row_count, q4b_weight **weight,
                      char *error_message, size_t error_capacity);
/* Same, from separate scale and bias planes in fp16 or bf16 -- the un-converted
 * MLX metadata that minimax_h3_q4_projection carries (compiler/minimax-h3/
 * apple-m3-pro/minimax_h3_q4_layer.h:14-24); bf16 is converted like the packer
 * does (qwen38_m3_pack.c:173-178): bf16 -> fp32 -> fp16, round to nearest even.
 * The device holds fp16 records, so the reference kernel that reads bf16 planes
 * as they are (minimax_h3_q4_gemm_bf16_meta, minimax_h3_attention.metal:416-506,
 * dequantising in fp32) is matched exactly where every scale and bias is an fp16
 * number -- every bf16 value with 2^-14 <= |v| <= 65504 is -- and not otherwise:
 * smaller magnitudes lose bits or become zero, larger ones become infinite.
 * q4b_planes_narrowed counts the values of a plane pair that would change (host
 * only, no GPU needed): 0 means the upload is exact. */
uint64_t q4b_planes_narrowed(const void *scales, const void *biases, int meta_dtype, uint64_t values_per_plane);
int q4b_weight_upload_planes(q4b_context *context, const void *quants, const void *scales,
                             const void *biases, int meta_dtype, uint32_t rows,
                             uint32_t groups_per_row, uint32_t row_begin, uint32_t row_count,
                             q4b_weight **weight, char *error_message, size_t error_capacity);
/* Same as q4b_weight_upload with the two segments already in device memory. */
int q4b_weight_from_device(q4b_context *context, const void *device_quants,
                           const void *device_meta, uint32_t rows, uint32_t groups_per_row,
                           uint32_t row_begin, uint32_t row_count, q4b_weight **weight,
                           char *error_message, size_t error_capacity);
/* Seeded synthetic matrix generated on the device in the image layout and then
 * loaded like any other (the role of fill_weights, qwen38_m3.m:64-87).  The same
 * counter-based generator exists in C for the CPU checker. */
int q4b_weight_synth(q4b_context *context, uint64_t seed, uint32_t projection, uint32_t rows,
                     uint32_t groups_per_row, uint32_t row_begin, uint32_t row_count,
                     q4b_weight **weight, char *error_message, size_t error_capacity);
int q4b_synth_x(q4b_context *context, uint64_t seed, uint64_t stream_id, void *device_x_f16,
                uint64_t begin, uint64_t count, char *error_message, size_t error_capacity);
void q4b_weight_free(q4b_context *context, q4b_weight *weight);
int q4b_weight_info(const q4b_weight *weight, uint32_t *rows, uint32_t *groups_per_row,
                    uint64_t *device_bytes);
/* Embedding lookup: replaces qwen38_q4_embedding_lookup (qwen38_global.metal:13-28).
 * out[i][k] = scale * (float)q + bias of row rows[i] (rounded to fp16 when out_dtype
 * is fp16, as the reference does), i < count.  rows (DEVICE memory) are numbered in
 * the whole matrix; a shard (row slice) writes zeros for rows it does not hold, so
 * the shards of a split vocabulary add up.  Asynchronous. */
int q4b_embedding_lookup(q4b_context *context, const q4b_weight *embedding, const uint32_t *rows,
                         uint32_t count, void *out, int out_dtype,
                         char *error_message, size_t error_capacity);

/* ---- the step before a layer's matmuls: RMS norm of the hidden state into the fp16 x
 * that the in-projections and the MLP read.  Replaces qwen38_rmsnorm_f16_to_f16 and
 * qwen38_rmsnorm_f32_to_f16 (qwen38_layer.metal:21-69) and their batched forms:
 * output[b][i] = half(input[b][i] * inv_rms(b) * weight[i]) with
 * inv_rms = 1 / sqrt(mean(input[b]^2) + epsilon), in the reference's order of
 * operations (256 strided partial sums, a halving tree, two fp32 products), every
 * operation rounded on its own.  input is [batch_rows][hidden] fp16 or fp32, weight
 * fp32 [hidden] (the layer image's constants hold it), output fp16; DEVICE pointers;
 * asynchronous on the context's stream.  The reference's epsilon is 1e-6. */
int q4b_rmsnorm(q4b_context *context, const void *input, int input_dtype, const float *weight, void *output_f16,
                uint32_t hidden, uint32_t batch_rows, float epsilon, char *error_message, size_t error_capacity);
/* The affine-Q8 sibling (minimax_h3_q8_gemm_bf16_meta, minimax_h3_attention.metal:594-676; host
 * minimax_h3_m3_run_q8_gemm_benchmark, minimax_h3_m3_gemm.m:387-): one code BYTE per weight, 64 per group
 * (quants [rows][K] bytes), bf16 scales and biases [rows][K/64], w = half(float(scale) * q + float(bias)).
 * The metadata stay bf16 on the device, as that kernel reads them.  A Q8 weight is served by q4b_matmul (and
 * q4b_matmul_host) alone, on the tcgen05 GEMM at every M, with fp16 or fp32 activations; q4b_weight_unpack
 * returns its codes and dequantised values; the other entry points refuse it with status 1. */
int q4b_weight_upload_q8(q4b_context *context, const void *quants, const void *scales_bf16, const void *biases_bf16,
                         uint32_t rows, uint32_t groups_per_row, uint32_t row_begin, uint32_t row_count,
                         q4b_weight **weight, char *error_message, size_t error_capacity);
/* Dequantisation in isolation (the job of qwen38_q4_embedding_lookup,
 * qwen38_global.metal:13-28) over the whole shard, written to HOST buffers, any
 * of which may be NULL: codes uint8 [rows][K], w32 float [rows][K] =
 * scale*(float)q+bias, w16 fp16 bits [rows][K] = the value the tensor-core GEMM
 * multiplies.  Synchronous. */
int q4b_weight_unpack(q4b_context *context, const q4b_weight *weight, uint8_t *codes,
                      float *w32, uint16_t *w16, char *error_message, size_t error_capacity);

/* ---- matmul: replaces the decode row kernels and encode_prefill_gemm_f16 /
 * encode_prefill_gemm_residual (qwen38_m3_decode.m:639-660, :885-1001).
 * y[m][n] = sum_k w(n,k) x[m][k] (+ residual[m][n]), fp32 accumulation.
 * x is [M][K] row-major fp16 or fp32, y is [M][ldy] fp16 or fp32 (ldy >= rows
 * of the shard lets a shard write its column slice of a wider matrix),
 * residual is [M][ld_residual] fp16 or fp32 or NULL.  DEVICE pointers, 16-byte
 * aligned; asynchronous.  The kernel is chosen by M: the decode kernel for
 * M <= 16, the tcgen05 GEMM above.
 *
 * How the decode kernel takes x.  At M <= 4 it multiplies on the integer tensor
 * pipe: every 64-column group of an activation row becomes two signed 8-bit
 * digits per value with one power-of-two step for the group (15 bits relative to
 * the group's largest |x|; fp16 itself carries 11 per value), the sums of
 * code x digit are exact integers, and scale, step and bias are applied per group
 * in fp32.  Measured max|y - ref| / max|ref| = 3e-5 .. 8e-5 on fp32 outputs, far
 * inside 2e-3 (an fp16 output rounds at 5e-4).  At M = 5..16 the codes meet x as
 * fp16 on the tensor pipe with fp32 accumulation (1e-6 on fp32 outputs).  Either
 * way a row's result does not depend on M (within the same form) or on the other
 * rows, nor on timing.  Bit 4 of q4b_context_set_variant (or Q4B_VARIANT) keeps
 * the fp16 form at M <= 4 too.
 * fp32 x (the reference's second projections multiply in fp32,
 * qwen38_m3_layer.m:375-393) is not narrowed to fp16's range: each group is
 * scaled by the power of two of its largest magnitude before it is cut into
 * digits (M <= 4) or rounded to fp16 (M = 5..16: 11 bits per value relative to
 * the value itself), so magnitudes up to 2^100 are served with the same relative
 * accuracy.  The tensor-core GEMM (M > 16) does round fp32 x to fp16 as it is:
 * there |x| above 65504 overflows.
 * A group that holds an infinity or a NaN (or, for fp32 x, a magnitude of 2^100
 * or more) makes every output of that activation row NaN.
 *
 * bf16 activations (x_dtype = Q4B_BF16) select the arithmetic of the H3
 * projections (minimax_h3_q4_gemm_bf16_activation, minimax_h3_attention.metal:
 * 512-592; CPU check benchmarks/minimax_h3_m3_real_gemm.c:25-42): every weight
 * is rounded to bf16, w = bf16(scale * q + bias), multiplied with bf16 x on the
 * tensor cores and summed in fp32 over the whole of K; y and the residual are
 * then bf16 or fp32.  The tcgen05 GEMM serves this at every M.  Meant for
 * weights uploaded from bf16 planes (q4b_weight_upload_planes with Q4B_BF16):
 * scale and bias are taken from the fp16 records and rounded to bf16, which
 * gives the plane's own values back wherever they lie in fp16's normal range.
 * Sequences, q4b_matmul_no_alloc and mixed pairs (fp16/fp32 x with bf16 y, bf16
 * x with fp16 y) are refused with status 1. */
int q4b_matmul(q4b_context *context, const q4b_weight *weight, const void *x, int x_dtype,
               uint32_t m_rows, void *y, int y_dtype, uint32_t ldy, const void *residual,
               int residual_dtype, uint32_t ld_residual,
               char *error_message, size_t error_capacity);
/* The same product for callers that must not allocate.  (This entry point has no
 * counterpart in the reference; it exists for hosts built around this library.)
 *
 * q4b_matmul keeps a scratch buffer for row blocks whose K range is split over
 * several thread blocks, and grows it with cudaMalloc the first time a shape
 * needs more.  That is wrong for a caller that has handed all device memory to
 * its own pool, that runs where an implicit device-wide synchronisation (which
 * cudaMalloc and cudaFree cause) would stall other streams mid-token, or that
 * must give the same latency on the first token as on the thousandth.  This
 * variant runs the same kernel with its scratch in an array that is part of the
 * library image itself: 1 MiB of partial sums plus 4096 arrival counters, held
 * by every GPU that loads the library until the process exits.  It calls no
 * cudaMalloc, cudaFree or other allocating routine.
 *
 * Limits and rules:
 *   - only a matrix with fewer 128-row blocks than the GPU runs thread blocks at
 *     once (296 on a B200, i.e. up to about 37,000 rows) has its K range split and
 *     uses the scratch at all; larger matrices (the 248,320-row lm_head among
 *     them) need none and are served as they are.  A split matrix needs at most
 *     2 KB (M <= 4), 4 KB (M <= 8) or 8 KB (M <= 16) per resident thread block:
 *     everything at M <= 4 -- decode and the verify step -- fits on a B200 (at
 *     most 0.6 MB); at M = 5..16 a matrix cut into more than 256 (M <= 8) or 128
 *     pieces (17408 -> 5120 is cut into 240 or 280, which M = 16 cannot park) is
 *     refused with status 1 and a message that states both sizes: use q4b_matmul
 *     for it;
 *   - no residual input; otherwise the arguments of q4b_matmul;
 *   - the first call on a device looks the array's device address up (once per
 *     device); make that first call before any stream capture begins;
 *   - every call on a device shares the one array and finds what the last call
 *     left in it: the call clears its counters itself, but two calls whose
 *     kernels overlap on the GPU (two contexts, two streams) race on it -- keep
 *     calls to this entry point on one stream per device. */
int q4b_matmul_no_alloc(q4b_context *context, const q4b_weight *weight, const void *x, int x_dtype,
                        uint32_t m_rows, void *y, int y_dtype, uint32_t ldy,
                        char *error_message, size_t error_capacity);
/* The restricted head of the draft passes (qwen38_m3_decode.m:1847-1866): the first
 * `draft_vocab` rows of the lm_head as an ordinary matmul, then the listed extra
 * rows after them.
 * q4b_weight_rows: a handle on rows [row_begin, row_begin + row_count) of a loaded
 * weight, without a copy (row_begin a multiple of 128); usable wherever a weight
 * is, freed with q4b_weight_free before the weight it was taken from.
 * q4b_matmul_rows replaces qwen38_q4_lm_head_gathered (qwen38_global.metal:68-96):
 * y[m][slot] = sum_k w(row_ids[slot], k) x[m][k] for `count` row ids in DEVICE
 * memory, numbered in the whole matrix; 1 <= m_rows <= 16; w = scale * q + bias in
 * fp32 as there.  The reference writes logits[base + slot]: pass y + base.  Ids of
 * rows another rank's shard holds leave their slot untouched. */
int q4b_weight_rows(const q4b_weight *weight, uint32_t row_begin, uint32_t row_count, q4b_weight **rows,
                    char *error_message, size_t error_capacity);
int q4b_matmul_rows(q4b_context *context, const q4b_weight *weight, const uint32_t *row_ids, uint32_t count,
                    const void *x, int x_dtype, uint32_t m_rows, void *y, int y_dtype, uint32_t ldy,
                    char *error_message, size_t error_capacity);
/* Up to 4 matrices that share x in one launch, e.g. q/k/v, which the reference
 * fuses into one matrix (qwen38_attention.metal:4-8). */
int q4b_matmul_group(q4b_context *context, const q4b_weight *const *weights, int count,
                     const void *x, int x_dtype, uint32_t m_rows, void *const *y, int y_dtype,
                     const uint32_t *ldy, char *error_message, size_t error_capacity);
/* Fused gate/up with SiLU-gate epilogue: out = silu(gate x) * (up x), replaces
 * qwen38_q4_gate_up_silu (qwen38_q4.metal:129-151, qwen38_m3_decode.m:643-651)
 * and the prefill pair + qwen38_prefill_silu_mul (:1019-1033).
 * Activations are taken as q4b_matmul takes them (integer form at M <= 4). */
int q4b_gate_up_silu(q4b_context *context, const q4b_weight *gate, const q4b_weight *up,
                     const void *x, int x_dtype, uint32_t m_rows, void *y, int y_dtype,
                     uint32_t ldy, char *error_message, size_t error_capacity);

/* ---- operator-level calls with HOST buffers: the shape of
 * minimax_h3_m3_run_q4_projection_bf16 (minimax_h3_m3_gemm.h:57-66): copy in,
 * run, copy out, report device milliseconds of the kernel.  Synchronous. */
int q4b_matmul_host(q4b_context *context, const q4b_weight *weight, const void *x_host,
                    int x_dtype, uint32_t m_rows, void *y_host, int y_dtype, double *gpu_ms,
                    char *error_message, size_t error_capacity);
int q4b_gate_up_silu_host(q4b_context *context, const q4b_weight *gate, const q4b_weight *up,
                          const void *x_host, int x_dtype, uint32_t m_rows, void *y_host,
                          int y_dtype, double *gpu_ms, char *error_message,
                          size_t error_capacity);

/* ---- completion and timing: replaces qwen38_m3_model_forward_wait
 * (qwen38_m3_decode.h:77-92).  q4b_timer_start records an event on the stream;
 * q4b_sync waits for all queued work, surfaces asynchronous errors as a nonzero
 * status and, when device_ms is not NULL, returns the device time since the
 * last q4b_timer_start. */
int q4b_timer_start(q4b_context *context, char *error_message, size_t error_capacity);
int q4b_sync(q4b_context *context, double *device_ms, char *error_message, size_t error_capacity);

/* ---- decode sequences: one token's chain of projections in ONE launch.
 * The reference encodes a whole token into one command buffer
 * (qwen38_m3_model_forward_submit, qwen38_m3_decode.m:1614-1690: per layer
 * encode_delta / encode_attention / encode_mlp back to back).  A sequence is the
 * same idea for the Q4 matmuls: jobs are added in execution order, each either a
 * group of 1..4 matrices that share x (q4b_matmul_group) or a fused gate/up pair
 * (q4b_gate_up_silu); job j may read what job j-1 wrote (the kernel treats
 * every job as depending on the one before it; the next job's weights are
 * already streaming while it waits).  All pointers are DEVICE pointers,
 * 1 <= m_rows <= 16; q4b_sequence_add_matmul and _add_gate_up take fp16 x,
 * q4b_sequence_add_projection one matrix with fp16 or fp32 x and an optional
 * residual (the second projections, qwen38_layer.metal:193-255).
 * q4b_sequence_finalize plans the work split and allocates the sequence's own
 * scratch (synchronous, never while recording); q4b_sequence_launch queues one
 * cooperative kernel on the context's stream.  The count of launches lives in
 * device memory and advances when a launch ends, so a launch recorded into a
 * graph (q4b_graph_begin) replays correctly.
 *
 * Column-parallel ranks (one process per GPU): create with (world, rank), give
 * every job the slice this rank owns, and with q4b_sequence_set_peer_output name
 * where that slice goes in each peer's copy of y (a pointer obtained with
 * q4b_ipc_open, column offset applied).  After finalize exchange
 * q4b_sequence_done_counters between the ranks (q4b_ipc_export / q4b_ipc_open)
 * and install them with q4b_sequence_set_peer_counters.  The kernel then stores
 * every output on every rank and a job starts only when all ranks have published
 * the previous one: the all-gather is part of the launch.  All ranks must launch
 * the same sequence the same number of times. */
int q4b_sequence_create(q4b_context *context, uint32_t m_rows, uint32_t world, uint32_t rank,
                        q4b_sequence **sequence, char *error_message, size_t error_capacity);
int q4b_sequence_add_matmul(q4b_sequence *sequence, const q4b_weight *const *weights, int count,
                            const void *x, void *const *y, const uint32_t *ldy, int y_dtype,
                            char *error_message, size_t error_capacity);
int q4b_sequence_add_gate_up(q4b_sequence *sequence, const q4b_weight *gate, const q4b_weight *up,
                             const void *x, void *y, uint32_t ldy, int y_dtype,
                             char *error_message, size_t error_capacity);
int q4b_sequence_add_projection(q4b_sequence *sequence, const q4b_weight *weight, const void *x, int x_dtype,
                                void *y, int y_dtype, uint32_t ldy, const void *residual, int residual_dtype,
                                uint32_t ld_residual, char *error_message, size_t error_capacity);
int q4b_sequence_set_peer_output(q4b_sequence *sequence, uint32_t job, uint32_t segment,
                                 uint32_t peer_rank, void *peer_y);
/* Ranks whose slices differ in size: the number of 64-row blocks (summed over the
 * job's matrices, each rounded up) that ALL ranks together compute for `job`;
 * the next job starts when that many have been published.  Default: this rank's
 * own count times world (equal slices). */
int q4b_sequence_set_job_blocks(q4b_sequence *sequence, uint32_t job, uint32_t blocks_on_all_ranks);
int q4b_sequence_finalize(q4b_context *context, q4b_sequence *sequence,
                          char *error_message, size_t error_capacity);
void *q4b_sequence_done_counters(q4b_sequence *sequence);
int q4b_sequence_set_peer_counters(q4b_sequence *sequence, uint32_t peer_rank, void *peer_counters);
int q4b_sequence_launch(q4b_context *context, q4b_sequence *sequence,
                        char *error_message, size_t error_capacity);
/* Where a sequence's time goes (the role of QWEN38_PROFILE, qwen38_m3_decode.m:1217-1283, which splits the
 * command buffer by region).  The first call switches the clocks on (one allocation); every later call waits
 * for the stream, copies out what the launches since the last call added up and clears it.  clocks receives,
 * per resident thread block, six sums of SM clock ticks as one of its consumer warps saw them: waiting for the
 * previous job's outputs; turning activations into tensor-pipe operands; waiting for weights to arrive from
 * HBM; multiplying; finishing units (split sums, epilogue, publishing); and the whole launch.  capacity is in
 * values (thread_blocks x 6 are needed; *thread_blocks is always set).  Synchronous; not while recording. */
int q4b_sequence_profile(q4b_context *context, q4b_sequence *sequence, uint64_t *clocks, uint32_t capacity,
                         uint32_t *thread_blocks, char *error_message, size_t error_capacity);
void q4b_sequence_free(q4b_context *context, q4b_sequence *sequence);

/* ---- column-parallel ranks, one launch per projection: the kernel stores a
 * rank's slice straight into every rank's copy of the output, and a one-thread
 * barrier kernel per gather point replaces the all-gather (the reference has one
 * GPU; this is the NCCL all-gather of the slices done by the producing kernel).
 * Works at every M: the tensor-core GEMM above M = 16, the decode kernel up to it
 * (where a sequence, above, is the other way to share outputs).
 *
 * q4b_context_push_outputs: for the NEXT q4b_matmul / q4b_matmul_group /
 * q4b_gate_up_silu call, name where its output block(s) live in the other ranks'
 * memory: peer_y[s * world + r] is segment s's block on rank r, obtained with
 * q4b_ipc_open, pointing at the same element as the call's own y[s]; NULL entries
 * (the own rank) are skipped.  q4b_matmul_no_alloc ignores it.
 *
 * q4b_barrier_*: create one per context, exchange q4b_barrier_counter between the
 * ranks (q4b_ipc_export / q4b_ipc_open), install with q4b_barrier_set_peer.
 * q4b_barrier_queue puts a kernel on the stream that tells every rank "all I
 * queued before this is stored" and waits (bounded, status 2 at the next
 * q4b_sync when it expires) until every rank has said so; work queued after it
 * may read what the peers pushed.  Every rank must queue the same barriers in
 * the same order.  The round number lives in device memory, so barriers may be
 * recorded into a graph (q4b_graph_begin) together with the launches between
 * them; the barrier is a programmatic dependent of the launch before it and lets
 * the launch after it start early, so the next projection's weights stream while
 * the ranks meet. */
/* q4b_push_rows: the other way to put a finished slice into the peers' copies, for
 * large M: one kernel after the launch that copies a block of m_rows rows of
 * row_bytes each (rows ld_bytes apart, the same pitch on every rank) from this
 * rank's output into the same place of every peer's (peers[r]: the block's address
 * there, from q4b_ipc_open) with whole 512-byte requests per warp on every link at
 * once.  A GEMM epilogue stores 32-64 bytes per thread per peer between tiles and
 * reaches a fraction of the link's rate; at M = 512 on eight ranks this call is
 * the difference.  Queue the barrier after it. */
int q4b_push_rows(q4b_context *context, const void *local, void *const *peers, uint32_t peer_count, uint32_t m_rows,
                  uint32_t row_bytes, uint32_t ld_bytes, char *error_message, size_t error_capacity);
typedef struct q4b_barrier q4b_barrier;
int q4b_context_push_outputs(q4b_context *context, uint32_t world, void *const *peer_y, int count);
int q4b_barrier_create(q4b_context *context, uint32_t world, uint32_t rank, q4b_barrier **barrier,
                       char *error_message, size_t error_capacity);
void *q4b_barrier_counter(q4b_barrier *barrier);
int q4b_barrier_set_peer(q4b_barrier *barrier, uint32_t peer_rank, void *peer_counter);
int q4b_barrier_queue(q4b_context *context, q4b_barrier *barrier, char *error_message, size_t error_capacity);
void q4b_barrier_free(q4b_context *context, q4b_barrier *barrier);

/* ---- device memory shared between the ranks of one node (thin wrappers of the
 * CUDA IPC calls; the reference is single-device and has no counterpart).  A
 * 64-byte handle made by the owner is opened by a peer process, which may then
 * store into that memory over NVLink. */
int q4b_ipc_export(q4b_context *context, void *device_pointer, void *handle_64_bytes,
                   char *error_message, size_t error_capacity);
int q4b_ipc_open(q4b_context *context, const void *handle_64_bytes, void **peer_pointer,
                 char *error_message, size_t error_capacity);
int q4b_ipc_close(q4b_context *context, void *peer_pointer);

/* ---- NCCL all-gather of the output slices over NVLink (the reference is
 * single-device and has no collective; this is the plain form of the gather that
 * the sequences and q4b_context_push_outputs fuse into the producing kernels, kept
 * as their baseline and cross-check).  One process per GPU: one rank calls
 * q4b_comm_unique_id and hands the 128 bytes to the others by any means; every
 * rank then calls q4b_comm_create (collective: returns when all have).  NCCL is
 * loaded at run time (libnccl.so.2) by the first of these calls; status 3 when
 * it cannot be.
 *
 * q4b_all_gather: ncclAllGather of `bytes_per_rank` bytes on the context's
 * stream; `gathered` holds world x bytes_per_rank, rank-major; in place when
 * slice == gathered + rank * bytes_per_rank.  Asynchronous.
 * q4b_all_gather_columns: this rank's [m_rows][slice_columns] block (dense) into
 * the whole [m_rows][world * slice_columns] row-major matrix every rank needs
 * next.  m_rows = 1 is the plain all-gather; above that NCCL's rank-major blocks
 * land in `staging` (world x m_rows x slice bytes, device) and a copy kernel
 * interleaves them.  All ranks pass equal slices. */
typedef struct q4b_comm q4b_comm;
int q4b_comm_unique_id(void *id_128_bytes, char *error_message, size_t error_capacity);
int q4b_comm_create(q4b_context *context, uint32_t world, uint32_t rank, const void *id_128_bytes,
                    q4b_comm **comm, char *error_message, size_t error_capacity);
uint32_t q4b_comm_world(const q4b_comm *comm);
uint32_t q4b_comm_rank(const q4b_comm *comm);
int q4b_all_gather(q4b_context *context, q4b_comm *comm, const void *slice, void *gathered,
                   size_t bytes_per_rank, char *error_message, size_t error_capacity);
int q4b_all_gather_columns(q4b_context *context, q4b_comm *comm, const void *slice, void *full,
                           uint32_t m_rows, uint32_t slice_columns, uint32_t element_bytes, void *staging,
                           char *error_message, size_t error_capacity);
void q4b_comm_free(q4b_context *context, q4b_comm *comm);

/* ---- layer-image files: replaces map_file, validate_delta_header,
 * validate_attention_header, load_delta_layer and load_attention_layer
 * (qwen38_m3_decode.m:374-625) for the Q4 matrices of a layer.  File layouts:
 * qwen38_m3_image.h:26-94 (magic "Q38M3Q4\0", version 3) and
 * qwen38_m3_attention_image.h:21-72 (magic "Q38M3ATT", version 1).
 *
 * q4b_image_open maps the file read-only and validates it as the reference does:
 * at least one page, magic, version, one-page header, group size 64, the layer
 * index asked for (DeltaNet images never at layers 3 mod 4, attention images only
 * there or at the MTP layer 64), every segment page-aligned (mapped_buffer,
 * :398-407), the file ending with the output metadata; and, beyond the
 * reference, every segment inside the file and large enough for its matrix.
 * check_27b_shapes adds the fixed shapes the reference runtime insists on
 * (:412-421, :433-443).  allowed_sha256 (may be NULL) is the list of source
 * digests the caller accepts, the role of pinned_sha.  Failures return
 * Q4B_LOAD_FAILURE with a message.  No GPU is needed to open an image. */
typedef struct q4b_image q4b_image;
enum { Q4B_IMAGE_DELTA = 0, Q4B_IMAGE_ATTENTION = 1, Q4B_IMAGE_GLOBAL = 2, Q4B_IMAGE_MTP = 3 };
enum { Q4B_MATRIX_GATE = 0, Q4B_MATRIX_UP = 1, Q4B_MATRIX_DOWN = 2, Q4B_MATRIX_INPUT = 3, Q4B_MATRIX_OUTPUT = 4 };
/* the global image (qwen38_m3_global_image.h:14-38, magic "Q38M3GLB", version 1; load_global, :462-498) holds two
 * [vocabulary, hidden] matrices; its info reports the vocabulary as intermediate_size, the embedding's source
 * digest as source_sha256 and the lm_head's as mlp_source_sha256; layer_index is ignored */
enum { Q4B_MATRIX_EMBEDDING = 0, Q4B_MATRIX_LM_HEAD = 1 };
/* the MTP extras image (qwen38_m3_mtp_image.h:21-51, magic "Q38M3MTP", version 1; validated as
 * qwen38_m3_model_mtp_open does, qwen38_m3_decode.m:2365-2380) holds one matrix, the fused fc projection
 * [hidden, 2 x hidden] that encode_mtp_pass runs through encode_prefill_gemm_f16 (:1818-1821), and three norm
 * vectors of hidden_size floats inside its constants: info.constants_index gives where the embedding norm, the
 * hidden norm and the final norm begin; intermediate_size repeats the fc rows; layer_index is ignored.  The MTP
 * transformer layer itself is an attention image with layer index 64. */
enum { Q4B_MATRIX_FC = 0 };
typedef struct {
    uint32_t kind, version, layer_index, hidden_size, intermediate_size, group_size;
    uint32_t rows[5], groups[5];          /* by Q4B_MATRIX_*: output rows and K/64 */
    uint32_t constants_f32_count;
    uint32_t reference_counts[3];         /* how many of the eight values below the packer filled */
    float gate_up_reference_first_8[8];   /* silu(gate x) * up x, rows 0..7 (qwen38_m3_pack.c:448-505) */
    float mlp_reference_first_8[8];       /* whole MLP + residual, rows 0..7 */
    float layer_reference_first_8[8];
    char source_sha256[65], mlp_source_sha256[65];
    uint64_t constants_index[3];          /* MTP extras only: embedding norm, hidden norm, final norm */
} q4b_image_info;
int q4b_image_open(const char *path, int kind, uint32_t layer_index, int check_27b_shapes,
                   const char *const *allowed_sha256, int allowed_count, q4b_image **image,
                   char *error_message, size_t error_capacity);
int q4b_image_describe(const q4b_image *image, q4b_image_info *info);
/* the fp32 constants block (norm weights and the like), a host pointer into the mapping */
const float *q4b_image_constants(const q4b_image *image, uint32_t *count);
/* host pointers to the two segments of one matrix, as the packer wrote them */
int q4b_image_segments(const q4b_image *image, int matrix, const void **quants, const void **metadata);
/* rows [row_begin, row_begin+row_count) of one matrix, repacked and uploaded (q4b_weight_upload) */
int q4b_image_weight(q4b_context *context, const q4b_image *image, int matrix, uint32_t row_begin,
                     uint32_t row_count, q4b_weight **weight, char *error_message, size_t error_capacity);
void q4b_image_close(q4b_image *image);

/* ---- one decoder layer's Q4 matmuls, as the reference's encoders issue them
 * (qwen38_m3_decode.m): the in-projection at the head of encode_delta (:668-674)
 * and encode_attention (:747-753), the out-projection with residual at their
 * tails (:716-723, :788-795), encode_mlp (:639-660): fused gate/up + SiLU, then
 * down with the residual added; and their batched forms encode_prefill_gemm_f16
 * (:885-928), encode_prefill_gemm_residual (:930-1001), encode_prefill_mlp
 * (:1016-1038) -- one entry point each, the kernel is chosen by `batch`.
 *
 * A layer holds, of every matrix, the rows this rank owns (column-parallel over
 * `world` ranks; q4b_layer_slice gives the rule: contiguous, 16-row granular).
 * All activations are DEVICE pointers, [batch, width] row-major with the FULL
 * width of the matrix's output: a call writes columns [begin, begin+count) and
 * leaves the rest to the other ranks (gather is the caller's; with world = 1 the
 * slice is everything).  Inputs: fp16, except where a dtype is passed (the
 * reference feeds fp32 to the second projections, qwen38_layer.metal:193-255).
 * q4b_layer_encode_mlp runs both halves and therefore needs world = 1;
 * q4b_layer_encode_mlp_gathered is the same for world > 1: gate/up on this rank's
 * rows, q4b_layer_gather of the intermediate, down, gather of the output, all
 * queued on the context's stream.  q4b_layer_gather completes a full-width
 * [batch, rows] buffer of which every rank has written its own columns (NCCL
 * all-gather; equal slices on all ranks; batch > 1 needs `staging`, device
 * memory of (world + 1) x batch x slice bytes). */
typedef struct q4b_layer q4b_layer;
void q4b_layer_slice(uint32_t rows, uint32_t rank, uint32_t world, uint32_t *row_begin, uint32_t *row_count);
int q4b_layer_load(q4b_context *context, const q4b_image *image, uint32_t rank, uint32_t world,
                   q4b_layer **layer, char *error_message, size_t error_capacity);
/* a layer over matrices the caller already holds (Q4B_MATRIX_* order, entries may be NULL);
 * rows_total = rows of the whole matrix, row_begin = first row the given shard holds */
int q4b_layer_wrap(const q4b_weight *const *matrices, const uint32_t *rows_total, const uint32_t *row_begin,
                   uint32_t rank, uint32_t world, q4b_layer **layer);
void q4b_layer_free(q4b_context *context, q4b_layer *layer);
int q4b_layer_encode_input(q4b_context *context, const q4b_layer *layer, const void *normalized_f16,
                           uint32_t batch, void *projected, int projected_dtype,
                           char *error_message, size_t error_capacity);
int q4b_layer_encode_output(q4b_context *context, const q4b_layer *layer, const void *mixer_output,
                            int mixer_dtype, uint32_t batch, const void *residual, int residual_dtype,
                            void *hidden, int hidden_dtype, char *error_message, size_t error_capacity);
int q4b_layer_encode_gate_up(q4b_context *context, const q4b_layer *layer, const void *post_normalized_f16,
                             uint32_t batch, void *intermediate, int intermediate_dtype,
                             char *error_message, size_t error_capacity);
int q4b_layer_encode_down(q4b_context *context, const q4b_layer *layer, const void *intermediate,
                          int intermediate_dtype, uint32_t batch, const void *residual, int residual_dtype,
                          void *layer_output, int output_dtype, char *error_message, size_t error_capacity);
int q4b_layer_encode_mlp(q4b_context *context, const q4b_layer *layer, const void *post_normalized_f16,
                         uint32_t batch, void *intermediate, int intermediate_dtype, const void *residual,
                         int residual_dtype, void *layer_output, int output_dtype,
                         char *error_message, size_t error_capacity);

int q4b_layer_gather(q4b_context *context, const q4b_layer *layer, q4b_comm *comm, int matrix, void *full_width,
                     int dtype, uint32_t batch, void *staging, char *error_message, size_t error_capacity);
int q4b_layer_encode_mlp_gathered(q4b_context *context, const q4b_layer *layer, q4b_comm *comm,
                                  const void *post_normalized_f16, uint32_t batch, void *intermediate,
                                  int intermediate_dtype, const void *residual, int residual_dtype,
                                  void *layer_output, int output_dtype, void *staging,
                                  char *error_message, size_t error_capacity);

/* ---- read-bandwidth probe: the role of the reference's device-memory probe
 * (models/qwen3.8-27b/targets/jetson-orin/qwen38_jetson_memory_probe.cu:25-49):
 * reads `bytes` of device memory `iterations` times and reports GB/s from CUDA
 * events.  mode 0 = plain 16-byte loads; 1 = the GEMV kernel's bulk-copy ring
 * with idle consumers; 2 = the same ring with the consumers reading the staged
 * bytes.  ctas_per_sm, stages and stage_bytes shape the ring modes.  Synchronous;
 * allocates and frees its own buffer. */
int q4b_probe_read(q4b_context *context, int mode, size_t bytes, int ctas_per_sm, uint32_t stages,
                   uint32_t stage_bytes, int iterations, double *gigabytes_per_second,
                   char *error_message, size_t error_capacity);

/* One side of a ping-pong between two GPUs (no reference counterpart: the
 * reference has one GPU).  Both ranks call it at about the same time, one with
 * initiator = 1.  own_words / peer_words: 256 + payload_bytes of zeroed device
 * memory on this GPU and the same buffer of the peer (q4b_ipc_open); word 0 is
 * the flag.  A round trip is: payload stores into the peer, a system-scope fence,
 * an addition to the peer's flag, and the wait for the answer -- the exchange a
 * column-parallel decode sequence makes twice per gather point.  rounds_before:
 * rounds earlier calls have already played on these buffers.  mode 0 is that
 * exchange; bit 0 raises the flag with one release store instead of fence +
 * addition, bit 1 polls with relaxed loads and fences once at the end, bit 2
 * drops the sender's fence (not an ordering to rely on: it prices the fence).
 * Waits are bounded
 * (about a second); a peer that never answers gives status 2 and a message
 * naming the round.  Synchronous. */
int q4b_probe_signal(q4b_context *context, void *own_words, void *peer_words, uint32_t payload_bytes,
                     uint32_t rounds, uint32_t rounds_before, int initiator, int mode,
                     double *microseconds_per_round_trip, char *error_message, size_t error_capacity);

/* ---- replay of a recorded call sequence (one command buffer per token in the
 * reference, qwen38_m3_decode.m:1614-1690): calls between begin and end are
 * captured instead of executed. */
int q4b_graph_begin(q4b_context *context, char *error_message, size_t error_capacity);
int q4b_graph_end(q4b_context *context, q4b_graph **graph, char *error_message,
                  size_t error_capacity);
int q4b_graph_launch(q4b_context *context, q4b_graph *graph, char *error_message,
                     size_t error_capacity);
void q4b_graph_free(q4b_graph *graph);

#ifdef __cplusplus
}
#endif
#endif
