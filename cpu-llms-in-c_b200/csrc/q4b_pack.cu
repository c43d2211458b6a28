// Image loader kernels: raw reference planes -> tile stream, its inverse
// (the dequantisation-in-isolation hook, cf. qwen38_global.metal:13-28), and the
// seeded synthetic generator.
#include "q4b_kernels.h"

namespace q4b {

__device__ inline uint16_t meta_to_f16_bits(const void *plane, int dtype, size_t index) {
    uint16_t bits = reinterpret_cast<const uint16_t *>(plane)[index];
    if (dtype == kBF16) {
        // BF16 plane -> fp16 record: widen, round once to nearest even
        // (compiler/qwen3.8-27b/apple-m3-pro/qwen38_m3_pack.c:173-178)
        float value = __uint_as_float((uint32_t)bits << 16);
        return __half_as_ushort(__float2half_rn(value));
    }
    return bits;
}

// one thread per (tile, lane); lanes 0..7 also write the metadata records
__global__ void __launch_bounds__(256)
repack_kernel(const uint8_t *__restrict__ quants, const void *__restrict__ meta,
              const void *__restrict__ biases, int meta_dtype, uint32_t groups,
              uint32_t row_begin, uint32_t row_count, uint32_t padded_row_tiles,
              uint8_t *__restrict__ tiles) {
    uint64_t thread = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t tile = thread >> 5;
    uint32_t lane = thread & 31u;
    if (tile >= (uint64_t)padded_row_tiles * groups) {
        return;
    }
    uint32_t rt = (uint32_t)(tile / groups);
    uint32_t g = (uint32_t)(tile % groups);
    uint32_t gid = lane >> 2, t = lane & 3u;
    uint32_t local_lo = rt * 16 + gid, local_hi = local_lo + 8;
    uint64_t piece_lo = 0, piece_hi = 0;
    if (local_lo < row_count) {
        size_t byte = ((size_t)(row_begin + local_lo) * groups + g) * 32 + 8 * t;
        piece_lo = *reinterpret_cast<const uint64_t *>(quants + byte);
    }
    if (local_hi < row_count) {
        size_t byte = ((size_t)(row_begin + local_hi) * groups + g) * 32 + 8 * t;
        piece_hi = *reinterpret_cast<const uint64_t *>(quants + byte);
    }
    uint8_t *out = tiles + tile_offset(rt, g, groups);
    reinterpret_cast<uint4 *>(out)[piece_index(lane)] = swizzle_lane(piece_lo, piece_hi);
    if (lane < 8) {
        uint16_t record[4] = {0, 0, 0, 0};
        uint32_t rows[2] = {rt * 16 + lane, rt * 16 + lane + 8};
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (rows[half] < row_count) {
                size_t block = (size_t)(row_begin + rows[half]) * groups + g;
                if (biases == nullptr) {
                    record[2 * half] = meta_to_f16_bits(meta, kF16, 2 * block);
                    record[2 * half + 1] = meta_to_f16_bits(meta, kF16, 2 * block + 1);
                } else {
                    record[2 * half] = meta_to_f16_bits(meta, meta_dtype, block);
                    record[2 * half + 1] = meta_to_f16_bits(biases, meta_dtype, block);
                }
            }
        }
        uint2 packed = make_uint2(record[0] | ((uint32_t)record[1] << 16),
                                  record[2] | ((uint32_t)record[3] << 16));
        reinterpret_cast<uint2 *>(out + kTileCodeBytes)[lane] = packed;
    }
}

cudaError_t launch_repack(const uint8_t *quants, const void *meta, const void *biases,
                          int meta_dtype, uint32_t groups, uint32_t row_begin,
                          uint32_t row_count, uint8_t *tiles, cudaStream_t stream) {
    uint32_t row_tiles = ceil_div(row_count, kTileRows);
    uint32_t padded = ceil_div(row_tiles, kRowTilePad) * kRowTilePad;
    uint64_t threads = (uint64_t)padded * groups * 32;
    if (threads == 0) {
        return cudaSuccess;
    }
    uint64_t blocks = (threads + 255) / 256;
    repack_kernel<<<(unsigned)blocks, 256, 0, stream>>>(quants, meta, biases, meta_dtype,
                                                         groups, row_begin, row_count, padded,
                                                         tiles);
    return cudaGetLastError();
}

// one thread per (tile, lane): 2 rows x 16 columns
__global__ void __launch_bounds__(256)
unpack_kernel(WeightView w, uint8_t *__restrict__ codes, float *__restrict__ w32,
              __half *__restrict__ w16) {
    uint64_t thread = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint64_t tile = thread >> 5;
    uint32_t lane = thread & 31u;
    if (tile >= (uint64_t)w.row_tiles * w.groups) {
        return;
    }
    uint32_t rt = (uint32_t)(tile / w.groups);
    uint32_t g = (uint32_t)(tile % w.groups);
    uint32_t gid = lane >> 2, t = lane & 3u;
    const uint8_t *in = w.tiles + tile_offset(rt, g, w.groups);
    uint4 words = reinterpret_cast<const uint4 *>(in)[piece_index(lane)];
    uint2 record = reinterpret_cast<const uint2 *>(in + kTileCodeBytes)[gid];
    const uint32_t word[4] = {words.x, words.y, words.z, words.w};
    size_t columns = (size_t)w.groups * kGroup;
    uint32_t row[2] = {rt * 16 + gid, rt * 16 + gid + 8};
    __half2 meta16[2] = {*reinterpret_cast<__half2 *>(&record.x),
                         *reinterpret_cast<__half2 *>(&record.y)};
    if (codes != nullptr) {
        uint64_t piece[2];
        unswizzle_lane(words, piece[0], piece[1]);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (row[half] < w.rows) {
                uint8_t *out = codes + (size_t)row[half] * columns + g * kGroup + 16 * t;
                uint32_t bytes[4];
#pragma unroll
                for (int quad = 0; quad < 4; ++quad) {
                    uint32_t nibbles = (uint32_t)(piece[half] >> (16 * quad)) & 0xffffu;
                    bytes[quad] = (nibbles & 0xfu) | ((nibbles & 0xf0u) << 4) |
                                  ((nibbles & 0xf00u) << 8) | ((nibbles & 0xf000u) << 12);
                }
                *reinterpret_cast<uint4 *>(out) = make_uint4(bytes[0], bytes[1], bytes[2], bytes[3]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 regs[4];
        word_to_codes_f16(word[i], regs);  // the same extraction the matmul kernels use
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (row[half] >= w.rows) {
                continue;
            }
            size_t base = (size_t)row[half] * columns + g * kGroup + 16 * t + 4 * i;
            __half2 scale = __half2half2(__low2half(meta16[half]));
            __half2 bias = __half2half2(__high2half(meta16[half]));
            __half2 pair01 = regs[half], pair23 = regs[2 + half];
            if (w16 != nullptr) {
                __half2 out01 = dequant_w16(pair01, scale, bias);
                __half2 out23 = dequant_w16(pair23, scale, bias);
                uint2 packed = make_uint2(*reinterpret_cast<uint32_t *>(&out01),
                                          *reinterpret_cast<uint32_t *>(&out23));
                *reinterpret_cast<uint2 *>(w16 + base) = packed;
            }
            if (w32 != nullptr) {
                float s = __low2float(meta16[half]), b = __high2float(meta16[half]);
                float4 out;
                out.x = dequant_w32((uint32_t)__half2float(__low2half(pair01)), s, b);
                out.y = dequant_w32((uint32_t)__half2float(__high2half(pair01)), s, b);
                out.z = dequant_w32((uint32_t)__half2float(__low2half(pair23)), s, b);
                out.w = dequant_w32((uint32_t)__half2float(__high2half(pair23)), s, b);
                *reinterpret_cast<float4 *>(w32 + base) = out;
            }
        }
    }
}

cudaError_t launch_unpack(WeightView w, uint8_t *codes, float *w32, __half *w16,
                          cudaStream_t stream) {
    uint64_t threads = (uint64_t)w.row_tiles * w.groups * 32;
    if (threads == 0) {
        return cudaSuccess;
    }
    uint64_t blocks = (threads + 255) / 256;
    unpack_kernel<<<(unsigned)blocks, 256, 0, stream>>>(w, codes, w32, w16);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// affine Q8: planes [N][G][64] bytes + bf16 scales / biases [N][G] -> the Q8 stream, and its inverse
// ---------------------------------------------------------------------------
// one thread per (128-row block, group, row, piece)
__global__ void __launch_bounds__(256)
repack_q8_kernel(const uint8_t *__restrict__ quants, const uint16_t *__restrict__ scales,
                 const uint16_t *__restrict__ biases, uint32_t groups, uint32_t row_begin, uint32_t row_count,
                 uint32_t blocks, uint8_t *__restrict__ tiles) {
    const uint64_t thread = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (thread >= (uint64_t)blocks * groups * kQ8Rows * 4) return;
    const uint32_t piece = (uint32_t)(thread & 3u), row = (uint32_t)((thread >> 2) & (kQ8Rows - 1));
    const uint64_t tile = thread >> 9;  // block * groups + g
    const uint32_t g = (uint32_t)(tile % groups), local = (uint32_t)(tile / groups) * kQ8Rows + row;
    uint8_t *out = tiles + tile * kQ8TileBytes;
    uint4 codes = make_uint4(0u, 0u, 0u, 0u);
    uint32_t record = 0;
    if (local < row_count) {
        const size_t at = (size_t)(row_begin + local) * groups + g;
        codes = *reinterpret_cast<const uint4 *>(quants + at * kGroup + 16 * piece);
        record = (uint32_t)scales[at] | ((uint32_t)biases[at] << 16);
    }
    reinterpret_cast<uint4 *>(out)[q8_piece_index(row, piece)] = codes;
    if (piece == 0) reinterpret_cast<uint32_t *>(out + kQ8CodeBytes)[row] = record;
}

cudaError_t launch_repack_q8(const uint8_t *quants, const uint16_t *scales, const uint16_t *biases, uint32_t groups,
                             uint32_t row_begin, uint32_t row_count, uint8_t *tiles, cudaStream_t stream) {
    const uint32_t blocks = ceil_div(row_count, kQ8Rows);
    const uint64_t threads = (uint64_t)blocks * groups * kQ8Rows * 4;
    if (threads == 0) return cudaSuccess;
    repack_q8_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(quants, scales, biases, groups, row_begin,
                                                                            row_count, blocks, tiles);
    return cudaGetLastError();
}

// The Q8 dequantisation contract: half(float(scale) * float(q) + float(bias)), the product exact in fp32, the sum
// rounded once in fp32, then once to fp16 (minimax_h3_attention.metal:627-633).
__device__ inline float dequant_q8_w32(uint32_t code, uint32_t record) {
    const float scale = __uint_as_float(record << 16), bias = __uint_as_float(record & 0xffff0000u);
    return __fmaf_rn(scale, (float)code, bias);
}

__global__ void __launch_bounds__(256)
unpack_q8_kernel(WeightView w, uint8_t *__restrict__ codes, float *__restrict__ w32, __half *__restrict__ w16) {
    const uint64_t thread = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t blocks = ceil_div(w.rows, kQ8Rows);
    if (thread >= (uint64_t)blocks * w.groups * kQ8Rows * 4) return;
    const uint32_t piece = (uint32_t)(thread & 3u), row = (uint32_t)((thread >> 2) & (kQ8Rows - 1));
    const uint64_t tile = thread >> 9;
    const uint32_t g = (uint32_t)(tile % w.groups), local = (uint32_t)(tile / w.groups) * kQ8Rows + row;
    if (local >= w.rows) return;
    const uint8_t *in = w.tiles + tile * kQ8TileBytes;
    const uint4 words = reinterpret_cast<const uint4 *>(in)[q8_piece_index(row, piece)];
    const uint32_t record = reinterpret_cast<const uint32_t *>(in + kQ8CodeBytes)[row];
    const size_t base = (size_t)local * w.groups * kGroup + (size_t)g * kGroup + 16 * piece;
    if (codes != nullptr) *reinterpret_cast<uint4 *>(codes + base) = words;
    const uint32_t word[4] = {words.x, words.y, words.z, words.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float value = dequant_q8_w32((word[i >> 2] >> (8 * (i & 3))) & 0xffu, record);
        if (w32 != nullptr) w32[base + i] = value;
        if (w16 != nullptr) w16[base + i] = __float2half_rn(value);
    }
}

cudaError_t launch_unpack_q8(WeightView w, uint8_t *codes, float *w32, __half *w16, cudaStream_t stream) {
    const uint64_t threads = (uint64_t)ceil_div(w.rows, kQ8Rows) * w.groups * kQ8Rows * 4;
    if (threads == 0) return cudaSuccess;
    unpack_q8_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(w, codes, w32, w16);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// rows of a matrix, dequantised: the embedding lookup
// (qwen38_q4_embedding_lookup, qwen38_global.metal:13-28: out[c] = half(float(scale) * float(q) + float(bias)))
// ---------------------------------------------------------------------------
// one thread per (requested row, group, quarter of the group): 16 columns
__global__ void __launch_bounds__(256)
lookup_rows_kernel(WeightView w, const uint32_t *__restrict__ rows, uint32_t count, uint32_t row_base,
                   void *__restrict__ out, int out_dtype) {
    const uint64_t thread = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t per_row = w.groups * 4;
    const uint64_t which = thread / per_row;
    if (which >= count) return;
    const uint32_t rest = (uint32_t)(thread % per_row), g = rest >> 2, t = rest & 3u;
    const uint32_t row = rows[which] - row_base;  // rows outside this shard wrap to huge values
    const size_t columns = (size_t)w.groups * kGroup;
    const size_t at = which * columns + (size_t)g * kGroup + 16 * t;
    if (row >= w.rows) {  // not held here: zeros, so that the shards of a split vocabulary add up
        if (out_dtype == kF32) {
            for (int i = 0; i < 16; ++i) reinterpret_cast<float *>(out)[at + i] = 0.0f;
        } else {
            for (int i = 0; i < 16; ++i) reinterpret_cast<__half *>(out)[at + i] = __float2half_rn(0.0f);
        }
        return;
    }
    const uint32_t rt = row >> 4, within = row & 15u, gid = within & 7u, upper = within >> 3;
    const uint8_t *in = w.tiles + tile_offset(rt, g, w.groups);
    const uint4 words = reinterpret_cast<const uint4 *>(in)[piece_index(gid * 4 + t)];
    const uint2 record = reinterpret_cast<const uint2 *>(in + kTileCodeBytes)[gid];
    const __half2 meta = *reinterpret_cast<const __half2 *>(upper ? &record.y : &record.x);
    const float scale = __low2float(meta), bias = __high2float(meta);
    const uint32_t word[4] = {words.x, words.y, words.z, words.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            // column 4 i + c of this lane's 16 sits in nibble 4 (c % 2) + 2 (c / 2) of word i, rows gid + 8 one nibble up
            const uint32_t nibble = 4u * (c & 1) + 2u * (c >> 1) + upper;
            const float value = dequant_w32((word[i] >> (4u * nibble)) & 0xfu, scale, bias);
            if (out_dtype == kF32) {
                reinterpret_cast<float *>(out)[at + 4 * i + c] = value;
            } else {
                reinterpret_cast<__half *>(out)[at + 4 * i + c] = __float2half_rn(value);
            }
        }
    }
}

cudaError_t launch_lookup_rows(WeightView w, const uint32_t *rows, uint32_t count, uint32_t row_base, void *out,
                               int out_dtype, cudaStream_t stream) {
    if (count == 0) return cudaSuccess;
    const uint64_t threads = (uint64_t)count * w.groups * 4;
    lookup_rows_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(w, rows, count, row_base, out, out_dtype);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Listed rows only: y[m][slot] = sum_k w(ids[slot], k) x[m][k] -- the draft head's extra vocabulary rows
// (qwen38_q4_lm_head_gathered, qwen38_global.metal:68-96: one simdgroup per gathered row id, w =
// float(scale) * q + float(bias), fp32 sum).  One warp per listed row: lane = (group phase lane / 4, quarter
// lane % 4) reads the 16 codes of that row in each of its (group, quarter) cells and the cell's 16 activations;
// a butterfly over the warp finishes the row.  A listed row costs 64 bytes per group (its tile partner's
// nibbles ride along), which matters not at all for the few hundred rows such a list holds.
// ---------------------------------------------------------------------------
template <typename X>
__global__ void __launch_bounds__(256)
matmul_rows_kernel(WeightView w, const uint32_t *__restrict__ ids, uint32_t count, uint32_t row_base,
                   const X *__restrict__ x, uint32_t m_rows, void *__restrict__ y, int y_dtype, uint32_t ldy) {
    const uint32_t slot = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (slot >= count) return;
    const uint32_t row = ids[slot] - row_base;  // rows outside this shard wrap to huge values
    if (row >= w.rows) return;                  // not held here: the rank that holds it writes the slot
    const uint32_t rt = row >> 4, within = row & 15u, gid = within & 7u, upper = within >> 3;
    const uint32_t t = lane & 3u;
    const size_t K = (size_t)w.groups * kGroup;
    float acc[16];
#pragma unroll
    for (int m = 0; m < 16; ++m) acc[m] = 0.0f;
    for (uint32_t g = lane >> 2; g < w.groups; g += 8) {
        const uint8_t *in = w.tiles + tile_offset(rt, g, w.groups);
        const uint4 words = reinterpret_cast<const uint4 *>(in)[piece_index(gid * 4 + t)];
        const uint2 record = reinterpret_cast<const uint2 *>(in + kTileCodeBytes)[gid];
        const __half2 meta = *reinterpret_cast<const __half2 *>(upper ? &record.y : &record.x);
        const float scale = __low2float(meta), bias = __high2float(meta);
        const uint32_t word[4] = {words.x, words.y, words.z, words.w};
        float weight[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t nibble = 4u * (c & 1) + 2u * (c >> 1) + upper;
                weight[4 * i + c] = dequant_w32((word[i] >> (4u * nibble)) & 0xfu, scale, bias);
            }
        }
        for (uint32_t m = 0; m < m_rows; ++m) {
            const X *cell = x + (size_t)m * K + (size_t)g * kGroup + 16 * t;
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float value;
                if constexpr (sizeof(X) == 2) value = __half2float(cell[i]);
                else value = cell[i];
                sum = fmaf(weight[i], value, sum);
            }
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                if ((uint32_t)q == m) acc[q] += sum;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < 16; ++m) {
        float total = acc[m];
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) total += __shfl_xor_sync(0xffffffffu, total, offset);
        if (lane == 0 && (uint32_t)m < m_rows) {
            const size_t at = (size_t)m * ldy + slot;
            if (y_dtype == kF32) reinterpret_cast<float *>(y)[at] = total;
            else reinterpret_cast<__half *>(y)[at] = __float2half_rn(total);
        }
    }
}

cudaError_t launch_matmul_rows(WeightView w, const uint32_t *ids, uint32_t count, uint32_t row_base, const void *x,
                               int x_dtype, uint32_t m_rows, void *y, int y_dtype, uint32_t ldy, cudaStream_t stream) {
    if (count == 0) return cudaSuccess;
    if (m_rows == 0 || m_rows > 16) return cudaErrorInvalidValue;
    const unsigned blocks = (count + 7) / 8;
    if (x_dtype == kF32) {
        matmul_rows_kernel<float><<<blocks, 256, 0, stream>>>(w, ids, count, row_base, static_cast<const float *>(x),
                                                              m_rows, y, y_dtype, ldy);
    } else {
        matmul_rows_kernel<__half><<<blocks, 256, 0, stream>>>(w, ids, count, row_base, static_cast<const __half *>(x),
                                                               m_rows, y, y_dtype, ldy);
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// RMS norm: the step that produces the fp16 x of a layer's in-projections and of the MLP
// (qwen38_rmsnorm_f16_to_f16 / qwen38_rmsnorm_f32_to_f16, qwen38_layer.metal:21-69; one thread block per
// activation row as in their batched forms).  Same order of operations as the reference: 256 strided partial
// sums of squares, a halving tree over them, out = half(x * inv_rms * weight) with both products in fp32.
// Every operation is rounded on its own (no fused multiply-add, IEEE square root and division), so the result
// is a function of the inputs alone and a CPU restatement reproduces it bit for bit.
// ---------------------------------------------------------------------------
template <typename In>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const In *__restrict__ input, const float *__restrict__ weight, __half *__restrict__ output,
               uint32_t hidden, float epsilon) {
    __shared__ float partials[256];
    const uint32_t tid = threadIdx.x;
    const In *row = input + (size_t)blockIdx.x * hidden;
    auto value_at = [&](uint32_t index) {
        if constexpr (sizeof(In) == 2) return __half2float(row[index]);
        else return (float)row[index];
    };
    float sum = 0.0f;
    for (uint32_t index = tid; index < hidden; index += 256) {
        const float value = value_at(index);
        sum = __fadd_rn(sum, __fmul_rn(value, value));
    }
    partials[tid] = sum;
    __syncthreads();
    for (uint32_t stride = 128; stride != 0; stride >>= 1) {
        if (tid < stride) partials[tid] = __fadd_rn(partials[tid], partials[tid + stride]);
        __syncthreads();
    }
    const float mean = __fadd_rn(__fdiv_rn(partials[0], (float)hidden), epsilon);
    const float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(mean));
    __half *out = output + (size_t)blockIdx.x * hidden;
    for (uint32_t index = tid; index < hidden; index += 256) {
        out[index] = __float2half_rn(__fmul_rn(__fmul_rn(value_at(index), inv_rms), weight[index]));
    }
}

cudaError_t launch_rmsnorm(const void *input, int input_dtype, const float *weight, void *output, uint32_t hidden,
                           uint32_t batch, float epsilon, cudaStream_t stream) {
    if (batch == 0) return cudaSuccess;
    if (input_dtype == kF32) {
        rmsnorm_kernel<float><<<batch, 256, 0, stream>>>(static_cast<const float *>(input), weight,
                                                         static_cast<__half *>(output), hidden, epsilon);
    } else {
        rmsnorm_kernel<__half><<<batch, 256, 0, stream>>>(static_cast<const __half *>(input), weight,
                                                          static_cast<__half *>(output), hidden, epsilon);
    }
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// seeded generator
// ---------------------------------------------------------------------------
__global__ void synth_codes_kernel(uint64_t key, uint32_t *words, uint64_t word_begin,
                                   uint64_t word_count) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t offset = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
         offset < word_count; offset += stride) {
        uint64_t word = word_begin + offset;
        uint64_t bits = keyed(key, word >> 1);
        words[offset] = (uint32_t)(bits >> (32u * (word & 1u)));
    }
}

__global__ void synth_meta_kernel(uint64_t key, __half *meta, uint64_t group_begin,
                                  uint64_t group_count) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t offset = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
         offset < group_count; offset += stride) {
        uint64_t group = group_begin + offset;
        float uniform = (float)(keyed(key, 4ull * group) >> 40) * (1.0f / 16777216.0f);
        __half scale = __float2half_rn(__fmaf_rn(uniform, 3.5e-3f, 5.0e-4f));
        float noise = normal12(keyed(key, 4ull * group + 1), keyed(key, 4ull * group + 2),
                               keyed(key, 4ull * group + 3));
        float bias = __fmaf_rn(noise, 1.0e-3f, __fmul_rn(-8.0f, __half2float(scale)));
        meta[2 * offset] = scale;
        meta[2 * offset + 1] = __float2half_rn(bias);
    }
}

__global__ void synth_x_kernel(uint64_t key, __half *x, uint64_t begin, uint64_t count) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t offset = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; offset < count;
         offset += stride) {
        uint64_t index = begin + offset;
        x[offset] = __float2half_rn(normal12(keyed(key, 3ull * index),
                                             keyed(key, 3ull * index + 1),
                                             keyed(key, 3ull * index + 2)));
    }
}

static unsigned synth_blocks(uint64_t count) {
    uint64_t blocks = (count + 255) / 256;
    return (unsigned)(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

cudaError_t launch_synth_codes(uint64_t seed, uint64_t stream_id, uint32_t *words,
                               uint64_t word_begin, uint64_t word_count, cudaStream_t stream) {
    if (word_count == 0) return cudaSuccess;
    synth_codes_kernel<<<synth_blocks(word_count), 256, 0, stream>>>(
        stream_key(seed, stream_id), words, word_begin, word_count);
    return cudaGetLastError();
}
cudaError_t launch_synth_meta(uint64_t seed, uint64_t stream_id, __half *meta,
                              uint64_t group_begin, uint64_t group_count, cudaStream_t stream) {
    if (group_count == 0) return cudaSuccess;
    synth_meta_kernel<<<synth_blocks(group_count), 256, 0, stream>>>(
        stream_key(seed, stream_id), meta, group_begin, group_count);
    return cudaGetLastError();
}
cudaError_t launch_synth_x(uint64_t seed, uint64_t stream_id, __half *x, uint64_t begin,
                           uint64_t count, cudaStream_t stream) {
    if (count == 0) return cudaSuccess;
    synth_x_kernel<<<synth_blocks(count), 256, 0, stream>>>(stream_key(seed, stream_id), x,
                                                            begin, count);
    return cudaGetLastError();
}

}  // namespace q4b
