// Shared definitions of the affine-Q4 CUDA library (sm_100a).
//
// HBM layout of one weight matrix ("tile stream")
// -----------------------------------------------
// The reference image keeps two planes per matrix W[N][K], G = K/64
// (models/qwen3.8-27b/targets/apple-m3-pro/qwen38_q4.metal:10-37):
//   quants [N][G][32 bytes]   byte j>>1 of a group holds code j (low nibble even)
//   meta   [N][G]{fp16 scale, fp16 bias}
// On upload the two planes are fused into one linear stream of 576-byte tiles.
// Tile (rt, g) covers rows 16*rt .. 16*rt+15 and columns 64*g .. 64*g+63.  Four
// row tiles form a 64-row block; the stream is ordered [block][group][tile in
// block], so tile (rt, g) sits at byte offset ((rt/4)*G + g) * 2304 + (rt%4) * 576
// and everything one 64-row block needs for a range of groups is one contiguous
// byte range (one bulk copy).  Inside a tile:
//
//   [  0,512)  32 lane pieces of 16 bytes, lane l's piece at index piece_index(l)
//              (a rotation inside each 64-byte gid group that keeps the
//              row-per-thread readers of the tensor-core GEMM free of bank
//              conflicts).  Lane l = 4*gid + t owns rows
//              (gid, gid+8) and columns 16*t .. 16*t+15 of the tile.  Its four
//              32-bit words i = 0..3 each carry the eight codes of one
//              m16n8k16 A fragment, nibble p (bits 4p..4p+3):
//                p = 0: (gid  , 16t+4i  )   p = 4: (gid  , 16t+4i+1)
//                p = 2: (gid  , 16t+4i+2)   p = 6: (gid  , 16t+4i+3)
//                p = 1: (gid+8, 16t+4i  )   p = 5: (gid+8, 16t+4i+1)
//                p = 3: (gid+8, 16t+4i+2)   p = 7: (gid+8, 16t+4i+3)
//              so `w & 0x000F000F`, `w & 0x00F000F0`, and the same two masks
//              on `w >> 8` yield the four half2 registers of the fragment.
//   [512,576)  8 records of 8 bytes, record gid = {scale[gid], bias[gid],
//              scale[gid+8], bias[gid+8]} as fp16.
//
// A warp consumes a tile with one 16-byte read per lane plus an 8-byte metadata
// read; CTAs fetch whole [block][group range] byte ranges with bulk copies.
// Rows are padded with zero tiles up to a multiple of 128.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace q4b {

constexpr int kGroup = 64;           // columns per quantisation group
constexpr int kTileRows = 16;        // rows per tile
constexpr int kTileCodeBytes = 512;  // 16 rows x 64 codes / 2
constexpr int kTileMetaBytes = 64;   // 16 x {scale, bias} fp16
constexpr int kTileBytes = kTileCodeBytes + kTileMetaBytes;  // 576
constexpr int kRowTilePad = 8;       // row tiles padded to a multiple of this
constexpr int kBlockTiles = 4;       // row tiles per 64-row block
constexpr int kUnitBytes = kBlockTiles * kTileBytes;  // one block x one group: 2304

enum DType : int { kF16 = 0, kF32 = 1, kBF16 = 2, kNone = -1 };

enum WeightKind : uint32_t { kQ4 = 0, kQ8 = 1 };

struct WeightView {
    const uint8_t *tiles;  // tile stream
    uint32_t rows;         // logical rows held (N of this shard)
    uint32_t groups;       // G = K / 64
    uint32_t row_tiles;    // ceil(rows / 16)
    uint32_t kind;         // kQ4: the 576-byte tiles above; kQ8: the affine-Q8 stream below
};

// Affine Q8 (minimax_h3_q8_gemm_bf16_meta, minimax_h3_attention.metal:594-676): one code BYTE per weight,
// 64 per group, bf16 scale and bias per (row, group), w = half(float(scale) * q + float(bias)).  Stream of
// 8704-byte tiles of 128 rows x one group, ordered [128-row block][group]:
//   [0, 8192)     row r's 64 code bytes as four 16-byte pieces, piece p (columns 16 p .. 16 p + 15) at index
//                 4 r + ((p + r / 2) & 3): a warp whose lanes read piece p of 32 consecutive rows then touches
//                 every bank group four times, the minimum for 512 bytes
//   [8192, 8704)  128 records {bf16 scale, bf16 bias}, kept as bf16
constexpr int kQ8Rows = 128;
constexpr int kQ8CodeBytes = kQ8Rows * kGroup;          // 8192
constexpr int kQ8TileBytes = kQ8CodeBytes + kQ8Rows * 4;  // 8704
__host__ __device__ inline uint32_t q8_piece_index(uint32_t row, uint32_t piece) {
    return 4u * row + ((piece + (row >> 1)) & 3u);
}

__host__ __device__ inline uint32_t ceil_div(uint32_t a, uint32_t b) {
    return (a + b - 1) / b;
}

// position (in 16-byte pieces) of lane l's piece inside a tile: pieces of one gid
// stay in their 64-byte group, rotated by gid/2.  A warp reading piece t of 16
// different rows then touches every bank group instead of two.
__host__ __device__ inline uint32_t piece_index(uint32_t lane) {
    return (lane & ~3u) | (((lane & 3u) + (lane >> 3)) & 3u);
}

// byte offset of tile (rt, g) in a stream with G groups per row
__host__ __device__ inline size_t tile_offset(uint32_t rt, uint32_t g, uint32_t G) {
    return ((size_t)(rt / kBlockTiles) * G + g) * kUnitBytes + (size_t)(rt % kBlockTiles) * kTileBytes;
}

// ---------------------------------------------------------------------------
// nibble order of one 32-bit word: position p holds element kWordRow/kWordCol
// ---------------------------------------------------------------------------
// row offset (0 -> gid, 1 -> gid+8) and column offset (0..3) of nibble p
__host__ __device__ inline int word_row(int p) { return p & 1; }
__host__ __device__ inline int word_col(int p) {
    // p: 0 1 2 3 4 5 6 7 -> col 0 0 2 2 1 1 3 3
    return ((p >> 1) & 1) * 2 + (p >> 2);
}

// Build the four words of one lane from the two 64-bit raw row pieces
// (16 codes each, code c in nibble c).
__device__ inline uint4 swizzle_lane(uint64_t row_lo, uint64_t row_hi) {
    uint32_t out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t a = (uint32_t)(row_lo >> (16 * i)) & 0xffffu;
        uint32_t b = (uint32_t)(row_hi >> (16 * i)) & 0xffffu;
        uint32_t word = 0;
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            uint32_t source = word_row(p) ? b : a;
            word |= ((source >> (4 * word_col(p))) & 0xfu) << (4 * p);
        }
        out[i] = word;
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

// Inverse of swizzle_lane.
__device__ inline void unswizzle_lane(uint4 words, uint64_t &row_lo, uint64_t &row_hi) {
    const uint32_t in[4] = {words.x, words.y, words.z, words.w};
    row_lo = 0;
    row_hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            uint64_t code = (in[i] >> (4 * p)) & 0xfu;
            int shift = 16 * i + 4 * word_col(p);
            if (word_row(p)) {
                row_hi |= code << shift;
            } else {
                row_lo |= code << shift;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// dequantisation
// ---------------------------------------------------------------------------
// The four half2 registers of one word as exact small integers.
//   regs[0] = (gid  ; col 0,1)  regs[1] = (gid+8; col 0,1)
//   regs[2] = (gid  ; col 2,3)  regs[3] = (gid+8; col 2,3)
// 0x6400 | q is the fp16 number 1024 + q; 0x6400 | (q << 4) is 1024 + 16 q.
// Both subtractions / the fused multiply-add below are exact in fp16.
__device__ inline void word_to_codes_f16(uint32_t w, __half2 regs[4]) {
    const uint32_t kMagic = 0x64006400u;
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const __half2 kSixteenth = __half2half2(__ushort_as_half(0x2c00));  // 1/16
    const __half2 kMinus64 = __half2half2(__ushort_as_half(0xd400));    // -64
    uint32_t lo0, hi0, lo1, hi1;
    asm("lop3.b32 %0, %1, 0x000F000F, %2, 0xEA;" : "=r"(lo0) : "r"(w), "r"(kMagic));
    asm("lop3.b32 %0, %1, 0x00F000F0, %2, 0xEA;" : "=r"(hi0) : "r"(w), "r"(kMagic));
    uint32_t w8 = w >> 8;
    asm("lop3.b32 %0, %1, 0x000F000F, %2, 0xEA;" : "=r"(lo1) : "r"(w8), "r"(kMagic));
    asm("lop3.b32 %0, %1, 0x00F000F0, %2, 0xEA;" : "=r"(hi1) : "r"(w8), "r"(kMagic));
    regs[0] = __hsub2(*reinterpret_cast<__half2 *>(&lo0), k1024);
    regs[1] = __hfma2(*reinterpret_cast<__half2 *>(&hi0), kSixteenth, kMinus64);
    regs[2] = __hsub2(*reinterpret_cast<__half2 *>(&lo1), k1024);
    regs[3] = __hfma2(*reinterpret_cast<__half2 *>(&hi1), kSixteenth, kMinus64);
}

// Same registers as fp16 SUBNORMALS: the bit pattern q (or q << 4) is the fp16
// number q * 2^-24 (or 16 q * 2^-24).  No arithmetic at all; the caller folds
// 2^24 (rows gid) and 2^20 (rows gid+8) into the scale.
__device__ inline void word_to_codes_subnormal(uint32_t w, uint32_t regs[4]) {
    regs[0] = w & 0x000F000Fu;
    regs[1] = w & 0x00F000F0u;
    uint32_t w8 = w >> 8;
    regs[2] = w8 & 0x000F000Fu;
    regs[3] = w8 & 0x00F000F0u;
}

// W16 contract: fp16_rn(exact(scale * q + bias)), i.e. one fused multiply-add in
// fp16 on the exact integer code (qwen38_global.metal:26-27 rounds the fp32
// value once; for exact s*q+b the two agree).  No flush-to-zero: small results
// are fp16 subnormals and must survive.
__device__ inline __half2 dequant_w16(__half2 codes, __half2 scale, __half2 bias) {
    return __hfma2(scale, codes, bias);
}

// W32 contract: scale * (float)q + bias in fp32 (qwen38_m3.m:116).  s*q is exact
// in fp32, so the fused form rounds identically to multiply-then-add.
__device__ inline float dequant_w32(uint32_t code, float scale, float bias) {
    return __fmaf_rn(scale, (float)code, bias);
}

// ---------------------------------------------------------------------------
// seeded synthetic inputs (same counter-based generator as the CPU checker)
// ---------------------------------------------------------------------------
__host__ __device__ inline uint64_t finalize64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ inline uint64_t stream_key(uint64_t seed, uint64_t stream) {
    return finalize64(seed * 0x9E3779B97F4A7C15ull + finalize64(stream + 1ull));
}
__host__ __device__ inline uint64_t keyed(uint64_t key, uint64_t index) {
    return finalize64(key + (index + 1ull) * 0x9E3779B97F4A7C15ull);
}
__host__ __device__ inline float normal12(uint64_t a, uint64_t b, uint64_t c) {
    uint32_t sum = 0;
#pragma unroll
    for (int part = 0; part < 4; ++part) {
        sum += (uint32_t)((a >> (16 * part)) & 0xffffu);
        sum += (uint32_t)((b >> (16 * part)) & 0xffffu);
        sum += (uint32_t)((c >> (16 * part)) & 0xffffu);
    }
    return (float)((int32_t)sum - 393210) * (1.0f / 65536.0f);
}

}  // namespace q4b
