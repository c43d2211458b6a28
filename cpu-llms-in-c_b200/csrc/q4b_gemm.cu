// Prefill GEMM on the Q4 tile stream: tcgen05 tensor cores, accumulators in TMEM.
//
// Replaces the reference's batched tensor kernels: qwen38_prefill_q4_gemm_*_mma /
// _mma2 / _mma3 (qwen38_prefill.metal:811-1502) and minimax_h3_q4_gemm_f16_mma[_wide]
// (minimax_h3_attention.metal:211-404): Y[m][n] = sum_k w(n,k) X[m][k], fp16
// operands, fp32 accumulation over the whole K (no half-precision window).
//
// One CTA computes a 128 (weight rows) x BN (activation rows) output tile:
//   D[128][BN] (TMEM, fp32) += A[128][64] (TMEM, fp16) * B[BN][64]^T (shared memory)
// per quantisation group.  The WEIGHTS are the A operand and never exist as fp16
// in shared memory: warp 0 brings the group's 4.6 KB of Q4 tiles in with bulk
// copies and the X tile with a TMA tensor copy (128-byte swizzle); eight
// dequantisation warps (thread = weight row) turn the codes into
// w16 = fma(scale, q, bias) -- the bit-exact W16 contract -- and write them
// straight into TMEM with tcgen05.st; warp 1 issues four tcgen05.mma (K = 16 each)
// per group and commits to mbarriers that free the A slot and the stage.  A
// dequantised tile written to and re-read from shared memory next to the X tile
// would exceed one SM's shared-memory bandwidth; through TMEM it costs none.
// After the last group the same eight warps read D with tcgen05.ld, apply the
// epilogue (optional residual) and store Y.  Fused gate/up puts the 64 gate rows
// and the 64 up rows of the same 64 output features into one 128-row A tile, so
// the tensor cores still run full-width tiles; the epilogue pairs the two halves
// through shared memory and stores silu(gate) * up.  Every wait is bounded; on expiry the kernel records a code in the
// status word, releases its TMEM and returns.
#include "q4b_kernels.h"

#include <cstdlib>
#include <cuda.h>

namespace q4b {

namespace {

// ring stages (one quantisation group each); a multiple of the number of warpgroups, see the dequantisation loop
template <int BN, bool FUSED, bool Q8 = false>
struct TcStages {
    static constexpr int value = BN == 256 || Q8 ? 4 : 8;  // a Q8 stage holds 8.7 KB of weights, not 4.6
};
constexpr int kTcSlots = 8;        // A-operand slots in TMEM (32 columns each)
constexpr int kTcWarpgroups = 4;   // dequantisation warpgroups; group g belongs to warpgroup g % 4
static_assert(TcStages<256, false>::value % kTcWarpgroups == 0 && TcStages<128, false>::value % kTcWarpgroups == 0,
              "a warpgroup must meet every fill of the stages it uses");
constexpr int kTcThreads = 64 + kTcWarpgroups * 128;  // warp 0 producer, warp 1 MMA, then the warpgroups
constexpr long long kTcWaitLimit = 4000000000ll;

struct TcParams {
    CUtensorMap x_map;  // X [M][K] fp16, box 64 x BN, 128-byte swizzle
    WeightView w[kMaxSegments];  // matrices that share X (one launch), e.g. q, k, v
    WeightView up;               // second matrix of fused gate/up (single segment)
    void *y[kMaxSegments];
    uint32_t ldy[kMaxSegments];
    uint32_t block_begin[kMaxSegments + 1];  // prefix sums of row blocks over the segments
    int segments;
    const void *residual;        // segment 0 only
    uint32_t *status;
    uint32_t ld_residual;
    uint32_t m_rows, groups, n_blocks, m_blocks;
    uint32_t m_group;            // activation blocks walked together (see tc_tile_of)
    // stream-K (split != 0): the (tile, group) iterations are cut into equal contiguous ranges, one per CTA
    uint32_t split, iters_per_cta, iters_extra;
    void *peer_y[kMaxSegments][kMaxPeers];  // the same output block in the other ranks' memory (null: none)
    uint32_t peers;              // entries of peer_y in use (0 on a single GPU)
    float *workspace;            // [CTA][128][BN] fp32 partial tiles
    uint32_t *flags;             // [CTA] 1 while that CTA's partial tile waits to be added, else 0
    int y_dtype, residual_dtype;
};

__device__ inline uint32_t tc_smem_u32(const void *pointer) {
    return (uint32_t)__cvta_generic_to_shared(pointer);
}
__device__ inline void tc_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ inline void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ inline void tc_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ inline bool tc_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// false when the wait expired
__device__ inline bool tc_wait(uint32_t bar, uint32_t parity) {
    if (tc_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!tc_try_wait(bar, parity)) {
        if (clock64() - start > kTcWaitLimit) return false;
    }
    return true;
}
__device__ inline void tc_bulk_copy(uint32_t destination, const void *source, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(destination), "l"(source), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ inline void tc_tensor_copy_2d(uint32_t destination, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(destination), "l"(map), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
__device__ inline void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ inline void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ inline void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem_d] (+)= A[tmem_a] * B[desc]^T, M = 128, K = 16
__device__ inline void tc_mma(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ inline void tc_store_32(uint32_t address, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ inline void tc_load_16(uint32_t address, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address));
}


// Tile order: the activation blocks are walked in groups of `m_group`; inside a group every weight block
// meets every activation block of the group before the next weight block starts.  CTAs that run together
// then share a few weight blocks and a slice of X small enough to stay in L2, whatever M is.
__device__ inline void tc_tile_of(uint32_t tile, uint32_t n_blocks, uint32_t m_blocks, uint32_t m_group,
                                  uint32_t &nb_all, uint32_t &mb) {
    const uint32_t per_group = n_blocks * m_group;
    const uint32_t group = tile / per_group, rest = tile % per_group;
    const uint32_t first = group * m_group;
    const uint32_t width = min(m_group, m_blocks - first);   // the last group may be narrower
    nb_all = rest / width;
    mb = first + rest % width;
}

// The work of one CTA as all its roles walk it: a list of segments (tile, groups [g0, g1)).
// Without splitting a segment is a whole tile and the tiles are dealt round-robin.  With splitting
// (few tiles for many SMs) the tile-major sequence of (tile, group) iterations is cut into equal
// contiguous ranges; a tile cut in two or more is summed by the CTA that holds its first groups, which
// reaches them last in time -- the others left their partial tiles in the workspace long before.
struct TcWalk {
    uint32_t split, tile, tiles, step, i, i1, G;
    __device__ inline void start(const TcParams &p, uint32_t tiles_total) {
        split = p.split;
        G = p.groups;
        tiles = tiles_total;
        tile = blockIdx.x;
        step = gridDim.x;
        i = blockIdx.x * p.iters_per_cta + min(blockIdx.x, p.iters_extra);
        i1 = i + p.iters_per_cta + (blockIdx.x < p.iters_extra ? 1u : 0u);
    }
    __device__ inline bool next(uint32_t &t, uint32_t &g0, uint32_t &g1) {
        if (split == 0) {
            if (tile >= tiles) return false;
            t = tile;
            g0 = 0;
            g1 = G;
            tile += step;
            return true;
        }
        if (i >= i1) return false;
        t = i / G;
        g0 = i % G;
        g1 = min(G, g0 + (i1 - i));
        i += g1 - g0;
        return true;
    }
};
__device__ inline uint32_t tc_cta_of_iteration(const TcParams &p, uint32_t iteration) {
    const uint32_t boundary = p.iters_extra * (p.iters_per_cta + 1);
    return iteration < boundary ? iteration / (p.iters_per_cta + 1)
                                : p.iters_extra + (iteration - boundary) / p.iters_per_cta;
}

// BN   : activation rows per tile (columns of D)
// FUSED: the A tile is 64 rows of `w` (gate) over 64 rows of `up`; epilogue silu(gate) * up
// BF   : bf16 activations against weights rounded to bf16 (the arithmetic of
//        minimax_h3_q4_gemm_bf16_activation, minimax_h3_attention.metal:512-592, and of its CPU check,
//        minimax_h3_m3_real_gemm.c:25-42); otherwise fp16 activations against fp16 weights
// Q8   : the weights are an affine-Q8 stream (minimax_h3_q8_gemm_bf16_meta, minimax_h3_attention.metal:594-676):
//        one 8704-byte tile per group, w = half(float(scale) * q + float(bias)) with bf16 scale and bias
template <int BN, bool FUSED, bool BF, bool Q8 = false>
__global__ void __launch_bounds__(kTcThreads, 1)
tc_gemm_kernel(const __grid_constant__ TcParams p) {
    static_assert(!Q8 || (!FUSED && !BF), "the Q8 sibling is a plain fp16 GEMM");
    constexpr int kTcStages = TcStages<BN, FUSED, Q8>::value;
    constexpr uint32_t kXBytes = BN * 128;               // one group of X: BN rows x 64 halves
    constexpr uint32_t kWBytes = Q8 ? kQ8TileBytes : 2 * kUnitBytes;  // 128 rows of one group
    constexpr uint32_t kDCols = BN;
    constexpr uint32_t kTmemCols = kDCols + kTcSlots * 32 <= 256 ? 256 : 512;
    static_assert(kDCols + kTcSlots * 32 <= 512, "accumulators and A slots must fit the 512 TMEM columns");
    extern __shared__ uint8_t tc_smem_raw[];
    // 128-byte swizzle atoms need 1024-byte alignment in the shared window
    uint8_t *base = tc_smem_raw + ((1024u - (tc_smem_u32(tc_smem_raw) & 1023u)) & 1023u);
    uint8_t *xbuf = base;
    uint8_t *wbuf = base + kTcStages * kXBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(wbuf + kTcStages * kWBytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kTcStages + 2 * kTcSlots + 2);
    float *exchange = reinterpret_cast<float *>(tmem_slot + 4);  // epilogue staging: [warpgroups][16][128]
    const uint32_t full0 = tc_smem_u32(bars), empty0 = full0 + 8 * kTcStages;
    const uint32_t a_full0 = empty0 + 8 * kTcStages, a_free0 = a_full0 + 8 * kTcSlots;
    const uint32_t d_full = a_free0 + 8 * kTcSlots, d_free = d_full + 8;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t G = p.groups;
    const uint32_t tiles = p.n_blocks * p.m_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; ++s) {
            tc_mbar_init(full0 + 8 * s, 1);
            tc_mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < kTcSlots; ++a) {
            tc_mbar_init(a_full0 + 8 * a, 4);
            tc_mbar_init(a_free0 + 8 * a, 1);
        }
        tc_mbar_init(d_full, 1);
        tc_mbar_init(d_free, 4 * kTcWarpgroups);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tc_smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;          // D: columns [0, BN)
    const uint32_t tmem_a = tmem_d + kDCols;     // A slots: 32 columns each

    bool ok = true;
    if (warp == 0) {
        // ---- producer: Q4 tiles by bulk copy, X tile by TMA tensor copy ----
        if (lane == 0) {
            uint32_t it = 0, tile, g0, g1;
            TcWalk walk;
            walk.start(p, tiles);
            while (ok && walk.next(tile, g0, g1)) {
                uint32_t nb_all, mb;
                tc_tile_of(tile, p.n_blocks, p.m_blocks, p.m_group, nb_all, mb);
                int segment = 0;
#pragma unroll
                for (int q = 1; q < kMaxSegments; ++q) {
                    if (q < p.segments && nb_all >= p.block_begin[q]) segment = q;
                }
                const uint32_t nb = nb_all - p.block_begin[segment];
                const uint8_t *tiles = p.w[segment].tiles;
                for (uint32_t g = g0; g < g1; ++g, ++it) {
                    const uint32_t s = it % kTcStages;
                    if (it >= kTcStages && !tc_wait(empty0 + 8 * s, ((it / kTcStages) - 1) & 1)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = full0 + 8 * s;
                    tc_mbar_expect_tx(bar, kWBytes + kXBytes);
                    const uint32_t wdst = tc_smem_u32(wbuf) + s * kWBytes;
                    if constexpr (Q8) {
                        tc_bulk_copy(wdst, tiles + ((size_t)nb * G + g) * kQ8TileBytes, kQ8TileBytes, bar);
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint8_t *stream = FUSED && h == 1 ? p.up.tiles : tiles;
                            const uint32_t block = FUSED ? nb : nb * 2 + h;  // 64-row block of that stream
                            const size_t offset = ((size_t)block * G + g) * kUnitBytes;
                            tc_bulk_copy(wdst + h * kUnitBytes, stream + offset, kUnitBytes, bar);
                        }
                    }
                    tc_tensor_copy_2d(tc_smem_u32(xbuf) + s * kXBytes, &p.x_map, (int)(g * kGroup), (int)(mb * BN), bar);
                }
            }
            if (!ok) {
                atomicExch(p.status, 0x71u);
                // let copies already issued land before the shared memory is released
                for (uint32_t back = 0; back < kTcStages && back < it; ++back) {
                    const uint32_t j = it - 1 - back;
                    tc_wait(full0 + 8 * (j % kTcStages), (j / kTcStages) & 1);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            // D fp32; A and B fp16 (format 0) or bf16 (format 1, bits 7 and 10); N and M
            const uint32_t idesc = (1u << 4) | (BF ? (1u << 7) | (1u << 10) : 0u) | ((uint32_t)(BN >> 3) << 17) |
                                   ((128u >> 4) << 24);
            const uint64_t desc_base = ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
                                       ((uint64_t)2 << 61);
            uint32_t it = 0, unit = 0, tile_iter = 0, tile, g0, g1;
            TcWalk walk;
            walk.start(p, tiles);
            for (; ok && walk.next(tile, g0, g1); ++tile_iter) {
                if (tile_iter > 0 && !tc_wait(d_free, (tile_iter - 1) & 1)) { ok = false; break; }
                tc_fence_after();
                for (uint32_t g = g0; g < g1 && ok; ++g, ++it) {
                    const uint32_t s = it % kTcStages;
                    if (!tc_wait(full0 + 8 * s, (it / kTcStages) & 1)) { ok = false; break; }
                    const uint32_t xaddr = tc_smem_u32(xbuf) + s * kXBytes;
                    const uint32_t a = unit % kTcSlots;
                    if (!tc_wait(a_full0 + 8 * a, (unit / kTcSlots) & 1)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint64_t desc = desc_base | (uint64_t)(((xaddr + kk * 32) >> 4) & 0x3fffu);
                        tc_mma(tmem_d, tmem_a + a * 32 + kk * 8, desc, idesc, (g > g0 || kk > 0) ? 1u : 0u);
                    }
                    ++unit;
                    tc_commit(a_free0 + 8 * a);  // the slot may be rewritten once these MMAs retire
                    tc_commit(empty0 + 8 * s);   // and the stage refilled
                }
                if (ok) tc_commit(d_full);
            }
            if (!ok) atomicExch(p.status, 0x72u);
        }
    } else {
        // ---- dequantisation (thread = weight row) and epilogue ----
        const uint32_t wg = (uint32_t)(warp - 2) >> 2, quad = warp & 3;
        const uint32_t row = quad * 32 + lane;  // row of the 128-row tile == TMEM lane
        const uint32_t lane_field = (quad * 32) << 16;
        const uint32_t r64 = row & 63, gid = r64 & 7, hi = (r64 >> 3) & 1;
        const uint32_t tile_offset_bytes = (row >> 6) * kUnitBytes + (r64 >> 4) * kTileBytes;
        // rows gid+8 sit in the odd nibbles: 0x6400 | (q << 4) is 1024 + 16 q
        const uint32_t mask = hi ? 0x00F000F0u : 0x000F000Fu;
        const __half2 to_code_mul = __half2half2(__ushort_as_half(hi ? 0x2c00 : 0x3c00));  // 1/16 or 1
        const __half2 to_code_add = __half2half2(__ushort_as_half(hi ? 0xd400 : 0xe400));  // -64 or -1024
        uint32_t it = 0, unit = 0, tile_iter = 0, tile, g0, g1;
        TcWalk walk;
        walk.start(p, tiles);
        for (; ok && walk.next(tile, g0, g1); ++tile_iter) {
            uint32_t nb_all, mb;
            tc_tile_of(tile, p.n_blocks, p.m_blocks, p.m_group, nb_all, mb);
            int segment = 0;
#pragma unroll
            for (int q = 1; q < kMaxSegments; ++q) {
                if (q < p.segments && nb_all >= p.block_begin[q]) segment = q;
            }
            const uint32_t nb = nb_all - p.block_begin[segment];
            for (uint32_t g = g0; g < g1 && ok; ++g, ++it) {
                const uint32_t s = it % kTcStages;
                for (int once = 0; once < 1; ++once, ++unit) {
                    if (unit % kTcWarpgroups != wg) continue;  // the warpgroups take groups in turn
                    const uint32_t a = unit % kTcSlots;
                    // A warpgroup waits only for its own groups' stages.  That is sound because the number of
                    // stages is a multiple of the number of warpgroups: it then meets every fill of the stages it
                    // uses (a parity wait that skips a fill is satisfied by the fill before last), and a stage it is
                    // still waiting for cannot be refilled, since the MMA that frees it needs this warpgroup's A tile.
                    if (!tc_wait(full0 + 8 * s, (it / kTcStages) & 1)) { ok = false; break; }
                    uint32_t regs[32];
                    if constexpr (Q8) {
                        // thread = weight row: 64 code bytes in four pieces, one {bf16 scale, bf16 bias} record;
                        // 0x4B0000qq is the float 8388608 + q, so q comes out exact with one subtraction; the
                        // product with the bf16 scale is exact in fp32, the sum rounds once, then once to fp16
                        const uint8_t *tile_q8 = wbuf + s * kWBytes;
                        const uint32_t record = reinterpret_cast<const uint32_t *>(tile_q8 + kQ8CodeBytes)[row];
                        const float scale_f = __uint_as_float(record << 16), bias_f = __uint_as_float(record & 0xffff0000u);
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const uint4 piece = reinterpret_cast<const uint4 *>(tile_q8)[q8_piece_index(row, t)];
                            const uint32_t word[4] = {piece.x, piece.y, piece.z, piece.w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                float value[4];
#pragma unroll
                                for (int b = 0; b < 4; ++b) {
                                    const uint32_t bits = __byte_perm(word[i], 0x4B000000u, 0x7540 + b);
                                    value[b] = __fmaf_rn(scale_f, __uint_as_float(bits) - 8388608.0f, bias_f);
                                }
                                const __half2 w01 = __floats2half2_rn(value[0], value[1]);
                                const __half2 w23 = __floats2half2_rn(value[2], value[3]);
                                regs[8 * t + 2 * i] = *reinterpret_cast<const uint32_t *>(&w01);
                                regs[8 * t + 2 * i + 1] = *reinterpret_cast<const uint32_t *>(&w23);
                            }
                        }
                    } else {
                    const uint8_t *tile_bytes = wbuf + s * kWBytes + tile_offset_bytes;
                    const uint32_t record = *reinterpret_cast<const uint32_t *>(tile_bytes + kTileCodeBytes + gid * 8 + hi * 4);
                    const __half2 sb = *reinterpret_cast<const __half2 *>(&record);
                    const __half2 scale = __half2half2(__low2half(sb)), bias = __half2half2(__high2half(sb));
                    // bf16 weights: scale and bias come back from the fp16 record unchanged when the planes were
                    // bf16 to begin with (every bf16 in fp16's normal range is an fp16)
                    const __nv_bfloat162 scale_b = __float2bfloat162_rn(__low2float(sb));
                    const __nv_bfloat162 bias_b = __float2bfloat162_rn(__high2float(sb));
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const uint4 piece = *reinterpret_cast<const uint4 *>(tile_bytes + piece_index(gid * 4 + t) * 16);
                        const uint32_t word[4] = {piece.x, piece.y, piece.z, piece.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if constexpr (BF) {
                                // 0x4300 | q is 128 + q in bf16 (seven fraction bits), so the odd nibbles are
                                // shifted down first; q = (128 + q) - 128 exactly, then one fused multiply-add
                                // rounds s q + b to bf16 once
                                const uint32_t wa = word[i] >> (hi ? 4 : 0), wb = word[i] >> (hi ? 12 : 8);
                                uint32_t v01, v23;
                                asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(v01) : "r"(wa));
                                asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(v23) : "r"(wb));
                                const __nv_bfloat162 offset = __float2bfloat162_rn(128.0f);
                                const __nv_bfloat162 q01 = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&v01), offset);
                                const __nv_bfloat162 q23 = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&v23), offset);
                                const __nv_bfloat162 w01 = __hfma2(q01, scale_b, bias_b);
                                const __nv_bfloat162 w23 = __hfma2(q23, scale_b, bias_b);
                                regs[8 * t + 2 * i] = *reinterpret_cast<const uint32_t *>(&w01);
                                regs[8 * t + 2 * i + 1] = *reinterpret_cast<const uint32_t *>(&w23);
                                continue;
                            }
                            uint32_t v01, v23;
                            const uint32_t w8 = word[i] >> 8;
                            asm("lop3.b32 %0, %1, %2, 0x64006400, 0xEA;" : "=r"(v01) : "r"(word[i]), "r"(mask));
                            asm("lop3.b32 %0, %1, %2, 0x64006400, 0xEA;" : "=r"(v23) : "r"(w8), "r"(mask));
                            const __half2 q01 = __hfma2(*reinterpret_cast<__half2 *>(&v01), to_code_mul, to_code_add);
                            const __half2 q23 = __hfma2(*reinterpret_cast<__half2 *>(&v23), to_code_mul, to_code_add);
                            const __half2 w01 = dequant_w16(q01, scale, bias);
                            const __half2 w23 = dequant_w16(q23, scale, bias);
                            regs[8 * t + 2 * i] = *reinterpret_cast<const uint32_t *>(&w01);
                            regs[8 * t + 2 * i + 1] = *reinterpret_cast<const uint32_t *>(&w23);
                        }
                    }
                    }
                    if (unit >= kTcSlots && !tc_wait(a_free0 + 8 * a, ((unit / kTcSlots) - 1) & 1)) { ok = false; break; }
                    tc_fence_after();
                    tc_store_32(tmem_a + a * 32 + lane_field, regs);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc_mbar_arrive(a_full0 + 8 * a);
                }
            }
            if (!ok) break;
            // ---- epilogue: this warp's 32 rows x half of the columns ----
            if (!tc_wait(d_full, tile_iter & 1)) { ok = false; break; }
            tc_fence_after();
            void *y_out = p.y[segment];
            const uint32_t ldy = p.ldy[segment];
            float *swap = exchange + wg * (16 * 128);   // this warpgroup's 8 KB of the output staging buffer
            constexpr uint32_t kColumnsPerGroup = BN / kTcWarpgroups;
            if (g0 > 0) {
                // ---- a later part of a split tile: leave the partial sums for the CTA that holds the first groups ----
                float *mine = p.workspace + ((size_t)blockIdx.x * 128 + row) * BN;
#pragma unroll 1
                for (uint32_t c = wg * kColumnsPerGroup; c < (wg + 1) * kColumnsPerGroup; c += 16) {
                    uint32_t d0[16];
                    tc_load_16(tmem_d + c + lane_field, d0);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        *reinterpret_cast<float4 *>(mine + c + j) =
                            make_float4(__uint_as_float(d0[j]), __uint_as_float(d0[j + 1]), __uint_as_float(d0[j + 2]),
                                        __uint_as_float(d0[j + 3]));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(d_free);
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"r"(kTcWarpgroups * 128) : "memory");
                if (threadIdx.x == 64) {
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.flags + blockIdx.x), "r"(1u) : "memory");
                }
                continue;
            }
            uint32_t partial_first = 0, partial_count = 0;
            if (g1 < G) {
                // ---- the first part of a split tile: every later part was finished long ago by its CTA ----
                partial_first = blockIdx.x + 1;
                partial_count = tc_cta_of_iteration(p, tile * G + G - 1) - blockIdx.x;
                if (threadIdx.x == 64) {
                    const long long start = clock64();
                    for (uint32_t q = 0; q < partial_count; ++q) {
                        uint32_t ready = 0;
                        for (;;) {
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(ready) : "l"(p.flags + partial_first + q) : "memory");
                            if (ready != 0) break;
                            if (clock64() - start > kTcWaitLimit) {
                                atomicExch(p.status, 0x74u);
                                break;
                            }
                            __nanosleep(64);
                        }
                        p.flags[partial_first + q] = 0;  // consumed: ready for the next launch
                    }
                    __threadfence();
                }
                asm volatile("bar.sync 1, %0;" ::"r"(kTcWarpgroups * 128) : "memory");
            }
#pragma unroll 1
            for (uint32_t c = wg * kColumnsPerGroup; c < (wg + 1) * kColumnsPerGroup; c += 16) {
                uint32_t d0[16];
                tc_load_16(tmem_d + c + lane_field, d0);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                for (uint32_t q = 0; q < partial_count; ++q) {  // partial tiles in CTA order
                    const float *theirs = p.workspace + ((size_t)(partial_first + q) * 128 + row) * BN + c;
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const float4 v = __ldcg(reinterpret_cast<const float4 *>(theirs + j));
                        d0[j] = __float_as_uint(__uint_as_float(d0[j]) + v.x);
                        d0[j + 1] = __float_as_uint(__uint_as_float(d0[j + 1]) + v.y);
                        d0[j + 2] = __float_as_uint(__uint_as_float(d0[j + 2]) + v.z);
                        d0[j + 3] = __float_as_uint(__uint_as_float(d0[j + 3]) + v.w);
                    }
                }
                // The chunk (16 activation rows x this warpgroup's output features) goes through shared memory
                // transposed, so that the stores are 32 or 64 contiguous bytes per thread and whole 128/256-byte
                // rows per eight threads -- for the peers' copies over NVLink as much as for the own.
                constexpr uint32_t kFeatures = FUSED ? 64 : 128;   // output features of the tile
                float *tile_out = swap;                             // [16][kFeatures]
                if (FUSED) {
                    // rows 64..127 hold `up` of the feature whose `gate` sits 64 rows above
                    if (row >= 64) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) tile_out[j * kFeatures + (row - 64)] = __uint_as_float(d0[j]);
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + wg) : "memory");
                    if (row < 64) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            // silu(g) * u from the un-rounded accumulators (qwen38_q4.metal:146-149)
                            const float gate = __uint_as_float(d0[j]);
                            tile_out[j * kFeatures + row] = (gate / (1.0f + __expf(-gate))) * tile_out[j * kFeatures + row];
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) tile_out[j * kFeatures + row] = __uint_as_float(d0[j]);
                }
                asm volatile("bar.sync %0, 128;" ::"r"(2 + wg) : "memory");
                {
                    const uint32_t unit = row;                          // 0..127: (activation row j, span of 16 features)
                    constexpr uint32_t kSpans = kFeatures / 16;
                    const uint32_t j = unit / kSpans, span = unit % kSpans;
                    const uint32_t m = mb * BN + c + j;
                    const uint32_t n0 = (FUSED ? nb * 64 : nb * 128) + span * 16;
                    const uint32_t rows_total = p.w[segment].rows;
                    if (unit < 16 * kSpans && m < p.m_rows && n0 < rows_total) {
                        float v[16];
#pragma unroll
                        for (int q = 0; q < 16; q += 4) {
                            const float4 f = *reinterpret_cast<const float4 *>(tile_out + j * kFeatures + span * 16 + q);
                            v[q] = f.x; v[q + 1] = f.y; v[q + 2] = f.z; v[q + 3] = f.w;
                        }
                        const uint32_t valid = min(16u, rows_total - n0);
                        if (p.residual != nullptr && segment == 0) {
                            const size_t at = (size_t)m * p.ld_residual + n0;
#pragma unroll
                            for (int q = 0; q < 16; ++q) {
                                if ((uint32_t)q < valid) {
                                    v[q] += p.residual_dtype == kF32
                                                ? reinterpret_cast<const float *>(p.residual)[at + q]
                                            : p.residual_dtype == kBF16
                                                ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p.residual)[at + q])
                                                : __half2float(reinterpret_cast<const __half *>(p.residual)[at + q]);
                                }
                            }
                        }
                        const size_t at = (size_t)m * ldy + n0;
                        const bool f32 = p.y_dtype == kF32;
                        const bool wide = valid == 16 && ((at * (f32 ? 4 : 2)) & 15u) == 0;
                        uint4 packed[4];
                        if (f32) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                packed[q] = make_uint4(__float_as_uint(v[4 * q]), __float_as_uint(v[4 * q + 1]),
                                                       __float_as_uint(v[4 * q + 2]), __float_as_uint(v[4 * q + 3]));
                            }
                        } else if (p.y_dtype == kBF16) {
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                __nv_bfloat162 h[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[8 * q + 2 * e], v[8 * q + 2 * e + 1]);
                                packed[q] = make_uint4(*reinterpret_cast<uint32_t *>(&h[0]), *reinterpret_cast<uint32_t *>(&h[1]),
                                                       *reinterpret_cast<uint32_t *>(&h[2]), *reinterpret_cast<uint32_t *>(&h[3]));
                            }
                        } else {
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                __half2 h[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(v[8 * q + 2 * e], v[8 * q + 2 * e + 1]);
                                packed[q] = make_uint4(*reinterpret_cast<uint32_t *>(&h[0]), *reinterpret_cast<uint32_t *>(&h[1]),
                                                       *reinterpret_cast<uint32_t *>(&h[2]), *reinterpret_cast<uint32_t *>(&h[3]));
                            }
                        }
                        // own copy first, then every peer's (column-parallel ranks: plain stores over NVLink)
                        for (uint32_t r = 0; r <= p.peers; ++r) {
                            void *destination = r == 0 ? y_out : p.peer_y[segment][r - 1];
                            if (destination == nullptr) continue;
                            if (wide) {
                                uint4 *out = reinterpret_cast<uint4 *>(static_cast<uint8_t *>(destination) + at * (f32 ? 4 : 2));
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    if (f32 || q < 2) out[q] = packed[q];
                                }
                            } else {
#pragma unroll
                                for (int q = 0; q < 16; ++q) {
                                    if ((uint32_t)q >= valid) continue;
                                    if (f32) {
                                        reinterpret_cast<float *>(destination)[at + q] = v[q];
                                    } else if (p.y_dtype == kBF16) {
                                        reinterpret_cast<__nv_bfloat16 *>(destination)[at + q] = __float2bfloat16_rn(v[q]);
                                    } else {
                                        reinterpret_cast<__half *>(destination)[at + q] = __float2half_rn(v[q]);
                                    }
                                }
                            }
                        }
                    }
                }
                asm volatile("bar.sync %0, 128;" ::"r"(2 + wg) : "memory");  // the buffer is free for the next chunk
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(d_free);
        }
        if (!ok && lane == 0) atomicExch(p.status, 0x73u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime, so the library links libcudart only
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn function = nullptr;
    if (function == nullptr) {
        void *pointer = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pointer, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess) {
            function = reinterpret_cast<EncodeTiledFn>(pointer);
        }
    }
    return function;
}

template <int BN, bool FUSED, bool BF, bool Q8 = false>
cudaError_t launch_tc_instance(TcParams &p, const TcGemmArgs &args, int sm_count, cudaStream_t stream) {
    EncodeTiledFn encode = encode_tiled();
    if (encode == nullptr) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {(cuuint64_t)args.w[0].groups * kGroup, (cuuint64_t)args.m_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)args.w[0].groups * kGroup * sizeof(__half)};
    const cuuint32_t box[2] = {(cuuint32_t)kGroup, (cuuint32_t)BN};
    const cuuint32_t element_strides[2] = {1, 1};
    if (encode(&p.x_map, BF ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(args.x), dims, strides, box,
               element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
        return cudaErrorInvalidValue;
    }
    p.m_blocks = ceil_div(args.m_rows, BN);
    // about 32 MB of X per group of activation blocks
    const size_t block_bytes = (size_t)BN * args.w[0].groups * kGroup * sizeof(__half);
    p.m_group = (uint32_t)((size_t)(32u << 20) / block_bytes);
    if (p.m_group < 1) p.m_group = 1;
    if (p.m_group > p.m_blocks) p.m_group = p.m_blocks;
    const uint32_t tiles = p.n_blocks * p.m_blocks;
    constexpr int kTcStages = TcStages<BN, FUSED, Q8>::value;
    const size_t smem_bytes = (size_t)kTcStages * (BN * 128 + (Q8 ? kQ8TileBytes : 2 * kUnitBytes)) +
                              (2 * kTcStages + 2 * kTcSlots + 2) * 8 + 16 + kTcWarpgroups * 16 * 128 * 4 + 1024;
    auto kernel = tc_gemm_kernel<BN, FUSED, BF, Q8>;
    static bool configured[kMaxDevices];  // per instantiation and device
    const int slot = device_slot();
    if (slot < 0 || !configured[slot]) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        if (status != cudaSuccess) return status;
        if (slot >= 0) configured[slot] = true;
    }
    unsigned grid = tiles < (uint32_t)sm_count ? tiles : (unsigned)sm_count;
    // Few tiles for many SMs: whole tiles would leave SMs idle (80 tiles on 148 SMs) or a thin last wave
    // (160 on 148).  The iterations can be split evenly over any number of CTAs instead.  In units of one
    // group's MMAs a CTA then works through iterations / CTAs, and a tile that is cut costs about 48 for leaving
    // and adding the first partial tile plus 25 for every further part, which its owner adds one after the
    // other (fitted: 17408 -> 5120 at M = 512 whole 129 us, over 148 CTAs 104 us; an eighth of it over 148
    // CTAs 108 us, i.e. worse than whole).  The cheapest count wins, whole tiles included.
    const uint32_t rounds = ceil_div(tiles, (uint32_t)sm_count);
    const uint64_t iterations = (uint64_t)tiles * p.groups;
    const double whole_cost = (double)rounds * p.groups;
    double best_cost = whole_cost;
    unsigned best_grid = 0;
    if (args.workspace != nullptr && getenv("Q4B_GEMM_WHOLE_TILES") == nullptr &&
        (size_t)sm_count * 128 * BN * sizeof(float) <= args.workspace_bytes) {
        for (unsigned candidate = 2; candidate <= (unsigned)sm_count; ++candidate) {
            if (iterations < (uint64_t)candidate * 8) break;
            const double parts = (double)candidate / tiles;  // CTAs per tile (tiles per CTA when below one)
            const double cut = parts > 1.0 ? 48.0 + 25.0 * (parts - 1.0) : 48.0;
            const double cost = (double)ceil_div((uint32_t)iterations, candidate) + cut;
            if (cost < 0.92 * whole_cost && cost < best_cost) {
                best_cost = cost;
                best_grid = candidate;
            }
        }
    }
    p.split = 0;
    if (best_grid != 0) {
        p.split = 1;
        grid = best_grid;
        p.iters_per_cta = (uint32_t)(iterations / grid);
        p.iters_extra = (uint32_t)(iterations % grid);
        p.workspace = args.workspace;
        p.flags = args.flags;
        // CTAs wait on one another: all of them must be resident
        void *arguments[] = {&p};
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(kernel), dim3(grid), dim3(kTcThreads), arguments,
                                           smem_bytes, stream);
    }
    kernel<<<grid, kTcThreads, smem_bytes, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_tc_gemm(const TcGemmArgs &args, int sm_count, cudaStream_t stream) {
    if (args.m_rows == 0 || args.segments < 1 || args.segments > kMaxSegments) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(args.x) & 15u) != 0) return cudaErrorInvalidValue;
    if (args.fused_silu && args.segments != 1) return cudaErrorInvalidValue;
    TcParams p = {};
    uint32_t blocks = 0;
    for (int s = 0; s < args.segments; ++s) {
        p.w[s] = args.w[s];
        p.y[s] = args.y[s];
        p.ldy[s] = args.ldy[s];
        p.block_begin[s] = blocks;
        blocks += ceil_div(args.w[s].rows, args.fused_silu ? 64 : 128);
    }
    for (int s = args.segments; s <= kMaxSegments; ++s) p.block_begin[s] = blocks;
    p.segments = args.segments;
    p.up = args.up;
    p.peers = args.peers;
    for (int s = 0; s < kMaxSegments; ++s) {
        for (int r = 0; r < kMaxPeers; ++r) p.peer_y[s][r] = (uint32_t)r < args.peers ? args.peer_y[s][r] : nullptr;
    }
    p.residual = args.residual;
    p.status = args.status;
    p.ld_residual = args.ld_residual;
    p.m_rows = args.m_rows;
    p.groups = args.w[0].groups;
    p.n_blocks = blocks;
    if (blocks == 0) return cudaSuccess;
    p.y_dtype = args.y_dtype;
    p.residual_dtype = args.residual_dtype;
    if (args.w[0].kind == kQ8) {
        if (args.x_bf16 || args.fused_silu || args.segments != 1) return cudaErrorInvalidValue;
        return args.m_rows <= 128 ? launch_tc_instance<128, false, false, true>(p, args, sm_count, stream)
                                  : launch_tc_instance<256, false, false, true>(p, args, sm_count, stream);
    }
    if (args.x_bf16) {
        if (args.fused_silu) {
            return args.m_rows <= 128 ? launch_tc_instance<128, true, true>(p, args, sm_count, stream)
                                      : launch_tc_instance<256, true, true>(p, args, sm_count, stream);
        }
        return args.m_rows <= 128 ? launch_tc_instance<128, false, true>(p, args, sm_count, stream)
                                  : launch_tc_instance<256, false, true>(p, args, sm_count, stream);
    }
    if (args.fused_silu) {
        return args.m_rows <= 128 ? launch_tc_instance<128, true, false>(p, args, sm_count, stream)
                                  : launch_tc_instance<256, true, false>(p, args, sm_count, stream);
    }
    return args.m_rows <= 128 ? launch_tc_instance<128, false, false>(p, args, sm_count, stream)
                              : launch_tc_instance<256, false, false>(p, args, sm_count, stream);
}

// fp32 activations -> fp16 (the tensor pipe multiplies fp16)
__global__ void convert_f32_to_f16_kernel(const float *in, __half *out, size_t count) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        out[i] = __float2half_rn(in[i]);
    }
}

struct RankBarrierParams {
    uint32_t *counters[kMaxPeers];
    uint32_t world, rank;
    uint32_t *round;  // device word of this rank: barriers passed so far
    uint32_t *status;
};
// Kernels of different GPUs wait for one another here, never two launches on one GPU.  Launched as a programmatic
// dependent of the kernel before it and letting its own successor start early: the next projection's weights
// stream while the ranks meet.
__global__ void rank_barrier_kernel(const RankBarrierParams p) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the launches before this one are complete and visible
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const uint32_t round = *p.round + 1;
    *p.round = round;
    // everything this GPU stored into the peers' memory before this launch is ordered before the adds
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    for (uint32_t r = 0; r < p.world; ++r) {
        asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.counters[r]), "r"(1u) : "memory");
    }
    const uint32_t expected = p.world * round;
    const long long start = clock64();
    for (;;) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.counters[p.rank]) : "memory");
        if ((int32_t)(seen - expected) >= 0) break;
        if (clock64() - start > kTcWaitLimit) {
            atomicExch(p.status, 0x91u);
            break;
        }
    }
}

cudaError_t launch_rank_barrier(uint32_t *const *counters, uint32_t world, uint32_t rank, uint32_t *round,
                                uint32_t *status, cudaStream_t stream) {
    if (world == 0 || world > (uint32_t)kMaxPeers || rank >= world) return cudaErrorInvalidValue;
    RankBarrierParams p = {};
    for (uint32_t r = 0; r < world; ++r) p.counters[r] = counters[r];
    p.world = world;
    p.rank = rank;
    p.round = round;
    p.status = status;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(1);
    config.blockDim = dim3(32);
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, rank_barrier_kernel, p);
}

cudaError_t launch_convert_f32_to_f16(const float *in, __half *out, size_t count, cudaStream_t stream) {
    if (count == 0) return cudaSuccess;
    size_t blocks = (count + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    convert_f32_to_f16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(in, out, count);
    return cudaGetLastError();
}

}  // namespace q4b
