// Decode sequences: a list of Q4 projections executed by ONE persistent launch.
//
// The reference encodes a whole token -- every layer's fixed chain of Q4 matmuls --
// into one command buffer (qwen38_m3_decode.m:1614-1690).  At M = 1 on a B200 each
// projection streams for only a few microseconds, so a kernel boundary per
// projection (drain, launch, refill the pipeline) costs as much as the work.  Here
// the chain is a job table in device memory and one cooperative grid walks it:
//
//   * the producer warp of every CTA streams job after job through the same
//     shared-memory ring (cp.async.bulk + mbarrier) without ever draining it:
//     weights never depend on earlier jobs, so the next job's tiles arrive while
//     this job's sums are still being combined;
//   * jobs form a chain: before a CTA reads x of job j it waits (bounded) until
//     every CTA has published job j-1's outputs -- the same ordering as separate
//     dependent launches, at the cost of one counter in L2;
//   * the per-job work split, arithmetic and cross-CTA sums are those of the
//     single-projection kernel (q4b_gemv.cu): mma.sync m16n8k16 on the exact codes,
//     per-group scale/bias in fp32, deterministic slot sums for split row blocks.
//
// With peers set (column-parallel ranks, one process per GPU) the epilogue stores
// this rank's output slice into every rank's copy of y over NVLink and the
// completion counter of every rank is advanced, so the gather is part of the same
// kernel: no collective call per projection.
#include "q4b_kernels.h"

#include <cstdlib>

#include <cooperative_groups.h>

#ifdef Q4B_TRACE
__device__ long long q4b_decode_trace[1024 * 8];
#define SQ_CLOCK() clock64()
#define SQ_ADD(slot, since) do { if (threadIdx.x == 0) q4b_decode_trace[blockIdx.x * 8 + (slot)] += clock64() - (since); } while (0)
extern "C" int q4b_decode_trace_read(long long *out, int count) {
    return (int)cudaMemcpyFromSymbol(out, q4b_decode_trace, sizeof(long long) * count);
}
#else
#define SQ_CLOCK() 0ll
#define SQ_ADD(slot, since) do { } while (0)
#endif

namespace q4b {

namespace {

constexpr int kSeqMaxStages = 8;
constexpr int kSeqWarps = 8;  // consumer warps; warp 8 produces
constexpr long long kSeqWaitLimit = 4000000000ll;

struct SeqParams {
    const DecodeJob *jobs;
    uint32_t job_count;
    uint32_t stages;
    uint32_t m_rows;
    uint32_t max_local_blocks;
    uint32_t world;           // ranks that publish into `done` (1 without peers)
    uint32_t rank;
    uint32_t epoch;           // launches so far, this one included: `done` counts up across launches
    uint32_t *done;           // [job_count] CTAs (of all ranks) that published the job's outputs
    uint32_t *peer_done[kMaxPeers];  // the same array on every rank (index `rank` = own)
    float *scratch;
    uint32_t *counters;
    uint32_t *status;
};

__device__ inline uint32_t sq_smem_u32(const void *pointer) { return (uint32_t)__cvta_generic_to_shared(pointer); }
__device__ inline void sq_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ inline void sq_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ inline void sq_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ inline bool sq_try_wait(uint32_t bar, uint32_t parity) {
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
__device__ inline bool sq_wait(uint32_t bar, uint32_t parity) {  // false when the wait expired
    if (sq_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!sq_try_wait(bar, parity)) {
        if (clock64() - start > kSeqWaitLimit) return false;
    }
    return true;
}
__device__ inline void sq_bulk_copy(uint32_t destination, const void *source, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(destination), "l"(source), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ inline void sq_consumer_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ inline void sq_mma(float d[4], const uint32_t a[4], uint32_t b0, uint32_t b1, bool first) {
    if (first) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
    } else {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

__device__ inline uint32_t sq_cta_of_unit(uint32_t unit, uint32_t share, uint32_t extra) {
    const uint32_t boundary = extra * (share + 1);
    return unit < boundary ? unit / (share + 1) : extra + (unit - boundary) / share;
}

// unit range [u0, u0 + range) of CTA `cta` in job `job`
__device__ inline void sq_range(const DecodeJob &job, uint32_t cta, uint32_t &u0, uint32_t &range) {
    if (cta >= job.active_ctas) {
        u0 = 0;
        range = 0;
    } else if (job.parts > 0) {
        const uint32_t block = cta / job.parts, j = cta % job.parts;
        const uint32_t from = job.groups * j / job.parts, to = job.groups * (j + 1) / job.parts;
        u0 = block * job.groups + from;
        range = to - from;
    } else {
        u0 = cta * job.units_per_cta + min(cta, job.units_extra);
        range = job.units_per_cta + (cta < job.units_extra ? 1u : 0u);
    }
}

__device__ inline int sq_segment_of(const DecodeJob &job, uint32_t grb) {
    int segment = 0;
#pragma unroll
    for (int q = 1; q < kMaxSegments; ++q) {
        if (q < (int)job.segments && grb >= job.block_begin[q]) segment = q;
    }
    return segment;
}


// NT: 8-column output tiles per warp (M <= 8*NT).  Warps 0..7 consume, warp 8
// produces.  A ring stage holds 16 sub-units of 2304 bytes of ONE 64-row block:
// 16 consecutive groups, or 8 groups of gate followed by the same 8 groups of up.
// Consumer warp w takes sub-units w and w + 8.
template <int NT>
__global__ void __launch_bounds__(288, NT > 1 ? 1 : 2)
decode_sequence_kernel(const SeqParams p) {
    constexpr int W = kSeqWarps;
    constexpr uint32_t kStageBytes = 16 * kUnitBytes;       // 36,864
    constexpr uint32_t kPerBlock = 2 * NT * 4 * 128;         // floats of one 64-row block (gate + up planes)
    extern __shared__ __align__(128) uint8_t sq_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, t = lane & 3;
    const uint32_t cta = blockIdx.x, stages = p.stages;

    uint64_t *bars = reinterpret_cast<uint64_t *>(sq_smem);  // full[8], empty[8]
    uint8_t *ring = sq_smem + 128;
    float *red = reinterpret_cast<float *>(ring + (size_t)stages * kStageBytes);   // [L][kPerBlock]
    uint32_t *flags = reinterpret_cast<uint32_t *>(red + (size_t)p.max_local_blocks * kPerBlock);
    float *part = reinterpret_cast<float *>(flags + ((p.max_local_blocks + 3u) & ~3u));  // [W][512], M <= 4 only
    const uint32_t full0 = sq_smem_u32(bars), empty0 = sq_smem_u32(bars + kSeqMaxStages);
    const uint32_t ring0 = sq_smem_u32(ring);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) {
            sq_mbar_init(full0 + 8 * s, 1);
            sq_mbar_init(empty0 + 8 * s, W);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        flags[0] = 0;
    }
    __syncthreads();

    if (warp == W) {
        // ---- producer: stream every job's byte range, never draining the ring ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t j = 0; j < p.job_count && ok; ++j) {
                const DecodeJob &job = p.jobs[j];
                const uint32_t G = job.groups, per_stage = job.fused ? 8u : 16u;
                uint32_t u0, range;
                sq_range(job, cta, u0, range);
                uint32_t ua = u0, g = range > 0 ? u0 % G : 0;
                const uint32_t u1 = u0 + range;
                while (ua < u1) {
                    const uint32_t s = it % stages;
                    if (it >= stages && !sq_wait(empty0 + 8 * s, ((it / stages) - 1) & 1)) {
                        ok = false;
                        break;
                    }
                    const uint32_t count = min(min(per_stage, G - g), u1 - ua);  // never across a row block
                    const uint32_t bytes = count * kUnitBytes;
                    sq_mbar_expect_tx(full0 + 8 * s, job.fused ? 2 * bytes : bytes);
                    const uint32_t grb = ua / G;
                    const int segment = sq_segment_of(job, grb);
                    const size_t offset = (size_t)(ua - job.block_begin[segment] * G) * kUnitBytes;
                    sq_bulk_copy(ring0 + s * kStageBytes, job.tiles[segment] + offset, bytes, full0 + 8 * s);
                    if (job.fused) {
                        sq_bulk_copy(ring0 + s * kStageBytes + 8 * kUnitBytes, job.up_tiles + offset, bytes, full0 + 8 * s);
                    }
                    ua += count;
                    g += count;
                    if (g == G) g = 0;
                    ++it;
                }
            }
            if (!ok) {
                atomicExch(p.status, 0x81u);
                for (uint32_t back = 0; back < stages && back < it; ++back) {  // let issued copies land
                    const uint32_t i = it - 1 - back;
                    sq_wait(full0 + 8 * (i % stages), (i / stages) & 1);
                }
            }
        }
        return;  // the producer warp takes part in no later barrier
    }

    // ---- consumers ----
    const uint32_t m_rows = p.m_rows;
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t j = 0; j < p.job_count && ok; ++j) {
        const DecodeJob &job = p.jobs[j];
        const uint32_t G = job.groups;
        const bool fused = job.fused != 0;
        const uint32_t per_stage = fused ? 8u : 16u;
        const size_t K = (size_t)G * kGroup;
        uint32_t u0, range;
        sq_range(job, cta, u0, range);
        const uint32_t u1 = u0 + range;
        const uint32_t grb0 = range > 0 ? u0 / G : 0, g_first = range > 0 ? u0 % G : 0;

        for (uint32_t i = threadIdx.x; i < job.local_blocks * kPerBlock; i += 256) red[i] = 0.0f;
        // x of this job may be what the previous job wrote (on this or any rank): wait for all of it
        const long long t_dep = SQ_CLOCK();
        if (j > 0 && range > 0 && threadIdx.x == 0) {
            // every row block of the previous job, on every rank, announces itself once
            const uint32_t expected = p.jobs[j - 1].expected_blocks * p.epoch;
            const long long start = clock64();
            uint32_t seen = 0;
            for (;;) {
                if (p.world > 1) {  // peers add to the counter over NVLink after a system-scope fence
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.done + (j - 1)) : "memory");
                } else {
                    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.done + (j - 1)) : "memory");
                }
                if ((int32_t)(seen - expected) >= 0) break;
                if (clock64() - start > kSeqWaitLimit) { flags[0] = 0xdeadu; break; }
                __nanosleep(32);
            }
            // the acquire above (system scope with peers) ordered the peers' stores; a system-scope fence here
            // measured 3 us per job, the device-scope one passes the order on to the CTA's other threads
            asm volatile("fence.acq_rel.gpu;" ::: "memory");
        }
        sq_consumer_barrier();
        if (flags[0] == 0xdeadu) {
            ok = false;
            if (threadIdx.x == 0) atomicExch(p.status, 0x83u);
            break;
        }
        SQ_ADD(0, t_dep);
        const long long t_loop = SQ_CLOCK();

        float acc[2][4][NT][4];
#pragma unroll
        for (int k = 0; k < 2; ++k)
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int q = 0; q < 4; ++q) acc[k][r][n][q] = 0.0f;

        // add every warp's sums of a finished row block into the block sums, in warp order
        auto flush_in_turns = [&](uint32_t lrb) {
            float *target = red + (size_t)lrb * kPerBlock;
            for (int turn = 0; turn < W; ++turn) {
                if (warp == turn) {
#pragma unroll
                    for (int k = 0; k < 2; ++k)
#pragma unroll
                        for (int n = 0; n < NT; ++n)
#pragma unroll
                            for (int r = 0; r < 4; ++r) {
                                float4 *at = reinterpret_cast<float4 *>(target + k * (NT * 512)) + (n * 4 + r) * 32 + lane;
                                float4 v = *at;
                                v.x += acc[k][r][n][0]; v.y += acc[k][r][n][1];
                                v.z += acc[k][r][n][2]; v.w += acc[k][r][n][3];
                                *at = v;
                                acc[k][r][n][0] = acc[k][r][n][1] = acc[k][r][n][2] = acc[k][r][n][3] = 0.0f;
                            }
                }
                sq_consumer_barrier();
            }
        };

        // The same for M <= 4 in two barriers: only columns 0..3 of the 8-wide tiles carry activations,
        // so every warp parks those (2 planes x 64 rows x 4 columns) in its own slice and the CTA's
        // threads add the eight slices in warp order.
        auto flush_small = [&](uint32_t lrb) {
            float *mine = part + (size_t)warp * 512;
            if (t < 2) {
#pragma unroll
                for (int k = 0; k < 2; ++k)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const uint32_t row = r * 16 + gid;
                        *reinterpret_cast<float2 *>(mine + (k * 64 + row) * 4 + 2 * t) =
                            make_float2(acc[k][r][0][0], acc[k][r][0][1]);
                        *reinterpret_cast<float2 *>(mine + (k * 64 + row + 8) * 4 + 2 * t) =
                            make_float2(acc[k][r][0][2], acc[k][r][0][3]);
                    }
            }
#pragma unroll
            for (int k = 0; k < 2; ++k)
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[k][r][0][0] = acc[k][r][0][1] = acc[k][r][0][2] = acc[k][r][0][3] = 0.0f;
            sq_consumer_barrier();
            float *target = red + (size_t)lrb * kPerBlock;
            for (uint32_t o = threadIdx.x; o < 512; o += 256) {
                const uint32_t k = o >> 8, row = (o >> 2) & 63u, col = o & 3u;
                float total = 0.0f;
#pragma unroll
                for (int w = 0; w < W; ++w) total += part[(size_t)w * 512 + o];
                // fragment layout of the block sums: tile r = row / 16, lane = 4 (row % 8) + col / 2,
                // element 2 (row / 8 % 2) + col % 2
                const uint32_t index = k * (NT * 512) + (row >> 4) * 128 + ((row & 7u) * 4 + (col >> 1)) * 4 +
                                       ((row >> 3) & 1u) * 2 + (col & 1u);
                target[index] += total;
            }
            sq_consumer_barrier();
        };
        auto flush = [&](uint32_t lrb) {
            if (NT == 1 && m_rows <= 4) {
                flush_small(lrb);
            } else {
                flush_in_turns(lrb);
            }
        };

        uint32_t ua = u0, g = g_first, cur_grb = grb0, grb = grb0;
        while (ua < u1) {
            const uint32_t s = it % stages;
            const uint32_t count = min(min(per_stage, G - g), u1 - ua);
            if (grb != cur_grb) {
                flush(cur_grb - grb0);
                cur_grb = grb;
            }
            if (!sq_wait(full0 + 8 * s, (it / stages) & 1)) {
                ok = false;
                break;
            }
            const uint8_t *stage = ring + (size_t)s * kStageBytes;
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                // fused: sub = matrix (gate, up) of group `warp`; else sub selects group warp or warp + 8
                const uint32_t j_group = fused ? (uint32_t)warp : (uint32_t)warp + 8u * sub;
                if (j_group >= count) continue;
                const int plane = fused ? sub : 0;
                const uint32_t group = g + j_group;
                uint32_t xb[NT][8];
                float2 sums[NT];
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const uint32_t m = n * 8 + gid;
                    if (m < m_rows) {
                        const uint4 *src = reinterpret_cast<const uint4 *>(
                            reinterpret_cast<const __half *>(job.x) + (size_t)m * K + (size_t)group * kGroup + 16 * t);
                        const uint4 a = __ldg(src), b = __ldg(src + 1);
                        xb[n][0] = a.x; xb[n][1] = a.y; xb[n][2] = a.z; xb[n][3] = a.w;
                        xb[n][4] = b.x; xb[n][5] = b.y; xb[n][6] = b.z; xb[n][7] = b.w;
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) xb[n][i] = 0u;
                    }
                    // group sums of x on the tensor pipe: a fragment of ones times the same B
                    const uint32_t ones[4] = {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u};
                    float total[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) sq_mma(total, ones, xb[n][2 * i], xb[n][2 * i + 1], i == 0);
                    sums[n] = make_float2(total[0], total[1]);
                }
                const uint8_t *unit = stage + (size_t)((fused ? 8u * sub : 0u) + j_group) * kUnitBytes;
                uint4 codes[4];
                uint2 meta[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const uint8_t *tile = unit + r * kTileBytes;
                    codes[r] = *reinterpret_cast<const uint4 *>(tile + piece_index(lane) * 16);
                    meta[r] = *reinterpret_cast<const uint2 *>(tile + kTileCodeBytes + gid * 8);
                }
                float c[4][NT][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const uint32_t word = i == 0 ? codes[r].x : i == 1 ? codes[r].y : i == 2 ? codes[r].z : codes[r].w;
                        uint32_t a[4];
                        word_to_codes_subnormal(word, a);
#pragma unroll
                        for (int n = 0; n < NT; ++n) sq_mma(c[r][n], a, xb[n][2 * i], xb[n][2 * i + 1], i == 0);
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&meta[r].x));
                    float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&meta[r].y));
                    lo.x *= 16777216.0f;  // codes arrive as q * 2^-24
                    hi.x *= 1048576.0f;   // and 16 q * 2^-24
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        if (plane == 0) {
                            acc[0][r][n][0] = fmaf(lo.x, c[r][n][0], fmaf(lo.y, sums[n].x, acc[0][r][n][0]));
                            acc[0][r][n][1] = fmaf(lo.x, c[r][n][1], fmaf(lo.y, sums[n].y, acc[0][r][n][1]));
                            acc[0][r][n][2] = fmaf(hi.x, c[r][n][2], fmaf(hi.y, sums[n].x, acc[0][r][n][2]));
                            acc[0][r][n][3] = fmaf(hi.x, c[r][n][3], fmaf(hi.y, sums[n].y, acc[0][r][n][3]));
                        } else {
                            acc[1][r][n][0] = fmaf(lo.x, c[r][n][0], fmaf(lo.y, sums[n].x, acc[1][r][n][0]));
                            acc[1][r][n][1] = fmaf(lo.x, c[r][n][1], fmaf(lo.y, sums[n].y, acc[1][r][n][1]));
                            acc[1][r][n][2] = fmaf(hi.x, c[r][n][2], fmaf(hi.y, sums[n].x, acc[1][r][n][2]));
                            acc[1][r][n][3] = fmaf(hi.x, c[r][n][3], fmaf(hi.y, sums[n].y, acc[1][r][n][3]));
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) sq_mbar_arrive(empty0 + 8 * s);
            ++it;
            ua += count;
            g += count;
            if (g == G) { g = 0; ++grb; }
        }
        if (!ok) {
            if (lane == 0) atomicExch(p.status, 0x82u);
            break;
        }
        if (range == 0) continue;
        SQ_ADD(1, t_loop);
        const long long t_flush = SQ_CLOCK();
        flush(cur_grb - grb0);  // ends with a consumer barrier
        SQ_ADD(2, t_flush);
        const long long t_finish = SQ_CLOCK();
        // ---- finish every row block this CTA touched ----
        const uint32_t grb_last = (u1 - 1) / G;
        const uint32_t share = job.units_per_cta, extra = job.units_extra, parts = job.parts;
        const uint32_t floats = fused ? kPerBlock : kPerBlock / 2;  // planes in use
        // (1) park the sums of row blocks that other CTAs share
        for (uint32_t b = grb0; b <= grb_last; ++b) {
            const uint32_t contributed = min(u1, (b + 1) * G) - max(u0, b * G);
            if (contributed == G) continue;
            const uint32_t first_cta = parts > 0 ? b * parts : sq_cta_of_unit(b * G, share, extra);
            const float *mine = red + (size_t)(b - grb0) * kPerBlock;
            float *slot = p.scratch + ((size_t)b * job.slots + (cta - first_cta)) * kPerBlock;
            for (uint32_t o = threadIdx.x; o < floats; o += 256) slot[o] = mine[o];
        }
        sq_consumer_barrier();
        // (2) one thread per row block publishes and learns whether this CTA completes the block
        if (threadIdx.x <= grb_last - grb0) {
            const uint32_t b = grb0 + threadIdx.x;
            const uint32_t contributed = min(u1, (b + 1) * G) - max(u0, b * G);
            uint32_t finish = 1;
            if (contributed != G) {
                // release: the CTA's parked sums (ordered before this by the barrier) are visible to whoever reads
                // the count; acquire: the last arriver sees everybody else's
                uint32_t before;
                asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;"
                             : "=r"(before) : "l"(p.counters + b), "r"(contributed) : "memory");
                finish = before + contributed == G ? 2u : 0u;
                if (finish) p.counters[b] = 0;  // ready for the next job (ordered by the publishing release below)
            }
            flags[threadIdx.x] = finish;
        }
        sq_consumer_barrier();
        // (3) outputs of the blocks that are complete here, stored on every rank
        for (uint32_t b = grb0; b <= grb_last; ++b) {
            const uint32_t finish = flags[b - grb0];
            if (finish == 0) continue;
            const float *mine = red + (size_t)(b - grb0) * kPerBlock;
            const uint32_t first_cta = parts > 0 ? b * parts : sq_cta_of_unit(b * G, share, extra);
            const uint32_t last_cta = parts > 0 ? first_cta + parts - 1 : sq_cta_of_unit((b + 1) * G - 1, share, extra);
            const uint32_t contributors = last_cta - first_cta + 1;
            const float *slots = p.scratch + ((size_t)b * job.slots) * kPerBlock;
            const int segment = sq_segment_of(job, b);
            const uint32_t rb = b - job.block_begin[segment];
            const uint32_t rows = job.rows[segment], ldy = job.ldy[segment];
            for (uint32_t o = threadIdx.x; o < NT * 4 * 128; o += 256) {
                const uint32_t n = o / 512, rr = (o >> 7) & 3u, ln = (o >> 2) & 31u, q = o & 3u;
                const uint32_t row = rb * 64 + rr * kTileRows + (ln >> 2) + 8 * (q >> 1);
                const uint32_t m = n * 8 + 2 * (ln & 3u) + (q & 1u);
                if (row >= rows || m >= m_rows) continue;
                float value = 0.0f, second = 0.0f;
                if (finish == 1) {
                    value = mine[o];
                    if (fused) second = mine[NT * 512 + o];
                } else {  // the slots in CTA order: the same sum whichever CTA arrives last
                    for (uint32_t c0 = 0; c0 < contributors; c0 += 4) {  // four loads in flight at a time
                        float a[4], b[4];
#pragma unroll
                        for (uint32_t q = 0; q < 4; ++q) {
                            const bool live = c0 + q < contributors;
                            a[q] = live ? __ldcg(slots + (size_t)(c0 + q) * kPerBlock + o) : 0.0f;
                            b[q] = live && fused ? __ldcg(slots + (size_t)(c0 + q) * kPerBlock + NT * 512 + o) : 0.0f;
                        }
#pragma unroll
                        for (uint32_t q = 0; q < 4; ++q) {
                            value += a[q];
                            second += b[q];
                        }
                    }
                }
                if (fused) {
                    // silu(g) * u from the un-rounded accumulators (qwen38_q4.metal:146-149)
                    value = (value / (1.0f + __expf(-value))) * second;
                }
                const size_t at = (size_t)m * ldy + row;
                for (uint32_t r = 0; r < p.world; ++r) {
                    void *destination = job.y[segment][r];
                    if (destination == nullptr) continue;
                    if (job.y_dtype == kF32) {
                        reinterpret_cast<float *>(destination)[at] = value;
                    } else {
                        reinterpret_cast<__half *>(destination)[at] = __float2half_rn(value);
                    }
                }
            }
        }
        // (4) publish the row blocks whose outputs this CTA wrote (CTAs that only
        // contributed partial sums have nothing more to say and move on)
        uint32_t finished = 0;
        for (uint32_t b = grb0; b <= grb_last; ++b) finished += flags[b - grb0] != 0 ? 1u : 0u;
        sq_consumer_barrier();
        if (threadIdx.x == 0 && finished > 0) {
            if (p.world > 1) {
                const long long t_publish = SQ_CLOCK();
                // one system-scope fence for the CTA's stores to all ranks, then one add per rank
                asm volatile("fence.acq_rel.sys;" ::: "memory");
                for (uint32_t r = 0; r < p.world; ++r)
                    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.peer_done[r] + j), "r"(finished) : "memory");
                SQ_ADD(5, t_publish);
            } else {
                asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.done + j), "r"(finished) : "memory");
            }
        }
        SQ_ADD(3, t_finish);
    }
}

template <int NT>
cudaError_t sequence_attributes(size_t smem_bytes, int *blocks_per_sm) {
    auto kernel = decode_sequence_kernel<NT>;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
    if (status != cudaSuccess) return status;
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, kernel, 288, smem_bytes);
}

}  // namespace

void plan_decode_job(DecodeJob *job, uint32_t m_rows, uint32_t ctas, size_t *scratch_bytes, size_t *counter_bytes) {
    const uint32_t G = job->groups;
    const int NT = m_rows <= 8 ? 1 : 2;
    uint32_t blocks = 0;
    for (uint32_t s = 0; s < job->segments; ++s) {
        job->block_begin[s] = blocks;
        blocks += ceil_div(job->rows[s], 64);
    }
    for (uint32_t s = job->segments; s <= kMaxSegments; ++s) job->block_begin[s] = blocks;
    const uint32_t units = blocks * G;
    job->total_units = units;
    // every row block cut into the same number of parts when all parts fit the grid
    // Every row block cut into the same number of K parts when all parts fit the grid: one CTA then touches
    // one row block only.  (Equal unit ranges over the whole grid balance the bytes better but make every CTA
    // share two or three row blocks; measured 80 against 68 us per 27B layer.)
    uint32_t parts = 0;
    if (blocks <= ctas && getenv("Q4B_SEQUENCE_EQUAL_RANGES") == nullptr) {
        for (uint32_t k = 1; k <= G; ++k) {
            if (blocks * k <= ctas && (G / k >= 4 || k == 1)) parts = k;
        }
    }
    job->parts = parts;
    uint32_t max_range;
    if (parts > 0) {
        job->active_ctas = blocks * parts;
        job->units_per_cta = 0;
        job->units_extra = 0;
        job->slots = parts;
        job->local_blocks = 1;
        max_range = ceil_div(G, parts);
    } else {
        uint32_t active = ctas;
        const uint32_t by_work = units / 8 > 0 ? units / 8 : 1;
        if (active > by_work) active = by_work;
        job->active_ctas = active;
        job->units_per_cta = units / active;
        job->units_extra = units % active;
        max_range = ceil_div(units, active);
        job->slots = ceil_div(G, job->units_per_cta > 0 ? job->units_per_cta : 1) + 1;
        job->local_blocks = (max_range - 1) / G + 2;
    }
    (void)max_range;
    *scratch_bytes = (size_t)blocks * job->slots * (2 * NT * 4 * 128) * sizeof(float);
    *counter_bytes = (size_t)blocks * sizeof(uint32_t);
}

cudaError_t sequence_geometry(uint32_t m_rows, int sm_count, uint32_t stages, uint32_t max_local_blocks,
                              uint32_t *ctas, size_t *smem_bytes) {
    const int NT = m_rows <= 8 ? 1 : 2;
    if (m_rows == 0 || m_rows > 16 || stages < 2 || stages > (uint32_t)kSeqMaxStages) return cudaErrorInvalidValue;
    const size_t bytes = 128 + (size_t)stages * 16 * kUnitBytes +
                         (size_t)max_local_blocks * (2 * NT * 4 * 128) * sizeof(float) +
                         ((max_local_blocks + 3u) & ~3u) * 4 + (m_rows <= 4 ? 8 * 512 * sizeof(float) : 0) + 16;
    if (bytes > 220 * 1024) return cudaErrorInvalidValue;
    int per_sm = 0;
    cudaError_t status = NT == 1 ? sequence_attributes<1>(bytes, &per_sm) : sequence_attributes<2>(bytes, &per_sm);
    if (status != cudaSuccess) return status;
    if (per_sm < 1) return cudaErrorInvalidValue;
    if (per_sm > 2) per_sm = 2;
    *ctas = (uint32_t)(per_sm * sm_count);
    *smem_bytes = bytes;
    return cudaSuccess;
}

cudaError_t launch_sequence(const SequenceLaunch &launch, cudaStream_t stream) {
    SeqParams p = {};
    p.jobs = launch.jobs;
    p.job_count = launch.job_count;
    p.stages = launch.stages;
    p.m_rows = launch.m_rows;
    p.max_local_blocks = launch.max_local_blocks;
    p.world = launch.world;
    p.rank = launch.rank;
    p.epoch = launch.epoch;
    p.done = launch.done;
    for (int r = 0; r < kMaxPeers; ++r) p.peer_done[r] = launch.peer_done[r];
    p.scratch = launch.scratch;
    p.counters = launch.counters;
    p.status = launch.status;
    void *arguments[] = {&p};
    const void *kernel = launch.m_rows <= 8 ? reinterpret_cast<const void *>(decode_sequence_kernel<1>)
                                            : reinterpret_cast<const void *>(decode_sequence_kernel<2>);
    // cooperative: the CTAs wait on one another, so all of them must be resident
    return cudaLaunchCooperativeKernel(kernel, dim3(launch.ctas), dim3(288), arguments, launch.smem_bytes, stream);
}

}  // namespace q4b
