// Decode GEMV (M = 1) and small-M verify GEMM (M <= 16) on the Q4 tile stream.
//
// Replaces the reference's row kernels: qwen38_q4_matvec / qwen38_q4_gate_up_silu
// (qwen38_q4.metal:111-151), the fused in-projections (qwen38_layer.metal:71-100,
// qwen38_attention.metal:28-52), the residual second projections
// (qwen38_layer.metal:193-255) and the small-batch verify GEMMs
// (qwen38_prefill.metal:144-248, :1090-1363).
//
// HBM bound: every weight byte is read once.  The work of one launch is the
// linear sequence of "units" (one 64-row block x one 64-column group, 2304
// contiguous bytes of the tile stream; two matrices for fused gate/up).  The
// grid is persistent -- one or two CTAs per SM -- and CTA c owns the contiguous
// unit range [c*U/n, (c+1)*U/n): equal bytes for every CTA whatever the shape,
// and a single contiguous byte range per CTA, which a producer warp streams into
// a shared-memory ring with bulk asynchronous copies (cp.async.bulk + mbarrier)
// several stages ahead of the consumer warps.
//
// Arithmetic: y[m][n] = sum_g ( s[n][g] * sum_j q[n][g][j] x[m][64g+j]
//                             + b[n][g] * sum_j x[m][64g+j] ).
// The integer-code dot products run on the tensor pipe (m16n8k16; the fp16
// operands hold the exact codes, fp32 accumulate), scale and bias are applied per
// group in fp32 on the CUDA cores, x and its group sums are staged once per CTA.
// Consumer warp w takes units w, w+W, ... of the CTA's range and keeps the
// 64 x M accumulators of the current row block in registers; when its row block
// changes it adds them into the CTA's shared-memory block sums.  A row block that
// one CTA covered completely is finished locally; otherwise each contributing CTA
// parks its partial sums in a global scratch slot and the last one to arrive adds
// the slots in CTA order (deterministic) and writes the output.
// Every wait is bounded: on expiry the kernel records a code in the status word
// and runs to its normal end.
#include "q4b_kernels.h"

#ifdef Q4B_TRACE
__device__ long long q4b_trace_buffer[1024 * 16];
#define Q4B_STAMP(slot) do { if (threadIdx.x == 0) q4b_trace_buffer[blockIdx.x * 16 + (slot)] = clock64(); } while (0)
#define Q4B_ADD(slot, value) do { if (threadIdx.x == 0) q4b_trace_buffer[blockIdx.x * 16 + (slot)] += (value); } while (0)
extern "C" int q4b_trace_read(long long *out, int count) {
    return (int)cudaMemcpyFromSymbol(out, q4b_trace_buffer, sizeof(long long) * count);
}
extern "C" int q4b_trace_clear(void) {
    static long long zeros[1024 * 16];
    return (int)cudaMemcpyToSymbol(q4b_trace_buffer, zeros, sizeof(zeros));
}
#else
#define Q4B_STAMP(slot) do { } while (0)
#define Q4B_ADD(slot, value) do { } while (0)
#endif

namespace q4b {

namespace {

constexpr int kMaxStages = 8;
constexpr long long kWaitLimitCycles = 4000000000ll;  // every wait gives up after ~2 s of SM clocks

struct GemvParams {
    WeightView w[kMaxSegments];
    WeightView up;
    void *y[kMaxSegments];
    uint32_t ldy[kMaxSegments];
    uint32_t block_begin[kMaxSegments + 1];  // prefix sums of 64-row blocks
    int segments;
    const void *x;
    const void *residual;
    uint32_t *status;
    float *scratch;        // [blocks][slots][PER_CTA] partial sums
    uint32_t *counters;    // [blocks] units contributed so far (self-resetting)
    uint32_t slots;
    uint32_t ld_residual;
    uint32_t m_rows;
    uint32_t groups;
    uint32_t stages;
    uint32_t units_per_cta, units_extra;  // U / ctas and U % ctas (equal-range mode)
    uint32_t parts;                       // > 0: every row block is cut into `parts` CTAs
    uint32_t local_blocks; // row blocks a CTA's range can touch
    uint32_t total_units;
    int y_dtype, residual_dtype;
};

__device__ inline uint32_t smem_u32(const void *pointer) {
    return (uint32_t)__cvta_generic_to_shared(pointer);
}
__device__ inline void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ inline void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ inline void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ inline bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
__device__ inline bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > kWaitLimitCycles) return false;
    }
    return true;
}
__device__ inline void bulk_copy_to_shared(uint32_t destination, const void *source, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(destination), "l"(source), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ inline void consumer_barrier(uint32_t threads) {
    asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

// the CTA whose range holds unit `unit` when the first `extra` CTAs own share+1 units and the rest share
__device__ inline uint32_t cta_of_unit(uint32_t unit, uint32_t share, uint32_t extra) {
    const uint32_t boundary = extra * (share + 1);
    return unit < boundary ? unit / (share + 1) : extra + (unit - boundary) / share;
}

// D = A * B + C with C given (first == false) or zero (first == true)
__device__ inline void mma_16816(float d[4], const uint32_t a[4], uint32_t b0, uint32_t b1, bool first) {
    if (first) {
        asm(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
    } else {
        asm(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// 16 consecutive activations of row m as 8 half2 registers (zeros past M)
template <bool X32>
__device__ inline void load_x16(const void *x, size_t element, bool valid, uint32_t out[8]) {
    if (!valid) {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = 0u;
        return;
    }
    if constexpr (X32) {
        const float4 *p = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + element);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float4 v = __ldg(p + i);
            __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
            out[2 * i] = *reinterpret_cast<uint32_t *>(&lo);
            out[2 * i + 1] = *reinterpret_cast<uint32_t *>(&hi);
        }
    } else {
        const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(x) + element);
        uint4 a = __ldg(p), b = __ldg(p + 1);
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    }
}

// u8 x s8 -> s32, m16n8k32: the codes as bytes against activations as signed 8-bit digits
__device__ inline void mma_16832_u8s8(int d[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

// NT   : 8-column output tiles per warp (M <= 8*NT)
// FUSED: second matrix (`up`) shares x; epilogue silu(gate) * up
// SUBN : feed the codes to the tensor pipe as fp16 subnormals (no unpack math)
// X32  : x arrives as fp32 and is rounded to fp16 while it is staged
// I8   : (fused gate/up, M <= 4, fp16 x) integer form: every consumer warp turns its group of x into two signed
//        8-bit digits per value with one power-of-two step per group and row (15 bits relative to the group's
//        largest value, where fp16 itself carries 11 per value), the codes go to the tensor pipe as bytes
//        (mma.sync m16n8k32 u8 x s8, exact s32 sums) and scale, step and bias are applied per group in fp32
//
// Warps 0..7 consume, warp 8 produces.  A ring stage holds up to 8 consecutive
// groups of one 64-row block (8 x 2304 bytes, one bulk copy; fused gate/up adds the
// same groups of the second matrix as a second copy).  Consumer warp w takes group
// w of the stage: four independent tiles (eight when fused, sharing one read of
// x), accumulated in registers across stages.
template <int NT, bool FUSED, bool SUBN, bool X32, bool I8 = false>
__global__ void __launch_bounds__(288, (FUSED && NT > 1) ? 1 : 2)
gemv_kernel(const GemvParams p) {
    static_assert(!I8 || (NT == 1 && FUSED && !X32), "the integer form serves fused gate/up at M <= 4 with fp16 x");
    constexpr int NW = FUSED ? 2 : 1;
    constexpr int W = 8;                             // consumer warps
    constexpr uint32_t S = W;                        // groups per full stage
    constexpr uint32_t PER_CTA = NW * NT * 4 * 128;  // partial sums of one 64-row block
    constexpr uint32_t kStageBytes = NW * W * kUnitBytes;  // larger copies stream faster
    constexpr uint32_t kConsumers = W * 32;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    // dependents may start at once: all they do before their own wait is prefetch weights
    asm volatile("griddepcontrol.launch_dependents;");

    Q4B_STAMP(0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, t = lane & 3;
    const uint32_t G = p.groups, U = p.total_units, ctas = gridDim.x, cta = blockIdx.x;
    // CTA c owns units [u0, u1): the first U % ctas CTAs take one unit more
    const uint32_t share = p.units_per_cta, extra = p.units_extra, parts = p.parts;
    uint32_t u0, range;
    if (parts > 0) {  // CTA = (row block, part): groups [G*j/parts, G*(j+1)/parts) of that block
        const uint32_t block = cta / parts, j = cta % parts;
        const uint32_t from = G * j / parts, to = G * (j + 1) / parts;
        u0 = block * G + from;
        range = to - from;
    } else {
        u0 = cta * share + min(cta, extra);
        range = share + (cta < extra ? 1u : 0u);
    }
    const uint32_t u1 = u0 + range;
    (void)U;
    (void)ctas;
    const uint32_t stages = p.stages;
    const uint32_t grb0 = u0 / G, g_first = u0 % G;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);  // full[kMaxStages], empty[kMaxStages]
    uint8_t *ring = smem_raw + 128;
    float *red = reinterpret_cast<float *>(ring + (size_t)stages * kStageBytes);   // [L][PER_CTA]
    uint32_t *flags = reinterpret_cast<uint32_t *>(red + (size_t)p.local_blocks * PER_CTA);  // [L]
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kMaxStages);
    const uint32_t ring0 = smem_u32(ring);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, W);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    Q4B_STAMP(10);
    for (uint32_t i = threadIdx.x; i < p.local_blocks * PER_CTA; i += blockDim.x) red[i] = 0.0f;
    Q4B_STAMP(11);
    __syncthreads();
    Q4B_STAMP(12);

    bool ok = true;
    if (warp == W && lane == 0) {
        // ---- producer: stream this CTA's byte range of the tile stream(s) ----
        uint32_t issued = 0, ua = u0, g = g_first;
        for (uint32_t it = 0; ua < u1; ++it) {
            const uint32_t s = it % stages;
            if (it >= stages && !mbar_wait(empty0 + 8 * s, ((it / stages) - 1) & 1)) {
                ok = false;
                break;
            }
            const uint32_t count = min(min(S, G - g), u1 - ua);  // never across a row block
            const uint32_t bytes = count * kUnitBytes;
            mbar_expect_tx(full0 + 8 * s, NW * bytes);
            const uint32_t grb = ua / G;
            int segment = 0;
#pragma unroll
            for (int q = 1; q < kMaxSegments; ++q) {
                if (q < p.segments && grb >= p.block_begin[q]) segment = q;
            }
            const size_t offset = (size_t)(ua - p.block_begin[segment] * G) * kUnitBytes;
            bulk_copy_to_shared(ring0 + s * kStageBytes, p.w[segment].tiles + offset, bytes, full0 + 8 * s);
            if constexpr (FUSED) {
                bulk_copy_to_shared(ring0 + s * kStageBytes + S * kUnitBytes, p.up.tiles + offset, bytes,
                                    full0 + 8 * s);
            }
            ua += count;
            g += count;
            if (g == G) g = 0;
            issued = it + 1;
        }
        if (!ok) {
            atomicExch(p.status, 0x51u);
            // let the copies already issued land before this CTA's memory is released
            for (uint32_t it = issued > stages ? issued - stages : 0; it < issued; ++it) {
                mbar_wait(full0 + 8 * (it % stages), (it / stages) & 1);
            }
        }
    }

    // The weights never depend on the previous kernels of the stream; x and y may.
    // Under programmatic dependent launch this kernel starts while its predecessors
    // still run: the copies above overlap them, everything below waits for them.
    Q4B_STAMP(1);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    Q4B_STAMP(2);

    if (warp < W) {
        const size_t K = (size_t)G * kGroup;
        const uint32_t m_rows = p.m_rows;
        const uint32_t j_mine = (uint32_t)warp;  // this warp's group inside a stage
        Q4B_STAMP(3);
        Q4B_STAMP(4);

        float acc[NW][4][NT][4];
#pragma unroll
        for (int k = 0; k < NW; ++k)
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[k][r][n][j] = 0.0f;
        // Add every warp's sums of a finished row block into the CTA's block sums,
        // one warp at a time in warp order, so the result does not depend on timing.
        auto flush = [&](uint32_t lrb) {
            float *target = red + (size_t)lrb * PER_CTA;
            for (int turn = 0; turn < W; ++turn) {
                if (warp == turn) {
#pragma unroll
                    for (int k = 0; k < NW; ++k)
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
                consumer_barrier(kConsumers);
            }
        };

        // Integer form: lane (gid, t) accumulates rows gid (slot 0) and gid + 8 (slot 2) of activation row m = t.
        // The block sums expect the fp16 form's layout -- slots 0..3 = (gid, m = 2t), (gid, 2t+1), (gid+8, 2t),
        // (gid+8, 2t+1) -- so the sums change lanes once per finished row block.
        auto settle = [&]() {
            if constexpr (I8) {
                const int base = lane & ~3, from = (2 * t) & 3;
#pragma unroll
                for (int k = 0; k < NW; ++k)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const float top = acc[k][r][0][0], low = acc[k][r][0][2];
                        const float top0 = __shfl_sync(0xffffffffu, top, base + from);
                        const float top1 = __shfl_sync(0xffffffffu, top, base + from + 1);
                        const float low0 = __shfl_sync(0xffffffffu, low, base + from);
                        const float low1 = __shfl_sync(0xffffffffu, low, base + from + 1);
                        const bool holds = t < 2;  // activation rows 2t, 2t+1 exist only below 4
                        acc[k][r][0][0] = holds ? top0 : 0.0f;
                        acc[k][r][0][1] = holds ? top1 : 0.0f;
                        acc[k][r][0][2] = holds ? low0 : 0.0f;
                        acc[k][r][0][3] = holds ? low1 : 0.0f;
                    }
            }
        };

        // B fragments come straight from global memory (x is small and stays in L1/L2): lane (gid, t)
        // holds x[m = gid][64 g + 16 t .. +15] for each column tile.  They are fetched one stage ahead,
        // so that their latency hides behind the tiles of the stage before.
        uint32_t x_ahead[NT][8];
        auto fetch_x = [&](uint32_t group) {
            if constexpr (I8) {
                const uint32_t m = (uint32_t)gid >> 1;  // column gid of B = (row m, digit gid & 1)
                // the same 16 consecutive columns as in the fp16 form: this lane's code words cover 16t .. 16t+15
                load_x16<false>(p.x, (size_t)m * K + (size_t)group * kGroup + 16 * t, m < m_rows, x_ahead[0]);
                return;
            }
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const uint32_t m = n * 8 + gid;
                load_x16<X32>(p.x, (size_t)m * K + (size_t)group * kGroup + 16 * t, m < m_rows, x_ahead[n]);
            }
        };
        if (range > 0 && j_mine < min(min(S, G - g_first), range)) fetch_x(g_first + j_mine);

        // ---- main loop: the same stage sequence the producer issues ----
        uint32_t ua = u0, g = g_first, cur_grb = grb0, grb = grb0;
        for (uint32_t it = 0; ua < u1; ++it) {
            const uint32_t s = it % stages;
            const uint32_t count = min(min(S, G - g), u1 - ua);
            if (grb != cur_grb) {
                settle();
                flush(cur_grb - grb0);
                cur_grb = grb;
            }
#ifdef Q4B_TRACE
            const long long wait_begin = clock64();
#endif
            if (!mbar_wait(full0 + 8 * s, (it / stages) & 1)) {
                ok = false;
                break;
            }
            Q4B_ADD(8, clock64() - wait_begin);
            Q4B_ADD(9, 1);
            // what the next stage holds, for the fetch ahead
            const uint32_t ua_next = ua + count, g_next = g + count == G ? 0u : g + count;
            const uint32_t count_next = ua_next < u1 ? min(min(S, G - g_next), u1 - ua_next) : 0u;
            if constexpr (I8) {
              if (j_mine < count) {
                uint32_t raw[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) raw[i] = x_ahead[0][i];
                if (j_mine < count_next) fetch_x(g_next + j_mine);
                // one power-of-two step per (group, activation row): the largest |x| of the 64 columns
                __half2 biggest = __habs2(*reinterpret_cast<__half2 *>(&raw[0]));
#pragma unroll
                for (int i = 1; i < 8; ++i) biggest = __hmax2(biggest, __habs2(*reinterpret_cast<__half2 *>(&raw[i])));
                float top = fmaxf(__low2float(biggest), __high2float(biggest));
                top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
                top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
                int e = (int)((__float_as_uint(top) >> 23) & 0xffu) - 127;  // top in [2^e, 2^(e+1))
                e = min(max(e, -10), 15);  // 2^(5-e) must be an fp16; smaller groups keep fewer bits, of a tiny value
                const float factor = __uint_as_float((uint32_t)(127 + 5 - e) << 23);     // |x| * factor < 64
                const float step_here = __uint_as_float((uint32_t)(127 + e - 13) << 23);  // one unit of the low digit
                const __half2 f_hi = __float2half2_rn(factor);
                const __half2 magic = __float2half2_rn(1536.0f), times256 = __float2half2_rn(256.0f);
                const __half2 cap = __float2half2_rn(127.0f);
                const bool low_digit = (gid & 1) != 0;
                uint32_t b[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t digit[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        // x * 2^(13-e) = 256 hi + lo: v = x * 2^(5-e) lies in (-64, 64); hi = v rounded to nearest in
                        // the 1536 binade (one unit per ulp), lo = 256 (v - hi) exactly, in [-128, 128], capped at 127
                        // (a tie leaves 128: one unit of error, 2^-14 of the group's top) and rounded the same way
                        const __half2 x2 = *reinterpret_cast<__half2 *>(&raw[2 * i + h]);
                        const __half2 v = __hmul2(x2, f_hi);
                        const __half2 hi_m = __hadd2(v, magic);
                        const __half2 hi = __hsub2(hi_m, magic);
                        const __half2 lo = __hmul2(__hsub2(v, hi), times256);
                        const __half2 lo_m = __hadd2(__hmin2(lo, cap), magic);
                        digit[h] = low_digit ? *reinterpret_cast<const uint32_t *>(&lo_m)
                                             : *reinterpret_cast<const uint32_t *>(&hi_m);
                    }
                    // bytes in the order of the code bytes of word i: columns 4i, 4i+2, 4i+1, 4i+3 of this lane's 16
                    b[i] = __byte_perm(digit[0], digit[1], 0x6240);
                }
                // as an accumulator owner this lane serves activation row m = t: that row's step sits in lane 8t
                const float step = __shfl_sync(0xffffffffu, step_here, 8 * t);
                // the group's sum of x, exact: a row of ones against the digits
                const uint32_t ones[4] = {0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u};
                int s0[4], s1[4];
                mma_16832_u8s8(s0, ones, b[0], b[1]);
                mma_16832_u8s8(s1, ones, b[2], b[3]);
                const float sum_x = step * (float)((s0[0] + s1[0]) * 256 + (s0[1] + s1[1]));
#pragma unroll
                for (int k = 0; k < NW; ++k) {
                    const uint8_t *unit = ring + (size_t)s * kStageBytes + (size_t)(k * S + j_mine) * kUnitBytes;
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const uint8_t *tile = unit + r * kTileBytes;
                        const uint4 codes = *reinterpret_cast<const uint4 *>(tile + piece_index(lane) * 16);
                        const uint2 meta = *reinterpret_cast<const uint2 *>(tile + kTileCodeBytes + gid * 8);
                        // even nibbles: row gid, odd nibbles: row gid + 8; word i covers columns 4i .. 4i+3
                        const uint32_t a0[4] = {codes.x & 0x0F0F0F0Fu, (codes.x >> 4) & 0x0F0F0F0Fu,
                                                codes.y & 0x0F0F0F0Fu, (codes.y >> 4) & 0x0F0F0F0Fu};
                        const uint32_t a1[4] = {codes.z & 0x0F0F0F0Fu, (codes.z >> 4) & 0x0F0F0F0Fu,
                                                codes.w & 0x0F0F0F0Fu, (codes.w >> 4) & 0x0F0F0F0Fu};
                        int c0[4], c1[4];
                        mma_16832_u8s8(c0, a0, b[0], b[1]);
                        mma_16832_u8s8(c1, a1, b[2], b[3]);
                        const float top_row = (float)((c0[0] + c1[0]) * 256 + (c0[1] + c1[1]));
                        const float low_row = (float)((c0[2] + c1[2]) * 256 + (c0[3] + c1[3]));
                        const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&meta.x));
                        const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&meta.y));
                        acc[k][r][0][0] = fmaf(lo.x * step, top_row, fmaf(lo.y, sum_x, acc[k][r][0][0]));
                        acc[k][r][0][2] = fmaf(hi.x * step, low_row, fmaf(hi.y, sum_x, acc[k][r][0][2]));
                    }
                }
              } else if (j_mine < count_next) {
                fetch_x(g_next + j_mine);
              }
            } else
            if (j_mine < count) {
                uint32_t xb[NT][8];
                float2 sums[NT];
#pragma unroll
                for (int n = 0; n < NT; ++n) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) xb[n][i] = x_ahead[n][i];
                }
                if (j_mine < count_next) fetch_x(g_next + j_mine);
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    // group sums of x on the tensor pipe: a fragment of ones times the same B
                    const uint32_t ones[4] = {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u};
                    float total[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) mma_16816(total, ones, xb[n][2 * i], xb[n][2 * i + 1], i == 0);
                    sums[n] = make_float2(total[0], total[1]);
                }
#pragma unroll
                for (int k = 0; k < NW; ++k) {
                const uint8_t *unit = ring + (size_t)s * kStageBytes + (size_t)(k * S + j_mine) * kUnitBytes;
                // the four tiles of the sub-unit advance together, word by word, so that
                // consecutive MMAs in the instruction stream are independent of each other
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
                        if constexpr (SUBN) {
                            word_to_codes_subnormal(word, a);
                        } else {
                            __half2 h[4];
                            word_to_codes_f16(word, h);
#pragma unroll
                            for (int q = 0; q < 4; ++q) a[q] = *reinterpret_cast<uint32_t *>(&h[q]);
                        }
#pragma unroll
                        for (int n = 0; n < NT; ++n) mma_16816(c[r][n], a, xb[n][2 * i], xb[n][2 * i + 1], i == 0);
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&meta[r].x));
                    float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&meta[r].y));
                    if constexpr (SUBN) {
                        lo.x *= 16777216.0f;  // codes arrived as q * 2^-24
                        hi.x *= 1048576.0f;   // and 16 q * 2^-24
                    }
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        acc[k][r][n][0] = fmaf(lo.x, c[r][n][0], fmaf(lo.y, sums[n].x, acc[k][r][n][0]));
                        acc[k][r][n][1] = fmaf(lo.x, c[r][n][1], fmaf(lo.y, sums[n].y, acc[k][r][n][1]));
                        acc[k][r][n][2] = fmaf(hi.x, c[r][n][2], fmaf(hi.y, sums[n].x, acc[k][r][n][2]));
                        acc[k][r][n][3] = fmaf(hi.x, c[r][n][3], fmaf(hi.y, sums[n].y, acc[k][r][n][3]));
                    }
                }
                }
            }
            else if (j_mine < count_next) {
                fetch_x(g_next + j_mine);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
            ua += count;
            g += count;
            if (g == G) { g = 0; ++grb; }
        }
        Q4B_STAMP(5);
        if (ok && range > 0) {
            // Last row block of the range: the ring is drained, so every warp parks its
            // sums in its own slice of it at once and the block sums are formed in one
            // pass, still in warp order.
            settle();
            consumer_barrier(kConsumers);
            float *parked = reinterpret_cast<float *>(ring);  // [W][PER_CTA]
#pragma unroll
            for (int k = 0; k < NW; ++k)
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        reinterpret_cast<float4 *>(parked + (size_t)warp * PER_CTA + k * (NT * 512))[(n * 4 + r) * 32 + lane] =
                            make_float4(acc[k][r][n][0], acc[k][r][n][1], acc[k][r][n][2], acc[k][r][n][3]);
                    }
            consumer_barrier(kConsumers);
            float *target = red + (size_t)(cur_grb - grb0) * PER_CTA;
            for (uint32_t o = threadIdx.x; o < PER_CTA; o += kConsumers) {
                float total = target[o];
#pragma unroll
                for (int wv = 0; wv < W; ++wv) total += parked[(size_t)wv * PER_CTA + o];
                target[o] = total;
            }
        }
        if (!ok && lane == 0) atomicExch(p.status, 0x52u);
    }
    __syncthreads();
    Q4B_STAMP(6);

    // ---- finish every row block this CTA touched ----
    if (range == 0) return;
    const uint32_t grb_last = (u1 - 1) / G;
    // (1) park the sums of row blocks that other CTAs share
    for (uint32_t grb = grb0; grb <= grb_last; ++grb) {
        const uint32_t contributed = min(u1, (grb + 1) * G) - max(u0, grb * G);
        if (contributed == G) continue;
        const uint32_t first_cta = parts > 0 ? grb * parts : cta_of_unit(grb * G, share, extra);
        const float *mine = red + (size_t)(grb - grb0) * PER_CTA;
        float *slot = p.scratch + ((size_t)grb * p.slots + (cta - first_cta)) * PER_CTA;
        for (uint32_t o = threadIdx.x; o < PER_CTA; o += blockDim.x) slot[o] = mine[o];
    }
    __syncthreads();
    // (2) one thread publishes them and learns which blocks this CTA completes
    if (threadIdx.x <= grb_last - grb0) {  // one thread per row block, their round trips overlap
        const uint32_t grb = grb0 + threadIdx.x;
        const uint32_t contributed = min(u1, (grb + 1) * G) - max(u0, grb * G);
        uint32_t finish = 1;
        if (contributed != G) {
            __threadfence();
            const uint32_t before = atomicAdd(p.counters + grb, contributed);
            finish = before + contributed == G ? 2u : 0u;
            if (finish) {
                p.counters[grb] = 0;  // ready for the next launch
                __threadfence();
            }
        }
        flags[grb - grb0] = finish;
    }
    __syncthreads();
    // (3) outputs of the blocks that are complete here
    for (uint32_t grb = grb0; grb <= grb_last; ++grb) {
        const uint32_t finish = flags[grb - grb0];
        if (finish == 0) continue;
        const float *mine = red + (size_t)(grb - grb0) * PER_CTA;
        const uint32_t first_cta = parts > 0 ? grb * parts : cta_of_unit(grb * G, share, extra);
        const uint32_t last_cta = parts > 0 ? first_cta + parts - 1 : cta_of_unit((grb + 1) * G - 1, share, extra);
        const uint32_t contributors = last_cta - first_cta + 1;
        const float *slots = p.scratch + ((size_t)grb * p.slots) * PER_CTA;
        int segment = 0;
#pragma unroll
        for (int q = 1; q < kMaxSegments; ++q) {
            if (q < p.segments && grb >= p.block_begin[q]) segment = q;
        }
        const uint32_t rb = grb - p.block_begin[segment];
        const uint32_t rows = p.w[segment].rows;
        for (uint32_t o = threadIdx.x; o < NT * 4 * 128; o += blockDim.x) {
            const uint32_t n = o / 512, rr = (o >> 7) & 3u, ln = (o >> 2) & 31u, j = o & 3u;
            const uint32_t row = rb * 64 + rr * kTileRows + (ln >> 2) + 8 * (j >> 1);
            const uint32_t m = n * 8 + 2 * (ln & 3u) + (j & 1u);
            if (row >= rows || m >= p.m_rows) continue;
            float value = 0.0f, second = 0.0f;
            if (finish == 1) {
                value = mine[o];
                if constexpr (FUSED) second = mine[NT * 512 + o];
            } else {  // the slots in CTA order: the same sum whichever CTA arrives last
                for (uint32_t q = 0; q < contributors; ++q) {
                    value += __ldcg(slots + (size_t)q * PER_CTA + o);
                    if constexpr (FUSED) second += __ldcg(slots + (size_t)q * PER_CTA + NT * 512 + o);
                }
            }
            if constexpr (FUSED) {
                // silu(g) * u from the un-rounded accumulators (qwen38_q4.metal:146-149)
                value = (value / (1.0f + __expf(-value))) * second;
            }
            if (p.residual != nullptr && segment == 0) {
                const size_t at = (size_t)m * p.ld_residual + row;
                value += p.residual_dtype == kF32 ? reinterpret_cast<const float *>(p.residual)[at]
                                                  : __half2float(reinterpret_cast<const __half *>(p.residual)[at]);
            }
            const size_t at = (size_t)m * p.ldy[segment] + row;
            if (p.y_dtype == kF32) {
                reinterpret_cast<float *>(p.y[segment])[at] = value;
            } else {
                reinterpret_cast<__half *>(p.y[segment])[at] = __float2half_rn(value);
            }
        }
    }
    Q4B_STAMP(7);
}

template <int NT, bool FUSED, bool SUBN, bool X32, bool I8 = false>
cudaError_t launch_instance(const GemvParams &p, unsigned ctas, int threads, size_t smem_bytes,
                            bool dependent_launch, cudaStream_t stream) {
    auto kernel = gemv_kernel<NT, FUSED, SUBN, X32, I8>;
    static size_t configured = 0;  // per instantiation
    if (smem_bytes > configured) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)smem_bytes);
        if (status != cudaSuccess) return status;
        configured = smem_bytes;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(ctas);
    config.blockDim = dim3(threads);
    config.dynamicSmemBytes = smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dependent_launch ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, p);
}

template <int NT, bool FUSED>
cudaError_t launch_by_flags(const GemvParams &p, bool subnormal, bool x32, unsigned ctas, int threads,
                            size_t smem_bytes, bool pdl, cudaStream_t stream) {
    if (subnormal) {
        return x32 ? launch_instance<NT, FUSED, true, true>(p, ctas, threads, smem_bytes, pdl, stream)
                   : launch_instance<NT, FUSED, true, false>(p, ctas, threads, smem_bytes, pdl, stream);
    }
    return x32 ? launch_instance<NT, FUSED, false, true>(p, ctas, threads, smem_bytes, pdl, stream)
               : launch_instance<NT, FUSED, false, false>(p, ctas, threads, smem_bytes, pdl, stream);
}

}  // namespace

uint32_t gemv_max_m() { return 16; }

// ---------------------------------------------------------------------------
// Scratch that exists without any allocation call: file-scope device arrays,
// part of the library image, held by every GPU that loads it until the process
// exits.  In host code the names below are only stand-ins for the symbols; the
// device addresses come from cudaGetSymbolAddress, looked up once per device
// with that device current.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB of partial-sum slots
constexpr size_t kStaticCounterCount = 4096;      // one arrival counter per 64-row block
static __device__ __align__(256) float q4b_static_scratch[kStaticScratchBytes / sizeof(float)];
static __device__ __align__(256) uint32_t q4b_static_counters[kStaticCounterCount];

cudaError_t gemv_static_scratch(float **scratch, uint32_t **counters, size_t *scratch_bytes,
                                size_t *counter_bytes) {
    constexpr int kMaxDevices = 64;
    static float *scratch_of[kMaxDevices];
    static uint32_t *counters_of[kMaxDevices];
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return status;
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    if (scratch_of[device] == nullptr) {
        float *scratch_address = nullptr;
        uint32_t *counter_address = nullptr;
        status = cudaGetSymbolAddress(reinterpret_cast<void **>(&scratch_address), q4b_static_scratch);
        if (status != cudaSuccess) return status;
        status = cudaGetSymbolAddress(reinterpret_cast<void **>(&counter_address), q4b_static_counters);
        if (status != cudaSuccess) return status;
        counters_of[device] = counter_address;
        scratch_of[device] = scratch_address;
    }
    *scratch = scratch_of[device];
    *counters = counters_of[device];
    *scratch_bytes = kStaticScratchBytes;
    *counter_bytes = kStaticCounterCount * sizeof(uint32_t);
    return cudaSuccess;
}

// variant encoding (0 = heuristics): bits 0-3 CTAs per SM, 8-11 ring stages,
// bit 12 equal unit ranges even when an even split of the row blocks exists,
// bit 13 exact-fp16 codes instead of subnormals, bit 14 no programmatic
// dependent launch, bit 4 the fp16 form also for fused gate/up at M <= 4 (default there: the integer form)
cudaError_t plan_gemv(const GemvArgs &args, int variant, int sm_count, GemvPlan *plan) {
    const uint32_t G = args.w[0].groups;
    const int NT = args.m_rows <= 8 ? 1 : 2;
    const int NW = args.fused_silu ? 2 : 1;
    uint32_t blocks = 0;
    for (int s = 0; s < args.segments; ++s) blocks += ceil_div(args.w[s].row_tiles, kBlockTiles);
    const uint64_t units64 = (uint64_t)blocks * G;
    if (units64 == 0 || units64 > 0x7fffffffull) return cudaErrorInvalidValue;
    const uint32_t units = (uint32_t)units64;

    int per_sm = variant & 0xf, stages = (variant >> 8) & 0xf;
    if (per_sm == 0) per_sm = 2;
    if (stages == 0) stages = NW == 2 ? 2 : 4;
    if (stages > kMaxStages) stages = kMaxStages;
    const uint32_t slots_on_chip = (uint32_t)sm_count * per_sm;
    uint32_t ctas = slots_on_chip;
    const uint32_t stage_groups = 8;
    const uint32_t by_work = units / stage_groups > 0 ? units / stage_groups : 1;  // a stage or more per CTA
    if (ctas > by_work) ctas = by_work;
    // Prefer an even split: every CTA inside one row block, every block cut into
    // the same number of parts (one part = no cross-CTA sum at all).  All CTAs
    // are resident at once and stream equal shares, so they finish together.
    uint32_t parts = 0;
    if (blocks <= slots_on_chip && ((variant >> 12) & 1) == 0) {
        for (uint32_t k = 1; k <= G; ++k) {
            if (blocks * k <= slots_on_chip && (G / k >= 4 || k == 1)) parts = k;
        }
        if (parts > 0) ctas = blocks * parts;
    }
    plan->parts = parts;
    const uint32_t max_range = parts > 0 ? ceil_div(G, parts) : ceil_div(units, ctas);
    const uint32_t needed = ceil_div(max_range, stage_groups) + 1;
    if ((uint32_t)stages > needed) stages = needed < 2 ? 2 : needed;

    plan->ctas = ctas;
    plan->threads = 9 * 32;
    plan->stages = stages;
    plan->stage_units = stage_groups;
    plan->total_units = units;
    plan->blocks = blocks;
    plan->local_blocks = (max_range - 1) / G + 2;
    plan->slots = parts > 0 ? parts : ceil_div(G, units / ctas > 0 ? units / ctas : 1) + 1;
    const size_t per_cta_floats = (size_t)NW * NT * 4 * 128;
    plan->scratch_bytes = (size_t)blocks * plan->slots * per_cta_floats * 4;
    plan->counter_bytes = (size_t)blocks * 4;
    plan->smem_bytes = 128 + (size_t)stages * NW * 8 * kUnitBytes +
                       (size_t)plan->local_blocks * per_cta_floats * 4 + (size_t)plan->local_blocks * 4 + 16;
    if (plan->smem_bytes > 220 * 1024) return cudaErrorInvalidValue;
    return cudaSuccess;
}

cudaError_t launch_gemv(const GemvArgs &args, const GemvPlan &plan, int variant, cudaStream_t stream) {
    GemvParams p = {};
    uint32_t blocks = 0;
    for (int s = 0; s < args.segments; ++s) {
        p.w[s] = args.w[s];
        p.y[s] = args.y[s];
        p.ldy[s] = args.ldy[s];
        p.block_begin[s] = blocks;
        blocks += ceil_div(args.w[s].row_tiles, kBlockTiles);
    }
    for (int s = args.segments; s <= kMaxSegments; ++s) p.block_begin[s] = blocks;
    p.segments = args.segments;
    p.up = args.up;
    p.x = args.x;
    p.residual = args.residual;
    p.status = args.status;
    p.scratch = args.scratch;
    p.counters = args.counters;
    p.slots = plan.slots;
    p.ld_residual = args.ld_residual;
    p.m_rows = args.m_rows;
    p.groups = args.w[0].groups;
    p.stages = plan.stages;
    p.units_per_cta = plan.total_units / plan.ctas;
    p.units_extra = plan.total_units % plan.ctas;
    p.parts = plan.parts;
    p.local_blocks = plan.local_blocks;
    p.total_units = plan.total_units;
    p.y_dtype = args.y_dtype;
    p.residual_dtype = args.residual_dtype;
    const bool exact_codes = (variant >> 13) & 1, pdl = ((variant >> 14) & 1) == 0;
    const bool subnormal = !exact_codes, x32 = args.x_dtype == kF32;
    const int NT = args.m_rows <= 8 ? 1 : 2;
    if (args.fused_silu && ((variant >> 4) & 1) == 0 && subnormal && args.m_rows <= 4 && !x32) {
        return launch_instance<1, true, true, false, true>(p, plan.ctas, plan.threads, plan.smem_bytes, pdl, stream);
    }
    if (args.fused_silu) {
        return NT == 1 ? launch_by_flags<1, true>(p, subnormal, x32, plan.ctas, plan.threads, plan.smem_bytes, pdl, stream)
                       : launch_by_flags<2, true>(p, subnormal, x32, plan.ctas, plan.threads, plan.smem_bytes, pdl, stream);
    }
    return NT == 1 ? launch_by_flags<1, false>(p, subnormal, x32, plan.ctas, plan.threads, plan.smem_bytes, pdl, stream)
                   : launch_by_flags<2, false>(p, subnormal, x32, plan.ctas, plan.threads, plan.smem_bytes, pdl, stream);
}

}  // namespace q4b
