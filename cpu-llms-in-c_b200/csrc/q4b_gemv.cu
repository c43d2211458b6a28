// Decode GEMV (M = 1) and small-M verify GEMM (M <= 32) on the Q4 tile stream.
//
// Replaces the reference's row kernels: qwen38_q4_matvec / qwen38_q4_gate_up_silu
// (qwen38_q4.metal:111-151), the fused in-projections (qwen38_layer.metal:71-100,
// qwen38_attention.metal:28-52), the residual second projections
// (qwen38_layer.metal:193-255) and the small-batch verify GEMMs
// (qwen38_prefill.metal:144-248, :1090-1363).
//
// HBM bound: every weight byte is read once, straight into registers, with one
// coalesced 16-byte load per lane per tile and several tiles in flight per warp.
// The arithmetic is y[m][n] = sum_g ( s[n][g] * sum_j q[n][g][j] x[m][64g+j]
//                                   + b[n][g] * sum_j x[m][64g+j] ):
// the inner integer-code dot products run on the tensor pipe (m16n8k16, fp16
// operands that hold the exact codes, fp32 accumulate), the per-group scale and
// bias are applied in fp32 on the CUDA cores, and the group sums of x are
// computed once per CTA.  K is split over the warps of a CTA and, for short
// matrices, over the CTAs of a thread-block cluster whose partial sums meet in
// the leader's shared memory (distributed shared memory, no global scratch).
#include "q4b_kernels.h"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace q4b {

namespace {

struct GemvParams {
    WeightView w[kMaxSegments];
    WeightView up;
    void *y[kMaxSegments];
    uint32_t ldy[kMaxSegments];
    uint32_t tile_begin[kMaxSegments + 1];  // prefix sums of CTA row-tile blocks
    int segments;
    const void *x;
    const void *residual;
    uint32_t ld_residual;
    uint32_t m_rows;
    uint32_t groups;
    uint32_t row_tiles_per_cta;  // R
    int x_dtype, y_dtype, residual_dtype;
};

__device__ inline uint4 load_stream_16(const void *address) {
    uint4 value;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
                 : "l"(address));
    return value;
}
__device__ inline uint2 load_stream_8(const void *address) {
    uint2 value;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(value.x), "=r"(value.y)
                 : "l"(address));
    return value;
}

__device__ inline void mma_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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

template <bool X32>
__device__ inline float sum_x16(const void *x, size_t element) {
    float total = 0.0f;
    if constexpr (X32) {
        const float4 *p = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + element);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float4 v = __ldg(p + i);
            // the tensor pipe sees x rounded to fp16; sum the same values
            float2 lo = __half22float2(__floats2half2_rn(v.x, v.y));
            float2 hi = __half22float2(__floats2half2_rn(v.z, v.w));
            total += (lo.x + lo.y) + (hi.x + hi.y);
        }
    } else {
        const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(x) + element);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint4 v = __ldg(p + i);
            const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&r[k]));
                total += f.x + f.y;
            }
        }
    }
    return total;
}

struct TileRegs {
    uint4 codes;
    uint2 meta;
};

// NT   : 8-column output tiles per warp (M <= 8*NT)
// FUSED: second matrix (`up`) shares x; epilogue silu(gate) * up
// SUBN : feed the codes to the tensor pipe as fp16 subnormals (no unpack math)
// U    : tiles in flight per warp
template <int NT, bool FUSED, bool SUBN, bool X32, int U>
__global__ void __launch_bounds__(256)
gemv_kernel(const GemvParams p) {
    constexpr int NW = FUSED ? 2 : 1;
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const int gid = lane >> 2, t = lane & 3;
    const uint32_t R = p.row_tiles_per_cta;
    const uint32_t ksplit = gridDim.x, kslice = blockIdx.x;

    // which matrix and which block of row tiles
    int segment = 0;
#pragma unroll
    for (int s = 1; s < kMaxSegments; ++s) {
        if (s < p.segments && blockIdx.y >= p.tile_begin[s]) segment = s;
    }
    const WeightView w0 = p.w[segment];
    const uint32_t rt0 = (blockIdx.y - p.tile_begin[segment]) * R;
    const uint32_t G = p.groups;
    const uint32_t g0 = (uint32_t)((uint64_t)G * kslice / ksplit);
    const uint32_t g1 = (uint32_t)((uint64_t)G * (kslice + 1) / ksplit);
    const uint32_t slice_groups = g1 - g0;
    // this warp's groups: g0 + warp, g0 + warp + warps, ...
    const uint32_t ns = slice_groups > (uint32_t)warp ? (slice_groups - warp + warps - 1) / warps : 0;
    const uint32_t row_tiles_here = min(R, w0.row_tiles > rt0 ? w0.row_tiles - rt0 : 0u);
    const uint32_t total = ns * row_tiles_here;

    // shared memory carve-up
    float *sx = smem;                                       // [slice_groups][8*NT]
    float *red = smem + (size_t)(((G + ksplit - 1) / ksplit) + 1) * 8 * NT;  // [R][warps][NW*NT][32][4]
    float *part = red + (size_t)R * warps * NW * NT * 128;  // [ksplit][R][NW*NT][128] (leader)

    const uint8_t *base[NW];
    base[0] = w0.tiles;
    if constexpr (FUSED) base[1] = p.up.tiles;

    auto tile_offset = [&](uint32_t r, uint32_t j) -> size_t {
        return ((size_t)(rt0 + r) * G + g0 + warp + (size_t)j * warps) * kTileBytes;
    };

    // ---- start the weight stream before anything else ----
    TileRegs buffer[U][NW];
    uint32_t load_r = 0, load_j = 0, issued = 0;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        if (issued < total) {
            size_t offset = tile_offset(load_r, load_j);
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                buffer[u][k].codes = load_stream_16(base[k] + offset + lane * 16);
                buffer[u][k].meta = load_stream_8(base[k] + offset + kTileCodeBytes + gid * 8);
            }
            ++issued;
            if (++load_j == ns) { load_j = 0; ++load_r; }
        }
    }

    // ---- group sums of x for this K slice (overlaps the loads above) ----
    {
        const uint32_t items = slice_groups * (8 * NT) * 4;  // (group, m, quarter)
        const size_t K = (size_t)G * kGroup;
        for (uint32_t first = warp * 32; first < items; first += blockDim.x) {
            uint32_t item = first + lane;
            uint32_t quarter = item & 3u, m = (item >> 2) % (8 * NT), g = (item >> 2) / (8 * NT);
            float value = 0.0f;
            if (item < items && m < p.m_rows) {
                value = sum_x16<X32>(p.x, (size_t)m * K + (size_t)(g0 + g) * kGroup + 16 * quarter);
            }
            value += __shfl_xor_sync(0xffffffffu, value, 1);
            value += __shfl_xor_sync(0xffffffffu, value, 2);
            if (quarter == 0 && item < items) sx[g * (8 * NT) + m] = value;
        }
    }
    __syncthreads();

    float acc[NW][NT][4];
#pragma unroll
    for (int k = 0; k < NW; ++k)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[k][n][j] = 0.0f;

    const size_t K = (size_t)G * kGroup;
    uint32_t cur_r = 0, cur_j = 0;
    for (uint32_t s0 = 0; s0 < total; s0 += U) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (s0 + u >= total) break;
            TileRegs cur[NW];
#pragma unroll
            for (int k = 0; k < NW; ++k) cur[k] = buffer[u][k];
            if (issued < total) {  // refill this slot with the tile U steps ahead
                size_t offset = tile_offset(load_r, load_j);
#pragma unroll
                for (int k = 0; k < NW; ++k) {
                    buffer[u][k].codes = load_stream_16(base[k] + offset + lane * 16);
                    buffer[u][k].meta = load_stream_8(base[k] + offset + kTileCodeBytes + gid * 8);
                }
                ++issued;
                if (++load_j == ns) { load_j = 0; ++load_r; }
            }
            const uint32_t g_local = warp + cur_j * warps;  // group index inside the slice
            const uint32_t g = g0 + g_local;
            // B fragments: x[m][64 g + 16 t .. +15]
            uint32_t xb[NT][8];
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                uint32_t m = n * 8 + gid;
                load_x16<X32>(p.x, (size_t)m * K + (size_t)g * kGroup + 16 * t, m < p.m_rows, xb[n]);
            }
            float c[NW][NT][4];
#pragma unroll
            for (int k = 0; k < NW; ++k)
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int j = 0; j < 4; ++j) c[k][n][j] = 0.0f;
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                const uint32_t word[4] = {cur[k].codes.x, cur[k].codes.y, cur[k].codes.z, cur[k].codes.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t a[4];
                    if constexpr (SUBN) {
                        word_to_codes_subnormal(word[i], a);
                    } else {
                        __half2 h[4];
                        word_to_codes_f16(word[i], h);
#pragma unroll
                        for (int r = 0; r < 4; ++r) a[r] = *reinterpret_cast<uint32_t *>(&h[r]);
                    }
#pragma unroll
                    for (int n = 0; n < NT; ++n) mma_16816(c[k][n], a, xb[n][2 * i], xb[n][2 * i + 1]);
                }
            }
            // per-group scale and bias in fp32
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                float2 lo = __half22float2(*reinterpret_cast<__half2 *>(&cur[k].meta.x));
                float2 hi = __half22float2(*reinterpret_cast<__half2 *>(&cur[k].meta.y));
                if constexpr (SUBN) {
                    lo.x *= 16777216.0f;  // codes arrived as q * 2^-24
                    hi.x *= 1048576.0f;   // and 16 q * 2^-24
                }
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    float2 sums = *reinterpret_cast<const float2 *>(&sx[g_local * (8 * NT) + n * 8 + 2 * t]);
                    acc[k][n][0] = fmaf(lo.x, c[k][n][0], fmaf(lo.y, sums.x, acc[k][n][0]));
                    acc[k][n][1] = fmaf(lo.x, c[k][n][1], fmaf(lo.y, sums.y, acc[k][n][1]));
                    acc[k][n][2] = fmaf(hi.x, c[k][n][2], fmaf(hi.y, sums.x, acc[k][n][2]));
                    acc[k][n][3] = fmaf(hi.x, c[k][n][3], fmaf(hi.y, sums.y, acc[k][n][3]));
                }
            }
            if (++cur_j == ns) {  // row tile finished: park this warp's partial sums
#pragma unroll
                for (int k = 0; k < NW; ++k)
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        float4 v = make_float4(acc[k][n][0], acc[k][n][1], acc[k][n][2], acc[k][n][3]);
                        reinterpret_cast<float4 *>(red)[(((size_t)cur_r * warps + warp) * (NW * NT) + k * NT + n) * 32 + lane] = v;
                        acc[k][n][0] = acc[k][n][1] = acc[k][n][2] = acc[k][n][3] = 0.0f;
                    }
                cur_j = 0;
                ++cur_r;
            }
        }
    }
    __syncthreads();

    // ---- sum over warps, then over the cluster, then the epilogue ----
    const uint32_t active_warps = min((uint32_t)warps, slice_groups);
    const uint32_t per_tile = NW * NT * 128;
    const uint32_t outputs = row_tiles_here * per_tile;
    cg::cluster_group cluster = cg::this_cluster();
    float *leader_part = ksplit > 1 ? cluster.map_shared_rank(part, 0) : part;
    for (uint32_t o = threadIdx.x; o < outputs; o += blockDim.x) {
        uint32_t r = o / per_tile, inner = o % per_tile;
        float total_value = 0.0f;
        for (uint32_t wv = 0; wv < active_warps; ++wv) {
            total_value += red[((size_t)r * warps + wv) * per_tile + inner];
        }
        leader_part[(size_t)kslice * R * per_tile + o] = total_value;
    }
    if (ksplit > 1) {
        cluster.sync();
        if (kslice != 0) return;
    } else {
        __syncthreads();
    }

    const uint32_t results = row_tiles_here * NT * 128;  // fused: gate/up pairs collapse
    for (uint32_t o = threadIdx.x; o < results; o += blockDim.x) {
        uint32_t r = o / (NT * 128), inner = o % (NT * 128);
        uint32_t n = inner >> 7, ln = (inner >> 2) & 31u, j = inner & 3u;
        uint32_t row = (rt0 + r) * kTileRows + (ln >> 2) + 8 * (j >> 1);
        uint32_t m = n * 8 + 2 * (ln & 3u) + (j & 1u);
        if (row >= w0.rows || m >= p.m_rows) continue;
        float value = 0.0f, second = 0.0f;
        for (uint32_t ks = 0; ks < ksplit; ++ks) {
            const float *src = part + ((size_t)ks * R + r) * per_tile;
            value += src[inner];
            if constexpr (FUSED) second += src[NT * 128 + inner];
        }
        if constexpr (FUSED) {
            // silu(g) * u from the un-rounded accumulators (qwen38_q4.metal:146-149)
            value = (value / (1.0f + __expf(-value))) * second;
        }
        if (p.residual != nullptr && segment == 0) {
            size_t at = (size_t)m * p.ld_residual + row;
            value += p.residual_dtype == kF32 ? reinterpret_cast<const float *>(p.residual)[at]
                                              : __half2float(reinterpret_cast<const __half *>(p.residual)[at]);
        }
        size_t at = (size_t)m * p.ldy[segment] + row;
        if (p.y_dtype == kF32) {
            reinterpret_cast<float *>(p.y[segment])[at] = value;
        } else {
            reinterpret_cast<__half *>(p.y[segment])[at] = __float2half_rn(value);
        }
    }
}

template <int NT, bool FUSED, bool SUBN, bool X32, int U>
cudaError_t launch_instance(const GemvParams &p, dim3 grid, int threads, size_t smem_bytes,
                            cudaStream_t stream) {
    auto kernel = gemv_kernel<NT, FUSED, SUBN, X32, U>;
    if (smem_bytes > 48 * 1024) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  (int)smem_bytes);
        if (status != cudaSuccess) return status;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(threads);
    config.dynamicSmemBytes = smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = grid.x;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, p);
}

template <int NT, bool FUSED, bool X32>
cudaError_t launch_by_flags(const GemvParams &p, bool subnormal, int depth, dim3 grid, int threads,
                            size_t smem_bytes, cudaStream_t stream) {
    if (subnormal) {
        return depth >= 8 ? launch_instance<NT, FUSED, true, X32, (FUSED || NT > 1) ? 4 : 8>(p, grid, threads, smem_bytes, stream)
                          : launch_instance<NT, FUSED, true, X32, (FUSED || NT > 2) ? 2 : 4>(p, grid, threads, smem_bytes, stream);
    }
    return depth >= 8 ? launch_instance<NT, FUSED, false, X32, (FUSED || NT > 1) ? 4 : 8>(p, grid, threads, smem_bytes, stream)
                      : launch_instance<NT, FUSED, false, X32, (FUSED || NT > 2) ? 2 : 4>(p, grid, threads, smem_bytes, stream);
}

}  // namespace

uint32_t gemv_max_m() { return 32; }

// variant encoding (0 = heuristics): bits 0-3 ksplit, 4-7 warps, 8-11 R,
// bit 12 deep prefetch, bit 13 exact-fp16 code path instead of subnormals
cudaError_t launch_gemv(const GemvArgs &args, int variant, int sm_count, cudaStream_t stream) {
    GemvParams p = {};
    const uint32_t G = args.w[0].groups;
    uint32_t total_row_tiles = 0;
    for (int s = 0; s < args.segments; ++s) total_row_tiles += args.w[s].row_tiles;

    int ksplit = variant & 0xf, warps = (variant >> 4) & 0xf, R = (variant >> 8) & 0xf;
    const bool deep = (variant >> 12) & 1, exact_codes = (variant >> 13) & 1;
    if (warps == 0) warps = 8;
    const int NT = args.m_rows <= 8 ? 1 : (args.m_rows <= 16 ? 2 : 4);
    if (R == 0) {
        // enough CTAs for ~4 per SM, but rows*K per CTA not tiny
        R = 1;
        while (R < 4 && NT == 1 && total_row_tiles / (R * 2) >= (uint32_t)sm_count * 4 && G * R < 256) R *= 2;
    }
    if (ksplit == 0) {
        ksplit = 1;
        uint32_t ctas = ceil_div(total_row_tiles, R);
        while (ksplit < 8 && ctas * ksplit < (uint32_t)sm_count * 4 && G / (ksplit * 2) >= (uint32_t)warps * 2) ksplit *= 2;
    }
    if ((uint32_t)ksplit > G) ksplit = 1;

    uint32_t blocks = 0;
    for (int s = 0; s < args.segments; ++s) {
        p.w[s] = args.w[s];
        p.y[s] = args.y[s];
        p.ldy[s] = args.ldy[s];
        p.tile_begin[s] = blocks;
        blocks += ceil_div(args.w[s].row_tiles, R);
    }
    p.tile_begin[args.segments] = blocks;
    p.segments = args.segments;
    p.up = args.up;
    p.x = args.x;
    p.residual = args.residual;
    p.ld_residual = args.ld_residual;
    p.m_rows = args.m_rows;
    p.groups = G;
    p.row_tiles_per_cta = R;
    p.x_dtype = args.x_dtype;
    p.y_dtype = args.y_dtype;
    p.residual_dtype = args.residual_dtype;
    if (blocks == 0) return cudaSuccess;

    const int NW = args.fused_silu ? 2 : 1;
    size_t smem_floats = (size_t)(ceil_div(G, ksplit) + 1) * 8 * NT      // sx
                         + (size_t)R * warps * NW * NT * 128             // red
                         + (size_t)ksplit * R * NW * NT * 128;           // part
    size_t smem_bytes = smem_floats * sizeof(float);
    if (smem_bytes > 200 * 1024) return cudaErrorInvalidValue;
    dim3 grid(ksplit, blocks);
    const int threads = warps * 32;
    const bool subnormal = !exact_codes;
    const bool x32 = args.x_dtype == kF32;
    const int depth = deep ? 8 : 4;

#define Q4B_DISPATCH(NTV, FUSEDV)                                                                   \
    return x32 ? launch_by_flags<NTV, FUSEDV, true>(p, subnormal, depth, grid, threads, smem_bytes, stream) \
               : launch_by_flags<NTV, FUSEDV, false>(p, subnormal, depth, grid, threads, smem_bytes, stream)
    if (args.fused_silu) {
        if (NT == 1) { Q4B_DISPATCH(1, true); }
        if (NT == 2) { Q4B_DISPATCH(2, true); }
        Q4B_DISPATCH(4, true);
    }
    if (NT == 1) { Q4B_DISPATCH(1, false); }
    if (NT == 2) { Q4B_DISPATCH(2, false); }
    Q4B_DISPATCH(4, false);
#undef Q4B_DISPATCH
}

}  // namespace q4b
