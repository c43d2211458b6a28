// HBM read-bandwidth probes (the job of read_once in the reference's
// models/qwen3.8-27b/targets/jetson-orin/qwen38_jetson_memory_probe.cu:25-35):
// what this GPU delivers to a kernel that only reads, (0) with plain 16-byte
// loads, and (1, 2) with the producer/consumer bulk-copy ring of the GEMV kernel,
// without (1) or with (2) the consumers reading the staged bytes.  And a ping-pong between two GPUs: what one
// publish-and-wait of the column-parallel decode sequence costs over NVLink.
#include "q4b_kernels.h"

namespace q4b {

namespace {

__global__ void __launch_bounds__(256) probe_ldg_kernel(const uint4 *data, size_t count, uint32_t *sink) {
    uint4 total = make_uint4(0, 0, 0, 0);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 7 * stride < count; i += 8 * stride) {
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[k].x), "=r"(v[k].y), "=r"(v[k].z), "=r"(v[k].w)
                         : "l"(data + i + k * stride));
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) { total.x ^= v[k].x; total.y ^= v[k].y; total.z ^= v[k].z; total.w ^= v[k].w; }
    }
    for (; i < count; i += stride) { uint4 v = data[i]; total.x ^= v.x ^ v.y ^ v.z ^ v.w; }
    if ((total.x ^ total.y ^ total.z ^ total.w) == 0x12345678u) *sink = 1;
}

__device__ inline uint32_t probe_smem_u32(const void *pointer) { return (uint32_t)__cvta_generic_to_shared(pointer); }
__device__ inline bool probe_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
__device__ inline bool probe_wait(uint32_t bar, uint32_t parity) {
    if (probe_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!probe_try_wait(bar, parity)) {
        if (clock64() - start > 4000000000ll) return false;
    }
    return true;
}

// CTA c streams bytes [c*B/n, (c+1)*B/n) (rounded to stage multiples) through a ring
__global__ void __launch_bounds__(288) probe_ring_kernel(const uint8_t *data, size_t stages_total,
                                                         uint32_t stage_bytes, uint32_t stages, int read_back,
                                                         uint32_t *sink) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);
    uint8_t *ring = smem_raw + 128;
    const uint32_t full0 = probe_smem_u32(bars), empty0 = probe_smem_u32(bars + 8), ring0 = probe_smem_u32(ring);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t first = stages_total * blockIdx.x / gridDim.x, last = stages_total * (blockIdx.x + 1) / gridDim.x;
    const uint32_t iterations = (uint32_t)(last - first);
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(full0 + 8 * s), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty0 + 8 * s), "r"(8) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (warp == 8) {
        if (lane == 0) {
            for (uint32_t it = 0; it < iterations; ++it) {
                const uint32_t s = it % stages;
                if (it >= stages && !probe_wait(empty0 + 8 * s, ((it / stages) - 1) & 1)) break;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full0 + 8 * s), "r"(stage_bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(ring0 + s * stage_bytes), "l"(data + (first + it) * stage_bytes), "r"(stage_bytes),
                             "r"(full0 + 8 * s) : "memory");
            }
        }
        return;
    }
    uint32_t total = 0;
    for (uint32_t it = 0; it < iterations; ++it) {
        const uint32_t s = it % stages;
        if (!probe_wait(full0 + 8 * s, (it / stages) & 1)) break;
        if (read_back) {
            const uint4 *mine = reinterpret_cast<const uint4 *>(ring + (size_t)s * stage_bytes) + warp * (stage_bytes / 128);
            for (uint32_t i = lane; i < stage_bytes / 128; i += 32) { uint4 v = mine[i]; total ^= v.x ^ v.y ^ v.z ^ v.w; }
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty0 + 8 * s) : "memory");
    }
    if (total == 0x12345678u) *sink = 1;
}

}  // namespace

// One side of a ping-pong between two GPUs, the exchange the column-parallel decode sequence makes after every job:
// `payload_words` plain stores into the peer's memory, a system-scope fence, one addition to the peer's flag; then
// a wait for the own flag to reach the same round.  The initiator sends first, the responder answers.  Every wait
// is bounded; *status receives the round at which a wait gave up (0: none did).
// mode: 0 as described; bit 0: the flag is raised by one st.release.sys instead of fence + red; bit 1: the
// waiter polls with relaxed loads and makes one system-scope fence once the flag is up; bit 2: no fence on the
// sender at all and a relaxed flag store (NOT an ordering a consumer may rely on: it shows what the fence costs)
__global__ void __launch_bounds__(32) probe_signal_kernel(uint32_t *own_flag, uint32_t *peer_flag, uint32_t *peer_payload,
                                                          uint32_t payload_words, uint32_t rounds, uint32_t base,
                                                          int initiator, int mode, uint32_t *status) {
    const uint32_t lane = threadIdx.x;
    bool alive = true;
    for (uint32_t round = 1; round <= rounds && alive; ++round) {
        for (int turn = 0; turn < 2; ++turn) {
            const bool sending = (turn == 0) == (initiator != 0);
            if (sending) {
                for (uint32_t w = lane; w < payload_words; w += 32) peer_payload[w] = round;
                __syncwarp();
                if (lane == 0) {
                    if (mode & 4) {
                        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(peer_flag), "r"(base + round) : "memory");
                    } else if (mode & 1) {
                        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flag), "r"(base + round) : "memory");
                    } else {
                        asm volatile("fence.acq_rel.sys;" ::: "memory");
                        asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(peer_flag), "r"(1u) : "memory");
                    }
                }
            } else {
                uint32_t seen = 0;
                const long long start = clock64();
                for (;;) {
                    if (lane == 0) {
                        if (mode & 2) {
                            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(own_flag) : "memory");
                        } else {
                            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(own_flag) : "memory");
                        }
                    }
                    seen = __shfl_sync(0xffffffffu, seen, 0);
                    if ((int32_t)(seen - (base + round)) >= 0) break;
                    if (clock64() - start > 2000000000ll) {  // about a second: the peer is not there
                        alive = false;
                        break;
                    }
                }
                if (!alive) {
                    if (lane == 0) *status = round;
                    break;
                }
                if (mode & 2) asm volatile("fence.acq_rel.sys;" ::: "memory");
            }
        }
    }
}

cudaError_t launch_probe_signal(uint32_t *own_flag, uint32_t *peer_flag, uint32_t *peer_payload, uint32_t payload_words,
                                uint32_t rounds, uint32_t base, int initiator, int mode, uint32_t *status,
                                cudaStream_t stream) {
    probe_signal_kernel<<<1, 32, 0, stream>>>(own_flag, peer_flag, peer_payload, payload_words, rounds, base, initiator,
                                              mode, status);
    return cudaGetLastError();
}

cudaError_t launch_probe(int mode, const uint8_t *data, size_t bytes, int ctas, uint32_t stages, uint32_t stage_bytes,
                         uint32_t *sink, cudaStream_t stream) {
    if (mode == 0) {
        probe_ldg_kernel<<<ctas, 256, 0, stream>>>(reinterpret_cast<const uint4 *>(data), bytes / 16, sink);
        return cudaGetLastError();
    }
    if (stages < 2 || stages > 8 || stage_bytes % 128 != 0 || stage_bytes == 0) return cudaErrorInvalidValue;
    const size_t smem = 128 + (size_t)stages * stage_bytes;
    if (smem > 220 * 1024) return cudaErrorInvalidValue;
    cudaError_t status = cudaFuncSetAttribute(probe_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) return status;
    probe_ring_kernel<<<ctas, 288, smem, stream>>>(data, bytes / stage_bytes, stage_bytes, stages, mode == 2, sink);
    return cudaGetLastError();
}

}  // namespace q4b
