// Decode GEMV (M = 1) and small-M verify GEMM (M <= 16) on the Q4 tile stream: one
// kernel, launched either once per projection or once for a whole chain of
// projections ("sequence": one persistent cooperative grid walks a job table).
//
// Replaces the reference's row kernels: qwen38_q4_matvec / qwen38_q4_gate_up_silu
// (qwen38_q4.metal:111-151), the fused in-projections (qwen38_layer.metal:71-100,
// qwen38_attention.metal:28-52), the residual second projections
// (qwen38_layer.metal:193-255), the lm_head (qwen38_global.metal:37-61) and the
// small-batch verify GEMMs (qwen38_prefill.metal:144-248, :1090-1363); the sequence
// form is the counterpart of the reference encoding a whole token into one command
// buffer (qwen38_m3_decode.m:1614-1690).
//
// HBM bound: every weight byte is read once.  Work is cut into units: one "pair
// block" (128 output rows = two 64-row blocks of the tile stream, or 64 gate rows
// and the same 64 up rows when fused) times one contiguous range of K groups.  A
// CTA has two kinds of warps:
//
//   * warp 8, the weight producer: one thread streams the CTA's units -- job after
//     job in a sequence, never draining -- through a shared-memory ring with bulk
//     asynchronous copies (cp.async.bulk + mbarrier), 8 groups x 2 blocks = 36 KB
//     per stage.  Weights never depend on earlier work, so the ring runs ahead of
//     the consumers across job boundaries and kernel boundaries (programmatic
//     dependent launch): the wait for the previous projection's output is hidden
//     behind loads that are needed anyway.
//   * warps 0..7, the consumers.  Warp w owns ONE 16-row tile of the pair block
//     (tile w & 3 of block w >> 2) and multiplies it with every group of the
//     unit, so a row's sum lives in one lane from the first group to the last: no
//     reduction inside the CTA, no barrier among the consumers.  Per group:
//     y += (s * step) * (q . x') + b * sum(x) in fp32, the reference's arithmetic
//     re-associated per group.  The activations reach the tensor pipe as "entries"
//     in shared memory, eight per ring stage, which the same warps make in turn,
//     two stages ahead of their use (three sets, mbarrier hand-over).  For M <= 4
//     an entry is the integer form: two signed 8-bit digits per value with one
//     power-of-two step per (group, activation row), 15 bits relative to the
//     group's largest value (fp16 itself carries 11 per value), so the codes go
//     to the tensor pipe as bytes (mma.sync m16n8k32 u8 x s8, exact s32 sums); one
//     pass of a warp serves four groups at M = 1, two at M = 2.  For M = 5..16 it
//     is the fp16 form (codes as fp16 subnormal bit patterns, m16n8k16, fp32
//     accumulate).  fp32 activations are scaled per group by a power of two
//     first, so their magnitude does not matter.  In a sequence the consumers are
//     also the ones that wait for the previous job's outputs.
//
// Units that share a pair block (K split over CTAs when a job has fewer pair
// blocks than the grid has CTAs) park their sums in global slots; the last warp
// to arrive for a tile adds the slots in part order -- results do not depend on
// timing -- applies the epilogue (SiLU gate, residual) and stores y, on every
// rank's copy when the ranks of a column-parallel job share outputs.  In a
// sequence it then advances the job's completion counters; the next job's
// consumers start when every tile of every rank has been counted.
//
// Every wait is bounded.  The first wait that expires sets a CTA-wide flag and a
// code in the status word; from then on no wait in that CTA waits, every role
// walks the rest of its control flow (so every barrier still gets its arrivals),
// and the host turns the status word into an error.
#include "q4b_kernels.h"

#include <mutex>

namespace q4b {

namespace {

constexpr int kConsumers = 8;                 // consumer warps
constexpr int kProducerWarp = 8;
constexpr int kDecodeThreads = 32 * (kConsumers + 1);
constexpr uint32_t kStageGroups = 8;          // groups per ring stage, both blocks of the pair
constexpr uint32_t kStageBytes = 2 * kStageGroups * kUnitBytes;  // 36,864
constexpr uint32_t kEntrySets = 3;            // sets of eight entries: they are made two stages ahead of their use
constexpr uint32_t kMaxSharedBytes = 115712;  // what lets two CTAs share an SM (228 KB less 1 KB per CTA)
constexpr long long kWaitLimitCycles = 4000000000ll;  // every wait gives up after ~2 s of SM clocks
// phases of a consumer's time (see SequenceLaunch::profile): waiting for the previous job's outputs, making and
// waiting for activation entries, waiting for weights, multiplying, finishing units; the whole launch
enum ProfileSlot { kProfileDependency = 0, kProfileEntries, kProfileWeights, kProfileTiles, kProfileFinish, kProfileTotal };

// MODE 0: integer form, M <= 4.  MODE 1 / 2: fp16 form, M <= 8 / M <= 16.
// An "entry" is what one group's activations take in shared memory once they are B operands.
template <int MODE> struct Form;
template <> struct Form<0> {
    static constexpr int NT = 1, VALS = 2, SUM_UNROLL = 8;
    static constexpr uint32_t XCHG_VALS = 1;  // values per lane handed from an up warp to its gate warp at a time
    // per activation row: 128 B of digit fragments (lanes 0 .. 8 M - 1), then {step, sum} per row; entries
    // are read with 16-byte loads, so their size is a multiple of 16
    __host__ __device__ static constexpr uint32_t entry_bytes(uint32_t m_rows) { return (136 * m_rows + 15) / 16 * 16; }
};
template <> struct Form<1> {
    static constexpr int NT = 1, VALS = 4, SUM_UNROLL = 4;
    static constexpr uint32_t XCHG_VALS = 4;
    __host__ __device__ static constexpr uint32_t entry_bytes(uint32_t) { return 1088; }  // 1024 B of fp16 fragments + 8 x {step, sum}
};
template <> struct Form<2> {
    static constexpr int NT = 2, VALS = 8, SUM_UNROLL = 2;
    static constexpr uint32_t XCHG_VALS = 8;
    __host__ __device__ static constexpr uint32_t entry_bytes(uint32_t) { return 2176; }
};

// shared memory of a CTA: barriers and flags, the weight ring, three sets of eight entries, the exchange buffer
// of fused gate/up.  Three ring stages when two CTAs then still share an SM, else two.
template <int MODE> uint32_t smem_bytes_of(uint32_t m_rows, uint32_t *stages) {
    const uint32_t fixed = 128 + kEntrySets * kStageGroups * Form<MODE>::entry_bytes(m_rows) +
                           4 * 32 * Form<MODE>::XCHG_VALS * 4 + 64;  // the last 64: the optional phase clocks
    *stages = fixed + 3 * kStageBytes <= kMaxSharedBytes ? 3u : 2u;
    return fixed + *stages * kStageBytes;
}

struct PassParams {
    DecodeJob job;                   // one projection per launch: the job itself
    const DecodeJob *jobs;           // sequence: the job table in device memory
    uint32_t job_count;
    uint32_t m_rows;
    uint32_t world;
    uint32_t stages;                 // ring stages (2 or 3)
    uint32_t cluster;                // single launch: the CTAs of one pair block are one thread-block cluster
    uint32_t throttle;               // single launch: hold the last stage of the first ring fill back
    uint32_t *epoch;                 // sequence: launches completed so far (device word)
    uint32_t *exit_count;            // sequence: CTAs of this launch that have finished
    uint32_t *done;                  // sequence: [job][8] completion counters, kDoneStride words apart
    uint32_t *peer_done[kMaxPeers];  // the same array on every rank (own rank included)
    float *scratch;
    uint32_t *counters;
    uint32_t *status;
    unsigned long long *profile;     // optional: [CTA][kProfileSlots] SM clocks by phase, added up by consumer warp 0
};

// ---------------------------------------------------------------------------
// small PTX wrappers
// ---------------------------------------------------------------------------
__device__ inline uint32_t smem_u32(const void *pointer) { return (uint32_t)__cvta_generic_to_shared(pointer); }
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
// the same, asking the hardware to keep the warp suspended for up to about `nanoseconds` while the phase is open
__device__ inline bool mbar_try_wait_for(uint32_t bar, uint32_t parity, uint32_t nanoseconds) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(nanoseconds)
        : "memory");
    return done != 0;
}
// Bounded wait.  Once any wait of the CTA has expired (*failed != 0) nobody waits any more.  A waiting warp sleeps
// inside try_wait and looks at the failure word and the clock only every sixteenth time it wakes: a spinning warp
// takes issue slots from the warps that multiply.
__device__ inline bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *failed, uint32_t code) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*failed != 0) return false;
    const long long start = clock64();
    uint32_t woken = 0;
    while (!mbar_try_wait_for(bar, parity, 4000u)) {
        if ((++woken & 15u) != 0) continue;
        if (*failed != 0) return false;
        if (clock64() - start > kWaitLimitCycles) {
            *failed = code;
            return false;
        }
    }
    return true;
}
// weights are read once per pass: they leave L2 first, the activations and partial sums that are read again stay
__device__ inline uint64_t stream_once_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ inline void bulk_copy_to_shared(uint32_t destination, const void *source, uint32_t bytes, uint32_t bar,
                                           uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(destination), "l"(source), "r"(bytes), "r"(bar), "l"(policy)
                 : "memory");
}
// every thread of every CTA of the cluster, the same number of times
__device__ inline void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// the address, in the cluster's shared window, of this CTA's shared address `local` inside CTA `rank`
__device__ inline uint32_t cluster_address(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ inline void cluster_store(uint32_t address, float value) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(value) : "memory");
}
__device__ inline void pair_barrier(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

// D = A * B + C (C zero when first), fp16 operands, fp32 accumulate
__device__ inline void mma_16816(float d[4], const uint32_t a[4], uint32_t b0, uint32_t b1, bool first) {
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
// u8 x s8 -> s32, m16n8k32: codes as bytes against activations as signed 8-bit digits
__device__ inline void mma_16832_u8s8(int d[4], const uint32_t a[4], uint32_t b0, uint32_t b1, bool first) {
    if (first) {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
    } else {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// ---------------------------------------------------------------------------
// geometry of a job, the same in every role
// ---------------------------------------------------------------------------
struct Unit {
    uint32_t pair;      // pair block, counted over the job's segments
    uint32_t part;      // which K range of it
    uint32_t g0, g1;    // groups [g0, g1)
    int segment;
    uint32_t local;     // pair block inside its segment
    bool has_b;         // the pair's second block exists (always when fused)
};

__device__ inline Unit unit_of(const DecodeJob &job, uint32_t index) {
    Unit u;
    u.pair = index / job.parts;
    u.part = index % job.parts;
    u.g0 = job.groups * u.part / job.parts;
    u.g1 = job.groups * (u.part + 1) / job.parts;
    u.segment = 0;
#pragma unroll
    for (int q = 1; q < kMaxSegments; ++q) {
        if (q < (int)job.segments && u.pair >= job.pair_begin[q]) u.segment = q;
    }
    u.local = u.pair - job.pair_begin[u.segment];
    u.has_b = job.fused != 0 || 2 * u.local + 1 < ceil_div(job.rows[u.segment], 64);
    return u;
}

// ---------------------------------------------------------------------------
// activations of one group -> B operands in shared memory (all 32 lanes of one consumer warp)
// ---------------------------------------------------------------------------
// 16 consecutive fp16 activations of this lane in one group (8 registers), zeros when not `live`
__device__ inline void fetch_x16(const void *x, size_t element, bool live, uint32_t raw[8]) {
    uint4 lo = make_uint4(0u, 0u, 0u, 0u), hi = lo;
    if (live) {
        const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(x) + element);
        lo = __ldcg(p);
        hi = __ldcg(p + 1);
    }
    raw[0] = lo.x; raw[1] = lo.y; raw[2] = lo.z; raw[3] = lo.w;
    raw[4] = hi.x; raw[5] = hi.y; raw[6] = hi.z; raw[7] = hi.w;
}
__device__ inline void fetch_x32(const void *x, size_t element, bool live, float v[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float4 f = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (live) f = __ldcg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + element) + i);
        v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
    }
}

// Integer form.  Lane (gid, t): activation row m = gid >> 1, digit gid & 1 (0 high, 1 low), the 16 columns
// 16 t .. 16 t + 15 of the group -- the columns this lane's code words cover in a tile.  An entry receives:
//   [lane * 16, +16)    for lanes 0 .. 8 M - 1: the four B registers of the two m16n8k32 MMAs of a tile
//                       (column n = 2 m + digit), bytes of register i in the order of the code bytes of word i:
//                       columns 4i, 4i+2, 4i+1, 4i+3; the other lanes' registers are zero and are not stored
//   [128 M + 8 m, +8)   {step, sum}: one unit of the low digit as a float, and the sum of the group's 64 values
//                       as the digits represent them (exact)
// A group whose largest magnitude is infinite, NaN (or, for fp32 input, 2^100 or more) gets step = NaN, so
// that every output row of that activation row comes out NaN as the reference's arithmetic would have it.
//
// fp16 input: x * 2^(13-e) = 256 hi + lo with v = x * 2^(5-e) in (-64, 64); hi = v rounded to nearest in the
// 1536 binade of fp16 (one unit per ulp: the digit is the low byte of the sum), lo = 256 (v - hi) exactly, in
// [-128, 128], capped at 127 (a tie leaves 128: one unit of error, 2^-14 of the group's top) and rounded the
// same way.
__device__ inline void digits_of_f16(const uint32_t raw[8], bool low_digit, uint32_t b[4], float &step_here) {
    // largest |x| of the 64 columns by bit pattern: NaN patterns sort above infinity, infinity above the rest
    uint32_t big = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) big = __vmaxu2(big, raw[i] & 0x7fff7fffu);
    uint32_t top = max(big & 0xffffu, big >> 16);
    top = max(top, __shfl_xor_sync(0xffffffffu, top, 1));
    top = max(top, __shfl_xor_sync(0xffffffffu, top, 2));
    const bool finite = top < 0x7c00u;
    int e = (int)(top >> 10) - 15;  // largest |x| in [2^e, 2^(e+1)) (subnormals: below 2^-14)
    e = min(max(e, -10), 15);       // 2^(5-e) must be an fp16; smaller groups keep fewer bits, of a tiny value
    const float factor = __uint_as_float((uint32_t)(127 + 5 - e) << 23);
    step_here = finite ? __uint_as_float((uint32_t)(127 + e - 13) << 23) : __uint_as_float(0x7fc00000u);
    const __half2 f_hi = __float2half2_rn(factor);
    const __half2 magic = __float2half2_rn(1536.0f), times256 = __float2half2_rn(256.0f);
    const __half2 cap = __float2half2_rn(127.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t digit[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t bits = finite ? raw[2 * i + h] : 0u;
            const __half2 x2 = *reinterpret_cast<const __half2 *>(&bits);
            const __half2 v = __hmul2(x2, f_hi);
            const __half2 hi_m = __hadd2(v, magic);
            const __half2 hi = __hsub2(hi_m, magic);
            const __half2 lo = __hmul2(__hsub2(v, hi), times256);
            const __half2 lo_m = __hadd2(__hmin2(lo, cap), magic);
            digit[h] = low_digit ? *reinterpret_cast<const uint32_t *>(&lo_m)
                                 : *reinterpret_cast<const uint32_t *>(&hi_m);
        }
        b[i] = __byte_perm(digit[0], digit[1], 0x6240);
    }
}
// fp32 input: the same digits from v = x * 2^(5-e) in fp32, e the exponent of the group's largest magnitude
__device__ inline void digits_of_f32(const float v[16], bool low_digit, uint32_t b[4], float &step_here) {
    uint32_t big = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) big = max(big, __float_as_uint(v[i]) & 0x7fffffffu);
    big = max(big, __shfl_xor_sync(0xffffffffu, big, 1));
    big = max(big, __shfl_xor_sync(0xffffffffu, big, 2));
    const bool finite = big < (227u << 23);  // below 2^100
    int e = (int)(big >> 23) - 127;           // largest |x| in [2^e, 2^(e+1))
    e = min(max(e, -100), 100);
    const float factor = __uint_as_float((uint32_t)(127 + 5 - e) << 23);  // |x| * factor < 64
    step_here = finite ? __uint_as_float((uint32_t)(127 + e - 13) << 23) : __uint_as_float(0x7fc00000u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t word = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int column = 4 * i + ((q & 1) << 1) + (q >> 1);  // 4i, 4i+2, 4i+1, 4i+3
            const float scaled = finite ? v[column] * factor : 0.0f;
            const float hi = rintf(scaled);
            const float lo = fminf(rintf((scaled - hi) * 256.0f), 127.0f);
            const int digit = (int)(low_digit ? lo : hi);
            word |= ((uint32_t)digit & 0xffu) << (8 * q);
        }
        b[i] = word;
    }
}
// One pass of a warp makes the entries of P = 4 >> shift consecutive groups, shift = 0, 1, 2 for M = 1, 2, 3..4:
// the eight (activation row, digit) columns of the B operand are four "slots" of two digits, and with fewer than
// four activation rows the spare slots take the same rows of the following groups.  Lane (gid, t): slot gid >> 1
// = (group q = slot >> shift of the pass, activation row m = slot & (2^shift - 1)), digit gid & 1.
struct Pass {
    uint32_t q, m;      // this lane's group of the pass and activation row
    bool live;          // that group and row exist
};
__device__ inline Pass pass_of(int lane, uint32_t shift, uint32_t count, uint32_t m_rows) {
    const uint32_t slot = (uint32_t)lane >> 3;
    Pass pass;
    pass.q = slot >> shift;
    pass.m = slot & ((1u << shift) - 1u);
    pass.live = pass.q < count && pass.m < m_rows;
    return pass;
}
// digits in hand (b, step_here): the sums of the pass's groups on the tensor pipe, then everything to the entries
__device__ inline void pass_store(const uint32_t b[4], float step_here, const Pass &pass, uint32_t shift, uint32_t count,
                                  uint32_t m_rows, uint8_t *first_entry, uint32_t entry_bytes, int lane) {
    const int gid = lane >> 2, t = lane & 3;
    // accumulator column pair t belongs to slot t, whose step sits in lane 8 t
    const float step = __shfl_sync(0xffffffffu, step_here, 8 * t);
    // the sum of a group's 64 values, exact: a row of ones against the digits
    const uint32_t ones[4] = {0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u};
    int s[4];
    mma_16832_u8s8(s, ones, b[0], b[1], true);
    mma_16832_u8s8(s, ones, b[2], b[3], false);
    if (pass.live) {
        *reinterpret_cast<uint4 *>(first_entry + pass.q * entry_bytes + (pass.m * 8 + (gid & 1) * 4 + t) * 16) =
            make_uint4(b[0], b[1], b[2], b[3]);
    }
    const uint32_t q = (uint32_t)t >> shift, m = (uint32_t)t & ((1u << shift) - 1u);
    if (gid == 0 && q < count && m < m_rows) {
        const float sum = step * (float)(s[0] * 256 + s[1]);
        *reinterpret_cast<float2 *>(first_entry + q * entry_bytes + 128 * m_rows + m * 8) = make_float2(step, sum);
    }
}
// the whole pass for groups [group, group + count): fp16 x from `raw` (fetched earlier by pass_fetch), fp32 x from memory
__device__ inline void pass_fetch(const DecodeJob &job, size_t K, uint32_t group, const Pass &pass, int lane,
                                  uint32_t raw[8]) {
    fetch_x16(job.x, (size_t)pass.m * K + (size_t)(group + pass.q) * kGroup + 16 * (lane & 3), pass.live, raw);
}
__device__ inline void pass_finish(const DecodeJob &job, size_t K, uint32_t group, const Pass &pass, uint32_t shift,
                                   uint32_t count, uint32_t m_rows, const uint32_t raw[8], uint8_t *first_entry,
                                   uint32_t entry_bytes, int lane) {
    const bool low_digit = ((lane >> 2) & 1) != 0;
    uint32_t b[4];
    float step_here;
    if (job.x_dtype == kF32) {
        float v[16];
        fetch_x32(job.x, (size_t)pass.m * K + (size_t)(group + pass.q) * kGroup + 16 * (lane & 3), pass.live, v);
        digits_of_f32(v, low_digit, b, step_here);
    } else {
        digits_of_f16(raw, low_digit, b, step_here);
    }
    pass_store(b, step_here, pass, shift, count, m_rows, first_entry, entry_bytes, lane);
}

// fp16 form.  Lane (gid, t), column tile n: activation row m = 8 n + gid, columns 16 t .. 16 t + 15.  An entry gets:
//   [n * 1024 + lane * 32, +32)           the eight B registers of the four m16n8k16 MMAs of a tile
//   [NT * 1024 + 8 (8 n + m'), +8)        {step, step * sum} of activation row 8 n + m'
// fp16 input passes through unchanged (step = 1); fp32 input is scaled by the power of two that brings the
// group's largest magnitude into [1, 2) and then rounded to fp16, the power going into step.
// `held` (fp16 input only): the registers fetched a stage ahead, [n][8].
template <int NT>
__device__ inline void entry_f16(const DecodeJob &job, uint32_t m_rows, size_t K, uint32_t group, const uint32_t *held,
                                 uint8_t *entry, int lane) {
    const int gid = lane >> 2, t = lane & 3;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const uint32_t m = n * 8 + gid;
        uint32_t raw[8];
        float step_here = 1.0f;
        if (job.x_dtype == kF32) {
            float v[16];
            fetch_x32(job.x, (size_t)m * K + (size_t)group * kGroup + 16 * t, m < m_rows, v);
            uint32_t big = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) big = max(big, __float_as_uint(v[i]) & 0x7fffffffu);
            big = max(big, __shfl_xor_sync(0xffffffffu, big, 1));
            big = max(big, __shfl_xor_sync(0xffffffffu, big, 2));
            const bool finite = big < (227u << 23);
            int e = (int)(big >> 23) - 127;
            e = min(max(e, -100), 100);
            const float down = __uint_as_float((uint32_t)(127 - e) << 23);
            step_here = finite ? __uint_as_float((uint32_t)(127 + e) << 23) : __uint_as_float(0x7fc00000u);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const __half2 pair = finite ? __floats2half2_rn(v[2 * i] * down, v[2 * i + 1] * down)
                                            : __float2half2_rn(0.0f);
                raw[i] = *reinterpret_cast<const uint32_t *>(&pair);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) raw[i] = held[n * 8 + i];
        }
        // group sums of x on the tensor pipe: a fragment of ones times the same B
        const uint32_t ones[4] = {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u};
        float total[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) mma_16816(total, ones, raw[2 * i], raw[2 * i + 1], i == 0);
        // accumulator columns 2t, 2t+1 are activation rows 8n + 2t, 8n + 2t + 1: their steps sit in lanes 8t, 8t + 4
        const float step0 = __shfl_sync(0xffffffffu, step_here, 8 * t);
        const float step1 = __shfl_sync(0xffffffffu, step_here, 8 * t + 4);
        uint4 *out = reinterpret_cast<uint4 *>(entry + n * 1024 + lane * 32);
        out[0] = make_uint4(raw[0], raw[1], raw[2], raw[3]);
        out[1] = make_uint4(raw[4], raw[5], raw[6], raw[7]);
        if (gid == 0) {
            *reinterpret_cast<float4 *>(entry + NT * 1024 + (n * 8 + 2 * t) * 8) =
                make_float4(step0, step0 * total[0], step1, step1 * total[1]);
        }
    }
}

// fp16 form: this lane's fp16 activations of one group into `held` [NT][8] (rows 8 n + gid)
template <int NT>
__device__ inline void fetch_held(const DecodeJob &job, uint32_t m_rows, size_t K, uint32_t group, int lane,
                                  uint32_t *held) {
    const int gid = lane >> 2, t = lane & 3;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const uint32_t m = n * 8 + gid;
        fetch_x16(job.x, (size_t)m * K + (size_t)group * kGroup + 16 * t, m < m_rows, held + n * 8);
    }
}

// ---------------------------------------------------------------------------
// a consumer warp's work on one tile of one group
// ---------------------------------------------------------------------------
// Integer form: lane (gid, t) accumulates rows gid (acc[0]) and gid + 8 (acc[1]) of activation row t.
__device__ inline void tile_digits(const uint8_t *tile, const uint8_t *entry, uint32_t digits_at, uint32_t steps_at,
                                   int lane, float acc[2]) {
    const int gid = lane >> 2;
    const uint4 codes = *reinterpret_cast<const uint4 *>(tile + piece_index(lane) * 16);
    const uint2 meta = *reinterpret_cast<const uint2 *>(tile + kTileCodeBytes + gid * 8);
    // B columns beyond the activation rows there are read some valid lane's digits and steps instead of zeros
    // (digits_at, steps_at): their sums land in accumulators nobody stores, and the loads need no predicate
    const uint4 b = *reinterpret_cast<const uint4 *>(entry + digits_at);
    const float2 ss = *reinterpret_cast<const float2 *>(entry + steps_at);
    // Word i covers columns 4i .. 4i+3 of this lane's 16; its even nibbles are row gid, its odd nibbles row gid + 8.
    // Row gid gets the masked nibbles.  Row gid + 8 gets the RAW bytes, 16 * (its code) + (row gid's code): its
    // integer sum is then 16 * (the wanted sum) + (row gid's sum), and one subtraction after the MMAs replaces
    // eight shift-and-mask instructions before them (bytes up to 255 times digits up to 128 over 64 columns stay
    // far inside 32 bits).
    const uint32_t a0[4] = {codes.x & 0x0F0F0F0Fu, codes.x, codes.y & 0x0F0F0F0Fu, codes.y};
    const uint32_t a1[4] = {codes.z & 0x0F0F0F0Fu, codes.z, codes.w & 0x0F0F0F0Fu, codes.w};
    int c[4];
    mma_16832_u8s8(c, a0, b.x, b.y, true);
    mma_16832_u8s8(c, a1, b.z, b.w, false);
    const int top = c[0] * 256 + c[1];
    const float top_row = (float)top;
    const float low_row = (float)(c[2] * 256 + c[3] - top);  // 16 x the sum of row gid + 8
    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&meta.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&meta.y));
    acc[0] = fmaf(lo.x * ss.x, top_row, fmaf(lo.y, ss.y, acc[0]));
    acc[1] = fmaf(hi.x * (0.0625f * ss.x), low_row, fmaf(hi.y, ss.y, acc[1]));
}

// fp16 form: lane (gid, t), column tile n: acc[4n + j] = (row gid + 8 (j >> 1), activation row 8n + 2t + (j & 1))
template <int NT>
__device__ inline void tile_f16(const uint8_t *tile, const uint8_t *slot, int lane, float acc[4 * NT]) {
    const int gid = lane >> 2, t = lane & 3;
    const uint4 codes = *reinterpret_cast<const uint4 *>(tile + piece_index(lane) * 16);
    const uint2 meta = *reinterpret_cast<const uint2 *>(tile + kTileCodeBytes + gid * 8);
    float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&meta.x));
    float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&meta.y));
    lo.x *= 16777216.0f;  // the codes go to the tensor pipe as q * 2^-24 (fp16 subnormal bit patterns)
    hi.x *= 1048576.0f;   // and 16 q * 2^-24
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const uint4 *xs = reinterpret_cast<const uint4 *>(slot + n * 1024 + lane * 32);
        const uint4 x0 = xs[0], x1 = xs[1];
        const float4 ss = *reinterpret_cast<const float4 *>(slot + NT * 1024 + (n * 8 + 2 * t) * 8);
        const uint32_t xb[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        float c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t word = i == 0 ? codes.x : i == 1 ? codes.y : i == 2 ? codes.z : codes.w;
            uint32_t a[4];
            word_to_codes_subnormal(word, a);
            mma_16816(c, a, xb[2 * i], xb[2 * i + 1], i == 0);
        }
        acc[4 * n + 0] = fmaf(lo.x * ss.x, c[0], fmaf(lo.y, ss.y, acc[4 * n + 0]));
        acc[4 * n + 1] = fmaf(lo.x * ss.z, c[1], fmaf(lo.y, ss.w, acc[4 * n + 1]));
        acc[4 * n + 2] = fmaf(hi.x * ss.x, c[2], fmaf(hi.y, ss.y, acc[4 * n + 2]));
        acc[4 * n + 3] = fmaf(hi.x * ss.z, c[3], fmaf(hi.y, ss.w, acc[4 * n + 3]));
    }
}

// row offset inside the 16-row tile and activation row of accumulator v of lane (gid, t)
template <int MODE>
__device__ inline void place_of(int v, int gid, int t, uint32_t &row, uint32_t &m) {
    if (MODE == 0) {
        row = gid + 8 * v;
        m = t;
    } else {
        row = gid + 8 * ((v >> 1) & 1);
        m = 8 * (v >> 2) + 2 * t + (v & 1);
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int MODE, bool SEQ>
__global__ void __launch_bounds__(kDecodeThreads, 2)
decode_kernel(const __grid_constant__ PassParams p) {
    using F = Form<MODE>;
    constexpr int NT = F::NT, VALS = F::VALS;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    if (!SEQ) asm volatile("griddepcontrol.launch_dependents;");  // the next launch may start prefetching weights

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, t = lane & 3;
    const uint32_t cta = blockIdx.x, ctas = gridDim.x;
    const uint32_t m_rows = p.m_rows, stages = p.stages;
    const uint32_t entry_bytes = F::entry_bytes(m_rows);

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);  // full[3], empty[3], xfull[3], xempty[3]
    volatile uint32_t *failed = reinterpret_cast<volatile uint32_t *>(smem_raw + 96);
    uint32_t *published = reinterpret_cast<uint32_t *>(smem_raw + 100);  // tiles this CTA finished since it last said so
    uint8_t *ring = smem_raw + 128;
    uint8_t *entries = ring + stages * kStageBytes;  // [kEntrySets][8 groups][entry_bytes]
    float *xchg = reinterpret_cast<float *>(entries + kEntrySets * kStageGroups * entry_bytes);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 24, xfull0 = full0 + 48, xempty0 = full0 + 72;
    const uint32_t opened0 = full0 + 104;  // completes once: the first entries of a single launch are in place
    const uint32_t ring0 = smem_u32(ring);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kConsumers);
        }
        for (uint32_t c = 0; c < kEntrySets; ++c) {
            mbar_init(xfull0 + 8 * c, kConsumers);
            mbar_init(xempty0 + 8 * c, kConsumers);
        }
        mbar_init(opened0, kConsumers);
        *failed = 0;
        *published = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const uint32_t job_count = SEQ ? p.job_count : 1u;
    // One launch, K split over the CTAs of a cluster (CTA rank = part, one unit per CTA): the partial sums meet in
    // the shared memory of the cluster's first CTA instead of global memory.  The same answer in every thread.
    const bool clustered = !SEQ && p.cluster != 0 && p.job.parts > 1 && gridDim.x == p.job.units;

    if (warp == kProducerWarp) {
        // ---- weight producer: one thread streams every unit of every job, never draining the ring ----
        if (lane == 0) {
            uint32_t it = 0, issued = 0, slot = 0, lap_parity = 0;
            auto ring_step = [stages](uint32_t &at, uint32_t &parity) {
                if (++at == stages) {
                    at = 0;
                    parity ^= 1u;
                }
            };
            const uint64_t policy = stream_once_policy();
            const bool throttle = p.throttle != 0;
            for (uint32_t j = 0; j < job_count; ++j) {
                const DecodeJob &job = SEQ ? p.jobs[j] : p.job;
                if (SEQ) {
                    // This thread reads its way through the job table far ahead of the consumers, one dependent
                    // load after another: the descriptors of the next two jobs start for L1 now, so that walking
                    // into them later costs no round trip to L2 with the copy engine idle meanwhile.
                    for (uint32_t ahead = 1; ahead <= 2 && j + ahead < job_count; ++ahead) {
                        const uint8_t *next = reinterpret_cast<const uint8_t *>(p.jobs + j + ahead);
                        for (uint32_t line = 0; line < sizeof(DecodeJob); line += 128) {
                            asm volatile("prefetch.global.L1 [%0];" ::"l"(next + line));
                        }
                    }
                }
                const uint32_t G = job.groups;
                for (uint32_t index = cta; index < job.units; index += ctas) {
                    const Unit u = unit_of(job, index);
                    const uint8_t *a = job.tiles[u.segment] +
                                       (size_t)(job.fused ? u.local : 2 * u.local) * G * kUnitBytes;
                    const uint8_t *b = job.fused ? job.up_tiles + (size_t)u.local * G * kUnitBytes
                                                 : a + (size_t)G * kUnitBytes;
                    for (uint32_t g = u.g0; g < u.g1; g += kStageGroups, ++it, ring_step(slot, lap_parity)) {
                        const uint32_t s = slot;  // it % stages, and lap_parity = (it / stages) & 1, kept without dividing
                        if (it >= stages) mbar_wait(empty0 + 8 * s, lap_parity ^ 1u, failed, 0x91u);
                        // A single launch starts before the launch it depends on has finished, and the ring would
                        // fill while the consumers wait for their activations; then their first loads queue behind
                        // a whole ring of weight requests.  The last stage of the first fill waits for the first
                        // entries instead (a barrier of its own that completes once: one that keeps cycling could
                        // run two phases ahead of a thread that only watches it, and the watcher would wait for
                        // a third).
                        if (!SEQ && throttle && it == stages - 1) mbar_wait(opened0, 0, failed, 0x96u);
                        if (*failed != 0) continue;  // no new copies once a wait has expired
                        const uint32_t bytes = min(kStageGroups, u.g1 - g) * kUnitBytes;
                        mbar_expect_tx(full0 + 8 * s, u.has_b ? 2 * bytes : bytes);
                        bulk_copy_to_shared(ring0 + s * kStageBytes, a + (size_t)g * kUnitBytes, bytes, full0 + 8 * s, policy);
                        if (u.has_b) {
                            bulk_copy_to_shared(ring0 + s * kStageBytes + kStageGroups * kUnitBytes,
                                                b + (size_t)g * kUnitBytes, bytes, full0 + 8 * s, policy);
                        }
                        issued = it + 1;
                    }
                }
            }
            if (*failed != 0) {
                // the copies already issued must land before this CTA's shared memory is released: the last
                // fill of every stage (a bounded spin of its own, whatever the failure flag says)
                for (uint32_t i = issued > stages ? issued - stages : 0; i < issued; ++i) {
                    const long long start = clock64();
                    while (!mbar_try_wait(full0 + 8 * (i % stages), (i / stages) & 1) &&
                           clock64() - start < kWaitLimitCycles) {
                    }
                }
            }
        }
        __syncwarp();
        if (clustered) {  // the two barriers of the consumers' split-K exchange count every thread of the cluster
            cluster_barrier();
            cluster_barrier();
        }
    } else {
        // ---- consumers: warp w owns tile w & 3 of block w >> 2 of every pair block this CTA visits ----
        const int k = warp >> 2, r = warp & 3;
        bool in_stream_order = SEQ;  // a single launch: whether the launches before it are known to be complete
        bool opened = false;         // a single launch: whether this warp has reported its first entries
        uint32_t epoch = 0;
        if (SEQ) epoch = *reinterpret_cast<volatile uint32_t *>(p.epoch) + 1;
        // the stage counter, and what it says about the rings, kept without dividing: slot = it % stages with
        // lap_parity = (it / stages) & 1, entry set e = it % kEntrySets with e_parity = (it / kEntrySets) & 1
        uint32_t it = 0, slot = 0, lap_parity = 0, e = 0, e_parity = 0;
        // entry set and lap parity of the stage `ahead` (0..2) stages after the current one
        auto set_at = [&](uint32_t ahead, uint32_t &index, uint32_t &parity) {
            index = e + ahead;
            parity = e_parity;
            if (index >= kEntrySets) {
                index -= kEntrySets;
                parity ^= 1u;
            }
        };
        // optional phase clocks: consumer warp 0 stamps its own progress (its lane 0 adds them up at the end)
        const bool stamp = SEQ && p.profile != nullptr && warp == 0 && lane == 0;
        long long *phase = reinterpret_cast<long long *>(xchg + 4 * 32 * F::XCHG_VALS);  // [kProfileSlots], this lane's alone
        if (stamp) {
            for (int slot = 0; slot < kProfileSlots; ++slot) phase[slot] = 0;
        }
        long long mark = stamp ? clock64() : 0;
        const long long begun = mark;
        auto lap = [&](int slot) {
            if (stamp) {
                const long long now = clock64();
                phase[slot] += now - mark;
                mark = now;
            }
        };
        // Entries are made in passes: in the integer form one pass of a warp serves 4, 2 or 1 groups (M = 1, 2,
        // 3..4), in the fp16 form one.  The warps take the passes of successive stages in turn, and every pass
        // runs TWO stages ahead of the tiles that use it (three sets of entries, handed over through the mbarrier
        // pairs xfull / xempty, eight arrivals each): a warp busy with a pass delays nobody, there is no barrier
        // among the consumers.
        const uint32_t shift = MODE != 0 ? 2u : m_rows == 1 ? 0u : m_rows == 2 ? 1u : 2u;
        const uint32_t per_pass = 4u >> shift, pass_log = 2u - shift;  // groups per pass and their logarithm
        const uint8_t *lane_tiles = ring + (size_t)k * kStageGroups * kUnitBytes + r * kTileBytes;
        // integer form: where this lane reads its B registers and its row's steps inside an entry
        const uint32_t digits_at = ((uint32_t)lane < 8 * m_rows ? (uint32_t)lane : (uint32_t)lane & 7u) * 16u;
        const uint32_t steps_at = 128u * m_rows + min((uint32_t)t, m_rows - 1) * 8u;
        for (uint32_t j = 0; j < job_count; ++j) {
            const DecodeJob &job = SEQ ? p.jobs[j] : p.job;
            const bool fused = job.fused != 0;
            const bool x16 = job.x_dtype != kF32;
            const size_t K = (size_t)job.groups * kGroup;
            if (SEQ) {
                // the next job's descriptor on its way into L1 while this job runs
                if (warp == 0 && j + 1 < job_count && lane * 128u < sizeof(DecodeJob)) {
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const uint8_t *>(p.jobs + j + 1) + lane * 128));
                }
                if (j > 0 && cta < job.units) {
                    // x of this job may be what the previous job wrote, on this or any rank: wait until every
                    // 16-row tile of it, on every rank, has been counted in this launch.  One warp per CTA asks
                    // (with a pause between questions: thousands of askers on eight lines of L2 would delay the
                    // very additions they wait for); a barrier passes its answer on to the others.
                    if (warp == 0) {
                        const uint32_t expected = 4u * p.jobs[j - 1].expected_blocks * epoch;
                        const uint32_t *counter = p.done + ((size_t)(j - 1) * 8 + (lane & 7)) * kDoneStride;
                        const long long start = clock64();
                        for (;;) {
                            uint32_t seen = 0;
                            if (lane < 8) {
                                if (p.world > 1) {
                                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                                } else {
                                    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                                }
                            }
                            seen += __shfl_xor_sync(0xffffffffu, seen, 1);
                            seen += __shfl_xor_sync(0xffffffffu, seen, 2);
                            seen += __shfl_xor_sync(0xffffffffu, seen, 4);
                            seen = __shfl_sync(0xffffffffu, seen, 0);
                            if ((int32_t)(seen - expected) >= 0 || *failed != 0) break;
                            if (clock64() - start > kWaitLimitCycles) {
                                *failed = 0x95u;
                                break;
                            }
                            __nanosleep(100);
                        }
                        asm volatile("fence.acq_rel.gpu;" ::: "memory");
                    }
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                    lap(kProfileDependency);
                }
            }
            for (uint32_t index = cta; index < job.units; index += ctas) {
                const Unit u = unit_of(job, index);
                const bool active = k == 0 || u.has_b;
                float acc[VALS];
#pragma unroll
                for (int v = 0; v < VALS; ++v) acc[v] = 0.0f;
                // this warp's pass of the stage with counter `counter` (groups from `g`), if it has one: [first, +count)
                auto my_pass = [&](uint32_t counter, uint32_t g, uint32_t &first, uint32_t &count) {
                    const uint32_t groups_in_stage = min(kStageGroups, u.g1 - g);
                    const uint32_t passes = (groups_in_stage + per_pass - 1) >> pass_log;
                    const uint32_t mine = ((uint32_t)warp - counter * (kStageGroups >> pass_log)) & 7u;
                    first = mine * per_pass;
                    count = mine < passes ? min(per_pass, groups_in_stage - first) : 0u;
                };
                uint32_t raw[MODE == 0 ? 8 : 8 * NT];
                // fetch == true: only send the loads off (fp16 x); false: make the entries from what was fetched
                auto pass_step = [&](uint32_t ahead, uint32_t g, bool fetch) {  // the stage `ahead` after the current
                    uint32_t first, count, index, parity;
                    my_pass(it + ahead, g, first, count);
                    if (count == 0) return;
                    set_at(ahead, index, parity);
                    uint8_t *first_entry = entries + (size_t)index * kStageGroups * entry_bytes + first * entry_bytes;
                    if constexpr (MODE == 0) {
                        const Pass pass = pass_of(lane, shift, count, m_rows);
                        if (fetch) {
                            if (x16) pass_fetch(job, K, g + first, pass, lane, raw);
                        } else {
                            pass_finish(job, K, g + first, pass, shift, count, m_rows, raw, first_entry, entry_bytes, lane);
                        }
                    } else {
                        if (fetch) {
                            if (x16) fetch_held<NT>(job, m_rows, K, g + first, lane, raw);
                        } else {
                            entry_f16<NT>(job, m_rows, K, g + first, raw, first_entry, lane);
                        }
                    }
                };
                auto hand_over = [&](uint32_t ahead) {  // this warp's part of that stage's entries is in place
                    uint32_t index, parity;
                    set_at(ahead, index, parity);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(xfull0 + 8 * index);
                };
                auto wait_set_free = [&](uint32_t ahead) {  // the tiles of three stages before that one are done with the set
                    if (it + ahead >= kEntrySets) {
                        uint32_t index, parity;
                        set_at(ahead, index, parity);
                        mbar_wait(xempty0 + 8 * index, parity ^ 1u, failed, 0x94u);
                    }
                };
                if (!in_stream_order) {
                    // x, y, residual and scratch belong to stream order; everything above (and the weights) does not
                    asm volatile("griddepcontrol.wait;" ::: "memory");
                    in_stream_order = true;
                }
                // the unit's first two stages: nothing to hide their entries behind.  With several groups to a pass
                // a warp has a pass in at most one of the two, so the stages' passes run side by side on
                // different warps; otherwise a warp makes its two passes one after the other.
                if (per_pass > 1) {
                    const uint32_t g2 = u.g0 + kStageGroups;
                    uint32_t first, count;
                    my_pass(it, u.g0, first, count);
                    const bool second = count == 0 && g2 < u.g1;  // no pass in the first stage: maybe in the second
                    wait_set_free(0);
                    if (g2 < u.g1) wait_set_free(1);
                    pass_step(second ? 1u : 0u, second ? g2 : u.g0, true);
                    pass_step(second ? 1u : 0u, second ? g2 : u.g0, false);
                    hand_over(0);
                    if (g2 < u.g1) hand_over(1);
                } else {
#pragma unroll
                    for (uint32_t d = 0; d < 2; ++d) {
                        const uint32_t g = u.g0 + d * kStageGroups;
                        if (g < u.g1) {
                            wait_set_free(d);
                            pass_step(d, g, true);
                            pass_step(d, g, false);
                            hand_over(d);
                        }
                    }
                }
                if (!SEQ && !opened) {  // this warp's share of the launch's first entries is in place
                    opened = true;
                    if (lane == 0) mbar_arrive(opened0);
                }
                lap(kProfileEntries);
                auto next_stage = [&]() {
                    ++it;
                    if (++slot == stages) {
                        slot = 0;
                        lap_parity ^= 1u;
                    }
                    if (++e == kEntrySets) {
                        e = 0;
                        e_parity ^= 1u;
                    }
                };
                for (uint32_t g = u.g0; g < u.g1; g += kStageGroups, next_stage()) {
                    const uint32_t s = slot;
                    const uint32_t in_stage = min(kStageGroups, u.g1 - g);
                    const uint8_t *set = entries + (size_t)e * kStageGroups * entry_bytes;
                    const uint32_t g_ahead = g + 2 * kStageGroups;
                    if (g_ahead < u.g1) pass_step(2, g_ahead, true);  // loads first: they pass under the tiles
                    mbar_wait(xfull0 + 8 * e, e_parity, failed, 0x93u);
                    lap(kProfileEntries);
                    mbar_wait(full0 + 8 * s, lap_parity, failed, 0x92u);
                    lap(kProfileWeights);
                    if (active) {
                        const uint8_t *tiles = lane_tiles + s * kStageBytes;
                        if (in_stage == kStageGroups) {  // the common case without a branch between the tiles
#pragma unroll
                            for (uint32_t q = 0; q < kStageGroups; ++q) {
                                if (MODE == 0) {
                                    tile_digits(tiles + q * kUnitBytes, set + q * entry_bytes, digits_at, steps_at, lane, acc);
                                } else {
                                    tile_f16<NT>(tiles + q * kUnitBytes, set + q * entry_bytes, lane, acc);
                                }
                            }
                        } else {
                            for (uint32_t q = 0; q < in_stage; ++q) {
                                if (MODE == 0) {
                                    tile_digits(tiles + q * kUnitBytes, set + q * entry_bytes, digits_at, steps_at, lane, acc);
                                } else {
                                    tile_f16<NT>(tiles + q * kUnitBytes, set + q * entry_bytes, lane, acc);
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(xempty0 + 8 * e);
                        mbar_arrive(empty0 + 8 * s);
                    }
                    lap(kProfileTiles);
                    if (g_ahead < u.g1) {
                        wait_set_free(2);
                        pass_step(2, g_ahead, false);
                        hand_over(2);
                        lap(kProfileEntries);
                    }
                }

                // ---- the unit is done: finish this warp's tile ----
                float second[VALS];  // the up half of a fused pair, once known
#pragma unroll
                for (int v = 0; v < VALS; ++v) second[v] = 0.0f;
                bool finisher;
                if (job.parts == 1) {
                    if (fused) {
                        // the up warp hands its sums to the gate warp of the same tile through shared memory
                        float *mine = xchg + (size_t)(r * 32 + lane) * F::XCHG_VALS;
#pragma unroll
                        for (int round = 0; round < VALS / (int)F::XCHG_VALS; ++round) {
                            if (k == 1) {
#pragma unroll
                                for (int v = 0; v < (int)F::XCHG_VALS; ++v) mine[v] = acc[round * F::XCHG_VALS + v];
                            }
                            pair_barrier(2 + r);
                            if (k == 0) {
#pragma unroll
                                for (int v = 0; v < (int)F::XCHG_VALS; ++v) second[round * F::XCHG_VALS + v] = mine[v];
                            }
                            pair_barrier(2 + r);
                        }
                    }
                    finisher = fused ? k == 0 : active;
                } else if (clustered) {
                    // K is split over the CTAs of this cluster.  Once every CTA is through with its ring (first
                    // barrier), each warp puts its sums into the first CTA's ring, part by part; after the
                    // second barrier that CTA adds them in part order, the order of the path through global
                    // memory below, so both give the same bits.
                    cluster_barrier();
                    if (active) {
                        const uint32_t slot = cluster_address(ring0 + (((u.part * VALS) * 8 + warp) * 32 + lane) * 4u, 0u);
#pragma unroll
                        for (int v = 0; v < VALS; ++v) cluster_store(slot + (uint32_t)v * 8u * 32u * 4u, acc[v]);
                    }
                    cluster_barrier();
                    finisher = u.part == 0 && (fused ? k == 0 : active);
                    if (finisher) {
                        const float *base = reinterpret_cast<const float *>(ring);
                        const int gate_warp = fused ? r : warp;
#pragma unroll
                        for (int v = 0; v < VALS; ++v) acc[v] = 0.0f;
                        for (uint32_t q = 0; q < job.parts; ++q) {
#pragma unroll
                            for (int v = 0; v < VALS; ++v) {
                                acc[v] += base[((q * VALS + v) * 8 + gate_warp) * 32 + lane];
                                if (fused) second[v] += base[((q * VALS + v) * 8 + gate_warp + 4) * 32 + lane];
                            }
                        }
                    }
                } else {
                    // K is split over CTAs: park the sums; the last warp to arrive for this tile adds every
                    // part's in part order (the same sum whoever is last)
                    finisher = false;
                    if (active) {
                        float *slot = p.scratch + (size_t)index * (8 * 32 * VALS);
#pragma unroll
                        for (int v = 0; v < VALS; ++v) slot[(v * 8 + warp) * 32 + lane] = acc[v];
                        __syncwarp();
                        uint32_t before = 0;
                        uint32_t *counter = p.counters + (size_t)u.pair * 8 + (fused ? r : warp);
                        if (lane == 0) {
                            asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;"
                                         : "=r"(before) : "l"(counter), "r"(1u) : "memory");
                        }
                        before = __shfl_sync(0xffffffffu, before, 0);
                        __syncwarp();
                        const uint32_t needed = fused ? 2 * job.parts : job.parts;
                        if (before + 1 == needed) {
                            finisher = true;
                            if (lane == 0) *counter = 0;  // ready for the next job or launch (ordered by what follows)
                            asm volatile("fence.acq_rel.gpu;" ::: "memory");
                            const float *base = p.scratch + (size_t)(u.pair * job.parts) * (8 * 32 * VALS);
                            const int gate_warp = fused ? r : warp;
#pragma unroll
                            for (int v = 0; v < VALS; ++v) acc[v] = 0.0f;
                            // several parts' loads in flight at a time, added in part order
                            for (uint32_t q0 = 0; q0 < job.parts; q0 += F::SUM_UNROLL) {
                                float first[F::SUM_UNROLL][VALS], other[F::SUM_UNROLL][VALS];
#pragma unroll
                                for (int i = 0; i < F::SUM_UNROLL; ++i) {
                                    const bool live = q0 + i < job.parts;
                                    const float *from = base + (size_t)(q0 + i) * (8 * 32 * VALS);
#pragma unroll
                                    for (int v = 0; v < VALS; ++v) {
                                        first[i][v] = live ? __ldcg(from + (v * 8 + gate_warp) * 32 + lane) : 0.0f;
                                        other[i][v] = live && fused ? __ldcg(from + (v * 8 + gate_warp + 4) * 32 + lane) : 0.0f;
                                    }
                                }
#pragma unroll
                                for (int i = 0; i < F::SUM_UNROLL; ++i) {
#pragma unroll
                                    for (int v = 0; v < VALS; ++v) {
                                        acc[v] += first[i][v];
                                        second[v] += other[i][v];
                                    }
                                }
                            }
                        }
                    }
                }
                if (finisher) {
                    const int out_k = fused ? 0 : k;
                    const uint32_t row0 = (fused ? u.local * 64 : u.local * 128 + out_k * 64) + r * kTileRows;
                    const uint32_t rows = job.rows[u.segment], ldy = job.ldy[u.segment];
#pragma unroll
                    for (int v = 0; v < VALS; ++v) {
                        uint32_t row, m;
                        place_of<MODE>(v, gid, t, row, m);
                        row += row0;
                        if (row >= rows || m >= m_rows) continue;
                        float value = acc[v];
                        // silu(g) * u from the un-rounded accumulators (qwen38_q4.metal:146-149)
                        if (fused) value = (value / (1.0f + __expf(-value))) * second[v];
                        if (job.residual != nullptr && u.segment == 0) {
                            const size_t at = (size_t)m * job.ld_residual + row;
                            value += job.residual_dtype == kF32
                                         ? reinterpret_cast<const float *>(job.residual)[at]
                                         : __half2float(reinterpret_cast<const __half *>(job.residual)[at]);
                        }
                        const size_t at = (size_t)m * ldy + row;
                        for (uint32_t rank = 0; rank < p.world; ++rank) {
                            void *destination = job.y[u.segment][rank];
                            if (destination == nullptr) continue;
                            if (job.y_dtype == kF32) {
                                reinterpret_cast<float *>(destination)[at] = value;
                            } else {
                                reinterpret_cast<__half *>(destination)[at] = __float2half_rn(value);
                            }
                        }
                    }
                    if (SEQ) {
                        __syncwarp();
                        if (lane == 0) atomicAdd(published, 1u);  // this tile is stored everywhere
                    }
                }
                if (SEQ) {
                    // One thread counts the CTA's finished tiles on every rank: one fence for all the warps'
                    // stores (the barrier orders them before it), one addition per rank.
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                    if (warp == 0 && lane == 0) {
                        const uint32_t tiles_done = atomicExch(published, 0u);
                        if (tiles_done > 0) {
                            const size_t at = ((size_t)j * 8 + (cta & 7u)) * kDoneStride;
                            if (p.world > 1) {
                                asm volatile("fence.acq_rel.sys;" ::: "memory");
                                for (uint32_t rank = 0; rank < p.world; ++rank) {
                                    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;"
                                                 ::"l"(p.peer_done[rank] + at), "r"(tiles_done) : "memory");
                                }
                            } else {
                                asm volatile("red.release.gpu.global.add.u32 [%0], %1;"
                                             ::"l"(p.done + at), "r"(tiles_done) : "memory");
                            }
                        }
                    }
                }
                lap(kProfileFinish);
            }
        }
        if (stamp) {
            phase[kProfileTotal] = clock64() - begun;
            for (int slot = 0; slot < kProfileSlots; ++slot) {
                p.profile[(size_t)cta * kProfileSlots + slot] += (unsigned long long)phase[slot];
            }
        }
    }

    __syncthreads();
    if (threadIdx.x == 0) {
        if (*failed != 0) atomicExch(p.status, *failed);
        if (SEQ) {
            // the last CTA to leave closes the launch: the next one expects one more round of completions
            __threadfence();
            const uint32_t left = atomicAdd(p.exit_count, 1u);
            if (left + 1 == ctas) {
                *p.exit_count = 0;
                *reinterpret_cast<volatile uint32_t *>(p.epoch) = *reinterpret_cast<volatile uint32_t *>(p.epoch) + 1;
            }
        }
    }
}

int mode_of(uint32_t m_rows, int variant) {
    if (m_rows <= 4 && ((variant >> 4) & 1) == 0) return 0;
    return m_rows <= 8 ? 1 : 2;
}

size_t smem_of(int mode, uint32_t m_rows, uint32_t *stages) {
    return mode == 0 ? smem_bytes_of<0>(m_rows, stages) : mode == 1 ? smem_bytes_of<1>(m_rows, stages)
                                                                    : smem_bytes_of<2>(m_rows, stages);
}

template <int MODE, bool SEQ>
cudaError_t configure(size_t smem_bytes, int *blocks_per_sm) {
    auto kernel = decode_kernel<MODE, SEQ>;
    // per instantiation and device: the dynamic shared memory granted so far, and the last occupancy answer
    static size_t granted[kMaxDevices], asked[kMaxDevices];
    static int resident[kMaxDevices];
    const int slot = device_slot();
    if (slot >= 0 && resident[slot] > 0 && asked[slot] == smem_bytes) {
        *blocks_per_sm = resident[slot];
        return cudaSuccess;
    }
    if (slot < 0 || smem_bytes > granted[slot]) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        if (status != cudaSuccess) return status;
        if (slot >= 0) granted[slot] = smem_bytes;
    }
    cudaError_t status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, kernel, kDecodeThreads, smem_bytes);
    if (status != cudaSuccess) return status;
    if (*blocks_per_sm < 1) return cudaErrorInvalidConfiguration;
    if (slot >= 0) {
        resident[slot] = *blocks_per_sm;
        asked[slot] = smem_bytes;
    }
    return cudaSuccess;
}

// How many clusters of `parts` CTAs the device holds at once (0 when it cannot say): per instantiation, device,
// cluster size and shared-memory size, asked once.
template <int MODE>
uint32_t resident_clusters(uint32_t parts, size_t smem_bytes) {
    static int known[kMaxDevices][9];
    static size_t asked[kMaxDevices][9];
    static std::mutex guard;
    const int slot = device_slot();
    if (slot < 0 || parts < 2 || parts > 8) return 0;
    std::lock_guard<std::mutex> lock(guard);
    if (known[slot][parts] == 0 || asked[slot][parts] != smem_bytes) {
        int unused = 0;
        if (configure<MODE, false>(smem_bytes, &unused) != cudaSuccess) return 0;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(parts * 64);
        config.blockDim = dim3(kDecodeThreads);
        config.dynamicSmemBytes = smem_bytes;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = parts;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, decode_kernel<MODE, false>, &config) != cudaSuccess) {
            cudaGetLastError();
            clusters = -1;
        }
        known[slot][parts] = clusters > 0 ? clusters : -1;
        asked[slot][parts] = smem_bytes;
    }
    return known[slot][parts] > 0 ? (uint32_t)known[slot][parts] : 0u;
}

cudaError_t configure_mode(int mode, bool sequence, size_t smem_bytes, int *per_sm) {
    if (sequence) {
        return mode == 0 ? configure<0, true>(smem_bytes, per_sm)
               : mode == 1 ? configure<1, true>(smem_bytes, per_sm) : configure<2, true>(smem_bytes, per_sm);
    }
    return mode == 0 ? configure<0, false>(smem_bytes, per_sm)
           : mode == 1 ? configure<1, false>(smem_bytes, per_sm) : configure<2, false>(smem_bytes, per_sm);
}

}  // namespace

uint32_t decode_max_m() { return 16; }

// ---------------------------------------------------------------------------
// Scratch that exists without any allocation call: file-scope device arrays,
// part of the library image, held by every GPU that loads it until the process
// exits.  In host code the names below are only stand-ins for the symbols; the
// device addresses come from cudaGetSymbolAddress, looked up once per device
// with that device current.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 1u << 20;  // 1 MiB of partial-sum slots
constexpr size_t kStaticCounterCount = 4096;      // one arrival counter per 16-row tile of a split pair block
static __device__ __align__(256) float q4b_static_scratch[kStaticScratchBytes / sizeof(float)];
static __device__ __align__(256) uint32_t q4b_static_counters[kStaticCounterCount];

cudaError_t decode_static_scratch(float **scratch, uint32_t **counters, size_t *scratch_bytes,
                                  size_t *counter_bytes) {
    static float *scratch_of[kMaxDevices];
    static uint32_t *counters_of[kMaxDevices];
    static std::mutex guard;  // two contexts on two threads may make their first call at the same time
    const int device = device_slot();
    if (device < 0) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(guard);
    if (scratch_of[device] == nullptr) {
        float *scratch_address = nullptr;
        uint32_t *counter_address = nullptr;
        cudaError_t status = cudaGetSymbolAddress(reinterpret_cast<void **>(&scratch_address), q4b_static_scratch);
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

// variant encoding (0 = heuristics): bits 0-3 CTAs per SM (at most what fits), bit 4 the fp16 form also at
// M <= 4 (default there: the integer form), bits 8-11 an upper limit on the K parts of a pair block,
// bit 13 no thread-block clusters for a split K, bit 14 no programmatic dependent launch, bit 16 the first ring
// fill of a single launch is not held back
cudaError_t decode_geometry(uint32_t m_rows, int variant, int sm_count, bool sequence, DecodeGeometry *geometry) {
    if (m_rows == 0 || m_rows > decode_max_m()) return cudaErrorInvalidValue;
    geometry->mode = mode_of(m_rows, variant);
    geometry->smem_bytes = smem_of(geometry->mode, m_rows, &geometry->stages);
    // The K split is planned around the clusters the device can hold of the integer form at M = 1 (asked once per
    // device), so that every form, every M and a sequence split a projection alike; a launch then uses clusters
    // when its own form's fit as well.
    uint32_t stages_unused = 0;
    const size_t plan_smem = smem_of(0, 1u, &stages_unused);
    const size_t form_smem = smem_of(geometry->mode, geometry->mode == 0 ? 1u : m_rows, &stages_unused);
    for (uint32_t k = 0; k <= 8; ++k) {
        geometry->plan_room[k] = k < 2 ? 0u : resident_clusters<0>(k, plan_smem);
        geometry->cluster_room[k] = k < 2                ? 0u
                                    : geometry->mode == 0 ? geometry->plan_room[k]
                                    : geometry->mode == 1 ? resident_clusters<1>(k, form_smem)
                                                          : resident_clusters<2>(k, form_smem);
    }
    int per_sm = 0;
    cudaError_t status = configure_mode(geometry->mode, sequence, geometry->smem_bytes, &per_sm);
    if (status != cudaSuccess) return status;
    if (per_sm > 2) per_sm = 2;
    const int wanted = variant & 0xf;
    if (wanted >= 1 && wanted < per_sm) per_sm = wanted;
    geometry->ctas = (uint32_t)(per_sm * sm_count);
    // the K split is planned for two thread blocks per SM whatever is resident, so that a row's sum is grouped the
    // same way in every form of the kernel (a grid that is smaller takes the units in turns)
    geometry->plan_ctas = (uint32_t)(2 * sm_count);
    geometry->threads = kDecodeThreads;
    geometry->max_parts = (uint32_t)((variant >> 8) & 0xf);
    return cudaSuccess;
}

void plan_decode_job(DecodeJob *job, uint32_t m_rows, const DecodeGeometry &geometry, size_t *scratch_bytes,
                     size_t *counter_bytes) {
    (void)m_rows;
    const uint32_t G = job->groups;
    uint32_t pairs = 0;
    for (uint32_t s = 0; s < job->segments; ++s) {
        job->pair_begin[s] = pairs;
        pairs += job->fused ? ceil_div(job->rows[s], 64) : ceil_div(job->rows[s], 128);
    }
    for (uint32_t s = job->segments; s <= (uint32_t)kMaxSegments; ++s) job->pair_begin[s] = pairs;
    // Fewer pair blocks than CTAs: cut K into equal parts so that the whole grid streams, a part no shorter
    // than four groups.  Otherwise every CTA takes whole pair blocks in turn.
    uint32_t parts = 1;
    if (pairs < geometry.plan_ctas) {
        for (uint32_t k = 1; k <= G; ++k) {
            if (pairs * k <= geometry.plan_ctas && (G / k >= 4 || k == 1)) parts = k;
        }
    }
    if (geometry.max_parts > 0 && parts > geometry.max_parts) parts = geometry.max_parts;
    // A small matrix (a rank's slice of a projection, say) would be cut into more than eight parts: eight parts
    // that meet in a cluster's shared memory finish sooner than many that meet in global memory, as long as a
    // part stays within a few ring stages
    if (parts > 8 && geometry.plan_room[8] >= pairs && G / 8 <= 5 * kStageGroups) parts = 8;
    // 2..8 parts meet in the shared memory of a thread-block cluster when all the clusters fit on the device at
    // once: rather one part fewer than a sum through global memory
    while (parts >= 2 && parts <= 8 && geometry.plan_room[parts] < pairs) {
        uint32_t fewer = parts - 1;
        while (fewer >= 2 && geometry.plan_room[fewer] < pairs) --fewer;
        if (fewer < 2) break;  // no cluster size fits: keep the split, summed through global memory
        parts = fewer;
    }
    job->parts = parts;
    job->units = pairs * parts;
    const size_t vals = geometry.mode == 0 ? 2 : geometry.mode == 1 ? 4 : 8;
    *scratch_bytes = parts > 1 ? (size_t)job->units * 8 * 32 * vals * sizeof(float) : 0;
    *counter_bytes = parts > 1 ? (size_t)pairs * 8 * sizeof(uint32_t) : 0;
}

namespace {

template <int MODE, bool SEQ>
cudaError_t launch_kernel(const PassParams &p, uint32_t ctas, size_t smem_bytes, bool dependent_launch,
                          cudaStream_t stream) {
    auto kernel = decode_kernel<MODE, SEQ>;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(ctas);
    config.blockDim = dim3(kDecodeThreads);
    config.dynamicSmemBytes = smem_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    config.numAttrs = 0;
    if (SEQ) {
        // the CTAs wait on one another: all of them must be resident
        attribute[0].id = cudaLaunchAttributeCooperative;
        attribute[0].val.cooperative = 1;
        config.numAttrs = 1;
    } else {
        if (dependent_launch) {
            attribute[config.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attribute[config.numAttrs].val.programmaticStreamSerializationAllowed = 1;
            ++config.numAttrs;
        }
        if (p.cluster != 0) {
            attribute[config.numAttrs].id = cudaLaunchAttributeClusterDimension;
            attribute[config.numAttrs].val.clusterDim.x = p.job.parts;
            attribute[config.numAttrs].val.clusterDim.y = 1;
            attribute[config.numAttrs].val.clusterDim.z = 1;
            ++config.numAttrs;
        }
    }
    config.attrs = attribute;
    return cudaLaunchKernelEx(&config, kernel, p);
}

}  // namespace

cudaError_t launch_decode(const DecodeJob &job, uint32_t m_rows, uint32_t world, const DecodeGeometry &geometry, int variant,
                          float *scratch, uint32_t *counters, uint32_t *status, cudaStream_t stream) {
    PassParams p = {};
    p.job = job;
    p.job_count = 1;
    p.m_rows = m_rows;
    p.world = world;  // the own copy of the outputs and world - 1 peers' (job.y[segment][0 .. world - 1])
    p.stages = geometry.stages;
    p.scratch = scratch;
    p.counters = counters;
    p.status = status;
    const uint32_t ctas = job.units < geometry.ctas ? job.units : geometry.ctas;
    const bool pdl = ((variant >> 14) & 1) == 0;
    p.throttle = ((variant >> 16) & 1) == 0 ? 1u : 0u;
    // K split over 2..8 CTAs, every unit with a CTA of its own, and all the clusters resident at once: the parts of
    // a pair block meet in shared memory
    if (((variant >> 13) & 1) == 0 && job.parts >= 2 && job.parts <= 8 && ctas == job.units &&
        geometry.cluster_room[job.parts] * job.parts >= job.units) {
        p.cluster = 1;
    }
    switch (geometry.mode) {
        case 0: return launch_kernel<0, false>(p, ctas, geometry.smem_bytes, pdl, stream);
        case 1: return launch_kernel<1, false>(p, ctas, geometry.smem_bytes, pdl, stream);
        default: return launch_kernel<2, false>(p, ctas, geometry.smem_bytes, pdl, stream);
    }
}

cudaError_t launch_sequence(const SequenceLaunch &launch, cudaStream_t stream) {
    PassParams p = {};
    p.jobs = launch.jobs;
    p.job_count = launch.job_count;
    p.m_rows = launch.m_rows;
    p.world = launch.world;
    p.stages = launch.geometry.stages;
    p.epoch = launch.epoch;
    p.exit_count = launch.exit_count;
    p.done = launch.done;
    for (int r = 0; r < kMaxPeers; ++r) p.peer_done[r] = launch.peer_done[r];
    p.scratch = launch.scratch;
    p.counters = launch.counters;
    p.status = launch.status;
    p.profile = launch.profile;
    switch (launch.geometry.mode) {
        case 0: return launch_kernel<0, true>(p, launch.geometry.ctas, launch.geometry.smem_bytes, false, stream);
        case 1: return launch_kernel<1, true>(p, launch.geometry.ctas, launch.geometry.smem_bytes, false, stream);
        default: return launch_kernel<2, true>(p, launch.geometry.ctas, launch.geometry.smem_bytes, false, stream);
    }
}

}  // namespace q4b
