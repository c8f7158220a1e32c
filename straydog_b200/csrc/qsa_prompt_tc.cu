// Causal prompt attention over Q8_0 K/V on the 5th-generation tensor cores (tcgen05.mma, accumulators
// and the A operands in TMEM): the Blackwell-native form of sdx_qsa_prompt.
//
// K and V enter the tensor cores as two FP16 planes: hi = FP16(int8 * scale), the rounding of the reference's own tensor-core kernel
// (gpu/kernels.cpp:46-54), and lo = int8 * scale - hi, the part that rounding drops (an int8 times an FP16 scale has at most 18
// significant bits, so hi + lo is the value itself and one FP16 fused multiply-add gives lo exactly). Every product is issued
// twice, once per plane, into the same FP32 accumulator: K and V enter exactly, as they enter the reference's FP32 kernels
// (gpu/sparse_attention_compute.hpp:177-415), and only the softmax weights are rounded to FP16. The planes are made inside the
// kernel from the raw Q8_0 rows: a CTA streams 272 bytes a row from L2, not the 1024 bytes of two FP16 planes (with the planes
// prepared in memory by a kernel of their own, this kernel was bound by the L2's bandwidth at about 7 TB/s over all SMs).
//
// A CTA owns 128 M-rows: 128 / group consecutive query tokens x the `group` (<= 16) query heads of one K/V head (a group that does not
// divide 128 leaves the last rows idle: the reference's own 12 heads a K/V head use 120 of them).
// It walks the causal key range in tiles of 64 keys:
//   S[128 x 64]  = Q[128 x 256] . (K_hi + K_lo)^T   2 x 16 tcgen05.mma (M 128, N 64, K 16), FP16 in, FP32 in TMEM
//   O[128 x 256] += P[128 x 64] . (V_hi + V_lo)     2 x 4 tcgen05.mma (M 128, N 256, K 16)
// TMEM (all 512 columns): O in 0..255; two S buffers in 256..319 and 320..383; Q (FP16, two values a column) in
// 384..511. P is written over the first 32 columns of the S buffer it was made from, so both products take their A
// operand from TMEM and shared memory only holds K and V tiles: one ring of five 32 KB slots that the dequantising warps fill
// and the MMA thread drains in the same fixed order (K_hi, K_lo of tile i, then V_hi, V_lo of tile i - 1).
//
// Warp roles (19 warps):
//   warps 0-7   softmax: two threads per M-row (32 of the tile's 64 columns each; warp w works on the TMEM lanes
//               32 (w % 4).. a warp may touch). tcgen05.ld of the scores, mask, row maximum exchanged with the partner
//               warp through shared memory, P rounded to FP16 and stored to TMEM; O is rescaled in TMEM only when a
//               row's maximum has grown by more than 2^8 (the stale maximum stays exact arithmetic: weights are at
//               most 256 and the final division uses the same maximum); epilogue O / l.
//   warp 8      one thread issues the score products' tcgen05.mma and commits them to mbarriers.
//   warp 9      one thread issues the value products' (a thread each: the tensor pipe's queue is short, and one issuer's waits
//               for tiles, weights and buffers let it run dry; with two, one's waits pass while the other issues).
//   warp 10     one thread brings the raw rows: a bulk copy (TMA engine) of a tile's 64 consecutive rows of one plane
//               (17408 contiguous bytes) into a ring of three raw slots.
//   warps 11-18 dequantise a raw slot into an FP16 hi tile and an FP16 lo tile, written in the 128-byte-swizzled
//               [64 rows][128 bytes] blocks that are the K-major / MN-major operand layout the MMA's descriptors read.
// S is double buffered, so the tensor pipe works on S(i+1) while the softmax warps work on S(i). Every wait is bounded; a wait
// that gives up raises a flag that ends all roles, frees TMEM and reports through the status word.
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

#include <algorithm>

namespace sdb {
namespace tc {

constexpr int kM = 128, kN = 64, kD = 256;
constexpr int kSoftmaxWarps = 8, kScoreWarp = 8, kValueWarp = 9, kTmaWarp = 10, kDequantWarp0 = 11, kDequantWarps = 8;
constexpr int kThreads = 32 * (kDequantWarp0 + kDequantWarps);   // 8 softmax warps, two MMA warps, the copy warp, 8 dequantising warps
constexpr int kKVBytes = kN * kD * 2;               // one operand tile: 64 positions x 256 FP16
constexpr int kSlots = 5;                            // the operand ring (FP16 tiles)
constexpr int kRawSlots = 3, kRawBytes = kN * int(kv_row_q8);   // raw Q8_0 tiles: 64 rows of one plane, 17408 contiguous bytes
constexpr int kOffRing = 0, kOffRaw = kOffRing + kSlots * kKVBytes, kOffBars = kOffRaw + kRawSlots * kRawBytes + 256;
constexpr int kOffStats = kOffBars + 256;            // [2 halves][128 rows] floats exchanged between the two warps of a row block
constexpr size_t kSmem = kOffStats + 2 * kM * 4 + 1024;   // + slack to align the base to 1024 bytes
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;

struct Args {
    const uint8_t* state;   // 2 * kv_heads planes of `context` Q8_0 rows
    size_t context, first, rows, heads, kv_heads, group;
    const __half* q;
    float* out;
    float scale_log2;
    int* status;
    long long* trace;   // -DSDX_TRACE only
};

enum Bar { kFull = 0, kFree = kSlots, kSFull = 2 * kSlots, kSFree = kSFull + 2, kPFull = kSFree + 2, kPvDone = kPFull + 2,
           kRawFull = kPvDone + 1, kRawFree = kRawFull + kRawSlots, kBars = kRawFree + kRawSlots };

// A shared-memory operand descriptor: start address, leading and stride byte offsets in 16-byte units; descriptor version 1;
// 128-byte swizzle. Its high word (stride 1024 bytes between 8-row groups, version, swizzle) never changes here and its low word is
// (address >> 4) | (leading offset >> 4) << 16, so the descriptor a few bytes further on is one 32-bit add away: the issuing thread
// does nothing else, and a descriptor built from scratch costs it a dozen dependent instructions per MMA.
constexpr uint32_t kDescHigh = 0x40004040u;
__device__ __forceinline__ uint32_t desc_low(uint32_t address, uint32_t leading_bytes) { return ((address & 0x3ffffu) >> 4) | ((leading_bytes >> 4) << 16); }
__device__ __forceinline__ uint64_t desc_of(uint32_t low) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(low), "r"(kDescHigh));
    return d;
}
// Built with -DSDX_TRACE the MMA thread adds up the cycles it spends in each of its waits (eight 64-bit counters a CTA: total, wait
// for a tile, for the weights, for a free score buffer, the value thread's wait for a tile, tiles, the value thread's total, softmax thread 0's wait for the scores): the figures the profile summary of this kernel quotes.
#if defined(SDX_TRACE)
#define SDX_TRACE_ADD(slot, since) trace[slot] += clock64() - (since)
#else
#define SDX_TRACE_ADD(slot, since) ((void)0)
#endif
// kind::f16 instruction descriptor: FP32 accumulator, FP16 A and B, A K-major, B K-major or MN-major, shape M x N
__device__ __forceinline__ uint32_t instr_desc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
}
// the same with the A operand in TMEM (lane = row; a 32-bit column holds two consecutive K elements)
__device__ __forceinline__ void umma_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    #pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "f"(v[8]), "f"(v[9]),
                   "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]), "f"(v[15]), "f"(v[16]), "f"(v[17]), "f"(v[18]), "f"(v[19]),
                   "f"(v[20]), "f"(v[21]), "f"(v[22]), "f"(v[23]), "f"(v[24]), "f"(v[25]), "f"(v[26]), "f"(v[27]), "f"(v[28]), "f"(v[29]),
                   "f"(v[30]), "f"(v[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_st32_bits(uint32_t taddr, const uint32_t (&v)[32]) {
    float f[32];
    #pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
    tmem_st32(taddr, f);
}
__device__ __forceinline__ void tmem_st16_bits(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
                   "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void pair_barrier(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

__global__ void __launch_bounds__(kThreads, 1) qsa_prompt_tc_kernel(const Args a) {
    constexpr int kBlockThreads = kThreads;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* stats = reinterpret_cast<float*>(smem + kOffStats);

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const size_t tokens_per_block = kM / a.group;
    const size_t blocks = (a.rows + tokens_per_block - 1) / tokens_per_block;
    const size_t block = blocks - 1 - blockIdx.x, kv = blockIdx.y;   // longest blocks first
    const size_t r0 = block * tokens_per_block;

    if (tid == 0) {
        // (a barrier is completed by one arrival - a copy's byte count or an MMA commit - except p_full, one arrival per softmax warp, and
        //  the barriers the dequantising warps arrive on, one arrival per such warp)
        for (int i = 0; i < kBars; ++i) {
            const bool by_dequant = (i >= kFull && i < kFull + kSlots) || (i >= kRawFree && i < kRawFree + kRawSlots);
            mbar_init(&bars[i], i == kPFull || i == kPFull + 1 ? kSoftmaxWarps : by_dequant ? kDequantWarps : 1);
        }
        *abort_flag = 0;
    }
    fence_barrier_init();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // Q -> TMEM columns 384..511 as the A operand of the score products (lane = M-row, a 32-bit column = two consecutive
    // columns of Q): the tensor core then reads only K from shared memory. A softmax thread stores its half row.
    if (warp < kSoftmaxWarps) {
        const int rb = warp & 3, half = warp >> 2, m = rb * 32 + lane;
        // (a group that does not divide 128, the reference's own 12 among them, leaves the block's last M-rows without a token: zeros)
        const size_t row = size_t(m) < tokens_per_block * a.group ? r0 + m / a.group : a.rows, head = kv * a.group + m % a.group;
        const uint4* source = reinterpret_cast<const uint4*>(a.q + (row * a.heads + head) * kD + half * 128);
        #pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint32_t words[32];
            #pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 v = row < a.rows ? __ldg(source + c * 8 + i) : make_uint4(0, 0, 0, 0);
                words[4 * i] = v.x; words[4 * i + 1] = v.y; words[4 * i + 2] = v.z; words[4 * i + 3] = v.w;
            }
            tmem_st32_bits(tmem + (uint32_t(rb * 32) << 16) + 384 + half * 64 + c * 32, words);
        }
        tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    const size_t last_row = min(a.rows, r0 + tokens_per_block) - 1;
    const size_t keys_total = a.first + last_row + 1;
    const uint32_t tiles = uint32_t((keys_total + kN - 1) / kN);

    // a bounded wait that also ends when another role has given up
    auto wait = [&](int bar, uint32_t parity) -> bool {
        if (mbar_try_wait(&bars[bar], parity)) return true;
        const uint64_t start = global_timer_ns();
        for (;;) {
            #pragma unroll 1
            for (int spin = 0; spin < 32; ++spin)
                if (mbar_try_wait(&bars[bar], parity)) return true;
            if (*abort_flag) return false;
            if (global_timer_ns() - start > 2000000000ull) { *abort_flag = 1; atomicExch(a.status, 1); return false; }
        }
    };

    if (warp < kSoftmaxWarps) {
        // ================= softmax, correction, epilogue: two threads per M-row, 32 of the tile's 64 columns each =================
        // Warp w works on TMEM lanes 32 (w % 4) .. (the lanes a warp may touch) and columns 32 (w / 4) .. ; the two warps of a row
        // block exchange their row maxima through shared memory, so both take the same decisions and keep their own partial sums.
        const int rb = warp & 3, half = warp >> 2, m = rb * 32 + lane;
        const size_t token = r0 + m / a.group, head = kv * a.group + m % a.group;
        const bool valid = token < a.rows && size_t(m) < tokens_per_block * a.group;
        const long long limit = valid ? (long long)(a.first + token) : -1;
        const uint32_t lane_base = uint32_t(rb * 32) << 16;
        float* mine_stat = stats + half * kM + m;
        const float* other_stat = stats + (half ^ 1) * kM + m;
        float m_run = -INFINITY, l_run = 0.0f;
        bool alive = true;
        for (uint32_t j = 0; j < tiles && alive; ++j) {
            const uint32_t slot = j & 1;
#if defined(SDX_TRACE)
            const long long since = clock64();
#endif
            if (!wait(kSFull + slot, (j >> 1) & 1)) { alive = false; break; }
#if defined(SDX_TRACE)
            if (tid == 0) a.trace[(size_t(blockIdx.y) * gridDim.x + blockIdx.x) * 8 + 7] += clock64() - since;
#endif
            tc_fence_after();
            float s[32];
            tmem_ld32(tmem + lane_base + 256 + slot * 64 + half * 32, s);
            const long long begin = (long long)j * kN + half * 32;
            const bool edge = (long long)j * kN + kN - 1 > (long long)(a.first + r0) || (long long)j * kN + kN > (long long)keys_total;
            // (four independent maxima, then their maximum: one chain of 32 dependent fmnmx cost a third of the tile's softmax time)
            // the scores stay unscaled: the scale (positive) is applied to the maximum once and folded into each exponent's argument
            float tops[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (edge) {
                #pragma unroll
                for (int n = 0; n < 32; ++n)
                    if (begin + n > limit) s[n] = -INFINITY;
            }
            #pragma unroll
            for (int n = 0; n < 32; ++n) tops[n & 3] = fmaxf(tops[n & 3], s[n]);
            const float top = fmaxf(fmaxf(tops[0], tops[1]), fmaxf(tops[2], tops[3])) * a.scale_log2;
            *mine_stat = top;
            pair_barrier(1 + rb);
            const float m_new = fmaxf(m_run, fmaxf(top, *other_stat));
            pair_barrier(1 + rb);   // (the partner has read this tile's maximum before the next one is written)
            // keep the old maximum while the new one is within 2^8 of it: no pass over O in TMEM
            const bool grow = m_new > m_run + kRescaleThreshold || m_run == -INFINITY;
            const float m_use = grow ? m_new : m_run;
            if (j >= 1 && __any_sync(0xffffffffu, grow && m_run != -INFINITY)) {
                // a maximum of this warp's rows has grown past the threshold: O (this half's 128 columns) is rescaled in TMEM once every
                // product issued so far has landed
                if (!wait(kPvDone, (j - 1) & 1)) { alive = false; break; }
                tc_fence_after();
                const float factor = grow && m_run != -INFINITY ? fast_exp2(m_run - m_use) : 1.0f;
                #pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    float o[32];
                    tmem_ld32(tmem + lane_base + half * 128 + c * 32, o);
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= factor;
                    tmem_st32(tmem + lane_base + half * 128 + c * 32, o);
                }
                tmem_st_wait();
                l_run *= factor;
            }
            if (grow && m_run == -INFINITY) l_run = 0.0f;
            m_run = m_use;
            const float u = m_run == -INFINITY ? 0.0f : m_run;
            // This half of the P row, 32 FP16 as 16 TMEM columns, over the first columns of the S buffer it came from (every thread of the
            // row block has its scores in registers by now: both halves passed the barriers above). The product reads P from TMEM.
            uint32_t packed[16];
            float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            #pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float p0 = fast_exp2(fmaf(s[2 * i], a.scale_log2, -u)), p1 = fast_exp2(fmaf(s[2 * i + 1], a.scale_log2, -u));
                packed[i] = pack_half2(p0, p1);
                // the denominator adds the weights as the product sees them, rounded to FP16: the output stays a convex combination of the
                // values, and a rounding of a weight moves it by (value - output), not by the value (the worst errors, rows that one or two
                // keys of large values dominate, shrink two to three times)
                const float2 seen = __half22float2(*reinterpret_cast<const __half2*>(&packed[i]));
                sums[i & 3] += seen.x + seen.y;
            }
            l_run += (sums[0] + sums[1]) + (sums[2] + sums[3]);
            tmem_st16_bits(tmem + lane_base + 256 + slot * 64 + half * 16, packed);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kPFull + slot]);
        }
        // epilogue: O / l, this half's 128 columns; the row's denominator is the two halves' sums
        *mine_stat = l_run;
        pair_barrier(1 + rb);
        const float denominator = l_run + *other_stat;
        if (alive && tiles >= 2 && !wait(kSFree + ((tiles - 2) & 1), ((tiles - 2) >> 1) & 1)) alive = false;   // (all but the last product done)
        if (alive && tiles > 0 && wait(kPvDone, (tiles - 1) & 1)) {
            tc_fence_after();
            const float inverse = 1.0f / denominator;
            float* mine = a.out + (token * a.heads + head) * kD + half * 128;
            #pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float o[32];
                tmem_ld32(tmem + lane_base + half * 128 + c * 32, o);
                if (valid) {
                    #pragma unroll
                    for (int i = 0; i < 32; i += 2) *reinterpret_cast<float2*>(mine + c * 32 + i) = make_float2(o[i] * inverse, o[i + 1] * inverse);
                }
            }
        }
    } else if (warp == kScoreWarp) {
        // ================= the score products' issuer =================
        // The ring is drained in the order the dequantising warps fill it: plane tile t sits in slot t % 5, in its (t / 5)-th use. The
        // planes of K(i) are tiles 4 i - 2 and 4 i - 1 (0 and 1 for the first tile), those of V(j) 4 j + 4 and 4 j + 5 (4 j + 2 and
        // 4 j + 3 for the last tile, which no K follows). Scores and values have a thread each, so that one's waits pass while the
        // other issues: the tensor pipe's queue is short, and a single issuer let it run dry at every wait.
        if (lane == 0) {
            long long trace[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long started = clock64();
            (void)started;
            const uint32_t ring = smem_u32(smem + kOffRing);
            const uint32_t idesc_s = instr_desc(kM, kN, false);
            bool alive = true;
            for (uint32_t i = 0; i < tiles && alive; ++i) {
                const uint32_t buffer = i & 1, s_tmem = tmem + 256 + buffer * 64;
                long long since = clock64();
                if (i >= 2 && !wait(kSFree + buffer, ((i - 2) >> 1) & 1)) break;
                SDX_TRACE_ADD(3, since);
                uint32_t item = i == 0 ? 0u : 4 * i - 2;
                #pragma unroll 1
                for (int part = 0; part < 2 && alive; ++part, ++item) {   // K_hi, then K_lo into the same accumulator
                    const uint32_t slot = item % kSlots, tile = desc_low(ring + slot * kKVBytes, 16);
                    since = clock64();
                    if (!wait(kFull + slot, (item / kSlots) & 1)) { alive = false; break; }
                    SDX_TRACE_ADD(1, since);
                    #pragma unroll
                    for (int kk = 0; kk < 16; ++kk)
                        umma_a_tmem(s_tmem, tmem + 384 + kk * 8, desc_of(tile + (((kk / 4) * (kN * 128) + (kk % 4) * 32) >> 4)), idesc_s, part > 0 || kk > 0);
                    umma_commit(&bars[kFree + slot]);
                }
                if (!alive) break;
                umma_commit(&bars[kSFull + buffer]);
            }
#if defined(SDX_TRACE)
            trace[0] = clock64() - started; trace[5] = tiles;
            long long* mine = a.trace + (size_t(blockIdx.y) * gridDim.x + blockIdx.x) * 8;
            mine[0] = trace[0]; mine[1] = trace[1]; mine[3] = trace[3]; mine[5] = trace[5];
#endif
        }
    } else if (warp == kValueWarp) {
        // ================= the value products' issuer =================
        if (lane == 0) {
            long long trace[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long started = clock64();
            (void)started;
            const uint32_t ring = smem_u32(smem + kOffRing);
            const uint32_t idesc_o = instr_desc(kM, kD, true);
            bool alive = true;
            for (uint32_t j = 0; j < tiles && alive; ++j) {
                const uint32_t buffer = j & 1, p_tmem = tmem + 256 + buffer * 64;
                long long since = clock64();
                if (!wait(kPFull + buffer, (j >> 1) & 1)) break;
                SDX_TRACE_ADD(2, since);
                tc_fence_after();
                uint32_t item = j + 1 == tiles ? 4 * j + 2 : 4 * j + 4;
                #pragma unroll 1
                for (int part = 0; part < 2 && alive; ++part, ++item) {   // V_hi, then V_lo
                    const uint32_t slot = item % kSlots, tile = desc_low(ring + slot * kKVBytes, kN * 128);
                    since = clock64();
                    if (!wait(kFull + slot, (item / kSlots) & 1)) { alive = false; break; }
                    SDX_TRACE_ADD(4, since);
                    #pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_a_tmem(tmem, p_tmem + kk * 8, desc_of(tile + ((kk * (16 * 128)) >> 4)), idesc_o, j > 0 || part > 0 || kk > 0);
                    umma_commit(&bars[kFree + slot]);
                }
                if (!alive) break;
                umma_commit(&bars[kPvDone]);
                umma_commit(&bars[kSFree + buffer]);   // P sat in the S buffer: free once the product has read it
            }
#if defined(SDX_TRACE)
            trace[6] = clock64() - started;
            long long* mine = a.trace + (size_t(blockIdx.y) * gridDim.x + blockIdx.x) * 8;
            mine[2] = trace[2]; mine[4] = trace[4]; mine[6] = trace[6];
#endif
        }
    } else if (warp == kTmaWarp) {
        // ================= the copy thread: raw Q8_0 rows by bulk copies =================
        // Raw item r is the K rows of tile i or the V rows of tile i - 1, in the order the MMA thread wants them: K(0), K(1), V(0), K(2), ...
        if (lane == 0) {
            uint32_t item = 0;
            bool ok = true;
            for (uint32_t i = 0; i <= tiles && ok; ++i) {
                #pragma unroll 1
                for (int which = 0; which < 2 && ok; ++which) {
                    const bool value = which == 1;
                    if (value ? i == 0 : i == tiles) continue;
                    const uint32_t tile_index = value ? i - 1 : i, slot = item % kRawSlots;
                    const size_t plane = value ? a.kv_heads + kv : kv, begin = size_t(tile_index) * kN;
                    const uint32_t rows = uint32_t(min(size_t(kN), keys_total - begin));
                    if (item >= uint32_t(kRawSlots) && !wait(kRawFree + slot, (item / kRawSlots - 1) & 1)) { ok = false; break; }
                    mbar_expect_tx(&bars[kRawFull + slot], rows * kv_row_q8);
                    bulk_g2s(smem + kOffRaw + slot * kRawBytes, a.state + (plane * a.context + begin) * kv_row_q8, rows * kv_row_q8, &bars[kRawFull + slot]);
                    ++item;
                }
            }
        }
    } else {
        // ================= the dequantising warps: a raw slot -> an FP16 hi tile and an FP16 lo tile =================
        // Thread t takes a quarter of a row (row t % 64, columns 64 (t / 64) ..: one 128-byte segment of the operand tile): four 16-byte
        // pieces of raw values, two block scales. A warp's 32 rows are 272 bytes apart in the raw slot and 128 bytes apart, swizzled, in
        // the tile: neither its loads nor its stores meet in a bank.
        const int dt = tid - 32 * kDequantWarp0, row = dt % kN, quarter = dt / kN;
        const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));   // 1152 = 1024 + 128
        const uint32_t total_items = 2 * tiles;
        for (uint32_t item = 0; item < total_items; ++item) {
            const uint32_t raw_slot = item % kRawSlots, hi_slot = (2 * item) % kSlots, lo_slot = (2 * item + 1) % kSlots;
            // which tile the item is (K(0), K(1), V(0), K(2), V(1), ..., V(tiles - 1)) and how many of its 64 rows exist
            const uint32_t tile_index = item == 0 ? 0u : item + 1 == total_items ? tiles - 1 : (item & 1 ? (item + 1) / 2 : item / 2 - 1);
            const uint32_t rows = uint32_t(min(size_t(kN), keys_total - size_t(tile_index) * kN));
            if (!wait(kRawFull + raw_slot, (item / kRawSlots) & 1)) break;
            if (2 * item >= uint32_t(kSlots) && !wait(kFree + hi_slot, ((2 * item) / kSlots - 1) & 1)) break;
            if (2 * item + 1 >= uint32_t(kSlots) && !wait(kFree + lo_slot, ((2 * item + 1) / kSlots - 1) & 1)) break;
            const uint8_t* raw = smem + kOffRaw + raw_slot * kRawBytes + row * kv_row_q8;
            uint8_t* hi_row = smem + kOffRing + hi_slot * kKVBytes + quarter * (kN * 128) + row * 128;
            uint8_t* lo_row = smem + kOffRing + lo_slot * kKVBytes + quarter * (kN * 128) + row * 128;
            const bool exists = uint32_t(row) < rows;   // (rows past the chunk's last position: zeros, never stale bytes)
            const uint32_t scales = exists ? *reinterpret_cast<const uint32_t*>(raw + 256 + quarter * 4) : 0u;
            #pragma unroll
            for (int piece = 0; piece < 4; ++piece) {
                uint4 bytes = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
                if (exists) bytes = *reinterpret_cast<const uint4*>(raw + quarter * 64 + piece * 16);
                const __half scale_h = __ushort_as_half(uint16_t(piece / 2 ? scales >> 16 : scales & 0xffffu));
                const __half2 scale2 = __halves2half2(scale_h, scale_h);
                const uint32_t words[4] = {bytes.x ^ 0x80808080u, bytes.y ^ 0x80808080u, bytes.z ^ 0x80808080u, bytes.w ^ 0x80808080u};
                uint32_t hi[8], lo[8];
                #pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t pair0 = prmt(words[w], 0x64646464u, 0x4140u), pair1 = prmt(words[w], 0x64646464u, 0x4342u);
                    const __half2 v0 = __hsub2(*reinterpret_cast<const __half2*>(&pair0), bias), v1 = __hsub2(*reinterpret_cast<const __half2*>(&pair1), bias);
                    const __half2 h0 = __hmul2(v0, scale2), h1 = __hmul2(v1, scale2);
                    const __half2 l0 = __hfma2(v0, scale2, __hneg2(h0)), l1 = __hfma2(v1, scale2, __hneg2(h1));   // exact: the product has 18 bits at most
                    hi[2 * w] = *reinterpret_cast<const uint32_t*>(&h0); hi[2 * w + 1] = *reinterpret_cast<const uint32_t*>(&h1);
                    lo[2 * w] = *reinterpret_cast<const uint32_t*>(&l0); lo[2 * w + 1] = *reinterpret_cast<const uint32_t*>(&l1);
                }
                // 16 values = two 16-byte pieces of the row's 128-byte segment, swizzled by the row
                const uint32_t at0 = ((2 * piece) ^ (row % 8)) * 16, at1 = ((2 * piece + 1) ^ (row % 8)) * 16;
                *reinterpret_cast<uint4*>(hi_row + at0) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(hi_row + at1) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                *reinterpret_cast<uint4*>(lo_row + at0) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint4*>(lo_row + at1) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
            }
            fence_proxy_async();   // (the tensor core reads the tiles through the async proxy)
            __syncwarp();
            if (lane == 0) { mbar_arrive(&bars[kFull + hi_slot]); mbar_arrive(&bars[kFull + lo_slot]); mbar_arrive(&bars[kRawFree + raw_slot]); }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

}  // namespace tc

static void launch_prompt_tc(Device& d, const uint8_t* state, size_t context, size_t first, size_t rows, size_t heads, size_t kv_heads,
                             float scale, const void* q, float* out) {
    tc::Args args{};
    args.state = state; args.context = context;
    args.first = first; args.rows = rows; args.heads = heads; args.kv_heads = kv_heads; args.group = heads / kv_heads;
    args.q = static_cast<const __half*>(q);
    args.out = out;
    args.scale_log2 = scale * 1.4426950408889634f;
    args.status = status_word(d);
    const size_t tokens_per_block = tc::kM / args.group;
    const dim3 grid{unsigned((rows + tokens_per_block - 1) / tokens_per_block), unsigned(kv_heads)};
    static bool configured[64] = {};
    if (!configured[d.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(tc::qsa_prompt_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(tc::kSmem)));
        configured[d.ordinal & 63] = true;
    }
#if defined(SDX_TRACE)
    {
        const size_t ctas = size_t(grid.x) * grid.y;
        args.trace = static_cast<long long*>(ensure(d, d.work, d.work_bytes, ctas * 64));
        SDB_CHECK(cudaMemsetAsync(args.trace, 0, ctas * 64, d.stream));
        d.trace = args.trace; d.trace_ctas = ctas;
    }
#endif
    tc::qsa_prompt_tc_kernel<<<grid, tc::kThreads, tc::kSmem, d.stream>>>(args);
    ++d.launches;
}

}  // namespace sdb

using namespace sdb;

// Causal prompt attention over a Q8_0 K/V state: a chunk of `rows` new tokens at positions first .. first + rows - 1 attends every
// cached position up to its own. What it replaces in the reference: qsa_flash / qsa_flash_wide (FP32,
// gpu/sparse_attention_compute.hpp:177-415) and qsa_flash_mma (mma.sync per token, :416-584) behind qsa_flash_launch (:589-608), in
// their dense causal form. The reference walks one token per block, so sixteen neighbouring tokens that share almost all their
// keys each read and dequantise them again; here a CTA takes 128 / group consecutive tokens for all the query heads of one K/V head.
extern "C" int sdx_qsa_prompt(void* handle, const void* state, uint64_t context, uint64_t first, uint64_t rows, uint64_t heads,
                              uint64_t kv_heads, float scale, const void* q, float* out) {
    SDB_OP_BEGIN
    if (value.kv_row != kv_row_q8) throw std::runtime_error("this Straydog build's attention reads Q8_0 K/V rows only");
    const uint64_t group = kv_heads ? heads / kv_heads : 0;
    if (!context || context > (uint64_t(1) << 24) || !rows || first > context || rows > context - first || !heads || !kv_heads ||
        heads % kv_heads || group > 16 || kv_heads > 65535 || !(scale > 0.0f) || !(scale < 1e30f))
        throw std::runtime_error("invalid Straydog attention dimensions");
    span(value, state, checked_product({context, 2 * kv_heads, kv_row_q8}), "a K/V state");
    span(value, q, checked_product({rows, heads, 256, 2}), "attention queries");
    span(value, out, checked_product({rows, heads, 256, 4}), "an attention output");
    if (reinterpret_cast<uintptr_t>(state) % 16 || reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(out) % 8)
        throw std::runtime_error("Straydog prompt attention operands must be 16-byte aligned");
    launch_prompt_tc(value, static_cast<const uint8_t*>(state), context, first, rows, heads, kv_heads, scale, q, out);
    SDB_OP_END
}
