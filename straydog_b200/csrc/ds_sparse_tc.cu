// Latent sparse attention on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM): the kernel sd_op_sparse_attention
// prefers for BF16-tagged compressed rows and head counts that are multiples of 16.
//
// What it replaces: op_attention_scores_kernel + op_attention_output_kernel (gpu/ops.hpp:1329-1434, 1542-1661) and, as a design,
// the reference's all-heads-of-a-row-per-block WMMA form (gpu/ds_attention_wmma.hpp:25-326: every key row read once for all the
// heads of a query row, weights formed once per row).
//
// A CTA owns one query row, up to 64 of its heads and a split of its selected rows, walked in tiles of 32 keys:
//   S[64 x 32]      = Q[64 heads x dim] . K_tile^T          M 64, N 32, K 16 per instruction; Q (BF16) and the tile in shared memory
//   O^T[dim x heads] += V_tile^T[dim x 32] . P^T[32 x heads]  M 128 (two 64-column blocks of the tile), N = heads, K 16
// The output is held TRANSPOSED in TMEM (a lane = an output column, a column = a head): 5 x 64 columns for dim 576 and 64 heads,
// where O itself (heads x 576 FP32) would not fit the 512 columns. The keys are the values (gpu/ops.hpp:1309-1316), so one tile in
// shared memory serves both products: as the K-major B operand of the scores and as the MN-major A operand of the output.
//
// A tile is gathered by four copy warps: 16-byte cp.async copies, a warp instruction covering 512 consecutive bytes of one row, each
// piece written where the 128-byte swizzle of the tensor core's shared-memory descriptors expects it (a bulk copy of a whole row
// cannot swizzle); absent rows (-1) are zero-filled by the copy itself. Three tiles are in flight per CTA.
//
// Warps: 0-3 softmax (a thread per head row of S: mask, running maximum with a lazy rescale, weights to shared memory as BF16) and
// epilogue (a thread per output column); 4 issues every MMA; 5-8 copy. The CTA leaves a partial (sums, maximum, denominator) per
// head for its split; the window rows' partial comes from the FP32 kernel and sparse_combine_kernel merges them with the sink and
// turns the rotated columns back (gpu/ops.hpp:1561-1583, 1528-1538). Every wait is bounded and reports through the status word.
#include "ds_sparse.cuh"

#include <algorithm>

namespace sdb {
namespace tcl {

constexpr int kKeys = 32, kSlots = 3, kRows = 64;          // keys a tile, tiles in the ring, head rows of S (M of the score product)
constexpr int kSoftmaxWarps = 4, kMmaWarp = 4, kCopyWarp0 = 5, kCopyWarps = 4, kThreads = 32 * (kCopyWarp0 + kCopyWarps);
constexpr float kRescaleThreshold = 8.0f;

template<int DIM> struct Shape {
    static constexpr int kBlocks = DIM / 64;                // 64-column blocks of a row
    static constexpr int kTile = kBlocks * kKeys * 128;     // a tile: [block][32 keys][128 bytes], swizzled
    static constexpr int kMTiles = (DIM + 127) / 128;       // output M-tiles of 128 columns (the last half empty for dim 576)
    static constexpr int kOffRing = 0;
    static constexpr int kOffQ = kSlots * kTile + 4096;     // (+ one block of slack: the last M-tile of dim 576 names a block past the tile)
    static constexpr int kOffQlo = kOffQ + kBlocks * kRows * 128;
    static constexpr int kOffP = kOffQlo + 2 * kRows * 128; // low parts of the rotated columns: at most two blocks (rope_dims <= 128)
    static constexpr int kOffBars = kOffP + 2 * kRows * 128;
    static constexpr int kOffMisc = kOffBars + 128;
    static constexpr size_t kSmem = kOffMisc + 1024 + 1024; // misc (masks, factors, flags) + slack to align the base to 1024 bytes
    static_assert(kSmem <= 232448, "shared memory of one CTA");
};

enum Bar { kFull = 0, kFree = kSlots, kSFull = 2 * kSlots, kSFree = kSFull + 2, kPFull = kSFree + 2, kPFree = kPFull + 2, kDone = kPFree + 2, kBars = kDone + 1 };

// Built with -DSDX_TRACE the kernel adds up, per CTA, the cycles its MMA thread and its first copy thread spend in each wait, and
// leaves them behind the partials (eight 64-bit counters a CTA: total, wait for a tile, for the weights, for a free score buffer,
// copy thread's wait for a free slot, tiles): the figures the profile summary of this kernel quotes.
#if defined(SDX_TRACE)
#define SDX_TRACE_ADD(slot, since) trace[slot] += clock64() - (since)
#else
#define SDX_TRACE_ADD(slot, since) ((void)0)
#endif

struct Args {
    SparseArgs a;
    const float* q;
    size_t pairs;
    const double2* forward;
    float scale_log2;
    int* status;
    float* partial;          // [(row * heads + head) * parts + 1 + split][dim + 2]
    uint32_t parts, splits;
    long long* trace;        // -DSDX_TRACE only
};

__device__ __forceinline__ uint64_t smem_desc(uint32_t address, uint32_t leading_bytes, uint32_t stride_bytes) {
    return uint64_t((address & 0x3ffffu) >> 4) | (uint64_t(leading_bytes >> 4) << 16) | (uint64_t(stride_bytes >> 4) << 32) |
           (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// The same descriptor from its two words: the high word (stride 1024 bytes between 8-row groups, version 1, 128-byte swizzle) never
// changes, and the low word is (address >> 4) | (leading offset >> 4) << 16, so a descriptor a few bytes further on is one 32-bit add
// away (the issuing thread does nothing else, and a descriptor built from scratch costs it a dozen dependent instructions).
constexpr uint32_t kDescHigh = 0x40004040u;
__device__ __forceinline__ uint32_t desc_low(uint32_t address, uint32_t leading_bytes) { return ((address & 0x3ffffu) >> 4) | ((leading_bytes >> 4) << 16); }
__device__ __forceinline__ uint64_t desc_of(uint32_t low) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(low), "r"(kDescHigh));
    return d;
}
// kind::f16 instruction descriptor: FP32 accumulator, BF16 A and B, each K-major or MN-major, shape M x N
__device__ __forceinline__ uint32_t instr_desc(int m, int n, bool a_mn, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(a_mn) << 15) | (uint32_t(b_mn) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    #pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "f"(v[8]), "f"(v[9]),
                   "f"(v[10]), "f"(v[11]), "f"(v[12]), "f"(v[13]), "f"(v[14]), "f"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Byte offset of element (row, column) in a K-major operand of [rows][columns] BF16 laid out as 64-column blocks of
// [rows][128 bytes] with the 128-byte swizzle (16-byte pieces of a row exchanged by the row's low three bits).
__device__ __forceinline__ uint32_t swizzled(uint32_t rows, uint32_t row, uint32_t column) {
    return (column / 64) * rows * 128 + row * 128 + ((((column % 64) / 8) ^ (row % 8)) * 16) + (column % 8) * 2;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t bytes) {   // bytes 0: zeros are written
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {   // arrives (counted in the barrier's expected arrivals) once this thread's copies have landed
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// the four softmax warps' barrier, which also ORs a flag over them: a wait that gave up takes all four out of the loop together
__device__ __forceinline__ bool softmax_barrier_or(bool flag) {
    uint32_t any;
    asm volatile("{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.or.pred p, 1, 128, q; selp.u32 %0, 1, 0, p; }"
                 : "=r"(any) : "r"(uint32_t(flag)) : "memory");
    return any != 0;
}

template<int DIM>
__global__ void __launch_bounds__(kThreads, 1) sparse_tc_kernel(const Args g) {
    using S = Shape<DIM>;
    constexpr int kChunks = DIM / 8;                        // 16-byte pieces of a row
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kOffBars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::kOffMisc + 4);
    volatile uint32_t* masks = reinterpret_cast<volatile uint32_t*>(smem + S::kOffMisc + 16);        // [kSlots]: which keys of the tile exist
    volatile int* rescale = reinterpret_cast<volatile int*>(smem + S::kOffMisc + 32);                // [2]: some head of tile j rescales
    float* factors = reinterpret_cast<float*>(smem + S::kOffMisc + 64);                              // [64]

    const SparseArgs& a = g.a;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const size_t split = blockIdx.x, row = blockIdx.z, head0 = size_t(blockIdx.y) * kRows;
    const int nheads = int(min(size_t(kRows), a.heads - head0)), nh = (nheads + 15) / 16 * 16;
    const uint32_t all_tiles = uint32_t((a.selections + kKeys - 1) / kKeys);
    const uint32_t per_split = (all_tiles + g.splits - 1) / g.splits;
    const uint32_t tile_begin = min(all_tiles, uint32_t(split) * per_split), tile_end = min(all_tiles, tile_begin + per_split);
    const uint32_t tiles = tile_end - tile_begin;
    const size_t nlo_blocks = (2 * g.pairs + 63) / 64;     // blocks of the row's tail that hold rotated columns
    float* partial = g.partial + ((row * a.heads + head0) * g.parts + 1 + split) * (DIM + 2);   // head h: + h * parts * (DIM + 2)
    const size_t head_stride = size_t(g.parts) * (DIM + 2);

    if (tiles == 0) {   // nothing selected for this split: an empty partial (zeros, maximum -inf)
        for (int i = tid; i < nheads * (DIM + 2); i += kThreads) {
            const int h = i / (DIM + 2), c = i % (DIM + 2);
            partial[h * head_stride + c] = c == DIM ? -INFINITY : 0.0f;
        }
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < kBars; ++i) {
            const bool copies = i >= kFull && i < kFull + kSlots, warps4 = (i >= kSFree && i < kSFree + 2) || (i >= kPFull && i < kPFull + 2);
            mbar_init(&bars[i], copies ? 32 * kCopyWarps : warps4 ? kSoftmaxWarps : 1);
        }
        *abort_flag = 0;
        rescale[0] = rescale[1] = 0;
    }
    fence_barrier_init();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // ---- the CTA's 64 query rows: rotated (double), BF16, in the swizzled K-major layout; the low parts of the tail blocks. Only the
    //      real head rows are read (four column pairs a thread in flight at a time); the others are zeros. ----
    {
        uint8_t* q_hi = smem + S::kOffQ;
        uint8_t* q_lo = smem + S::kOffQlo;
        const size_t plain = DIM - 2 * g.pairs, lo_from = DIM - 64 * nlo_blocks;
        for (int i = tid; i < (kRows - nheads) * kChunks; i += kThreads) {   // 16-byte pieces of the empty rows (all zeros: the swizzle does not matter)
            const int piece = i % kChunks, empty_row = nheads + i / kChunks;
            *reinterpret_cast<uint4*>(q_hi + (piece / 8) * (kRows * 128) + empty_row * 128 + (piece % 8) * 16) = make_uint4(0, 0, 0, 0);
        }
        for (int i = tid; i < kRows * int(nlo_blocks) * 8; i += kThreads)
            *reinterpret_cast<uint4*>(q_lo + i * 16) = make_uint4(0, 0, 0, 0);
        __syncthreads();
        const int real = nheads * (DIM / 2);
        for (int base = 0; base < real; base += 4 * kThreads) {
            float2 v[4];
            #pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = base + k * kThreads + tid, h = i / (DIM / 2), col = 2 * (i % (DIM / 2));
                v[k] = make_float2(0.0f, 0.0f);
                if (i < real) {
                    const float* src = g.q + (row * a.heads + head0 + h) * DIM + col;   // (only known to be 4-byte aligned)
                    v[k] = make_float2(src[0], src[1]);
                }
            }
            #pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = base + k * kThreads + tid, h = i / (DIM / 2), col = 2 * (i % (DIM / 2));
                if (i >= real) continue;
                if (size_t(col) >= plain) {
                    const double2 turn = g.forward[row * g.pairs + (col - plain) / 2];
                    const double x = v[k].x, y = v[k].y;
                    v[k] = make_float2(float(x * turn.x - y * turn.y), float(x * turn.y + y * turn.x));
                }
                const __nv_bfloat16 h0 = __float2bfloat16_rn(v[k].x), h1 = __float2bfloat16_rn(v[k].y);
                *reinterpret_cast<__nv_bfloat162*>(q_hi + swizzled(kRows, h, col)) = __halves2bfloat162(h0, h1);
                if (size_t(col) >= lo_from)
                    *reinterpret_cast<__nv_bfloat162*>(q_lo + swizzled(kRows, h, col - lo_from)) =
                        __halves2bfloat162(__float2bfloat16_rn(v[k].x - __bfloat162float(h0)), __float2bfloat16_rn(v[k].y - __bfloat162float(h1)));
            }
        }
    }
    fence_proxy_async();   // (the tensor core reads these bytes through the async proxy)
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // a bounded wait that also ends when another role has given up
    auto wait = [&](int bar, uint32_t parity) -> bool {
        if (mbar_try_wait(&bars[bar], parity)) return true;
        const uint64_t start = global_timer_ns();
        for (;;) {
            #pragma unroll 1
            for (int spin = 0; spin < 32; ++spin)
                if (mbar_try_wait(&bars[bar], parity)) return true;
            if (*abort_flag) return false;
            if (global_timer_ns() - start > 2000000000ull) { *abort_flag = 1; atomicExch(g.status, 1); return false; }
        }
    };
    const int32_t* chosen = a.selected + row * a.selections;

    if (warp < kSoftmaxWarps) {
        // ================= softmax (lanes 0-15 of a warp own head rows 16 warp + lane: where an M = 64 accumulator keeps them) =================
        const uint32_t lane_base = uint32_t(warp * 32) << 16;
        const int head = 16 * warp + lane;                  // (meaningful for lane < 16)
        const bool owner = lane < 16;
        float m_run = -INFINITY, l_run = 0.0f;
        bool alive = true;
        for (uint32_t j = 0; j < tiles && alive; ++j) {
            const uint32_t b = j & 1, slot = j % kSlots;
            // (both waits of the tile come before its first barrier, which carries their outcome to all four warps)
            bool failed = !wait(kSFull + b, (j >> 1) & 1);
            if (j >= 2) failed = !wait(kPFree + b, ((j - 2) >> 1) & 1) || failed;
            tc_fence_after();
            float s[32];
            tmem_ld32(tmem + lane_base + 320 + b * 32, s);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kSFree + b]);
            const uint32_t mask = masks[slot];
            float top = -INFINITY;
            #pragma unroll
            for (int n = 0; n < 32; ++n) top = fmaxf(top, (mask >> n) & 1u ? s[n] : -INFINITY);
            top *= g.scale_log2;
            const float m_new = fmaxf(m_run, top);
            // the old maximum stays while the new one is within 2^8 of it: no pass over O^T in TMEM
            const bool grow = m_new > m_run + kRescaleThreshold || (m_run == -INFINITY && m_new > -INFINITY);
            const float m_use = grow ? m_new : m_run;
            const bool rescales = owner && grow && m_run != -INFINITY;
            const float factor = rescales ? fast_exp2(m_run - m_use) : 1.0f;
            if (owner) factors[head] = factor;
            if (__any_sync(0xffffffffu, rescales) && lane == 0) rescale[b] = 1;
            if (softmax_barrier_or(failed)) { alive = false; break; }
            if (rescale[b]) {
                // some head's maximum has grown past the threshold: its column of O^T is rescaled once every product issued so far
                // has landed (and before this tile's product can start: it waits for the weights below)
                failed = j >= 1 && !wait(kDone, (j - 1) & 1);
                tc_fence_after();
                if (j >= 1 && !failed) {
                    #pragma unroll 1
                    for (int mt = 0; mt < S::kMTiles; ++mt)
                        #pragma unroll 1
                        for (int c0 = 0; c0 < nh; c0 += 16) {
                            float o[16];
                            tmem_ld16(tmem + lane_base + mt * 64 + c0, o);
                            #pragma unroll
                            for (int i = 0; i < 16; ++i) o[i] *= factors[c0 + i];
                            tmem_st16(tmem + lane_base + mt * 64 + c0, o);
                        }
                    tmem_st_wait();
                }
                tc_fence_before();
                if (softmax_barrier_or(failed)) { alive = false; break; }
                if (tid == 0) rescale[b] = 0;
            }
            l_run *= factor;
            m_run = m_use;
            const float u = m_run == -INFINITY ? 0.0f : m_run;
            // this head's weights for the tile's 32 keys: a row of P^T (BF16, K-major: 64 bytes of a 128-byte row)
            uint32_t packed[16];
            float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            #pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float p0 = (mask >> (2 * i)) & 1u ? fast_exp2(fmaf(s[2 * i], g.scale_log2, -u)) : 0.0f;
                const float p1 = (mask >> (2 * i + 1)) & 1u ? fast_exp2(fmaf(s[2 * i + 1], g.scale_log2, -u)) : 0.0f;
                packed[i] = pack_bf16x2(p0, p1);
                // (the denominator sums what the product will use: the rounded weights)
                sums[i & 3] += __uint_as_float(packed[i] << 16) + __uint_as_float(packed[i] & 0xffff0000u);
            }
            l_run += (sums[0] + sums[1]) + (sums[2] + sums[3]);
            if (owner) {
                uint8_t* p_row = smem + S::kOffP + b * (kRows * 128) + head * 128;
                #pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(p_row + ((c ^ (head % 8)) * 16)) = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kPFull + b]);
        }
        // ---- epilogue: a thread per output column (TMEM lane), the heads along the columns ----
        // (first the product before the last: a barrier that every product commits to may otherwise be read a phase early)
        if (alive && tiles >= 2 && !wait(kPFree + ((tiles - 2) & 1), ((tiles - 2) >> 1) & 1)) alive = false;
        if (alive && wait(kDone, (tiles - 1) & 1)) {
            tc_fence_after();
            #pragma unroll 1
            for (int mt = 0; mt < S::kMTiles; ++mt) {
                const int d = mt * 128 + warp * 32 + lane;
                #pragma unroll 1
                for (int c0 = 0; c0 < nh; c0 += 16) {
                    float o[16];
                    tmem_ld16(tmem + lane_base + mt * 64 + c0, o);
                    if (d < DIM) {
                        #pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (c0 + i < nheads) partial[(c0 + i) * head_stride + d] = o[i];
                    }
                }
            }
            if (owner && head < nheads) {
                partial[head * head_stride + DIM] = m_run * 0.6931471805599453f;   // (the partials' maxima are natural logarithms)
                partial[head * head_stride + DIM + 1] = l_run;
            }
        }
    } else if (warp == kMmaWarp) {
        // ================= the MMA issuer =================
        if (lane == 0) {
            long long trace[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long started = clock64();
            (void)started;
            const uint32_t ring = smem_u32(smem + S::kOffRing);
            const uint32_t q_hi = desc_low(smem_u32(smem + S::kOffQ), 16), q_lo = desc_low(smem_u32(smem + S::kOffQlo), 16);
            const uint32_t p_low = desc_low(smem_u32(smem + S::kOffP), 16);
            const uint32_t idesc_s = instr_desc(kRows, kKeys, false, false), idesc_o = instr_desc(128, nh, true, false);
            const int lo_first = S::kBlocks - int(nlo_blocks);
            for (uint32_t i = 0; i <= tiles; ++i) {
                if (i < tiles) {
                    const uint32_t b = i & 1, slot = i % kSlots, tile = desc_low(ring + slot * S::kTile, 16), s_tmem = tmem + 320 + b * 32;
                    long long since = clock64();
                    if (i >= 2 && !wait(kSFree + b, ((i - 2) >> 1) & 1)) break;
                    SDX_TRACE_ADD(3, since);
                    since = clock64();
                    if (!wait(kFull + slot, (i / kSlots) & 1)) break;
                    SDX_TRACE_ADD(1, since);
                    fence_proxy_async();   // (the copies wrote through the generic proxy)
                    tc_fence_after();
                    #pragma unroll
                    for (int blk = 0; blk < S::kBlocks; ++blk)
                        #pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma(s_tmem, desc_of(q_hi + ((blk * (kRows * 128) + kk * 32) >> 4)), desc_of(tile + ((blk * (kKeys * 128) + kk * 32) >> 4)),
                                 idesc_s, blk > 0 || kk > 0);
                    #pragma unroll
                    for (int lb = 0; lb < 2; ++lb) {
                        if (lb >= int(nlo_blocks)) break;
                        #pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            umma(s_tmem, desc_of(q_lo + ((lb * (kRows * 128) + kk * 32) >> 4)),
                                 desc_of(tile + (((lo_first + lb) * (kKeys * 128) + kk * 32) >> 4)), idesc_s, true);
                    }
                    umma_commit(&bars[kSFull + b]);
                }
                if (i >= 1) {
                    const uint32_t j = i - 1, b = j & 1, slot = j % kSlots;
                    const uint32_t tile = desc_low(ring + slot * S::kTile, kKeys * 128), p_tile = p_low + ((b * (kRows * 128)) >> 4);
                    const long long since = clock64();
                    if (!wait(kPFull + b, (j >> 1) & 1)) break;
                    SDX_TRACE_ADD(2, since);
                    tc_fence_after();
                    #pragma unroll
                    for (int mt = 0; mt < S::kMTiles; ++mt)
                        #pragma unroll
                        for (int ks = 0; ks < kKeys / 16; ++ks)
                            umma(tmem + mt * 64, desc_of(tile + ((2 * mt * (kKeys * 128) + ks * (16 * 128)) >> 4)), desc_of(p_tile + ((ks * 32) >> 4)),
                                 idesc_o, j > 0 || ks > 0);
                    umma_commit(&bars[kFree + slot]);
                    umma_commit(&bars[kPFree + b]);
                    umma_commit(&bars[kDone]);
                }
            }
#if defined(SDX_TRACE)
            trace[0] = clock64() - started; trace[5] = tiles;
            long long* mine = g.trace + ((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8;
            for (int i = 0; i < 8; ++i) if (i != 4) mine[i] = trace[i];
#endif
        }
    } else {
        // ================= the copy warps: 16-byte copies into the swizzled tile, a warp instruction = 512 bytes of one row =================
        const uint8_t* halves = reinterpret_cast<const uint8_t*>(state_halves(a.compressed));
        const int ctid = tid - 32 * kCopyWarp0;
        const size_t sel_begin = size_t(tile_begin) * kKeys;
        auto index_at = [&](uint32_t t) -> int32_t {
            const size_t index = sel_begin + size_t(t) * kKeys + lane;
            int32_t at = t < tiles && index < a.selections ? chosen[index] : -1;
            if (at >= 0 && size_t(at) >= a.compressed_rows) { atomicExch(g.status, 2); at = -1; }   // (a row number past the cache: taken as absent, reported)
            return at;
        };
        int32_t at = index_at(0);
        for (uint32_t t = 0; t < tiles; ++t) {
            const uint32_t slot = t % kSlots;
            const int32_t next = index_at(t + 1);   // (the list comes from HBM like the rows: asked for a tile ahead)
            const long long since = clock64();
            (void)since;
            if (t >= uint32_t(kSlots) && !wait(kFree + slot, (t / kSlots - 1) & 1)) break;
#if defined(SDX_TRACE)
            if (ctid == 0) atomicAdd(reinterpret_cast<unsigned long long*>(g.trace + ((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + 4),
                                     (unsigned long long)(clock64() - since));
#endif
            const uint32_t live = __ballot_sync(0xffffffffu, at >= 0);
            if (ctid == 0) masks[slot] = live;
            const uint32_t tile = smem_u32(smem + S::kOffRing + slot * S::kTile);
            #pragma unroll 3
            for (int i = 0; i < kKeys * kChunks / (32 * kCopyWarps); ++i) {
                const int piece = ctid + 32 * kCopyWarps * i, key = piece / kChunks, chunk = piece % kChunks;
                const int32_t from = __shfl_sync(0xffffffffu, at, key);
                const uint32_t dst = tile + (chunk / 8) * (kKeys * 128) + key * 128 + (((chunk % 8) ^ (key % 8)) * 16);
                cp_async16(dst, halves + (from >= 0 ? size_t(from) * DIM * 2 + chunk * 16 : 0), from >= 0 ? 16u : 0u);
            }
            cp_async_arrive(&bars[kFull + slot]);
            at = next;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");   // (nothing in flight into this CTA's shared memory when it exits)
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
}

}  // namespace tcl

// The FP32 kernel and the combine of ds_sparse.cu: the window rows' partial and the merge of all partials.
void sparse_window_partial(Device& d, const SparseArgs& a, const float* q, size_t rows, size_t pairs, const double2* forward, float* rotated,
                           float* partial, size_t parts, cudaStream_t stream = nullptr);
void sparse_combine(Device& d, const float* partial, size_t parts, size_t rows, size_t heads, size_t dim, const float* sinks, size_t pairs,
                    const double2* inverse, float* out);

// Where the tcgen05 kernel is the faster one: 128 heads or more a call, BF16 rows, a short window. Measured on a B200 (32 rows x
// top-2048, dim 576): 128 heads 114 us against the mma.sync kernel's 146 us (which reads every row once per 16 heads: eight times);
// 64 heads 74 us against 75 us; 16 heads 73 us against 29 us. The kernel is bound by the tensor pipe's instruction rate, not its
// arithmetic: an instruction of 64 x 32 x 16 or 128 x 64 x 16 costs the pipe about as long as one four times its size (48 cycles at
// the least, about 70 with these operands), and dim 576 leaves shared memory for tiles of 32 keys only.
bool sparse_tc_supported(const SparseArgs& a) {
    return (a.dim == 512 || a.dim == 576) && a.heads % 16 == 0 && a.heads >= 128 && a.selections >= 64 && a.window <= 16 &&
           state_is_bf16(a.compressed) && reinterpret_cast<uintptr_t>(state_halves(a.compressed)) % 16 == 0;
}

template<int DIM>
static void launch_tc(Device& d, const tcl::Args& args, size_t rows, size_t head_tiles) {
    using S = tcl::Shape<DIM>;
    static bool configured[64] = {};
    if (!configured[d.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(tcl::sparse_tc_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::kSmem)));
        configured[d.ordinal & 63] = true;
    }
    tcl::sparse_tc_kernel<DIM><<<dim3(args.splits, unsigned(head_tiles), unsigned(rows)), tcl::kThreads, S::kSmem, d.stream>>>(args);
    ++d.launches;
}

void sparse_tc_launch(Device& d, const SparseArgs& a, const float* q, const float* sinks, size_t rows, size_t pairs, const double2* forward,
                      const double2* inverse, float* out) {
    const size_t head_tiles = (a.heads + tcl::kRows - 1) / tcl::kRows;
    const size_t all_tiles = (a.selections + tcl::kKeys - 1) / tcl::kKeys;
    // one wave of CTAs where the call is small: as many splits of a row's keys as fill the SMs, each of at least four tiles
    size_t splits = std::max<size_t>(1, size_t(d.sms) / std::max<size_t>(1, rows * head_tiles));
    splits = std::min<size_t>({splits, std::max<size_t>(1, all_tiles / 4), size_t(32)});
    const size_t parts = splits + 1;   // part 0: the window rows (FP32 kernel)
    const size_t partial_bytes = checked_product({rows, a.heads, parts, a.dim + 2, 4});
    const size_t q_bytes = pairs ? (checked_product({rows, a.heads, a.dim, 4}) + 255) / 256 * 256 : 0;
    size_t trace_bytes = 0;
#if defined(SDX_TRACE)
    const size_t trace_at = (q_bytes + partial_bytes + 255) / 256 * 256;
    trace_bytes = 256 + splits * head_tiles * rows * 64;   // the counters follow the partials in the workspace
#endif
    auto* work = static_cast<uint8_t*>(ensure(d, d.partial, d.partial_bytes, q_bytes + partial_bytes + trace_bytes));
    auto* partial = reinterpret_cast<float*>(work + q_bytes);
    sparse_window_partial(d, a, q, rows, pairs, forward, reinterpret_cast<float*>(work), partial, parts);
    tcl::Args args{};
    args.a = a; args.q = q; args.pairs = pairs; args.forward = forward;
    args.scale_log2 = a.scale * 1.4426950408889634f;
    args.status = status_word(d);
    args.partial = partial;
    args.parts = uint32_t(parts); args.splits = uint32_t(splits);
#if defined(SDX_TRACE)
    args.trace = reinterpret_cast<long long*>(work + trace_at);
    SDB_CHECK(cudaMemsetAsync(args.trace, 0, splits * head_tiles * rows * 64, d.stream));
    d.trace = args.trace; d.trace_ctas = splits * head_tiles * rows;
#endif
    if (a.dim == 576) launch_tc<576>(d, args, rows, head_tiles); else launch_tc<512>(d, args, rows, head_tiles);
    SDB_CHECK(cudaGetLastError());
    sparse_combine(d, partial, parts, rows, a.heads, a.dim, sinks, pairs, inverse, out);
}

}  // namespace sdb

// The counters of the last traced launch on this handle (eight per CTA), for builds with -DSDX_TRACE; 0 CTAs in any other build.
extern "C" int sdx_trace_read(void* handle, int64_t* out, uint64_t capacity) {
    try {
        auto& value = sdb::device(handle);
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        const size_t ctas = std::min<size_t>(value.trace_ctas, size_t(capacity / 8));
        if (ctas) SDB_CHECK(cudaMemcpy(out, value.trace, ctas * 64, cudaMemcpyDeviceToHost));
        return int(ctas);
    } catch (const std::exception& e) { sdb::last_error = e.what(); return -1; }
}
