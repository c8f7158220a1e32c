// Latent sparse attention on the 5th-generation tensor cores for 128 heads and more: a pair of CTAs (a thread-block cluster of two)
// takes one query row with 128 of its heads and splits the COLUMNS of the latent rows between them.
//
// What it replaces: op_attention_scores_kernel + op_attention_output_kernel (gpu/ops.hpp:1329-1434, 1542-1661) and, as a design,
// the reference's all-heads-of-a-row-per-block WMMA form (gpu/ds_attention_wmma.hpp:25-326: every key row read once for all the
// heads of a query row, weights formed once per row).
//
// Why a pair: a tcgen05.mma costs the tensor pipe about max(48, N / 2) cycles whatever its M, so the products must be few and large.
// 128 heads x 576 output columns are 576 TMEM columns (of 512) and 128 x 576 BF16 queries are 144 KB of shared memory: one CTA holds
// neither. Split by columns, CTA h of the pair holds the queries' and the gathered rows' columns of its half (320 + 256 of 576,
// 256 + 256 of 512), forms the scores' PARTIAL sums over them,
//     S_h[128 heads x 32 keys] = Q[:, half h] . K_tile[:, half h]^T        M 128, N 32, K 16: 20 (or 16) instructions a tile
// and the two partial sums meet through distributed shared memory: a softmax warp (a thread per head, in both CTAs) lays its 32 rows of
// S_h down in shared memory, sends them into the partner's receive buffer with one bulk copy (TMA engine) that completes on the
// partner's mbarrier, waits for the partner's rows and adds them. Both CTAs then hold the same scores (an FP32 addition commutes) and
// form the same weights; each accumulates ITS columns of the output,
//     O_h[128 x half] += P[128 x 32] . K_tile[:, half h]                   M 128, N 256 (+ N 64): 2 (or 4) instructions a tile
// with P written over the scores in TMEM as the A operand (as the prompt kernel does) and the tile, which served as the K-major B
// operand of the scores, now read as an MN-major B operand: the keys are the values (gpu/ops.hpp:1309-1316). Per 64 keys and 128
// heads the pair issues 96 instructions where the single-CTA kernel (ds_sparse_tc.cu: 64 heads, 32 keys, O transposed) issues 184;
// tiles of 64 keys would halve that again, but their exchange buffers (four of 32 KB) do not fit beside Q and the ring.
//
// Warps (14): 0-3 softmax and epilogue (thread = head = TMEM lane), 4-7 take the partial scores out of TMEM and send them to the
// partner, 8 issues the score products, 9 the output products (a thread each, so that one's waits pass while the other issues),
// 10-13 gather the tile's half rows with 16-byte cp.async copies written where
// the 128-byte swizzle of the tensor core's shared-memory descriptors expects them (a ring of four tiles; four score buffers in
// TMEM). The CTA leaves a partial (its columns' sums; the maximum and the denominator by CTA 0) per head for its split; the window
// rows' partial comes from the FP32 kernel and sparse_combine_kernel merges them with the sink and turns the rotated columns back
// (gpu/ops.hpp:1561-1583, 1528-1538). Every wait is bounded and reports through the status word; nobody leaves before the pair
// has met at a cluster barrier.
//
// Measured on a B200 (32 rows x top-2048, dim 576, 128 heads): 104 us a call against the single-CTA kernel's 115 us and the
// mma.sync kernel's 146 us; 16 spans x 8 rows in one launch 349 us against 401 us and 534 us. (Asking a tile's rows into L2
// several tiles ahead made both slower; so did tiles of 48 keys in a ring of three.) Of the pair kernel's 80 us a CTA
// spends 7 us preparing Q, 54 us in its 32 tiles (the softmax warps are the busy ones: 2600 of a tile's 3200 cycles, most of it the
// fixed cost of a tile - TMEM load and store with their waits, the proxy fence, the copy's issue - not its 32 exponentials) and 9 us
// writing its partial.
#include "ds_sparse.cuh"

#include <algorithm>

namespace sdb {
namespace tc2 {

constexpr int kHeads = 128, kKeys = 32, kSlots = 4;   // heads a CTA, keys a tile, tiles in the ring
constexpr int kSoftmaxWarps = 4, kSendWarp0 = 4, kScoreWarp = 8, kValueWarp = 9, kCopyWarp0 = 10, kCopyWarps = 4, kThreads = 32 * (kCopyWarp0 + kCopyWarps);
constexpr int kSCol = 320, kSStride = kKeys, kScoreBuffers = (512 - kSCol) / kSStride >= 4 ? 4 : 3, kExchange = kHeads * kKeys * 4;   // the score buffers' first TMEM column and their distance; bytes of one exchange buffer
static_assert(kKeys == 32 || kKeys == 48 || kKeys == 64, "a tile: whole 16-key steps of the output product, at most two words of indices a lane");
constexpr float kRescaleThreshold = 8.0f;

template<int DIM> struct Shape {
    static constexpr int kDims0 = DIM == 576 ? 320 : 256, kDims1 = DIM - kDims0;   // the halves' columns: whole 64-column blocks
    static constexpr int kHalf0 = kSlots * (kDims0 / 64) * kKeys * 128 + (kDims0 / 64) * kHeads * 128 + 4 * kExchange;       // ring | Q | exchange (two to send from, two to receive into)
    static constexpr int kHalf1 = kSlots * (kDims1 / 64) * kKeys * 128 + (kDims1 / 64 + 2) * kHeads * 128 + 4 * kExchange;   // ring | Q | two low blocks | exchange
    static constexpr int kBytes = kHalf0 > kHalf1 ? kHalf0 : kHalf1;
    static constexpr size_t kSmem = kBytes + 512 + 1024;   // + barriers and flags + slack to align the base to 1024 bytes
    static_assert(kSmem <= 232448, "shared memory of one CTA");
};

enum Bar { kFull = 0, kFree = kSlots, kSFull = 2 * kSlots, kSFree = kSFull + kScoreBuffers, kPFull = kSFree + kScoreBuffers, kRecv = kPFull + kScoreBuffers, kAck = kRecv + 8, kStaged = kAck + 8, kRead = kStaged + 8, kBars = kRead + 8 };   // kRecv, kAck: [buffer][softmax warp]   // kRecv: [buffer][softmax warp]

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

// Built with -DSDX_TRACE: eight 64-bit counters a CTA (0 the score thread's cycles in its loop, 1 of them waiting for a tile, 5 tiles;
// of head 0's softmax thread: 3 the cycles before its loop (Q's preparation), 7 in its loop, 4 of them waiting for the two halves'
// rows, 2 after it (the last products and the partial's stores); 6 head 0's sender's wait for the scores).
#if defined(SDX_TRACE)
#define SDX_TRACE_ADD(slot, since) trace[slot] += clock64() - (since)
#define SDX_TRACE_OUT(slot) g.trace[((size_t(blockIdx.z) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + (slot)] = trace[slot]
#else
#define SDX_TRACE_ADD(slot, since) ((void)0)
#define SDX_TRACE_OUT(slot) ((void)0)
#endif

constexpr uint32_t kDescHigh = 0x40004040u;   // stride 1024 bytes between 8-row groups, descriptor version 1, 128-byte swizzle
__device__ __forceinline__ uint32_t desc_low(uint32_t address, uint32_t leading_bytes) { return ((address & 0x3ffffu) >> 4) | ((leading_bytes >> 4) << 16); }
__device__ __forceinline__ uint64_t desc_of(uint32_t low) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(low), "r"(kDescHigh));
    return d;
}
// kind::f16 instruction descriptor: FP32 accumulator, BF16 A and B, A K-major, B K-major or MN-major, shape M x N
__device__ __forceinline__ uint32_t instr_desc(int m, int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(b_mn) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
}
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
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
                   "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]),
                   "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
                   "r"(v[30]), "r"(v[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    #pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
                   "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
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
// ---- the pair ----
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_address(uint32_t local, uint32_t rank) {   // the same shared-memory offset in CTA `rank` of the cluster
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, unsigned parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}

template<int DIM>
__global__ void __launch_bounds__(kThreads, 1) sparse_tc2_kernel(const Args g) {
    using S = Shape<DIM>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const SparseArgs& a = g.a;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const long long kernel_started = clock64();
    (void)kernel_started;
    const uint32_t half = blockIdx.y, partner = half ^ 1u;                     // (cluster dimensions (1, 2, 1): the rank in the pair is blockIdx.y)
    const int d0 = half ? S::kDims0 : 0, dims = half ? S::kDims1 : S::kDims0, blocks = dims / 64;
    const size_t nlo_blocks = (2 * g.pairs + 63) / 64;                         // blocks of a row's tail that hold rotated columns: all in half 1
    const int lo_blocks = half ? int(nlo_blocks) : 0;
    // this half's shared memory: ring | Q | Q's low parts | exchange | barriers and flags
    const int tile_bytes = blocks * kKeys * 128;
    uint8_t* ring = smem;
    uint8_t* q_hi = ring + kSlots * tile_bytes;
    uint8_t* q_lo = q_hi + blocks * kHeads * 128;
    uint8_t* exchange = smem + S::kBytes - 4 * kExchange;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBars + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile unsigned long long* masks = reinterpret_cast<volatile unsigned long long*>(bars + kBars + 3);   // [kSlots]: which keys of the tile exist

    const size_t head_tiles = (a.heads + kHeads - 1) / kHeads;
    const size_t split = blockIdx.x % g.splits, head0 = size_t(blockIdx.x / g.splits) * kHeads, row = blockIdx.z;
    (void)head_tiles;
    const int nheads = int(min(size_t(kHeads), a.heads - head0));
    const uint32_t all_tiles = uint32_t((a.selections + kKeys - 1) / kKeys);
    const uint32_t per_split = (all_tiles + g.splits - 1) / g.splits;
    const uint32_t tile_begin = min(all_tiles, uint32_t(split) * per_split), tile_end = min(all_tiles, tile_begin + per_split);
    const uint32_t tiles = tile_end - tile_begin;
    const size_t head_stride = size_t(g.parts) * (DIM + 2);
    float* partial = g.partial + ((row * a.heads + head0) * g.parts + 1 + split) * (DIM + 2);   // head h: + h * head_stride

    if (tiles == 0) {   // nothing selected for this split (both CTAs of the pair see the same): an empty partial, this half's columns
        for (int i = tid; i < nheads * (dims + 2); i += kThreads) {
            const int h = i / (dims + 2), c = i % (dims + 2);
            if (c < dims) partial[h * head_stride + d0 + c] = 0.0f;
            else if (half == 0) partial[h * head_stride + DIM + (c - dims)] = c == dims ? -INFINITY : 0.0f;
        }
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < kBars; ++i) {
            const bool copies = i >= kFull && i < kFull + kSlots, warps4 = i >= kPFull && i < kPFull + kScoreBuffers;
            mbar_init(&bars[i], copies ? 32 * kCopyWarps : warps4 ? kSoftmaxWarps : 1);
        }
        *abort_flag = 0;
    }
    fence_barrier_init();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // ---- this half's columns of the 128 query rows: rotated (double), BF16, in the swizzled K-major layout; the low parts of the tail
    //      blocks (the rotated columns are F32 values, the plain ones are taken as BF16). Rows past the call's heads are zeros. A thread
    //      takes eight columns at a time: two 16-byte loads where the queries are 16-byte aligned, one 16-byte store a plane. ----
    {
        const size_t plain = DIM - 2 * g.pairs, lo_from = DIM - 64 * nlo_blocks;
        const int chunks = dims / 8;
        const bool aligned = reinterpret_cast<uintptr_t>(g.q) % 16 == 0;
        #pragma unroll 4
        for (int i = tid; i < kHeads * chunks; i += kThreads) {
            const int h = i / chunks, col = 8 * (i % chunks);   // (col: within the half)
            const size_t gcol = size_t(d0 + col);
            float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
            if (h < nheads) {
                const float* src = g.q + (row * a.heads + head0 + h) * DIM + gcol;
                if (aligned) {
                    const float4 x = __ldg(reinterpret_cast<const float4*>(src)), y = __ldg(reinterpret_cast<const float4*>(src) + 1);
                    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
                } else {
                    #pragma unroll
                    for (int k = 0; k < 8; ++k) v[k] = src[k];
                }
                if (gcol + 8 > plain) {
                    #pragma unroll
                    for (int k = 0; k < 8; k += 2) {
                        if (gcol + k < plain) continue;
                        const double2 turn = g.forward[row * g.pairs + (gcol + k - plain) / 2];
                        const double x = v[k], y = v[k + 1];
                        v[k] = float(x * turn.x - y * turn.y); v[k + 1] = float(x * turn.y + y * turn.x);
                    }
                }
            }
            uint32_t hi[4], lo[4];
            #pragma unroll
            for (int k = 0; k < 4; ++k) {
                hi[k] = pack_bf16x2(v[2 * k], v[2 * k + 1]);
                lo[k] = pack_bf16x2(v[2 * k] - __uint_as_float(hi[k] << 16), v[2 * k + 1] - __uint_as_float(hi[k] & 0xffff0000u));
            }
            *reinterpret_cast<uint4*>(q_hi + swizzled(kHeads, h, col)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            if (lo_blocks && gcol >= lo_from)
                *reinterpret_cast<uint4*>(q_lo + swizzled(kHeads, h, uint32_t(gcol - lo_from))) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
    }
    fence_proxy_async();   // (the tensor core reads these bytes through the async proxy)
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // (the partner's barriers are initialised before anything is sent to them)
    cluster_arrive(); cluster_wait();

    // a bounded wait that also ends when another role has given up
    auto wait = [&](int bar, uint32_t parity) -> bool {
        if (mbar_try_wait_cluster(&bars[bar], parity)) return true;
        const uint64_t start = global_timer_ns();
        for (;;) {
            #pragma unroll 1
            for (int spin = 0; spin < 32; ++spin)
                if (mbar_try_wait_cluster(&bars[bar], parity)) return true;
            if (*abort_flag) return false;
            if (global_timer_ns() - start > 2000000000ull) { *abort_flag = 1; atomicExch(g.status, 1); return false; }
        }
    };
    const int32_t* chosen = a.selected + row * a.selections;

    if (warp < kSendWarp0 + kSoftmaxWarps) {
        // ================= softmax and epilogue (warps 0-3) and their senders (warps 4-7): a thread per head (TMEM lane 32 (warp % 4) + lane) =================
        const int quad = warp % 4;
        const bool sender = warp >= kSendWarp0;
        // A tile's work comes in two halves with a warp each, so that the exchange of one tile's partial sums is under way while an earlier
        // tile's weights are formed:
        //   send(j)   (warps 4-7) the quadrant's 32 rows of S_h leave TMEM for the local send buffer j % 2 ([quadrant][piece][lane]: neither
        //             these stores nor the loads later meet in a bank) and lane 0 sends them (one bulk copy, TMA engine, through distributed
        //             shared memory) to the same place of the partner's receive buffer j % 2, completing on the mbarrier the partner's
        //             same quadrant waits on (it needs its own heads' sums only). Before that, for j >= 2, it waits for the partner's word
        //             that it has read tile j - 2's rows (then this CTA's copy of tile j - 2 has landed and the partner's receive buffer may
        //             be overwritten) and for this CTA's softmax warp to have read its own rows of tile j - 2 back.
        //   finish(j) (warps 0-3) waits for this CTA's rows to be laid down and for the partner's to arrive, adds them, tells both senders
        //             that they are read, and forms the weights.
        const int head = 32 * quad + lane;
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        const uint32_t at = uint32_t(quad) * (kExchange / 4) + uint32_t(lane) * 16;   // + piece * 512, within one exchange buffer
        uint8_t* send_buffers = exchange;                     // [2]
        uint8_t* receive_buffers = exchange + 2 * kExchange;  // [2]
        const uint32_t their_receive = cluster_address(smem_u32(receive_buffers), partner);
        const uint32_t their_recv_bar = cluster_address(smem_u32(&bars[kRecv]), partner), their_ack_bar = cluster_address(smem_u32(&bars[kAck]), partner);
        float m_run = -INFINITY, l_run = 0.0f;
        bool alive = true;
        long long trace[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const long long started = clock64();
        (void)started;
        const long long prologue_cycles = started - kernel_started;
        (void)prologue_cycles;
        auto send = [&](uint32_t j) {
            const uint32_t b = j & 1;
            long long since = clock64();
            (void)since;
            const uint32_t sb = j % kScoreBuffers;
            if (__any_sync(0xffffffffu, !wait(kSFull + sb, (j / kScoreBuffers) & 1))) { alive = false; return; }   // (a warp decides as one: its TMEM accesses are warp-wide)
            SDX_TRACE_ADD(6, since);
            tc_fence_after();
            float s[kKeys];
            tmem_ld32(tmem + lane_base + kSCol + sb * kSStride, s);
            if (kKeys == 64) tmem_ld32(tmem + lane_base + kSCol + sb * kSStride + 32, s + 32);
            else if (kKeys == 48) tmem_ld16(tmem + lane_base + kSCol + sb * kSStride + 32, s + 32);
            since = clock64();
            // (the partner has read tile j - 2's rows: this CTA's copy of them has landed and the partner's receive buffer is free; and this
            //  CTA's softmax warp has read its own rows of tile j - 2 back from the send buffer)
            if (j >= 2 && __any_sync(0xffffffffu, !wait(kAck + 4 * b + quad, ((j - 2) >> 1) & 1) || !wait(kRead + 4 * b + quad, ((j - 2) >> 1) & 1))) { alive = false; return; }
            uint8_t* mine = send_buffers + b * kExchange + at;
            #pragma unroll
            for (int piece = 0; piece < kKeys / 4; ++piece)
                *reinterpret_cast<float4*>(mine + piece * 512) = make_float4(s[4 * piece], s[4 * piece + 1], s[4 * piece + 2], s[4 * piece + 3]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars[kStaged + 4 * b + quad]);                   // (this CTA's softmax warp may read the rows back)
                mbar_expect_tx(&bars[kRecv + 4 * b + quad], kExchange / 4);   // (the partner's copy into this CTA)
                asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(their_receive + b * kExchange + uint32_t(quad) * (kExchange / 4)), "r"(smem_u32(mine)), "r"(uint32_t(kExchange / 4)),
                               "r"(their_recv_bar + (4 * b + quad) * 8) : "memory");
            }
        };
        if (sender) {
            for (uint32_t j = 0; j < tiles && alive; ++j) send(j);
#if defined(SDX_TRACE)
            if (head == 0) SDX_TRACE_OUT(6);
#endif
        }
        for (uint32_t j = 0; j < tiles && alive && !sender; ++j) {
            const uint32_t b = j & 1;
            long long since = clock64();
            (void)since;
            if (__any_sync(0xffffffffu, !wait(kStaged + 4 * b + quad, (j >> 1) & 1) || !wait(kRecv + 4 * b + quad, (j >> 1) & 1))) { alive = false; break; }
            SDX_TRACE_ADD(4, since);
            float s[kKeys];
            #pragma unroll
            for (int piece = 0; piece < kKeys / 4; ++piece) {
                const float4 own = *reinterpret_cast<const float4*>(send_buffers + b * kExchange + at + piece * 512);
                const float4 other = *reinterpret_cast<const float4*>(receive_buffers + b * kExchange + at + piece * 512);
                s[4 * piece] = own.x + other.x; s[4 * piece + 1] = own.y + other.y; s[4 * piece + 2] = own.z + other.z; s[4 * piece + 3] = own.w + other.w;
            }
            __syncwarp();
            if (lane == 0) {   // (release at cluster scope, after the warp's loads: the partner may now overwrite the receive buffer and reuse its send buffer)
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(their_ack_bar + (4 * b + quad) * 8) : "memory");
                mbar_arrive(&bars[kRead + 4 * b + quad]);
            }
            const unsigned long long mask = masks[j % kSlots];
            const uint32_t mask_lo = uint32_t(mask), mask_hi = uint32_t(mask >> 32);
            (void)mask_hi;
            if (mask != (kKeys == 64 ? ~0ull : (1ull << kKeys) - 1)) {   // (a tile with absent rows: their scores never count)
                #pragma unroll
                for (int n = 0; n < (kKeys < 32 ? kKeys : 32); ++n)
                    if (!((mask_lo >> n) & 1u)) s[n] = -INFINITY;
                #pragma unroll
                for (int n = 0; n < kKeys - 32; ++n)
                    if (!((mask_hi >> n) & 1u)) s[32 + n] = -INFINITY;
            }
            float tops[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            #pragma unroll
            for (int n = 0; n < kKeys; ++n) tops[n & 3] = fmaxf(tops[n & 3], s[n]);
            const float top = fmaxf(fmaxf(tops[0], tops[1]), fmaxf(tops[2], tops[3])) * g.scale_log2;
            const float m_new = fmaxf(m_run, top);
            // the old maximum stays while the new one is within 2^8 of it: no pass over O in TMEM
            const bool grow = m_new > m_run + kRescaleThreshold || (m_run == -INFINITY && m_new > -INFINITY);
            const float m_use = grow ? m_new : m_run;
            const bool rescales = grow && m_run != -INFINITY;
            const float factor = rescales ? fast_exp2(m_run - m_use) : 1.0f;
            if (j >= 1 && __any_sync(0xffffffffu, rescales)) {
                // a head's maximum has grown past the threshold: its row of O is rescaled once every product issued so far has landed
                // (this tile's product cannot start before: it waits for the weights below)
                // (tile j - 1's product frees its score buffer when it is done, and the products run in order; that barrier's phase is known to
                //  within one, where a barrier every product commits to may be two or more phases behind this thread)
                if (__any_sync(0xffffffffu, !wait(kSFree + (j - 1) % kScoreBuffers, ((j - 1) / kScoreBuffers) & 1))) { alive = false; break; }
                tc_fence_after();
                #pragma unroll 1
                for (int c0 = 0; c0 < dims; c0 += 32) {
                    float o[32];
                    tmem_ld32(tmem + lane_base + c0, o);
                    uint32_t bits[32];
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) bits[i] = __float_as_uint(o[i] * factor);
                    tmem_st32(tmem + lane_base + c0, bits);
                }
                tmem_st_wait();
            }
            l_run *= factor;
            m_run = m_use;
            const float u = m_run == -INFINITY ? 0.0f : m_run;
            // the head's weights for the tile's keys: BF16 pairs over the first columns of the score buffer they came from
            uint32_t packed[kKeys / 2];
            float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            #pragma unroll
            for (int i = 0; i < kKeys / 2; ++i) {
                // (an absent key's score is -inf: its weight is exp2(-inf) = 0)
                const float p0 = fast_exp2(fmaf(s[2 * i], g.scale_log2, -u)), p1 = fast_exp2(fmaf(s[2 * i + 1], g.scale_log2, -u));
                packed[i] = pack_bf16x2(p0, p1);
                // (the denominator sums what the product will use: the rounded weights)
                sums[i & 3] += __uint_as_float(packed[i] << 16) + __uint_as_float(packed[i] & 0xffff0000u);
            }
            l_run += (sums[0] + sums[1]) + (sums[2] + sums[3]);
            const uint32_t sb = j % kScoreBuffers;
            if (kKeys == 64) tmem_st32(tmem + lane_base + kSCol + sb * kSStride, packed);
            else if (kKeys == 48) { tmem_st16(tmem + lane_base + kSCol + sb * kSStride, packed); tmem_st8(tmem + lane_base + kSCol + sb * kSStride + 16, packed + 16); }
            else tmem_st16(tmem + lane_base + kSCol + sb * kSStride, packed);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kPFull + sb]);
        }
#if defined(SDX_TRACE)
        const long long loop_ended = clock64();
        if (head == 0 && !sender) { trace[7] = loop_ended - started; trace[3] = prologue_cycles; SDX_TRACE_OUT(4); SDX_TRACE_OUT(6); SDX_TRACE_OUT(7); SDX_TRACE_OUT(3); }
#endif
        // ---- epilogue: the head's row of O, this half's columns ----
        if (!sender && alive && wait(kSFree + (tiles - 1) % kScoreBuffers, ((tiles - 1) / kScoreBuffers) & 1)) {   // (the last product, so every product, is done)
            tc_fence_after();
            // 32 heads x 32 columns at a time through a padded tile of the (idle) ring, so that a store instruction writes 128 consecutive
            // bytes of one head's partial instead of 8 bytes of each of 32 heads'
            float* tile = reinterpret_cast<float*>(ring) + warp * (32 * 33);
            #pragma unroll 1
            for (int c0 = 0; c0 < dims; c0 += 32) {
                float o[32];
                tmem_ld32(tmem + lane_base + c0, o);
                __syncwarp();
                #pragma unroll
                for (int i = 0; i < 32; ++i) tile[lane * 33 + i] = o[i];
                __syncwarp();
                #pragma unroll 8
                for (int h = 0; h < 32; ++h)
                    if (32 * warp + h < nheads) partial[(32 * warp + h) * head_stride + d0 + c0 + lane] = tile[h * 33 + lane];
            }
            if (half == 0 && head < nheads) {
                partial[head * head_stride + DIM] = m_run * 0.6931471805599453f;   // (the partials' maxima are natural logarithms)
                partial[head * head_stride + DIM + 1] = l_run;
            }
        }
#if defined(SDX_TRACE)
        if (head == 0 && !sender) { trace[2] = clock64() - loop_ended; SDX_TRACE_OUT(2); }
#endif
    } else if (warp == kScoreWarp) {
        // ================= the score products' issuer =================
        if (lane == 0) {
            const uint32_t q_low = desc_low(smem_u32(q_hi), 16), qlo_low = desc_low(smem_u32(q_lo), 16);
            const uint32_t idesc_s = instr_desc(kHeads, kKeys, false);
            const int lo_first = blocks - lo_blocks;
            long long trace[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long started = clock64();
            (void)started;
            for (uint32_t i = 0; i < tiles; ++i) {
                const uint32_t b = i % kScoreBuffers, slot = i % kSlots, tile = desc_low(smem_u32(ring) + slot * tile_bytes, 16), s_tmem = tmem + kSCol + b * kSStride;
                long long since = clock64();
                (void)since;
                if (i >= uint32_t(kScoreBuffers) && !wait(kSFree + b, (i / kScoreBuffers - 1) & 1)) break;
                since = clock64();
                if (!wait(kFull + slot, (i / kSlots) & 1)) break;
                SDX_TRACE_ADD(1, since);
                fence_proxy_async();   // (the copies wrote through the generic proxy)
                tc_fence_after();
                for (int blk = 0; blk < blocks; ++blk)
                    #pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma(s_tmem, desc_of(q_low + ((blk * (kHeads * 128) + kk * 32) >> 4)), desc_of(tile + ((blk * (kKeys * 128) + kk * 32) >> 4)),
                             idesc_s, blk > 0 || kk > 0);
                for (int lb = 0; lb < lo_blocks; ++lb)
                    #pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma(s_tmem, desc_of(qlo_low + ((lb * (kHeads * 128) + kk * 32) >> 4)),
                             desc_of(tile + (((lo_first + lb) * (kKeys * 128) + kk * 32) >> 4)), idesc_s, true);
                umma_commit(&bars[kSFull + b]);
            }
#if defined(SDX_TRACE)
            trace[0] = clock64() - started; trace[5] = tiles;
            SDX_TRACE_OUT(0); SDX_TRACE_OUT(1); SDX_TRACE_OUT(5);
#endif
        }
    } else if (warp == kValueWarp) {
        // ================= the output products' issuer =================
        if (lane == 0) {
            const uint32_t idesc_256 = instr_desc(kHeads, 256, true), idesc_64 = instr_desc(kHeads, 64, true);
            long long trace[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (uint32_t j = 0; j < tiles; ++j) {
                const uint32_t b = j % kScoreBuffers, slot = j % kSlots, tile = desc_low(smem_u32(ring) + slot * tile_bytes, kKeys * 128), p_tmem = tmem + kSCol + b * kSStride;
                const long long since = clock64();
                (void)since;
                if (!wait(kPFull + b, (j / kScoreBuffers) & 1)) break;
                SDX_TRACE_ADD(2, since);
                tc_fence_after();
                #pragma unroll
                for (int ks = 0; ks < kKeys / 16; ++ks) {
                    umma_a_tmem(tmem, p_tmem + ks * 8, desc_of(tile + ((ks * (16 * 128)) >> 4)), idesc_256, j > 0 || ks > 0);
                    if (blocks > 4)
                        umma_a_tmem(tmem + 256, p_tmem + ks * 8, desc_of(tile + ((4 * (kKeys * 128) + ks * (16 * 128)) >> 4)), idesc_64, j > 0 || ks > 0);
                }
                umma_commit(&bars[kFree + slot]);
                umma_commit(&bars[kSFree + b]);   // the weights sat in the score buffer: free once the product has read them
            }
        }
    } else {
        // ================= the copy warps: 16-byte copies of this half's columns into the swizzled tile =================
        const uint8_t* halves = reinterpret_cast<const uint8_t*>(state_halves(a.compressed)) + size_t(d0) * 2;
        const int ctid = tid - 32 * kCopyWarp0, chunks = dims / 8;   // 16-byte pieces of a half row
        const size_t sel_begin = size_t(tile_begin) * kKeys;
        auto index_at = [&](uint32_t t, int part) -> int32_t {
            const size_t index = sel_begin + size_t(t) * kKeys + part * 32 + lane;
            int32_t at = t < tiles && part * 32 + lane < kKeys && index < a.selections ? chosen[index] : -1;
            if (at >= 0 && size_t(at) >= a.compressed_rows) { atomicExch(g.status, 2); at = -1; }   // (a row number past the cache: taken as absent, reported)
            return at;
        };
        int32_t at0 = index_at(0, 0), at1 = index_at(0, 1);
        for (uint32_t t = 0; t < tiles; ++t) {
            const uint32_t slot = t % kSlots;
            const int32_t next0 = index_at(t + 1, 0), next1 = index_at(t + 1, 1);   // (the list comes from HBM like the rows: asked for a tile ahead)
            if (t >= uint32_t(kSlots) && !wait(kFree + slot, (t / kSlots - 1) & 1)) break;
            const unsigned long long live = (unsigned long long)__ballot_sync(0xffffffffu, at0 >= 0) | ((unsigned long long)__ballot_sync(0xffffffffu, at1 >= 0) << 32);
            if (ctid == 0) masks[slot] = live;
            const uint32_t tile = smem_u32(ring) + slot * tile_bytes;
            const int pieces = kKeys * chunks;
            #pragma unroll 4
            for (int piece = ctid; piece < pieces; piece += 32 * kCopyWarps) {
                const int key = piece / chunks, chunk = piece % chunks;
                const int32_t from_lo = __shfl_sync(0xffffffffu, at0, key % 32), from_hi = __shfl_sync(0xffffffffu, at1, key % 32);
                const int32_t from = key < 32 ? from_lo : from_hi;
                const uint32_t dst = tile + (chunk / 8) * (kKeys * 128) + key * 128 + (((chunk % 8) ^ (key % 8)) * 16);
                cp_async16(dst, halves + (from >= 0 ? size_t(from) * DIM * 2 + chunk * 16 : 0), from >= 0 ? 16u : 0u);
            }
            cp_async_arrive(&bars[kFull + slot]);
            at0 = next0; at1 = next1;
        }
        asm volatile("cp.async.wait_all;" ::: "memory");   // (nothing in flight into this CTA's shared memory when it exits)
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
    }
    cluster_arrive(); cluster_wait();   // (nobody leaves while its partner may still write into its exchange buffers)
}

}  // namespace tc2

void sparse_window_partial(Device& d, const SparseArgs& a, const float* q, size_t rows, size_t pairs, const double2* forward, float* rotated,
                           float* partial, size_t parts, cudaStream_t stream = nullptr);
void sparse_combine(Device& d, const float* partial, size_t parts, size_t rows, size_t heads, size_t dim, const float* sinks, size_t pairs,
                    const double2* inverse, float* out);

template<int DIM>
static void launch_tc2(Device& d, const tc2::Args& args, size_t rows, size_t head_tiles) {
    using S = tc2::Shape<DIM>;
    static bool configured[64] = {};
    if (!configured[d.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(tc2::sparse_tc2_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::kSmem)));
        configured[d.ordinal & 63] = true;
    }
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(unsigned(args.splits * head_tiles), 2, unsigned(rows));
    config.blockDim = dim3(tc2::kThreads);
    config.dynamicSmemBytes = S::kSmem;
    config.stream = d.stream;
    cudaLaunchAttribute cluster{};
    cluster.id = cudaLaunchAttributeClusterDimension;
    cluster.val.clusterDim.x = 1; cluster.val.clusterDim.y = 2; cluster.val.clusterDim.z = 1;
    config.attrs = &cluster; config.numAttrs = 1;
    SDB_CHECK(cudaLaunchKernelEx(&config, tc2::sparse_tc2_kernel<DIM>, args));
    ++d.launches;
}

// The pair kernel for the shapes sparse_tc_supported accepts (128 heads and more).
void sparse_tc2_launch(Device& d, const SparseArgs& a, const float* q, const float* sinks, size_t rows, size_t pairs, const double2* forward,
                       const double2* inverse, float* out) {
    const size_t head_tiles = (a.heads + tc2::kHeads - 1) / tc2::kHeads;
    const size_t all_tiles = (a.selections + tc2::kKeys - 1) / tc2::kKeys;
    // one wave of pairs where the call is small: as many splits of a row's keys as fill half the SMs, each of at least four tiles
    size_t splits = std::max<size_t>(1, size_t(d.sms) / 2 / std::max<size_t>(1, rows * head_tiles));
    splits = std::min<size_t>({splits, std::max<size_t>(1, all_tiles / 4), size_t(32)});
    const size_t parts = splits + 1;   // part 0: the window rows (FP32 kernel)
    const size_t partial_bytes = checked_product({rows, a.heads, parts, a.dim + 2, 4});
    const size_t q_bytes = pairs ? (checked_product({rows, a.heads, a.dim, 4}) + 255) / 256 * 256 : 0;
    size_t trace_bytes = 0;
#if defined(SDX_TRACE)
    const size_t trace_at = (q_bytes + partial_bytes + 255) / 256 * 256, trace_ctas = splits * head_tiles * 2 * rows;
    trace_bytes = 256 + trace_ctas * 64;   // the counters follow the partials in the workspace
#endif
    auto* work = static_cast<uint8_t*>(ensure(d, d.partial, d.partial_bytes, q_bytes + partial_bytes + trace_bytes));
    auto* partial = reinterpret_cast<float*>(work + q_bytes);
    // the window rows' partial (slot 0 of every head's partials) has nothing to do with the selected rows' (slots 1 ..): it runs on the
    // handle's side stream beside the pair kernel (whose grid leaves SMs idle when a call is small), and the combine waits for both
    sparse_window_partial(d, a, q, rows, pairs, forward, reinterpret_cast<float*>(work), partial, parts, side_stream_begin(d));
    tc2::Args args{};
#if defined(SDX_TRACE)
    args.trace = reinterpret_cast<long long*>(work + trace_at);
    SDB_CHECK(cudaMemsetAsync(args.trace, 0, trace_ctas * 64, d.stream));
    d.trace = args.trace; d.trace_ctas = trace_ctas;
#endif
    args.a = a; args.q = q; args.pairs = pairs; args.forward = forward;
    args.scale_log2 = a.scale * 1.4426950408889634f;
    args.status = status_word(d);
    args.partial = partial;
    args.parts = uint32_t(parts); args.splits = uint32_t(splits);
    if (a.dim == 576) launch_tc2<576>(d, args, rows, head_tiles); else launch_tc2<512>(d, args, rows, head_tiles);
    SDB_CHECK(cudaGetLastError());
    side_stream_end(d);
    sparse_combine(d, partial, parts, rows, a.heads, a.dim, sinks, pairs, inverse, out);
}

}  // namespace sdb
