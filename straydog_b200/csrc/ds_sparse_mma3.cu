// Tensor-core kernel of the latent sparse attention (sd_op_sparse_attention) for sm_100a, third form:
// sixteen compute warps and four copy warps a CTA; scores split by KEYS and the weighted sum split by
// COLUMNS, so that a score is exponentiated once (not once per warp) and a warp issues about a third of
// the instructions per key of the second form; the gather is taken off the compute warps altogether.
// Measured on the second form and on a first draft of this one: a compute warp that issues its own
// 16-byte cp.async copies sits in that issue for a third of a tile's time, and the index list has to be
// read a whole tile ahead because it comes from HBM like the rows.
//
// What it replaces: op_attention_scores_kernel + op_attention_output_kernel + combine
// (gpu/ops.hpp:1329-1434, 1542-1677). A CTA holds 16 heads of one query row and streams a split of that
// row's selected compressed rows once; the queries are rotated and split into BF16 parts by the CTA itself
// (gpu/ops.hpp:1318-1327, 1366-1377), and the CTAs of a (row, head tile) are a thread-block cluster that merges its splits through distributed
// shared memory, so one launch makes a call and no partial goes to HBM.
//
// CTA = 640 threads. Warps 0-15 are two groups of eight; the groups take alternate 32-key tiles of a
// four-slot ring (group g owns slots g and g + 2), each with its own softmax state and its own partial.
// Warps 16 + g and 18 + g are group g's copy warps (16 keys of a tile each; one warp alone needs two thirds of a
// tile's time to issue 32 copies): a lane per key, one bulk copy (TMA engine) of a whole row into a
// padded shared-memory row, completion counted on the slot's full barrier; absent rows are zero-filled
// by the lane itself. A slot returns through an empty barrier on which the group's warps arrive as they
// leave the tile. Per tile a group runs three phases:
//   scores   warp (kh, kq): keys 16 kh .. 16 kh + 15 of the tile, quarter kq of the contraction; Q and K
//            fragments by ldmatrix, two accumulator pairs so that consecutive MMAs do not depend on each
//            other. The four partial sums of a score go to a shared slab.                    [barrier A]
//   softmax  warp w: heads 2w and 2w + 1, a lane per key pair: the four parts are added in part order,
//            scaled and masked; running maximum and denominator of the head live in these lanes; the
//            weights are rounded to BF16 once and stored with the rescale factor of the head. [barrier B]
//   output   warp w: columns w * dim / 8 ..: O = O * factor + P V, P by ldmatrix from shared memory,
//            V by transposing ldmatrix from the same rows that served as keys (keys are the values).
// Exactness: as in the other forms, F32 operands are split into BF16 high and low parts and both are
// multiplied, so BF16-tagged and F32 rows of equal values give equal bits (tests/ds_state_bf16_gpu.rs:99-102).
// Every wait is bounded; a wait that gives up is voted through barrier A so that a group leaves together.
#include "ds_sparse.cuh"

#include <algorithm>
#include <type_traits>

namespace sdb {
namespace v3 {

constexpr int kT = 32;            // keys a tile
constexpr int kStages = 4;        // tiles in the ring
constexpr int kGroups = 2, kGroupWarps = 8, kGroupThreads = 32 * kGroupWarps;
constexpr int kScalarWindow = 4;   // window rows up to which the window is taken by FP32 arithmetic, a row at a time
constexpr int kCopyWarps = 2;     // copy warps a group, 16 rows of a tile each
constexpr int kComputeThreads = kGroups * kGroupThreads, kThreads = kComputeThreads + 32 * kGroups * kCopyWarps;

template<int DIM> struct Shape {
    static constexpr int kRow = (DIM + 8) * 2;          // padded shared-memory row, bytes
    static constexpr int kPlane = kT * kRow;
    static constexpr int kKS = DIM / 64;                // k-steps (16 columns) of one contraction quarter
    static constexpr int kCols = DIM / 8;               // output columns a warp owns
    static constexpr int kNT = kCols / 8;               // its n-tiles (8 columns)
    static constexpr int kSlabRow = kT + 8;             // floats
    static constexpr int kSlab = 16 * kSlabRow;         // one contraction quarter's partial scores
    static constexpr int kPRow = (kT + 8) * 2;          // bytes of a row of weights
    static constexpr int kOffQhi = kStages * kPlane;
    static constexpr int kOffQlo = kOffQhi + 16 * kRow;
    static constexpr int kOffSlabs = kOffQlo + 16 * kRow;
    static constexpr int kOffP = kOffSlabs + kGroups * 4 * kSlab * 4;
    static constexpr int kOffFactors = kOffP + kGroups * 16 * kPRow;
    static constexpr int kOffBars = kOffFactors + kGroups * 16 * 4;         // full[kStages], empty[kStages]
    static constexpr int kOffPtrs = kOffBars + 2 * kStages * 8;             // F32 phase: a tile's key pointers
    static constexpr int kOffMisc = kOffPtrs + kT * 8;                      // abort flag, live mask of an F32 tile
    static constexpr size_t kSmem = kOffMisc + 16;
    static_assert(kSmem <= 232448, "shared memory of one CTA");
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(address));
}
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ void group_barrier(int id) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(kGroupThreads) : "memory");
}
// a group barrier that also ORs a flag over the group
__device__ __forceinline__ bool group_barrier_or(int id, bool flag) {
    uint32_t any;
    asm volatile("{ .reg .pred p, q; setp.ne.u32 q, %2, 0; bar.red.or.pred p, %1, %3, q; selp.u32 %0, 1, 0, p; }"
                 : "=r"(any) : "r"(id), "r"(uint32_t(flag)), "n"(kGroupThreads) : "memory");
    return any != 0;
}

// thread-block cluster: the CTAs of one (row, head tile) are a cluster, a CTA per split of the selected keys
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_address(uint32_t local, uint32_t rank) {   // the same shared-memory offset in CTA `rank`
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ float2 cluster_load2(uint32_t address) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(address) : "memory");
    return v;
}

template<int DIM>
__global__ void __launch_bounds__(kThreads, 1) sparse_mma3_kernel(
        const SparseArgs a, const float* __restrict__ q, size_t pairs, const double2* __restrict__ forward,
        float scale_log2, int* __restrict__ status, const float* __restrict__ sinks, const double2* __restrict__ inverse, float* __restrict__ out,
        const GatherTargets gather) {
    using S = Shape<DIM>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* planes = smem;
    uint8_t* q_hi = smem + S::kOffQhi;
    uint8_t* q_lo = smem + S::kOffQlo;
    float* slabs = reinterpret_cast<float*>(smem + S::kOffSlabs);
    uint8_t* weights = smem + S::kOffP;
    float* factors = reinterpret_cast<float*>(smem + S::kOffFactors);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::kOffBars);
    uint64_t* empty = full + kStages;
    const float** key_ptrs = reinterpret_cast<const float**>(smem + S::kOffPtrs);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::kOffMisc);
    uint32_t* f32_live = reinterpret_cast<uint32_t*>(smem + S::kOffMisc + 4);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane / 4, t = lane % 4;
    const bool copier = warp >= kGroups * kGroupWarps;
    const int group = copier ? (warp - kGroups * kGroupWarps) % kGroups : warp / kGroupWarps, gw = warp % kGroupWarps;
    const int copy_half = (warp - kGroups * kGroupWarps) / kGroups;   // of a copy warp: which 16 rows of a tile
    const int kh = gw % 2, kq = gw / 2;                        // scores: key half of the tile, contraction quarter
    const size_t split = blockIdx.x, splits = gridDim.x, row = blockIdx.z, head0 = size_t(blockIdx.y) * 16;
    // (the compute threads ask for their share of the queries before anything else: the load's latency covers the set-up)
    constexpr int kEach = 16 * (DIM / 2) / kComputeThreads;   // column pairs a thread prepares
    static_assert(16 * (DIM / 2) % kComputeThreads == 0, "the query rows divide evenly over the threads");
    float2 loaded[kEach];
    if (!copier) {
        #pragma unroll
        for (int it = 0; it < kEach; ++it) {
            const int i = threadIdx.x + it * kComputeThreads, head = i / (DIM / 2), col = 2 * (i % (DIM / 2));
            loaded[it] = make_float2(0.0f, 0.0f);
            if (head0 + head < a.heads) {
                const float* src = q + (row * a.heads + head0 + head) * DIM + col;   // (only known to be 4-byte aligned)
                loaded[it] = make_float2(src[0], src[1]);
            }
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 32); mbar_init(&empty[s], kGroupWarps); }
        *abort_flag = 0;
    }
    fence_barrier_init();
    __syncthreads();

    // a bounded wait that also ends when another warp has given up
    auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
        if (mbar_try_wait(bar, parity)) return true;
        const uint64_t start = global_timer_ns();
        for (;;) {
            #pragma unroll 1
            for (int spin = 0; spin < 32; ++spin)
                if (mbar_try_wait(bar, parity)) return true;
            if (*abort_flag) return false;
            if (global_timer_ns() - start > 2000000000ull) { *abort_flag = 1; atomicExch(status, 1); return false; }
        }
    };

    const KeyList list = key_list(a, row);
    const bool rows_bf16 = state_is_bf16(a.compressed);
    // The selected rows are dealt in whole tiles. Split 0 also has the window rows, an F32 tile of which costs one of its groups
    // about three streamed tiles (read, converted on the spot, both parts multiplied): it takes that many fewer streamed tiles.
    // (a window of up to kScalarWindow rows goes through FP32 arithmetic instead: next to free. When the call's window is that
    //  short, the dealing does not wait for the row's position to come from HBM: the copy warps start a round trip earlier.)
    const bool short_window = a.window <= size_t(kScalarWindow);
    const uint32_t all_tiles = uint32_t((a.selections + kT - 1) / kT);
    const uint32_t window_tiles = short_window ? 0u : uint32_t((list.raw_count + kT - 1) / kT);
    const bool scalar_window = short_window || (list.raw_count > 0 && list.raw_count <= size_t(kScalarWindow));
    const uint32_t window_cost = scalar_window ? 0u : 3 * window_tiles;   // (the same for both row formats, so that they are dealt alike)
    const uint32_t per_split = (all_tiles + window_cost + uint32_t(splits) - 1) / uint32_t(splits);
    const uint32_t first_share = per_split > window_cost ? per_split - window_cost : (splits == 1 ? all_tiles : 0u);
    const uint32_t tile_begin = split == 0 ? 0u : min(all_tiles, first_share + (uint32_t(split) - 1) * per_split);
    const uint32_t tile_end = split + 1 == splits ? all_tiles : min(all_tiles, first_share + uint32_t(split) * per_split);
    const size_t sel_begin = min(a.selections, size_t(tile_begin) * kT), sel_end = min(a.selections, size_t(tile_end) * kT);
    const uint32_t stream_tiles = rows_bf16 ? tile_end - tile_begin : 0u;
    // F32 keys. BF16 rows: only split 0's window rows, which its group 0 converts and consumes by itself in its own two slots
    // while group 1 already streams. Untagged F32 rows: every key, tile by tile, by the whole CTA in the last two slots.
    const bool window_here = rows_bf16 && split == 0 && window_tiles > 0 && !scalar_window;
    const size_t f32_begin = rows_bf16 ? 0 : (split == 0 && !scalar_window ? 0 : list.raw_count + sel_begin);
    const size_t f32_end = rows_bf16 ? 0 : list.raw_count + sel_end;
    const uint32_t f32_tiles = [&] {
        uint32_t n = 0;
        for (size_t first = f32_begin; first < f32_end; ++n) first += min(size_t(kT), (first < list.raw_count ? list.raw_count : f32_end) - first);
        return n;
    }();

    const int32_t* chosen = a.selected + row * a.selections;
    auto index_at = [&](uint32_t tile, int key) -> int32_t {   // row number of key `key` of `tile`, -1: none
        const size_t index = sel_begin + size_t(tile) * kT + key;
        return tile < stream_tiles && index < sel_end ? chosen[index] : -1;
    };

    // =========================== the copy warps of a group ===========================
    if (copier) {
        const uint8_t* halves = reinterpret_cast<const uint8_t*>(state_halves(a.compressed));
        const bool active = lane < kT / kCopyWarps;
        const int key = copy_half * (kT / kCopyWarps) + lane;
        auto fill = [&](uint32_t tile, int32_t at) {
            if (!active) return;
            if (at >= 0 && size_t(at) >= a.compressed_rows) { atomicExch(status, 2); at = -1; }   // (a row number past the cache: taken as absent, reported)
            const int slot = int(tile % kStages);
            uint8_t* dst = planes + size_t(slot) * S::kPlane + size_t(key) * S::kRow;
            if (at >= 0) {
                mbar_expect_tx(&full[slot], DIM * 2);
                bulk_g2s(dst, halves + size_t(at) * DIM * 2, DIM * 2, &full[slot]);
            } else {   // an absent row: zeros, so that a zero weight never meets stale bits
                #pragma unroll 4
                for (int c = 0; c < DIM * 2 / 16; ++c) *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(0, 0, 0, 0);
                fence_proxy_async();   // (a later bulk copy lands on the same bytes)
                mbar_arrive(&full[slot]);
            }
        };
        // indices are read two tiles before they are used: the list comes from HBM like the rows
        int32_t at = active ? index_at(uint32_t(group), key) : -1, next = active ? index_at(uint32_t(group) + kGroups, key) : -1;
        for (uint32_t i = 0; i < f32_tiles; ++i) { __syncthreads(); __syncthreads(); __syncthreads(); }   // (untagged rows: no stream)
        // (group 0's slots first hold the window tiles' planes where there are any: they are released like a streamed tile)
        const uint32_t shift = window_here && group == 0 ? 1u : 0u;
        for (uint32_t tile = uint32_t(group); tile < stream_tiles; tile += kGroups) {
            const uint32_t use = tile / kStages + shift;
            if (use >= 1 && !wait(&empty[tile % kStages], (use - 1) & 1)) break;
            fill(tile, at);
            at = next;
            next = active ? index_at(tile + 2 * kGroups, key) : -1;
        }
        // (the merge at the end is the compute warps' work; every thread of the cluster meets at its two barriers)
        cluster_arrive(); cluster_wait();
        cluster_arrive(); cluster_wait();
        return;
    }

    // =========================== the compute warps ===========================
    // ---- the CTA's 16 query rows: rotated (double), split into BF16 high and low parts ----
    bool any_lo = false;
    {
        const size_t plain = DIM - 2 * pairs;
        #pragma unroll
        for (int it = 0; it < kEach; ++it) {
            const int i = threadIdx.x + it * kComputeThreads, head = i / (DIM / 2), col = 2 * (i % (DIM / 2));
            float2 v = loaded[it];
            if (size_t(col) >= plain && head0 + head < a.heads) {
                const double2 turn = forward[row * pairs + (col - plain) / 2];
                const double x = v.x, y = v.y;
                v = make_float2(float(x * turn.x - y * turn.y), float(x * turn.y + y * turn.x));
            }
            const __nv_bfloat16 h0 = __float2bfloat16_rn(v.x), h1 = __float2bfloat16_rn(v.y);
            const float r0 = v.x - __bfloat162float(h0), r1 = v.y - __bfloat162float(h1);
            *reinterpret_cast<__nv_bfloat162*>(q_hi + head * S::kRow + col * 2) = __halves2bfloat162(h0, h1);
            *reinterpret_cast<__nv_bfloat162*>(q_lo + head * S::kRow + col * 2) = __halves2bfloat162(__float2bfloat16_rn(r0), __float2bfloat16_rn(r1));
            if (size_t(col) < plain && (r0 != 0.0f || r1 != 0.0f)) any_lo = true;
        }
    }
    // (low parts matter from the first rotated column on, or everywhere when some plain column is not a BF16 value)
    uint32_t some_lo;
    asm volatile("{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.or.pred p, 4, %2, q; selp.u32 %0, 1, 0, p; }"
                 : "=r"(some_lo) : "r"(uint32_t(any_lo)), "n"(kComputeThreads) : "memory");   // (the compute threads alone: the copy warps are busy)
    const int lo_from = some_lo ? 0 : int((DIM - 2 * pairs) / 16);

    float o[S::kNT][4];
    #pragma unroll
    for (int n = 0; n < S::kNT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    float m = -INFINITY, l = 0.0f;   // of head 2 gw + lane / 16 (the softmax phase's lanes)

    // ---- lane constants of the three phases ----
    const int frag_row = 8 * (lane / 16) + lane % 8, frag_half = (lane / 8) % 2;
    const uint32_t k_lane = uint32_t((16 * kh + frag_row) * S::kRow + (16 * kq * S::kKS + 8 * frag_half) * 2);
    const int a_row = lane % 8 + 8 * ((lane / 8) % 2), a_col = 8 * (lane / 16);     // A operand by ldmatrix: queries and weights
    const uint32_t qhi_lane = smem_u32(q_hi) + uint32_t(a_row * S::kRow + (16 * kq * S::kKS + a_col) * 2);
    const uint32_t qlo_lane = smem_u32(q_lo) + uint32_t(a_row * S::kRow + (16 * kq * S::kKS + a_col) * 2);
    const uint32_t p_lane = smem_u32(weights) + uint32_t(group * 16 * S::kPRow + a_row * S::kPRow + a_col * 2);
    const int v_key = 8 * ((lane / 8) % 2) + lane % 8, v_dim = 8 * (lane / 16);
    const uint32_t v_lane = uint32_t(v_key * S::kRow + (gw * S::kCols + v_dim) * 2);
    float* slab_out = slabs + (group * 4 + kq) * S::kSlab + g * S::kSlabRow + 16 * kh + 2 * t;
    const int soft_head = 2 * gw + lane / 16, soft_key = 2 * (lane % 16);
    const float* slab_in = slabs + group * 4 * S::kSlab + soft_head * S::kSlabRow + soft_key;
    uint32_t* p_out = reinterpret_cast<uint32_t*>(weights + group * 16 * S::kPRow + soft_head * S::kPRow + soft_key * 2);
    float* group_factors = factors + group * 16;

    // ---- one tile for one group. has_lo: the tile has a low-part plane (F32 keys). failed: this warp's wait gave up.
    //      Returns false when the group gives up. ----
    auto compute = [&](uint32_t hi_plane, uint32_t lo_plane, uint32_t live, bool failed, auto lo_tag) -> bool {
        constexpr bool has_lo = decltype(lo_tag)::value;
        float s[2][2][4];   // [k-step parity][n-tile]: consecutive k-steps feed different accumulators
        #pragma unroll
        for (int i = 0; i < 2; ++i)
            #pragma unroll
            for (int j = 0; j < 2; ++j) { s[i][j][0] = s[i][j][1] = s[i][j][2] = s[i][j][3] = 0.0f; }
        uint32_t qa[2][4], kb[2][4];
        ldmatrix_x4(qa[0], qhi_lane);
        ldmatrix_x4(kb[0], hi_plane + k_lane);
        #pragma unroll
        for (int ks = 0; ks < S::kKS; ++ks) {
            const int cur = ks & 1, nxt = cur ^ 1;
            if (ks + 1 < S::kKS) {   // (the next step's fragments are on their way while this step multiplies)
                ldmatrix_x4(qa[nxt], qhi_lane + 32 * (ks + 1));
                ldmatrix_x4(kb[nxt], hi_plane + k_lane + 32 * (ks + 1));
            }
            mma_bf16(s[cur][0], qa[cur], kb[cur][0], kb[cur][1]);
            mma_bf16(s[cur][1], qa[cur], kb[cur][2], kb[cur][3]);
            if (kq * S::kKS + ks >= lo_from) {
                uint32_t al[4];
                ldmatrix_x4(al, qlo_lane + 32 * ks);
                mma_bf16(s[cur][0], al, kb[cur][0], kb[cur][1]);
                mma_bf16(s[cur][1], al, kb[cur][2], kb[cur][3]);
            }
            if constexpr (has_lo) {
                uint32_t bl[4];
                ldmatrix_x4(bl, lo_plane + k_lane + 32 * ks);
                mma_bf16(s[cur][0], qa[cur], bl[0], bl[1]);
                mma_bf16(s[cur][1], qa[cur], bl[2], bl[3]);
            }
        }
        #pragma unroll
        for (int j = 0; j < 2; ++j) {
            *reinterpret_cast<float2*>(slab_out + 8 * j) = make_float2(s[0][j][0] + s[1][j][0], s[0][j][1] + s[1][j][1]);
            *reinterpret_cast<float2*>(slab_out + 8 * S::kSlabRow + 8 * j) = make_float2(s[0][j][2] + s[1][j][2], s[0][j][3] + s[1][j][3]);
        }
        if (group_barrier_or(1 + group, failed)) return false;                         // barrier A
        {   // softmax of heads 2 gw, 2 gw + 1: a lane per key pair
            float2 sum = make_float2(0.0f, 0.0f);
            #pragma unroll
            for (int part = 0; part < 4; ++part) {
                const float2 x = *reinterpret_cast<const float2*>(slab_in + part * S::kSlab);
                sum.x += x.x; sum.y += x.y;
            }
            const float s0 = (live >> soft_key) & 1u ? sum.x * scale_log2 : -INFINITY;
            const float s1 = (live >> (soft_key + 1)) & 1u ? sum.y * scale_log2 : -INFINITY;
            float top = fmaxf(s0, s1);
            #pragma unroll
            for (int offset = 1; offset < 16; offset *= 2) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
            const float next = fmaxf(m, top);
            const float factor = m == next ? 1.0f : (m == -INFINITY ? 0.0f : fast_exp2(m - next));
            const float used = next == -INFINITY ? 0.0f : next;   // (no live key yet: weights 0, not NaN)
            const uint32_t p = pack_bf16x2(fast_exp2(s0 - used), fast_exp2(s1 - used));
            float total = bf16_lo(p) + bf16_hi(p);
            #pragma unroll
            for (int offset = 1; offset < 16; offset *= 2) total += __shfl_xor_sync(0xffffffffu, total, offset);
            l = l * factor + total;
            m = next;
            *p_out = p;
            if (lane % 16 == 0) group_factors[soft_head] = factor;
        }
        group_barrier(1 + group);                                                       // barrier B
        {   // O = O * factor + P V over this warp's columns
            const float f0 = group_factors[g], f1 = group_factors[g + 8];
            if (__any_sync(0xffffffffu, f0 != 1.0f || f1 != 1.0f)) {
                #pragma unroll
                for (int n = 0; n < S::kNT; ++n) { o[n][0] *= f0; o[n][1] *= f0; o[n][2] *= f1; o[n][3] *= f1; }
            }
            #pragma unroll
            for (int kk = 0; kk < kT / 16; ++kk) {
                uint32_t pa[4], vb[S::kNT / 2][4], tail0 = 0, tail1 = 0;
                ldmatrix_x4(pa, p_lane + 32 * kk);
                #pragma unroll
                for (int np = 0; np < S::kNT / 2; ++np) ldmatrix_x4_trans(vb[np], hi_plane + v_lane + uint32_t(16 * kk * S::kRow + 32 * np));
                if constexpr (S::kNT % 2 == 1) ldmatrix_x2_trans(tail0, tail1, hi_plane + v_lane + uint32_t(16 * kk * S::kRow + 32 * (S::kNT / 2)));
                #pragma unroll
                for (int np = 0; np < S::kNT / 2; ++np) {
                    mma_bf16(o[2 * np], pa, vb[np][0], vb[np][1]);
                    mma_bf16(o[2 * np + 1], pa, vb[np][2], vb[np][3]);
                }
                if constexpr (S::kNT % 2 == 1) mma_bf16(o[S::kNT - 1], pa, tail0, tail1);
                if constexpr (has_lo) {
                    #pragma unroll
                    for (int np = 0; np < S::kNT / 2; ++np) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, lo_plane + v_lane + uint32_t(16 * kk * S::kRow + 32 * np));
                        mma_bf16(o[2 * np], pa, b[0], b[1]);
                        mma_bf16(o[2 * np + 1], pa, b[2], b[3]);
                    }
                    if constexpr (S::kNT % 2 == 1) {
                        ldmatrix_x2_trans(tail0, tail1, lo_plane + v_lane + uint32_t(16 * kk * S::kRow + 32 * (S::kNT / 2)));
                        mma_bf16(o[S::kNT - 1], pa, tail0, tail1);
                    }
                }
            }
        }
        return true;
    };

    // ---- F32 keys: a tile at a time, converted into a high and a low plane ----
    auto key_in_range = [&](const float* key) -> bool {
        const size_t rings = (gridDim.z + a.span_rows - 1) / a.span_rows;
        if (state_is_bf16(key)) {
            const uint16_t* at = state_halves(key), *base = state_halves(a.compressed);
            return state_is_bf16(a.compressed) && at >= base && at + DIM <= base + a.compressed_rows * DIM;
        }
        if (key >= a.raw && key + DIM <= a.raw + rings * a.raw_rows * DIM) return true;
        return !state_is_bf16(a.compressed) && key >= a.compressed && key + DIM <= a.compressed + a.compressed_rows * DIM;
    };
    auto convert_tile = [&](size_t first, size_t count, int tid, int threads, uint8_t* hi, uint8_t* lo, auto&& barrier) {
        barrier();   // the planes' last readers are done
        if (tid < 32) {
            const float* key = size_t(lane) < count ? key_pointer(a, list, row, first + lane) : nullptr;
            key_ptrs[lane] = key;
            const uint32_t mask = __ballot_sync(0xffffffffu, key != nullptr);
            if (lane == 0) *f32_live = mask;
        }
        barrier();
        for (int i = tid; i < kT * (DIM / 2); i += threads) {
            const int r = i / (DIM / 2), c = 2 * (i % (DIM / 2));
            const float* key = key_ptrs[r];
            if (key && !key_in_range(key)) { atomicExch(status, 3); key = nullptr; }   // (never expected: a corrupted pointer table is reported, not followed)
            float2 v = make_float2(0.0f, 0.0f);
            if (key) v = state_is_bf16(key) ? make_float2(__uint_as_float(uint32_t(state_halves(key)[c]) << 16), __uint_as_float(uint32_t(state_halves(key)[c + 1]) << 16))
                                            : make_float2(key[c], key[c + 1]);
            const __nv_bfloat16 h0 = __float2bfloat16_rn(v.x), h1 = __float2bfloat16_rn(v.y);
            *reinterpret_cast<__nv_bfloat162*>(hi + r * S::kRow + c * 2) = __halves2bfloat162(h0, h1);
            *reinterpret_cast<__nv_bfloat162*>(lo + r * S::kRow + c * 2) =
                __halves2bfloat162(__float2bfloat16_rn(v.x - __bfloat162float(h0)), __float2bfloat16_rn(v.y - __bfloat162float(h1)));
        }
        fence_proxy_async();   // (bulk copies will land on these bytes later)
        barrier();
    };
    if (scalar_window && split == 0 && group == 0) {
        // A short window (a decode step's own row, a verify span's few rows): FP32 arithmetic, a row at a time, by group 0 before its
        // stream. A half warp forms the score of its head (the softmax phase's lanes), every warp adds the weighted row to its columns.
        float* all_staged = slabs;                                // [rows][DIM] in group 0's slab (idle until its first tile)
        static_assert(kScalarWindow * DIM <= 4 * S::kSlab, "the window's rows fit the group's slab");
        float* window_weights = reinterpret_cast<float*>(weights);   // [16] in group 0's weight rows (idle too)
        const int part = lane % 16;
        for (size_t j = 0; j < list.raw_count; ++j) {             // (every row is asked for before the first is used)
            const float* key = key_pointer(a, list, row, j);
            for (int c = threadIdx.x; c < DIM; c += kGroupThreads) all_staged[j * DIM + c] = key[c];
        }
        group_barrier(1);
        for (size_t j = 0; j < list.raw_count; ++j) {
            const float* staged = all_staged + j * DIM;
            float sum = 0.0f;
            {
                const uint8_t* hi = q_hi + soft_head * S::kRow, *lo = q_lo + soft_head * S::kRow;
                #pragma unroll 4
                for (int c = 2 * part; c < DIM; c += 32) {   // (column pairs interleaved over the 16 lanes: conflict-free)
                    const uint32_t h = *reinterpret_cast<const uint32_t*>(hi + c * 2), w = *reinterpret_cast<const uint32_t*>(lo + c * 2);
                    const float2 k = *reinterpret_cast<const float2*>(staged + c);
                    sum = fmaf(bf16_lo(h) + bf16_lo(w), k.x, sum);
                    sum = fmaf(bf16_hi(h) + bf16_hi(w), k.y, sum);
                }
            }
            #pragma unroll
            for (int offset = 1; offset < 16; offset *= 2) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
            const float score = sum * scale_log2;
            const float next = fmaxf(m, score);
            const float factor = m == next ? 1.0f : (m == -INFINITY ? 0.0f : fast_exp2(m - next));
            const float weight = fast_exp2(score - next);
            l = l * factor + weight;
            m = next;
            if (part == 0) { group_factors[soft_head] = factor; window_weights[soft_head] = weight; }
            group_barrier(1);
            {
                const float f0 = group_factors[g], f1 = group_factors[g + 8], w0 = window_weights[g], w1 = window_weights[g + 8];
                #pragma unroll
                for (int n = 0; n < S::kNT; ++n) {
                    const float2 k = *reinterpret_cast<const float2*>(staged + gw * S::kCols + 8 * n + 2 * t);
                    o[n][0] = fmaf(w0, k.x, o[n][0] * f0); o[n][1] = fmaf(w0, k.y, o[n][1] * f0);
                    o[n][2] = fmaf(w1, k.x, o[n][2] * f1); o[n][3] = fmaf(w1, k.y, o[n][3] * f1);
                }
            }
            group_barrier(1);   // the weights have been read
        }
    }
    if (window_here && group == 0) {
        // split 0 of BF16 rows: group 0 alone, in its own slots 0 and 2; its copy warp waits for the slots' first release
        uint8_t* hi = planes, *lo = planes + 2 * size_t(S::kPlane);
        for (size_t first = 0; first < list.raw_count; first += kT) {
            convert_tile(first, min(size_t(kT), list.raw_count - first), threadIdx.x, kGroupThreads, hi, lo, [&] { group_barrier(1); });
            compute(smem_u32(hi), smem_u32(lo), *f32_live, false, std::true_type{});
        }
        __syncwarp();
        if (lane == 0) { mbar_arrive(&empty[0]); mbar_arrive(&empty[2]); }
    }
    {
        // untagged F32 rows: the whole CTA, the last two slots (there is no stream). A tile never mixes window rows with selected
        // rows, and selected tiles alternate between the groups exactly as the stream's tiles do, so that F32 rows and BF16
        // rows of equal values are summed in the same order.
        uint8_t* hi = planes + size_t(kStages - 2) * S::kPlane, *lo = hi + S::kPlane;
        for (size_t first = f32_begin; first < f32_end;) {
            const size_t limit = first < list.raw_count ? list.raw_count : f32_end;
            const size_t count = min(size_t(kT), limit - first);
            convert_tile(first, count, threadIdx.x, kComputeThreads, hi, lo, [] { __syncthreads(); });
            const int consumer = first < list.raw_count ? 0 : int(((first - list.raw_count - sel_begin) / kT) % kGroups);
            if (group == consumer) compute(smem_u32(hi), smem_u32(lo), *f32_live, false, std::true_type{});
            first += count;
        }
    }

    // ---- BF16 selected rows: tile t is consumed by group t % 2 from slot t % kStages ----
    {
        int32_t live_at = index_at(uint32_t(group), lane);   // (read a tile ahead; the copy warp has had the same line a tile earlier still)
        for (uint32_t tile = uint32_t(group); tile < stream_tiles; tile += kGroups) {
            const int slot = int(tile % kStages);
            const uint32_t live = __ballot_sync(0xffffffffu, live_at >= 0);
            live_at = index_at(tile + kGroups, lane);
            const bool arrived = wait(&full[slot], (tile / kStages) & 1);
            const uint32_t plane = smem_u32(planes) + uint32_t(slot) * S::kPlane;
            if (!compute(plane, plane, live, !arrived, std::false_type{})) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
        }
    }

    // ---- the merge of the splits (gpu/ops.hpp:1561-1583, 1648-1677) runs inside the cluster: every group leaves its partial in
    //      its CTA's shared memory (the ring is idle by now), and after a cluster barrier CTA r merges columns r * dim / splits ..
    //      of all 16 heads, reading the other CTAs' partials through distributed shared memory: no partial goes to HBM. ----
    constexpr int kPartRow = DIM + 8;                          // floats (a part is exactly one slot of the ring)
    static_assert(16 * kPartRow * 4 <= S::kPlane, "a group's partial fits a slot");
    float* parts_area = reinterpret_cast<float*>(planes);      // [group][16 heads][kPartRow]
    float* part_stats = reinterpret_cast<float*>(weights);     // [group][16 heads][max, denominator], in the group's own weight rows
    group_barrier(1 + group);                                  // the group's last tile has been read by all of its warps
    {
        float* mine = parts_area + size_t(group) * 16 * kPartRow + gw * S::kCols + 2 * t;
        #pragma unroll
        for (int n = 0; n < S::kNT; ++n) {
            *reinterpret_cast<float2*>(mine + g * kPartRow + 8 * n) = make_float2(o[n][0], o[n][1]);
            *reinterpret_cast<float2*>(mine + (g + 8) * kPartRow + 8 * n) = make_float2(o[n][2], o[n][3]);
        }
        if (lane % 16 == 0) { part_stats[group * (16 * S::kPRow / 4) + soft_head * 2] = m; part_stats[group * (16 * S::kPRow / 4) + soft_head * 2 + 1] = l; }
    }
    cluster_arrive(); cluster_wait();
    const int parts = int(splits) * kGroups;                   // (at most 16: a lane each)
    float* merge_factors = slabs;                              // [16 heads][32]
    float* denominators = slabs + 16 * 32;
    // This CTA's columns (splits divides dim / 2). A thread merges up to kWide column pairs; the first eight parts of all of
    // them are asked for before the factors are formed, so that the two latencies overlap.
    const int cols = DIM / int(splits), col0 = int(split) * cols, half = cols / 2;
    constexpr int kWide = (16 * (DIM / 2) / 4 + kComputeThreads - 1) / kComputeThreads;   // pairs a thread at four or more splits
    auto pair_source = [&](int i, int& head_local, int& d) -> bool {
        head_local = i / half; d = col0 + 2 * (i % half);
        return i < 16 * half && head0 + head_local < a.heads;
    };
    auto load_parts = [&](int i, int part0, float2 (&x)[8]) {
        int head_local, d;
        const bool real = pair_source(i, head_local, d);
        const uint32_t from = smem_u32(parts_area + (real ? head_local * kPartRow + d : 0));
        #pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int part = part0 + k;
            x[k] = real && part < parts ? cluster_load2(cluster_address(from + uint32_t((part % kGroups) * 16 * kPartRow * 4), uint32_t(part / kGroups)))
                                        : make_float2(0.0f, 0.0f);
        }
    };
    float2 early[kWide][8];
    #pragma unroll
    for (int w = 0; w < kWide; ++w) load_parts(threadIdx.x + w * kComputeThreads, 0, early[w]);
    {   // warp = head, lane = part
        const size_t head = head0 + warp;
        float top_part = -INFINITY, sum_part = 0.0f, sink = -INFINITY;
        if (head < a.heads) sink = sinks[head] * 1.4426950408889634f;
        if (lane < parts) {
            const float2 stats = cluster_load2(cluster_address(smem_u32(part_stats + (lane % kGroups) * (16 * S::kPRow / 4) + warp * 2), uint32_t(lane / kGroups)));
            top_part = stats.x; sum_part = stats.y;
        }
        float top = fmaxf(top_part, sink);
        #pragma unroll
        for (int offset = 16; offset; offset /= 2) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
        const float factor = top_part == -INFINITY ? 0.0f : exp2f(top_part - top);
        float denominator = factor * sum_part;
        #pragma unroll
        for (int offset = 16; offset; offset /= 2) denominator += __shfl_xor_sync(0xffffffffu, denominator, offset);
        merge_factors[warp * 32 + lane] = factor;
        // (a sink of -inf adds 0; top is finite whenever any key or the sink is)
        if (lane == 0) denominators[warp] = denominator + exp2f(sink - top);
    }
    asm volatile("bar.sync 3, %0;" ::"n"(kComputeThreads) : "memory");
    {
        const size_t plain = DIM - 2 * pairs;
        auto add_parts = [&](float2& sum, int head_local, int part0, const float2 (&x)[8]) {
            #pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (part0 + k < parts) {
                    const float factor = merge_factors[head_local * 32 + part0 + k];
                    sum.x = fmaf(x[k].x, factor, sum.x); sum.y = fmaf(x[k].y, factor, sum.y);
                }
            }
        };
        auto finish = [&](float2 sum, int head_local, int d) {
            const float denominator = denominators[head_local];
            sum.x /= denominator; sum.y /= denominator;
            if (size_t(d) >= plain) {
                const double2 turn = inverse[row * pairs + (d - plain) / 2];
                const double x0 = sum.x, y0 = sum.y;
                sum = make_float2(float(x0 * turn.x - y0 * turn.y), float(x0 * turn.y + y0 * turn.x));
            }
            if (gather.world) {   // slot `rank` of every GPU's gathered copy (8-byte aligned: checked by the entry)
                const size_t at = ((size_t(gather.rank) * gridDim.z + row) * a.heads + head0 + head_local) * DIM + d;
                #pragma unroll 1
                for (uint32_t peer = 0; peer < gather.world; ++peer) *reinterpret_cast<float2*>(gather.out[peer] + at) = sum;
                return;
            }
            float* to = out + (row * a.heads + head0 + head_local) * DIM + d;   // (only known to be 4-byte aligned)
            to[0] = sum.x; to[1] = sum.y;
        };
        #pragma unroll
        for (int w = 0; w < kWide; ++w) {
            int head_local, d;
            if (!pair_source(threadIdx.x + w * kComputeThreads, head_local, d)) continue;
            float2 sum = make_float2(0.0f, 0.0f);
            add_parts(sum, head_local, 0, early[w]);
            if (parts > 8) {
                float2 more[8];
                load_parts(threadIdx.x + w * kComputeThreads, 8, more);
                add_parts(sum, head_local, 8, more);
            }
            finish(sum, head_local, d);
        }
        // (fewer than four splits: more pairs a thread than were asked for early)
        for (int i = threadIdx.x + kWide * kComputeThreads; i < 16 * half; i += kComputeThreads) {
            int head_local, d;
            if (!pair_source(i, head_local, d)) continue;
            float2 x[8];
            load_parts(i, 0, x);
            float2 sum = make_float2(0.0f, 0.0f);
            add_parts(sum, head_local, 0, x);
            finish(sum, head_local, d);
        }
    }
    cluster_arrive(); cluster_wait();   // (nobody leaves while its partial may still be read)
    if (gather.world > 1) {
        // The gathered form's hand-over, by the last CTA of the grid to finish: a CTA's peer stores are ordered before its arrival
        // (the barrier orders every thread's stores before thread 0's system-scope fence, which is cumulative: one fence a CTA, not
        // one a thread, each of which would wait on seven links), the arrivals before the counters this rank raises on every GPU
        // (release, system scope); then the same thread waits, bounded to a second, until every rank has raised this GPU's counters
        // to `step`: work queued behind this kernel sees the whole gathered buffer. A rank that never arrives ends the wait with
        // status 4 instead of hanging the GPU.
        asm volatile("bar.sync 3, %0;" ::"n"(kComputeThreads) : "memory");
        if (threadIdx.x == 0) {
            __threadfence_system();
            const unsigned total = gridDim.x * gridDim.y * gridDim.z;
            if (atomicInc(gather.arrivals, total - 1) == total - 1) {   // (wraps to zero: ready for the next call)
                __threadfence_system();
                for (uint32_t peer = 0; peer < gather.world; ++peer)
                    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(gather.flags[peer] + gather.rank), "r"(gather.step) : "memory");
                const uint64_t start = global_timer_ns();
                for (uint32_t peer = 0; peer < gather.world; ++peer) {
                    const int* mine = gather.flags[gather.rank] + peer;
                    for (;;) {
                        int seen;
                        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
                        if (seen - gather.step >= 0) break;   // (counters only grow; the difference survives a wrap)
                        if (global_timer_ns() - start > 1000000000ull) { atomicExch(status, 4); peer = gather.world; break; }
                        __nanosleep(100);
                    }
                }
            }
        }
    }
}

}  // namespace v3

template<int DIM>
static void launch_v3(Device& d, const SparseArgs& a, const float* q, size_t pairs, const double2* forward, size_t rows, size_t splits,
                      int* status, const float* sinks, const double2* inverse, float* out, const GatherTargets& gather) {
    using S = v3::Shape<DIM>;
    static bool configured[64] = {};
    if (!configured[d.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(v3::sparse_mma3_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::kSmem)));
        configured[d.ordinal & 63] = true;
    }
    cudaLaunchConfig_t config{};
    config.gridDim = dim3{unsigned(splits), unsigned((a.heads + 15) / 16), unsigned(rows)};
    config.blockDim = dim3{unsigned(v3::kThreads), 1, 1};
    config.dynamicSmemBytes = S::kSmem;
    config.stream = d.stream;
    cudaLaunchAttribute cluster{};
    cluster.id = cudaLaunchAttributeClusterDimension;
    cluster.val.clusterDim.x = unsigned(splits); cluster.val.clusterDim.y = 1; cluster.val.clusterDim.z = 1;
    config.attrs = &cluster; config.numAttrs = 1;
    // A cluster of this size must fit the device (one 640-thread CTA with all its shared memory per SM, the cluster's SMs in one
    // GPC): asked of the driver once per device and size; a size that does not fit is halved (the kernel reads the split count
    // from the grid, so any power of two is a valid launch).
    static int fits[64][4] = {};   // [device][log2 size]: 0 unknown, 1 fits, -1 does not
    for (;;) {
        const unsigned size = config.gridDim.x;
        const int slot = size >= 8 ? 3 : size >= 4 ? 2 : size >= 2 ? 1 : 0;
        int& known = fits[d.ordinal & 63][slot];
        if (size > 1 && !known) {
            int clusters = 0;
            const cudaError_t asked = cudaOccupancyMaxActiveClusters(&clusters, v3::sparse_mma3_kernel<DIM>, &config);
            if (asked != cudaSuccess) cudaGetLastError();
            known = asked == cudaSuccess && clusters > 0 ? 1 : -1;
        }
        if (size == 1 || known > 0) break;
        config.gridDim.x = size / 2;
        cluster.val.clusterDim.x = size / 2;
    }
    SDB_CHECK(cudaLaunchKernelEx(&config, v3::sparse_mma3_kernel<DIM>, a, q, pairs, forward, a.scale * 1.4426950408889634f, status, sinks, inverse, out, gather));
    ++d.launches;
}

void sparse_mma3_launch(Device& d, const SparseArgs& a, const float* q, const float* sinks, size_t rows, size_t pairs,
                        const double2* forward, const double2* inverse, float* out, const GatherTargets* gather) {
    const size_t head_tiles = (a.heads + 15) / 16;
    // One wave of CTAs (one per SM). The splits of a (row, head tile) are a thread-block cluster: 1, 2, 4 or 8 of them, as many
    // as keep rows * head tiles * splits within the SM count, each group of a split at least two tiles.
    const size_t room = size_t(d.sms) / std::max<size_t>(1, rows * head_tiles);
    const size_t useful = std::max<size_t>(1, a.selections / (2 * v3::kT * v3::kGroups));
    size_t splits = 1;
    while (splits * 2 <= std::min<size_t>({room, useful, size_t(8)})) splits *= 2;
    int* status = status_word(d);
    GatherTargets targets{};
    if (gather) { targets = *gather; targets.arrivals = reinterpret_cast<unsigned*>(status) + 16; }   // (a word of the status block, zero at rest)
    if (a.dim == 576) launch_v3<576>(d, a, q, pairs, forward, rows, splits, status, sinks, inverse, out, targets);
    else launch_v3<512>(d, a, q, pairs, forward, rows, splits, status, sinks, inverse, out, targets);
    SDB_CHECK(cudaGetLastError());
}

}  // namespace sdb
