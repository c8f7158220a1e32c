// Tensor-core kernel of the latent sparse attention (sd_op_sparse_attention) for sm_100a, second form:
// a dedicated producer warp and a five-tile ring, so that four tiles of gathered rows are always in
// flight per SM (random 1152-byte rows from HBM need about 2 us: 6.4 TB/s x 2 us / 148 SMs = 86 KB).
//
// What it replaces: op_attention_scores_kernel + op_attention_output_kernel + combine
// (gpu/ops.hpp:1329-1434, 1542-1677), which write every score to HBM and re-read each key row once
// per 16-head group and again per (64 dims x 8 heads) output block. Here a CTA holds 16 or 32 heads
// of one query row and streams that row's selected compressed rows once.
//
// CTA = 8 compute warps + 1 producer warp, one CTA per SM.
//   * Producer: walks the split's selection list with the next tile's indices already in registers
//     and gathers each BF16 row HBM -> shared memory by one bulk copy (TMA engine) of dim * 2 bytes into
//     a ring of five 32-key tiles; a full and an empty mbarrier per slot. Rows that are absent (-1, or
//     past the list) are zero-filled so that a zero weight never meets stale bits.
//   * Compute warp (mt, dp) of a group: head tile mt (16 heads), dimension part dp (a quarter of the
//     columns). With 32 heads the eight warps are one group (2 head tiles x 4 parts); with 16 heads
//     they are two groups of four warps that take alternate tiles, each with its own softmax state and
//     its own partial. A warp's Q fragments for its quarter of the contraction stay in registers; the
//     four partial score tiles of a head tile are summed through shared memory in a fixed order, every
//     warp then forms the same softmax weights and multiplies them into its own quarter of the output
//     columns (keys are also the values). Both products run on mma.sync.m16n8k16 (BF16) with ldmatrix
//     operands from padded rows (the 8 rows of a fragment hit 32 distinct banks).
// Exactness: BF16 rows are exact operands. F32 operands (queries after rope, window rows, untagged
// compressed rows) are split into BF16 high and low parts, x = hi + lo up to 2^-17 relative, and both
// parts are multiplied; a low part that is zero adds exact zeros, so BF16 rows and F32 rows holding the
// same values give the same bits (tests/ds_state_bf16_gpu.rs:99-102). The weights are rounded to BF16
// once; the same rounded values form the denominator.
#include "ds_sparse.cuh"

#include <algorithm>
#include <type_traits>

namespace sdb {
namespace v2 {

constexpr int kT = 32;          // keys a tile
constexpr int kStages = 5;      // tiles in the ring
constexpr int kComputeWarps = 8;

template<int DIM> struct Shape {
    static constexpr int kRow = (DIM + 8) * 2;          // padded shared-memory row
    static constexpr int kPlane = kT * kRow;
    static constexpr int kKS = DIM / 64;                // k-steps (16 dims) of one dimension part
    static constexpr int kNT = DIM / 32;                // output n-tiles (8 dims) of one dimension part
    static constexpr int kSlabRow = kT + 8;             // floats
    static constexpr int kSlab = 16 * kSlabRow;         // one warp's partial scores
    static constexpr size_t kSlabBytes = size_t(2) * kComputeWarps * kSlab * 4;   // double buffered, one per compute warp
    static constexpr size_t kSmem = size_t(kStages) * kPlane + kSlabBytes + 2 * kStages * 8 + kStages * 4 + 64;
};

// (32-bit shared addresses: a lane's base is formed once per tile and every fragment is base + a compile-time offset)
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ void group_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// WM: head tiles of 16 a group holds (1: two groups of four warps; 2: one group of eight)
template<int DIM, int WM>
__global__ void __launch_bounds__(kComputeWarps * 32, 1) sparse_mma2_kernel(
        const SparseArgs a, const __nv_bfloat16* __restrict__ q_hi, const __nv_bfloat16* __restrict__ q_lo,
        const int* __restrict__ inexact, int lo_rope_from, float scale_log2, float* __restrict__ partial, int* __restrict__ status) {
    using S = Shape<DIM>;
    constexpr int kGroups = 2 / WM, kGroupWarps = 4 * WM, kGroupThreads = 32 * kGroupWarps;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* planes = smem;
    float* slabs = reinterpret_cast<float*>(smem + size_t(kStages) * S::kPlane);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + size_t(kStages) * S::kPlane + S::kSlabBytes);
    uint64_t* empty = full + kStages;
    uint32_t* live_masks = reinterpret_cast<uint32_t*>(empty + kStages);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(live_masks + kStages);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane / 4, t = lane % 4;
    constexpr bool producer = false;   // (no separate producer warp: the first warp of a group refills the slot its group has just consumed)
    const int group = warp / kGroupWarps, gw = warp % kGroupWarps;   // the warp within its group
    const int mt = gw % WM, dp = gw / WM;
    const size_t split = blockIdx.x, splits = gridDim.x, row = blockIdx.z;
    const size_t head0 = size_t(blockIdx.y) * 16 * WM + 16 * mt;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], kGroupThreads); mbar_init(&empty[s], kGroupWarps); }
        *abort_flag = 0;
    }
    fence_barrier_init();
    __syncthreads();

    // a bounded wait that also ends when another role has given up
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
    const size_t per_split = ((a.selections + splits - 1) / splits + kT - 1) / kT * kT;
    const size_t sel_begin = min(a.selections, split * per_split), sel_end = min(a.selections, sel_begin + per_split);
    const uint32_t stream_tiles = rows_bf16 ? uint32_t((sel_end - sel_begin + kT - 1) / kT) : 0u;
    // F32 keys: the window rows (split 0) and untagged compressed rows, taken tile by tile by group 0 before the stream
    const size_t f32_begin = split == 0 ? 0 : list.raw_count + sel_begin;
    const size_t f32_end = rows_bf16 ? (split == 0 ? list.raw_count : f32_begin) : list.raw_count + sel_end;

    // ---- this warp's query fragments: heads head0 + g and head0 + g + 8, its quarter of the columns ----
    const int lo_from = *inexact ? 0 : lo_rope_from;
    uint32_t qh[S::kKS][4], ql[S::kKS][4];
    if (!producer) {
        const size_t ha = head0 + g, hb = head0 + g + 8;
        const uint32_t* rows_hi[2] = {ha < a.heads ? reinterpret_cast<const uint32_t*>(q_hi + (row * a.heads + ha) * DIM) : nullptr,
                                      hb < a.heads ? reinterpret_cast<const uint32_t*>(q_hi + (row * a.heads + hb) * DIM) : nullptr};
        const uint32_t* rows_lo[2] = {ha < a.heads ? reinterpret_cast<const uint32_t*>(q_lo + (row * a.heads + ha) * DIM) : nullptr,
                                      hb < a.heads ? reinterpret_cast<const uint32_t*>(q_lo + (row * a.heads + hb) * DIM) : nullptr};
        #pragma unroll
        for (int ks = 0; ks < S::kKS; ++ks) {
            const int word = (16 * (dp * S::kKS + ks) + 2 * t) / 2;
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int which = i & 1, off = word + (i >> 1) * 4;
                qh[ks][i] = rows_hi[which] ? rows_hi[which][off] : 0u;
                ql[ks][i] = rows_lo[which] && (dp * S::kKS + ks) >= lo_from ? rows_lo[which][off] : 0u;
            }
        }
    }
    float o[S::kNT][4];
    #pragma unroll
    for (int n = 0; n < S::kNT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    unsigned tiles_done = 0;

    // ---- one tile for one group: scores, softmax, weighted sum; has_lo: the tile has a low-part plane (F32 keys) ----
    const int frag_row = 8 * (lane / 16) + lane % 8, frag_half = (lane / 8) % 2;
    const uint32_t k_lane = uint32_t(frag_row * S::kRow + (16 * dp * S::kKS + 8 * frag_half) * 2);
    const int v_key = 8 * ((lane / 8) % 2) + lane % 8, v_dim = 8 * (lane / 16);
    const uint32_t v_lane = uint32_t(v_key * S::kRow + (dp * (DIM / 4) + v_dim) * 2);
    auto compute = [&](const uint8_t* hi, const uint8_t* lo, uint32_t live, auto lo_tag) {
        constexpr bool has_lo = decltype(lo_tag)::value;
        const uint32_t hi_k = smem_u32(hi) + k_lane, lo_k = smem_u32(lo) + k_lane, hi_v = smem_u32(hi) + v_lane, lo_v = smem_u32(lo) + v_lane;
        float s[4][4];
        #pragma unroll
        for (int j = 0; j < 4; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
        #pragma unroll
        for (int ks = 0; ks < S::kKS; ++ks) {
            const int kk = dp * S::kKS + ks;
            #pragma unroll
            for (int jp = 0; jp < 2; ++jp) {
                const uint32_t at = uint32_t(16 * jp * S::kRow + 32 * ks);
                uint32_t b[4];
                ldmatrix_x4(b, hi_k + at);
                mma_bf16(s[2 * jp], qh[ks], b[0], b[1]);
                mma_bf16(s[2 * jp + 1], qh[ks], b[2], b[3]);
                if (kk >= lo_from) {
                    mma_bf16(s[2 * jp], ql[ks], b[0], b[1]);
                    mma_bf16(s[2 * jp + 1], ql[ks], b[2], b[3]);
                }
                if constexpr (has_lo) {
                    ldmatrix_x4(b, lo_k + at);
                    mma_bf16(s[2 * jp], qh[ks], b[0], b[1]);
                    mma_bf16(s[2 * jp + 1], qh[ks], b[2], b[3]);
                }
            }
        }
        // the four dimension parts of a head tile summed in part order through shared memory (this group's slabs)
        float* mine = slabs + size_t((tiles_done & 1) * kComputeWarps + group * kGroupWarps + mt * 4) * S::kSlab;
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<float2*>(mine + dp * S::kSlab + g * S::kSlabRow + 8 * j + 2 * t) = make_float2(s[j][0], s[j][1]);
            *reinterpret_cast<float2*>(mine + dp * S::kSlab + (g + 8) * S::kSlabRow + 8 * j + 2 * t) = make_float2(s[j][2], s[j][3]);
        }
        group_barrier(1 + group, kGroupThreads);
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 top = make_float2(0.0f, 0.0f), bottom = make_float2(0.0f, 0.0f);
            #pragma unroll
            for (int part = 0; part < 4; ++part) {
                const float2 x = *reinterpret_cast<const float2*>(mine + part * S::kSlab + g * S::kSlabRow + 8 * j + 2 * t);
                const float2 y = *reinterpret_cast<const float2*>(mine + part * S::kSlab + (g + 8) * S::kSlabRow + 8 * j + 2 * t);
                top.x += x.x; top.y += x.y; bottom.x += y.x; bottom.y += y.y;
            }
            const bool live0 = (live >> (8 * j + 2 * t)) & 1u, live1 = (live >> (8 * j + 2 * t + 1)) & 1u;
            s[j][0] = live0 ? top.x * scale_log2 : -INFINITY; s[j][1] = live1 ? top.y * scale_log2 : -INFINITY;
            s[j][2] = live0 ? bottom.x * scale_log2 : -INFINITY; s[j][3] = live1 ? bottom.y * scale_log2 : -INFINITY;
        }
        float top[2] = {-INFINITY, -INFINITY};
        #pragma unroll
        for (int j = 0; j < 4; ++j) { top[0] = fmaxf(top[0], fmaxf(s[j][0], s[j][1])); top[1] = fmaxf(top[1], fmaxf(s[j][2], s[j][3])); }
        #pragma unroll
        for (int i = 0; i < 2; ++i) {
            top[i] = fmaxf(top[i], __shfl_xor_sync(0xffffffffu, top[i], 1));
            top[i] = fmaxf(top[i], __shfl_xor_sync(0xffffffffu, top[i], 2));
        }
        const float n0 = fmaxf(m[0], top[0]), n1 = fmaxf(m[1], top[1]);
        if (__any_sync(0xffffffffu, n0 > m[0] || n1 > m[1])) {
            const float f0 = m[0] == -INFINITY ? 0.0f : fast_exp2(m[0] - n0), f1 = m[1] == -INFINITY ? 0.0f : fast_exp2(m[1] - n1);
            l[0] *= f0; l[1] *= f1;
            #pragma unroll
            for (int n = 0; n < S::kNT; ++n) { o[n][0] *= f0; o[n][1] *= f0; o[n][2] *= f1; o[n][3] *= f1; }
            m[0] = n0; m[1] = n1;
        }
        const float u0 = m[0] == -INFINITY ? 0.0f : m[0], u1 = m[1] == -INFINITY ? 0.0f : m[1];   // (no live key yet: weights 0, not NaN)
        uint32_t pa[2][4];
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t p01 = pack_bf16x2(fast_exp2(s[j][0] - u0), fast_exp2(s[j][1] - u0));
            const uint32_t p23 = pack_bf16x2(fast_exp2(s[j][2] - u1), fast_exp2(s[j][3] - u1));
            l[0] += bf16_lo(p01) + bf16_hi(p01);
            l[1] += bf16_lo(p23) + bf16_hi(p23);
            pa[j / 2][(j & 1) * 2] = p01;
            pa[j / 2][(j & 1) * 2 + 1] = p23;
        }
        // O += P V over this warp's quarter of the columns
        #pragma unroll
        for (int kk2 = 0; kk2 < kT / 16; ++kk2) {
            #pragma unroll
            for (int np = 0; np < S::kNT / 2; ++np) {
                const uint32_t at = uint32_t(16 * kk2 * S::kRow + 32 * np);
                uint32_t b[4];
                ldmatrix_x4_trans(b, hi_v + at);
                mma_bf16(o[2 * np], pa[kk2], b[0], b[1]);
                mma_bf16(o[2 * np + 1], pa[kk2], b[2], b[3]);
                if constexpr (has_lo) {
                    ldmatrix_x4_trans(b, lo_v + at);
                    mma_bf16(o[2 * np], pa[kk2], b[0], b[1]);
                    mma_bf16(o[2 * np + 1], pa[kk2], b[2], b[3]);
                }
            }
        }
        ++tiles_done;
    };

    // ---- F32 keys: converted into a high and a low plane (slots 0 and 1), a tile at a time, by all compute warps; group 0 consumes ----
    // (8-byte aligned: the flag sits 100 bytes past the 8-aligned barriers)
    const float** key_ptrs = reinterpret_cast<const float**>((reinterpret_cast<uintptr_t>(const_cast<int*>(abort_flag)) + 4 + 7) & ~uintptr_t(7));
    for (size_t first = f32_begin; first < f32_end;) {
        // (a tile never mixes window rows with selected rows, so that the selected rows tile alike in both formats)
        const size_t limit = first < list.raw_count ? list.raw_count : f32_end;
        const size_t count = min(size_t(kT), limit - first);
        if (!producer) {
            group_barrier(3, kComputeWarps * 32);   // the planes' last readers are done
            if (warp == 0) {
                const float* key = size_t(lane) < count ? key_pointer(a, list, row, first + lane) : nullptr;
                key_ptrs[lane] = key;
                const uint32_t mask = __ballot_sync(0xffffffffu, key != nullptr);
                if (lane == 0) live_masks[0] = mask;
            }
            group_barrier(3, kComputeWarps * 32);
            for (size_t i = threadIdx.x; i < size_t(kT) * (DIM / 2); i += kComputeWarps * 32) {
                const size_t r = i / (DIM / 2), c = 2 * (i % (DIM / 2));
                const float* key = key_ptrs[r];
                float2 v = make_float2(0.0f, 0.0f);
                if (key) v = state_is_bf16(key) ? make_float2(__uint_as_float(uint32_t(state_halves(key)[c]) << 16), __uint_as_float(uint32_t(state_halves(key)[c + 1]) << 16))
                                                : make_float2(key[c], key[c + 1]);
                const __nv_bfloat16 h0 = __float2bfloat16_rn(v.x), h1 = __float2bfloat16_rn(v.y);
                *reinterpret_cast<__nv_bfloat162*>(planes + r * S::kRow + c * 2) = __halves2bfloat162(h0, h1);
                *reinterpret_cast<__nv_bfloat162*>(planes + S::kPlane + r * S::kRow + c * 2) =
                    __halves2bfloat162(__float2bfloat16_rn(v.x - __bfloat162float(h0)), __float2bfloat16_rn(v.y - __bfloat162float(h1)));
            }
            group_barrier(3, kComputeWarps * 32);
            if (group == 0) compute(planes, planes + S::kPlane, live_masks[0], std::true_type{});
        }
        first += count;
    }
    __syncthreads();   // the F32 tiles are consumed: the ring belongs to the producer from here

    // ---- BF16 selected rows: a ring of kStages tiles; the groups consume alternate tiles and refill the slot they have just left ----
    // The gather runs on 16-byte asynchronous copies (cp.async, zero-filling absent rows) issued by every thread of a group, a
    // quarter of a tile per warp: one bulk copy per 1152-byte row kept the copy engine at about one row per 70 ns per SM, a third
    // of what HBM delivers.
    {
        const int32_t* chosen = a.selected + row * a.selections;
        const uint8_t* halves = reinterpret_cast<const uint8_t*>(state_halves(a.compressed));
        constexpr int kChunks = DIM * 2 / 16;   // 16-byte pieces of a row
        auto index_of = [&](uint32_t tile) -> int32_t {   // this lane's row of `tile`
            const size_t index = sel_begin + size_t(tile) * kT + lane;
            return tile < stream_tiles && index < sel_end ? chosen[index] : -1;
        };
        auto issue = [&](uint32_t tile, int32_t at) {   // every warp of a group: warp gw copies pieces gw, gw + kGroupWarps, ... of each run of 32
            const int slot = int(tile % kStages);
            uint8_t* plane = planes + size_t(slot) * S::kPlane;
            if (gw == 0) {
                const uint32_t mask = __ballot_sync(0xffffffffu, at >= 0);
                if (lane == 0) { live_masks[slot] = mask; __threadfence_block(); }
            }
            #pragma unroll 2
            for (int i = gw * 32 + lane; i < kT * kChunks; i += kGroupThreads) {
                const int r = i / kChunks, c = i % kChunks;
                const int32_t source = __shfl_sync(0xffffffffu, at, r);
                const uint8_t* src = halves + (source >= 0 ? size_t(source) * DIM * 2 + size_t(c) * 16 : 0);
                const uint32_t bytes = source >= 0 ? 16u : 0u;   // 0: the piece is zero-filled
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(plane + size_t(r) * S::kRow + c * 16)), "l"(src), "r"(bytes) : "memory");
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[slot])) : "memory");
        };
        // the first kStages tiles: a group fills alternate ones
        for (uint32_t s = uint32_t(group); s < uint32_t(kStages) && s < stream_tiles; s += kGroups) issue(s, index_of(s));
        for (uint32_t tile = uint32_t(group); tile < stream_tiles; tile += kGroups) {
            const int slot = int(tile % kStages);
            const uint32_t refill = tile + kStages;
            const int32_t refill_at = index_of(refill);   // (in flight while this tile is computed)
            if (!wait(&full[slot], (tile / kStages) & 1)) break;
            const uint32_t live = live_masks[slot];
            const uint8_t* plane = planes + size_t(slot) * S::kPlane;
            compute(plane, plane, live, std::false_type{});
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
            if (refill < stream_tiles) {
                if (!wait(&empty[slot], (tile / kStages) & 1)) break;   // the whole group is past the slot
                issue(refill, refill_at);
            }
        }
        // ---- the group's partial: [DIM sums | max (exp2 domain) | denominator] per head ----
        #pragma unroll
        for (int i = 0; i < 2; ++i) {
            l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
            l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        }
        #pragma unroll
        for (int i = 0; i < 2; ++i) {
            const size_t head = head0 + g + 8 * i;
            if (head >= a.heads) continue;
            float* mine = partial + ((row * a.heads + head) * (splits * kGroups) + split * kGroups + group) * (DIM + 2);
            #pragma unroll
            for (int n = 0; n < S::kNT; ++n)
                *reinterpret_cast<float2*>(mine + dp * (DIM / 4) + 8 * n + 2 * t) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
            if (dp == 0 && t == 0) { mine[DIM] = m[i]; mine[DIM + 1] = l[i]; }
        }
    }
}

}  // namespace v2

template<int DIM, int WM>
static void launch_v2(Device& d, const SparseArgs& a, const __nv_bfloat16* hi, const __nv_bfloat16* lo, const int* inexact, int lo_rope_from,
                      size_t rows, size_t splits, float* partial, int* status) {
    using S = v2::Shape<DIM>;
    static bool configured[64] = {};
    if (!configured[d.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(v2::sparse_mma2_kernel<DIM, WM>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::kSmem + 320)));
        configured[d.ordinal & 63] = true;
    }
    const dim3 grid{unsigned(splits), unsigned((a.heads + 16 * WM - 1) / (16 * WM)), unsigned(rows)};
    v2::sparse_mma2_kernel<DIM, WM><<<grid, v2::kComputeWarps * 32, S::kSmem + 320, d.stream>>>(
        a, hi, lo, inexact, lo_rope_from, a.scale * 1.4426950408889634f, partial, status);
    ++d.launches;
}

void sparse_mma2_launch(Device& d, const SparseArgs& a, const float* q, const float* sinks, size_t rows, size_t pairs,
                        const double2* forward, const double2* inverse, float* out) {
    const int wm = a.heads > 16 ? 2 : 1;
    const size_t head_groups = (a.heads + 16 * wm - 1) / (16 * wm), key_groups = 2 / wm;
    // one wave of CTAs (one per SM): as many splits as keep rows * head groups * splits within the SM count,
    // each group of a split at least two tiles
    size_t splits = size_t(d.sms) / std::max<size_t>(1, rows * head_groups);
    splits = std::max<size_t>(1, std::min<size_t>({splits, size_t(16), std::max<size_t>(1, a.selections / (2 * v2::kT * key_groups))}));
    const size_t partials = splits * key_groups;
    const size_t q_values = checked_product({rows, a.heads, a.dim});
    const size_t hi_at = 256, lo_at = hi_at + (q_values * 2 + 255) / 256 * 256, partial_at = lo_at + (q_values * 2 + 255) / 256 * 256;
    const size_t total = partial_at + checked_product({rows, a.heads, partials, a.dim + 2, 4});
    auto* work = static_cast<uint8_t*>(ensure(d, d.partial, d.partial_bytes, total));
    int* flags = reinterpret_cast<int*>(work);              // [0]: queries not BF16-exact outside the rotated columns
    auto* hi = reinterpret_cast<__nv_bfloat16*>(work + hi_at);
    auto* lo = reinterpret_cast<__nv_bfloat16*>(work + lo_at);
    auto* partial = reinterpret_cast<float*>(work + partial_at);
    SDB_CHECK(cudaMemsetAsync(flags, 0, 8, d.stream));
    sparse_prepare_q_kernel<<<dim3(unsigned(a.heads), unsigned(rows)), 128, 0, d.stream>>>(q, a.heads, a.dim, pairs, forward, nullptr, hi, lo, flags);
    ++d.launches;
    const int lo_rope_from = pairs ? int((a.dim - 2 * pairs) / 16) : int(a.dim / 16);
    int* status = status_word(d);
    if (a.dim == 576) {
        if (wm == 2) launch_v2<576, 2>(d, a, hi, lo, flags, lo_rope_from, rows, splits, partial, status);
        else launch_v2<576, 1>(d, a, hi, lo, flags, lo_rope_from, rows, splits, partial, status);
    } else {
        if (wm == 2) launch_v2<512, 2>(d, a, hi, lo, flags, lo_rope_from, rows, splits, partial, status);
        else launch_v2<512, 1>(d, a, hi, lo, flags, lo_rope_from, rows, splits, partial, status);
    }
    SDB_CHECK(cudaGetLastError());
    sparse_combine_kernel<<<unsigned(rows * a.heads), 128, 0, d.stream>>>(partial, partials, a.heads, a.dim, sinks, pairs, inverse, 1, out);
    ++d.launches;
}

}  // namespace sdb
