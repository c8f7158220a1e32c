// Tensor-core kernel of the latent sparse attention (sd_op_sparse_attention) for sm_100a: BF16
// operands, FP32 accumulation, flash decoding over each row's key list.
//
// What it replaces: op_attention_scores_kernel + op_attention_output_kernel + combine
// (gpu/ops.hpp:1329-1434, 1542-1677), which write every score to HBM and re-read each key row once
// per 16-head group and again per (64 dims x 8 heads) output block. Here a CTA holds 16 or 32 heads
// of one query row and streams that row's selected compressed rows once: BF16 rows are gathered
// HBM -> shared memory by one bulk copy (TMA engine) per 1152-byte row, three tiles of 32 keys in
// flight, and both products run on mma.sync.m16n8k16 (BF16) straight from the tile.
//
// Warp roles. Warp (mt, dp): head tile mt (16 heads), dimension part dp (a quarter of the columns).
// Its Q fragments for its quarter of the contraction stay in registers for the whole kernel; the four
// partial score tiles of a head tile are summed through shared memory in a fixed order, every warp
// then forms the same softmax weights and multiplies them into its own quarter of the output columns
// (keys are also the values). Exactness: BF16 rows are exact operands. F32 operands (queries after
// rope, window rows, untagged compressed rows) are split into BF16 high and low parts, x = hi + lo up
// to 2^-17 relative, and both parts are multiplied; a low part that is zero adds exact zeros, so BF16
// rows and F32 rows holding the same values give the same bits (tests/ds_state_bf16_gpu.rs:99-102).
// The weights are rounded to BF16 once; the same rounded values form the denominator.
#include "ds_sparse.cuh"

#include <algorithm>

namespace sdb {

constexpr int kT = 32;   // keys a tile

template<int DIM, int WM, int STAGES> struct MmaShape {
    static constexpr int kRow = (DIM + 8) * 2;          // padded shared-memory row: 8 rows of a fragment load hit 32 distinct banks
    static constexpr int kPlane = kT * kRow;
    static constexpr int kKS = DIM / 64;                // k-steps (16 dims) of one dimension part
    static constexpr int kNT = DIM / 32;                // output n-tiles (8 dims) of one dimension part
    static constexpr int kSlabRow = kT + 8;             // floats
    static constexpr int kSlab = 16 * kSlabRow;         // one warp's partial scores
    static constexpr size_t kSmem = size_t(STAGES) * kPlane + size_t(2) * WM * 4 * kSlab * 4 + STAGES * 8 + STAGES * 4 + 64;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }

template<int DIM, int WM, int STAGES>
__global__ void __launch_bounds__(128 * WM, 1) sparse_mma_kernel(const SparseArgs a, const __nv_bfloat16* __restrict__ q_hi,
                                                                const __nv_bfloat16* __restrict__ q_lo, const int* __restrict__ inexact,
                                                                int lo_rope_from, float scale_log2, float* __restrict__ partial,
                                                                int* __restrict__ status) {
    using S = MmaShape<DIM, WM, STAGES>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* planes = smem;
    float* slabs = reinterpret_cast<float*>(smem + size_t(STAGES) * S::kPlane);
    uint64_t* full = reinterpret_cast<uint64_t*>(slabs + 2 * WM * 4 * S::kSlab);
    uint32_t* live_masks = reinterpret_cast<uint32_t*>(full + STAGES);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane / 4, t = lane % 4;
    const int mt = warp % WM, dp = warp / WM;
    const size_t split = blockIdx.x, splits = gridDim.x, row = blockIdx.z;
    const size_t head0 = size_t(blockIdx.y) * 16 * WM + 16 * mt;
    if (threadIdx.x == 0)
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
    fence_barrier_init();
    __syncthreads();

    // ---- this warp's query fragments: heads head0 + g and head0 + g + 8, its quarter of the columns ----
    const int lo_from = *inexact ? 0 : lo_rope_from;
    uint32_t qh[S::kKS][4], ql[S::kKS][4];
    {
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

    // ---- one tile: scores, softmax, weighted sum. LO: the tile has a low-part plane (F32 keys) ----
    auto compute = [&](const uint8_t* hi, const uint8_t* lo, uint32_t live, bool has_lo) {
        float s[4][4];
        #pragma unroll
        for (int j = 0; j < 4; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
        const int frag_row = 8 * (lane / 16) + lane % 8, frag_half = (lane / 8) % 2;
        #pragma unroll
        for (int ks = 0; ks < S::kKS; ++ks) {
            const int kk = dp * S::kKS + ks;
            #pragma unroll
            for (int jp = 0; jp < 2; ++jp) {
                const size_t at = size_t(16 * jp + frag_row) * S::kRow + size_t(16 * kk + 8 * frag_half) * 2;
                uint32_t b[4];
                ldmatrix_x4(b, hi + at);
                mma_bf16(s[2 * jp], qh[ks], b[0], b[1]);
                mma_bf16(s[2 * jp + 1], qh[ks], b[2], b[3]);
                if (kk >= lo_from) {
                    mma_bf16(s[2 * jp], ql[ks], b[0], b[1]);
                    mma_bf16(s[2 * jp + 1], ql[ks], b[2], b[3]);
                }
                if (has_lo) {
                    ldmatrix_x4(b, lo + at);
                    mma_bf16(s[2 * jp], qh[ks], b[0], b[1]);
                    mma_bf16(s[2 * jp + 1], qh[ks], b[2], b[3]);
                }
            }
        }
        // the four dimension parts of a head tile summed in part order through shared memory
        float* mine = slabs + size_t((tiles_done & 1) * WM * 4 + mt * 4) * S::kSlab;
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<float2*>(mine + dp * S::kSlab + g * S::kSlabRow + 8 * j + 2 * t) = make_float2(s[j][0], s[j][1]);
            *reinterpret_cast<float2*>(mine + dp * S::kSlab + (g + 8) * S::kSlabRow + 8 * j + 2 * t) = make_float2(s[j][2], s[j][3]);
        }
        __syncthreads();
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
        const int v_key = 8 * ((lane / 8) % 2) + lane % 8, v_dim = 8 * (lane / 16);
        #pragma unroll
        for (int kk2 = 0; kk2 < kT / 16; ++kk2) {
            #pragma unroll
            for (int np = 0; np < S::kNT / 2; ++np) {
                const size_t at = size_t(16 * kk2 + v_key) * S::kRow + size_t(dp * (DIM / 4) + 16 * np + v_dim) * 2;
                uint32_t b[4];
                ldmatrix_x4_trans(b, hi + at);
                mma_bf16(o[2 * np], pa[kk2], b[0], b[1]);
                mma_bf16(o[2 * np + 1], pa[kk2], b[2], b[3]);
                if (has_lo) {
                    ldmatrix_x4_trans(b, lo + at);
                    mma_bf16(o[2 * np], pa[kk2], b[0], b[1]);
                    mma_bf16(o[2 * np + 1], pa[kk2], b[2], b[3]);
                }
            }
        }
        ++tiles_done;
    };

    const KeyList list = key_list(a, row);
    const bool rows_bf16 = state_is_bf16(a.compressed);
    const size_t per_split = ((a.selections + splits - 1) / splits + kT - 1) / kT * kT;
    const size_t sel_begin = min(a.selections, split * per_split), sel_end = min(a.selections, sel_begin + per_split);

    // ---- F32 keys (the window rows, on split 0; untagged compressed rows): converted into a high and a low plane, tile by tile ----
    const size_t f32_begin = split == 0 ? 0 : list.raw_count + sel_begin;
    const size_t f32_end = rows_bf16 ? (split == 0 ? list.raw_count : f32_begin) : list.raw_count + sel_end;
    for (size_t first = f32_begin; first < f32_end;) {
        // (a tile never mixes window rows with selected rows, so that the selected rows tile alike in both formats)
        const size_t limit = first < list.raw_count ? list.raw_count : f32_end;
        const size_t count = min(size_t(kT), limit - first);
        __syncthreads();   // the planes' last readers are done
        for (size_t i = threadIdx.x; i < size_t(kT) * (DIM / 2); i += blockDim.x) {
            const size_t r = i / (DIM / 2), c = 2 * (i % (DIM / 2));
            const float* key = r < count ? key_pointer(a, list, row, first + r) : nullptr;
            float2 v = make_float2(0.0f, 0.0f);
            if (key) v = state_is_bf16(key) ? make_float2(__uint_as_float(uint32_t(state_halves(key)[c]) << 16), __uint_as_float(uint32_t(state_halves(key)[c + 1]) << 16))
                                            : make_float2(key[c], key[c + 1]);
            const __nv_bfloat16 h0 = __float2bfloat16_rn(v.x), h1 = __float2bfloat16_rn(v.y);
            const __nv_bfloat162 hi2 = __halves2bfloat162(h0, h1);
            const __nv_bfloat162 lo2 = __halves2bfloat162(__float2bfloat16_rn(v.x - __bfloat162float(h0)), __float2bfloat16_rn(v.y - __bfloat162float(h1)));
            *reinterpret_cast<__nv_bfloat162*>(planes + r * S::kRow + c * 2) = hi2;
            *reinterpret_cast<__nv_bfloat162*>(planes + S::kPlane + r * S::kRow + c * 2) = lo2;
        }
        if (warp == 0) {
            const bool live = size_t(lane) < count && key_pointer(a, list, row, first + lane) != nullptr;
            const uint32_t mask = __ballot_sync(0xffffffffu, live);
            if (lane == 0) live_masks[0] = mask;
        }
        __syncthreads();
        compute(planes, planes + S::kPlane, live_masks[0], true);
        first += count;
    }

    // ---- BF16 selected rows: gathered by bulk copies, STAGES tiles deep ----
    if (rows_bf16 && sel_end > sel_begin) {
        __syncthreads();   // the planes are free
        const uint32_t tiles = uint32_t((sel_end - sel_begin + kT - 1) / kT);
        const int32_t* chosen = a.selected + row * a.selections;
        const uint16_t* halves = state_halves(a.compressed);
        auto issue = [&](uint32_t tile) {   // warp 0, all lanes: lane = the tile's row
            const int slot = int(tile % STAGES);
            uint8_t* dst = planes + size_t(slot) * S::kPlane + size_t(lane) * S::kRow;
            const size_t index = sel_begin + size_t(tile) * kT + lane;
            const int32_t at = index < sel_end ? chosen[index] : -1;
            const bool live = at >= 0;
            if (!live)
                for (int i = 0; i < DIM * 2 / 16; ++i) reinterpret_cast<uint4*>(dst)[i] = make_uint4(0, 0, 0, 0);
            const uint32_t mask = __ballot_sync(0xffffffffu, live);
            __syncwarp();
            if (lane == 0) {
                live_masks[slot] = mask;
                mbar_expect_tx(&full[slot], uint32_t(__popc(mask)) * DIM * 2);
            }
            __syncwarp();
            if (live) bulk_g2s(dst, halves + size_t(at) * DIM, DIM * 2, &full[slot]);
        };
        if (warp == 0)
            for (uint32_t s = 0; s < uint32_t(STAGES - 1) && s < tiles; ++s) issue(s);
        for (uint32_t tile = 0; tile < tiles; ++tile) {
            const int slot = int(tile % STAGES);
            if (!mbar_wait(&full[slot], (tile / STAGES) & 1)) { if (threadIdx.x == 0) atomicExch(status, 1); drain_delay(); return; }
            const uint32_t live = live_masks[slot];
            // (the refill of the slot read one tile ago follows the barrier inside compute: every warp is past that tile by then)
            const uint8_t* plane = planes + size_t(slot) * S::kPlane;
            // scores, then the shared-memory sum's barrier, then the refill, then the rest: written out here so that the
            // issue sits right behind the barrier
            compute(plane, plane, live, false);
            if (warp == 0 && tile + STAGES - 1 < tiles) {
                // every warp finished tile - 1's reads before it reached this tile's barrier; tile's own slot is not touched
                issue(tile + STAGES - 1);
            }
        }
    }

    // ---- the split's partial: [DIM sums | max (exp2 domain) | denominator] per head ----
    #pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    #pragma unroll
    for (int i = 0; i < 2; ++i) {
        const size_t head = head0 + g + 8 * i;
        if (head >= a.heads) continue;
        float* mine = partial + ((row * a.heads + head) * splits + split) * (DIM + 2);
        #pragma unroll
        for (int n = 0; n < S::kNT; ++n)
            *reinterpret_cast<float2*>(mine + dp * (DIM / 4) + 8 * n + 2 * t) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
        if (dp == 0 && t == 0) { mine[DIM] = m[i]; mine[DIM + 1] = l[i]; }
    }
}

bool sparse_mma_supported(const SparseArgs& a) {
    if (a.dim != 512 && a.dim != 576) return false;
    if (a.selections && state_is_bf16(a.compressed) && reinterpret_cast<uintptr_t>(state_halves(a.compressed)) % 16) return false;
    return true;
}

template<int DIM, int WM, int STAGES>
static void launch_shape(Device& d, const SparseArgs& a, const __nv_bfloat16* hi, const __nv_bfloat16* lo, const int* inexact, int lo_rope_from,
                         size_t rows, size_t splits, float* partial, int* status) {
    using S = MmaShape<DIM, WM, STAGES>;
    SDB_CHECK(cudaFuncSetAttribute(sparse_mma_kernel<DIM, WM, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::kSmem)));
    const dim3 grid{unsigned(splits), unsigned((a.heads + 16 * WM - 1) / (16 * WM)), unsigned(rows)};
    sparse_mma_kernel<DIM, WM, STAGES><<<grid, 128 * WM, S::kSmem, d.stream>>>(a, hi, lo, inexact, lo_rope_from,
                                                                                 a.scale * 1.4426950408889634f, partial, status);
    ++d.launches;
}

void sparse_mma_launch(Device& d, const SparseArgs& a, const float* q, const float* sinks, size_t rows, size_t pairs,
                       const double2* forward, const double2* inverse, float* out) {
    const int wm = a.heads > 16 ? 2 : 1;
    const size_t groups = (a.heads + 16 * wm - 1) / (16 * wm);
    // one wave of CTAs: as many splits as keep rows * groups * splits within the resident CTA slots, each split at least two tiles
    const size_t slots = size_t(d.sms) * (wm == 1 ? 2 : 1);
    size_t splits = slots / std::max<size_t>(1, rows * groups);
    splits = std::max<size_t>(1, std::min<size_t>({splits, size_t(16), std::max<size_t>(1, a.selections / (2 * kT))}));
    const size_t q_values = checked_product({rows, a.heads, a.dim});
    const size_t hi_at = 256, lo_at = hi_at + (q_values * 2 + 255) / 256 * 256, partial_at = lo_at + (q_values * 2 + 255) / 256 * 256;
    const size_t total = partial_at + checked_product({rows, a.heads, splits, a.dim + 2, 4});
    auto* work = static_cast<uint8_t*>(ensure(d, d.partial, d.partial_bytes, total));
    int* flags = reinterpret_cast<int*>(work);              // [0]: queries not BF16-exact outside the rotated columns; [1]: a wait gave up
    auto* hi = reinterpret_cast<__nv_bfloat16*>(work + hi_at);
    auto* lo = reinterpret_cast<__nv_bfloat16*>(work + lo_at);
    auto* partial = reinterpret_cast<float*>(work + partial_at);
    SDB_CHECK(cudaMemsetAsync(flags, 0, 8, d.stream));
    sparse_prepare_q_kernel<<<dim3(unsigned(a.heads), unsigned(rows)), 128, 0, d.stream>>>(q, a.heads, a.dim, pairs, forward, nullptr, hi, lo, flags);
    ++d.launches;
    const int lo_rope_from = pairs ? int((a.dim - 2 * pairs) / 16) : int(a.dim / 16);
    if (a.dim == 576) {
        if (wm == 2) launch_shape<576, 2, 3>(d, a, hi, lo, flags, lo_rope_from, rows, splits, partial, flags + 1);
        else launch_shape<576, 1, 2>(d, a, hi, lo, flags, lo_rope_from, rows, splits, partial, flags + 1);
    } else {
        if (wm == 2) launch_shape<512, 2, 3>(d, a, hi, lo, flags, lo_rope_from, rows, splits, partial, flags + 1);
        else launch_shape<512, 1, 2>(d, a, hi, lo, flags, lo_rope_from, rows, splits, partial, flags + 1);
    }
    SDB_CHECK(cudaGetLastError());
    sparse_combine_kernel<<<unsigned(rows * a.heads), 128, 0, d.stream>>>(partial, splits, a.heads, a.dim, sinks, pairs, inverse, 1, out);
    ++d.launches;
}

}  // namespace sdb
