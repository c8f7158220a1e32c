// Selection-list decode attention over Q8_0 K/V rows on the tensor cores: each row (a decoded token, or one row of a
// verification span) attends its own list of selected key positions.
//
// What it replaces in the reference: qsa_decode_parts + qsa_decode_merge (gpu/sparse_attention_compute.hpp:41-170) as
// qsa_attention (one token, :609-627) and qsa_attention_rows (a verification's rows, :631-647) launch them. Same inputs: the
// packed F32 rows of `steps` tokens (queries | keys | values | selected positions as floats | counts as floats,
// gpu/core.hpp:392), the same rule for a live slot (slot < count, 0 <= position <= the row's own position, position < context:
// :58-64), the same ring-mirror addressing (:65-68), the same optional sigmoid gate in the merge (:168).
//
// Contract kept bit for bit (lines 40-41 of the reference's own design notes under docs/, gpu/qsa_decode.hpp:46-50): a row's result does not depend on how many rows
// share the launch. The work is cut at fixed places: a chunk is 64 consecutive slots of one row, a CTA owns one (chunk, K/V
// head, row), the merge combines a row's chunks in chunk order.
//
// Design: a CTA gathers its chunk's rows into shared memory with one bulk copy (TMA engine) per 272-byte row, four tiles of 16
// slots each with its own mbarrier, all issued up front; a warp per eight query heads of the group then runs the decode
// kernel's arithmetic on each tile: int8 -> FP16 exactly, K.Q^T on mma.sync.m16n8k16 per 32-column block with the block's
// scale applied in FP32, softmax in FP32 (exp2 domain), V^T.P' with the value block's scale folded into P'. The queries arrive
// as F32 and the weights are F32, so both enter the tensor cores as FP16 hi + lo pairs (two products each): nothing is rounded
// to 11 bits on the way, and the result differs from the reference's FP32 kernels by summation order only.
// FP16 rows (sd_kv_format(512): 256 halves a row) take the same kernel without the int8 steps: the rows' halves are the tensor
// cores' operands as they lie (a row every 528 bytes of shared memory, so that eight rows fall on eight bank groups), the value
// fragments come through transposing ldmatrix loads of 16-bit units, and the rows of dead slots are zeroed (a stale NaN times a
// zero weight would be a NaN).
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

namespace sdb {

constexpr int kSelTile = 16, kSelTiles = 4, kSelChunk = kSelTile * kSelTiles;      // slots a tile, tiles a chunk
template <bool F16> struct SelShape {
    static constexpr int kRow = F16 ? int(kv_row_f16) : int(kv_row_q8);            // a row in memory
    static constexpr int kPitch = F16 ? int(kv_row_f16) + 16 : int(kv_row_q8);     // a row in shared memory
    static constexpr int kTileBytes = 2 * kSelTile * kPitch;                       // K rows then V rows
    static constexpr size_t kSmem = size_t(kSelTiles) * kTileBytes + kSelTiles * 8 + kSelChunk * 4 + 16;
};

struct SelectArgs {
    const uint8_t* state;      // 2 * kv_heads planes of `context` rows
    const uint8_t* mirror;     // ring of the newest rows (2 * kv_heads planes of mirror_rows), or null
    size_t context, mirror_rows, base, steps, selected, heads, kv_heads, group, chunks;
    size_t row0;               // the launch's first row (a launch may take a part of the packed rows)
    const uint32_t* position;  // a row's own position, or null: base + row
    const float* input;        // the packed rows
    float* partial;            // [row][head][chunk][258]
    float scale_log2;
    int* status;
};

__device__ __forceinline__ int sel_tile_row(int g) { return 2 * (g & 3) + (g >> 2); }
__device__ __forceinline__ uint32_t sel_bytes01(uint32_t x) {
    const uint32_t h = prmt(x, 0x64646464u, 0x4140u);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t sel_bytes23(uint32_t x) {
    const uint32_t h = prmt(x, 0x64646464u, 0x4342u);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ float sel_half_at(const uint4& v, int i) {
    const uint32_t w = i < 2 ? v.x : i < 4 ? v.y : i < 6 ? v.z : v.w;
    return __half2float(__ushort_as_half(uint16_t(i & 1 ? w >> 16 : w & 0xffffu)));
}
// Two F32 values as an FP16 pair and the pair of what that rounding dropped.
__device__ __forceinline__ void split_pair(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __half ah = __float2half_rn(a), bh = __float2half_rn(b);
    hi = uint32_t(__half_as_ushort(ah)) | uint32_t(__half_as_ushort(bh)) << 16;
    lo = pack_half2(a - __half2float(ah), b - __half2float(bh));
}

// grid (chunks, kv_heads, steps); block = 32 x ceil(group / 8) threads: warp w takes query heads 8w .. of the group
template <bool F16>
__global__ void __launch_bounds__(64) qsa_select_kernel(const SelectArgs a) {
    using S = SelShape<F16>;
    constexpr int kRow = S::kRow, kPitch = S::kPitch, kSelTileBytes = S::kTileBytes;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + size_t(kSelTiles) * kSelTileBytes);
    int* tokens = reinterpret_cast<int*>(bars + kSelTiles);
    // the merge launched behind this kernel may take its place on the SMs now: it waits for this grid's end before it reads
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t chunk = blockIdx.x, kv = blockIdx.y, row = a.row0 + blockIdx.z;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane / 4, t = lane % 4;
    const size_t index_start = a.steps * (a.heads * 256 + a.kv_heads * 512);
    const size_t count = size_t(a.input[index_start + a.steps * a.selected + row]);
    const size_t first = chunk * kSelChunk;
    if (first >= count) return;   // (the merge reads ceil(count / 64) chunks of this row)

    if (warp == 0) {
        // ---- the chunk's 64 slots: validation, then one bulk copy per live key row and value row ----
        const size_t limit = a.position ? size_t(a.position[row]) : a.base + row;
        const size_t last = a.position ? size_t(a.position[a.steps - 1]) : a.base + a.steps - 1;
        if (lane < kSelTiles) mbar_init(&bars[lane], 1);
        fence_barrier_init();
        __syncwarp();
        #pragma unroll
        for (int half = 0; half < 2; ++half) {
            const size_t slot = first + half * 32 + lane;
            int token = -1;
            if (slot < count && slot < a.selected) {
                const float raw = a.input[index_start + row * a.selected + slot];
                if (raw >= 0 && raw <= float(limit) && raw < float(a.context)) token = int(raw);
            }
            tokens[half * 32 + lane] = token;
            // two tiles per half: lanes 0-15 and 16-31
            const unsigned live = __ballot_sync(0xffffffffu, token >= 0);
            if (lane == 0 && (live & 0xffffu)) mbar_expect_tx(&bars[2 * half], __popc(live & 0xffffu) * 2 * kRow);
            if (lane == 16 && (live >> 16)) mbar_expect_tx(&bars[2 * half + 1], __popc(live >> 16) * 2 * kRow);
            __syncwarp();
            const int tile = 2 * half + lane / 16, r = lane % 16;
            uint8_t* dst = smem + size_t(tile) * kSelTileBytes + r * kPitch;
            if (token >= 0) {
                // a recent position is read from the ring mirror of a host-resident state (gpu/sparse_attention_compute.hpp:65-68)
                const bool cached = a.mirror && size_t(token) + a.mirror_rows > last + 8;
                const uint8_t* source = cached ? a.mirror : a.state;
                const size_t capacity = cached ? a.mirror_rows : a.context, at = cached ? size_t(token) % a.mirror_rows : size_t(token);
                bulk_g2s(dst, source + (kv * capacity + at) * kRow, kRow, &bars[tile]);
                bulk_g2s(dst + kSelTile * kPitch, source + ((a.kv_heads + kv) * capacity + at) * kRow, kRow, &bars[tile]);
            } else if (F16) {   // (a dead slot's halves enter the products as they lie: zeros)
                for (int i = 0; i < kRow / 16; ++i) {
                    reinterpret_cast<uint4*>(dst)[i] = make_uint4(0, 0, 0, 0);
                    reinterpret_cast<uint4*>(dst + kSelTile * kPitch)[i] = make_uint4(0, 0, 0, 0);
                }
            }
        }
    }
    __syncthreads();

    const size_t head_in_group = size_t(warp) * 8 + g;
    const bool head_live = head_in_group < a.group;
    // this warp's queries as B fragments, hi and lo
    uint32_t qh[8][4], ql[8][4];
    {
        const float* q = a.input + (row * a.heads + kv * a.group + (head_live ? head_in_group : 0)) * 256 + 8 * t;
        #pragma unroll
        for (int b = 0; b < 8; ++b) {
            float4 x = make_float4(0, 0, 0, 0), y = x;
            if (head_live) { x = *reinterpret_cast<const float4*>(q + 32 * b); y = *reinterpret_cast<const float4*>(q + 32 * b + 4); }
            split_pair(x.x, x.y, qh[b][0], ql[b][0]); split_pair(x.z, x.w, qh[b][1], ql[b][1]);
            split_pair(y.x, y.y, qh[b][2], ql[b][2]); split_pair(y.z, y.w, qh[b][3], ql[b][3]);
        }
    }
    float o[8][2][4];
    #pragma unroll
    for (int b = 0; b < 8; ++b)
        #pragma unroll
        for (int i = 0; i < 2; ++i)
            #pragma unroll
            for (int c = 0; c < 4; ++c) o[b][i][c] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;   // heads 2t and 2t+1 of this warp's eight
    const int r0 = sel_tile_row(g), r1 = r0 + 8;
    const int ka = sel_tile_row(2 * t), kb = sel_tile_row(2 * t + 1);
    // (a block's value bytes come through one transposing ldmatrix, as in the dense decode kernel: matrix m holds the keys
    //  k-index j -> sel_tile_row(j) + 8 (m & 1) and the 16-bit units of columns 16 (m >> 1) ..)
    //  FP16 rows: matrix m holds the keys sel_tile_row(j) + 8 (m >> 1) and the columns 8 (m & 1) .. of a 16-column piece: the A fragment's order)
    const uint32_t v_lane = F16 ? uint32_t((sel_tile_row(lane % 8) + 8 * (lane / 16)) * kPitch + 16 * ((lane / 8) & 1))
                                : uint32_t((sel_tile_row(lane % 8) + 8 * ((lane / 8) & 1)) * kPitch + 16 * (lane / 16));

    #pragma unroll 1
    for (int tile = 0; tile < kSelTiles; ++tile) {
        unsigned live = 0;   // bit r: slot r of the tile holds a key
        #pragma unroll
        for (int r = 0; r < kSelTile; ++r) live |= unsigned(tokens[tile * kSelTile + r] >= 0) << r;
        if (!live) continue;
        if (!mbar_wait(&bars[tile], 0)) { if (lane == 0) atomicExch(a.status, 1); drain_delay(); return; }
        const uint8_t* kt = smem + size_t(tile) * kSelTileBytes;
        const uint8_t* vt = kt + kSelTile * kPitch;
        const uint32_t vt_address = smem_u32(vt);
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if constexpr (F16) {
            // ---- S = K Q^T: the rows' halves are the A fragments (columns 32 b + 8 t .. + 7 of rows r0 and r1 a block) ----
            #pragma unroll
            for (int b = 0; b < 8; ++b) {
                const uint4 w0 = *reinterpret_cast<const uint4*>(kt + r0 * kPitch + 64 * b + 16 * t);
                const uint4 w1 = *reinterpret_cast<const uint4*>(kt + r1 * kPitch + 64 * b + 16 * t);
                const uint32_t af[4] = {w0.x, w1.x, w0.y, w1.y}, ag[4] = {w0.z, w1.z, w0.w, w1.w};
                mma_f16(s, af, ql[b][0], ql[b][1]);
                mma_f16(s, af, qh[b][0], qh[b][1]);
                mma_f16(s, ag, ql[b][2], ql[b][3]);
                mma_f16(s, ag, qh[b][2], qh[b][3]);
            }
        } else {
        // ---- S = K Q^T per 32-column block, then the block's scale (rows nobody fetched hold stale bytes: masked below) ----
        const uint4 ks0 = *reinterpret_cast<const uint4*>(kt + r0 * kv_row_q8 + 256);
        const uint4 ks1 = *reinterpret_cast<const uint4*>(kt + r1 * kv_row_q8 + 256);
        #pragma unroll
        for (int b = 0; b < 8; ++b) {
            uint2 w0 = *reinterpret_cast<const uint2*>(kt + r0 * kv_row_q8 + 32 * b + 8 * t);
            uint2 w1 = *reinterpret_cast<const uint2*>(kt + r1 * kv_row_q8 + 32 * b + 8 * t);
            w0.x ^= 0x80808080u; w0.y ^= 0x80808080u; w1.x ^= 0x80808080u; w1.y ^= 0x80808080u;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const uint32_t af[4] = {sel_bytes01(w0.x), sel_bytes01(w1.x), sel_bytes23(w0.x), sel_bytes23(w1.x)};
            mma_f16(acc, af, ql[b][0], ql[b][1]);
            mma_f16(acc, af, qh[b][0], qh[b][1]);
            const uint32_t ag[4] = {sel_bytes01(w0.y), sel_bytes01(w1.y), sel_bytes23(w0.y), sel_bytes23(w1.y)};
            mma_f16(acc, ag, ql[b][2], ql[b][3]);
            mma_f16(acc, ag, qh[b][2], qh[b][3]);
            const float c0 = (live >> r0 & 1) ? sel_half_at(ks0, b) : 0.0f, c1 = (live >> r1 & 1) ? sel_half_at(ks1, b) : 0.0f;
            s[0] = fmaf(acc[0], c0, s[0]); s[1] = fmaf(acc[1], c0, s[1]);
            s[2] = fmaf(acc[2], c1, s[2]); s[3] = fmaf(acc[3], c1, s[3]);
        }
        }
        const bool live0 = live >> r0 & 1, live1 = live >> r1 & 1;
        float x[4] = {live0 ? s[0] * a.scale_log2 : -INFINITY, live0 ? s[1] * a.scale_log2 : -INFINITY,
                      live1 ? s[2] * a.scale_log2 : -INFINITY, live1 ? s[3] * a.scale_log2 : -INFINITY};
        float top0 = fmaxf(x[0], x[2]), top1 = fmaxf(x[1], x[3]);
        #pragma unroll
        for (int offset = 4; offset < 32; offset *= 2) {
            top0 = fmaxf(top0, __shfl_xor_sync(0xffffffffu, top0, offset));
            top1 = fmaxf(top1, __shfl_xor_sync(0xffffffffu, top1, offset));
        }
        const float n0 = fmaxf(m0, top0), n1 = fmaxf(m1, top1);
        // (a score may be -inf or NaN only through a query that is: the maxima of a tile with a live key are taken as they come)
        const float f0 = m0 == n0 ? 1.0f : fast_exp2(m0 - n0), f1 = m1 == n1 ? 1.0f : fast_exp2(m1 - n1);
        l0 *= f0; l1 *= f1;
        #pragma unroll
        for (int b = 0; b < 8; ++b)
            #pragma unroll
            for (int i = 0; i < 2; ++i) { o[b][i][0] *= f0; o[b][i][1] *= f1; o[b][i][2] *= f0; o[b][i][3] *= f1; }
        m0 = n0; m1 = n1;
        float p[4] = {live0 ? fast_exp2(x[0] - m0) : 0.0f, live0 ? fast_exp2(x[1] - m1) : 0.0f,
                      live1 ? fast_exp2(x[2] - m0) : 0.0f, live1 ? fast_exp2(x[3] - m1) : 0.0f};
        l0 += p[0] + p[2]; l1 += p[1] + p[3];
        // ---- transpose P (keys x heads) into B-fragment order: lane (g, t) gets head g, keys ka, kb, ka + 8, kb + 8 ----
        float pa, pb, pc, pd;
        {
            const uint32_t u0 = __float_as_uint(p[0]), u1 = __float_as_uint(p[1]), u2 = __float_as_uint(p[2]), u3 = __float_as_uint(p[3]);
            const uint32_t lo = movmatrix_trans(prmt(u0, u1, 0x5410u)), hi = movmatrix_trans(prmt(u0, u1, 0x7632u));
            pa = __uint_as_float(prmt(lo, hi, 0x5410u)); pb = __uint_as_float(prmt(lo, hi, 0x7632u));
            const uint32_t lo2 = movmatrix_trans(prmt(u2, u3, 0x5410u)), hi2 = movmatrix_trans(prmt(u2, u3, 0x7632u));
            pc = __uint_as_float(prmt(lo2, hi2, 0x5410u)); pd = __uint_as_float(prmt(lo2, hi2, 0x7632u));
        }
        if constexpr (F16) {
            // ---- O^T += V^T P: P as hi + lo; the value fragments of a 16-column piece through one transposing ldmatrix ----
            uint32_t ph0, pl0, ph1, pl1;
            split_pair(pa, pb, ph0, pl0);
            split_pair(pc, pd, ph1, pl1);
            #pragma unroll
            for (int b = 0; b < 8; ++b)
                #pragma unroll
                for (int i = 0; i < 2; ++i) {
                    uint32_t w[4];
                    ldmatrix_x4_trans(w, vt_address + v_lane + 64 * b + 32 * i);
                    mma_f16(o[b][i], w, pl0, pl1);
                    mma_f16(o[b][i], w, ph0, ph1);
                }
            continue;
        }
        // ---- O^T += V^T P': the value block's scale folded into P' in FP32, P' as hi + lo ----
        uint4 va = *reinterpret_cast<const uint4*>(vt + ka * kv_row_q8 + 256);
        uint4 vb = *reinterpret_cast<const uint4*>(vt + kb * kv_row_q8 + 256);
        uint4 vc = *reinterpret_cast<const uint4*>(vt + (ka + 8) * kv_row_q8 + 256);
        uint4 vd = *reinterpret_cast<const uint4*>(vt + (kb + 8) * kv_row_q8 + 256);
        if (!(live >> ka & 1)) va = make_uint4(0, 0, 0, 0);
        if (!(live >> kb & 1)) vb = make_uint4(0, 0, 0, 0);
        if (!(live >> (ka + 8) & 1)) vc = make_uint4(0, 0, 0, 0);
        if (!(live >> (kb + 8) & 1)) vd = make_uint4(0, 0, 0, 0);
        #pragma unroll
        for (int b = 0; b < 8; ++b) {
            uint32_t ph0, pl0, ph1, pl1;
            split_pair(pa * sel_half_at(va, b), pb * sel_half_at(vb, b), ph0, pl0);
            split_pair(pc * sel_half_at(vc, b), pd * sel_half_at(vd, b), ph1, pl1);
            // w[0], w[1]: columns 32b + 2g, + 1 of keys (ka, kb) and (ka + 8, kb + 8); w[2], w[3]: columns 32b + 16 + 2g, + 1
            uint32_t w[4];
            ldmatrix_x4_trans(w, vt_address + v_lane + 32 * b);
            w[0] ^= 0x80808080u; w[1] ^= 0x80808080u; w[2] ^= 0x80808080u; w[3] ^= 0x80808080u;
            const uint32_t af[4] = {bytes02_to_half2(w[0]), bytes13_to_half2(w[0]), bytes02_to_half2(w[1]), bytes13_to_half2(w[1])};
            mma_f16(o[b][0], af, pl0, pl1);
            mma_f16(o[b][0], af, ph0, ph1);
            const uint32_t ag[4] = {bytes02_to_half2(w[2]), bytes13_to_half2(w[2]), bytes02_to_half2(w[3]), bytes13_to_half2(w[3])};
            mma_f16(o[b][1], ag, pl0, pl1);
            mma_f16(o[b][1], ag, ph0, ph1);
        }
    }
    // ---- the chunk's partial: o[b][i][c] is head 2t + (c & 1) of this warp's eight, column 32b + 16i + 2g + (c >> 1)
    //      (FP16 rows: column 32b + 16i + g + 8 (c >> 1), the tensor cores' own order) ----
    #pragma unroll
    for (int offset = 4; offset < 32; offset *= 2) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, offset);
        l1 += __shfl_xor_sync(0xffffffffu, l1, offset);
    }
    #pragma unroll
    for (int which = 0; which < 2; ++which) {
        const size_t head = size_t(warp) * 8 + 2 * t + which;
        if (head >= a.group) continue;
        float* mine = a.partial + ((row * a.heads + kv * a.group + head) * a.chunks + chunk) * 258;
        #pragma unroll
        for (int b = 0; b < 8; ++b)
            #pragma unroll
            for (int i = 0; i < 2; ++i) {
                if constexpr (F16) {
                    mine[32 * b + 16 * i + g] = o[b][i][which];
                    mine[32 * b + 16 * i + g + 8] = o[b][i][2 + which];
                } else {
                    const int column = 32 * b + 16 * i + 2 * g;
                    *reinterpret_cast<float2*>(mine + column) = make_float2(o[b][i][which], o[b][i][2 + which]);
                }
            }
        if (g == 0) { mine[256] = which ? m1 : m0; mine[257] = which ? l1 : l0; }
    }
}

// Block = (query head, row); thread = output column. A row's chunks combined in chunk order as qsa_decode_merge does
// (gpu/sparse_attention_compute.hpp:139-170; maxima in the exp2 domain here): M = max of maxima, factor = exp2(max - M), 0 for a
// chunk without a live key, out = sum factor * acc / sum factor * denominator, times sigmoid(gate) when gates are given (:168).
__global__ void __launch_bounds__(256) qsa_select_merge_kernel(const SelectArgs a, const float* __restrict__ gates, size_t gate_stride,
                                                               float* __restrict__ out) {
    const size_t head = blockIdx.x, row = a.row0 + blockIdx.y, column = threadIdx.x;
    const size_t index_start = a.steps * (a.heads * 256 + a.kv_heads * 512);
    const size_t count = size_t(a.input[index_start + a.steps * a.selected + row]);
    const size_t used = min((count + kSelChunk - 1) / kSelChunk, a.chunks);
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the chunks' partials are complete and visible from here on
    const float* source = a.partial + (row * a.heads + head) * a.chunks * 258;
    float top = -INFINITY;
    for (size_t c = 0; c < used; ++c) top = fmaxf(top, source[c * 258 + 256]);
    float numerator = 0.0f, denominator = 0.0f;
    for (size_t c = 0; c < used; ++c) {
        const float own = source[c * 258 + 256];
        const float factor = own == -INFINITY ? 0.0f : fast_exp2(own - top);
        denominator = fmaf(factor, source[c * 258 + 257], denominator);
        numerator = fmaf(factor, source[c * 258 + column], numerator);
    }
    float value = numerator / denominator;
    if (gates) {
        const float x = gates[row * gate_stride + head * 512 + 256 + column];   // (a head's query and gate lie side by side)
        const float e = expf(-fabsf(x));
        value *= x >= 0 ? 1.0f / (1.0f + e) : e / (1.0f + e);   // gpu/core.hpp:1108-1111
    }
    out[(row * a.heads + head) * 256 + column] = value;
}

// Rows [row0, row0 + rows) of the packed rows: the chunks' kernel, then the merge.
static void launch_select(Device& value, SelectArgs& args, size_t row0, size_t rows, float scale, const float* gates, size_t gate_stride, float* out) {
    args.row0 = row0;
    // the chunks' partials: a library-owned workspace, grown on the first call of a size (make that call outside a stream capture)
    args.partial = static_cast<float*>(ensure(value, value.partial, value.partial_bytes, checked_product({args.steps, args.heads, args.chunks, 258, 4})));
    args.scale_log2 = scale * 1.4426950408889634f;
    args.status = status_word(value);
    static bool configured[64] = {};
    if (!configured[value.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(qsa_select_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SelShape<false>::kSmem)));
        SDB_CHECK(cudaFuncSetAttribute(qsa_select_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SelShape<true>::kSmem)));
        configured[value.ordinal & 63] = true;
    }
    const unsigned warps = unsigned((args.group + 7) / 8);
    const dim3 grid(unsigned(args.chunks), unsigned(args.kv_heads), unsigned(rows));
    if (value.kv_row == kv_row_f16) qsa_select_kernel<true><<<grid, 32 * warps, SelShape<true>::kSmem, value.stream>>>(args);
    else qsa_select_kernel<false><<<grid, 32 * warps, SelShape<false>::kSmem, value.stream>>>(args);
    // programmatic dependent launch: the merge's blocks are placed while the chunks' kernel drains and start at its end
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(unsigned(args.heads), unsigned(rows));
    config.blockDim = dim3(256);
    config.stream = value.stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    SDB_CHECK(cudaLaunchKernelEx(&config, qsa_select_merge_kernel, static_cast<const SelectArgs>(args), gates, gate_stride, out));
    value.launches += 2;
}

// ---- a batch's selections over a K/V in host memory: the union of the selected 4-row blocks copied into the VRAM stage once ----
// What it replaces in the reference: qsa_mark_selection, qsa_place_union, qsa_gather_union, qsa_renumber_selection
// (gpu/sparse_attention_compute.hpp:680-734) under qsa_attention_gathered (gpu/prefill_batch.hpp:227-252). Nearby tokens select
// overlapping blocks; read over the bus once per token they would cost the bus many times over, so the union goes to the stage in
// block order and every selection is renumbered to it: a row reads the same keys and values in the same order, so the same bits.
// marks[block] = 1 for every block a live slot of rows [first, first + gridDim.x) names (a live slot: the chunks' kernel's rule).
__global__ void __launch_bounds__(256) union_mark_kernel(const SelectArgs a, size_t first, uint32_t* __restrict__ marks) {
    const size_t row = first + blockIdx.x, index_start = a.steps * (a.heads * 256 + a.kv_heads * 512);
    const float* indices = a.input + index_start + row * a.selected;
    const size_t count = min(a.selected, size_t(a.input[index_start + a.steps * a.selected + row]));
    const float limit = float(a.position ? size_t(a.position[row]) : a.base + row);
    for (size_t i = threadIdx.x; i < count; i += 256) {
        const float raw = indices[i];
        if (raw >= 0 && raw <= limit && raw < float(a.context)) marks[size_t(raw) / 4] = 1u;
    }
}
// marks[block] becomes the number of marked blocks before it, blocks[place] the block in that place, marks[end] the count: one
// CTA of 1024 threads, each a run of blocks, the runs' counts scanned by warp shuffles.
__global__ void __launch_bounds__(1024) union_place_kernel(uint32_t* __restrict__ marks, size_t end, uint32_t* __restrict__ blocks) {
    __shared__ unsigned warp_totals[32];
    const unsigned t = threadIdx.x, lane = t % 32, warp = t / 32;
    const size_t per = (end + 1023) / 1024, from = min(end, size_t(t) * per), to = min(end, from + per);
    unsigned own = 0;
    for (size_t block = from; block < to; ++block) own += marks[block] != 0;
    unsigned inclusive = own;
    #pragma unroll
    for (int offset = 1; offset < 32; offset *= 2) {
        const unsigned other = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if (lane >= unsigned(offset)) inclusive += other;
    }
    if (lane == 31) warp_totals[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
        unsigned total = warp_totals[lane], scanned = total;
        #pragma unroll
        for (int offset = 1; offset < 32; offset *= 2) {
            const unsigned other = __shfl_up_sync(0xffffffffu, scanned, offset);
            if (lane >= unsigned(offset)) scanned += other;
        }
        warp_totals[lane] = scanned - total;   // exclusive
        if (lane == 31) marks[end] = scanned;
    }
    __syncthreads();
    unsigned at = warp_totals[warp] + inclusive - own;
    for (size_t block = from; block < to; ++block) {
        const bool marked = marks[block] != 0;
        marks[block] = at;
        if (marked) blocks[at++] = uint32_t(block);
    }
}
// Union place p's four rows of every plane, from the K/V into rows 4 p .. 4 p + 3 of the stage; a CTA per place, 16-byte pieces.
__global__ void __launch_bounds__(256) union_gather_kernel(const uint8_t* __restrict__ state, size_t context, size_t planes,
                                                           const uint32_t* __restrict__ blocks, const uint32_t* __restrict__ total,
                                                           uint8_t* __restrict__ stage, size_t capacity, size_t kv_row) {
    const size_t pieces = kv_row / 16;
    const size_t place = blockIdx.x;
    if (place >= *total) return;
    const size_t block = blocks[place];
    for (size_t i = threadIdx.x; i < planes * 4 * pieces; i += 256) {
        const size_t plane = i / (4 * pieces), row = i / pieces % 4, piece = i % pieces, position = block * 4 + row;
        if (position >= context) continue;
        reinterpret_cast<uint4*>(stage + (plane * capacity + place * 4 + row) * kv_row)[piece] =
            __ldg(reinterpret_cast<const uint4*>(state + (plane * context + position) * kv_row) + piece);
    }
}
// Rows [first, first + gridDim.x)'s selections renumbered to the union's places, into the library's copy of the packed rows (the
// caller's stay as they are); a slot that was not live becomes -1, which no rule makes live.
__global__ void __launch_bounds__(256) union_renumber_kernel(const SelectArgs a, size_t first, const uint32_t* __restrict__ places,
                                                             float* __restrict__ renumbered) {
    const size_t row = first + blockIdx.x, index_start = a.steps * (a.heads * 256 + a.kv_heads * 512);
    const float* indices = a.input + index_start + row * a.selected;
    float* target = renumbered + index_start + row * a.selected;
    const size_t count = min(a.selected, size_t(a.input[index_start + a.steps * a.selected + row]));
    const float limit = float(a.position ? size_t(a.position[row]) : a.base + row);
    for (size_t i = threadIdx.x; i < count; i += 256) {
        const float raw = indices[i];
        const bool live = raw >= 0 && raw <= limit && raw < float(a.context);
        const size_t index = live ? size_t(raw) : 0;
        target[i] = live ? float(size_t(places[index / 4]) * 4 + index % 4) : -1.0f;
    }
}

}  // namespace sdb

using namespace sdb;

extern "C" int sdx_qsa_attention_rows(void* handle, const void* state, uint64_t context, uint64_t base, const uint32_t* positions,
                                      uint64_t steps, uint64_t selected, uint64_t heads, uint64_t kv_heads, float scale, const float* input,
                                      const void* mirror, uint64_t mirror_rows, const float* gates, uint64_t gate_stride, float* out) {
    SDB_OP_BEGIN
    const uint64_t group = kv_heads ? heads / kv_heads : 0;
    if (!context || context > (uint64_t(1) << 24) || !steps || steps > max_batch || !selected || selected > 8192 || !heads || !kv_heads ||
        heads % kv_heads || group > 16 || kv_heads > 65535 || (mirror && !mirror_rows) || base > context)
        throw std::runtime_error("invalid Straydog attention dimensions");
    const size_t packed = checked_product({steps, heads * 256 + kv_heads * 512 + selected + 1, 4});
    span(value, state, checked_product({context, 2 * kv_heads, value.kv_row}), "a K/V state");
    span(value, input, packed, "packed attention rows");
    span(value, out, checked_product({steps, heads, 256, 4}), "an attention output");
    if (positions) span(value, positions, steps * 4, "attention positions");
    if (mirror) span(value, mirror, checked_product({mirror_rows, 2 * kv_heads, value.kv_row}), "a K/V mirror");
    if (gates) span(value, gates, checked_product({(steps - 1) * gate_stride + heads * 512, 4}), "attention gates");
    if (reinterpret_cast<uintptr_t>(state) % 16 || reinterpret_cast<uintptr_t>(mirror) % 16 || reinterpret_cast<uintptr_t>(input) % 16)
        throw std::runtime_error("Straydog attention operands must be 16-byte aligned");
    SelectArgs args{};
    args.state = static_cast<const uint8_t*>(state);
    args.mirror = static_cast<const uint8_t*>(mirror);
    args.context = context; args.mirror_rows = mirror_rows; args.base = base; args.steps = steps; args.selected = selected;
    args.heads = heads; args.kv_heads = kv_heads; args.group = group;
    args.chunks = (selected + kSelChunk - 1) / kSelChunk;
    args.position = positions;
    args.input = input;
    launch_select(value, args, 0, steps, scale, gates, gate_stride, out);
    SDB_OP_END
}

// Selection-list attention over a K/V that lies in host memory (sd_host_state), through the VRAM stage registered with sd_kv_stage:
// as many rows at a time as the stage holds the union of (halved until it does, one host read of the union's size per attempt, as
// gpu/prefill_batch.hpp:232-250 does); a stage that cannot hold one row's selection is refused. The result is
// sdx_qsa_attention_rows' over the same state bit for bit. `passes` (optional) receives how many groups of rows the call made.
extern "C" int sdx_qsa_attention_gathered(void* handle, const void* state, uint64_t context, uint64_t base, const uint32_t* positions,
                                          uint64_t steps, uint64_t selected, uint64_t heads, uint64_t kv_heads, float scale, const float* input,
                                          const float* gates, uint64_t gate_stride, float* out, uint64_t* passes) {
    SDB_OP_BEGIN
    const uint64_t group = kv_heads ? heads / kv_heads : 0;
    if (!context || context > (uint64_t(1) << 24) || !steps || steps > max_batch || !selected || selected > 8192 || !heads || !kv_heads ||
        heads % kv_heads || group > 16 || kv_heads > 65535 || base > context)
        throw std::runtime_error("invalid Straydog attention dimensions");
    if (!value.kv_stage) throw std::runtime_error("no Straydog K/V stage is registered");
    const size_t planes = 2 * kv_heads, capacity = size_t(value.kv_stage_rows) * 4096 / (value.kv_row * planes);
    if (capacity < 4) throw std::runtime_error("invalid Straydog K/V stage");
    const size_t packed = checked_product({steps, heads * 256 + kv_heads * 512 + selected + 1, 4});
    span(value, state, checked_product({context, planes, value.kv_row}), "a K/V state");
    span(value, input, packed, "packed attention rows");
    span(value, out, checked_product({steps, heads, 256, 4}), "an attention output");
    if (positions) span(value, positions, steps * 4, "attention positions");
    if (gates) span(value, gates, checked_product({(steps - 1) * gate_stride + heads * 512, 4}), "attention gates");
    if (reinterpret_cast<uintptr_t>(state) % 16 || reinterpret_cast<uintptr_t>(input) % 16)
        throw std::runtime_error("Straydog attention operands must be 16-byte aligned");
    SelectArgs args{};
    args.state = static_cast<const uint8_t*>(state);
    args.context = context; args.base = base; args.steps = steps; args.selected = selected;
    args.heads = heads; args.kv_heads = kv_heads; args.group = group;
    args.chunks = (selected + kSelChunk - 1) / kSelChunk;
    args.position = positions;
    args.input = input;
    // the workspace: places (end + 1 words), blocks (end words), then the renumbered copy of the packed rows
    const size_t end = (context + 3) / 4, words = (2 * end + 1 + 3) / 4 * 4;
    auto* places = static_cast<uint32_t*>(ensure(value, value.unions, value.unions_bytes, words * 4 + packed));
    uint32_t* blocks = places + end + 1;
    float* renumbered = reinterpret_cast<float*>(places + words);
    SDB_CHECK(cudaMemcpyAsync(renumbered, input, packed, cudaMemcpyDeviceToDevice, value.stream));
    auto* stage = static_cast<uint8_t*>(value.kv_stage);
    uint64_t made = 0;
    for (size_t first = 0; first < steps; ++made) {
        size_t count = steps - first;
        uint32_t total = 0;
        for (;;) {
            SDB_CHECK(cudaMemsetAsync(places, 0, (end + 1) * 4, value.stream));
            union_mark_kernel<<<unsigned(count), 256, 0, value.stream>>>(args, first, places);
            union_place_kernel<<<1, 1024, 0, value.stream>>>(places, end, blocks);
            value.launches += 2;
            SDB_CHECK(cudaMemcpyAsync(&total, places + end, 4, cudaMemcpyDeviceToHost, value.stream));
            SDB_CHECK(cudaStreamSynchronize(value.stream));
            if (size_t(total) * 4 <= capacity || count == 1) break;
            count = (count + 1) / 2;
        }
        if (size_t(total) * 4 <= capacity) {
            if (total) {
                union_gather_kernel<<<total, 256, 0, value.stream>>>(args.state, context, planes, blocks, places + end, stage, capacity, value.kv_row);
                ++value.launches;
            }
            union_renumber_kernel<<<unsigned(count), 256, 0, value.stream>>>(args, first, places, renumbered);
            ++value.launches;
            SelectArgs staged = args;
            staged.state = stage; staged.context = capacity; staged.input = renumbered;
            launch_select(value, staged, first, count, scale, gates, gate_stride, out);
        } else
            // (the reference lets such a row read the host rows directly; the chunks' kernel fetches rows with the bulk-copy engine, which is
            //  kept to device memory here, so a stage that cannot hold one row's selection is refused: 4 * selected positions always do)
            throw std::runtime_error("the Straydog K/V stage is too small for one row's selection");
        first += count;
    }
    if (passes) *passes = made;
    SDB_OP_END
}
