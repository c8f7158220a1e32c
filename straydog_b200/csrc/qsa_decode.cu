// Grouped-query decode attention over Q8_0 K/V rows, split-K flash decoding for sm_100a.
//
// What it replaces in the reference: qsa_decode_parts + qsa_decode_merge
// (gpu/sparse_attention_compute.hpp:41-170) behind qsa_attention / qsa_attention_rows (:609-647),
// generalised from "24 query / 2 KV heads, <= 2052 selected keys of one sequence" to any group of
// <= 8 query heads per KV head (an even group of up to 16, the reference's own 12 among them, as two halves that stream
// the K/V head's rows once each), dense causal key ranges and many sequences in one launch.
//
// Design (one persistent CTA per SM, 8 independent warps):
//   * The batch's (sequence, KV head) segments are laid end to end as a sequence of 16-key tiles and
//     cut into equal contiguous runs, one per warp (stream-K): every warp streams the same number of
//     bytes whatever the sequences' lengths. A run crosses segment borders as separate "pieces".
//   * Each warp owns a ring of STAGES tiles in shared memory. A tile is 16 consecutive K rows and the
//     same 16 V rows (2 x 4352 contiguous bytes), fetched by two bulk copies (TMA engine) that complete
//     on the tile's mbarrier; the warp refills a slot as soon as it has consumed it, so STAGES-1 tiles
//     per warp are always in flight.
//   * Arithmetic: int8 -> FP16 is exact, so Q.K^T runs on mma.sync.m16n8k16 with the 16 keys as M,
//     the 8 query heads of the group as N and one 32-column Q8_0 block per two MMAs; the block's FP32
//     sum is multiplied by the key's FP16 block scale in FP32 (the reference multiplies each value by
//     the scale before its FMA: the same number up to one rounding). P.V runs as V^T (16 columns x 16
//     keys, raw int8 as FP16) times P' (keys x heads), where P' = p * (value block scale) rounded to
//     FP16 once; accumulation is FP32 throughout. Online softmax per warp in the exp2 domain.
//   * Every piece leaves (unnormalised sum[8][256], max, denominator) in a partial slot; a merge
//     kernel combines a segment's pieces exactly as qsa_decode_merge does (:139-170).
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

#include <algorithm>
#include <cstdlib>
#include <utility>

namespace sdb {

constexpr int kWarps = 8, kTileKeys = 16, kStages = 3;
constexpr int kTileBytes = 2 * kTileKeys * int(kv_row_q8);   // K rows then V rows: 8704
constexpr int kPartialFloats = 8 * 258;                      // per piece: 8 heads x (256 sums, max, denominator)
constexpr size_t kDecodeSmem = size_t(kWarps) * kStages * kTileBytes + size_t(kWarps) * kStages * 8 + 16;

struct Piece { uint32_t segment, begin, end, slot; };   // slot: the piece's partial, counted in the segment's own order

struct DecodeArgs {
    const Segment* segments;
    const Piece* pieces;
    const uint32_t* warp_piece;   // [virtual warps + 1]
    const __half* q;
    float* partial;
    uint32_t virtual_warps, ctas;
    uint32_t group;               // query heads a segment (<= 8)
    float scale_log2;             // softmax scale * log2(e)
    int* status;                  // set to 1 when a bounded wait gave up
};

// Row of the tile held by the MMA fragment row `g` (0..7); rows g + 8 follow the same map + 8.
// Even rows go to lanes 0..15 and odd rows to lanes 16..31, which keeps the 8-byte key loads of a
// half warp on 32 distinct banks with 272-byte rows.
__device__ __forceinline__ int tile_row(int g) { return 2 * (g & 3) + (g >> 2); }

// Four int8 (a 32-bit word, already xor 0x80808080) -> two FP16 pairs, exactly: 0x64xx is 1024 + xx.
__device__ __forceinline__ uint32_t bytes01_to_half2(uint32_t x) {
    const uint32_t h = prmt(x, 0x64646464u, 0x4140u);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bytes23_to_half2(uint32_t x) {
    const uint32_t h = prmt(x, 0x64646464u, 0x4342u);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ float half_at(const uint4& v, int i) {
    const uint32_t w = i < 2 ? v.x : i < 4 ? v.y : i < 6 ? v.z : v.w;
    return __half2float(__ushort_as_half(uint16_t(i & 1 ? w >> 16 : w & 0xffffu)));
}

// The walk of one warp over its pieces' tiles, used twice: by the cursor that issues copies and by
// the one that consumes them.
struct Cursor {
    uint32_t piece, piece_end, key, key_end;
    const uint8_t* keys;
    const uint8_t* values;
    __device__ __forceinline__ void load(const DecodeArgs& a) {
        if (piece >= piece_end) return;
        const Piece p = a.pieces[piece];
        const Segment s = a.segments[p.segment];
        key = p.begin; key_end = min(p.end, s.length); keys = s.keys; values = s.values;
    }
    __device__ __forceinline__ bool done() const { return piece >= piece_end; }
};

__global__ void __launch_bounds__(kWarps * 32, 1) qsa_decode_kernel(const DecodeArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane / 4, t = lane % 4;
    uint8_t* ring = smem + size_t(warp) * kStages * kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + size_t(kWarps) * kStages * kTileBytes) + warp * kStages;
    if (lane == 0)
        for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    __syncthreads();
    // the merge launched behind this kernel may take its place on the SMs now: it waits for this grid's end before it reads
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // virtual warp v runs on CTA v % ctas: few warps spread over many SMs rather than filling one
    const uint32_t vwarp = uint32_t(warp) * a.ctas + blockIdx.x;
    if (vwarp >= a.virtual_warps) return;

    Cursor issue{a.warp_piece[vwarp], a.warp_piece[vwarp + 1], 0, 0, nullptr, nullptr};
    Cursor use = issue;
    if (issue.done()) return;
    issue.load(a);
    use.load(a);

    // lane 0 issues the tile at the issue cursor into `slot`
    auto fetch = [&](int slot) {
        if (issue.done()) return;
        const uint32_t rows = min(uint32_t(kTileKeys), issue.key_end - issue.key), bytes = rows * kv_row_q8;
        if (lane == 0) {
            uint8_t* dst = ring + slot * kTileBytes;
            mbar_expect_tx(&bars[slot], 2 * bytes);
            bulk_g2s(dst, issue.keys + size_t(issue.key) * kv_row_q8, bytes, &bars[slot]);
            bulk_g2s(dst + kTileKeys * kv_row_q8, issue.values + size_t(issue.key) * kv_row_q8, bytes, &bars[slot]);
        }
        issue.key += rows;
        if (issue.key >= issue.key_end) { ++issue.piece; issue.load(a); }
    };
    #pragma unroll
    for (int s = 0; s < kStages - 1; ++s) fetch(s);

    const int r0 = tile_row(g), r1 = r0 + 8;
    const int ka = tile_row(2 * t), kb = tile_row(2 * t + 1);   // the keys whose P this lane holds after the transpose
    // The value bytes of a 32-column block reach the lanes through one transposing ldmatrix: a 16-bit unit is two columns of one key,
    // matrix m holds keys (k-index j -> key tile_row(j) + 8 (m & 1)) and the units of columns 16 (m >> 1) ..: lane (g, t) then has,
    // per matrix, columns 2g and 2g + 1 of the keys ka (+8) and kb (+8), the k-indices 2t and 2t + 1 its weights sit at.
    const uint32_t v_lane = uint32_t((tile_row(lane % 8) + 8 * ((lane / 8) & 1)) * int(kv_row_q8) + 16 * (lane / 16));
    uint32_t slot = 0, phase = 0, fill = kStages - 1;

    while (!use.done()) {
        // ---- per piece: this segment's queries as B fragments, fresh softmax state ----
        const Piece piece = a.pieces[use.piece];
        const Segment segment = a.segments[piece.segment];
        uint32_t qf[8][4];
        {
            const __half* q = a.q + segment.q_offset + size_t(g) * 256 + 8 * t;
            #pragma unroll
            for (int b = 0; b < 8; ++b) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (uint32_t(g) < a.group) v = *reinterpret_cast<const uint4*>(q + 32 * b);
                qf[b][0] = v.x; qf[b][1] = v.y; qf[b][2] = v.z; qf[b][3] = v.w;
            }
        }
        float o[8][2][4];
        #pragma unroll
        for (int b = 0; b < 8; ++b)
            #pragma unroll
            for (int i = 0; i < 2; ++i)
                #pragma unroll
                for (int c = 0; c < 4; ++c) o[b][i][c] = 0.0f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;   // heads 2t and 2t+1

        while (use.key < use.key_end) {
            const uint32_t rows = min(uint32_t(kTileKeys), use.key_end - use.key);
            // refill the slot consumed last iteration (all lanes are past their reads of it)
            __syncwarp();
            fetch(int(fill));
            fill = fill + 1 == kStages ? 0 : fill + 1;
            if (!mbar_wait(&bars[slot], phase)) { if (lane == 0) atomicExch(a.status, 1); drain_delay(); return; }
            const uint8_t* kt = ring + slot * kTileBytes;
            const uint8_t* vt = kt + kTileKeys * kv_row_q8;
            const uint32_t vt_address = smem_u32(vt);

            // ---- S = K Q^T: per 32-column block two MMAs into a fresh accumulator, then the block's scale ----
            const uint4 ks0 = *reinterpret_cast<const uint4*>(kt + r0 * kv_row_q8 + 256);
            const uint4 ks1 = *reinterpret_cast<const uint4*>(kt + r1 * kv_row_q8 + 256);
            float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            #pragma unroll
            for (int b = 0; b < 8; ++b) {
                uint2 w0 = *reinterpret_cast<const uint2*>(kt + r0 * kv_row_q8 + 32 * b + 8 * t);
                uint2 w1 = *reinterpret_cast<const uint2*>(kt + r1 * kv_row_q8 + 32 * b + 8 * t);
                w0.x ^= 0x80808080u; w0.y ^= 0x80808080u; w1.x ^= 0x80808080u; w1.y ^= 0x80808080u;
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                uint32_t af[4] = {bytes01_to_half2(w0.x), bytes01_to_half2(w1.x), bytes23_to_half2(w0.x), bytes23_to_half2(w1.x)};
                mma_f16(acc, af, qf[b][0], qf[b][1]);
                uint32_t ag[4] = {bytes01_to_half2(w0.y), bytes01_to_half2(w1.y), bytes23_to_half2(w0.y), bytes23_to_half2(w1.y)};
                mma_f16(acc, ag, qf[b][2], qf[b][3]);
                const float c0 = half_at(ks0, b), c1 = half_at(ks1, b);
                s[0] = fmaf(acc[0], c0, s[0]); s[1] = fmaf(acc[1], c0, s[1]);
                s[2] = fmaf(acc[2], c1, s[2]); s[3] = fmaf(acc[3], c1, s[3]);
            }
            // ---- online softmax (exp2 domain); s[0], s[1]: key r0, heads 2t, 2t+1; s[2], s[3]: key r1 ----
            const bool live0 = uint32_t(r0) < rows, live1 = uint32_t(r1) < rows;
            float x[4] = {live0 ? s[0] * a.scale_log2 : -INFINITY, live0 ? s[1] * a.scale_log2 : -INFINITY,
                          live1 ? s[2] * a.scale_log2 : -INFINITY, live1 ? s[3] * a.scale_log2 : -INFINITY};
            float top0 = fmaxf(x[0], x[2]), top1 = fmaxf(x[1], x[3]);
            #pragma unroll
            for (int offset = 4; offset < 32; offset *= 2) {
                top0 = fmaxf(top0, __shfl_xor_sync(0xffffffffu, top0, offset));
                top1 = fmaxf(top1, __shfl_xor_sync(0xffffffffu, top1, offset));
            }
            const float n0 = fmaxf(m0, top0), n1 = fmaxf(m1, top1);   // finite: every tile has a live key (row 0)
            if (__any_sync(0xffffffffu, n0 > m0 || n1 > m1)) {
                const float f0 = fast_exp2(m0 - n0), f1 = fast_exp2(m1 - n1);   // exp2(-inf) = 0 at the first tile
                l0 *= f0; l1 *= f1;
                #pragma unroll
                for (int b = 0; b < 8; ++b)
                    #pragma unroll
                    for (int i = 0; i < 2; ++i) { o[b][i][0] *= f0; o[b][i][1] *= f1; o[b][i][2] *= f0; o[b][i][3] *= f1; }
                m0 = n0; m1 = n1;
            }
            float p[4] = {fast_exp2(x[0] - m0), fast_exp2(x[1] - m1), fast_exp2(x[2] - m0), fast_exp2(x[3] - m1)};
            l0 += p[0] + p[2]; l1 += p[1] + p[3];
            // ---- transpose P (keys x heads, FP32) into B-fragment order: lane (g, t) gets head g, keys ka, kb, ka+8, kb+8 ----
            float pa, pb, pc, pd;
            {
                const uint32_t u0 = __float_as_uint(p[0]), u1 = __float_as_uint(p[1]), u2 = __float_as_uint(p[2]), u3 = __float_as_uint(p[3]);
                const uint32_t lo = movmatrix_trans(prmt(u0, u1, 0x5410u)), hi = movmatrix_trans(prmt(u0, u1, 0x7632u));
                pa = __uint_as_float(prmt(lo, hi, 0x5410u)); pb = __uint_as_float(prmt(lo, hi, 0x7632u));
                const uint32_t lo2 = movmatrix_trans(prmt(u2, u3, 0x5410u)), hi2 = movmatrix_trans(prmt(u2, u3, 0x7632u));
                pc = __uint_as_float(prmt(lo2, hi2, 0x5410u)); pd = __uint_as_float(prmt(lo2, hi2, 0x7632u));
            }
            // ---- O^T += V^T P': the value block's scale folded into P (FP32 product, one rounding to FP16) ----
            uint4 va = *reinterpret_cast<const uint4*>(vt + ka * kv_row_q8 + 256);
            uint4 vb = *reinterpret_cast<const uint4*>(vt + kb * kv_row_q8 + 256);
            uint4 vc = *reinterpret_cast<const uint4*>(vt + (ka + 8) * kv_row_q8 + 256);
            uint4 vd = *reinterpret_cast<const uint4*>(vt + (kb + 8) * kv_row_q8 + 256);
            if (rows < uint32_t(kTileKeys)) {   // rows past the piece hold stale bytes: their weights are 0, their scales must be too
                if (uint32_t(ka) >= rows) va = make_uint4(0, 0, 0, 0);
                if (uint32_t(kb) >= rows) vb = make_uint4(0, 0, 0, 0);
                if (uint32_t(ka + 8) >= rows) vc = make_uint4(0, 0, 0, 0);
                if (uint32_t(kb + 8) >= rows) vd = make_uint4(0, 0, 0, 0);
            }
            #pragma unroll
            for (int b = 0; b < 8; ++b) {
                const uint32_t pb0 = pack_half2(pa * half_at(va, b), pb * half_at(vb, b));
                const uint32_t pb1 = pack_half2(pc * half_at(vc, b), pd * half_at(vd, b));
                // w[0], w[1]: columns 32b + 2g, + 1 of keys (ka, kb) and (ka + 8, kb + 8); w[2], w[3]: columns 32b + 16 + 2g, + 1
                uint32_t w[4];
                ldmatrix_x4_trans(w, vt_address + v_lane + 32 * b);
                w[0] ^= 0x80808080u; w[1] ^= 0x80808080u; w[2] ^= 0x80808080u; w[3] ^= 0x80808080u;
                uint32_t af[4] = {bytes02_to_half2(w[0]), bytes13_to_half2(w[0]), bytes02_to_half2(w[1]), bytes13_to_half2(w[1])};
                mma_f16(o[b][0], af, pb0, pb1);
                uint32_t ag[4] = {bytes02_to_half2(w[2]), bytes13_to_half2(w[2]), bytes02_to_half2(w[3]), bytes13_to_half2(w[3])};
                mma_f16(o[b][1], ag, pb0, pb1);
            }
            use.key += rows;
            if (++slot == kStages) { slot = 0; phase ^= 1; }
        }
        // ---- the piece's partial: o[b][i][c] is head 2t + (c & 1), column 32b + 16i + 2g + (c >> 1) ----
        #pragma unroll
        for (int offset = 4; offset < 32; offset *= 2) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, offset);
            l1 += __shfl_xor_sync(0xffffffffu, l1, offset);
        }
        float* mine = a.partial + size_t(piece.slot) * kPartialFloats;
        #pragma unroll
        for (int b = 0; b < 8; ++b)
            #pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int column = 32 * b + 16 * i + 2 * g;
                *reinterpret_cast<float2*>(mine + (2 * t) * 258 + column) = make_float2(o[b][i][0], o[b][i][2]);
                *reinterpret_cast<float2*>(mine + (2 * t + 1) * 258 + column) = make_float2(o[b][i][1], o[b][i][3]);
            }
        if (g == 0) {
            mine[(2 * t) * 258 + 256] = m0; mine[(2 * t) * 258 + 257] = l0;
            mine[(2 * t + 1) * 258 + 256] = m1; mine[(2 * t + 1) * 258 + 257] = l1;
        }
        ++use.piece;
        use.load(a);
    }
}

// Block = (segment, head of the group); thread = output column. The pieces' partials combined as
// gpu/sparse_attention_compute.hpp:139-170 does: M = max of maxima, factor = exp(max - M) (here
// exp2: the maxima are kept in the exp2 domain), out = sum factor * acc / sum factor * denominator.
__global__ void __launch_bounds__(256) qsa_decode_merge_kernel(const Segment* __restrict__ segments, const float* __restrict__ partial,
                                                               uint32_t group, float* __restrict__ out) {
    const Segment segment = segments[blockIdx.x];   // (the work list: written before the streaming kernel was launched)
    const uint32_t head = blockIdx.y, column = threadIdx.x;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the streaming kernel's partials are complete and visible from here on
    const float* first = partial + size_t(segment.first_piece) * kPartialFloats + head * 258;
    float top = -INFINITY;
    for (uint32_t piece = 0; piece < segment.pieces; ++piece) top = fmaxf(top, first[size_t(piece) * kPartialFloats + 256]);
    float numerator = 0.0f, denominator = 0.0f;
    for (uint32_t piece = 0; piece < segment.pieces; ++piece) {
        const float* at = first + size_t(piece) * kPartialFloats;
        const float factor = fast_exp2(at[256] - top);
        denominator = fmaf(factor, at[257], denominator);
        numerator = fmaf(factor, at[column], numerator);
    }
    out[size_t(segment.q_offset) + size_t(head) * 256 + column] = numerator / denominator;
    (void)group;
}

// ---- host: the work list ----
struct DecodePlan {
    uint32_t segments = 0, pieces = 0, virtual_warps = 0, ctas = 0, group = 0;
    uint64_t sequences = 0, heads = 0, kv_heads = 0;
    uint64_t kv_bytes = 0;
    // device tables, one allocation: segments | pieces | warp_piece
    void* tables = nullptr;
    size_t segment_offset = 0, piece_offset = 0, warp_offset = 0, table_bytes = 0;
    float* partial = nullptr;
    int* status = nullptr;
    bool owns = false;
};

struct HostTables {
    std::vector<Segment> segments;
    std::vector<Piece> pieces;
    std::vector<uint32_t> warp_piece;
};

// The work list in its two forms.
//
// Fixed cuts (the default): a segment is cut at places that depend on its own length only - chunks of 32 tiles (512 keys; 8 tiles
// for a segment shorter than 512 tiles) and a tail that halves down to single tiles - and a chunk is never shared by two warps.
// The chunks are dealt to the warps longest first, each to the warp with the least work so far; the halving tails are what lets
// that come out even. A segment's partials are merged in chunk order, so a sequence's result has the same bits in any batch (the
// reference's verification contract, lines 40-41 of the reference's own design notes under docs/, kept for this library's own batched decode).
//
// Moving cuts: the segments' tiles laid end to end and cut into equal runs, one per warp. Fewer partials (one per warp and one
// per segment border), but where a segment is cut depends on what else is in the batch. Kept for sdx_qsa_decode_static, whose
// fixed scratch bounds the number of partials.
static void chunk_sizes(uint64_t tiles, std::vector<uint32_t>& out) {
    const uint64_t chunk = tiles >= 512 ? 32 : 8;
    out.clear();
    while (tiles >= 2 * chunk) { out.push_back(uint32_t(chunk)); tiles -= chunk; }
    while (tiles > 2) { const uint64_t take = (tiles + 1) / 2; out.push_back(uint32_t(take)); tiles -= take; }
    if (tiles) out.push_back(uint32_t(tiles));
}

// Segments a (sequence, K/V head): 1 for a group of up to eight query heads, 2 for a larger one (even, up to 16).
static uint64_t group_parts(uint64_t heads, uint64_t kv_heads) { return heads / kv_heads > 8 ? 2 : 1; }

static void build_tables(const std::vector<const uint8_t*>& states, const uint64_t* contexts, const uint64_t* lengths, uint64_t sequences,
                         uint64_t heads, uint64_t kv_heads, uint32_t warps_available, HostTables& out, bool fixed_cuts = true) {
    // A warp holds eight query heads: a larger (even) group is two segments a (sequence, K/V head), half the group's heads each.
    const uint64_t group = heads / kv_heads, parts = group_parts(heads, kv_heads), part_heads = group / parts;
    uint64_t total_tiles = 0;
    for (uint64_t s = 0; s < sequences; ++s) total_tiles += (lengths[s] + kTileKeys - 1) / kTileKeys * kv_heads * parts;
    constexpr uint64_t min_tiles = 8;
    out.segments.clear(); out.pieces.clear(); out.warp_piece.clear();
    auto segment_of = [&](uint64_t s, uint64_t unit) {   // unit = kv * parts + part
        const uint64_t kv = unit / parts, part = unit % parts;
        Segment segment{};
        segment.keys = states[s] + kv * contexts[s] * kv_row_q8;
        segment.values = states[s] + (kv_heads + kv) * contexts[s] * kv_row_q8;
        segment.q_offset = uint32_t((s * heads + kv * group + part * part_heads) * 256);
        segment.length = uint32_t(lengths[s]);
        return segment;
    };
    const uint64_t units = kv_heads * parts;
    if (fixed_cuts) {
        struct Chunk { uint32_t segment, begin, end, slot, tiles; };
        std::vector<Chunk> chunks;
        std::vector<uint32_t> sizes;
        for (uint64_t s = 0; s < sequences; ++s)
            for (uint64_t kv = 0; kv < units; ++kv) {
                Segment segment = segment_of(s, kv);
                segment.first_piece = uint32_t(chunks.size());
                chunk_sizes((lengths[s] + kTileKeys - 1) / kTileKeys, sizes);
                uint64_t key = 0;
                for (uint32_t tiles : sizes) {
                    // (a chunk ends at a tile border; the kernel stops at the segment's length, so a work list stays valid while
                    // its segments keep their tile counts)
                    const uint64_t end = key + uint64_t(tiles) * kTileKeys;
                    chunks.push_back(Chunk{uint32_t(out.segments.size()), uint32_t(key), uint32_t(end), uint32_t(chunks.size()), tiles});
                    key = end;
                }
                segment.pieces = uint32_t(chunks.size()) - segment.first_piece;
                out.segments.push_back(segment);
            }
        const uint32_t warps = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>(warps_available, total_tiles / min_tiles)));
        std::vector<uint32_t> order(chunks.size());
        for (uint32_t i = 0; i < order.size(); ++i) order[i] = i;
        std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return chunks[a].tiles > chunks[b].tiles; });
        // least-loaded warp first: a heap of (tiles so far, warp)
        std::vector<std::pair<uint64_t, uint32_t>> heap(warps);
        for (uint32_t w = 0; w < warps; ++w) heap[w] = {0, w};
        auto later = [](const std::pair<uint64_t, uint32_t>& a, const std::pair<uint64_t, uint32_t>& b) { return a > b; };
        std::vector<std::vector<uint32_t>> dealt(warps);
        for (uint32_t index : order) {
            std::pop_heap(heap.begin(), heap.end(), later);
            auto& least = heap.back();
            dealt[least.second].push_back(index);
            least.first += chunks[index].tiles;
            std::push_heap(heap.begin(), heap.end(), later);
        }
        for (uint32_t w = 0; w < warps; ++w) {
            out.warp_piece.push_back(uint32_t(out.pieces.size()));
            for (uint32_t index : dealt[w]) out.pieces.push_back(Piece{chunks[index].segment, chunks[index].begin, chunks[index].end, chunks[index].slot});
        }
        out.warp_piece.push_back(uint32_t(out.pieces.size()));
        return;
    }
    const uint64_t per_warp = std::max<uint64_t>(min_tiles, (total_tiles + warps_available - 1) / warps_available);
    out.warp_piece.push_back(0);
    uint64_t room = per_warp;   // tiles the current warp may still take
    for (uint64_t s = 0; s < sequences; ++s)
        for (uint64_t kv = 0; kv < units; ++kv) {
            Segment segment = segment_of(s, kv);
            segment.first_piece = uint32_t(out.pieces.size());
            uint64_t key = 0;
            while (key < lengths[s]) {
                if (!room) { out.warp_piece.push_back(uint32_t(out.pieces.size())); room = per_warp; }
                const uint64_t tiles_left = (lengths[s] - key + kTileKeys - 1) / kTileKeys, take = std::min(room, tiles_left);
                // (a piece ends at a tile border; the kernel stops at the segment's length, so a work list stays valid while its
                // segments keep their tile counts)
                const uint64_t end = key + take * kTileKeys;
                out.pieces.push_back(Piece{uint32_t(out.segments.size()), uint32_t(key), uint32_t(end), uint32_t(out.pieces.size())});
                room -= take;
                key = end;
            }
            segment.pieces = uint32_t(out.pieces.size()) - segment.first_piece;
            out.segments.push_back(segment);
        }
    out.warp_piece.push_back(uint32_t(out.pieces.size()));
}

static void validate_batch(Device& d, const void* const* states, const uint64_t* contexts, const uint64_t* lengths, uint64_t sequences,
                           uint64_t heads, uint64_t kv_heads, std::vector<const uint8_t*>& checked, uint64_t& kv_bytes) {
    if (d.kv_row != kv_row_q8) throw std::runtime_error("this Straydog build's decode attention reads Q8_0 K/V rows only");
    if (!states || !contexts || !lengths || !sequences || sequences > 65535 || !heads || !kv_heads || heads % kv_heads ||
        heads / kv_heads > 16 || (heads / kv_heads > 8 && heads / kv_heads % 2) || heads > 1024)
        throw std::runtime_error("invalid Straydog attention dimensions");
    checked.resize(sequences);
    kv_bytes = 0;
    for (uint64_t s = 0; s < sequences; ++s) {
        if (!contexts[s] || contexts[s] > (uint64_t(1) << 24) || !lengths[s] || lengths[s] > contexts[s])
            throw std::runtime_error("invalid Straydog attention dimensions");
        span(d, states[s], checked_product({contexts[s], 2 * kv_heads, kv_row_q8}), "a K/V state");
        if (reinterpret_cast<uintptr_t>(states[s]) % 16) throw std::runtime_error("a Straydog K/V state must be 16-byte aligned");
        checked[s] = static_cast<const uint8_t*>(states[s]);
        kv_bytes += lengths[s] * 2 * kv_heads * kv_row_q8;
    }
}

static void upload_tables(Device& d, const HostTables& host, DecodePlan& plan, void* tables, void* staging) {
    plan.segment_offset = 0;
    plan.piece_offset = (host.segments.size() * sizeof(Segment) + 255) / 256 * 256;
    plan.warp_offset = plan.piece_offset + (host.pieces.size() * sizeof(Piece) + 255) / 256 * 256;
    auto* stage = static_cast<uint8_t*>(staging);
    std::memcpy(stage + plan.segment_offset, host.segments.data(), host.segments.size() * sizeof(Segment));
    std::memcpy(stage + plan.piece_offset, host.pieces.data(), host.pieces.size() * sizeof(Piece));
    std::memcpy(stage + plan.warp_offset, host.warp_piece.data(), host.warp_piece.size() * 4);
    SDB_CHECK(cudaMemcpyAsync(tables, stage, plan.table_bytes, cudaMemcpyHostToDevice, d.stream));
    plan.tables = tables;
}

static size_t table_bytes_of(const HostTables& host) {
    return (host.segments.size() * sizeof(Segment) + 255) / 256 * 256 + (host.pieces.size() * sizeof(Piece) + 255) / 256 * 256 +
           host.warp_piece.size() * 4 + 256;
}

static void fill_plan(Device& d, const HostTables& host, DecodePlan& plan, uint64_t sequences, uint64_t heads, uint64_t kv_heads) {
    plan.segments = uint32_t(host.segments.size());
    plan.pieces = uint32_t(host.pieces.size());
    plan.virtual_warps = uint32_t(host.warp_piece.size() - 1);
    plan.ctas = std::min<uint32_t>(uint32_t(d.sms), plan.virtual_warps);
    plan.group = uint32_t(heads / kv_heads / group_parts(heads, kv_heads));   // query heads a segment
    plan.sequences = sequences; plan.heads = heads; plan.kv_heads = kv_heads;
    plan.table_bytes = table_bytes_of(host);
}

static void run_plan(Device& d, const DecodePlan& plan, float scale, const void* q, float* out, cudaEvent_t before = nullptr,
                     cudaEvent_t after = nullptr) {
    static bool configured[64] = {};
    if (!configured[d.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(qsa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kDecodeSmem)));
        configured[d.ordinal & 63] = true;
    }
    DecodeArgs args{};
    auto* base = static_cast<uint8_t*>(plan.tables);
    args.segments = reinterpret_cast<const Segment*>(base + plan.segment_offset);
    args.pieces = reinterpret_cast<const Piece*>(base + plan.piece_offset);
    args.warp_piece = reinterpret_cast<const uint32_t*>(base + plan.warp_offset);
    args.q = static_cast<const __half*>(q);
    args.partial = plan.partial;
    args.virtual_warps = plan.virtual_warps;
    args.ctas = plan.ctas;
    args.group = plan.group;
    args.scale_log2 = scale * 1.4426950408889634f;
    args.status = plan.status;
    if (before) SDB_CHECK(cudaEventRecord(before, d.stream));
    qsa_decode_kernel<<<plan.ctas, kWarps * 32, kDecodeSmem, d.stream>>>(args);
    if (after) SDB_CHECK(cudaEventRecord(after, d.stream));
    // programmatic dependent launch: the merge's blocks are placed while the streaming kernel drains and start at its end
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(plan.segments, plan.group);
    config.blockDim = dim3(256);
    config.stream = d.stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = after ? 0 : 1;   // (an event recorded between the two launches keeps the plain order)
    SDB_CHECK(cudaLaunchKernelEx(&config, qsa_decode_merge_kernel, args.segments, static_cast<const float*>(plan.partial), plan.group, out));
    d.launches += 2;
}

// The status word of the device's decode kernels (a wait that gave up sets it), read after a synchronising call.
int* status_word(Device& d) {
    static std::map<int, int*> words;
    static std::mutex mutex;
    std::lock_guard<std::mutex> lock(mutex);
    auto found = words.find(d.ordinal);
    if (found != words.end()) return found->second;
    int* word = nullptr;
    SDB_CHECK(cudaMalloc(&word, 256));
    SDB_CHECK(cudaMemset(word, 0, 256));
    words[d.ordinal] = word;
    return word;
}

void launch_kv_append(Device& d, const Segment* segments, size_t count, const float* keys, const float* values, cudaStream_t stream);

void qsa_decode_dense(Device& d, const void* const* states, const uint64_t* contexts, const uint64_t* lengths, uint64_t sequences,
                      uint64_t heads, uint64_t kv_heads, float scale, const void* q, float* out) {
    std::vector<const uint8_t*> checked;
    uint64_t kv_bytes = 0;
    validate_batch(d, states, contexts, lengths, sequences, heads, kv_heads, checked, kv_bytes);
    HostTables host;
    build_tables(checked, contexts, lengths, sequences, heads, kv_heads, uint32_t(d.sms) * kWarps, host, d.fixed_cuts);
    DecodePlan plan;
    fill_plan(d, host, plan, sequences, heads, kv_heads);
    ensure(d, d.pinned, d.pinned_bytes, plan.table_bytes, true);
    ensure(d, d.tables, d.tables_bytes, plan.table_bytes);
    ensure(d, d.partial, d.partial_bytes, size_t(plan.pieces) * kPartialFloats * 4);
    plan.partial = static_cast<float*>(d.partial);
    plan.status = status_word(d);
    // (the staging buffer is reused by the next call: wait for the previous upload to have left it)
    SDB_CHECK(cudaStreamSynchronize(d.stream));
    upload_tables(d, host, plan, d.tables, d.pinned);
    run_plan(d, plan, scale, q, out);
}

// sdx_attention_batch's work list, kept from call to call. A decode step makes every sequence one position longer, and the cuts
// lie at tile borders: the list of the step before serves this step with the segments' new lengths, and a sequence that has crossed
// into a new 16-key tile gets that tile added to its last piece (moving cuts only: the fixed cuts are a function of the length and
// are rebuilt). The host builds a new list when the batch changes or once a sequence has grown by more than kCacheGrowth tiles since
// the list was built (the warps that hold last pieces would otherwise drift ahead of the others); in between, the segments and the
// pieces go to the device as they are (a few tens of KB) and the host builds nothing.
constexpr uint32_t kCacheGrowth = 8;
struct BatchCache {
    std::vector<const uint8_t*> states;
    std::vector<uint64_t> contexts;
    std::vector<uint32_t> built, tiles;   // a sequence's tiles when the list was built, and now
    uint64_t heads = 0, kv_heads = 0;
    bool fixed = false;
    HostTables host;
    DecodePlan plan;
    // the list on the device and its page-locked staging area: allocations of the cache's own (the other decode entries use the handle's,
    // and may still be copying out of theirs when this entry is called; this entry ends with a synchronisation, so its own are free)
    void* tables = nullptr; size_t tables_bytes = 0;
    void* staging = nullptr; size_t staging_bytes = 0;
    ~BatchCache() { if (tables) cudaFree(tables); if (staging) cudaFreeHost(staging); }
};

// One decode step of a batch from host buffers: the new rows are appended and the batch is decoded by one pass over one work
// list. The host builds the list (when the step before's does not serve) while the copies of the queries and the new rows are in flight.
void attention_batch(Device& d, void* const* states, const uint64_t* contexts, const uint64_t* bases, uint64_t sequences, uint64_t heads,
                     uint64_t kv_heads, float scale, const void* q, const float* k, const float* v, float* out) {
    // everything is checked before anything is queued: a refused call leaves the K/V states as they were
    if (!states || !contexts || !bases || !q || !k || !v || !out || !sequences || sequences > 65535)
        throw std::runtime_error("invalid Straydog attention dimensions");
    std::vector<uint64_t> lengths(sequences);
    for (uint64_t s = 0; s < sequences; ++s) {
        if (!contexts[s] || bases[s] >= contexts[s]) throw std::runtime_error("invalid Straydog attention dimensions");
        lengths[s] = bases[s] + 1;
    }
    // (the append runs over the work list's segments, one a (sequence, K/V head): groups of up to eight query heads here)
    if (kv_heads && heads / kv_heads > 8) throw std::runtime_error("invalid Straydog attention dimensions");
    std::vector<const uint8_t*> checked;
    uint64_t kv_bytes = 0;
    validate_batch(d, reinterpret_cast<const void* const*>(states), contexts, lengths.data(), sequences, heads, kv_heads, checked, kv_bytes);
    {
        std::vector<const uint8_t*> sorted(checked);
        std::sort(sorted.begin(), sorted.end());
        if (std::adjacent_find(sorted.begin(), sorted.end()) != sorted.end())
            throw std::runtime_error("a Straydog K/V state is listed twice in one batch: its new row would be written twice");
    }
    // device work buffer: q (FP16) | k | v | out
    const size_t q_bytes = size_t(sequences * heads) * 256 * 2, new_bytes = size_t(sequences * kv_heads) * 256 * 4,
                 out_bytes = size_t(sequences * heads) * 256 * 4;
    const size_t k_at = (q_bytes + 255) / 256 * 256, v_at = k_at + (new_bytes + 255) / 256 * 256,
                 out_at = v_at + (new_bytes + 255) / 256 * 256, total = out_at + out_bytes;
    auto* work = static_cast<uint8_t*>(ensure(d, d.work, d.work_bytes, total));
    // Page-locked host buffers are read and written in place by the kernels (the device's view of the same memory): the new rows by the
    // append, the outputs by the merge, whose stores cross the bus while it runs instead of in a copy behind it. The queries, which every
    // piece of a sequence reads again, are copied. Pageable buffers take the copies.
    const auto in_place = [&](const void* host) -> void* {
        cudaPointerAttributes attributes{};
        if (cudaPointerGetAttributes(&attributes, host) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        return attributes.type == cudaMemoryTypeHost ? attributes.devicePointer : nullptr;
    };
    const float* k_device = static_cast<const float*>(in_place(k));
    const float* v_device = static_cast<const float*>(in_place(v));
    float* out_device = static_cast<float*>(in_place(out));
    if (!d.batch_cache) d.batch_cache = std::make_shared<BatchCache>();
    BatchCache& cache = *static_cast<BatchCache*>(d.batch_cache.get());
    std::vector<uint32_t> tiles(sequences);
    for (uint64_t s = 0; s < sequences; ++s) tiles[s] = uint32_t((lengths[s] + kTileKeys - 1) / kTileKeys);
    bool serves = cache.tables && cache.heads == heads && cache.kv_heads == kv_heads && cache.fixed == d.fixed_cuts && cache.states == checked &&
                  std::equal(cache.contexts.begin(), cache.contexts.end(), contexts);
    for (uint64_t s = 0; serves && s < sequences; ++s)
        serves = tiles[s] == cache.tiles[s] || (!d.fixed_cuts && tiles[s] > cache.tiles[s] && tiles[s] - cache.built[s] <= kCacheGrowth);
    HostTables& host = cache.host;
    DecodePlan& plan = cache.plan;
    // The order of the queue: the work list first (a few tens of KB), then the append on the side stream (it needs the list's segments,
    // and reads the new rows over the bus while it runs) beside the queries' copy on the main one; the decode waits for both. A list
    // that has to be built is built while the queries' copy is in flight instead.
    bool q_queued = false;
    if (!serves) { SDB_CHECK(cudaMemcpyAsync(work, q, q_bytes, cudaMemcpyHostToDevice, d.stream)); q_queued = true; }
    // (the buffers grow on the first call of a size only)
    if (serves) {
        for (size_t i = 0; i < host.segments.size(); ++i) {
            Segment& segment = host.segments[i];
            const uint64_t sequence = i / kv_heads;
            segment.length = uint32_t(lengths[sequence]);
            // (moving cuts: a segment's pieces lie one behind the other in the list, its last piece ends where its last tile does)
            if (tiles[sequence] != cache.tiles[sequence]) host.pieces[segment.first_piece + segment.pieces - 1].end = tiles[sequence] * kTileKeys;
        }
        cache.tiles = tiles;
        const size_t bytes = plan.piece_offset + host.pieces.size() * sizeof(Piece);   // segments | pieces, as upload_tables lays them out
        auto* stage = static_cast<uint8_t*>(cache.staging);
        std::memcpy(stage + plan.segment_offset, host.segments.data(), host.segments.size() * sizeof(Segment));
        std::memcpy(stage + plan.piece_offset, host.pieces.data(), host.pieces.size() * sizeof(Piece));
        SDB_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(cache.tables), stage, bytes, cudaMemcpyHostToDevice, d.stream));
    } else {
        cache.states.clear();   // (not a valid list until the new one is in place)
        build_tables(checked, contexts, lengths.data(), sequences, heads, kv_heads, uint32_t(d.sms) * kWarps, host, d.fixed_cuts);
        plan = DecodePlan{};
        fill_plan(d, host, plan, sequences, heads, kv_heads);
        ensure(d, cache.staging, cache.staging_bytes, plan.table_bytes, true);
        ensure(d, cache.tables, cache.tables_bytes, plan.table_bytes);
        upload_tables(d, host, plan, cache.tables, cache.staging);
        cache.states = checked; cache.contexts.assign(contexts, contexts + sequences); cache.tiles = tiles; cache.built = tiles;
        cache.heads = heads; cache.kv_heads = kv_heads; cache.fixed = d.fixed_cuts;
    }
    ensure(d, d.partial, d.partial_bytes, size_t(plan.pieces) * kPartialFloats * 4);
    plan.partial = static_cast<float*>(d.partial);
    plan.status = status_word(d);
    // the new rows, appended by one launch over the work list's segments (plane bases and lengths)
    const cudaStream_t side = side_stream_begin(d);
    if (!k_device) { SDB_CHECK(cudaMemcpyAsync(work + k_at, k, new_bytes, cudaMemcpyHostToDevice, side)); k_device = reinterpret_cast<const float*>(work + k_at); }
    if (!v_device) { SDB_CHECK(cudaMemcpyAsync(work + v_at, v, new_bytes, cudaMemcpyHostToDevice, side)); v_device = reinterpret_cast<const float*>(work + v_at); }
    launch_kv_append(d, reinterpret_cast<const Segment*>(static_cast<uint8_t*>(cache.tables) + plan.segment_offset), host.segments.size(),
                     k_device, v_device, side);
    SDB_CHECK(cudaGetLastError());
    if (!q_queued) SDB_CHECK(cudaMemcpyAsync(work, q, q_bytes, cudaMemcpyHostToDevice, d.stream));
    side_stream_end(d);
    run_plan(d, plan, scale, work, out_device ? out_device : reinterpret_cast<float*>(work + out_at));
    SDB_CHECK(cudaGetLastError());
    if (!out_device) SDB_CHECK(cudaMemcpyAsync(out, work + out_at, out_bytes, cudaMemcpyDeviceToHost, d.stream));
    SDB_CHECK(cudaStreamSynchronize(d.stream));
}

}  // namespace sdb

using namespace sdb;

extern "C" {

int sdx_qsa_decode(void* handle, const void* const* states, const uint64_t* contexts, const uint64_t* lengths, uint64_t sequences,
                   uint64_t heads, uint64_t kv_heads, float scale, const void* q, float* out) {
    SDB_OP_BEGIN
    span(value, q, checked_product({sequences, heads, 256, 2}), "attention queries");
    span(value, out, checked_product({sequences, heads, 256, 4}), "an attention output");
    qsa_decode_dense(value, states, contexts, lengths, sequences, heads, kv_heads, scale, q, out);
    SDB_OP_END
}

int sdx_attention_batch(void* handle, void* const* states, const uint64_t* contexts, const uint64_t* bases, uint64_t sequences,
                        uint64_t heads, uint64_t kv_heads, float scale, const void* q, const float* k, const float* v, float* out) {
    SDB_OP_BEGIN
    attention_batch(value, states, contexts, bases, sequences, heads, kv_heads, scale, q, k, v, out);
    SDB_OP_END
}

// The work list's cuts without a device (host arithmetic only): stats = {pieces, warps used, most tiles a warp got, tiles in all};
// begins[0 .. result) = where the pieces of sequence `probe`'s first K/V head start. For tests and for a caller that sizes scratch.
int sdx_qsa_cuts(const uint64_t* lengths, uint64_t sequences, uint64_t kv_heads, uint64_t warps, int fixed, uint64_t probe,
                 uint32_t* begins, uint64_t capacity, uint64_t* stats) {
    try {
        if (!lengths || !sequences || !kv_heads || !warps || probe >= sequences) throw std::runtime_error("invalid Straydog attention dimensions");
        std::vector<const uint8_t*> states(sequences, nullptr);
        std::vector<uint64_t> contexts(lengths, lengths + sequences);
        for (uint64_t s = 0; s < sequences; ++s)
            if (!lengths[s] || lengths[s] > (uint64_t(1) << 24)) throw std::runtime_error("invalid Straydog attention dimensions");
        HostTables host;
        build_tables(states, contexts.data(), lengths, sequences, kv_heads, kv_heads, uint32_t(warps), host, fixed != 0);
        if (stats) {
            uint64_t most = 0, total = 0;
            for (size_t w = 0; w + 1 < host.warp_piece.size(); ++w) {
                uint64_t tiles = 0;
                for (uint32_t i = host.warp_piece[w]; i < host.warp_piece[w + 1]; ++i) {
                    const Piece& piece = host.pieces[i];
                    tiles += (std::min(piece.end, host.segments[piece.segment].length) - piece.begin + kTileKeys - 1) / kTileKeys;
                }
                most = std::max(most, tiles);
                total += tiles;
            }
            stats[0] = host.pieces.size(); stats[1] = host.warp_piece.size() - 1; stats[2] = most; stats[3] = total;
        }
        std::vector<uint32_t> mine;
        for (const Piece& piece : host.pieces)
            if (piece.segment == probe * kv_heads) mine.push_back(piece.begin);
        std::sort(mine.begin(), mine.end());
        if (begins)
            for (size_t i = 0; i < mine.size() && i < capacity; ++i) begins[i] = mine[i];
        return int(mine.size());
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

int sdx_decode_cuts(void* handle, int fixed) {
    SDB_OP_BEGIN
    value.fixed_cuts = fixed != 0;
    SDB_OP_END
}

void* sdx_qsa_plan(void* handle, const void* const* states, const uint64_t* contexts, const uint64_t* lengths, uint64_t sequences,
                   uint64_t heads, uint64_t kv_heads) {
    try {
        auto& value = device(handle);
        std::vector<const uint8_t*> checked;
        uint64_t kv_bytes = 0;
        validate_batch(value, states, contexts, lengths, sequences, heads, kv_heads, checked, kv_bytes);
        HostTables host;
        build_tables(checked, contexts, lengths, sequences, heads, kv_heads, uint32_t(value.sms) * kWarps, host, value.fixed_cuts);
        auto plan = std::make_unique<DecodePlan>();
        fill_plan(value, host, *plan, sequences, heads, kv_heads);
        plan->kv_bytes = kv_bytes;
        plan->owns = true;
        void* tables = nullptr;
        SDB_CHECK(cudaMalloc(&tables, plan->table_bytes));
        void* partial = nullptr;
        if (cudaMalloc(&partial, size_t(plan->pieces) * kPartialFloats * 4) != cudaSuccess) { cudaFree(tables); SDB_CHECK(cudaGetLastError()); }
        plan->partial = static_cast<float*>(partial);
        plan->status = status_word(value);
        std::vector<uint8_t> staging(plan->table_bytes);
        upload_tables(value, host, *plan, tables, staging.data());
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        return plan.release();
    } catch (const std::exception& e) { last_error = e.what(); return nullptr; }
}

int sdx_qsa_plan_run(void* handle, void* plan, float scale, const void* q, float* out) {
    SDB_OP_BEGIN
    if (!plan) throw std::runtime_error("null Straydog decode plan");
    const auto& p = *static_cast<const DecodePlan*>(plan);
    span(value, q, checked_product({p.sequences, p.heads, 256, 2}), "attention queries");
    span(value, out, checked_product({p.sequences, p.heads, 256, 4}), "an attention output");
    run_plan(value, p, scale, q, out);
    SDB_OP_END
}

int sdx_qsa_plan_run_marked(void* handle, void* plan, float scale, const void* q, float* out, void* before, void* after) {
    SDB_OP_BEGIN
    if (!plan) throw std::runtime_error("null Straydog decode plan");
    const auto& p = *static_cast<const DecodePlan*>(plan);
    span(value, q, checked_product({p.sequences, p.heads, 256, 2}), "attention queries");
    span(value, out, checked_product({p.sequences, p.heads, 256, 4}), "an attention output");
    run_plan(value, p, scale, q, out, static_cast<cudaEvent_t>(before), static_cast<cudaEvent_t>(after));
    SDB_OP_END
}

int sdx_qsa_plan_info(void* plan, uint64_t* kv_bytes, uint64_t* pieces, uint64_t* ctas, uint64_t* virtual_warps) {
    if (!plan) { last_error = "null Straydog decode plan"; return -1; }
    const auto& p = *static_cast<const DecodePlan*>(plan);
    if (kv_bytes) *kv_bytes = p.kv_bytes;
    if (pieces) *pieces = p.pieces;
    if (ctas) *ctas = p.ctas;
    if (virtual_warps) *virtual_warps = p.virtual_warps;
    return 0;
}

int sdx_qsa_plan_release(void* handle, void* plan) {
    SDB_OP_BEGIN
    if (!plan) throw std::runtime_error("null Straydog decode plan");
    auto* p = static_cast<DecodePlan*>(plan);
    SDB_CHECK(cudaStreamSynchronize(value.stream));
    if (p->owns) { cudaFree(p->tables); cudaFree(p->partial); }
    delete p;
    SDB_OP_END
}

// ---- the decode that allocates nothing ----
// Every other decode entry keeps its work list and its split partials in memory it allocates on demand
// (cudaMalloc / cudaMallocHost the first time a batch of a new size arrives). Some hosts cannot allow
// that: an engine that has handed its whole VRAM budget to weights and K/V and must never see an
// allocation fail mid-request, or a serving loop that forbids driver allocations after start-up because
// they synchronise the device. For them this entry keeps all of its scratch in one array that is part
// of the library's device image: every GPU that loads the image holds it until exit. The CUDA runtime
// loads a library's device image lazily by default (at the first use of one of its kernels or symbols, which
// is when the array's 16.3 MiB are taken), so the call that must never allocate is any call AFTER the first
// one on that device: make one warm-up call at start-up, or run with CUDA_MODULE_LOADING=EAGER.
constexpr size_t kStaticSequences = 64;                                  // sequences a call
constexpr size_t kStaticKvHeads = 8;                                     // K/V heads
constexpr size_t kStaticPieces = 2048;                                   // pieces a call's work list may hold
constexpr size_t kStaticTableBytes = size_t(128) << 10;                  // segments | pieces | warp ranges
constexpr size_t kStaticScratchBytes = kStaticTableBytes + kStaticPieces * size_t(kPartialFloats) * 4 + 256;   // about 16.3 MiB
static __device__ __align__(256) uint8_t static_decode_scratch[kStaticScratchBytes];

// The array's device address, per device. The symbol's name is only a host-side stand-in: the address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
static uint8_t* static_scratch_address(Device& d) {
    static std::mutex mutex;
    static std::map<int, uint8_t*> known;
    std::lock_guard<std::mutex> lock(mutex);
    auto found = known.find(d.ordinal);
    if (found != known.end()) return found->second;
    void* address = nullptr;
    SDB_CHECK(cudaGetSymbolAddress(&address, static_decode_scratch));   // (device(handle) made d.ordinal current)
    known[d.ordinal] = static_cast<uint8_t*>(address);
    return static_cast<uint8_t*>(address);
}

int sdx_qsa_decode_static(void* handle, const void* const* states, const uint64_t* contexts, const uint64_t* lengths,
                          uint64_t sequences, uint64_t heads, uint64_t kv_heads, float scale, const void* q, float* out) {
    SDB_OP_BEGIN
    if (sequences > kStaticSequences || kv_heads > kStaticKvHeads)
        throw std::runtime_error("sdx_qsa_decode_static holds scratch for at most 64 sequences of at most 8 K/V heads: use sdx_qsa_decode for a larger batch");
    span(value, q, checked_product({sequences, heads, 256, 2}), "attention queries");
    span(value, out, checked_product({sequences, heads, 256, 4}), "an attention output");
    std::vector<const uint8_t*> checked;
    uint64_t kv_bytes = 0;
    validate_batch(value, states, contexts, lengths, sequences, heads, kv_heads, checked, kv_bytes);
    HostTables host;
    build_tables(checked, contexts, lengths, sequences, heads, kv_heads, uint32_t(value.sms) * kWarps, host, false);   // (moving cuts: fewest partials)
    DecodePlan plan;
    fill_plan(value, host, plan, sequences, heads, kv_heads);
    if (plan.pieces > kStaticPieces || plan.table_bytes > kStaticTableBytes)
        throw std::runtime_error("sdx_qsa_decode_static: this batch's work list is larger than the static scratch (2048 pieces)");
    uint8_t* scratch = static_scratch_address(value);
    plan.partial = reinterpret_cast<float*>(scratch + kStaticTableBytes);
    plan.status = reinterpret_cast<int*>(scratch + kStaticScratchBytes - 256);
    // The tables travel from ordinary host memory: the copy is staged by the runtime before the call returns, so the
    // vector may go; nothing is allocated on the device. The status word is the only part that must start at zero.
    std::vector<uint8_t> staging(plan.table_bytes);
    SDB_CHECK(cudaMemsetAsync(plan.status, 0, 4, value.stream));
    upload_tables(value, host, plan, scratch, staging.data());
    run_plan(value, plan, scale, q, out);
    SDB_CHECK(cudaGetLastError());
    int gave_up = 0;
    SDB_CHECK(cudaMemcpyAsync(&gave_up, plan.status, 4, cudaMemcpyDeviceToHost, value.stream));
    SDB_CHECK(cudaStreamSynchronize(value.stream));
    if (gave_up) throw std::runtime_error("sdx_qsa_decode_static: a bounded wait inside the decode kernel gave up");
    SDB_OP_END
}

// What a kernel reported since the last call (the word is cleared): 0 nothing, 1 a bounded wait on a copy gave up, 2 / 3 a row
// number / key pointer out of range in the latent kernel, 4 a gather's peer never arrived.
int sdx_decode_status(void* handle) {
    try {
        auto& value = device(handle);
        int* word = status_word(value);
        int host = 0;
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        SDB_CHECK(cudaMemcpy(&host, word, 4, cudaMemcpyDeviceToHost));
        if (host) SDB_CHECK(cudaMemset(word, 0, 4));
        return host;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

}  // extern "C"
