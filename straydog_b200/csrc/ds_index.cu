// The producers of the latent attention's index lists (DeepSeek-V4.1's indexer) and its compressed rows:
//   sd_op_rope              gpu/straydog_gpu.h:271, gpu/ops.hpp:107-120, entry gpu/kernels.cpp:4942-4956
//   sd_op_compress          gpu/straydog_gpu.h:407, gpu/ops.hpp:1679-1695, entry gpu/kernels.cpp:5478-5485
//   sd_op_index_scores      gpu/straydog_gpu.h:408, gpu/ops.hpp:1697-1745, entry gpu/kernels.cpp:5487-5499
//   sd_op_index_candidates  gpu/straydog_gpu.h:410-414, gpu/ops.hpp:1942-1966, entry gpu/kernels.cpp:5546-5566
//   sd_op_index_select      gpu/straydog_gpu.h:415-419, gpu/ops.hpp:1978-2300, entry gpu/kernels.cpp:5568-5618
//   sd_op_index_select_proj gpu/straydog_gpu.h:422, entry gpu/kernels.cpp:5620-5667 (plain weight kinds)
// The contract is bit-exact: a score is scale * sum over heads in order of relu(q_h . key) * weight_h, each dot one chain of fused
// multiply-adds over the columns in order, each term one rounded product, the terms added in head order; sd_op_index_select gives
// the scores and indices that sd_op_rope, sd_op_index_scores and sd_op_top_k give one after the other
// (crates/straydog-engine/tests/fused_gpu.rs:391-431). The kernels here keep that order of operations with another division of
// the work: a thread owns a register tile of (place, head) running dots fed by 16-byte shared-memory reads (16 x 8 with two fused
// multiply-adds an instruction in index_scores_wide_kernel, 4 x 4 in index_scores_kernel for the widths that one does not take),
// BF16-tagged keys are widened as they land. The tensor cores are not used: their summation order is not the contract's.
#include "common.cuh"
#include "ds_sparse.cuh"
#include "../../include/straydog_gpu_b200.h"

#include <algorithm>

namespace sdb {

void launch_top_k(Device& d, const float* scores, size_t rows, size_t groups, size_t k, int32_t* out, const int32_t* candidates, size_t blocks, size_t block,
                  bool dependent, const TopKExpand* expand);

__global__ void __launch_bounds__(256) rope_kernel(float* __restrict__ x, size_t count, size_t vectors, size_t width, size_t pairs,
                                                   const int32_t* __restrict__ positions, const float* __restrict__ frequencies, int inverse) {
    const size_t index = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= count) return;
    const size_t pair = index % pairs, vector = index / pairs % vectors, row = index / (pairs * vectors);
    float* v = x + (row * vectors + vector) * width + (width - 2 * pairs) + 2 * pair;
    double s, c;
    sincos(double(positions[row]) * double(frequencies[pair]) * (inverse ? -1.0 : 1.0), &s, &c);   // (the angle times -1.0: its own sincos)
    const double a = v[0], b = v[1];
    v[0] = float(a * c - b * s);
    v[1] = float(a * s + b * c);
}

// out[group][col] = sum_r softmax_r(gate[group * ratio + r][col]) * kv[group * ratio + r][col]; no gate: the row itself
__global__ void __launch_bounds__(256) compress_kernel(const float* __restrict__ kv, const float* __restrict__ gate, size_t groups, size_t ratio,
                                                       size_t dim, float* __restrict__ out) {
    const size_t index = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= groups * dim) return;
    const size_t group = index / dim, col = index % dim;
    if (!gate) { out[index] = kv[group * dim + col]; return; }
    const float* g = gate + group * ratio * dim + col;
    const float* v = kv + group * ratio * dim + col;
    float top = -INFINITY;
    for (size_t r = 0; r < ratio; ++r) top = fmaxf(top, g[r * dim]);
    float sum = 0.0f, acc = 0.0f;
    for (size_t r = 0; r < ratio; ++r) {
        const float w = expf(g[r * dim] - top);
        sum = __fadd_rn(sum, w);
        acc = fmaf(w, v[r * dim], acc);   // (what the reference's `acc += w * kv` compiles to)
    }
    out[index] = __fdiv_rn(acc, sum);
}

// The projection in front of sd_op_index_select_proj: weights[h] = W[h] . x for the (<= 64) index heads, W a row-major matrix of the
// reference's plain kinds (0: F32, 1: F16, 30: BF16). The sum's order is the reference GEMV's for such a matrix (gpu/gemv_common.hpp:42-86,
// 784-812 with the lanes gpu/gemv.hpp:24-36 gives a matrix of so few rows: a warp a row): lane l takes the units l, l + 32, ... (a unit
// = 4 F32 or 8 half values), a unit's dot is one chain (F32: from the last value inwards; halves: from the first), the lane adds
// its units in order, the lanes' sums meet in a butterfly (xor 16, 8, 4, 2, 1). Rows or inputs that are not 16-byte aligned take
// the reference's element path (gpu/gemv_common.hpp:814-836): lane l takes the columns l, l + 32, ... in one chain.
__device__ __forceinline__ float proj_half(uint32_t bits, int kind) {
    return kind == 1 ? __half2float(__ushort_as_half(uint16_t(bits))) : __uint_as_float(bits << 16);
}
__global__ void __launch_bounds__(256) index_proj_kernel(const uint8_t* __restrict__ w, int kind, size_t row_bytes, size_t rows, size_t cols,
                                                         const float* __restrict__ x, bool units_path, float* __restrict__ out) {
    const size_t row = size_t(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    const unsigned lane = threadIdx.x % 32;
    if (row >= rows) return;
    const uint8_t* data = w + row * row_bytes;
    float sum = 0.0f;
    if (units_path && kind == 0) {
        for (size_t unit = lane; unit < cols / 4; unit += 32) {
            const float4 m = reinterpret_cast<const float4*>(data)[unit], a = reinterpret_cast<const float4*>(x)[unit];
            sum = __fadd_rn(sum, fmaf(m.x, a.x, fmaf(m.y, a.y, fmaf(m.z, a.z, __fmul_rn(m.w, a.w)))));
        }
    } else if (units_path) {
        for (size_t unit = lane; unit < cols / 8; unit += 32) {
            const uint4 q = reinterpret_cast<const uint4*>(data)[unit];
            const float4 a = reinterpret_cast<const float4*>(x)[2 * unit], b = reinterpret_cast<const float4*>(x)[2 * unit + 1];
            float dot = __fmul_rn(proj_half(q.x & 0xffffu, kind), a.x);
            dot = fmaf(proj_half(q.x >> 16, kind), a.y, dot); dot = fmaf(proj_half(q.y & 0xffffu, kind), a.z, dot);
            dot = fmaf(proj_half(q.y >> 16, kind), a.w, dot); dot = fmaf(proj_half(q.z & 0xffffu, kind), b.x, dot);
            dot = fmaf(proj_half(q.z >> 16, kind), b.y, dot); dot = fmaf(proj_half(q.w & 0xffffu, kind), b.z, dot);
            dot = fmaf(proj_half(q.w >> 16, kind), b.w, dot);
            sum = __fadd_rn(sum, dot);
        }
    } else {
        for (size_t col = lane; col < cols; col += 32) {
            const float m = kind == 0 ? reinterpret_cast<const float*>(data)[col] : proj_half(reinterpret_cast<const uint16_t*>(data)[col], kind);
            sum = fmaf(m, x[col], sum);
        }
    }
    #pragma unroll
    for (unsigned offset = 16; offset; offset /= 2) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, offset));
    if (lane == 0) out[row] = sum;
}

constexpr int kIndexGroups = 64, kIndexCols = 32, kIndexHeads = 64, kIndexThreads = 256, kIndexStride = 68;   // (68 floats: 16-byte aligned rows)

// A CTA scores 64 places of one row against all (<= 64) heads: thread (tg, th) = (t % 16, t / 16) owns places 4 tg .. 4 tg + 3 and heads
// 4 th .. 4 th + 3, sixteen running dots, and per column reads one 16-byte piece of the key tile and one of the query tile (both kept
// column-major in shared memory) for sixteen fused multiply-adds: the arithmetic pipe, not the shared-memory pipe, sets the pace. The
// order of operations is the reference's: a dot is one chain over the columns in order, a head's term one rounded product, the terms
// are added in head order by one thread a place. With candidates, place v of a row stands for group candidates[v / block] * block +
// v % block (none where the slot is -1) and the scores are stored in candidate order.
__global__ void __launch_bounds__(kIndexThreads) index_scores_kernel(const float* __restrict__ q, const float* keys, const float* __restrict__ weights,
                                                                     const int32_t* __restrict__ visible, size_t groups, size_t heads, size_t dim,
                                                                     float scale, float* __restrict__ scores, const int32_t* __restrict__ candidates,
                                                                     size_t blocks, size_t block) {
    const size_t row = blockIdx.y, scored = candidates ? blocks * block : groups, place0 = size_t(blockIdx.x) * kIndexGroups;
    const unsigned t = threadIdx.x, tg = t % 16, th = t / 16;
    const size_t limit = min(groups, size_t(max(visible[row], 0)));
    __shared__ __align__(16) float tiles[2 * kIndexCols * kIndexStride];   // keys [column][place] | queries [column][head]; then the terms [head][place]
    __shared__ size_t tile_groups[kIndexGroups];
    float* ks = tiles;
    float* qs = tiles + kIndexCols * kIndexStride;
    if (t < kIndexGroups) {
        const size_t place = place0 + t;
        size_t g = groups;
        if (place < scored) {
            if (!candidates) g = place;
            else { const int32_t b = candidates[row * blocks + place / block]; g = b < 0 ? groups : size_t(b) * block + place % block; }
        }
        tile_groups[t] = g;
    }
    float acc[4][4];   // [place][head]
    #pragma unroll
    for (int i = 0; i < 4; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    const float* row_q = q + row * heads * dim;
    const bool bf16 = state_is_bf16(keys);
    for (size_t d0 = 0; d0 < dim; d0 += kIndexCols) {
        __syncthreads();
        // (a warp reads 32 consecutive columns of one key or one head's query, and writes them down a column of the tile)
        for (unsigned i = t; i < kIndexGroups * kIndexCols; i += kIndexThreads) {
            const unsigned r = i / kIndexCols, c = i % kIndexCols;
            const size_t at = tile_groups[r], col = d0 + c;
            float value = 0.0f;
            if (at < limit && col < dim)
                value = bf16 ? __uint_as_float(uint32_t(state_halves(keys)[at * dim + col]) << 16) : keys[at * dim + col];
            ks[c * kIndexStride + r] = value;
            qs[c * kIndexStride + r] = r < heads && col < dim ? row_q[r * dim + col] : 0.0f;
        }
        __syncthreads();
        const int width = int(min(size_t(kIndexCols), dim - d0));
        #pragma unroll 8
        for (int c = 0; c < width; ++c) {
            const float4 k4 = *reinterpret_cast<const float4*>(ks + c * kIndexStride + 4 * tg);
            const float4 q4 = *reinterpret_cast<const float4*>(qs + c * kIndexStride + 4 * th);
            const float k[4] = {k4.x, k4.y, k4.z, k4.w}, qv[4] = {q4.x, q4.y, q4.z, q4.w};
            #pragma unroll
            for (int i = 0; i < 4; ++i)
                #pragma unroll
                for (int h = 0; h < 4; ++h) acc[i][h] = fmaf(qv[h], k[i], acc[i][h]);
        }
    }
    __syncthreads();
    float* terms = tiles;   // [head][place], 64 x 68 floats
    #pragma unroll
    for (int h = 0; h < 4; ++h) {
        const size_t head = 4 * th + h;
        const float w = head < heads ? weights[row * heads + head] : 0.0f;
        *reinterpret_cast<float4*>(terms + head * kIndexStride + 4 * tg) =
            make_float4(__fmul_rn(fmaxf(acc[0][h], 0.0f), w), __fmul_rn(fmaxf(acc[1][h], 0.0f), w), __fmul_rn(fmaxf(acc[2][h], 0.0f), w), __fmul_rn(fmaxf(acc[3][h], 0.0f), w));
    }
    __syncthreads();
    if (t >= kIndexGroups || place0 + t >= scored) return;
    float total = 0.0f;
    for (size_t h = 0; h < heads; ++h) total = __fadd_rn(total, terms[h * kIndexStride + t]);
    scores[row * scored + place0 + t] = tile_groups[t] < limit ? __fmul_rn(total, scale) : -INFINITY;
}

// The same scores for the usual shapes (dim a multiple of 8, keys and queries 16-byte aligned): a CTA of 128 threads scores 256 places of
// one row against all (<= 64) heads, a thread a 16 x 8 register tile (places 4 tg + 64 j .. + 3 for j = 0 .. 3, heads 4 th .. + 3 and
// 32 + 4 th .. + 3). What bounds such a kernel is the path from shared memory to the registers, four cycles a 16-byte read of a warp
// whatever is broadcast: the 4 x 4 tile above pays two reads for 16 fused multiply-adds, an 8 x 8 tile four for 64 (the two pipes level),
// this tile six for 128, which leaves the arithmetic pipe the slower one; and the multiply-adds are issued two to an instruction
// (fma.rn.f32x2 over a pair of heads: each half one IEEE fma, the scalar chain's bits), which halves their issue slots. The columns come 8 at a time: a thread fetches two places' 8 key
// values (16 bytes of BF16 each) and a head's 4 query values into registers while the step before is being multiplied, and sets them
// down the tiles' columns (lanes on consecutive places: no bank conflict) between two barriers. Order of operations as above.
// Two fused multiply-adds an instruction (each half one IEEE fma, the same bits as two scalar ones): half the issue slots for the same arithmetic.
__device__ __forceinline__ uint64_t pair_of(float low, float high) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(low), "f"(high)); return r; }
__device__ __forceinline__ void fma_pair(uint64_t& acc, uint64_t a, uint64_t b) { asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b)); }
__device__ __forceinline__ float2 halves_of(uint64_t pair) { float2 r; asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(pair)); return r; }

namespace wide {
constexpr int kPlaces = 256, kHeads = 64, kStep = 8, kThreads = 128, kTermStride = kPlaces + 4;
constexpr size_t kSmem = size_t(kHeads) * kTermStride * 4;   // the terms [head][place]; the tiles [column][place] | [column][head] lie in the same bytes before
static_assert(kSmem >= size_t(kStep) * (kPlaces + kHeads) * 4, "the tiles fit the terms' area");
}  // namespace wide

__global__ void __launch_bounds__(wide::kThreads) index_scores_wide_kernel(const float* __restrict__ q, const float* keys, const float* __restrict__ weights,
                                                                           const int32_t* __restrict__ visible, size_t groups, size_t heads, size_t dim,
                                                                           float scale, float* __restrict__ scores, const int32_t* __restrict__ candidates,
                                                                           size_t blocks, size_t block) {
    using namespace wide;
    const size_t row = blockIdx.y, scored = candidates ? blocks * block : groups, place0 = size_t(blockIdx.x) * kPlaces;
    const unsigned t = threadIdx.x, tg = t % 16, th = t / 16;
    const size_t limit = min(groups, size_t(max(visible[row], 0)));
    extern __shared__ __align__(16) float wide_tiles[];
    float* ks = wide_tiles;                      // [column of the step][place]
    float* qs = wide_tiles + kStep * kPlaces;    // [column of the step][head]
    // this thread's two places (their key rows) and its part of a head's query step
    size_t mine[2];
    bool live[2];
    #pragma unroll
    for (int j = 0; j < 2; ++j) {
        const size_t place = place0 + t + kThreads * j;
        mine[j] = groups;
        if (place < scored) {
            if (!candidates) mine[j] = place;
            else { const int32_t b = candidates[row * blocks + place / block]; mine[j] = b < 0 ? groups : size_t(b) * block + place % block; }
        }
        live[j] = mine[j] < limit;
    }
    const bool bf16 = state_is_bf16(keys);
    const uint16_t* key_halves = state_halves(keys);
    const unsigned q_head = t % kHeads, q_part = t / kHeads;
    const float* q_from = q + (row * heads + q_head) * dim + 4 * q_part;
    const bool q_live = q_head < heads;

    float key_next[2][kStep];
    float4 q_next;
    const auto fetch = [&](size_t d0) {
        #pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (!live[j]) {
                #pragma unroll
                for (int i = 0; i < kStep; ++i) key_next[j][i] = 0.0f;
            } else if (bf16) {
                const uint4 x = *reinterpret_cast<const uint4*>(key_halves + mine[j] * dim + d0);
                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
                #pragma unroll
                for (int i = 0; i < 4; ++i) { key_next[j][2 * i] = __uint_as_float(w[i] << 16); key_next[j][2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
            } else {
                #pragma unroll
                for (int v = 0; v < 2; ++v) {
                    const float4 x = *reinterpret_cast<const float4*>(keys + mine[j] * dim + d0 + 4 * v);
                    key_next[j][4 * v] = x.x; key_next[j][4 * v + 1] = x.y; key_next[j][4 * v + 2] = x.z; key_next[j][4 * v + 3] = x.w;
                }
            }
        }
        q_next = q_live ? __ldg(reinterpret_cast<const float4*>(q_from + d0)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    };
    const auto set_down = [&]() {
        #pragma unroll
        for (int j = 0; j < 2; ++j)
            #pragma unroll
            for (int i = 0; i < kStep; ++i) ks[i * kPlaces + t + kThreads * j] = key_next[j][i];
        qs[(4 * q_part) * kHeads + q_head] = q_next.x; qs[(4 * q_part + 1) * kHeads + q_head] = q_next.y;
        qs[(4 * q_part + 2) * kHeads + q_head] = q_next.z; qs[(4 * q_part + 3) * kHeads + q_head] = q_next.w;
    };

    uint64_t acc[16][4];   // [place][pair of heads]
    #pragma unroll
    for (int i = 0; i < 16; ++i)
        #pragma unroll
        for (int h = 0; h < 4; ++h) acc[i][h] = 0;
    fetch(0);
    set_down();
    __syncthreads();
    for (size_t d0 = 0; d0 < dim; d0 += kStep) {
        const bool more = d0 + kStep < dim;
        if (more) fetch(d0 + kStep);
        #pragma unroll
        for (int c = 0; c < kStep; ++c) {
            uint64_t k[16], qv[4];
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 x = *reinterpret_cast<const float4*>(ks + c * kPlaces + 64 * j + 4 * tg);
                k[4 * j] = pair_of(x.x, x.x); k[4 * j + 1] = pair_of(x.y, x.y); k[4 * j + 2] = pair_of(x.z, x.z); k[4 * j + 3] = pair_of(x.w, x.w);
            }
            #pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float4 x = *reinterpret_cast<const float4*>(qs + c * kHeads + 32 * j + 4 * th);
                qv[2 * j] = pair_of(x.x, x.y); qv[2 * j + 1] = pair_of(x.z, x.w);
            }
            #pragma unroll
            for (int i = 0; i < 16; ++i)
                #pragma unroll
                for (int h = 0; h < 4; ++h) fma_pair(acc[i][h], qv[h], k[i]);
        }
        __syncthreads();
        if (more) { set_down(); __syncthreads(); }
    }
    float* terms = wide_tiles;   // [head][place]
    #pragma unroll
    for (int h = 0; h < 8; ++h) {
        const size_t head = (h < 4 ? 0 : 32) + 4 * th + (h & 3);
        const float w = head < heads ? weights[row * heads + head] : 0.0f;
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            float dot[4];
            #pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 both = halves_of(acc[4 * j + i][h / 2]); dot[i] = h & 1 ? both.y : both.x; }
            *reinterpret_cast<float4*>(terms + head * kTermStride + 64 * j + 4 * tg) =
                make_float4(__fmul_rn(fmaxf(dot[0], 0.0f), w), __fmul_rn(fmaxf(dot[1], 0.0f), w), __fmul_rn(fmaxf(dot[2], 0.0f), w), __fmul_rn(fmaxf(dot[3], 0.0f), w));
        }
    }
    __syncthreads();
    // a place's terms in head order: one chain of additions a place, two places a thread side by side
    float total[2] = {0.0f, 0.0f};
    for (size_t h = 0; h < heads; ++h) {
        total[0] = __fadd_rn(total[0], terms[h * kTermStride + t]);
        total[1] = __fadd_rn(total[1], terms[h * kTermStride + t + kThreads]);
    }
    #pragma unroll
    for (int j = 0; j < 2; ++j)
        if (place0 + t + kThreads * j < scored) scores[row * scored + place0 + t + kThreads * j] = live[j] ? __fmul_rn(total[j], scale) : -INFINITY;
}

// A block's highest score, a thread a block; the block of the row's last visible group +inf (always kept), blocks of only -inf stay -inf.
__global__ void __launch_bounds__(256) index_block_tops_kernel(const float* __restrict__ scores, const int32_t* __restrict__ visible, size_t groups,
                                                               size_t block, size_t count, float* __restrict__ tops) {
    const size_t row = blockIdx.y, b = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (b >= count) return;
    const float* s = scores + row * groups;
    const size_t seen = min(groups, size_t(max(visible[row], 0)));
    float top = seen && b == (seen - 1) / block ? INFINITY : -INFINITY;
    for (size_t g = b * block, end = min(groups, g + block); g < end; ++g) top = fmaxf(top, s[g]);
    tops[row * count + b] = top;
}

static void launch_index_scores(Device& d, const float* q, const float* keys, const float* weights, const int32_t* visible, size_t rows, size_t groups,
                                size_t heads, size_t dim, float scale, float* scores, const int32_t* candidates, size_t blocks, size_t block) {
    const size_t scored = candidates ? blocks * block : groups;
    const bool aligned = dim % 8 == 0 && reinterpret_cast<uintptr_t>(q) % 16 == 0 && reinterpret_cast<uintptr_t>(state_halves(keys)) % 16 == 0;
    if (aligned) {
        static bool configured[64] = {};
        if (!configured[d.ordinal & 63]) {
            SDB_CHECK(cudaFuncSetAttribute(index_scores_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(wide::kSmem)));
            configured[d.ordinal & 63] = true;
        }
        index_scores_wide_kernel<<<dim3(unsigned((scored + wide::kPlaces - 1) / wide::kPlaces), unsigned(rows)), wide::kThreads, wide::kSmem, d.stream>>>(
            q, keys, weights, visible, groups, heads, dim, scale, scores, candidates, blocks, block);
    } else {
        index_scores_kernel<<<dim3(unsigned((scored + kIndexGroups - 1) / kIndexGroups), unsigned(rows)), kIndexThreads, 0, d.stream>>>(
            q, keys, weights, visible, groups, heads, dim, scale, scores, candidates, blocks, block);
    }
    ++d.launches;
    SDB_CHECK(cudaGetLastError());
}

static void keys_span(Device& d, const float* keys, size_t values) {
    if (state_is_bf16(keys)) span(d, state_halves(keys), values * 2, "index keys");
    else span(d, keys, values * 4, "index keys");
}

}  // namespace sdb

using namespace sdb;

extern "C" {

int sd_op_rope(void* handle, float* x, uint64_t rows, uint64_t vectors, uint64_t width, uint64_t rope_dims, const int32_t* positions,
               const float* frequencies, int inverse) {
    SDB_OP_BEGIN
    if (!rows || !vectors || !rope_dims || rope_dims % 2 || rope_dims > width) throw std::runtime_error("invalid Straydog rope shape");
    span(value, x, checked_product({rows, vectors, width, 4}), "a rotated buffer");
    span(value, positions, checked_product({rows, 4}), "rope positions");
    span(value, frequencies, checked_product({rope_dims / 2, 4}), "rope frequencies");
    const size_t count = checked_product({rows, vectors, rope_dims / 2});
    rope_kernel<<<unsigned((count + 255) / 256), 256, 0, value.stream>>>(x, count, size_t(vectors), size_t(width), size_t(rope_dims / 2), positions, frequencies, inverse);
    ++value.launches;
    SDB_OP_END
}

int sd_op_compress(void* handle, const float* kv, const float* gate, uint64_t groups, uint64_t ratio, uint64_t dim, float* out) {
    SDB_OP_BEGIN
    if (!groups || !ratio || !dim) throw std::runtime_error("invalid Straydog compression shape");
    span(value, kv, checked_product({groups, ratio, dim, 4}), "rows to compress");
    if (gate) span(value, gate, checked_product({groups, ratio, dim, 4}), "a compression gate");
    span(value, out, checked_product({groups, dim, 4}), "compressed rows");
    const size_t count = checked_product({groups, dim});
    compress_kernel<<<unsigned((count + 255) / 256), 256, 0, value.stream>>>(kv, gate, size_t(groups), size_t(ratio), size_t(dim), out);
    ++value.launches;
    SDB_OP_END
}

int sd_op_index_scores(void* handle, const float* q, const float* keys, const float* weights, const int32_t* visible, uint64_t rows, uint64_t groups,
                       uint64_t heads, uint64_t dim, float scale, float* scores) {
    SDB_OP_BEGIN
    if (!rows || rows > 65535 || !groups || !heads || heads > uint64_t(kIndexHeads) || !dim) throw std::runtime_error("invalid Straydog index shape");
    span(value, q, checked_product({rows, heads, dim, 4}), "index queries");
    keys_span(value, keys, checked_product({groups, dim}));
    span(value, weights, checked_product({rows, heads, 4}), "index weights");
    span(value, visible, checked_product({rows, 4}), "visible counts");
    span(value, scores, checked_product({rows, groups, 4}), "index scores");
    launch_index_scores(value, q, keys, weights, visible, size_t(rows), size_t(groups), size_t(heads), size_t(dim), scale, scores, nullptr, 0, 1);
    SDB_OP_END
}

int sd_op_index_candidates(void* handle, const float* scores, const int32_t* visible, uint64_t rows, uint64_t groups, uint64_t blocks, uint64_t block,
                           int32_t* out, float* scratch, uint64_t scratch_bytes) {
    SDB_OP_BEGIN
    if (!rows || rows > 65535 || !groups || groups > (uint64_t(1) << 31) || !blocks || blocks > (uint64_t(1) << 20) || !block || block > 4096)
        throw std::runtime_error("invalid Straydog index candidates");
    const uint64_t count = (groups + block - 1) / block;
    span(value, scores, checked_product({rows, groups, 4}), "index scores");
    span(value, visible, checked_product({rows, 4}), "visible counts");
    span(value, out, checked_product({rows, blocks, 4}), "index candidates");
    if (checked_product({rows, count, 4}) > scratch_bytes) throw std::runtime_error("Straydog index candidates need more scratch");
    span(value, scratch, checked_product({rows, count, 4}), "index candidates' scratch");
    index_block_tops_kernel<<<dim3(unsigned((count + 255) / 256), unsigned(rows)), 256, 0, value.stream>>>(scores, visible, size_t(groups), size_t(block), size_t(count), scratch);
    ++value.launches;
    SDB_CHECK(cudaGetLastError());
    launch_top_k(value, scratch, size_t(rows), size_t(count), size_t(blocks), out, nullptr, 0, 1, false, nullptr);
    SDB_OP_END
}

int sd_op_index_select(void* handle, const float* q, const float* keys, const float* weights, const int32_t* visible, uint64_t rows, uint64_t groups,
                       uint64_t heads, uint64_t dim, float scale, uint64_t rope_dims, const int32_t* positions, const float* frequencies, float* scores,
                       uint64_t k, int32_t* out, const int32_t* candidates, uint64_t blocks, uint64_t block) {
    SDB_OP_BEGIN
    if (!rows || rows > 65535 || !groups || groups > (uint64_t(1) << 31) || !heads || heads > uint64_t(kIndexHeads) || !dim || !k ||
        k > (uint64_t(1) << 31) || rope_dims % 2 || rope_dims > dim || rope_dims > 128)
        throw std::runtime_error("invalid Straydog index shape");
    uint64_t scored = groups;
    if (candidates) {
        if (!blocks || !block || blocks > (uint64_t(1) << 20) || block > 4096) throw std::runtime_error("invalid Straydog index candidates");
        span(value, candidates, checked_product({rows, blocks, 4}), "index candidates");
        scored = blocks * block;
    }
    span(value, q, checked_product({rows, heads, dim, 4}), "index queries");
    keys_span(value, keys, checked_product({groups, dim}));
    span(value, weights, checked_product({rows, heads, 4}), "index weights");
    span(value, visible, checked_product({rows, 4}), "visible counts");
    span(value, positions, checked_product({rows, 4}), "query positions");
    if (rope_dims) span(value, frequencies, checked_product({rope_dims / 2, 4}), "rope frequencies");
    span(value, scores, checked_product({rows, std::max(groups, scored), 4}), "index scores");
    span(value, out, checked_product({rows, k, 4}), "top-k indices");
    // q rotated into a workspace of the library (q itself stays as it is), then the scores and the top k over them
    const float* q_used = q;
    if (rope_dims) {
        const size_t bytes = checked_product({rows, heads, dim, 4});
        auto* rotated = static_cast<float*>(ensure(value, value.work, value.work_bytes, bytes));
        SDB_CHECK(cudaMemcpyAsync(rotated, q, bytes, cudaMemcpyDeviceToDevice, value.stream));
        const size_t count = checked_product({rows, heads, rope_dims / 2});
        rope_kernel<<<unsigned((count + 255) / 256), 256, 0, value.stream>>>(rotated, count, size_t(heads), size_t(dim), size_t(rope_dims / 2), positions, frequencies, 0);
        ++value.launches;
        SDB_CHECK(cudaGetLastError());
        q_used = rotated;
    }
    launch_index_scores(value, q_used, keys, weights, visible, size_t(rows), size_t(groups), size_t(heads), size_t(dim), scale, scores, candidates, size_t(blocks), size_t(block ? block : 1));
    launch_top_k(value, scores, size_t(rows), size_t(scored), size_t(k), out, candidates, size_t(blocks), size_t(block ? block : 1), false, nullptr);
    SDB_OP_END
}

// gpu/straydog_gpu.h:422, entry gpu/kernels.cpp:5620-5667: sd_op_index_select for one row whose head weights are first projected from the
// row's input, weights = W . x (written to `weights`), W [heads][proj_cols] of a plain kind: 0 (F32), 1 (F16), 30 (BF16). The reference
// also takes its quantised GGML kinds there; those belong to its GEMV family and are refused here by name.
int sd_op_index_select_proj(void* handle, const void* proj_weights, int proj_kind, uint64_t proj_cols, const float* x, const float* q,
                            const float* keys, float* weights, const int32_t* visible, uint64_t groups, uint64_t heads, uint64_t dim,
                            float scale, uint64_t rope_dims, const int32_t* positions, const float* frequencies, float* scores, uint64_t k,
                            int32_t* out, const int32_t* candidates, uint64_t blocks, uint64_t block) {
    SDB_OP_BEGIN
    if (!proj_weights || !proj_cols || proj_cols > 8192 || !groups || groups > (uint64_t(1) << 31) || !heads || heads > uint64_t(kIndexHeads) ||
        !dim || !k || k > (uint64_t(1) << 31) || rope_dims % 2 || rope_dims > dim || rope_dims > 128)
        throw std::runtime_error("invalid Straydog index shape");
    if (proj_kind != 0 && proj_kind != 1 && proj_kind != 30) throw std::runtime_error("unsupported Straydog GPU matrix format");
    const size_t row_bytes = size_t(proj_cols) * (proj_kind == 0 ? 4 : 2), unit = proj_kind == 0 ? 4 : 8;
    span(value, proj_weights, checked_product({heads, row_bytes}), "a weight matrix");
    span(value, x, checked_product({proj_cols, 4}), "a linear input");
    span(value, weights, checked_product({heads, 4}), "index weights");
    const bool units_path = proj_cols % unit == 0 && reinterpret_cast<uintptr_t>(proj_weights) % 16 == 0 && row_bytes % 16 == 0 &&
                            reinterpret_cast<uintptr_t>(x) % 16 == 0;
    index_proj_kernel<<<unsigned((heads + 7) / 8), 256, 0, value.stream>>>(static_cast<const uint8_t*>(proj_weights), proj_kind, row_bytes,
                                                                            size_t(heads), size_t(proj_cols), x, units_path, weights);
    ++value.launches;
    SDB_CHECK(cudaGetLastError());
    if (sd_op_index_select(handle, q, keys, weights, visible, 1, groups, heads, dim, scale, rope_dims, positions, frequencies, scores, k, out,
                           candidates, blocks, block))
        throw std::runtime_error(last_error);
    SDB_OP_END
}

}  // extern "C"
