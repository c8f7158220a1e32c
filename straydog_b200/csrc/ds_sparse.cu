// sd_op_sparse_attention: DeepSeek-V4.1-style latent attention. Each query row attends the window
// rows of an F32 ring ending at its position and the compressed rows its selection lists (-1: none),
// keys being also the values, with a per-head sink in the softmax max and denominator; the last
// rope_dims columns of q are rotated by position * frequency (in double) and the output's rotated back.
// Reference: gpu/kernels.cpp:5311-5476 (entry, validation), gpu/ops.hpp:1203-1235 (BF16-tagged rows),
// :1240-1297 (definition), :1309-1327 (key order, rope table), :1528-1538 (inverse rope), :1561-1583 (sink).
//
// This file holds the entries, the rope table and the FP32 CUDA-core kernel (exact FP32 products for any
// operand values and any dim); ds_sparse_mma3.cu holds the tensor-core kernel the entries prefer when the
// shape allows it (dim 512 or 576).
#include "common.cuh"
#include "ds_sparse.cuh"
#include "../../include/straydog_gpu_b200.h"

#include <algorithm>
#include <cstdlib>

namespace sdb {

// One row's rope, once: forward (cos, sin) of p * f, then of that angle times -1.0 by its own sincos
// (gpu/ops.hpp:1318-1327: "not a negated sine").
__global__ void sparse_turns_kernel(const int32_t* __restrict__ positions, const float* __restrict__ frequencies, size_t pairs,
                                    double2* __restrict__ forward, double2* __restrict__ inverse) {
    const int64_t p = positions[blockIdx.x];
    for (size_t pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
        double s, c;
        sincos(double(p) * double(frequencies[pair]), &s, &c);
        forward[size_t(blockIdx.x) * pairs + pair] = make_double2(c, s);
        sincos(double(p) * double(frequencies[pair]) * -1.0, &s, &c);
        inverse[size_t(blockIdx.x) * pairs + pair] = make_double2(c, s);
    }
}

// q with its last 2 * pairs columns rotated in adjacent pairs (double arithmetic, rounded to F32: gpu/ops.hpp:1366-1377), for the
// FP32 kernel (the tensor-core kernel rotates its own queries).
__global__ void __launch_bounds__(128) sparse_rotate_q_kernel(const float* __restrict__ q, size_t heads, size_t dim, size_t pairs,
                                                              const double2* __restrict__ forward, float* __restrict__ rotated_q) {
    // block = (head, row); a thread takes adjacent column pairs (a rope pair never straddles two threads: dim - 2 * pairs columns come first)
    const size_t head = blockIdx.x, row = blockIdx.y, plain = dim - 2 * pairs;
    const size_t base = (row * heads + head) * dim;
    for (size_t col = threadIdx.x; col < plain; col += blockDim.x) rotated_q[base + col] = q[base + col];
    for (size_t pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
        const size_t col = plain + 2 * pair;
        const double2 g = forward[row * pairs + pair];
        const double a = q[base + col], b = q[base + col + 1];
        rotated_q[base + col] = float(a * g.x - b * g.y);
        rotated_q[base + col + 1] = float(a * g.y + b * g.x);
    }
}

// ---- FP32 kernel: block = (row, group of 4 heads, split); a warp per key ----
constexpr int kSimtHeads = 4, kSimtWarps = 8;

// The partial of split s of (row, head) goes to slot part0 + s of that pair's `parts` slots (parts == 0: one slot per split).
template<int PER_LANE>
__global__ void __launch_bounds__(kSimtWarps * 32) sparse_simt_kernel(const SparseArgs a, const float* __restrict__ q, float* __restrict__ partial,
                                                                      size_t parts, size_t part0) {
    const size_t row = blockIdx.x, head0 = size_t(blockIdx.y) * kSimtHeads, split = blockIdx.z, splits = gridDim.z;
    const unsigned lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const KeyList list = key_list(a, row);
    const size_t share = (list.total + splits - 1) / splits, begin = min(list.total, split * share), end = min(list.total, begin + share);
    if (!parts) parts = splits;
    extern __shared__ float shared[];
    float* qs = shared;                                  // [kSimtHeads][dim]
    float* merged = shared + kSimtHeads * a.dim;         // [kSimtHeads][dim]
    __shared__ float tops[kSimtWarps][kSimtHeads], sums[kSimtWarps][kSimtHeads];
    for (size_t i = threadIdx.x; i < kSimtHeads * a.dim; i += blockDim.x) {
        const size_t head = head0 + i / a.dim;
        qs[i] = head < a.heads ? q[(row * a.heads + head) * a.dim + i % a.dim] : 0.0f;
        merged[i] = 0.0f;
    }
    __syncthreads();
    float m[kSimtHeads], l[kSimtHeads], acc[kSimtHeads][PER_LANE];
    #pragma unroll
    for (int h = 0; h < kSimtHeads; ++h) {
        m[h] = -INFINITY; l[h] = 0.0f;
        #pragma unroll
        for (int j = 0; j < PER_LANE; ++j) acc[h][j] = 0.0f;
    }
    for (size_t index = begin + warp; index < end; index += kSimtWarps) {
        const float* key = key_pointer(a, list, row, index);
        if (!key) continue;
        float k[PER_LANE];
        if (state_is_bf16(key)) {
            const uint16_t* halves = state_halves(key);
            #pragma unroll
            for (int j = 0; j < PER_LANE; ++j) { const size_t d = lane + 32 * j; k[j] = d < a.dim ? __uint_as_float(uint32_t(halves[d]) << 16) : 0.0f; }
        } else {
            #pragma unroll
            for (int j = 0; j < PER_LANE; ++j) { const size_t d = lane + 32 * j; k[j] = d < a.dim ? key[d] : 0.0f; }
        }
        #pragma unroll
        for (int h = 0; h < kSimtHeads; ++h) {
            float dot = 0.0f;
            #pragma unroll
            for (int j = 0; j < PER_LANE; ++j) { const size_t d = lane + 32 * j; dot = fmaf(d < a.dim ? qs[h * a.dim + d] : 0.0f, k[j], dot); }
            #pragma unroll
            for (unsigned offset = 16; offset; offset /= 2) dot += __shfl_xor_sync(0xffffffffu, dot, offset);
            const float score = dot * a.scale, next = fmaxf(m[h], score);
            const float correction = expf(m[h] - next), p = expf(score - next);
            l[h] = fmaf(l[h], correction, p);
            #pragma unroll
            for (int j = 0; j < PER_LANE; ++j) acc[h][j] = fmaf(acc[h][j], correction, p * k[j]);
            m[h] = next;
        }
    }
    if (lane == 0)
        #pragma unroll
        for (int h = 0; h < kSimtHeads; ++h) { tops[warp][h] = m[h]; sums[warp][h] = l[h]; }
    __syncthreads();
    float top[kSimtHeads], total[kSimtHeads];
    #pragma unroll
    for (int h = 0; h < kSimtHeads; ++h) {
        top[h] = tops[0][h];
        for (int w = 1; w < kSimtWarps; ++w) top[h] = fmaxf(top[h], tops[w][h]);
        total[h] = 0.0f;
        for (int w = 0; w < kSimtWarps; ++w) total[h] += tops[w][h] == -INFINITY ? 0.0f : sums[w][h] * expf(tops[w][h] - top[h]);
    }
    for (int w = 0; w < kSimtWarps; ++w) {   // warps add in turn: a fixed order
        if (int(warp) == w) {
            #pragma unroll
            for (int h = 0; h < kSimtHeads; ++h) {
                if (m[h] == -INFINITY) continue;
                const float factor = expf(m[h] - top[h]);
                #pragma unroll
                for (int j = 0; j < PER_LANE; ++j) { const size_t d = lane + 32 * j; if (d < a.dim) merged[h * a.dim + d] += factor * acc[h][j]; }
            }
        }
        __syncthreads();
    }
    // the split's partial: [dim sums | max | denominator] per (row, head, split)
    for (size_t i = threadIdx.x; i < kSimtHeads * a.dim; i += blockDim.x) {
        const size_t h = i / a.dim, head = head0 + h;
        if (head < a.heads) partial[((row * a.heads + head) * parts + part0 + split) * (a.dim + 2) + i % a.dim] = merged[i];
    }
    if (threadIdx.x < kSimtHeads && head0 + threadIdx.x < a.heads) {
        float* at = partial + ((row * a.heads + head0 + threadIdx.x) * parts + part0 + split) * (a.dim + 2) + a.dim;
        at[0] = top[threadIdx.x]; at[1] = total[threadIdx.x];
    }
}

// The splits of a (row, head) combined with the head's sink (in the max and the denominator,
// gpu/ops.hpp:1561-1583), divided, and the rotated columns turned back (gpu/ops.hpp:1528-1538).
__global__ void __launch_bounds__(128) sparse_combine_kernel(const float* __restrict__ partial, size_t splits, size_t heads, size_t dim,
                                                             const float* __restrict__ sinks, size_t pairs, const double2* __restrict__ inverse,
                                                             float* __restrict__ out) {
    const size_t item = blockIdx.x, row = item / heads, head = item % heads, plain = dim - 2 * pairs;
    const float* first = partial + item * splits * (dim + 2);
    constexpr int kMaxSplits = 64;
    __shared__ float factors[kMaxSplits];
    __shared__ float denominator_shared;
    // (the usual shape - an even dim of at most 768, at most four partials - has its sums on their way from memory before the first
    //  warp has the factors: the kernel is a chain of two round trips to memory otherwise)
    constexpr int kEarlyPairs = 3, kEarlySplits = 4;
    const bool early = dim % 2 == 0 && dim / 2 <= size_t(kEarlyPairs) * 128 && splits <= size_t(kEarlySplits) && blockDim.x == 128;
    float2 sums_early[kEarlyPairs][kEarlySplits];
    if (early) {
        #pragma unroll
        for (int k = 0; k < kEarlyPairs; ++k)
            #pragma unroll
            for (int sp = 0; sp < kEarlySplits; ++sp) {
                const size_t pair = threadIdx.x + 128 * k;
                sums_early[k][sp] = pair < dim / 2 && size_t(sp) < splits ? *reinterpret_cast<const float2*>(first + sp * (dim + 2) + 2 * pair) : make_float2(0.0f, 0.0f);
            }
    }
    if (threadIdx.x < 32) {
        // the first warp: the head's maximum (with its sink), every split's factor and the denominator
        const float sink = sinks[head];
        float tops[kMaxSplits / 32], sums[kMaxSplits / 32], top = sink;
        #pragma unroll
        for (int i = 0; i < kMaxSplits / 32; ++i) {
            const size_t s = threadIdx.x + 32 * i;
            tops[i] = s < splits ? first[s * (dim + 2) + dim] : -INFINITY;
            sums[i] = s < splits ? first[s * (dim + 2) + dim + 1] : 0.0f;
            top = fmaxf(top, tops[i]);
        }
        #pragma unroll
        for (unsigned offset = 16; offset; offset /= 2) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
        float denominator = 0.0f;
        #pragma unroll
        for (int i = 0; i < kMaxSplits / 32; ++i) {
            const size_t s = threadIdx.x + 32 * i;
            const float factor = tops[i] == -INFINITY ? 0.0f : expf(tops[i] - top);
            if (s < splits) factors[s] = factor;
            denominator += factor * sums[i];
        }
        #pragma unroll
        for (unsigned offset = 16; offset; offset /= 2) denominator += __shfl_xor_sync(0xffffffffu, denominator, offset);
        // (a sink of -inf adds 0; top is finite whenever any key or the sink is)
        if (threadIdx.x == 0) denominator_shared = denominator + expf(sink - top);
    }
    __syncthreads();
    const float denominator = denominator_shared;
    for (size_t pair = threadIdx.x; pair < dim / 2 + dim % 2; pair += blockDim.x) {
        const size_t d = 2 * pair;
        float o[2] = {0.0f, 0.0f};
        if (early) {
            const int k = int(pair / 128);
            #pragma unroll
            for (int kk = 0; kk < kEarlyPairs; ++kk)
                if (kk == k) {
                    #pragma unroll
                    for (int sp = 0; sp < kEarlySplits; ++sp)
                        if (size_t(sp) < splits) { o[0] = fmaf(sums_early[kk][sp].x, factors[sp], o[0]); o[1] = fmaf(sums_early[kk][sp].y, factors[sp], o[1]); }
                }
        } else if (d + 1 < dim && dim % 2 == 0) {
            for (size_t s = 0; s < splits; ++s) {
                const float2 x = *reinterpret_cast<const float2*>(first + s * (dim + 2) + d);   // (rows of dim + 2 floats, d even: 8-byte aligned when dim is even)
                o[0] = fmaf(x.x, factors[s], o[0]);
                o[1] = fmaf(x.y, factors[s], o[1]);
            }
        } else {
            for (size_t s = 0; s < splits; ++s) {
                o[0] = fmaf(first[s * (dim + 2) + d], factors[s], o[0]);
                if (d + 1 < dim) o[1] = fmaf(first[s * (dim + 2) + d + 1], factors[s], o[1]);
            }
        }
        o[0] /= denominator; o[1] /= denominator;
        if (d >= plain && d + 1 < dim) {
            const double2 g = inverse[row * pairs + (d - plain) / 2];
            const double x = o[0], y = o[1];
            o[0] = float(x * g.x - y * g.y);
            o[1] = float(x * g.y + y * g.x);
        }
        out[item * dim + d] = o[0];
        if (d + 1 < dim) out[item * dim + d + 1] = o[1];
    }
}

static void turns_reserve(Device& d, size_t rows, size_t pairs) {
    if (!pairs || !rows) return;
    if (d.turns && d.turns_rows >= rows && d.turns_pairs == pairs) return;
    SDB_CHECK(cudaStreamSynchronize(d.stream));
    if (d.turns) SDB_CHECK(cudaFree(d.turns));
    d.turns = nullptr;
    SDB_CHECK(cudaMalloc(reinterpret_cast<void**>(&d.turns), rows * pairs * 2 * sizeof(double2)));
    d.turns_rows = rows; d.turns_pairs = pairs;
}

// The window rows' share of one (row, head), for the tcgen05 kernel: a warp walks the row's few window keys (lanes over the
// columns), exact FP32 arithmetic, online softmax in the natural domain; the result is slot 0 of the pair's `parts` partials.
template<int PER_LANE>
__global__ void __launch_bounds__(256) sparse_window_kernel(const SparseArgs a, const float* __restrict__ q, float* __restrict__ partial, size_t rows, size_t parts) {
    const size_t pair = size_t(blockIdx.x) * 8 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (pair >= rows * a.heads) return;
    const size_t row = pair / a.heads;
    const KeyList list = key_list(a, row);
    float qv[PER_LANE], acc[PER_LANE];
    #pragma unroll
    for (int j = 0; j < PER_LANE; ++j) { const size_t d = lane + 32 * j; qv[j] = d < a.dim ? q[pair * a.dim + d] : 0.0f; acc[j] = 0.0f; }
    float m = -INFINITY, l = 0.0f;
    for (size_t index = 0; index < list.raw_count; ++index) {
        const float* key = key_pointer(a, list, row, index);
        float k[PER_LANE], dot = 0.0f;
        #pragma unroll
        for (int j = 0; j < PER_LANE; ++j) { const size_t d = lane + 32 * j; k[j] = d < a.dim ? key[d] : 0.0f; dot = fmaf(qv[j], k[j], dot); }
        #pragma unroll
        for (unsigned offset = 16; offset; offset /= 2) dot += __shfl_xor_sync(0xffffffffu, dot, offset);
        const float score = dot * a.scale, next = fmaxf(m, score), correction = expf(m - next), p = expf(score - next);
        l = fmaf(l, correction, p);
        #pragma unroll
        for (int j = 0; j < PER_LANE; ++j) acc[j] = fmaf(acc[j], correction, p * k[j]);
        m = next;
    }
    float* mine = partial + pair * parts * (a.dim + 2);
    #pragma unroll
    for (int j = 0; j < PER_LANE; ++j) { const size_t d = lane + 32 * j; if (d < a.dim) mine[d] = acc[j]; }
    if (lane == 0) { mine[a.dim] = m; mine[a.dim + 1] = l; }
}

static void launch_simt(Device& d, const SparseArgs& args, const float* q_used, float* partial, size_t rows, size_t splits, size_t parts, size_t part0) {
    const size_t groups = (args.heads + kSimtHeads - 1) / kSimtHeads;
    const dim3 grid{unsigned(rows), unsigned(groups), unsigned(splits)};
    const size_t shared = 2 * kSimtHeads * size_t(args.dim) * 4;
    const int per_lane = int((args.dim + 31) / 32);
    // (the opt-in for more than 48 KB of dynamic shared memory is asked once per device and kernel, not per launch: a driver call)
    #define SDB_SIMT(N) do { \
        static size_t allowed[64] = {}; \
        if (allowed[d.ordinal & 63] < shared) { \
            SDB_CHECK(cudaFuncSetAttribute(sparse_simt_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(shared))); \
            allowed[d.ordinal & 63] = shared; } \
        sparse_simt_kernel<N><<<grid, kSimtWarps * 32, shared, d.stream>>>(args, q_used, partial, parts, part0); } while (0)
    if (per_lane <= 4) SDB_SIMT(4); else if (per_lane <= 8) SDB_SIMT(8); else if (per_lane <= 16) SDB_SIMT(16);
    else if (per_lane <= 18) SDB_SIMT(18); else SDB_SIMT(32);
    #undef SDB_SIMT
    ++d.launches;
    SDB_CHECK(cudaGetLastError());
}

// For the tcgen05 kernel: the window rows' share of every (row, head) as slot 0 of its `parts` partials, in exact FP32 arithmetic.
void sparse_window_partial(Device& d, const SparseArgs& a, const float* q, size_t rows, size_t pairs, const double2* forward, float* rotated,
                           float* partial, size_t parts, cudaStream_t stream) {
    if (!stream) stream = d.stream;
    const float* q_used = q;
    if (pairs) {
        sparse_rotate_q_kernel<<<dim3(unsigned(a.heads), unsigned(rows)), 128, 0, stream>>>(q, a.heads, a.dim, pairs, forward, rotated);
        ++d.launches;
        q_used = rotated;
    }
    SparseArgs window = a;
    window.selections = 0;   // (the key list of a row is then its window rows alone)
    const unsigned blocks = unsigned((rows * a.heads + 7) / 8);
    if (a.dim <= 512) sparse_window_kernel<16><<<blocks, 256, 0, stream>>>(window, q_used, partial, rows, parts);
    else sparse_window_kernel<18><<<blocks, 256, 0, stream>>>(window, q_used, partial, rows, parts);
    ++d.launches;
    SDB_CHECK(cudaGetLastError());
}

void sparse_combine(Device& d, const float* partial, size_t parts, size_t rows, size_t heads, size_t dim, const float* sinks, size_t pairs,
                    const double2* inverse, float* out) {
    sparse_combine_kernel<<<unsigned(rows * heads), 128, 0, d.stream>>>(partial, parts, heads, dim, sinks, pairs, inverse, out);
    ++d.launches;
    SDB_CHECK(cudaGetLastError());
}

// The tensor-core kernel holds dim 512 and 576 and needs 16-byte aligned BF16 rows (whole rows travel by bulk copies).
bool sparse_mma_supported(const SparseArgs& a) {
    if (a.dim != 512 && a.dim != 576) return false;
    if (a.selections && state_is_bf16(a.compressed) && reinterpret_cast<uintptr_t>(state_halves(a.compressed)) % 16) return false;
    return true;
}

static bool env_flag(const char* name) {
    const char* v = std::getenv(name);
    return v && v[0] == '1' && !v[1];
}

}  // namespace sdb

using namespace sdb;

extern "C" {

int sd_attention_turns_reserve(void* handle, uint64_t rows, uint64_t rope_dims) {
    try {
        if (rope_dims > 128 || rope_dims % 2) throw std::runtime_error("invalid Straydog attention rope");
        turns_reserve(device(handle), size_t(rows), size_t(rope_dims / 2));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

// In the reference the next norm+rope op of exactly `rows` rows then fills the table so that the
// attention skips its own rope launch (gpu/straydog_gpu.h:386-389). Those ops are outside this
// library, so nothing ever fills it early: arming is accepted and the attention fills the table itself.
int sd_attention_turns_arm(void* handle, uint64_t rows) {
    try {
        auto& value = device(handle);
        (void)rows;
        value.turns_ready = false;
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

// The body of both entries. spans > 1: `rows` = spans * span_rows query rows, span s with its own window ring
// raw + s * raw_rows * dim and positions counted in that ring; everything else as in a single call.
static int sparse_attention_call(void* handle, const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions,
                                 uint64_t window, const float* compressed, uint64_t compressed_rows, const int32_t* selected,
                                 uint64_t selections, const float* sinks, uint64_t rows, uint64_t heads, uint64_t dim, float scale,
                                 uint64_t rope_dims, const float* frequencies, float* scratch, uint64_t scratch_bytes, float* out,
                                 uint64_t spans, uint64_t span_rows, const GatherTargets* gather = nullptr) {
    SDB_OP_BEGIN
    if (!rows || rows > 65535 || !heads || !dim || !window || rope_dims % 2 || rope_dims > dim || rope_dims > 128)
        throw std::runtime_error("invalid Straydog attention shape");
    if (dim > 1024 || heads > 65535 * kSimtHeads || !raw_rows) throw std::runtime_error("invalid Straydog attention shape");
    if (rope_dims) span(value, frequencies, size_t(rope_dims / 2) * 4, "rope frequencies");
    span(value, q, checked_product({rows, heads, dim, 4}), "attention queries");
    span(value, raw, checked_product({spans, raw_rows, dim, 4}), "window rows");
    span(value, positions, checked_product({rows, 4}), "query positions");
    if (selections) {
        if (state_is_bf16(compressed)) span(value, state_halves(compressed), checked_product({compressed_rows, dim, 2}), "compressed rows");
        else span(value, compressed, checked_product({compressed_rows, dim, 4}), "compressed rows");
        span(value, selected, checked_product({rows, selections, 4}), "selected rows");
    }
    span(value, sinks, checked_product({heads, 4}), "attention sinks");
    if (!gather) span(value, out, checked_product({rows, heads, dim, 4}), "an attention output");
    if (scratch && scratch_bytes) span(value, scratch, size_t(scratch_bytes), "attention scratch");

    const size_t pairs = size_t(rope_dims / 2);
    double2* forward = nullptr;
    double2* inverse = nullptr;
    if (pairs) {
        turns_reserve(value, size_t(rows), pairs);
        forward = reinterpret_cast<double2*>(value.turns);
        inverse = forward + value.turns_rows * pairs;
        sparse_turns_kernel<<<unsigned(rows), 64, 0, value.stream>>>(positions, frequencies, pairs, forward, inverse);
        ++value.launches;
    }
    value.turns_ready = false;

    SparseArgs args{};
    args.raw = raw; args.raw_rows = raw_rows; args.positions = positions; args.window = window; args.compressed = compressed;
    args.compressed_rows = compressed_rows; args.selected = selected; args.selections = selections; args.heads = heads; args.dim = dim;
    args.scale = scale;
    args.span_rows = spans > 1 ? span_rows : rows;   // (one span: every row in ring 0)

    if (gather) {   // (the gathered form exists in the third tensor-core kernel only)
        if (!sparse_mma_supported(args)) throw std::runtime_error("the gathered latent attention needs dim 512 or 576 and 16-byte aligned rows");
        sparse_mma3_launch(value, args, q, sinks, rows, pairs, forward, inverse, nullptr, gather);
        SDB_CHECK(cudaGetLastError());
        return 0;
    }
    const bool force_simt = env_flag("SDX_SPARSE_SIMT");
    // (SDX_SPARSE_KERNEL=mma3, read at each call, keeps the mma.sync kernel where the tcgen05 kernel would run: the in-library A/B)
    const char* form = std::getenv("SDX_SPARSE_KERNEL");
    if (!force_simt && sparse_tc_supported(args) && !(form && std::string(form) == "mma3")) {
        // (SDX_SPARSE_KERNEL=tc1 keeps the single-CTA tcgen05 kernel where the pair kernel would run)
        if (form && std::string(form) == "tc1") sparse_tc_launch(value, args, q, sinks, rows, pairs, forward, inverse, out);
        else sparse_tc2_launch(value, args, q, sinks, rows, pairs, forward, inverse, out);
        SDB_CHECK(cudaGetLastError());
        return 0;
    }
    if (!force_simt && sparse_mma_supported(args)) {
        sparse_mma3_launch(value, args, q, sinks, rows, pairs, forward, inverse, out);
        SDB_CHECK(cudaGetLastError());
        return 0;
    }

    // FP32 path. Workspace (library-owned, grown on the first call of a size): rotated q, then the splits' partials.
    const size_t stride = size_t(window + selections);
    const size_t groups = (heads + kSimtHeads - 1) / kSimtHeads;
    size_t splits = std::max<size_t>(1, std::min<size_t>({size_t(32), (stride + 63) / 64, size_t(value.sms) * 4 / std::max<size_t>(1, rows * groups)}));
    splits = std::max<size_t>(splits, 1);
    const size_t q_bytes = pairs ? (checked_product({rows, heads, dim, 4}) + 255) / 256 * 256 : 0;
    const size_t partial_bytes = checked_product({rows, heads, splits, dim + 2, 4});
    auto* work = static_cast<uint8_t*>(ensure(value, value.partial, value.partial_bytes, q_bytes + partial_bytes));
    const float* q_used = q;
    if (pairs) {
        auto* rotated = reinterpret_cast<float*>(work);
        sparse_rotate_q_kernel<<<dim3(unsigned(heads), unsigned(rows)), 128, 0, value.stream>>>(q, heads, dim, pairs, forward, rotated);
        ++value.launches;
        q_used = rotated;
    }
    auto* partial = reinterpret_cast<float*>(work + q_bytes);
    launch_simt(value, args, q_used, partial, rows, splits, 0, 0);
    sparse_combine_kernel<<<unsigned(rows * heads), 128, 0, value.stream>>>(partial, splits, heads, dim, sinks, pairs, inverse, out);
    ++value.launches;
    SDB_OP_END
}

int sd_op_sparse_attention(void* handle, const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions,
                           uint64_t window, const float* compressed, uint64_t compressed_rows, const int32_t* selected,
                           uint64_t selections, const float* sinks, uint64_t rows, uint64_t heads, uint64_t dim, float scale,
                           uint64_t rope_dims, const float* frequencies, float* scratch, uint64_t scratch_bytes, float* out) {
    return sparse_attention_call(handle, q, raw, raw_rows, positions, window, compressed, compressed_rows, selected, selections, sinks, rows,
                                 heads, dim, scale, rope_dims, frequencies, scratch, scratch_bytes, out, 1, rows);
}

int sdx_sparse_attention_spans(void* handle, const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions,
                               uint64_t window, const float* compressed, uint64_t compressed_rows, const int32_t* selected,
                               uint64_t selections, const float* sinks, uint64_t spans, uint64_t span_rows, uint64_t heads, uint64_t dim,
                               float scale, uint64_t rope_dims, const float* frequencies, float* out) {
    try {
        if (!spans || !span_rows || spans > 65535 || span_rows > 65535) throw std::runtime_error("invalid Straydog attention shape");
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
    return sparse_attention_call(handle, q, raw, raw_rows, positions, window, compressed, compressed_rows, selected, selections, sinks,
                                 spans * span_rows, heads, dim, scale, rope_dims, frequencies, nullptr, 0, out, spans, span_rows);
}


int sdx_sparse_attention_gather(void* handle, const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions,
                                uint64_t window, const float* compressed, uint64_t compressed_rows, const int32_t* selected,
                                uint64_t selections, const float* sinks, uint64_t rows, uint64_t heads, uint64_t dim, float scale,
                                uint64_t rope_dims, const float* frequencies, uint64_t world, uint64_t rank, void* const* outs,
                                void* const* flags, int32_t step) {
    GatherTargets gather{};
    try {
        auto& value = device(handle);
        if (!world || world > uint64_t(kMaxGatherWorld) || rank >= world || !outs || !flags) throw std::runtime_error("invalid gather of Straydog attention outputs");
        const size_t bytes = checked_product({world, rows, heads, dim, 4});
        for (uint64_t peer = 0; peer < world; ++peer) {
            span_or_peer(value, outs[peer], bytes, "a gathered attention output");
            span_or_peer(value, flags[peer], size_t(world) * 4, "a gather's arrival counters");
            if (reinterpret_cast<uintptr_t>(outs[peer]) % 8 || dim % 2) throw std::runtime_error("a gathered attention output must be 8-byte aligned");
            gather.out[peer] = static_cast<float*>(outs[peer]);
            gather.flags[peer] = static_cast<int*>(flags[peer]);
        }
        gather.world = uint32_t(world); gather.rank = uint32_t(rank); gather.step = step;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
    return sparse_attention_call(handle, q, raw, raw_rows, positions, window, compressed, compressed_rows, selected, selections, sinks, rows,
                                 heads, dim, scale, rope_dims, frequencies, nullptr, 0, nullptr, 1, rows, &gather);
}

}  // extern "C"
