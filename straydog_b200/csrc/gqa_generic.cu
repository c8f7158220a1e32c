// sd_op_attention: generic dense causal grouped-query attention over F32 keys and values
// [context][kv_heads][dim] (gpu/token_mixing.hpp:340-520, 652-694; declared gpu/straydog_gpu.h:453).
// FP32 throughout: the reference's own test holds every output to an FP32-level error bound
// (crates/straydog-engine/tests/attention_gpu.rs:42-49), so no operand is narrowed here.
//
// Flash decoding on CUDA cores: block = (row, head, split of the row's keys); each warp walks its
// keys four at a time (lanes over the dimensions, coalesced), keeps its own online softmax and
// its slice of the weighted sum in registers, and the block's warps merge through shared memory.
// One split writes the output itself; several leave (sum[dim], max, denominator) in the caller's
// scratch, in the reference's partial layout, for the combine kernel.
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

#include <algorithm>

namespace sdb {

constexpr int kGenericMaxDim = 1024;     // gpu/token_mixing.hpp:342
constexpr int kGenericMaxSplits = 64;    // gpu/token_mixing.hpp:343
constexpr int kGenericWarps = 8;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

template<int PER_LANE>   // dimensions per lane: dim <= 32 * PER_LANE
__global__ void __launch_bounds__(kGenericWarps * 32) generic_attention_kernel(
        const float* __restrict__ q, const float* __restrict__ keys, const float* __restrict__ values, size_t context,
        const int32_t* __restrict__ positions, size_t heads, size_t kv_heads, size_t dim, float scale, const float* __restrict__ gate,
        float* __restrict__ partial, float* __restrict__ out) {
    const size_t pair = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const size_t row = pair / heads, h = pair % heads, kh = h / (heads / kv_heads);
    const unsigned lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    // (a position past the cache reads no key past it: tests/attention_gpu.rs:96-101)
    const size_t length = min(size_t(positions[row]) + 1, context);
    const size_t share = (length + splits - 1) / splits;
    const size_t begin = min(length, split * share), end = min(length, begin + share);
    float qv[PER_LANE], acc[PER_LANE];
    #pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        const size_t d = lane + 32 * j;
        qv[j] = d < dim ? q[pair * dim + d] : 0.0f;
        acc[j] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const size_t stride = kv_heads * dim;
    for (size_t key = begin + warp; key < end; key += kGenericWarps) {
        const float* k = keys + key * stride + kh * dim;
        const float* v = values + key * stride + kh * dim;
        float sum = 0.0f, vv[PER_LANE];
        #pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
            const size_t d = lane + 32 * j;
            sum = fmaf(qv[j], d < dim ? k[d] : 0.0f, sum);
            vv[j] = d < dim ? v[d] : 0.0f;
        }
        #pragma unroll
        for (unsigned offset = 16; offset; offset /= 2) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        const float score = sum * scale, next = fmaxf(m, score);
        const float correction = expf(m - next), p = expf(score - next);   // (correction 0 at the first key: m = -inf)
        l = fmaf(l, correction, p);
        #pragma unroll
        for (int j = 0; j < PER_LANE; ++j) acc[j] = fmaf(acc[j], correction, p * vv[j]);
        m = next;
    }
    // merge the block's warps
    __shared__ float tops[kGenericWarps], sums[kGenericWarps];
    __shared__ float merged[kGenericMaxDim];
    if (lane == 0) { tops[warp] = m; sums[warp] = l; }
    for (unsigned d = threadIdx.x; d < dim; d += blockDim.x) merged[d] = 0.0f;
    __syncthreads();
    float top = tops[0];
    #pragma unroll
    for (int w = 1; w < kGenericWarps; ++w) top = fmaxf(top, tops[w]);
    float total = 0.0f;
    #pragma unroll
    for (int w = 0; w < kGenericWarps; ++w) total += tops[w] == -INFINITY ? 0.0f : sums[w] * expf(tops[w] - top);
    const float factor = m == -INFINITY ? 0.0f : expf(m - top);
    // warps add in turn (a fixed order: the same bits every run)
    for (int w = 0; w < kGenericWarps; ++w) {
        if (int(warp) == w && factor != 0.0f) {
            #pragma unroll
            for (int j = 0; j < PER_LANE; ++j) {
                const size_t d = lane + 32 * j;
                if (d < dim) merged[d] += factor * acc[j];
            }
        }
        __syncthreads();
    }
    if (splits == 1) {
        for (unsigned d = threadIdx.x; d < dim; d += blockDim.x) {
            const size_t at = pair * dim + d;
            float value = merged[d] / total;
            if (gate) value *= sigmoid_f(gate[at]);
            out[at] = value;
        }
        return;
    }
    float* mine = partial + (pair * splits + split) * (dim + 2);
    for (unsigned d = threadIdx.x; d < dim; d += blockDim.x) mine[d] = merged[d];
    if (threadIdx.x == 0) { mine[dim] = top; mine[dim + 1] = total; }
}

// The splits of a (row, head) combined: each scaled by exp(its max - the max), normalised, times
// sigmoid(gate) when given (gpu/token_mixing.hpp:486-520).
__global__ void __launch_bounds__(256) generic_attention_combine_kernel(const float* __restrict__ partial, size_t splits, size_t dim,
                                                                        const float* __restrict__ gate, float* __restrict__ out) {
    const size_t pair = blockIdx.x;
    const float* first = partial + pair * splits * (dim + 2);
    __shared__ float scales[kGenericMaxSplits];
    __shared__ float total_shared;
    if (threadIdx.x < 32) {
        float top = -INFINITY;
        for (size_t s = threadIdx.x; s < splits; s += 32) top = fmaxf(top, first[s * (dim + 2) + dim]);
        #pragma unroll
        for (unsigned offset = 16; offset; offset /= 2) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
        for (size_t s = threadIdx.x; s < splits; s += 32) {
            const float own = first[s * (dim + 2) + dim];
            scales[s] = own == -INFINITY ? 0.0f : expf(own - top);
        }
        __syncwarp();
        if (threadIdx.x == 0) {
            float total = 0.0f;
            for (size_t s = 0; s < splits; ++s) total += first[s * (dim + 2) + dim + 1] * scales[s];
            total_shared = total;
        }
    }
    __syncthreads();
    const float total = total_shared;
    for (size_t d = threadIdx.x; d < dim; d += blockDim.x) {
        float sum = 0.0f;
        for (size_t s = 0; s < splits; ++s) sum = fmaf(first[s * (dim + 2) + d], scales[s], sum);
        const size_t at = pair * dim + d;
        float value = sum / total;
        if (gate) value *= sigmoid_f(gate[at]);
        out[at] = value;
    }
}

}  // namespace sdb

using namespace sdb;

extern "C" int sd_op_attention(void* handle, const float* q, const float* keys, const float* values, uint64_t context,
                               const int32_t* positions, uint64_t rows, uint64_t heads, uint64_t kv_heads, uint64_t dim, float scale,
                               const float* gate, float* scratch, uint64_t scratch_bytes, float* out) {
    SDB_OP_BEGIN
    if (!rows || !heads || !kv_heads || heads % kv_heads || !dim || dim > kGenericMaxDim || !context ||
        checked_product({rows, heads}) > 65535ull * 64)
        throw std::runtime_error("invalid Straydog attention shape");
    span(value, q, checked_product({rows, heads, dim, 4}), "attention queries");
    span(value, keys, checked_product({context, kv_heads, dim, 4}), "attention keys");
    span(value, values, checked_product({context, kv_heads, dim, 4}), "attention values");
    span(value, positions, checked_product({rows, 4}), "attention positions");
    if (gate) span(value, gate, checked_product({rows, heads, dim, 4}), "an attention gate");
    span(value, out, checked_product({rows, heads, dim, 4}), "an attention output");
    const size_t pairs = size_t(rows * heads);
    // Many rows (a prefill pass) fill the device by themselves and need no scratch, as in the reference
    // (gpu/token_mixing.hpp:667); few rows split their keys (the reference's split count, :683).
    size_t splits = 1;
    if (!(rows >= 16 && dim == 256)) {
        splits = std::min<size_t>(kGenericMaxSplits, std::max<size_t>(1, 256 / pairs));
        if (splits > 1) {
            const size_t partial_bytes = pairs * splits * (size_t(dim) + 2) * 4;
            if (!scratch || scratch_bytes < partial_bytes) throw std::runtime_error("Straydog attention scratch too small");
            span(value, scratch, partial_bytes, "attention scratch");
        }
    }
    const dim3 grid{unsigned(pairs), unsigned(splits)};
    const int per_lane = int((dim + 31) / 32);
    #define SDB_GENERIC(N) generic_attention_kernel<N><<<grid, kGenericWarps * 32, 0, value.stream>>>( \
        q, keys, values, size_t(context), positions, size_t(heads), size_t(kv_heads), size_t(dim), scale, gate, scratch, out)
    if (per_lane <= 2) SDB_GENERIC(2); else if (per_lane <= 4) SDB_GENERIC(4); else if (per_lane <= 8) SDB_GENERIC(8);
    else if (per_lane <= 16) SDB_GENERIC(16); else SDB_GENERIC(32);
    #undef SDB_GENERIC
    ++value.launches;
    if (splits > 1) {
        SDB_CHECK(cudaGetLastError());
        generic_attention_combine_kernel<<<unsigned(pairs), 256, 0, value.stream>>>(scratch, splits, size_t(dim), gate, out);
        ++value.launches;
    }
    SDB_OP_END
}
