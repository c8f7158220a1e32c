// sd_op_top_k and sd_op_to_bf16: the index-list producer's contract and the BF16 rounding op.
//
// Top-k (gpu/straydog_gpu.h:409; rule: gpu/ops.hpp:1741-1742, 1766-1769, 1797-1874 and
// crates/straydog-engine/tests/fused_gpu.rs:325-357): per row the k highest scores' indices in
// ascending index order; ties at the threshold keep the lowest indices; -inf is never kept; -0 ties
// +0; unused slots hold -1. Bit-exact integer work: a most-significant-byte-first radix select over
// order-preserving keys finds the k-th key, then one ordered pass compacts the kept indices.
//
// One block of 1024 threads per row; a row's scores are read five times (four histogram passes
// and the compaction), all but the first from L2 for the row sizes the indexer produces (<= 1 MB).
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

namespace sdb {

constexpr int kTopThreads = 1024, kTopRun = 4;   // consecutive scores a thread takes in the ordered pass

__device__ __forceinline__ uint32_t order_key(float value) {
    const uint32_t bits = __float_as_uint(value == 0.0f ? 0.0f : value);   // -0 ties +0, as the floats compare
    return bits & 0x80000000u ? ~bits : bits | 0x80000000u;
}

// Exclusive prefix of `value` over the block in thread order, and the block's total.
__device__ __forceinline__ uint32_t block_scan(uint32_t value, uint32_t* warp_sums, uint32_t& total) {
    const unsigned lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    uint32_t inclusive = value;
    #pragma unroll
    for (unsigned offset = 1; offset < 32; offset *= 2) {
        const uint32_t other = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if (lane >= offset) inclusive += other;
    }
    __syncthreads();   // (warp_sums may still be read from the previous scan)
    if (lane == 31) warp_sums[warp] = inclusive;
    __syncthreads();
    uint32_t before = 0, sum = 0;
    #pragma unroll
    for (unsigned w = 0; w < kTopThreads / 32; ++w) {
        const uint32_t c = warp_sums[w];
        before += w < warp ? c : 0u;
        sum += c;
    }
    total = sum;
    return before + inclusive - value;
}

__global__ void __launch_bounds__(kTopThreads) top_k_kernel(const float* __restrict__ scores, size_t groups, size_t k, int32_t* __restrict__ out) {
    const float* row = scores + size_t(blockIdx.x) * groups;
    int32_t* mine = out + size_t(blockIdx.x) * k;
    const unsigned t = threadIdx.x;
    const uint32_t floor_key = order_key(-INFINITY);
    __shared__ uint32_t bins[256];
    __shared__ uint32_t warp_sums[kTopThreads / 32];
    __shared__ uint32_t picked_bin, picked_left, picked_count, live_total;
    uint32_t prefix = 0, rank = uint32_t(k);
    bool all = false;
    uint32_t equal_count = 0;
    for (int byte = 3; byte >= 0; --byte) {
        for (unsigned bin = t; bin < 256; bin += kTopThreads) bins[bin] = 0;
        __syncthreads();
        const int shift = 8 * byte;
        for (size_t g = t; g < groups; g += kTopThreads) {
            const uint32_t key = order_key(row[g]);
            if (key > floor_key && (byte == 3 || (key >> (shift + 8)) == (prefix >> (shift + 8)))) atomicAdd(&bins[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        // the first warp walks the bins from the top: lane i takes bins 255 - 8i .. 248 - 8i
        if (t < 32) {
            uint32_t counts[8], sum = 0;
            #pragma unroll
            for (int i = 0; i < 8; ++i) { counts[i] = bins[255 - (8 * t + i)]; sum += counts[i]; }
            uint32_t inclusive = sum;
            #pragma unroll
            for (unsigned offset = 1; offset < 32; offset *= 2) {
                const uint32_t other = __shfl_up_sync(0xffffffffu, inclusive, offset);
                if (t >= offset) inclusive += other;
            }
            const uint32_t every = __shfl_sync(0xffffffffu, inclusive, 31);
            uint32_t above = inclusive - sum;
            if (t == 0) live_total = every;
            if (every < rank) {            // fewer candidates than wanted: the lowest bin stands (all are kept)
                if (t == 31) { picked_bin = 0; picked_left = rank - (every - counts[7]); picked_count = counts[7]; }
            } else if (above < rank && above + sum >= rank) {
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (above < rank && above + counts[i] >= rank) { picked_bin = 255 - (8 * t + i); picked_left = rank - above; picked_count = counts[i]; }
                    above += counts[i];
                }
            }
        }
        __syncthreads();
        if (byte == 3 && live_total <= k) { all = true; break; }
        prefix |= picked_bin << shift;
        rank = picked_left;
        equal_count = picked_count;
        __syncthreads();
    }
    const uint32_t threshold = prefix, need = all ? 0u : rank;   // `need` of the keys equal to the threshold are kept
    const bool every_tie = all || equal_count <= need;
    uint32_t slot = 0, ties_seen = 0;
    const size_t tile = size_t(kTopThreads) * kTopRun;
    for (size_t start = 0; start < groups; start += tile) {
        const size_t first = start + size_t(t) * kTopRun;
        uint32_t keys[kTopRun], ties = 0;
        #pragma unroll
        for (int i = 0; i < kTopRun; ++i) {
            keys[i] = first + i < groups ? order_key(row[first + i]) : floor_key;
            ties += !all && keys[i] == threshold && keys[i] > floor_key;
        }
        uint32_t tie_before = 0, tile_ties = 0;
        if (!every_tie) tie_before = ties_seen + block_scan(ties, warp_sums, tile_ties);
        bool keep[kTopRun];
        uint32_t kept = 0;
        #pragma unroll
        for (int i = 0; i < kTopRun; ++i) {
            const bool live = keys[i] > floor_key, equal = !all && live && keys[i] == threshold;
            keep[i] = live && (all || keys[i] > threshold || (equal && (every_tie || tie_before < need)));
            tie_before += equal;
            kept += keep[i];
        }
        uint32_t tile_kept;
        uint32_t at = slot + block_scan(kept, warp_sums, tile_kept);
        #pragma unroll
        for (int i = 0; i < kTopRun; ++i)
            if (keep[i] && at < k) mine[at++] = int32_t(first + i);
        slot += tile_kept;
        ties_seen += tile_ties;
    }
    for (size_t i = slot + t; i < k; i += kTopThreads) mine[i] = -1;
}

// out[i] = x[i] as BF16: nearest, ties to even; a NaN stays a NaN (gpu/token_mixing.hpp:728-735).
__global__ void __launch_bounds__(256) to_bf16_kernel(const float* __restrict__ x, size_t count, uint16_t* __restrict__ out) {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x) {
        const uint32_t bits = __float_as_uint(x[i]);
        out[i] = (bits & 0x7fffffffu) > 0x7f800000u ? uint16_t((bits >> 16) | 0x40u) : uint16_t((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
    }
}

}  // namespace sdb

using namespace sdb;

extern "C" {

int sd_op_top_k(void* handle, const float* scores, uint64_t rows, uint64_t groups, uint64_t k, int32_t* out) {
    SDB_OP_BEGIN
    if (!rows || !groups || !k || groups > (uint64_t(1) << 31) || k > (uint64_t(1) << 31) || rows > 0x7fffffffull)
        throw std::runtime_error("invalid Straydog top-k shape");
    span(value, scores, checked_product({rows, groups, 4}), "scores");
    span(value, out, checked_product({rows, k, 4}), "top-k indices");
    top_k_kernel<<<unsigned(rows), kTopThreads, 0, value.stream>>>(scores, size_t(groups), size_t(k), out);
    ++value.launches;
    SDB_OP_END
}

int sd_op_to_bf16(void* handle, const float* x, uint64_t count, void* out) {
    SDB_OP_BEGIN
    if (!count) return 0;
    span(value, x, checked_product({count, 4}), "values to round");
    span(value, out, checked_product({count, 2}), "BF16 values");
    const unsigned grid = unsigned(std::min<uint64_t>((count + 255) / 256, uint64_t(value.sms) * 16));
    to_bf16_kernel<<<grid, 256, 0, value.stream>>>(x, size_t(count), static_cast<uint16_t*>(out));
    ++value.launches;
    SDB_OP_END
}

}  // extern "C"
