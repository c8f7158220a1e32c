// sd_op_top_k and sd_op_to_bf16: the index-list producer's contract and the BF16 rounding op.
//
// Top-k contract (gpu/straydog_gpu.h:409; rule: gpu/ops.hpp:1741-1742, crates/straydog-engine/tests/fused_gpu.rs:325-357): per
// row the k highest scores' indices in ascending index order; scores equal to the k-th keep the lowest indices; -inf is never
// kept; -0 ties +0; unused slots hold -1. All integer work, bit-exact.
//
// Kernel: one block of 1024 threads a row, built around reading the row from memory twice.
//   read 1   a 2048-bin histogram of the top 11 bits of every live score's sortable key (sixteen private histograms filled by
//            plain shared-memory atomics and added up). The bin in which the running count from the top reaches k is the
//            band: everything above it is kept for sure, everything below is dropped.
//   read 2   in index order: the sure indices go to one shared list, the band's (key, index) pairs to another.
//   then, in shared memory only: the band's next 11 and last 10 key bits are histogrammed the same way, which gives the k-th
//            key itself and how many of its equals are wanted; the band's chosen entries are compacted in index order; the
//            two ascending lists are merged by rank (each entry's place = its own rank + a binary search in the other list).
// A row whose band (or k) does not fit the shared lists - more than 8192 scores sharing their top 11 bits with the k-th, k over
// 4096 - takes the general path: the two refinements read the row again, then one ordered pass compacts straight to the output.
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

namespace sdb {
namespace topk {

constexpr int kThreads = 1024, kWarps = kThreads / 32, kPerThread = 8;
constexpr uint32_t kBins = 2048, kBandCap = 8192, kKeepCap = 4096;
constexpr size_t kSmem = (kBins + kKeepCap + 2 * kBandCap + kKeepCap) * 4;   // histogram | sure | band keys | band indices | chosen

// Order-preserving map of a score to an unsigned key; the two zeros share a key.
__device__ __forceinline__ uint32_t sortable(float score) {
    uint32_t bits = __float_as_uint(score);
    if ((bits << 1) == 0) bits = 0;
    return bits ^ (uint32_t(int32_t(bits) >> 31) | 0x80000000u);
}
constexpr uint32_t kDead = 0x007fffffu;   // sortable(-inf): nothing at or below it is ever kept

struct Shared {
    uint32_t warp_totals[kWarps];
    uint32_t found_bin, found_above, found_count, live;
};

// Exclusive prefix of `mine` over the block in thread order; `total` = the block's sum.
__device__ __forceinline__ uint32_t prefix_before(uint32_t mine, Shared& sh, uint32_t& total) {
    const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t running = mine;
    #pragma unroll
    for (int step = 1; step < 32; step <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, running, step);
        running += lane >= unsigned(step) ? up : 0u;
    }
    __syncthreads();                       // the totals of an earlier call have been read
    if (lane == 31) sh.warp_totals[warp] = running;
    __syncthreads();
    uint32_t mine_total = lane < kWarps ? sh.warp_totals[lane] : 0u, scanned = mine_total;
    #pragma unroll
    for (int step = 1; step < 32; step <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, scanned, step);
        scanned += lane >= unsigned(step) ? up : 0u;
    }
    total = __shfl_sync(0xffffffffu, scanned, 31);
    const uint32_t warps_before = __shfl_sync(0xffffffffu, scanned - mine_total, warp);
    return warps_before + running - mine;
}

// bins[bin] += 1 for every thread with `counted`; equal bins of a warp add once.
__device__ __forceinline__ void count_in(uint32_t* bins, uint32_t bin, bool counted) {
    const unsigned voters = __ballot_sync(0xffffffffu, counted);
    if (!counted) return;
    const unsigned same = __match_any_sync(voters, bin);
    if ((threadIdx.x & 31) == unsigned(__ffs(same) - 1)) atomicAdd(&bins[bin], uint32_t(__popc(same)));
}

// From the highest bin down: the bin in which the running count reaches `wanted` (found_bin, the count above it, its own count), and
// the count of all bins (live). When all bins together hold fewer than `wanted`, found_bin stays at `bins` (no such bin).
__device__ __forceinline__ void find_band(const uint32_t* hist, uint32_t bins, uint32_t wanted, Shared& sh) {
    const uint32_t each = (bins + kThreads - 1) / kThreads;   // bins a thread, taken from the top
    uint32_t counts[2] = {0, 0}, sum = 0;
    for (uint32_t i = 0; i < each; ++i) {
        const uint32_t at = threadIdx.x * each + i;
        counts[i] = at < bins ? hist[bins - 1 - at] : 0u;
        sum += counts[i];
    }
    if (threadIdx.x == 0) sh.found_bin = bins;
    uint32_t total;
    uint32_t above = prefix_before(sum, sh, total);
    for (uint32_t i = 0; i < each; ++i) {
        if (above < wanted && above + counts[i] >= wanted) { sh.found_bin = bins - 1 - (threadIdx.x * each + i); sh.found_above = above; sh.found_count = counts[i]; }
        above += counts[i];
    }
    if (threadIdx.x == 0) sh.live = total;
    __syncthreads();
}

// With `candidates` (a row's `blocks` block numbers in index order, -1 past the last; gpu/ops.hpp:1942-1951) the row's scores are
// those of its candidate groups in candidate order, and a kept place v is written as the group it stands for,
// candidates[v / block] * block + v % block: index order both ways, so the list still ascends.
__global__ void __launch_bounds__(kThreads) top_k_kernel(const float* __restrict__ scores, size_t groups, size_t k, int32_t* __restrict__ out,
                                                         const int32_t* __restrict__ candidates, size_t blocks, size_t block) {
    extern __shared__ __align__(16) uint32_t dynamic[];
    uint32_t* hist = dynamic;
    uint32_t* sure = hist + kBins;              // indices kept for sure, ascending
    uint32_t* band_key = sure + kKeepCap;       // the band in index order
    uint32_t* band_index = band_key + kBandCap;
    uint32_t* chosen = band_index + kBandCap;   // the band's kept indices, ascending
    __shared__ Shared sh;
    const float* row = scores + size_t(blockIdx.x) * groups;
    int32_t* mine = out + size_t(blockIdx.x) * k;
    const unsigned t = threadIdx.x;
    const int32_t* mapped = candidates ? candidates + size_t(blockIdx.x) * blocks : nullptr;
    const auto group_of = [&](uint32_t place) { return mapped ? int32_t(size_t(mapped[place / block]) * block + place % block) : int32_t(place); };

    // ---- read 1: the top 11 key bits ----
    for (uint32_t i = t; i < kBins; i += kThreads) hist[i] = 0;
    __syncthreads();
    // Rows of up to a million scores: sixteen private histograms (a pair of warps each), two 16-bit counts a word (bins b and b + 1024),
    // filled by plain shared-memory atomics and added up afterwards. A warp-wide match (one add per distinct bin of a warp) cost three
    // fifths of the whole kernel; an atomic's worst case, a warp of equal scores, is 32 adds to one word, still a fraction of a match,
    // and the copies (a word apart in the banks) keep the warps off each other's words. Longer rows keep the matching count.
    constexpr int kAhead = 8;
    constexpr uint32_t kCopies = 16, kCopyWords = kBins / 2 + 1;
    static_assert(kCopies * kCopyWords <= 2 * kBandCap + kKeepCap, "the private histograms fit the lists' area, idle during the first read");
    if (groups <= (size_t(1) << 20) - 1024) {
        uint32_t* copies = band_key;   // (band_key, band_index and chosen lie one behind the other)
        for (uint32_t i = t; i < kCopies * kCopyWords; i += kThreads) copies[i] = 0;
        __syncthreads();
        uint32_t* my_copy = copies + (t / 64) * kCopyWords;
        for (size_t base = 0; base < groups; base += size_t(kThreads) * kAhead) {
            uint32_t keys[kAhead];
            #pragma unroll
            for (int i = 0; i < kAhead; ++i) {
                const size_t g = base + size_t(i) * kThreads + t;
                keys[i] = g < groups ? sortable(row[g]) : kDead;
            }
            #pragma unroll
            for (int i = 0; i < kAhead; ++i)
                if (keys[i] > kDead) atomicAdd(&my_copy[(keys[i] >> 21) & 1023u], keys[i] >> 31 ? 65536u : 1u);
        }
        __syncthreads();
        for (uint32_t bin = t; bin < kBins; bin += kThreads) {
            uint32_t sum = 0;
            #pragma unroll
            for (uint32_t c = 0; c < kCopies; ++c) sum += (copies[c * kCopyWords + (bin & 1023u)] >> (bin >> 10 ? 16 : 0)) & 0xffffu;
            hist[bin] = sum;
        }
    } else {
        for (size_t base = 0; base < groups; base += kThreads) {
            const size_t g = base + t;
            const uint32_t key = g < groups ? sortable(row[g]) : kDead;
            count_in(hist, key >> 21, key > kDead);
        }
    }
    __syncthreads();
    const uint32_t wanted = uint32_t(min(k, size_t(0xffffffffu)));
    find_band(hist, kBins, wanted, sh);
    const bool keep_all_live = sh.found_bin == kBins;          // fewer live scores than k: every one of them is kept
    uint32_t prefix = keep_all_live ? 0u : sh.found_bin << 21;  // the k-th key's bits so far
    uint32_t above = keep_all_live ? 0u : sh.found_above;       // scores above the band
    const uint32_t band_count = keep_all_live ? 0u : sh.found_count;
    const bool in_shared = !keep_all_live && band_count <= kBandCap && k <= kKeepCap;
    __syncthreads();

    uint32_t threshold = kDead, need = 0;   // kept: key > threshold, and the first `need` (by index) of key == threshold
    if (in_shared) {
        // ---- read 2: the sure indices and the band, both in index order ----
        uint32_t sure_count = 0, band_seen = 0;
        // (the next iteration's scores are asked for before this iteration's scan: the scan's two barriers then cover the load)
        float ahead[kPerThread];
        #pragma unroll
        for (int i = 0; i < kPerThread; ++i) { const size_t g = size_t(t) * kPerThread + i; ahead[i] = g < groups ? row[g] : -INFINITY; }
        for (size_t base = 0; base < groups; base += size_t(kThreads) * kPerThread) {
            const size_t first = base + size_t(t) * kPerThread;
            uint32_t keys[kPerThread], packed = 0;
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) keys[i] = first + i < groups ? sortable(ahead[i]) : kDead;
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) { const size_t g = first + size_t(kThreads) * kPerThread + i; ahead[i] = g < groups ? row[g] : -INFINITY; }
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) {
                const uint32_t top = keys[i] >> 21;
                packed += keys[i] > kDead ? (top > (prefix >> 21) ? 1u : top == (prefix >> 21) ? 0x10000u : 0u) : 0u;
            }
            uint32_t tile_total;
            const uint32_t before = prefix_before(packed, sh, tile_total);   // (two counts in one scan: neither passes 16 bits)
            uint32_t sure_at = sure_count + (before & 0xffffu), band_at = band_seen + (before >> 16);
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) {
                if (keys[i] <= kDead) continue;
                const uint32_t top = keys[i] >> 21;
                if (top > (prefix >> 21)) sure[sure_at++] = uint32_t(first + i);
                else if (top == (prefix >> 21)) { band_key[band_at] = keys[i]; band_index[band_at] = uint32_t(first + i); ++band_at; }
            }
            sure_count += tile_total & 0xffffu;
            band_seen += tile_total >> 16;
        }
        __syncthreads();
        // ---- the band's remaining 21 bits, in shared memory ----
        for (int round = 0; round < 2; ++round) {
            const int shift = round == 0 ? 10 : 0;
            const uint32_t bins = round == 0 ? 2048u : 1024u, decided = round == 0 ? 21u : 10u;
            for (uint32_t i = t; i < bins; i += kThreads) hist[i] = 0;
            __syncthreads();
            for (uint32_t base = 0; base < band_count; base += kThreads) {
                const uint32_t key = base + t < band_count ? band_key[base + t] : 0u;
                count_in(hist, (key >> shift) & (bins - 1), base + t < band_count && (key >> decided) == (prefix >> decided));
            }
            __syncthreads();
            find_band(hist, bins, wanted - above, sh);
            prefix |= sh.found_bin << shift;
            above += sh.found_above;
            __syncthreads();
        }
        threshold = prefix;
        need = wanted - above;
        // ---- the band's kept entries, in index order ----
        uint32_t chosen_count = 0, ties_seen = 0;
        for (uint32_t base = 0; base < band_count; base += kThreads * kPerThread) {
            const uint32_t first = base + t * kPerThread;
            uint32_t keys[kPerThread], ties = 0;
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) {
                keys[i] = first + i < band_count ? band_key[first + i] : kDead;
                ties += keys[i] == threshold;
            }
            uint32_t tile_ties;
            uint32_t tie_rank = ties_seen + prefix_before(ties, sh, tile_ties);
            uint32_t kept = 0;
            bool keep[kPerThread];
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) {
                keep[i] = keys[i] > threshold || (keys[i] == threshold && tie_rank < need);
                tie_rank += keys[i] == threshold;
                kept += keep[i];
            }
            uint32_t tile_kept;
            uint32_t at = chosen_count + prefix_before(kept, sh, tile_kept);
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i)
                if (keep[i]) chosen[at++] = band_index[first + i];
            chosen_count += tile_kept;
            ties_seen += tile_ties;
        }
        __syncthreads();
        // ---- two ascending lists into one: an entry's place is its own rank plus the other list's entries before it ----
        auto before_in = [](const uint32_t* list, uint32_t count, uint32_t index) {
            uint32_t low = 0, high = count;
            while (low < high) { const uint32_t mid = (low + high) / 2; if (list[mid] < index) low = mid + 1; else high = mid; }
            return low;
        };
        for (uint32_t i = t; i < sure_count; i += kThreads) mine[i + before_in(chosen, chosen_count, sure[i])] = group_of(sure[i]);
        for (uint32_t i = t; i < chosen_count; i += kThreads) mine[i + before_in(sure, sure_count, chosen[i])] = group_of(chosen[i]);
        for (size_t i = size_t(sure_count) + chosen_count + t; i < k; i += kThreads) mine[i] = -1;
        return;
    }

    // ---- the general path: refinements over the row itself, then one ordered pass ----
    if (!keep_all_live) {
        for (int round = 0; round < 2; ++round) {
            const int shift = round == 0 ? 10 : 0;
            const uint32_t bins = round == 0 ? 2048u : 1024u, decided = round == 0 ? 21u : 10u;
            for (uint32_t i = t; i < bins; i += kThreads) hist[i] = 0;
            __syncthreads();
            for (size_t base = 0; base < groups; base += kThreads) {
                const size_t g = base + t;
                const uint32_t key = g < groups ? sortable(row[g]) : kDead;
                count_in(hist, (key >> shift) & (bins - 1), key > kDead && (key >> decided) == (prefix >> decided));
            }
            __syncthreads();
            find_band(hist, bins, wanted - above, sh);
            prefix |= sh.found_bin << shift;
            above += sh.found_above;
            __syncthreads();
        }
        threshold = prefix;
        need = wanted - above;
    }
    size_t written = 0;
    uint32_t ties_seen = 0;
    for (size_t base = 0; base < groups; base += size_t(kThreads) * kPerThread) {
        const size_t first = base + size_t(t) * kPerThread;
        uint32_t keys[kPerThread], ties = 0;
        #pragma unroll
        for (int i = 0; i < kPerThread; ++i) {
            keys[i] = first + i < groups ? sortable(row[first + i]) : kDead;
            ties += !keep_all_live && keys[i] == threshold;
        }
        uint32_t tile_ties = 0, tie_rank = 0;
        if (!keep_all_live) tie_rank = ties_seen + prefix_before(ties, sh, tile_ties);
        uint32_t kept = 0;
        bool keep[kPerThread];
        #pragma unroll
        for (int i = 0; i < kPerThread; ++i) {
            const bool tie = !keep_all_live && keys[i] == threshold;
            keep[i] = keys[i] > kDead && (keep_all_live || keys[i] > threshold || (tie && tie_rank < need));
            tie_rank += tie;
            kept += keep[i];
        }
        uint32_t tile_kept;
        size_t at = written + prefix_before(kept, sh, tile_kept);
        #pragma unroll
        for (int i = 0; i < kPerThread; ++i)
            if (keep[i] && at < k) mine[at++] = group_of(uint32_t(first + i));
        written += tile_kept;
        ties_seen += tile_ties;
    }
    for (size_t i = written + t; i < k; i += kThreads) mine[i] = -1;
}

}  // namespace topk

// rows x groups scores -> rows x k indices (with candidates: see top_k_kernel)
void launch_top_k(Device& d, const float* scores, size_t rows, size_t groups, size_t k, int32_t* out, const int32_t* candidates, size_t blocks, size_t block) {
    static bool configured[64] = {};
    if (!configured[d.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(topk::top_k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(topk::kSmem)));
        configured[d.ordinal & 63] = true;
    }
    topk::top_k_kernel<<<unsigned(rows), topk::kThreads, topk::kSmem, d.stream>>>(scores, groups, k, out, candidates, blocks, block);
    ++d.launches;
    SDB_CHECK(cudaGetLastError());
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
    launch_top_k(value, scores, size_t(rows), size_t(groups), size_t(k), out, nullptr, 0, 1);
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
