// sd_op_top_k and sd_op_to_bf16: the index-list producer's contract and the BF16 rounding op.
//
// Top-k contract (gpu/straydog_gpu.h:409; rule: gpu/ops.hpp:1741-1742, crates/straydog-engine/tests/fused_gpu.rs:325-357): per
// row the k highest scores' indices in ascending index order; scores equal to the k-th keep the lowest indices; -inf is never
// kept; -0 ties +0; unused slots hold -1. All integer work, bit-exact.
//
// Kernel: blocks of 1024 threads, built around reading the row from memory twice. A row belongs to a thread-block cluster of 1, 2, 4
// or 8 blocks (as many as keep rows x blocks within the SM count, each block at least 8192 scores): block r takes the r-th
// contiguous slice of the row, every histogram is the sum of the blocks' histograms read through distributed shared memory, and
// block r writes its kept indices behind those of the blocks before it, so the list still ascends.
//   read 1   a 2048-bin histogram of the top 11 bits of every live score's sortable key (sixteen private histograms filled by
//            plain shared-memory atomics and added up). The bin in which the running count from the top reaches k is the
//            band: everything above it is kept for sure, everything below is dropped.
//   read 2   in index order: the sure indices go to one shared list, the band's (key, index) pairs to another.
//   then, in shared memory only: the band's next 11 and last 10 key bits are histogrammed the same way, which gives the k-th
//            key itself and how many of its equals are wanted; the band's chosen entries are compacted in index order; the
//            two ascending lists are merged by rank (each entry's place = its own rank + a binary search in the other list).
// A row whose band (or k) does not fit the shared lists - more than 8192 scores sharing their top 11 bits with the k-th, k over
// 4096 - takes the general path in the cluster's first block alone: the two refinements read the row again, then one ordered pass
// compacts straight to the output.
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

namespace sdb {
namespace topk {

constexpr int kThreads = 1024, kWarps = kThreads / 32, kPerThread = 8;
constexpr uint32_t kBins = 2048, kBandCap = 8192, kKeepCap = 4096;
constexpr size_t kSmem = (2 * kBins + kKeepCap + 2 * kBandCap + kKeepCap) * 4;   // two histograms | sure | band keys | band indices | chosen

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
    uint32_t kept;   // this block's share of the row's list
};

// The row's cluster. Both barrier halves are executed by every thread of every block of the cluster, the same number of times.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_blocks() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
// the word / the four words at this shared-memory address in block `rank` of the cluster
__device__ __forceinline__ uint32_t word_of(const uint32_t* local, uint32_t rank) {
    uint32_t remote, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ uint4 words_of(const uint32_t* local, uint32_t rank) {
    uint32_t remote;
    uint4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(remote) : "memory");
    return v;
}

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
// With `blocks` > 1 a bin's count is the sum over the cluster's blocks of their `hist` (every block finds the same band); the
// caller does not touch this `hist` again before the cluster's next barrier. The sums are made four bins a load (a load from
// another block's shared memory costs the same for 16 bytes as for 4): the threads' lower half adds the even blocks', the upper
// half the odd blocks' into `scratch` (2 x bins words of this block), and a thread's bins are the two halves' sum.
__device__ __forceinline__ void find_band(const uint32_t* hist, uint32_t bins, uint32_t wanted, Shared& sh, uint32_t blocks, uint32_t* scratch) {
    const uint32_t each = (bins + kThreads - 1) / kThreads;   // bins a thread, taken from the top
    uint32_t counts[2] = {0, 0}, sum = 0;
    if (blocks > 1) {
        cluster_arrive(); cluster_wait();                     // every block's histogram is complete
        const uint32_t half = threadIdx.x / (kThreads / 2), four = threadIdx.x % (kThreads / 2);
        if (four < bins / 4) {
            uint4 total = make_uint4(0, 0, 0, 0);
            for (uint32_t r = half; r < blocks; r += 2) {
                const uint4 theirs = words_of(&hist[4 * four], r);
                total.x += theirs.x; total.y += theirs.y; total.z += theirs.z; total.w += theirs.w;
            }
            *reinterpret_cast<uint4*>(&scratch[half * bins + 4 * four]) = total;
        }
        __syncthreads();
    }
    for (uint32_t i = 0; i < each; ++i) {
        const uint32_t at = threadIdx.x * each + i;
        if (at < bins) counts[i] = blocks == 1 ? hist[bins - 1 - at] : scratch[bins - 1 - at] + scratch[bins + bins - 1 - at];
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

// With `expand.packed` the kept indices are not written as they are: the rows are Qwen's block scores, and a row's list goes into its
// packed attention row as the reference's selection does (gpu/sparse_attention.hpp:172-243, 307-395): four positions a chosen block,
// then the positions of the row's incomplete block, then the count; a row with no more whole blocks than `keep` lists every position
// and takes no part in the choice.

// With `candidates` (a row's `blocks` block numbers in index order, -1 past the last; gpu/ops.hpp:1942-1951) the row's scores are
// those of its candidate groups in candidate order, and a kept place v is written as the group it stands for,
// candidates[v / block] * block + v % block: index order both ways, so the list still ascends.
__global__ void __launch_bounds__(kThreads) top_k_kernel(const float* __restrict__ scores, size_t groups, size_t k, int32_t* __restrict__ out,
                                                         const int32_t* __restrict__ candidates, size_t blocks, size_t block, const TopKExpand expand) {
    extern __shared__ __align__(16) uint32_t dynamic[];
    uint32_t* hist_a = dynamic;                 // the histograms of the first read and of the band's last bits
    uint32_t* hist_b = hist_a + kBins;          // the histogram between them: a block may still be reading the one before in another block
    uint32_t* sure = hist_b + kBins;            // indices kept for sure, ascending
    uint32_t* band_key = sure + kKeepCap;       // the band in index order
    uint32_t* band_index = band_key + kBandCap;
    uint32_t* chosen = band_index + kBandCap;   // the band's kept indices, ascending
    __shared__ Shared sh;
    const uint32_t ranks = cluster_blocks(), rank = cluster_rank();
    const size_t row_number = blockIdx.x / ranks;
    const float* row = scores + row_number * groups;
    int32_t* mine = out + row_number * k;
    const unsigned t = threadIdx.x;
    const int32_t* mapped = candidates ? candidates + row_number * blocks : nullptr;
    const auto group_of = [&](uint32_t place) { return mapped ? int32_t(size_t(mapped[place / block]) * block + place % block) : int32_t(place); };
    float* listed = nullptr;   // expand: the row's list in its packed row
    if (expand.packed) {
        const size_t position = expand.positions ? expand.positions[row_number] : expand.base + row_number, complete = (position + 1) / 4;
        listed = expand.packed + expand.index_start + row_number * expand.selected;
        float* count = expand.packed + expand.index_start + expand.steps * expand.selected + row_number;
        const size_t head = size_t(expand.keep) * 4;
        if (rank == 0) {
            if (complete <= expand.keep) {
                for (size_t i = threadIdx.x; i <= position; i += kThreads) listed[i] = float(i);
                if (threadIdx.x == 0) *count = float(position + 1);
            } else {
                for (size_t i = threadIdx.x; complete * 4 + i <= position; i += kThreads) listed[head + i] = float(complete * 4 + i);
                if (threadIdx.x == 0) *count = float(head + position + 1 - complete * 4);
            }
        }
        if (complete <= expand.keep) return;   // (the same for every block of the row's cluster, before its first barrier)
    }
    // place `at` of the row's list takes the group standing at `place`
    const auto put = [&](size_t at, uint32_t place) {
        if (!listed) { mine[at] = group_of(place); return; }
        const float first_position = float(size_t(place) * 4);
        float* four = listed + 4 * at;
        if (reinterpret_cast<uintptr_t>(four) % 16 == 0) *reinterpret_cast<float4*>(four) = make_float4(first_position, first_position + 1.0f, first_position + 2.0f, first_position + 3.0f);
        else { four[0] = first_position; four[1] = first_position + 1.0f; four[2] = first_position + 2.0f; four[3] = first_position + 3.0f; }
    };
    // this block's slice of the row
    const size_t slice = ((groups + ranks - 1) / ranks + 3) & ~size_t(3);
    const size_t low = min(groups, size_t(rank) * slice), high = min(groups, low + slice);

    // (launched as a programmatic dependent, this grid was placed while the kernel before it drained: that kernel's scores are complete
    //  behind the wait; the kernel after this one may be placed now and waits for this grid's end the same way. Plain launches: no-ops.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // ---- read 1: the top 11 key bits ----
    for (uint32_t i = t; i < kBins; i += kThreads) hist_a[i] = 0;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();
    // Slices of up to a million scores: sixteen private histograms (a pair of warps each), two 16-bit counts a word (bins b and b + 1024),
    // filled by plain shared-memory atomics and added up afterwards. A warp-wide match (one add per distinct bin of a warp) cost three
    // fifths of the whole kernel; an atomic's worst case, a warp of equal scores, is 32 adds to one word, still a fraction of a match,
    // and the copies (a word apart in the banks) keep the warps off each other's words. Longer slices keep the matching count.
    constexpr int kAhead = 16;
    constexpr uint32_t kCopies = 16, kCopyWords = kBins / 2 + 1;
    static_assert(kCopies * kCopyWords <= 2 * kBandCap + kKeepCap, "the private histograms fit the lists' area, idle during the first read");
    static_assert(2 * kBins <= kKeepCap, "find_band's two halves fit the chosen list's area");
    if (high - low <= (size_t(1) << 20) - 1024) {
        uint32_t* copies = band_key;   // (band_key, band_index and chosen lie one behind the other)
        static_assert(kCopies * kCopyWords % 4 == 0, "zeroed 16 bytes a store");
        for (uint32_t i = t; i < kCopies * kCopyWords / 4; i += kThreads) reinterpret_cast<uint4*>(copies)[i] = make_uint4(0, 0, 0, 0);
        __syncthreads();
        uint32_t* my_copy = copies + (t / 64) * kCopyWords;
        for (size_t base = low; base < high; base += size_t(kThreads) * kAhead) {
            uint32_t keys[kAhead];
            #pragma unroll
            for (int i = 0; i < kAhead; ++i) {
                const size_t g = base + size_t(i) * kThreads + t;
                keys[i] = g < high ? sortable(row[g]) : kDead;
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
            hist_a[bin] = sum;
        }
    } else {
        for (size_t base = low; base < high; base += kThreads) {
            const size_t g = base + t;
            const uint32_t key = g < high ? sortable(row[g]) : kDead;
            count_in(hist_a, key >> 21, key > kDead);
        }
    }
    __syncthreads();
    const uint32_t wanted = uint32_t(min(k, size_t(0xffffffffu)));
    find_band(hist_a, kBins, wanted, sh, ranks, chosen);   // (chosen: idle until the band's entries are picked)
    const bool keep_all_live = sh.found_bin == kBins;          // fewer live scores than k: every one of them is kept
    uint32_t prefix = keep_all_live ? 0u : sh.found_bin << 21;  // the k-th key's bits so far
    uint32_t above = keep_all_live ? 0u : sh.found_above;       // scores above the band
    const uint32_t band_count = keep_all_live ? 0u : sh.found_count;   // the band over the whole row
    const bool in_shared = !keep_all_live && band_count <= kBandCap && k <= kKeepCap;
    __syncthreads();

    uint32_t threshold = kDead, need = 0;   // kept: key > threshold, and the first `need` (by index) of key == threshold
    if (in_shared) {
        // ---- read 2: the slice's sure indices and its part of the band, both in index order ----
        uint32_t sure_count = 0, band_seen = 0;
        const uint32_t count = uint32_t(high - low), first_index = uint32_t(low);
        const float* part = row + low;
        // a key above band_top is kept for sure; the band's keys are band_low .. band_top (one unsigned compare of key - band_low)
        const uint32_t band_top = prefix | 0x1fffffu, band_low = max(prefix, kDead + 1), band_width = band_top - band_low;
        // (the next iteration's scores are asked for before this iteration's scan: the scan's two barriers then cover the load)
        float ahead[kPerThread];
        const bool whole = (reinterpret_cast<uintptr_t>(part) & 15) == 0;   // a thread's eight scores are two 16-byte loads
        const auto fetch = [&](uint32_t first, float* v) {
            if (whole && first + kPerThread <= count) {
                #pragma unroll
                for (int i = 0; i < kPerThread; i += 4) {
                    const float4 x = __ldg(reinterpret_cast<const float4*>(part + first + i));
                    v[i] = x.x; v[i + 1] = x.y; v[i + 2] = x.z; v[i + 3] = x.w;
                }
            } else {
                #pragma unroll
                for (int i = 0; i < kPerThread; ++i) v[i] = first + i < count ? part[first + i] : -INFINITY;   // (-inf: neither sure nor band)
            }
        };
        fetch(t * kPerThread, ahead);
        for (uint32_t base = 0; base < count; base += kThreads * kPerThread) {
            const uint32_t first = base + t * kPerThread;
            uint32_t keys[kPerThread], packed = 0;
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) keys[i] = sortable(ahead[i]);
            fetch(first + kThreads * kPerThread, ahead);
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) packed += (keys[i] > band_top ? 1u : 0u) + (keys[i] - band_low <= band_width ? 0x10000u : 0u);
            uint32_t tile_total;
            const uint32_t before = prefix_before(packed, sh, tile_total);   // (two counts in one scan: neither passes 16 bits)
            uint32_t sure_at = sure_count + (before & 0xffffu), band_at = band_seen + (before >> 16);
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) {
                if (keys[i] > band_top) sure[sure_at++] = first_index + first + i;
                else if (keys[i] - band_low <= band_width) { band_key[band_at] = keys[i]; band_index[band_at] = first_index + first + i; ++band_at; }
            }
            sure_count += tile_total & 0xffffu;
            band_seen += tile_total >> 16;
        }
        __syncthreads();
        // ---- the band's remaining 21 bits, in shared memory (band_seen: this block's part of the band) ----
        for (int round = 0; round < 2; ++round) {
            const int shift = round == 0 ? 10 : 0;
            const uint32_t bins = round == 0 ? 2048u : 1024u, decided = round == 0 ? 21u : 10u;
            uint32_t* hist = round == 0 ? hist_b : hist_a;   // (hist_a: every block has passed the barrier of the round before, so has read it)
            for (uint32_t i = t; i < bins; i += kThreads) hist[i] = 0;
            __syncthreads();
            for (uint32_t i = t; i < band_seen; i += kThreads) {   // (a band is a few thousand keys over 2048 bins: plain atomics)
                const uint32_t key = band_key[i];
                if ((key >> decided) == (prefix >> decided)) atomicAdd(&hist[(key >> shift) & (bins - 1)], 1u);
            }
            __syncthreads();
            find_band(hist, bins, wanted - above, sh, ranks, chosen);
            prefix |= sh.found_bin << shift;
            above += sh.found_above;
            __syncthreads();
        }
        threshold = prefix;
        need = wanted - above;
        // Of the `need` equals of the k-th key the blocks before this one take theirs first (hist_a holds every block's count of them).
        for (uint32_t r = 0; r < rank; ++r) {
            const uint32_t theirs = word_of(&hist_a[threshold & 1023u], r);
            need -= min(need, theirs);
        }
        // ---- the band's kept entries, in index order ----
        uint32_t chosen_count = 0, ties_seen = 0;
        for (uint32_t base = 0; base < band_seen; base += kThreads * kPerThread) {
            const uint32_t first = base + t * kPerThread;
            uint32_t keys[kPerThread], ties = 0;
            #pragma unroll
            for (int i = 0; i < kPerThread; ++i) {
                keys[i] = first + i < band_seen ? band_key[first + i] : kDead;
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
        // ---- where this block's entries start in the row's list: behind those of the blocks before it ----
        uint32_t start = 0, total = sure_count + chosen_count;
        if (ranks > 1) {
            if (t == 0) sh.kept = sure_count + chosen_count;
            cluster_arrive(); cluster_wait();
            total = 0;
            for (uint32_t r = 0; r < ranks; ++r) {
                const uint32_t theirs = word_of(&sh.kept, r);
                start += r < rank ? theirs : 0u;
                total += theirs;
            }
            cluster_arrive();   // (this block has read what it needs of the others; the wait is at the end)
        }
        // ---- two ascending lists into one: an entry's place is its own rank plus the other list's entries before it ----
        auto before_in = [](const uint32_t* list, uint32_t count, uint32_t index) {
            uint32_t low = 0, high = count;
            while (low < high) { const uint32_t mid = (low + high) / 2; if (list[mid] < index) low = mid + 1; else high = mid; }
            return low;
        };
        for (uint32_t i = t; i < sure_count; i += kThreads) put(start + i + before_in(chosen, chosen_count, sure[i]), sure[i]);
        for (uint32_t i = t; i < chosen_count; i += kThreads) put(start + i + before_in(sure, sure_count, chosen[i]), chosen[i]);
        if (!listed)
            for (size_t i = size_t(total) + rank * kThreads + t; i < k; i += size_t(ranks) * kThreads) mine[i] = -1;
        if (ranks > 1) cluster_wait();   // nobody leaves while its shared memory may still be read
        return;
    }

    // ---- the general path: the cluster's first block alone; refinements over the row itself, then one ordered pass ----
    if (rank != 0) {   // (the others meet the first block at the cluster's last barrier: it may still be reading their first histogram)
        cluster_arrive(); cluster_wait();
        return;
    }
    if (!keep_all_live) {
        for (int round = 0; round < 2; ++round) {
            const int shift = round == 0 ? 10 : 0;
            const uint32_t bins = round == 0 ? 2048u : 1024u, decided = round == 0 ? 21u : 10u;
            for (uint32_t i = t; i < bins; i += kThreads) hist_b[i] = 0;   // (hist_a may still be read by the other blocks)
            __syncthreads();
            for (size_t base = 0; base < groups; base += kThreads) {
                const size_t g = base + t;
                const uint32_t key = g < groups ? sortable(row[g]) : kDead;
                count_in(hist_b, (key >> shift) & (bins - 1), key > kDead && (key >> decided) == (prefix >> decided));
            }
            __syncthreads();
            find_band(hist_b, bins, wanted - above, sh, 1, nullptr);
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
            if (keep[i] && at < k) put(at++, uint32_t(first + i));
        written += tile_kept;
        ties_seen += tile_ties;
    }
    if (!listed)
        for (size_t i = written + t; i < k; i += kThreads) mine[i] = -1;
    if (ranks > 1) { cluster_arrive(); cluster_wait(); }
}

}  // namespace topk

// rows x groups scores -> rows x k indices (with candidates: see top_k_kernel)
// dependent: launched as a programmatic dependent of the kernel queued before it (which issues griddepcontrol.launch_dependents)
void launch_top_k(Device& d, const float* scores, size_t rows, size_t groups, size_t k, int32_t* out, const int32_t* candidates, size_t blocks, size_t block,
                  bool dependent, const TopKExpand* expand) {
    static bool configured[64] = {};
    if (!configured[d.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(topk::top_k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(topk::kSmem)));
        configured[d.ordinal & 63] = true;
    }
    // A row's cluster: as many blocks (1, 2, 4, 8) as keep the launch within one block per SM and a block's slice at 8192 scores or more
    // (the cluster's five barriers cost a shorter slice more than the split saves it).
    unsigned ranks = 1;
    while (ranks < 8 && rows * ranks * 2 <= size_t(d.sms) && groups / (ranks * 2) >= 8192) ranks *= 2;
    cudaLaunchConfig_t config{};
    config.blockDim = dim3{unsigned(topk::kThreads), 1, 1};
    config.dynamicSmemBytes = topk::kSmem;
    config.stream = d.stream;
    cudaLaunchAttribute attributes[2] = {};
    cudaLaunchAttribute& cluster = attributes[0];
    cluster.id = cudaLaunchAttributeClusterDimension;
    cluster.val.clusterDim.y = 1; cluster.val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes; config.numAttrs = dependent ? 2 : 1;
    // A cluster of this size must fit the device (a 1024-thread block with all its shared memory per SM, the cluster's SMs in one
    // GPC): asked of the driver once per device and size; a size that does not fit is halved.
    static int fits[64][4] = {};   // [device][log2 size]: 0 unknown, 1 fits, -1 does not
    for (;; ranks /= 2) {
        config.gridDim = dim3{unsigned(rows * ranks), 1, 1};
        cluster.val.clusterDim.x = ranks;
        if (ranks == 1) break;
        int& known = fits[d.ordinal & 63][ranks >= 8 ? 3 : ranks >= 4 ? 2 : 1];
        if (!known) {
            int clusters = 0;
            const cudaError_t asked = cudaOccupancyMaxActiveClusters(&clusters, topk::top_k_kernel, &config);
            if (asked != cudaSuccess) cudaGetLastError();
            known = asked == cudaSuccess && clusters > 0 ? 1 : -1;
        }
        if (known > 0) break;
    }
    SDB_CHECK(cudaLaunchKernelEx(&config, topk::top_k_kernel, scores, groups, k, out, candidates, blocks, block, expand ? *expand : TopKExpand{}));
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
    launch_top_k(value, scores, size_t(rows), size_t(groups), size_t(k), out, nullptr, 0, 1, false, nullptr);
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
