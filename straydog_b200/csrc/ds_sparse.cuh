// Shared by the latent sparse attention kernels: the argument block, the key order of a row
// (window rows, then selected compressed rows: gpu/ops.hpp:1309-1316) and the BF16 pointer tag
// (bit 0 of the pointer marks BF16 rows: gpu/ops.hpp:1208-1222).
#pragma once
#include "common.cuh"

namespace sdb {

struct SparseArgs {
    const float* raw; size_t raw_rows;
    const int32_t* positions; size_t window;
    const float* compressed; size_t compressed_rows;   // may carry the BF16 tag
    const int32_t* selected; size_t selections;
    size_t heads, dim;
    float scale;
    size_t span_rows;   // rows of one span: a call may hold several spans, each with its own window ring (never 0; one span: all the rows)
};

// Head-sharded runs: every GPU of the node keeps the gathered outputs [world][rows][heads][dim] (rank-major), and a rank's
// kernel stores its own outputs into slot `rank` of every GPU's copy over NVLink (peer pointers), so that the all-gather
// is part of the attention kernel's merge instead of a collective behind it.
constexpr int kMaxGatherWorld = 8;
struct GatherTargets {
    float* out[kMaxGatherWorld];     // every rank's gathered buffer (this rank's own included)
    int* flags[kMaxGatherWorld];     // every rank's arrival counters [world]
    uint32_t world, rank;            // world == 0: no gather, plain `out`
    int32_t step;                    // value a rank's counter takes when its outputs of this call have been stored
    unsigned* arrivals;              // this GPU's count of the grid's finished CTAs (zero at rest: the last CTA wraps it)
};

__host__ __device__ inline bool state_is_bf16(const void* p) { return reinterpret_cast<uintptr_t>(p) & 1u; }
__host__ __device__ inline const uint16_t* state_halves(const void* p) {
    return reinterpret_cast<const uint16_t*>(reinterpret_cast<uintptr_t>(p) & ~uintptr_t(1));
}

#if defined(__CUDACC__)
struct KeyList { int64_t first; size_t raw_count, total; };

__device__ __forceinline__ KeyList key_list(const SparseArgs& a, size_t row) {
    const int64_t p = a.positions[row];
    const int64_t first = p - int64_t(a.window) + 1 < 0 ? 0 : p - int64_t(a.window) + 1;
    const size_t raw_count = size_t(p - first + 1);
    return KeyList{first, raw_count, raw_count + a.selections};
}
// Key `index` of a row: an F32 window row, a compressed row (tagged as `compressed` is), or null for an empty selection.
__device__ __forceinline__ const float* key_pointer(const SparseArgs& a, const KeyList& list, size_t row, size_t index) {
    if (index < list.raw_count) {
        const float* ring = a.raw + row / a.span_rows * a.raw_rows * a.dim;   // (a span's own ring)
        return ring + size_t(list.first + int64_t(index)) % a.raw_rows * a.dim;
    }
    if (index >= list.total) return nullptr;
    const int32_t at = a.selected[row * a.selections + (index - list.raw_count)];
    if (at < 0) return nullptr;
    if (state_is_bf16(a.compressed))
        return reinterpret_cast<const float*>(reinterpret_cast<uintptr_t>(state_halves(a.compressed) + size_t(at) * a.dim) | 1u);
    return a.compressed + size_t(at) * a.dim;
}
#endif

bool sparse_mma_supported(const SparseArgs& a);
bool sparse_tc_supported(const SparseArgs& a);
void sparse_tc_launch(Device& d, const SparseArgs& a, const float* q, const float* sinks, size_t rows, size_t pairs,
                      const double2* forward, const double2* inverse, float* out);
void sparse_tc2_launch(Device& d, const SparseArgs& a, const float* q, const float* sinks, size_t rows, size_t pairs,
                       const double2* forward, const double2* inverse, float* out);
void sparse_mma3_launch(Device& d, const SparseArgs& a, const float* q, const float* sinks, size_t rows, size_t pairs,
                        const double2* forward, const double2* inverse, float* out, const GatherTargets* gather = nullptr);

}  // namespace sdb
