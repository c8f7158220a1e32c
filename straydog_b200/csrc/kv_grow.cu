// A sequence's K/V and its indexer state grown to a longer context: the data movement of sd_kv_grow (gpu/kernels.cpp:4048-4203).
// The reference's entry finds the state in its decoder-layer registry and rewires the registry's plans afterwards; the registry is the
// engine's side of the call and is not part of this library, so this entry takes and returns the two pointers themselves.
//
// A state is 2 * kv_heads planes of `context` rows: a longer context moves every plane but the first. In VRAM the new state is a new
// allocation of the handle (zeroed), every plane's `from` positions copied on the device (all of them, not only the `valid` ones: a later
// read finds what it would have found in a state that had the whole context from the start), and the old one released. A host-resident
// state (sd_host_state) is grown in host memory, its `valid` positions copied by the CPU. The indexer's pooled blocks
// [128][from / 4 + 1] take their new pitch [128][to / 4 + 1] (the first min(old pitch, valid / 4 + 1) blocks of every column), the
// 16 x 128 history ring follows them; the index state is replaced by a new allocation only when the old one is too small.
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

#include <algorithm>

namespace sdb {
namespace {

constexpr size_t kRing = 16 * 128;   // gpu/sparse_attention.hpp:85: the history ring, floats

// `before`: the old index state (a copy). `after`: the new one, zeroed. A thread a float of the new layout that has a source.
__global__ void __launch_bounds__(256) index_repitch_kernel(const float* __restrict__ before, size_t old_pool, size_t pool, size_t keep,
                                                            float* __restrict__ after) {
    const size_t total = 128 * keep + kRing;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
        if (i < 128 * keep) after[(i / keep) * pool + i % keep] = before[(i / keep) * old_pool + i % keep];
        else after[128 * pool + (i - 128 * keep)] = before[128 * old_pool + (i - 128 * keep)];
    }
}

}  // namespace
}  // namespace sdb

using namespace sdb;

extern "C" int sdx_kv_grow(void* handle, uint64_t kv_heads, uint64_t from, uint64_t to, uint64_t valid, void** state, void** index_state) {
    SDB_OP_BEGIN
    if (!state || !index_state || !*state || !*index_state || !kv_heads || kv_heads > 65535 || !from || to <= from || to > 262144 || valid > from)
        throw std::runtime_error("invalid Straydog K/V growth");
    const size_t row = value.kv_row, planes = 2 * kv_heads, old_pool = from / 4 + 1, pool = to / 4 + 1;
    const size_t old_bytes = checked_product({from, planes, row}), new_bytes = checked_product({to, planes, row});
    const size_t old_index_bytes = (old_pool * 128 + kRing) * 4, new_index_bytes = (pool * 128 + kRing) * 4;
    void* old_state = *state;
    void* old_index = *index_state;
    const size_t index_have = allocation_bytes(value, old_index);
    bool on_host = false;
    void* old_host = nullptr;
    {
        std::lock_guard<std::mutex> lock(value.mutex);
        auto host = value.host_states.find(static_cast<const uint8_t*>(old_state));
        on_host = host != value.host_states.end();
        if (on_host) old_host = host->second;
    }
    const size_t state_have = allocation_bytes(value, old_state);
    if (!state_have || !index_have || (on_host ? state_have < old_bytes : state_have != old_bytes) || index_have < old_index_bytes)
        throw std::runtime_error("invalid Straydog K/V growth");
    SDB_CHECK(cudaStreamSynchronize(value.stream));
    // Everything that can fail for want of memory comes first: a growth that is refused leaves both states as they were.
    void* grown = nullptr;
    void* grown_index = nullptr;
    float* before = static_cast<float*>(ensure(value, value.work, value.work_bytes, old_index_bytes));   // the old index state's copy
    try {
        grown = on_host ? sd_host_state(handle, new_bytes) : raw_allocate(value, new_bytes, true);
        if (!grown) throw std::runtime_error(last_error);
        if (index_have < new_index_bytes) grown_index = raw_allocate(value, new_index_bytes, true);
    } catch (...) {
        if (grown) raw_release(value, grown);
        throw;
    }
    if (on_host) {
        void* grown_host = nullptr;
        {
            std::lock_guard<std::mutex> lock(value.mutex);
            grown_host = value.host_states.at(static_cast<const uint8_t*>(grown));
        }
        for (size_t plane = 0; plane < planes; ++plane)
            std::memcpy(static_cast<uint8_t*>(grown_host) + plane * to * row, static_cast<const uint8_t*>(old_host) + plane * from * row, valid * row);
    } else {
        SDB_CHECK(cudaMemcpy2DAsync(grown, to * row, old_state, from * row, from * row, planes, cudaMemcpyDeviceToDevice, value.stream));
    }
    // the indexer's blocks at their new pitch, then its ring
    float* after = static_cast<float*>(grown_index ? grown_index : old_index);
    SDB_CHECK(cudaMemcpyAsync(before, old_index, old_index_bytes, cudaMemcpyDeviceToDevice, value.stream));
    if (!grown_index) SDB_CHECK(cudaMemsetAsync(after, 0, new_index_bytes, value.stream));
    const size_t keep = std::min<size_t>(old_pool, valid / 4 + 1);
    index_repitch_kernel<<<unsigned(std::min<size_t>((128 * keep + kRing + 255) / 256, size_t(value.sms) * 8)), 256, 0, value.stream>>>(
        before, old_pool, pool, keep, after);
    ++value.launches;
    SDB_CHECK(cudaGetLastError());
    SDB_CHECK(cudaStreamSynchronize(value.stream));
    raw_release(value, old_state);
    if (grown_index) raw_release(value, old_index);
    *state = grown;
    *index_state = after;
    SDB_OP_END
}
