// Handles, allocations and transfers of the C ABI: the subset of the reference's memory entries the
// attention path's callers use (gpu/straydog_gpu.h:17,33-34,42-67,113-114,157-159;
// gpu/kernels.cpp:3511-3611, 3646-3712, 3771, 4364-4386, 4555-4593). Same conventions: a negative
// result or a null pointer is a failure that sd_error() describes for the calling thread; the
// library owns every allocation and each op checks that its pointers lie inside one of them.
#include "common.cuh"

#include <cstring>
#include "../../include/straydog_gpu_b200.h"

namespace sdb {

thread_local std::string last_error;

Device& device(void* handle) {
    if (!handle) throw std::runtime_error("null Straydog device handle");
    auto& value = *static_cast<Device*>(handle);
    SDB_CHECK(cudaSetDevice(value.ordinal));
    return value;
}

static std::string budget_exceeded(const Device& d, uint64_t bytes) {
    return "Straydog VRAM budget exceeded: " + std::to_string(bytes) + " bytes requested, " + std::to_string(d.used) + " of " +
           std::to_string(d.budget) + " in use";
}

void* raw_allocate(Device& d, size_t bytes, bool zero) {
    std::lock_guard<std::mutex> lock(d.mutex);
    const uint64_t available = d.budget > d.used ? d.budget - d.used : 0;
    if (!bytes || bytes > available || allocation_tail > available - bytes) throw std::runtime_error(budget_exceeded(d, bytes));
    void* pointer = nullptr;
    SDB_CHECK(cudaMalloc(&pointer, bytes + allocation_tail));
    d.allocations.emplace(static_cast<const uint8_t*>(pointer), bytes);
    d.used += bytes + allocation_tail;
    if (zero) {
        SDB_CHECK(cudaMemsetAsync(pointer, 0, bytes + allocation_tail, d.stream));
        SDB_CHECK(cudaStreamSynchronize(d.stream));
    }
    return pointer;
}

void raw_release(Device& d, void* pointer) {
    std::lock_guard<std::mutex> lock(d.mutex);
    auto found = d.allocations.find(static_cast<const uint8_t*>(pointer));
    if (found == d.allocations.end()) throw std::runtime_error("unknown Straydog allocation");
    SDB_CHECK(cudaStreamSynchronize(d.stream));
    auto host = d.host_states.find(found->first);
    if (host != d.host_states.end()) {   // a host-resident state: page-locked host memory, outside the VRAM budget
        SDB_CHECK(cudaFreeHost(host->second));
        d.host_states.erase(host);
        d.allocations.erase(found);
        return;
    }
    SDB_CHECK(cudaFree(pointer));
    d.used -= found->second + allocation_tail;
    d.allocations.erase(found);
}

// The range [pointer, pointer + bytes) lies inside one allocation of this device (gpu/ops.hpp:8-26).
void span(Device& d, const void* pointer, size_t bytes, const char* what) {
    if (d.adopted) {   // the adopting library has checked its own pointers (gpu/ops.hpp:8-26 runs before any kernel of its ops)
        if (!pointer) throw std::runtime_error(std::string("Straydog op: ") + what + " is null");
        return;
    }
    const auto* at = static_cast<const uint8_t*>(pointer);
    std::lock_guard<std::mutex> lock(d.mutex);
    auto next = d.allocations.upper_bound(at);
    if (next != d.allocations.begin()) {
        --next;
        if (bytes <= next->second && size_t(at - next->first) <= next->second - bytes) return;
    }
    throw std::runtime_error(std::string("Straydog op: ") + what + " is outside this device's allocations");
}

void span_or_peer(Device& d, const void* pointer, size_t bytes, const char* what) {
    const auto* at = static_cast<const uint8_t*>(pointer);
    {
        std::lock_guard<std::mutex> lock(d.mutex);
        auto next = d.peers.upper_bound(at);
        if (next != d.peers.begin()) {
            --next;
            if (bytes <= next->second && size_t(at - next->first) <= next->second - bytes) return;
        }
    }
    span(d, pointer, bytes, what);
}

size_t allocation_bytes(Device& d, const void* base) {
    std::lock_guard<std::mutex> lock(d.mutex);
    auto found = d.allocations.find(static_cast<const uint8_t*>(base));
    return found == d.allocations.end() ? 0 : found->second;
}

// Library-owned workspaces (not in the allocation map: callers never see them), grown on demand.
void* ensure(Device& d, void*& slot, size_t& have, size_t bytes, bool pinned_host) {
    if (have >= bytes && slot) return slot;
    SDB_CHECK(cudaStreamSynchronize(d.stream));
    if (slot) { if (pinned_host) SDB_CHECK(cudaFreeHost(slot)); else SDB_CHECK(cudaFree(slot)); slot = nullptr; have = 0; }
    const size_t grown = bytes + bytes / 4 + 4096;
    if (pinned_host) SDB_CHECK(cudaMallocHost(&slot, grown)); else SDB_CHECK(cudaMalloc(&slot, grown));
    have = grown;
    return slot;
}

cudaStream_t side_stream_begin(Device& d) {
    if (!d.side) {
        SDB_CHECK(cudaStreamCreateWithFlags(&d.side, cudaStreamNonBlocking));
        SDB_CHECK(cudaEventCreateWithFlags(&d.side_fork, cudaEventDisableTiming));
        SDB_CHECK(cudaEventCreateWithFlags(&d.side_join, cudaEventDisableTiming));
    }
    SDB_CHECK(cudaEventRecord(d.side_fork, d.stream));
    SDB_CHECK(cudaStreamWaitEvent(d.side, d.side_fork, 0));
    return d.side;
}

void side_stream_end(Device& d) {
    SDB_CHECK(cudaEventRecord(d.side_join, d.side));
    SDB_CHECK(cudaStreamWaitEvent(d.stream, d.side_join, 0));
}

static void copy_in(Device& d, void* target, const void* data, size_t bytes) {
    SDB_CHECK(cudaMemcpyAsync(target, data, bytes, cudaMemcpyDefault, d.stream));   // (the target may be a host-resident state)
}

}  // namespace sdb

using namespace sdb;

extern "C" {

const char* sd_error(void) { return last_error.c_str(); }

int sd_device_count(void) {
    int count = 0;
    const cudaError_t error = cudaGetDeviceCount(&count);
    if (error != cudaSuccess) { last_error = cudaGetErrorString(error); cudaGetLastError(); return -1; }
    return count;
}

void* sd_create(int ordinal, uint64_t budget) {
    try {
        int count = 0;
        SDB_CHECK(cudaGetDeviceCount(&count));
        if (ordinal < 0 || ordinal >= count) throw std::runtime_error("unknown Straydog device ordinal");
        auto value = std::make_unique<Device>(ordinal);
        SDB_CHECK(cudaSetDevice(ordinal));
        cudaDeviceProp prop{};
        SDB_CHECK(cudaGetDeviceProperties(&prop, ordinal));
        // This library holds sm_100a code only: refuse any other device instead of failing at the first launch.
        if (prop.major != 10)
            throw std::runtime_error(std::string("this Straydog build holds code for B200-class GPUs (sm_100a) only, not for ") + prop.name);
        value->sms = prop.multiProcessorCount;
        size_t available = 0, total = 0;
        SDB_CHECK(cudaMemGetInfo(&available, &total));
        if (budget < (1u << 20) || budget > available) throw std::runtime_error("Straydog VRAM budget is unavailable");
        value->budget = budget;
        SDB_CHECK(cudaStreamCreateWithFlags(&value->stream, cudaStreamNonBlocking));
        return value.release();
    } catch (const std::exception& e) { last_error = e.what(); return nullptr; }
}

// A handle over another library's device state: its stream (work is queued there, in order with that library's own kernels) and
// its allocations (pointers are taken as that library checked them). For the reference's own build when it calls this library's
// kernels from inside its spans (include/qsa_b200.hpp). Owns only this library's workspaces; sd_destroy frees those.
void* sdx_adopt(int ordinal, void* stream) {
    try {
        int count = 0;
        SDB_CHECK(cudaGetDeviceCount(&count));
        if (ordinal < 0 || ordinal >= count) throw std::runtime_error("unknown Straydog device ordinal");
        auto value = std::make_unique<Device>(ordinal);
        SDB_CHECK(cudaSetDevice(ordinal));
        cudaDeviceProp prop{};
        SDB_CHECK(cudaGetDeviceProperties(&prop, ordinal));
        if (prop.major != 10)
            throw std::runtime_error(std::string("this Straydog build holds code for B200-class GPUs (sm_100a) only, not for ") + prop.name);
        value->sms = prop.multiProcessorCount;
        value->stream = static_cast<cudaStream_t>(stream);
        value->adopted = true;
        return value.release();
    } catch (const std::exception& e) { last_error = e.what(); return nullptr; }
}

void sd_destroy(void* handle) {
    if (!handle) return;
    auto* value = static_cast<Device*>(handle);
    if (cudaSetDevice(value->ordinal) == cudaSuccess) {
        cudaStreamSynchronize(value->stream);
        for (auto& entry : value->peers) cudaIpcCloseMemHandle(const_cast<uint8_t*>(entry.first));
        for (auto& entry : value->allocations) {
            auto host = value->host_states.find(entry.first);
            if (host != value->host_states.end()) cudaFreeHost(host->second);
            else cudaFree(const_cast<uint8_t*>(entry.first));
        }
        if (value->pinned) cudaFreeHost(value->pinned);
        for (void* p : {value->work, value->partial, value->tables, value->unions, static_cast<void*>(value->turns), static_cast<void*>(value->rope_rows)}) if (p) cudaFree(p);
        if (value->side) { cudaStreamDestroy(value->side); cudaEventDestroy(value->side_fork); cudaEventDestroy(value->side_join); }
        if (!value->adopted) cudaStreamDestroy(value->stream);
        cudaGetLastError();
    }
    delete value;
}

int sd_memory(void* handle, uint64_t* used, uint64_t* budget) {
    try {
        auto& value = device(handle);
        if (used) *used = value.used;
        if (budget) *budget = value.budget;
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

void* sd_allocate(void* handle, uint64_t bytes) {
    try { return raw_allocate(device(handle), bytes, false); }
    catch (const std::exception& e) { last_error = e.what(); return nullptr; }
}

void* sd_upload(void* handle, const void* data, uint64_t bytes) {
    try {
        auto& value = device(handle);
        if (!data) throw std::runtime_error("invalid Straydog upload");
        void* pointer = raw_allocate(value, bytes, false);
        copy_in(value, pointer, data, bytes);
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        return pointer;
    } catch (const std::exception& e) { last_error = e.what(); return nullptr; }
}

int sd_write(void* handle, void* pointer, const void* data, uint64_t bytes) {
    try {
        auto& value = device(handle);
        if (!data || !bytes || allocation_bytes(value, pointer) != bytes) throw std::runtime_error("invalid Straydog write");
        copy_in(value, pointer, data, bytes);
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

int sd_release(void* handle, void* pointer) {
    try {
        auto& value = device(handle);
        if (pointer == value.kv_stage) { value.kv_stage = nullptr; value.kv_stage_rows = 0; }
        raw_release(value, pointer);
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

int sd_allocation_bytes(void* handle, const void* pointer, uint64_t* bytes) {
    try {
        auto& value = device(handle);
        const size_t requested = allocation_bytes(value, pointer);
        if (!bytes || !requested) throw std::runtime_error("unknown Straydog allocation");
        *bytes = requested + allocation_tail;
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

int sd_zero(void* handle, void* pointer) {
    try {
        auto& value = device(handle);
        const size_t requested = allocation_bytes(value, pointer);
        if (!requested) throw std::runtime_error("unknown Straydog state allocation");
        SDB_CHECK(cudaMemsetAsync(pointer, 0, requested, value.stream));
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

int sd_download(void* handle, void* pointer, void* output, uint64_t bytes) {
    try {
        auto& value = device(handle);
        if (!output || !bytes || allocation_bytes(value, pointer) != bytes)
            throw std::runtime_error("Straydog state readback size mismatch");
        SDB_CHECK(cudaMemcpyAsync(output, pointer, bytes, cudaMemcpyDefault, value.stream));
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

void* sd_buffer(void* handle, uint64_t bytes) {
    try { return raw_allocate(device(handle), bytes, true); }
    catch (const std::exception& e) { last_error = e.what(); return nullptr; }
}

int sd_buffer_write(void* handle, void* buffer, uint64_t offset, const void* data, uint64_t bytes) {
    try {
        auto& value = device(handle);
        if (!data || offset > UINT64_MAX - bytes) throw std::runtime_error("invalid Straydog buffer write");
        span(value, static_cast<uint8_t*>(buffer) + offset, bytes, "a written buffer");
        copy_in(value, static_cast<uint8_t*>(buffer) + offset, data, bytes);
        // (the caller's memory may be pageable and reused at once: the copy is finished before returning)
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

int sd_buffer_read(void* handle, const void* buffer, uint64_t offset, void* output, uint64_t bytes) {
    try {
        auto& value = device(handle);
        if (!output || offset > UINT64_MAX - bytes) throw std::runtime_error("invalid Straydog buffer read");
        span(value, static_cast<const uint8_t*>(buffer) + offset, bytes, "a read buffer");
        SDB_CHECK(cudaMemcpyAsync(output, static_cast<const uint8_t*>(buffer) + offset, bytes, cudaMemcpyDefault, value.stream));
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

// gpu/kernels.cpp:4266-4275: 512 (FP16 rows) or 272 (Q8_0 rows). The codec, the fused fronts and the FP32 check path
// (sd_attention_sequence) handle both, and so does the selection-list attention of the decode seam (sdx_qsa_attention_rows, _gathered);
// the dense batch decode and the prompt kernel stream Q8_0 rows only and refuse FP16 rows at the call.
int sd_kv_format(void* handle, uint32_t row) {
    try {
        auto& value = device(handle);
        if (row != kv_row_f16 && row != kv_row_q8) throw std::runtime_error("invalid Straydog K/V format");
        value.kv_row = row;
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

// gpu/kernels.cpp:4277-4290: registers the VRAM stage of host-resident K/V. With every K/V plane in
// HBM (180 GB) there is nothing to stage: the registration is validated and kept, and the decode
// view stays {state, context} (gpu/kv_stage.hpp:105-109, mirror = none).
int sd_kv_stage(void* handle, void* pointer, uint64_t rows) {
    try {
        auto& value = device(handle);
        if (!rows || rows > (uint64_t(1) << 22) || allocation_bytes(value, pointer) != size_t(rows) * 1024 * 4)
            throw std::runtime_error("invalid Straydog K/V stage");
        value.kv_stage = pointer;
        value.kv_stage_rows = rows;
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

// gpu/kernels.cpp:3876-3902: a zeroed state in page-locked host memory the GPU reads in place (a K/V that does not fit the VRAM budget);
// the pointer returned is the device's view of it, an allocation of the handle like any other (sd_release frees it).
void* sd_host_state(void* handle, uint64_t bytes) {
    try {
        auto& value = device(handle);
        if (!bytes) throw std::runtime_error("invalid Straydog host state");
        void* host = nullptr;
        SDB_CHECK(cudaHostAlloc(&host, size_t(bytes) + allocation_tail, cudaHostAllocMapped));
        void* pointer = nullptr;
        try {
            std::memset(host, 0, size_t(bytes) + allocation_tail);
            SDB_CHECK(cudaHostGetDevicePointer(&pointer, host, 0));
            std::lock_guard<std::mutex> lock(value.mutex);
            value.host_states.emplace(static_cast<const uint8_t*>(pointer), host);
            value.allocations.emplace(static_cast<const uint8_t*>(pointer), size_t(bytes));
        } catch (...) { cudaFreeHost(host); throw; }
        return pointer;
    } catch (const std::exception& e) { last_error = e.what(); return nullptr; }
}

// gpu/kernels.cpp (sd_host_state_supported): whether the device reads mapped host memory (every B200 does: unified addressing)
int sd_host_state_supported(void* handle) {
    try {
        auto& value = device(handle);
        int can = 0;
        SDB_CHECK(cudaDeviceGetAttribute(&can, cudaDevAttrCanMapHostMemory, value.ordinal));
        return can ? 1 : 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

int sdx_synchronize(void* handle) {
    try {
        auto& value = device(handle);
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

void* sdx_stream(void* handle) {
    try { return device(handle).stream; }
    catch (const std::exception& e) { last_error = e.what(); return nullptr; }
}

void* sdx_event_create(void) {
    cudaEvent_t event = nullptr;
    const cudaError_t error = cudaEventCreate(&event);
    if (error != cudaSuccess) { last_error = cudaGetErrorString(error); return nullptr; }
    return event;
}

int sdx_event_record(void* handle, void* event) {
    try {
        auto& value = device(handle);
        SDB_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(event), value.stream));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

int sdx_event_elapsed_ms(void* before, void* after, float* ms) {
    try {
        SDB_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(after)));
        SDB_CHECK(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(before), static_cast<cudaEvent_t>(after)));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

void sdx_event_destroy(void* event) { if (event) cudaEventDestroy(static_cast<cudaEvent_t>(event)); }

uint64_t sdx_launch_count(void* handle) {
    try { return device(handle).launches; }
    catch (const std::exception& e) { last_error = e.what(); return 0; }
}


// ---- another process's allocation on another GPU of the node, for kernels that store to peers over NVLink ----
int sdx_ipc_export(void* handle, const void* pointer, void* out_handle) {
    SDB_OP_BEGIN
    {
        std::lock_guard<std::mutex> lock(value.mutex);
        if (!value.allocations.count(static_cast<const uint8_t*>(pointer))) throw std::runtime_error("unknown Straydog allocation");
    }
    if (!out_handle) throw std::runtime_error("no room for the handle");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the exported handle is 64 bytes");
    cudaIpcMemHandle_t exported;
    SDB_CHECK(cudaIpcGetMemHandle(&exported, const_cast<void*>(pointer)));
    std::memcpy(out_handle, &exported, sizeof exported);
    SDB_OP_END
}

void* sdx_ipc_open(void* handle, const void* in_handle, uint64_t bytes) {
    try {
        auto& value = device(handle);
        if (!in_handle || !bytes) throw std::runtime_error("no handle to open");
        cudaIpcMemHandle_t imported;
        std::memcpy(&imported, in_handle, sizeof imported);
        void* pointer = nullptr;
        SDB_CHECK(cudaIpcOpenMemHandle(&pointer, imported, cudaIpcMemLazyEnablePeerAccess));
        // the size the caller states must fit the range that was mapped: a kernel given this pointer stores into another GPU
        size_t mapped = 0;
        {
            using Range = int (*)(unsigned long long*, size_t*, unsigned long long);
            void* entry = nullptr;
            cudaDriverEntryPointQueryResult found;
            if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &entry, cudaEnableDefault, &found) == cudaSuccess && entry &&
                found == cudaDriverEntryPointSuccess) {
                unsigned long long base = 0;
                if (reinterpret_cast<Range>(entry)(&base, &mapped, reinterpret_cast<unsigned long long>(pointer)) != 0) mapped = 0;
                else mapped -= size_t(reinterpret_cast<unsigned long long>(pointer) - base);
            }
        }
        if (mapped && bytes > mapped) {   // (a driver that cannot answer leaves the stated size as it is)
            cudaIpcCloseMemHandle(pointer);
            throw std::runtime_error("the mapped peer allocation is smaller than the size stated for it");
        }
        std::lock_guard<std::mutex> lock(value.mutex);
        value.peers.emplace(static_cast<const uint8_t*>(pointer), size_t(bytes));
        return pointer;
    } catch (const std::exception& e) { last_error = e.what(); return nullptr; }
}

int sdx_ipc_close(void* handle, void* pointer) {
    SDB_OP_BEGIN
    {
        std::lock_guard<std::mutex> lock(value.mutex);
        auto found = value.peers.find(static_cast<const uint8_t*>(pointer));
        if (found == value.peers.end()) throw std::runtime_error("unknown peer mapping");
        value.peers.erase(found);
    }
    SDB_CHECK(cudaStreamSynchronize(value.stream));
    SDB_CHECK(cudaIpcCloseMemHandle(pointer));
    SDB_OP_END
}

}  // extern "C"
