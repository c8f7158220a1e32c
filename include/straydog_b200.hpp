// C++ host side above the C ABI of straydog_gpu_b200.h: the mirror of the reference engine's Rust wrappers for the attention path
// (straydog_engine::gpu::Backend, crates/straydog-engine/src/gpu.rs:491-561,735; straydog_engine::ops::Ops,
// crates/straydog-engine/src/ops.rs:195-256,878-886,1021-1024,1141-1171,1241-1244): the same method names and argument meaning;
// where the Rust returns Err(String) with the library's message, these throw straydog::Error with the same message.
// Header only; link against libstraydog_gpu_b200.so.
#pragma once
#include "straydog_gpu_b200.h"

#include <cstdint>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace straydog {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// A device allocation of one Backend (ops.rs:170-193: pointer and size; freed by Backend::release or with the Backend).
struct Buffer {
    void* pointer = nullptr;
    uint64_t bytes = 0;
    template<class T = void> T* at(uint64_t byte_offset = 0) const { return reinterpret_cast<T*>(static_cast<uint8_t*>(pointer) + byte_offset); }
    // the BF16 tag of latent rows: bit 0 of the pointer (ops.hpp:1208-1222)
    const float* tagged_bf16() const { return reinterpret_cast<const float*>(reinterpret_cast<uintptr_t>(pointer) | 1u); }
};

class Backend {
  public:
    // gpu.rs Backend::new: a handle on device `ordinal` that may hold `budget` bytes.
    Backend(int ordinal, uint64_t budget) : handle_(sd_create(ordinal, budget)) {
        if (!handle_) throw Error(sd_error());
    }
    ~Backend() { sd_destroy(handle_); }
    Backend(const Backend&) = delete;
    Backend& operator=(const Backend&) = delete;
    Backend(Backend&& other) noexcept : handle_(std::exchange(other.handle_, nullptr)) {}

    static int device_count() { return check(sd_device_count()); }
    void* handle() const { return handle_; }

    // ---- ops.rs:195-256 ----
    Buffer buffer(uint64_t bytes) { return made(sd_buffer(handle_, bytes), bytes); }            // zeroed
    Buffer buffer_unset(uint64_t bytes) { return made(sd_allocate(handle_, bytes), bytes); }
    template<class T> Buffer upload(const std::vector<T>& values) { return made(sd_upload(handle_, values.data(), values.size() * sizeof(T)), values.size() * sizeof(T)); }
    void release(Buffer& b) { check(sd_release(handle_, b.pointer)); b = Buffer{}; }
    template<class T> void write_buffer(const Buffer& b, uint64_t offset_bytes, const std::vector<T>& values) {
        check(sd_buffer_write(handle_, b.pointer, offset_bytes, values.data(), values.size() * sizeof(T)));
    }
    // waits for the stream, then copies out.size() values from the buffer, `offset` values in
    template<class T> void read_buffer(const Buffer& b, size_t offset, std::vector<T>& out) {
        check(sd_buffer_read(handle_, b.pointer, offset * sizeof(T), out.data(), out.size() * sizeof(T)));
    }
    void synchronize() { check(sdx_synchronize(handle_)); }
    std::pair<uint64_t, uint64_t> memory() {   // (bytes in use, budget)
        uint64_t used = 0, budget = 0;
        check(sd_memory(handle_, &used, &budget));
        return {used, budget};
    }

    // ---- K/V format and the scalar check path (gpu.rs:491-523, 735) ----
    void kv_format(uint32_t row_bytes) { check(sd_kv_format(handle_, row_bytes)); }
    void attention_sequence(const Buffer& state, uint64_t context, uint64_t base, uint64_t steps, uint64_t selected,
                            const std::vector<float>& input, std::vector<float>& output) {
        check(sd_attention_sequence(handle_, state.pointer, context, base, steps, selected, input.data(), input.size(), output.data(), output.size()));
    }

    // ---- ops.rs:878-886: dense causal GQA over F32 K/V ----
    void attention(const float* q, const float* keys, const float* values, uint64_t context, const int32_t* positions, uint64_t rows,
                   uint64_t heads, uint64_t kv_heads, uint64_t dim, float scale, const float* gate, const Buffer& scratch, float* out) {
        check(sd_op_attention(handle_, q, keys, values, context, positions, rows, heads, kv_heads, dim, scale, gate,
                              static_cast<float*>(scratch.pointer), scratch.bytes, out));
    }

    // ---- ops.rs:1141-1171: latent sparse attention ----
    void attention_turns_reserve(uint64_t rows, uint64_t rope_dims) { check(sd_attention_turns_reserve(handle_, rows, rope_dims)); }
    void attention_turns_arm(uint64_t rows) { check(sd_attention_turns_arm(handle_, rows)); }
    using Rows = std::optional<std::pair<const float*, uint64_t>>;        // (pointer, rows): compressed rows, may carry the BF16 tag
    using Picks = std::optional<std::pair<const int32_t*, uint64_t>>;     // (pointer, selections)
    using Rope = std::optional<std::pair<uint64_t, const Buffer*>>;       // (dims, frequencies)
    void sparse_attention(const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions, uint64_t window, Rows compressed,
                          Picks selected, const float* sinks, uint64_t rows, uint64_t heads, uint64_t dim, float scale, Rope rope,
                          const Buffer* scratch, float* out) {
        check(sd_op_sparse_attention(handle_, q, raw, raw_rows, positions, window, compressed ? compressed->first : nullptr,
                                     compressed ? compressed->second : 0, selected ? selected->first : nullptr, selected ? selected->second : 0,
                                     sinks, rows, heads, dim, scale, rope ? rope->first : 0,
                                     rope ? static_cast<const float*>(rope->second->pointer) : nullptr,
                                     scratch ? static_cast<float*>(scratch->pointer) : nullptr, scratch ? scratch->bytes : 0, out));
    }
    // (an addition) `spans` calls of sparse_attention with rows = span_rows in one launch
    void sparse_attention_spans(const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions, uint64_t window, Rows compressed,
                                Picks selected, const float* sinks, uint64_t spans, uint64_t span_rows, uint64_t heads, uint64_t dim,
                                float scale, Rope rope, float* out) {
        check(sdx_sparse_attention_spans(handle_, q, raw, raw_rows, positions, window, compressed ? compressed->first : nullptr,
                                         compressed ? compressed->second : 0, selected ? selected->first : nullptr,
                                         selected ? selected->second : 0, sinks, spans, span_rows, heads, dim, scale, rope ? rope->first : 0,
                                         rope ? static_cast<const float*>(rope->second->pointer) : nullptr, out));
    }

    // ---- ops.rs:1021-1024, 1241-1244 ----
    void to_bf16(const float* x, uint64_t count, void* out) { check(sd_op_to_bf16(handle_, x, count, out)); }
    void top_k(const float* scores, uint64_t rows, uint64_t groups, uint64_t k, int32_t* out) { check(sd_op_top_k(handle_, scores, rows, groups, k, out)); }

    // ---- additions for Q8_0 GQA (no counterpart in the reference ABI: it reaches these kernels inside its span calls) ----
    void kv_write(const Buffer& state, uint64_t context, uint64_t kv_heads, uint64_t base, uint64_t steps, const float* keys, const float* values) {
        check(sdx_kv_write(handle_, state.pointer, context, kv_heads, base, steps, keys, values));
    }
    void qsa_decode(const std::vector<const void*>& states, const std::vector<uint64_t>& contexts, const std::vector<uint64_t>& lengths,
                    uint64_t heads, uint64_t kv_heads, float scale, const void* q_f16, float* out) {
        if (contexts.size() != states.size() || lengths.size() != states.size()) throw Error("one context and one length per state");
        check(sdx_qsa_decode(handle_, states.data(), contexts.data(), lengths.data(), states.size(), heads, kv_heads, scale, q_f16, out));
    }
    void qsa_prompt(const Buffer& state, uint64_t context, uint64_t first, uint64_t rows, uint64_t heads, uint64_t kv_heads, float scale,
                    const void* q_f16, float* out) {
        check(sdx_qsa_prompt(handle_, state.pointer, context, first, rows, heads, kv_heads, scale, q_f16, out));
    }
    int decode_status() { return check(sdx_decode_status(handle_)); }

  private:
    static int check(int result) {
        if (result < 0) throw Error(sd_error());
        return result;
    }
    static Buffer made(void* pointer, uint64_t bytes) {
        if (!pointer) throw Error(sd_error());
        return Buffer{pointer, bytes};
    }
    void* handle_;
};

}  // namespace straydog
