// The seam inside the reference's own build: its internal decode-attention functions, with their signatures, over this
// library's tensor-core kernels.
//
// The reference's layer spans (sd_decode_span, sd_verify_span, sd_qsa_sequence) do not reach the attention kernels through the
// C ABI but through two internal function templates, qsa_attention<P> and qsa_attention_rows<P>
// (gpu/sparse_attention_compute.hpp:609-647), called from gpu/qsa_decode.hpp:42,126 and gpu/verify_span.hpp. A maintainer who
// wants those spans on the B200 kernels includes this header in gpu/kernels.cpp in place of the two definitions (after
// gpu/core.hpp, which brings Device, QwenHeads<P>, kv_t and kv_row_q8; before gpu/qsa_decode.hpp) and links
// libstraydog_gpu_b200.so. Everything else in the span stays the reference's: the packed rows in d.input, the selection
// written by qsa_select_rows, write_attention_kv, the gate's place in the projections.
//
// What is the same: arguments and their meaning; which slots are live (gpu/sparse_attention_compute.hpp:58-64); ring-mirror
// addressing (:65-68); the gate folded into the merge (:168); a verification row has the bits of the one-token decode of the
// same token (gpu/qsa_decode.hpp:46-50). What differs: the partials live in this library's own workspace, not in
// d.attention_scores; a prompt batch (steps > 1 in qsa_attention) keeps the reference's own qsa_flash_launch, because its rows
// attend selection lists, which this library's prompt kernel (dense causal) does not take.
#pragma once
#include "straydog_gpu_b200.h"

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

namespace qsa_b200 {

// One adopted handle per reference Device: this library queues on the reference's stream, so its kernels run in order with the
// span's other kernels and inside the span's graph captures.
template <class DeviceT>
inline void* handle_of(DeviceT& d) {
    static std::mutex mutex;
    static std::map<int, void*> handles;
    std::lock_guard<std::mutex> lock(mutex);
    auto found = handles.find(d.ordinal);
    if (found != handles.end()) return found->second;
    void* made = sdx_adopt(d.ordinal, reinterpret_cast<void*>(d.stream));
    if (!made) throw std::runtime_error(std::string("B200 attention library: ") + sd_error());
    handles[d.ordinal] = made;
    return made;
}
inline void check(int result) {
    if (result < 0) throw std::runtime_error(std::string("B200 attention library: ") + sd_error());
}

}  // namespace qsa_b200

#if defined(QSA_B200_REFERENCE_TYPES)   // set by the including translation unit once Device, QwenHeads and kv_t are declared

// gpu/sparse_attention_compute.hpp:609-627
template <int P = 1>
void qsa_attention(Device& d, void* kv, size_t context, size_t base, size_t steps, size_t selected, const float* input, float* output,
                   const uint32_t* position = nullptr, const kv_t* mirror = nullptr, size_t mirror_rows = 0) {
    using H = QwenHeads<P>;
    if (steps > 1) {   // a prompt batch: the reference's own flash kernels
        qsa_flash_launch<P>(d, dim3(unsigned(steps), unsigned(H::kv)), static_cast<const kv_t*>(kv), context, base, steps, selected, input, output);
        return;
    }
    if (d.kv_row != kv_row_q8) throw std::runtime_error("the B200 attention library reads Q8_0 K/V rows (sd_kv_format(272))");
    qsa_b200::check(sdx_qsa_attention_rows(qsa_b200::handle_of(d), kv, context, base, position, 1, selected, H::query, H::kv, 0.0625f, input,
                                           mirror, mirror_rows, nullptr, 0, output));
}

// gpu/sparse_attention_compute.hpp:631-647
template <int P = 1>
void qsa_attention_rows(Device& d, void* kv, size_t context, size_t steps, size_t selected, const float* input, float* output,
                        const uint32_t* position, const kv_t* mirror = nullptr, size_t mirror_rows = 0, const float* gates = nullptr,
                        size_t gate_stride = 0) {
    using H = QwenHeads<P>;
    if (d.kv_row != kv_row_q8) throw std::runtime_error("the B200 attention library reads Q8_0 K/V rows (sd_kv_format(272))");
    qsa_b200::check(sdx_qsa_attention_rows(qsa_b200::handle_of(d), kv, context, 0, position, steps, selected, H::query, H::kv, 0.0625f, input,
                                           mirror, mirror_rows, gates, gate_stride, output));
}

#endif
