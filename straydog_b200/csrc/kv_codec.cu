// Q8_0 K/V rows: the write path (append new tokens' keys and values to a state) and a plain decode
// of rows to F32. Bit-exact with the reference's codec: gpu/kernels.cpp:38-44 (kv_scale, kv_load),
// :58-74 (kv_encode, kv_put), :79-98 (write_attention_kv); Rust twin
// crates/straydog-engine/src/gpu.rs:536-561.
//
// Row layout (gpu/core.hpp:398-403): 256 int8 values, then the 8 FP16 scales of their 32-value
// blocks, 272 bytes; or, under sd_kv_format(512), 256 FP16 values (the nearest FP16 of each value,
// gpu/kernels.cpp:42, 70). State layout: 2 * kv_heads planes of `context` rows, keys of head 0.., then
// values of head 0...
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

namespace sdb {

// One warp encodes one 32-value block: lane = column % 32. Grid-stride over blocks so that any
// number of rows runs in one launch sized to the SM count.
template<bool F16>
__global__ void __launch_bounds__(256) kv_write_kernel(uint8_t* __restrict__ state, size_t context, size_t kv_heads, size_t base,
                                                        const uint32_t* __restrict__ position, size_t steps,
                                                        const float* __restrict__ keys, const float* __restrict__ values) {
    constexpr size_t kRow = F16 ? kv_row_f16 : kv_row_q8;
    if (position) base = *position;
    const size_t width = kv_heads * 256, blocks = steps * width / 32 * 2;   // key blocks, then value blocks
    const unsigned lane = threadIdx.x % 32;
    for (size_t block = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) / 32; block < blocks;
         block += size_t(gridDim.x) * blockDim.x / 32) {
        const bool is_value = block >= blocks / 2;
        const size_t index = (is_value ? block - blocks / 2 : block) * 32 + lane;   // into [steps][kv_heads][256]
        const size_t step = index / width, head = (index % width) / 256, column = index % 256;
        uint8_t* row = state + (((is_value ? kv_heads : 0) + head) * context + base + step) * kRow;
        if constexpr (F16) {
            reinterpret_cast<__half*>(row)[column] = __float2half_rn((is_value ? values : keys)[index]);
        } else {
            __half scale_h;
            const int8_t q = q8_encode((is_value ? values : keys)[index], scale_h);
            reinterpret_cast<int8_t*>(row)[column] = q;
            if (lane == 0) reinterpret_cast<__half*>(row + 256)[column / 32] = scale_h;
        }
    }
}

// The same encode for a batch of sequences, one new token each: segment i (a sequence's K/V head) takes keys / values
// [i][256] into row `length - 1` of its planes.
__global__ void __launch_bounds__(256) kv_append_kernel(const Segment* __restrict__ segments, size_t count,
                                                         const float* __restrict__ keys, const float* __restrict__ values) {
    const unsigned lane = threadIdx.x % 32;
    const size_t blocks = count * 8 * 2;
    for (size_t block = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) / 32; block < blocks; block += size_t(gridDim.x) * blockDim.x / 32) {
        const bool is_value = block >= blocks / 2;
        const size_t index = (is_value ? block - blocks / 2 : block) * 32 + lane, segment = index / 256, column = index % 256;
        __half scale_h;
        const int8_t q = q8_encode((is_value ? values : keys)[index], scale_h);
        const Segment s = segments[segment];
        uint8_t* row = const_cast<uint8_t*>(is_value ? s.values : s.keys) + size_t(s.length - 1) * kv_row_q8;
        reinterpret_cast<int8_t*>(row)[column] = q;
        if (lane == 0) reinterpret_cast<__half*>(row + 256)[column / 32] = scale_h;
    }
}

// The same append with a warp a row (a segment's 256 keys or values): a lane takes 8 consecutive values in two 16-byte loads, so a row
// crosses the bus (the new rows may lie in page-locked host memory, read in place) in two requests of 512 bytes instead of eight of
// 128; a block is four lanes, its largest magnitude two shuffles. The arithmetic is q8_encode's, value by value.
__global__ void __launch_bounds__(256) kv_append_wide_kernel(const Segment* __restrict__ segments, size_t count,
                                                              const float* __restrict__ keys, const float* __restrict__ values) {
    const unsigned lane = threadIdx.x % 32;
    const size_t rows = 2 * count;
    for (size_t row = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) / 32; row < rows; row += size_t(gridDim.x) * blockDim.x / 32) {
        const bool is_value = row >= count;
        const size_t segment = is_value ? row - count : row;
        const float4* source = reinterpret_cast<const float4*>((is_value ? values : keys) + segment * 256) + 2 * lane;
        const float4 a = source[0], b = source[1];
        const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        float top = 0.0f;
        #pragma unroll
        for (int i = 0; i < 8; ++i) top = fmaxf(top, fabsf(x[i]));
        top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
        top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
        const __half scale_h = __float2half_rn(__fdiv_rn(top, 127.0f));
        const float scale = __half2float(scale_h);
        uint32_t packed[2] = {0, 0};
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            int q = scale > 0.0f ? __float2int_rn(__fdiv_rn(x[i], scale)) : 0;
            q = q > 127 ? 127 : q < -127 ? -127 : q;
            packed[i / 4] |= uint32_t(uint8_t(int8_t(q))) << (8 * (i % 4));
        }
        const Segment s = segments[segment];
        uint8_t* target = const_cast<uint8_t*>(is_value ? s.values : s.keys) + size_t(s.length - 1) * kv_row_q8;
        *reinterpret_cast<uint2*>(target + 8 * lane) = make_uint2(packed[0], packed[1]);
        if (lane % 4 == 0) reinterpret_cast<__half*>(target + 256)[lane / 4] = scale_h;
    }
}

// rows of 272 bytes -> rows of 256 F32: value = float(int8) * float(scale), one FP32 multiply; rows of 512 bytes: the FP16 values widened.
template<bool F16>
__global__ void __launch_bounds__(256) kv_decode_rows_kernel(const uint8_t* __restrict__ rows, size_t count, float* __restrict__ out) {
    for (size_t index = size_t(blockIdx.x) * blockDim.x + threadIdx.x; index < count * 256; index += size_t(gridDim.x) * blockDim.x) {
        const uint8_t* row = rows + index / 256 * (F16 ? kv_row_f16 : kv_row_q8);
        const size_t column = index % 256;
        if constexpr (F16) {
            out[index] = __half2float(reinterpret_cast<const __half*>(row)[column]);
        } else {
            const float scale = __half2float(reinterpret_cast<const __half*>(row + 256)[column / 32]);
            out[index] = __fmul_rn(float(reinterpret_cast<const int8_t*>(row)[column]), scale);
        }
    }
}

void launch_kv_write(Device& d, uint8_t* state, size_t context, size_t kv_heads, size_t base, const uint32_t* position, size_t steps,
                     const float* keys, const float* values) {
    const size_t warps = steps * kv_heads * 8 * 2;
    const unsigned grid = unsigned(std::min<size_t>((warps + 7) / 8, size_t(d.sms) * 8));
    if (d.kv_row == kv_row_f16) kv_write_kernel<true><<<grid, 256, 0, d.stream>>>(state, context, kv_heads, base, position, steps, keys, values);
    else kv_write_kernel<false><<<grid, 256, 0, d.stream>>>(state, context, kv_heads, base, position, steps, keys, values);
    ++d.launches;
}

void launch_kv_append(Device& d, const Segment* segments, size_t count, const float* keys, const float* values, cudaStream_t stream) {
    if (reinterpret_cast<uintptr_t>(keys) % 16 == 0 && reinterpret_cast<uintptr_t>(values) % 16 == 0) {
        kv_append_wide_kernel<<<unsigned(std::min<size_t>((count * 2 + 7) / 8, size_t(d.sms) * 8)), 256, 0, stream>>>(segments, count, keys, values);
    } else {
        const unsigned grid = unsigned(std::min<size_t>((count * 16 + 7) / 8, size_t(d.sms) * 8));
        kv_append_kernel<<<grid, 256, 0, stream>>>(segments, count, keys, values);
    }
    ++d.launches;
}

}  // namespace sdb

using namespace sdb;

extern "C" {

int sdx_kv_write(void* handle, void* state, uint64_t context, uint64_t kv_heads, uint64_t base, uint64_t steps, const float* keys,
                 const float* values) {
    SDB_OP_BEGIN
    if (!context || !kv_heads || !steps || base > context || steps > context - base) throw std::runtime_error("invalid Straydog K/V write");
    span(value, state, checked_product({2, kv_heads, context, value.kv_row}), "a K/V state");
    span(value, keys, checked_product({steps, kv_heads, 256, 4}), "new keys");
    span(value, values, checked_product({steps, kv_heads, 256, 4}), "new values");
    launch_kv_write(value, static_cast<uint8_t*>(state), context, kv_heads, base, nullptr, steps, keys, values);
    SDB_OP_END
}

int sdx_kv_decode_rows(void* handle, const void* rows, uint64_t count, float* out) {
    SDB_OP_BEGIN
    if (!count) throw std::runtime_error("invalid Straydog K/V row count");
    span(value, rows, checked_product({count, value.kv_row}), "K/V rows");
    span(value, out, checked_product({count, 256, 4}), "decoded K/V rows");
    const unsigned grid = unsigned(std::min<size_t>((count * 256 + 255) / 256, size_t(value.sms) * 16));
    if (value.kv_row == kv_row_f16) kv_decode_rows_kernel<true><<<grid, 256, 0, value.stream>>>(static_cast<const uint8_t*>(rows), count, out);
    else kv_decode_rows_kernel<false><<<grid, 256, 0, value.stream>>>(static_cast<const uint8_t*>(rows), count, out);
    ++value.launches;
    SDB_OP_END
}

}  // extern "C"
