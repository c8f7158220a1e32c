// sd_attention_sequence: the reference's standalone selection-attention entry (host floats in,
// host floats out; gpu/kernels.cpp:4387-4419 over attention_scores / attention_reduce, :100-165).
//
// Both K/V row formats (sd_kv_format: Q8_0 rows of 272 bytes, FP16 rows of 512, gpu/kernels.cpp:36-43): this entry is the check path,
// and the FP16 rows are what the Q8_0 rows are checked against. The selection kernel keeps FP32 arithmetic throughout (queries arrive as F32 and the reference
// computes in F32): one block per (step, query head), a warp per selected key for the scores
// (lanes over the 256 columns, 8 consecutive columns each), the probabilities in shared memory, then
// a thread per output column summing p * v in slot order, as attention_reduce does.
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

namespace sdb {

void launch_kv_write(Device& d, uint8_t* state, size_t context, size_t kv_heads, size_t base, const uint32_t* position, size_t steps,
                     const float* keys, const float* values);

constexpr int kMaxSelected = 2052;   // gpu/kernels.cpp:4392

// kv_load (gpu/kernels.cpp:40-43): a row's value as it is read, Q8_0 (one FP32 multiply) or FP16
template<bool F16>
__device__ __forceinline__ float kv_at(const uint8_t* row, unsigned column) {
    if constexpr (F16) return __half2float(reinterpret_cast<const __half*>(row)[column]);
    return __fmul_rn(float(reinterpret_cast<const int8_t*>(row)[column]),
                     __half2float(reinterpret_cast<const __half*>(row + 256)[column / 32]));
}

template<bool F16>
__global__ void __launch_bounds__(256) selection_attention_kernel(const uint8_t* __restrict__ state, size_t context, size_t base,
                                                                  size_t steps, size_t selected, size_t heads, size_t kv_heads,
                                                                  float scale, const float* __restrict__ input, float* __restrict__ output) {
    const size_t item = blockIdx.x, step = item / heads, head = item % heads, kv = head / (heads / kv_heads);
    const unsigned t = threadIdx.x, lane = t % 32, warp = t / 32;
    const size_t index_start = steps * (heads * 256 + kv_heads * 512);
    const float* indices = input + index_start + step * selected;
    const size_t count = size_t(input[index_start + steps * selected + step]);
    __shared__ float query[256];
    __shared__ float weights[kMaxSelected];
    __shared__ int tokens[kMaxSelected];
    __shared__ float reduce[8];
    query[t] = input[item * 256 + t];
    __syncthreads();
    // scores: a warp per slot
    constexpr size_t kRow = F16 ? kv_row_f16 : kv_row_q8;
    const uint8_t* keys = state + kv * context * kRow;
    for (size_t slot = warp; slot < selected; slot += 8) {
        int token = -1;
        if (slot < count) {
            const float raw = indices[slot];
            if (raw >= 0 && raw <= float(base + step) && raw < float(context)) token = int(raw);
        }
        float sum = 0.0f;
        if (token >= 0) {
            const uint8_t* row = keys + size_t(token) * kRow;
            if constexpr (F16) {
                const uint4 halves = *reinterpret_cast<const uint4*>(row + 16 * lane);
                const uint32_t words[4] = {halves.x, halves.y, halves.z, halves.w};
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float k = __half2float(__ushort_as_half(uint16_t(i & 1 ? words[i / 2] >> 16 : words[i / 2] & 0xffffu)));
                    sum = fmaf(k, query[8 * lane + i], sum);
                }
            } else {
                const uint2 bytes = *reinterpret_cast<const uint2*>(row + 8 * lane);
                const float block_scale = __half2float(reinterpret_cast<const __half*>(row + 256)[lane / 4]);
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t word = i < 4 ? bytes.x : bytes.y;
                    const float k = __fmul_rn(float(int8_t(word >> (8 * (i & 3)))), block_scale);
                    sum = fmaf(k, query[8 * lane + i], sum);
                }
            }
            #pragma unroll
            for (unsigned offset = 16; offset; offset /= 2) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        }
        if (lane == 0) { weights[slot] = token >= 0 ? sum * scale : -INFINITY; tokens[slot] = token; }
    }
    __syncthreads();
    float top = -INFINITY;
    for (size_t slot = t; slot < selected; slot += 256) top = fmaxf(top, weights[slot]);
    #pragma unroll
    for (unsigned offset = 16; offset; offset /= 2) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
    if (lane == 0) reduce[warp] = top;
    __syncthreads();
    top = reduce[0];
    #pragma unroll
    for (int w = 1; w < 8; ++w) top = fmaxf(top, reduce[w]);
    __syncthreads();
    float total = 0.0f;
    for (size_t slot = t; slot < selected; slot += 256) {
        const float p = expf(weights[slot] - top);
        weights[slot] = p;
        total += p;
    }
    #pragma unroll
    for (unsigned offset = 16; offset; offset /= 2) total += __shfl_xor_sync(0xffffffffu, total, offset);
    if (lane == 0) reduce[warp] = total;
    __syncthreads();
    total = 0.0f;
    #pragma unroll
    for (int w = 0; w < 8; ++w) total += reduce[w];
    for (size_t slot = t; slot < selected; slot += 256) weights[slot] = __fdiv_rn(weights[slot], total);
    __syncthreads();
    const uint8_t* values = state + (kv_heads + kv) * context * kRow;
    float result = 0.0f;
    const size_t live = count < selected ? count : selected;
    for (size_t slot = 0; slot < live; ++slot) {
        const int token = tokens[slot];
        if (token >= 0) result = fmaf(weights[slot], kv_at<F16>(values + size_t(token) * kRow, t), result);
    }
    output[item * 256 + t] = result;
}

}  // namespace sdb

using namespace sdb;

extern "C" {

int sd_attention_sequence(void* handle, void* state, uint64_t context, uint64_t base, uint64_t steps, uint64_t selected,
                          const float* input, uint64_t input_count, float* output, uint64_t output_count) {
    try {
        auto& value = device(handle);
        constexpr uint64_t heads = 24, kv_heads = 2;   // gpu/core.hpp:390 (QwenHeads<1>)
        if (!input || !output || !context || context > 262144 || !steps || steps > max_batch || base > context ||
            steps > context - base || !selected || selected > kMaxSelected)
            throw std::runtime_error("invalid Straydog attention dimensions");
        if (allocation_bytes(value, state) != context * 4 * value.kv_row)
            throw std::runtime_error("Straydog attention state size mismatch");
        if (input_count != steps * (heads * 256 + kv_heads * 512 + selected + 1) || output_count != steps * heads * 256)
            throw std::runtime_error("Straydog attention workspace mismatch");
        // Counts are host-readable metadata: validated before any kernel reads them (gpu/kernels.cpp:4400-4406).
        const size_t count_offset = size_t(steps * (heads * 256 + kv_heads * 512 + selected));
        for (size_t step = 0; step < steps; ++step) {
            const float count = input[count_offset + step];
            if (!(count >= 1 && count <= float(selected)) || count != float(size_t(count)))
                throw std::runtime_error("invalid Straydog attention selection count");
        }
        const size_t in_bytes = size_t(input_count) * 4, out_bytes = size_t(output_count) * 4;
        auto* work = static_cast<float*>(ensure(value, value.work, value.work_bytes, in_bytes + out_bytes + 256));
        float* device_out = work + (in_bytes + 255) / 256 * 64;
        SDB_CHECK(cudaMemcpyAsync(work, input, in_bytes, cudaMemcpyHostToDevice, value.stream));
        launch_kv_write(value, static_cast<uint8_t*>(state), context, kv_heads, base, nullptr, steps, work + steps * heads * 256,
                        work + steps * (heads + kv_heads) * 256);
        if (value.kv_row == kv_row_f16)
            selection_attention_kernel<true><<<unsigned(steps * heads), 256, 0, value.stream>>>(
                static_cast<const uint8_t*>(state), context, base, steps, selected, heads, kv_heads, 0.0625f, work, device_out);
        else
            selection_attention_kernel<false><<<unsigned(steps * heads), 256, 0, value.stream>>>(
                static_cast<const uint8_t*>(state), context, base, steps, selected, heads, kv_heads, 0.0625f, work, device_out);
        ++value.launches;
        SDB_CHECK(cudaGetLastError());
        SDB_CHECK(cudaMemcpyAsync(output, device_out, out_bytes, cudaMemcpyDeviceToHost, value.stream));
        SDB_CHECK(cudaStreamSynchronize(value.stream));
        return 0;
    } catch (const std::exception& e) { last_error = e.what(); return -1; }
}

}  // extern "C"
