// sd_op_dspark_attention: the drafter's noncausal block attention (gpu/dspark_attention.hpp:1-101, entry gpu/kernels.cpp region of
// sd_op_dspark_attention; declared gpu/straydog_gpu.h:399-406). Every query of a block (1 to 5 slots, a device's 1 to 64 heads, 512
// columns, rope already applied) sees the history positions [anchor - history, anchor) of the K = V ring of 128 rows and ALL of the
// block's own keys; scale 1 / sqrt(512); a head's sink enters the softmax maximum and the denominator, never the output.
//
// Every query row of the call attends the same keys, so a CTA takes one head with all of the block's slots: a key row is read once
// for the (up to) five queries of the head instead of once per query row. Scores: a warp per key, lanes over the 512 columns, the
// slots' queries in registers; then the weights in shared memory and a thread per column pair for the output, again one read of a
// key for all slots. Exact FP32 arithmetic (the contract is an FP32 error bound: tests/dspark_attention_gpu.rs:42-51).
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

namespace sdb {

constexpr int kDsparkDim = 512, kDsparkRing = 128, kDsparkSlots = 5, kDsparkKeys = kDsparkRing + kDsparkSlots;

__global__ void __launch_bounds__(256) dspark_attention_kernel(const float* __restrict__ q, const float* __restrict__ ring, const float* __restrict__ block,
                                                               const float* __restrict__ sinks, size_t heads, size_t slots, uint32_t anchor,
                                                               const int32_t* __restrict__ anchor_at, size_t history, float scale, float* __restrict__ out) {
    const size_t head = blockIdx.x;
    const unsigned t = threadIdx.x, lane = t % 32, warp = t / 32;
    const int64_t end = anchor_at ? int64_t(anchor_at[0]) : int64_t(anchor);             // history positions [end - history, end)
    const int64_t first = end - int64_t(history) < 0 ? 0 : end - int64_t(history);
    const size_t raw_count = size_t(end - first), total = raw_count + slots;
    __shared__ float weights[kDsparkSlots][kDsparkKeys];
    __shared__ float denominators[kDsparkSlots];
    const auto key_row = [&](size_t index) {
        return index < raw_count ? ring + size_t(first + int64_t(index)) % kDsparkRing * kDsparkDim : block + (index - raw_count) * kDsparkDim;
    };
    // ---- scores: lane l holds columns 4 l .. 4 l + 3 of each 128-column quarter of every slot's query ----
    float4 qv[kDsparkSlots][4];
    #pragma unroll
    for (int s = 0; s < kDsparkSlots; ++s)
        #pragma unroll
        for (int part = 0; part < 4; ++part)
            qv[s][part] = size_t(s) < slots ? *reinterpret_cast<const float4*>(q + (s * heads + head) * kDsparkDim + part * 128 + 4 * lane) : make_float4(0, 0, 0, 0);
    for (size_t index = warp; index < total; index += 8) {
        const float* k = key_row(index);
        float4 kv[4];
        #pragma unroll
        for (int part = 0; part < 4; ++part) kv[part] = *reinterpret_cast<const float4*>(k + part * 128 + 4 * lane);
        #pragma unroll
        for (int s = 0; s < kDsparkSlots; ++s) {
            float dot = 0.0f;
            #pragma unroll
            for (int part = 0; part < 4; ++part) {
                dot = fmaf(qv[s][part].x, kv[part].x, dot); dot = fmaf(qv[s][part].y, kv[part].y, dot);
                dot = fmaf(qv[s][part].z, kv[part].z, dot); dot = fmaf(qv[s][part].w, kv[part].w, dot);
            }
            #pragma unroll
            for (unsigned offset = 16; offset; offset /= 2) dot += __shfl_xor_sync(0xffffffffu, dot, offset);
            if (lane == 0) weights[s][index] = dot * scale;
        }
    }
    __syncthreads();
    // ---- softmax per slot: warp s takes slot s ----
    if (warp < slots) {
        const float sink = sinks[head];
        float top = sink;
        for (size_t index = lane; index < total; index += 32) top = fmaxf(top, weights[warp][index]);
        #pragma unroll
        for (unsigned offset = 16; offset; offset /= 2) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
        float sum = 0.0f;
        for (size_t index = lane; index < total; index += 32) {
            const float score = weights[warp][index];
            const float w = score == -INFINITY ? 0.0f : expf(score - top);
            weights[warp][index] = w;
            sum += w;
        }
        #pragma unroll
        for (unsigned offset = 16; offset; offset /= 2) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        if (lane == 0) denominators[warp] = sum + expf(sink - top);
    }
    __syncthreads();
    // ---- output: a thread per column pair, one read of a key for all the slots ----
    const size_t dim = 2 * size_t(t);
    float2 acc[kDsparkSlots];
    #pragma unroll
    for (int s = 0; s < kDsparkSlots; ++s) acc[s] = make_float2(0.0f, 0.0f);
    #pragma unroll 4
    for (size_t index = 0; index < total; ++index) {
        const float2 v = *reinterpret_cast<const float2*>(key_row(index) + dim);
        #pragma unroll
        for (int s = 0; s < kDsparkSlots; ++s) {
            const float w = size_t(s) < slots ? weights[s][index] : 0.0f;
            acc[s].x = fmaf(w, v.x, acc[s].x); acc[s].y = fmaf(w, v.y, acc[s].y);
        }
    }
    #pragma unroll
    for (int s = 0; s < kDsparkSlots; ++s)
        if (size_t(s) < slots) {
            float* o = out + (s * heads + head) * kDsparkDim + dim;
            o[0] = acc[s].x / denominators[s];
            o[1] = acc[s].y / denominators[s];
        }
}

}  // namespace sdb

using namespace sdb;

extern "C" int sd_op_dspark_attention(void* handle, const float* q, const float* ring, const float* block, const float* sinks, uint64_t heads,
                                      uint64_t slots, uint32_t anchor, const int32_t* anchor_at, uint64_t history, float* out) {
    SDB_OP_BEGIN
    if (!heads || heads > 64 || !slots || slots > uint64_t(kDsparkSlots) || history > uint64_t(kDsparkRing) || anchor > uint32_t(INT32_MAX) || history > anchor)
        throw std::runtime_error("invalid DSpark attention block or history range");
    span(value, q, checked_product({slots, heads, kDsparkDim, 4}), "DSpark rotated queries");
    span(value, ring, size_t(kDsparkRing) * kDsparkDim * 4, "DSpark history K ring");
    span(value, block, checked_product({slots, kDsparkDim, 4}), "DSpark rotated block keys");
    span(value, sinks, checked_product({heads, 4}), "DSpark attention sinks");
    span(value, out, checked_product({slots, heads, kDsparkDim, 4}), "DSpark attention output");
    if (anchor_at) span(value, anchor_at, 4, "DSpark anchor position");
    if (reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(ring) % 16 || reinterpret_cast<uintptr_t>(block) % 16 || reinterpret_cast<uintptr_t>(out) % 8)
        throw std::runtime_error("DSpark attention operands must be 16-byte aligned");
    dspark_attention_kernel<<<unsigned(heads), 256, 0, value.stream>>>(q, ring, block, sinks, size_t(heads), size_t(slots), anchor, anchor_at,
                                                                       size_t(history), 1.0f / sqrtf(float(kDsparkDim)), out);
    ++value.launches;
    SDB_OP_END
}
