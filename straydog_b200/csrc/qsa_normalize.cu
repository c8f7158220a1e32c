// The front of Qwen's decode and verification attention in one launch: RMS normalisation and rotation of the rows' queries, keys
// and index queries, the rows' keys and values written to the Q8_0 K/V state (and its mirror), the index keys pooled into the
// indexer's blocks. What it replaces: qsa_normalize_rows (gpu/qsa_decode.hpp:86-111) and, for one row, qsa_normalize_decode +
// qsa_pool_one + write_attention_kv as qsa_decode_attend launches them (gpu/qsa_decode.hpp:5-23, 28-44; gpu/sparse_attention.hpp:2-6,
// 55-79), for any number of query and K/V heads.
//
// A row of projections (stride floats apart) is  qgate [heads][query 256 | gate 256] | key [kv_heads][256] | value [kv_heads][256] |
// index query [4][128] | index key [128]. The grid is (heads + kv_heads + 5, rows), 256 threads:
//   blocks 0 .. heads - 1         a query head: normalised, rotated, into packed[row][head][256]
//   the next kv_heads blocks      a key head: normalised, rotated, into packed's keys, then encoded with the head's value row
//                                 into row positions[row] of the state's planes (a warp is one Q8_0 block)
//   the next four                 an index-query head of 128, in place
//   the last, for row 0 only      the rows' index keys enter the 16-position history ring one after the other; a row that
//                                 completes a 4-position block pools it (mean of the four, normalised, rotated at the
//                                 block's first position) into blocks[column][position / 4]
// Arithmetic, so that the values are the reference's: x * norm and x * x per column; the squares are summed by halving (column c
// takes c + 128, then c + 64, ... c + 1: the reference's tree, here through shared memory down to a warp and by shuffles inside
// it); the divisor is sqrtf(sum / width + 1e-6f); the rotation pairs column c < 64 with (c + 32) % 64 at the angle
// position / 1e7^((c % 32) / 32), columns from 64 on pass.
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

namespace sdb {

namespace {

constexpr size_t kHistory = 16;   // gpu/sparse_attention.hpp:85

struct NormalizeArgs {
    float* projections; size_t stride, rows, heads, kv_heads;
    const float* qnorm; const float* knorm; const float* iqnorm; const float* pool_norm;
    const uint32_t* positions; const uint32_t* ropes;
    float* packed;
    uint8_t* state; size_t context;
    uint8_t* mirror; size_t mirror_rows;
    float* blocks; size_t pool;   // [128][pool], then the history ring [16][128]
    int* status;
};

// gpu/sparse_attention.hpp:2-6
__device__ __forceinline__ float rotate(float own, float partner, size_t column, size_t position) {
    if (column >= 64) return own;
    const float angle = float(position) / powf(1e7f, float(column % 32) / 32.0f);
    return own * cosf(angle) + (column < 32 ? -partner : partner) * sinf(angle);
}

// The sum of sums[0 .. width) by halving, in every thread: the shared-memory levels down to 32, the rest by shuffles (lane c adds
// lane c + offset: the same pairs as the reference's loop). Every thread of the block calls it.
__device__ __forceinline__ float halving_sum(float* sums, size_t width, size_t column, float* total) {
    __syncthreads();
    for (unsigned offset = unsigned(width / 2); offset >= 32; offset /= 2) {
        if (column < offset) sums[column] += sums[column + offset];
        __syncthreads();
    }
    if (column < 32) {
        float s = sums[column];
        #pragma unroll
        for (unsigned offset = 16; offset; offset /= 2) s += __shfl_down_sync(0xffffffffu, s, offset);
        if (column == 0) *total = s;
    }
    __syncthreads();
    return *total;
}

// one head of `width` columns: normalised and rotated into target[column]; returns this thread's value (0 past the width)
__device__ __forceinline__ float normalize_head(const float* source, const float* norm, size_t width, size_t position, float* target,
                                                float* values, float* sums, float* total) {
    const size_t column = threadIdx.x;
    const bool own = column < width;
    if (own) { const float x = source[column]; values[column] = x * norm[column]; sums[column] = x * x; }
    const float sum = halving_sum(sums, width, column, total);
    if (!own) return 0.0f;
    const float denominator = sqrtf(sum / float(width) + 1e-6f);
    const float mine = values[column] / denominator;
    const float partner = column < 64 ? values[(column + 32) % 64] / denominator : 0.0f;
    const float result = rotate(mine, partner, column, position);
    target[column] = result;
    return result;
}

__global__ void __launch_bounds__(256) qsa_normalize_rows_kernel(const NormalizeArgs a) {
    __shared__ float values[256], sums[256], total;
    const size_t block = blockIdx.x, row = blockIdx.y, column = threadIdx.x;
    const size_t keys = a.heads * 512, vals = keys + a.kv_heads * 256, index = keys + a.kv_heads * 512;
    float* own = a.projections + row * a.stride;
    const size_t rope = a.ropes[row];
    if (block < a.heads) {
        normalize_head(own + block * 512, a.qnorm, 256, rope, a.packed + (row * a.heads + block) * 256, values, sums, &total);
    } else if (block < a.heads + a.kv_heads) {
        const size_t head = block - a.heads, position = a.positions[row];
        if (position >= a.context) {   // (a position past the state: nothing of the row is written, and the host is told)
            if (column == 0) atomicExch(a.status, 5);
            return;
        }
        float* normalized = a.packed + a.rows * a.heads * 256 + (row * a.kv_heads + head) * 256;
        const float key = normalize_head(own + keys + head * 256, a.knorm, 256, rope, normalized, values, sums, &total);
        __half key_scale, value_scale;
        const int8_t k8 = q8_encode(key, key_scale), v8 = q8_encode(own[vals + head * 256 + column], value_scale);
        auto put = [&](uint8_t* planes, size_t rows_of_plane, size_t at) {
            uint8_t* k_row = planes + (head * rows_of_plane + at) * kv_row_q8;
            uint8_t* v_row = planes + ((a.kv_heads + head) * rows_of_plane + at) * kv_row_q8;
            reinterpret_cast<int8_t*>(k_row)[column] = k8;
            reinterpret_cast<int8_t*>(v_row)[column] = v8;
            if (column % 32 == 0) {
                reinterpret_cast<__half*>(k_row + 256)[column / 32] = key_scale;
                reinterpret_cast<__half*>(v_row + 256)[column / 32] = value_scale;
            }
        };
        put(a.state, a.context, position);
        if (a.mirror_rows) put(a.mirror, a.mirror_rows, position % a.mirror_rows);
    } else if (block < a.heads + a.kv_heads + 4) {
        const size_t head = block - a.heads - a.kv_heads;
        normalize_head(own + index + head * 128, a.iqnorm, 128, rope, own + index + head * 128, values, sums, &total);
    } else if (row == 0) {
        float* history = a.blocks + a.pool * 128;
        const bool mine = column < 128;
        for (size_t r = 0; r < a.rows; ++r) {
            const size_t position = a.positions[r];
            if (position >= a.context) continue;   // (reported by the row's key blocks; the same for every thread)
            if (mine) history[(position % kHistory) * 128 + column] = a.projections[r * a.stride + index + 512 + column];
            if ((position + 1) % 4 == 0) {   // (the same for every thread: all of them pass the barriers)
                if (mine) {
                    float x = 0.0f;
                    for (size_t tap = 0; tap < 4; ++tap) x += history[((position - 3 + tap) % kHistory) * 128 + column];
                    x /= 4.0f;
                    values[column] = x * a.pool_norm[column];
                    sums[column] = x * x;
                }
                const float sum = halving_sum(sums, 128, column, &total);
                if (mine) {
                    const float denominator = sqrtf(sum / 128.0f + 1e-6f);
                    const float value = values[column] / denominator;
                    const float partner = column < 64 ? values[(column + 32) % 64] / denominator : 0.0f;
                    a.blocks[column * a.pool + position / 4] = rotate(value, partner, column, size_t(a.ropes[r]) - 3);
                }
            }
            __syncthreads();   // (the next row may overwrite `values`, and reads the history this row wrote)
        }
    }
}

}  // namespace
}  // namespace sdb

using namespace sdb;

// The rows' projections -> packed queries and keys, the K/V rows, normalised index queries (in place) and the pooled index blocks.
// All pointers are device pointers; positions and ropes hold `rows` values each (a row's K/V position and its rotation position:
// the same number unless the sequence holds images, gpu/qsa_decode.hpp:1-4). `index_state` is the indexer's state of one layer:
// [128][pool] pooled blocks, pool = context / 4 + 1, followed by the history ring of 16 x 128 (gpu/sparse_attention.hpp:462).
extern "C" int sdx_qsa_normalize_rows(void* handle, float* projections, uint64_t stride, uint64_t rows, uint64_t heads, uint64_t kv_heads,
                                      const float* qnorm, const float* knorm, const float* iqnorm, const float* pool_norm,
                                      const uint32_t* positions, const uint32_t* ropes, float* packed, uint64_t selected, void* state,
                                      uint64_t context, void* mirror, uint64_t mirror_rows, float* index_state) {
    SDB_OP_BEGIN
    if (value.kv_row != kv_row_q8) throw std::runtime_error("this Straydog build writes Q8_0 K/V rows only");
    if (!rows || rows > max_batch || !heads || !kv_heads || heads > 65535 || kv_heads > heads || !context || context > (uint64_t(1) << 24) ||
        stride < heads * 512 + kv_heads * 512 + 640 || (mirror_rows && !mirror) || mirror_rows > context)
        throw std::runtime_error("invalid Straydog attention dimensions");
    const uint64_t pool = context / 4 + 1;
    span(value, projections, checked_product({rows - 1, stride, 4}) + (heads * 512 + kv_heads * 512 + 640) * 4, "the rows' projections");
    span(value, qnorm, 256 * 4, "a query norm"); span(value, knorm, 256 * 4, "a key norm");
    span(value, iqnorm, 128 * 4, "an index-query norm"); span(value, pool_norm, 128 * 4, "an index-key norm");
    span(value, positions, rows * 4, "row positions"); span(value, ropes, rows * 4, "rotation positions");
    span(value, packed, checked_product({rows, heads * 256 + kv_heads * 512 + selected + 1, 4}), "packed attention rows");
    span(value, state, checked_product({context, 2 * kv_heads, kv_row_q8}), "a K/V state");
    if (mirror_rows) span(value, mirror, checked_product({mirror_rows, 2 * kv_heads, kv_row_q8}), "a K/V mirror");
    span(value, index_state, checked_product({pool + 16, 128, 4}), "an index state");
    NormalizeArgs a{};
    a.projections = projections; a.stride = stride; a.rows = rows; a.heads = heads; a.kv_heads = kv_heads;
    a.qnorm = qnorm; a.knorm = knorm; a.iqnorm = iqnorm; a.pool_norm = pool_norm; a.positions = positions; a.ropes = ropes;
    a.packed = packed; a.state = static_cast<uint8_t*>(state); a.context = context;
    a.mirror = static_cast<uint8_t*>(mirror); a.mirror_rows = mirror_rows; a.blocks = index_state; a.pool = pool; a.status = status_word(value);
    qsa_normalize_rows_kernel<<<dim3(unsigned(heads + kv_heads + 5), unsigned(rows)), 256, 0, value.stream>>>(a);
    ++value.launches;
    SDB_OP_END
}
