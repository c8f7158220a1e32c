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
// sdx_qsa_normalize_chunk is the same front for a prompt chunk (gpu/prefill_batch.hpp:342-370, gpu/sparse_attention.hpp:87-106, 135-139,
// 493-506: qsa_normalize x 3, the values' copy, qsa_pool, qsa_save_history, write_attention_kv): `count` consecutive tokens from
// `position`, their five projections in arrays of their own; the per-token blocks are the same, the pooling is a second small launch
// (a block of 128 threads per completed 4-position block, all at once: only the chunk's first block reaches back into the ring).
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
    // the rows' five projections, each with its own distance between rows (one array and one stride for decode rows)
    const float* qgate; size_t qgate_stride;
    const float* key; size_t key_stride;
    const float* value; size_t value_stride;
    float* iq; size_t iq_stride;
    const float* ik; size_t ik_stride;
    size_t rows, heads, kv_heads;
    size_t base;              // positions == null: row r sits and turns at base + r (a prompt chunk)
    bool copy_values;         // a prompt chunk's values also go into the packed rows (gpu/sparse_attention.hpp:495)
    const float* qnorm; const float* knorm; const float* iqnorm; const float* pool_norm;
    const uint32_t* positions; const uint32_t* ropes;
    const uint32_t* axes; size_t axes_first;   // a prompt chunk of a sequence with images: three rotation positions (t, h, w) a position from axes_first
    float* packed;
    uint8_t* state; size_t context; unsigned kv_row;
    uint8_t* mirror; size_t mirror_rows;
    float* blocks; size_t pool;   // [128][pool], then the history ring [16][128]
    int* status;
};

// gpu/sparse_attention.hpp:2-6 (qsa_rope), and :27-32 (qsa_rope_axes) with `axes`: pair p of the 32 turns by the position of axis p % 3
// (text holds one position on all three axes, which is the first form's angle)
__device__ __forceinline__ float rotate(float own, float partner, size_t column, size_t position, const uint32_t* axes = nullptr) {
    if (column >= 64) return own;
    const size_t pair = column % 32;
    const float angle = float(axes ? size_t(axes[pair % 3]) : position) / powf(1e7f, float(pair) / 32.0f);
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
                                                float* values, float* sums, float* total, const uint32_t* axes = nullptr) {
    const size_t column = threadIdx.x;
    const bool own = column < width;
    if (own) { const float x = source[column]; values[column] = x * norm[column]; sums[column] = x * x; }
    const float sum = halving_sum(sums, width, column, total);
    if (!own) return 0.0f;
    const float denominator = sqrtf(sum / float(width) + 1e-6f);
    const float mine = values[column] / denominator;
    const float partner = column < 64 ? values[(column + 32) % 64] / denominator : 0.0f;
    const float result = rotate(mine, partner, column, position, axes);
    target[column] = result;
    return result;
}

__global__ void __launch_bounds__(256) qsa_normalize_rows_kernel(const NormalizeArgs a) {
    __shared__ float values[256], sums[256], total;
    const size_t block = blockIdx.x, row = blockIdx.y, column = threadIdx.x;
    const size_t rope = a.positions ? a.ropes[row] : a.base + row;
    const uint32_t* axes = a.axes ? a.axes + (a.base + row - a.axes_first) * 3 : nullptr;   // (a prompt chunk's rows only)
    if (block < a.heads) {
        normalize_head(a.qgate + row * a.qgate_stride + block * 512, a.qnorm, 256, rope, a.packed + (row * a.heads + block) * 256, values, sums, &total, axes);
    } else if (block < a.heads + a.kv_heads) {
        const size_t head = block - a.heads, position = a.positions ? a.positions[row] : a.base + row;
        if (position >= a.context) {   // (a position past the state: nothing of the row is written, and the host is told)
            if (column == 0) atomicExch(a.status, 5);
            return;
        }
        float* normalized = a.packed + a.rows * a.heads * 256 + (row * a.kv_heads + head) * 256;
        const float key = normalize_head(a.key + row * a.key_stride + head * 256, a.knorm, 256, rope, normalized, values, sums, &total, axes);
        const float value = a.value[row * a.value_stride + head * 256 + column];
        if (a.copy_values) a.packed[a.rows * (a.heads + a.kv_heads) * 256 + (row * a.kv_heads + head) * 256 + column] = value;
        __half key_scale, value_scale;
        const int8_t k8 = q8_encode(key, key_scale), v8 = q8_encode(value, value_scale);
        auto put = [&](uint8_t* planes, size_t rows_of_plane, size_t at) {
            uint8_t* k_row = planes + (head * rows_of_plane + at) * a.kv_row;
            uint8_t* v_row = planes + ((a.kv_heads + head) * rows_of_plane + at) * a.kv_row;
            if (a.kv_row == kv_row_f16) {   // FP16 rows: the nearest FP16 of each value (gpu/kernels.cpp:70)
                reinterpret_cast<__half*>(k_row)[column] = __float2half_rn(key);
                reinterpret_cast<__half*>(v_row)[column] = __float2half_rn(value);
                return;
            }
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
        float* mine = a.iq + row * a.iq_stride + head * 128;
        normalize_head(mine, a.iqnorm, 128, rope, mine, values, sums, &total, axes);
    } else if (row == 0) {
        float* history = a.blocks + a.pool * 128;
        const bool mine = column < 128;
        for (size_t r = 0; r < a.rows; ++r) {
            const size_t position = a.positions[r];
            if (position >= a.context) continue;   // (reported by the row's key blocks; the same for every thread)
            if (mine) history[(position % kHistory) * 128 + column] = a.ik[r * a.ik_stride + column];
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

// A prompt chunk's pooling (gpu/sparse_attention.hpp:87-106 qsa_pool, 135-139 qsa_save_history): block b of the grid pools the b-th
// 4-position block the chunk completes, positions before the chunk from the ring, the rest from the chunk's own index keys. Only the
// first completed block reads the ring, and the ring's new entries (the chunk's last four tokens at most) may land on the slots it
// reads: the grid's block 0 pools it, then, behind a barrier, saves the history. With no block completed block 0 only saves.
__global__ void __launch_bounds__(128) qsa_pool_chunk_kernel(const NormalizeArgs a, size_t completed) {
    __shared__ float values[128], sums[128], total;
    const size_t column = threadIdx.x;
    float* history = a.blocks + a.pool * 128;
    if (blockIdx.x < completed) {
        const size_t block = a.base / 4 + blockIdx.x, begin = block * 4;
        float x = 0.0f;
        for (size_t tap = 0; tap < 4; ++tap) {
            const size_t position = begin + tap;
            x += position < a.base ? history[(position % kHistory) * 128 + column] : a.ik[(position - a.base) * a.ik_stride + column];
        }
        x /= 4.0f;
        values[column] = x * a.pool_norm[column];
        sums[column] = x * x;
        const float sum = halving_sum(sums, 128, column, &total);
        const float denominator = sqrtf(sum / 128.0f + 1e-6f);
        const float value = values[column] / denominator;
        const float partner = column < 64 ? values[(column + 32) % 64] / denominator : 0.0f;
        a.blocks[column * a.pool + block] = rotate(value, partner, column, begin, a.axes ? a.axes + (begin - a.axes_first) * 3 : nullptr);   // (:111-131 qsa_pool_axes)
    }
    if (blockIdx.x == 0) {
        __syncthreads();   // (the ring has been read)
        const size_t kept = a.rows < 4 ? a.rows : 4;
        for (size_t t = a.rows - kept; t < a.rows; ++t) history[((a.base + t) % kHistory) * 128 + column] = a.ik[t * a.ik_stride + column];
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
    if (!rows || rows > max_batch || !heads || !kv_heads || heads > 65535 || kv_heads > heads || !context || context > (uint64_t(1) << 24) ||
        stride < heads * 512 + kv_heads * 512 + 640 || (mirror_rows && !mirror) || mirror_rows > context)
        throw std::runtime_error("invalid Straydog attention dimensions");
    const uint64_t pool = context / 4 + 1;
    span(value, projections, checked_product({rows - 1, stride, 4}) + (heads * 512 + kv_heads * 512 + 640) * 4, "the rows' projections");
    span(value, qnorm, 256 * 4, "a query norm"); span(value, knorm, 256 * 4, "a key norm");
    span(value, iqnorm, 128 * 4, "an index-query norm"); span(value, pool_norm, 128 * 4, "an index-key norm");
    span(value, positions, rows * 4, "row positions"); span(value, ropes, rows * 4, "rotation positions");
    span(value, packed, checked_product({rows, heads * 256 + kv_heads * 512 + selected + 1, 4}), "packed attention rows");
    span(value, state, checked_product({context, 2 * kv_heads, value.kv_row}), "a K/V state");
    if (mirror_rows) span(value, mirror, checked_product({mirror_rows, 2 * kv_heads, value.kv_row}), "a K/V mirror");
    span(value, index_state, checked_product({pool + 16, 128, 4}), "an index state");
    NormalizeArgs a{};
    const size_t keys_at = heads * 512, values_at = keys_at + kv_heads * 256, index_at = keys_at + kv_heads * 512;
    a.qgate = projections; a.key = projections + keys_at; a.value = projections + values_at; a.iq = projections + index_at; a.ik = projections + index_at + 512;
    a.qgate_stride = a.key_stride = a.value_stride = a.iq_stride = a.ik_stride = stride;
    a.rows = rows; a.heads = heads; a.kv_heads = kv_heads;
    a.qnorm = qnorm; a.knorm = knorm; a.iqnorm = iqnorm; a.pool_norm = pool_norm; a.positions = positions; a.ropes = ropes;
    a.packed = packed; a.state = static_cast<uint8_t*>(state); a.context = context;
    a.mirror = static_cast<uint8_t*>(mirror); a.mirror_rows = mirror_rows; a.blocks = index_state; a.pool = pool; a.status = status_word(value); a.kv_row = value.kv_row;
    qsa_normalize_rows_kernel<<<dim3(unsigned(heads + kv_heads + 5), unsigned(rows)), 256, 0, value.stream>>>(a);
    ++value.launches;
    SDB_OP_END
}

// The same front for a prompt chunk: `count` consecutive tokens from `position` (a token's rotation position is its own), their
// projections in five arrays: qgate [count][heads][512], key and value [count][kv_heads][256], iq [count][4][128] (normalised in
// place), ik [count][128]. Also copies the values into the packed rows (the layout sd_attention_sequence reads).
extern "C" int sdx_qsa_normalize_chunk(void* handle, const float* qgate, const float* key, const float* value_rows, float* iq, const float* ik,
                                       uint64_t count, uint64_t position, uint64_t heads, uint64_t kv_heads, const float* qnorm,
                                       const float* knorm, const float* iqnorm, const float* pool_norm, float* packed, uint64_t selected,
                                       void* state, uint64_t context, void* mirror, uint64_t mirror_rows, float* index_state) {
    SDB_OP_BEGIN
    if (!count || count > 65535 || !heads || !kv_heads || heads > 65535 || kv_heads > heads || !context || context > (uint64_t(1) << 24) ||
        position > context || count > context - position || (mirror_rows && !mirror) || mirror_rows > context)
        throw std::runtime_error("invalid Straydog attention dimensions");
    const uint64_t pool = context / 4 + 1;
    span(value, qgate, checked_product({count, heads, 512, 4}), "query projections");
    span(value, key, checked_product({count, kv_heads, 256, 4}), "key projections");
    span(value, value_rows, checked_product({count, kv_heads, 256, 4}), "value projections");
    span(value, iq, checked_product({count, 512, 4}), "index queries");
    span(value, ik, checked_product({count, 128, 4}), "index keys");
    span(value, qnorm, 256 * 4, "a query norm"); span(value, knorm, 256 * 4, "a key norm");
    span(value, iqnorm, 128 * 4, "an index-query norm"); span(value, pool_norm, 128 * 4, "an index-key norm");
    span(value, packed, checked_product({count, heads * 256 + kv_heads * 512 + selected + 1, 4}), "packed attention rows");
    span(value, state, checked_product({context, 2 * kv_heads, value.kv_row}), "a K/V state");
    if (mirror_rows) span(value, mirror, checked_product({mirror_rows, 2 * kv_heads, value.kv_row}), "a K/V mirror");
    span(value, index_state, checked_product({pool + 16, 128, 4}), "an index state");
    NormalizeArgs a{};
    a.qgate = qgate; a.qgate_stride = heads * 512; a.key = key; a.key_stride = kv_heads * 256; a.value = value_rows; a.value_stride = kv_heads * 256;
    a.iq = iq; a.iq_stride = 512; a.ik = ik; a.ik_stride = 128;
    a.rows = count; a.heads = heads; a.kv_heads = kv_heads; a.base = position; a.copy_values = true;
    a.qnorm = qnorm; a.knorm = knorm; a.iqnorm = iqnorm; a.pool_norm = pool_norm;
    if (value.rope_count) {   // (gpu/prefill_batch.hpp:344, 360-362: the table covers the chunk's rows and the block its first row is in)
        const uint64_t first_read = (position + count) / 4 > position / 4 ? position / 4 * 4 : position;
        if (first_read < value.rope_first || position + count > value.rope_first + value.rope_count)
            throw std::runtime_error("invalid Straydog rope table");
        a.axes = value.rope_rows; a.axes_first = value.rope_first;
    }
    a.packed = packed; a.state = static_cast<uint8_t*>(state); a.context = context;
    a.mirror = static_cast<uint8_t*>(mirror); a.mirror_rows = mirror_rows; a.blocks = index_state; a.pool = pool; a.status = status_word(value); a.kv_row = value.kv_row;
    qsa_normalize_rows_kernel<<<dim3(unsigned(heads + kv_heads + 4), unsigned(count)), 256, 0, value.stream>>>(a);
    const uint64_t completed = (position + count) / 4 - position / 4;
    qsa_pool_chunk_kernel<<<unsigned(std::max<uint64_t>(completed, 1)), 128, 0, value.stream>>>(a, completed);
    value.launches += 2;
    SDB_OP_END
}

// gpu/straydog_gpu.h:607-609, gpu/kernels.cpp:1526-1536. The rope positions of a sequence with images for the next prompt chunks:
// three (t, h, w) a position from `first`, `count` positions (a host array), covering each chunk's rows and the block its first
// row is in; count 0: the rows' own positions again. sdx_qsa_normalize_chunk turns by the table while one is set.
extern "C" int sd_rope_rows(void* handle, uint64_t first, uint64_t count, const uint32_t* axes) {
    SDB_OP_BEGIN
    constexpr size_t most = 4096 + 4;
    if (count > most || (count && !axes)) throw std::runtime_error("invalid Straydog rope table");
    if (count && !value.rope_rows) SDB_CHECK(cudaMalloc(reinterpret_cast<void**>(&value.rope_rows), most * 3 * 4));
    if (count) {
        SDB_CHECK(cudaMemcpyAsync(value.rope_rows, axes, size_t(count) * 3 * 4, cudaMemcpyHostToDevice, value.stream));
        SDB_CHECK(cudaStreamSynchronize(value.stream));   // (the host array is the caller's again on return)
    }
    value.rope_first = size_t(first); value.rope_count = size_t(count);
    SDB_OP_END
}
