// Qwen's indexer, the producer of the selection lists sdx_qsa_attention_rows consumes: block scores and the exact choice of the 512
// best 4-position blocks of every row, written into the packed rows in the reference's layout.
//
// What it replaces in the reference: qsa_block_scores / qsa_block_scores_tiled (gpu/sparse_attention.hpp:141-157, 247-296) and
// qsa_select / qsa_select_rows (:172-243, 307-395) as qsa_index_exact launches them (:398-410). The reference reaches them only from
// inside sd_qsa_sequence and its spans, so there is no entry of its library to hold this one to: parity here rests on the oracle's
// restatement of those lines (bit for bit: the scores are chains of fused multiply-adds in column order, the choice is integer work).
//
// Contract kept: a row at position p has complete = (p + 1) / 4 whole blocks. Up to 512 of them: every position 0 .. p is selected, in
// order. More: score(block) = sum over the four index heads of max(0, sum_col key[col][block] * query[head][col]) (each dot one chain
// of fused multiply-adds over the 128 columns in order, the four terms added in head order); the 512 blocks of highest score are
// kept, equal scores by lowest block, listed in block order, four positions each; then the positions of the incomplete block,
// 4 * complete .. p; the count is 2048 + (p + 1 - 4 * complete).
//
// Here: one scores kernel for any number of rows (a thread owns a block and four rows' four running dots, so a key column value is
// loaded once for 16 fused multiply-adds; the rows' queries sit in shared memory, a column's 32 values side by side), then the library's top-k kernel (two reads of a
// row, ties by lowest index, ascending output: the same rule), which writes the chosen blocks into the packed rows as positions itself.
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

namespace sdb {

void launch_top_k(Device& d, const float* scores, size_t rows, size_t groups, size_t k, int32_t* out, const int32_t* candidates, size_t blocks, size_t block,
                  bool dependent, const TopKExpand* expand);

constexpr int kIndexRows = 8, kIndexBlocks = 64, kIndexKeep = 512, kIndexOwn = 4;

// grid (ceil(pool / 64), ceil(steps / 8)), 128 threads; scores [steps][pool], -inf from a row's first incomplete block on. A thread owns
// a block and four of the CTA's eight rows. Its 128 key column values are all asked for before the first is used (a row's pooled keys are
// read once a step, from memory: loads issued a few at a time left the kernel waiting on memory one batch after the other), and a
// column's 16 query values (4 rows x 4 heads) are four 16-byte shared-memory reads.
__global__ void __launch_bounds__(2 * kIndexBlocks) qsa_block_scores_kernel(const float* __restrict__ queries, size_t query_stride, const float* __restrict__ blocks,
                                                                            size_t pool, size_t base, const uint32_t* __restrict__ positions, size_t steps,
                                                                            float* __restrict__ scores) {
    __shared__ __align__(16) float q[128][kIndexRows * 4];   // [column][row * 4 + head]
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // (the choice queued behind this kernel waits for its end before it reads the scores)
    const int t = threadIdx.x % kIndexBlocks, part = threadIdx.x / kIndexBlocks;   // (a warp is of one part: its query reads are broadcasts)
    const size_t row0 = size_t(blockIdx.y) * kIndexRows, block = size_t(blockIdx.x) * kIndexBlocks + t;
    const int rows = int(min(size_t(kIndexRows), steps - row0));
    size_t most = 0;   // the most whole blocks a row of this CTA has
    for (int r = 0; r < rows; ++r) most = max(most, (size_t(positions ? positions[row0 + r] : base + row0 + r) + 1) / 4);
    const bool wanted = most > size_t(kIndexKeep) && size_t(blockIdx.x) * kIndexBlocks < most;
    const bool mine = wanted && block < pool && part * kIndexOwn < rows;
    float key[128];
    if (mine) {
        #pragma unroll
        for (int col = 0; col < 128; ++col) key[col] = blocks[size_t(col) * pool + block];
    }
    if (wanted) {
        // (a lane a (row, head), four columns a load: all of a thread's loads are in flight at once, and the stores fall on 32 banks)
        constexpr int kEach = 128 * kIndexRows / (2 * kIndexBlocks);
        if (reinterpret_cast<uintptr_t>(queries) % 16 == 0 && query_stride % 4 == 0) {
            float4 got[kEach];
            #pragma unroll
            for (int n = 0; n < kEach; ++n) {
                const int i = n * 2 * kIndexBlocks + threadIdx.x, four = i / (kIndexRows * 4), r = i % (kIndexRows * 4) / 4, h = i % 4;
                got[n] = r < rows ? __ldg(reinterpret_cast<const float4*>(queries + (row0 + r) * query_stride + h * 128 + 4 * four)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
            #pragma unroll
            for (int n = 0; n < kEach; ++n) {
                const int i = n * 2 * kIndexBlocks + threadIdx.x, four = i / (kIndexRows * 4), rh = i % (kIndexRows * 4);
                q[4 * four][rh] = got[n].x; q[4 * four + 1][rh] = got[n].y; q[4 * four + 2][rh] = got[n].z; q[4 * four + 3][rh] = got[n].w;
            }
        } else {
            for (int i = threadIdx.x; i < 128 * kIndexRows * 4; i += 2 * kIndexBlocks) {
                const int col = i / (kIndexRows * 4), r = i % (kIndexRows * 4) / 4, h = i % 4;
                q[col][r * 4 + h] = r < rows ? queries[(row0 + r) * query_stride + h * 128 + col] : 0.0f;
            }
        }
    }
    __syncthreads();
    float acc[kIndexOwn][4];
    #pragma unroll
    for (int r = 0; r < kIndexOwn; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.0f;
    if (mine) {
        #pragma unroll
        for (int col = 0; col < 128; ++col)
            #pragma unroll
            for (int r = 0; r < kIndexOwn; ++r) {
                const float4 x = *reinterpret_cast<const float4*>(&q[col][4 * (part * kIndexOwn + r)]);
                acc[r][0] = fmaf(key[col], x.x, acc[r][0]); acc[r][1] = fmaf(key[col], x.y, acc[r][1]);
                acc[r][2] = fmaf(key[col], x.z, acc[r][2]); acc[r][3] = fmaf(key[col], x.w, acc[r][3]);
            }
    }
    if (block >= pool) return;
    #pragma unroll
    for (int r = 0; r < kIndexOwn; ++r) {
        const int row = part * kIndexOwn + r;
        if (row >= rows) break;
        const size_t complete = (size_t(positions ? positions[row0 + row] : base + row0 + row) + 1) / 4;
        const float score = __fadd_rn(__fadd_rn(__fadd_rn(fmaxf(acc[r][0], 0.0f), fmaxf(acc[r][1], 0.0f)), fmaxf(acc[r][2], 0.0f)), fmaxf(acc[r][3], 0.0f));
        scores[(row0 + row) * pool + block] = complete > size_t(kIndexKeep) && block < complete ? score : -INFINITY;
    }
}

}  // namespace sdb

using namespace sdb;

extern "C" int sdx_qsa_index_select(void* handle, const float* queries, uint64_t query_stride, const float* blocks, uint64_t pool, uint64_t base,
                                    const uint32_t* positions, uint64_t steps, uint64_t selected, uint64_t heads, uint64_t kv_heads, float* packed) {
    SDB_OP_BEGIN
    if (!steps || steps > 65535 || !pool || pool > (uint64_t(1) << 22) || query_stride < 512 || selected < 2052 || selected > 8192 || !heads || !kv_heads ||
        (!positions && (base + steps - 1) / 4 >= pool))
        throw std::runtime_error("invalid Straydog indexer dimensions");
    const size_t row_floats = heads * 256 + kv_heads * 512;
    span(value, queries, checked_product({steps - 1, query_stride, 4}) + 512 * 4, "index queries");
    span(value, blocks, checked_product({128, pool, 4}), "pooled index keys");
    span(value, packed, checked_product({steps, row_floats + selected + 1, 4}), "packed attention rows");
    if (positions) span(value, positions, steps * 4, "attention positions");
    // scores [steps][pool]: a library-owned workspace (make the first call of a size outside a capture)
    auto* scores = static_cast<float*>(ensure(value, value.work, value.work_bytes, checked_product({steps, pool, 4})));
    qsa_block_scores_kernel<<<dim3(unsigned((pool + kIndexBlocks - 1) / kIndexBlocks), unsigned((steps + kIndexRows - 1) / kIndexRows)), 2 * kIndexBlocks, 0, value.stream>>>(
        queries, size_t(query_stride), blocks, size_t(pool), size_t(base), positions, size_t(steps), scores);
    ++value.launches;
    SDB_CHECK(cudaGetLastError());
    // (the choice as a programmatic dependent of the scores: placed while they drain; it writes the rows' lists itself)
    TopKExpand expand{};
    expand.packed = packed; expand.index_start = size_t(steps) * row_floats; expand.selected = size_t(selected); expand.steps = size_t(steps);
    expand.base = size_t(base); expand.positions = positions; expand.keep = uint32_t(kIndexKeep);
    launch_top_k(value, scores, size_t(steps), size_t(pool), size_t(kIndexKeep), nullptr, nullptr, 0, 1, true, &expand);
    SDB_OP_END
}
