// Causal prompt attention over a Q8_0 K/V state (sdx_qsa_prompt): a chunk of `rows` new tokens at
// positions first .. first + rows - 1 attends every cached position up to its own.
//
// What it replaces in the reference: qsa_flash / qsa_flash_wide (FP32, gpu/sparse_attention_compute.hpp:177-415)
// and qsa_flash_mma (mma.sync per token, :416-584) behind qsa_flash_launch (:589-608), in their dense
// causal form. The reference walks one token per block, so sixteen neighbouring tokens that share
// almost all their keys each read and dequantise them again; here a CTA takes a block of query rows
// for all the query heads of one K/V head (128 M-rows: 16 rows x 8 heads, 32 x 4, ...) and every 64-key
// tile is fetched and dequantised once for all of them.
//
// Pipeline per CTA (8 warps): raw Q8_0 tiles (64 K rows + 64 V rows, 2 x 17408 contiguous bytes) arrive
// by bulk copies (TMA engine) into a two-slot ring, one tile ahead of the math; all warps turn a raw
// tile into FP16 tiles in shared memory: value = FP16(int8 * scale), the single rounding the reference's
// own tensor-core kernel applies (kv_half4, gpu/kernels.cpp:46-54); then each warp runs S = Q K^T and
// O += P V for its 16 M-rows on mma.sync.m16n8k16 (FP16 operands, FP32 accumulation) with ldmatrix
// operands from padded, conflict-free rows, online softmax in the exp2 domain.
#include "common.cuh"
#include "../../include/straydog_gpu_b200.h"

#include <cstdlib>

namespace sdb {

void launch_prompt_tc(Device& d, const uint8_t* state, size_t context, size_t first, size_t rows, size_t heads, size_t kv_heads,
                      float scale, const void* q, float* out);

constexpr int kPromptKeys = 64;                    // keys a tile
constexpr int kPromptRow = (256 + 8) * 2;          // padded FP16 row in shared memory: 528 bytes
constexpr int kPromptRaw = kPromptKeys * int(kv_row_q8);   // one plane's raw tile: 17408 bytes
constexpr size_t kPromptSmem = size_t(128) * kPromptRow      // Q: 128 M-rows
                             + size_t(2) * kPromptKeys * kPromptRow   // K and V tiles as FP16
                             + size_t(2) * 2 * kPromptRaw            // two slots of raw K rows + raw V rows
                             + 64;

struct PromptArgs {
    const uint8_t* keys;      // this state's key planes: plane stride context * 272
    const uint8_t* values;
    size_t context, first, rows, heads, kv_heads, group;
    const __half* q;
    float* out;
    float scale_log2;
    int* status;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}

__global__ void __launch_bounds__(256, 1) qsa_prompt_kernel(const PromptArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* qs = smem;
    uint8_t* ks = qs + 128 * kPromptRow;
    uint8_t* vs = ks + kPromptKeys * kPromptRow;
    uint8_t* raw = vs + kPromptKeys * kPromptRow;
    uint64_t* full = reinterpret_cast<uint64_t*>(raw + 2 * 2 * kPromptRaw);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane / 4, t = lane % 4;
    const size_t rows_per_block = 16 * (8 / a.group);
    // longest blocks first: the last row blocks see the most keys
    const size_t blocks = (a.rows + rows_per_block - 1) / rows_per_block;
    const size_t block = blocks - 1 - blockIdx.x, kv = blockIdx.y;
    const size_t r0 = block * rows_per_block;
    const size_t head = kv * a.group + warp % a.group;          // this warp's query head
    const size_t warp_row0 = r0 + 16 * (warp / a.group);        // and its 16 rows

    if (threadIdx.x == 0) { mbar_init(&full[0], 1); mbar_init(&full[1], 1); }
    fence_barrier_init();

    // Q: warp's 16 rows x 256 columns into its 16 shared rows (zero past the chunk)
    for (int i = lane; i < 16 * 32; i += 32) {
        const int r = i / 32, piece = i % 32;
        const size_t row = warp_row0 + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < a.rows) v = *reinterpret_cast<const uint4*>(a.q + (row * a.heads + head) * 256 + piece * 8);
        *reinterpret_cast<uint4*>(qs + (warp * 16 + r) * kPromptRow + piece * 16) = v;
    }
    __syncthreads();

    const size_t last_row = min(a.rows, r0 + rows_per_block) - 1;
    const size_t keys_total = min(a.context, a.first + last_row + 1);
    const uint32_t tiles = uint32_t((keys_total + kPromptKeys - 1) / kPromptKeys);
    const uint8_t* key_plane = a.keys + kv * a.context * kv_row_q8;
    const uint8_t* value_plane = a.values + kv * a.context * kv_row_q8;

    auto fetch = [&](uint32_t tile) {   // thread 0
        const size_t begin = size_t(tile) * kPromptKeys;
        const uint32_t count = uint32_t(min(size_t(kPromptKeys), keys_total - begin)), bytes = count * kv_row_q8;
        uint8_t* slot = raw + (tile & 1) * 2 * kPromptRaw;
        mbar_expect_tx(&full[tile & 1], 2 * bytes);
        bulk_g2s(slot, key_plane + begin * kv_row_q8, bytes, &full[tile & 1]);
        bulk_g2s(slot + kPromptRaw, value_plane + begin * kv_row_q8, bytes, &full[tile & 1]);
    };
    if (threadIdx.x == 0) fetch(0);

    float o[32][4];
    #pragma unroll
    for (int n = 0; n < 32; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    // positions this thread's two rows may see
    const long long limit0 = warp_row0 + g < a.rows ? (long long)(a.first + warp_row0 + g) : -1;
    const long long limit1 = warp_row0 + g + 8 < a.rows ? (long long)(a.first + warp_row0 + g + 8) : -1;

    for (uint32_t tile = 0; tile < tiles; ++tile) {
        const size_t begin = size_t(tile) * kPromptKeys;
        const uint32_t count = uint32_t(min(size_t(kPromptKeys), keys_total - begin));
        if (!mbar_wait(&full[tile & 1], (tile >> 1) & 1)) { if (threadIdx.x == 0) atomicExch(a.status, 1); drain_delay(); return; }
        __syncthreads();   // every warp is done with the FP16 tiles of the previous step (and with the other raw slot)
        if (threadIdx.x == 0 && tile + 1 < tiles) fetch(tile + 1);
        // ---- raw Q8_0 -> FP16 tiles: a thread takes 16 consecutive columns of a row at a time ----
        {
            const uint8_t* slot = raw + (tile & 1) * 2 * kPromptRaw;
            for (int i = threadIdx.x; i < 2 * kPromptKeys * 16; i += 256) {
                const int plane = i / (kPromptKeys * 16), r = (i / 16) % kPromptKeys, piece = i % 16;
                uint8_t* dst = (plane ? vs : ks) + r * kPromptRow + piece * 32;
                if (uint32_t(r) >= count) {   // rows past the last key: zeros, so that a zero weight never meets stale bits
                    reinterpret_cast<uint4*>(dst)[0] = make_uint4(0, 0, 0, 0);
                    reinterpret_cast<uint4*>(dst)[1] = make_uint4(0, 0, 0, 0);
                    continue;
                }
                const uint8_t* src = slot + plane * kPromptRaw + r * kv_row_q8;
                const uint4 bytes = *reinterpret_cast<const uint4*>(src + piece * 16);
                const __half scale_h = reinterpret_cast<const __half*>(src + 256)[piece / 2];
                const __half2 scale2 = __halves2half2(scale_h, scale_h);
                const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));   // 1152
                const uint32_t words[4] = {bytes.x ^ 0x80808080u, bytes.y ^ 0x80808080u, bytes.z ^ 0x80808080u, bytes.w ^ 0x80808080u};
                uint32_t halves[8];
                #pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t lo = prmt(words[w], 0x64646464u, 0x4140u), hi = prmt(words[w], 0x64646464u, 0x4342u);
                    const __half2 a0 = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&lo), bias), scale2);
                    const __half2 a1 = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&hi), bias), scale2);
                    halves[2 * w] = *reinterpret_cast<const uint32_t*>(&a0);
                    halves[2 * w + 1] = *reinterpret_cast<const uint32_t*>(&a1);
                }
                reinterpret_cast<uint4*>(dst)[0] = make_uint4(halves[0], halves[1], halves[2], halves[3]);
                reinterpret_cast<uint4*>(dst)[1] = make_uint4(halves[4], halves[5], halves[6], halves[7]);
            }
        }
        __syncthreads();

        // ---- S = Q K^T for this warp's 16 rows x 64 keys ----
        float s[8][4];
        #pragma unroll
        for (int j = 0; j < 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
        const int a_row = lane % 16, a_half = lane / 16;                      // A operand: rows 0..15, column halves
        const int b_row = 8 * (lane / 16) + lane % 8, b_half = (lane / 8) % 2;   // B operand: two n-tiles x two column halves
        #pragma unroll 4
        for (int kk = 0; kk < 16; ++kk) {
            uint32_t af[4];
            ldsm_x4(af, qs + (warp * 16 + a_row) * kPromptRow + (16 * kk + 8 * a_half) * 2);
            #pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                uint32_t b[4];
                ldsm_x4(b, ks + (16 * jp + b_row) * kPromptRow + (16 * kk + 8 * b_half) * 2);
                mma_f16(s[2 * jp], af, b[0], b[1]);
                mma_f16(s[2 * jp + 1], af, b[2], b[3]);
            }
        }
        // ---- causal mask and online softmax ----
        const bool edge = (long long)(begin + kPromptKeys - 1) > (long long)(a.first + warp_row0) || count < uint32_t(kPromptKeys);
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            #pragma unroll
            for (int c = 0; c < 4; ++c) {
                float x = s[j][c] * a.scale_log2;
                if (edge) {
                    const long long position = (long long)begin + 8 * j + 2 * t + (c & 1);
                    if (position > (c < 2 ? limit0 : limit1)) x = -INFINITY;
                }
                s[j][c] = x;
            }
        }
        float top[2] = {-INFINITY, -INFINITY};
        #pragma unroll
        for (int j = 0; j < 8; ++j) { top[0] = fmaxf(top[0], fmaxf(s[j][0], s[j][1])); top[1] = fmaxf(top[1], fmaxf(s[j][2], s[j][3])); }
        #pragma unroll
        for (int i = 0; i < 2; ++i) {
            top[i] = fmaxf(top[i], __shfl_xor_sync(0xffffffffu, top[i], 1));
            top[i] = fmaxf(top[i], __shfl_xor_sync(0xffffffffu, top[i], 2));
        }
        const float n0 = fmaxf(m[0], top[0]), n1 = fmaxf(m[1], top[1]);
        if (__any_sync(0xffffffffu, n0 > m[0] || n1 > m[1])) {
            const float f0 = m[0] == -INFINITY ? 0.0f : fast_exp2(m[0] - n0), f1 = m[1] == -INFINITY ? 0.0f : fast_exp2(m[1] - n1);
            l[0] *= f0; l[1] *= f1;
            #pragma unroll
            for (int n = 0; n < 32; ++n) { o[n][0] *= f0; o[n][1] *= f0; o[n][2] *= f1; o[n][3] *= f1; }
            m[0] = n0; m[1] = n1;
        }
        const float u0 = m[0] == -INFINITY ? 0.0f : m[0], u1 = m[1] == -INFINITY ? 0.0f : m[1];
        uint32_t pa[4][4];
        #pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p0 = fast_exp2(s[j][0] - u0), p1 = fast_exp2(s[j][1] - u0), p2 = fast_exp2(s[j][2] - u1), p3 = fast_exp2(s[j][3] - u1);
            const uint32_t p01 = pack_half2(p0, p1), p23 = pack_half2(p2, p3);
            // the denominator sums the weights as the tensor cores see them (rounded to FP16)
            const float2 r01 = __half22float2(*reinterpret_cast<const __half2*>(&p01)), r23 = __half22float2(*reinterpret_cast<const __half2*>(&p23));
            l[0] += r01.x + r01.y; l[1] += r23.x + r23.y;
            pa[j / 2][(j & 1) * 2] = p01;
            pa[j / 2][(j & 1) * 2 + 1] = p23;
        }
        // ---- O += P V ----
        const int v_key = 8 * ((lane / 8) % 2) + lane % 8, v_dim = 8 * (lane / 16);
        #pragma unroll
        for (int kk2 = 0; kk2 < 4; ++kk2) {
            #pragma unroll
            for (int np = 0; np < 16; ++np) {
                uint32_t b[4];
                ldsm_x4_trans(b, vs + (16 * kk2 + v_key) * kPromptRow + (16 * np + v_dim) * 2);
                mma_f16(o[2 * np], pa[kk2], b[0], b[1]);
                mma_f16(o[2 * np + 1], pa[kk2], b[2], b[3]);
            }
        }
    }
    // ---- normalise and store ----
    #pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    #pragma unroll
    for (int i = 0; i < 2; ++i) {
        const size_t row = warp_row0 + g + 8 * i;
        if (row >= a.rows) continue;
        const float inverse = 1.0f / l[i];
        float* mine = a.out + (row * a.heads + head) * 256;
        #pragma unroll
        for (int n = 0; n < 32; ++n)
            *reinterpret_cast<float2*>(mine + 8 * n + 2 * t) = make_float2(o[n][2 * i] * inverse, o[n][2 * i + 1] * inverse);
    }
}

}  // namespace sdb

using namespace sdb;

extern "C" int sdx_qsa_prompt(void* handle, const void* state, uint64_t context, uint64_t first, uint64_t rows, uint64_t heads,
                              uint64_t kv_heads, float scale, const void* q, float* out) {
    SDB_OP_BEGIN
    if (value.kv_row != kv_row_q8) throw std::runtime_error("this Straydog build's attention reads Q8_0 K/V rows only");
    const uint64_t group = kv_heads ? heads / kv_heads : 0;
    if (!context || context > (uint64_t(1) << 24) || !rows || first > context || rows > context - first || !heads || !kv_heads ||
        heads % kv_heads || (group != 1 && group != 2 && group != 4 && group != 8) || kv_heads > 65535)
        throw std::runtime_error("invalid Straydog attention dimensions");
    span(value, state, checked_product({context, 2 * kv_heads, kv_row_q8}), "a K/V state");
    span(value, q, checked_product({rows, heads, 256, 2}), "attention queries");
    span(value, out, checked_product({rows, heads, 256, 4}), "an attention output");
    if (reinterpret_cast<uintptr_t>(state) % 16 || reinterpret_cast<uintptr_t>(q) % 16 || reinterpret_cast<uintptr_t>(out) % 8)
        throw std::runtime_error("Straydog prompt attention operands must be 16-byte aligned");
    // The tcgen05/TMEM kernel is the default; SDX_PROMPT_KERNEL=mma (read at each call) selects the mma.sync kernel for A/B runs.
    const char* choice = std::getenv("SDX_PROMPT_KERNEL");
    if (!(choice && std::string(choice) == "mma")) {
        launch_prompt_tc(value, static_cast<const uint8_t*>(state), context, first, rows, heads, kv_heads, scale, q, out);
        SDB_CHECK(cudaGetLastError());
        return 0;
    }
    static bool configured[64] = {};
    if (!configured[value.ordinal & 63]) {
        SDB_CHECK(cudaFuncSetAttribute(qsa_prompt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPromptSmem)));
        configured[value.ordinal & 63] = true;
    }
    PromptArgs args{};
    args.keys = static_cast<const uint8_t*>(state);
    args.values = args.keys + kv_heads * context * kv_row_q8;
    args.context = context; args.first = first; args.rows = rows; args.heads = heads; args.kv_heads = kv_heads; args.group = group;
    args.q = static_cast<const __half*>(q);
    args.out = out;
    args.scale_log2 = scale * 1.4426950408889634f;
    args.status = status_word(value);
    const size_t rows_per_block = 16 * (8 / group);
    const dim3 grid{unsigned((rows + rows_per_block - 1) / rows_per_block), unsigned(kv_heads)};
    qsa_prompt_kernel<<<grid, 256, kPromptSmem, value.stream>>>(args);
    ++value.launches;
    SDB_OP_END
}
