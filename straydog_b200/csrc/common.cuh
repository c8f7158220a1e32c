// Shared host-side state and device-side primitives of the B200 attention library.
// One Device per sd_create handle: its stream, its allocation map (every op range-checks its
// pointers against it, as the reference's op_span does: gpu/ops.hpp:8-26) and lazily made scratch.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <initializer_list>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace sdb {

constexpr unsigned kv_row_f16 = 512, kv_row_q8 = 272;   // gpu/core.hpp:403
constexpr size_t max_batch = 256;                        // gpu/core.hpp:178
constexpr size_t allocation_tail = 64;                   // gpu/core.hpp:211

extern thread_local std::string last_error;

inline void check_at(cudaError_t error, const char* file, int line) {
    if (error == cudaSuccess) return;
    const std::string path(file);
    const char* text = cudaGetErrorString(error);
    throw std::runtime_error(std::string(text ? text : "GPU error") + " (" + path.substr(path.find_last_of("/\\") + 1) + ":" +
                             std::to_string(line) + ", code " + std::to_string(int(error)) + ")");
}
#define SDB_CHECK(error) ::sdb::check_at((error), __FILE__, __LINE__)

struct DecodePlan;

// One (sequence, K/V head) of a decode batch: the work list's unit, also what a batched K/V append addresses.
struct Segment {
    const uint8_t* keys;    // plane base
    const uint8_t* values;
    uint32_t q_offset;      // (sequence * heads + kv_head * group) * 256, in query elements
    uint32_t first_piece, pieces, length;
};

struct Device {
    int ordinal = 0;
    int sms = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t side = nullptr; cudaEvent_t side_fork = nullptr, side_join = nullptr;   // a second stream for work that may run beside a kernel of `stream` (made on first use)
    uint64_t budget = 0, used = 0;
    unsigned kv_row = kv_row_q8;
    std::mutex mutex;
    std::map<const uint8_t*, size_t> allocations;   // base -> requested bytes
    std::map<const uint8_t*, void*> host_states;    // device pointer -> the page-locked host allocation behind it (sd_host_state)
    std::map<const uint8_t*, size_t> peers;         // base -> bytes of other processes' allocations mapped by sdx_ipc_open
    // staging for host-pointer entries (page-locked) and device-side workspaces, grown on demand
    void* pinned = nullptr; size_t pinned_bytes = 0;
    void* work = nullptr; size_t work_bytes = 0;        // packed inputs / outputs of host-pointer entries
    void* partial = nullptr; size_t partial_bytes = 0;  // split partials of the decode kernels
    void* tables = nullptr; size_t tables_bytes = 0;    // work lists of the decode kernels
    std::shared_ptr<void> batch_cache;                  // sdx_attention_batch's last work list, kept while the batch keeps its tile counts
    void* unions = nullptr; size_t unions_bytes = 0;    // places and blocks of a gathered selection union, the renumbered rows
    long long* trace = nullptr; size_t trace_ctas = 0;   // -DSDX_TRACE builds: the last traced launch's counters
    bool fixed_cuts = false;                            // the decode work list's cuts (sdx_decode_cuts)
    double* turns = nullptr; size_t turns_rows = 0, turns_pairs = 0;   // rope sincos table (forward, inverse)
    bool turns_ready = false; size_t turns_ready_rows = 0, turns_ready_pairs = 0;
    void* kv_stage = nullptr; uint64_t kv_stage_rows = 0;
    uint32_t* rope_rows = nullptr; size_t rope_first = 0, rope_count = 0;   // a sequence with images: three rotation positions a row (sd_rope_rows)
    uint64_t launches = 0;   // kernels launched through this handle (the benchmark's gpu_launches)
    bool adopted = false;    // made by sdx_adopt over another library's stream and allocations: no range checks, nothing owned but workspaces
    explicit Device(int o) : ordinal(o) {}
};

Device& device(void* handle);   // sets the CUDA device; throws on a null handle
void* raw_allocate(Device& d, size_t bytes, bool zero);
void raw_release(Device& d, void* pointer);
void span(Device& d, const void* pointer, size_t bytes, const char* what);
void span_or_peer(Device& d, const void* pointer, size_t bytes, const char* what);   // also accepts a mapped peer allocation
size_t allocation_bytes(Device& d, const void* base);   // requested bytes of the allocation that starts at `base`, 0 if none (takes the lock)
void* ensure(Device& d, void*& slot, size_t& have, size_t bytes, bool pinned_host = false);
int* status_word(Device& d);
// top_k_kernel's other output (csrc/topk.cu): a row's chosen 4-position blocks written into its packed attention row as positions
struct TopKExpand {
    float* packed;               // null: off
    size_t index_start, selected, steps, base;
    const uint32_t* positions;   // a row's position, or null: base + row
    uint32_t keep;
};

cudaStream_t side_stream_begin(Device& d);   // the side stream, made to wait for everything queued on d.stream so far
void side_stream_end(Device& d);             // d.stream made to wait for everything queued on the side stream so far   // the device's word a kernel's bounded wait sets when it gives up (read by sdx_decode_status)

// a * b * c ... with overflow refusal (gpu/core.hpp:1413 region: an op_span check never passes on a wrapped size)
inline size_t checked_product(std::initializer_list<uint64_t> factors) {
    unsigned __int128 total = 1;
    for (uint64_t f : factors) {
        total *= f;
        if (total > (unsigned __int128)(SIZE_MAX / 8)) throw std::runtime_error("Straydog op: a shape overflows the address space");
    }
    return size_t(total);
}

#define SDB_OP_BEGIN try { auto& value = ::sdb::device(handle); (void)value;
#define SDB_OP_END SDB_CHECK(cudaGetLastError()); return 0; } catch (const std::exception& e) { ::sdb::last_error = e.what(); return -1; }

#if defined(__CUDACC__)
// ---- device primitives (sm_100a) ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// A bounded wait: gives up two seconds after the first failed poll and reports failure, so that a
// copy that never lands ends the kernel with a status the host reads instead of hanging it.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    for (;;) {
        #pragma unroll 1
        for (int spin = 0; spin < 64; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - start > 2000000000ull) return false;
    }
}
// After a wait gave up: let copies still in flight into this CTA's shared memory land (or not) for a
// bounded millisecond before the CTA exits.
__device__ __forceinline__ void drain_delay() {
    const uint64_t start = global_timer_ns();
    while (global_timer_ns() - start < 1000000ull) __nanosleep(1000);
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Untiled bulk copy global -> shared (TMA engine), completion on an mbarrier. Both addresses
// 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// D(16x8, f32) += A(16x16, row) * B(16x8, col); f16 or bf16 operands.
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
    uint32_t out;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(a), "r"(b), "r"(selector));
    return out;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    uint32_t out;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
    return out;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t out;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
    return out;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Bytes 0 and 2 (or 1 and 3) of a word (already xor 0x80808080) -> an FP16 pair, exactly.
__device__ __forceinline__ uint32_t bytes02_to_half2(uint32_t x) {
    const uint32_t h = prmt(x, 0x64646464u, 0x4240u);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bytes13_to_half2(uint32_t x) {
    const uint32_t h = prmt(x, 0x64646464u, 0x4341u);
    const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&h), __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480)));
    return *reinterpret_cast<const uint32_t*>(&r);
}
// Four 8 x 8 matrices of 16-bit units, transposed on the way: lane i gives the address of row i % 8 of matrix i / 8, and lane (g, t)
// receives, per matrix, unit g of rows 2t (low half) and 2t + 1 (high half).
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
// kv_encode (gpu/kernels.cpp:58-69) for one 32-value block held by a warp, a value a lane: the block's scale is
// FP16(max |v| / 127), a value is v / scale rounded to nearest even and clamped to +-127, 0 under a zero scale.
__device__ __forceinline__ int8_t q8_encode(float value, __half& scale_h) {
    float top = fabsf(value);
    #pragma unroll
    for (unsigned offset = 16; offset; offset /= 2) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
    scale_h = __float2half_rn(__fdiv_rn(top, 127.0f));
    const float scale = __half2float(scale_h);
    int q = scale > 0.0f ? __float2int_rn(__fdiv_rn(value, scale)) : 0;
    q = q > 127 ? 127 : q < -127 ? -127 : q;
    return int8_t(q);
}
#endif

}  // namespace sdb
