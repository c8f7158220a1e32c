/* C ABI of the B200 (sm_100a) attention library: libstraydog_gpu_b200.so.
 *
 * The sd_* entries keep the names, argument meaning and error behaviour of the reference's
 * gpu/straydog_gpu.h for the attention path, so that the engine's existing FFI binds them
 * unchanged; each declaration cites the reference declaration it replaces. The sdx_* entries are
 * additions the reference has no counterpart for (several sequences in one call, plans that keep
 * the host work out of the step); they collide with nothing in the reference.
 *
 * Conventions (gpu/straydog_gpu.h:1-5): an int result < 0 or a null pointer is a failure which
 * sd_error() then describes for the calling thread; other int results are 0 or a query's answer.
 * Handles are opaque. Nothing throws across this boundary. Every device pointer passed to an op
 * must lie inside an allocation this library made for the same handle (sd_allocate, sd_upload,
 * sd_buffer): every op checks. Work is queued on the handle's stream; reads synchronise.
 * No entry falls back to the CPU: without a B200-class GPU sd_create fails.
 */
#ifndef STRAYDOG_GPU_B200_H
#define STRAYDOG_GPU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- errors, devices, memory ---- */
/* gpu/straydog_gpu.h:17 */
const char* sd_error(void);
/* gpu/straydog_gpu.h:18 */
int sd_device_count(void);
/* gpu/straydog_gpu.h:33-34. budget: bytes this handle may allocate, at most the free memory. */
/* (the budget bounds what sd_allocate / sd_buffer / sd_upload hand out; the library's own workspaces - split partials, work lists,
   staging of host-pointer entries - are grown beside it on the first call of a size.) */
void* sd_create(int ordinal, uint64_t budget);
void sd_destroy(void* handle);
/* gpu/straydog_gpu.h:35 */
int sd_memory(void* handle, uint64_t* used, uint64_t* budget);
/* gpu/straydog_gpu.h:42,47,57,63,65-67 */
void* sd_upload(void* handle, const void* data, uint64_t bytes);
void* sd_allocate(void* handle, uint64_t bytes);
int sd_write(void* handle, void* pointer, const void* data, uint64_t bytes);
int sd_release(void* handle, void* pointer);
int sd_allocation_bytes(void* handle, const void* pointer, uint64_t* bytes);
int sd_zero(void* handle, void* pointer);
int sd_download(void* handle, void* pointer, void* output, uint64_t bytes);
/* gpu/straydog_gpu.h:157-159: a zeroed buffer; byte-range writes and reads. */
void* sd_buffer(void* handle, uint64_t bytes);
int sd_buffer_write(void* handle, void* buffer, uint64_t offset, const void* data, uint64_t bytes);
int sd_buffer_read(void* handle, const void* buffer, uint64_t offset, void* output, uint64_t bytes);

/* ---- K/V format and staging ---- */
/* gpu/straydog_gpu.h:113. row: 272 (Q8_0) or 512 (FP16: a value's nearest FP16). FP16 rows are written (sdx_kv_write, the fused
   fronts), decoded, grown and attended by sd_attention_sequence and by the decode seam's selection-list attention
   (sdx_qsa_attention_rows, sdx_qsa_attention_gathered: the rows' halves are the tensor cores' operands as they lie); the dense batch
   decode and the prompt kernel (sdx_qsa_decode*, sdx_attention_batch, sdx_qsa_prompt) read Q8_0 rows only and refuse a handle set to
   FP16 rows. */
int sd_kv_format(void* handle, uint32_t row);
/* gpu/straydog_gpu.h:114. The VRAM stage of host-resident K/V: an allocation of rows * 4096 bytes. With K/V resident in HBM the
   stage is registered and validated but never needed; sdx_qsa_attention_gathered copies a host-resident state's selected blocks
   into it. */
int sd_kv_stage(void* handle, void* pointer, uint64_t rows);
/* gpu/straydog_gpu.h:100. A zeroed state of `bytes` in page-locked host memory that the GPU reads in place (a K/V beyond the VRAM
   budget): the pointer returned is the device's view of it and an allocation of the handle like any other (sd_write, sd_download,
   sd_release; outside the VRAM budget). Null on failure. */
void* sd_host_state(void* handle, uint64_t bytes);
/* gpu/straydog_gpu.h:112. 1 when the device reads mapped host memory. */
int sd_host_state_supported(void* handle);
/* The data movement of sd_kv_grow (gpu/straydog_gpu.h:109, gpu/kernels.cpp:4048-4203): a sequence's K/V state of `from` positions and
   its indexer state grown to `to` positions (from < to <= 262144; valid <= from positions written). The reference's entry looks the
   two up in its decoder-layer registry and rewires the registry afterwards; the registry is the engine's, so here the caller passes
   the two pointers and gets the new ones back in their place. *state: 2 * kv_heads planes of `from` rows, an allocation of exactly
   that size in VRAM, or a host-resident state (sd_host_state). In VRAM the new state is a new zeroed allocation with every plane's
   `from` positions copied on the device, and the old one is released; a host-resident state is grown in host memory and its `valid`
   positions copied by the CPU. *index_state: [128][from / 4 + 1] pooled blocks + the 16 x 128 ring; the blocks take the pitch
   to / 4 + 1 (the first min(from / 4 + 1, valid / 4 + 1) of every column, the rest zeros), the ring follows; it is replaced by a
   new allocation only when the old one is too small (then the old one is released). A growth the budget refuses leaves both states
   as they were. Returns after the copies are complete. */
int sdx_kv_grow(void* handle, uint64_t kv_heads, uint64_t from, uint64_t to, uint64_t valid, void** state, void** index_state);

/* ---- Qwen3.8-style grouped-query attention over Q8_0 K/V ---- */
/* gpu/straydog_gpu.h:528. Host pointers. The reference's own shapes: 24 query / 2 K/V heads of 256,
   scale 1/16, `selected` <= 2052 key positions per step given as floats, then one count per step.
   input: [steps][24][256] q | [steps][2][256] k | [steps][2][256] v | [steps][selected] | [steps], all F32.
   Writes rows base..base+steps-1 of `state` (quantised to Q8_0), then attends. output [steps][24][256]. */
int sd_attention_sequence(void* handle, void* state, uint64_t context, uint64_t base, uint64_t steps, uint64_t selected,
                          const float* input, uint64_t input_count, float* output, uint64_t output_count);
/* gpu/straydog_gpu.h:453. Generic dense causal GQA over F32 keys/values [context][kv_heads][dim];
   device pointers. scratch >= rows * heads * 64 * (dim + 2) * 4 bytes always suffices. */
int sd_op_attention(void* handle, const float* q, const float* keys, const float* values, uint64_t context,
                    const int32_t* positions, uint64_t rows, uint64_t heads, uint64_t kv_heads, uint64_t dim, float scale,
                    const float* gate, float* scratch, uint64_t scratch_bytes, float* out);

/* ---- DeepSeek-V4.1-style latent sparse attention ---- */
/* gpu/straydog_gpu.h:385-389 */
int sd_attention_turns_reserve(void* handle, uint64_t rows, uint64_t rope_dims);
int sd_attention_turns_arm(void* handle, uint64_t rows);
/* gpu/straydog_gpu.h:398. `compressed` may carry the BF16 tag in bit 0 of the pointer. */
int sd_op_sparse_attention(void* handle, const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions,
                           uint64_t window, const float* compressed, uint64_t compressed_rows, const int32_t* selected,
                           uint64_t selections, const float* sinks, uint64_t rows, uint64_t heads, uint64_t dim, float scale,
                           uint64_t rope_dims, const float* frequencies, float* scratch, uint64_t scratch_bytes, float* out);
/* gpu/straydog_gpu.h:399-406. The drafter's noncausal block attention: q / out [slots][heads][512] (1..5 slots, 1..64 heads), K = V ring
   [128][512], the block's keys [slots][512], sinks [heads]; rope already applied. Every query sees history positions
   [anchor - history, anchor) of the ring and ALL block keys; history 0..128 <= anchor <= INT32_MAX; anchor_at (device, or null)
   overrides `anchor` at run time; scale 1 / sqrt(512); the sink enters the maximum and the denominator only. */
int sd_op_dspark_attention(void* handle, const float* q, const float* ring, const float* block, const float* sinks, uint64_t heads,
                           uint64_t slots, uint32_t anchor, const int32_t* anchor_at, uint64_t history, float* out);
/* ---- the producers of the latent attention's rows and index lists (DeepSeek-V4.1's indexer) ---- */
/* gpu/straydog_gpu.h:271. The last rope_dims values of each of rows x vectors vectors of `width`, rotated in adjacent pairs by
   positions[row] * frequencies[pair] (the angle times -1.0 with `inverse`), in double, in place. */
int sd_op_rope(void* handle, float* x, uint64_t rows, uint64_t vectors, uint64_t width, uint64_t rope_dims, const int32_t* positions,
               const float* frequencies, int inverse);
/* gpu/straydog_gpu.h:407. `ratio` consecutive rows pooled into one per group by a per-channel softmax of the gate (no gate: ratio 1). */
int sd_op_compress(void* handle, const float* kv, const float* gate, uint64_t groups, uint64_t ratio, uint64_t dim, float* out);
/* gpu/straydog_gpu.h:408. scores[row][g] = scale * sum_h relu(q[row][h] . keys[g]) * weights[row][h] for g < visible[row], -inf beyond;
   heads <= 64; `keys` may carry the BF16 tag in bit 0. */
int sd_op_index_scores(void* handle, const float* q, const float* keys, const float* weights, const int32_t* visible, uint64_t rows,
                       uint64_t groups, uint64_t heads, uint64_t dim, float scale, float* scores);
/* gpu/straydog_gpu.h:410-414. Each row's `blocks` blocks of `block` groups whose highest score is highest (the block of the row's last
   visible group always kept, blocks of only -inf never), in index order, -1 past the last; scratch holds rows * ceil(groups / block)
   floats. */
int sd_op_index_candidates(void* handle, const float* scores, const int32_t* visible, uint64_t rows, uint64_t groups, uint64_t blocks,
                           uint64_t block, int32_t* out, float* scratch, uint64_t scratch_bytes);
/* gpu/straydog_gpu.h:415-419. sd_op_rope of q (q itself unchanged), sd_op_index_scores and sd_op_top_k in one call: the same scores and
   indices. With candidates (rows x blocks) a row's groups scored and chosen are its candidates' (scores rows x blocks * block in
   candidate order), the indices the groups'. */
int sd_op_index_select(void* handle, const float* q, const float* keys, const float* weights, const int32_t* visible, uint64_t rows,
                       uint64_t groups, uint64_t heads, uint64_t dim, float scale, uint64_t rope_dims, const int32_t* positions,
                       const float* frequencies, float* scores, uint64_t k, int32_t* out, const int32_t* candidates, uint64_t blocks,
                       uint64_t block);
/* gpu/straydog_gpu.h:422. sd_op_index_select for one row whose head weights are projected first: weights = W . x, W [heads][proj_cols]
   row-major of kind 0 (F32), 1 (F16) or 30 (BF16), summed in the reference GEMV's order (bit-equal weights); `weights` receives them. The
   reference's quantised GGML kinds are refused ("unsupported Straydog GPU matrix format"): its GEMV family is outside this library. */
int sd_op_index_select_proj(void* handle, const void* proj_weights, int proj_kind, uint64_t proj_cols, const float* x, const float* q,
                            const float* keys, float* weights, const int32_t* visible, uint64_t groups, uint64_t heads, uint64_t dim,
                            float scale, uint64_t rope_dims, const int32_t* positions, const float* frequencies, float* scores, uint64_t k,
                            int32_t* out, const int32_t* candidates, uint64_t blocks, uint64_t block);
/* gpu/straydog_gpu.h:409 */
int sd_op_top_k(void* handle, const float* scores, uint64_t rows, uint64_t groups, uint64_t k, int32_t* out);
/* gpu/straydog_gpu.h:459 */
int sd_op_to_bf16(void* handle, const float* x, uint64_t count, void* out);

/* ---- additions (no counterpart in the reference) ---- */
/* A handle over another library's CUDA stream and allocations on device `ordinal` (no counterpart in the reference: it is what the
   reference's own build holds when its spans call this library's kernels, include/qsa_b200.hpp). Ops queue on `stream`; pointers
   are taken as checked by the caller; sd_allocate and friends are refused. Released by sd_destroy, which leaves the stream alone. */
void* sdx_adopt(int ordinal, void* stream);
/* Waits for everything queued on the handle's stream. */
int sdx_synchronize(void* handle);
/* The handle's CUDA stream (a cudaStream_t), for timing with events on the launching stream. */
void* sdx_stream(void* handle);
/* Kernels launched through the handle so far. */
uint64_t sdx_launch_count(void* handle);
/* CUDA events on the handle's stream, for timing a region or one kernel from a host language without CUDA bindings. */
void* sdx_event_create(void);
int sdx_event_record(void* handle, void* event);
int sdx_event_elapsed_ms(void* before, void* after, float* ms);
void sdx_event_destroy(void* event);

/* Appends `steps` tokens' keys and values ([steps][kv_heads][256] F32, device) to a Q8_0 state at rows
   base..: the reference's write_attention_kv (gpu/kernels.cpp:79-98) for any number of K/V heads. */
int sdx_kv_write(void* handle, void* state, uint64_t context, uint64_t kv_heads, uint64_t base, uint64_t steps,
                 const float* keys, const float* values);
/* `count` Q8_0 rows (272 bytes each, device) as F32 [count][256]: float(int8) * float(block scale). */
int sdx_kv_decode_rows(void* handle, const void* rows, uint64_t count, float* out);

/* Ragged batch of one-token decodes: sequence s attends rows 0..lengths[s]-1 of states[s] (a Q8_0
   state of contexts[s] positions, 2 * kv_heads planes). states/contexts/lengths are HOST arrays;
   q ([sequences][heads][256] FP16) and out ([sequences][heads][256] F32) are device pointers.
   heads / kv_heads <= 8, or an even number up to 16 (the reference's own 24 / 2 among them: a K/V head's rows are then streamed
   once for each half of its query heads). */
int sdx_qsa_decode(void* handle, const void* const* states, const uint64_t* contexts, const uint64_t* lengths,
                   uint64_t sequences, uint64_t heads, uint64_t kv_heads, float scale, const void* q, float* out);
/* The same in two steps: the plan holds the batch's work list on the device, so that a run is
   kernel launches only (no host work, no allocation: safe inside a captured graph). */
void* sdx_qsa_plan(void* handle, const void* const* states, const uint64_t* contexts, const uint64_t* lengths,
                   uint64_t sequences, uint64_t heads, uint64_t kv_heads);
int sdx_qsa_plan_run(void* handle, void* plan, float scale, const void* q, float* out);
/* sdx_qsa_plan_run with `before` recorded ahead of the streaming kernel and `after` behind it (ahead of the merge). */
int sdx_qsa_plan_run_marked(void* handle, void* plan, float scale, const void* q, float* out, void* before, void* after);
int sdx_qsa_plan_info(void* plan, uint64_t* kv_bytes, uint64_t* pieces, uint64_t* ctas, uint64_t* virtual_warps);
int sdx_qsa_plan_release(void* handle, void* plan);
/* How the batched decode entries of this handle (sdx_qsa_decode, sdx_qsa_plan, sdx_attention_batch) cut a batch into pieces.
   fixed = 0 (the default), moving cuts: the batch's 16-key tiles laid end to end and cut into equal runs, one per warp: the fewest
   partials and an even load whatever the batch, but where a sequence is cut depends on its batch, so its result is the same
   value to FP32 rounding, not bit for bit. fixed = 1: a sequence is cut at places that depend on its own length only (chunks of
   512 keys and a halving tail, 128 keys for sequences under 8192) and its chunks are merged in order: the same bits in any batch,
   at the cost of more partials and of an uneven load when a batch is small. (The reference's own bit-for-bit contract, verification
   rows = one-token decodes, is the selection-list entry's, sdx_qsa_attention_rows, which keeps it always.) */
int sdx_decode_cuts(void* handle, int fixed);
/* The cuts of a batch for `warps` warps, without a device (host arithmetic): fixed as above. Returns the number of pieces of sequence `probe`'s first K/V head and writes where they begin to begins[0 ..
   capacity); stats (or null) = {pieces in all, warps used, most 16-key tiles a warp got, tiles in all}. */
int sdx_qsa_cuts(const uint64_t* lengths, uint64_t sequences, uint64_t kv_heads, uint64_t warps, int fixed, uint64_t probe,
                 uint32_t* begins, uint64_t capacity, uint64_t* stats);
/* No counterpart in the reference. sdx_qsa_decode for hosts that may not allocate once they serve (an engine
   whose VRAM budget is fully handed out, a loop that forbids driver allocations because they stall the
   device): the work list and the split partials live in a 16.3 MiB array inside the library's device image,
   held by every GPU that loads the library until exit. Limits: at most 64 sequences, 8 K/V heads and 2048
   work-list pieces a call; a larger batch is refused with an error, nothing is truncated. The first call on a
   device looks up the array's device address and, under the CUDA runtime's default lazy loading, is also when the GPU takes the
   library's device image with the array in it: make that call at start-up (before any stream capture); it is every later call
   that touches no allocator. Calls share the
   array: two calls that overlap on the GPU, from any handles or threads, race; the call returns after its
   result is complete. It calls no cudaMalloc, cudaFree or allocating library routine. */
int sdx_qsa_decode_static(void* handle, const void* const* states, const uint64_t* contexts, const uint64_t* lengths,
                          uint64_t sequences, uint64_t heads, uint64_t kv_heads, float scale, const void* q, float* out);
/* What a kernel reported instead of hanging or faulting since the last call (cleared by the call), 0 if nothing:
   1 a bounded wait on a copy gave up (decode, prompt or latent kernel); 2 a selected row number lay past the latent cache (the
   row was taken as absent); 3 a key pointer lay outside the call's buffers (skipped); 4 a rank of a gathered latent attention
   never raised its counter within a second; 5 a row of sdx_qsa_normalize_rows sat at a position past the K/V state (nothing of the
   row was written). Synchronises the handle's stream. */
int sdx_decode_status(void* handle);

/* For builds of the library with -DSDX_TRACE (python -m straydog_b200.build --define SDX_TRACE --out <path>): the cycle counters the
   latent tcgen05 kernel's last launch on this handle left, eight int64 per CTA (total, the MMA thread's waits for a tile, for the
   weights and for a free score buffer, the copy thread's wait for a free slot, tiles, 0, 0). Returns the number of CTAs written
   (0 in an ordinary build). */
int sdx_trace_read(void* handle, int64_t* out, uint64_t capacity);

/* Causal prompt attention of a chunk: `rows` new tokens at positions first .. first + rows - 1 of a Q8_0 state
   (their K/V rows already written, e.g. by sdx_kv_write) attend positions 0 .. their own. q [rows][heads][256]
   FP16 and out [rows][heads][256] F32 are device pointers; heads / kv_heads is at most 16 (a group that does not divide 128, like the reference's own 12, leaves some of a block's 128 rows idle). The dense causal
   form of the reference's qsa_flash_launch (gpu/sparse_attention_compute.hpp:589-608). */
int sdx_qsa_prompt(void* handle, const void* state, uint64_t context, uint64_t first, uint64_t rows, uint64_t heads,
                   uint64_t kv_heads, float scale, const void* q, float* out);

/* Latent sparse attention of several spans in one call (no reference counterpart: the reference verifies one sequence per call,
   gpu/straydog_gpu.h:398, crates/straydog-engine/src/arch/deepseek41/engine.rs:3838). Equal to `spans` calls of
   sd_op_sparse_attention with rows = span_rows: span s takes q, positions, selected and out at row offset s * span_rows and its
   own window ring raw + s * raw_rows * dim (positions count in that ring); `compressed`, `sinks`, `frequencies` are shared, so the
   caller keeps the sequences' caches in one allocation and points `selected` into it. No scratch: the library owns its workspaces. */
int sdx_sparse_attention_spans(void* handle, const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions,
                               uint64_t window, const float* compressed, uint64_t compressed_rows, const int32_t* selected,
                               uint64_t selections, const float* sinks, uint64_t spans, uint64_t span_rows, uint64_t heads, uint64_t dim,
                               float scale, uint64_t rope_dims, const float* frequencies, float* out);

/* Head-sharded latent attention with the all-gather inside the kernel (no reference counterpart: the reference shards by
   pipeline stage, not by head). Rank `rank` of `world` (<= 8) GPUs of one node computes this call's `heads` heads (its share) over
   the whole latent cache; every GPU keeps a gathered buffer [world][rows][heads][dim] F32 (rank-major). The call stores this rank's
   outputs into slot `rank` of EVERY GPU's buffer (outs[peer]: this handle's own allocation for peer == rank, mappings made by
   sdx_ipc_open for the others: plain stores over NVLink from the kernel's merge); the last CTA of the kernel then raises counter
   `rank` in every GPU's `flags[peer]` (int32 [world], zeroed once) to `step` and waits, bounded to a second, until its own
   counters all show `step`: work queued behind the call sees the whole gathered buffer. `step` grows by one per call.
   The caller keeps TWO gathered buffers per GPU and passes them in turn (step odd / even): a rank may run one call ahead of
   its peers, never two (it cannot leave call n + 1 before every peer has entered its own call n + 1, which the peer's stream
   orders behind the peer's readers of call n), so with two buffers a store never lands in a buffer a peer still reads; with one
   buffer it could. */
int sdx_sparse_attention_gather(void* handle, const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions,
                                uint64_t window, const float* compressed, uint64_t compressed_rows, const int32_t* selected,
                                uint64_t selections, const float* sinks, uint64_t rows, uint64_t heads, uint64_t dim, float scale,
                                uint64_t rope_dims, const float* frequencies, uint64_t world, uint64_t rank, void* const* outs,
                                void* const* flags, int32_t step);
/* Sharing an allocation with the other ranks' processes (CUDA IPC): export writes a 64-byte handle for an allocation's base
   pointer; open maps another process's exported allocation of `bytes` bytes (peer access over NVLink) and lets this handle's
   entries accept pointers into it where they say so; close unmaps. */
int sdx_ipc_export(void* handle, const void* pointer, void* out_handle);
void* sdx_ipc_open(void* handle, const void* in_handle, uint64_t bytes);
int sdx_ipc_close(void* handle, void* pointer);

/* Selection-list decode attention of `steps` rows on the tensor cores: the reference's qsa_attention (steps = 1) and
   qsa_attention_rows (a verification's rows) as their callers use them (gpu/sparse_attention_compute.hpp:609-647 over
   qsa_decode_parts / qsa_decode_merge, :41-170), for any heads / kv_heads <= 16. All pointers are device pointers. `input` holds
   the packed F32 rows in the reference's layout (gpu/core.hpp:392): [steps][heads][256] queries | [steps][kv_heads][256] keys |
   [steps][kv_heads][256] values | [steps][selected] key positions as floats | [steps] counts as floats. Row r sits at position
   positions[r] (or base + r when positions is null); slot s of a row is live when s < count, 0 <= position <= the row's own and
   position < context. `mirror` (or null) is the ring of the newest mirror_rows positions of a host-resident state, read as
   gpu/sparse_attention_compute.hpp:65-68 does. `gates` (or null): out is multiplied by sigmoid(gates[r * gate_stride + head * 512
   + 256 + column]) (:168). out [steps][heads][256] F32. A row's result has the same bits whatever `steps` is. selected <= 8192. */
int sdx_qsa_attention_rows(void* handle, const void* state, uint64_t context, uint64_t base, const uint32_t* positions,
                           uint64_t steps, uint64_t selected, uint64_t heads, uint64_t kv_heads, float scale, const float* input,
                           const void* mirror, uint64_t mirror_rows, const float* gates, uint64_t gate_stride, float* out);

/* Qwen's indexer, the producer of the lists above (the reference's qsa_block_scores[_tiled] and qsa_select[_rows],
   gpu/sparse_attention.hpp:141-157, 172-243, 247-296, 307-395, as qsa_index_exact launches them, :398-410; the reference has no entry of
   its own for them). queries: `steps` rows of 4 index heads x 128 F32, query_stride floats apart (>= 512); blocks: the pooled index keys,
   [128 columns][pool] F32. Row r at position positions[r] (or base + r) has complete = (position + 1) / 4 whole blocks: up to 512, every
   position 0 .. position is listed; more, the 512 blocks of highest score = sum over the heads of max(0, query . key) are listed in block
   order (equal scores by lowest block), four positions each, then the positions of the incomplete block. The lists and counts are
   written into `packed` (the layout of sdx_qsa_attention_rows, whose queries, keys and values this call leaves alone); selected >= 2052. */
int sdx_qsa_index_select(void* handle, const float* queries, uint64_t query_stride, const float* blocks, uint64_t pool, uint64_t base,
                         const uint32_t* positions, uint64_t steps, uint64_t selected, uint64_t heads, uint64_t kv_heads, float* packed);

/* The front of Qwen's decode and verification attention in one launch, for `rows` <= 256 rows: the reference's qsa_normalize_rows
   (gpu/qsa_decode.hpp:86-111; for one row qsa_normalize_decode + qsa_pool_one + write_attention_kv as qsa_decode_attend launches
   them, :5-23, 28-44; the rotation and normalisation of gpu/sparse_attention.hpp:2-6, 55-71), for any heads and kv_heads. Row r of
   `projections` (stride floats apart, stride >= heads * 512 + kv_heads * 512 + 640) holds  qgate [heads][query 256 | gate 256] |
   key [kv_heads][256] | value [kv_heads][256] | index query [4][128] | index key [128].  The call writes the RMS-normalised, rotated
   queries and keys into `packed` (the layout of sdx_qsa_attention_rows for `rows` rows and `selected` slots; its values, lists and
   counts are left alone), encodes each row's normalised keys and its values into row positions[r] of the Q8_0 `state` (and of
   `mirror`, the ring of mirror_rows positions of a host-resident state, or null / 0), normalises and rotates the four index-query
   heads in place, and passes the rows' index keys through the history ring: a row whose position completes a 4-position block
   pools it into index_state ([128][context / 4 + 1] pooled blocks followed by the ring of 16 x 128, gpu/sparse_attention.hpp:462).
   positions: the rows' K/V positions; ropes: their rotation positions (the same numbers unless the sequence holds images). Then
   sdx_qsa_index_select (queries = projections + heads * 512 + kv_heads * 512, blocks = index_state) and sdx_qsa_attention_rows
   (gates = projections) finish what the reference's qsa_decode_attend_rows does (gpu/qsa_decode.hpp:113-129). A position past the
   state writes nothing and reports status 5. */
int sdx_qsa_normalize_rows(void* handle, float* projections, uint64_t stride, uint64_t rows, uint64_t heads, uint64_t kv_heads,
                           const float* qnorm, const float* knorm, const float* iqnorm, const float* pool_norm,
                           const uint32_t* positions, const uint32_t* ropes, float* packed, uint64_t selected, void* state,
                           uint64_t context, void* mirror, uint64_t mirror_rows, float* index_state);

/* The same front for a prompt chunk: `count` consecutive tokens from `position` (a token turns at its own position), as the
   reference's prefill runs it in seven launches (gpu/prefill_batch.hpp:342-370, gpu/sparse_attention.hpp:493-506: qsa_normalize of the
   queries, keys and index queries, the values' copy, qsa_pool :87-106, qsa_save_history :135-139, write_attention_kv), here in two.
   The projections come in five arrays: qgate [count][heads][512] (query 256 | gate 256 a head), key and value_rows
   [count][kv_heads][256], iq [count][4][128] (normalised and rotated in place), ik [count][128]. Queries, keys and values go into
   `packed` (all three: the layout sd_attention_sequence and sdx_qsa_attention_rows read, for `count` rows), keys and values into rows
   position .. position + count - 1 of the Q8_0 state (and the mirror ring), every 4-position block the chunk completes is pooled into
   index_state (positions before the chunk from the ring), and the chunk's last four index keys enter the ring. The same bits as
   sdx_qsa_normalize_rows over the same tokens. While a rope table is set (sd_rope_rows: a sequence with images) the tokens and the
   pooled blocks turn by the table's three positions a row (qsa_normalize_axes, qsa_pool_axes: gpu/sparse_attention.hpp:27-50,
   111-131); a chunk the table does not cover is refused ("invalid Straydog rope table"). */
int sdx_qsa_normalize_chunk(void* handle, const float* qgate, const float* key, const float* value_rows, float* iq, const float* ik,
                            uint64_t count, uint64_t position, uint64_t heads, uint64_t kv_heads, const float* qnorm,
                            const float* knorm, const float* iqnorm, const float* pool_norm, float* packed, uint64_t selected,
                            void* state, uint64_t context, void* mirror, uint64_t mirror_rows, float* index_state);

/* gpu/straydog_gpu.h:607-609. The rope positions of a sequence with images for the next prompt chunks: three (t, h, w) a position
   from `first`, `count` (<= 4100) positions in a host array, covering each chunk's rows and the 4-position block its first row is
   in. count 0: the rows' own positions again. */
int sd_rope_rows(void* handle, uint64_t first, uint64_t count, const uint32_t* axes);

/* sdx_qsa_attention_rows over a state in host memory (sd_host_state), through the stage registered with sd_kv_stage: the union of
   the rows' selected 4-position blocks is copied into the stage once, in block order, and the selections are renumbered to it
   (the reference's qsa_attention_gathered, gpu/prefill_batch.hpp:227-252 over gpu/sparse_attention_compute.hpp:680-734), as many
   rows at a time as the stage holds the union of; one host read of the union's size per attempt; a stage that cannot hold one
   row's selection (4 * selected positions always do) is refused. The same bits as
   sdx_qsa_attention_rows over the same state. `input` is left as it is. passes (or null): the groups of rows the call made. */
int sdx_qsa_attention_gathered(void* handle, const void* state, uint64_t context, uint64_t base, const uint32_t* positions,
                               uint64_t steps, uint64_t selected, uint64_t heads, uint64_t kv_heads, float scale, const float* input,
                               const float* gates, uint64_t gate_stride, float* out, uint64_t* passes);

/* One decode step of a batch from HOST buffers (the batched twin of sd_attention_sequence): for
   sequence s the new token's keys/values (k, v: [sequences][kv_heads][256] F32, host) are written
   to row bases[s] of states[s], then its query (q: [sequences][heads][256] FP16, host) attends rows
   0..bases[s]; out [sequences][heads][256] F32, host. Copies both ways are inside the call; page-locked k, v and out are read and
   written in place by the kernels instead (the same bits), which takes three of the four copies off the call. */
int sdx_attention_batch(void* handle, void* const* states, const uint64_t* contexts, const uint64_t* bases, uint64_t sequences,
                        uint64_t heads, uint64_t kv_heads, float scale, const void* q, const float* k, const float* v, float* out);

#ifdef __cplusplus
}
#endif
#endif
