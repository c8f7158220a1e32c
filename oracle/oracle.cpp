// CPU restatement of the reference's attention arithmetic. TEST INFRASTRUCTURE ONLY: this file is
// the checker the parity tests, the smoke test and the benchmark's CPU-baseline leg compare the
// CUDA path against. Nothing in the shipped library links or calls it.
//
// Every function names the reference source it restates (paths inside the reference project).
// Parity status: the Q8_0 codec is pinned by the properties of the reference's own unit tests
// (crates/straydog-engine/src/gpu.rs kv_format_tests); the dense GQA attention by the reference's
// F64 error-bound test (crates/straydog-engine/tests/attention_gpu.rs); top-k by its rule
// (tests/fused_gpu.rs top_k_reference); the latent sparse attention by
// tests/ds_state_bf16_gpu.rs shapes. Golden fixtures produced by the reference's own GPU library
// (tests/golden/) pin the restatement where a GPU run of the reference was available: its sd_* entries directly, and Qwen's front,
// indexer and selection-list decode through sd_qsa_sequence over selection matrices (tests/golden/make_golden.py --qsa).
//
// Build: g++ -O3 -march=native -fopenmp -shared -fPIC (see oracle/build.py). -ffast-math is never used.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---- IEEE binary16 <-> binary32, round to nearest even (what __float2half_rn / __half2float do) ----
inline uint16_t f32_to_f16(float value) {
    uint32_t x;
    std::memcpy(&x, &value, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return uint16_t(sign | (x > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (x >= 0x477ff000u) return uint16_t(sign | 0x7c00u);          // rounds to infinity
    if (x < 0x33000001u) return uint16_t(sign);                      // rounds to zero (<= 2^-25)
    int exponent = int(x >> 23) - 127;
    uint32_t mantissa = (x & 0x7fffffu) | 0x800000u;
    int shift;
    if (exponent < -14) { shift = 13 + (-14 - exponent); exponent = -15; } else shift = 13;
    uint32_t half = mantissa >> shift;
    const uint32_t rest = mantissa & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rest > halfway || (rest == halfway && (half & 1))) ++half;
    // (a carry out of the mantissa moves into the exponent field, which is what is wanted)
    if (exponent == -15) return uint16_t(sign | half);
    return uint16_t(sign | ((uint32_t(exponent + 15) << 10) + (half - 0x400u)));
}
inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = uint32_t(h & 0x8000u) << 16;
    uint32_t exponent = (h >> 10) & 31, mantissa = h & 0x3ffu, bits;
    if (exponent == 31) bits = sign | 0x7f800000u | (mantissa << 13);
    else if (exponent) bits = sign | ((exponent + 112) << 23) | (mantissa << 13);
    else if (!mantissa) bits = sign;
    else {
        int e = -1;
        do { ++e; mantissa <<= 1; } while (!(mantissa & 0x400u));
        bits = sign | (uint32_t(112 - e) << 23) | ((mantissa & 0x3ffu) << 13);
    }
    float out;
    std::memcpy(&out, &bits, 4);
    return out;
}
// tests/ds_state_bf16_gpu.rs:27-37 (nearest BF16, ties to even; a NaN stays one) and gpu/ops.hpp:1215 (widening).
inline uint16_t f32_to_bf16(float value) {
    uint32_t bits;
    std::memcpy(&bits, &value, 4);
    if (value != value) return uint16_t((bits >> 16) | 0x40);
    return uint16_t((bits + 0x7fffu + ((bits >> 16) & 1)) >> 16);
}
inline float bf16_to_f32(uint16_t half) {
    const uint32_t bits = uint32_t(half) << 16;
    float out;
    std::memcpy(&out, &bits, 4);
    return out;
}

constexpr size_t kRowQ8 = 272, kDim = 256;

// gpu/kernels.cpp:38-44 (kv_scale, kv_load): value = float(int8) * float(fp16 scale of the column's block).
inline float q8_value(const uint8_t* row, size_t column) {
    uint16_t scale;
    std::memcpy(&scale, row + 256 + 2 * (column / 32), 2);
    return float(int8_t(row[column])) * f16_to_f32(scale);
}

// gpu/kernels.cpp:58-74 (kv_encode, kv_put); crates/straydog-engine/src/gpu.rs:536-550 (kv_q8_row).
void q8_encode_row(const float* values, uint8_t* row) {
    for (size_t block = 0; block < 8; ++block) {
        float top = 0.0f;
        for (size_t i = 0; i < 32; ++i) top = std::fmax(top, std::fabs(values[block * 32 + i]));
        const uint16_t half = f32_to_f16(top / 127.0f);
        const float scale = f16_to_f32(half);
        for (size_t i = 0; i < 32; ++i) {
            int q = 0;
            if (scale > 0.0f) {
                const float quotient = values[block * 32 + i] / scale;
                // __float2int_rn: nearest, ties to even, saturating; a NaN gives 0
                if (quotient != quotient) q = 0;
                else if (quotient >= 2147483520.0f) q = 2147483647;
                else if (quotient <= -2147483648.0f) q = -2147483647 - 1;
                else q = int(std::nearbyintf(quotient));
            }
            q = q > 127 ? 127 : q < -127 ? -127 : q;
            row[block * 32 + i] = uint8_t(int8_t(q));
        }
        std::memcpy(row + 256 + 2 * block, &half, 2);
    }
}

// The halving-tree sum of 256 partials as gpu/kernels.cpp:141-145 forms it.
inline float tree_sum(float* partial) {
    for (unsigned stride = 128; stride; stride /= 2)
        for (unsigned i = 0; i < stride; ++i) partial[i] += partial[i + stride];
    return partial[0];
}

inline float sigmoid(float x) { return 1.0f / (1.0f + std::exp(-x)); }

}  // namespace

extern "C" {

uint16_t orc_f32_to_f16(float value) { return f32_to_f16(value); }
float orc_f16_to_f32(uint16_t half) { return f16_to_f32(half); }

void orc_q8_encode_rows(const float* values, uint64_t rows, uint8_t* out) {
    for (uint64_t r = 0; r < rows; ++r) q8_encode_row(values + r * kDim, out + r * kRowQ8);
}
void orc_q8_decode_rows(const uint8_t* packed, uint64_t rows, float* out) {
    for (uint64_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < kDim; ++c) out[r * kDim + c] = q8_value(packed + r * kRowQ8, c);
}

// gpu/kernels.cpp:79-98 (write_attention_kv): rows base..base+steps-1 of every plane, planes ordered
// K(head 0..kv-1) then V(head 0..kv-1), plane stride context rows. keys/values: [steps][kv_heads][256] F32.
void orc_kv_write(uint8_t* state, uint64_t context, uint64_t kv_heads, uint64_t base, uint64_t steps, const float* keys,
                  const float* values) {
    for (uint64_t step = 0; step < steps; ++step)
        for (uint64_t head = 0; head < kv_heads; ++head) {
            q8_encode_row(keys + (step * kv_heads + head) * kDim, state + (head * context + base + step) * kRowQ8);
            q8_encode_row(values + (step * kv_heads + head) * kDim, state + ((kv_heads + head) * context + base + step) * kRowQ8);
        }
}

// gpu/kernels.cpp:100-165 (attention_scores, attention_reduce) behind sd_attention_sequence
// (gpu/kernels.cpp:4387-4419), for any head counts: `input` is the packed layout
// [steps][heads][256] q | [steps][kv][256] k | [steps][kv][256] v | [steps][selected] positions as floats | [steps] counts as floats.
// The state's rows base.. are written first (as the entry does), then every (step, head) attends.
// scale is the reference's hard-coded 0.0625 when called for its own shapes.
void orc_attention_sequence(uint8_t* state, uint64_t context, uint64_t heads, uint64_t kv_heads, uint64_t base, uint64_t steps,
                            uint64_t selected, const float* input, float scale, float* output) {
    const uint64_t group = heads / kv_heads;
    const float* keys = input + steps * heads * kDim;
    const float* values = keys + steps * kv_heads * kDim;
    const float* indices = values + steps * kv_heads * kDim;
    const float* counts = indices + steps * selected;
    orc_kv_write(state, context, kv_heads, base, steps, keys, values);
    #pragma omp parallel for collapse(2) schedule(dynamic)
    for (uint64_t step = 0; step < steps; ++step)
        for (uint64_t head = 0; head < heads; ++head) {
            const uint64_t item = step * heads + head, kv = head / group;
            const uint64_t count = uint64_t(counts[step]);
            std::vector<float> scores(selected), probabilities(selected);
            std::vector<int64_t> token(selected, -1);
            for (uint64_t slot = 0; slot < selected; ++slot) {
                float result = -INFINITY;
                if (slot < count) {
                    const float raw = indices[step * selected + slot];
                    if (raw >= 0 && raw <= float(base + step) && raw < float(context)) {
                        token[slot] = int64_t(raw);
                        const uint8_t* row = state + (kv * context + uint64_t(raw)) * kRowQ8;
                        result = 0;
                        for (size_t column = 0; column < kDim; ++column)
                            result = std::fmaf(q8_value(row, column), input[item * kDim + column], result);
                        result *= scale;
                    }
                }
                scores[slot] = result;
            }
            float maximum = -INFINITY;
            for (uint64_t slot = 0; slot < selected; ++slot) maximum = std::fmax(maximum, scores[slot]);
            float partial[256];
            for (unsigned t = 0; t < 256; ++t) {
                float sum = 0;
                for (uint64_t slot = t; slot < selected; slot += 256) {
                    probabilities[slot] = std::exp(scores[slot] - maximum);
                    sum += probabilities[slot];
                }
                partial[t] = sum;
            }
            const float denominator = tree_sum(partial);
            for (uint64_t slot = 0; slot < selected; ++slot) probabilities[slot] /= denominator;
            for (size_t column = 0; column < kDim; ++column) {
                float result = 0;
                for (uint64_t slot = 0; slot < count && slot < selected; ++slot)
                    if (token[slot] >= 0)
                        result = std::fmaf(probabilities[slot],
                                           q8_value(state + ((kv_heads + kv) * context + uint64_t(token[slot])) * kRowQ8, column), result);
                output[item * kDim + column] = result;
            }
        }
}

// Dense causal decode over a Q8_0 state: one query token per sequence attending positions 0..length-1
// (the selection attention above with the identity selection, gpu/kernels.cpp:100-165, and the
// flash kernels' "divide at the end" form, gpu/sparse_attention_compute.hpp:139-170). q is FP16 bits
// [heads][256]; accumulation FP32 (accumulate64 = 0) or F64 (accumulate64 = 1, the tight checker).
void orc_gqa_decode_q8(const uint8_t* state, uint64_t context, uint64_t length, uint64_t heads, uint64_t kv_heads,
                       const uint16_t* q, float scale, int accumulate64, float* out) {
    const uint64_t group = heads / kv_heads;
    #pragma omp parallel for schedule(dynamic)
    for (uint64_t head = 0; head < heads; ++head) {
        const uint64_t kv = head / group;
        float query[kDim];
        for (size_t c = 0; c < kDim; ++c) query[c] = f16_to_f32(q[head * kDim + c]);
        std::vector<double> scores(length);
        double top = -INFINITY;
        for (uint64_t key = 0; key < length; ++key) {
            const uint8_t* row = state + (kv * context + key) * kRowQ8;
            double score;
            if (accumulate64) {
                double sum = 0;
                for (size_t c = 0; c < kDim; ++c) sum += double(q8_value(row, c)) * double(query[c]);
                score = sum * double(scale);
            } else {
                float sum = 0;
                for (size_t c = 0; c < kDim; ++c) sum = std::fmaf(q8_value(row, c), query[c], sum);
                score = double(sum * scale);
            }
            scores[key] = score;
            top = std::max(top, score);
        }
        double denominator = 0;
        float denominator32 = 0;
        std::vector<double> acc(kDim, 0.0);
        std::vector<float> acc32(kDim, 0.0f);
        for (uint64_t key = 0; key < length; ++key) {
            const uint8_t* row = state + ((kv_heads + kv) * context + key) * kRowQ8;
            if (accumulate64) {
                const double p = std::exp(scores[key] - top);
                denominator += p;
                for (size_t c = 0; c < kDim; ++c) acc[c] += p * double(q8_value(row, c));
            } else {
                const float p = std::exp(float(scores[key]) - float(top));
                denominator32 += p;
                for (size_t c = 0; c < kDim; ++c) acc32[c] = std::fmaf(p, q8_value(row, c), acc32[c]);
            }
        }
        for (size_t c = 0; c < kDim; ++c)
            out[head * kDim + c] = accumulate64 ? float(acc[c] / denominator) : acc32[c] / denominator32;
    }
}

// Causal prompt attention over a Q8_0 state (the dense form of gpu/sparse_attention_compute.hpp:177-279
// qsa_flash: F32 online softmax, output = accumulator / running sum): query row r sits at position
// first + r and attends keys 0..first+r. q FP16 bits [rows][heads][256]; rows row_begin..row_end-1 are computed.
void orc_gqa_prompt_q8(const uint8_t* state, uint64_t context, uint64_t first, uint64_t rows, uint64_t row_begin, uint64_t row_end,
                       uint64_t row_step, uint64_t heads, uint64_t kv_heads, const uint16_t* q, float scale, int accumulate64, float* out) {
    (void)rows;
    std::vector<uint64_t> list;
    for (uint64_t r = row_begin; r < row_end; r += row_step) list.push_back(r);
    #pragma omp parallel for schedule(dynamic)
    for (size_t i = 0; i < list.size(); ++i) {
        const uint64_t r = list[i];
        orc_gqa_decode_q8(state, context, std::min<uint64_t>(first + r + 1, context), heads, kv_heads, q + r * heads * kDim, scale,
                          accumulate64, out + r * heads * kDim);
    }
}

// gpu/token_mixing.hpp:435-520 (tm_attention_split_kernel + combine; semantics only: one split) and
// crates/straydog-engine/tests/attention_gpu.rs:50-87 (the F64 reference and its per-output bound).
// keys/values [context][kv_heads][dim] F32. out64/bound (optional, F64) receive the reference and its bound.
void orc_op_attention(const float* q, const float* keys, const float* values, uint64_t context, const int32_t* positions,
                      uint64_t rows, uint64_t heads, uint64_t kv_heads, uint64_t dim, float scale, const float* gate, float* out,
                      double* out64, double* bound) {
    const auto gamma = [](size_t operations) {
        const double nu = double(operations) * std::ldexp(1.0, -24);
        return nu / (1.0 - nu);
    };
    #pragma omp parallel for collapse(2) schedule(dynamic)
    for (uint64_t row = 0; row < rows; ++row)
        for (uint64_t head = 0; head < heads; ++head) {
            const uint64_t length = std::min<uint64_t>(uint64_t(positions[row]) + 1, context), kh = head / (heads / kv_heads);
            const float* query = q + (row * heads + head) * dim;
            std::vector<float> scores(length);
            std::vector<double> scores64(length);
            double error = 0;
            float top = -INFINITY;
            double top64 = -INFINITY;
            for (uint64_t key = 0; key < length; ++key) {
                const float* k = keys + (key * kv_heads + kh) * dim;
                float sum = 0;
                double sum64 = 0, absolute = 0;
                for (uint64_t d = 0; d < dim; ++d) {
                    sum = std::fmaf(query[d], k[d], sum);
                    const double product = double(query[d]) * double(k[d]);
                    sum64 += product;
                    absolute += std::fabs(product);
                }
                error = std::max(error, gamma(2 * dim + 1) * absolute * std::fabs(double(scale)));
                scores[key] = sum * scale;
                scores64[key] = sum64 * double(scale);
                top = std::fmax(top, scores[key]);
                top64 = std::max(top64, scores64[key]);
            }
            float total = 0;
            double total64 = 0;
            for (uint64_t key = 0; key < length; ++key) {
                scores[key] = std::exp(scores[key] - top);
                total += scores[key];
                scores64[key] = std::exp(scores64[key] - top64);
                total64 += scores64[key];
            }
            for (uint64_t d = 0; d < dim; ++d) {
                float sum = 0;
                double sum64 = 0, largest = 0;
                for (uint64_t key = 0; key < length; ++key) {
                    const float v = values[(key * kv_heads + kh) * dim + d];
                    sum = std::fmaf(scores[key], v, sum);
                    sum64 += scores64[key] * double(v);
                    largest = std::max(largest, std::fabs(double(v)));
                }
                const uint64_t at = (row * heads + head) * dim + d;
                float value = sum / total;
                double gating = 1.0;
                if (gate) {
                    value *= sigmoid(gate[at]);
                    gating = 1.0 / (1.0 + std::exp(-double(gate[at])));
                }
                out[at] = value;
                if (out64) out64[at] = sum64 / total64 * gating;
                if (bound) bound[at] = largest * (std::expm1(2.0 * error) + gamma(8 * length + 32) + 16.0 * std::ldexp(1.0, -24));
            }
        }
}

// gpu/ops.hpp:1240-1297 (op_sparse_attention_kernel: the definition), gpu/ops.hpp:1309-1327 and
// 1366-1377 (key order; q's last rope_dims rotated in adjacent pairs by double(p) * double(freq), in
// double, rounded to F32), gpu/ops.hpp:1528-1538 (the output rotated back by that angle times -1.0,
// its own sincos), gpu/ops.hpp:1561-1583 (sink in the max and the denominator).
// compressed_bf16 != 0: `compressed` holds BF16 rows (uint16 bits), else F32 rows.
// accumulate64: scores and sums in F64 (crates/straydog-engine/examples/ds41_reference.rs:385-411).
void orc_sparse_attention(const float* q, const float* raw, uint64_t raw_rows, const int32_t* positions, uint64_t window,
                          const void* compressed, int compressed_bf16, const int32_t* selected, uint64_t selections,
                          const float* sinks, uint64_t rows, uint64_t heads, uint64_t dim, float scale, uint64_t rope_dims,
                          const float* frequencies, int accumulate64, float* out) {
    const uint64_t pairs = rope_dims / 2, rotated = dim - rope_dims;
    #pragma omp parallel for collapse(2) schedule(dynamic)
    for (uint64_t row = 0; row < rows; ++row)
        for (uint64_t head = 0; head < heads; ++head) {
            const int64_t p = positions[row];
            const int64_t first = p - int64_t(window) + 1 < 0 ? 0 : p - int64_t(window) + 1;
            const uint64_t raw_count = uint64_t(p - first + 1), total = raw_count + selections;
            std::vector<float> query(q + (row * heads + head) * dim, q + (row * heads + head + 1) * dim);
            for (uint64_t pair = 0; pair < pairs; ++pair) {
                const double angle = double(p) * double(frequencies[pair]);
                const double c = std::cos(angle), s = std::sin(angle);
                const double a = query[rotated + 2 * pair], b = query[rotated + 2 * pair + 1];
                query[rotated + 2 * pair] = float(a * c - b * s);
                query[rotated + 2 * pair + 1] = float(a * s + b * c);
            }
            std::vector<float> key_row(dim);
            const auto key = [&](uint64_t index, float* into) -> bool {
                if (index < raw_count) {
                    std::memcpy(into, raw + uint64_t(first + int64_t(index)) % raw_rows * dim, dim * 4);
                    return true;
                }
                const int32_t at = selected[row * selections + (index - raw_count)];
                if (at < 0) return false;
                if (compressed_bf16) {
                    const uint16_t* halves = static_cast<const uint16_t*>(compressed) + uint64_t(at) * dim;
                    for (uint64_t i = 0; i < dim; ++i) into[i] = bf16_to_f32(halves[i]);
                } else std::memcpy(into, static_cast<const float*>(compressed) + uint64_t(at) * dim, dim * 4);
                return true;
            };
            std::vector<double> scores(total);
            double top = sinks[head];
            for (uint64_t index = 0; index < total; ++index) {
                if (!key(index, key_row.data())) { scores[index] = -INFINITY; continue; }
                if (accumulate64) {
                    double dot = 0;
                    for (uint64_t i = 0; i < dim; ++i) dot += double(query[i]) * double(key_row[i]);
                    scores[index] = dot * double(scale);
                } else {
                    float dot = 0;
                    for (uint64_t i = 0; i < dim; ++i) dot = std::fmaf(query[i], key_row[i], dot);
                    scores[index] = double(dot * scale);
                }
                top = std::max(top, scores[index]);
            }
            std::vector<double> acc(dim, 0.0);
            std::vector<float> acc32(dim, 0.0f);
            double sum = 0;
            float sum32 = 0;
            for (uint64_t index = 0; index < total; ++index) {
                if (scores[index] == -INFINITY) continue;
                key(index, key_row.data());
                if (accumulate64) {
                    const double w = std::exp(scores[index] - top);
                    sum += w;
                    for (uint64_t i = 0; i < dim; ++i) acc[i] += w * double(key_row[i]);
                } else {
                    const float w = std::exp(float(scores[index]) - float(top));
                    if (w == 0.0f) continue;
                    sum32 += w;
                    for (uint64_t i = 0; i < dim; ++i) acc32[i] = std::fmaf(w, key_row[i], acc32[i]);
                }
            }
            float* o = out + (row * heads + head) * dim;
            if (accumulate64) {
                const double denominator = sum + std::exp(double(sinks[head]) - top);
                for (uint64_t i = 0; i < dim; ++i) o[i] = float(acc[i] / denominator);
            } else {
                const float denominator = sum32 + std::exp(sinks[head] - float(top));
                for (uint64_t i = 0; i < dim; ++i) o[i] = acc32[i] / denominator;
            }
            for (uint64_t pair = 0; pair < pairs; ++pair) {
                const double angle = double(p) * double(frequencies[pair]) * -1.0;
                const double c = std::cos(angle), s = std::sin(angle);
                const double a = o[rotated + 2 * pair], b = o[rotated + 2 * pair + 1];
                o[rotated + 2 * pair] = float(a * c - b * s);
                o[rotated + 2 * pair + 1] = float(a * s + b * c);
            }
        }
}

// crates/straydog-engine/tests/fused_gpu.rs:325-357 (top_k_key, top_k_reference): the rule
// gpu/ops.hpp:1766-1941 (top_k_row) implements. out [rows][k] int32, ascending index order, -1 padding.
void orc_top_k(const float* scores, uint64_t rows, uint64_t groups, uint64_t k, int32_t* out) {
    const auto key_of = [](float value) {
        if (value == 0.0f) value = 0.0f;   // -0 ties +0
        uint32_t bits;
        std::memcpy(&bits, &value, 4);
        return bits & 0x80000000u ? ~bits : bits | 0x80000000u;
    };
    const uint32_t floor = key_of(-INFINITY);
    #pragma omp parallel for schedule(dynamic)
    for (uint64_t row = 0; row < rows; ++row) {
        const float* s = scores + row * groups;
        std::vector<uint32_t> keys(groups);
        std::vector<uint64_t> live;
        for (uint64_t g = 0; g < groups; ++g) {
            keys[g] = key_of(s[g]);
            if (keys[g] > floor) live.push_back(g);
        }
        std::vector<int32_t> kept;
        if (live.size() <= k) for (uint64_t g : live) kept.push_back(int32_t(g));
        else {
            std::vector<uint32_t> sorted;
            for (uint64_t g : live) sorted.push_back(keys[g]);
            std::nth_element(sorted.begin(), sorted.begin() + (k - 1), sorted.end(), std::greater<uint32_t>());
            const uint32_t threshold = sorted[k - 1];
            uint64_t above = 0;
            for (uint64_t g : live) above += keys[g] > threshold;
            uint64_t need = k - above;
            for (uint64_t g : live) {
                if (keys[g] > threshold) kept.push_back(int32_t(g));
                else if (keys[g] == threshold && need > 0) { kept.push_back(int32_t(g)); --need; }
            }
        }
        kept.resize(k, -1);
        std::memcpy(out + row * k, kept.data(), k * 4);
    }
}

// gpu/ops.hpp:107-120 (op_rope_kernel): the last 2 * pairs values of each of rows x vectors vectors of `width`, rotated in adjacent
// pairs by positions[row] * frequencies[pair] (times -1.0 with `inverse`), angle and rotation in double, in place.
void orc_rope(float* x, uint64_t rows, uint64_t vectors, uint64_t width, uint64_t rope_dims, const int32_t* positions,
              const float* frequencies, int inverse) {
    const uint64_t pairs = rope_dims / 2;
    for (uint64_t row = 0; row < rows; ++row)
        for (uint64_t vector = 0; vector < vectors; ++vector)
            for (uint64_t pair = 0; pair < pairs; ++pair) {
                float* v = x + (row * vectors + vector) * width + (width - rope_dims) + 2 * pair;
                const double angle = double(positions[row]) * double(frequencies[pair]) * (inverse ? -1.0 : 1.0);
                const double s = std::sin(angle), c = std::cos(angle), a = v[0], b = v[1];
                v[0] = float(a * c - b * s);
                v[1] = float(a * s + b * c);
            }
}

// gpu/ops.hpp:1679-1695 (op_compress_kernel): `ratio` rows pooled per group and channel by the softmax of the gate; the weighted sum
// one chain of fused multiply-adds over the rows in order (what the kernel's `acc += w * kv` compiles to), the weights' sum plain adds.
void orc_compress(const float* kv, const float* gate, uint64_t groups, uint64_t ratio, uint64_t dim, float* out) {
    for (uint64_t group = 0; group < groups; ++group)
        for (uint64_t col = 0; col < dim; ++col) {
            if (!gate) { out[group * dim + col] = kv[group * dim + col]; continue; }
            float top = -INFINITY;
            for (uint64_t r = 0; r < ratio; ++r) top = std::fmax(top, gate[(group * ratio + r) * dim + col]);
            float sum = 0.0f, acc = 0.0f;
            for (uint64_t r = 0; r < ratio; ++r) {
                const float w = std::exp(gate[(group * ratio + r) * dim + col] - top);
                sum += w;
                acc = std::fmaf(w, kv[(group * ratio + r) * dim + col], acc);
            }
            out[group * dim + col] = acc / sum;
        }
}

// gpu/ops.hpp:1697-1745 (op_index_scores_kernel), with gpu/ops.hpp:1942-1951 (index_candidate) when `candidates` is given (then the
// scores are rows x blocks * block in candidate order, as gpu/ops.hpp:1978-2075 stores them). A dot is one chain of fused multiply-adds
// over the columns in order from 0; a head's term relu(dot) * weight, one rounded product; the terms added in head order; then * scale.
// keys_bf16: the keys are BF16 halves (widened exactly).
void orc_index_scores(const float* q, const void* keys, int keys_bf16, const float* weights, const int32_t* visible, uint64_t rows, uint64_t groups,
                      uint64_t heads, uint64_t dim, float scale, const int32_t* candidates, uint64_t blocks, uint64_t block, float* scores) {
    const uint64_t scored = candidates ? blocks * block : groups;
    #pragma omp parallel for collapse(2) schedule(static)
    for (uint64_t row = 0; row < rows; ++row)
        for (uint64_t place = 0; place < scored; ++place) {
            const uint64_t limit = std::min<uint64_t>(groups, uint64_t(std::max(visible[row], 0)));
            uint64_t g = place;
            if (candidates) { const int32_t b = candidates[row * blocks + place / block]; g = b < 0 ? groups : uint64_t(b) * block + place % block; }
            if (g >= limit) { scores[row * scored + place] = -INFINITY; continue; }
            float total = 0.0f;
            for (uint64_t h = 0; h < heads; ++h) {
                const float* qv = q + (row * heads + h) * dim;
                float acc = 0.0f;
                for (uint64_t d = 0; d < dim; ++d) {
                    float k;
                    if (keys_bf16) { const uint32_t bits = uint32_t(static_cast<const uint16_t*>(keys)[g * dim + d]) << 16; std::memcpy(&k, &bits, 4); }
                    else k = static_cast<const float*>(keys)[g * dim + d];
                    acc = std::fmaf(qv[d], k, acc);
                }
                const float term = std::fmax(acc, 0.0f) * weights[row * heads + h];
                total += term;
            }
            scores[row * scored + place] = total * scale;
        }
}

// The projection of sd_op_index_select_proj (gpu/kernels.cpp:5620-5667): out[h] = W[h] . x, W [rows][cols] of kind 0 (F32), 1 (F16) or 30
// (BF16), in the order the reference's GEMV sums a matrix of so few rows (gpu/gemv.hpp:24-36: 32 lanes a row; gpu/gemv_common.hpp:42-86,
// 784-812): lane l takes the units l, l + 32, ... (4 F32 values: a chain from the last inwards; 8 halves: a chain from the first), adds them
// in order, and the lanes meet in a butterfly (xor 16 .. 1). `units` = 0: the element path of gpu/gemv_common.hpp:814-836 (a matrix or an
// input off 16-byte alignment, or a width that is no whole number of units): lane l takes the columns l, l + 32, ... in one chain.
void orc_index_proj(const void* w, int kind, uint64_t rows, uint64_t cols, const float* x, int units, float* out) {
    auto at = [&](uint64_t row, uint64_t col) -> float {
        if (kind == 0) return static_cast<const float*>(w)[row * cols + col];
        const uint16_t bits = static_cast<const uint16_t*>(w)[row * cols + col];
        if (kind == 1) return f16_to_f32(bits);
        uint32_t wide = uint32_t(bits) << 16;
        float value;
        std::memcpy(&value, &wide, 4);
        return value;
    };
    for (uint64_t row = 0; row < rows; ++row) {
        float lanes[32];
        for (uint64_t lane = 0; lane < 32; ++lane) {
            float sum = 0.0f;
            if (!units) {
                for (uint64_t col = lane; col < cols; col += 32) sum = std::fmaf(at(row, col), x[col], sum);
            } else if (kind == 0) {
                for (uint64_t unit = lane; unit < cols / 4; unit += 32) {
                    const uint64_t c = unit * 4;
                    sum += std::fmaf(at(row, c), x[c], std::fmaf(at(row, c + 1), x[c + 1], std::fmaf(at(row, c + 2), x[c + 2], at(row, c + 3) * x[c + 3])));
                }
            } else {
                for (uint64_t unit = lane; unit < cols / 8; unit += 32) {
                    const uint64_t c = unit * 8;
                    float dot = at(row, c) * x[c];
                    for (uint64_t i = 1; i < 8; ++i) dot = std::fmaf(at(row, c + i), x[c + i], dot);
                    sum += dot;
                }
            }
            lanes[lane] = sum;
        }
        for (uint64_t offset = 16; offset; offset /= 2) {
            float next[32];
            for (uint64_t lane = 0; lane < 32; ++lane) next[lane] = lanes[lane] + lanes[lane ^ offset];
            std::memcpy(lanes, next, sizeof(lanes));
        }
        out[row] = lanes[0];
    }
}

// gpu/ops.hpp:1952-1966 (op_index_block_tops_kernel): a block's highest score, +inf for the block of the row's last visible group.
void orc_index_block_tops(const float* scores, const int32_t* visible, uint64_t rows, uint64_t groups, uint64_t block, float* tops) {
    const uint64_t count = (groups + block - 1) / block;
    for (uint64_t row = 0; row < rows; ++row) {
        const uint64_t seen = std::min<uint64_t>(groups, uint64_t(std::max(visible[row], 0)));
        for (uint64_t b = 0; b < count; ++b) {
            float top = seen && b == (seen - 1) / block ? INFINITY : -INFINITY;
            for (uint64_t g = b * block, end = std::min(groups, g + block); g < end; ++g) top = std::fmax(top, scores[row * groups + g]);
            tops[row * count + b] = top;
        }
    }
}

// gpu/sparse_attention.hpp:141-157 (qsa_block_scores; :247-296 its tiled twin with the same bits) and :172-243 (qsa_select): a row at
// position p has complete = (p + 1) / 4 whole blocks; up to 512, every position 0 .. p; more, the 512 blocks of highest score (a dot =
// one chain of fused multiply-adds over the 128 columns, the four heads' positive parts added in head order), equal scores by lowest
// block, in block order, four positions each, then the positions of the incomplete block. Lists and counts go into `packed`.
void orc_qsa_index_select(const float* queries, uint64_t query_stride, const float* blocks, uint64_t pool, uint64_t base, const uint32_t* positions,
                          uint64_t steps, uint64_t selected, uint64_t row_floats, float* packed) {
    const uint64_t index_start = steps * row_floats;
    #pragma omp parallel for schedule(dynamic)
    for (uint64_t token = 0; token < steps; ++token) {
        const uint64_t position = positions ? positions[token] : base + token, complete = (position + 1) / 4;
        float* indices = packed + index_start + token * selected;
        if (complete <= 512) {
            for (uint64_t i = 0; i <= position; ++i) indices[i] = float(i);
            packed[index_start + steps * selected + token] = float(position + 1);
            continue;
        }
        std::vector<float> scores(complete);
        for (uint64_t block = 0; block < complete; ++block) {
            float sums[4] = {0, 0, 0, 0};
            for (uint64_t col = 0; col < 128; ++col) {
                const float key = blocks[col * pool + block];
                for (int h = 0; h < 4; ++h) sums[h] = std::fmaf(key, queries[token * query_stride + h * 128 + col], sums[h]);
            }
            scores[block] = std::fmax(sums[0], 0.0f) + std::fmax(sums[1], 0.0f) + std::fmax(sums[2], 0.0f) + std::fmax(sums[3], 0.0f);
        }
        std::vector<uint32_t> order(complete);
        for (uint64_t i = 0; i < complete; ++i) order[i] = uint32_t(i);
        std::stable_sort(order.begin(), order.end(), [&](uint32_t x, uint32_t y) { return scores[x] > scores[y]; });   // (stable: equal scores by block)
        std::vector<uint32_t> kept(order.begin(), order.begin() + 512);
        std::sort(kept.begin(), kept.end());
        for (uint64_t j = 0; j < 512; ++j)
            for (uint64_t tap = 0; tap < 4; ++tap) indices[4 * j + tap] = float(uint64_t(kept[j]) * 4 + tap);
        for (uint64_t i = 0; complete * 4 + i <= position; ++i) indices[2048 + i] = float(complete * 4 + i);
        packed[index_start + steps * selected + token] = float(2048 + position + 1 - complete * 4);
    }
}

// gpu/sparse_attention.hpp:2-6 (qsa_rope): column c < 64 turns with its partner (c + 32) % 64 by position / 1e7^((c % 32) / 32);
// columns from 64 on pass. (The kernel's own * cos + partner * sin is written out as the two products and their sum.)
static float qsa_rope(float own, float partner, uint64_t column, uint64_t position) {
    if (column >= 64) return own;
    const float angle = float(position) / std::pow(1e7f, float(column % 32) / 32.0f);
    return own * std::cos(angle) + (column < 32 ? -partner : partner) * std::sin(angle);
}
// gpu/sparse_attention.hpp:27-32 (qsa_rope_axes): a row of a sequence with images has a position for each axis (t, h, w); pair p of
// the 32 turns by the position of axis p % 3. No table: qsa_rope.
static float qsa_rope_at(float own, float partner, uint64_t column, uint64_t position, const uint32_t* axes) {
    if (!axes) return qsa_rope(own, partner, column, position);
    if (column >= 64) return own;
    const uint64_t pair = column % 32;
    const float angle = float(axes[pair % 3]) / std::pow(1e7f, float(pair) / 32.0f);
    return own * std::cos(angle) + (column < 32 ? -partner : partner) * std::sin(angle);
}
// The sum of width squares as the reference's shared-memory loop forms it: column c takes c + width / 2, then c + width / 4, ...
static float qsa_halving_sum(float* sums, uint64_t width) {
    for (uint64_t offset = width / 2; offset; offset /= 2)
        for (uint64_t c = 0; c < offset; ++c) sums[c] += sums[c + offset];
    return sums[0];
}
// gpu/sparse_attention.hpp:55-71 (qsa_normalize_block): one head of `width` columns, RMS-normalised, scaled by `norm`, rotated.
static void qsa_normalize_head(const float* source, const float* norm, uint64_t width, uint64_t position, float* target,
                               const uint32_t* axes = nullptr) {
    float values[256], sums[256];
    for (uint64_t c = 0; c < width; ++c) { values[c] = source[c] * norm[c]; sums[c] = source[c] * source[c]; }
    const float denominator = std::sqrt(qsa_halving_sum(sums, width) / float(width) + 1e-6f);
    float result[256];
    for (uint64_t c = 0; c < width; ++c) {
        const float own = values[c] / denominator, partner = c < 64 ? values[(c + 32) % 64] / denominator : 0.0f;
        result[c] = qsa_rope_at(own, partner, c, position, axes);
    }
    std::memcpy(target, result, width * sizeof(float));   // (the index queries are normalised in place)
}
// gpu/qsa_decode.hpp:86-111 (qsa_normalize_rows) with :51-83 (qsa_pool_rows_block; for one row :5-23, qsa_pool_one): the rows'
// queries and keys normalised and rotated into `packed` ([rows][heads][256] | [rows][kv_heads][256] | ...), the keys (normalised)
// and values encoded into row positions[r] of the Q8_0 state, the four index-query heads normalised in place, the index keys passed
// through the history ring (16 positions) and pooled four by four into blocks[column][position / 4]. index_state: [128][pool]
// blocks, then the ring [16][128]. A projections row: qgate [heads][512] | key [kv][256] | value [kv][256] | index query [4][128] |
// index key [128].
void orc_qsa_normalize_rows(float* projections, uint64_t stride, uint64_t rows, uint64_t heads, uint64_t kv_heads, const float* qnorm,
                            const float* knorm, const float* iqnorm, const float* pool_norm, const uint32_t* positions,
                            const uint32_t* ropes, float* packed, uint8_t* state, uint64_t context, float* index_state) {
    const uint64_t keys = heads * 512, values = keys + kv_heads * 256, index = keys + kv_heads * 512, pool = context / 4 + 1;
    for (uint64_t row = 0; row < rows; ++row) {
        float* own = projections + row * stride;
        for (uint64_t head = 0; head < heads; ++head)
            qsa_normalize_head(own + head * 512, qnorm, 256, ropes[row], packed + (row * heads + head) * 256);
        for (uint64_t head = 0; head < kv_heads; ++head) {
            float* normalized = packed + rows * heads * 256 + (row * kv_heads + head) * 256;
            qsa_normalize_head(own + keys + head * 256, knorm, 256, ropes[row], normalized);
            q8_encode_row(normalized, state + (head * context + positions[row]) * kRowQ8);
            q8_encode_row(own + values + head * 256, state + ((kv_heads + head) * context + positions[row]) * kRowQ8);
        }
        for (uint64_t head = 0; head < 4; ++head)
            qsa_normalize_head(own + index + head * 128, iqnorm, 128, ropes[row], own + index + head * 128);
    }
    float* history = index_state + pool * 128;
    for (uint64_t row = 0; row < rows; ++row) {
        const uint64_t pos = positions[row];
        for (uint64_t c = 0; c < 128; ++c) history[(pos % 16) * 128 + c] = projections[row * stride + index + 512 + c];
        if ((pos + 1) % 4) continue;
        float vals[128], sums[128];
        for (uint64_t c = 0; c < 128; ++c) {
            float x = 0.0f;
            for (uint64_t tap = 0; tap < 4; ++tap) x += history[((pos - 3 + tap) % 16) * 128 + c];
            x /= 4.0f;
            vals[c] = x * pool_norm[c]; sums[c] = x * x;
        }
        const float denominator = std::sqrt(qsa_halving_sum(sums, 128) / 128.0f + 1e-6f);
        for (uint64_t c = 0; c < 128; ++c) {
            const float value = vals[c] / denominator, partner = c < 64 ? vals[(c + 32) % 64] / denominator : 0.0f;
            index_state[c * pool + pos / 4] = qsa_rope(value, partner, c, uint64_t(ropes[row]) - 3);
        }
    }
}

// A prompt chunk's front (gpu/prefill_batch.hpp:342-370 and gpu/sparse_attention.hpp:493-506: qsa_normalize of the queries, keys and
// index queries, the values copied into the packed rows, qsa_pool :87-106 over the blocks the chunk completes, qsa_save_history
// :135-139, write_attention_kv): `count` tokens from `position`, a token's rotation position its own. The arrays: qgate
// [count][heads][512], key and value [count][kv_heads][256], iq [count][4][128] (normalised in place), ik [count][128].
void orc_qsa_normalize_chunk(const float* qgate, const float* key, const float* value, float* iq, const float* ik, uint64_t count,
                             uint64_t position, uint64_t heads, uint64_t kv_heads, const float* qnorm, const float* knorm,
                             const float* iqnorm, const float* pool_norm, float* packed, uint8_t* state, uint64_t context,
                             float* index_state, const uint32_t* rope_rows, uint64_t rope_first) {
    // (rope_rows: the table of a sequence with images, three positions a row from rope_first, gpu/prefill_batch.hpp:344 and :360-362
    // with qsa_normalize_axes / qsa_pool_axes, gpu/sparse_attention.hpp:36-50, 111-131; null: every token turns at its own position)
    const uint64_t pool = context / 4 + 1, Q = heads * 256, K = kv_heads * 256;
    for (uint64_t t = 0; t < count; ++t) {
        const uint32_t* axes = rope_rows ? rope_rows + (position + t - rope_first) * 3 : nullptr;
        for (uint64_t head = 0; head < heads; ++head)
            qsa_normalize_head(qgate + (t * heads + head) * 512, qnorm, 256, position + t, packed + t * Q + head * 256, axes);
        for (uint64_t head = 0; head < kv_heads; ++head) {
            float* normalized = packed + count * Q + t * K + head * 256;
            qsa_normalize_head(key + t * K + head * 256, knorm, 256, position + t, normalized, axes);
            std::memcpy(packed + count * (Q + K) + t * K + head * 256, value + t * K + head * 256, 256 * sizeof(float));
            q8_encode_row(normalized, state + (head * context + position + t) * kRowQ8);
            q8_encode_row(value + t * K + head * 256, state + ((kv_heads + head) * context + position + t) * kRowQ8);
        }
        for (uint64_t head = 0; head < 4; ++head)
            qsa_normalize_head(iq + t * 512 + head * 128, iqnorm, 128, position + t, iq + t * 512 + head * 128, axes);
    }
    float* history = index_state + pool * 128;
    for (uint64_t block = position / 4; block < (position + count) / 4; ++block) {
        const uint64_t begin = block * 4;
        float vals[128], sums[128];
        for (uint64_t c = 0; c < 128; ++c) {
            float x = 0.0f;
            for (uint64_t tap = 0; tap < 4; ++tap) {
                const uint64_t pos = begin + tap;
                x += pos < position ? history[(pos % 16) * 128 + c] : ik[(pos - position) * 128 + c];
            }
            x /= 4.0f;
            vals[c] = x * pool_norm[c]; sums[c] = x * x;
        }
        const float denominator = std::sqrt(qsa_halving_sum(sums, 128) / 128.0f + 1e-6f);
        for (uint64_t c = 0; c < 128; ++c) {
            const float own = vals[c] / denominator, partner = c < 64 ? vals[(c + 32) % 64] / denominator : 0.0f;
            index_state[c * pool + block] = qsa_rope_at(own, partner, c, begin, rope_rows ? rope_rows + (begin - rope_first) * 3 : nullptr);
        }
    }
    const uint64_t kept = count < 4 ? count : 4;
    for (uint64_t t = count - kept; t < count; ++t) std::memcpy(history + ((position + t) % 16) * 128, ik + t * 128, 128 * sizeof(float));
}

// gpu/dspark_attention.hpp:9-100 (dspark_attention_kernel) and crates/straydog-engine/tests/dspark_attention_gpu.rs:25-39 (its F64
// oracle): every query row [slots][heads][512] attends the ring's history positions [anchor - history, anchor) (ring of 128 rows,
// K = V) and all `slots` block keys; scale 1 / sqrt(512); the head's sink in the maximum and in the denominator.
// accumulate64 = 0: the kernel's FP32 arithmetic (a score one chain of fused multiply-adds over the columns in order, an output
// column one chain over the keys in order); 1: F64 throughout.
void orc_dspark_attention(const float* q, const float* ring, const float* block, const float* sinks, uint64_t heads, uint64_t slots,
                          uint64_t anchor, uint64_t history, int accumulate64, float* out) {
    constexpr uint64_t dim = 512, ring_rows = 128;
    const uint64_t first = anchor >= history ? anchor - history : 0, raw_count = anchor - first, total = raw_count + slots;
    auto key = [&](uint64_t index) { return index < raw_count ? ring + (first + index) % ring_rows * dim : block + (index - raw_count) * dim; };
    #pragma omp parallel for schedule(dynamic)
    for (uint64_t item = 0; item < slots * heads; ++item) {
        const float* query = q + item * dim;
        const double sink = sinks[item % heads];
        std::vector<double> scores(total);
        double top = sink;
        for (uint64_t i = 0; i < total; ++i) {
            if (accumulate64) {
                double dot = 0;
                for (uint64_t d = 0; d < dim; ++d) dot += double(query[d]) * double(key(i)[d]);
                scores[i] = dot / std::sqrt(double(dim));
            } else {
                float dot = 0;
                for (uint64_t d = 0; d < dim; ++d) dot = std::fmaf(query[d], key(i)[d], dot);
                scores[i] = dot * (1.0f / std::sqrt(float(dim)));
            }
            top = std::max(top, scores[i]);
        }
        double denominator = 0;
        for (uint64_t i = 0; i < total; ++i) {
            scores[i] = accumulate64 ? std::exp(scores[i] - top) : double(std::exp(float(scores[i]) - float(top)));
            denominator = accumulate64 ? denominator + scores[i] : double(float(denominator) + float(scores[i]));
        }
        denominator = accumulate64 ? denominator + std::exp(sink - top) : double(float(denominator) + std::exp(float(sink) - float(top)));
        for (uint64_t d = 0; d < dim; ++d) {
            if (accumulate64) {
                double sum = 0;
                for (uint64_t i = 0; i < total; ++i) sum += scores[i] * double(key(i)[d]);
                out[item * dim + d] = float(sum / denominator);
            } else {
                float sum = 0;
                for (uint64_t i = 0; i < total; ++i) sum = std::fmaf(float(scores[i]), key(i)[d], sum);
                out[item * dim + d] = sum / float(denominator);
            }
        }
    }
}

// gpu/straydog_gpu.h:458-459 (sd_op_to_bf16: nearest, ties to even); tests/ds_state_bf16_gpu.rs:27-37.
void orc_to_bf16(const float* x, uint64_t count, uint16_t* out) {
    for (uint64_t i = 0; i < count; ++i) out[i] = f32_to_bf16(x[i]);
}

// torchrun exports OMP_NUM_THREADS=1 to its ranks: the timed baseline asks for the host's cores explicitly.
void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_threads(void) {
#ifdef _OPENMP
    int n = 1;
    #pragma omp parallel
    {
        #pragma omp single
        n = omp_get_num_threads();
    }
    return n;
#else
    return 1;
#endif
}

}  // extern "C"
