// Parity of the attention path through the C++ host mirror (include/straydog_b200.hpp), in the manner of the reference's
// own model-free GPU tests (crates/straydog-engine/tests/attention_gpu.rs, ds_state_bf16_gpu.rs): seeded inputs, an F64
// restatement computed here, the library's outputs held to it. Prints "ok <checks>" and exits 0, or the first failure and 1.
#include "straydog_b200.hpp"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>

using namespace straydog;

namespace {

struct Random {   // xorshift64
    uint64_t state;
    explicit Random(uint64_t seed) : state(seed ? seed : 1) {}
    uint64_t next() { state ^= state << 13; state ^= state >> 7; state ^= state << 17; return state; }
    float unit() { return float(next() >> 40) / float(1 << 24) * 2.0f - 1.0f; }   // [-1, 1)
};

int failures = 0, checks = 0;
void expect(bool ok, const char* what, double value = 0.0) {
    ++checks;
    if (!ok) { std::printf("FAILED: %s (%g)\n", what, value); ++failures; }
}

// max-abs 2e-3 or max-rel 1e-2 per element
bool close(const std::vector<float>& got, const std::vector<double>& want, double& worst) {
    worst = 0.0;
    bool ok = got.size() == want.size();
    for (size_t i = 0; ok && i < got.size(); ++i) {
        const double error = std::fabs(double(got[i]) - want[i]);
        worst = std::max(worst, error);
        if (!(error <= 2e-3 || error <= 1e-2 * std::fabs(want[i]))) ok = false;
    }
    return ok;
}

// dense causal GQA over F32 K/V [context][kv_heads][dim]: length = min(position + 1, context)
void dense_gqa(Backend& gpu, uint64_t rows, uint64_t heads, uint64_t kv_heads, uint64_t dim, uint64_t context) {
    Random random(0x51ED270B5EEDull ^ rows ^ (dim << 16) ^ (context << 32));
    std::vector<float> q(rows * heads * dim), keys(context * kv_heads * dim), values(keys.size());
    for (auto& x : q) x = random.unit();
    for (auto& x : keys) x = random.unit();
    for (auto& x : values) x = random.unit();
    std::vector<int32_t> positions(rows);
    for (uint64_t r = 0; r < rows; ++r) positions[r] = int32_t(context - rows + r);
    const float scale = 1.0f / std::sqrt(float(dim));
    std::vector<double> want(q.size());
    const uint64_t group = heads / kv_heads;
    for (uint64_t r = 0; r < rows; ++r)
        for (uint64_t h = 0; h < heads; ++h) {
            const uint64_t length = std::min<uint64_t>(uint64_t(positions[r]) + 1, context), kv = h / group;
            std::vector<double> score(length);
            double top = -std::numeric_limits<double>::infinity();
            for (uint64_t k = 0; k < length; ++k) {
                double dot = 0.0;
                for (uint64_t d = 0; d < dim; ++d) dot += double(q[(r * heads + h) * dim + d]) * double(keys[(k * kv_heads + kv) * dim + d]);
                score[k] = dot * scale;
                top = std::max(top, score[k]);
            }
            double denominator = 0.0;
            for (auto& s : score) { s = std::exp(s - top); denominator += s; }
            for (uint64_t d = 0; d < dim; ++d) {
                double sum = 0.0;
                for (uint64_t k = 0; k < length; ++k) sum += score[k] * double(values[(k * kv_heads + kv) * dim + d]);
                want[(r * heads + h) * dim + d] = sum / denominator;
            }
        }
    Buffer qb = gpu.upload(q), kb = gpu.upload(keys), vb = gpu.upload(values), pb = gpu.upload(positions);
    Buffer scratch = gpu.buffer(std::max<uint64_t>(4096, rows * heads * 64 * (dim + 2) * 4)), out = gpu.buffer(q.size() * 4);
    gpu.attention(qb.at<float>(), kb.at<float>(), vb.at<float>(), context, pb.at<int32_t>(), rows, heads, kv_heads, dim, scale, nullptr, scratch,
                  out.at<float>());
    std::vector<float> got(q.size());
    gpu.read_buffer(out, 0, got);
    double worst;
    expect(close(got, want, worst), "dense causal GQA against the F64 restatement", worst);
    for (Buffer* b : {&qb, &kb, &vb, &pb, &scratch, &out}) gpu.release(*b);
}

uint16_t half_bits(float x) {   // round to nearest even, normal range and zero only (the test's values)
    uint32_t bits; std::memcpy(&bits, &x, 4);
    const uint32_t sign = (bits >> 16) & 0x8000u;
    int32_t exponent = int32_t((bits >> 23) & 0xff) - 127 + 15;
    uint32_t mantissa = bits & 0x7fffffu;
    if (exponent <= 0) return uint16_t(sign);
    uint32_t rounded = mantissa + 0xfffu + ((mantissa >> 13) & 1u);
    if (rounded & 0x800000u) { rounded = 0; ++exponent; }
    return uint16_t(sign | uint32_t(exponent << 10) | (rounded >> 13));
}
float half_value(uint16_t h) {
    const uint32_t sign = uint32_t(h & 0x8000u) << 16, exponent = (h >> 10) & 0x1f, mantissa = h & 0x3ffu;
    if (!exponent) return 0.0f;
    const uint32_t bits = sign | ((exponent - 15 + 127) << 23) | (mantissa << 13);
    float x; std::memcpy(&x, &bits, 4); return x;
}

// decode of one sequence over Q8_0 rows written by the library itself (kv_write), against F64 over the decoded rows
void q8_decode(Backend& gpu, uint64_t length) {
    const uint64_t heads = 16, kv_heads = 2, dim = 256, context = length;
    Random random(0xD0D0CAFEull + length);
    std::vector<float> keys(length * kv_heads * dim), values(keys.size());
    for (auto& x : keys) x = random.unit() * 0.7f;
    for (auto& x : values) x = random.unit() * 0.7f;
    gpu.kv_format(272);
    Buffer state = gpu.buffer(context * 2 * kv_heads * 272);
    Buffer kb = gpu.upload(keys), vb = gpu.upload(values);
    gpu.kv_write(state, context, kv_heads, 0, length, kb.at<float>(), vb.at<float>());
    std::vector<uint8_t> packed(state.bytes);
    gpu.read_buffer(state, 0, packed);
    // Q8_0 row: 256 int8 then 8 FP16 block scales; planes: keys of head 0.., then values of head 0..
    auto element = [&](uint64_t plane, uint64_t row, uint64_t d) {
        const uint8_t* at = packed.data() + (plane * context + row) * 272;
        uint16_t scale; std::memcpy(&scale, at + 256 + 2 * (d / 32), 2);
        return double(float(int8_t(at[d])) * half_value(scale));
    };
    expect(std::fabs(element(0, 3, 17) - keys[(3 * kv_heads + 0) * dim + 17]) <= 0.7 / 127.0, "a written key decodes to within half a step of its value");
    std::vector<uint16_t> q(heads * dim);
    std::vector<double> qd(q.size());
    for (size_t i = 0; i < q.size(); ++i) { q[i] = half_bits(random.unit() * 2.0f); qd[i] = half_value(q[i]); }
    std::vector<double> want(heads * dim);
    for (uint64_t h = 0; h < heads; ++h) {
        const uint64_t kv = h / (heads / kv_heads);
        std::vector<double> score(length);
        double top = -std::numeric_limits<double>::infinity();
        for (uint64_t k = 0; k < length; ++k) {
            double dot = 0.0;
            for (uint64_t d = 0; d < dim; ++d) dot += qd[h * dim + d] * element(kv, k, d);
            score[k] = dot * 0.0625;
            top = std::max(top, score[k]);
        }
        double denominator = 0.0;
        for (auto& s : score) { s = std::exp(s - top); denominator += s; }
        for (uint64_t d = 0; d < dim; ++d) {
            double sum = 0.0;
            for (uint64_t k = 0; k < length; ++k) sum += score[k] * element(kv_heads + kv, k, d);
            want[h * dim + d] = sum / denominator;
        }
    }
    Buffer qb = gpu.upload(q), out = gpu.buffer(heads * dim * 4);
    gpu.qsa_decode({state.pointer}, {context}, {length}, heads, kv_heads, 0.0625f, qb.pointer, out.at<float>());
    std::vector<float> got(heads * dim);
    gpu.read_buffer(out, 0, got);
    double worst;
    expect(close(got, want, worst), "Q8_0 GQA decode against the F64 restatement", worst);
    expect(gpu.decode_status() == 0, "no bounded wait gave up");
    for (Buffer* b : {&state, &kb, &vb, &qb, &out}) gpu.release(*b);
}

void errors(Backend& gpu) {
    bool thrown = false;
    try { Buffer b = gpu.buffer(64); float host = 0; gpu.to_bf16(&host, 1, b.pointer); } catch (const Error& e) { thrown = std::strlen(e.what()) > 0; }
    expect(thrown, "a pointer outside the device's allocations is refused with the library's message");
    thrown = false;
    try { Backend other(Backend::device_count() + 7, 1 << 20); } catch (const Error&) { thrown = true; }
    expect(thrown, "an unknown device ordinal is refused");
}

}  // namespace

int main() {
    try {
        Backend gpu(0, 1ull << 30);
        dense_gqa(gpu, 15, 4, 2, 256, 33);
        dense_gqa(gpu, 17, 16, 2, 256, 137);
        dense_gqa(gpu, 1, 2, 1, 128, 35);
        q8_decode(gpu, 700);
        q8_decode(gpu, 4096);
        errors(gpu);
    } catch (const std::exception& e) {
        std::printf("FAILED: %s\n", e.what());
        return 1;
    }
    if (failures) return 1;
    std::printf("ok %d\n", checks);
    return 0;
}
