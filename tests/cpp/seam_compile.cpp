// include/qsa_b200.hpp compiled against stand-ins for the reference's declarations it relies on (Device with ordinal, stream
// and kv_row; QwenHeads<P>::query / ::kv; kv_t; kv_row_q8; qsa_flash_launch<P>): the two seam functions must instantiate with
// the reference's call shapes (gpu/qsa_decode.hpp:42,126) and link against the library. Nothing runs.
#include <cstddef>
#include <cstdint>

typedef uint8_t kv_t;
constexpr unsigned kv_row_q8 = 272;
struct dim3 { unsigned x, y, z; dim3(unsigned a = 1, unsigned b = 1, unsigned c = 1) : x(a), y(b), z(c) {} };
struct Device { int ordinal = 0; void* stream = nullptr; unsigned kv_row = kv_row_q8; };
template <int P> struct QwenHeads { static constexpr size_t query = 24 / P, kv = 2 / P; };
template <int P> void qsa_flash_launch(Device&, dim3, const kv_t*, size_t, size_t, size_t, size_t, const float*, float*, size_t = 0) {}

#define QSA_B200_REFERENCE_TYPES
#include "qsa_b200.hpp"

int main(int argc, char**) {
    if (argc > 100) {   // instantiated, never run
        Device d;
        qsa_attention<1>(d, nullptr, 0, 0, 1, 2052, nullptr, nullptr, nullptr, nullptr, 0);
        qsa_attention<2>(d, nullptr, 0, 0, 1, 2052, nullptr, nullptr);
        qsa_attention_rows<1>(d, nullptr, 0, 8, 2052, nullptr, nullptr, nullptr, nullptr, 0, nullptr, 0);
        qsa_attention_rows<2>(d, nullptr, 0, 8, 2052, nullptr, nullptr, nullptr);
    }
    return 0;
}
