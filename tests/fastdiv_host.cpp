// Host build of the multiply-high division (compressed_tensors_b200/csrc/ctb_fastdiv.h) for the CPU test suite.
#include <cstdint>

#include "ctb_fastdiv.h"

extern "C" {

// number of n in `ns` (plus the edges 0, d - 1, d, k * d - 1, k * d, 2^31 - 1) where fastdiv(n, d) != n / d
int64_t fastdiv_mismatches(uint32_t d, const uint32_t *ns, int64_t count) {
    const ctb::FastDiv f = ctb::make_fastdiv(d);
    int64_t bad = 0;
    for (int64_t i = 0; i < count; ++i) bad += ctb::fastdiv(ns[i], f) != ns[i] / d;
    const uint32_t top = 0x7FFFFFFFu;
    const uint32_t k = top / d;
    const uint32_t edges[] = {0u, d - 1, d, k * d - 1, k * d, top, top - 1, (k / 2) * d, (k / 2) * d - 1};
    for (uint32_t n : edges)
        if (n <= top) bad += ctb::fastdiv(n, f) != n / d;
    return bad;
}
}
