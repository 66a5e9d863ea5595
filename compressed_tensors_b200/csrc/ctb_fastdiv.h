// Division of a 31-bit number by a run-time constant as a multiply-high, an add and a shift.
// Plain integer logic shared by the CUDA kernels and a host build (tests compile it with g++).
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define CTB_HD __host__ __device__ __forceinline__
#else
#define CTB_HD inline
#endif

namespace ctb {

// For a divisor d >= 1 and l = ceil(log2 d):  mul = floor(2^32 * (2^l - d) / d) + 1.  Then for every n < 2^31
//   n / d == (mulhi(n, mul) + n) >> l          (Granlund & Montgomery, "Division by invariant integers");
// mulhi(n, mul) <= n < 2^31, so the sum stays below 2^32.
struct FastDiv {
    uint32_t mul, shift;
};

inline FastDiv make_fastdiv(uint32_t d) {
    uint32_t l = 0;
    while ((1ull << l) < d) ++l;
    FastDiv f;
    f.mul = (uint32_t)((((1ull << l) - d) << 32) / d + 1);
    f.shift = l;
    return f;
}

CTB_HD uint32_t fastdiv(uint32_t n, FastDiv f) {
#if defined(__CUDA_ARCH__)
    return (__umulhi(n, f.mul) + n) >> f.shift;
#else
    return (uint32_t)((((uint64_t)n * f.mul) >> 32) + n) >> f.shift;
#endif
}

}  // namespace ctb
