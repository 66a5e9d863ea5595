// CPU oracle, TEST INFRASTRUCTURE ONLY: the 2:4 keep-mask of
// compressors/sparse_compressors/sparse_24_bitmask.py:227-260 get_24_bytemasks.
//
// The reference takes abs() of every run of 4 consecutive elements (flat view) and keeps the
// two positions returned by torch.topk(2).  torch's CPU top-k for a slice this small is
// std::nth_element on (value, index) pairs with the comparator "NaN first, then greater",
// followed by a sort of the leading k-1 entries; which index survives a tie is therefore
// whatever libstdc++'s introselect does.  This file restates that by calling the same
// standard-library algorithm with the same comparator.  fp8 tensors are ranked by the
// absolute value of their int8 bit pattern (sparse_24_bitmask.py:244-245), where abs(-128)
// wraps to -128.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <utility>
#include <vector>

namespace {

template <typename T>
inline bool is_nan(T) { return false; }
template <>
inline bool is_nan<float>(float v) { return std::isnan(v); }

template <typename T>
inline unsigned keep_mask(const T a[4]) {
    std::vector<std::pair<T, int64_t>> queue(4);
    for (int64_t j = 0; j < 4; ++j) queue[j] = {a[j], j};
    auto cmp = [](const std::pair<T, int64_t>& x, const std::pair<T, int64_t>& y) -> bool {
        return (is_nan<T>(x.first) && !is_nan<T>(y.first)) || (x.first > y.first);
    };
    const int k = 2;
    std::nth_element(queue.begin(), queue.begin() + k - 1, queue.end(), cmp);
    std::sort(queue.begin(), queue.begin() + k - 1, cmp);
    return (1u << queue[0].second) | (1u << queue[1].second);
}

inline float bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline float f16_to_f32(uint16_t h) { _Float16 x; std::memcpy(&x, &h, 2); return (float)x; }

}  // namespace

// dtype codes: 0 bf16, 1 f16, 2 f32, 4 int8, 5 e4m3 (ranked through its int8 view)
extern "C" int orc_sparse24_mask(const void* x, int dt, int64_t numel, uint8_t* bytemask) {
    if (numel % 4) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < numel / 4; ++g) {
        unsigned m;
        if (dt == 4 || dt == 5) {
            int8_t a[4];
            for (int j = 0; j < 4; ++j) {
                int8_t v = ((const int8_t*)x)[4 * g + j];
                a[j] = (int8_t)(v < 0 ? (uint8_t)(-(int)v) : v);  // int8 abs, -128 stays -128
            }
            m = keep_mask<int8_t>(a);
        } else {
            float a[4];
            for (int j = 0; j < 4; ++j) {
                float v = dt == 0 ? bf16_to_f32(((const uint16_t*)x)[4 * g + j])
                        : dt == 1 ? f16_to_f32(((const uint16_t*)x)[4 * g + j])
                                  : ((const float*)x)[4 * g + j];
                a[j] = std::fabs(v);
            }
            m = keep_mask<float>(a);
        }
        for (int j = 0; j < 4; ++j) bytemask[4 * g + j] = (m >> j) & 1u;
    }
    return 0;
}
