// Host build of the SIMD 2:4 selection (compressed_tensors_b200/csrc/ctb_sparse24_simd.cuh) for the CPU test
// suite: the same bit logic the CUDA kernels run, exported over flat arrays so that it can be compared with the
// oracle on every weak ordering and on random data without a GPU.
#include <cstdint>
#include <cstring>

#include "ctb_sparse24_simd.cuh"

extern "C" {

// x: n16 * 16 int8-view elements -> values: n16 * 8 bytes, mask: n16 * 2 bytes
void simd24_pack_u8(const uint8_t *x, int64_t n16, uint8_t *values, uint8_t *mask) {
    for (int64_t i = 0; i < n16; ++i) {
        uint32_t w[4], v0, v1, m;
        std::memcpy(w, x + 16 * i, 16);
        ctb::sparse24_pack_u8x16(w[0], w[1], w[2], w[3], v0, v1, m);
        std::memcpy(values + 8 * i, &v0, 4);
        std::memcpy(values + 8 * i + 4, &v1, 4);
        mask[2 * i] = (uint8_t)m;
        mask[2 * i + 1] = (uint8_t)(m >> 8);
    }
}

// x: n8 * 8 16-bit elements -> values: n8 * 4 elements, mask: n8 bytes
void simd24_pack_u16(const uint16_t *x, int64_t n8, uint16_t *values, uint8_t *mask) {
    for (int64_t i = 0; i < n8; ++i) {
        uint32_t w[4], v0, v1, m;
        std::memcpy(w, x + 8 * i, 16);
        ctb::sparse24_pack_u16x8(w[0], w[1], w[2], w[3], v0, v1, m);
        std::memcpy(values + 4 * i, &v0, 4);
        std::memcpy(values + 4 * i + 2, &v1, 4);
        mask[i] = (uint8_t)m;
    }
}

// x: n16 * 16 int8-view elements -> mask: one 0/1 byte per element
void simd24_bytemask_u8(const uint8_t *x, int64_t n16, uint8_t *mask) {
    for (int64_t i = 0; i < n16; ++i) {
        uint32_t w[4], o[4];
        std::memcpy(w, x + 16 * i, 16);
        ctb::sparse24_bytemask_u8x16(w[0], w[1], w[2], w[3], o[0], o[1], o[2], o[3]);
        std::memcpy(mask + 16 * i, o, 16);
    }
}

// x: n8 * 8 16-bit elements -> mask: one 0/1 byte per element
void simd24_bytemask_u16(const uint16_t *x, int64_t n8, uint8_t *mask) {
    for (int64_t i = 0; i < n8; ++i) {
        uint32_t w[4], o[2];
        std::memcpy(w, x + 8 * i, 16);
        ctb::sparse24_bytemask_u16x8(w[0], w[1], w[2], w[3], o[0], o[1]);
        std::memcpy(mask + 8 * i, o, 8);
    }
}
}
