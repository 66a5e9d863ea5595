// Sparse codecs: 2:4 keep-mask and compaction (compressors/sparse_compressors/sparse_24_bitmask.py),
// unstructured bitmask compress / decompress (compressors/sparse_compressors/sparse_bitmask.py).
//
// Layout facts shared with the reference: values are row-major, bitmask byte k of a row holds
// columns 8k..8k+7 with column 8k+j in bit j (numpy.packbits, bitorder="little"), row_offsets is the
// int64 exclusive prefix of the per-row counts.
#include <atomic>

#include "ctb_codec.cuh"
#include "ctb_fastdiv.h"
#include "ctb_sparse24_simd.cuh"

namespace ctb {

constexpr int kThreads = 256;

// A kernel launched as the fallback of another one runs only if *flag holds `value`.  The value is a per-call
// ticket rather than 1, so the flag word never has to be cleared between calls: a stale word matches a new ticket
// with probability 2^-32, and a false match only costs the time of the (correct) generic kernels.
struct Gate {
    const int *flag;
    int value;
};


// element classes by storage size; `nz_mask` selects the bits that make an element non-zero
// (sign bit excluded for float types so that -0.0 counts as zero, sparse_bitmask.py:137)
struct ElemInfo {
    int esize;
    uint32_t nz_mask;
    int is_int8;  // magnitudes ranked through the int8 view (int8 and e4m3 tensors)
};

static bool elem_info(int dt, ElemInfo *e) {
    switch (dt) {
    case CTB_BF16: case CTB_F16: *e = {2, 0x7FFFu, 0}; return true;
    case CTB_F32: *e = {4, 0x7FFFFFFFu, 0}; return true;
    case CTB_E4M3: *e = {1, 0x7Fu, 1}; return true;
    case CTB_I8: case CTB_U8: *e = {1, 0xFFu, 1}; return true;
    default: return false;
    }
}

// 8 consecutive elements as raw bit patterns
template <int ES>
__device__ __forceinline__ void load8_bits(const void *x, int64_t unit, uint32_t (&b)[8]) {
    if constexpr (ES == 2) {
        uint4 v = ld_stream((const char *)x + unit * 16);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { b[2 * i] = w[i] & 0xFFFFu; b[2 * i + 1] = w[i] >> 16; }
    } else if constexpr (ES == 1) {
        uint2 v = ld_stream8((const char *)x + unit * 8);
        const uint32_t w[2] = {v.x, v.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = (w[i >> 2] >> (8 * (i & 3))) & 0xFFu;
    } else {
        uint4 v0 = ld_stream((const char *)x + unit * 32), v1 = ld_stream((const char *)x + unit * 32 + 16);
        b[0] = v0.x; b[1] = v0.y; b[2] = v0.z; b[3] = v0.w;
        b[4] = v1.x; b[5] = v1.y; b[6] = v1.z; b[7] = v1.w;
    }
}

__device__ __forceinline__ uint32_t load_bits(const void *x, int es, int64_t i) {
    return es == 1 ? ((const uint8_t *)x)[i] : es == 2 ? ((const uint16_t *)x)[i] : ((const uint32_t *)x)[i];
}
__device__ __forceinline__ void store_bits(void *x, int es, int64_t i, uint32_t v) {
    if (es == 1) ((uint8_t *)x)[i] = (uint8_t)v;
    else if (es == 2) ((uint16_t *)x)[i] = (uint16_t)v;
    else ((uint32_t *)x)[i] = v;
}

// sparse_24_bitmask.py:244-256: magnitude used for ranking.  Float types: |x| orders like its
// magnitude bits.  int8 view (int8 / e4m3 tensors): torch's int8 abs, where abs(-128) wraps to -128.
template <bool IS_INT8>
__device__ __forceinline__ int32_t rank_key(uint32_t bits, uint32_t nz_mask) {
    if constexpr (IS_INT8) {
        int32_t v = (int32_t)(int8_t)bits;
        return (int32_t)(int8_t)(v < 0 ? -v : v);
    } else {
        return (int32_t)(bits & nz_mask);
    }
}

// keep-mask (4 bits) of one run of four magnitudes: the positions abs().topk(2) returns on CPU.
// torch's top-k breaks ties towards the higher index ("i beats j" below), with one family of exceptions
// that comes from the partition step of std::nth_element: when element 0 is strictly the largest and the
// second place is tied, the winner of the tie is fixed per tie set ({1,2}->1, {1,3}->1, {2,3}->2,
// {1,2,3}->2).  The rule is checked against torch.topk on all 75 weak orderings of four values (tests/golden).
__device__ __forceinline__ uint32_t keep24(int32_t k0, int32_t k1, int32_t k2, int32_t k3) {
    const bool b01 = k0 > k1, b02 = k0 > k2, b03 = k0 > k3, b12 = k1 > k2, b13 = k1 > k3, b23 = k2 > k3;
    const int w0 = b01 + b02 + b03, w1 = !b01 + b12 + b13, w2 = !b02 + !b12 + b23, w3 = !b03 + !b13 + !b23;
    uint32_t m = (w0 >= 2 ? 1u : 0u) | (w1 >= 2 ? 2u : 0u) | (w2 >= 2 ? 4u : 0u) | (w3 >= 2 ? 8u : 0u);
    if (b01 && b02 && b03) {
        const int32_t mx = max(k1, max(k2, k3));
        const uint32_t t = (k1 == mx ? 1u : 0u) | (k2 == mx ? 2u : 0u) | (k3 == mx ? 4u : 0u);
        m = 1u | ((0x44282420u >> (4 * t)) & 0xFu);
    }
    return m;
}

// get_24_bytemasks on the flat view: one thread per run of 4
template <bool IS_INT8>
__global__ void __launch_bounds__(kThreads) sparse24_mask_kernel(const void *x, int es, uint32_t nzm, int64_t groups, uint8_t *out) {
    for (int64_t g = (int64_t)blockIdx.x * kThreads + threadIdx.x; g < groups; g += (int64_t)gridDim.x * kThreads) {
        int32_t k[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) k[j] = rank_key<IS_INT8>(load_bits(x, es, 4 * g + j), nzm);
        uint32_t m = keep24(k[0], k[1], k[2], k[3]);
        *reinterpret_cast<uint32_t *>(out + 4 * g) = (m & 1) | ((m >> 1 & 1) << 8) | ((m >> 2 & 1) << 16) | ((m >> 3 & 1) << 24);
    }
}

// get_24_bytemasks for 8- and 16-bit elements on SIMD lanes: 16 bytes in per thread, one 0/1 byte per element out
template <int ES>
__global__ void __launch_bounds__(kThreads) sparse24_mask_simd_kernel(const void *x, int64_t chunks, uint8_t *out) {
    static_assert(ES == 1 || ES == 2, "SIMD lanes are 8 or 16 bits");
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kThreads) {
        const uint4 w = ld_stream((const char *)x + c * 16);
        if constexpr (ES == 1) {
            uint4 o;
            sparse24_bytemask_u8x16(w.x, w.y, w.z, w.w, o.x, o.y, o.z, o.w);
            st_stream(out + c * 16, o);
        } else {
            uint2 o;
            sparse24_bytemask_u16x8(w.x, w.y, w.z, w.w, o.x, o.y);
            st_stream8(out + c * 8, o);
        }
    }
}

// sparse24_bitmask_compress, cols % 8 == 0, 8- and 16-bit elements: one thread per 16 elements (two bitmask bytes,
// eight kept values).  The keep rule runs on SIMD lanes of 32-bit words (ctb_sparse24_simd.cuh), about six integer
// instructions per element, so the kernel stays bound by memory rather than by the selection logic.
template <int ES>
__global__ void __launch_bounds__(kThreads) sparse24_compress_simd_kernel(const void *x, int64_t units, void *values, uint8_t *bitmask) {
    static_assert(ES == 1 || ES == 2, "SIMD lanes are 8 or 16 bits");
    if constexpr (ES == 2) {
        // 16 bytes per unit: lane l of a warp takes units 64 t + l and 64 t + 32 + l, so that every load and
        // store instruction of the warp covers one contiguous span
        const int64_t items = ((units + 63) >> 6) << 5;
        for (int64_t it = (int64_t)blockIdx.x * kThreads + threadIdx.x; it < items; it += (int64_t)gridDim.x * kThreads) {
            const int64_t ua = ((it >> 5) << 6) + (it & 31), ub = ua + 32;
            uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
            if (ua < units) a = ld_stream((const char *)x + ua * 16);
            if (ub < units) b = ld_stream((const char *)x + ub * 16);
            uint32_t v0, v1, v2, v3, m0, m1;
            sparse24_pack_u16x8(a.x, a.y, a.z, a.w, v0, v1, m0);
            sparse24_pack_u16x8(b.x, b.y, b.z, b.w, v2, v3, m1);
            if (ua < units) {
                st_stream8((char *)values + ua * 8, make_uint2(v0, v1));
                bitmask[ua] = (uint8_t)m0;
            }
            if (ub < units) {
                st_stream8((char *)values + ub * 8, make_uint2(v2, v3));
                bitmask[ub] = (uint8_t)m1;
            }
        }
    } else {
        const int64_t items = (units + 1) >> 1;
        for (int64_t it = (int64_t)blockIdx.x * kThreads + threadIdx.x; it < items; it += (int64_t)gridDim.x * kThreads) {
            const int64_t u = it * 2;
            const bool both = u + 1 < units;
            uint4 w = make_uint4(0, 0, 0, 0);
            if (both) w = ld_stream((const char *)x + u * 8);
            else {
                const uint2 t = ld_stream8((const char *)x + u * 8);
                w.x = t.x;
                w.y = t.y;
            }
            uint32_t v0, v1, m;
            sparse24_pack_u8x16(w.x, w.y, w.z, w.w, v0, v1, m);
            if (both) {
                st_stream8((char *)values + u * 4, make_uint2(v0, v1));
                *reinterpret_cast<uint16_t *>(bitmask + u) = (uint16_t)m;
            } else {
                st_stream4((char *)values + u * 4, v0);
                bitmask[u] = (uint8_t)m;
            }
        }
    }
}

// the same for 32-bit elements (and the model the SIMD kernels are tested against): one thread per 8 elements =
// 2 runs = 4 kept values and one bitmask byte; four neighbouring lanes merge their bytes into one 32-bit store.
template <int ES, bool IS_INT8>
__global__ void __launch_bounds__(kThreads) sparse24_compress_kernel(const void *x, uint32_t nzm, int64_t units, void *values, uint8_t *bitmask) {
    const int64_t padded = (units + 31) & ~(int64_t)31;
    for (int64_t u = (int64_t)blockIdx.x * kThreads + threadIdx.x; u < padded; u += (int64_t)gridDim.x * kThreads) {
        uint32_t b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const bool live = u < units;
        if (live) load8_bits<ES>(x, u, b);
        int32_t k[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) k[j] = rank_key<IS_INT8>(b[j], nzm);
        uint32_t m = keep24(k[0], k[1], k[2], k[3]) | (keep24(k[4], k[5], k[6], k[7]) << 4);
        // the four kept elements in column order: per run, the lower and the upper of its two set bits
        uint32_t kept[4];
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            uint32_t mm = (m >> (4 * g)) & 0xFu;
            kept[2 * g] = (mm & 1) ? b[4 * g] : ((mm & 2) ? b[4 * g + 1] : b[4 * g + 2]);
            kept[2 * g + 1] = (mm & 8) ? b[4 * g + 3] : ((mm & 4) ? b[4 * g + 2] : b[4 * g + 1]);
        }
        if (live) {
            if constexpr (ES == 2) st_stream8((char *)values + u * 8, make_uint2(kept[0] | (kept[1] << 16), kept[2] | (kept[3] << 16)));
            else if constexpr (ES == 1) st_stream4((char *)values + u * 4, kept[0] | (kept[1] << 8) | (kept[2] << 16) | (kept[3] << 24));
            else st_stream((char *)values + u * 16, make_uint4(kept[0], kept[1], kept[2], kept[3]));
        }
        // gather 4 mask bytes; whole quads are live or dead together only when units % 4 == 0
        uint32_t w = m << (8 * (threadIdx.x & 3));
        w |= __shfl_xor_sync(0xFFFFFFFFu, w, 1);
        w |= __shfl_xor_sync(0xFFFFFFFFu, w, 2);
        if ((threadIdx.x & 3) == 0 && live) {
            if (u + 3 < units) *reinterpret_cast<uint32_t *>(bitmask + u) = w;
            else
                for (int64_t t = u; t < units; ++t) bitmask[t] = (uint8_t)(w >> (8 * (t - u)));
        }
    }
}

// Fast expansion of a 2:4 compressed tensor (cols % 8 == 0), 8- and 16-bit elements: every run of four columns
// keeps exactly two, so the values of bitmask byte u start at 4u and no prefix sum is needed.  One thread per 16
// elements; a run is rebuilt by ONE byte permute of its two values whose selector comes from a 16-entry table
// indexed by the run's mask nibble.  A bitmask that breaks the two-per-run rule raises *irregular; the generic
// kernels then redo the tensor (they are launched right behind this one and return at once when the flag is clear).
template <int ES>
__global__ void __launch_bounds__(kThreads) sparse24_expand_simd_kernel(const void *values, const uint8_t *bitmask, int64_t units, void *out, int *irregular, int irregular_value) {
    static_assert(ES == 1 || ES == 2, "byte-permute expansion is for 8- and 16-bit elements");
    // selector of a run with mask nibble n: the lower set bit takes the first value, the upper one the second, the
    // rest a zero byte (source byte 4).  ES == 1: four byte selectors; ES == 2: two words of two halfword selectors.
    __shared__ uint32_t lut[16];
    if (threadIdx.x < 16) {
        const uint32_t n = threadIdx.x;
        uint32_t sel = 0;
        int seen = 0;
        for (int i = 0; i < 4; ++i) {
            uint32_t src = 4;  // zero
            if ((n >> i) & 1) src = seen++ ? 1 : 0;
            if (ES == 1) sel |= src << (4 * i);
            else sel |= (src == 4 ? 0x44u : src == 0 ? 0x10u : 0x32u) << (8 * i);
        }
        lut[n] = sel;
    }
    __syncthreads();
    bool bad = false;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    if constexpr (ES == 2) {
        // lane l of a warp takes units 64 t + l and 64 t + 32 + l: every load and store instruction of the warp
        // covers one contiguous span (16 bytes out per unit)
        const int64_t items = ((units + 63) >> 6) << 5;
        constexpr int U = 2;
        for (int64_t it0 = (int64_t)blockIdx.x * kThreads + threadIdx.x; it0 < items; it0 += U * stride) {
            uint32_t m[U][2];
            uint2 v[U][2];
#pragma unroll
            for (int k = 0; k < U; ++k) {
                const int64_t it = it0 + k * stride;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int64_t u = ((it >> 5) << 6) + (it & 31) + 32 * h;
                    m[k][h] = 0x33u;  // an absent unit counts as regular
                    v[k][h] = make_uint2(0, 0);
                    if (it < items && u < units) {
                        m[k][h] = bitmask[u];
                        v[k][h] = ld_stream8((const char *)values + u * 8);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < U; ++k) {
                const int64_t it = it0 + k * stride;
                if (it >= items) break;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int64_t u = ((it >> 5) << 6) + (it & 31) + 32 * h;
                    const uint32_t mm = m[k][h];
                    uint32_t c = mm - ((mm >> 1) & 0x55u);
                    c = (c & 0x33u) + ((c >> 2) & 0x33u);
                    bad |= c != 0x22u;  // each nibble must have exactly two bits set
                    const uint32_t s0 = lut[mm & 0xFu], s1 = lut[mm >> 4];
                    if (u < units)
                        st_stream((char *)out + u * 16, make_uint4(prmt(v[k][h].x, 0, s0 & 0xFFFFu), prmt(v[k][h].x, 0, s0 >> 16),
                                                                   prmt(v[k][h].y, 0, s1 & 0xFFFFu), prmt(v[k][h].y, 0, s1 >> 16)));
                }
            }
        }
    } else {
        const int64_t items = (units + 1) >> 1;
        constexpr int U = 4;  // items in flight per thread: the loads of all of them are issued before the first is used
        for (int64_t it0 = (int64_t)blockIdx.x * kThreads + threadIdx.x; it0 < items; it0 += U * stride) {
            uint32_t m[U];
            uint2 v[U];
#pragma unroll
            for (int k = 0; k < U; ++k) {
                const int64_t u = (it0 + k * stride) * 2;
                m[k] = 0;
                v[k] = make_uint2(0, 0);
                if (u + 1 < units) {
                    m[k] = *reinterpret_cast<const uint16_t *>(bitmask + u);
                    v[k] = ld_stream8((const char *)values + u * 4);
                } else if (u < units) {
                    m[k] = bitmask[u];
                    v[k].x = ld_stream4((const char *)values + u * 4);
                }
            }
#pragma unroll
            for (int k = 0; k < U; ++k) {
                const int64_t u = (it0 + k * stride) * 2;
                if (u >= units) break;
                const bool both = u + 1 < units;
                {  // every nibble must have exactly two bits set (the absent second unit counts as regular)
                    uint32_t c = m[k] - ((m[k] >> 1) & 0x5555u);
                    c = (c & 0x3333u) + ((c >> 2) & 0x3333u);
                    bad |= c != (both ? 0x2222u : 0x0022u);
                }
                const uint32_t s0 = lut[m[k] & 0xFu], s1 = lut[(m[k] >> 4) & 0xFu], s2 = lut[(m[k] >> 8) & 0xFu], s3 = lut[(m[k] >> 12) & 0xFu];
                const uint32_t o0 = prmt(v[k].x, 0, s0), o1 = prmt(v[k].x >> 16, 0, s1);
                const uint32_t o2 = prmt(v[k].y, 0, s2), o3 = prmt(v[k].y >> 16, 0, s3);
                if (both) st_stream((char *)out + u * 8, make_uint4(o0, o1, o2, o3));
                else st_stream8((char *)out + u * 8, make_uint2(o0, o1));
            }
        }
    }
    if (__any_sync(0xFFFFFFFFu, bad) && (threadIdx.x & 31) == 0) atomicExch(irregular, irregular_value);
}

// the same for 32-bit elements: one thread per 8 elements
template <int ES>
__global__ void __launch_bounds__(kThreads) sparse24_expand_kernel(const void *values, const uint8_t *bitmask, int64_t units, void *out, int *irregular, int irregular_value) {
    bool bad = false;
    for (int64_t u = (int64_t)blockIdx.x * kThreads + threadIdx.x; u < units; u += (int64_t)gridDim.x * kThreads) {
        const uint32_t m = bitmask[u];
        bad |= (__popc(m & 0xFu) != 2) | (__popc(m >> 4) != 2);
        uint32_t v[4];
        if constexpr (ES == 2) {
            uint2 t = ld_stream8((const char *)values + u * 8);
            v[0] = t.x & 0xFFFFu; v[1] = t.x >> 16; v[2] = t.y & 0xFFFFu; v[3] = t.y >> 16;
        } else if constexpr (ES == 1) {
            uint32_t t = ld_stream4((const char *)values + u * 4);
            v[0] = t & 0xFFu; v[1] = (t >> 8) & 0xFFu; v[2] = (t >> 16) & 0xFFu; v[3] = t >> 24;
        } else {
            uint4 t = ld_stream((const char *)values + u * 16);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        }
        uint32_t b[8];
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            const uint32_t mm = (m >> (4 * g)) & 0xFu;
            const uint32_t lo = v[2 * g], hi = v[2 * g + 1];
            // a kept position holds the run's first value if no lower bit is set, else the second
            b[4 * g + 0] = (mm & 1) ? lo : 0u;
            b[4 * g + 1] = (mm & 2) ? ((mm & 1) ? hi : lo) : 0u;
            b[4 * g + 2] = (mm & 4) ? ((mm & 3) ? hi : lo) : 0u;
            b[4 * g + 3] = (mm & 8) ? hi : 0u;
        }
        if constexpr (ES == 2) st_stream((char *)out + u * 16, make_uint4(b[0] | (b[1] << 16), b[2] | (b[3] << 16), b[4] | (b[5] << 16), b[6] | (b[7] << 16)));
        else if constexpr (ES == 1) st_stream8((char *)out + u * 8, make_uint2(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24), b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24)));
        else {
            st_stream((char *)out + u * 32, make_uint4(b[0], b[1], b[2], b[3]));
            st_stream((char *)out + u * 32 + 16, make_uint4(b[4], b[5], b[6], b[7]));
        }
    }
    if (__any_sync(0xFFFFFFFFu, bad) && (threadIdx.x & 31) == 0) atomicExch(irregular, irregular_value);
}

}  // namespace ctb

// ------------------------------------------------------------------ unstructured bitmask codec

namespace ctb {

// 8-bit keep mask of unit `u` (8 elements of one row; cols % 8 == 0 fast path) plus the raw bits
template <int ES>
__device__ __forceinline__ uint32_t unit_mask(const void *x, int64_t unit, uint32_t nzm, uint32_t (&b)[8]) {
    load8_bits<ES>(x, unit, b);
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) m |= ((b[j] & nzm) != 0 ? 1u : 0u) << j;
    return m;
}

// mask of up to 8 elements starting at column c0 of `row`, scalar loads (ragged / unaligned rows);
// `pred` (optional bytemask) replaces the non-zero test
__device__ __forceinline__ uint32_t unit_mask_scalar(const void *x, const uint8_t *pred, int es, uint32_t nzm, int64_t row, int64_t c0, int64_t cols, uint32_t (&b)[8]) {
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        b[j] = 0;
        if (c0 + j < cols) {
            int64_t i = row * cols + c0 + j;
            b[j] = load_bits(x, es, i);
            bool keep = pred ? (pred[i] != 0) : ((b[j] & nzm) != 0);
            m |= (keep ? 1u : 0u) << j;
        }
    }
    return m;
}

__device__ __forceinline__ int block_sum(int v) {
    __shared__ int part[kThreads / 32];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    int t = 0;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) t += part[i];
    return t;
}

// exclusive prefix of v over the block, and the block total
__device__ __forceinline__ int block_excl_scan(int v, int &total) {
    __shared__ int wsum[kThreads / 32];
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int inc = v;
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) wsum[w] = inc;
    __syncthreads();
    int base = 0;
    total = 0;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) {
        if (i < w) base += wsum[i];
        total += wsum[i];
    }
    return base + inc - v;
}

// pass 1: bitmask bytes and per-row counts.  One block per row.
template <int ES, bool VEC>
__global__ void __launch_bounds__(kThreads) bm_count_kernel(const void *x, const uint8_t *pred, int es, uint32_t nzm, int64_t rows, int64_t cols, uint8_t *bitmask, int64_t *row_counts) {
    const int64_t upr = (cols + 7) / 8;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        int cnt = 0;
        for (int64_t u = threadIdx.x; u < upr; u += kThreads) {
            uint32_t b[8];
            uint32_t m = VEC ? unit_mask<ES>(x, r * upr + u, nzm, b) : unit_mask_scalar(x, pred, es, nzm, r, u * 8, cols, b);
            if (bitmask) bitmask[r * upr + u] = (uint8_t)m;
            cnt += __popc(m);
        }
        cnt = block_sum(cnt);
        if (threadIdx.x == 0) row_counts[r] = cnt;
    }
}

// per-row counts straight from a bitmask (decompress)
__global__ void __launch_bounds__(kThreads) bm_popcount_kernel(const uint8_t *bitmask, int64_t rows, int64_t cols, int64_t *row_counts, Gate gate) {
    if (gate.flag != nullptr && *gate.flag != gate.value) return;  // the fast 2:4 expansion already produced the tensor
    const int64_t upr = (cols + 7) / 8;
    const int tail = (int)(cols & 7);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        int cnt = 0;
        for (int64_t u = threadIdx.x; u < upr; u += kThreads) {
            uint32_t m = bitmask[r * upr + u];
            if (tail && u == upr - 1) m &= (1u << tail) - 1;  // unpackbits(count=cols) ignores pad bits
            cnt += __popc(m);
        }
        cnt = block_sum(cnt);
        if (threadIdx.x == 0) row_counts[r] = cnt;
    }
}

// pass 2: in-place exclusive scan of the row counts (single block), total to *nnz
__global__ void __launch_bounds__(1024) row_scan_kernel(int64_t *counts, int64_t rows, int64_t *nnz, Gate gate = Gate{nullptr, 0}) {
    if (gate.flag != nullptr && *gate.flag != gate.value) return;
    __shared__ int64_t wsum[32];
    __shared__ int64_t carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int64_t base = 0; base < rows; base += 1024) {
        int64_t i = base + threadIdx.x;
        int64_t v = i < rows ? counts[i] : 0, inc = v;
        for (int o = 1; o < 32; o <<= 1) {
            int64_t t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) wsum[w] = inc;
        __syncthreads();
        int64_t off = carry_s;
        for (int k = 0; k < w; ++k) off += wsum[k];
        if (i < rows) counts[i] = off + inc - v;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = off + inc;
        __syncthreads();
    }
    if (threadIdx.x == 0 && nnz) *nnz = carry_s;
}

// pass 3 (compress): compact each row's kept elements to values[row_offsets[r] ...], staged through
// shared memory so that global stores are contiguous.  One block per row, 2048 elements per round.
template <int ES, bool VEC>
__global__ void __launch_bounds__(kThreads) bm_scatter_kernel(const void *x, const uint8_t *pred, int es, uint32_t nzm, int64_t rows, int64_t cols, const int64_t *row_offsets, void *values) {
    __shared__ uint32_t stage[kThreads * 8];
    const int64_t upr = (cols + 7) / 8;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        int64_t out = row_offsets[r];
        for (int64_t u0 = 0; u0 < upr; u0 += kThreads) {
            int64_t u = u0 + threadIdx.x;
            uint32_t b[8], m = 0;
            if (u < upr) m = VEC ? unit_mask<ES>(x, r * upr + u, nzm, b) : unit_mask_scalar(x, pred, es, nzm, r, u * 8, cols, b);
            int total, pos = block_excl_scan(__popc(m), total);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if ((m >> j) & 1) stage[pos++] = b[j];
            __syncthreads();
            for (int i = threadIdx.x; i < total; i += kThreads) store_bits(values, es, out + i, stage[i]);
            out += total;
            __syncthreads();
        }
    }
}

// decompress: zeros, then values scattered to the set bits.  One block per row; every thread owns
// 8 output elements per round and writes them with one vector store when the row layout allows.
template <int ES, bool VEC>
__global__ void __launch_bounds__(kThreads) bm_expand_kernel(const void *values, const uint8_t *bitmask, int es, int64_t rows, int64_t cols, const int64_t *row_offsets, void *out,
                                                               Gate gate) {
    if (gate.flag != nullptr && *gate.flag != gate.value) return;
    const int64_t upr = (cols + 7) / 8;
    const int tail = (int)(cols & 7);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        int64_t in = row_offsets[r];
        for (int64_t u0 = 0; u0 < upr; u0 += kThreads) {
            int64_t u = u0 + threadIdx.x;
            uint32_t m = 0;
            if (u < upr) {
                m = bitmask[r * upr + u];
                if (tail && u == upr - 1) m &= (1u << tail) - 1;
            }
            int total, pos = block_excl_scan(__popc(m), total);
            uint32_t b[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) b[j] = ((m >> j) & 1) ? load_bits(values, es, in + pos++) : 0u;
            if (u < upr) {
                if constexpr (VEC && ES == 2) {
                    st_stream((char *)out + (r * upr + u) * 16, make_uint4(b[0] | (b[1] << 16), b[2] | (b[3] << 16), b[4] | (b[5] << 16), b[6] | (b[7] << 16)));
                } else if constexpr (VEC && ES == 1) {
                    st_stream8((char *)out + (r * upr + u) * 8, make_uint2(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24), b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24)));
                } else if constexpr (VEC && ES == 4) {
                    st_stream((char *)out + (r * upr + u) * 32, make_uint4(b[0], b[1], b[2], b[3]));
                    st_stream((char *)out + (r * upr + u) * 32 + 16, make_uint4(b[4], b[5], b[6], b[7]));
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (u * 8 + j < cols) store_bits(out, es, r * cols + u * 8 + j, b[j]);
                }
            }
            in += total;
        }
    }
}

}  // namespace ctb


// ------------------------------------------------------------------ block-tile bitmask codec (cols % 8 == 0)
//
// The flat tensor is a sequence of units of 8 elements (one bitmask byte each).  Every block of the grid owns a
// CONTIGUOUS range of units and walks it in tiles of kBmTile units (8192 elements), thread t taking units
// t, t + 256, t + 512, t + 768 of a tile, so that each load or store instruction of a warp covers one contiguous span.
//   kernel 1 streams over the tensor (compress: writes the bitmask) or over the bitmask (decompress) and leaves the
//            kept count of every block;
//   kernel 2, launched with the same grid, sums the counts of the blocks before it (at most 4096 words) and walks
//            its range with a running offset.  Per tile: one block-wide exclusive scan of the per-unit counts
//            (packed pairs through the warp shuffles, then 32 warp totals through one more warp scan), a
//            data-dependent placement of single elements into (out of) a shared-memory window that mirrors the
//            16-byte alignment of `values`, and the window is written (read) as whole 16-byte words; only the
//            ragged head and tail of a tile move element by element.
// Nothing waits on another block, and scratch is one count per block whatever the tensor size.  The second read
// of the dense tensor comes from L2 when the tensor fits there.
namespace ctb {

constexpr int kWarps = kThreads / 32;
constexpr int kBmRows = 4;                   // units per thread and tile
constexpr int kBmTile = kThreads * kBmRows;  // units per block and step
constexpr int kTileMaxGrid = 4096;           // blocks per launch (bounds the scratch: one count per block)
static_assert(kWarps == 8 && kBmRows == 4, "tile_scan maps (row, warp) onto the 32 lanes of one warp");

// The per-element placement, written as predicated instructions: `if (bit) { store; advance; }` in C++ becomes a
// branch with its divergence bookkeeping per element, which is most of what these kernels would execute.
// `saddr` is a shared-window byte address (32-bit shared state space) and advances by ES when the bit is set.
template <int ES>
__device__ __forceinline__ void stage_put_if(uint32_t &saddr, uint32_t v, uint32_t bit) {
    if constexpr (ES == 1)
        asm volatile("{ .reg .pred p; setp.ne.u32 p, %2, 0; @p st.shared.u8 [%0], %1; @p add.u32 %0, %0, 1; }" : "+r"(saddr) : "r"(v), "r"(bit) : "memory");
    else if constexpr (ES == 2)
        asm volatile("{ .reg .pred p; setp.ne.u32 p, %2, 0; @p st.shared.u16 [%0], %1; @p add.u32 %0, %0, 2; }" : "+r"(saddr) : "r"(v), "r"(bit) : "memory");  // the low half of v
    else
        asm volatile("{ .reg .pred p; setp.ne.u32 p, %2, 0; @p st.shared.u32 [%0], %1; @p add.u32 %0, %0, 4; }" : "+r"(saddr) : "r"(v), "r"(bit) : "memory");
}
// the mirror image: the element at `saddr` when the bit is set (and advance), zero otherwise
template <int ES>
__device__ __forceinline__ uint32_t stage_get_if(uint32_t &saddr, uint32_t bit) {
    uint32_t v;
    if constexpr (ES == 1)
        asm volatile("{ .reg .pred p; setp.ne.u32 p, %2, 0; mov.u32 %0, 0; @p ld.shared.u8 %0, [%1]; @p add.u32 %1, %1, 1; }" : "=r"(v), "+r"(saddr) : "r"(bit) : "memory");
    else if constexpr (ES == 2)
        asm volatile("{ .reg .pred p; setp.ne.u32 p, %2, 0; mov.u32 %0, 0; @p ld.shared.u16 %0, [%1]; @p add.u32 %1, %1, 2; }" : "=r"(v), "+r"(saddr) : "r"(bit) : "memory");
    else
        asm volatile("{ .reg .pred p; setp.ne.u32 p, %2, 0; mov.u32 %0, 0; @p ld.shared.u32 %0, [%1]; @p add.u32 %1, %1, 4; }" : "=r"(v), "+r"(saddr) : "r"(bit) : "memory");
    return v;
}

// units [first, last) of this block when the units are dealt to the blocks of the grid in contiguous ranges of
// whole rows of kThreads units
__device__ __forceinline__ void block_range(int64_t units, int64_t &first, int64_t &last) {
    const int64_t rows = (units + kThreads - 1) / kThreads;
    const int64_t per = (rows + gridDim.x - 1) / gridDim.x;
    const int64_t r0 = min((int64_t)blockIdx.x * per, rows);
    const int64_t r1 = min(r0 + per, rows);
    first = r0 * kThreads;
    last = min(r1 * kThreads, units);
}

// kernel 1 epilogue: the kept count of the block
__device__ __forceinline__ void publish_count(unsigned long long c, unsigned long long *block_tot) {
    __shared__ unsigned long long wt[kWarps];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
    if ((threadIdx.x & 31) == 0) wt[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
#pragma unroll
        for (int i = 0; i < kWarps; ++i) t += wt[i];
        block_tot[blockIdx.x] = t;
    }
}

// kernel 2 prologue: index of the first kept value of this block's range; the last block also stores the grand total
__device__ __forceinline__ unsigned long long block_first_value(const unsigned long long *block_tot, int64_t *nnz) {
    __shared__ unsigned long long red[kWarps];
    unsigned long long s = 0;
    for (int i = threadIdx.x; i < (int)blockIdx.x; i += kThreads) s += block_tot[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    unsigned long long base = 0;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) base += red[i];
    if (nnz != nullptr && blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) *nnz = (int64_t)(base + block_tot[blockIdx.x]);
    return base;
}

// Exclusive prefixes, in tile order (row j of the tile before row j + 1, threads in order inside a row), of the
// per-unit counts c[j] <= 8 of this thread, and the tile total.  Two barriers; `wt` and `pre` are block-shared.
__device__ __forceinline__ void tile_scan(const uint32_t (&c)[kBmRows], uint32_t (&excl)[kBmRows], uint32_t &total, uint32_t (*wt)[2],
                                          uint32_t *pre) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    uint32_t p01 = c[0] | (c[1] << 16), p23 = c[2] | (c[3] << 16);  // a warp's sums stay below 2^16
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, p01, o), b = __shfl_up_sync(0xFFFFFFFFu, p23, o);
        if (lane >= o) {
            p01 += a;
            p23 += b;
        }
    }
    if (lane == 31) {
        wt[w][0] = p01;
        wt[w][1] = p23;
    }
    __syncthreads();
    if (w == 0) {
        // lane = row * kWarps + warp: the 32 (row, warp) totals in tile order
        const int j = lane >> 3, ww = lane & 7;
        const uint32_t packed = wt[ww][j >> 1];
        const uint32_t v = (j & 1) ? (packed >> 16) : (packed & 0xFFFFu);
        uint32_t inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += a;
        }
        pre[lane] = inc - v;
        if (lane == 31) pre[32] = inc;
    }
    __syncthreads();
    total = pre[32];
    excl[0] = pre[0 * kWarps + w] + (p01 & 0xFFFFu) - c[0];
    excl[1] = pre[1 * kWarps + w] + (p01 >> 16) - c[1];
    excl[2] = pre[2 * kWarps + w] + (p23 & 0xFFFFu) - c[2];
    excl[3] = pre[3 * kWarps + w] + (p23 >> 16) - c[3];
}

// raw 16-byte (ES = 2), 8-byte (ES = 1) or 32-byte (ES = 4) image of one 8-element unit; KEEP = the dense tensor is
// read again by the next kernel, so leave it in L2 (default policy) instead of streaming it through
template <int ES, bool KEEP>
__device__ __forceinline__ Raw8 load_unit_raw(const void *x, int64_t unit) {
    Raw8 r;
    r.a = make_uint4(0, 0, 0, 0);
    r.b = make_uint4(0, 0, 0, 0);
    const char *p = (const char *)x + unit * (8 * ES);
    if constexpr (ES == 2) r.a = KEEP ? *reinterpret_cast<const uint4 *>(p) : ld_stream(p);
    else if constexpr (ES == 1) {
        const uint2 t = KEEP ? *reinterpret_cast<const uint2 *>(p) : ld_stream8(p);
        r.a.x = t.x;
        r.a.y = t.y;
    } else {
        r.a = KEEP ? *reinterpret_cast<const uint4 *>(p) : ld_stream(p);
        r.b = KEEP ? *reinterpret_cast<const uint4 *>(p + 16) : ld_stream(p + 16);
    }
    return r;
}
template <int ES>
__device__ __forceinline__ void unit_bits(const Raw8 &r, uint32_t (&b)[8]) {
    if constexpr (ES == 2) {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { b[2 * i] = w[i] & 0xFFFFu; b[2 * i + 1] = w[i] >> 16; }
    } else if constexpr (ES == 1) {
        const uint32_t w[2] = {r.a.x, r.a.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = (w[i >> 2] >> (8 * (i & 3))) & 0xFFu;
    } else {
        b[0] = r.a.x; b[1] = r.a.y; b[2] = r.a.z; b[3] = r.a.w;
        b[4] = r.b.x; b[5] = r.b.y; b[6] = r.b.z; b[7] = r.b.w;
    }
}

// The top bits of the four bytes of t (bits 7, 15, 23, 31) as a nibble in bits 28..31: one multiply moves bit 7 + 8i
// to bit 28 + i, and no two partial products share a bit, so nothing carries.
__device__ __forceinline__ uint32_t top_bits_to_high_nibble(uint32_t t) { return (t & 0x80808080u) * 0x00204081u; }

// 8-bit non-zero mask of one unit straight from its packed words.  16- and 8-bit elements: adding the magnitude mask
// to the magnitude bits carries into the element's top bit exactly when one of them is set (an integer type's own
// top bit is OR-ed in); the top bits are then gathered with a byte permute and a multiply.
template <int ES>
__device__ __forceinline__ uint32_t unit_nz_mask(const Raw8 &r, uint32_t nzm) {
    if constexpr (ES == 2) {
        const uint32_t k = 0x7FFF7FFFu;  // the 16-bit types here are floating point: sign excluded, -0.0 is a zero
        const uint32_t t0 = (r.a.x & k) + k, t1 = (r.a.y & k) + k, t2 = (r.a.z & k) + k, t3 = (r.a.w & k) + k;
        const uint32_t lo = top_bits_to_high_nibble(prmt_b32(t0, t1, 0x7531)), hi = top_bits_to_high_nibble(prmt_b32(t2, t3, 0x7531));
        return (lo >> 28) | ((hi >> 24) & 0xF0u);
    } else if constexpr (ES == 1) {
        const uint32_t k = 0x7F7F7F7Fu;
        uint32_t t0 = (r.a.x & k) + k, t1 = (r.a.y & k) + k;
        if (nzm & 0x80u) {
            t0 |= r.a.x;
            t1 |= r.a.y;
        }
        return (top_bits_to_high_nibble(t0) >> 28) | ((top_bits_to_high_nibble(t1) >> 24) & 0xF0u);
    } else {
        uint32_t m = 0;
        const uint32_t w[8] = {r.a.x, r.a.y, r.a.z, r.a.w, r.b.x, r.b.y, r.b.z, r.b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) m |= ((w[i] & nzm) != 0 ? 1u : 0u) << i;
        return m;
    }
}

// compress, kernel 1: bitmask bytes and the kept count of the block
template <int ES>
__global__ void __launch_bounds__(kThreads) bm_block_count_kernel(const void *x, uint32_t nzm, int64_t units, uint8_t *bitmask,
                                                                  unsigned long long *block_tot) {
    int64_t first, last;
    block_range(units, first, last);
    uint32_t cnt = 0;
    constexpr int DEPTH = 4;  // units in flight per thread
    for (int64_t base = first; base < last; base += DEPTH * kThreads) {
        Raw8 raw[DEPTH];
        bool ok[DEPTH];
#pragma unroll
        for (int j = 0; j < DEPTH; ++j) {  // all loads first
            const int64_t u = base + j * kThreads + threadIdx.x;
            ok[j] = u < last;
            if (ok[j]) raw[j] = load_unit_raw<ES, true>(x, u);
        }
#pragma unroll
        for (int j = 0; j < DEPTH; ++j) {
            if (!ok[j]) continue;
            const uint32_t m = unit_nz_mask<ES>(raw[j], nzm);
            bitmask[base + j * kThreads + threadIdx.x] = (uint8_t)m;
            cnt += __popc(m);
        }
    }
    publish_count((unsigned long long)cnt, block_tot);
}

// decompress, kernel 1: the same counts from the bitmask
__global__ void __launch_bounds__(kThreads) bm_block_popcount_kernel(const uint8_t *bitmask, int64_t units, unsigned long long *block_tot,
                                                                     Gate gate) {
    if (gate.flag != nullptr && *gate.flag != gate.value) return;  // the fast 2:4 expansion already produced the tensor
    int64_t first, last;
    block_range(units, first, last);
    unsigned long long c = 0;
    int64_t i = first + (int64_t)threadIdx.x * 16;  // `first` is a multiple of 256: 16-byte steps keep the base's alignment
    if ((reinterpret_cast<uintptr_t>(bitmask) & 15u) == 0) {
        for (; i + 16 <= last; i += kThreads * 16) {
            const uint4 v = *reinterpret_cast<const uint4 *>(bitmask + i);
            c += __popc(v.x) + __popc(v.y) + __popc(v.z) + __popc(v.w);
        }
    }
    // ragged end (and unaligned bitmasks): a thread's first leftover piece may be partial, later ones are whole
    for (; i < last; i += kThreads * 16)
        for (int64_t j = i; j < i + 16 && j < last; ++j) c += __popc((uint32_t)bitmask[j]);
    publish_count(c, block_tot);
}

// Kept elements of the bitmask bytes [first, last) counted by the whole block (every thread returns the sum).
// `first` is a multiple of 256 or 0: 16-byte steps keep the alignment of the bitmask's base.
__device__ __forceinline__ unsigned long long block_popcount_range(const uint8_t *bitmask, int64_t first, int64_t last) {
    __shared__ unsigned long long pc[kWarps];
    unsigned long long c = 0;
    int64_t i = first + (int64_t)threadIdx.x * 16;
    if ((reinterpret_cast<uintptr_t>(bitmask) & 15u) == 0) {
        for (; i + 16 <= last; i += kThreads * 16) {
            const uint4 v = *reinterpret_cast<const uint4 *>(bitmask + i);
            c += __popc(v.x) + __popc(v.y) + __popc(v.z) + __popc(v.w);
        }
    }
    for (; i < last; i += kThreads * 16)
        for (int64_t j = i; j < i + 16 && j < last; ++j) c += __popc((uint32_t)bitmask[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
    __syncthreads();  // `pc` may still be read by a previous call
    if ((threadIdx.x & 31) == 0) pc[threadIdx.x >> 5] = c;
    __syncthreads();
    unsigned long long t = 0;
#pragma unroll
    for (int i2 = 0; i2 < kWarps; ++i2) t += pc[i2];
    return t;
}

// what the dequantizing form of the expand kernel needs besides the arguments of the plain form
struct ExpandExtra {
    const uint16_t *scale;  // one bf16 scale per row
    FastDiv by_upr;         // unit -> row
};

template <int ES>
struct BmWindow {
    static constexpr int kBytes = kBmTile * 8 * ES + 32;  // a tile's elements, shifted by up to 15 bytes
};

// compress, kernel 2 (same grid as kernel 1): compact every tile of the block's range into `values`, and the row offsets
template <int ES>
__global__ void __launch_bounds__(kThreads, ES == 4 ? 4 : 6) bm_block_scatter_kernel(const void *x, const uint8_t *bitmask, int64_t units, FastDiv by_upr, uint32_t upr,
                                                                    const unsigned long long *block_tot, void *values, int64_t *row_offsets,
                                                                    int64_t *nnz) {
    __shared__ __align__(16) unsigned char win[BmWindow<ES>::kBytes];
    __shared__ uint32_t wt[kWarps][2], pre[kBmRows * kWarps + 1];
    asm volatile("griddepcontrol.wait;" ::: "memory");  // a programmatic dependent of the count kernel (see launch_dependent)
    const uint32_t win_addr = (uint32_t)__cvta_generic_to_shared(win);
    int64_t first, last;
    block_range(units, first, last);
    Raw8 raw[kBmRows];
    uint32_t mask[kBmRows];
    auto fetch = [&](int64_t base) {
#pragma unroll
        for (int j = 0; j < kBmRows; ++j) {
            const int64_t u = base + j * kThreads + threadIdx.x;
            mask[j] = 0;
            if (u < last) {
                mask[j] = bitmask[u];
                raw[j] = load_unit_raw<ES, false>(x, u);
            }
        }
    };
    if (first < last) fetch(first);  // in flight during the prologue
    unsigned long long prefix = block_first_value(block_tot, nnz);
    for (int64_t base = first; base < last; base += kBmTile) {
        uint32_t c[kBmRows], excl[kBmRows], total;
#pragma unroll
        for (int j = 0; j < kBmRows; ++j) c[j] = __popc(mask[j]);
        tile_scan(c, excl, total, wt, pre);
        char *dst = (char *)values + prefix * ES;
        const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15u);  // the window mirrors the destination's alignment
#pragma unroll
        for (int j = 0; j < kBmRows; ++j) {
            if (mask[j] == 0) continue;
            uint32_t b[8];
            unit_bits<ES>(raw[j], b);
            uint32_t sa = win_addr + shift + excl[j] * ES;
#pragma unroll
            for (int e = 0; e < 8; ++e) stage_put_if<ES>(sa, b[e], mask[j] & (1u << e));
        }
        // rows that begin at one of this thread's units (cols is a multiple of 8, so a row starts on a unit)
#pragma unroll
        for (int j = 0; j < kBmRows; ++j) {
            const int64_t u = base + j * kThreads + threadIdx.x;
            if (u < last) {
                const uint32_t r = fastdiv((uint32_t)u, by_upr);
                if (r * upr == (uint32_t)u) row_offsets[r] = (int64_t)(prefix + excl[j]);
            }
        }
        if (base + kBmTile < last) fetch(base + kBmTile);  // the next tile's loads fly while this one is copied out
        __syncthreads();
        // whole 16-byte words of the window that belong to this tile alone, then the ragged head and tail by element
        const uint32_t nbytes = shift + total * ES;
        const uint32_t first_full = shift ? 1u : 0u, end_full = nbytes >> 4;
        char *dst0 = dst - shift;
        for (uint32_t wv = first_full + threadIdx.x; wv < end_full; wv += kThreads)
            *reinterpret_cast<uint4 *>(dst0 + 16 * wv) = *reinterpret_cast<const uint4 *>(win + 16 * wv);
        {
            const uint32_t head_end = min(16u * first_full, nbytes);
            const uint32_t tail0 = max(16u * end_full, head_end);
            const uint32_t per = 16 / ES;  // elements in one 16-byte word
            if (threadIdx.x < per) {
                const uint32_t p = shift + threadIdx.x * ES;
                if (p < head_end) store_bits(values, ES, (int64_t)prefix + threadIdx.x, load_bits(win, ES, p / ES));
            } else if (threadIdx.x >= 32 && threadIdx.x < 32 + per) {
                const uint32_t p = tail0 + (threadIdx.x - 32) * ES;
                if (p < nbytes) store_bits(values, ES, (int64_t)prefix + (p - shift) / ES, load_bits(win, ES, p / ES));
            }
        }
        prefix += total;
        __syncthreads();  // the window is reused by the next tile
    }
}

// decompress, kernel 2 (same grid as kernel 1): every tile's kept values are one contiguous run of `values`: bring it
// into the window (whole 16-byte words that lie inside the run, its ragged ends by element, so nothing outside
// `values` is ever read), then every thread rebuilds its units from the window
// SELFCOUNT: no count kernel runs in front and nothing is exchanged between blocks: every block counts the bits before
// its own range itself.  That reads half the bitmask per block on average, which is the price of a launch that needs
// no scratch, no ticket and no other block; it is the form of the gated fallback of the 2:4 kernels, which returns at
// once unless a bitmask is not two-per-four, so that the common case pays for one empty launch and not two.
// DEQ (8-bit elements): the rebuilt e4m3 codes are dequantized with the row's bf16 scale and `out` is bf16.
template <int ES, bool SELFCOUNT = false, bool DEQ = false>
__global__ void __launch_bounds__(kThreads, ES == 4 ? 4 : 6) bm_block_expand_kernel(const void *values, const uint8_t *bitmask, int64_t units,
                                                                   unsigned long long *block_tot, void *out, Gate gate,
                                                                   ExpandExtra extra = ExpandExtra{}) {
    static_assert(!DEQ || ES == 1, "the dequantizing form is for e4m3 codes");
    // launched as a programmatic dependent of the kernel in front (the count kernel, or the 2:4 kernel that may raise the
    // flag): its blocks may be resident before that kernel has finished, and wait here for its completion and the
    // visibility of its writes (without the launch attribute this returns at once)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (gate.flag != nullptr && *gate.flag != gate.value) return;
    __shared__ __align__(16) unsigned char win[BmWindow<ES>::kBytes];
    __shared__ uint32_t wt[kWarps][2], pre[kBmRows * kWarps + 1];
    const uint32_t win_addr = (uint32_t)__cvta_generic_to_shared(win);
    int64_t first, last;
    block_range(units, first, last);
    uint32_t mask_n[kBmRows];
    auto fetch = [&](int64_t base) {
#pragma unroll
        for (int j = 0; j < kBmRows; ++j) {
            const int64_t u = base + j * kThreads + threadIdx.x;
            mask_n[j] = u < last ? (uint32_t)bitmask[u] : 0u;
        }
    };
    unsigned long long src;
    if constexpr (SELFCOUNT) {
        if (first < last) fetch(first);
        src = block_popcount_range(bitmask, 0, first);
    } else {
        if (first < last) fetch(first);
        src = block_first_value(block_tot, nullptr);
    }
    for (int64_t base = first; base < last; base += kBmTile) {
        uint32_t mask[kBmRows], c[kBmRows], excl[kBmRows], total;
#pragma unroll
        for (int j = 0; j < kBmRows; ++j) {
            mask[j] = mask_n[j];
            c[j] = __popc(mask[j]);
        }
        if (base + kBmTile < last) fetch(base + kBmTile);  // one tile ahead
        tile_scan(c, excl, total, wt, pre);
        const char *a = (const char *)values + src * ES;
        const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(a) & 15u);
        const uint32_t nbytes = shift + total * ES;
        const uint32_t first_full = shift ? 1u : 0u, end_full = nbytes >> 4;
        const char *a0 = a - shift;
        for (uint32_t wv = first_full + threadIdx.x; wv < end_full; wv += kThreads)
            *reinterpret_cast<uint4 *>(win + 16 * wv) = ld_stream(a0 + 16 * wv);
        {
            const uint32_t head_end = min(16u * first_full, nbytes);
            const uint32_t tail0 = max(16u * end_full, head_end);
            const uint32_t per = 16 / ES;
            if (threadIdx.x < per) {
                const uint32_t p = shift + threadIdx.x * ES;
                if (p < head_end) store_bits(win, ES, p / ES, load_bits(values, ES, (int64_t)src + threadIdx.x));
            } else if (threadIdx.x >= 32 && threadIdx.x < 32 + per) {
                const uint32_t p = tail0 + (threadIdx.x - 32) * ES;
                if (p < nbytes) store_bits(win, ES, p / ES, load_bits(values, ES, (int64_t)src + (p - shift) / ES));
            }
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < kBmRows; ++j) {
            const int64_t u = base + j * kThreads + threadIdx.x;
            if (u >= last) continue;
            uint32_t sa = win_addr + shift + excl[j] * ES;
            uint32_t b[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) b[e] = stage_get_if<ES>(sa, mask[j] & (1u << e));
            char *q = (char *)out + u * 8 * ES;
            if constexpr (DEQ) {
                Raw8 r;
                r.a = make_uint4(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24), b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24), 0, 0);
                r.b = make_uint4(0, 0, 0, 0);
                float f[8];
                decode8<F_E4M3>(r, f);
                const uint32_t sb = __ldg(extra.scale + fastdiv((uint32_t)u, extra.by_upr));
                st_stream((char *)out + u * 16, dequant8_to_bf16<false>(f, __uint_as_float(sb << 16)));
            } else if constexpr (ES == 2) st_stream(q, make_uint4(b[0] | (b[1] << 16), b[2] | (b[3] << 16), b[4] | (b[5] << 16), b[6] | (b[7] << 16)));
            else if constexpr (ES == 1) st_stream8(q, make_uint2(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24), b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24)));
            else {
                st_stream(q, make_uint4(b[0], b[1], b[2], b[3]));
                st_stream(q + 16, make_uint4(b[4], b[5], b[6], b[7]));
            }
        }
        src += total;
        __syncthreads();  // the window is reused by the next tile
    }
}

// ------------------------------------------------------------------ single-pass bitmask compress
//
// One cooperative kernel that reads the dense tensor from HBM exactly once.  The flat tensor is cut into tiles of
// kFzThreads * ITEMS * 4 elements (16 KiB of 16-bit data); tile T belongs to block T % gridDim.x, so the tiles a
// block works on at the same time as its neighbours (one "slab" of gridDim.x tiles) are adjacent in memory.
//   * thread 0 of a block keeps kFzStages bulk copies (cp.async.bulk, completion on an mbarrier) in flight: the
//     tiles after the current one stream into shared memory while it is worked on, and nothing is read twice;
//   * every thread owns ITEMS runs of 4 elements of the tile (thread t the runs t, t + 256, ...: neighbouring
//     lanes place their kept elements about 4 bytes apart, which keeps the placement free of bank conflicts);
//     masks and counts come straight from shared memory, one block-wide scan orders them;
//   * an iteration first COUNTS the block's next tile and publishes that count, then PLACES the current one, so a count
//     is out a whole iteration before anyone needs it and no block runs in lockstep with another; the count goes out as (ticket, count) in one 64-bit word of the scratch (the 48-bit ticket of
//     the call makes a stale or uninitialised word recognisable, so the scratch never needs clearing); the block then
//     needs the counts of every tile before its own: all tiles of the slab before (read once per slab by the whole
//     block) and the lower-numbered tiles of this slab.  Counts do not depend on anyone else's offsets, so
//     there is no chain to wait along: a block only ever waits for other blocks to have COUNTED;
//   * kept elements go through a shared-memory window that mirrors the 16-byte alignment of their place in
//     `values` and leave as whole 16-byte words.
// All blocks must be resident at once (a block waits for counts of higher-numbered blocks of the slab before),
// hence the cooperative launch.  Every wait is bounded; on expiry the kernel stores -1 in *nnz and returns.
constexpr int kFzThreads = 256;
constexpr int kFzWarps = kFzThreads / 32;
constexpr int kFzStages = 3;
constexpr int kFzMaxTiles = 16384;  // count words in the scratch
constexpr long long kFzSpinCycles = 2000000000LL;

template <int ES>
struct Fz {
    static constexpr int kItems = ES == 4 ? 4 : 8;               // runs of 4 elements per thread and tile
    static constexpr int kTileElems = kFzThreads * kItems * 4;   // 8192 (4096 for 32-bit elements)
    static constexpr int kTileBytes = kTileElems * ES;           // 16 KiB (8 KiB for 8-bit elements)
    static constexpr int kWindowBytes = kTileBytes + 32;
    static constexpr int kSmemBytes = kFzStages * kTileBytes + kWindowBytes + 128 /*barriers*/ + 16 /*alignment*/;
};

__device__ __forceinline__ uint32_t fz_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool fz_mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when the budget ran out
__device__ __forceinline__ bool fz_mbar_wait(uint32_t bar, uint32_t parity) {
    if (fz_mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!fz_mbar_try(bar, parity))
        if (clock64() - t0 > kFzSpinCycles) return false;
    return true;
}
__device__ __forceinline__ void fz_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fz_publish(unsigned long long *flag, unsigned long long v) {
    asm volatile("st.global.release.gpu.u64 [%0], %1;" ::"l"(flag), "l"(v) : "memory");
}
// the count another block published for this ticket; bounded, false on expiry
__device__ __forceinline__ bool fz_await(const unsigned long long *flag, unsigned long long ticket, unsigned long long &count) {
    const long long t0 = clock64();
    for (;;) {
        unsigned long long v;
        asm volatile("ld.global.acquire.gpu.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
        if ((v >> 16) == ticket) {  // a tile keeps at most 8192 elements: 16 bits of count, 48 bits of ticket
            count = v & 0xFFFFull;
            return true;
        }
        if (clock64() - t0 > kFzSpinCycles) return false;
        __nanosleep(32);
    }
}

// 4-bit non-zero mask of a run of 4 elements at `p` in shared memory
template <int ES>
__device__ __forceinline__ uint32_t fz_run_mask(const unsigned char *p, uint32_t nzm) {
    if constexpr (ES == 2) {
        const uint2 v = *reinterpret_cast<const uint2 *>(p);
        const uint32_t k = 0x7FFF7FFFu;
        return top_bits_to_high_nibble(prmt_b32((v.x & k) + k, (v.y & k) + k, 0x7531)) >> 28;
    } else if constexpr (ES == 1) {
        const uint32_t v = *reinterpret_cast<const uint32_t *>(p);
        uint32_t t0 = (v & 0x7F7F7F7Fu) + 0x7F7F7F7Fu;
        if (nzm & 0x80u) t0 |= v;
        return top_bits_to_high_nibble(t0) >> 28;
    } else {
        const uint4 v = *reinterpret_cast<const uint4 *>(p);
        return ((v.x & nzm) != 0 ? 1u : 0u) | ((v.y & nzm) != 0 ? 2u : 0u) | ((v.z & nzm) != 0 ? 4u : 0u) | ((v.w & nzm) != 0 ? 8u : 0u);
    }
}

template <int ES>
__global__ void __launch_bounds__(kFzThreads, 3)
bm_single_pass_compress_kernel(const void *x, uint32_t nzm, int64_t units, FastDiv by_upr, uint32_t upr, unsigned long long *flags,
                               unsigned long long ticket, void *values, uint8_t *bitmask, int64_t *row_offsets, int64_t *nnz) {
    using F = Fz<ES>;
    constexpr int ITEMS = F::kItems;
    extern __shared__ unsigned char fz_raw[];
    unsigned char *base = fz_raw + ((16u - (fz_smem_u32(fz_raw) & 15u)) & 15u);
    unsigned char *win = base + kFzStages * F::kTileBytes;
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(win + F::kWindowBytes + 8);
    __shared__ uint32_t wt[kFzWarps][2], pre[ITEMS * kFzWarps + 1];
    __shared__ unsigned long long red[kFzWarps][2];
    __shared__ int failed;
    const uint32_t win_addr = fz_smem_u32(win);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t elems = units * 8;
    const int64_t ntiles = (elems + F::kTileElems - 1) / F::kTileElems;
    const int64_t G = gridDim.x;

    auto tile_bytes_of = [&](int64_t T) -> uint32_t {
        const int64_t n = min((int64_t)F::kTileElems, elems - T * F::kTileElems);
        return (uint32_t)(n * ES);
    };
    if (threadIdx.x == 0) {
        failed = 0;
        for (int i = 0; i < kFzStages; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(fz_smem_u32(&bars[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int i = 0; i < kFzStages; ++i) {
            const int64_t T = blockIdx.x + (int64_t)i * G;
            if (T < ntiles) fz_bulk_load(fz_smem_u32(base + i * F::kTileBytes), (const char *)x + T * F::kTileBytes, tile_bytes_of(T), fz_smem_u32(&bars[i]));
        }
    }
    __syncthreads();

    // What the counting half of an iteration leaves for the placing half of the next one.
    struct Counted {
        uint32_t masks;        // the run masks of this thread, 4 bits per run
        uint32_t excl[ITEMS];  // exclusive prefixes of its runs within the tile
        uint32_t total;        // kept elements of the tile
    };
    // ---- count tile number `it` of this block (masks, bitmask bytes, block-wide scan) and publish its count
    auto count_tile = [&](int64_t it, int64_t T, Counted &out) {
        const int sidx = (int)(it % kFzStages);
        if (!fz_mbar_wait(fz_smem_u32(&bars[sidx]), (uint32_t)((it / kFzStages) & 1))) failed = 1;  // benign race: every writer stores 1
        const unsigned char *src = base + sidx * F::kTileBytes;
        const uint32_t tile_elems = tile_bytes_of(T) / ES;
        uint32_t c[ITEMS], mine = 0;
#pragma unroll
        for (int j = 0; j < ITEMS; ++j) {
            const uint32_t r = j * kFzThreads + threadIdx.x;  // run index in tile order
            // tiles are whole units of 8 elements: a run is inside or outside as a whole
            const uint32_t m = r * 4 < tile_elems ? fz_run_mask<ES>(src + r * 4 * ES, nzm) : 0u;
            c[j] = __popc(m);
            mine |= m << (4 * j);
        }
        out.masks = mine;
        // bitmask bytes: a unit is the pair of runs of an even lane and its odd neighbour; the even lane writes the bytes of
        // the first half of the rows, the odd lane those of the second half
        {
            const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, mine, 1);
            const uint32_t lo = (lane & 1) ? other : mine, hi = (lane & 1) ? mine : other;
#pragma unroll
            for (int jj = 0; jj < ITEMS / 2; ++jj) {
                const int j = jj + ((lane & 1) ? ITEMS / 2 : 0);
                const uint32_t r = j * kFzThreads + (threadIdx.x & ~1u);
                if (r * 4 < tile_elems) bitmask[T * (F::kTileElems / 8) + (r >> 1)] = (uint8_t)(((lo >> (4 * j)) & 15u) | (((hi >> (4 * j)) & 15u) << 4));
            }
        }
        // block-wide exclusive scan in tile order (row j before row j + 1, threads in order inside a row)
        uint32_t p0 = 0, p1 = 0;  // byte fields: a warp's sum of one row is at most 128
#pragma unroll
        for (int j = 0; j < ITEMS && j < 4; ++j) p0 |= c[j] << (8 * j);
#pragma unroll
        for (int j = 4; j < ITEMS; ++j) p1 |= c[j] << (8 * (j - 4));
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, p0, o), b = __shfl_up_sync(0xFFFFFFFFu, p1, o);
            if (lane >= o) {
                p0 += a;
                p1 += b;
            }
        }
        if (lane == 31) {
            wt[w][0] = p0;
            wt[w][1] = p1;
        }
        __syncthreads();
        if (w == 0) {
            // ITEMS * kFzWarps (row, warp) totals in tile order, PER consecutive ones per lane
            constexpr int PER = ITEMS * kFzWarps / 32;
            static_assert(PER >= 1 && PER * 32 == ITEMS * kFzWarps, "one warp covers the (row, warp) totals");
            uint32_t v[PER], sum = 0;
#pragma unroll
            for (int q = 0; q < PER; ++q) {
                const int e = lane * PER + q, j = e / kFzWarps, ww = e % kFzWarps;
                v[q] = (wt[ww][j >> 2] >> (8 * (j & 3))) & 0xFFu;
                sum += v[q];
            }
            uint32_t inc = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if (lane >= o) inc += a;
            }
            uint32_t run = inc - sum;
#pragma unroll
            for (int q = 0; q < PER; ++q) {
                pre[lane * PER + q] = run;
                run += v[q];
            }
            if (lane == 31) {
                pre[ITEMS * kFzWarps] = inc;
                // other blocks wait for counts only: out it goes, a whole iteration before this block places the tile
                fz_publish(&flags[T], (ticket << 16) | (unsigned long long)inc);
            }
        }
        __syncthreads();
        out.total = pre[ITEMS * kFzWarps];
#pragma unroll
        for (int j = 0; j < ITEMS; ++j) {
            const uint32_t incl = ((j < 4 ? p0 : p1) >> (8 * (j & 3))) & 0xFFu;
            out.excl[j] = pre[j * kFzWarps + w] + incl - c[j];
        }
        __syncthreads();  // `pre` and `wt` are free again (the next scan may start before everyone has read them otherwise)
    };

    unsigned long long before_slab = 0;  // kept elements in all slabs before the current one (block-uniform)
    Counted cur, nxt;
    int64_t it = 0;
    if ((int64_t)blockIdx.x < ntiles) count_tile(0, blockIdx.x, cur);
    for (int64_t T = blockIdx.x; T < ntiles; T += G, ++it) {
        const bool more = T + G < ntiles;
        if (more) count_tile(it + 1, T + G, nxt);  // published one iteration ahead: nobody runs in lockstep
        const int sidx = (int)(it % kFzStages);
        const unsigned char *src = base + sidx * F::kTileBytes;
        const uint32_t tile_elems = tile_bytes_of(T) / ES;
        // ---- kept elements before this tile: every tile of the slab before (all blocks), lower tiles of this slab
        {
            const int64_t slab0 = T - blockIdx.x;  // first tile of this slab
            unsigned long long prev = 0, here = 0;
            bool ok = true;
            if (slab0 > 0)
                for (int64_t b = threadIdx.x; b < G; b += kFzThreads) {
                    unsigned long long cnt = 0;
                    ok = fz_await(&flags[slab0 - G + b], ticket, cnt) && ok;
                    prev += cnt;
                }
            for (int64_t b = threadIdx.x; b < (int64_t)blockIdx.x; b += kFzThreads) {
                unsigned long long cnt = 0;
                ok = fz_await(&flags[slab0 + b], ticket, cnt) && ok;
                here += cnt;
            }
            if (!ok) failed = 1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                prev += __shfl_xor_sync(0xFFFFFFFFu, prev, o);
                here += __shfl_xor_sync(0xFFFFFFFFu, here, o);
            }
            if (lane == 0) {
                red[w][0] = prev;
                red[w][1] = here;
            }
        }
        __syncthreads();
        unsigned long long slab_prev = 0, slab_here = 0;
#pragma unroll
        for (int i = 0; i < kFzWarps; ++i) {
            slab_prev += red[i][0];
            slab_here += red[i][1];
        }
        before_slab += slab_prev;
        const unsigned long long prefix = before_slab + slab_here;
        if (failed) break;  // block-uniform: every write to `failed` precedes the barrier above
        // ---- place the kept elements in the window, which mirrors the 16-byte alignment of their place in `values`
        char *dst = (char *)values + prefix * ES;
        const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15u);
#pragma unroll
        for (int j = 0; j < ITEMS; ++j) {
            const uint32_t m = (cur.masks >> (4 * j)) & 15u;
            if (m == 0) continue;
            const unsigned char *p = src + (j * kFzThreads + threadIdx.x) * 4 * ES;
            uint32_t sa = win_addr + shift + cur.excl[j] * ES;
            if constexpr (ES == 2) {
                const uint2 v = *reinterpret_cast<const uint2 *>(p);
                stage_put_if<2>(sa, v.x, m & 1u);
                stage_put_if<2>(sa, v.x >> 16, m & 2u);
                stage_put_if<2>(sa, v.y, m & 4u);
                stage_put_if<2>(sa, v.y >> 16, m & 8u);
            } else if constexpr (ES == 1) {
                const uint32_t v = *reinterpret_cast<const uint32_t *>(p);
                stage_put_if<1>(sa, v, m & 1u);
                stage_put_if<1>(sa, v >> 8, m & 2u);
                stage_put_if<1>(sa, v >> 16, m & 4u);
                stage_put_if<1>(sa, v >> 24, m & 8u);
            } else {
                const uint4 v = *reinterpret_cast<const uint4 *>(p);
                stage_put_if<4>(sa, v.x, m & 1u);
                stage_put_if<4>(sa, v.y, m & 2u);
                stage_put_if<4>(sa, v.z, m & 4u);
                stage_put_if<4>(sa, v.w, m & 8u);
            }
        }
        // ---- rows that begin at one of this thread's units (cols is a multiple of 8: a row starts on a unit, i.e. at
        //      the run of an even thread)
        if ((threadIdx.x & 1) == 0) {
#pragma unroll
            for (int j = 0; j < ITEMS; ++j) {
                const uint32_t r = j * kFzThreads + threadIdx.x;
                if (r * 4 < tile_elems) {
                    const uint32_t u = (uint32_t)(T * (F::kTileElems / 8)) + (r >> 1);
                    const uint32_t row = fastdiv(u, by_upr);
                    if (row * upr == u) row_offsets[row] = (int64_t)(prefix + cur.excl[j]);
                }
            }
        }
        __syncthreads();  // the stage buffer has been read by everyone, the window is complete
        const uint32_t total = cur.total;
        if (threadIdx.x == 0) {
            const int64_t Tn = T + (int64_t)kFzStages * G;  // the tile that reuses this stage buffer
            if (Tn < ntiles) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic reads above, async-proxy writes below
                fz_bulk_load(fz_smem_u32(base + sidx * F::kTileBytes), (const char *)x + Tn * F::kTileBytes, tile_bytes_of(Tn), fz_smem_u32(&bars[sidx]));
            }
            if (T == ntiles - 1) *nnz = (int64_t)(prefix + total);
        }
        // ---- the window leaves as whole 16-byte words; its ragged head and tail by element
        {
            const uint32_t nbytes = shift + total * ES;
            const uint32_t first_full = shift ? 1u : 0u, end_full = nbytes >> 4;
            char *dst0 = dst - shift;
            for (uint32_t wv = first_full + threadIdx.x; wv < end_full; wv += kFzThreads)
                st_stream(dst0 + 16 * wv, *reinterpret_cast<const uint4 *>(win + 16 * wv));
            const uint32_t head_end = min(16u * first_full, nbytes);
            const uint32_t tail0 = max(16u * end_full, head_end);
            constexpr uint32_t per = 16 / ES;
            if (threadIdx.x < per) {
                const uint32_t p = shift + threadIdx.x * ES;
                if (p < head_end) store_bits(values, ES, (int64_t)prefix + threadIdx.x, load_bits(win, ES, p / ES));
            } else if (threadIdx.x >= 32 && threadIdx.x < 32 + per) {
                const uint32_t p = tail0 + (threadIdx.x - 32) * ES;
                if (p < nbytes) store_bits(values, ES, (int64_t)prefix + (p - shift) / ES, load_bits(win, ES, p / ES));
            }
        }
        __syncthreads();  // the window is reused by the next tile
        cur = nxt;
    }
    if (failed) {
        // let the copies still in flight land before the block gives its shared memory back, then report
        if (threadIdx.x == 0) {
            for (int64_t j = it; j < it + kFzStages; ++j) {
                const int64_t Tj = blockIdx.x + j * G;
                if (Tj < ntiles) fz_mbar_wait(fz_smem_u32(&bars[j % kFzStages]), (uint32_t)((j / kFzStages) & 1));
            }
            *nnz = -1;
        }
    }
}

}  // namespace ctb

// ------------------------------------------------------------------ entry points

using namespace ctb;

extern "C" int ctb_sparse24_mask(const void *x, int32_t dtype, int64_t numel, uint8_t *out, void *stream) {
    if (numel != 0 && (!x || !out)) return fail(CTB_EINVAL_NULL, "null buffer");  // an empty tensor has no storage
    ElemInfo e;
    if (!elem_info(dtype, &e)) return fail(CTB_EINVAL_DTYPE, "unsupported dtype for 2:4 masks");
    if (numel % 4 != 0) return fail(CTB_EINVAL_SHAPE, "Tensor size must be a multiple of 4 for TWO_FOUR sparsity");
    if (numel == 0) return CTB_OK;
    cudaStream_t st = as_stream(stream);
    int64_t done = 0;  // elements covered by the SIMD kernel; the scalar kernel takes what is left (less than one chunk)
    if (e.esize != 4 && aligned16(x) && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
        const int per = 16 / e.esize;  // elements per 16-byte chunk
        const int64_t chunks = numel / per;
        if (chunks > 0) {
            const int grid = grid_for(chunks, kThreads, 8);
            if (e.esize == 1) sparse24_mask_simd_kernel<1><<<grid, kThreads, 0, st>>>(x, chunks, out);
            else sparse24_mask_simd_kernel<2><<<grid, kThreads, 0, st>>>(x, chunks, out);
            int rc = after_launch("sparse24_mask_simd_kernel");
            if (rc) return rc;
        }
        done = chunks * per;
    }
    if (done == numel) return CTB_OK;
    const void *xr = (const char *)x + done * e.esize;
    const int64_t groups = (numel - done) / 4;
    int grid = grid_for(groups, kThreads, 8);
    if (e.is_int8) sparse24_mask_kernel<true><<<grid, kThreads, 0, st>>>(xr, e.esize, e.nz_mask, groups, out + done);
    else sparse24_mask_kernel<false><<<grid, kThreads, 0, st>>>(xr, e.esize, e.nz_mask, groups, out + done);
    return after_launch("sparse24_mask_kernel");
}

extern "C" int ctb_sparse24_compress(const void *x, int32_t dtype, int64_t rows, int64_t cols, void *values, uint8_t *bitmask, void *stream) {
    if (rows != 0 && cols != 0 && (!x || !values || !bitmask)) return fail(CTB_EINVAL_NULL, "null buffer");
    ElemInfo e;
    if (!elem_info(dtype, &e)) return fail(CTB_EINVAL_DTYPE, "unsupported dtype for 2:4 compression");
    if ((rows * cols) % 4 != 0) return fail(CTB_EINVAL_SHAPE, "Tensor size must be a multiple of 4 for TWO_FOUR sparsity");
    if (cols % 8 != 0) return fail(CTB_EUNSUPPORTED, "fused 2:4 compression needs cols %% 8 == 0; use ctb_sparse24_mask + ctb_masked_compress");
    if (!aligned16(x) || !aligned16(values)) return fail(CTB_EINVAL_ALIGN, "buffers must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(bitmask) & 3u) return fail(CTB_EINVAL_ALIGN, "bitmask must be 4-byte aligned");
    int64_t units = rows * cols / 8;
    if (units == 0) return CTB_OK;
    cudaStream_t st = as_stream(stream);
    if (e.esize == 4) {
        sparse24_compress_kernel<4, false><<<grid_for(units, kThreads, 8), kThreads, 0, st>>>(x, e.nz_mask, units, values, bitmask);
        return after_launch("sparse24_compress_kernel");
    }
    const int grid = grid_for((units + 1) / 2, kThreads, 8);
    if (e.esize == 2) sparse24_compress_simd_kernel<2><<<grid, kThreads, 0, st>>>(x, units, values, bitmask);
    else sparse24_compress_simd_kernel<1><<<grid, kThreads, 0, st>>>(x, units, values, bitmask);
    return after_launch("sparse24_compress_simd_kernel");
}

// Launch `kernel` as a programmatic dependent of the kernel before it on the stream: its launch latency is spent while
// that kernel still runs, and its blocks wait at their `griddepcontrol.wait` for that kernel to have completed.
template <typename... KArgs, typename... Args>
static cudaError_t launch_dependent(void (*kernel)(KArgs...), int grid, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// 1 keeps ctb_bitmask_compress on the two-kernel path (the default: on the tensor sizes of a model's weights the pair
// is the faster of the two; the single-pass kernel reads the tensor from HBM only once and is there for tensors that do
// not fit the L2 cache).  ctb_bitmask_force_two_kernels(0) selects the single-pass kernel where it can run.
static std::atomic<int> g_two_kernel_bitmask{1};

static int64_t tile_bytes() {
    return 8 * (int64_t)kFzMaxTiles;  // one count per block of the two-kernel codec (4096) or per tile of the single-pass kernel
}
// the 2:4 decompress keeps its "bitmask is irregular" flag behind whichever scratch layout is used
static int64_t flag_offset(int64_t rows) {
    const int64_t a = tile_bytes(), b = rows * 8;
    return a > b ? a : b;
}
// Blocks of the two-kernel tile codec: both kernels must see the same grid, it defines the ranges.  A range is a whole
// number of rows of kThreads units; a handful of resident blocks per SM keeps enough loads in flight for the
// streaming kernel and enough warps for the placement kernel.
static int tile_grid(int64_t units, int blocks_per_sm = 6) {
    const int g = grid_for(units, kThreads, blocks_per_sm);
    return g < kTileMaxGrid ? g : kTileMaxGrid;
}

// The single-pass kernel, when the device can hold the whole grid at once and one count word per tile fits the
// scratch.  *launched = false leaves the call to the two-kernel path.
template <int ES>
static int launch_single_pass(const void *x, const ElemInfo &e, int64_t units, uint32_t upr, unsigned long long *flags, void *values,
                              uint8_t *bitmask, int64_t *row_offsets, int64_t *nnz, cudaStream_t st, bool *launched) {
    using F = Fz<ES>;
    *launched = false;
    const int64_t ntiles = cdiv(units * 8, F::kTileElems);
    if (ntiles > kFzMaxTiles) return CTB_OK;
    // The per-tile counts are told apart from stale scratch by a ticket chosen per launch CALL.  A launch recorded into
    // a CUDA graph would replay with the ticket it was recorded with and could take the counts of the replay before for
    // its own: a capturing stream gets the two-kernel path, which exchanges nothing through tagged scratch.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return CTB_OK;
    }
    int dev = 0, coop = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return CTB_OK;
    static std::atomic<int> per_sm[64];  // resident blocks per SM of this instantiation on each device (0: not asked yet, -1: cannot run)
    int occ = per_sm[dev].load(std::memory_order_acquire);
    auto *kernel = bm_single_pass_compress_kernel<ES>;
    if (occ == 0) {
        occ = -1;
        if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && coop &&
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F::kSmemBytes) == cudaSuccess) {
            int n = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kFzThreads, F::kSmemBytes) == cudaSuccess && n > 0) occ = n;
        }
        cudaGetLastError();  // a refusal above is not an error of this call
        per_sm[dev].store(occ, std::memory_order_release);
    }
    if (occ <= 0) return CTB_OK;
    const int64_t cap = (int64_t)occ * sm_count();
    const int grid = (int)(ntiles < cap ? ntiles : cap);
    static std::atomic<unsigned long long> s_ticket{0x5DEECE66Dull};
    unsigned long long ticket = s_ticket.fetch_add(0x9E3779B97F4Aull, std::memory_order_relaxed) & ((1ull << 48) - 1);
    FastDiv by_upr = make_fastdiv(upr);
    uint32_t nzm = e.nz_mask;
    void *args[] = {(void *)&x, (void *)&nzm, (void *)&units, (void *)&by_upr, (void *)&upr, (void *)&flags, (void *)&ticket,
                    (void *)&values, (void *)&bitmask, (void *)&row_offsets, (void *)&nnz};
    cudaError_t err = cudaLaunchCooperativeKernel((const void *)kernel, dim3(grid), dim3(kFzThreads), args, F::kSmemBytes, st);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return CTB_OK;  // e.g. another context holds part of the device: the two-kernel path needs no co-residency
    }
    *launched = true;
    return after_launch("bm_single_pass_compress_kernel");
}

static int compress_impl(const void *x, const uint8_t *pred, int32_t dtype, int64_t rows, int64_t cols, void *values, uint8_t *bitmask,
                         int64_t *row_offsets, int64_t *nnz, void *workspace, void *stream) {
    if (!nnz || (rows != 0 && cols != 0 && (!x || !values || !bitmask || !row_offsets))) return fail(CTB_EINVAL_NULL, "null buffer");
    ElemInfo e;
    if (!elem_info(dtype, &e)) return fail(CTB_EINVAL_DTYPE, "unsupported dtype for bitmask compression");
    if (rows < 0 || cols < 0) return fail(CTB_EINVAL_SHAPE, "negative shape");
    cudaStream_t st = as_stream(stream);
    if (rows == 0 || cols == 0) {
        cudaMemsetAsync(nnz, 0, sizeof(int64_t), st);
        if (rows) cudaMemsetAsync(row_offsets, 0, sizeof(int64_t) * rows, st);
        return CTB_OK;
    }
    const bool vec = !pred && cols % 8 == 0 && aligned16(x);
    if (vec && workspace != nullptr && (reinterpret_cast<uintptr_t>(values) & 3u) == 0 && rows * cols / 8 < (1LL << 31)) {
        // block tiles: count, then scatter (both kernels must see the same grid: it defines the ranges)
        unsigned long long *block_tot = static_cast<unsigned long long *>(workspace);
        const int64_t units = rows * cols / 8;
        const uint32_t upr = (uint32_t)(cols / 8);  // units per row
        const FastDiv by_upr = make_fastdiv(upr);
        int rc;
        if (aligned16(x) && (units * 8 * e.esize) % 16 == 0 && !g_two_kernel_bitmask.load(std::memory_order_relaxed)) {
            bool launched = false;
            if (e.esize == 2) rc = launch_single_pass<2>(x, e, units, upr, block_tot, values, bitmask, row_offsets, nnz, st, &launched);
            else if (e.esize == 1) rc = launch_single_pass<1>(x, e, units, upr, block_tot, values, bitmask, row_offsets, nnz, st, &launched);
            else rc = launch_single_pass<4>(x, e, units, upr, block_tot, values, bitmask, row_offsets, nnz, st, &launched);
            if (rc || launched) return rc;
        }
        const int g1 = tile_grid(units);
        if (e.esize == 2) bm_block_count_kernel<2><<<g1, kThreads, 0, st>>>(x, e.nz_mask, units, bitmask, block_tot);
        else if (e.esize == 1) bm_block_count_kernel<1><<<g1, kThreads, 0, st>>>(x, e.nz_mask, units, bitmask, block_tot);
        else bm_block_count_kernel<4><<<g1, kThreads, 0, st>>>(x, e.nz_mask, units, bitmask, block_tot);
        if ((rc = after_launch("bm_block_count_kernel"))) return rc;
        cudaError_t le;
        if (e.esize == 2) le = launch_dependent(bm_block_scatter_kernel<2>, g1, st, x, bitmask, units, by_upr, upr, block_tot, values, row_offsets, nnz);
        else if (e.esize == 1) le = launch_dependent(bm_block_scatter_kernel<1>, g1, st, x, bitmask, units, by_upr, upr, block_tot, values, row_offsets, nnz);
        else le = launch_dependent(bm_block_scatter_kernel<4>, g1, st, x, bitmask, units, by_upr, upr, block_tot, values, row_offsets, nnz);
        if (le != cudaSuccess) return fail(CTB_ECUDA, "bm_block_scatter_kernel: %s", cudaGetErrorString(le));
        return after_launch("bm_block_scatter_kernel");
    }
    int grid = grid_for(rows, 1, 8);
    int rc;
#define CTB_BM(KERNEL, ...)                                                                              \
    if (vec && e.esize == 2) KERNEL<2, true><<<grid, kThreads, 0, st>>>(__VA_ARGS__);                     \
    else if (vec && e.esize == 1) KERNEL<1, true><<<grid, kThreads, 0, st>>>(__VA_ARGS__);                \
    else if (vec && e.esize == 4) KERNEL<4, true><<<grid, kThreads, 0, st>>>(__VA_ARGS__);                \
    else KERNEL<0, false><<<grid, kThreads, 0, st>>>(__VA_ARGS__);
    CTB_BM(bm_count_kernel, x, pred, e.esize, e.nz_mask, rows, cols, bitmask, row_offsets)
    if ((rc = after_launch("bm_count_kernel"))) return rc;
    row_scan_kernel<<<1, 1024, 0, st>>>(row_offsets, rows, nnz);
    if ((rc = after_launch("row_scan_kernel"))) return rc;
    CTB_BM(bm_scatter_kernel, x, pred, e.esize, e.nz_mask, rows, cols, row_offsets, values)
    return after_launch("bm_scatter_kernel");
}

extern "C" void ctb_bitmask_force_two_kernels(int32_t on) { g_two_kernel_bitmask.store(on ? 1 : 0, std::memory_order_relaxed); }

extern "C" int64_t ctb_bitmask_workspace_bytes(int64_t rows, int64_t cols) {
    return flag_offset(rows) + 16;
}

extern "C" int ctb_bitmask_compress(const void *x, int32_t dtype, int64_t rows, int64_t cols, void *values, uint8_t *bitmask,
                                    int64_t *row_offsets, int64_t *nnz, void *workspace, void *stream) {
    return compress_impl(x, nullptr, dtype, rows, cols, values, bitmask, row_offsets, nnz, workspace, stream);
}

extern "C" int ctb_masked_compress(const void *x, const uint8_t *bytemask, int32_t dtype, int64_t rows, int64_t cols, void *values,
                                   uint8_t *bitmask, int64_t *row_offsets, int64_t *nnz, void *stream) {
    if (rows != 0 && cols != 0 && !bytemask) return fail(CTB_EINVAL_NULL, "null mask");
    return compress_impl(x, bytemask, dtype, rows, cols, values, bitmask, row_offsets, nnz, nullptr, stream);
}

static int decompress_impl(const void *values, const uint8_t *bitmask, int32_t dtype, int64_t rows, int64_t cols, void *out, void *workspace,
                           Gate gate, void *stream, bool tiles_ok = false, const uint16_t *deq_scale = nullptr) {
    if (rows != 0 && cols != 0 && (!bitmask || !out || !workspace)) return fail(CTB_EINVAL_NULL, "null buffer");
    ElemInfo e;
    if (!elem_info(dtype, &e)) return fail(CTB_EINVAL_DTYPE, "unsupported dtype for bitmask decompression");
    if (rows <= 0 || cols <= 0) return rows < 0 || cols < 0 ? fail(CTB_EINVAL_SHAPE, "negative shape") : CTB_OK;
    if (!values) return fail(CTB_EINVAL_NULL, "null values");
    cudaStream_t st = as_stream(stream);
    if (tiles_ok && cols % 8 == 0 && aligned16(out) && (reinterpret_cast<uintptr_t>(values) & 3u) == 0) {
        unsigned long long *block_tot = static_cast<unsigned long long *>(workspace);
        const int64_t units = rows * cols / 8;
        // both kernels must see the same grid: it defines the ranges.  As the gated fallback of the 2:4
        // expansion the launches almost always return at once: keep them small.
        const int g1 = tile_grid(units, gate.flag ? 1 : 6);
        ExpandExtra extra{};
        extra.scale = deq_scale;
        extra.by_upr = make_fastdiv((uint32_t)(cols / 8));
        if (deq_scale != nullptr && (e.esize != 1 || units >= (1ll << 31))) return fail(CTB_EUNSUPPORTED, "the dequantizing expansion takes at most 2^34 e4m3 values");
        if (gate.flag != nullptr) {
            // the gated fallback: one launch that needs no count kernel in front (see SELFCOUNT), queued as a programmatic
            // dependent of the kernel before it, so that its launch latency is spent while that kernel still runs
            cudaError_t le;
            if (deq_scale != nullptr) le = launch_dependent(bm_block_expand_kernel<1, true, true>, g1, st, values, bitmask, units, block_tot, out, gate, extra);
            else if (e.esize == 2) le = launch_dependent(bm_block_expand_kernel<2, true, false>, g1, st, values, bitmask, units, block_tot, out, gate, extra);
            else if (e.esize == 1) le = launch_dependent(bm_block_expand_kernel<1, true, false>, g1, st, values, bitmask, units, block_tot, out, gate, extra);
            else le = launch_dependent(bm_block_expand_kernel<4, true, false>, g1, st, values, bitmask, units, block_tot, out, gate, extra);
            if (le != cudaSuccess) return fail(CTB_ECUDA, "bm_block_expand_kernel: %s", cudaGetErrorString(le));
            return after_launch("bm_block_expand_kernel");
        }
        bm_block_popcount_kernel<<<g1, kThreads, 0, st>>>(bitmask, units, block_tot, gate);
        int rc0 = after_launch("bm_block_popcount_kernel");
        if (rc0) return rc0;
        cudaError_t le;
        if (deq_scale != nullptr) le = launch_dependent(bm_block_expand_kernel<1, false, true>, g1, st, values, bitmask, units, block_tot, out, gate, extra);
        else if (e.esize == 2) le = launch_dependent(bm_block_expand_kernel<2, false, false>, g1, st, values, bitmask, units, block_tot, out, gate, extra);
        else if (e.esize == 1) le = launch_dependent(bm_block_expand_kernel<1, false, false>, g1, st, values, bitmask, units, block_tot, out, gate, extra);
        else le = launch_dependent(bm_block_expand_kernel<4, false, false>, g1, st, values, bitmask, units, block_tot, out, gate, extra);
        if (le != cudaSuccess) return fail(CTB_ECUDA, "bm_block_expand_kernel: %s", cudaGetErrorString(le));
        return after_launch("bm_block_expand_kernel");
    }
    if (deq_scale != nullptr) return fail(CTB_EUNSUPPORTED, "the dequantizing expansion needs cols %% 8 == 0 and aligned buffers");
    int64_t *offs = (int64_t *)workspace;
    int grid = grid_for(rows, 1, 8);
    int rc;
    bm_popcount_kernel<<<grid, kThreads, 0, st>>>(bitmask, rows, cols, offs, gate);
    if ((rc = after_launch("bm_popcount_kernel"))) return rc;
    row_scan_kernel<<<1, 1024, 0, st>>>(offs, rows, nullptr, gate);
    if ((rc = after_launch("row_scan_kernel"))) return rc;
    const bool vec = cols % 8 == 0 && aligned16(out);
    if (vec && e.esize == 2) bm_expand_kernel<2, true><<<grid, kThreads, 0, st>>>(values, bitmask, e.esize, rows, cols, offs, out, gate);
    else if (vec && e.esize == 1) bm_expand_kernel<1, true><<<grid, kThreads, 0, st>>>(values, bitmask, e.esize, rows, cols, offs, out, gate);
    else if (vec && e.esize == 4) bm_expand_kernel<4, true><<<grid, kThreads, 0, st>>>(values, bitmask, e.esize, rows, cols, offs, out, gate);
    else bm_expand_kernel<0, false><<<grid, kThreads, 0, st>>>(values, bitmask, e.esize, rows, cols, offs, out, gate);
    return after_launch("bm_expand_kernel");
}

extern "C" int ctb_bitmask_decompress(const void *values, const uint8_t *bitmask, int32_t dtype, int64_t rows, int64_t cols, void *out,
                                      void *workspace, void *stream) {
    return decompress_impl(values, bitmask, dtype, rows, cols, out, workspace, Gate{nullptr, 0}, stream, true);
}

extern "C" int ctb_sparse24_decompress(const void *values, int64_t nvalues, const uint8_t *bitmask, int32_t dtype, int64_t rows,
                                       int64_t cols, void *out, void *workspace, void *stream) {
    if (rows != 0 && cols != 0 && (!values || !bitmask || !out || !workspace)) return fail(CTB_EINVAL_NULL, "null buffer");
    ElemInfo e;
    if (!elem_info(dtype, &e)) return fail(CTB_EINVAL_DTYPE, "unsupported dtype for bitmask decompression");
    if (rows <= 0 || cols <= 0) return rows < 0 || cols < 0 ? fail(CTB_EINVAL_SHAPE, "negative shape") : CTB_OK;
    if (nvalues < 0) return fail(CTB_EINVAL_SHAPE, "negative value count");
    // The scan-free kernels read two values for every four columns whatever the bitmask says, so they may run only
    // over a buffer that holds rows * cols / 2 elements: a shorter one (fewer bits set than two per four) goes to
    // the generic kernels, which read exactly as many values as the bitmask has bits.
    if (nvalues < rows * cols / 2 || cols % 8 != 0 || !aligned16(out) || (reinterpret_cast<uintptr_t>(values) & 15u))
        return decompress_impl(values, bitmask, dtype, rows, cols, out, workspace, Gate{nullptr, 0}, stream, nvalues < rows * cols / 2);
    cudaStream_t st = as_stream(stream);
    int *flag = reinterpret_cast<int *>(static_cast<char *>(workspace) + flag_offset(rows));
    static std::atomic<int> s_ticket{1};
    const int ticket = s_ticket.fetch_add(1, std::memory_order_relaxed);  // see Gate: no clearing of the flag word
    const int64_t units = rows * cols / 8;
    const bool simd = e.esize != 4 && (reinterpret_cast<uintptr_t>(bitmask) & 1u) == 0;
    if (simd && e.esize == 2) sparse24_expand_simd_kernel<2><<<grid_for((units + 1) / 2, kThreads, 8), kThreads, 0, st>>>(values, bitmask, units, out, flag, ticket);
    else if (simd) sparse24_expand_simd_kernel<1><<<grid_for((units + 1) / 2, kThreads, 8), kThreads, 0, st>>>(values, bitmask, units, out, flag, ticket);
    else if (e.esize == 2) sparse24_expand_kernel<2><<<grid_for(units, kThreads, 8), kThreads, 0, st>>>(values, bitmask, units, out, flag, ticket);
    else if (e.esize == 1) sparse24_expand_kernel<1><<<grid_for(units, kThreads, 8), kThreads, 0, st>>>(values, bitmask, units, out, flag, ticket);
    else sparse24_expand_kernel<4><<<grid_for(units, kThreads, 8), kThreads, 0, st>>>(values, bitmask, units, out, flag, ticket);
    int rc = after_launch("sparse24_expand_kernel");
    if (rc) return rc;
    // generic path, gated on the flag: returns immediately unless the bitmask was not two-per-run
    return decompress_impl(values, bitmask, dtype, rows, cols, out, workspace, Gate{flag, ticket}, stream, true);
}

// ------------------------------------------------------------------ 2:4 decompress fused with the FP8 dequantize
//
// The decompress walk of a stacked sparse-24-bitmask + float-quantized module (model_compressor.py:580-611: the sparsity
// compressor rebuilds the dense e4m3 weight, the quantization compressor dequantizes it) in one pass: kept e4m3 values
// (0.5 B / element) and the bitmask (0.125) in, bf16 weight (2) out; the dense e4m3 tensor is never written.

// One thread per 8 elements: the unit's two runs are rebuilt by byte permutes (selector table by mask nibble, as in
// sparse24_expand_simd_kernel), decoded, multiplied by the row's scale and rounded once to bf16, which is
// (x_q.to(bf16) * scale) of forward.py:504-512 for a bf16 scale and no zero point.
__global__ void __launch_bounds__(kThreads) sparse24_expand_dequant_fp8_kernel(const void *values, const uint8_t *bitmask, const uint16_t *scale,
                                                                               uint32_t units, FastDiv by_upr, void *out, int *irregular,
                                                                               int irregular_value) {
    __shared__ uint32_t lut[16];
    if (threadIdx.x < 16) {
        const uint32_t n = threadIdx.x;
        uint32_t sel = 0;
        int seen = 0;
        for (int i = 0; i < 4; ++i) {
            uint32_t src = 4;  // a zero byte (the second permute operand)
            if ((n >> i) & 1) src = seen++ ? 1 : 0;
            sel |= src << (4 * i);
        }
        lut[n] = sel;
    }
    __syncthreads();
    bool bad = false;
    constexpr int U = 4;  // units in flight per thread
    const uint32_t stride = gridDim.x * (uint32_t)kThreads;
    for (uint32_t u0 = blockIdx.x * (uint32_t)kThreads + threadIdx.x; u0 < units; u0 += U * stride) {
        uint32_t m[U], v[U], sb[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {  // all loads first; a warp instruction covers one contiguous span
            const uint32_t u = u0 + k * stride;
            m[k] = 0x33u;  // an absent unit counts as regular
            v[k] = 0;
            sb[k] = 0;
            if (u < units) {
                m[k] = bitmask[u];
                v[k] = ld_stream4((const char *)values + (size_t)u * 4);
                sb[k] = __ldg(scale + fastdiv(u, by_upr));
            }
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const uint32_t u = u0 + k * stride;
            if (u >= units) break;
            uint32_t c = m[k] - ((m[k] >> 1) & 0x55u);
            c = (c & 0x33u) + ((c >> 2) & 0x33u);
            bad |= c != 0x22u;  // each nibble must have exactly two bits set
            Raw8 r;
            r.a = make_uint4(prmt(v[k], 0, lut[m[k] & 0xFu]), prmt(v[k] >> 16, 0, lut[m[k] >> 4]), 0, 0);
            r.b = make_uint4(0, 0, 0, 0);
            float f[8];
            decode8<F_E4M3>(r, f);
            st_stream((char *)out + (size_t)u * 16, dequant8_to_bf16<false>(f, __uint_as_float(sb[k] << 16)));
        }
    }
    if (__any_sync(0xFFFFFFFFu, bad) && (threadIdx.x & 31) == 0) atomicExch(irregular, irregular_value);
}

extern "C" int64_t ctb_sparse24_dequantize_workspace_bytes(int64_t rows, int64_t cols) { return ctb_bitmask_workspace_bytes(rows, cols); }

extern "C" int ctb_sparse24_decompress_dequantize_fp8(const void *values, int64_t nvalues, const uint8_t *bitmask, const void *scale, int64_t rows,
                                                      int64_t cols, void *out, void *workspace, void *stream) {
    if (rows != 0 && cols != 0 && (!values || !bitmask || !scale || !out || !workspace)) return fail(CTB_EINVAL_NULL, "null buffer");
    if (rows <= 0 || cols <= 0) return rows < 0 || cols < 0 ? fail(CTB_EINVAL_SHAPE, "negative shape") : CTB_OK;
    if (nvalues < 0) return fail(CTB_EINVAL_SHAPE, "negative value count");
    if (cols % 8 != 0) return fail(CTB_EINVAL_SHAPE, "fused 2:4 decompress + dequantize needs cols %% 8 == 0, got %lld", (long long)cols);
    if (!aligned16(out) || (reinterpret_cast<uintptr_t>(values) & 3u) || (reinterpret_cast<uintptr_t>(scale) & 1u))
        return fail(CTB_EINVAL_ALIGN, "out must be 16-byte, values 4-byte, scale 2-byte aligned");
    const int64_t units64 = rows * cols / 8;
    if (units64 >= (1ll << 31) - 4 * 148 * 8 * kThreads) return fail(CTB_EUNSUPPORTED, "more than 2^34 elements in one call");
    const uint32_t units = (uint32_t)units64;
    const FastDiv by_upr = make_fastdiv((uint32_t)(cols / 8));
    const uint16_t *sp = reinterpret_cast<const uint16_t *>(scale);
    cudaStream_t st = as_stream(stream);
    if (nvalues < rows * cols / 2)
        // fewer values than two per run of four: the bitmask decides where they go (generic codec, dequantizing form)
        return decompress_impl(values, bitmask, CTB_E4M3, rows, cols, out, workspace, Gate{nullptr, 0}, stream, true, sp);
    int *flag = reinterpret_cast<int *>(static_cast<char *>(workspace) + flag_offset(rows));
    static std::atomic<int> s_ticket{0x40000001};
    const int ticket = s_ticket.fetch_add(1, std::memory_order_relaxed);  // see Gate: no clearing of the flag word
    sparse24_expand_dequant_fp8_kernel<<<grid_for(units64, (int64_t)kThreads * 4, 16), kThreads, 0, st>>>(values, bitmask, sp, units, by_upr, out, flag, ticket);
    int rc = after_launch("sparse24_expand_dequant_fp8_kernel");
    if (rc) return rc;
    // a bitmask that is not two-per-run opened the gate: the generic codec (dequantizing form) redoes the tensor
    return decompress_impl(values, bitmask, CTB_E4M3, rows, cols, out, workspace, Gate{flag, ticket}, stream, true, sp);
}

// ------------------------------------------------------------------ decompress without caller scratch
//
// Some hosts of this library may not allocate device memory at the point where they decompress:
// an inference server that handed its whole memory budget to a fixed arena at start-up, or a
// loader hook that runs while another component owns the allocator.  For them the per-row start
// offsets that ctb_bitmask_decompress keeps in caller-provided scratch live in this fixed array
// instead.  Every GPU that loads the library holds these 512 KiB until the process exits.
constexpr int64_t kStaticMaxRows = 65536;
static __device__ __align__(256) int64_t g_row_offsets_static[kStaticMaxRows];

// Device address of the array above for the current device.  In host code the array's name is only
// a stand-in for the symbol, so the address is asked of the runtime once per device, with that
// device current, and cached.
static int static_scratch(int64_t **out) {
    static std::atomic<int64_t *> cached[64];  // zero-initialised; two host threads may make their first call at once
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(CTB_ECUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(CTB_EUNSUPPORTED, "device index %d is outside the table of cached scratch addresses", dev);
    int64_t *addr = cached[dev].load(std::memory_order_acquire);
    if (addr == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_row_offsets_static);
        if (e != cudaSuccess || p == nullptr) return fail(CTB_ECUDA, "cudaGetSymbolAddress(g_row_offsets_static): %s", cudaGetErrorString(e));
        addr = static_cast<int64_t *>(p);
        cached[dev].store(addr, std::memory_order_release);
    }
    *out = addr;
    return CTB_OK;
}

extern "C" int ctb_bitmask_decompress_static(const void *values, const uint8_t *bitmask, int32_t dtype, int64_t rows, int64_t cols,
                                             void *out, void *stream) {
    if (rows > kStaticMaxRows)
        return fail(CTB_EINVAL_SHAPE, "ctb_bitmask_decompress_static takes at most %lld rows (got %lld); use ctb_bitmask_decompress with caller scratch",
                    (long long)kStaticMaxRows, (long long)rows);
    int64_t *scratch = nullptr;
    int rc = static_scratch(&scratch);
    if (rc) return rc;
    // every row's slot is rewritten by the popcount pass before the scan reads it: nothing has to start at zero
    const bool fits = rows > 0 && cols > 0 && tile_bytes() <= kStaticMaxRows * 8;
    return decompress_impl(values, bitmask, dtype, rows, cols, out, scratch, Gate{nullptr, 0}, stream, fits);
}
