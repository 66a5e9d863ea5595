// Eight bf16 values of one output channel -> eight e4m3 codes, static per-channel bf16 scale (compute dtype bf16):
// quantization/lifecycle/forward.py:462-489 _quantize with dtype float8_e4m3fn.  Shared by the kernels that quantize
// whole rows with one scale per row (the one-pass FP8 + 2:4 kernel and the whole-shard FP8 kernel).
#pragma once

#include "ctb_codec.cuh"

namespace ctb {

// One chunk by the float arithmetic of the generic quantize tier, an element at a time: the rare path (a scale outside
// the range where the reciprocal product is proven to round like the quotient, a zero point other than zero, or a
// NaN among the inputs, whose code must carry the input's sign).  `chunk` points at the 8 bf16 values.
template <bool HAS_ZP>
__device__ __noinline__ uint2 fp8_codes8_exact(const uint4 *chunk, const uint16_t *scale, const void *zp, int zdt, uint32_t row) {
    const QP q = load_qp(scale, CTB_BF16, HAS_ZP ? zp : nullptr, zdt, nullptr, row);
    const uint16_t *x = reinterpret_cast<const uint16_t *>(chunk);
    uint64_t acc = 0;
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
        float t = scaled_div<CTB_BF16>(bf16_bits_to_f32(x[i]), q);  // forward.py:471
        if (HAS_ZP) t = round_to<CTB_BF16>(t + q.zp);               // forward.py:474
        t = clamp_nan(t, -448.0f, 448.0f);
        uint32_t code = (uint32_t)__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3);
        if (t != t) code = 0x7Fu | ((__float_as_uint(t) >> 24) & 0x80u);  // Tensor.to(float8_e4m3fn) keeps a NaN's sign
        acc |= (uint64_t)code << (8 * i);
    }
    return make_uint2((uint32_t)acc, (uint32_t)(acc >> 32));
}

// The packed tier: q = bf16(x * rcp(s)) ("+ 0" where the module carries a zero point, which turns -0.0 into +0.0),
// then the saturating e4m3 convert, which equals the reference's clamp to +-448 followed by Tensor.to(float8_e4m3fn)
// for every non-NaN value.  `raw` is the chunk already in registers, `chunk` its address for the exact routine.
template <bool HAS_ZP>
__device__ __forceinline__ uint2 fp8_codes8(const uint4 &raw, const uint4 *chunk, const uint16_t *scale, const void *zp, int zdt, uint32_t row) {
    const uint32_t sbits = __ldg(scale + row);
    bool exact = ((sbits >> 7) & 0xFFu) - 28u > 197u;  // biased exponent outside [28, 225]
    if (HAS_ZP) exact = exact || load_f32(zp, zdt, row) != 0.0f;
    if (exact) return fp8_codes8_exact<HAS_ZP>(chunk, scale, zp, zdt, row);
    const float r = rcp_approx(__uint_as_float(sbits << 16));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t c[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t b = bf162_as_u32(HAS_ZP ? scale_pair_plus_zero(w[k], r) : scale_pair(w[k], r));
        c[k] = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__uint_as_float(b << 16), __uint_as_float(b & 0xFFFF0000u)), __NV_SATFINITE,
                                                  __NV_E4M3);
    }
    const uint32_t c0 = c[0] | (c[1] << 16), c1 = c[2] | (c[3] << 16);
    if (((((c0 & 0x7F7F7F7Fu) + 0x01010101u) | ((c1 & 0x7F7F7F7Fu) + 0x01010101u)) & 0x80808080u) != 0)
        return fp8_codes8_exact<HAS_ZP>(chunk, scale, zp, zdt, row);
    return make_uint2(c0, c1);
}

}  // namespace ctb
