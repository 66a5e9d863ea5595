// Per-chunk (8 consecutive elements of one row) load / store / arithmetic used by the quantize,
// dequantize and fused kernels.  Every function restates one step of
// quantization/lifecycle/forward.py:455-514 (_quantize / _dequantize) with the intermediate
// roundings torch performs made explicit.
#pragma once

#include "ctb_common.cuh"

namespace ctb {

// storage format of one side of a kernel
enum Fmt : int {
    F_BF16 = 0,
    F_F16 = 1,
    F_F32 = 2,
    F_I8 = 3,
    F_E4M3 = 4,
    F_PACK4 = 5,  // int4 codes, 8 per int32 word, offset binary (pack_to_int32, num_bits=4)
    F_PACK8 = 6,  // int8 codes, 4 per int32 word, offset binary (pack_to_int32, num_bits=8)
    F_FP4X2 = 7,  // e2m1 codes, 2 per byte, even element in the low nibble
    F_NONE = 8
};

enum QKind : int { QK_INT = 0, QK_FP8 = 1, QK_FP4 = 2 };

#ifdef __CUDACC__

// bytes one 8-element chunk occupies in a format
__host__ __device__ constexpr int chunk_bytes(int f) {
    return f == F_F32 ? 32 : (f == F_BF16 || f == F_F16) ? 16 : (f == F_I8 || f == F_E4M3 || f == F_PACK8) ? 8 : 4;
}

// raw register image of one chunk (enough for the widest format)
struct Raw8 {
    uint4 a, b;
};

template <int F>
__device__ __forceinline__ Raw8 load_raw(const void *base, int64_t chunk) {
    Raw8 r;
    const char *p = (const char *)base + chunk * chunk_bytes(F);
    if constexpr (F == F_F32) {
        r.a = ld_stream(p);
        r.b = ld_stream(p + 16);
    } else if constexpr (F == F_BF16 || F == F_F16) {
        r.a = ld_stream(p);
    } else if constexpr (F == F_I8 || F == F_E4M3 || F == F_PACK8) {
        uint2 t = ld_stream8(p);
        r.a.x = t.x;
        r.a.y = t.y;
    } else {
        r.a.x = ld_stream4(p);
    }
    return r;
}

__device__ __forceinline__ float2 half2_bits_to_float2(uint32_t u) {
    __half2 h = *reinterpret_cast<__half2 *>(&u);
    return __half22float2(h);
}

template <int F>
__device__ __forceinline__ void decode8(const Raw8 &r, float (&v)[8]) {
    if constexpr (F == F_F32) {
        v[0] = __uint_as_float(r.a.x); v[1] = __uint_as_float(r.a.y);
        v[2] = __uint_as_float(r.a.z); v[3] = __uint_as_float(r.a.w);
        v[4] = __uint_as_float(r.b.x); v[5] = __uint_as_float(r.b.y);
        v[6] = __uint_as_float(r.b.z); v[7] = __uint_as_float(r.b.w);
    } else if constexpr (F == F_BF16) {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    } else if constexpr (F == F_F16) {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = half2_bits_to_float2(w[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    } else if constexpr (F == F_I8 || F == F_PACK8) {
        const uint32_t w[2] = {r.a.x, r.a.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t b = (w[i >> 2] >> (8 * (i & 3))) & 0xFFu;
            if constexpr (F == F_PACK8) b ^= 0x80u;  // stored as value + 128
            v[i] = (float)(int)(int8_t)b;
        }
    } else if constexpr (F == F_E4M3) {
        const uint32_t w[2] = {r.a.x, r.a.y};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w[i >> 1] >> (16 * (i & 1))) & 0xFFFFu), __NV_E4M3);
            float2 f = __half22float2(__half2(h));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    } else if constexpr (F == F_PACK4) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (float)((int)((r.a.x >> (4 * i)) & 0xFu) - 8);
    } else if constexpr (F == F_FP4X2) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((r.a.x >> (8 * i)) & 0xFFu), __NV_E2M1);
            float2 f = __half22float2(__half2(h));
            v[2 * i] = f.x;      // low nibble = even element; nibble 0x8 decodes to -0.0
            v[2 * i + 1] = f.y;
        }
    }
}

// store 8 plain values (already exactly representable in the target float dtype, or to be rounded to it)
template <int F>
__device__ __forceinline__ void store8_float(void *base, int64_t chunk, const float (&v)[8]) {
    char *p = (char *)base + chunk * chunk_bytes(F);
    if constexpr (F == F_F32) {
        st_stream(p, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])));
        st_stream(p + 16, make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7])));
    } else if constexpr (F == F_BF16) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        st_stream(p, make_uint4(w[0], w[1], w[2], w[3]));
    } else if constexpr (F == F_F16) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        st_stream(p, make_uint4(w[0], w[1], w[2], w[3]));
    }
}

// Final rounding of 8 clamped values to the quantized grid (quantization/quant_args.py:384-408
// round_to_quantized_type) fused with the store in format F.
//   INT : torch.round (half to even)                      -> I8 / PACK4 / PACK8 / float dtype
//   FP8 : Tensor.to(float8_e4m3fn), NaN keeps its sign   -> E4M3 / float dtype
//   FP4 : FP4_E2M1_DATA.cast_to_fp4 (quant_args.py:55-68) -> FP4X2 / float dtype
// In FP4 an input that is exactly +-0 encodes as +0 while a negative value that rounds to zero
// keeps its sign (nibble 0x8), because the reference multiplies by torch.sign(x).
template <int QK, int F>
__device__ __forceinline__ void encode_store8(void *base, int64_t chunk, float (&v)[8]) {
    char *p = (char *)base + chunk * chunk_bytes(F);
    if constexpr (QK == QK_INT) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = rintf(v[i]);
        if constexpr (F == F_PACK4) {
            uint32_t w = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) w |= (uint32_t)(((int)v[i] + 8) & 0xF) << (4 * i);
            st_stream4(p, w);
        } else if constexpr (F == F_I8 || F == F_PACK8) {
            uint32_t w[2] = {0u, 0u};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                uint32_t b = (uint32_t)((int)v[i]) & 0xFFu;
                if constexpr (F == F_PACK8) b ^= 0x80u;
                w[i >> 2] |= b << (8 * (i & 3));
            }
            st_stream8(p, make_uint2(w[0], w[1]));
        } else {
            store8_float<F>(base, chunk, v);
        }
    } else if constexpr (QK == QK_FP8) {
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t c = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(v[2 * i], v[2 * i + 1]), __NV_SATFINITE, __NV_E4M3);
            if (v[2 * i] != v[2 * i]) c = (c & 0xFF00u) | 0x7Fu | ((__float_as_uint(v[2 * i]) >> 24) & 0x80u);
            if (v[2 * i + 1] != v[2 * i + 1]) c = (c & 0x00FFu) | 0x7F00u | ((__float_as_uint(v[2 * i + 1]) >> 16) & 0x8000u);
            w[i >> 1] |= c << (16 * (i & 1));
        }
        if constexpr (F == F_E4M3) {
            st_stream8(p, make_uint2(w[0], w[1]));
        } else {
            Raw8 r;
            r.a.x = w[0];
            r.a.y = w[1];
            decode8<F_E4M3>(r, v);
            store8_float<F>(base, chunk, v);
        }
    } else {
        uint32_t w = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t c = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(v[2 * i], v[2 * i + 1]), __NV_E2M1, cudaRoundNearest);
            if (v[2 * i] == 0.0f) c &= 0xF7u;      // exact zero in -> +0 out
            if (v[2 * i + 1] == 0.0f) c &= 0x7Fu;
            w |= c << (8 * i);
        }
        if constexpr (F == F_FP4X2) {
            st_stream4(p, w);
        } else {
            Raw8 r;
            r.a.x = w;
            float q[8];
            decode8<F_FP4X2>(r, q);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = (v[i] != v[i]) ? v[i] : q[i];  // NaN stays NaN
            store8_float<F>(base, chunk, v);
        }
    }
}

// Values (not codes) of the quantized grid for 8 clamped inputs: what round_to_quantized_type
// returns before any cast.  Used by fake-quantize, which feeds them straight to the dequantize step.
template <int QK>
__device__ __forceinline__ void round8(float (&v)[8]) {
    if constexpr (QK == QK_INT) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = rintf(v[i]);
    } else if constexpr (QK == QK_FP8) {
        Raw8 r;
        r.a.x = r.a.y = 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t c = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(v[2 * i], v[2 * i + 1]), __NV_SATFINITE, __NV_E4M3);
            if (i < 2) r.a.x |= c << (16 * (i & 1)); else r.a.y |= c << (16 * (i & 1));
        }
        float q[8];
        decode8<F_E4M3>(r, q);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (v[i] != v[i]) ? v[i] : q[i];
    } else {
        Raw8 r;
        r.a.x = 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t c = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(v[2 * i], v[2 * i + 1]), __NV_E2M1, cudaRoundNearest);
            if (v[2 * i] == 0.0f) c &= 0xF7u;
            if (v[2 * i + 1] == 0.0f) c &= 0x7Fu;
            r.a.x |= c << (8 * i);
        }
        float q[8];
        decode8<F_FP4X2>(r, q);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (v[i] != v[i]) ? v[i] : q[i];
    }
}

// ---- packed bf16x2 fast paths for int4 <-> bf16 with a bf16 scale ---------------------------------

__device__ __forceinline__ uint32_t bf162_as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __nv_bfloat162 u32_as_bf162(uint32_t v) { return *reinterpret_cast<__nv_bfloat162 *>(&v); }

// A packed pair of bf16 values already divided by the scale -> clamp to [-8, 7], then add 200: the sum lies in
// [192, 207], where a bf16 step is 1, so the addition rounds half to even and the low byte of each half is
// 0x40 | (code + 8), i.e. its low nibble is the offset-binary int4 code.
__device__ __forceinline__ uint32_t int4_pair_magic(__nv_bfloat162 q) {
    const __nv_bfloat162 lo = u32_as_bf162(0xC100C100u);     // -8, -8
    const __nv_bfloat162 hi = u32_as_bf162(0x40E040E0u);     //  7,  7
    const __nv_bfloat162 magic = u32_as_bf162(0x43484348u);  // 200, 200
    return bf162_as_u32(__hadd2(__hmin2(__hmax2(q, lo), hi), magic));
}

// byte permute by the PTX instruction (selector nibble i picks the source byte of result byte i)
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// 8 bf16 inputs (4 packed words) -> one pack_to_int32 word of int4 codes, compute dtype bf16:
//   q = bf16_rn(x * rcp(s)) [+ zero point, rounded to bf16]; clamp to [-8, 7]; round half to even.
// `zp2` is the zero point replicated in both halves (bf16x2), ignored unless has_zp.
// The eight code bytes are gathered with byte permutes and their low nibbles merged two at a time.
__device__ __forceinline__ uint32_t quant_int4_word_bf16(const uint32_t (&w)[4], float r, bool has_zp, __nv_bfloat162 zp2) {
    uint32_t m[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float f0 = __uint_as_float(w[k] << 16), f1 = __uint_as_float(w[k] & 0xFFFF0000u);
        __nv_bfloat162 q = __floats2bfloat162_rn(f0 * r, f1 * r);
        if (has_zp) q = __hadd2(q, zp2);
        m[k] = int4_pair_magic(q);
    }
    const uint32_t a = prmt_b32(m[0], m[1], 0x6420), b = prmt_b32(m[2], m[3], 0x6420);  // code bytes of elements 0-3, 4-7
    const uint32_t ta = (a & 0x0F0F0F0Fu) | ((a >> 4) & 0xF0F0F0F0u);  // byte 0: elements 0, 1; byte 2: elements 2, 3
    const uint32_t tb = (b & 0x0F0F0F0Fu) | ((b >> 4) & 0xF0F0F0F0u);
    return prmt_b32(ta, tb, 0x6420);
}

// one pack_to_int32 word of int4 codes -> 8 bf16 outputs (4 packed words), compute dtype bf16:
//   (code - zero_point) * scale, both steps exact-or-single-rounded in bf16x2 arithmetic.
// 0x4300 | nibble is the bf16 number 128 + nibble, so subtracting 136 + zp gives code - zp exactly.
__device__ __forceinline__ uint4 dequant_int4_word_bf16(uint32_t word, __nv_bfloat162 s2, __nv_bfloat162 bias2) {
    uint32_t t[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) t[k] = ((word >> (4 * k)) & 0x000F000Fu) | 0x43004300u;  // low half: nibble k, high half: nibble k + 4
    uint32_t p[4] = {__byte_perm(t[0], t[1], 0x5410), __byte_perm(t[2], t[3], 0x5410),   // (n0, n1), (n2, n3)
                     __byte_perm(t[0], t[1], 0x7632), __byte_perm(t[2], t[3], 0x7632)};  // (n4, n5), (n6, n7)
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = bf162_as_u32(__hmul2(__hsub2(u32_as_bf162(p[k]), bias2), s2));
    return make_uint4(p[0], p[1], p[2], p[3]);
}

// 8 bf16 inputs (4 packed words) -> 8 e4m3 codes, compute dtype bf16 (bf16 tensor, bf16 scale):
//   q = bf16_rn(x * rcp(s)) + 0  (the all-zero zero point of a symmetric scheme turns -0.0 into +0.0; folded
//   into the multiply as fma(x, r, +0.0)), then the saturating round-to-nearest-even e4m3 convert, which
//   equals the reference's clamp to +-448 followed by Tensor.to(float8_e4m3fn) for every non-NaN input.
__device__ __forceinline__ uint2 quant_fp8_codes_bf16(const uint32_t (&w)[4], float r) {
    uint32_t c[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float f0 = __uint_as_float(w[k] << 16), f1 = __uint_as_float(w[k] & 0xFFFF0000u);
        const uint32_t q = bf162_as_u32(__floats2bfloat162_rn(fmaf(f0, r, 0.0f), fmaf(f1, r, 0.0f)));
        c[k] = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__uint_as_float(q << 16), __uint_as_float(q & 0xFFFF0000u)),
                                                  __NV_SATFINITE, __NV_E4M3);
    }
    return make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
}

// 8 bf16 inputs (4 packed words) -> 8 e2m1 codes (one 32-bit word, even element in the low nibble), fp32 effective
// scale (NVFP4: e4m3 group scale / fp32 global scale).  x / s is the correctly rounded fp32 quotient (reciprocal +
// Markstein correction; for x = -0.0 the correction step itself yields +0.0, which is also what the reference's
// cast produces for a zero input), and the saturating round-to-nearest-even e2m1 convert equals the reference's
// clamp to +-6 followed by FP4_E2M1_DATA.cast_to_fp4 (ties to the even code, a negative value that rounds to zero
// keeps its sign bit).  Callers guarantee finite inputs and a scale in the normal range.
__device__ __forceinline__ uint32_t quant_fp4_codes_f32(const uint32_t (&w)[4], float s, float r) {
    uint32_t out = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float x0 = __uint_as_float(w[k] << 16), x1 = __uint_as_float(w[k] & 0xFFFF0000u);
        const float a0 = x0 * r, a1 = x1 * r;
        const float q0 = fmaf(fmaf(-a0, s, x0), r, a0), q1 = fmaf(fmaf(-a1, s, x1), r, a1);
        out |= (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(q0, q1), __NV_E2M1, cudaRoundNearest) << (8 * k);
    }
    return out;
}

// 8 values exactly representable in the scale's compute dtype (int8 / e4m3 / e2m1 codes), no zero point:
// value * scale rounded once to bf16 -- what (x_q.to(scale.dtype) * scale).to(bf16) gives for a bf16 scale,
// and, with an fp32 effective scale, the fp32 product rounded to bf16 (NVFP4 decompress).
template <bool F32_PRODUCT>
__device__ __forceinline__ uint4 dequant8_to_bf16(const float (&v)[8], float s) {
    uint32_t p[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = bf162_as_u32(__floats2bfloat162_rn(v[2 * k] * s, v[2 * k + 1] * s));
    return make_uint4(p[0], p[1], p[2], p[3]);
}

// ---- packed bf16x2 quantize helpers shared by the given-qparam tier and the fused calibrate kernels ---------------

__device__ __forceinline__ float rcp_approx(float s) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(s));
    return r;
}

// both halves of one packed word times r, each rounded once to bf16
__device__ __forceinline__ __nv_bfloat162 scale_pair(uint32_t w, float r) {
    return __floats2bfloat162_rn(__uint_as_float(w << 16) * r, __uint_as_float(w & 0xFFFF0000u) * r);
}

// like scale_pair, then "+ 0" (an all-zero zero point turns -0.0 into +0.0)
__device__ __forceinline__ __nv_bfloat162 scale_pair_plus_zero(uint32_t w, float r) {
    return __floats2bfloat162_rn(fmaf(__uint_as_float(w << 16), r, 0.0f), fmaf(__uint_as_float(w & 0xFFFF0000u), r, 0.0f));
}

// int8 codes of four sign-magnitude halves (two words of u = q + copysign(128, q)): |code| bytes, a 0x00 / 0xFF
// sign byte each, then a per-byte negate whose "+ 1" cannot carry into the neighbouring byte
__device__ __forceinline__ uint32_t int8_codes_of(uint32_t u0, uint32_t u1) {
    const uint32_t mag = prmt_b32(u0, u1, 0x6420), neg = prmt_b32(u0, u1, 0xFDB9);
    const uint32_t x = mag ^ neg;
    return ((x & 0x7F7F7F7Fu) + (neg & 0x01010101u)) ^ (x & 0x80808080u);
}

// fake quantize of one packed word to an integer grid, compute dtype bf16 (forward.py:471-512): q = bf16(x * r)
// [+ zero point], clamp (a NaN stays a NaN), u = q + copysign(128, q) rounds half to even because |u| is in
// [128, 256] where a bf16 step is 1, back by the same constant with q's sign put on a zero, [- zero point], * scale.
__device__ __forceinline__ uint32_t fake_int_pair_bf16(uint32_t w, float r, bool has_zp, __nv_bfloat162 z2, __nv_bfloat162 lo2,
                                                       __nv_bfloat162 hi2, __nv_bfloat162 s2) {
    __nv_bfloat162 q = scale_pair(w, r);
    if (has_zp) q = __hadd2(q, z2);
    q = __hmin2_nan(__hmax2_nan(q, lo2), hi2);
    const uint32_t sign = bf162_as_u32(q) & 0x80008000u;
    const __nv_bfloat162 m = u32_as_bf162(sign | 0x43004300u);
    __nv_bfloat162 t = u32_as_bf162(bf162_as_u32(__hsub2(__hadd2(q, m), m)) | sign);
    if (has_zp) t = __hsub2(t, z2);
    return bf162_as_u32(__hmul2(t, s2));
}

// fake quantize of one packed word to e4m3, compute dtype bf16, symmetric (no zero point, or the all-zero one)
__device__ __forceinline__ uint32_t fake_fp8_pair_bf16(uint32_t w, float r, bool plus_zero, float s) {
    const uint32_t q = bf162_as_u32(plus_zero ? scale_pair_plus_zero(w, r) : scale_pair(w, r));
    const uint32_t code = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__uint_as_float(q << 16), __uint_as_float(q & 0xFFFF0000u)),
                                                             __NV_SATFINITE, __NV_E4M3);
    const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)code, __NV_E4M3)));
    return bf162_as_u32(__floats2bfloat162_rn(f.x * s, f.y * s));
}

// qparam for a chunk, as fp32
struct QP {
    float s;   // effective scale (scale or scale / global_scale)
    float r;   // 1 / s, correctly rounded
    float zp;  // zero point value (0 when absent)
    bool slow; // scale outside the range where the reciprocal path is proven exact
};

__device__ __forceinline__ QP load_qp(const void *scale, int sdt, const void *zp, int zdt, const float *gs, int64_t qi) {
    QP q;
    q.s = load_f32(scale, sdt, qi);
    if (gs != nullptr) q.s = __fdiv_rn(q.s, __ldg(gs));  // forward.py:468-469 scale.to(f32) / global_scale
    q.r = __frcp_rn(q.s);
    q.zp = (zp != nullptr) ? load_f32(zp, zdt, qi) : 0.0f;
    float a = fabsf(q.s);
    q.slow = !(a >= 1.0e-30f && a <= 1.0e30f);
    return q;
}

// x / scale rounded to the compute dtype T (forward.py:471 `scaled = x / scale`).
//  T = bf16: both operands carry 8 significant bits, so the exact quotient is at least 2^-17
//            (relative) away from every bf16 rounding boundary while x * rcp(s) is within 2^-23
//            of it: rounding the product gives the same bf16 as rounding the IEEE quotient.
//  otherwise: correctly rounded fp32 quotient (Markstein correction), then the rounding to T.
template <int T>
__device__ __forceinline__ float scaled_div(float x, const QP &q) {
    if (q.slow) return round_to<T>(__fdiv_rn(x, q.s));
    if constexpr (T == CTB_BF16) return round_to<T>(x * q.r);
    else return round_to<T>(div_by_rcp(x, q.s, q.r));
}

// forward.py:471-481: scale, add zero point, clamp.  zp_x is zero_point.to(x.dtype).
template <int T>
__device__ __forceinline__ void quant_prepare8(float (&v)[8], const QP &q, bool has_zp, float zp_x, float qmin, float qmax) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float t = scaled_div<T>(v[i], q);
        if (has_zp) t = round_to<T>(t + zp_x);
        v[i] = clamp_nan(t, qmin, qmax);
    }
}

// the same steps for one element with its own qparam (activation-ordered groups: every column names its group)
template <int T>
__device__ __forceinline__ float quant_prepare1(float x, const QP &q, bool has_zp, float qmin, float qmax) {
    float t = scaled_div<T>(x, q);
    if (has_zp) t = round_to<T>(t + q.zp);
    return clamp_nan(t, qmin, qmax);
}

template <int TS>
__device__ __forceinline__ float dequant1(float v, const QP &q, bool has_zp) {
    float t = round_to<TS>(v);
    if (has_zp) t = round_to<TS>(t - round_to<TS>(q.zp));
    return round_to<TS>(t * q.s);
}

// forward.py:504-512: x_q.to(scale.dtype), subtract zero point, multiply by scale; all in Ts.
template <int TS>
__device__ __forceinline__ void dequant8(float (&v)[8], const QP &q, bool has_zp) {
    float z = round_to<TS>(q.zp);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float t = round_to<TS>(v[i]);
        if (has_zp) t = round_to<TS>(t - z);
        v[i] = round_to<TS>(t * q.s);
    }
}

#endif  // __CUDACC__

}  // namespace ctb
