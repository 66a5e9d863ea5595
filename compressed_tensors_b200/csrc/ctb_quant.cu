// quantize / dequantize / fake_quantize (quantization/lifecycle/forward.py:45-189, :455-514)
// with pack_to_int32 / pack_fp4_to_uint8 and their inverses fused on the quantized side.
//
// Two tiers:
//   vec8    : 8 consecutive elements per step, 128-bit streaming loads, formats and compute
//             dtypes fixed at compile time; needs cols % 8 == 0, col_group % 8 == 0, no g_idx and
//             16-byte aligned buffers.  Bound by HBM: every input byte is read once and every
//             output byte written once.
//   generic : one output unit (element, packed word or fp4 byte) per thread, everything decided
//             at run time; covers ragged shapes, any num_bits, g_idx column maps.
#include "ctb_codec.cuh"
#include "ctb_fastdiv.h"

namespace ctb {

struct QArgs {
    const void *in;
    const void *scale;
    const void *zp;
    const int32_t *g_idx;
    const float *gs;
    void *out;
    int64_t rows, cols, col_group, row_group, srs;
    int64_t chunks;  // rows * cols / 8
    int64_t cpr;     // chunks per row
    int gshift;      // >= 0: qparam index = (8 * chunk) >> gshift; < 0: general indexing
    float qmin, qmax;
    int sdt, zdt;    // scale / zero-point dtypes
    int xdt;         // dense-side dtype
    int T, TS;       // compute dtypes of the quantize and the dequantize half
    int qk;          // QKind
    int bits;
    int fin, fout;   // Fmt of both sides (generic tier)
    FastDiv by_cpr;  // chunk -> row (g_idx tier, BLOCK layouts)
    FastDiv by_row_group, by_col_chunks;  // row -> block row, chunk of a row -> block column
    int idx32;       // chunk indices fit 31 bits: BLOCK layouts index qparams through the dividers
};

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

__device__ __forceinline__ int64_t qp_index_chunk(const QArgs &a, int64_t chunk) {
    if (a.gshift >= 0) return (chunk << 3) >> a.gshift;
    if (a.idx32) {
        const uint32_t c = (uint32_t)chunk, row = fastdiv(c, a.by_cpr);
        return (int64_t)fastdiv(row, a.by_row_group) * a.srs + fastdiv(c - row * (uint32_t)a.cpr, a.by_col_chunks);
    }
    int64_t row = chunk / a.cpr;
    int64_t col = (chunk - row * a.cpr) << 3;
    return (row / a.row_group) * a.srs + col / a.col_group;
}

// MODE 0 quantize, 1 dequantize, 2 fake quantize
template <int MODE, int T, int TS, int QK, int FIN, int FOUT>
__global__ void __launch_bounds__(kThreads) qdq_vec8_kernel(const QArgs a) {
    const bool has_zp = a.zp != nullptr;
    const int64_t stride = (int64_t)gridDim.x * kThreads * kUnroll;
    for (int64_t base = (int64_t)blockIdx.x * kThreads * kUnroll + threadIdx.x; base < a.chunks; base += stride) {
        Raw8 raw[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int64_t c = base + (int64_t)u * kThreads;
            if (c < a.chunks) raw[u] = load_raw<FIN>(a.in, c);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int64_t c = base + (int64_t)u * kThreads;
            if (c >= a.chunks) continue;
            QP q = load_qp(a.scale, a.sdt, a.zp, a.zdt, a.gs, qp_index_chunk(a, c));
            // int4 <-> bf16 with a bf16 scale: packed bf16x2 arithmetic, a few instructions per element
            if constexpr (MODE == 1 && FIN == F_PACK4 && FOUT == F_BF16 && TS == CTB_BF16) {
                uint4 o = dequant_int4_word_bf16(raw[u].a.x, __float2bfloat162_rn(q.s), __float2bfloat162_rn(136.0f + q.zp));
                st_stream((char *)a.out + c * 16, o);
                continue;
            }
            if constexpr (MODE == 0 && FIN == F_BF16 && FOUT == F_PACK4 && T == CTB_BF16 && QK == QK_INT) {
                if (!q.slow) {
                    const uint32_t w[4] = {raw[u].a.x, raw[u].a.y, raw[u].a.z, raw[u].a.w};
                    st_stream4((char *)a.out + c * 4, quant_int4_word_bf16(w, q.r, has_zp, __float2bfloat162_rn(q.zp)));
                    continue;
                }
            }
            if constexpr (MODE == 0 && FIN == F_BF16 && FOUT == F_E4M3 && T == CTB_BF16 && QK == QK_FP8) {
                // symmetric schemes (no zero point, or the all-zero one calculate_qparams returns for them)
                if (!q.slow && (!has_zp || q.zp == 0.0f)) {
                    const uint32_t w[4] = {raw[u].a.x, raw[u].a.y, raw[u].a.z, raw[u].a.w};
                    if (has_zp) {
                        st_stream8((char *)a.out + c * 8, quant_fp8_codes_bf16(w, q.r));
                        continue;
                    }
                }
            }
            float v[8];
            decode8<FIN>(raw[u], v);
            if constexpr (MODE == 1 && FOUT == F_BF16 && (FIN == F_E4M3 || FIN == F_I8 || FIN == F_PACK8 || FIN == F_FP4X2)) {
                if (!has_zp) {  // codes are exact in the compute dtype: one multiply, one rounding to bf16
                    st_stream((char *)a.out + c * 16, dequant8_to_bf16<TS == CTB_F32>(v, q.s));
                    continue;
                }
            }
            if constexpr (MODE == 0) {
                quant_prepare8<T>(v, q, has_zp, q.zp, a.qmin, a.qmax);
                encode_store8<QK, FOUT>(a.out, c, v);
            } else if constexpr (MODE == 1) {
                dequant8<TS>(v, q, has_zp);
                store8_float<FOUT>(a.out, c, v);
            } else {
                quant_prepare8<T>(v, q, has_zp, q.zp, a.qmin, a.qmax);
                round8<QK>(v);
                dequant8<TS>(v, q, has_zp);
                store8_float<FOUT>(a.out, c, v);
            }
        }
    }
}

// The vec8 tier with a column -> group map (g_idx, forward.py:300-352: activation-ordered groups).  The reference
// permutes the columns so that groups become contiguous, quantizes group by group and permutes back; element for
// element that is "column c uses qparam g_idx[c] of its row".  Loads and stores stay 8 elements wide; the eight
// group numbers of a chunk are two 16-byte loads and the qparams eight small gathers that hit in L1 / L2.
template <int MODE, int T, int TS, int QK, int FIN, int FOUT>
__device__ __forceinline__ void gidx_chunk_float(const QArgs &a, uint32_t c, uint32_t row, uint32_t col0) {
    const bool has_zp = a.zp != nullptr;
    const Raw8 raw = load_raw<FIN>(a.in, c);
    const int4 g0 = __ldg(reinterpret_cast<const int4 *>(a.g_idx + col0)), g1 = __ldg(reinterpret_cast<const int4 *>(a.g_idx + col0 + 4));
    const int g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const int64_t base = (int64_t)row * a.srs;
    float v[8];
    decode8<FIN>(raw, v);
    QP q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = load_qp(a.scale, a.sdt, a.zp, a.zdt, a.gs, base + g[i]);
    if constexpr (MODE != 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = quant_prepare1<T>(v[i], q[i], has_zp, a.qmin, a.qmax);
    }
    if constexpr (MODE == 0) {
        encode_store8<QK, FOUT>(a.out, c, v);
    } else {
        if constexpr (MODE == 2) round8<QK>(v);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = dequant1<TS>(v[i], q[i], has_zp);
        store8_float<FOUT>(a.out, c, v);
    }
}

template <int MODE, int T, int TS, int QK, int FIN, int FOUT>
__global__ void __launch_bounds__(kThreads) qdq_vec8_gidx_kernel(const QArgs a) {
    const FastDiv by_cpr = a.by_cpr;
    for (uint32_t c = blockIdx.x * kThreads + threadIdx.x; c < (uint32_t)a.chunks; c += gridDim.x * kThreads) {
        const uint32_t row = fastdiv(c, by_cpr);
        gidx_chunk_float<MODE, T, TS, QK, FIN, FOUT>(a, c, row, (c - row * (uint32_t)a.cpr) * 8);
    }
}

// ---- lean tier: bf16 tensor, bf16 scale (compute dtype bf16), 32-bit chunk indices ---------------------------
//
// The vec8 kernel above spends as many instructions per chunk on bookkeeping (64-bit indices, a run-time switch
// per qparam load, an IEEE reciprocal) as on arithmetic, and its quantize half works one float at a time.  This
// tier keeps every step in packed bf16x2 registers:
//   q    = bf16_rn(x * rcp(s))          rcp.approx is within 1 ulp, far inside the 2^-17 margin that keeps the
//                                       rounded product equal to the rounded IEEE quotient of two bf16 numbers
//   q   += zero_point (bf16 add), clamp to [q_min, q_max]
//   INT : u = q + copysign(128, q) is exact-or-rounded-half-to-even to an integer because |u| lies in [128, 256],
//         where a bf16 step is 1; the low byte of each half of u is |code| and its sign bit the code's sign.
//         u - copysign(128, q) is the rounded value itself (fake quantize), with q's sign put back on a zero.
//   FP8 : saturating e4m3 convert of q.
// A chunk whose scale lies outside [2^-99, 2^99), an FP8 chunk that produced a NaN code, or an FP8 zero point
// other than zero, is recomputed by the float path of the vec8 tier (lean_exact_chunk).
struct LeanArgs {
    const uint4 *in;
    const void *scale;  // bf16 or fp32 (template parameter ST of the kernel)
    const void *zp;
    void *out;
    uint32_t chunks, cpr, srs;
    int shift;  // >= 0: qparam index = chunk >> shift; < 0: [row_group x col_group] blocks through the dividers
    FastDiv by_cpr, by_row_group, by_col_chunks;
    float qmin, qmax;
    int zdt;
};

// One chunk by the float arithmetic of the vec8 tier, an element at a time (few registers: this is the rare path
// and its register count would otherwise bound the occupancy of the whole kernel).
template <int MODE, int QK, int FOUT, int ST>
__device__ __noinline__ void lean_exact_chunk(const LeanArgs &a, uint32_t c, uint32_t qi) {
    const bool has_zp = a.zp != nullptr;
    const QP q = load_qp(a.scale, ST, a.zp, a.zdt, nullptr, qi);
    const uint16_t *x = reinterpret_cast<const uint16_t *>(a.in + c);
    uint64_t acc = 0;
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
        float t = scaled_div<ST>(bf16_bits_to_f32(x[i]), q);       // forward.py:471-481
        if (has_zp) t = round_to<ST>(t + q.zp);
        t = clamp_nan(t, a.qmin, a.qmax);
        float val;
        if constexpr (QK == QK_INT) {
            val = rintf(t);
            const uint32_t code = (uint32_t)(int)val;
            if constexpr (FOUT == F_PACK4) acc |= (uint64_t)((code + 8u) & 0xFu) << (4 * i);
            else if constexpr (FOUT == F_PACK8) acc |= (uint64_t)((code & 0xFFu) ^ 0x80u) << (8 * i);
            else acc |= (uint64_t)(code & 0xFFu) << (8 * i);
        } else {
            uint32_t code = (uint32_t)__nv_cvt_float_to_fp8(t, __NV_SATFINITE, __NV_E4M3);
            if (t != t) code = 0x7Fu | ((__float_as_uint(t) >> 24) & 0x80u);  // Tensor.to(float8_e4m3fn) keeps a NaN's sign
            acc |= (uint64_t)code << (8 * i);
            val = (t != t) ? t : e4m3_to_f32((uint8_t)code);
        }
        if constexpr (MODE == 2) {  // forward.py:504-512, every step rounded to the scale dtype, the result to bf16
            float d = round_to<ST>(val);
            if (has_zp) d = round_to<ST>(d - round_to<ST>(q.zp));
            store_f32(a.out, CTB_BF16, (int64_t)c * 8 + i, round_to<ST>(d * q.s));
        }
    }
    if constexpr (MODE == 0) {
        if constexpr (FOUT == F_PACK4) st_stream4((char *)a.out + (size_t)c * 4, (uint32_t)acc);
        else st_stream8((char *)a.out + (size_t)c * 8, make_uint2((uint32_t)acc, (uint32_t)(acc >> 32)));
    }
}

constexpr int kLeanUnroll = 2;

// 32 registers (a few bytes of spill in the rare path): eight resident blocks per SM measured faster than six at 40
template <int MODE, int QK, int FOUT, int ST>
__global__ void __launch_bounds__(kThreads, ST == CTB_BF16 ? 8 : 6) quant_bf16_lean_kernel(const __grid_constant__ LeanArgs a) {
    const bool has_zp = a.zp != nullptr;
    const __nv_bfloat162 lo2 = __float2bfloat162_rn(a.qmin), hi2 = __float2bfloat162_rn(a.qmax);
    const uint32_t stride = gridDim.x * (uint32_t)(kThreads * kLeanUnroll);
    for (uint32_t base = blockIdx.x * (uint32_t)(kThreads * kLeanUnroll) + threadIdx.x; base < a.chunks; base += stride) {
        uint4 raw[kLeanUnroll];
#pragma unroll
        for (int u = 0; u < kLeanUnroll; ++u) {
            const uint32_t c = base + u * kThreads;
            if (c < a.chunks) raw[u] = ld_stream(a.in + c);
        }
#pragma unroll
        for (int u = 0; u < kLeanUnroll; ++u) {
            const uint32_t c = base + u * kThreads;
            if (c >= a.chunks) break;
            uint32_t qi;
            if (a.shift >= 0) {
                qi = c >> a.shift;
            } else {
                const uint32_t row = fastdiv(c, a.by_cpr);
                qi = fastdiv(row, a.by_row_group) * a.srs + fastdiv(c - row * a.cpr, a.by_col_chunks);
            }
            uint32_t sbits;  // the scale's bits (bf16: low half)
            if constexpr (ST == CTB_BF16) sbits = __ldg(reinterpret_cast<const uint16_t *>(a.scale) + qi);
            else sbits = __ldg(reinterpret_cast<const uint32_t *>(a.scale) + qi);
            const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
            bool exact = ((sbits >> (ST == CTB_BF16 ? 7 : 23)) & 0xFFu) - 28u > 197u;  // biased exponent outside [28, 225]
            float zf = 0.0f;
            if (has_zp) {
                zf = load_f32(a.zp, a.zdt, qi);
                if constexpr (QK == QK_FP8) exact = exact || zf != 0.0f;
            }
            if (exact) {
                lean_exact_chunk<MODE, QK, FOUT, ST>(a, c, qi);
                continue;
            }
            if constexpr (ST == CTB_F32) {
                // fp32 scale: compute dtype fp32.  x / s is the correctly rounded quotient (reciprocal + Markstein step),
                // the zero point an fp32 add, rounding to the grid by the convert instructions.
                const float sc = __uint_as_float(sbits), r = __frcp_rn(sc);
                float q[8];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    q[2 * k] = div_by_rcp(__uint_as_float(w[k] << 16), sc, r);
                    q[2 * k + 1] = div_by_rcp(__uint_as_float(w[k] & 0xFFFF0000u), sc, r);
                }
                if (has_zp) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) q[i] += zf;
                }
                if constexpr (QK == QK_INT) {
                    if constexpr (MODE == 0) {
                        int code[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) code[i] = __float2int_rn(fminf(fmaxf(q[i], a.qmin), a.qmax));
                        const uint32_t b0 = prmt_b32(prmt_b32(code[0], code[1], 0x0040), prmt_b32(code[2], code[3], 0x0040), 0x5410);
                        const uint32_t b1 = prmt_b32(prmt_b32(code[4], code[5], 0x0040), prmt_b32(code[6], code[7], 0x0040), 0x5410);
                        if constexpr (FOUT == F_PACK4) {  // (code + 8) & 15 == (code & 15) ^ 8; then two nibbles per byte
                            const uint32_t n0 = (b0 & 0x0F0F0F0Fu) ^ 0x08080808u, n1 = (b1 & 0x0F0F0F0Fu) ^ 0x08080808u;
                            const uint32_t t0 = n0 | ((n0 >> 4) & 0xF0F0F0F0u), t1 = n1 | ((n1 >> 4) & 0xF0F0F0F0u);
                            st_stream4((char *)a.out + (size_t)c * 4, prmt_b32(t0, t1, 0x6420));
                        } else if constexpr (FOUT == F_PACK8) {
                            st_stream8((char *)a.out + (size_t)c * 8, make_uint2(b0 ^ 0x80808080u, b1 ^ 0x80808080u));
                        } else {
                            st_stream8((char *)a.out + (size_t)c * 8, make_uint2(b0, b1));
                        }
                    } else {
                        uint32_t o[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float d0 = rintf(clamp_nan(q[2 * k], a.qmin, a.qmax)), d1 = rintf(clamp_nan(q[2 * k + 1], a.qmin, a.qmax));
                            if (has_zp) { d0 -= zf; d1 -= zf; }
                            o[k] = bf162_as_u32(__floats2bfloat162_rn(d0 * sc, d1 * sc));
                        }
                        st_stream((char *)a.out + (size_t)c * 16, make_uint4(o[0], o[1], o[2], o[3]));
                    }
                } else {
                    uint32_t code[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        code[k] = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(q[2 * k], q[2 * k + 1]), __NV_SATFINITE, __NV_E4M3);
                    const uint32_t c0 = code[0] | (code[1] << 16), c1 = code[2] | (code[3] << 16);
                    if constexpr (MODE == 0) {
                        if (((((c0 & 0x7F7F7F7Fu) + 0x01010101u) | ((c1 & 0x7F7F7F7Fu) + 0x01010101u)) & 0x80808080u) != 0) {
                            lean_exact_chunk<MODE, QK, FOUT, ST>(a, c, qi);  // a NaN code must carry its input's sign
                            continue;
                        }
                        st_stream8((char *)a.out + (size_t)c * 8, make_uint2(c0, c1));
                    } else {
                        uint32_t o[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)code[k], __NV_E4M3)));
                            o[k] = bf162_as_u32(__floats2bfloat162_rn(f.x * sc, f.y * sc));
                        }
                        st_stream((char *)a.out + (size_t)c * 16, make_uint4(o[0], o[1], o[2], o[3]));
                    }
                }
                continue;
            }
            const float r = rcp_approx(__uint_as_float(sbits << 16));
            const __nv_bfloat162 z2 = __float2bfloat162_rn(zf);
            if constexpr (QK == QK_INT && FOUT == F_PACK4) {
                st_stream4((char *)a.out + (size_t)c * 4, quant_int4_word_bf16(w, r, has_zp, z2));
            } else if constexpr (QK == QK_INT) {
                const __nv_bfloat162 s2 = u32_as_bf162(sbits * 0x00010001u);
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if constexpr (MODE == 0) {
                        // codes: a NaN input takes q_min (its integer cast is unspecified in the reference)
                        __nv_bfloat162 q = scale_pair(w[k], r);
                        if (has_zp) q = __hadd2(q, z2);
                        q = __hmin2(__hmax2(q, lo2), hi2);
                        const uint32_t sign = bf162_as_u32(q) & 0x80008000u;
                        o[k] = bf162_as_u32(__hadd2(q, u32_as_bf162(sign | 0x43004300u)));  // sign-magnitude: 128 + |code|
                    } else {
                        o[k] = fake_int_pair_bf16(w[k], r, has_zp, z2, lo2, hi2, s2);
                    }
                }
                if constexpr (MODE == 0) {
                    uint32_t c0 = int8_codes_of(o[0], o[1]), c1 = int8_codes_of(o[2], o[3]);
                    if constexpr (FOUT == F_PACK8) { c0 ^= 0x80808080u; c1 ^= 0x80808080u; }
                    st_stream8((char *)a.out + (size_t)c * 8, make_uint2(c0, c1));
                } else {
                    st_stream((char *)a.out + (size_t)c * 16, make_uint4(o[0], o[1], o[2], o[3]));
                }
            } else {  // FP8
                uint32_t code[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t q = bf162_as_u32(has_zp ? scale_pair_plus_zero(w[k], r) : scale_pair(w[k], r));
                    code[k] = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(__uint_as_float(q << 16), __uint_as_float(q & 0xFFFF0000u)),
                                                                 __NV_SATFINITE, __NV_E4M3);
                }
                const uint32_t c0 = code[0] | (code[1] << 16), c1 = code[2] | (code[3] << 16);
                if constexpr (MODE == 0) {
                    // a NaN code (0x7F under the sign bit) must carry its input's sign: rare, take the float path
                    if (((((c0 & 0x7F7F7F7Fu) + 0x01010101u) | ((c1 & 0x7F7F7F7Fu) + 0x01010101u)) & 0x80808080u) != 0) {
                        lean_exact_chunk<MODE, QK, FOUT, ST>(a, c, qi);
                        continue;
                    }
                    st_stream8((char *)a.out + (size_t)c * 8, make_uint2(c0, c1));
                } else {
                    const float s = __uint_as_float(sbits << 16);
                    uint32_t o[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)code[k], __NV_E4M3)));
                        o[k] = bf162_as_u32(__floats2bfloat162_rn(f.x * s, f.y * s));
                    }
                    st_stream((char *)a.out + (size_t)c * 16, make_uint4(o[0], o[1], o[2], o[3]));
                }
            }
        }
    }
}

// ---- activation-ordered groups on the packed tier -----------------------------------------------------------
// bf16 tensor, bf16 scales, int codes.  A block takes a row: the row's qparams (one per group, a few hundred) are
// staged in shared memory once -- reciprocal, scale and zero point ready to use -- and every element then costs one
// shared-memory lookup by its group number instead of a global gather, a reciprocal and a range check.  The
// arithmetic is that of the packed tier, with a different scale in each half of a bf16x2 register.  A row with a
// scale outside [2^-99, 2^99) is redone by the float path (gidx_chunk_float).
struct GidxSmem {
    float r;      // 1 / scale (rcp.approx: within 1 ulp, see the packed tier)
    uint32_t sz;  // scale bits | zero point (bf16 bits) << 16
};

constexpr int kGidxThreads = 128;  // short rows per block: more blocks in different phases hide the per-row barriers

template <int MODE, int FC>  // FC: format of the codes (F_PACK4 / F_I8); unused for fake quantize
__global__ void __launch_bounds__(kGidxThreads) gidx_row_kernel(const QArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    GidxSmem *qp = reinterpret_cast<GidxSmem *>(smem_raw);  // [srs]
    const bool has_zp = a.zp != nullptr;
    const uint32_t srs = (uint32_t)a.srs, cpr = (uint32_t)a.cpr;
    const __nv_bfloat162 lo2 = __float2bfloat162_rn(a.qmin), hi2 = __float2bfloat162_rn(a.qmax);
    const uint16_t *scale = reinterpret_cast<const uint16_t *>(a.scale);
    for (uint32_t row = blockIdx.x; row < (uint32_t)a.rows; row += gridDim.x) {
        __syncthreads();  // the previous row is done with the table
        int bad = 0;
        for (uint32_t j = threadIdx.x; j < srs; j += kGidxThreads) {
            const uint32_t sb = __ldg(scale + (size_t)row * srs + j);
            bad |= ((sb >> 7) & 0xFFu) - 28u > 197u;
            const float zf = has_zp ? load_f32(a.zp, a.zdt, (int64_t)row * srs + j) : 0.0f;
            const __nv_bfloat16 zb = __float2bfloat16_rn(zf);
            qp[j].r = rcp_approx(__uint_as_float(sb << 16));
            qp[j].sz = sb | ((uint32_t)(*reinterpret_cast<const uint16_t *>(&zb)) << 16);
        }
        const bool exact = __syncthreads_or(bad) != 0;
        for (uint32_t cc = threadIdx.x; cc < cpr; cc += kGidxThreads) {
            const uint32_t c = row * cpr + cc, col0 = cc * 8;
            if (exact) {
                if constexpr (MODE == 0) gidx_chunk_float<0, CTB_BF16, CTB_F32, QK_INT, F_BF16, FC>(a, c, row, col0);
                else if constexpr (MODE == 1) gidx_chunk_float<1, CTB_F32, CTB_BF16, QK_INT, FC, F_BF16>(a, c, row, col0);
                else gidx_chunk_float<2, CTB_BF16, CTB_BF16, QK_INT, F_BF16, F_BF16>(a, c, row, col0);
                continue;
            }
            const int4 g0 = __ldg(reinterpret_cast<const int4 *>(a.g_idx + col0)), g1 = __ldg(reinterpret_cast<const int4 *>(a.g_idx + col0 + 4));
            const int gi[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            float r[8];
            uint32_t s2[4], z2[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // an out-of-range group number reads the last entry instead of faulting
                const GidxSmem e0 = qp[min((uint32_t)gi[2 * k], srs - 1)], e1 = qp[min((uint32_t)gi[2 * k + 1], srs - 1)];
                r[2 * k] = e0.r;
                r[2 * k + 1] = e1.r;
                s2[k] = prmt_b32(e0.sz, e1.sz, 0x5410);
                z2[k] = prmt_b32(e0.sz, e1.sz, 0x7632);
            }
            if constexpr (MODE == 1) {
                uint32_t p[4];  // the codes as bf16 pairs, exactly
                if constexpr (FC == F_PACK4) {
                    const uint32_t word = ld_stream4(reinterpret_cast<const uint32_t *>(a.in) + c);
                    uint32_t t[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) t[k] = ((word >> (4 * k)) & 0x000F000Fu) | 0x43004300u;  // 128 + nibble; low half k, high half k + 4
                    p[0] = prmt_b32(t[0], t[1], 0x5410); p[1] = prmt_b32(t[2], t[3], 0x5410);
                    p[2] = prmt_b32(t[0], t[1], 0x7632); p[3] = prmt_b32(t[2], t[3], 0x7632);
#pragma unroll
                    for (int k = 0; k < 4; ++k)  // (128 + nibble) - 136 = code, exact
                        p[k] = bf162_as_u32(__hsub2(u32_as_bf162(p[k]), u32_as_bf162(0x43084308u)));
                } else {
                    const uint2 w = ld_stream8(reinterpret_cast<const uint2 *>(a.in) + c);
                    const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t h = ww[k >> 1] >> (16 * (k & 1));
                        p[k] = bf162_as_u32(__floats2bfloat162_rn((float)(int)(int8_t)(h & 0xFFu), (float)(int)(int8_t)((h >> 8) & 0xFFu)));
                    }
                }
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    __nv_bfloat162 t = u32_as_bf162(p[k]);
                    if (has_zp) t = __hsub2(t, u32_as_bf162(z2[k]));
                    o[k] = bf162_as_u32(__hmul2(t, u32_as_bf162(s2[k])));
                }
                st_stream((char *)a.out + (size_t)c * 16, make_uint4(o[0], o[1], o[2], o[3]));
            } else {
                const uint4 raw = ld_stream(reinterpret_cast<const uint4 *>(a.in) + c);
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    __nv_bfloat162 q = __floats2bfloat162_rn(__uint_as_float(w[k] << 16) * r[2 * k], __uint_as_float(w[k] & 0xFFFF0000u) * r[2 * k + 1]);
                    if (has_zp) q = __hadd2(q, u32_as_bf162(z2[k]));
                    if constexpr (MODE == 0) q = __hmin2(__hmax2(q, lo2), hi2);
                    else q = __hmin2_nan(__hmax2_nan(q, lo2), hi2);
                    const uint32_t sign = bf162_as_u32(q) & 0x80008000u;
                    const __nv_bfloat162 m = u32_as_bf162(sign | 0x43004300u);
                    const __nv_bfloat162 uu = __hadd2(q, m);  // |uu| in [128, 256]: the add rounds half to even to an integer
                    if constexpr (MODE == 0) {
                        o[k] = bf162_as_u32(uu);
                    } else {
                        __nv_bfloat162 t = u32_as_bf162(bf162_as_u32(__hsub2(uu, m)) | sign);
                        if (has_zp) t = __hsub2(t, u32_as_bf162(z2[k]));
                        o[k] = bf162_as_u32(__hmul2(t, u32_as_bf162(s2[k])));
                    }
                }
                if constexpr (MODE == 2) {
                    st_stream((char *)a.out + (size_t)c * 16, make_uint4(o[0], o[1], o[2], o[3]));
                } else {
                    const uint32_t c0 = int8_codes_of(o[0], o[1]), c1 = int8_codes_of(o[2], o[3]);
                    if constexpr (FC == F_I8) {
                        st_stream8((char *)a.out + (size_t)c * 8, make_uint2(c0, c1));
                    } else {  // (code + 8) & 15 == (code & 15) ^ 8, two nibbles per byte
                        const uint32_t n0 = (c0 & 0x0F0F0F0Fu) ^ 0x08080808u, n1 = (c1 & 0x0F0F0F0Fu) ^ 0x08080808u;
                        const uint32_t t0 = n0 | ((n0 >> 4) & 0xF0F0F0F0u), t1 = n1 | ((n1 >> 4) & 0xF0F0F0F0u);
                        st_stream4((char *)a.out + (size_t)c * 4, prmt_b32(t0, t1, 0x6420));
                    }
                }
            }
        }
    }
}

// NVFP4 decompress (compressors/quantized_compressors/fp4_quantized.py:123-148 unpack, lifecycle/forward.py:468-469
// and :500-509 for the arithmetic): e2m1 codes, e4m3 group scales under an fp32 global scale, bf16 out.  One lane
// per 8 elements (4 code bytes in, 16 bytes out, both fully coalesced); the two lanes of a group read the same
// scale byte.  There are only 256 possible scale bytes, so the effective scales float(e4m3) / global_scale are
// divided once per block (IEEE division, exactly what the reference computes) into a shared table, and a chunk
// costs one table read instead of a division.
__global__ void __launch_bounds__(kThreads) dequant_fp4_g16_bf16_kernel(const void *codes, const uint8_t *scale, const float *gs, int64_t chunks, void *out) {
    __shared__ float s_eff[256];
    static_assert(kThreads == 256, "one table entry per thread");
    s_eff[threadIdx.x] = __fdiv_rn(e4m3_to_f32((uint8_t)threadIdx.x), __ldg(gs));
    __syncthreads();
    constexpr int U = 8;
    const int64_t stride = (int64_t)gridDim.x * kThreads * U;
    for (int64_t base = (int64_t)blockIdx.x * kThreads * U + threadIdx.x; base < chunks; base += stride) {
        uint32_t w[U], sb[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t c = base + (int64_t)u * kThreads;
            w[u] = 0;
            sb[u] = 0;
            if (c < chunks) {
                w[u] = ld_stream4((const char *)codes + c * 4);
                sb[u] = scale[c >> 1];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t c = base + (int64_t)u * kThreads;
            if (c >= chunks) break;
            const float s = s_eff[sb[u]];
            uint32_t p[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // low nibble = even element; nibble 0x8 decodes to -0.0, which the product keeps
                const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((w[u] >> (8 * i)) & 0xFFu), __NV_E2M1);
                const float2 f = __half22float2(__half2(h));
                p[i] = bf162_as_u32(__floats2bfloat162_rn(f.x * s, f.y * s));  // fp32 product, then one rounding to bf16
            }
            st_stream((char *)out + c * 16, make_uint4(p[0], p[1], p[2], p[3]));
        }
    }
}

// ------------------------------------------------------------------ generic tier

__device__ __forceinline__ float quant_scalar(const QArgs &a, float x, float s, bool has_zp, float zp) {
    float t = round_to_rt(a.T, __fdiv_rn(x, s));
    if (has_zp) t = round_to_rt(a.T, t + zp);
    t = clamp_nan(t, a.qmin, a.qmax);
    if (a.qk == QK_INT) return rintf(t);
    if (a.qk == QK_FP8) return (t != t) ? t : e4m3_to_f32(f32_to_e4m3(t));
    // FP4_E2M1_DATA.cast_to_fp4, quant_args.py:55-68
    if (t != t) return t;
    float sign = (t > 0.0f) ? 1.0f : ((t < 0.0f) ? -1.0f : 0.0f);
    float m = fabsf(t), r;
    if (m <= 0.25f) r = 0.0f;
    else if (m < 0.75f) r = 0.5f;
    else if (m <= 1.25f) r = 1.0f;
    else if (m < 1.75f) r = 1.5f;
    else if (m <= 2.5f) r = 2.0f;
    else if (m < 3.5f) r = 3.0f;
    else if (m <= 5.0f) r = 4.0f;
    else r = 6.0f;
    return r * sign;
}

__device__ __forceinline__ float dequant_scalar(const QArgs &a, float q, float s, bool has_zp, float zp) {
    float t = round_to_rt(a.TS, q);
    if (has_zp) t = round_to_rt(a.TS, t - round_to_rt(a.TS, zp));
    return round_to_rt(a.TS, t * s);
}

__device__ __forceinline__ uint32_t e2m1_nibble(float v) {
    // index of the grid magnitude (exact for grid values) with the sign bit of v
    float m = fabsf(v);
    uint32_t idx = m < 0.25f ? 0 : m < 0.75f ? 1 : m < 1.25f ? 2 : m < 1.75f ? 3 : m < 2.5f ? 4 : m < 3.5f ? 5 : m < 5.0f ? 6 : 7;
    return idx | ((__float_as_uint(v) >> 31) << 3);
}

__device__ __forceinline__ float e2m1_value(uint32_t nib) {
    const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float m = mag[nib & 7];
    return (nib & 8) ? -m : m;
}

__device__ __forceinline__ int fmt_dtype(int f) {
    return f == F_BF16 ? CTB_BF16 : f == F_F16 ? CTB_F16 : f == F_F32 ? CTB_F32 : f == F_I8 ? CTB_I8 : CTB_E4M3;
}

// load the quantized-side value of element (row, col) for the generic dequantize
__device__ __forceinline__ float load_code(const QArgs &a, int64_t row, int64_t col) {
    if (a.fin == F_PACK4 || a.fin == F_PACK8) {
        int pf = 32 / a.bits;
        int64_t pc = (a.cols + pf - 1) / pf;
        int32_t w = ((const int32_t *)a.in)[row * pc + col / pf];
        int32_t u = (w >> (a.bits * (int)(col % pf))) & ((1 << a.bits) - 1);
        return (float)(u - (1 << (a.bits - 1)));
    }
    if (a.fin == F_FP4X2) {
        uint8_t b = ((const uint8_t *)a.in)[(row * a.cols + col) >> 1];
        return e2m1_value((col & 1) ? (b >> 4) : (b & 0xF));
    }
    return load_f32(a.in, fmt_dtype(a.fin), row * a.cols + col);
}

template <int MODE>
__global__ void __launch_bounds__(kThreads) qdq_generic_kernel(const QArgs a) {
    const bool has_zp = a.zp != nullptr;
    const bool pack32 = (MODE == 0) && (a.fout == F_PACK4 || a.fout == F_PACK8);
    const bool fp4x2 = (MODE == 0) && (a.fout == F_FP4X2);
    const int per = pack32 ? 32 / a.bits : (fp4x2 ? 2 : 1);
    const int64_t upr = (a.cols + per - 1) / per;  // units per row
    const int64_t units = a.rows * upr;
    for (int64_t u = (int64_t)blockIdx.x * kThreads + threadIdx.x; u < units; u += (int64_t)gridDim.x * kThreads) {
        int64_t row = u / upr, c0 = (u - row * upr) * per;
        uint32_t word = 0;
        for (int k = 0; k < per; ++k) {
            int64_t col = c0 + k;
            if (col >= a.cols) break;
            int64_t g = a.g_idx ? (int64_t)a.g_idx[col] : col / a.col_group;
            int64_t qi = (row / a.row_group) * a.srs + g;
            float s = load_f32(a.scale, a.sdt, qi);
            if (a.gs) s = __fdiv_rn(s, a.gs[0]);
            float zp = has_zp ? load_f32(a.zp, a.zdt, qi) : 0.0f;
            int64_t i = row * a.cols + col;
            if (MODE == 1) {
                float v = dequant_scalar(a, load_code(a, row, col), s, has_zp, zp);
                store_f32(a.out, fmt_dtype(a.fout), i, v);
                continue;
            }
            float q = quant_scalar(a, load_f32(a.in, a.xdt, i), s, has_zp, zp);
            if (MODE == 2) {
                store_f32(a.out, fmt_dtype(a.fout), i, dequant_scalar(a, q, s, has_zp, zp));
            } else if (pack32) {
                // pack_quantized.py:219-242: (value + offset).to(uint8) << (bits * k)
                word |= (uint32_t)(uint8_t)((int)q + (1 << (a.bits - 1))) << (a.bits * k);
            } else if (fp4x2) {
                word |= e2m1_nibble(q) << (4 * k);
            } else {
                store_f32(a.out, fmt_dtype(a.fout), i, q);
            }
        }
        if (pack32) ((int32_t *)a.out)[u] = (int32_t)word;
        if (fp4x2) ((uint8_t *)a.out)[u] = (uint8_t)word;
    }
}

}  // namespace ctb

// ------------------------------------------------------------------ host dispatch

namespace ctb {

static int dtype_to_fmt(int dt) {
    switch (dt) {
    case CTB_BF16: return F_BF16;
    case CTB_F16: return F_F16;
    case CTB_F32: return F_F32;
    case CTB_I8: return F_I8;
    case CTB_E4M3: return F_E4M3;
    default: return F_NONE;
    }
}

// format of the quantized side
static int code_fmt(const ctb_qdesc *d) {
    if (d->codec == CTB_CODE_PACK32) return d->num_bits == 4 ? F_PACK4 : F_PACK8;  // other widths: generic only
    if (d->codec == CTB_CODE_FP4X2) return F_FP4X2;
    return dtype_to_fmt(d->q_dtype);
}

static int validate(const ctb_qdesc *d, const void *in, const void *scale, const void *out, int mode) {
    if (!d) return fail(CTB_EINVAL_NULL, "null descriptor");
    if (d->rows != 0 && d->cols != 0 && (!in || !scale || !out)) return fail(CTB_EINVAL_NULL, "null buffer");  // an empty tensor has no storage
    if (d->rows < 0 || d->cols < 0) return fail(CTB_EINVAL_SHAPE, "negative shape");
    if (d->col_group <= 0 || d->row_group <= 0) return fail(CTB_EINVAL_SHAPE, "group sizes must be positive");
    // forward.py:277-282 / :215-224: columns (rows) must divide into whole groups (blocks)
    if (d->cols % d->col_group != 0)
        return fail(CTB_EINVAL_SHAPE, "tensor column shape must be divisble by the given group_size %lld but got %lld",
                    (long long)d->col_group, (long long)d->cols);
    if (d->rows % d->row_group != 0)
        return fail(CTB_EINVAL_SHAPE, "Tensor height %lld is not divisible by block_height %lld.",
                    (long long)d->rows, (long long)d->row_group);
    if (!is_float_dtype(d->x_dtype)) return fail(CTB_EINVAL_DTYPE, "dense side must be bf16, f16 or f32");
    if (!(is_float_dtype(d->scale_dtype) || d->scale_dtype == CTB_E4M3)) return fail(CTB_EINVAL_DTYPE, "unsupported scale dtype");
    if (d->qtype == CTB_QINT) {
        if (d->num_bits < 1 || d->num_bits > 8) return fail(CTB_EUNSUPPORTED, "int quantization supports 1..8 bits");
    } else if (d->qtype == CTB_QFLOAT) {
        if (d->num_bits != 8 && d->num_bits != 4) return fail(CTB_EUNSUPPORTED, "Only num_bits in (4, 8) are supported");
    } else {
        return fail(CTB_EINVAL_DTYPE, "Invalid quantization type %d", d->qtype);
    }
    if (d->codec == CTB_CODE_PACK32 && d->qtype != CTB_QINT) return fail(CTB_EINVAL_DTYPE, "PACK32 needs an int type");
    if (d->codec == CTB_CODE_FP4X2) {
        if (!(d->qtype == CTB_QFLOAT && d->num_bits == 4)) return fail(CTB_EINVAL_DTYPE, "FP4X2 needs the fp4 type");
        if (d->cols % 2) return fail(CTB_EINVAL_SHAPE, "tensor must have an even number of columns for nvfp4 compression");
    }
    if (d->codec == CTB_CODE_DTYPE && dtype_to_fmt(d->q_dtype) == F_NONE) return fail(CTB_EINVAL_DTYPE, "unsupported q_dtype");
    if (mode == 2 && !is_float_dtype(d->q_dtype)) return fail(CTB_EINVAL_DTYPE, "fake quantize writes a float dtype");
    return CTB_OK;
}

template <int MODE, int T, int TS, int QK, int FIN, int FOUT>
static int launch_vec8(const QArgs &a, cudaStream_t st) {
    // dequantize writes 2-8x what it reads: many more blocks than are resident (they sweep the output as one moving
    // window) measured faster than a persistent grid, as for the batched dequantize kernel
    int grid = grid_for(a.chunks, (int64_t)kThreads * kUnroll, MODE == 1 ? 256 : 8);
    qdq_vec8_kernel<MODE, T, TS, QK, FIN, FOUT><<<grid, kThreads, 0, st>>>(a);
    return after_launch("qdq_vec8_kernel");
}

// the combinations built for the vec8 tier; anything else runs on the generic tier
#define CTB_TRY(MODE, T_, TS_, QK_, FIN_, FOUT_)                                                        \
    if (mode == MODE && (MODE == 1 || a.T == T_) && (MODE == 0 || a.TS == TS_) && a.qk == QK_ &&        \
        a.fin == FIN_ && a.fout == FOUT_)                                                                \
        return launch_vec8<MODE, T_, TS_, QK_, FIN_, FOUT_>(a, st);

static int dispatch_vec8(int mode, const QArgs &a, cudaStream_t st, bool *handled) {
    *handled = true;
    constexpr int B = CTB_BF16, H = CTB_F16, S = CTB_F32;
    // quantize
    CTB_TRY(0, B, S, QK_INT, F_BF16, F_PACK4) CTB_TRY(0, B, S, QK_INT, F_BF16, F_PACK8)
    CTB_TRY(0, B, S, QK_INT, F_BF16, F_I8) CTB_TRY(0, B, S, QK_INT, F_BF16, F_BF16)
    CTB_TRY(0, S, S, QK_INT, F_BF16, F_PACK4) CTB_TRY(0, S, S, QK_INT, F_BF16, F_I8)
    CTB_TRY(0, S, S, QK_INT, F_F32, F_PACK4) CTB_TRY(0, S, S, QK_INT, F_F32, F_I8) CTB_TRY(0, S, S, QK_INT, F_F32, F_F32)
    CTB_TRY(0, H, S, QK_INT, F_F16, F_PACK4) CTB_TRY(0, H, S, QK_INT, F_F16, F_I8)
    CTB_TRY(0, B, S, QK_FP8, F_BF16, F_E4M3) CTB_TRY(0, B, S, QK_FP8, F_BF16, F_BF16)
    CTB_TRY(0, S, S, QK_FP8, F_BF16, F_E4M3) CTB_TRY(0, S, S, QK_FP8, F_F32, F_E4M3)
    CTB_TRY(0, H, S, QK_FP8, F_F16, F_E4M3)
    CTB_TRY(0, S, S, QK_FP4, F_BF16, F_FP4X2) CTB_TRY(0, S, S, QK_FP4, F_BF16, F_BF16)
    // dequantize
    CTB_TRY(1, S, B, QK_INT, F_PACK4, F_BF16) CTB_TRY(1, S, B, QK_INT, F_PACK8, F_BF16)
    CTB_TRY(1, S, B, QK_INT, F_I8, F_BF16) CTB_TRY(1, S, B, QK_FP8, F_E4M3, F_BF16)
    CTB_TRY(1, S, S, QK_INT, F_PACK4, F_F32) CTB_TRY(1, S, S, QK_INT, F_I8, F_F32)
    CTB_TRY(1, S, S, QK_FP8, F_E4M3, F_F32) CTB_TRY(1, S, S, QK_FP8, F_E4M3, F_BF16)
    CTB_TRY(1, S, H, QK_INT, F_PACK4, F_F16) CTB_TRY(1, S, H, QK_FP8, F_E4M3, F_F16)
    CTB_TRY(1, S, S, QK_FP4, F_FP4X2, F_BF16) CTB_TRY(1, S, S, QK_FP4, F_BF16, F_BF16)
    // fake quantize
    CTB_TRY(2, B, B, QK_INT, F_BF16, F_BF16) CTB_TRY(2, B, B, QK_FP8, F_BF16, F_BF16)
    CTB_TRY(2, S, S, QK_FP4, F_BF16, F_BF16) CTB_TRY(2, S, S, QK_FP8, F_BF16, F_F32)
    CTB_TRY(2, S, S, QK_INT, F_F32, F_F32)
    *handled = false;
    return CTB_OK;
}

template <int MODE, int QK, int FOUT>
static int launch_lean(const LeanArgs &l, int sdt, cudaStream_t st) {
    const int grid = grid_for(l.chunks, (int64_t)kThreads * kLeanUnroll, sdt == CTB_BF16 ? 16 : 12);
    if (sdt == CTB_BF16) quant_bf16_lean_kernel<MODE, QK, FOUT, CTB_BF16><<<grid, kThreads, 0, st>>>(l);
    else quant_bf16_lean_kernel<MODE, QK, FOUT, CTB_F32><<<grid, kThreads, 0, st>>>(l);
    return after_launch("quant_bf16_lean_kernel");
}

// bf16 tensor with a bf16 or fp32 scale: quantize to packed int4 / int8 / e4m3 codes, or fake-quantize back to bf16
static int dispatch_lean(int mode, const QArgs &a, cudaStream_t st, bool *handled) {
    *handled = false;
    if (a.xdt != CTB_BF16 || !(a.sdt == CTB_BF16 || a.sdt == CTB_F32) || a.gs || a.chunks >= (1LL << 31) || a.srs >= (1LL << 31)) return CTB_OK;
    if (!(mode == 0 || (mode == 2 && a.fout == F_BF16)) || a.qk == QK_FP4) return CTB_OK;
    LeanArgs l{};
    l.in = (const uint4 *)a.in; l.scale = a.scale; l.zp = a.zp; l.out = a.out;
    l.chunks = (uint32_t)a.chunks; l.cpr = (uint32_t)a.cpr; l.srs = (uint32_t)a.srs;
    l.shift = a.gshift >= 3 ? a.gshift - 3 : -1;
    l.by_cpr = make_fastdiv((uint32_t)a.cpr);
    l.by_row_group = make_fastdiv((uint32_t)a.row_group);
    l.by_col_chunks = make_fastdiv((uint32_t)(a.col_group / 8));
    l.qmin = a.qmin; l.qmax = a.qmax; l.zdt = a.zdt;
    *handled = true;
    if (mode == 0 && a.qk == QK_INT && a.fout == F_PACK4) return launch_lean<0, QK_INT, F_PACK4>(l, a.sdt, st);
    if (mode == 0 && a.qk == QK_INT && a.fout == F_PACK8) return launch_lean<0, QK_INT, F_PACK8>(l, a.sdt, st);
    if (mode == 0 && a.qk == QK_INT && a.fout == F_I8) return launch_lean<0, QK_INT, F_I8>(l, a.sdt, st);
    if (mode == 0 && a.qk == QK_FP8 && a.fout == F_E4M3) return launch_lean<0, QK_FP8, F_E4M3>(l, a.sdt, st);
    if (mode == 2 && a.qk == QK_INT) return launch_lean<2, QK_INT, F_BF16>(l, a.sdt, st);
    if (mode == 2 && a.qk == QK_FP8) return launch_lean<2, QK_FP8, F_BF16>(l, a.sdt, st);
    *handled = false;
    return CTB_OK;
}

#define CTB_TRY_GIDX(MODE, T_, TS_, QK_, FIN_, FOUT_)                                                   \
    if (mode == MODE && (MODE == 1 || a.T == T_) && (MODE == 0 || a.TS == TS_) && a.qk == QK_ &&        \
        a.fin == FIN_ && a.fout == FOUT_) {                                                              \
        qdq_vec8_gidx_kernel<MODE, T_, TS_, QK_, FIN_, FOUT_><<<grid_for(a.chunks, kThreads, 8), kThreads, 0, st>>>(a); \
        return after_launch("qdq_vec8_gidx_kernel");                                                     \
    }

// group-strategy int codes of a 16-bit tensor with a column -> group map; anything else runs on the generic tier
static int dispatch_gidx(int mode, const QArgs &a, cudaStream_t st, bool *handled) {
    *handled = true;
    if (a.xdt == CTB_BF16 && a.sdt == CTB_BF16 && !a.gs && a.qk == QK_INT && a.srs <= 4096 && a.rows < (1LL << 31)) {
        const size_t smem = (size_t)a.srs * sizeof(GidxSmem);
        const int grid = grid_for(a.rows, 1, 32);  // bound by the shared-memory lookups; 8 .. 64 per SM measured within 10 %
#define CTB_GIDX_ROW(MODE_, FC_)                                                 \
    {                                                                            \
        gidx_row_kernel<MODE_, FC_><<<grid, kGidxThreads, smem, st>>>(a);        \
        return after_launch("gidx_row_kernel");                                  \
    }
        if (mode == 0 && a.T == CTB_BF16 && a.fout == F_PACK4) CTB_GIDX_ROW(0, F_PACK4)
        if (mode == 0 && a.T == CTB_BF16 && a.fout == F_I8) CTB_GIDX_ROW(0, F_I8)
        if (mode == 1 && a.TS == CTB_BF16 && a.fin == F_PACK4 && a.fout == F_BF16) CTB_GIDX_ROW(1, F_PACK4)
        if (mode == 1 && a.TS == CTB_BF16 && a.fin == F_I8 && a.fout == F_BF16) CTB_GIDX_ROW(1, F_I8)
        if (mode == 2 && a.T == CTB_BF16 && a.TS == CTB_BF16 && a.fout == F_BF16) CTB_GIDX_ROW(2, F_BF16)
#undef CTB_GIDX_ROW
    }
    constexpr int B = CTB_BF16, H = CTB_F16, S = CTB_F32;
    CTB_TRY_GIDX(0, B, S, QK_INT, F_BF16, F_PACK4) CTB_TRY_GIDX(0, B, S, QK_INT, F_BF16, F_I8)
    CTB_TRY_GIDX(0, H, S, QK_INT, F_F16, F_PACK4) CTB_TRY_GIDX(0, H, S, QK_INT, F_F16, F_I8)
    CTB_TRY_GIDX(1, S, B, QK_INT, F_PACK4, F_BF16) CTB_TRY_GIDX(1, S, B, QK_INT, F_I8, F_BF16)
    CTB_TRY_GIDX(1, S, H, QK_INT, F_PACK4, F_F16) CTB_TRY_GIDX(1, S, H, QK_INT, F_I8, F_F16)
    CTB_TRY_GIDX(2, B, B, QK_INT, F_BF16, F_BF16) CTB_TRY_GIDX(2, H, H, QK_INT, F_F16, F_F16)
    *handled = false;
    return CTB_OK;
}

static int run(int mode, const ctb_qdesc *d, const void *in, const void *scale, const void *zp,
               const int32_t *g_idx, const float *gs, void *out, void *stream) {
    int rc = validate(d, in, scale, out, mode);
    if (rc) return rc;
    if (d->rows == 0 || d->cols == 0) return CTB_OK;
    QArgs a{};
    a.in = in; a.scale = scale; a.zp = zp; a.g_idx = g_idx; a.gs = gs; a.out = out;
    a.rows = d->rows; a.cols = d->cols; a.col_group = d->col_group; a.row_group = d->row_group;
    a.srs = d->scale_row_stride;
    a.sdt = d->scale_dtype; a.zdt = d->zp_dtype; a.xdt = d->x_dtype; a.bits = d->num_bits;
    a.qk = d->qtype == CTB_QINT ? QK_INT : (d->num_bits == 8 ? QK_FP8 : QK_FP4);
    if (a.qk == QK_INT) { a.qmax = (float)(1 << d->num_bits) / 2 - 1; a.qmin = -(float)(1 << d->num_bits) / 2; }
    else if (a.qk == QK_FP8) { a.qmax = 448.0f; a.qmin = -448.0f; }
    else { a.qmax = 6.0f; a.qmin = -6.0f; }
    int sdt_eff = gs ? CTB_F32 : d->scale_dtype;      // scale.to(global_scale.dtype) / global_scale
    if (sdt_eff == CTB_E4M3) return fail(CTB_EINVAL_DTYPE, "an e4m3 scale needs a global_scale");
    a.T = promote(d->x_dtype, sdt_eff);
    a.TS = sdt_eff;
    int dense = dtype_to_fmt(d->x_dtype), code = code_fmt(d);
    if (mode == 0) { a.fin = dense; a.fout = code; }
    else if (mode == 1) { a.fin = code; a.fout = dense; }
    else { a.fin = dense; a.fout = dtype_to_fmt(d->q_dtype); }
    cudaStream_t st = as_stream(stream);

    bool pack_other = d->codec == CTB_CODE_PACK32 && d->num_bits != 4 && d->num_bits != 8;
    bool vec_ok = !g_idx && !pack_other && d->cols % 8 == 0 && d->col_group % 8 == 0 && aligned16(in) && aligned16(out);
    if (vec_ok) {
        a.chunks = d->rows * d->cols / 8;
        a.cpr = d->cols / 8;
        a.gshift = -1;
        a.idx32 = a.chunks < (1LL << 31);
        if (a.idx32) {
            a.by_cpr = make_fastdiv((uint32_t)a.cpr);
            a.by_row_group = make_fastdiv((uint32_t)d->row_group);
            a.by_col_chunks = make_fastdiv((uint32_t)(d->col_group / 8));
        }
        bool flat = d->row_group == 1 && (d->scale_row_stride == d->cols / d->col_group);
        if (flat && (d->col_group & (d->col_group - 1)) == 0) {
            int sh = 0;
            while ((1LL << sh) < d->col_group) ++sh;
            a.gshift = sh;
        }
        if (mode == 1 && a.qk == QK_FP4 && a.fin == F_FP4X2 && a.fout == F_BF16 && d->scale_dtype == CTB_E4M3 && gs && !zp && flat &&
            d->col_group == 16) {
            dequant_fp4_g16_bf16_kernel<<<grid_for(a.chunks, (int64_t)kThreads * 8, 32), kThreads, 0, st>>>(in, (const uint8_t *)scale, gs, a.chunks, out);
            return after_launch("dequant_fp4_g16_bf16_kernel");
        }
        if (mode == 0 && a.qk == QK_FP4 && a.fin == F_BF16 && a.fout == F_FP4X2 && d->scale_dtype == CTB_E4M3 && gs && flat &&
            d->col_group == 16 && a.idx32 && (!zp || dtype_size(d->zp_dtype) != 0)) {
            // NVFP4 with given scales: the whole-shard kernel on a table of one (a lane per group of 16, the effective
            // scale divided once per group)
            return quant_fp4_g16_one(in, scale, gs, zp, d->zp_dtype, d->rows, d->cols, out, st);
        }
        bool handled = false;
        rc = dispatch_lean(mode, a, st, &handled);
        if (handled) return rc;
        rc = dispatch_vec8(mode, a, st, &handled);
        if (handled) return rc;
    }
    if (g_idx && !pack_other && d->row_group == 1 && d->cols % 8 == 0 && aligned16(in) && aligned16(out) && aligned16(g_idx) &&
        d->rows * d->cols / 8 < (1LL << 31)) {
        a.chunks = d->rows * d->cols / 8;
        a.cpr = d->cols / 8;
        a.by_cpr = make_fastdiv((uint32_t)a.cpr);
        bool handled = false;
        rc = dispatch_gidx(mode, a, st, &handled);
        if (handled) return rc;
    }
    int per = (mode == 0 && d->codec == CTB_CODE_PACK32) ? 32 / d->num_bits : ((mode == 0 && d->codec == CTB_CODE_FP4X2) ? 2 : 1);
    int64_t units = d->rows * cdiv(d->cols, per);
    int grid = grid_for(units, kThreads, 8);
    if (mode == 0) qdq_generic_kernel<0><<<grid, kThreads, 0, st>>>(a);
    else if (mode == 1) qdq_generic_kernel<1><<<grid, kThreads, 0, st>>>(a);
    else qdq_generic_kernel<2><<<grid, kThreads, 0, st>>>(a);
    return after_launch("qdq_generic_kernel");
}

}  // namespace ctb

extern "C" int ctb_quantize(const ctb_qdesc *desc, const void *x, const void *scale, const void *zero_point,
                            const int32_t *g_idx, const float *global_scale, void *out, void *stream) {
    return ctb::run(0, desc, x, scale, zero_point, g_idx, global_scale, out, stream);
}
extern "C" int ctb_dequantize(const ctb_qdesc *desc, const void *q, const void *scale, const void *zero_point,
                              const int32_t *g_idx, const float *global_scale, void *out, void *stream) {
    return ctb::run(1, desc, q, scale, zero_point, g_idx, global_scale, out, stream);
}
extern "C" int ctb_fake_quantize(const ctb_qdesc *desc, const void *x, const void *scale, const void *zero_point,
                                 const int32_t *g_idx, const float *global_scale, void *out, void *stream) {
    return ctb::run(2, desc, x, scale, zero_point, g_idx, global_scale, out, stream);
}

// ------------------------------------------------------------------ whole-shard unpack + dequantize (int4, group 128, bf16)

namespace ctb {

constexpr int kDQBatchMax = 256;

struct DQBatch {
    int count;
    int64_t ustart[kDQBatchMax + 1];  // first global unit of each tensor (unit = 1024 chunks = 8192 elements); ustart[count] = total
    int64_t nchunks[kDQBatchMax];     // chunks (8 elements) of each tensor
    const void *in[kDQBatchMax];      // packed words
    const void *scale[kDQBatchMax];   // bf16, one per 16 chunks
    void *out[kDQBatchMax];           // bf16
};

constexpr int kDQUnit = kThreads * kUnroll;  // chunks per block-iteration

// One launch for every tensor of the table.  The units of all tensors form one index space that the grid strides
// over; the tensor lookup happens once per unit (uniform across the block), addressing inside a unit is 32-bit,
// and the next unit's words and scales are loaded before the current unit is written.
__global__ void __launch_bounds__(kThreads) dequant_int4_batch_kernel(const __grid_constant__ DQBatch B) {
    const int64_t total = B.ustart[B.count];
    int t = 0;
    uint32_t word[kUnroll], sbits[kUnroll];
    bool ok[kUnroll];
    char *obase = nullptr;
    auto fetch = [&](int64_t unit) {
        while (t + 1 < B.count && unit >= B.ustart[t + 1]) ++t;
        const int64_t cbase = (unit - B.ustart[t]) * kDQUnit;
        const uint32_t left = (uint32_t)min((int64_t)kDQUnit, B.nchunks[t] - cbase);
        const char *ip = (const char *)B.in[t] + cbase * 4;
        const unsigned short *sp = (const unsigned short *)B.scale[t] + (cbase >> 4);
        obase = (char *)B.out[t] + cbase * 16;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t c = u * kThreads + threadIdx.x;
            ok[u] = c < left;
            if (ok[u]) {
                word[u] = ld_stream4(ip + c * 4);
                sbits[u] = __ldg(sp + (c >> 4));
            }
        }
    };
    int64_t unit = blockIdx.x;
    if (unit < total) fetch(unit);
    const __nv_bfloat162 bias = __float2bfloat162_rn(136.0f);
    while (unit < total) {
        uint32_t w[kUnroll], s[kUnroll];
        bool k[kUnroll];
        char *o = obase;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) { w[u] = word[u]; s[u] = sbits[u]; k[u] = ok[u]; }
        const int64_t next = unit + gridDim.x;
        if (next < total) fetch(next);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (k[u]) st_stream(o + (uint32_t)(u * kThreads + threadIdx.x) * 16, dequant_int4_word_bf16(w[u], u32_as_bf162(s[u] | (s[u] << 16)), bias));
        unit = next;
    }
}

}  // namespace ctb

namespace ctb {

// The mirror of the kernel above for the compress direction when the scales are GIVEN (a calibrated model:
// compressors/quantized_compressors/base.py:91-122 calling pack_quantized.py:88-145 once per weight): symmetric int4,
// group 128, bf16 weights and bf16 scales, every tensor of the table in one grid.  Same table type; `in` is the dense
// weight, `scale` is read, `out` receives the pack_to_int32 words.  The arithmetic is the packed-bf16x2 tier of
// quant_bf16_lean_kernel (and its float routine for a scale outside [2^-99, 2^99)), so the words equal ctb_quantize's.
__global__ void __launch_bounds__(kThreads) quant_int4_batch_kernel(const __grid_constant__ DQBatch B) {
    const int64_t total = B.ustart[B.count];
    int t = 0;
    uint4 raw[kUnroll];
    uint32_t sbits[kUnroll];
    bool ok[kUnroll];
    int64_t cbase = 0;
    auto fetch = [&](int64_t unit) {
        while (t + 1 < B.count && unit >= B.ustart[t + 1]) ++t;
        cbase = (unit - B.ustart[t]) * kDQUnit;
        const uint32_t left = (uint32_t)min((int64_t)kDQUnit, B.nchunks[t] - cbase);
        const char *ip = (const char *)B.in[t] + cbase * 16;
        const unsigned short *sp = (const unsigned short *)B.scale[t] + (cbase >> 4);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const uint32_t c = u * kThreads + threadIdx.x;
            ok[u] = c < left;
            if (ok[u]) {
                raw[u] = ld_stream(ip + (size_t)c * 16);
                sbits[u] = __ldg(sp + (c >> 4));
            }
        }
    };
    int64_t unit = blockIdx.x;
    if (unit < total) fetch(unit);
    while (unit < total) {
        uint4 w[kUnroll];
        uint32_t s[kUnroll];
        bool k[kUnroll];
        const int ct = t;
        const int64_t cb = cbase;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) { w[u] = raw[u]; s[u] = sbits[u]; k[u] = ok[u]; }
        const int64_t next = unit + gridDim.x;
        if (next < total) fetch(next);
        char *o = (char *)B.out[ct] + cb * 4;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (!k[u]) continue;
            const uint32_t c = u * kThreads + threadIdx.x;
            if (((s[u] >> 7) & 0xFFu) - 28u > 197u) {  // scale outside the range the reciprocal form is proved for
                LeanArgs l{};
                l.in = (const uint4 *)B.in[ct] + cb; l.scale = (const unsigned short *)B.scale[ct] + (cb >> 4); l.zp = nullptr;
                l.out = o; l.qmin = -8.0f; l.qmax = 7.0f; l.zdt = CTB_I8;
                lean_exact_chunk<0, QK_INT, F_PACK4, CTB_BF16>(l, c, c >> 4);
                continue;
            }
            const uint32_t x4[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
            st_stream4(o + (size_t)c * 4, quant_int4_word_bf16(x4, rcp_approx(__uint_as_float(s[u] << 16)), false, u32_as_bf162(0u)));
        }
        unit = next;
    }
}

}  // namespace ctb

extern "C" int ctb_quantize_pack_int4_batch(const ctb_tensor_ref *tensors, int32_t count, void *stream) {
    using namespace ctb;
    if (!tensors && count > 0) return fail(CTB_EINVAL_NULL, "null tensor table");
    static thread_local DQBatch B;
    for (int32_t base = 0; base < count; base += kDQBatchMax) {
        const int32_t n = count - base < kDQBatchMax ? count - base : kDQBatchMax;
        int64_t g = 0;
        for (int32_t i = 0; i < n; ++i) {
            const ctb_tensor_ref &t = tensors[base + i];
            if (!t.in || !t.out || !t.scale) return fail(CTB_EINVAL_NULL, "tensor %d has a null buffer", base + i);
            if (t.rows < 0 || t.cols <= 0 || t.cols % 128) return fail(CTB_EINVAL_SHAPE, "tensor %d: columns %lld are not a multiple of 128", base + i, (long long)t.cols);
            if (!aligned16(t.in) || (reinterpret_cast<uintptr_t>(t.out) & 3u) || (reinterpret_cast<uintptr_t>(t.scale) & 1u))
                return fail(CTB_EINVAL_ALIGN, "tensor %d is misaligned", base + i);
            B.ustart[i] = g;
            B.nchunks[i] = t.rows * t.cols / 8;
            B.in[i] = t.in;
            B.scale[i] = t.scale;
            B.out[i] = t.out;
            g += cdiv(B.nchunks[i], kDQUnit);
        }
        B.count = n;
        B.ustart[n] = g;
        if (g == 0) continue;
        int grid = grid_for(g, 1, 8);
        quant_int4_batch_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(B);
        int rc = after_launch("quant_int4_batch_kernel");
        if (rc) return rc;
    }
    return CTB_OK;
}

extern "C" int ctb_unpack_dequantize_int4_batch(const ctb_tensor_ref *tensors, int32_t count, void *stream) {
    using namespace ctb;
    if (!tensors && count > 0) return fail(CTB_EINVAL_NULL, "null tensor table");
    static thread_local DQBatch B;
    for (int32_t base = 0; base < count; base += kDQBatchMax) {
        const int32_t n = count - base < kDQBatchMax ? count - base : kDQBatchMax;
        int64_t g = 0;
        for (int32_t i = 0; i < n; ++i) {
            const ctb_tensor_ref &t = tensors[base + i];
            if (!t.in || !t.out || !t.scale) return fail(CTB_EINVAL_NULL, "tensor %d has a null buffer", base + i);
            if (t.rows < 0 || t.cols <= 0 || t.cols % 128) return fail(CTB_EINVAL_SHAPE, "tensor %d: columns %lld are not a multiple of 128", base + i, (long long)t.cols);
            if (!aligned16(t.out) || (reinterpret_cast<uintptr_t>(t.in) & 3u)) return fail(CTB_EINVAL_ALIGN, "tensor %d is misaligned", base + i);
            B.ustart[i] = g;
            B.nchunks[i] = t.rows * t.cols / 8;
            B.in[i] = t.in;
            B.scale[i] = t.scale;
            B.out[i] = t.out;
            g += cdiv(B.nchunks[i], kDQUnit);
        }
        B.count = n;
        B.ustart[n] = g;
        if (g == 0) continue;
        // many more blocks than fit at once (a handful of units each): the resident ones then sweep the output as one
        // moving window, which measured 6 % faster on this write-heavy kernel than one persistent block per slot
        int grid = grid_for(g, 1, 256);
        dequant_int4_batch_kernel<<<grid, kThreads, 0, as_stream(stream)>>>(B);
        int rc = after_launch("dequant_int4_batch_kernel");
        if (rc) return rc;
    }
    return CTB_OK;
}
