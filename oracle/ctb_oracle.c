/*
 * CPU oracle for the tensor-codec path of compressed-tensors.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of what the
 * reference's torch-CPU code computes, written so that every intermediate
 * rounding the reference performs (bf16 / fp16 / fp32 / e4m3) is explicit.  It
 * is the checker for the CUDA kernels and the timed CPU baseline; nothing in
 * the shipped package calls it.
 *
 * Each function cites the reference file:line it follows (paths are relative
 * to the reference project root, src/compressed_tensors/...).
 *
 * The arithmetic itself lives in a third-party dependency of the reference,
 * PyTorch (CPU eager kernels) and numpy.packbits; the facts restated here are
 *   - bf16/fp16 binary ops compute in fp32 and round the result to nearest-even,
 *   - Tensor.to(float8_e4m3fn) is round-to-nearest-even with NaN above 464,
 *   - torch.round is round-half-to-even,
 *   - numpy.packbits(bitorder="little") puts column 8k+j in bit j of byte k.
 * Parity is pinned by golden vectors generated from the reference itself
 * (tests/golden/).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* dtype codes (same numbering as the product header, restated independently) */
enum {
    ORC_BF16 = 0,
    ORC_F16 = 1,
    ORC_F32 = 2,
    ORC_F64 = 3,
    ORC_I8 = 4,
    ORC_E4M3 = 5,
    ORC_U8 = 6,
    ORC_I32 = 7,
    ORC_I64 = 8,
};

enum { ORC_QINT = 0, ORC_QFLOAT = 1 };

/* ------------------------------------------------------------------ scalars */

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* round-to-nearest-even fp32 -> bf16; NaN becomes the canonical quiet NaN */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if (isnan(f)) return 0x7FC0;
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) { _Float16 x; memcpy(&x, &h, 2); return (float)x; }
static inline uint16_t f32_to_f16(float f) { _Float16 x = (_Float16)f; uint16_t h; memcpy(&h, &x, 2); return h; }

/* value of an e4m3fn byte (1-4-3, bias 7, no inf, 0x7f/0xff = NaN) */
static inline float e4m3_to_f32(uint8_t b) {
    int s = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0xF && m == 7) v = NAN;
    else if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf((float)(8 + m), e - 10);
    return s ? -v : v;
}

/* fp32 -> e4m3fn, round-to-nearest-even.  Matches Tensor.to(float8_e4m3fn):
 * magnitudes that round above 448 (i.e. >= 464) and inf/NaN give NaN (0x7f | sign). */
static inline uint8_t f32_to_e4m3(float f) {
    uint8_t sign = (f32_bits(f) >> 31) ? 0x80 : 0;
    float a = fabsf(f);
    if (!(a < INFINITY)) return sign | 0x7F; /* inf or NaN */
    if (a == 0.0f) return sign;
    int e;
    (void)frexpf(a, &e); /* a = m * 2^e, m in [0.5,1)  => floor(log2 a) = e-1 */
    int lg = e - 1;
    if (lg < -6) lg = -6;             /* subnormal range shares the 2^-9 grid */
    float step = ldexpf(1.0f, lg - 3); /* spacing of representable values here */
    float q = rintf(a / step) * step;  /* exact: power-of-two scaling, ties-to-even */
    if (q > 448.0f) return sign | 0x7F;
    if (q == 0.0f) return sign;
    (void)frexpf(q, &e);
    lg = e - 1;
    if (lg < -6) { /* subnormal */
        int m = (int)(q / ldexpf(1.0f, -9));
        return sign | (uint8_t)m;
    }
    int m = (int)(q / ldexpf(1.0f, lg - 3)) - 8;
    return sign | (uint8_t)(((lg + 7) << 3) | m);
}

/* round a float to the nearest value of a storage dtype and come back as float */
static inline float round_to(int dt, float v) {
    switch (dt) {
    case ORC_BF16: return bf16_to_f32(f32_to_bf16(v));
    case ORC_F16: return f16_to_f32(f32_to_f16(v));
    default: return v;
    }
}

static inline float load_as_f32(const void *p, int dt, int64_t i) {
    switch (dt) {
    case ORC_BF16: return bf16_to_f32(((const uint16_t *)p)[i]);
    case ORC_F16: return f16_to_f32(((const uint16_t *)p)[i]);
    case ORC_F32: return ((const float *)p)[i];
    case ORC_F64: return (float)((const double *)p)[i];
    case ORC_I8: return (float)((const int8_t *)p)[i];
    case ORC_U8: return (float)((const uint8_t *)p)[i];
    case ORC_E4M3: return e4m3_to_f32(((const uint8_t *)p)[i]);
    case ORC_I32: return (float)((const int32_t *)p)[i];
    default: return NAN;
    }
}

static inline void store_from_f32(void *p, int dt, int64_t i, float v) {
    switch (dt) {
    case ORC_BF16: ((uint16_t *)p)[i] = f32_to_bf16(v); break;
    case ORC_F16: ((uint16_t *)p)[i] = f32_to_f16(v); break;
    case ORC_F32: ((float *)p)[i] = v; break;
    case ORC_F64: ((double *)p)[i] = (double)v; break;
    case ORC_I8: ((int8_t *)p)[i] = (int8_t)v; break;
    case ORC_E4M3: ((uint8_t *)p)[i] = f32_to_e4m3(v); break;
    default: break;
    }
}

/* torch type promotion between two floating tensors of dim > 0 */
static inline int promote(int a, int b) {
    if (a == b) return a;
    if (a == ORC_F64 || b == ORC_F64) return ORC_F64;
    return ORC_F32; /* bf16+f16, x+f32 */
}

/* quantization/quant_args.py:55-68  FP4_E2M1_DATA.cast_to_fp4
 * thresholds with ties going to the code with an even mantissa; the result is
 * |x| snapped to the grid times sign(x), where sign(+-0) = 0 so an exact zero
 * input comes out as +0 while a small negative comes out as -0. */
static inline float cast_to_fp4(float x) {
    if (isnan(x)) return x;
    float sign = (x > 0.0f) ? 1.0f : ((x < 0.0f) ? -1.0f : 0.0f);
    float a = fabsf(x), r;
    if (a <= 0.25f) r = 0.0f;
    else if (a < 0.75f) r = 0.5f;
    else if (a <= 1.25f) r = 1.0f;
    else if (a < 1.75f) r = 1.5f;
    else if (a <= 2.5f) r = 2.0f;
    else if (a < 3.5f) r = 3.0f;
    else if (a <= 5.0f) r = 4.0f;
    else r = 6.0f;
    return r * sign;
}

/* quantization/utils/helpers.py:208-234  calculate_range */
static inline void qrange(int qtype, int bits, float *qmin, float *qmax) {
    if (qtype == ORC_QINT) {
        float r = (float)(1 << bits);
        *qmax = r / 2 - 1;
        *qmin = -r / 2;
    } else if (bits == 8) {
        *qmax = 448.0f; *qmin = -448.0f;
    } else {
        *qmax = 6.0f; *qmin = -6.0f;
    }
}

/* torch.clamp propagates NaN */
static inline float clampf(float v, float lo, float hi) {
    if (isnan(v)) return v;
    return v < lo ? lo : (v > hi ? hi : v);
}

/* --------------------------------------------------- quantize / dequantize */

typedef struct {
    int64_t rows, cols;     /* x viewed as [rows, cols] (leading dims flattened) */
    int64_t col_group;      /* columns sharing one scale (group size; cols for channel/token/tensor) */
    int64_t row_group;      /* rows sharing one scale (1 except BLOCK) */
    int64_t scale_row_stride; /* scale index = (r/row_group)*scale_row_stride + c/col_group */
    int32_t qtype, bits;
    int32_t x_dtype, scale_dtype, zp_dtype, out_dtype;
} orc_desc;

static inline int64_t qp_index(const orc_desc *d, const int32_t *g_idx, int64_t r, int64_t c) {
    int64_t g = g_idx ? (int64_t)g_idx[c] : c / d->col_group;
    return (r / d->row_group) * d->scale_row_stride + g;
}

/* quantization/lifecycle/forward.py:455-487 _quantize, quant_args.py:384-408
 * round_to_quantized_type.  Returns the quantized value as a float that is
 * exactly representable in the compute dtype T = promote(x, scale'). */
static inline float quant_core(float x, float s, int T, int has_zp, float zp,
                               int qtype, int bits, float qmin, float qmax) {
    float v = round_to(T, x / s);
    if (has_zp) v = round_to(T, v + zp);
    v = clampf(v, qmin, qmax);
    if (qtype == ORC_QINT) v = rintf(v);
    else if (bits == 8) v = e4m3_to_f32(f32_to_e4m3(v));
    else v = cast_to_fp4(v);
    return v;
}

/* forward.py:491-514 _dequantize */
static inline float dequant_core(float q, float s, int Ts, int has_zp, float zp) {
    float v = round_to(Ts, q);
    if (has_zp) v = round_to(Ts, v - round_to(Ts, zp));
    return round_to(Ts, v * s);
}

/* effective scale: forward.py:468-469 / :501-502 */
static inline float eff_scale(const orc_desc *d, const void *scale, const float *gs, int64_t i) {
    float s = load_as_f32(scale, d->scale_dtype, i);
    if (gs) s = s / gs[0];
    return s;
}

/* mode 0: quantize; out dtype from desc (float dtypes, I8 or E4M3)
 * mode 1: dequantize (x holds codes in x_dtype: I8 / E4M3 / float)
 * mode 2: fake quantize (quantize then dequantize, forward.py:157-189)      */
int orc_qdq(const orc_desc *d, int mode, const void *x, const void *scale, const void *zp,
            const int32_t *g_idx, const float *gs, void *out) {
    float qmin, qmax;
    qrange(d->qtype, d->bits, &qmin, &qmax);
    int sdt = gs ? ORC_F32 : d->scale_dtype;
    int T = promote(d->x_dtype, sdt);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < d->rows; ++r) {
        for (int64_t c = 0; c < d->cols; ++c) {
            int64_t i = r * d->cols + c, qi = qp_index(d, g_idx, r, c);
            float s = eff_scale(d, scale, gs, qi);
            float z = zp ? load_as_f32(zp, d->zp_dtype, qi) : 0.0f;
            float xv = load_as_f32(x, d->x_dtype, i), v;
            if (mode == 1) {
                v = dequant_core(xv, s, sdt, zp != NULL, z);
            } else {
                /* zero_point.to(x.dtype), forward.py:474 */
                v = quant_core(xv, s, T, zp != NULL, round_to(d->x_dtype, z), d->qtype, d->bits, qmin, qmax);
                if (mode == 2) v = dequant_core(v, s, sdt, zp != NULL, z);
            }
            store_from_f32(out, d->out_dtype, i, v);
        }
    }
    return 0;
}

/* ---------------------------------------------------------------- qparams */

/* amin / amax over [row_group x col_group] tiles (helpers.py:168-203); outputs in x dtype */
int orc_minmax(const void *x, int xdt, int64_t rows, int64_t cols, int64_t row_group,
               int64_t col_group, void *out_min, void *out_max) {
    int64_t gr = rows / row_group, gc = cols / col_group;
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t a = 0; a < gr; ++a)
        for (int64_t b = 0; b < gc; ++b) {
            float mn = INFINITY, mx = -INFINITY;
            for (int64_t r = a * row_group; r < (a + 1) * row_group; ++r)
                for (int64_t c = b * col_group; c < (b + 1) * col_group; ++c) {
                    float v = load_as_f32(x, xdt, r * cols + c);
                    mn = v < mn ? v : mn;
                    mx = v > mx ? v : mx;
                }
            store_from_f32(out_min, xdt, a * gc + b, mn);
            store_from_f32(out_max, xdt, a * gc + b, mx);
        }
    return 0;
}

/* quantization/utils/helpers.py:67-146 calculate_qparams.
 * M = dtype of min/max.  Scale comes out in M (or e4m3 for fp4 with a global
 * scale); zero point in zp_dtype (int8 for int, e4m3 for float types). */
int orc_calculate_qparams(const void *mins, const void *maxs, int M, int64_t n, int qtype, int bits,
                          int symmetric, const float *gs, void *out_scale, void *out_zp, int zp_dtype) {
    float qmin, qmax;
    qrange(qtype, bits, &qmin, &qmax);
    float bit_range = qmax - qmin;
    const float eps = 1.1920928955078125e-07f; /* torch.finfo(float32).eps */
    int fp4 = (qtype == ORC_QFLOAT && bits == 4);
    if (!symmetric && fp4) return -1; /* helpers.py:126-129 */
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float mn = load_as_f32(mins, M, i), mx = load_as_f32(maxs, M, i);
        mn = mn < 0.0f ? mn : 0.0f; /* :87-88 zero must be representable */
        mx = mx > 0.0f ? mx : 0.0f;
        float zpv = 0.0f;
        if (symmetric) {
            float mvp = fmaxf(fabsf(mn), fabsf(mx));
            if (fp4 && gs) {
                /* :103-106: fp32 global scale times the M-rounded amax/6, saturate, cast e4m3 */
                float sc = gs[0] * round_to(M, mvp / 6.0f);
                sc = clampf(sc, -448.0f, 448.0f);
                uint8_t b = f32_to_e4m3(sc);
                if ((b & 0x7F) == 0) b = 0x20; /* :114-120 zero -> 0.125 */
                ((uint8_t *)out_scale)[i] = b;
            } else {
                float sc = round_to(M, mvp / (bit_range / 2.0f)); /* :110 */
                sc = sc < eps ? eps : sc;                          /* :122 */
                store_from_f32(out_scale, M, i, sc);
            }
        } else {
            float sc = round_to(M, round_to(M, mx - mn) / bit_range); /* :131 */
            sc = sc < eps ? eps : sc;
            sc = round_to(M, sc);
            zpv = round_to(M, qmin - round_to(M, mn / sc)); /* :133 */
            zpv = clampf(zpv, qmin, qmax);
            store_from_f32(out_scale, M, i, sc);
        }
        if (qtype == ORC_QINT) zpv = rintf(zpv); /* :138-139 */
        store_from_f32(out_zp, zp_dtype, i, zpv);
    }
    return 0;
}

/* helpers.py:414-434 generate_gparam: `448 * 6 / amax` with a Python scalar on the left, which torch evaluates as
 * amax.reciprocal() * 2688 (Tensor.__rtruediv__): two roundings in the min/max dtype, then fp32 */
float orc_generate_gparam(const void *mn_p, const void *mx_p, int M) {
    float mn = load_as_f32(mn_p, M, 0), mx = load_as_f32(mx_p, M, 0);
    mn = mn < 0.0f ? mn : 0.0f;
    mx = mx > 0.0f ? mx : 0.0f;
    float mvp = fmaxf(fabsf(mn), fabsf(mx));
    return round_to(M, round_to(M, 1.0f / mvp) * 2688.0f);
}

/* ------------------------------------------------------------ int32 packing */

/* compressors/quantized_compressors/pack_quantized.py:186-246 pack_to_int32, packed_dim=1.
 * value int8 [rows, cols] -> int32 [rows, ceil(cols/pf)], pf = 32/bits; element i of a run
 * sits in bits [bits*i, bits*i+bits) after adding 2^(bits-1); pad fields are zero. */
int orc_pack_int32(const int8_t *q, int64_t rows, int64_t cols, int bits, int32_t *out) {
    int pf = 32 / bits;
    int64_t pc = (cols + pf - 1) / pf;
    int offset = 1 << (bits - 1);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t w = 0; w < pc; ++w) {
            uint32_t word = 0; /* the reference sums int32 fields; fields never overlap when value < 2^bits */
            int32_t acc = 0;
            for (int k = 0; k < pf; ++k) {
                int64_t c = w * pf + k;
                if (c >= cols) break;
                uint8_t u = (uint8_t)(q[r * cols + c] + offset); /* :220 (value+offset).to(uint8) */
                acc = (int32_t)((uint32_t)acc + ((uint32_t)u << (bits * k))); /* :241-242 shift then int32 sum */
            }
            word = (uint32_t)acc;
            out[r * pc + w] = (int32_t)word;
        }
    return 0;
}

/* pack_quantized.py:249-309 unpack_from_int32, packed_dim=1 */
int orc_unpack_int32(const int32_t *w, int64_t rows, int64_t cols, int bits, int8_t *out) {
    int pf = 32 / bits;
    int64_t pc = (cols + pf - 1) / pf;
    int32_t mask = (1 << bits) - 1, offset = (1 << bits) / 2;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) {
            int32_t word = w[r * pc + c / pf];
            int32_t u = (word >> (bits * (c % pf))) & mask; /* arithmetic shift then mask */
            out[r * cols + c] = (int8_t)(u - offset);
        }
    return 0;
}

/* ---------------------------------------------------------------- fp4 pack */

static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* compressors/quantized_compressors/fp4_quantized.py:135-178 pack_fp4_to_uint8:
 * index of the nearest grid magnitude (first minimum wins, as torch.argmin), sign bit from
 * signbit(x), even column in the low nibble. */
int orc_pack_fp4(const void *x, int xdt, int64_t m, int64_t n, uint8_t *out) {
    if (n % 2) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m * n / 2; ++i) {
        uint8_t nib[2];
        for (int h = 0; h < 2; ++h) {
            float v = load_as_f32(x, xdt, 2 * i + h);
            float a = fabsf(v);
            int best = 0;
            float bd = round_to(xdt, fabsf(round_to(xdt, a - kE2M1[0])));
            for (int k = 1; k < 8; ++k) {
                float dk = round_to(xdt, fabsf(round_to(xdt, a - kE2M1[k])));
                if (dk < bd) { bd = dk; best = k; }
            }
            nib[h] = (uint8_t)(best | ((f32_bits(v) >> 31) << 3));
        }
        out[i] = nib[0] | (nib[1] << 4);
    }
    return 0;
}

/* fp4_quantized.py:187-221 unpack_fp4_from_uint8 */
int orc_unpack_fp4(const uint8_t *a, int64_t m, int64_t n, void *out, int odt) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m * n / 2; ++i) {
        uint8_t b = a[i];
        for (int h = 0; h < 2; ++h) {
            uint8_t nb = h ? (b >> 4) : (b & 0xF);
            float v = kE2M1[nb & 7] * ((nb & 8) ? -1.0f : 1.0f);
            store_from_f32(out, odt, 2 * i + h, v);
        }
    }
    return 0;
}

/* ------------------------------------------------------------ bitmask codec */

static inline int elem_nonzero(const void *x, int esize, int is_float_dt, int dt, int64_t i) {
    /* `tensor != 0` (sparse_bitmask.py:137): -0.0 compares equal to zero, NaN does not */
    if (is_float_dt) {
        float v = load_as_f32(x, dt, i);
        return !(v == 0.0f);
    }
    (void)esize;
    return ((const int8_t *)x)[i] != 0;
}

/* utils/helpers.py:302-313 pack_bitmasks: numpy.packbits(axis=-1, bitorder="little") */
int orc_pack_bitmasks(const uint8_t *bytemask, int64_t rows, int64_t cols, uint8_t *out) {
    int64_t pc = (cols + 7) / 8;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t k = 0; k < pc; ++k) {
            uint8_t b = 0;
            for (int j = 0; j < 8; ++j) {
                int64_t c = 8 * k + j;
                if (c < cols && bytemask[r * cols + c]) b |= (uint8_t)(1u << j);
            }
            out[r * pc + k] = b;
        }
    return 0;
}

/* utils/helpers.py:316-339 unpack_bitmasks */
int orc_unpack_bitmasks(const uint8_t *packed, int64_t rows, int64_t cols, uint8_t *out) {
    int64_t pc = (cols + 7) / 8;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) out[r * cols + c] = (packed[r * pc + c / 8] >> (c % 8)) & 1;
    return 0;
}

static size_t dt_size(int dt) {
    switch (dt) {
    case ORC_BF16: case ORC_F16: return 2;
    case ORC_F32: case ORC_I32: return 4;
    case ORC_F64: case ORC_I64: return 8;
    default: return 1;
    }
}

/* compressors/sparse_compressors/sparse_bitmask.py:131-149 bitmask_compress.
 * values: row-major nonzeros; row_offsets: exclusive prefix of per-row counts (int64).
 * e4m3 tensors are compared as floats (`tensor != 0` on the fp8 tensor) and moved as bytes.
 * Returns nnz. */
int64_t orc_bitmask_compress(const void *x, int dt, int64_t rows, int64_t cols, void *values,
                             uint8_t *bitmask, int64_t *row_offsets) {
    size_t es = dt_size(dt);
    int64_t pc = (cols + 7) / 8, nnz = 0;
    memset(bitmask, 0, (size_t)(rows * pc));
    for (int64_t r = 0; r < rows; ++r) {
        row_offsets[r] = nnz;
        for (int64_t c = 0; c < cols; ++c) {
            int64_t i = r * cols + c;
            if (elem_nonzero(x, (int)es, 1, dt, i)) {
                memcpy((char *)values + (size_t)nnz * es, (const char *)x + (size_t)i * es, es);
                bitmask[r * pc + c / 8] |= (uint8_t)(1u << (c % 8));
                ++nnz;
            }
        }
    }
    return nnz;
}

/* sparse_bitmask.py:152-169 bitmask_decompress (row_offsets are not consulted);
 * also sparse_24_bitmask.py:206-224 */
int orc_bitmask_decompress(const void *values, const uint8_t *bitmask, int dt, int64_t rows,
                           int64_t cols, void *out) {
    size_t es = dt_size(dt);
    int64_t pc = (cols + 7) / 8, k = 0;
    memset(out, 0, (size_t)(rows * cols) * es);
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c)
            if ((bitmask[r * pc + c / 8] >> (c % 8)) & 1) {
                memcpy((char *)out + (size_t)(r * cols + c) * es, (const char *)values + (size_t)k * es, es);
                ++k;
            }
    return 0;
}

/* sparse_24_bitmask.py:162-203 sparse24_bitmask_compress given the 2:4 bytemask
 * (the mask itself comes from orc_sparse24_mask in sparse24_topk.cpp). */
int orc_sparse24_gather(const void *x, int dt, const uint8_t *bytemask, int64_t rows, int64_t cols,
                        void *values, uint8_t *bitmask) {
    size_t es = dt_size(dt);
    int64_t k = 0;
    for (int64_t i = 0; i < rows * cols; ++i)
        if (bytemask[i]) {
            memcpy((char *)values + (size_t)k * es, (const char *)x + (size_t)i * es, es);
            ++k;
        }
    orc_pack_bitmasks(bytemask, rows, cols, bitmask);
    return (k == rows * cols / 2) ? 0 : -1;
}

/* ----------------------------------------------------------------- Hadamard */

/* transform/utils/hadamard.py:33-62 deterministic_hadamard_matrix (Sylvester): H[i][j] = (-1)^popcount(i&j) */
/* ---- MXFP4 scale helpers (quantization/utils/mxfp4_utils.py) ------------------------------------ */

/* mxfp4_utils.py:43-72 round_to_power_2: on the bf16 bit pattern, add a quarter of the mantissa range
 * (1 << 5) and keep sign + exponent; sums that overflow 16 bits wrap (the cast back to uint16). */
int orc_mxfp4_round_pow2(const uint16_t *x, int64_t n, uint16_t *out) {
    for (int64_t i = 0; i < n; ++i) out[i] = (uint16_t)(((uint32_t)x[i] + 32u) & 0xFF80u);
    return 0;
}

/* mxfp4_utils.py:75-97 generate_mxfp4_scales: 127 + floor(log2(p)) - 2 clamped to uint8, p the rounded power of
 * two.  For p = 2^e that is e + 125.  log2 of zero, of a negative number and of inf gives -inf / NaN / inf, whose
 * conversion to int32 is INT_MIN on the reference's hosts, so all of them clamp to 0. */
int orc_mxfp4_generate_scales(const uint16_t *x, int64_t n, uint8_t *out) {
    for (int64_t i = 0; i < n; ++i) {
        const uint32_t p = ((uint32_t)x[i] + 32u) & 0xFF80u;
        const int sign = (p >> 15) & 1, be = (p >> 7) & 0xFF;  /* the mantissa of p is zero */
        int v = 0;
        if (!sign && be != 0 && be != 0xFF) {
            v = (be - 127) + 125;
            if (v < 0) v = 0;
            if (v > 255) v = 255;
        }
        out[i] = (uint8_t)v;
    }
    return 0;
}

/* mxfp4_utils.py:25-40 convert_mxfp4_exp_scale: 2.0 ** (scale - 127) in fp32 (2^-127 is an fp32 subnormal,
 * 2^128 overflows to inf), then the cast to the dense dtype. */
int orc_mxfp4_convert_scales(const uint8_t *scale, int64_t n, int odt, void *out) {
    for (int64_t i = 0; i < n; ++i) {
        const float v = scale[i] ? bits_f32((uint32_t)scale[i] << 23) : bits_f32(0x00400000u);
        store_from_f32(out, odt, i, v);
    }
    return 0;
}

/* ---- Marlin-24 (compressors/sparse_quantized_compressors/marlin_24.py) --------------------------- */

/* utils/semi_structured_conversions.py:79-209 sparse_semi_structured_from_dense_cutlass for a 16-bit dense
 * dtype (int16 meta, four quadruples per meta element), on int8 codes standing for the fp16 tensor of the
 * same integers: per run of four, two values are kept by the non-zero pattern (:160-176), their indices
 * form a 4-bit code, four codes make a meta element, and the meta matrix is scattered into CUTLASS's
 * reordered, column-interleaved layout (:43-73). */
int orc_cutlass24_compress(const int8_t *dense, int64_t m, int64_t k, int8_t *sparse, int16_t *meta_reordered) {
    if (m % 32 || k % 16) return 1;
    const int64_t ncols = k / 16;
    for (int64_t r = 0; r < m; ++r)
        for (int64_t c = 0; c < ncols; ++c) {
            uint32_t elem = 0;
            for (int j = 0; j < 4; ++j) {
                const int8_t *d = dense + r * k + (c * 4 + j) * 4;
                const int m0 = d[0] != 0, m1 = d[1] != 0, m3 = d[3] != 0;
                const int e0 = m0 && m1, e1 = !m0 && m1, e2 = !m0 && !m1;
                const int i0 = e1 | (e2 << 1), i1 = (e0 | e2 | m3) | ((e1 | !m1) << 1);
                sparse[r * (k / 2) + (c * 4 + j) * 2] = d[i0];
                sparse[r * (k / 2) + (c * 4 + j) * 2 + 1] = d[i1];
                elem |= (uint32_t)(i0 | (i1 << 2)) << (4 * j);
            }
            int64_t dr = r / 64 * 64 + (r % 2) * 2 + (r % 8) / 4 + ((r % 32) % 4) / 2 * 32 + ((r % 64) / 8) * 4, dc = c;
            const int tr = (dr % 2 == 0) && (dc % 2 == 1), bl = (dr % 2 == 1) && (dc % 2 == 0);
            dr += tr - bl;
            dc -= tr - bl;
            meta_reordered[(dc / 2) * m * 2 + dr * 2 + dc % 2] = (int16_t)elem;
        }
    return 0;
}

/* utils/semi_structured_conversions.py:216-308 sparse_semi_structured_to_dense_cutlass (int16 meta): undo the
 * reordering, then scatter every kept value to the position its 2-bit index names; everything else is zero. */
int orc_cutlass24_decompress(const int8_t *sparse, const int16_t *meta_reordered, int64_t m, int64_t k2, int8_t *dense) {
    const int64_t ncols = k2 / 8, k = k2 * 2;
    if (m % 32 || k2 % 8) return 1;
    memset(dense, 0, (size_t)(m * k));
    for (int64_t r = 0; r < m; ++r)
        for (int64_t c = 0; c < ncols; ++c) {
            int64_t dr = r / 64 * 64 + (r % 2) * 2 + (r % 8) / 4 + ((r % 32) % 4) / 2 * 32 + ((r % 64) / 8) * 4, dc = c;
            const int tr = (dr % 2 == 0) && (dc % 2 == 1), bl = (dr % 2 == 1) && (dc % 2 == 0);
            dr += tr - bl;
            dc -= tr - bl;
            const uint32_t elem = (uint16_t)meta_reordered[(dc / 2) * m * 2 + dr * 2 + dc % 2];
            for (int j = 0; j < 4; ++j) {
                const int i0 = (elem >> (4 * j)) & 3, i1 = (elem >> (4 * j + 2)) & 3;
                int8_t *d = dense + r * k + (c * 4 + j) * 4;
                d[i0] = sparse[r * k2 + (c * 4 + j) * 2];      /* scatter order: a later write wins */
                d[i1] = sparse[r * k2 + (c * 4 + j) * 2 + 1];
            }
        }
    return 0;
}

/* utils/permutations_24.py:32-65 */
static void marlin24_perm(int bits, int *perm /* 1024 */) {
    int list[1024], n = 0;
    for (int i = 0; i < 32; ++i) {
        int perm1[8], p = 0;
        const int col = i / 4, col_o = col / 2;
        for (int block = 0; block < 2; ++block) {
            const int rows4[4] = {2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1};
            for (int t = 0; t < 4; ++t) perm1[p++] = 16 * rows4[t] + col_o * 256 + 8 * (col % 2) + 4 * block;
        }
        for (int j = 0; j < 4; ++j)
            for (int t = 0; t < 8; ++t) list[n++] = perm1[t] + j;
    }
    static const int il4[8] = {0, 2, 4, 6, 1, 3, 5, 7}, il8[4] = {0, 2, 1, 3};
    const int L = bits == 4 ? 8 : 4;
    for (int b = 0; b < 1024 / L; ++b)
        for (int t = 0; t < L; ++t) perm[b * L + t] = list[b * L + (bits == 4 ? il4[t] : il8[t])];
}

/* marlin_24.py:208-249 marlin_permute_weights + pack_weight_24 on the transposed, offset codes:
 * sparse is [n, k2] (k2 = in_features / 2); out is [k2 / 16, n * 16 / (32 / bits)] int32. */
int orc_marlin24_pack_weight(const int8_t *sparse, int64_t n, int64_t k2, int bits, int32_t *out) {
    if ((bits != 4 && bits != 8) || k2 % 16 || n % 64) return 1;
    int perm[1024];
    marlin24_perm(bits, perm);
    const int pf = 32 / bits, half = (1 << bits) / 2;
    const int64_t row_elems = n * 16;
    for (int64_t kt = 0; kt < k2 / 16; ++kt)
        for (int64_t j = 0; j < row_elems / pf; ++j) {
            uint32_t word = 0;
            for (int i = 0; i < pf; ++i) {
                const int64_t idx = j * pf + i, src = idx / 1024 * 1024 + perm[idx % 1024];
                const int64_t nt = src / 256, ki = (src % 256) / 16, ni = src % 16;
                const uint32_t v = (uint32_t)((int)sparse[(nt * 16 + ni) * k2 + kt * 16 + ki] + half);
                word |= v << (bits * i);
            }
            out[kt * (row_elems / pf) + j] = (int32_t)word;
        }
    return 0;
}

/* marlin_24.py:252-273 pack_scales_24: scale is [n, g] (16-bit), out is [g, n]; `grouped` selects the
 * group permutation (group size below in_features / 2), otherwise the per-channel one (the identity). */
int orc_marlin24_pack_scales(const uint16_t *scale, int64_t n, int64_t g, int grouped, uint16_t *out) {
    if (n % 64) return 1;
    static const int inner[8] = {0, 4, 1, 5, 2, 6, 3, 7};
    for (int64_t f = 0; f < g * n; ++f) {  /* flat index of the transposed [g, n] tensor */
        const int64_t blk = f / 64, w = f % 64;
        const int64_t src = blk * 64 + (grouped ? (w / 8) * 8 + inner[w % 8] : w);
        out[f] = scale[(src % n) * g + src / n];
    }
    return 0;
}

static inline double sylvester(int64_t i, int64_t j) { return (__builtin_popcountll(i & j) & 1) ? -1.0 : 1.0; }

/* transform/factory/hadamard.py:104-121 HadamardTransform.forward with the offline precision float64
 * and transform/utils/matrix.py:115-122, :160-169 for torch.nn.Linear weights.
 *
 * Wh = diag(signs) @ H_n (hadamard.py:85-89; signs = NULL for the deterministic matrix), transposed
 * when `inverse`.  side 0 (weight_input): out = W @ Wh^T per n-column block;
 * side 1 (weight_output): out = Wh^T @ W per n-row block.  Result / sqrt(n), cast to the value dtype. */
int orc_hadamard(const void *x, int dt, int64_t rows, int64_t cols, int64_t n, const int8_t *signs,
                 int inverse, int side, void *out) {
    double *Wh = (double *)malloc(sizeof(double) * (size_t)(n * n));
    if (!Wh) return -2;
    for (int64_t i = 0; i < n; ++i)
        for (int64_t j = 0; j < n; ++j) {
            double v = (signs ? (double)signs[i] : 1.0) * sylvester(i, j); /* diag(Q) @ H */
            if (inverse) Wh[j * n + i] = v; else Wh[i * n + j] = v;
        }
    double scale = sqrt((double)n);
    if (side == 0) {
        if (cols % n) { free(Wh); return -1; }
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; ++r)
            for (int64_t b = 0; b < cols / n; ++b)
                for (int64_t i = 0; i < n; ++i) {
                    double acc = 0.0; /* (W @ Wh^T)[r, i] = sum_j W[r, j] * Wh[i, j] */
                    for (int64_t j = 0; j < n; ++j) {
                        double w = (dt == ORC_F64) ? ((const double *)x)[r * cols + b * n + j]
                                                   : (double)load_as_f32(x, dt, r * cols + b * n + j);
                        acc += w * Wh[i * n + j];
                    }
                    double v = acc / scale;
                    if (dt == ORC_F64) ((double *)out)[r * cols + b * n + i] = v;
                    else store_from_f32(out, dt, r * cols + b * n + i, (float)v);
                }
    } else {
        if (rows % n) { free(Wh); return -1; }
#pragma omp parallel for schedule(static)
        for (int64_t c = 0; c < cols; ++c)
            for (int64_t b = 0; b < rows / n; ++b)
                for (int64_t i = 0; i < n; ++i) {
                    double acc = 0.0; /* (Wh^T @ W)[i, c] = sum_j Wh[j, i] * W[j, c] */
                    for (int64_t j = 0; j < n; ++j) {
                        double w = (dt == ORC_F64) ? ((const double *)x)[(b * n + j) * cols + c]
                                                   : (double)load_as_f32(x, dt, (b * n + j) * cols + c);
                        acc += Wh[j * n + i] * w;
                    }
                    double v = acc / scale;
                    if (dt == ORC_F64) ((double *)out)[(b * n + i) * cols + c] = v;
                    else store_from_f32(out, dt, (b * n + i) * cols + c, (float)v);
                }
    }
    free(Wh);
    return 0;
}
