// Quantization parameters: tile min/max (quantization/utils/helpers.py:149-205), calculate_qparams
// (:67-146) and generate_gparam (:414-434).
#include <algorithm>
#include <cfloat>

#include "ctb_codec.cuh"

namespace ctb {

constexpr int kThreads = 256;

__device__ __forceinline__ void warp_minmax(float &mn, float &mx, int width) {
    for (int o = width >> 1; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    }
}

__device__ __forceinline__ void block_minmax(float &mn, float &mx) {
    __shared__ float smn[kThreads / 32], smx[kThreads / 32];
    warp_minmax(mn, mx, 32);
    int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();  // protects reuse of the shared arrays across calls
    if (l == 0) { smn[w] = mn; smx[w] = mx; }
    __syncthreads();
    mn = (l < kThreads / 32) ? smn[l] : FLT_MAX;
    mx = (l < kThreads / 32) ? smx[l] : -FLT_MAX;
    mn = (threadIdx.x < 32) ? mn : FLT_MAX;
    warp_minmax(mn, mx, 32);  // every warp ends with the block result in all lanes of warp 0
}

template <int F>
__device__ __forceinline__ void chunk_minmax(const void *x, int64_t chunk, float &mn, float &mx) {
    float v[8];
    Raw8 r = load_raw<F>(x, chunk);
    decode8<F>(r, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) { mn = fminf(mn, v[i]); mx = fmaxf(mx, v[i]); }
}

// ---- 16-bit element types: min / max stay packed two to a register (like fminf / fmaxf, a NaN operand is ignored)
template <int F>
__device__ __forceinline__ uint32_t min2(uint32_t a, uint32_t b) {
    if constexpr (F == F_BF16) return bf162_as_u32(__hmin2(u32_as_bf162(a), u32_as_bf162(b)));
    else { const __half2 r = __hmin2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b)); return *reinterpret_cast<const uint32_t *>(&r); }
}
template <int F>
__device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b) {
    if constexpr (F == F_BF16) return bf162_as_u32(__hmax2(u32_as_bf162(a), u32_as_bf162(b)));
    else { const __half2 r = __hmax2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b)); return *reinterpret_cast<const uint32_t *>(&r); }
}
template <int F> struct Packed16 {  // +inf / -inf in both halves
    static constexpr uint32_t kPosInf = F == F_BF16 ? 0x7F807F80u : 0x7C007C00u;
    static constexpr uint32_t kNegInf = kPosInf | 0x80008000u;
};

// running packed min / max over one 8-element chunk
template <int F, typename Index>
__device__ __forceinline__ void chunk_minmax16(const void *x, Index chunk, uint32_t &mn2, uint32_t &mx2) {
    const uint4 q = ld_stream(reinterpret_cast<const uint4 *>(x) + chunk);
    mn2 = min2<F>(min2<F>(mn2, q.x), min2<F>(min2<F>(q.y, q.z), q.w));
    mx2 = max2<F>(max2<F>(mx2, q.x), max2<F>(max2<F>(q.y, q.z), q.w));
}

// one register holding (min, -max) of both halves: a single packed min then reduces both at once
template <int F>
__device__ __forceinline__ uint32_t fold_minmax16(uint32_t mn2, uint32_t mx2) {
    const uint32_t nmx = mx2 ^ 0x80008000u;
    return min2<F>(prmt_b32(mn2, nmx, 0x5410), prmt_b32(mn2, nmx, 0x7632));
}

template <int F>
__device__ __forceinline__ void unpack_minmax16(uint32_t mn2, uint32_t mx2, float &mn, float &mx) {
    const uint32_t k = fold_minmax16<F>(mn2, mx2);
    if constexpr (F == F_BF16) { mn = bf16_bits_to_f32(k & 0xFFFFu); mx = -bf16_bits_to_f32(k >> 16); }
    else { const float2 f = half2_bits_to_float2(k); mn = f.x; mx = -f.y; }
}

// (a16) the group kernel for bf16 / f16: one chunk per lane, L lanes reduce one packed (min, -max) register.
//       32-bit chunk indices (the host checks the range).
template <int F, int L>
__global__ void __launch_bounds__(kThreads) minmax_group16_kernel(const uint4 *x, uint32_t chunks, uint16_t *out_min, uint16_t *out_max) {
    constexpr int kShift = L == 1 ? 0 : L == 2 ? 1 : L == 4 ? 2 : L == 8 ? 3 : L == 16 ? 4 : 5;
    const uint32_t stride = gridDim.x * kThreads;
    const uint32_t padded = (chunks + 31u) & ~31u;  // whole warps stay in the loop for the shuffles
    for (uint32_t c = blockIdx.x * kThreads + threadIdx.x; c < padded; c += 2 * stride) {
        const uint32_t c1 = c + stride;
        uint32_t mn0 = Packed16<F>::kPosInf, mx0 = Packed16<F>::kNegInf, mn1 = mn0, mx1 = mx0;
        if (c < chunks) chunk_minmax16<F>(x, c, mn0, mx0);
        if (c1 < chunks) chunk_minmax16<F>(x, c1, mn1, mx1);
        uint32_t k0 = fold_minmax16<F>(mn0, mx0), k1 = fold_minmax16<F>(mn1, mx1);
#pragma unroll
        for (int o = L >> 1; o > 0; o >>= 1) {
            k0 = min2<F>(k0, __shfl_xor_sync(0xFFFFFFFFu, k0, o));
            k1 = min2<F>(k1, __shfl_xor_sync(0xFFFFFFFFu, k1, o));
        }
        if ((c & (L - 1)) == 0) {
            if (c < chunks) { out_min[c >> kShift] = (uint16_t)k0; out_max[c >> kShift] = (uint16_t)((k0 >> 16) ^ 0x8000u); }
            if (c1 < chunks) { out_min[c1 >> kShift] = (uint16_t)k1; out_max[c1 >> kShift] = (uint16_t)((k1 >> 16) ^ 0x8000u); }
        }
    }
}

template <int F>
static void launch_group16(int L, int grid, cudaStream_t st, const void *x, int64_t chunks, void *out_min, void *out_max) {
    const uint4 *p = (const uint4 *)x;
    uint16_t *mn = (uint16_t *)out_min, *mx = (uint16_t *)out_max;
    const uint32_t n = (uint32_t)chunks;
    switch (L) {
    case 1: minmax_group16_kernel<F, 1><<<grid, kThreads, 0, st>>>(p, n, mn, mx); break;
    case 2: minmax_group16_kernel<F, 2><<<grid, kThreads, 0, st>>>(p, n, mn, mx); break;
    case 4: minmax_group16_kernel<F, 4><<<grid, kThreads, 0, st>>>(p, n, mn, mx); break;
    case 8: minmax_group16_kernel<F, 8><<<grid, kThreads, 0, st>>>(p, n, mn, mx); break;
    case 16: minmax_group16_kernel<F, 16><<<grid, kThreads, 0, st>>>(p, n, mn, mx); break;
    default: minmax_group16_kernel<F, 32><<<grid, kThreads, 0, st>>>(p, n, mn, mx); break;
    }
}

// (a) groups of 8*L consecutive elements inside a row, L a power of two <= 32: one chunk per lane,
//     L lanes cooperate through shuffles.  Flat indexing: group g covers chunks [g*L, (g+1)*L).
template <int F>
__global__ void __launch_bounds__(kThreads) minmax_group_kernel(const void *x, int64_t chunks, int L, int dt, void *out_min, void *out_max) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t padded = (chunks + 31) & ~(int64_t)31;  // whole warps stay in the loop for the shuffles
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < padded; c += stride) {
        float mn = FLT_MAX, mx = -FLT_MAX;
        if (c < chunks) chunk_minmax<F>(x, c, mn, mx);
        warp_minmax(mn, mx, L);
        if (c < chunks && (c & (L - 1)) == 0) {
            const int64_t gi = c >> (31 - __clz(L));  // L is a power of two
            store_f32(out_min, dt, gi, mn);
            store_f32(out_max, dt, gi, mx);
        }
    }
}

// (b) one block per [row_group x col_group] tile, any shape and alignment (scalar loads)
__global__ void __launch_bounds__(kThreads) minmax_tile_kernel(const void *x, int dt, int64_t rows, int64_t cols, int64_t rg, int64_t cg,
                                                                void *out_min, void *out_max) {
    const int64_t tiles_c = cols / cg, tiles = (rows / rg) * tiles_c;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        int64_t r0 = (t / tiles_c) * rg, c0 = (t % tiles_c) * cg;
        float mn = FLT_MAX, mx = -FLT_MAX;
        for (int64_t i = threadIdx.x; i < rg * cg; i += kThreads) {
            float v = load_f32(x, dt, (r0 + i / cg) * cols + c0 + i % cg);
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
        block_minmax(mn, mx);
        if (threadIdx.x == 0) { store_f32(out_min, dt, t, mn); store_f32(out_max, dt, t, mx); }
    }
}

// (b'') one block per [row_group x col_group] tile whose rows are whole 16-byte chunks (BLOCK strategy): 128-bit loads
template <int F>
__global__ void __launch_bounds__(kThreads) minmax_tile_vec_kernel(const void *x, int dt, int64_t rows, int64_t cols, int rg, int cg,
                                                                    void *out_min, void *out_max) {
    const int64_t tiles_c = cols / cg, tiles = (rows / rg) * tiles_c, cpr = cols / 8;
    const int cpt = cg / 8, per_tile = rg * cpt;  // chunks per tile row / per tile
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t tr = t / tiles_c, base = tr * rg * cpr + (t - tr * tiles_c) * cpt;  // first chunk of the tile
        float mn = FLT_MAX, mx = -FLT_MAX;
        if constexpr (F == F_F32) {
            for (int i = threadIdx.x; i < per_tile; i += kThreads) {
                const int r = i / cpt;
                chunk_minmax<F>(x, base + (int64_t)r * cpr + (i - r * cpt), mn, mx);
            }
        } else {
            uint32_t mn2 = Packed16<F>::kPosInf, mx2 = Packed16<F>::kNegInf;
            // thread i walks chunks i, i + kThreads, ... of the tile: (row, column) advance by a fixed step with one carry
            const int dr = kThreads / cpt, dj = kThreads - dr * cpt;
            int r = (int)threadIdx.x / cpt, j = (int)threadIdx.x - r * cpt;
            const uint4 *p = reinterpret_cast<const uint4 *>(x) + base;
#pragma unroll 4
            for (int i = threadIdx.x; i < per_tile; i += kThreads) {
                chunk_minmax16<F>(p, (int64_t)r * cpr + j, mn2, mx2);
                j += dj;
                r += dr;
                if (j >= cpt) { j -= cpt; ++r; }
            }
            unpack_minmax16<F>(mn2, mx2, mn, mx);
        }
        block_minmax(mn, mx);
        if (threadIdx.x == 0) { store_f32(out_min, dt, t, mn); store_f32(out_max, dt, t, mx); }
    }
}

// (b') one block per row, 128-bit loads (CHANNEL / TOKEN: the tile is a whole row)
template <int F>
__global__ void __launch_bounds__(kThreads) minmax_row_kernel(const void *x, int dt, int64_t rows, int64_t cpr, void *out_min, void *out_max) {
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        float mn = FLT_MAX, mx = -FLT_MAX;
        if constexpr (F == F_F32) {
            for (int64_t c = threadIdx.x; c < cpr; c += kThreads) chunk_minmax<F>(x, r * cpr + c, mn, mx);
        } else {
            uint32_t mn2 = Packed16<F>::kPosInf, mx2 = Packed16<F>::kNegInf;
#pragma unroll 4
            for (int64_t c = threadIdx.x; c < cpr; c += kThreads) chunk_minmax16<F>(x, r * cpr + c, mn2, mx2);
            unpack_minmax16<F>(mn2, mx2, mn, mx);
        }
        block_minmax(mn, mx);
        if (threadIdx.x == 0) { store_f32(out_min, dt, r, mn); store_f32(out_max, dt, r, mx); }
    }
}

// (b16) CHANNEL / TOKEN for bf16 / f16 rows of up to 4096 chunks: a warp per row, no block barrier; the lanes read
//       32 consecutive chunks per step (512 contiguous bytes), four steps in flight
template <int F>
__global__ void __launch_bounds__(kThreads) minmax_warprow16_kernel(const uint4 *x, int64_t rows, int cpr, uint16_t *out_min, uint16_t *out_max) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
    for (int64_t r = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
        const uint4 *row = x + r * cpr;
        uint32_t mn2 = Packed16<F>::kPosInf, mx2 = Packed16<F>::kNegInf;
#pragma unroll 4
        for (int c = lane; c < cpr; c += 32) chunk_minmax16<F>(row, c, mn2, mx2);
        uint32_t k = fold_minmax16<F>(mn2, mx2);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) k = min2<F>(k, __shfl_xor_sync(0xFFFFFFFFu, k, o));
        if (lane == 0) { out_min[r] = (uint16_t)k; out_max[r] = (uint16_t)((k >> 16) ^ 0x8000u); }
    }
}

// (c) one tile = the whole tensor: per-block partials into the workspace, then a one-block finish
template <int F>
__global__ void __launch_bounds__(kThreads, 8) minmax_flat_kernel(const void *x, int dt, int64_t n, float *partial) {
    float mn = FLT_MAX, mx = -FLT_MAX;
    const int64_t chunks = n / 8;
    if constexpr (F == F_F32) {
        for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kThreads)
            chunk_minmax<F>(x, c, mn, mx);
    } else {
        uint32_t mn2 = Packed16<F>::kPosInf, mx2 = Packed16<F>::kNegInf;
#pragma unroll 8
        for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kThreads)
            chunk_minmax16<F>(x, c, mn2, mx2);
        unpack_minmax16<F>(mn2, mx2, mn, mx);
    }
    if (blockIdx.x == 0)
        for (int64_t i = chunks * 8 + threadIdx.x; i < n; i += kThreads) {  // ragged tail
            float v = load_f32(x, dt, i);
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
    block_minmax(mn, mx);
    if (threadIdx.x == 0) { partial[2 * blockIdx.x] = mn; partial[2 * blockIdx.x + 1] = mx; }
}

__global__ void __launch_bounds__(kThreads) minmax_finish_kernel(const float *partial, int n, int dt, void *out_min, void *out_max) {
    float mn = FLT_MAX, mx = -FLT_MAX;
    for (int i = threadIdx.x; i < n; i += kThreads) { mn = fminf(mn, partial[2 * i]); mx = fmaxf(mx, partial[2 * i + 1]); }
    block_minmax(mn, mx);
    if (threadIdx.x == 0) { store_f32(out_min, dt, 0, mn); store_f32(out_max, dt, 0, mx); }
}

// helpers.py:67-146, one thread per (min, max) pair
__global__ void __launch_bounds__(kThreads) qparams_kernel(const void *mins, const void *maxs, int M, int64_t n, int qtype, int bits, int symmetric,
                                                            const float *gs, void *out_scale, void *out_zp, int zdt) {
    const float eps = 1.1920928955078125e-07f;  // torch.finfo(torch.float32).eps
    float qmin, qmax;
    if (qtype == CTB_QINT) { qmax = (float)(1 << bits) / 2 - 1; qmin = -(float)(1 << bits) / 2; }
    else if (bits == 8) { qmax = 448.0f; qmin = -448.0f; }
    else { qmax = 6.0f; qmin = -6.0f; }
    const float bit_range = qmax - qmin;
    const bool fp4 = qtype == CTB_QFLOAT && bits == 4;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads) {
        float mn = fminf(load_f32(mins, M, i), 0.0f);  // :87-88 zero stays representable
        float mx = fmaxf(load_f32(maxs, M, i), 0.0f);
        float zp = 0.0f;
        if (symmetric) {
            float mvp = fmaxf(fabsf(mn), fabsf(mx));
            if (fp4 && gs != nullptr) {
                // :103-120  e4m3(clamp(global_scale * (amax / 6))) with 0 replaced by 0.125
                float sc = gs[0] * round_to_rt(M, __fdiv_rn(mvp, 6.0f));
                sc = clamp_nan(sc, -448.0f, 448.0f);
                uint8_t b = f32_to_e4m3(sc);
                if ((b & 0x7F) == 0) b = 0x20;
                ((uint8_t *)out_scale)[i] = b;
            } else {
                float sc = round_to_rt(M, __fdiv_rn(mvp, bit_range / 2.0f));  // :110
                store_f32(out_scale, M, i, fmaxf(sc, eps));                  // :122
            }
        } else {
            float sc = round_to_rt(M, __fdiv_rn(round_to_rt(M, mx - mn), bit_range));  // :131
            sc = round_to_rt(M, fmaxf(sc, eps));
            zp = round_to_rt(M, qmin - round_to_rt(M, __fdiv_rn(mn, sc)));             // :133
            zp = clamp_nan(zp, qmin, qmax);
            store_f32(out_scale, M, i, sc);
        }
        if (qtype == CTB_QINT) zp = rintf(zp);  // :138-139
        store_f32(out_zp, zdt, i, zp);
    }
}

// helpers.py:414-434.  The reference writes `448 * 6 / amax` with a Python scalar on the left, which torch evaluates
// as amax.reciprocal() * 2688 (Tensor.__rtruediv__): the reciprocal is rounded to the min/max dtype before the product is.
__global__ void gparam_kernel(const void *mn_p, const void *mx_p, int M, float *out) {
    float mn = fminf(load_f32(mn_p, M, 0), 0.0f), mx = fmaxf(load_f32(mx_p, M, 0), 0.0f);
    const float r = round_to_rt(M, __frcp_rn(fmaxf(fabsf(mn), fabsf(mx))));
    out[0] = round_to_rt(M, __fmul_rn(r, 2688.0f));
}

// quantization/utils/mxfp4_utils.py.  MODE 0: round_to_power_2 (bf16 bits in, bf16 bits out); MODE 1:
// generate_mxfp4_scales (bf16 in, uint8 exponent out).  Both work on the bit pattern: add a quarter of the mantissa
// range and keep sign + exponent (a sum past 16 bits wraps, as the reference's cast back to uint16 does); the
// exponent byte is e + 125 for a positive normal power of two 2^e and 0 for everything whose log2 is not finite
// (zero, negatives, inf), which is what the reference's float -> int32 conversion and clamp leave.
template <int MODE>
__global__ void __launch_bounds__(256) mxfp4_scale_kernel(const uint16_t *x, int64_t n, void *out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t p = ((uint32_t)x[i] + 32u) & 0xFF80u;
        if constexpr (MODE == 0) {
            ((uint16_t *)out)[i] = (uint16_t)p;
        } else {
            const int be = (int)((p >> 7) & 0xFFu);
            int v = 0;
            if ((p >> 15) == 0 && be != 0 && be != 0xFF) v = max(be - 2, 0);  // (be - 127) + 125
            ((uint8_t *)out)[i] = (uint8_t)v;
        }
    }
}

// convert_mxfp4_exp_scale: 2 ** (scale - 127) in fp32 (2^-127 is an fp32 subnormal, exponent byte 255 overflows to
// inf, which is also what shifting it into the exponent field gives), then the cast to the dense dtype
__global__ void __launch_bounds__(256) mxfp4_convert_kernel(const uint8_t *scale, int64_t n, int odt, void *out) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t b = scale[i];
        store_f32(out, odt, i, __uint_as_float(b ? b << 23 : 0x00400000u));
    }
}

static int flat_blocks() { return sm_count() * 8; }

}  // namespace ctb

using namespace ctb;

extern "C" int64_t ctb_minmax_workspace_bytes(int64_t rows, int64_t cols, int64_t row_group, int64_t col_group) {
    if (row_group == rows && col_group == cols) return (int64_t)flat_blocks() * 2 * sizeof(float);
    return 0;
}

extern "C" int ctb_minmax(const void *x, int32_t dt, int64_t rows, int64_t cols, int64_t rg, int64_t cg, void *out_min, void *out_max,
                          void *workspace, void *stream) {
    if (!x || !out_min || !out_max) return fail(CTB_EINVAL_NULL, "null buffer");
    if (!is_float_dtype(dt)) return fail(CTB_EINVAL_DTYPE, "min/max needs bf16, f16 or f32");
    if (rows <= 0 || cols <= 0 || rg <= 0 || cg <= 0 || rows % rg || cols % cg) return fail(CTB_EINVAL_SHAPE, "tiles must divide the tensor");
    cudaStream_t st = as_stream(stream);
    const int F = dt == CTB_BF16 ? F_BF16 : dt == CTB_F16 ? F_F16 : F_F32;
    const bool vec = aligned16(x) && cols % 8 == 0;
    if (rg == rows && cg == cols) {  // whole tensor
        if (!workspace) return fail(CTB_EINVAL_NULL, "whole-tensor min/max needs the workspace");
        if (!aligned16(x)) return fail(CTB_EINVAL_ALIGN, "x must be 16-byte aligned");
        int blocks = (int)std::min<int64_t>(flat_blocks(), std::max<int64_t>(1, cdiv(rows * cols / 8, kThreads)));
        float *part = (float *)workspace;
        if (F == F_BF16) minmax_flat_kernel<F_BF16><<<blocks, kThreads, 0, st>>>(x, dt, rows * cols, part);
        else if (F == F_F16) minmax_flat_kernel<F_F16><<<blocks, kThreads, 0, st>>>(x, dt, rows * cols, part);
        else minmax_flat_kernel<F_F32><<<blocks, kThreads, 0, st>>>(x, dt, rows * cols, part);
        int rc = after_launch("minmax_flat_kernel");
        if (rc) return rc;
        minmax_finish_kernel<<<1, kThreads, 0, st>>>(part, blocks, dt, out_min, out_max);
        return after_launch("minmax_finish_kernel");
    }
    if (vec && rg == 1 && cg % 8 == 0) {
        int64_t L = cg / 8;
        if (L <= 32 && (L & (L - 1)) == 0) {
            int64_t chunks = rows * cols / 8;
            int grid = grid_for(chunks, kThreads, 8);
            if (F == F_BF16 && chunks < (1LL << 31)) launch_group16<F_BF16>((int)L, grid, st, x, chunks, out_min, out_max);
            else if (F == F_F16 && chunks < (1LL << 31)) launch_group16<F_F16>((int)L, grid, st, x, chunks, out_min, out_max);
            else if (F == F_BF16) minmax_group_kernel<F_BF16><<<grid, kThreads, 0, st>>>(x, chunks, (int)L, dt, out_min, out_max);
            else if (F == F_F16) minmax_group_kernel<F_F16><<<grid, kThreads, 0, st>>>(x, chunks, (int)L, dt, out_min, out_max);
            else minmax_group_kernel<F_F32><<<grid, kThreads, 0, st>>>(x, chunks, (int)L, dt, out_min, out_max);
            return after_launch("minmax_group_kernel");
        }
        if (cg == cols && F != F_F32 && cols / 8 <= 4096) {
            const int grid = grid_for(rows, kThreads / 32, 8);
            if (F == F_BF16) minmax_warprow16_kernel<F_BF16><<<grid, kThreads, 0, st>>>((const uint4 *)x, rows, (int)(cols / 8), (uint16_t *)out_min, (uint16_t *)out_max);
            else minmax_warprow16_kernel<F_F16><<<grid, kThreads, 0, st>>>((const uint4 *)x, rows, (int)(cols / 8), (uint16_t *)out_min, (uint16_t *)out_max);
            return after_launch("minmax_warprow16_kernel");
        }
        if (cg == cols) {
            int grid = grid_for(rows, 1, 64);
            if (F == F_BF16) minmax_row_kernel<F_BF16><<<grid, kThreads, 0, st>>>(x, dt, rows, cols / 8, out_min, out_max);
            else if (F == F_F16) minmax_row_kernel<F_F16><<<grid, kThreads, 0, st>>>(x, dt, rows, cols / 8, out_min, out_max);
            else minmax_row_kernel<F_F32><<<grid, kThreads, 0, st>>>(x, dt, rows, cols / 8, out_min, out_max);
            return after_launch("minmax_row_kernel");
        }
    }
    int grid = grid_for((rows / rg) * (cols / cg), 1, 8);
    if (cols % 8 == 0 && cg % 8 == 0 && aligned16(x) && rg * (cg / 8) < 0x7FFFFFFF) {
        if (dt == CTB_BF16) minmax_tile_vec_kernel<F_BF16><<<grid, kThreads, 0, st>>>(x, dt, rows, cols, (int)rg, (int)cg, out_min, out_max);
        else if (dt == CTB_F16) minmax_tile_vec_kernel<F_F16><<<grid, kThreads, 0, st>>>(x, dt, rows, cols, (int)rg, (int)cg, out_min, out_max);
        else minmax_tile_vec_kernel<F_F32><<<grid, kThreads, 0, st>>>(x, dt, rows, cols, (int)rg, (int)cg, out_min, out_max);
        return after_launch("minmax_tile_vec_kernel");
    }
    minmax_tile_kernel<<<grid, kThreads, 0, st>>>(x, dt, rows, cols, rg, cg, out_min, out_max);
    return after_launch("minmax_tile_kernel");
}

extern "C" int ctb_calculate_qparams(const void *mins, const void *maxs, int32_t dtype, int64_t n, int32_t qtype, int32_t bits,
                                     int32_t symmetric, const float *gs, void *out_scale, void *out_zp, int32_t zdt, void *stream) {
    if (n != 0 && (!mins || !maxs || !out_scale || !out_zp)) return fail(CTB_EINVAL_NULL, "null buffer");  // an empty tensor has no storage
    if (!is_float_dtype(dtype)) return fail(CTB_EINVAL_DTYPE, "min/max must be bf16, f16 or f32");
    if (qtype == CTB_QFLOAT && bits == 4 && !symmetric) return fail(CTB_EUNSUPPORTED, "Asymmetric Quantization is not supported for FP4");
    if (qtype == CTB_QFLOAT && bits != 4 && bits != 8) return fail(CTB_EUNSUPPORTED, "Range calculation only supported for 4 and 8 bits");
    if (qtype == CTB_QINT && (bits < 1 || bits > 8)) return fail(CTB_EUNSUPPORTED, "int quantization supports 1..8 bits");
    if (zdt != CTB_I8 && zdt != CTB_E4M3) return fail(CTB_EINVAL_DTYPE, "zero point dtype must be int8 or e4m3");
    if (n <= 0) return CTB_OK;
    qparams_kernel<<<grid_for(n, kThreads, 4), kThreads, 0, as_stream(stream)>>>(mins, maxs, dtype, n, qtype, bits, symmetric, gs, out_scale, out_zp, zdt);
    return after_launch("qparams_kernel");
}

extern "C" int ctb_generate_gparam(const void *mn, const void *mx, int32_t dtype, float *out, void *stream) {
    if (!mn || !mx || !out) return fail(CTB_EINVAL_NULL, "null buffer");
    if (!is_float_dtype(dtype)) return fail(CTB_EINVAL_DTYPE, "min/max must be bf16, f16 or f32");
    gparam_kernel<<<1, 1, 0, as_stream(stream)>>>(mn, mx, dtype, out);
    return after_launch("gparam_kernel");
}

extern "C" int ctb_mxfp4_round_pow2(const void *x, int64_t n, void *out, void *stream) {
    if (n != 0 && (!x || !out)) return fail(CTB_EINVAL_NULL, "null buffer");
    if (n < 0) return fail(CTB_EINVAL_SHAPE, "negative size");
    if (n == 0) return CTB_OK;
    mxfp4_scale_kernel<0><<<grid_for(n, 256, 8), 256, 0, as_stream(stream)>>>((const uint16_t *)x, n, out);
    return after_launch("mxfp4_scale_kernel");
}

extern "C" int ctb_mxfp4_generate_scales(const void *x, int64_t n, uint8_t *out, void *stream) {
    if (n != 0 && (!x || !out)) return fail(CTB_EINVAL_NULL, "null buffer");
    if (n < 0) return fail(CTB_EINVAL_SHAPE, "negative size");
    if (n == 0) return CTB_OK;
    mxfp4_scale_kernel<1><<<grid_for(n, 256, 8), 256, 0, as_stream(stream)>>>((const uint16_t *)x, n, out);
    return after_launch("mxfp4_scale_kernel");
}

extern "C" int ctb_mxfp4_convert_scales(const uint8_t *scale, int64_t n, int32_t out_dtype, void *out, void *stream) {
    if (n != 0 && (!scale || !out)) return fail(CTB_EINVAL_NULL, "null buffer");
    if (!is_float_dtype(out_dtype)) return fail(CTB_EINVAL_DTYPE, "dense scales are bf16, f16 or f32");
    if (n < 0) return fail(CTB_EINVAL_SHAPE, "negative size");
    if (n == 0) return CTB_OK;
    mxfp4_convert_kernel<<<grid_for(n, 256, 8), 256, 0, as_stream(stream)>>>(scale, n, out_dtype, out);
    return after_launch("mxfp4_convert_kernel");
}
