// Block Hadamard rotation of Linear weights (transform/factory/hadamard.py:104-121 with
// transform/utils/matrix.py:65-134) and the fused calibrate + quantize + pack kernels.
//
// Wh = diag(signs) @ H_n with H_n the Sylvester matrix, H[i][j] = (-1)^popcount(i & j)
// (transform/utils/hadamard.py:33-89).  For a Linear weight W:
//   weight_input,  forward: out[r, i] = signs[i] * FWHT(W[r, block])[i]
//   weight_input,  inverse: out[r, i] = FWHT(signs * W[r, block])[i]
//   weight_output, forward: out[i, c] = FWHT over the block's rows of (signs[row] * W[row, c])
//   weight_output, inverse: out[i, c] = signs[i] * FWHT over rows of W[:, c]
// each divided by sqrt(n) and rounded to the dtype of W.  The reference computes in float64; sums of
// at most 256 bf16/fp16 values are exact in float64 whatever the order, so the float64 butterfly
// below reproduces its matmul bit for bit.  The float32 mode trades that for speed.
#include <algorithm>

#include "ctb_codec.cuh"
#include "ctb_rotquant.cuh"

namespace ctb {

constexpr int kThreads = 256;

template <typename A>
__device__ __forceinline__ A shfl_xor(A v, int o) {
    if constexpr (sizeof(A) == 8) {
        int lo = __double2loint(v), hi = __double2hiint(v);
        lo = __shfl_xor_sync(0xFFFFFFFFu, lo, o);
        hi = __shfl_xor_sync(0xFFFFFFFFu, hi, o);
        return __hiloint2double(hi, lo);
    } else {
        return __shfl_xor_sync(0xFFFFFFFFu, v, o);
    }
}

// t / c for a run-time constant c = sqrt(n) with rc = 1 / c (both correctly rounded): exact when c is a power of
// two, otherwise the reciprocal product plus one Markstein correction, which is the correctly rounded quotient for
// operands this far from the overflow / underflow ends.  (A zero keeps no sign: every caller adds +0.0 afterwards.)
template <typename A>
__device__ __forceinline__ A div_const(A t, A c, A rc) {
    const A q0 = t * rc;
    return fma(fma(-q0, c, t), rc, q0);
}

// in-register butterfly over the 8 elements a lane holds (index bits 0..2 of the block position)
template <typename A>
__device__ __forceinline__ void fwht8(A (&v)[8]) {
#pragma unroll
    for (int h = 1; h < 8; h <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if ((i & h) == 0) {
                A a = v[i], b = v[i | h];
                v[i] = a + b;
                v[i | h] = a - b;
            }
}

// cross-lane stages: lane bit k of the L lanes that share a block is index bit 3+k
template <typename A>
__device__ __forceinline__ void fwht_lanes(A (&v)[8], int L, int lane_in_block) {
    for (int o = 1; o < L; o <<= 1) {
        const A sgn = (lane_in_block & o) != 0 ? (A)-1 : (A)1;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            A other = shfl_xor<A>(v[i], o);
            v[i] = fma(sgn, v[i], other);  // other - v in the upper half, v + other in the lower: one exact fma
        }
    }
}

// Sign-bit masks (bit 31 where the +-1 entry is negative) of 8 consecutive entries of the diagonal: multiplying a
// float by +-1 is flipping its sign bit.  One 8-byte load where the address allows it.
__device__ __forceinline__ void sign_masks8(const int8_t *signs, int base, uint32_t (&m)[8]) {
    if (signs == nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) m[i] = 0u;
    } else if ((reinterpret_cast<uintptr_t>(signs) & 7u) == 0) {
        const uint2 w = __ldg(reinterpret_cast<const uint2 *>(signs + base));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            m[i] = (w.x << (24 - 8 * i)) & 0x80000000u;
            m[4 + i] = (w.y << (24 - 8 * i)) & 0x80000000u;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) m[i] = signs[base + i] < 0 ? 0x80000000u : 0u;
    }
}

__device__ __forceinline__ float flip(float v, uint32_t mask) { return __uint_as_float(__float_as_uint(v) ^ mask); }

struct HArgs {
    const void *x;
    const int8_t *signs;
    void *out;        // rotated tensor (plain rotation) or quantized output (fused)
    void *out_scale;  // fused only
    const float *gs;  // fused fp4 only
    int64_t chunks;   // rows * cols / 8
    int n;            // Hadamard size (0 = no rotation, fused calibrate+quantize only)
    int L;            // lanes per Hadamard block = n / 8
    int inverse;
    int normalize;    // divide by sqrt(n) (the reference's HadamardTransform) or leave the raw product
    int GL;           // lanes per quantization group = col_group / 8 (fused)
    int gl_shift;     // log2(GL)
    int xdt;
    float qmin, qmax, half_range;
};

// rotate the 8 values of this lane in place; returns them rounded to the dtype XF of the tensor
template <typename A, int XF>
__device__ __forceinline__ void rotate8(const HArgs &a, int64_t c, float (&v)[8]) {
    const int lane_in_block = (int)(c & (a.L - 1));
    uint32_t sg[8];
    sign_masks8(a.signs, lane_in_block * 8, sg);
    A t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = (A)(a.inverse ? flip(v[i], sg[i]) : v[i]);
    fwht8<A>(t);
    fwht_lanes<A>(t, a.L, lane_in_block);
    if constexpr (sizeof(A) == 8) {
        const double s = a.normalize ? sqrt((double)a.n) : 1.0, rs = 1.0 / s;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (float)div_const<double>(t[i], s, rs);  // float64 quotient, then the cast chain of .to(dtype)
    } else {
        const float s = a.normalize ? 1.0f / sqrtf((float)a.n) : 1.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = t[i] * s;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (!a.inverse) v[i] = flip(v[i], sg[i]);
        v[i] += 0.0f;  // an exact zero comes out of the reference's matmul as +0.0, whatever the signs
        v[i] = round_to<XF == F_BF16 ? CTB_BF16 : XF == F_F16 ? CTB_F16 : CTB_F32>(v[i]);
    }
}

// weight_input rotation: one 8-element chunk per lane
template <typename A, int XF>
__global__ void __launch_bounds__(kThreads, sizeof(A) == 8 ? 5 : 8) hadamard_cols_kernel(const HArgs a) {
    const int64_t padded = (a.chunks + 31) & ~(int64_t)31;
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < padded; c += (int64_t)gridDim.x * kThreads) {
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const bool live = c < a.chunks;
        if (live) {
            Raw8 r = load_raw<XF>(a.x, c);
            decode8<XF>(r, v);
        }
        rotate8<A, XF>(a, c, v);
        if (live) store8_float<XF>(a.out, c, v);
    }
}

// weight_input rotation for n = 512 .. 8192 (a whole hidden dimension): one Hadamard block of n = 256 * M elements
// per thread block.  Index bits 0-2 run in registers and bits 3-7 across the lanes of a warp exactly as in the small
// kernel (a 256-point transform per warp and chunk); the remaining log2(M) bits go through shared memory, where
// thread r gathers the M elements j * 256 + r, runs an M-point butterfly in registers and puts them back.
template <typename A>
__device__ __forceinline__ void smem_put8(A *dst, const A (&t)[8]) {
    if constexpr (sizeof(A) == 8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) reinterpret_cast<double2 *>(dst)[i] = make_double2(t[2 * i], t[2 * i + 1]);
    } else {
        reinterpret_cast<float4 *>(dst)[0] = make_float4(t[0], t[1], t[2], t[3]);
        reinterpret_cast<float4 *>(dst)[1] = make_float4(t[4], t[5], t[6], t[7]);
    }
}

template <typename A>
__device__ __forceinline__ void smem_get8(const A *src, A (&t)[8]) {
    if constexpr (sizeof(A) == 8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) { const double2 d = reinterpret_cast<const double2 *>(src)[i]; t[2 * i] = d.x; t[2 * i + 1] = d.y; }
    } else {
        const float4 a = reinterpret_cast<const float4 *>(src)[0], b = reinterpret_cast<const float4 *>(src)[1];
        t[0] = a.x; t[1] = a.y; t[2] = a.z; t[3] = a.w; t[4] = b.x; t[5] = b.y; t[6] = b.z; t[7] = b.w;
    }
}

template <typename A, int XF, int LOG_M>
__global__ void __launch_bounds__(kThreads) hadamard_cols_big_kernel(const void *x, int64_t blocks, const int8_t *signs, int inverse,
                                                                      int normalize, void *out) {
    constexpr int M = 1 << LOG_M, N = 256 * M, CH = N / 8;  // CH: 8-element chunks per Hadamard block, a multiple of 32
    extern __shared__ __align__(16) unsigned char smem_raw[];
    A *buf = reinterpret_cast<A *>(smem_raw);  // [N]
    const int lane = threadIdx.x & 31;
    for (int64_t b = blockIdx.x; b < blocks; b += gridDim.x) {
        const int64_t c0 = b * CH;
        for (int ci = threadIdx.x; ci < CH; ci += kThreads) {  // whole warps: the lane stages shuffle
            float v[8];
            decode8<XF>(load_raw<XF>(x, c0 + ci), v);
            A t[8];
            if (inverse) {
                uint32_t sg[8];
                sign_masks8(signs, ci * 8, sg);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = flip(v[i], sg[i]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = (A)v[i];
            fwht8<A>(t);
            fwht_lanes<A>(t, 32, lane);
            smem_put8<A>(buf + ci * 8, t);
        }
        __syncthreads();
        {
            A t[M];
#pragma unroll
            for (int j = 0; j < M; ++j) t[j] = buf[j * 256 + threadIdx.x];
#pragma unroll
            for (int h = 1; h < M; h <<= 1)
#pragma unroll
                for (int j = 0; j < M; ++j)
                    if ((j & h) == 0) {
                        const A u = t[j], w = t[j | h];
                        t[j] = u + w;
                        t[j | h] = u - w;
                    }
#pragma unroll
            for (int j = 0; j < M; ++j) buf[j * 256 + threadIdx.x] = t[j];
        }
        __syncthreads();
        for (int ci = threadIdx.x; ci < CH; ci += kThreads) {
            A t[8];
            smem_get8<A>(buf + ci * 8, t);
            float v[8];
            if constexpr (sizeof(A) == 8) {
                const double sc = normalize ? sqrt((double)N) : 1.0, rsc = 1.0 / sc;
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (float)div_const<double>(t[i], sc, rsc);  // float64 quotient, then the cast chain of .to(dtype)
            } else {
                const float sc = normalize ? 1.0f / sqrtf((float)N) : 1.0f;
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = t[i] * sc;
            }
            uint32_t sg[8];
            sign_masks8(inverse ? nullptr : signs, ci * 8, sg);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = flip(v[i], sg[i]);
                v[i] += 0.0f;  // an exact zero comes out of the reference's matmul as +0.0, whatever the signs
                v[i] = round_to<XF == F_BF16 ? CTB_BF16 : XF == F_F16 ? CTB_F16 : CTB_F32>(v[i]);
            }
            store8_float<XF>(out, c0 + ci, v);
        }
        __syncthreads();  // the next block's first phase overwrites the buffer
    }
}

template <typename A, int XF>
static int launch_cols_big(int n, int64_t blocks, const void *x, const int8_t *signs, int inverse, int normalize, void *out, cudaStream_t st) {
    const size_t smem = (size_t)n * sizeof(A);
    const int grid = grid_for(blocks, 1, 4);
#define CTB_HCB(LM_)                                                                                                       \
    {                                                                                                                      \
        cudaFuncSetAttribute(hadamard_cols_big_kernel<A, XF, LM_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        hadamard_cols_big_kernel<A, XF, LM_><<<grid, kThreads, smem, st>>>(x, blocks, signs, inverse, normalize, out);     \
    }
    switch (n) {
    case 512: CTB_HCB(1) break;
    case 1024: CTB_HCB(2) break;
    case 2048: CTB_HCB(3) break;
    case 4096: CTB_HCB(4) break;
    default: CTB_HCB(5) break;
    }
#undef CTB_HCB
    return after_launch("hadamard_cols_big_kernel");
}

// weight_output rotation: a [n rows x W cols] tile per block (W a power of two <= 32, as many as fit in shared memory),
// butterflies over rows in shared memory
template <typename A>
__global__ void __launch_bounds__(kThreads) hadamard_rows_kernel(const void *x, int dt, int64_t rows, int64_t cols, int n, int wshift,
                                                                  const int8_t *signs, int inverse, int normalize, void *out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    A *tile = reinterpret_cast<A *>(smem_raw);  // [n][W + 1]
    const int W = 1 << wshift, pitch = W + 1;
    const int64_t col_tiles = (cols + W - 1) >> wshift, tiles = (rows / n) * col_tiles;
    const A scale = normalize ? (A)sqrt((double)n) : (A)1, rscale = (A)1 / scale;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t tr = t / col_tiles, r0 = tr * n, c0 = (t - tr * col_tiles) << wshift;
        for (int i = threadIdx.x; i < n * W; i += kThreads) {
            int r = i >> wshift, c = i & (W - 1);
            A v = 0;
            if (c0 + c < cols) {
                v = (A)load_f32(x, dt, (r0 + r) * cols + c0 + c);
                if (!inverse && signs) v *= (A)signs[r];
            }
            tile[r * pitch + c] = v;
        }
        __syncthreads();
        for (int h = 1; h < n; h <<= 1) {
            for (int i = threadIdx.x; i < (n / 2) * W; i += kThreads) {
                int p = i >> wshift, c = i & (W - 1);
                int r = ((p & ~(h - 1)) << 1) | (p & (h - 1));  // row with bit h clear
                A u = tile[r * pitch + c], w = tile[(r | h) * pitch + c];
                tile[r * pitch + c] = u + w;
                tile[(r | h) * pitch + c] = u - w;
            }
            __syncthreads();
        }
        for (int i = threadIdx.x; i < n * W; i += kThreads) {
            int r = i >> wshift, c = i & (W - 1);
            if (c0 + c < cols) {
                A v = div_const<A>(tile[r * pitch + c], scale, rscale);
                float f = (float)v;
                if (inverse && signs) f *= (float)signs[r];
                f += 0.0f;  // exact zeros are +0.0 in the reference's matmul
                store_f32(out, dt, (r0 + r) * cols + c0 + c, f);
            }
        }
        __syncthreads();
    }
}

// weight_output rotation for 16-bit tensors and n = 512 .. 8192 (a whole output dimension).  A block takes a tile of
// n rows x W columns (W * 2 bytes of every row), stores it TRANSPOSED in shared memory, so that each column becomes a
// contiguous length-n vector, and then runs the three phases of the wide weight_input kernel on the W vectors:
// 256-point transforms in registers and across lanes, M-point transforms through strided gathers, and the scaled,
// signed, rounded write back.  W is as wide as 128 KiB of shared memory allows.
constexpr int kBigThreads = 512;
constexpr int kRowsBigBytes = 131072;  // most shared memory a tile may take

template <typename A, int LOG_M>
struct RowsBig {
    static constexpr int N = 256 << LOG_M;
    static constexpr int kFit = (kRowsBigBytes / (int)sizeof(A)) / N;
    static constexpr int W = kFit >= 8 ? 8 : kFit >= 2 ? kFit : 2;  // 8, 4 or 2
};

template <typename A, int XF, int LOG_M>
__global__ void __launch_bounds__(kBigThreads) hadamard_rows_big_kernel(const void *x, int64_t rows, int64_t cols, const int8_t *signs,
                                                                         int inverse, int normalize, void *out) {
    constexpr int M = 1 << LOG_M, N = RowsBig<A, LOG_M>::N, W = RowsBig<A, LOG_M>::W, CH = N / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    A *col = reinterpret_cast<A *>(smem_raw);  // [W][N]
    const A sc = normalize ? (A)sqrt((double)N) : (A)1, rsc = (A)1 / sc;
    const int lane = threadIdx.x & 31;
    const int64_t col_tiles = cols / W, tiles = (rows / N) * col_tiles;
    const uint16_t *xin = reinterpret_cast<const uint16_t *>(x);
    uint16_t *xout = reinterpret_cast<uint16_t *>(out);
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t tr = t / col_tiles, r0 = tr * N, c0 = (t - tr * col_tiles) * W;
        // rows of the tile -> columns in shared memory
#pragma unroll 4
        for (int r = threadIdx.x; r < N; r += kBigThreads) {
            const uint16_t *src = xin + (r0 + r) * cols + c0;
            uint32_t w[W / 2];
            if constexpr (W == 8) { const uint4 q = ld_stream(src); w[0] = q.x; w[1] = q.y; w[2] = q.z; w[3] = q.w; }
            else if constexpr (W == 4) { const uint2 q = ld_stream8(src); w[0] = q.x; w[1] = q.y; }
            else { w[0] = ld_stream4(src); }
            const float sg = (!inverse && signs) ? (float)signs[r] : 1.0f;
#pragma unroll
            for (int k = 0; k < W / 2; ++k) {
                float lo, hi;
                if constexpr (XF == F_BF16) { lo = __uint_as_float(w[k] << 16); hi = __uint_as_float(w[k] & 0xFFFF0000u); }
                else { const float2 f = half2_bits_to_float2(w[k]); lo = f.x; hi = f.y; }
                col[(2 * k) * N + r] = (A)(lo * sg);
                col[(2 * k + 1) * N + r] = (A)(hi * sg);
            }
        }
        __syncthreads();
        for (int q = threadIdx.x; q < W * CH; q += kBigThreads) {  // whole warps; a chunk never straddles two columns
            A v[8];
            smem_get8<A>(col + q * 8, v);
            fwht8<A>(v);
            fwht_lanes<A>(v, 32, lane);
            smem_put8<A>(col + q * 8, v);
        }
        __syncthreads();
        for (int q = threadIdx.x; q < W * 256; q += kBigThreads) {
            A *base = col + (q >> 8) * N + (q & 255);
            A v[M];
#pragma unroll
            for (int j = 0; j < M; ++j) v[j] = base[j * 256];
#pragma unroll
            for (int h = 1; h < M; h <<= 1)
#pragma unroll
                for (int j = 0; j < M; ++j)
                    if ((j & h) == 0) {
                        const A u = v[j], w2 = v[j | h];
                        v[j] = u + w2;
                        v[j | h] = u - w2;
                    }
#pragma unroll
            for (int j = 0; j < M; ++j) base[j * 256] = v[j];
        }
        __syncthreads();
#pragma unroll 4
        for (int r = threadIdx.x; r < N; r += kBigThreads) {
            const float sg = (inverse && signs) ? (float)signs[r] : 1.0f;
            uint32_t w[W / 2];
#pragma unroll
            for (int k = 0; k < W / 2; ++k) {
                float f[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const A v = col[(2 * k + e) * N + r];
                    f[e] = (float)div_const<A>(v, sc, rsc);
                    f[e] = f[e] * sg + 0.0f;  // exact zeros are +0.0 in the reference's matmul
                }
                if constexpr (XF == F_BF16) { const __nv_bfloat162 h = __floats2bfloat162_rn(f[0], f[1]); w[k] = *reinterpret_cast<const uint32_t *>(&h); }
                else { const __half2 h = __floats2half2_rn(f[0], f[1]); w[k] = *reinterpret_cast<const uint32_t *>(&h); }
            }
            uint16_t *dst = xout + (r0 + r) * cols + c0;
            if constexpr (W == 8) st_stream(dst, make_uint4(w[0], w[1], w[2], w[3]));
            else if constexpr (W == 4) st_stream8(dst, make_uint2(w[0], w[1]));
            else st_stream4(dst, w[0]);
        }
        __syncthreads();
    }
}

template <typename A, int XF>
static int launch_rows_big(int n, const void *x, int64_t rows, int64_t cols, const int8_t *signs, int inverse, int normalize, void *out,
                           cudaStream_t st) {
#define CTB_HRB(LM_)                                                                                                        \
    {                                                                                                                       \
        const int smem = RowsBig<A, LM_>::N * RowsBig<A, LM_>::W * (int)sizeof(A);                                          \
        const int grid = grid_for((rows / n) * (cols / RowsBig<A, LM_>::W), 1, std::min(4, std::max(1, 200 * 1024 / smem)));                                          \
        cudaFuncSetAttribute(hadamard_rows_big_kernel<A, XF, LM_>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);      \
        hadamard_rows_big_kernel<A, XF, LM_><<<grid, kBigThreads, smem, st>>>(x, rows, cols, signs, inverse, normalize, out); \
    }
    switch (n) {
    case 512: CTB_HRB(1) break;
    case 1024: CTB_HRB(2) break;
    case 2048: CTB_HRB(3) break;
    case 4096: CTB_HRB(4) break;
    default: CTB_HRB(5) break;
    }
#undef CTB_HRB
    return after_launch("hadamard_rows_big_kernel");
}

// tile width of the wide weight_output kernel for a Hadamard size and accumulator
static int rows_big_width(int n, bool f64) {
    const int fit = (kRowsBigBytes / (f64 ? 8 : 4)) / n;
    return fit >= 8 ? 8 : fit >= 2 ? fit : 2;
}

// weight_output rotation for 16-bit tensors and n = 32 .. 256: the butterflies run over ROWS, so a column is an
// independent length-n transform.  A block takes a tile of n rows x 32*CPT columns; a warp owns a strip of 4*CPT
// columns of it.  Row index bits 0-1 and 5+ of a lane's values live in registers, bits 2-4 across lanes
// (lane = 4 * bits[2..4] + column part), so three of the log2(n) stages are shuffles and the rest register
// arithmetic; every load instruction of a warp touches 8 rows x 32 (16) contiguous bytes and the block as a whole
// 256 (128) contiguous bytes of each row.  CPT = 4 columns per lane in float, 2 in double (register budget).
// Arithmetic and its order of roundings are those of hadamard_rows_kernel: signs before the transform (forward) or
// after it (inverse), quotient by sqrt(n) correctly rounded in A, cast chain A -> float -> tensor dtype, +0.0.
template <typename A, int XF, int LOG_HI>
__global__ void __launch_bounds__(kThreads) hadamard_rows_fast_kernel(const void *x, int64_t rows, int64_t cols, const int8_t *signs, int inverse,
                                                                       int normalize, void *out) {
    constexpr int CPT = sizeof(A) == 8 ? 2 : 4, HI = 1 << LOG_HI, N = 32 * HI, TILE_COLS = 32 * CPT;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, r_mid = lane >> 2, cpart = lane & 3;
    const int64_t col_tiles = (cols + TILE_COLS - 1) / TILE_COLS, tiles = (rows / N) * col_tiles;
    // x / sqrt(N): exact reciprocal multiply when sqrt(N) is a power of two, otherwise reciprocal + one Markstein
    // correction, which gives the correctly rounded quotient (the operands are far from the overflow / underflow ends)
    const A sc = normalize ? (A)sqrt((double)N) : (A)1, rsc = (A)1 / sc;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t tr = t / col_tiles, r0 = tr * N, c = (t - tr * col_tiles) * TILE_COLS + (warp * 4 + cpart) * CPT;
        const bool live = c < cols;
        A v[HI][4][CPT];
#pragma unroll
        for (int hi = 0; hi < HI; ++hi)
#pragma unroll
            for (int lo = 0; lo < 4; ++lo) {
                const int rr = lo + 4 * r_mid + 32 * hi;
                uint32_t w[2] = {0, 0};
                if (live) {
                    const char *p = (const char *)x + ((r0 + rr) * cols + c) * 2;
                    if constexpr (CPT == 4) {
                        const uint2 q = ld_stream8(p);
                        w[0] = q.x;
                        w[1] = q.y;
                    } else {
                        w[0] = ld_stream4(p);
                    }
                }
                const A sg = (!inverse && signs) ? (A)signs[rr] : (A)1;
#pragma unroll
                for (int k = 0; k < CPT; ++k) {
                    const uint32_t bits = (w[k >> 1] >> (16 * (k & 1))) & 0xFFFFu;
                    const float f = XF == F_BF16 ? __uint_as_float(bits << 16) : __half2float(__ushort_as_half((unsigned short)bits));
                    v[hi][lo][k] = (A)f * sg;
                }
            }
        // register stages: row bits 0, 1 (lo) and 5.. (hi)
#pragma unroll
        for (int h = 1; h < 4; h <<= 1)
#pragma unroll
            for (int hi = 0; hi < HI; ++hi)
#pragma unroll
                for (int lo = 0; lo < 4; ++lo)
                    if ((lo & h) == 0)
#pragma unroll
                        for (int k = 0; k < CPT; ++k) {
                            const A a = v[hi][lo][k], b = v[hi][lo | h][k];
                            v[hi][lo][k] = a + b;
                            v[hi][lo | h][k] = a - b;
                        }
#pragma unroll
        for (int h = 1; h < HI; h <<= 1)
#pragma unroll
            for (int hi = 0; hi < HI; ++hi)
                if ((hi & h) == 0)
#pragma unroll
                    for (int lo = 0; lo < 4; ++lo)
#pragma unroll
                        for (int k = 0; k < CPT; ++k) {
                            const A a = v[hi][lo][k], b = v[hi | h][lo][k];
                            v[hi][lo][k] = a + b;
                            v[hi | h][lo][k] = a - b;
                        }
        // shuffle stages: row bits 2, 3, 4 = lane bits 2, 3, 4
#pragma unroll
        for (int m = 4; m < 32; m <<= 1) {
            const A sgn = (lane & m) != 0 ? (A)-1 : (A)1;
#pragma unroll
            for (int hi = 0; hi < HI; ++hi)
#pragma unroll
                for (int lo = 0; lo < 4; ++lo)
#pragma unroll
                    for (int k = 0; k < CPT; ++k) {
                        const A mine = v[hi][lo][k], other = rq_shfl_xor<A>(mine, m);
                        v[hi][lo][k] = fma(sgn, mine, other);  // other - mine in the upper half, mine + other in the lower
                    }
        }
        if (!live) continue;
#pragma unroll
        for (int hi = 0; hi < HI; ++hi)
#pragma unroll
            for (int lo = 0; lo < 4; ++lo) {
                const int rr = lo + 4 * r_mid + 32 * hi;
                const float sg = (inverse && signs) ? (float)signs[rr] : 1.0f;
                uint32_t bits[CPT];
#pragma unroll
                for (int k = 0; k < CPT; ++k) {
                    const A tv = v[hi][lo][k];
                    A q = tv * rsc;
                    if constexpr (sizeof(A) == 8) q = fma(fma(-q, sc, tv), rsc, q);
                    else q = fmaf(fmaf(-q, sc, tv), rsc, q);
                    float f = (float)q * sg + 0.0f;  // exact zeros are +0.0 in the reference's matmul
                    bits[k] = XF == F_BF16 ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f)) : (uint32_t)__half_as_ushort(__float2half_rn(f));
                }
                char *p = (char *)out + ((r0 + rr) * cols + c) * 2;
                if constexpr (CPT == 4) st_stream8(p, make_uint2(bits[0] | (bits[1] << 16), bits[2] | (bits[3] << 16)));
                else st_stream4(p, bits[0] | (bits[1] << 16));
            }
    }
}

}  // namespace ctb

// ------------------------------------------------------------------ fused calibrate + quantize + pack

namespace ctb {

// symmetric scale of one group from its absolute maximum, helpers.py:99-122, in the dtype M of the
// tensor; returns the effective fp32 scale used by the quantize step and stores the qparam.
template <int M, int QK>
__device__ __forceinline__ float group_scale(float amax, float g, float rg, float half_range, float r_half, void *out_scale, int64_t gi, bool writer) {
    if constexpr (QK == QK_FP4) {
        // g = global scale, rg = 1 / g (both fp32); quotients by constants are correctly rounded (Markstein)
        float sc = g * round_to<M>(div_by_rcp(amax, 6.0f, 0.16666667163372040f));
        sc = clamp_nan(sc, -448.0f, 448.0f);  // NaN (all-zero tensor: inf * 0) stays NaN, as in the reference
        uint8_t b = f32_to_e4m3(sc);
        if ((b & 0x7F) == 0) b = 0x20;  // zero scale -> 0.125
        if (writer) ((uint8_t *)out_scale)[gi] = b;
        return div_by_rcp(e4m3_to_f32(b), g, rg);  // forward.py:468-469 scale.to(f32) / global_scale
    } else {
        float sc = fmaxf(round_to<M>(div_by_rcp(amax, half_range, r_half)), 1.1920928955078125e-07f);
        if (writer) store_f32(out_scale, M, gi, sc);
        return sc;
    }
}

// max |x| over 8 bf16 values held as four packed words (NaNs are skipped, as fmaxf skips them)
__device__ __forceinline__ __nv_bfloat162 amax2_bf16(const uint4 &w) {
    const __nv_bfloat162 a = __hmax2(__habs2(u32_as_bf162(w.x)), __habs2(u32_as_bf162(w.y)));
    const __nv_bfloat162 b = __hmax2(__habs2(u32_as_bf162(w.z)), __habs2(u32_as_bf162(w.w)));
    return __hmax2(a, b);
}
__device__ __forceinline__ float amax_of_pair(__nv_bfloat162 m) {
    const uint32_t u = bf162_as_u32(m);
    return fmaxf(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}

// W4A16 with groups of 128 on a bf16 weight, no rotation: calibrate + quantize + pack_to_int32 in one pass
// (quantization/utils/helpers.py:110-122 for the scale, lifecycle/forward.py:420-448 for the codes,
// compressors/quantized_compressors/pack_quantized.py:221 for the packing).  Two neighbouring lanes own a group:
// lane half h holds the 16-byte chunks 2a + h (a = 0..7), so the pair reads 32 contiguous bytes per step, the
// maximum stays in packed bf16 registers and the scale is computed once per 64 elements of a lane.
__global__ void __launch_bounds__(kThreads) absmax_quant_g128_int4_kernel(const void *x, void *out, void *scale, int64_t ngroups) {
    const int h = threadIdx.x & 1;
    const int ppb = blockDim.x >> 1;  // pairs per block
    const int64_t pairs = (int64_t)gridDim.x * ppb;
    const int64_t padded = (ngroups + 15) & ~(int64_t)15;  // whole warps stay in the loop for the shuffles
    for (int64_t g = (int64_t)blockIdx.x * ppb + (threadIdx.x >> 1); g < padded; g += pairs) {
        const bool live = g < ngroups;
        uint4 raw[8];
#pragma unroll
        for (int a = 0; a < 8; ++a) raw[a] = live ? ld_stream((const char *)x + (g * 16 + 2 * a + h) * 16) : make_uint4(0, 0, 0, 0);
        __nv_bfloat162 m2 = amax2_bf16(raw[0]);
#pragma unroll
        for (int a = 1; a < 8; ++a) m2 = __hmax2(m2, amax2_bf16(raw[a]));
        float amax = amax_of_pair(m2);
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
        // scale = bf16(amax / 7.5) clamped at fp32 eps
        const float s = fmaxf(round_to<CTB_BF16>(__fdiv_rn(amax, 7.5f)), 1.1920928955078125e-07f);
        const float r = __frcp_rn(s);
        if (live && h == 0) ((__nv_bfloat16 *)scale)[g] = __float2bfloat16_rn(s);
        uint32_t word[8];
#pragma unroll
        for (int a = 0; a < 8; ++a) {
            const uint32_t w[4] = {raw[a].x, raw[a].y, raw[a].z, raw[a].w};
            word[a] = quant_int4_word_bf16(w, r, false, u32_as_bf162(0u));
        }
        // word[a] is output word 2a + h of the group's 16.  Swap so that half 0 owns words 0..7 and half 1 words
        // 8..15, then two 16-byte stores per lane.
        uint32_t mine[8];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const uint32_t send = h ? word[a] : word[a + 4];
            const uint32_t got = __shfl_xor_sync(0xFFFFFFFFu, send, 1);
            const uint32_t keep = h ? word[a + 4] : word[a];
            mine[2 * a] = h ? got : keep;      // even word of the pair comes from half 0
            mine[2 * a + 1] = h ? keep : got;  // odd word from half 1
        }
        if (live) {
            char *o = (char *)out + g * 64 + h * 32;
            st_stream(o, make_uint4(mine[0], mine[1], mine[2], mine[3]));
            st_stream(o + 16, make_uint4(mine[4], mine[5], mine[6], mine[7]));
        }
    }
}

// groups of 8*GL consecutive elements (GL lanes, power of two <= 32), optional Hadamard in front.
// A = float / double selects the rotation precision; ROT = false skips the rotation.
template <typename A, bool ROT, int XF, int QK, int FOUT>
__global__ void __launch_bounds__(kThreads) absmax_quant_group_kernel(const HArgs a) {
    constexpr int M = XF == F_BF16 ? CTB_BF16 : XF == F_F16 ? CTB_F16 : CTB_F32;
    constexpr int T = QK == QK_FP4 ? CTB_F32 : M;
    constexpr int U = ROT ? 1 : 4;  // chunks in flight per thread
    const float gsv = (QK == QK_FP4) ? __ldg(a.gs) : 1.0f, rgs = __frcp_rn(gsv), r_half = __frcp_rn(a.half_range);
    const int64_t padded = (a.chunks + 31) & ~(int64_t)31;  // whole warps stay in the loop for the shuffles
    const int64_t stride = (int64_t)gridDim.x * kThreads * U;
    for (int64_t base = (int64_t)blockIdx.x * kThreads * U + threadIdx.x; base - threadIdx.x + (threadIdx.x & ~31) < padded; base += stride) {
        Raw8 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t c = base + (int64_t)u * kThreads;
            raw[u].a = make_uint4(0, 0, 0, 0);
            if (c < a.chunks) raw[u] = load_raw<XF>(a.x, c);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t c = base + (int64_t)u * kThreads;
            const bool live = c < a.chunks;
            float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            float amax = 0.0f;
            constexpr bool kPackedMax = XF == F_BF16 && !ROT;  // the maximum straight from the packed words
            if constexpr (kPackedMax) {
                amax = amax_of_pair(amax2_bf16(raw[u].a));
            } else {
                if (live) decode8<XF>(raw[u], v);
                if constexpr (ROT) rotate8<A, XF>(a, c, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            }
            for (int o = a.GL >> 1; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
            QP q;
            q.s = group_scale<M, QK>(amax, gsv, rgs, a.half_range, r_half, a.out_scale, c >> a.gl_shift, live && (c & (a.GL - 1)) == 0);
            q.r = __frcp_rn(q.s);
            q.zp = 0.0f;
            q.slow = !(fabsf(q.s) >= 1.0e-30f && fabsf(q.s) <= 1.0e30f);
            if constexpr (XF == F_BF16 && QK == QK_FP4 && FOUT == F_FP4X2 && !ROT) {
                // finite group (amax < inf) and a scale in the normal range: reciprocal + Markstein, saturating e2m1 convert
                if (!q.slow && amax <= 3.0e38f) {
                    const uint32_t w[4] = {raw[u].a.x, raw[u].a.y, raw[u].a.z, raw[u].a.w};
                    if (live) st_stream4((char *)a.out + c * 4, quant_fp4_codes_f32(w, q.s, q.r));
                    continue;
                }
            }
            if constexpr (XF == F_BF16 && ((QK == QK_INT && FOUT == F_PACK4) || (QK == QK_FP8 && FOUT == F_E4M3))) {
                if (!q.slow) {
                    uint32_t w[4];
                    if constexpr (ROT) {  // v[] hold bf16 values exactly, so re-packing them is lossless
#pragma unroll
                        for (int k = 0; k < 4; ++k) w[k] = bf162_as_u32(__floats2bfloat162_rn(v[2 * k], v[2 * k + 1]));
                    } else {
                        w[0] = raw[u].a.x; w[1] = raw[u].a.y; w[2] = raw[u].a.z; w[3] = raw[u].a.w;
                    }
                    if constexpr (QK == QK_INT) {
                        if (live) st_stream4((char *)a.out + c * 4, quant_int4_word_bf16(w, q.r, false, __float2bfloat162_rn(0.0f)));
                    } else {
                        if (live) st_stream8((char *)a.out + c * 8, quant_fp8_codes_bf16(w, q.r));
                    }
                    continue;
                }
            }
            if constexpr (XF == F_BF16 && FOUT == F_BF16 && !ROT) {  // dynamic fake quantize, packed bf16x2 arithmetic
                if (!q.slow) {
                    const uint32_t w[4] = {raw[u].a.x, raw[u].a.y, raw[u].a.z, raw[u].a.w};
                    uint32_t o[4];
                    if constexpr (QK == QK_INT) {
                        const __nv_bfloat162 lo2 = __float2bfloat162_rn(a.qmin), hi2 = __float2bfloat162_rn(a.qmax);
                        const __nv_bfloat162 s2 = u32_as_bf162((__float_as_uint(q.s) >> 16) * 0x00010001u), z2 = u32_as_bf162(0u);
#pragma unroll
                        for (int j = 0; j < 4; ++j) o[j] = fake_int_pair_bf16(w[j], q.r, true, z2, lo2, hi2, s2);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) o[j] = fake_fp8_pair_bf16(w[j], q.r, true, q.s);
                    }
                    if (live) st_stream((char *)a.out + c * 16, make_uint4(o[0], o[1], o[2], o[3]));
                    continue;
                }
            }
            // the zero point calculate_qparams returns is all zeros; adding it matters only for the sign of an
            // fp8 zero (-0.0 + 0.0 = +0.0) and of a fake-quantized zero
            if constexpr (kPackedMax) {
                if (live) decode8<XF>(raw[u], v);
            }
            if constexpr (FOUT == F_BF16) {
                quant_prepare8<T>(v, q, true, 0.0f, a.qmin, a.qmax);
                round8<QK>(v);
                dequant8<M>(v, q, true);
                if (live) store8_float<F_BF16>(a.out, c, v);
            } else {
                quant_prepare8<T>(v, q, QK == QK_FP8, 0.0f, a.qmin, a.qmax);
                if (live) encode_store8<QK, FOUT>(a.out, c, v);
            }
        }
    }
}

// NVFP4 (groups of 16, e4m3 group scales under an fp32 global scale) on a bf16 tensor: one lane owns a group, so
// the maximum needs no shuffle, the scale chain (e4m3 round trip, two corrected divisions, one reciprocal) runs
// once per 16 elements, and a lane moves 32 contiguous bytes in and 8 + 1 out.  Two groups in flight per lane.
__global__ void __launch_bounds__(kThreads) absmax_quant_g16_fp4_kernel(const HArgs a, int64_t ngroups) {
    constexpr int U = 2;
    const float gsv = __ldg(a.gs), rgs = __frcp_rn(gsv), r_half = __frcp_rn(a.half_range);
    const int64_t stride = (int64_t)gridDim.x * kThreads * U;
    for (int64_t base = (int64_t)blockIdx.x * kThreads * U + threadIdx.x; base < ngroups; base += stride) {
        uint4 raw[U][2];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t g = base + (int64_t)u * kThreads;
            raw[u][0] = raw[u][1] = make_uint4(0, 0, 0, 0);
            if (g < ngroups) {
                // a lane's two halves share a 32-byte sector: let L1 keep it between the two instructions
                raw[u][0] = __ldg(reinterpret_cast<const uint4 *>((const char *)a.x + g * 32));
                raw[u][1] = __ldg(reinterpret_cast<const uint4 *>((const char *)a.x + g * 32 + 16));
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t g = base + (int64_t)u * kThreads;
            if (g >= ngroups) break;
            const float amax = amax_of_pair(__hmax2(amax2_bf16(raw[u][0]), amax2_bf16(raw[u][1])));
            QP q;
            q.s = group_scale<CTB_BF16, QK_FP4>(amax, gsv, rgs, a.half_range, r_half, a.out_scale, g, true);
            q.r = __frcp_rn(q.s);
            q.zp = 0.0f;
            q.slow = !(fabsf(q.s) >= 1.0e-30f && fabsf(q.s) <= 1.0e30f);
            if (!q.slow && amax <= 3.0e38f) {
                // finite group and a scale in the normal range: reciprocal + Markstein, saturating e2m1 convert
                const uint32_t w0[4] = {raw[u][0].x, raw[u][0].y, raw[u][0].z, raw[u][0].w};
                const uint32_t w1[4] = {raw[u][1].x, raw[u][1].y, raw[u][1].z, raw[u][1].w};
                st_stream8((char *)a.out + g * 8, make_uint2(quant_fp4_codes_f32(w0, q.s, q.r), quant_fp4_codes_f32(w1, q.s, q.r)));
                continue;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                Raw8 r8;
                r8.a = raw[u][h];
                float v[8];
                decode8<F_BF16>(r8, v);
                quant_prepare8<CTB_F32>(v, q, false, 0.0f, a.qmin, a.qmax);
                encode_store8<QK_FP4, F_FP4X2>(a.out, g * 2 + h, v);
            }
        }
    }
}

// one warp per row, the whole row in registers (CHANNEL / TOKEN with cols <= 8 * 32 * CPL): a single pass with
// no shared memory and no block barrier.  CPL = 16-byte chunks per lane.
template <int CPL, int XF, int QK, int FOUT>
__global__ void __launch_bounds__(kThreads) absmax_quant_warprow_kernel(const HArgs a, int64_t rows, int cpr) {
    constexpr int M = XF == F_BF16 ? CTB_BF16 : XF == F_F16 ? CTB_F16 : CTB_F32;
    const int lane = threadIdx.x & 31;
    const float r_half = __frcp_rn(a.half_range);
    const int wpb = blockDim.x >> 5;  // launched with 128 or 256 threads: the block is only a bundle of independent warps
    const int64_t warps = (int64_t)gridDim.x * wpb;
    for (int64_t r = (int64_t)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += warps) {
        Raw8 raw[CPL];
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
            const int c = k * 32 + lane;
            if (c < cpr) raw[k] = load_raw<XF>(a.x, r * cpr + c);
        }
        float amax = 0.0f;
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
            if (k * 32 + lane < cpr) {
                float v[8];
                decode8<XF>(raw[k], v);
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            }
        }
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        QP q;
        q.s = group_scale<M, QK>(amax, 1.0f, 1.0f, a.half_range, r_half, a.out_scale, r, lane == 0);
        q.r = __frcp_rn(q.s);
        q.zp = 0.0f;
        q.slow = !(fabsf(q.s) >= 1.0e-30f && fabsf(q.s) <= 1.0e30f);
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
            const int c = k * 32 + lane;
            if (c < cpr) {
                if constexpr (QK == QK_FP8 && XF == F_BF16 && FOUT == F_E4M3) {
                    if (!q.slow) {
                        const uint32_t w[4] = {raw[k].a.x, raw[k].a.y, raw[k].a.z, raw[k].a.w};
                        st_stream8((char *)a.out + (r * cpr + c) * 8, quant_fp8_codes_bf16(w, q.r));
                        continue;
                    }
                }
                if constexpr (FOUT == F_BF16 && XF == F_BF16) {
                    if (!q.slow) {  // packed bf16x2 arithmetic; the scale is a bf16 value, so its top half is all of it
                        const uint32_t w[4] = {raw[k].a.x, raw[k].a.y, raw[k].a.z, raw[k].a.w};
                        uint32_t o[4];
                        if constexpr (QK == QK_INT) {
                            const __nv_bfloat162 lo2 = __float2bfloat162_rn(a.qmin), hi2 = __float2bfloat162_rn(a.qmax);
                            const __nv_bfloat162 s2 = u32_as_bf162((__float_as_uint(q.s) >> 16) * 0x00010001u), z2 = u32_as_bf162(0u);
#pragma unroll
                            for (int j = 0; j < 4; ++j) o[j] = fake_int_pair_bf16(w[j], q.r, true, z2, lo2, hi2, s2);
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) o[j] = fake_fp8_pair_bf16(w[j], q.r, true, q.s);
                        }
                        st_stream((char *)a.out + (r * cpr + c) * 16, make_uint4(o[0], o[1], o[2], o[3]));
                        continue;
                    }
                }
                float v[8];
                decode8<XF>(raw[k], v);
                if constexpr (FOUT == F_BF16) {
                    // dynamic fake quantize (forward.py:157-189 with the all-zero zero point calculate_qparams returns for a
                    // symmetric scheme): x / s + 0, clamp, round to the grid, (q - 0) * s, every step in the tensor dtype
                    quant_prepare8<M>(v, q, true, 0.0f, a.qmin, a.qmax);
                    round8<QK>(v);
                    dequant8<M>(v, q, true);
                    store8_float<F_BF16>(a.out, r * cpr + c, v);
                } else {
                    quant_prepare8<M>(v, q, QK == QK_FP8, 0.0f, a.qmin, a.qmax);
                    encode_store8<QK, FOUT>(a.out, r * cpr + c, v);
                }
            }
        }
    }
}

// one block per row (CHANNEL / TOKEN): first sweep finds the row's absolute maximum, second sweep
// re-reads the row (it is still in L1/L2) and quantizes it.
template <int XF, int QK, int FOUT>
__global__ void __launch_bounds__(kThreads) absmax_quant_row_kernel(const HArgs a, int64_t rows, int64_t cpr) {
    constexpr int M = XF == F_BF16 ? CTB_BF16 : XF == F_F16 ? CTB_F16 : CTB_F32;
    __shared__ float red[kThreads / 32];
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        float amax = 0.0f;
        for (int64_t c = threadIdx.x; c < cpr; c += kThreads) {
            const uint4 *p = reinterpret_cast<const uint4 *>((const char *)a.x + (r * cpr + c) * chunk_bytes(XF));
            Raw8 raw;
            raw.a = p[0];
            if constexpr (XF == F_F32) raw.b = p[1];
            float v[8];
            decode8<XF>(raw, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        }
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) amax = fmaxf(amax, red[i]);
        QP q;
        q.s = group_scale<M, QK>(amax, 1.0f, 1.0f, a.half_range, __frcp_rn(a.half_range), a.out_scale, r, threadIdx.x == 0);
        q.r = __frcp_rn(q.s);
        q.zp = 0.0f;
        q.slow = !(fabsf(q.s) >= 1.0e-30f && fabsf(q.s) <= 1.0e30f);
        for (int64_t c = threadIdx.x; c < cpr; c += kThreads) {
            Raw8 raw = load_raw<XF>(a.x, r * cpr + c);
            if constexpr (QK == QK_FP8 && XF == F_BF16 && FOUT == F_E4M3) {
                if (!q.slow) {
                    const uint32_t w[4] = {raw.a.x, raw.a.y, raw.a.z, raw.a.w};
                    st_stream8((char *)a.out + (r * cpr + c) * 8, quant_fp8_codes_bf16(w, q.r));
                    continue;
                }
            }
            float v[8];
            decode8<XF>(raw, v);
            quant_prepare8<M>(v, q, QK == QK_FP8, 0.0f, a.qmin, a.qmax);
            encode_store8<QK, FOUT>(a.out, r * cpr + c, v);
        }
    }
}

}  // namespace ctb

// ------------------------------------------------------------------ entry points

namespace ctb {

int rotquant_tc_launch(const ctb_tensor_ref *tensors, int32_t count, const int8_t *signs, bool quant, int32_t *status, cudaStream_t st,
                       long long spin_cycles = 0, int skip_tile = -1);

// launch the batched block-128 kernel over `B` (already filled except for nothing: starts, counts, pointers)
static int launch_rotquant(const RQBatch &B, const int8_t *signs, int precision, bool quant, cudaStream_t st) {
    const int64_t total = B.start[B.count];
    if (total == 0) return CTB_OK;
    int grid = grid_for(total, kRQThreads / 2, precision == CTB_F64 ? 2 : 4);
    if (precision == CTB_F64) {
        if (quant) rotquant128_kernel<double, true><<<grid, kRQThreads, 0, st>>>(B, signs);
        else rotquant128_kernel<double, false><<<grid, kRQThreads, 0, st>>>(B, signs);
    } else {
        if (quant) rotquant128_kernel<float, true><<<grid, kRQThreads, 0, st>>>(B, signs);
        else rotquant128_kernel<float, false><<<grid, kRQThreads, 0, st>>>(B, signs);
    }
    return after_launch("rotquant128_kernel");
}

static void rq_single(RQBatch &B, const void *x, void *out, void *scale, int64_t nblocks) {
    B.count = 1;
    B.start[0] = 0;
    B.start[1] = (nblocks + 15) & ~(int64_t)15;
    B.nblocks[0] = nblocks;
    B.x[0] = x;
    B.out[0] = out;
    B.scale[0] = scale;
}

}  // namespace ctb

using namespace ctb;

static bool pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }

extern "C" int ctb_hadamard(const void *x, int32_t dtype, int64_t rows, int64_t cols, int32_t n, const int8_t *signs, int32_t inverse,
                            int32_t side, int32_t precision, int32_t normalize, void *out, void *stream) {
    if (rows != 0 && cols != 0 && (!x || !out)) return fail(CTB_EINVAL_NULL, "null buffer");  // an empty tensor has no storage
    if (!is_float_dtype(dtype)) return fail(CTB_EINVAL_DTYPE, "weights must be bf16, f16 or f32");
    if (!pow2(n)) return fail(CTB_EUNSUPPORTED, "only Sylvester sizes (powers of two) are built");
    if (precision != CTB_F64 && precision != CTB_F32 && precision != CTB_ROT_TENSOR) return fail(CTB_EINVAL_DTYPE, "precision must be F64, F32 or CTB_ROT_TENSOR");
    if (rows < 0 || cols < 0) return fail(CTB_EINVAL_SHAPE, "negative shape");
    if (rows == 0 || cols == 0) return CTB_OK;
    cudaStream_t st = as_stream(stream);
    if (side == 0) {
        if (cols % n) return fail(CTB_EINVAL_SHAPE, "columns %lld are not a multiple of the Hadamard size %d", (long long)cols, n);
        if (precision == CTB_ROT_TENSOR) {
            if (!(n == 128 && dtype == CTB_BF16 && !inverse && normalize)) return fail(CTB_EUNSUPPORTED, "the tensor-core rotation is built for n = 128, bf16, forward, normalised");
            ctb_tensor_ref t{x, out, nullptr, rows, cols};
            return rotquant_tc_launch(&t, 1, signs, false, nullptr, st);
        }
        if (n == 128 && dtype == CTB_BF16 && !inverse && normalize && aligned16(x) && aligned16(out)) {
            static thread_local RQBatch B;
            rq_single(B, x, out, nullptr, rows * cols / 128);
            return launch_rotquant(B, signs, precision, false, st);
        }
        if (n >= 8 && n <= 256 && aligned16(x) && aligned16(out)) {
            HArgs a{};
            a.x = x; a.signs = signs; a.out = out; a.chunks = rows * cols / 8; a.n = n; a.L = n / 8; a.inverse = inverse; a.normalize = normalize; a.xdt = dtype;
            // whole waves of resident blocks: 8 per SM at 32 registers (fp32), 5 at 48 (fp64)
            int grid = grid_for(a.chunks, kThreads, precision == CTB_F64 ? 10 : 8);
#define CTB_HC(A_)                                                                                   \
    if (dtype == CTB_BF16) hadamard_cols_kernel<A_, F_BF16><<<grid, kThreads, 0, st>>>(a);            \
    else if (dtype == CTB_F16) hadamard_cols_kernel<A_, F_F16><<<grid, kThreads, 0, st>>>(a);         \
    else hadamard_cols_kernel<A_, F_F32><<<grid, kThreads, 0, st>>>(a);
            if (precision == CTB_F64) { CTB_HC(double) } else { CTB_HC(float) }
            return after_launch("hadamard_cols_kernel");
        }
        if (n >= 512 && n <= 8192 && aligned16(x) && aligned16(out)) {
            const int64_t blocks = rows * cols / n;
#define CTB_HCB_DT(A_)                                                                                                   \
    if (dtype == CTB_BF16) return launch_cols_big<A_, F_BF16>(n, blocks, x, signs, inverse, normalize, out, st);         \
    else if (dtype == CTB_F16) return launch_cols_big<A_, F_F16>(n, blocks, x, signs, inverse, normalize, out, st);      \
    else return launch_cols_big<A_, F_F32>(n, blocks, x, signs, inverse, normalize, out, st);
            if (precision == CTB_F64) { CTB_HCB_DT(double) } else { CTB_HCB_DT(float) }
        }
        return fail(CTB_EUNSUPPORTED, "weight_input rotation needs 8 <= n <= 8192 and 16-byte aligned buffers");
    }
    if (side != 1) return fail(CTB_EINVAL_SHAPE, "side must be 0 (weight_input) or 1 (weight_output)");
    if (rows % n) return fail(CTB_EINVAL_SHAPE, "rows %lld are not a multiple of the Hadamard size %d", (long long)rows, n);
    if (n > 8192) return fail(CTB_EUNSUPPORTED, "weight_output rotation is built for n <= 8192");
    if ((dtype == CTB_BF16 || dtype == CTB_F16) && (n == 32 || n == 64 || n == 128 || n == 256) && cols % 4 == 0 &&
        (reinterpret_cast<uintptr_t>(x) & 7u) == 0 && (reinterpret_cast<uintptr_t>(out) & 7u) == 0) {
        const bool f64 = precision == CTB_F64;
        const int tile_cols = f64 ? 64 : 128;
        const int fgrid = grid_for((rows / n) * cdiv(cols, tile_cols), 1, n <= 64 ? 4 : 2);
#define CTB_HR(A_, XF_, LH_) hadamard_rows_fast_kernel<A_, XF_, LH_><<<fgrid, kThreads, 0, st>>>(x, rows, cols, signs, inverse, normalize, out)
#define CTB_HR_N(A_, XF_)                                   \
    if (n == 32) CTB_HR(A_, XF_, 0);                        \
    else if (n == 64) CTB_HR(A_, XF_, 1);                   \
    else if (n == 128) CTB_HR(A_, XF_, 2);                  \
    else CTB_HR(A_, XF_, 3);
        if (f64) {
            if (dtype == CTB_BF16) { CTB_HR_N(double, F_BF16) } else { CTB_HR_N(double, F_F16) }
        } else {
            if (dtype == CTB_BF16) { CTB_HR_N(float, F_BF16) } else { CTB_HR_N(float, F_F16) }
        }
        return after_launch("hadamard_rows_fast_kernel");
    }
    if ((dtype == CTB_BF16 || dtype == CTB_F16) && n >= 512) {
        const int w = rows_big_width(n, precision == CTB_F64);
        if (cols % w == 0 && (reinterpret_cast<uintptr_t>(x) % (2 * w)) == 0 && (reinterpret_cast<uintptr_t>(out) % (2 * w)) == 0) {
            if (precision == CTB_F64) {
                if (dtype == CTB_BF16) return launch_rows_big<double, F_BF16>(n, x, rows, cols, signs, inverse, normalize, out, st);
                return launch_rows_big<double, F_F16>(n, x, rows, cols, signs, inverse, normalize, out, st);
            }
            if (dtype == CTB_BF16) return launch_rows_big<float, F_BF16>(n, x, rows, cols, signs, inverse, normalize, out, st);
            return launch_rows_big<float, F_F16>(n, x, rows, cols, signs, inverse, normalize, out, st);
        }
    }
    // widest power-of-two tile (<= 32 columns) whose [n][W + 1] buffer fits in 200 KiB of shared memory
    const size_t esize = precision == CTB_F64 ? sizeof(double) : sizeof(float);
    int wshift = 5;
    while (wshift > 0 && (size_t)n * ((1u << wshift) + 1) * esize > 200u * 1024u) --wshift;
    const size_t smem = (size_t)n * ((1u << wshift) + 1) * esize;
    int64_t tiles = (rows / n) * cdiv(cols, 1 << wshift);
    int grid = grid_for(tiles, 1, 2);
    if (precision == CTB_F64) {
        cudaFuncSetAttribute(hadamard_rows_kernel<double>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        hadamard_rows_kernel<double><<<grid, kThreads, smem, st>>>(x, dtype, rows, cols, n, wshift, signs, inverse, normalize, out);
    } else {
        cudaFuncSetAttribute(hadamard_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        hadamard_rows_kernel<float><<<grid, kThreads, smem, st>>>(x, dtype, rows, cols, n, wshift, signs, inverse, normalize, out);
    }
    return after_launch("hadamard_rows_kernel");
}

extern "C" int ctb_absmax_quantize(const ctb_qdesc *d, const void *x, const float *gs, void *out_scale, void *out, int32_t n,
                                   const int8_t *signs, int32_t precision, void *stream) {
    if (!d) return fail(CTB_EINVAL_NULL, "null descriptor");
    if (d->rows != 0 && (!x || !out_scale || !out)) return fail(CTB_EINVAL_NULL, "null buffer");  // an empty tensor has no storage
    if (d->x_dtype != CTB_BF16) return fail(CTB_EUNSUPPORTED, "fused calibration is built for bf16 tensors");
    if (d->rows < 0 || d->cols <= 0 || d->col_group <= 0 || d->cols % d->col_group) return fail(CTB_EINVAL_SHAPE, "tensor column shape must be divisble by the given group_size");
    if (d->row_group != 1) return fail(CTB_EUNSUPPORTED, "fused calibration does not take 2-D blocks");
    if (d->cols % 8 || d->col_group % 8 || !aligned16(x) || !aligned16(out)) return fail(CTB_EINVAL_ALIGN, "needs cols %% 8 == 0, group %% 8 == 0 and 16-byte aligned buffers");
    const int qk = d->qtype == CTB_QINT ? QK_INT : (d->num_bits == 8 ? QK_FP8 : QK_FP4);
    if (qk == QK_FP4 && (!gs || d->scale_dtype != CTB_E4M3)) return fail(CTB_EINVAL_DTYPE, "fp4 needs a global scale and e4m3 group scales");
    if (qk != QK_FP4 && d->scale_dtype != d->x_dtype) return fail(CTB_EINVAL_DTYPE, "scales are produced in the dtype of the tensor");
    int fout = F_NONE;
    if (d->codec == CTB_CODE_PACK32 && qk == QK_INT && d->num_bits == 4) fout = F_PACK4;
    else if (d->codec == CTB_CODE_PACK32 && qk == QK_INT && d->num_bits == 8) fout = F_PACK8;
    else if (d->codec == CTB_CODE_DTYPE && qk == QK_INT && d->q_dtype == CTB_I8) fout = F_I8;
    else if (d->codec == CTB_CODE_DTYPE && qk == QK_FP8 && d->q_dtype == CTB_E4M3) fout = F_E4M3;
    else if (d->codec == CTB_CODE_FP4X2 && qk == QK_FP4) fout = F_FP4X2;
    else if (d->codec == CTB_CODE_DTYPE && qk != QK_FP4 && d->q_dtype == CTB_BF16) fout = F_BF16;  // fake quantize: dequantized values
    else return fail(CTB_EUNSUPPORTED, "fused calibration writes PACK32 (4/8 bit), int8, e4m3, FP4X2 or (fake quantize) bf16");
    const bool whole_row = d->col_group == d->cols && d->scale_row_stride == 1;
    const int64_t lanes = d->col_group / 8;
    if (fout == F_BF16 && !(n <= 0 && ((whole_row && d->cols / 8 <= 32 * 32) ||
                                       (lanes <= 32 && (lanes & (lanes - 1)) == 0 && d->scale_row_stride == d->cols / d->col_group))))
        return fail(CTB_EUNSUPPORTED, "fused dynamic fake quantize is built for whole rows of up to 8192 elements and power-of-two groups of 8..256");
    if (d->rows == 0) return CTB_OK;
    HArgs a{};
    a.x = x; a.signs = signs; a.out = out; a.out_scale = out_scale; a.gs = gs;
    a.chunks = d->rows * d->cols / 8; a.n = n; a.L = n > 0 ? n / 8 : 1; a.inverse = 0; a.normalize = 1; a.xdt = d->x_dtype;
    if (qk == QK_INT) { a.qmax = (float)(1 << d->num_bits) / 2 - 1; a.qmin = -(float)(1 << d->num_bits) / 2; }
    else if (qk == QK_FP8) { a.qmax = 448.0f; a.qmin = -448.0f; }
    else { a.qmax = 6.0f; a.qmin = -6.0f; }
    a.half_range = (a.qmax - a.qmin) / 2.0f;
    cudaStream_t st = as_stream(stream);
    const int64_t GL = d->col_group / 8;
    if (n > 0) {
        if (!pow2(n) || n < 8 || n > 256 || d->cols % n) return fail(CTB_EINVAL_SHAPE, "Hadamard size must be a power of two in 8..256 dividing the columns");
        if (precision == CTB_ROT_TENSOR) {
            if (!(n == 128 && d->col_group == 128 && fout == F_PACK4)) return fail(CTB_EUNSUPPORTED, "the tensor-core path is built for n = 128, group 128, int4 PACK32");
            ctb_tensor_ref t{x, out, out_scale, d->rows, d->cols};
            return rotquant_tc_launch(&t, 1, signs, true, nullptr, st);
        }
        if (precision != CTB_F64 && precision != CTB_F32) return fail(CTB_EINVAL_DTYPE, "precision must be F64, F32 or CTB_ROT_TENSOR");
        if (!(pow2(GL) && GL <= 32)) return fail(CTB_EUNSUPPORTED, "with a rotation in front the group must be a power of two <= 256");
        if (fout != F_PACK4) return fail(CTB_EUNSUPPORTED, "the fused rotation is built for int4 PACK32 output");
        a.GL = (int)GL;
        a.gl_shift = 0;
        while ((1 << a.gl_shift) < a.GL) ++a.gl_shift;
        if (n == 128 && d->col_group == 128) {
            static thread_local RQBatch B;
            rq_single(B, x, out, out_scale, d->rows * d->cols / 128);
            return launch_rotquant(B, signs, precision, true, st);
        }
        int grid = grid_for(a.chunks, kThreads, 8);
        if (precision == CTB_F64) absmax_quant_group_kernel<double, true, F_BF16, QK_INT, F_PACK4><<<grid, kThreads, 0, st>>>(a);
        else absmax_quant_group_kernel<float, true, F_BF16, QK_INT, F_PACK4><<<grid, kThreads, 0, st>>>(a);
        return after_launch("absmax_quant_group_kernel");
    }
    if (fout == F_PACK4 && d->col_group == 128 && d->scale_row_stride == d->cols / 128) {
        const int64_t ngroups = d->rows * d->cols / 128;
        // 128-thread blocks, eight per SM, striding over the groups: measured 8.9 us on 4096 x 4096 against 9.2 us for one
        // wave and a partial second wave of 256-thread blocks
        const int gthreads = 128;
        absmax_quant_g128_int4_kernel<<<grid_for(ngroups, gthreads / 2, 8), gthreads, 0, st>>>(x, out, out_scale, ngroups);
        return after_launch("absmax_quant_g128_int4_kernel");
    }
    if (fout == F_FP4X2 && d->col_group == 16 && d->scale_row_stride == d->cols / 16) {
        const int64_t ngroups = d->rows * d->cols / 16;
        absmax_quant_g16_fp4_kernel<<<grid_for(ngroups, kThreads * 2, 10), kThreads, 0, st>>>(a, ngroups);  // 47 registers: 5 resident blocks per SM, two waves
        return after_launch("absmax_quant_g16_fp4_kernel");
    }
    if (!(fout == F_BF16 && whole_row) && pow2(GL) && GL <= 32 && d->scale_row_stride == d->cols / d->col_group) {
        a.GL = (int)GL;
        a.gl_shift = 0;
        while ((1 << a.gl_shift) < a.GL) ++a.gl_shift;
        int grid = grid_for(a.chunks, kThreads * 4, 8);
#define CTB_AQ(QK_, FOUT_) absmax_quant_group_kernel<float, false, F_BF16, QK_, FOUT_><<<grid, kThreads, 0, st>>>(a)
        if (fout == F_PACK4) CTB_AQ(QK_INT, F_PACK4);
        else if (fout == F_PACK8) CTB_AQ(QK_INT, F_PACK8);
        else if (fout == F_I8) CTB_AQ(QK_INT, F_I8);
        else if (fout == F_E4M3) CTB_AQ(QK_FP8, F_E4M3);
        else if (fout == F_FP4X2) CTB_AQ(QK_FP4, F_FP4X2);
        else if (fout == F_BF16 && qk == QK_INT) CTB_AQ(QK_INT, F_BF16);
        else if (fout == F_BF16 && qk == QK_FP8) CTB_AQ(QK_FP8, F_BF16);
        else return fail(CTB_EUNSUPPORTED, "no fused group kernel for this output format");
        return after_launch("absmax_quant_group_kernel");
    }
    if (d->col_group == d->cols && d->scale_row_stride == 1 && qk != QK_FP4) {
        const int64_t cpr = d->cols / 8;
        if (cpr <= 32 * 32 && (fout == F_E4M3 || fout == F_I8 || fout == F_BF16)) {
            // blocks of four warps: a block is only a bundle of independent rows, and small bundles spread a few thousand
            // rows evenly over the SMs (4096 rows in blocks of eight left every seventh SM with an extra block: 11.9 -> 10.9 us)
            const int wthreads = 128, wbps = cpr <= 512 ? 4 : 2;
            int wgrid = grid_for(d->rows, wthreads / 32, wbps);
#define CTB_WR(CPL_)                                                                                                              \
    if (fout == F_E4M3) absmax_quant_warprow_kernel<CPL_, F_BF16, QK_FP8, F_E4M3><<<wgrid, wthreads, 0, st>>>(a, d->rows, (int)cpr); \
    else if (fout == F_I8) absmax_quant_warprow_kernel<CPL_, F_BF16, QK_INT, F_I8><<<wgrid, wthreads, 0, st>>>(a, d->rows, (int)cpr); \
    else if (qk == QK_FP8) absmax_quant_warprow_kernel<CPL_, F_BF16, QK_FP8, F_BF16><<<wgrid, wthreads, 0, st>>>(a, d->rows, (int)cpr); \
    else absmax_quant_warprow_kernel<CPL_, F_BF16, QK_INT, F_BF16><<<wgrid, wthreads, 0, st>>>(a, d->rows, (int)cpr);
            if (cpr <= 128) { CTB_WR(4) } else if (cpr <= 256) { CTB_WR(8) } else if (cpr <= 512) { CTB_WR(16) } else { CTB_WR(32) }
            return after_launch("absmax_quant_warprow_kernel");
        }
        int grid = grid_for(d->rows, 1, 8);
        if (fout == F_E4M3) absmax_quant_row_kernel<F_BF16, QK_FP8, F_E4M3><<<grid, kThreads, 0, st>>>(a, d->rows, cpr);
        else if (fout == F_I8) absmax_quant_row_kernel<F_BF16, QK_INT, F_I8><<<grid, kThreads, 0, st>>>(a, d->rows, cpr);
        else if (fout == F_PACK8) absmax_quant_row_kernel<F_BF16, QK_INT, F_PACK8><<<grid, kThreads, 0, st>>>(a, d->rows, cpr);
        else if (fout == F_PACK4) absmax_quant_row_kernel<F_BF16, QK_INT, F_PACK4><<<grid, kThreads, 0, st>>>(a, d->rows, cpr);
        else return fail(CTB_EUNSUPPORTED, "no fused row kernel for this output format");
        return after_launch("absmax_quant_row_kernel");
    }
    return fail(CTB_EUNSUPPORTED, "fused calibration takes groups of 8..256 (power of two) or whole rows");
}



extern "C" int ctb_rotate_quantize_int4_batch_bounded(const ctb_tensor_ref *tensors, int32_t count, const int8_t *signs,
                                                      int32_t *device_status, int64_t spin_cycles, int32_t skip_tile, void *stream) {
    if (!tensors && count > 0) return fail(CTB_EINVAL_NULL, "null tensor table");
    if (spin_cycles <= 0) return fail(CTB_EINVAL_SHAPE, "the wait budget must be positive");
    return rotquant_tc_launch(tensors, count, signs, true, device_status, as_stream(stream), spin_cycles, skip_tile);
}

extern "C" int ctb_rotate_quantize_int4_batch(const ctb_tensor_ref *tensors, int32_t count, const int8_t *signs, int32_t precision,
                                              int32_t *device_status, void *stream) {
    if (!tensors && count > 0) return fail(CTB_EINVAL_NULL, "null tensor table");
    if (precision == CTB_ROT_TENSOR) return rotquant_tc_launch(tensors, count, signs, true, device_status, as_stream(stream));
    if (precision != CTB_F64 && precision != CTB_F32) return fail(CTB_EINVAL_DTYPE, "precision must be F64, F32 or CTB_ROT_TENSOR");
    static thread_local RQBatch B;
    for (int32_t base = 0; base < count; base += kBatchMax) {
        const int32_t n = count - base < kBatchMax ? count - base : kBatchMax;
        int64_t g = 0;
        for (int32_t i = 0; i < n; ++i) {
            const ctb_tensor_ref &t = tensors[base + i];
            if (!t.in || !t.out || !t.scale) return fail(CTB_EINVAL_NULL, "tensor %d has a null buffer", base + i);
            if (t.rows < 0 || t.cols <= 0 || t.cols % 128) return fail(CTB_EINVAL_SHAPE, "tensor %d: columns %lld are not a multiple of 128", base + i, (long long)t.cols);
            if (!aligned16(t.in) || !aligned16(t.out)) return fail(CTB_EINVAL_ALIGN, "tensor %d is not 16-byte aligned", base + i);
            const int64_t nb = t.rows * t.cols / 128;
            B.start[i] = g;
            B.nblocks[i] = nb;
            B.x[i] = t.in;
            B.out[i] = t.out;
            B.scale[i] = t.scale;
            g += (nb + 15) & ~(int64_t)15;
        }
        B.count = n;
        B.start[n] = g;
        int rc = launch_rotquant(B, signs, precision, true, as_stream(stream));
        if (rc) return rc;
    }
    return CTB_OK;
}
