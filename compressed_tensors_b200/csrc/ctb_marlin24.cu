// Marlin-24 packing (compressors/sparse_quantized_compressors/marlin_24.py): a quantized, 2:4-sparse weight
// becomes (1) the CUTLASS 2:4 compaction with its reordered metadata
// (utils/semi_structured_conversions.py:79-209), (2) the compacted codes transposed, shifted to unsigned,
// shuffled into Marlin's 16 x 64 tensor-core tiles and packed 8 (4) to an int32 (marlin_24.py:208-249,
// utils/permutations_24.py:32-65), (3) the scales transposed and permuted (marlin_24.py:252-273).
//
// Everything here is index arithmetic on small integers: one pass over the codes per step, every output element
// computed from its own index (gather), no scratch, no atomics.
#include "ctb_common.cuh"

namespace ctb {

constexpr int kMThreads = 256;

// ---- step 1: one thread per metadata element = 16 consecutive elements of a row = 4 runs of four; one block per
// tile of 64 rows x 8 metadata columns.
//
// A run keeps two values chosen by its non-zero pattern (semi_structured_conversions.py:160-176): with m_i the
// non-zero flags, index0 = (~m0 & m1) | ((~m0 & ~m1) << 1) and index1 = ((m0 & m1) | (~m0 & ~m1) | m3) |
// (((~m0 & m1) | ~m1) << 1); the run's 4-bit code is index0 | index1 << 2.  Four codes make an int16 metadata
// element, which goes to its place in CUTLASS's reordered, column-interleaved layout (:43-73).  That reordering
// permutes rows inside groups of 64 and swaps elements inside 2 x 2 blocks, so a 64-row tile of a column pair is one
// contiguous run of 128 elements of the output: the tile's elements are placed in shared memory and written out
// as whole runs.
// ES = 1: int8 codes (standing for the 16-bit tensor holding the same integers), ES = 2: fp16 / bf16 values.
template <int ES>
__global__ void __launch_bounds__(kMThreads) cutlass24_compress_kernel(const void *dense, int64_t m, int64_t k, void *sparse, int16_t *meta_reordered) {
    __shared__ __align__(4) int16_t smeta[4][128];  // [column pair of the tile][reordered row * 2 + column parity]
    const int64_t ncols = k / 16, tiles_c = (ncols + 7) / 8, tiles = (m / 64) * tiles_c;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t tr = tile / tiles_c, r0 = tr * 64, c0 = (tile - tr * tiles_c) * 8;
        for (int e = threadIdx.x; e < 512; e += kMThreads) {
            const int row = e >> 3;
            const int64_t r = r0 + row, c = c0 + (e & 7);
            if (c >= ncols) continue;
            uint32_t v[16];  // raw bits of the 16 elements
            if constexpr (ES == 1) {
                const uint4 w = ld_stream((const char *)dense + (r * k + c * 16));
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = (ww[i >> 2] >> (8 * (i & 3))) & 0xFFu;
            } else {
                const char *p = (const char *)dense + (r * k + c * 16) * 2;
                const uint4 a = ld_stream(p), b = ld_stream(p + 16);
                const uint32_t ww[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = (ww[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
            }
            const uint32_t nz = ES == 1 ? 0xFFu : 0x7FFFu;  // -0.0 is zero for the float types (`dense != 0`)
            uint32_t elem = 0, kept[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool m0 = (v[4 * j] & nz) != 0, m1 = (v[4 * j + 1] & nz) != 0, m3 = (v[4 * j + 3] & nz) != 0;
                const bool e0 = m0 && m1, e1 = !m0 && m1, e2 = !m0 && !m1;
                const int i0 = (int)e1 | ((int)e2 << 1), i1 = (int)(e0 || e2 || m3) | ((int)(e1 || !m1) << 1);
                // register arrays cannot be indexed dynamically: select
                kept[2 * j] = i0 == 0 ? v[4 * j] : i0 == 1 ? v[4 * j + 1] : v[4 * j + 2];  // index0 is never 3
                kept[2 * j + 1] = i1 == 1 ? v[4 * j + 1] : i1 == 2 ? v[4 * j + 2] : v[4 * j + 3];  // index1 is never 0
                elem |= (uint32_t)(i0 | (i1 << 2)) << (4 * j);
            }
            if constexpr (ES == 1) {
                st_stream8((char *)sparse + (r * (k / 2) + c * 8),
                           make_uint2(kept[0] | (kept[1] << 8) | (kept[2] << 16) | (kept[3] << 24), kept[4] | (kept[5] << 8) | (kept[6] << 16) | (kept[7] << 24)));
            } else {
                st_stream((char *)sparse + (r * (k / 2) + c * 8) * 2,
                          make_uint4(kept[0] | (kept[1] << 16), kept[2] | (kept[3] << 16), kept[4] | (kept[5] << 16), kept[6] | (kept[7] << 16)));
            }
            // reordered row inside the 64-row group (a permutation of the row's bits), then the 2 x 2 swap
            int dl = (row & 1) * 2 + ((row & 7) >> 2) + (((row & 3) >> 1) << 5) + ((row >> 3) << 2);
            int dcl = e & 7;
            const int swap = (int)(((dl & 1) == 0) && ((dcl & 1) == 1)) - (int)(((dl & 1) == 1) && ((dcl & 1) == 0));
            dl += swap;
            dcl -= swap;
            smeta[dcl >> 1][dl * 2 + (dcl & 1)] = (int16_t)elem;
        }
        __syncthreads();
        {  // 4 column pairs x 128 elements, two elements (one 32-bit word) per thread
            const int pair = threadIdx.x >> 6, within = (threadIdx.x & 63) * 2;
            if (c0 + pair * 2 < ncols)
                *reinterpret_cast<uint32_t *>(meta_reordered + (c0 / 2 + pair) * m * 2 + r0 * 2 + within) = *reinterpret_cast<const uint32_t *>(&smeta[pair][within]);
        }
        __syncthreads();  // smeta is reused by the next tile
    }
}

// The inverse (semi_structured_conversions.py:216-308): one thread per metadata element reads it from its
// reordered place, and writes its 16 dense elements: the two kept values of every run at the positions their 2-bit
// indices name (the second write wins when both name the same position, as in the reference's scatter), zeros
// elsewhere.
template <int ES>
__global__ void __launch_bounds__(kMThreads) cutlass24_decompress_kernel(const void *sparse, const int16_t *meta_reordered, int64_t m, int64_t k2, void *dense) {
    const int64_t ncols = k2 / 8, total = m * ncols;
    const bool small = total < 0x7FFFFFFF;
    for (int64_t t = (int64_t)blockIdx.x * kMThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kMThreads) {
        const int64_t r = small ? (int64_t)((uint32_t)t / (uint32_t)ncols) : t / ncols, c = t - r * ncols;
        const int rl = (int)(r & 63);
        int dl = (rl & 1) * 2 + ((rl & 7) >> 2) + (((rl & 3) >> 1) << 5) + ((rl >> 3) << 2);
        int64_t dc = c;
        const int swap = (int)(((dl & 1) == 0) && ((dc & 1) == 1)) - (int)(((dl & 1) == 1) && ((dc & 1) == 0));
        dl += swap;
        dc -= swap;
        const uint32_t elem = (uint16_t)meta_reordered[(dc >> 1) * m * 2 + ((r & ~(int64_t)63) + dl) * 2 + (dc & 1)];
        uint32_t kept[8];
        if constexpr (ES == 1) {
            const uint2 w = *reinterpret_cast<const uint2 *>((const char *)sparse + (r * k2 + c * 8));
#pragma unroll
            for (int i = 0; i < 8; ++i) kept[i] = ((i < 4 ? w.x : w.y) >> (8 * (i & 3))) & 0xFFu;
        } else {
            const uint4 w = *reinterpret_cast<const uint4 *>((const char *)sparse + (r * k2 + c * 8) * 2);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) kept[i] = (ww[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
        }
        uint32_t v[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i0 = (elem >> (4 * j)) & 3, i1 = (elem >> (4 * j + 2)) & 3;
#pragma unroll
            for (int p = 0; p < 4; ++p) v[4 * j + p] = p == i1 ? kept[2 * j + 1] : p == i0 ? kept[2 * j] : 0u;
        }
        if constexpr (ES == 1) {
            uint4 o;
            o.x = v[0] | (v[1] << 8) | (v[2] << 16) | (v[3] << 24);
            o.y = v[4] | (v[5] << 8) | (v[6] << 16) | (v[7] << 24);
            o.z = v[8] | (v[9] << 8) | (v[10] << 16) | (v[11] << 24);
            o.w = v[12] | (v[13] << 8) | (v[14] << 16) | (v[15] << 24);
            *reinterpret_cast<uint4 *>((char *)dense + (r * k2 * 2 + c * 16)) = o;
        } else {
            uint4 *o = reinterpret_cast<uint4 *>((char *)dense + (r * k2 * 2 + c * 16) * 2);
            o[0] = make_uint4(v[0] | (v[1] << 16), v[2] | (v[3] << 16), v[4] | (v[5] << 16), v[6] | (v[7] << 16));
            o[1] = make_uint4(v[8] | (v[9] << 16), v[10] | (v[11] << 16), v[12] | (v[13] << 16), v[14] | (v[15] << 16));
        }
    }
}

// utils/permutations_24.py:32-65: source position inside a 1024-element chunk for destination position d
__device__ __forceinline__ int marlin24_perm(int d, int bits) {
    const int L = bits == 4 ? 8 : 4;
    const int t = d % L, b = d / L;
    const int il = bits == 4 ? ((t & 3) * 2 + (t >> 2)) : (t == 1 ? 2 : t == 2 ? 1 : t);  // {0,2,4,6,1,3,5,7} / {0,2,1,3}
    const int e = b * L + il;  // index into the un-interleaved list: 32 blocks of 4 x 8
    const int i = e / 32, j = (e % 32) / 8, q = e % 8;
    const int col = i / 4, col_o = col / 2, block = q / 4, rr = q % 4;
    const int row = rr == 0 ? 2 * (i % 4) : rr == 1 ? 2 * (i % 4) + 1 : rr == 2 ? 2 * (i % 4 + 4) : 2 * (i % 4 + 4) + 1;
    return 16 * row + col_o * 256 + 8 * (col % 2) + 4 * block + j;
}

// ---- step 2: one block per 1024-element chunk = a 16 (k) x 64 (n) tile of the compacted codes.  sparse is
// [n, k2] int8 codes; out is [k2 / 16, n * 16 / pf] int32.  The tile comes in as 64 rows of 16 contiguous bytes,
// goes through shared memory, and leaves as 1024 / pf consecutive words.
constexpr int kPackThreads = 128;
__global__ void __launch_bounds__(kPackThreads) marlin24_pack_weight_kernel(const int8_t *sparse, int64_t n, int64_t k2, int bits, int32_t *out) {
    __shared__ uint16_t perm[1024];
    __shared__ __align__(16) uint8_t tile[64 * 16];  // tile[ni_global(64)][ki(16)]
    for (int d = threadIdx.x; d < 1024; d += kPackThreads) perm[d] = (uint16_t)marlin24_perm(d, bits);
    const int pf = 32 / bits, half = (1 << bits) / 2, words = 1024 / pf;
    const int64_t chunks_per_row = n / 64, total = (k2 / 16) * chunks_per_row;
    for (int64_t blk = blockIdx.x; blk < total; blk += gridDim.x) {
        const int64_t kt = blk / chunks_per_row, ch = blk - kt * chunks_per_row;
        __syncthreads();  // the previous tile has been consumed (and perm is complete)
        if (threadIdx.x < 64)
            *reinterpret_cast<uint4 *>(tile + threadIdx.x * 16) = *reinterpret_cast<const uint4 *>(sparse + (ch * 64 + threadIdx.x) * k2 + kt * 16);
        __syncthreads();
        for (int w = threadIdx.x; w < words; w += kPackThreads) {
            uint32_t word = 0;
            for (int i = 0; i < pf; ++i) {
                // position inside the chunk: (n tile of 16, k, n inside the tile), marlin_24.py:213-217
                const int src = perm[w * pf + i], nt = src >> 8, ki = (src & 255) >> 4, ni = src & 15;
                word |= (uint32_t)((int)(int8_t)tile[(nt * 16 + ni) * 16 + ki] + half) << (bits * i);
            }
            out[kt * (chunks_per_row * words) + ch * words + w] = (int32_t)word;
        }
    }
}

// ---- step 3: scale is [n, g] (16-bit elements), out is [g, n]
__global__ void __launch_bounds__(kMThreads) marlin24_pack_scales_kernel(const uint16_t *scale, int64_t n, int64_t g, int grouped, uint16_t *out) {
    const int64_t total = n * g;
    for (int64_t f = (int64_t)blockIdx.x * kMThreads + threadIdx.x; f < total; f += (int64_t)gridDim.x * kMThreads) {
        const int64_t blk = f >> 6;
        const int w = (int)(f & 63), q = w & 7;
        const int inner = (q & 1) * 4 + (q >> 1);  // {0,4,1,5,2,6,3,7}
        const int64_t src = blk * 64 + (grouped ? (w & ~7) + inner : w);
        out[f] = scale[(src % n) * g + src / n];
    }
}

}  // namespace ctb

using namespace ctb;

extern "C" int ctb_cutlass24_compress(const void *dense, int32_t dtype, int64_t rows, int64_t cols, void *out_sparse, int16_t *out_meta,
                                      void *stream) {
    if (rows != 0 && cols != 0 && (!dense || !out_sparse || !out_meta)) return fail(CTB_EINVAL_NULL, "null buffer");  // an empty tensor has no storage
    if (dtype != CTB_I8 && dtype != CTB_F16 && dtype != CTB_BF16) return fail(CTB_EINVAL_DTYPE, "dense must be int8 codes, f16 or bf16");
    if (rows < 0 || cols < 0) return fail(CTB_EINVAL_SHAPE, "negative shape");
    if (rows % 64 != 0) return fail(CTB_EINVAL_SHAPE, "Number of rows of dense matrix %lld must be divisible by 64", (long long)rows);
    // 16 in the reference's check, but with an odd number of metadata columns its 2 x 2 swap leaves the matrix
    if (cols % 32 != 0) return fail(CTB_EINVAL_SHAPE, "Number of columns of dense matrix %lld must be divisible by 32", (long long)cols);
    if (!aligned16(dense) || !aligned16(out_sparse) || (reinterpret_cast<uintptr_t>(out_meta) & 3u)) return fail(CTB_EINVAL_ALIGN, "buffers must be 16-byte aligned (the metadata 4-byte)");
    if (rows == 0 || cols == 0) return CTB_OK;
    const int grid = grid_for((rows / 64) * ((cols / 16 + 7) / 8), 1, 8);
    if (dtype == CTB_I8) cutlass24_compress_kernel<1><<<grid, kMThreads, 0, as_stream(stream)>>>(dense, rows, cols, out_sparse, out_meta);
    else cutlass24_compress_kernel<2><<<grid, kMThreads, 0, as_stream(stream)>>>(dense, rows, cols, out_sparse, out_meta);
    return after_launch("cutlass24_compress_kernel");
}

extern "C" int ctb_marlin24_pack_weight(const int8_t *sparse, int64_t n, int64_t k2, int32_t num_bits, int32_t *out, void *stream) {
    if (n != 0 && k2 != 0 && (!sparse || !out)) return fail(CTB_EINVAL_NULL, "null buffer");
    if (num_bits != 4 && num_bits != 8) return fail(CTB_EINVAL_SHAPE, "num_bits must be 4 or 8, got %d", num_bits);
    if (n < 0 || k2 < 0 || k2 % 16 != 0 || n % 64 != 0) return fail(CTB_EINVAL_SHAPE, "size_k must be a multiple of 16 and size_n of 64");
    if (n == 0 || k2 == 0) return CTB_OK;
    if (reinterpret_cast<uintptr_t>(sparse) & 15u) return fail(CTB_EINVAL_ALIGN, "codes must be 16-byte aligned");
    marlin24_pack_weight_kernel<<<grid_for((k2 / 16) * (n / 64), 1, 16), kPackThreads, 0, as_stream(stream)>>>(sparse, n, k2, num_bits, out);
    return after_launch("marlin24_pack_weight_kernel");
}

extern "C" int ctb_marlin24_pack_scales(const void *scale, int64_t n, int64_t groups, int32_t grouped, void *out, void *stream) {
    if (n != 0 && groups != 0 && (!scale || !out)) return fail(CTB_EINVAL_NULL, "null buffer");
    if (n < 0 || groups < 0 || n % 64 != 0) return fail(CTB_EINVAL_SHAPE, "size_n must be a multiple of 64");
    if (n == 0 || groups == 0) return CTB_OK;
    marlin24_pack_scales_kernel<<<grid_for(n * groups, kMThreads, 8), kMThreads, 0, as_stream(stream)>>>((const uint16_t *)scale, n, groups,
                                                                                                          grouped, (uint16_t *)out);
    return after_launch("marlin24_pack_scales_kernel");
}

extern "C" int ctb_cutlass24_decompress(const void *sparse, const int16_t *meta, int32_t dtype, int64_t rows, int64_t cols_sparse, void *out_dense,
                                        void *stream) {
    if (rows != 0 && cols_sparse != 0 && (!sparse || !meta || !out_dense)) return fail(CTB_EINVAL_NULL, "null buffer");
    if (dtype != CTB_I8 && dtype != CTB_F16 && dtype != CTB_BF16) return fail(CTB_EINVAL_DTYPE, "values must be int8 codes, f16 or bf16");
    if (rows < 0 || cols_sparse < 0) return fail(CTB_EINVAL_SHAPE, "negative shape");
    if (rows % 64 != 0 || cols_sparse % 16 != 0) return fail(CTB_EINVAL_SHAPE, "rows must be divisible by 64 and the compacted columns by 16");
    if (rows == 0 || cols_sparse == 0) return CTB_OK;
    if (!aligned16(sparse) || !aligned16(out_dense)) return fail(CTB_EINVAL_ALIGN, "buffers must be 16-byte aligned");
    const int grid = grid_for(rows * (cols_sparse / 8), kMThreads, 8);
    if (dtype == CTB_I8) cutlass24_decompress_kernel<1><<<grid, kMThreads, 0, as_stream(stream)>>>(sparse, meta, rows, cols_sparse, out_dense);
    else cutlass24_decompress_kernel<2><<<grid, kMThreads, 0, as_stream(stream)>>>(sparse, meta, rows, cols_sparse, out_dense);
    return after_launch("cutlass24_decompress_kernel");
}

