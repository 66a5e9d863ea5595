// Per-channel FP8 quantization fused with the 2:4 compaction: what a stacked float-quantized + sparse-24-bitmask
// checkpoint does to a bf16 weight in two passes (compressors/quantized_compressors/naive_quantized.py: compress_weight
// -> quantization/lifecycle/forward.py: _quantize, then compressors/sparse_compressors/sparse_24_bitmask.py:
// Sparse24BitMaskTensor.from_dense on the e4m3 result), in one pass over the weight.  The e4m3 tensor between the two
// never reaches memory: 2 bytes per element are read, 0.5 + 0.125 written.
//
// The arithmetic of each half is the arithmetic of the separate entry points (ctb_quantize and ctb_sparse24_compress),
// so the outputs are those of running the two one after the other, bit for bit: the kept pair of each run of four is
// chosen on the e4m3 codes (their int8 view, as the reference's topk on a float8 tensor does), not on the bf16 inputs.
#include "ctb_fastdiv.h"
#include "ctb_fp8_codes.cuh"
#include "ctb_sparse24_simd.cuh"

namespace ctb {

constexpr int kFusedThreads = 256;

struct QuantSparse24Args {
    const uint4 *in;        // bf16 [rows, cols], 8 elements per 16-byte unit
    const uint16_t *scale;  // bf16 [rows]
    const void *zp;         // [rows] of dtype zdt, or null
    int zdt;
    void *values;           // e4m3 [rows, cols / 2]
    uint8_t *bitmask;       // [rows, cols / 8]
    uint32_t units, upr;    // units in all, units per row
    FastDiv by_upr;
};

// Lane l of a warp takes units 64 t + l and 64 t + 32 + l, so that every load and store instruction of the warp
// covers one contiguous span; the four runs of four codes a thread then holds go through one 8-bit SIMD selection.
template <bool HAS_ZP>
__global__ void __launch_bounds__(kFusedThreads) quant_fp8_sparse24_kernel(const __grid_constant__ QuantSparse24Args a) {
    const uint32_t items = ((a.units + 63u) >> 6) << 5;
    const uint32_t stride = gridDim.x * (uint32_t)kFusedThreads;
    for (uint32_t it = blockIdx.x * (uint32_t)kFusedThreads + threadIdx.x; it < items; it += stride) {
        const uint32_t ua = ((it >> 5) << 6) + (it & 31u), ub = ua + 32u;
        const bool la = ua < a.units, lb = ub < a.units;
        uint4 ra = make_uint4(0, 0, 0, 0), rb = make_uint4(0, 0, 0, 0);
        if (la) ra = ld_stream(a.in + ua);
        if (lb) rb = ld_stream(a.in + ub);
        uint2 ca = make_uint2(0, 0), cb = make_uint2(0, 0);
        if (la) ca = fp8_codes8<HAS_ZP>(ra, a.in + ua, a.scale, a.zp, a.zdt, fastdiv(ua, a.by_upr));
        if (lb) cb = fp8_codes8<HAS_ZP>(rb, a.in + ub, a.scale, a.zp, a.zdt, fastdiv(ub, a.by_upr));
        uint32_t v0, v1, m;
        sparse24_pack_u8x16(ca.x, ca.y, cb.x, cb.y, v0, v1, m);
        if (la) {
            st_stream4((char *)a.values + (size_t)ua * 4, v0);
            a.bitmask[ua] = (uint8_t)m;
        }
        if (lb) {
            st_stream4((char *)a.values + (size_t)ub * 4, v1);
            a.bitmask[ub] = (uint8_t)(m >> 8);
        }
    }
}

}  // namespace ctb

using namespace ctb;

extern "C" int ctb_quantize_fp8_sparse24(const void *x, const void *scale, const void *zero_point, int32_t zp_dtype, int64_t rows,
                                         int64_t cols, void *values, uint8_t *bitmask, void *stream) {
    if (rows != 0 && cols != 0 && (!x || !scale || !values || !bitmask)) return fail(CTB_EINVAL_NULL, "null buffer");
    if (zero_point && dtype_size(zp_dtype) == 0) return fail(CTB_EINVAL_DTYPE, "unsupported zero point dtype %d", (int)zp_dtype);
    if (rows < 0 || cols < 0) return fail(CTB_EINVAL_SHAPE, "negative extent");
    if (cols % 8 != 0) return fail(CTB_EINVAL_SHAPE, "fused FP8 + 2:4 compression needs cols %% 8 == 0, got %lld", (long long)cols);
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(values) & 3u)) return fail(CTB_EINVAL_ALIGN, "x must be 16-byte, values 4-byte aligned");
    if (reinterpret_cast<uintptr_t>(scale) & 1u) return fail(CTB_EINVAL_ALIGN, "scale must be 2-byte aligned");
    const int64_t units = rows * cols / 8;
    if (units == 0) return CTB_OK;
    if (units >= (1ll << 31) - 64) return fail(CTB_EUNSUPPORTED, "more than 2^34 elements in one call");
    QuantSparse24Args a;
    a.in = reinterpret_cast<const uint4 *>(x);
    a.scale = reinterpret_cast<const uint16_t *>(scale);
    a.zp = zero_point;
    a.zdt = zp_dtype;
    a.values = values;
    a.bitmask = bitmask;
    a.units = (uint32_t)units;
    a.upr = (uint32_t)(cols / 8);
    a.by_upr = make_fastdiv(a.upr);
    cudaStream_t st = as_stream(stream);
    const int grid = grid_for((units + 1) / 2, kFusedThreads, 8);
    if (zero_point) quant_fp8_sparse24_kernel<true><<<grid, kFusedThreads, 0, st>>>(a);
    else quant_fp8_sparse24_kernel<false><<<grid, kFusedThreads, 0, st>>>(a);
    return after_launch("quant_fp8_sparse24_kernel");
}
