// Whole-shard FP8 per-channel quantize and dequantize: every Linear weight of a shard in ONE grid, the per-tensor loops
// of compressors/quantized_compressors/base.py:91-134 (compress -> naive_quantized.py compress_weight ->
// forward.py _quantize to float8_e4m3fn) and base.py:190-237 (decompress_weight -> forward.py dequantize) turned into
// two launches.  Static per-output-channel bf16 scales (one per row), bf16 weights; the arithmetic is that of
// ctb_quantize / ctb_dequantize for the same arguments, bit for bit.
#include "ctb_fastdiv.h"
#include "ctb_fp8_codes.cuh"

namespace ctb {

constexpr int kF8Threads = 256;
constexpr int kF8Unroll = 4;
constexpr int kF8Unit = kF8Threads * kF8Unroll;  // chunks (8 elements) per block-iteration
constexpr int kF8BatchMax = 256;

struct F8Batch {
    int count, zdt;
    int64_t ustart[kF8BatchMax + 1];  // first global unit of each tensor; ustart[count] = total
    uint32_t nchunks[kF8BatchMax];    // chunks of each tensor
    FastDiv by_cpr[kF8BatchMax];      // chunk -> row
    const void *in[kF8BatchMax];
    const void *scale[kF8BatchMax];   // bf16 [rows]
    const void *zp[kF8BatchMax];      // [rows] of dtype zdt or null (quantize only)
    void *out[kF8BatchMax];
};

// The units of all tensors form one index space that the grid strides over; the tensor lookup happens once per unit
// (uniform across the block), addressing inside a tensor is 32-bit, and the next unit's chunks are loaded before the
// current unit is computed and written.
__global__ void __launch_bounds__(kF8Threads) quant_fp8_channel_batch_kernel(const __grid_constant__ F8Batch B) {
    const int64_t total = B.ustart[B.count];
    int t = 0;
    uint4 raw[kF8Unroll];
    bool ok[kF8Unroll];
    uint32_t cbase = 0;
    auto fetch = [&](int64_t unit) {
        while (t + 1 < B.count && unit >= B.ustart[t + 1]) ++t;
        cbase = (uint32_t)(unit - B.ustart[t]) * (uint32_t)kF8Unit;
        const uint4 *ip = (const uint4 *)B.in[t];
#pragma unroll
        for (int u = 0; u < kF8Unroll; ++u) {
            const uint32_t c = cbase + u * kF8Threads + threadIdx.x;
            ok[u] = c < B.nchunks[t];
            if (ok[u]) raw[u] = ld_stream(ip + c);
        }
    };
    int64_t unit = blockIdx.x;
    if (unit < total) fetch(unit);
    while (unit < total) {
        uint4 w[kF8Unroll];
        bool k[kF8Unroll];
        const int ct = t;
        const uint32_t cb = cbase;
#pragma unroll
        for (int u = 0; u < kF8Unroll; ++u) { w[u] = raw[u]; k[u] = ok[u]; }
        const int64_t next = unit + gridDim.x;
        if (next < total) fetch(next);
        const uint4 *ip = (const uint4 *)B.in[ct];
        const uint16_t *sp = (const uint16_t *)B.scale[ct];
        const void *zp = B.zp[ct];
        const FastDiv by = B.by_cpr[ct];
        char *o = (char *)B.out[ct];
#pragma unroll
        for (int u = 0; u < kF8Unroll; ++u) {
            if (!k[u]) continue;
            const uint32_t c = cb + u * kF8Threads + threadIdx.x;
            const uint32_t row = fastdiv(c, by);
            const uint2 codes = zp ? fp8_codes8<true>(w[u], ip + c, sp, zp, B.zdt, row) : fp8_codes8<false>(w[u], ip + c, sp, nullptr, 0, row);
            st_stream8(o + (size_t)c * 8, codes);
        }
        unit = next;
    }
}

// e4m3 codes -> bf16: x_q.to(bf16) * scale, one rounding (the codes are exact in bf16)
__global__ void __launch_bounds__(kF8Threads) dequant_fp8_channel_batch_kernel(const __grid_constant__ F8Batch B) {
    const int64_t total = B.ustart[B.count];
    int t = 0;
    uint2 raw[kF8Unroll];
    uint32_t sbits[kF8Unroll];
    bool ok[kF8Unroll];
    uint32_t cbase = 0;
    auto fetch = [&](int64_t unit) {
        while (t + 1 < B.count && unit >= B.ustart[t + 1]) ++t;
        cbase = (uint32_t)(unit - B.ustart[t]) * (uint32_t)kF8Unit;
        const char *ip = (const char *)B.in[t];
        const uint16_t *sp = (const uint16_t *)B.scale[t];
        const FastDiv by = B.by_cpr[t];
#pragma unroll
        for (int u = 0; u < kF8Unroll; ++u) {
            const uint32_t c = cbase + u * kF8Threads + threadIdx.x;
            ok[u] = c < B.nchunks[t];
            if (ok[u]) {
                raw[u] = ld_stream8(ip + (size_t)c * 8);
                sbits[u] = __ldg(sp + fastdiv(c, by));
            }
        }
    };
    int64_t unit = blockIdx.x;
    if (unit < total) fetch(unit);
    while (unit < total) {
        uint2 w[kF8Unroll];
        uint32_t s[kF8Unroll];
        bool k[kF8Unroll];
        char *o = (char *)B.out[t] + (size_t)cbase * 16;
#pragma unroll
        for (int u = 0; u < kF8Unroll; ++u) { w[u] = raw[u]; s[u] = sbits[u]; k[u] = ok[u]; }
        const int64_t next = unit + gridDim.x;
        if (next < total) fetch(next);
#pragma unroll
        for (int u = 0; u < kF8Unroll; ++u) {
            if (!k[u]) continue;
            Raw8 r;
            r.a = make_uint4(w[u].x, w[u].y, 0, 0);
            r.b = make_uint4(0, 0, 0, 0);
            float v[8];
            decode8<F_E4M3>(r, v);
            st_stream(o + (size_t)(u * kF8Threads + threadIdx.x) * 16, dequant8_to_bf16<false>(v, __uint_as_float(s[u] << 16)));
        }
        unit = next;
    }
}

// fills the table for tensors [base, base + n); `elem_in` / `elem_out` are the element sizes of the two sides
static int fill(F8Batch &B, const ctb_tensor_ref *tensors, const void *const *zero_points, int32_t zp_dtype, int32_t base, int32_t n,
                int in_align, int out_align) {
    B.count = n;
    B.zdt = zp_dtype;
    int64_t units = 0;
    for (int32_t i = 0; i < n; ++i) {
        const ctb_tensor_ref &r = tensors[base + i];
        if (r.rows < 0 || r.cols < 0) return fail(CTB_EINVAL_SHAPE, "tensor %d: negative extent", base + i);
        if (r.cols % 8 != 0) return fail(CTB_EINVAL_SHAPE, "tensor %d: cols must be a multiple of 8, got %lld", base + i, (long long)r.cols);
        const int64_t chunks = r.rows * r.cols / 8;
        if (chunks >= (1ll << 31) - kF8Unit) return fail(CTB_EUNSUPPORTED, "tensor %d: more than 2^34 elements", base + i);
        if (chunks > 0 && (!r.in || !r.out || !r.scale)) return fail(CTB_EINVAL_NULL, "tensor %d: null buffer", base + i);
        if ((reinterpret_cast<uintptr_t>(r.in) & (in_align - 1)) || (reinterpret_cast<uintptr_t>(r.out) & (out_align - 1)))
            return fail(CTB_EINVAL_ALIGN, "tensor %d: the bf16 side must be 16-byte, the e4m3 side 8-byte aligned", base + i);
        if (reinterpret_cast<uintptr_t>(r.scale) & 1u) return fail(CTB_EINVAL_ALIGN, "tensor %d: scale must be 2-byte aligned", base + i);
        B.ustart[i] = units;
        B.nchunks[i] = (uint32_t)chunks;
        B.by_cpr[i] = make_fastdiv((uint32_t)(r.cols / 8 > 0 ? r.cols / 8 : 1));
        B.in[i] = r.in;
        B.scale[i] = r.scale;
        B.zp[i] = zero_points ? zero_points[base + i] : nullptr;
        B.out[i] = r.out;
        units += (chunks + kF8Unit - 1) / kF8Unit;
    }
    B.ustart[n] = units;
    return CTB_OK;
}

}  // namespace ctb

using namespace ctb;

extern "C" int ctb_quantize_fp8_channel_batch(const ctb_tensor_ref *tensors, int32_t count, const void *const *zero_points,
                                              int32_t zp_dtype, void *stream) {
    if (!tensors && count > 0) return fail(CTB_EINVAL_NULL, "null tensor table");
    if (zero_points && dtype_size(zp_dtype) == 0) return fail(CTB_EINVAL_DTYPE, "unsupported zero point dtype %d", (int)zp_dtype);
    static thread_local F8Batch B;
    for (int32_t base = 0; base < count; base += kF8BatchMax) {
        const int32_t n = count - base < kF8BatchMax ? count - base : kF8BatchMax;
        int rc = fill(B, tensors, zero_points, zp_dtype, base, n, 16, 8);
        if (rc) return rc;
        if (B.ustart[n] == 0) continue;
        const int grid = grid_for(B.ustart[n], 1, 8);
        quant_fp8_channel_batch_kernel<<<grid, kF8Threads, 0, as_stream(stream)>>>(B);
        rc = after_launch("quant_fp8_channel_batch_kernel");
        if (rc) return rc;
    }
    return CTB_OK;
}

extern "C" int ctb_dequantize_fp8_channel_batch(const ctb_tensor_ref *tensors, int32_t count, void *stream) {
    if (!tensors && count > 0) return fail(CTB_EINVAL_NULL, "null tensor table");
    static thread_local F8Batch B;
    for (int32_t base = 0; base < count; base += kF8BatchMax) {
        const int32_t n = count - base < kF8BatchMax ? count - base : kF8BatchMax;
        int rc = fill(B, tensors, nullptr, 0, base, n, 8, 16);
        if (rc) return rc;
        if (B.ustart[n] == 0) continue;
        // more blocks than are resident at once: the writes of finished blocks overlap the loads of new ones
        const int grid = grid_for(B.ustart[n], 1, 16);
        dequant_fp8_channel_batch_kernel<<<grid, kF8Threads, 0, as_stream(stream)>>>(B);
        rc = after_launch("dequant_fp8_channel_batch_kernel");
        if (rc) return rc;
    }
    return CTB_OK;
}
