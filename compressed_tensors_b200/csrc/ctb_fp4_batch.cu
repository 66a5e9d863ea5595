// Whole-shard NVFP4: every Linear weight of a shard in ONE grid per direction, the per-tensor loops of
// compressors/quantized_compressors/base.py:91-134 (compress -> fp4_quantized.py:84-105 compress_weight: quantize with
// e4m3 group-16 scales under an fp32 global scale, then pack_fp4_to_uint8) and base.py:190-237 (decompress_weight:
// unpack_fp4_from_uint8, dequantize).  The arithmetic is that of ctb_quantize / ctb_dequantize and of the fused
// calibrate kernel (same device functions), so the bytes are those of the per-tensor calls.
#include "ctb_codec.cuh"

namespace ctb {

constexpr int kF4Threads = 256;
constexpr int kF4Unroll = 4;
constexpr int kF4Unit = kF4Threads * kF4Unroll;  // chunks (8 elements) per block-iteration
constexpr int kF4BatchMax = 256;

struct F4Batch {
    int count, zdt;
    int64_t ustart[kF4BatchMax + 1];  // first global unit of each tensor; ustart[count] = total
    uint32_t nchunks[kF4BatchMax];
    const void *in[kF4BatchMax];
    const void *scale[kF4BatchMax];   // e4m3 [rows, cols / 16]
    const float *gs[kF4BatchMax];     // fp32 [1]
    const void *zp[kF4BatchMax];      // [rows, cols / 16] of dtype zdt or null (quantize only)
    void *out[kF4BatchMax];
};

// bf16 -> e2m1 codes, two per byte.  A lane takes whole groups of 16 elements (32 contiguous bytes in, 8 out), so the
// effective scale of a group, float(e4m3 scale) / global_scale (forward.py:468-469), is divided once per group.
// Finite groups with a scale in the normal range and no zero point other than zero go through the reciprocal +
// Markstein quotient and the saturating e2m1 convert (quant_fp4_codes_f32); everything else through the templates of
// the per-tensor vec8 tier.
__global__ void __launch_bounds__(kF4Threads) quant_fp4_g16_batch_kernel(const __grid_constant__ F4Batch B) {
    constexpr int U = kF4Unroll / 2;  // groups per lane and unit
    const int64_t total = B.ustart[B.count];
    int t = 0;
    uint4 raw[U][2];
    bool ok[U];
    uint32_t gbase = 0;
    auto fetch = [&](int64_t unit) {
        while (t + 1 < B.count && unit >= B.ustart[t + 1]) ++t;
        gbase = (uint32_t)(unit - B.ustart[t]) * (uint32_t)(kF4Unit / 2);
        const char *ip = (const char *)B.in[t];
        const uint32_t ngroups = B.nchunks[t] >> 1;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t g = gbase + u * kF4Threads + threadIdx.x;
            ok[u] = g < ngroups;
            if (ok[u]) {
                // a lane's two halves share a 32-byte sector: let L1 keep it between the two instructions
                raw[u][0] = __ldg(reinterpret_cast<const uint4 *>(ip + (size_t)g * 32));
                raw[u][1] = __ldg(reinterpret_cast<const uint4 *>(ip + (size_t)g * 32 + 16));
            }
        }
    };
    int64_t unit = blockIdx.x;
    if (unit < total) fetch(unit);
    while (unit < total) {
        uint4 w[U][2];
        bool k[U];
        const int ct = t;
        const uint32_t gb = gbase;
#pragma unroll
        for (int u = 0; u < U; ++u) { w[u][0] = raw[u][0]; w[u][1] = raw[u][1]; k[u] = ok[u]; }
        const int64_t next = unit + gridDim.x;
        if (next < total) fetch(next);
        const void *zp = B.zp[ct];
        const bool has_zp = zp != nullptr;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (!k[u]) continue;
            const uint32_t g = gb + u * kF4Threads + threadIdx.x;
            const QP q = load_qp(B.scale[ct], CTB_E4M3, zp, B.zdt, B.gs[ct], (int64_t)g);
            const uint32_t w0[4] = {w[u][0].x, w[u][0].y, w[u][0].z, w[u][0].w};
            const uint32_t w1[4] = {w[u][1].x, w[u][1].y, w[u][1].z, w[u][1].w};
            // an element with all exponent bits set (inf, NaN): adding 0x0080 to its magnitude carries into bit 15
            uint32_t nonfinite = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                nonfinite |= ((w0[i] & 0x7FFF7FFFu) + 0x00800080u) | ((w1[i] & 0x7FFF7FFFu) + 0x00800080u);
            if (!q.slow && q.zp == 0.0f && (nonfinite & 0x80008000u) == 0) {
                st_stream8((char *)B.out[ct] + (size_t)g * 8, make_uint2(quant_fp4_codes_f32(w0, q.s, q.r), quant_fp4_codes_f32(w1, q.s, q.r)));
                continue;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                Raw8 r8;
                r8.a = w[u][h];
                r8.b = make_uint4(0, 0, 0, 0);
                float v[8];
                decode8<F_BF16>(r8, v);
                quant_prepare8<CTB_F32>(v, q, has_zp, q.zp, -6.0f, 6.0f);
                encode_store8<QK_FP4, F_FP4X2>(B.out[ct], (int64_t)g * 2 + h, v);
            }
        }
        unit = next;
    }
}

// e2m1 codes -> bf16.  There are only 256 possible scale bytes, so the effective scales of the tensor a block is
// working on are divided once into a shared table (IEEE division, what the reference computes per group) and rebuilt
// when the block moves on to the next tensor.
__global__ void __launch_bounds__(kF4Threads) dequant_fp4_g16_batch_kernel(const __grid_constant__ F4Batch B) {
    __shared__ float s_eff[256];
    static_assert(kF4Threads == 256, "one table entry per thread");
    const int64_t total = B.ustart[B.count];
    int t = 0, table_of = -1;
    constexpr int U = 2 * kF4Unroll;  // a unit is kF4Unit chunks of the DENSE side; codes come 4 bytes per chunk
    for (int64_t unit = blockIdx.x; unit < total; unit += gridDim.x) {
        while (t + 1 < B.count && unit >= B.ustart[t + 1]) ++t;
        if (t != table_of) {  // uniform across the block
            __syncthreads();  // everyone is done with the previous tensor's table
            s_eff[threadIdx.x] = __fdiv_rn(e4m3_to_f32((uint8_t)threadIdx.x), __ldg(B.gs[t]));
            __syncthreads();
            table_of = t;
        }
        const uint32_t cbase = (uint32_t)(unit - B.ustart[t]) * (uint32_t)(kF4Threads * U);
        const char *ip = (const char *)B.in[t];
        const uint8_t *sp = (const uint8_t *)B.scale[t];
        char *op = (char *)B.out[t];
        uint32_t w[U], sb[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t c = cbase + u * kF4Threads + threadIdx.x;
            w[u] = 0;
            sb[u] = 0;
            if (c < B.nchunks[t]) {
                w[u] = ld_stream4(ip + (size_t)c * 4);
                sb[u] = sp[c >> 1];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t c = cbase + u * kF4Threads + threadIdx.x;
            if (c >= B.nchunks[t]) break;
            const float s = s_eff[sb[u]];
            uint32_t p[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // low nibble = even element; nibble 0x8 decodes to -0.0, which the product keeps
                const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((w[u] >> (8 * i)) & 0xFFu), __NV_E2M1);
                const float2 f = __half22float2(__half2(h));
                p[i] = bf162_as_u32(__floats2bfloat162_rn(f.x * s, f.y * s));  // fp32 product, then one rounding to bf16
            }
            st_stream(op + (size_t)c * 16, make_uint4(p[0], p[1], p[2], p[3]));
        }
    }
}

static int fill(F4Batch &B, const ctb_tensor_ref *tensors, const void *const *global_scales, const void *const *zero_points,
                int32_t zp_dtype, int32_t base, int32_t n, int unit_chunks, int in_align, int out_align) {
    B.count = n;
    B.zdt = zp_dtype;
    int64_t units = 0;
    for (int32_t i = 0; i < n; ++i) {
        const ctb_tensor_ref &r = tensors[base + i];
        if (r.rows < 0 || r.cols < 0) return fail(CTB_EINVAL_SHAPE, "tensor %d: negative extent", base + i);
        if (r.cols % 16 != 0) return fail(CTB_EINVAL_SHAPE, "tensor %d: cols must be a multiple of the group size 16, got %lld", base + i, (long long)r.cols);
        const int64_t chunks = r.rows * r.cols / 8;
        if (chunks >= (1ll << 31) - unit_chunks) return fail(CTB_EUNSUPPORTED, "tensor %d: more than 2^34 elements", base + i);
        if (chunks > 0 && (!r.in || !r.out || !r.scale || !global_scales || !global_scales[base + i]))
            return fail(CTB_EINVAL_NULL, "tensor %d: null buffer", base + i);
        if ((reinterpret_cast<uintptr_t>(r.in) & (in_align - 1)) || (reinterpret_cast<uintptr_t>(r.out) & (out_align - 1)))
            return fail(CTB_EINVAL_ALIGN, "tensor %d: the bf16 side must be 16-byte aligned, the packed side 8-byte (quantize) / 4-byte (dequantize)", base + i);
        if (reinterpret_cast<uintptr_t>(global_scales ? global_scales[base + i] : nullptr) & 3u)
            return fail(CTB_EINVAL_ALIGN, "tensor %d: global scale must be 4-byte aligned", base + i);
        B.ustart[i] = units;
        B.nchunks[i] = (uint32_t)chunks;
        B.in[i] = r.in;
        B.scale[i] = r.scale;
        B.gs[i] = global_scales ? reinterpret_cast<const float *>(global_scales[base + i]) : nullptr;
        B.zp[i] = zero_points ? zero_points[base + i] : nullptr;
        B.out[i] = r.out;
        units += (chunks + unit_chunks - 1) / unit_chunks;
    }
    B.ustart[n] = units;
    return CTB_OK;
}

int quant_fp4_g16_one(const void *x, const void *scale, const float *gs, const void *zp, int zdt, int64_t rows, int64_t cols, void *out,
                      cudaStream_t st) {
    static thread_local F4Batch B;
    ctb_tensor_ref r;
    r.in = x;
    r.out = out;
    r.scale = const_cast<void *>(scale);
    r.rows = rows;
    r.cols = cols;
    const void *g = gs, *z = zp;
    int rc = fill(B, &r, &g, zp ? &z : nullptr, zdt, 0, 1, kF4Unit, 16, 8);
    if (rc) return rc;
    if (B.ustart[1] == 0) return CTB_OK;
    quant_fp4_g16_batch_kernel<<<grid_for(B.ustart[1], 1, 8), kF4Threads, 0, st>>>(B);
    return after_launch("quant_fp4_g16_batch_kernel");
}

}  // namespace ctb

using namespace ctb;

extern "C" int ctb_quantize_fp4_g16_batch(const ctb_tensor_ref *tensors, int32_t count, const void *const *global_scales,
                                          const void *const *zero_points, int32_t zp_dtype, void *stream) {
    if (!tensors && count > 0) return fail(CTB_EINVAL_NULL, "null tensor table");
    if (zero_points && dtype_size(zp_dtype) == 0) return fail(CTB_EINVAL_DTYPE, "unsupported zero point dtype %d", (int)zp_dtype);
    static thread_local F4Batch B;
    for (int32_t base = 0; base < count; base += kF4BatchMax) {
        const int32_t n = count - base < kF4BatchMax ? count - base : kF4BatchMax;
        int rc = fill(B, tensors, global_scales, zero_points, zp_dtype, base, n, kF4Unit, 16, 8);
        if (rc) return rc;
        if (B.ustart[n] == 0) continue;
        quant_fp4_g16_batch_kernel<<<grid_for(B.ustart[n], 1, 8), kF4Threads, 0, as_stream(stream)>>>(B);
        rc = after_launch("quant_fp4_g16_batch_kernel");
        if (rc) return rc;
    }
    return CTB_OK;
}

extern "C" int ctb_dequantize_fp4_g16_batch(const ctb_tensor_ref *tensors, int32_t count, const void *const *global_scales, void *stream) {
    if (!tensors && count > 0) return fail(CTB_EINVAL_NULL, "null tensor table");
    static thread_local F4Batch B;
    for (int32_t base = 0; base < count; base += kF4BatchMax) {
        const int32_t n = count - base < kF4BatchMax ? count - base : kF4BatchMax;
        int rc = fill(B, tensors, global_scales, nullptr, 0, base, n, kF4Threads * 2 * kF4Unroll, 4, 16);
        if (rc) return rc;
        if (B.ustart[n] == 0) continue;
        // more blocks than are resident at once: the writes of finished blocks overlap the loads of new ones
        dequant_fp4_g16_batch_kernel<<<grid_for(B.ustart[n], 1, 16), kF4Threads, 0, as_stream(stream)>>>(B);
        rc = after_launch("dequant_fp4_g16_batch_kernel");
        if (rc) return rc;
    }
    return CTB_OK;
}
