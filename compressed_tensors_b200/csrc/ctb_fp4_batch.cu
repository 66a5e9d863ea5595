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

// One chunk by the templates of the per-tensor vec8 tier (any input, any scale, any zero point).  Out of line: it is
// the rare path and its registers would otherwise set the occupancy of the whole kernel.
__device__ __noinline__ void quant_fp4_chunk_general(const uint4 *chunk, const void *scale, const void *zp, int zdt, const float *gs, void *out,
                                                     uint32_t c) {
    const QP q = load_qp(scale, CTB_E4M3, zp, zdt, gs, (int64_t)(c >> 1));
    Raw8 r8;
    r8.a = __ldg(chunk);
    r8.b = make_uint4(0, 0, 0, 0);
    float v[8];
    decode8<F_BF16>(r8, v);
    quant_prepare8<CTB_F32>(v, q, zp != nullptr, q.zp, -6.0f, 6.0f);
    encode_store8<QK_FP4, F_FP4X2>(out, (int64_t)c, v);
}

// bf16 -> e2m1 codes, two per byte.  A lane takes a chunk of 8 elements, half a group, so that every warp instruction
// moves one contiguous span.  Finite chunks with a scale in the normal range and no zero point other than zero go
// through the reciprocal + Markstein quotient and the saturating e2m1 convert (quant_fp4_codes_f32); everything else
// through the templates of the per-tensor vec8 tier.
__global__ void __launch_bounds__(kF4Threads, 6) quant_fp4_g16_batch_kernel(const __grid_constant__ F4Batch B) {
    // (effective scale, its reciprocal) of every possible scale byte of the tensor the block is working on: 256 IEEE
    // divisions per tensor instead of one per group.  A reciprocal of 0 marks a scale outside the range where the
    // reciprocal + Markstein quotient is proven (or not finite): those chunks take the general routine.
    __shared__ float2 tab[256];
    static_assert(kF4Threads == 256, "one table entry per thread");
    const int64_t total = B.ustart[B.count];
    int t = 0, table_of = -1;
    for (int64_t unit = blockIdx.x; unit < total; unit += gridDim.x) {
        while (t + 1 < B.count && unit >= B.ustart[t + 1]) ++t;
        if (t != table_of) {  // uniform across the block
            __syncthreads();  // everyone is done with the previous tensor's table
            const float se = __fdiv_rn(e4m3_to_f32((uint8_t)threadIdx.x), __ldg(B.gs[t]));  // forward.py:468-469
            const bool fast = fabsf(se) >= 1.0e-30f && fabsf(se) <= 1.0e30f;
            tab[threadIdx.x] = make_float2(se, fast ? __frcp_rn(se) : 0.0f);
            __syncthreads();
            table_of = t;
        }
        const uint32_t cbase = (uint32_t)(unit - B.ustart[t]) * (uint32_t)kF4Unit;
        const uint4 *ip = (const uint4 *)B.in[t];
        const uint32_t nchunks = B.nchunks[t];
        const uint8_t *sp = (const uint8_t *)B.scale[t];
        const void *zp = B.zp[t];
        char *op = (char *)B.out[t];
        uint4 w[kF4Unroll];
        uint32_t sb[kF4Unroll];
        float zv[kF4Unroll];
#pragma unroll
        for (int u = 0; u < kF4Unroll; ++u) {  // all loads first (data, scale byte, zero point): one memory latency per unit
            const uint32_t c = cbase + u * kF4Threads + threadIdx.x;
            zv[u] = 0.0f;
            sb[u] = 0;
            w[u] = make_uint4(0, 0, 0, 0);
            if (c < nchunks) {
                w[u] = ld_stream(ip + c);  // a warp instruction covers 512 contiguous bytes
                sb[u] = __ldg(sp + (c >> 1));
                if (zp) zv[u] = load_f32(zp, B.zdt, (int64_t)(c >> 1));
            }
        }
#pragma unroll
        for (int u = 0; u < kF4Unroll; ++u) {
            const uint32_t c = cbase + u * kF4Threads + threadIdx.x;
            const float2 sr = tab[sb[u]];
            const uint32_t x[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
            // an element with all exponent bits set (inf, NaN): adding 0x0080 to its magnitude carries into bit 15
            const uint32_t nonfinite = (((x[0] & 0x7FFF7FFFu) + 0x00800080u) | ((x[1] & 0x7FFF7FFFu) + 0x00800080u) |
                                        ((x[2] & 0x7FFF7FFFu) + 0x00800080u) | ((x[3] & 0x7FFF7FFFu) + 0x00800080u)) & 0x80008000u;
            const uint32_t codes = quant_fp4_codes_f32(x, sr.x, sr.y);
            if (c < nchunks) {
                st_stream4(op + (size_t)c * 4, codes);
                // the rare cases redo the chunk with the per-tensor tier's templates and overwrite the word
                if (sr.y == 0.0f || zv[u] != 0.0f || nonfinite != 0) quant_fp4_chunk_general(ip + c, B.scale[t], zp, B.zdt, B.gs[t], op, c);
            }
        }
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
            return fail(CTB_EINVAL_ALIGN, "tensor %d: the bf16 side must be 16-byte, the packed side 4-byte aligned", base + i);
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
    int rc = fill(B, &r, &g, zp ? &z : nullptr, zdt, 0, 1, kF4Unit, 16, 4);
    if (rc) return rc;
    if (B.ustart[1] == 0) return CTB_OK;
    quant_fp4_g16_batch_kernel<<<grid_for(B.ustart[1], 1, 6), kF4Threads, 0, st>>>(B);
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
        int rc = fill(B, tensors, global_scales, zero_points, zp_dtype, base, n, kF4Unit, 16, 4);
        if (rc) return rc;
        if (B.ustart[n] == 0) continue;
        quant_fp4_g16_batch_kernel<<<grid_for(B.ustart[n], 1, 6), kF4Threads, 0, as_stream(stream)>>>(B);
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
