// Block-128 Hadamard rotation fused with int4 group-128 calibrate + quantize + pack, over a BATCH of
// tensors in one launch (the per-tensor loop of compressors/quantized_compressors/base.py:91 and
// transform/factory/base.py:95 turned into one grid).
//
// One 128-element Hadamard block is also one quantization group.  Two neighbouring lanes own a
// block: lane half h holds elements 16a + 8h + j (a, j = 0..7) as eight 16-byte chunks, so six of
// the seven butterfly stages (index bits 0-2 and 4-6) stay in registers and only bit 3 crosses
// lanes (one shuffle per element).  After the rotation the values are rounded to bf16 exactly as a
// separate rotate call would, the group maximum is reduced over the pair, and the int4 codes are
// produced with packed bf16x2 arithmetic (see quant_int4_word_bf16 / int4_pair_code).
//
// Work distribution: the blocks of all tensors form one index space (each tensor padded to a whole
// number of warps); the grid strides over it, so small tensors do not cost a launch or a tail each.
// The next block's 16-byte loads are issued before the current block is computed.
#pragma once

#include "ctb_codec.cuh"

namespace ctb {

constexpr int kRQThreads = 128;
constexpr int kBatchMax = 256;  // tensors per launch (the table travels as a kernel parameter)

struct RQBatch {
    int count;
    int64_t start[kBatchMax + 1];  // first global block index of each tensor (multiples of 16); start[count] = total
    int64_t nblocks[kBatchMax];    // real blocks of each tensor
    const void *x[kBatchMax];
    void *out[kBatchMax];          // packed words (QUANT) or rotated bf16 tensor (!QUANT)
    void *scale[kBatchMax];
};

template <typename A>
__device__ __forceinline__ A rq_shfl_xor(A v, int o) {
    if constexpr (sizeof(A) == 8) {
        int lo = __double2loint(v), hi = __double2hiint(v);
        lo = __shfl_xor_sync(0xFFFFFFFFu, lo, o);
        hi = __shfl_xor_sync(0xFFFFFFFFu, hi, o);
        return __hiloint2double(hi, lo);
    } else {
        return __shfl_xor_sync(0xFFFFFFFFu, v, o);
    }
}

// QUANT = false stops after the rotation and writes the rotated bf16 tensor (same arithmetic, so the
// fused output can be checked against quantize(rotate(x)) bit for bit in either precision).
template <typename A, bool QUANT>
__global__ void __launch_bounds__(kRQThreads, (sizeof(A) == 8 ? 2 : 4)) rotquant128_kernel(const __grid_constant__ RQBatch B, const int8_t *signs) {
    __shared__ float cs[128];  // sign_i / sqrt(128) (fp32 mode) or sign_i (fp64 mode)
    for (int i = threadIdx.x; i < 128; i += kRQThreads) {
        float s = signs ? (float)signs[i] : 1.0f;
        cs[i] = sizeof(A) == 8 ? s : s * 0.08838834764831845f;  // 1/sqrt(128)
    }
    __syncthreads();
    const int h = threadIdx.x & 1;
    const int64_t pairs = (int64_t)gridDim.x * (kRQThreads / 2);
    const int64_t total = B.start[B.count];

    int64_t g = (int64_t)blockIdx.x * (kRQThreads / 2) + (threadIdx.x >> 1);
    int t = 0;
    uint4 raw[8];
    auto fetch = [&](int64_t gi, int &ti, bool &live_out, int64_t &blk_out) {
        while (ti + 1 < B.count && gi >= B.start[ti + 1]) ++ti;
        blk_out = gi - B.start[ti];
        live_out = gi < total && blk_out < B.nblocks[ti];
#pragma unroll
        for (int a = 0; a < 8; ++a)
            raw[a] = live_out ? ld_stream((const char *)B.x[ti] + (blk_out * 16 + 2 * a + h) * 16) : make_uint4(0, 0, 0, 0);
    };
    bool live = false;
    int64_t blk = 0;
    if (g < total) fetch(g, t, live, blk);

    while (g < total) {
        A v[8][8];
#pragma unroll
        for (int a = 0; a < 8; ++a) {
            const uint32_t w[4] = {raw[a].x, raw[a].y, raw[a].z, raw[a].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                v[a][2 * k] = (A)__uint_as_float(w[k] << 16);
                v[a][2 * k + 1] = (A)__uint_as_float(w[k] & 0xFFFF0000u);
            }
        }
        // issue the next block's loads now; they complete while this block is computed
        const int cur_t = t;
        const bool cur_live = live;
        const int64_t cur_blk = blk;
        const int64_t gn = g + pairs;
        if (gn < total) fetch(gn, t, live, blk);

        // index bits 4..6 (a)
#pragma unroll
        for (int s = 1; s < 8; s <<= 1)
#pragma unroll
            for (int a = 0; a < 8; ++a)
                if ((a & s) == 0)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        A p = v[a][j], q = v[a | s][j];
                        v[a][j] = p + q;
                        v[a | s][j] = p - q;
                    }
        // index bits 0..2 (j)
#pragma unroll
        for (int a = 0; a < 8; ++a)
#pragma unroll
            for (int s = 1; s < 8; s <<= 1)
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if ((j & s) == 0) {
                        A p = v[a][j], q = v[a][j | s];
                        v[a][j] = p + q;
                        v[a][j | s] = p - q;
                    }
        // index bit 3 (the lane half)
        const A sg = h ? (A)-1 : (A)1;
#pragma unroll
        for (int a = 0; a < 8; ++a)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                A other = rq_shfl_xor<A>(v[a][j], 1);
                // exact: one rounding, same as other -/+ v.  The fused form is asked for by name: left to the
                // compiler, the float64 product by +-1 becomes a sign select per word in front of an add.
                if constexpr (sizeof(A) == 8) v[a][j] = __fma_rn(v[a][j], sg, other);
                else v[a][j] = __fmaf_rn(v[a][j], sg, other);
            }
        // normalise, apply the sign diagonal, round to bf16 (the rotated weight), group maximum
        uint32_t wq[8][4];  // rotated weights, packed bf16x2
        float amax = 0.0f;
#pragma unroll
        for (int a = 0; a < 8; ++a)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float f0, f1;
                const float c0 = cs[16 * a + 8 * h + 2 * k], c1 = cs[16 * a + 8 * h + 2 * k + 1];
                if constexpr (sizeof(A) == 8) {
                    // float64 quotient by sqrt(128), correctly rounded (reciprocal + one Markstein correction), then the
                    // float64 -> float32 -> bf16 cast chain of Tensor.to
                    const double c = sqrt(128.0), r = 1.0 / c;  // folded at compile time, both correctly rounded
                    double t0 = v[a][2 * k], t1 = v[a][2 * k + 1];
                    double q0 = t0 * r, q1 = t1 * r;
                    q0 = fma(fma(-q0, c, t0), r, q0);
                    q1 = fma(fma(-q1, c, t1), r, q1);
                    f0 = fmaf((float)q0, c0, 0.0f);
                    f1 = fmaf((float)q1, c1, 0.0f);
                } else {
                    f0 = fmaf((float)v[a][2 * k], c0, 0.0f);  // + 0.0: an exact zero is +0.0 in the reference's matmul
                    f1 = fmaf((float)v[a][2 * k + 1], c1, 0.0f);
                }
                amax = fmaxf(amax, fmaxf(fabsf(f0), fabsf(f1)));
                wq[a][k] = bf162_as_u32(__floats2bfloat162_rn(f0, f1));
            }
        if constexpr (!QUANT) {
            if (cur_live)
#pragma unroll
                for (int a = 0; a < 8; ++a)
                    st_stream((char *)B.out[cur_t] + (cur_blk * 16 + 2 * a + h) * 16, make_uint4(wq[a][0], wq[a][1], wq[a][2], wq[a][3]));
        } else {
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
            amax = round_to<CTB_BF16>(amax);  // max of the rounded values = rounded max (rounding is monotonic)
            // helpers.py:110,122: scale = bf16(amax / 7.5) clamped at fp32 eps
            const float s = fmaxf(round_to<CTB_BF16>(__fdiv_rn(amax, 7.5f)), 1.1920928955078125e-07f);
            const float r = __frcp_rn(s);
            if (cur_live && h == 0) ((__nv_bfloat16 *)B.scale[cur_t])[cur_blk] = __float2bfloat16_rn(s);
            uint32_t word[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) word[a] = quant_int4_word_bf16(wq[a], r, false, u32_as_bf162(0u));
            // word[a] covers elements 16a + 8h .. +7, i.e. output word 2a + h of the block's 16.  Swap so that
            // half 0 owns words 0..7 and half 1 words 8..15, then two 16-byte stores per lane.
            uint32_t mine[8];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                uint32_t send = h ? word[a] : word[a + 4];
                uint32_t got = __shfl_xor_sync(0xFFFFFFFFu, send, 1);
                uint32_t keep = h ? word[a + 4] : word[a];
                mine[2 * a] = h ? got : keep;      // even word of the pair comes from half 0
                mine[2 * a + 1] = h ? keep : got;  // odd word from half 1
            }
            if (cur_live) {
                char *o = (char *)B.out[cur_t] + cur_blk * 64 + h * 32;
                st_stream(o, make_uint4(mine[0], mine[1], mine[2], mine[3]));
                st_stream(o + 16, make_uint4(mine[4], mine[5], mine[6], mine[7]));
            }
        }
        g = gn;
    }
}

}  // namespace ctb
