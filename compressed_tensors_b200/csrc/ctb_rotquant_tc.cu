// Block-128 Hadamard rotation on the 5th-generation tensor cores (tcgen05 + TMEM), fused with the
// int4 group-128 calibrate + quantize + pack epilogue.
//
// A weight whose columns are a multiple of 128 is, in memory, a matrix of "blocks": row b of the
// [NB, 128] view is the b-th run of 128 consecutive elements, which is both one Hadamard block and
// one quantization group.  The rotation of 128 blocks is therefore one GEMM tile
//     D[128 blocks, 128] = A[128 blocks, 128] * B^T,     B[n][k] = signs[n] * H[n][k]  (+-1 in bf16)
// with bf16 operands (products are exact) and fp32 accumulators in TMEM.  TMEM lane m holds block m,
// so the epilogue thread that owns lane m has the whole quantization group in its registers: no
// shuffle is needed for the group maximum, and it writes the group's 16 packed words as 64
// contiguous bytes.
//
// Pipeline per SM (one persistent CTA, 10 warps):
//   warp 0      TMA producer : two 128B-swizzled [128 x 64] boxes per tile into a 4-stage smem ring
//   warp 1      MMA issuer   : 8 x tcgen05.mma (M128 N128 K16) per tile into one of two TMEM
//                              accumulators; tcgen05.commit frees the smem stage and publishes the tile
//   warps 2..9  epilogue     : two groups of 4 warps alternate tiles; tcgen05.ld the lane's 128 sums,
//                              release the accumulator, normalise, round to bf16, group max, scale,
//                              packed-bf16x2 int4 codes, 4 x 16-byte stores
// Every mbarrier wait is bounded (about a second of polling); on expiry an error word is set, all
// roles drain and the kernel returns CTB_ETIMEOUT to the host through the status buffer.
#include <cuda.h>

#include <atomic>

#include "ctb_codec.cuh"

namespace ctb {

constexpr int kTcThreads = 320;
constexpr int kTcStages = 4;
constexpr int kTcBatchMax = 256;
constexpr uint32_t kTcHalfBytes = 128 * 64 * 2;      // one 128B-swizzled [128 rows x 64 cols] bf16 box
constexpr uint32_t kTcTileBytes = 2 * kTcHalfBytes;  // 32 KiB: one A tile (or the B matrix)
constexpr size_t kTcSmemBytes = 1024 /*alignment slack*/ + kTcTileBytes * (1 + kTcStages) + 256;
constexpr long long kTcSpinCycles = 2000000000LL;    // default bound of every wait, in SM clocks

struct TCBatch {
    int count;
    int64_t tile_start[kTcBatchMax + 1];  // first global tile of each tensor; tile_start[count] = total
    int64_t row0[kTcBatchMax];            // row of the tensor's first block in the tensor map's [rows, 128] view
    void *out[kTcBatchMax];
    void *scale[kTcBatchMax];
    long long spin_cycles;                // bound of every device-side wait, in SM clocks
    int skip_tile;                        // >= 0: the producer leaves this tile's copy out (test hook: makes a wait run out)
};

// ---------------------------------------------------------------- PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when the budget ran out or another role already raised the error word
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *err, long long budget) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try(bar, parity)) {
        if (*err != 0) return false;
        if (clock64() - t0 > budget) {
            *err = 1;
            return false;
        }
    }
    return true;
}
// bounded wait that ignores the error word: used on the way out, for work this thread itself put in flight
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity, long long budget) {
    const long long t0 = clock64();
    while (!mbar_try(bar, parity) && clock64() - t0 < budget) {}
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major, 128-byte swizzle: rows 128 B apart inside an 8-row group, groups 1024 B apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                      // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                      // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                      // layout type SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace ctb

namespace ctb {

// QUANT = false writes the rotated bf16 tensor instead of codes (same arithmetic: used to check the fused
// output against quantize(rotate(x)) bit for bit).
template <bool QUANT>
__global__ void __launch_bounds__(kTcThreads, 1)
rotquant128_tc_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ TCBatch B, const int8_t *signs, int *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t base = (raw_u32 + 1023u) & ~1023u;  // the 128B swizzle pattern is defined on 1024-byte aligned tiles
    uint8_t *gbase = smem_raw + (base - raw_u32);
    const uint32_t b_smem = base;
    const uint32_t a_smem = base + kTcTileBytes;
    const uint32_t bars = base + kTcTileBytes * (1 + kTcStages);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kTcStages + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (2 * kTcStages + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (2 * kTcStages + 2 + b); };
    uint8_t *gctl = gbase + kTcTileBytes * (1 + kTcStages);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gctl + 8 * (2 * kTcStages + 4));
    volatile int *err = reinterpret_cast<volatile int *>(gctl + 8 * (2 * kTcStages + 4) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t total = B.tile_start[B.count];

    // ---- one-time setup: B = diag(signs) * H_128 in the swizzled K-major layout, barriers, TMEM
    for (int c = threadIdx.x; c < 128 * 16; c += kTcThreads) {
        const int n = c >> 4, ck = c & 15;
        const bool neg_row = signs != nullptr && signs[n] < 0;
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k0 = 8 * ck + 2 * j, k1 = k0 + 1;
            const uint32_t lo = ((__popc(n & k0) & 1) != 0) != neg_row ? 0xBF80u : 0x3F80u;
            const uint32_t hi = ((__popc(n & k1) & 1) != 0) != neg_row ? 0xBF80u : 0x3F80u;
            w[j] = lo | (hi << 16);
        }
        const int half = ck >> 3, c8 = ck & 7;
        *reinterpret_cast<uint4 *>(gbase + half * kTcHalfBytes + n * 128 + ((c8 ^ (n & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(accf_bar(b), 1);
            mbar_init(acce_bar(b), 4);  // one arrival per epilogue warp of the group
        }
        *err = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes of B -> visible to the tensor core
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            int t = 0;
            int64_t it = 0, skipped = -1;
            for (int64_t tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
                const int s = (int)(it % kTcStages);
                const uint32_t ph = (uint32_t)((it / kTcStages) & 1);
                if (!mbar_wait(empty_bar(s), ph ^ 1u, err, B.spin_cycles)) break;
                if (tile == (int64_t)B.skip_tile) { skipped = it; continue; }  // nothing is issued, nothing is in flight for this stage
                while (t + 1 < B.count && tile >= B.tile_start[t + 1]) ++t;
                const int64_t row = B.row0[t] + (tile - B.tile_start[t]) * 128;
                mbar_expect_tx(full_bar(s), kTcTileBytes);
                tma_load_2d(a_smem + s * kTcTileBytes, &tmap, full_bar(s), 0, (int)row);
                tma_load_2d(a_smem + s * kTcTileBytes + kTcHalfBytes, &tmap, full_bar(s), 64, (int)row);
            }
            if (*err != 0) {
                // let the copies still in flight land before the block gives its shared memory back
                // (default budget: a copy that was issued does land; the short budget of a test must not cut this wait)
                for (int64_t j = it > kTcStages ? it - kTcStages : 0; j < it; ++j)
                    if (j != skipped) mbar_drain(full_bar((int)(j % kTcStages)), (uint32_t)((j / kTcStages) & 1), kTcSpinCycles);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
            int64_t it = 0;
            for (int64_t tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
                const int s = (int)(it % kTcStages);
                const uint32_t ph = (uint32_t)((it / kTcStages) & 1);
                const int b = (int)(it & 1);
                const uint32_t bph = (uint32_t)((it >> 1) & 1);
                if (!mbar_wait(acce_bar(b), bph ^ 1u, err, B.spin_cycles)) break;
                if (!mbar_wait(full_bar(s), ph, err, B.spin_cycles)) break;
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t off = (k >> 2) * kTcHalfBytes + (k & 3) * 32;
                    umma_f16(tmem_base + b * 128, umma_desc_sw128(a_smem + s * kTcTileBytes + off), umma_desc_sw128(b_smem + off), idesc, k > 0);
                }
                umma_commit(empty_bar(s));  // the stage may be refilled once these MMAs have read it
                umma_commit(accf_bar(b));   // ... and the accumulator is complete
            }
            // On the error path nobody may be left to consume the last accumulator: wait here for the commit of
            // the MMAs already issued, so that none is in flight when the block frees its TMEM and shared memory.
            if (*err != 0 && it > 0) mbar_drain(accf_bar((int)((it - 1) & 1)), (uint32_t)(((it - 1) >> 1) & 1), kTcSpinCycles);
        }
    } else {
        // ------------------------------------------------ epilogue: two groups of four warps alternate tiles
        const int e = (warp - 2) >> 2;
        const int q = warp & 3;  // TMEM lanes [32q, 32q + 32) are the ones this warp may read
        int t = 0;
        int64_t it = 0;
        for (int64_t tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
            if ((int)(it & 1) != e) continue;
            const int b = e;
            const uint32_t bph = (uint32_t)((it >> 1) & 1);
            // the decision to leave is taken by the whole warp: tcgen05.ld below is a warp-wide (.sync.aligned) instruction
            if (!__all_sync(0xffffffffu, mbar_wait(accf_bar(b), bph, err, B.spin_cycles))) break;
            tc_fence_after();
            uint32_t acc[128];
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + b * 128;
            tmem_ld32(taddr + 0, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
            tmem_ld32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
            tmem_ld32(taddr + 64, *reinterpret_cast<uint32_t(*)[32]>(&acc[64]));
            tmem_ld32(taddr + 96, *reinterpret_cast<uint32_t(*)[32]>(&acc[96]));
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(b));  // the MMA warp may overwrite this accumulator now

            while (t + 1 < B.count && tile >= B.tile_start[t + 1]) ++t;
            const int64_t blk = (tile - B.tile_start[t]) * 128 + q * 32 + lane;
            uint32_t wq[64];  // the rotated weights of this block, packed bf16x2
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                const float f0 = fmaf(__uint_as_float(acc[2 * i]), 0.08838834764831845f, 0.0f);  // / sqrt(128); exact zeros come out +0.0
                const float f1 = fmaf(__uint_as_float(acc[2 * i + 1]), 0.08838834764831845f, 0.0f);
                amax = fmaxf(amax, fmaxf(fabsf(f0), fabsf(f1)));
                wq[i] = bf162_as_u32(__floats2bfloat162_rn(f0, f1));
            }
            if constexpr (!QUANT) {
                char *o = (char *)B.out[t] + blk * 256;
#pragma unroll
                for (int a = 0; a < 16; ++a) st_stream(o + 16 * a, make_uint4(wq[4 * a], wq[4 * a + 1], wq[4 * a + 2], wq[4 * a + 3]));
            } else {
                amax = round_to<CTB_BF16>(amax);
                const float s = fmaxf(round_to<CTB_BF16>(__fdiv_rn(amax, 7.5f)), 1.1920928955078125e-07f);  // helpers.py:110,122
                const float r = __frcp_rn(s);
                ((__nv_bfloat16 *)B.scale[t])[blk] = __float2bfloat16_rn(s);
                char *o = (char *)B.out[t] + blk * 64;
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    uint32_t word[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t w4[4] = {wq[16 * a + 4 * j], wq[16 * a + 4 * j + 1], wq[16 * a + 4 * j + 2], wq[16 * a + 4 * j + 3]};
                        word[j] = quant_int4_word_bf16(w4, r, false, u32_as_bf162(0u));
                    }
                    st_stream(o + 16 * a, make_uint4(word[0], word[1], word[2], word[3]));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
    }
    // a plain store: the status word may live in device memory or in page-locked host memory that the device reaches
    // over the bus, where it can be read without a copy on any stream
    if (threadIdx.x == 0 && *err != 0 && status != nullptr) {
        *reinterpret_cast<volatile int *>(status) = CTB_ETIMEOUT;
        __threadfence_system();
    }
}

}  // namespace ctb

// ---------------------------------------------------------------- host side

namespace ctb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Tensor-core path for a table of tensors.  Every tensor must be a whole number of 128-block tiles and
// sit a multiple of 256 bytes from the lowest one, so that ONE tensor map ([rows, 128] bf16 over the span
// of the table) addresses them all; only rows that belong to a tensor are ever requested.
int rotquant_tc_launch(const ctb_tensor_ref *tensors, int32_t count, const int8_t *signs, bool quant, int32_t *status, cudaStream_t st,
                       long long spin_cycles, int skip_tile) {
    if (count <= 0) return CTB_OK;
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return fail(CTB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    {
        // the opt-in to more than 48 KiB of dynamic shared memory is a per-device attribute of the function
        static std::atomic<bool> attr_set[64][2];
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return fail(CTB_ECUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
        const bool cacheable = dev >= 0 && dev < 64;
        if (!cacheable || !attr_set[dev][quant].load(std::memory_order_acquire)) {
            e = quant ? cudaFuncSetAttribute(rotquant128_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBytes)
                      : cudaFuncSetAttribute(rotquant128_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBytes);
            if (e != cudaSuccess) return fail(CTB_ECUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
            if (cacheable) attr_set[dev][quant].store(true, std::memory_order_release);
        }
    }
    static thread_local TCBatch B;
    B.spin_cycles = spin_cycles > 0 ? spin_cycles : kTcSpinCycles;
    B.skip_tile = skip_tile;
    for (int32_t base_i = 0; base_i < count; base_i += kTcBatchMax) {
        const int32_t n = count - base_i < kTcBatchMax ? count - base_i : kTcBatchMax;
        uintptr_t lo = UINTPTR_MAX, hi = 0;
        for (int32_t i = 0; i < n; ++i) {
            const ctb_tensor_ref &t = tensors[base_i + i];
            if (!t.in || !t.out || (quant && !t.scale)) return fail(CTB_EINVAL_NULL, "tensor %d has a null buffer", base_i + i);
            if (t.rows <= 0 || t.cols <= 0 || t.cols % 128 || (t.rows * t.cols) % (128 * 128))
                return fail(CTB_EUNSUPPORTED, "tensor %d: the tensor-core path takes whole tiles of 128 blocks of 128 elements", base_i + i);
            const uintptr_t a = reinterpret_cast<uintptr_t>(t.in);
            lo = a < lo ? a : lo;
            hi = a + (uintptr_t)t.rows * t.cols * 2 > hi ? a + (uintptr_t)t.rows * t.cols * 2 : hi;
        }
        int64_t tiles = 0;
        for (int32_t i = 0; i < n; ++i) {
            const ctb_tensor_ref &t = tensors[base_i + i];
            const uintptr_t a = reinterpret_cast<uintptr_t>(t.in);
            if ((a - lo) % 256 || !aligned16(t.out)) return fail(CTB_EINVAL_ALIGN, "tensor %d: inputs must be 256 bytes apart modulo alignment, outputs 16-byte aligned", base_i + i);
            B.tile_start[i] = tiles;
            B.row0[i] = (int64_t)((a - lo) / 256);
            B.out[i] = t.out;
            B.scale[i] = t.scale;
            tiles += t.rows * t.cols / (128 * 128);
        }
        B.count = n;
        B.tile_start[n] = tiles;
        const uint64_t rows = (hi - lo) / 256;
        if (rows >= (1ull << 31)) return fail(CTB_EUNSUPPORTED, "the table spans more than 2^31 blocks");
        CUtensorMap map;
        const cuuint64_t dims[2] = {128, rows};
        const cuuint64_t strides[1] = {256};
        const cuuint32_t box[2] = {64, 128};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, reinterpret_cast<void *>(lo), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CTB_ECUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
        const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
        if (quant) rotquant128_tc_kernel<true><<<grid, kTcThreads, kTcSmemBytes, st>>>(map, B, signs, status);
        else rotquant128_tc_kernel<false><<<grid, kTcThreads, kTcSmemBytes, st>>>(map, B, signs, status);
        int rc = after_launch("rotquant128_tc_kernel");
        if (rc) return rc;
    }
    return CTB_OK;
}

}  // namespace ctb
