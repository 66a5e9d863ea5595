// Shared host/device helpers for the ctb200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ctb200.h"

namespace ctb {

// ---------------------------------------------------------------- host side

void set_error(const char *fmt, ...);
int fail(int status, const char *fmt, ...);
void count_launch();
int sm_count();

// call after every launch: turns a launch failure into CTB_ECUDA and counts the launch
int after_launch(const char *what);

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int dtype_size(int dt) {
    switch (dt) {
    case CTB_BF16: case CTB_F16: return 2;
    case CTB_F32: case CTB_I32: return 4;
    case CTB_F64: case CTB_I64: return 8;
    case CTB_I8: case CTB_E4M3: case CTB_U8: return 1;
    default: return 0;
    }
}

inline bool is_float_dtype(int dt) { return dt == CTB_BF16 || dt == CTB_F16 || dt == CTB_F32; }

// torch's promotion between two floating tensors of dim > 0
inline int promote(int a, int b) { return a == b ? a : CTB_F32; }

// grid for a grid-stride kernel: enough blocks to cover `work` units of `per_block`, capped at a
// whole number of waves of resident blocks
// ctb_fp4_batch.cu: NVFP4 quantize + pack of ONE tensor with given e4m3 group-16 scales (the whole-shard kernel on a
// table of one entry); x 16-byte and out 8-byte aligned, cols % 16 == 0
int quant_fp4_g16_one(const void *x, const void *scale, const float *gs, const void *zp, int zdt, int64_t rows, int64_t cols, void *out,
                      cudaStream_t st);

inline int grid_for(int64_t work, int64_t per_block, int blocks_per_sm) {
    int64_t need = cdiv(work, per_block);
    int64_t cap = (int64_t)sm_count() * blocks_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

// ---------------------------------------------------------------- device side

#ifdef __CUDACC__

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// round-to-nearest-even to the storage dtype and back to fp32 (the rounding torch applies after
// every elementwise op on a reduced-precision tensor)
template <int DT>
__device__ __forceinline__ float round_to(float v) {
    if constexpr (DT == CTB_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    else if constexpr (DT == CTB_F16) return __half2float(__float2half_rn(v));
    else return v;
}

__device__ __forceinline__ float round_to_rt(int dt, float v) {
    if (dt == CTB_BF16) return round_to<CTB_BF16>(v);
    if (dt == CTB_F16) return round_to<CTB_F16>(v);
    return v;
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
    return __half2float(__half(h));
}

// Tensor.to(float8_e4m3fn): round-to-nearest-even; NaN keeps its sign bit (0x7f | sign).
// Callers clamp to +-448 first, as the reference does, so the saturating convert never saturates.
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
    uint8_t b = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    if (v != v) b = 0x7F | ((__float_as_uint(v) >> 24) & 0x80);
    return b;
}

// scalar load of element i of a typed buffer as fp32 (generic paths and qparams)
__device__ __forceinline__ float load_f32(const void *p, int dt, int64_t i) {
    switch (dt) {
    case CTB_BF16: return bf16_bits_to_f32(((const uint16_t *)p)[i]);
    case CTB_F16: return __half2float(((const __half *)p)[i]);
    case CTB_F32: return ((const float *)p)[i];
    case CTB_I8: return (float)((const int8_t *)p)[i];
    case CTB_U8: return (float)((const uint8_t *)p)[i];
    case CTB_E4M3: return e4m3_to_f32(((const uint8_t *)p)[i]);
    case CTB_F64: return (float)((const double *)p)[i];
    default: return 0.0f;
    }
}

__device__ __forceinline__ void store_f32(void *p, int dt, int64_t i, float v) {
    switch (dt) {
    case CTB_BF16: ((__nv_bfloat16 *)p)[i] = __float2bfloat16_rn(v); break;
    case CTB_F16: ((__half *)p)[i] = __float2half_rn(v); break;
    case CTB_F32: ((float *)p)[i] = v; break;
    case CTB_I8: ((int8_t *)p)[i] = (int8_t)(int)v; break;
    case CTB_E4M3: ((uint8_t *)p)[i] = f32_to_e4m3(v); break;
    case CTB_F64: ((double *)p)[i] = (double)v; break;
    default: break;
    }
}

// Correctly rounded fp32 quotient x / s from r = __frcp_rn(s): one multiply, one exact residual,
// one corrective fma (Markstein).  Falls back to the first product where the residual is not
// finite (x or s infinite, s == 0), which is what IEEE division returns there, and for x == +-0, whose
// residual (+0) + x would turn a negative zero quotient into +0.
__device__ __forceinline__ float div_by_rcp(float x, float s, float r) {
    float q0 = x * r;
    float e = fmaf(-q0, s, x);
    float q1 = fmaf(e, r, q0);
    return (fabsf(q1) <= 3.0e38f && x != 0.0f) ? q1 : q0;
}

// torch.clamp: NaN passes through
__device__ __forceinline__ float clamp_nan(float v, float lo, float hi) { return (v != v) ? v : fminf(fmaxf(v, lo), hi); }

// streaming 128-bit global accesses: every byte of these tensors is touched once
__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream8(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream4(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(void *p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_stream8(void *p, uint2 v) {
    asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
__device__ __forceinline__ void st_stream4(void *p, uint32_t v) {
    asm volatile("st.global.cs.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

#endif  // __CUDACC__

}  // namespace ctb
