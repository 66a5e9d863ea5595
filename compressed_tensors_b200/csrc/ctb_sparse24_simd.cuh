// 2:4 keep masks for several runs of four at once, with the magnitudes of the runs held as SIMD lanes of
// 32-bit words (sparse_24_bitmask.py:244-256: abs().topk(2) over runs of four).
//
// "Transposed" layout: word X_i holds element i of every run (four 8-bit lanes for the int8 view, two 16-bit
// lanes for bf16 / fp16).  All comparisons are lane-wise subtractions whose borrow lands in the lane's top bit,
// the selection rule is bitwise logic on those top bits, and only the four final keep masks are widened to whole
// lanes.  The rule itself (ties go to the higher index, except when element 0 is strictly largest and the second
// place is tied) is the one keep24() states for scalars; the two are compared on every weak ordering by the tests.
//
// The functions are __host__ __device__ so that the bit logic can be checked exhaustively without a GPU.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define CTB_HD __host__ __device__ __forceinline__
#else
#define CTB_HD inline
#endif

namespace ctb {

// byte permute of the 8 bytes {a (0-3), b (4-7)}; selector nibble bit 3 replicates the byte's top bit instead
CTB_HD uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
#if defined(__CUDA_ARCH__)
    uint32_t r;  // the PTX instruction itself: the __byte_perm intrinsic documents only the three index bits
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
#else
    const uint64_t src = ((uint64_t)b << 32) | a;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) {
        const uint32_t n = (sel >> (4 * i)) & 0xFu;
        uint32_t byte = (uint32_t)(src >> (8 * (n & 7u))) & 0xFFu;
        if (n & 8u) byte = (byte & 0x80u) ? 0xFFu : 0u;
        r |= byte << (8 * i);
    }
    return r;
#endif
}

struct Keep4 {
    uint32_t k0, k1, k2, k3;  // per lane: all ones where element i of the run is kept
};

// The selection rule on "greater or equal" bits.  g_ij has the lane's top bit set where key_i >= key_j; only the
// top bit of each lane of the results is meaningful.
CTB_HD Keep4 keep24_rule(uint32_t g10, uint32_t g20, uint32_t g30, uint32_t g21, uint32_t g31, uint32_t g32, uint32_t g12, uint32_t g13,
                         uint32_t g23) {
    // i beats j (i < j) iff key_i > key_j, i.e. not g_ji; j beats i iff g_ji.  Keep whoever beats two others.
    const uint32_t n10 = ~g10, n20 = ~g20, n30 = ~g30, n21 = ~g21, n31 = ~g31, n32 = ~g32;
    uint32_t k0 = (n10 & n20) | (n10 & n30) | (n20 & n30);
    uint32_t k1 = (g10 & n21) | (g10 & n31) | (n21 & n31);
    uint32_t k2 = (g20 & g21) | (g20 & n32) | (g21 & n32);
    uint32_t k3 = (g30 & g31) | (g30 & g32) | (g31 & g32);
    // element 0 strictly largest: the runner-up among 1..3 is the largest of them, ties resolved per tie set
    const uint32_t e = n10 & n20 & n30;
    const uint32_t e1 = g12 & g13, e2 = g21 & g23, e3 = g31 & g32;  // element is a maximum of {1, 2, 3}
    const uint32_t x1 = e1 & ~(e2 & e3);
    const uint32_t x2 = e2 & ~x1;
    const uint32_t x3 = e3 & ~e1 & ~e2;
    k1 = (e & x1) | (~e & k1);
    k2 = (e & x2) | (~e & k2);
    k3 = (e & x3) | (~e & k3);
    return {k0, k1, k2, k3};
}

// ---- four runs of int8-view elements (int8, uint8 and e4m3 tensors are ranked through torch's int8 abs, where
// abs(-128) stays -128 and therefore ranks lowest)

// a - b, placed on the multiply-add pipe on the GPU: the selection logic saturates the integer ALU pipe, and the
// dozen lane-wise subtractions and additions per 16 elements are the part of it that can run elsewhere
CTB_HD uint32_t sub_fma_pipe(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(0xFFFFFFFFu), "r"(a));
    return r;
#else
    return a - b;
#endif
}
CTB_HD uint32_t add_fma_pipe(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(1u), "r"(a));
    return r;
#else
    return a + b;
#endif
}

// lane-wise magnitude in torch's int8 arithmetic: m = abs_int8(v) as a byte, i.e. 0..127, and 0x80 for v = -128
// (which therefore has to rank LOWEST: see ge_abs8x4)
CTB_HD uint32_t abs_i8x4(uint32_t v) {
    const uint32_t s = prmt(v, 0, 0xBA98);  // 0xFF in negative lanes
    const uint32_t x = v ^ s;               // ~v in negative lanes; the lane's top bit is now clear
    return add_fma_pipe(x, s & 0x01010101u);  // + 1 completes the negation; the sum stays inside the lane
}

// top bit of each 8-bit lane set where rank(a) >= rank(b), for magnitudes from abs_i8x4 (the rank of a magnitude
// is the magnitude with its top bit flipped, so that 0x80 sorts below 0); ah = a | 0x80.., bl = b & 0x7F..
CTB_HD uint32_t ge_abs8x4(uint32_t a, uint32_t b, uint32_t ah, uint32_t bl) {
    const uint32_t t = sub_fma_pipe(ah, bl);  // per lane: 0x80 + (a & 0x7F) - (b & 0x7F), no borrow between lanes
    // with A = ~a, B = ~b the rank top bits:  (A & ~B) | (~(A ^ B) & t)
    return (~a & b) | (~(a ^ b) & t);
}

CTB_HD Keep4 keep24_u8x4(uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
    const uint32_t u0 = abs_i8x4(x0), u1 = abs_i8x4(x1), u2 = abs_i8x4(x2), u3 = abs_i8x4(x3);
    const uint32_t H = 0x80808080u;
    const uint32_t h1 = u1 | H, h2 = u2 | H, h3 = u3 | H;
    const uint32_t l0 = u0 & ~H, l1 = u1 & ~H, l2 = u2 & ~H, l3 = u3 & ~H;
    Keep4 k = keep24_rule(ge_abs8x4(u1, u0, h1, l0), ge_abs8x4(u2, u0, h2, l0), ge_abs8x4(u3, u0, h3, l0), ge_abs8x4(u2, u1, h2, l1),
                          ge_abs8x4(u3, u1, h3, l1), ge_abs8x4(u3, u2, h3, l2), ge_abs8x4(u1, u2, h1, l2), ge_abs8x4(u1, u3, h1, l3),
                          ge_abs8x4(u2, u3, h2, l3));
    k.k0 = prmt(k.k0, 0, 0xBA98);
    k.k1 = prmt(k.k1, 0, 0xBA98);
    k.k2 = prmt(k.k2, 0, 0xBA98);
    k.k3 = prmt(k.k3, 0, 0xBA98);
    return k;
}

// 4 x 4 byte transpose: w_g = the four elements of run g  ->  x_i = element i of runs 0..3 (and back: it is an involution)
CTB_HD void transpose_u8x4(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t &x0, uint32_t &x1, uint32_t &x2, uint32_t &x3) {
    const uint32_t t0 = prmt(w0, w1, 0x5140), t1 = prmt(w2, w3, 0x5140);
    const uint32_t t2 = prmt(w0, w1, 0x7362), t3 = prmt(w2, w3, 0x7362);
    x0 = prmt(t0, t1, 0x5410);
    x1 = prmt(t0, t1, 0x7632);
    x2 = prmt(t2, t3, 0x5410);
    x3 = prmt(t2, t3, 0x7632);
}

// Sixteen int8-view elements (four runs, two bitmask bytes): kept values in column order and the bitmask bytes.
CTB_HD void sparse24_pack_u8x16(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t &val0, uint32_t &val1, uint32_t &mask16) {
    uint32_t x0, x1, x2, x3;
    transpose_u8x4(w0, w1, w2, w3, x0, x1, x2, x3);
    const Keep4 k = keep24_u8x4(x0, x1, x2, x3);
    // per run: the lower and the upper of its two kept elements
    const uint32_t lo = (k.k0 & x0) | (~k.k0 & ((k.k1 & x1) | (~k.k1 & x2)));
    const uint32_t hi = (k.k3 & x3) | (~k.k3 & ((k.k2 & x2) | (~k.k2 & x1)));
    val0 = prmt(lo, hi, 0x5140);  // lo0 hi0 lo1 hi1
    val1 = prmt(lo, hi, 0x7362);  // lo2 hi2 lo3 hi3
    const uint32_t nib = (k.k0 & 0x01010101u) | (k.k1 & 0x02020202u) | (k.k2 & 0x04040404u) | (k.k3 & 0x08080808u);  // lane g: nibble of run g
    const uint32_t by = nib | (nib >> 4);  // lane 0: runs 0, 1; lane 2: runs 2, 3
    mask16 = prmt(by, 0, 0x4420);
}

// get_24_bytemasks for the same sixteen elements: one 0/1 byte per element, run g in word g
CTB_HD void sparse24_bytemask_u8x16(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t &o0, uint32_t &o1, uint32_t &o2, uint32_t &o3) {
    uint32_t x0, x1, x2, x3;
    transpose_u8x4(w0, w1, w2, w3, x0, x1, x2, x3);
    const Keep4 k = keep24_u8x4(x0, x1, x2, x3);
    transpose_u8x4(k.k0 & 0x01010101u, k.k1 & 0x01010101u, k.k2 & 0x01010101u, k.k3 & 0x01010101u, o0, o1, o2, o3);
}

// ---- two runs of 16-bit float elements (bf16 / fp16): keys are the 15 magnitude bits

CTB_HD Keep4 keep24_u16x2(uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3) {
    const uint32_t M = 0x7FFF7FFFu, H = 0x80008000u;
    const uint32_t u0 = x0 & M, u1 = x1 & M, u2 = x2 & M, u3 = x3 & M;
    const uint32_t h1 = u1 | H, h2 = u2 | H, h3 = u3 | H;
    // (a | H) - b keeps the lane's top bit iff a >= b (both below 0x8000); no borrow leaves a lane
    Keep4 k = keep24_rule(sub_fma_pipe(h1, u0), sub_fma_pipe(h2, u0), sub_fma_pipe(h3, u0), sub_fma_pipe(h2, u1), sub_fma_pipe(h3, u1),
                          sub_fma_pipe(h3, u2), sub_fma_pipe(h1, u2), sub_fma_pipe(h1, u3), sub_fma_pipe(h2, u3));
    k.k0 = prmt(k.k0, 0, 0xBB99);
    k.k1 = prmt(k.k1, 0, 0xBB99);
    k.k2 = prmt(k.k2, 0, 0xBB99);
    k.k3 = prmt(k.k3, 0, 0xBB99);
    return k;
}

// Eight 16-bit elements (two runs, one bitmask byte): w0 w1 = run a, w2 w3 = run b
CTB_HD void sparse24_pack_u16x8(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t &val0, uint32_t &val1, uint32_t &mask8) {
    const uint32_t x0 = prmt(w0, w2, 0x5410), x1 = prmt(w0, w2, 0x7632);  // element 0 / 1 of runs a, b
    const uint32_t x2 = prmt(w1, w3, 0x5410), x3 = prmt(w1, w3, 0x7632);
    const Keep4 k = keep24_u16x2(x0, x1, x2, x3);
    const uint32_t lo = (k.k0 & x0) | (~k.k0 & ((k.k1 & x1) | (~k.k1 & x2)));
    const uint32_t hi = (k.k3 & x3) | (~k.k3 & ((k.k2 & x2) | (~k.k2 & x1)));
    val0 = prmt(lo, hi, 0x5410);  // lo_a hi_a
    val1 = prmt(lo, hi, 0x7632);  // lo_b hi_b
    const uint32_t nib = (k.k0 & 0x00010001u) | (k.k1 & 0x00020002u) | (k.k2 & 0x00040004u) | (k.k3 & 0x00080008u);
    mask8 = (nib | (nib >> 12)) & 0xFFu;
}

// get_24_bytemasks for the same eight elements: one 0/1 byte per element, run a in o0 and run b in o1
CTB_HD void sparse24_bytemask_u16x8(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t &o0, uint32_t &o1) {
    const uint32_t x0 = prmt(w0, w2, 0x5410), x1 = prmt(w0, w2, 0x7632);
    const uint32_t x2 = prmt(w1, w3, 0x5410), x3 = prmt(w1, w3, 0x7632);
    const Keep4 k = keep24_u16x2(x0, x1, x2, x3);
    const uint32_t t0 = prmt(k.k0, k.k1, 0x6420), t1 = prmt(k.k2, k.k3, 0x6420);  // low bytes of both lanes of each mask
    o0 = prmt(t0, t1, 0x6420) & 0x01010101u;
    o1 = prmt(t0, t1, 0x7531) & 0x01010101u;
}

}  // namespace ctb
