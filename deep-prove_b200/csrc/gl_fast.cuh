// Device-only Goldilocks arithmetic for the hot kernels.
//
// The straightforward routines in field_gl.cuh keep every value canonical and
// spend most of their instructions on compares and conditional subtracts: the
// ALU pipe, not the multiplier, limits the kernels.  Here values are "loose":
// any 64-bit representative of the residue.  Rules (p = 2^64 - 2^32 + 1,
// EPS = 2^32 - 1 = 2^64 mod p):
//   add_c(a, c) / sub_c(a, c): a loose, c canonical -> loose, one correction
//   mul_wide: 64x64 -> 128 by four 32x32 multiply-adds
//   reduce128: 128 bits -> loose (2^64 = EPS, 2^96 = -1)
//   Acc160: sums of 128-bit products without reduction; one reduction at the
//           end of the thread's loop (2^128 = -2^32 mod p)
//   canon: loose -> canonical, before storing or publishing
#pragma once
#include <cstdint>

#include "field_gl.cuh"

namespace dpb {
namespace glf {

// The corrections below use the carry flag and a mask (all ones when the flag
// is set: subc m, 0, 0 after a subtraction, addc + neg after an addition) instead of a 64-bit compare and a
// predicated add: on sm_100a a compare-and-correct costs about twice the
// dispatch cycles of the five carry-chained 32-bit adds (measured 12-14 vs 6-8).

// a >= p  <=>  a + EPS carries out of 64 bits; then a + EPS (mod 2^64) = a - p
__device__ __forceinline__ uint64_t canon(uint64_t a) {
    uint64_t d;
    asm("{ .reg .u32 a0,a1,t,m; mov.b64 {a0,a1}, %1;\n\t"
        "add.cc.u32 t, a0, 0xffffffff; addc.cc.u32 t, a1, 0; addc.u32 m, 0, 0; neg.s32 m, m;\n\t"
        "add.cc.u32 a0, a0, m; addc.u32 a1, a1, 0; mov.b64 %0, {a0,a1}; }"
        : "=l"(d)
        : "l"(a));
    return d;
}

// a loose, c canonical: a + c - 2^64 < p, so adding EPS after a carry cannot carry again
__device__ __forceinline__ uint64_t add_c(uint64_t a, uint64_t c) {
    uint64_t d;
    asm("{ .reg .u32 a0,a1,c0,c1,m; mov.b64 {a0,a1}, %1; mov.b64 {c0,c1}, %2;\n\t"
        "add.cc.u32 a0, a0, c0; addc.cc.u32 a1, a1, c1; addc.u32 m, 0, 0; neg.s32 m, m;\n\t"
        "add.cc.u32 a0, a0, m; addc.u32 a1, a1, 0; mov.b64 %0, {a0,a1}; }"
        : "=l"(d)
        : "l"(a), "l"(c));
    return d;
}
// a loose, c canonical: after a borrow the wrapped value is >= 2^32, so subtracting EPS is safe
__device__ __forceinline__ uint64_t sub_c(uint64_t a, uint64_t c) {
    uint64_t d;
    asm("{ .reg .u32 a0,a1,c0,c1,m; mov.b64 {a0,a1}, %1; mov.b64 {c0,c1}, %2;\n\t"
        "sub.cc.u32 a0, a0, c0; subc.cc.u32 a1, a1, c1; subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 a0, a0, m; subc.u32 a1, a1, 0; mov.b64 %0, {a0,a1}; }"
        : "=l"(d)
        : "l"(a), "l"(c));
    return d;
}

__device__ __forceinline__ void mul_wide(uint64_t a, uint64_t b, uint64_t& lo, uint64_t& hi) {
    const uint32_t a0 = (uint32_t)a, a1 = (uint32_t)(a >> 32);
    const uint32_t b0 = (uint32_t)b, b1 = (uint32_t)(b >> 32);
    const uint64_t t0 = (uint64_t)a0 * b0;
    const uint64_t t1 = (uint64_t)a0 * b1 + (t0 >> 32);        // fits: (2^32-1)^2 + 2^32 - 1 < 2^64
    const uint64_t t2 = (uint64_t)a1 * b0 + (uint32_t)t1;
    const uint64_t t3 = (uint64_t)a1 * b1 + (t1 >> 32);
    hi = t3 + (t2 >> 32);
    lo = (t2 << 32) | (uint32_t)t0;
}

// lo + 2^64 hi = lo - hh + hl * EPS (hi = 2^32 hh + hl): subtract hh (borrow
// -> subtract EPS), add hl * EPS = (hl << 32) - hl built with one sub/subc
// (carry -> add EPS); neither correction can wrap a second time.
__device__ __forceinline__ uint64_t reduce128(uint64_t lo, uint64_t hi) {
    uint64_t d;
    asm("{ .reg .u32 l0,l1,h0,h1,m,y0,y1; mov.b64 {l0,l1}, %1; mov.b64 {h0,h1}, %2;\n\t"
        "sub.cc.u32 l0, l0, h1; subc.cc.u32 l1, l1, 0; subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 l0, l0, m; subc.u32 l1, l1, 0;\n\t"
        "sub.cc.u32 y0, 0, h0; subc.u32 y1, h0, 0;\n\t"
        "add.cc.u32 l0, l0, y0; addc.cc.u32 l1, l1, y1; addc.u32 m, 0, 0; neg.s32 m, m;\n\t"
        "add.cc.u32 l0, l0, m; addc.u32 l1, l1, 0; mov.b64 %0, {l0,l1}; }"
        : "=l"(d)
        : "l"(lo), "l"(hi));
    return d;
}

__device__ __forceinline__ uint64_t mul(uint64_t a, uint64_t b) {
    uint64_t lo, hi;
    mul_wide(a, b, lo, hi);
    return reduce128(lo, hi);
}

// 7 * a as a loose residue (a loose)
__device__ __forceinline__ uint64_t mul7(uint64_t a) {
    const uint64_t t0 = (uint64_t)(uint32_t)a * 7u;
    const uint64_t t1 = (uint64_t)(uint32_t)(a >> 32) * 7u + (t0 >> 32);
    const uint64_t lo = (t1 << 32) | (uint32_t)t0;
    const uint64_t hi = t1 >> 32;              // < 7
    const uint64_t add = (hi << 32) - hi;      // hi * EPS, canonical
    return add_c(lo, add);
}

// 160-bit accumulator of 128-bit products
struct Acc160 {
    uint64_t lo, hi;
    uint32_t ov;
};
__device__ __forceinline__ Acc160 acc_zero() {
    Acc160 a;
    a.lo = 0;
    a.hi = 0;
    a.ov = 0;
    return a;
}
__device__ __forceinline__ void acc_add(Acc160& a, uint64_t lo, uint64_t hi) {
    asm("add.cc.u64 %0, %0, %3;\n\t"
        "addc.cc.u64 %1, %1, %4;\n\t"
        "addc.u32 %2, %2, 0;"
        : "+l"(a.lo), "+l"(a.hi), "+r"(a.ov)
        : "l"(lo), "l"(hi));
}
__device__ __forceinline__ void acc_mac(Acc160& a, uint64_t x, uint64_t y) {
    uint64_t lo, hi;
    mul_wide(x, y, lo, hi);
    acc_add(a, lo, hi);
}
// acc += 7 * (x * y), the non-residue of the quadratic extension
__device__ __forceinline__ void acc_mac7(Acc160& a, uint64_t x, uint64_t y) {
    uint64_t lo, hi;
    mul_wide(x, y, lo, hi);
    const uint64_t t0 = (uint64_t)(uint32_t)lo * 7u;
    const uint64_t t1 = (uint64_t)(uint32_t)(lo >> 32) * 7u + (t0 >> 32);
    const uint64_t t2 = (uint64_t)(uint32_t)hi * 7u + (t1 >> 32);
    const uint64_t t3 = (uint64_t)(uint32_t)(hi >> 32) * 7u + (t2 >> 32);
    const uint64_t l7 = (t1 << 32) | (uint32_t)t0;
    const uint64_t h7 = (t3 << 32) | (uint32_t)t2;
    asm("add.cc.u64 %0, %0, %3;\n\t"
        "addc.cc.u64 %1, %1, %4;\n\t"
        "addc.u32 %2, %2, %5;"
        : "+l"(a.lo), "+l"(a.hi), "+r"(a.ov)
        : "l"(l7), "l"(h7), "r"((uint32_t)(t3 >> 32)));
}
// loose residue of the accumulator: lo + 2^64 hi - 2^32 ov
__device__ __forceinline__ uint64_t acc_reduce(const Acc160& a) {
    return sub_c(reduce128(a.lo, a.hi), (uint64_t)a.ov << 32);
}

// ---- quadratic extension, loose components -------------------------------
struct L2 {
    uint64_t c0, c1;
};

// (a0 + a1 X)(b0 + b1 X) with X^2 = 7: two lazy sums, two reductions
__device__ __forceinline__ L2 mul2(const L2& a, const L2& b) {
    Acc160 s0 = acc_zero(), s1 = acc_zero();
    acc_mac(s0, a.c0, b.c0);
    acc_mac7(s0, a.c1, b.c1);
    acc_mac(s1, a.c0, b.c1);
    acc_mac(s1, a.c1, b.c0);
    L2 r;
    r.c0 = acc_reduce(s0);
    r.c1 = acc_reduce(s1);
    return r;
}

}  // namespace glf
}  // namespace dpb
