// Goldilocks arithmetic on explicit 32-bit words, for the hottest kernels.
//
// Instruction counts measured on sm_100a show that a 64-bit formulation pays
// for packing and unpacking register pairs around every multiply: the C
// version of a 64x64 product issues ten multiply-pipe instructions where four
// are needed.  Measured issue costs per warp instruction: a 32x32->64 multiply
// (with or without a 64-bit addend and carry) about four cycles, a 32-bit
// multiply, logic op, shift or compare about two, a carry-chained add about
// one.  So the cheapest code is: exactly four wide multiplies per product, the
// additions of a sum of products folded into the multiplies' addends
// (mad.lo.cc / madc.hi.cc pairs on aligned word pairs become one instruction),
// everything else carry-chained 32-bit adds with corrections driven by the
// carry flag and a mask — no compares, no predicates, no shifts.
//
// Values are "loose" (any 64-bit representative of the residue) unless a
// comment says canonical.  p = 2^64 - 2^32 + 1, EPS = 2^32 - 1 = 2^64 mod p,
// 2^96 = -1, 2^128 = -2^32 (mod p).
#pragma once
#include <cstdint>

#include "field_gl.cuh"

namespace dpb {
namespace glw {

struct W {
    uint32_t lo, hi;
};
__host__ __device__ __forceinline__ W make_w(uint32_t lo, uint32_t hi) {
    W r;
    r.lo = lo;
    r.hi = hi;
    return r;
}
__device__ __forceinline__ uint64_t to_u64(const W& a) { return (uint64_t)a.lo | ((uint64_t)a.hi << 32); }

// a loose, c canonical -> loose.  A carry means the true sum is s + 2^64 = s + EPS;
// s < p then, so adding EPS cannot carry again.
__device__ __forceinline__ W add_c(const W& a, const W& c) {
    W d;
    asm("{ .reg .u32 m;\n\t"
        "add.cc.u32 %0, %2, %4; addc.cc.u32 %1, %3, %5; addc.u32 m, 0, 0; neg.s32 m, m;\n\t"
        "add.cc.u32 %0, %0, m; addc.u32 %1, %1, 0; }"
        : "=&r"(d.lo), "=&r"(d.hi)
        : "r"(a.lo), "r"(a.hi), "r"(c.lo), "r"(c.hi));
    return d;
}
// a loose, c canonical -> loose.  A borrow means the true difference is d - 2^64 = d - EPS;
// d >= 2^32 then, so subtracting EPS cannot borrow again.
__device__ __forceinline__ W sub_c(const W& a, const W& c) {
    W d;
    asm("{ .reg .u32 m;\n\t"
        "sub.cc.u32 %0, %2, %4; subc.cc.u32 %1, %3, %5; subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 %0, %0, m; subc.u32 %1, %1, 0; }"
        : "=&r"(d.lo), "=&r"(d.hi)
        : "r"(a.lo), "r"(a.hi), "r"(c.lo), "r"(c.hi));
    return d;
}
// loose -> canonical: a >= p  <=>  a + EPS carries; then a + EPS (mod 2^64) = a - p
__device__ __forceinline__ W canon(const W& a) {
    W d;
    asm("{ .reg .u32 t, m;\n\t"
        "add.cc.u32 t, %2, 0xffffffff; addc.cc.u32 t, %3, 0; addc.u32 m, 0, 0; neg.s32 m, m;\n\t"
        "add.cc.u32 %0, %2, m; addc.u32 %1, %3, 0; }"
        : "=&r"(d.lo), "=&r"(d.hi)
        : "r"(a.lo), "r"(a.hi));
    return d;
}

// 160-bit value, five words little-endian: what a reduction consumes.
struct A5 {
    uint32_t w0, w1, w2, w3, w4;
};

// Accumulator of 128-bit products, split so that every 64-bit partial product
// is added to an aligned word pair: e0..e4 hold the pairs at word positions
// (0,1), (2,3) and the carries out of them; o1..o3 hold the pair at (1,2) and
// its carries.  The value is e0 + 2^32 e1 + 2^64 e2 + 2^96 e3 + 2^128 e4
// + 2^32 o1 + 2^64 o2 + 2^96 o3.
struct A8 {
    uint32_t e0, e1, e2, e3, e4, o1, o2, o3;
};
__device__ __forceinline__ A8 acc_zero() {
    A8 a;
    a.e0 = a.e1 = a.e2 = a.e3 = a.e4 = a.o1 = a.o2 = a.o3 = 0;
    return a;
}
// accumulator that starts at the value v
__device__ __forceinline__ A8 acc_from(const W& v) {
    A8 a = acc_zero();
    a.e0 = v.lo;
    a.e1 = v.hi;
    return a;
}
// acc += a * b: four wide multiply-adds and three carry adds
__device__ __forceinline__ void acc_mac(A8& s, const W& a, const W& b) {
    asm("mad.lo.cc.u32 %0, %8, %10, %0; madc.hi.cc.u32 %1, %8, %10, %1;\n\t"
        "madc.lo.cc.u32 %2, %9, %11, %2; madc.hi.cc.u32 %3, %9, %11, %3; addc.u32 %4, %4, 0;\n\t"
        "mad.lo.cc.u32 %5, %8, %11, %5; madc.hi.cc.u32 %6, %8, %11, %6; addc.u32 %7, %7, 0;\n\t"
        "mad.lo.cc.u32 %5, %9, %10, %5; madc.hi.cc.u32 %6, %9, %10, %6; addc.u32 %7, %7, 0;"
        : "+r"(s.e0), "+r"(s.e1), "+r"(s.e2), "+r"(s.e3), "+r"(s.e4), "+r"(s.o1), "+r"(s.o2), "+r"(s.o3)
        : "r"(a.lo), "r"(a.hi), "r"(b.lo), "r"(b.hi));
}
// the accumulator as one 160-bit value
__device__ __forceinline__ A5 acc_merge(const A8& s) {
    A5 r;
    r.w0 = s.e0;
    asm("add.cc.u32 %0, %4, %8; addc.cc.u32 %1, %5, %9; addc.cc.u32 %2, %6, %10; addc.u32 %3, %7, 0;"
        : "=&r"(r.w1), "=&r"(r.w2), "=&r"(r.w3), "=&r"(r.w4)
        : "r"(s.e1), "r"(s.e2), "r"(s.e3), "r"(s.e4), "r"(s.o1), "r"(s.o2), "r"(s.o3));
    return r;
}

// The 128-bit product a * b as four words: four 32x32 products and six adds.
// It does not depend on any accumulator, so the adds that do (acc_add below)
// form a short chain.
struct P4 {
    uint32_t x0, x1, x2, x3;
};
__device__ __forceinline__ P4 prod(const W& a, const W& b) {
    P4 r;
    asm("{ .reg .u32 q0,q1,r0,r1; .reg .u64 t;\n\t"
        "mul.wide.u32 t, %4, %6; mov.b64 {%0,%1}, t;\n\t"
        "mul.wide.u32 t, %5, %7; mov.b64 {%2,%3}, t;\n\t"
        "mul.wide.u32 t, %4, %7; mov.b64 {q0,q1}, t;\n\t"
        "mul.wide.u32 t, %5, %6; mov.b64 {r0,r1}, t;\n\t"
        "add.cc.u32 %1, %1, q0; addc.cc.u32 %2, %2, q1; addc.u32 %3, %3, 0;\n\t"
        "add.cc.u32 %1, %1, r0; addc.cc.u32 %2, %2, r1; addc.u32 %3, %3, 0; }"
        : "=&r"(r.x0), "=&r"(r.x1), "=&r"(r.x2), "=&r"(r.x3)
        : "r"(a.lo), "r"(a.hi), "r"(b.lo), "r"(b.hi));
    return r;
}
// Loose residue of the accumulator.  With x = w0 + 2^32 w1, the value is
//   x + 2^64 w2 + 2^96 w3 + 2^128 w4 = x - (w3 + 2^32 w4) + w2 * EPS   (mod p).
// w4 counts overflows of a thread's sums and stays far below 2^31, so
// w3 + 2^32 w4 is canonical and the first step is a sub_c; w2 * EPS is
// (w2 << 32) - w2, built with one sub / subc, and added with the add_c fix.
__device__ __forceinline__ W acc_reduce(const A5& s) {
    W d;
    asm("{ .reg .u32 m, y0, y1;\n\t"
        "sub.cc.u32 %0, %2, %5; subc.cc.u32 %1, %3, %6; subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 %0, %0, m; subc.u32 %1, %1, 0;\n\t"
        "sub.cc.u32 y0, 0, %4; subc.u32 y1, %4, 0;\n\t"
        "add.cc.u32 %0, %0, y0; addc.cc.u32 %1, %1, y1; addc.u32 m, 0, 0; neg.s32 m, m;\n\t"
        "add.cc.u32 %0, %0, m; addc.u32 %1, %1, 0; }"
        : "=&r"(d.lo), "=&r"(d.hi)
        : "r"(s.w0), "r"(s.w1), "r"(s.w2), "r"(s.w3), "r"(s.w4));
    return d;
}

__device__ __forceinline__ W acc_reduce(const A8& s) { return acc_reduce(acc_merge(s)); }

// a * b as a loose residue
__device__ __forceinline__ W mul(const W& a, const W& b) {
    const P4 p = prod(a, b);
    A5 s;
    s.w0 = p.x0;
    s.w1 = p.x1;
    s.w2 = p.x2;
    s.w3 = p.x3;
    s.w4 = 0;
    return acc_reduce(s);
}

// 7 * a as a loose residue: 7a = x0 + 2^32 x1 + 2^64 x2 with x2 < 7, and 2^64 x2 = x2 * EPS
__device__ __forceinline__ W mul7(const W& a) {
    W d;
    asm("{ .reg .u32 x0, c0, y0, y1, x2, m, z0, z1; .reg .u64 t;\n\t"
        "mul.wide.u32 t, %2, 7; mov.b64 {x0,c0}, t;\n\t"
        "mul.wide.u32 t, %3, 7; mov.b64 {y0,y1}, t;\n\t"
        "add.cc.u32 y0, y0, c0; addc.u32 x2, y1, 0;\n\t"
        "sub.cc.u32 z0, 0, x2; subc.u32 z1, x2, 0;\n\t"
        "add.cc.u32 %0, x0, z0; addc.cc.u32 %1, y0, z1; addc.u32 m, 0, 0; neg.s32 m, m;\n\t"
        "add.cc.u32 %0, %0, m; addc.u32 %1, %1, 0; }"
        : "=&r"(d.lo), "=&r"(d.hi)
        : "r"(a.lo), "r"(a.hi));
    return d;
}

// ---- quadratic extension X^2 = 7, loose components ------------------------------
struct W2 {
    W c0, c1;
};
__device__ __forceinline__ W2 add_c(const W2& a, const W2& c) {
    W2 r;
    r.c0 = add_c(a.c0, c.c0);
    r.c1 = add_c(a.c1, c.c1);
    return r;
}
__device__ __forceinline__ W2 sub_c(const W2& a, const W2& c) {
    W2 r;
    r.c0 = sub_c(a.c0, c.c0);
    r.c1 = sub_c(a.c1, c.c1);
    return r;
}
// (a0 + a1 X)(b0 + b1 X): c0 = a0 b0 + (7 a1) b1, c1 = a0 b1 + a1 b0; two lazy sums, two reductions
__device__ __forceinline__ W2 mul(const W2& a, const W2& b) {
    A8 s0 = acc_zero(), s1 = acc_zero();
    acc_mac(s0, a.c0, b.c0);
    acc_mac(s0, mul7(a.c1), b.c1);
    acc_mac(s1, a.c0, b.c1);
    acc_mac(s1, a.c1, b.c0);
    W2 r;
    r.c0 = acc_reduce(s0);
    r.c1 = acc_reduce(s1);
    return r;
}

// What a fold needs of the challenge r = r0 + r1 X: r0, r1 and 7 r1, canonical.
struct Chal {
    W r0, r1, r1x7;
};
// canonical a0 + r (a1 - a0), a0 and a1 canonical extension elements
__device__ __forceinline__ W2 fold_ext(const W2& a0, const W2& a1, const Chal& r) {
    const W2 d = sub_c(a1, a0);
    A8 s0 = acc_from(a0.c0), s1 = acc_from(a0.c1);
    acc_mac(s0, d.c0, r.r0);
    acc_mac(s0, d.c1, r.r1x7);
    acc_mac(s1, d.c0, r.r1);
    acc_mac(s1, d.c1, r.r0);
    W2 f;
    f.c0 = canon(acc_reduce(s0));
    f.c1 = canon(acc_reduce(s1));
    return f;
}
// canonical a0 + r (a1 - a0), a0 and a1 canonical base elements
__device__ __forceinline__ W2 fold_base(const W& a0, const W& a1, const Chal& r) {
    const W d = sub_c(a1, a0);
    A8 s0 = acc_from(a0), s1 = acc_zero();
    acc_mac(s0, d, r.r0);
    acc_mac(s1, d, r.r1);
    W2 f;
    f.c0 = canon(acc_reduce(s0));
    f.c1 = canon(acc_reduce(s1));
    return f;
}

}  // namespace glw
}  // namespace dpb
