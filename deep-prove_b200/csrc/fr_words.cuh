// Device-side BN254 Fr arithmetic on 32-bit words.
//
// The portable routines of field_bn254.cuh multiply 64-bit limbs; on the GPU
// each 64x64 product expands into a long sequence of 32-bit multiply-adds and
// register shuffles.  Here a field element is eight 32-bit words and the
// Montgomery product is coarsely integrated operand scanning over words: per
// word of b, eight 32x32 products accumulate into the running sum through two
// carry chains (low halves, high halves), then eight more for the reduction
// step.  Multiplies are mul.wide.u32 (one per limb product), everything else is
// carry-chained 32-bit addition: the instruction mix the sm_100a integer pipes
// dispatch fastest (an add per cycle, a multiply every other cycle).
//
// The word layout is the little-endian split of the four 64-bit limbs, so a
// conversion is a register reinterpretation.
#pragma once
// Included by field_bn254.cuh (after the definition of Fr) and by nothing else.
#include <cstdint>

namespace dpb {
namespace frw {

struct F8 {
    uint32_t w[8];
};

__device__ __forceinline__ F8 from_fr(const Fr& a) {
    F8 r;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        r.w[2 * i] = (uint32_t)a.l[i];
        r.w[2 * i + 1] = (uint32_t)(a.l[i] >> 32);
    }
    return r;
}
__device__ __forceinline__ Fr to_fr(const F8& a) {
    Fr r;
#pragma unroll
    for (int i = 0; i < 4; i++) r.l[i] = (uint64_t)a.w[2 * i] | ((uint64_t)a.w[2 * i + 1] << 32);
    return r;
}

// modulus r, words little-endian
#define DPB_FRW_P0 0xf0000001u
#define DPB_FRW_P1 0x43e1f593u
#define DPB_FRW_P2 0x79b97091u
#define DPB_FRW_P3 0x2833e848u
#define DPB_FRW_P4 0x8181585du
#define DPB_FRW_P5 0xb85045b6u
#define DPB_FRW_P6 0xe131a029u
#define DPB_FRW_P7 0x30644e72u
#define DPB_FRW_INV 0xefffffffu  // -r^{-1} mod 2^32

// t (10 words) += a (8 words) * b (one word)
__device__ __forceinline__ void row_mac(uint32_t (&t)[10], const F8& a, uint32_t b) {
    asm("{ .reg .u32 l0,l1,l2,l3,l4,l5,l6,l7,h0,h1,h2,h3,h4,h5,h6,h7; .reg .u64 x;\n\t"
        "mul.wide.u32 x, %10, %18; mov.b64 {l0,h0}, x;\n\t"
        "mul.wide.u32 x, %11, %18; mov.b64 {l1,h1}, x;\n\t"
        "mul.wide.u32 x, %12, %18; mov.b64 {l2,h2}, x;\n\t"
        "mul.wide.u32 x, %13, %18; mov.b64 {l3,h3}, x;\n\t"
        "mul.wide.u32 x, %14, %18; mov.b64 {l4,h4}, x;\n\t"
        "mul.wide.u32 x, %15, %18; mov.b64 {l5,h5}, x;\n\t"
        "mul.wide.u32 x, %16, %18; mov.b64 {l6,h6}, x;\n\t"
        "mul.wide.u32 x, %17, %18; mov.b64 {l7,h7}, x;\n\t"
        "add.cc.u32 %0, %0, l0; addc.cc.u32 %1, %1, l1; addc.cc.u32 %2, %2, l2; addc.cc.u32 %3, %3, l3;\n\t"
        "addc.cc.u32 %4, %4, l4; addc.cc.u32 %5, %5, l5; addc.cc.u32 %6, %6, l6; addc.cc.u32 %7, %7, l7;\n\t"
        "addc.cc.u32 %8, %8, 0; addc.u32 %9, %9, 0;\n\t"
        "add.cc.u32 %1, %1, h0; addc.cc.u32 %2, %2, h1; addc.cc.u32 %3, %3, h2; addc.cc.u32 %4, %4, h3;\n\t"
        "addc.cc.u32 %5, %5, h4; addc.cc.u32 %6, %6, h5; addc.cc.u32 %7, %7, h6; addc.cc.u32 %8, %8, h7;\n\t"
        "addc.u32 %9, %9, 0; }"
        : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]), "+r"(t[4]), "+r"(t[5]), "+r"(t[6]), "+r"(t[7]), "+r"(t[8]),
          "+r"(t[9])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]),
          "r"(b));
}

// t += m * r with m chosen so that word 0 becomes zero; the caller then drops word 0.
__device__ __forceinline__ void row_reduce(uint32_t (&t)[10]) {
    asm("{ .reg .u32 m,l0,l1,l2,l3,l4,l5,l6,l7,h0,h1,h2,h3,h4,h5,h6,h7; .reg .u64 x;\n\t"
        "mul.lo.u32 m, %0, 0xefffffff;\n\t"
        "mul.wide.u32 x, m, 0xf0000001; mov.b64 {l0,h0}, x;\n\t"
        "mul.wide.u32 x, m, 0x43e1f593; mov.b64 {l1,h1}, x;\n\t"
        "mul.wide.u32 x, m, 0x79b97091; mov.b64 {l2,h2}, x;\n\t"
        "mul.wide.u32 x, m, 0x2833e848; mov.b64 {l3,h3}, x;\n\t"
        "mul.wide.u32 x, m, 0x8181585d; mov.b64 {l4,h4}, x;\n\t"
        "mul.wide.u32 x, m, 0xb85045b6; mov.b64 {l5,h5}, x;\n\t"
        "mul.wide.u32 x, m, 0xe131a029; mov.b64 {l6,h6}, x;\n\t"
        "mul.wide.u32 x, m, 0x30644e72; mov.b64 {l7,h7}, x;\n\t"
        "add.cc.u32 %0, %0, l0; addc.cc.u32 %1, %1, l1; addc.cc.u32 %2, %2, l2; addc.cc.u32 %3, %3, l3;\n\t"
        "addc.cc.u32 %4, %4, l4; addc.cc.u32 %5, %5, l5; addc.cc.u32 %6, %6, l6; addc.cc.u32 %7, %7, l7;\n\t"
        "addc.cc.u32 %8, %8, 0; addc.u32 %9, %9, 0;\n\t"
        "add.cc.u32 %1, %1, h0; addc.cc.u32 %2, %2, h1; addc.cc.u32 %3, %3, h2; addc.cc.u32 %4, %4, h3;\n\t"
        "addc.cc.u32 %5, %5, h4; addc.cc.u32 %6, %6, h5; addc.cc.u32 %7, %7, h6; addc.cc.u32 %8, %8, h7;\n\t"
        "addc.u32 %9, %9, 0; }"
        : "+r"(t[0]), "+r"(t[1]), "+r"(t[2]), "+r"(t[3]), "+r"(t[4]), "+r"(t[5]), "+r"(t[6]), "+r"(t[7]), "+r"(t[8]),
          "+r"(t[9]));
}

// a < 2r -> a mod r: subtract r; on a borrow add it back through a mask
__device__ __forceinline__ F8 reduce_once(const F8& a) {
    F8 d;
    asm("{ .reg .u32 m, q0,q1,q2,q3,q4,q5,q6,q7;\n\t"
        "sub.cc.u32 %0, %8, 0xf0000001; subc.cc.u32 %1, %9, 0x43e1f593; subc.cc.u32 %2, %10, 0x79b97091;\n\t"
        "subc.cc.u32 %3, %11, 0x2833e848; subc.cc.u32 %4, %12, 0x8181585d; subc.cc.u32 %5, %13, 0xb85045b6;\n\t"
        "subc.cc.u32 %6, %14, 0xe131a029; subc.cc.u32 %7, %15, 0x30644e72; subc.u32 m, 0, 0;\n\t"
        "and.b32 q0, m, 0xf0000001; and.b32 q1, m, 0x43e1f593; and.b32 q2, m, 0x79b97091; and.b32 q3, m, 0x2833e848;\n\t"
        "and.b32 q4, m, 0x8181585d; and.b32 q5, m, 0xb85045b6; and.b32 q6, m, 0xe131a029; and.b32 q7, m, 0x30644e72;\n\t"
        "add.cc.u32 %0, %0, q0; addc.cc.u32 %1, %1, q1; addc.cc.u32 %2, %2, q2; addc.cc.u32 %3, %3, q3;\n\t"
        "addc.cc.u32 %4, %4, q4; addc.cc.u32 %5, %5, q5; addc.cc.u32 %6, %6, q6; addc.u32 %7, %7, q7; }"
        : "=&r"(d.w[0]), "=&r"(d.w[1]), "=&r"(d.w[2]), "=&r"(d.w[3]), "=&r"(d.w[4]), "=&r"(d.w[5]), "=&r"(d.w[6]),
          "=&r"(d.w[7])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]));
    return d;
}

// Montgomery product a * b / 2^256 mod r
__device__ __forceinline__ F8 mul(const F8& a, const F8& b) {
    uint32_t t[10];
#pragma unroll
    for (int i = 0; i < 10; i++) t[i] = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        row_mac(t, a, b.w[i]);
        row_reduce(t);
        // word 0 is zero now: shift down one word
#pragma unroll
        for (int j = 0; j < 9; j++) t[j] = t[j + 1];
        t[9] = 0;
    }
    F8 r;
#pragma unroll
    for (int i = 0; i < 8; i++) r.w[i] = t[i];
    return reduce_once(r);  // the running sum stays below 2r (r has two spare top bits)
}

__device__ __forceinline__ F8 add(const F8& a, const F8& b) {
    F8 s;
    asm("add.cc.u32 %0, %8, %16; addc.cc.u32 %1, %9, %17; addc.cc.u32 %2, %10, %18; addc.cc.u32 %3, %11, %19;\n\t"
        "addc.cc.u32 %4, %12, %20; addc.cc.u32 %5, %13, %21; addc.cc.u32 %6, %14, %22; addc.u32 %7, %15, %23;"
        : "=&r"(s.w[0]), "=&r"(s.w[1]), "=&r"(s.w[2]), "=&r"(s.w[3]), "=&r"(s.w[4]), "=&r"(s.w[5]), "=&r"(s.w[6]),
          "=&r"(s.w[7])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]),
          "r"(b.w[0]), "r"(b.w[1]), "r"(b.w[2]), "r"(b.w[3]), "r"(b.w[4]), "r"(b.w[5]), "r"(b.w[6]), "r"(b.w[7]));
    return reduce_once(s);  // a + b < 2r < 2^255: no carry out of the top word
}

// a - b mod r: on a borrow add r back through a mask
__device__ __forceinline__ F8 sub(const F8& a, const F8& b) {
    F8 d;
    asm("{ .reg .u32 m, q0,q1,q2,q3,q4,q5,q6,q7;\n\t"
        "sub.cc.u32 %0, %8, %16; subc.cc.u32 %1, %9, %17; subc.cc.u32 %2, %10, %18; subc.cc.u32 %3, %11, %19;\n\t"
        "subc.cc.u32 %4, %12, %20; subc.cc.u32 %5, %13, %21; subc.cc.u32 %6, %14, %22; subc.cc.u32 %7, %15, %23;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "and.b32 q0, m, 0xf0000001; and.b32 q1, m, 0x43e1f593; and.b32 q2, m, 0x79b97091; and.b32 q3, m, 0x2833e848;\n\t"
        "and.b32 q4, m, 0x8181585d; and.b32 q5, m, 0xb85045b6; and.b32 q6, m, 0xe131a029; and.b32 q7, m, 0x30644e72;\n\t"
        "add.cc.u32 %0, %0, q0; addc.cc.u32 %1, %1, q1; addc.cc.u32 %2, %2, q2; addc.cc.u32 %3, %3, q3;\n\t"
        "addc.cc.u32 %4, %4, q4; addc.cc.u32 %5, %5, q5; addc.cc.u32 %6, %6, q6; addc.u32 %7, %7, q7; }"
        : "=&r"(d.w[0]), "=&r"(d.w[1]), "=&r"(d.w[2]), "=&r"(d.w[3]), "=&r"(d.w[4]), "=&r"(d.w[5]), "=&r"(d.w[6]),
          "=&r"(d.w[7])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]),
          "r"(b.w[0]), "r"(b.w[1]), "r"(b.w[2]), "r"(b.w[3]), "r"(b.w[4]), "r"(b.w[5]), "r"(b.w[6]), "r"(b.w[7]));
    return d;
}

}  // namespace frw
}  // namespace dpb
