// Goldilocks prime field (p = 2^64 - 2^32 + 1) and its quadratic extension
// F_p[X]/(X^2 - 7), for host and device code.
//
// Elements are canonical (< p) whenever they are stored to memory. Inside a
// kernel the multiply accepts any 64-bit representative and returns a canonical
// one, so callers may chain additions without re-normalising.
//
// The standalone sumcheck microbenchmark runs over this field: table entries
// are base-field values (8 bytes), verifier challenges are extension elements
// (16 bytes), and a table becomes extension-valued after its first fold.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define DPB_HD __host__ __device__ __forceinline__
#else
#define DPB_HD inline
#endif

namespace dpb {

constexpr uint64_t GL_P = 0xFFFFFFFF00000001ULL;
constexpr uint64_t GL_EPS = 0xFFFFFFFFULL;  // 2^64 mod p
constexpr uint64_t GL_NONRES = 7;           // X^2 = 7 in the extension

DPB_HD void mul64wide(uint64_t a, uint64_t b, uint64_t& lo, uint64_t& hi) {
#if defined(__CUDA_ARCH__)
    lo = a * b;
    hi = __umul64hi(a, b);
#else
    unsigned __int128 t = (unsigned __int128)a * b;
    lo = (uint64_t)t;
    hi = (uint64_t)(t >> 64);
#endif
}

// Canonical sum of two canonical values.
DPB_HD uint64_t gl_add(uint64_t a, uint64_t b) {
    uint64_t s = a + b;
    // a + b < 2p, so one correction is enough; overflow past 2^64 also means >= p
    if (s < a || s >= GL_P) s -= GL_P;
    return s;
}

DPB_HD uint64_t gl_sub(uint64_t a, uint64_t b) {
    uint64_t d = a - b;
    if (a < b) d += GL_P;
    return d;
}

DPB_HD uint64_t gl_neg(uint64_t a) { return a ? GL_P - a : 0; }

DPB_HD uint64_t gl_double(uint64_t a) { return gl_add(a, a); }

// Reduce a 128-bit value (hi:lo) to a canonical residue.
// 2^64 = 2^32 - 1 and 2^96 = -1 (mod p).
DPB_HD uint64_t gl_reduce128(uint64_t lo, uint64_t hi) {
    uint64_t hh = hi >> 32;
    uint64_t hl = hi & GL_EPS;
    uint64_t t0 = lo - hh;
    if (lo < hh) t0 -= GL_EPS;  // wrapped by 2^64 = EPS (mod p); t0 >= 2^64-2^32 here
    uint64_t t1 = (hl << 32) - hl;  // hl * (2^32 - 1)
    uint64_t r = t0 + t1;
    if (r < t0) r += GL_EPS;  // carry out: add 2^64 mod p; cannot carry again
    if (r >= GL_P) r -= GL_P;
    return r;
}

DPB_HD uint64_t gl_mul(uint64_t a, uint64_t b) {
    uint64_t lo, hi;
    mul64wide(a, b, lo, hi);
    return gl_reduce128(lo, hi);
}

DPB_HD uint64_t gl_sqr(uint64_t a) { return gl_mul(a, a); }

// Multiply a canonical value by a small constant (c < 2^32).
DPB_HD uint64_t gl_mul_small(uint64_t a, uint32_t c) {
    uint64_t lo, hi;
    mul64wide(a, (uint64_t)c, lo, hi);  // hi < 2^32
    uint64_t t1 = (hi << 32) - hi;
    uint64_t r = lo + t1;
    if (r < lo) r += GL_EPS;
    if (r >= GL_P) r -= GL_P;
    return r;
}

inline uint64_t gl_pow(uint64_t a, uint64_t e) {
    uint64_t r = 1;
    while (e) {
        if (e & 1) r = gl_mul(r, a);
        a = gl_mul(a, a);
        e >>= 1;
    }
    return r;
}
inline uint64_t gl_inv(uint64_t a) { return gl_pow(a, GL_P - 2); }

// ---------------------------------------------------------------- extension
struct alignas(16) Gl2 {
    uint64_t c0, c1;
};

DPB_HD Gl2 gl2_make(uint64_t c0, uint64_t c1) {
    Gl2 r;
    r.c0 = c0;
    r.c1 = c1;
    return r;
}
DPB_HD Gl2 gl2_zero() { return gl2_make(0, 0); }
DPB_HD Gl2 gl2_one() { return gl2_make(1, 0); }
DPB_HD Gl2 gl2_from_base(uint64_t a) { return gl2_make(a, 0); }
DPB_HD Gl2 gl2_add(Gl2 a, Gl2 b) { return gl2_make(gl_add(a.c0, b.c0), gl_add(a.c1, b.c1)); }
DPB_HD Gl2 gl2_sub(Gl2 a, Gl2 b) { return gl2_make(gl_sub(a.c0, b.c0), gl_sub(a.c1, b.c1)); }
DPB_HD Gl2 gl2_neg(Gl2 a) { return gl2_make(gl_neg(a.c0), gl_neg(a.c1)); }
DPB_HD bool gl2_eq(Gl2 a, Gl2 b) { return a.c0 == b.c0 && a.c1 == b.c1; }

// (a0 + a1 X)(b0 + b1 X) = (a0 b0 + 7 a1 b1) + ((a0+a1)(b0+b1) - a0 b0 - a1 b1) X
DPB_HD Gl2 gl2_mul(Gl2 a, Gl2 b) {
    uint64_t v0 = gl_mul(a.c0, b.c0);
    uint64_t v1 = gl_mul(a.c1, b.c1);
    // (a0+a1) and (b0+b1) may be taken without reduction only if they do not
    // wrap; reduce them instead (cheap next to the multiply).
    uint64_t sa = gl_add(a.c0, a.c1);
    uint64_t sb = gl_add(b.c0, b.c1);
    uint64_t m = gl_mul(sa, sb);
    Gl2 r;
    r.c0 = gl_add(v0, gl_mul_small(v1, (uint32_t)GL_NONRES));
    r.c1 = gl_sub(gl_sub(m, v0), v1);
    return r;
}

// extension element times base element
DPB_HD Gl2 gl2_mul_base(Gl2 a, uint64_t b) { return gl2_make(gl_mul(a.c0, b), gl_mul(a.c1, b)); }

inline Gl2 gl2_inv(Gl2 a) {
    // 1/(a0 + a1 X) = (a0 - a1 X) / (a0^2 - 7 a1^2)
    uint64_t n = gl_sub(gl_mul(a.c0, a.c0), gl_mul_small(gl_mul(a.c1, a.c1), (uint32_t)GL_NONRES));
    uint64_t ni = gl_inv(n);
    return gl2_make(gl_mul(a.c0, ni), gl_mul(gl_neg(a.c1), ni));
}

}  // namespace dpb
