/*
 * CPU oracle for the sumcheck / multilinear-fold / logup-GKR path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; it exists so that tests can compare the CUDA path with an
 * independent plain-C restatement, and so that the benchmark can time the same
 * algorithm on the host's cores.
 *
 * PARITY UNPINNED at the byte level: the reference's sumcheck, multilinear and
 * transcript code lives in the third-party crate dp-crypto 0.1.0 (git rev
 * 22e8e93cd0f94a7638616a1ae22190feb0a6b275, Cargo.lock:3773-3775), which is not
 * part of the reference tree, and the reference holds no golden proof or
 * transcript vector.  What IS pinned, by tests that replay the reference's own
 * algebraic checks against this file: little-endian evaluation
 * (zkml/src/lib.rs:357-369), which variables fix_high / fix_low bind
 * (zkml/src/layers/transformer/attention_mask/prove.rs:392-451), the tree
 * output identity (zkml/src/lookup/logup_gkr/circuit.rs:603-624) and the
 * logup claim identity (zkml/src/lookup/logup_gkr/mod.rs:24-79).
 *
 * Algorithms restated here (reference file:line beside each function):
 *   - the standard sumcheck round (evaluate product terms at 0..d over the
 *     remaining hypercube, low variable first) and the fold that binds it;
 *   - eq tables, fix_high / fix_low, evaluate;
 *   - LogUpLayer::next_layer for the three layer kinds.
 *
 * Layouts match the library's: Goldilocks base = uint64 (dtype 0), Goldilocks
 * quadratic extension X^2 = 7 = 2 x uint64 (dtype 1), BN254 Fr = 4 x uint64
 * Montgomery limbs (dtype 2).
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC oracle.c -o _build/liboracle.so
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef unsigned __int128 u128;

/* ------------------------------------------------------------ Goldilocks */
#define GLP 0xFFFFFFFF00000001ULL

static inline uint64_t gl_red(u128 x) {
    /* x = lo + 2^64 (hl + 2^32 hh); 2^64 = 2^32 - 1, 2^96 = -1 (mod p) */
    uint64_t lo = (uint64_t)x, hi = (uint64_t)(x >> 64);
    uint64_t hh = hi >> 32, hl = hi & 0xFFFFFFFFULL;
    u128 t = (u128)lo + (u128)hl * 0xFFFFFFFFULL + (u128)GLP - hh;
    /* t < 2^64 + 2^64 + 2^64: fold once more */
    uint64_t tl = (uint64_t)t, th = (uint64_t)(t >> 64); /* th <= 2 */
    u128 u = (u128)tl + (u128)th * 0xFFFFFFFFULL;
    uint64_t ul = (uint64_t)u, uh = (uint64_t)(u >> 64); /* uh <= 1 */
    u128 v = (u128)ul + (u128)uh * 0xFFFFFFFFULL;
    uint64_t r = (uint64_t)v;
    if ((v >> 64) != 0) r += 0xFFFFFFFFULL; /* cannot wrap again */
    if (r >= GLP) r -= GLP;
    return r;
}
static inline uint64_t gl_addc(uint64_t a, uint64_t b) {
    u128 s = (u128)a + b;
    if (s >= GLP) s -= GLP;
    return (uint64_t)s;
}
static inline uint64_t gl_subc(uint64_t a, uint64_t b) { return a >= b ? a - b : a + (GLP - b); }
static inline uint64_t gl_mulc(uint64_t a, uint64_t b) { return gl_red((u128)a * b); }

typedef struct { uint64_t c0, c1; } gl2;
static inline gl2 gl2_add(gl2 a, gl2 b) { gl2 r = {gl_addc(a.c0, b.c0), gl_addc(a.c1, b.c1)}; return r; }
static inline gl2 gl2_sub(gl2 a, gl2 b) { gl2 r = {gl_subc(a.c0, b.c0), gl_subc(a.c1, b.c1)}; return r; }
static inline gl2 gl2_mul(gl2 a, gl2 b) {
    /* schoolbook: (a0 b0 + 7 a1 b1) + (a0 b1 + a1 b0) X */
    uint64_t a1b1 = gl_mulc(a.c1, b.c1);
    gl2 r;
    r.c0 = gl_addc(gl_mulc(a.c0, b.c0), gl_mulc(a1b1, 7));
    r.c1 = gl_addc(gl_mulc(a.c0, b.c1), gl_mulc(a.c1, b.c0));
    return r;
}

/* ------------------------------------------------------------ BN254 Fr */
typedef struct { uint64_t l[4]; } fr;
static const uint64_t FRP[4] = {0x43e1f593f0000001ULL, 0x2833e84879b97091ULL, 0xb85045b68181585dULL,
                                0x30644e72e131a029ULL};
static const uint64_t FRINV = 0xc2e1f593efffffffULL; /* -r^-1 mod 2^64 */
static const fr FR_R2 = {{0x1bb8e645ae216da7ULL, 0x53fe3ab1e35c59e3ULL, 0x8c49833d53bb8085ULL,
                          0x0216d0b17f4e44a5ULL}};
static const fr FR_ONE = {{0xac96341c4ffffffbULL, 0x36fc76959f60cd29ULL, 0x666ea36f7879462eULL,
                           0x0e0a77c19a07df2fULL}};

static inline int fr_geq_p(const uint64_t* a) {
    for (int i = 3; i >= 0; i--) {
        if (a[i] > FRP[i]) return 1;
        if (a[i] < FRP[i]) return 0;
    }
    return 1;
}
static inline void fr_sub_p(uint64_t* a) {
    u128 bw = 0;
    for (int i = 0; i < 4; i++) {
        u128 d = (u128)a[i] - FRP[i] - bw;
        a[i] = (uint64_t)d;
        bw = (d >> 64) & 1;
    }
}
static inline fr fr_add(fr a, fr b) {
    fr r;
    u128 c = 0;
    for (int i = 0; i < 4; i++) {
        c += (u128)a.l[i] + b.l[i];
        r.l[i] = (uint64_t)c;
        c >>= 64;
    }
    if (fr_geq_p(r.l)) fr_sub_p(r.l);
    return r;
}
static inline fr fr_sub(fr a, fr b) {
    fr r;
    u128 bw = 0;
    for (int i = 0; i < 4; i++) {
        u128 d = (u128)a.l[i] - b.l[i] - bw;
        r.l[i] = (uint64_t)d;
        bw = (d >> 64) & 1;
    }
    if (bw) {
        u128 c = 0;
        for (int i = 0; i < 4; i++) {
            c += (u128)r.l[i] + FRP[i];
            r.l[i] = (uint64_t)c;
            c >>= 64;
        }
    }
    return r;
}
/* Montgomery product by separate multiply then reduce (SOS): an 8-limb
 * schoolbook product followed by four reduction steps. */
static inline fr fr_mul(fr a, fr b) {
    uint64_t t[9] = {0};
    for (int i = 0; i < 4; i++) {
        u128 c = 0;
        for (int j = 0; j < 4; j++) {
            c += (u128)a.l[j] * b.l[i] + t[i + j];
            t[i + j] = (uint64_t)c;
            c >>= 64;
        }
        t[i + 4] = (uint64_t)c;
    }
    for (int i = 0; i < 4; i++) {
        uint64_t m = t[i] * FRINV;
        u128 c = 0;
        for (int j = 0; j < 4; j++) {
            c += (u128)m * FRP[j] + t[i + j];
            t[i + j] = (uint64_t)c;
            c >>= 64;
        }
        for (int j = i + 4; j < 9 && c; j++) {
            c += t[j];
            t[j] = (uint64_t)c;
            c >>= 64;
        }
    }
    fr r = {{t[4], t[5], t[6], t[7]}};
    if (t[8] || fr_geq_p(r.l)) fr_sub_p(r.l);
    return r;
}

/* ------------------------------------------------------------ generic layer */
/* A "family" is the working element type: 0 = Goldilocks ext, 1 = BN254 Fr. */
#define FAM_GL 0
#define FAM_FR 1
#define DT_GL_BASE 0
#define DT_GL_EXT 1
#define DT_FR 2

static inline gl2 glf_ld(const void* p, int dt, uint64_t i) {
    if (dt == DT_GL_BASE) { gl2 r = {((const uint64_t*)p)[i], 0}; return r; }
    return ((const gl2*)p)[i];
}
static inline fr frf_ld(const void* p, int dt, uint64_t i) { (void)dt; return ((const fr*)p)[i]; }

typedef struct {
    uint8_t coeff[32];
    uint32_t n_factors;
    uint16_t idx[8];
} orc_term;

#define MAXD 8

/* One sumcheck round: evaluations at 0..=d of
 *   sum over pairs p of sum_t coeff_t prod_j f_tj(x; p),
 * where a table with all `vars` remaining variables contributes entries 2p
 * and 2p+1 (the low variable is the one being bound) and a table with fewer
 * variables depends on the LAST variables only, i.e. is constant in this round
 * (the convention of zkml/src/lookup/logup_gkr/prover.rs:217-249).  The body of
 * the reference's IOPProverState::prove is in dp-crypto (absent); this is the
 * textbook prover round its call sites imply
 * (zkml/src/layers/hadamard.rs:106-131). */
#define DEFINE_ROUND(NAME, T, LD, ADD, SUB, MUL)                                                     \
    void NAME(uint32_t vars, const void* const* tabs, const int* dts, const uint32_t* tvars,         \
              uint32_t k, const orc_term* terms, uint32_t n_terms, uint32_t d, void* out) {          \
        (void)k;                                                                                     \
        const uint64_t n_pairs = 1ULL << (vars - 1);                                                 \
        T tot[MAXD];                                                                                 \
        memset(tot, 0, sizeof tot);                                                                  \
        _Pragma("omp parallel") {                                                                    \
            T acc[MAXD];                                                                             \
            memset(acc, 0, sizeof acc);                                                              \
            _Pragma("omp for schedule(static)") for (uint64_t p = 0; p < n_pairs; p++) {             \
                for (uint32_t t = 0; t < n_terms; t++) {                                             \
                    T prod[MAXD];                                                                    \
                    T cf;                                                                            \
                    memcpy(&cf, terms[t].coeff, sizeof(T));                                          \
                    for (uint32_t x = 0; x <= d; x++) prod[x] = cf;                                  \
                    for (uint32_t j = 0; j < terms[t].n_factors; j++) {                              \
                        const uint32_t id = terms[t].idx[j];                                         \
                        T f0, f1;                                                                    \
                        if (tvars[id] >= vars) {                                                     \
                            f0 = LD(tabs[id], dts[id], 2 * p);                                       \
                            f1 = LD(tabs[id], dts[id], 2 * p + 1);                                   \
                        } else {                                                                     \
                            f0 = f1 = LD(tabs[id], dts[id], p >> (vars - 1 - tvars[id]));            \
                        }                                                                            \
                        T dl = SUB(f1, f0), v = f0;                                                  \
                        for (uint32_t x = 0; x <= d; x++) {                                          \
                            prod[x] = MUL(prod[x], v);                                               \
                            v = ADD(v, dl);                                                          \
                        }                                                                            \
                    }                                                                                \
                    for (uint32_t x = 0; x <= d; x++) acc[x] = ADD(acc[x], prod[x]);                 \
                }                                                                                    \
            }                                                                                        \
            _Pragma("omp critical") {                                                                \
                for (uint32_t x = 0; x <= d; x++) tot[x] = ADD(tot[x], acc[x]);                      \
            }                                                                                        \
        }                                                                                            \
        memcpy(out, tot, (d + 1) * sizeof(T));                                                       \
    }

DEFINE_ROUND(orc_round_gl, gl2, glf_ld, gl2_add, gl2_sub, gl2_mul)
DEFINE_ROUND(orc_round_fr, fr, frf_ld, fr_add, fr_sub, fr_mul)

/* Base-field fast path of the Goldilocks round for a single coefficient-one
 * product of k base tables (the first round of the f*g*h microbenchmark): the
 * same sums as orc_round_gl, computed with 64-bit multiplies. */
void orc_round_gl_base_product(uint32_t vars, const uint64_t* const* tabs, uint32_t k, void* out) {
    const uint64_t n_pairs = 1ULL << (vars - 1);
    uint64_t tot[MAXD] = {0};
#pragma omp parallel
    {
        uint64_t acc[MAXD] = {0};
#pragma omp for schedule(static)
        for (uint64_t p = 0; p < n_pairs; p++) {
            uint64_t v[8], dl[8];
            for (uint32_t j = 0; j < k; j++) {
                v[j] = tabs[j][2 * p];
                dl[j] = gl_subc(tabs[j][2 * p + 1], v[j]);
            }
            for (uint32_t x = 0; x <= k; x++) {
                uint64_t pr = v[0];
                for (uint32_t j = 1; j < k; j++) pr = gl_mulc(pr, v[j]);
                acc[x] = gl_addc(acc[x], pr);
                for (uint32_t j = 0; j < k; j++) v[j] = gl_addc(v[j], dl[j]);
            }
        }
#pragma omp critical
        for (uint32_t x = 0; x <= k; x++) tot[x] = gl_addc(tot[x], acc[x]);
    }
    gl2* o = (gl2*)out;
    for (uint32_t x = 0; x <= k; x++) { o[x].c0 = tot[x]; o[x].c1 = 0; }
}

/* Bind the low variable: out[p] = in[2p] + r (in[2p+1] - in[2p]).
 * (DensePolynomial::fix_low_variables for one variable; pinned by
 * zkml/src/layers/transformer/attention_mask/prove.rs:392-451.) */
void orc_fold_gl(const void* in, int dt, uint64_t n_out, const void* r_, void* out) {
    gl2 r; memcpy(&r, r_, sizeof r);
    gl2* o = (gl2*)out;
#pragma omp parallel for schedule(static)
    for (uint64_t p = 0; p < n_out; p++) {
        gl2 f0 = glf_ld(in, dt, 2 * p), f1 = glf_ld(in, dt, 2 * p + 1);
        o[p] = gl2_add(f0, gl2_mul(r, gl2_sub(f1, f0)));
    }
}
void orc_fold_fr(const void* in, int dt, uint64_t n_out, const void* r_, void* out) {
    (void)dt;
    fr r; memcpy(&r, r_, sizeof r);
    const fr* a = (const fr*)in;
    fr* o = (fr*)out;
#pragma omp parallel for schedule(static)
    for (uint64_t p = 0; p < n_out; p++) o[p] = fr_add(a[2 * p], fr_mul(r, fr_sub(a[2 * p + 1], a[2 * p])));
}

/* Bind the TOP variable: out[j] = in[j] + r (in[j + n_out] - in[j]).
 * (DensePolynomial::fix_high_variables for one variable.) */
void orc_fold_high_gl(const void* in, int dt, uint64_t n_out, const void* r_, void* out) {
    gl2 r; memcpy(&r, r_, sizeof r);
    gl2* o = (gl2*)out;
#pragma omp parallel for schedule(static)
    for (uint64_t p = 0; p < n_out; p++) {
        gl2 f0 = glf_ld(in, dt, p), f1 = glf_ld(in, dt, p + n_out);
        o[p] = gl2_add(f0, gl2_mul(r, gl2_sub(f1, f0)));
    }
}
void orc_fold_high_fr(const void* in, int dt, uint64_t n_out, const void* r_, void* out) {
    (void)dt;
    fr r; memcpy(&r, r_, sizeof r);
    const fr* a = (const fr*)in;
    fr* o = (fr*)out;
#pragma omp parallel for schedule(static)
    for (uint64_t p = 0; p < n_out; p++) o[p] = fr_add(a[p], fr_mul(r, fr_sub(a[p + n_out], a[p])));
}

/* eq(x, point) for all x, little-endian index, by doubling:
 * table over point[0..j] -> table over point[0..j+1]
 * (dp_crypto::poly::eq::evals; used as per-index weights in
 * zkml/src/layers/einsum/axis.rs:1032 and checked against
 * identity_eval, zkml/src/poly_commit/mod.rs:184-192). */
void orc_eq_gl(const void* point, uint32_t m, void* out) {
    const gl2* pt = (const gl2*)point;
    gl2* o = (gl2*)out;
    gl2 one = {1, 0};
    o[0] = one;
    for (uint32_t j = 0; j < m; j++) {
        uint64_t h = 1ULL << j;
        for (uint64_t i = 0; i < h; i++) {
            gl2 hi = gl2_mul(o[i], pt[j]);
            o[i + h] = hi;
            o[i] = gl2_sub(o[i], hi);
        }
    }
}
void orc_eq_fr(const void* point, uint32_t m, void* out) {
    const fr* pt = (const fr*)point;
    fr* o = (fr*)out;
    o[0] = FR_ONE;
    for (uint32_t j = 0; j < m; j++) {
        uint64_t h = 1ULL << j;
        for (uint64_t i = 0; i < h; i++) {
            fr hi = fr_mul(o[i], pt[j]);
            o[i + h] = hi;
            o[i] = fr_sub(o[i], hi);
        }
    }
}

/* LogUpLayer::next_layer (zkml/src/lookup/logup_gkr/circuit.rs:88-184).
 * kind 0: initial lookup (numerators -1), 1: initial table (numerators =
 * multiplicities), 2: generic (num/den arrays given as cols[0], cols[1]).
 * Denominator of the initial kinds: constant + sum_j sep^j col_j, powers
 * starting at one (circuit.rs:162-171).  Fractions add as
 * (n1 d2 + d1 n2, d1 d2) (zkml/src/lookup/logup_gkr/structs.rs:48-58). */
#define DEFINE_LOGUP(NAME, T, LD, ADD, SUB, MUL, ONE_EXPR)                                           \
    void NAME(int kind, const void* const* cols, const int* dts, uint32_t n_cols, const void* mult,  \
              int mult_dt, const void* constant_, const void* sep_, uint64_t half, void* num_out,    \
              void* den_out) {                                                                       \
        T* no = (T*)num_out;                                                                         \
        T* de = (T*)den_out;                                                                         \
        T cst, sep;                                                                                  \
        T zero;                                                                                      \
        memset(&zero, 0, sizeof zero);                                                               \
        if (kind != 2) { memcpy(&cst, constant_, sizeof(T)); memcpy(&sep, sep_, sizeof(T)); }        \
        _Pragma("omp parallel for schedule(static)") for (uint64_t i = 0; i < half; i++) {           \
            T n1, n2, d1, d2;                                                                        \
            if (kind == 2) {                                                                         \
                n1 = LD(cols[0], dts[0], i); n2 = LD(cols[0], dts[0], i + half);                     \
                d1 = LD(cols[1], dts[1], i); d2 = LD(cols[1], dts[1], i + half);                     \
            } else {                                                                                 \
                T pw = ONE_EXPR;                                                                     \
                d1 = cst; d2 = cst;                                                                  \
                for (uint32_t j = 0; j < n_cols; j++) {                                              \
                    d1 = ADD(d1, MUL(pw, LD(cols[j], dts[j], i)));                                   \
                    d2 = ADD(d2, MUL(pw, LD(cols[j], dts[j], i + half)));                            \
                    pw = MUL(pw, sep);                                                               \
                }                                                                                    \
                if (kind == 1) { n1 = LD(mult, mult_dt, i); n2 = LD(mult, mult_dt, i + half); }      \
                else { n1 = SUB(zero, ONE_EXPR); n2 = n1; }                                          \
            }                                                                                        \
            no[i] = ADD(MUL(n1, d2), MUL(d1, n2));                                                   \
            de[i] = MUL(d1, d2);                                                                     \
        }                                                                                            \
    }

static inline gl2 gl2_one_(void) { gl2 r = {1, 0}; return r; }
DEFINE_LOGUP(orc_logup_next_gl, gl2, glf_ld, gl2_add, gl2_sub, gl2_mul, gl2_one_())
DEFINE_LOGUP(orc_logup_next_fr, fr, frf_ld, fr_add, fr_sub, fr_mul, FR_ONE)

/* ---- scalar helpers for the Python side (conversions, single operations) -- */
void orc_fr_to_mont(const void* canon, void* mont, uint64_t n) {
    const fr* a = (const fr*)canon;
    fr* o = (fr*)mont;
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; i++) o[i] = fr_mul(a[i], FR_R2);
}
void orc_fr_from_mont(const void* mont, void* canon, uint64_t n) {
    const fr* a = (const fr*)mont;
    fr* o = (fr*)canon;
    fr one = {{1, 0, 0, 0}};
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; i++) o[i] = fr_mul(a[i], one);
}
/* Element (i64) -> field, negative x -> p - |x| (zkml/src/quantization/mod.rs:220-267) */
void orc_fr_from_i64(const int64_t* x, void* mont, uint64_t n) {
    fr* o = (fr*)mont;
    fr zero = {{0, 0, 0, 0}};
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; i++) {
        uint64_t mag = x[i] < 0 ? (uint64_t)0 - (uint64_t)x[i] : (uint64_t)x[i];
        fr a = {{mag, 0, 0, 0}};
        a = fr_mul(a, FR_R2);
        o[i] = x[i] < 0 ? fr_sub(zero, a) : a;
    }
}
void orc_gl_from_i64(const int64_t* x, uint64_t* out, uint64_t n) {
    for (uint64_t i = 0; i < n; i++)
        out[i] = x[i] < 0 ? GLP - ((uint64_t)0 - (uint64_t)x[i]) : (uint64_t)x[i];
}
void orc_fr_mul1(const void* a, const void* b, void* out) {
    fr x, y; memcpy(&x, a, 32); memcpy(&y, b, 32);
    fr r = fr_mul(x, y); memcpy(out, &r, 32);
}
void orc_gl2_mul1(const void* a, const void* b, void* out) {
    gl2 x, y; memcpy(&x, a, 16); memcpy(&y, b, 16);
    gl2 r = gl2_mul(x, y); memcpy(out, &r, 16);
}
int orc_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    n = omp_get_max_threads();
#endif
    return n;
}
/* Number of OpenMP threads later parallel regions use (a launcher may have exported OMP_NUM_THREADS=1). */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
