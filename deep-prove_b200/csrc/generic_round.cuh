// One-pass sumcheck round for any list of product terms.
//
// A round of the generic prover used to be two launches: bind the previous
// challenge into every table (read 2^v, write 2^(v-1)), then evaluate the terms
// (read 2^(v-1) again).  Here one kernel does both: a thread that owns pair p
// of this round reads the four previous-round entries 4p..4p+3 of every table,
// binds the challenge, stores the two new entries and evaluates the terms on
// them while they are still on chip.
//
// Three things cut the multiplies per pair:
//  * every table is loaded and bound once per pair, whatever the number of
//    terms that use it: the pair (value at 0, difference) of each table sits in
//    a per-thread slot of shared memory, and moving to the next evaluation point
//    is one addition per table;
//  * after round 0 the value at 1 is not computed: the host gets it from the
//    previous round polynomial (s(0) + s(1) = previous s(r));
//  * terms that share a table are grouped on the host, and that table
//    multiplies the group's sum once per point instead of once per term.
// Results are exact field sums, so they equal the two-pass kernels' bit for bit.
#pragma once
#include <algorithm>

#include "sumcheck_kernels.cuh"

namespace dpb {

// A table as one round's kernel sees it.
struct RoundTab {
    const void* in;    // fold mode: the table of the previous round; otherwise this round's table
    void* out;         // fold mode: where the bound table goes (2 entries per pair); else nullptr
    int32_t dtype_in;  // layout of `in`
    int32_t shift;     // < 0: entries 2p, 2p+1 (4p..4p+3 in fold mode); >= 0: constant this round, entry p >> shift
};

constexpr uint16_t kNoOuter = 0xFFFF;
constexpr int kMaxAccTail = 8;  // sums a round publishes (degree <= 7)

// Terms [term_begin, term_end) multiplied by table `outer` (kNoOuter: by nothing).
struct ProgGroup {
    uint16_t outer, term_begin, term_end, pad;
};

// One step of a group's inner sum (the group's outer table is not listed), which is evaluated as a Horner chain:
//   kOpTerm  adds coeff * product of idx[0..n_factors).  Terms with the same coefficient are stored next to each
//            other and the coefficient multiplies their sum, at the term with run_last set (neg: the coefficient
//            is -1 and the sum is subtracted);
//   kOpConst adds coeff;
//   kOpFold  multiplies everything added so far by the tables idx[0..n_factors).
// z*(z*(a - v) + b) + v is thus: const a, term -v, fold z, const b, fold z, term v: two products instead of the
// four (and three coefficient products) of its monomials.
constexpr uint8_t kOpTerm = 0, kOpConst = 1, kOpFold = 2;
template <class F>
struct ProgTerm {
    typename F::E coeff;
    uint16_t n_factors;
    uint8_t coeff_is_one;
    uint8_t run_last;
    uint8_t op;
    uint8_t neg;
    uint16_t idx[DPB_MAX_FACTORS];
};

// Per-thread slots in shared memory: slot s (= 2 * table + {0: value, 1: difference}) is W 16-byte words,
// word w of thread t at ((s * W + w) * blockDim + t): consecutive threads touch consecutive words.
template <class F>
struct Slots {
    typedef typename F::E E;
    static constexpr int W = sizeof(E) / 16;
    uint4* base;
    __device__ __forceinline__ E get(uint32_t s) const {
        E v;
        uint4* q = (uint4*)&v;
#pragma unroll
        for (int w = 0; w < W; w++) q[w] = base[((size_t)s * W + w) * blockDim.x + threadIdx.x];
        return v;
    }
    __device__ __forceinline__ void put(uint32_t s, const E& v) const {
        const uint4* q = (const uint4*)&v;
#pragma unroll
        for (int w = 0; w < W; w++) base[((size_t)s * W + w) * blockDim.x + threadIdx.x] = q[w];
    }
};

// sum over groups of outer * sum over terms of coeff * product, at the tables' current values
// (only the groups g with bit g of `mask` equal to `want`; mask = want = 0 takes all)
template <class F>
__device__ __noinline__ typename F::E eval_program(const Slots<F>& sl, const ProgGroup* __restrict__ groups,
                                                   uint32_t n_groups, const ProgTerm<F>* __restrict__ terms,
                                                   uint32_t mask = 0, uint32_t want = 0) {
    typedef typename F::E E;
    E total = F::zero();
    for (uint32_t g = 0; g < n_groups; g++) {
        if (((mask >> (g & 31)) & 1u) != want) continue;
        const ProgGroup pg = groups[g];
        E inner = F::zero(), run = F::zero();
        for (uint32_t t = pg.term_begin; t < pg.term_end; t++) {
            const ProgTerm<F>& tm = terms[t];
            const uint32_t nf = tm.n_factors;
            if (tm.op == kOpFold) {
                for (uint32_t j = 0; j < nf; j++) inner = F::mul(inner, sl.get(2 * tm.idx[j]));
                continue;
            }
            if (tm.op == kOpConst) {
                inner = F::add(inner, tm.coeff);
                continue;
            }
            E prod;
            if (nf == 0) {
                prod = F::one();
            } else {
                prod = sl.get(2 * tm.idx[0]);
                for (uint32_t j = 1; j < nf; j++) prod = F::mul(prod, sl.get(2 * tm.idx[j]));
            }
            run = F::add(run, prod);
            if (tm.run_last) {
                if (tm.neg) inner = F::sub(inner, run);
                else inner = F::add(inner, tm.coeff_is_one ? run : F::mul(run, tm.coeff));
                run = F::zero();
            }
        }
        if (pg.outer != kNoOuter) inner = F::mul(inner, sl.get(2 * pg.outer));
        total = F::add(total, inner);
    }
    return total;
}

// every table's current value moves one evaluation point on
template <class F>
__device__ __noinline__ void advance_point(const Slots<F>& sl, const RoundTab* __restrict__ tabs, uint32_t k) {
    for (uint32_t j = 0; j < k; j++) {
        if (tabs[j].shift >= 0) continue;  // constant in this round
        sl.put(2 * j, F::add(sl.get(2 * j), sl.get(2 * j + 1)));
    }
}

// acc[x] = sum over pairs of the program at point x, for x = 0..D; with SKIP_ONE, x = 1 is left at zero.
template <class F, int D, bool SKIP_ONE>
__global__ void __launch_bounds__(kThreads)
    sc_round_generic(const RoundTab* __restrict__ tabs, uint32_t k, const ProgGroup* __restrict__ groups,
                     uint32_t n_groups, const ProgTerm<F>* __restrict__ terms, typename F::FoldKey rk, uint64_t n_pairs,
                     ReduceScratch<F> rs, typename F::E* out) {
    typedef typename F::E E;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Slots<F> sl;
    sl.base = (uint4*)smem_raw;
    E acc[D + 1];
#pragma unroll
    for (int x = 0; x <= D; x++) acc[x] = F::zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        for (uint32_t j = 0; j < k; j++) {
            const RoundTab t = tabs[j];
            E f0, f1;
            if (t.out) {
                E a0, a1, b0, b1;
                F::load_pair(t.in, t.dtype_in, 2 * p, a0, a1);
                F::load_pair(t.in, t.dtype_in, 2 * p + 1, b0, b1);
                f0 = F::add(a0, F::mul_key(rk, F::sub(a1, a0)));
                f1 = F::add(b0, F::mul_key(rk, F::sub(b1, b0)));
                F::store(t.out, 2 * p, f0);
                F::store(t.out, 2 * p + 1, f1);
            } else if (t.shift < 0) {
                F::load_pair(t.in, t.dtype_in, p, f0, f1);
            } else {
                f0 = F::load(t.in, t.dtype_in, p >> t.shift);
                f1 = f0;
            }
            sl.put(2 * j, f0);
            sl.put(2 * j + 1, F::sub(f1, f0));
        }
#pragma unroll
        for (int x = 0; x <= D; x++) {
            if (!(SKIP_ONE && x == 1)) acc[x] = F::add(acc[x], eval_program<F>(sl, groups, n_groups, terms));
            if (x < D) advance_point<F>(sl, tabs, k);
        }
    }
    grid_sum_publish<F, D + 1>(acc, rs, out);
}

// ---- rounds in split-eq form -----------------------------------------------------
//
// When every group of the program is "an eq table times a sum of products", the
// round polynomial factors.  After the first i' variables of an eq table over the
// point q are bound to challenges c, its pair p is S * W[p] * ((1 - q_i'), q_i') with
// S = prod_k eq(q_k, c_k) and W the eq table of the remaining coordinates, and W[p] is
// the ORIGINAL table's entry p << (i' + 1) divided by prod_{k <= i'} (1 - q_k).  So
//     s(X) = ((1 - q) + (2 q - 1) X) * H(X) + C,    H(X) = sum_p kappa * eq[p << (i' + 1)] * G(X, p),
// with G the group's sum of products (one degree less than s), kappa a host-side scalar,
// and C the groups whose tables do not move in this round.  The kernel accumulates H at
// 0, 1, .., D - 1 (without 1 after round 0: the host gets H(1) from s(0) + s(1)) and C
// once per pair; the eq tables are neither bound nor stored.  One evaluation point and
// the eq table's folds less than the direct form; results are the same field elements.
constexpr int kMaxSplitEq = 4;
template <class F>
struct SplitEqArgs {
    uint32_t n_eq;                         // eq tables read in strided form this round
    uint32_t const_groups;                 // bit g: group g does not depend on this round's variable
    uint32_t table[kMaxSplitEq];           // their table ids
    uint32_t stride_log2[kMaxSplitEq];     // pair p reads entry p << stride_log2 of the original table
    typename F::E scale[kMaxSplitEq];      // kappa
};

// acc[x] = H(x) for x = 0..D-1 (x = 1 left at zero with SKIP_ONE), acc[D] = C.
template <class F, int D, bool SKIP_ONE>
__global__ void __launch_bounds__(kThreads)
    sc_round_spliteq(const RoundTab* __restrict__ tabs, uint32_t k, const ProgGroup* __restrict__ groups,
                     uint32_t n_groups, const ProgTerm<F>* __restrict__ terms, typename F::FoldKey rk,
                     SplitEqArgs<F> eq, uint64_t n_pairs, ReduceScratch<F> rs, typename F::E* out) {
    typedef typename F::E E;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Slots<F> sl;
    sl.base = (uint4*)smem_raw;
    E acc[D + 1];
#pragma unroll
    for (int x = 0; x <= D; x++) acc[x] = F::zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        for (uint32_t j = 0; j < k; j++) {
            const RoundTab t = tabs[j];
            E f0, f1;
            int e = -1;
            for (uint32_t q = 0; q < eq.n_eq; q++)
                if (eq.table[q] == j) e = (int)q;
            if (e >= 0) {
                // descriptors mark these tables constant (shift >= 0), so advance_point leaves them alone
                f0 = F::mul(eq.scale[e], F::load(t.in, t.dtype_in, p << eq.stride_log2[e]));
                f1 = f0;
            } else if (t.out) {
                E a0, a1, b0, b1;
                F::load_pair(t.in, t.dtype_in, 2 * p, a0, a1);
                F::load_pair(t.in, t.dtype_in, 2 * p + 1, b0, b1);
                f0 = F::add(a0, F::mul_key(rk, F::sub(a1, a0)));
                f1 = F::add(b0, F::mul_key(rk, F::sub(b1, b0)));
                F::store(t.out, 2 * p, f0);
                F::store(t.out, 2 * p + 1, f1);
            } else if (t.shift < 0) {
                F::load_pair(t.in, t.dtype_in, p, f0, f1);
            } else {
                f0 = F::load(t.in, t.dtype_in, p >> t.shift);
                f1 = f0;
            }
            sl.put(2 * j, f0);
            sl.put(2 * j + 1, F::sub(f1, f0));
        }
        if (eq.const_groups) acc[D] = F::add(acc[D], eval_program<F>(sl, groups, n_groups, terms, eq.const_groups, 1u));
#pragma unroll
        for (int x = 0; x < D; x++) {
            if (!(SKIP_ONE && x == 1))
                acc[x] = F::add(acc[x], eval_program<F>(sl, groups, n_groups, terms, eq.const_groups, 0u));
            if (x < D - 1) advance_point<F>(sl, tabs, k);
        }
    }
    grid_sum_publish<F, D + 1>(acc, rs, out);
}

// out[i] = scale * in[i << stride_log2]: an eq table in the bound form the direct kernels expect, made from the
// original when a sumcheck leaves the split-eq form (the resident last-rounds kernel takes over).
template <class F>
__global__ void __launch_bounds__(kThreads)
    eq_materialize(const void* __restrict__ in, int dtype_in, uint32_t stride_log2, typename F::E scale, uint64_t n,
                   typename F::E* __restrict__ out) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        F::store(out, i, F::mul(scale, F::load(in, dtype_in, i << stride_log2)));
}

// ---- one-pass rounds over a program cut into segments ------------------------------
//
// The kernels above keep (value, difference) of EVERY table in a thread's shared-memory slots, so a program over
// many tables leaves room for few threads per SM (13 BN254 tables: one block of 128), and one thread's chain of
// dependent products is then what the round waits for.  Most long programs are sums of independent parts, though:
// the instances of a logup batch, the heads of a stacked einsum.  Inside a group (terms sharing an outer table) the
// host finds the connected components of "terms that share a table"; each becomes a segment with its own few
// tables and its own Horner-chained term list over local table numbers.  A thread then walks the segments one
// after the other, reusing the same few slots: load (bind, store) the segment's tables, evaluate its terms at
// every point into the group's running sums, and multiply by the outer table once per group and point.  Same
// field sums as the unsegmented kernels, so the same messages.
constexpr int kSegTables = 6;
struct SegDesc {
    uint16_t group;                 // program group (bit of SplitEqArgs::const_groups)
    uint16_t outer;                 // the group's outer table, or kNoOuter
    uint16_t n_tabs;
    uint16_t term_begin, term_end;  // steps in the segmented program; their idx[] number the segment's tables
    uint8_t first, last;            // first / last segment of its group
    uint16_t tab[kSegTables];
};

// a group's inner sum over the steps [begin, end) at the slots' current values
template <class F>
__device__ __noinline__ typename F::E eval_steps(const Slots<F>& sl, const ProgTerm<F>* __restrict__ terms,
                                                 uint32_t begin, uint32_t end) {
    typedef typename F::E E;
    E inner = F::zero(), run = F::zero();
    for (uint32_t t = begin; t < end; t++) {
        const ProgTerm<F>& tm = terms[t];
        const uint32_t nf = tm.n_factors;
        if (tm.op == kOpFold) {
            for (uint32_t j = 0; j < nf; j++) inner = F::mul(inner, sl.get(2 * tm.idx[j]));
            continue;
        }
        if (tm.op == kOpConst) {
            inner = F::add(inner, tm.coeff);
            continue;
        }
        E prod;
        if (nf == 0) {
            prod = F::one();
        } else {
            prod = sl.get(2 * tm.idx[0]);
            for (uint32_t j = 1; j < nf; j++) prod = F::mul(prod, sl.get(2 * tm.idx[j]));
        }
        run = F::add(run, prod);
        if (tm.run_last) {
            if (tm.neg) inner = F::sub(inner, run);
            else inner = F::add(inner, tm.coeff_is_one ? run : F::mul(run, tm.coeff));
            run = F::zero();
        }
    }
    return inner;
}

// (value at 0, difference) of table t for pair p; binds the previous challenge and stores when the round folds
template <class F>
__device__ __forceinline__ void seg_load(const RoundTab& t, uint64_t p, const typename F::FoldKey& rk,
                                         typename F::E& f0, typename F::E& df) {
    typedef typename F::E E;
    E f1;
    if (t.out) {
        E a0, a1, b0, b1;
        F::load_pair(t.in, t.dtype_in, 2 * p, a0, a1);
        F::load_pair(t.in, t.dtype_in, 2 * p + 1, b0, b1);
        f0 = F::add(a0, F::mul_key(rk, F::sub(a1, a0)));
        f1 = F::add(b0, F::mul_key(rk, F::sub(b1, b0)));
        F::store(t.out, 2 * p, f0);
        F::store(t.out, 2 * p + 1, f1);
    } else if (t.shift < 0) {
        F::load_pair(t.in, t.dtype_in, p, f0, f1);
    } else {
        f0 = F::load(t.in, t.dtype_in, p >> t.shift);
        df = F::zero();
        return;
    }
    df = F::sub(f1, f0);
}

// SPLIT: the sums of sc_round_spliteq (H at 0..D-1, then C); otherwise those of sc_round_generic (0..D).
template <class F, int D, bool SKIP_ONE, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 2)
    sc_round_seg(const RoundTab* __restrict__ tabs, const SegDesc* __restrict__ segs, uint32_t n_segs,
                 const ProgTerm<F>* __restrict__ terms, typename F::FoldKey rk, SplitEqArgs<F> eq, uint64_t n_pairs,
                 uint32_t inner_slot, ReduceScratch<F> rs, typename F::E* out) {
    typedef typename F::E E;
    constexpr int NP = SPLIT ? D : D + 1;  // evaluation points per pair; the group's running sums live in the
                                           // slots inner_slot .. inner_slot + NP - 1 (registers are for the products)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Slots<F> sl;
    sl.base = (uint4*)smem_raw;
    E acc[D + 1];
#pragma unroll
    for (int x = 0; x <= D; x++) acc[x] = F::zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        for (uint32_t s = 0; s < n_segs; s++) {
            const SegDesc sd = segs[s];
            for (uint32_t j = 0; j < sd.n_tabs; j++) {
                E f0, df;
                seg_load<F>(tabs[sd.tab[j]], p, rk, f0, df);
                sl.put(2 * j, f0);
                sl.put(2 * j + 1, df);
            }
            if (sd.term_begin == sd.term_end && sd.outer == kNoOuter) continue;  // tables no term uses: bound, stored
            const bool cg = SPLIT && ((eq.const_groups >> (sd.group & 31)) & 1u);  // the group does not move this round
            if (sd.first) {
#pragma unroll
                for (int x = 0; x < NP; x++) sl.put(inner_slot + x, F::zero());
            }
            if (sd.term_begin != sd.term_end) {
#pragma unroll
                for (int x = 0; x < NP; x++) {
                    if (cg && x > 0) break;
                    if (!(SKIP_ONE && x == 1))
                        sl.put(inner_slot + x, F::add(sl.get(inner_slot + x), eval_steps<F>(sl, terms, sd.term_begin, sd.term_end)));
                    if (x < NP - 1 && !cg)
                        for (uint32_t j = 0; j < sd.n_tabs; j++) sl.put(2 * j, F::add(sl.get(2 * j), sl.get(2 * j + 1)));
                }
            }
            if (!sd.last) continue;
            if (sd.outer == kNoOuter) {
                if (cg) {
                    acc[D] = F::add(acc[D], sl.get(inner_slot));
                } else {
#pragma unroll
                    for (int x = 0; x < NP; x++) acc[x] = F::add(acc[x], sl.get(inner_slot + x));
                }
                continue;
            }
            E o, od;
            int e = -1;
            if (SPLIT)
                for (uint32_t q = 0; q < eq.n_eq; q++)
                    if (eq.table[q] == sd.outer) e = (int)q;
            if (e >= 0) {
                const RoundTab t = tabs[sd.outer];
                o = F::mul(eq.scale[e], F::load(t.in, t.dtype_in, p << eq.stride_log2[e]));
                od = F::zero();
            } else {
                seg_load<F>(tabs[sd.outer], p, rk, o, od);
            }
            if (cg) {
                acc[D] = F::add(acc[D], F::mul(sl.get(inner_slot), o));
            } else {
#pragma unroll
                for (int x = 0; x < NP; x++) {
                    if (!(SKIP_ONE && x == 1)) acc[x] = F::add(acc[x], F::mul(sl.get(inner_slot + x), o));
                    if (x < NP - 1 && e < 0) o = F::add(o, od);
                }
            }
        }
    }
    grid_sum_publish<F, D + 1>(acc, rs, out);
}

// ---- one-pass rounds of a logup-GKR layer, from the layer's own formula -------------
//
// The layer sumcheck of the batched logup prover (zkml/src/lookup/logup_gkr/circuit.rs:231-412) sums, per instance j,
//   alpha_j * eq * (n_lo d_hi + n_hi d_lo + lambda d_lo d_hi),
// where in an instance's input layer d = c + sum_i s^i column_i, the numerators of a lookup are -1 and those of a table
// its multiplicities.  As a list of product terms that is five products per instance and point (input layer of a
// two-column lookup: nine monomials); written as  A D + C (B + lambda D)  it is two, with lambda D, and then alpha_j
// times the sum, as products by per-launch constants.  Every table sits in registers as (value, difference), one
// instance after the other: no interpreter, no shared-memory slots.  The sums are those of sc_round_spliteq for
// degree 3 (H at 0, 1, 2, then C = 0), so the host side of the round is unchanged and so are the messages.
constexpr int kLogupInner = 0, kLogupLookup = 1, kLogupTable = 2;
constexpr uint32_t kLogupMaxInst = 128;
struct LogupInst {
    uint16_t kind;   // kLogup*
    uint16_t first;  // inner: n_lo, n_hi, d_lo, d_hi at first..first+3; lookup: ncol low halves, then ncol high halves;
                     // table: multiplicities' low and high halves, then the columns as for a lookup
    uint16_t ncol;   // input layers: 1 or 2 columns
    uint16_t pad;
};
template <class F>
struct LogupConsts {
    typename F::FoldKey alpha;  // alpha_j
    typename F::FoldKey sep;    // s (input layers with two columns)
    typename F::E c;            // the constant challenge (input layers)
};

template <class F, bool SKIP_ONE>
__global__ void __launch_bounds__(128, 3)
    sc_round_logup(const RoundTab* __restrict__ tabs, const LogupInst* __restrict__ inst_g,
                   const LogupConsts<F>* __restrict__ consts_g, uint32_t n_inst, typename F::FoldKey rk,
                   typename F::FoldKey lamk, uint32_t eq_table, typename F::E eq_scale, uint32_t eq_stride_log2,
                   uint64_t n_pairs, uint32_t blocks_x, uint32_t inst_per_slice, ReduceScratch<F> rs,
                   typename F::E* out) {
    typedef typename F::E E;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    LogupConsts<F>* consts = (LogupConsts<F>*)smem_raw;
    LogupInst* inst = (LogupInst*)(smem_raw + (size_t)n_inst * sizeof(LogupConsts<F>));
    {
        const uint32_t words = n_inst * (uint32_t)(sizeof(LogupConsts<F>) / 4);
        for (uint32_t i = threadIdx.x; i < words; i += blockDim.x) ((uint32_t*)consts)[i] = ((const uint32_t*)consts_g)[i];
        for (uint32_t i = threadIdx.x; i < n_inst * (uint32_t)(sizeof(LogupInst) / 4); i += blockDim.x)
            ((uint32_t*)inst)[i] = ((const uint32_t*)inst_g)[i];
    }
    __syncthreads();
    E acc[4];
#pragma unroll
    for (int x = 0; x < 4; x++) acc[x] = F::zero();
    const RoundTab eqt = tabs[eq_table];
    // The grid is blocks_x blocks over the pairs times slices of inst_per_slice instances: a round with few pairs
    // still fills the GPU, and a thread's chain of products is one slice long (the sums are linear in the instances).
    const uint32_t slice = blockIdx.x / blocks_x, bx = blockIdx.x % blocks_x;
    const uint32_t i_begin = slice * inst_per_slice, i_end = min(n_inst, i_begin + inst_per_slice);
    const uint64_t stride = (uint64_t)blocks_x * blockDim.x;
    for (uint64_t p = (uint64_t)bx * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        E g0 = F::zero(), g1 = F::zero(), g2 = F::zero();
        for (uint32_t i = i_begin; i < i_end; i++) {
            const LogupInst in = inst[i];
            const LogupConsts<F>& k = consts[i];
            E a0, da, c0, dc, d0, dd, u0, du;  // A, C, D and U = B + lambda D (lookups: lambda D - 1), each (value, difference)
            if (in.kind == kLogupInner) {
                seg_load<F>(tabs[in.first + 3], p, rk, d0, dd);
                seg_load<F>(tabs[in.first + 1], p, rk, u0, du);
                u0 = F::add(u0, F::mul_key(lamk, d0));
                du = F::add(du, F::mul_key(lamk, dd));
                seg_load<F>(tabs[in.first + 2], p, rk, c0, dc);
                seg_load<F>(tabs[in.first], p, rk, a0, da);
            } else {
                const uint32_t col = in.first + (in.kind == kLogupTable ? 2u : 0u);
                seg_load<F>(tabs[col], p, rk, c0, dc);
                seg_load<F>(tabs[col + in.ncol], p, rk, d0, dd);
                if (in.ncol == 2) {
                    E v, dv;
                    seg_load<F>(tabs[col + 1], p, rk, v, dv);
                    c0 = F::add(c0, F::mul_key(k.sep, v));
                    dc = F::add(dc, F::mul_key(k.sep, dv));
                    seg_load<F>(tabs[col + 3], p, rk, v, dv);
                    d0 = F::add(d0, F::mul_key(k.sep, v));
                    dd = F::add(dd, F::mul_key(k.sep, dv));
                }
                c0 = F::add(c0, k.c);
                d0 = F::add(d0, k.c);
                u0 = F::mul_key(lamk, d0);
                du = F::mul_key(lamk, dd);
                if (in.kind == kLogupTable) {
                    E v, dv;
                    seg_load<F>(tabs[in.first + 1], p, rk, v, dv);
                    u0 = F::add(u0, v);
                    du = F::add(du, dv);
                    seg_load<F>(tabs[in.first], p, rk, a0, da);
                } else {
                    u0 = F::sub(u0, F::one());  // numerators -1: C (lambda D - 1) - D
                    a0 = da = F::zero();
                }
            }
            const bool lookup = in.kind == kLogupLookup;
#pragma unroll
            for (int x = 0; x < 3; x++) {
                if (!(SKIP_ONE && x == 1)) {
                    E g = F::mul(c0, u0);
                    g = lookup ? F::sub(g, d0) : F::add(g, F::mul(a0, d0));
                    g = F::mul_key(k.alpha, g);
                    if (x == 0) g0 = F::add(g0, g);
                    else if (x == 1) g1 = F::add(g1, g);
                    else g2 = F::add(g2, g);
                }
                if (x < 2) {
                    c0 = F::add(c0, dc);
                    d0 = F::add(d0, dd);
                    u0 = F::add(u0, du);
                    if (!lookup) a0 = F::add(a0, da);
                }
            }
        }
        const E e = F::mul(eq_scale, F::load(eqt.in, eqt.dtype_in, p << eq_stride_log2));
        acc[0] = F::add(acc[0], F::mul(e, g0));
        if (!SKIP_ONE) acc[1] = F::add(acc[1], F::mul(e, g1));
        acc[2] = F::add(acc[2], F::mul(e, g2));
    }
    grid_sum_publish<F, 4>(acc, rs, out);
}

// ---- resident kernel for the last rounds ---------------------------------------
//
// Once a round has only a few hundred pairs, launching a kernel per round costs
// more than the round.  sc_tail_generic stays resident instead: one block runs
// every remaining round, hands each round's sums to the host through mapped
// memory and waits there for the challenge (about 4 us per exchange, measured).
// With so little work per round the latency of one thread's chain of
// multiplications is what counts, so the block spreads a round as widely as it
// can: binding over (pair, table), evaluation over (pair, point).  Every wait
// is bounded: when the host does not answer within wait_ns the kernel records
// that in the mailbox and returns.

constexpr uint32_t kTailAbort = 0xFFFFFFFFu;
constexpr unsigned long long kTailHelloNs = 50ull * 1000 * 1000;  // 50 ms for the host's first sign of life
constexpr uint32_t kTailMaxTables = 96;

// Mailbox in mapped pinned host memory.  Everything travels as 16-byte chunks
// {8 bytes of data, sequence number, pad}: a chunk is written and read as one
// transaction, so a reader that sees the sequence number it waits for has the
// data that belongs to it, and neither side needs a system-wide fence (those
// cost more than a microsecond each on the device).
struct TailBox {
    // host -> device: the challenge that ends round i carries sequence number i + 1; kTailAbort: leave now
    TailChunk chal[4];
    // host -> device, written right after the launch call returns: sequence number 1 = "the host runs beside you"
    TailChunk hello;
    uint32_t pad0[12];
    // device -> host
    volatile uint32_t status;  // 0 running, 2 gave up waiting for a challenge, 3 no hello: launches block the host
    uint32_t pad[15];
    TailChunk evals[kMaxAccTail * 4];      // sums of round i: sequence number i + 1
    TailChunk finals[kTailMaxTables * 4];  // final evaluations: sequence number n_rounds + 1
};

static_assert(sizeof(TailBox) <= 8192, "the context reserves 8 KiB for the mailbox");

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void chunk_load(const TailChunk* c, uint64_t& data, uint32_t& seq) {
    uint32_t lo, hi, unused = 0;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(lo), "=r"(hi), "=r"(seq), "+r"(unused) : "l"(c) : "memory");
    data = (uint64_t)lo | ((uint64_t)hi << 32);
}
// The kernel can only trade messages with a host that runs while it does.  Under a profiler that serialises
// launches, or with blocking launches, the launch call returns only when the kernel has ended: the hello never
// comes, the kernel says so and leaves at once, and the host goes back to one launch per round.
__device__ __forceinline__ bool tail_hello(TailBox* box, unsigned long long limit_ns) {
    const unsigned long long t0 = global_ns();
    for (;;) {
        uint64_t d;
        uint32_t s;
        chunk_load(&box->hello, d, s);
        if (s == 1) return true;
        if (s == kTailAbort) return false;
        if (global_ns() - t0 > limit_ns) {
            box->status = 3;
            return false;
        }
    }
}

// Waits for the challenge with sequence number `want`.  true: it is in r; false: abort or time-out.
template <class E>
__device__ __forceinline__ bool tail_wait(TailBox* box, uint32_t want, unsigned long long wait_ns, E& r) {
    const unsigned long long t0 = global_ns();
    uint64_t* rw = (uint64_t*)&r;
    for (int i = 0; i < (int)(sizeof(E) / 8); i++) {
        for (;;) {
            uint32_t s;
            chunk_load(&box->chal[i], rw[i], s);
            if (s == want) break;
            if (s == kTailAbort) return false;
            if (global_ns() - t0 > wait_ns) {
                box->status = 2;
                return false;
            }
        }
    }
    return true;
}

constexpr int kTailThreads = 512;
constexpr int kTailProgBytes = 8 * 1024;  // the term program is staged in shared memory when it fits

// Shared-memory slots addressed by pair instead of by thread: slot s of pair p, n pairs in the round.
template <class F>
struct PairSlots {
    typedef typename F::E E;
    static constexpr int W = sizeof(E) / 16;
    uint4* base;
    uint32_t n;
    __device__ __forceinline__ E get(uint32_t s, uint32_t p) const {
        E v;
        uint4* q = (uint4*)&v;
#pragma unroll
        for (int w = 0; w < W; w++) q[w] = base[((size_t)s * W + w) * n + p];
        return v;
    }
    __device__ __forceinline__ void put(uint32_t s, uint32_t p, const E& v) const {
        const uint4* q = (const uint4*)&v;
#pragma unroll
        for (int w = 0; w < W; w++) base[((size_t)s * W + w) * n + p] = q[w];
    }
    // value of table j at the integer point x: f(0) + x * (f(1) - f(0)) by repeated addition
    __device__ __forceinline__ E at(uint32_t j, uint32_t p, uint32_t x) const {
        E v = get(2 * j, p);
        if (x) {
            const E d = get(2 * j + 1, p);
            for (uint32_t q = 0; q < x; q++) v = F::add(v, d);
        }
        return v;
    }
};

template <class F>
__device__ __noinline__ typename F::E eval_program_at(const PairSlots<F>& sl, uint32_t p, uint32_t x,
                                                      const ProgGroup* groups, uint32_t n_groups,
                                                      const ProgTerm<F>* terms) {
    typedef typename F::E E;
    E total = F::zero();
    for (uint32_t g = 0; g < n_groups; g++) {
        const ProgGroup pg = groups[g];
        E inner = F::zero(), run = F::zero();
        for (uint32_t t = pg.term_begin; t < pg.term_end; t++) {
            const ProgTerm<F>& tm = terms[t];
            const uint32_t nf = tm.n_factors;
            if (tm.op == kOpFold) {
                for (uint32_t j = 0; j < nf; j++) inner = F::mul(inner, sl.at(tm.idx[j], p, x));
                continue;
            }
            if (tm.op == kOpConst) {
                inner = F::add(inner, tm.coeff);
                continue;
            }
            E prod;
            if (nf == 0) {
                prod = F::one();
            } else {
                prod = sl.at(tm.idx[0], p, x);
                for (uint32_t j = 1; j < nf; j++) prod = F::mul(prod, sl.at(tm.idx[j], p, x));
            }
            run = F::add(run, prod);
            if (tm.run_last) {
                if (tm.neg) inner = F::sub(inner, run);
                else inner = F::add(inner, tm.coeff_is_one ? run : F::mul(run, tm.coeff));
                run = F::zero();
            }
        }
        if (pg.outer != kNoOuter) inner = F::mul(inner, sl.at(pg.outer, p, x));
        total = F::add(total, inner);
    }
    return total;
}

// One block; round `round` has n_pairs = 2^(n_rounds - round - 1) <= max_pairs pairs.  Per round:
//   A. items (pair, table): load, bind the previous challenge, store, fill the pair's slots;
//   B. items (pair, point): evaluate the program at that point;
//   C. tree sum over the pairs of each point; thread 0 posts the sums and waits for the challenge.
// Dynamic shared memory: [program copy | round descriptors | slots (reused for the tree sum)].
template <class F, int D>
__global__ void __launch_bounds__(kTailThreads)
    sc_tail_generic(const RoundTab* __restrict__ tabs_all, uint32_t k, const ProgGroup* __restrict__ groups_g,
                    uint32_t n_groups, const ProgTerm<F>* __restrict__ terms_g, uint32_t n_prog_terms,
                    typename F::E r, uint32_t first_round, uint32_t n_rounds, TailBox* box,
                    unsigned long long wait_ns, uint32_t prog_in_smem, uint32_t slots_offset) {
    typedef typename F::E E;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ E sh_r;
    __shared__ int sh_stop;
    __shared__ typename F::FoldKey sh_key;  // the current challenge in the form the folds multiply by
    const ProgGroup* groups = groups_g;
    const ProgTerm<F>* terms = terms_g;
    unsigned char* cursor = smem_raw;
    if (prog_in_smem) {
        ProgTerm<F>* st = (ProgTerm<F>*)cursor;
        cursor += (size_t)n_prog_terms * sizeof(ProgTerm<F>);
        ProgGroup* sg = (ProgGroup*)cursor;
        for (uint32_t i = threadIdx.x; i < n_prog_terms; i += blockDim.x) st[i] = terms_g[i];
        for (uint32_t i = threadIdx.x; i < n_groups; i += blockDim.x) sg[i] = groups_g[i];
        groups = sg;
        terms = st;
    }
    // round descriptors, double-buffered: the next round's are fetched while this round computes
    RoundTab* tabs_buf[2] = {(RoundTab*)(smem_raw + slots_offset - 2 * (size_t)k * sizeof(RoundTab)),
                             (RoundTab*)(smem_raw + slots_offset - (size_t)k * sizeof(RoundTab))};
    for (uint32_t j = threadIdx.x; j < k; j += blockDim.x) tabs_buf[0][j] = tabs_all[(size_t)first_round * k + j];
    const RoundTab* tabs = tabs_buf[0];
    PairSlots<F> sl;
    sl.base = (uint4*)(smem_raw + slots_offset);
    E* tree = (E*)(smem_raw + slots_offset);  // [point][pair], after the slots have been consumed
    if (threadIdx.x == 0) sh_stop = tail_hello(box, kTailHelloNs) ? 0 : 1;
    F::fold_key_block(r, &sh_key);
    __syncthreads();
    if (sh_stop) return;
    for (uint32_t round = first_round; round < n_rounds; round++) {
        const uint32_t n_pairs = 1u << (n_rounds - round - 1);
        sl.n = n_pairs;
        tabs = tabs_buf[(round - first_round) & 1];
        if (round + 1 < n_rounds) {
            RoundTab* nxt = tabs_buf[(round + 1 - first_round) & 1];
            for (uint32_t j = threadIdx.x; j < k; j += blockDim.x) nxt[j] = tabs_all[(size_t)(round + 1) * k + j];
        }
        __syncthreads();
        // A
        for (uint32_t w = threadIdx.x; w < n_pairs * k; w += blockDim.x) {
            const uint32_t j = w / n_pairs, p = w % n_pairs;
            const RoundTab t = tabs[j];
            E f0, f1;
            if (t.out) {
                E a0, a1, b0, b1;
                F::load_pair(t.in, t.dtype_in, 2 * (uint64_t)p, a0, a1);
                F::load_pair(t.in, t.dtype_in, 2 * (uint64_t)p + 1, b0, b1);
                f0 = F::add(a0, F::mul_key(sh_key, F::sub(a1, a0)));
                f1 = F::add(b0, F::mul_key(sh_key, F::sub(b1, b0)));
                F::store(t.out, 2 * (uint64_t)p, f0);
                F::store(t.out, 2 * (uint64_t)p + 1, f1);
            } else if (t.shift < 0) {
                F::load_pair(t.in, t.dtype_in, p, f0, f1);
            } else {
                f0 = F::load(t.in, t.dtype_in, p >> t.shift);
                f1 = f0;
            }
            sl.put(2 * j, p, f0);
            sl.put(2 * j + 1, p, F::sub(f1, f0));
        }
        __syncthreads();
        // B: the points are 0, 1, .., D in round 0 and 0, 2, .., D later (index 1 is left out)
        const uint32_t n_points = round > 0 ? D : D + 1;
        E mine[2];  // at most two items per thread: n_pairs * n_points <= 2 * blockDim
        uint32_t n_mine = 0;
        for (uint32_t w = threadIdx.x; w < n_pairs * n_points; w += blockDim.x) {
            const uint32_t xi = w / n_pairs, p = w % n_pairs;
            const uint32_t x = (round > 0 && xi >= 1) ? xi + 1 : xi;
            mine[n_mine++] = eval_program_at<F>(sl, p, x, groups, n_groups, terms);
        }
        __syncthreads();  // every slot has been read: the region becomes the tree
        n_mine = 0;
        for (uint32_t w = threadIdx.x; w < n_pairs * n_points; w += blockDim.x) tree[w] = mine[n_mine++];
        __syncthreads();
        // C
        for (uint32_t s = n_pairs >> 1; s > 0; s >>= 1) {
            for (uint32_t w = threadIdx.x; w < s * n_points; w += blockDim.x) {
                const uint32_t xi = w / s, p = w % s;
                tree[xi * n_pairs + p] = F::add(tree[xi * n_pairs + p], tree[xi * n_pairs + p + s]);
            }
            __syncthreads();
        }
        if (threadIdx.x == 0) {
            constexpr int W8 = sizeof(E) / 8;
            for (uint32_t xi = 0; xi < n_points; xi++) {
                const uint32_t x = (round > 0 && xi >= 1) ? xi + 1 : xi;
                chunks_store<E>(&box->evals[x * W8], tree[xi * n_pairs], round + 1);
            }
            E rr;
            const bool ok = tail_wait<E>(box, round + 1, wait_ns, rr);
            if (ok) sh_r = rr;
            sh_stop = ok ? 0 : 1;
        }
        __syncthreads();  // also orders this round's table stores before the next round's loads
        if (sh_stop) return;
        r = sh_r;
        F::fold_key_block(r, &sh_key);  // visible after the barrier that follows the descriptor fetch of the next round
    }
    // r ends the last round: one value per table (tabs still holds the last round's descriptors)
    for (uint32_t j = threadIdx.x; j < k; j += blockDim.x) {
        const RoundTab t = tabs[j];
        E a0, a1;
        if (t.out) F::load_pair(t.out, F::kChalDtype, 0, a0, a1);
        else F::load_pair(t.in, t.dtype_in, 0, a0, a1);
        chunks_store<E>(&box->finals[j * (sizeof(E) / 8)], F::add(a0, F::mul(r, F::sub(a1, a0))), n_rounds + 1);
    }
}

// ---- host side ---------------------------------------------------------------

// A monomial of a group's inner sum on the host: coeff * product of f.
template <class F>
struct ProgMono {
    typename F::E coeff;
    std::vector<uint16_t> f;
};

// Steps and field multiplications of a monomial list evaluated as it stands: constants summed into one
// kOpConst, the rest sorted into runs of equal coefficients.
template <class F>
inline uint32_t emit_flat(std::vector<ProgMono<F>> monos, std::vector<ProgTerm<F>>& out) {
    typedef typename F::E E;
    uint32_t cost = 0;
    E c = F::zero();
    bool have_c = false;
    std::vector<ProgMono<F>> rest;
    for (auto& m : monos) {
        if (m.f.empty()) {
            c = F::add(c, m.coeff);
            have_c = true;
        } else {
            rest.push_back(std::move(m));
        }
    }
    if (have_c && !F::is_zero(c)) {
        ProgTerm<F> pt;
        memset(&pt, 0, sizeof pt);
        pt.coeff = c;
        pt.op = kOpConst;
        out.push_back(pt);
    }
    // equal coefficients next to each other (stable: otherwise the caller's order), the last of each run marked
    std::stable_sort(rest.begin(), rest.end(),
                     [](const ProgMono<F>& x, const ProgMono<F>& y) { return memcmp(&x.coeff, &y.coeff, sizeof(E)) < 0; });
    for (size_t t = 0; t < rest.size(); t++) {
        ProgTerm<F> pt;
        memset(&pt, 0, sizeof pt);
        pt.coeff = rest[t].coeff;
        pt.op = kOpTerm;
        pt.coeff_is_one = F::is_one(pt.coeff) ? 1 : 0;
        pt.neg = F::is_one(F::neg(pt.coeff)) ? 1 : 0;
        pt.n_factors = (uint16_t)rest[t].f.size();
        for (size_t j = 0; j < rest[t].f.size(); j++) pt.idx[j] = rest[t].f[j];
        pt.run_last = (t + 1 == rest.size() || memcmp(&rest[t].coeff, &rest[t + 1].coeff, sizeof(E)) != 0) ? 1 : 0;
        cost += pt.n_factors - 1;
        if (pt.run_last && !pt.coeff_is_one && !pt.neg) cost++;
        out.push_back(pt);
    }
    return cost;
}

// The cheaper of the list as it stands and  f * (monomials with f, f taken out once) + (monomials without f),
// f the table in most monomials, the first part planned the same way.  Returns the multiplications per
// evaluation; appends the steps to `out`.
template <class F>
inline uint32_t emit_chain(const std::vector<ProgMono<F>>& monos, uint32_t k, std::vector<ProgTerm<F>>& out) {
    std::vector<ProgTerm<F>> flat;
    const uint32_t flat_cost = emit_flat<F>(monos, flat);
    std::vector<uint32_t> count(k, 0);
    for (const auto& m : monos)
        for (size_t j = 0; j < m.f.size(); j++) {
            bool first = true;
            for (size_t q = 0; q < j; q++)
                if (m.f[q] == m.f[j]) first = false;
            if (first) count[m.f[j]]++;
        }
    uint32_t best = 0, best_n = 0;
    for (uint32_t j = 0; j < k; j++)
        if (count[j] > best_n) {
            best_n = count[j];
            best = j;
        }
    if (best_n >= 2 && monos.size() <= 4096) {
        std::vector<ProgMono<F>> with, without;
        for (const auto& m : monos) {
            size_t pos = m.f.size();
            for (size_t j = 0; j < m.f.size(); j++)
                if (m.f[j] == best) {
                    pos = j;
                    break;
                }
            if (pos == m.f.size()) {
                without.push_back(m);
            } else {
                ProgMono<F> r = m;
                r.f.erase(r.f.begin() + pos);
                with.push_back(std::move(r));
            }
        }
        std::vector<ProgTerm<F>> chain;
        uint32_t cost = emit_chain<F>(with, k, chain);
        ProgTerm<F> fold;
        memset(&fold, 0, sizeof fold);
        fold.op = kOpFold;
        fold.n_factors = 1;
        fold.idx[0] = (uint16_t)best;
        chain.push_back(fold);
        cost += 1 + emit_flat<F>(without, chain);
        if (cost < flat_cost) {
            out.insert(out.end(), chain.begin(), chain.end());
            return cost;
        }
    }
    out.insert(out.end(), flat.begin(), flat.end());
    return flat_cost;
}

// Groups terms by a shared table, greedily: the table that occurs in most of the
// still ungrouped terms (at least two) becomes the outer factor of those terms.
// Tables listed in `prefer` (eq tables) become outer factors first, whatever their counts.
// Inside a group the remaining monomials become a Horner chain where that saves multiplications (emit_chain).
template <class F>
inline void compile_program(const dpb_term* terms, uint32_t n_terms, uint32_t k, std::vector<ProgGroup>& groups,
                            std::vector<ProgTerm<F>>& prog, const std::vector<bool>& prefer = std::vector<bool>(),
                            uint32_t* mults_per_point = nullptr,
                            std::vector<std::vector<ProgMono<F>>>* group_monos = nullptr) {
    typedef typename F::E E;
    std::vector<bool> used(n_terms, false);
    uint32_t left = n_terms;
    std::vector<ProgMono<F>> monos;
    auto take = [&](uint32_t t, int drop) {  // drop: position of the factor that became the outer table, or -1
        ProgMono<F> m;
        memcpy(&m.coeff, terms[t].coeff, sizeof(E));
        for (uint32_t j = 0; j < terms[t].n_factors; j++)
            if ((int)j != drop) m.f.push_back(terms[t].idx[j]);
        monos.push_back(std::move(m));
    };
    while (left > 0) {
        std::vector<uint32_t> count(k, 0);
        for (uint32_t t = 0; t < n_terms; t++) {
            if (used[t]) continue;
            for (uint32_t j = 0; j < terms[t].n_factors; j++) {
                bool first = true;
                for (uint32_t q = 0; q < j; q++)
                    if (terms[t].idx[q] == terms[t].idx[j]) first = false;
                if (first) count[terms[t].idx[j]]++;
            }
        }
        uint32_t best = 0, best_n = 0;
        bool best_pref = false;
        for (uint32_t j = 0; j < k; j++) {
            const bool pref = j < prefer.size() && prefer[j] && count[j] > 0;
            if ((pref && !best_pref) || (pref == best_pref && count[j] > best_n)) {
                best_n = count[j];
                best = j;
                best_pref = pref;
            }
        }
        if (best_pref && best_n < 2) best_n = 2;  // an eq table leads its group even when a single term uses it
        ProgGroup g;
        g.pad = 0;
        g.term_begin = (uint16_t)prog.size();
        monos.clear();
        if (best_n >= 2) {
            g.outer = (uint16_t)best;
            for (uint32_t t = 0; t < n_terms; t++) {
                if (used[t]) continue;
                int pos = -1;
                for (uint32_t j = 0; j < terms[t].n_factors; j++)
                    if (terms[t].idx[j] == best) {
                        pos = (int)j;
                        break;
                    }
                if (pos < 0) continue;
                take(t, pos);
                used[t] = true;
                left--;
            }
        } else {
            g.outer = kNoOuter;
            for (uint32_t t = 0; t < n_terms; t++) {
                if (used[t]) continue;
                take(t, -1);
                used[t] = true;
                left--;
            }
        }
        if (group_monos) group_monos->push_back(monos);
        const uint32_t cost = emit_chain<F>(monos, k, prog) + (g.outer != kNoOuter ? 1 : 0);
        if (mults_per_point) *mults_per_point += cost;
        g.term_end = (uint16_t)prog.size();
        groups.push_back(g);
    }
}

// Cuts the groups compile_program made into segments for sc_round_seg: inside a group, the connected components of
// "monomials that share a table", in the order of their first monomial; a group's constants form a component
// without tables.  Every table no term touches gets a place in a segment without steps, so that it is still bound
// and stored.  Returns false when a component has more than kSegTables tables (the caller keeps the unsegmented
// kernels) or when nothing would be gained (a single segment holds every table).
template <class F>
inline bool compile_segments(const std::vector<ProgGroup>& groups, const std::vector<std::vector<ProgMono<F>>>& group_monos,
                             uint32_t k, std::vector<SegDesc>& segs, std::vector<ProgTerm<F>>& prog, uint32_t* max_tabs) {
    if (groups.size() != group_monos.size() || groups.size() > 32) return false;
    std::vector<bool> covered(k, false);
    uint32_t widest = 1;
    for (size_t g = 0; g < groups.size(); g++) {
        const auto& monos = group_monos[g];
        if (groups[g].outer != kNoOuter) covered[groups[g].outer] = true;
        // union-find over the tables of this group's monomials
        std::vector<int> parent(k);
        for (uint32_t j = 0; j < k; j++) parent[j] = (int)j;
        auto find = [&](int x) {
            while (parent[x] != x) x = parent[x] = parent[parent[x]];
            return x;
        };
        for (const auto& m : monos)
            for (size_t j = 1; j < m.f.size(); j++) parent[find(m.f[j])] = find(m.f[0]);
        std::vector<int> comp_of_root(k, -1);
        std::vector<std::vector<ProgMono<F>>> comp_monos;
        int const_comp = -1;
        for (const auto& m : monos) {
            int c;
            if (m.f.empty()) {
                if (const_comp < 0) {
                    const_comp = (int)comp_monos.size();
                    comp_monos.emplace_back();
                }
                c = const_comp;
            } else {
                const int root = find(m.f[0]);
                if (comp_of_root[root] < 0) {
                    comp_of_root[root] = (int)comp_monos.size();
                    comp_monos.emplace_back();
                }
                c = comp_of_root[root];
            }
            comp_monos[c].push_back(m);
        }
        if (comp_monos.empty()) comp_monos.emplace_back();  // a group of nothing but its outer table cannot occur; keep a segment
        for (size_t c = 0; c < comp_monos.size(); c++) {
            std::vector<uint16_t> tabs;
            for (const auto& m : comp_monos[c])
                for (uint16_t t : m.f)
                    if (std::find(tabs.begin(), tabs.end(), t) == tabs.end()) tabs.push_back(t);
            if (tabs.size() > (size_t)kSegTables) return false;
            std::sort(tabs.begin(), tabs.end());
            std::vector<ProgMono<F>> local = comp_monos[c];
            for (auto& m : local)
                for (auto& t : m.f) t = (uint16_t)(std::find(tabs.begin(), tabs.end(), t) - tabs.begin());
            if (prog.size() + 4 * local.size() + 8 > 65535) return false;
            SegDesc sd;
            memset(&sd, 0, sizeof sd);
            sd.group = (uint16_t)g;
            sd.outer = groups[g].outer;
            sd.n_tabs = (uint16_t)tabs.size();
            for (size_t j = 0; j < tabs.size(); j++) {
                sd.tab[j] = tabs[j];
                covered[tabs[j]] = true;
            }
            sd.term_begin = (uint16_t)prog.size();
            emit_chain<F>(local, (uint32_t)tabs.size(), prog);
            sd.term_end = (uint16_t)prog.size();
            sd.first = c == 0;
            sd.last = c + 1 == comp_monos.size();
            widest = std::max<uint32_t>(widest, (uint32_t)tabs.size());
            segs.push_back(sd);
        }
    }
    // tables outside every term: bound and stored by segments without steps
    SegDesc rest;
    memset(&rest, 0, sizeof rest);
    rest.outer = kNoOuter;
    for (uint32_t j = 0; j < k; j++) {
        if (covered[j]) continue;
        rest.tab[rest.n_tabs++] = (uint16_t)j;
        if (rest.n_tabs == kSegTables) {
            segs.push_back(rest);
            widest = std::max<uint32_t>(widest, rest.n_tabs);
            rest.n_tabs = 0;
        }
    }
    if (rest.n_tabs) {
        segs.push_back(rest);
        widest = std::max<uint32_t>(widest, rest.n_tabs);
    }
    *max_tabs = widest;
    return segs.size() > 1 && (uint32_t)(2 * widest) <= k;
}

// Value at x of the polynomial of degree <= D with the given values at 0..D.
// w[j] = 1 / prod_{m != j} (j - m), computed once by lagrange_weights.
template <class F>
inline void lagrange_weights(int D, typename F::E* w) {
    typedef typename F::E E;
    for (int j = 0; j <= D; j++) {
        E den = F::one();
        for (int m = 0; m <= D; m++) {
            if (m == j) continue;
            const E diff = j > m ? F::from_u64((uint64_t)(j - m)) : F::neg(F::from_u64((uint64_t)(m - j)));
            den = F::mul(den, diff);
        }
        w[j] = F::inv(den);
    }
}
template <class F>
inline typename F::E lagrange_eval(int D, const typename F::E* evals, const typename F::E* w, const typename F::E& x) {
    typedef typename F::E E;
    E total = F::zero();
    for (int j = 0; j <= D; j++) {
        E term = F::mul(evals[j], w[j]);
        for (int m = 0; m <= D; m++)
            if (m != j) term = F::mul(term, F::sub(x, F::from_u64((uint64_t)m)));
        total = F::add(total, term);
    }
    return total;
}

}  // namespace dpb
