// C ABI: the sumcheck prover state machine (begin / round / finish).
//
// All device buffers and the per-round table descriptors are laid out when the
// sumcheck begins, so a round is one launch that binds the previous challenge
// and evaluates (two launches on the fallback path for very many tables).  The
// kernel's last block writes the round polynomial straight into mapped host
// memory and raises a flag the host polls.
#include <atomic>
#include <chrono>
#include <mutex>

#include "common.cuh"
#include "fused_kernels.cuh"
#include "fused_v2.cuh"
#include "fused_v3.cuh"
#include "fused_v4.cuh"
#include "fused_int.cuh"
#include "generic_round.cuh"
#include "comm.cuh"

namespace dpb {

constexpr size_t kSlabCacheMax = (size_t)4 << 30;  // larger blocks (claim batching over a whole model) are not kept
constexpr int kOnePassMaxSmem = 200 * 1024;  // dynamic shared memory the one-pass generic rounds may use

struct MleTrack {
    const void* orig;
    int dtype;
    uint32_t nv;
    bool padded;   // fewer variables than the sumcheck and zero above its length (else: constant in early rounds)
    void* buf[2];  // ping-pong targets of the folds (challenge-element layout)
};

}  // namespace dpb

using namespace dpb;

struct dpb_sc {
    dpb_ctx* ctx = nullptr;
    bool gl = false;
    uint32_t n = 0, k = 0, d = 0, n_terms = 0;
    uint32_t round = 0;  // next round to run
    bool finished = false;
    std::vector<MleTrack> tr;
    void* slab = nullptr;        // fold buffers
    MleDesc* d_desc = nullptr;   // [n][k]
    FoldDesc* d_fold = nullptr;  // [n][k]   folds that run before round i (i >= 1)
    std::vector<uint32_t> n_fold;  // per round
    std::vector<uint64_t> max_fold_out;
    void* d_terms = nullptr;
    void* d_final = nullptr;  // k challenge elements
    int fused_shape = 0;      // see fused_kernels.cuh
    // one-pass generic rounds (generic_round.cuh); off when the tables' slots do not fit in shared memory
    // zero-padded tables: each term is evaluated over the pairs where all its padded factors hold data
    bool ranged = false;
    uint64_t* d_tile_prefix = nullptr;  // [n][n_terms + 1]
    uint64_t* d_term_pairs = nullptr;   // [n][n_terms]
    std::vector<uint64_t> total_tiles;  // per round
    // split-eq form of the large rounds (generic_round.cuh): every group of the program is led by an eq table
    struct EqLead {
        uint32_t table = 0;         // table id of the eq table
        uint32_t first_active = 0;  // round in which it starts to move
        uint32_t vars = 0;
        std::vector<uint8_t> q;       // its point (vars elements)
        std::vector<uint8_t> inv_zp;  // vars + 1 elements: 1 / prod_{k < j} (1 - q_k)
        alignas(16) uint8_t S[32] = {0}, S_prev[32] = {0};  // prod eq(q_k, c_k) over the bound variables, now / one round ago
    };
    bool spliteq = false;
    bool eq_unbound = false;      // split-eq rounds ran: the eq tables' bound copies do not exist
    std::vector<EqLead> eq_leads;
    std::vector<uint32_t> group_lead;  // per program group: index into eq_leads
    std::vector<uint8_t> round_q, round_inv_q;  // per round: the active groups' shared coordinate and its inverse
    RoundTab* d_rtab_eq = nullptr;  // [n][k] descriptors of split-eq rounds
    alignas(16) uint8_t lag_w_h[7 * 32] = {0};  // interpolation weights for the nodes 0..d-1
    bool one_pass = false;       // large generic rounds run sc_round_generic
    bool heavy = false;          // a long term program: small rounds are spread over the terms instead
    bool has_prog = false;       // d_rtab / d_groups / d_prog are laid out (every shape that fits)
    uint32_t tail_start = ~0u;   // first round the resident last-rounds kernel may take over
    bool tail_active = false;    // that kernel is running for this sumcheck
    uint32_t n_prog_terms = 0;
    bool tail_prog_in_smem = false;
    uint32_t tail_slots_offset = 0;
    size_t tail_smem = 0;
    RoundTab* d_rtab = nullptr;  // [n][k]
    void* d_groups = nullptr;
    void* d_prog = nullptr;
    uint32_t n_groups = 0;
    uint32_t op_threads = 0;
    size_t op_smem = 0;
    bool logup_ok = false;       // a usable hint of the logup prover: sc_round_logup runs the large rounds
    void* d_logup = nullptr;     // [LogupConsts[n] | LogupInst[n]] (own allocation)
    uint32_t logup_n = 0, logup_eq = 0;
    alignas(16) uint8_t logup_lambda[32] = {0};
    bool seg_ok = false;         // the program splits into segments over few tables each: sc_round_seg runs the large rounds
    void* d_segs = nullptr;
    void* d_seg_prog = nullptr;
    uint32_t n_segs = 0;
    size_t seg_smem = 0;
    uint32_t seg_inner_slot = 0;  // first of the slots that hold a group's running sums
    alignas(16) uint8_t prev_evals[7 * 32] = {0};  // previous round message (one-pass rounds derive s(1) from it)
    alignas(16) uint8_t lag_w[7 * 32] = {0};       // interpolation weights for the nodes 0..d
    alignas(16) uint8_t prev_coeffs[5 * 32] = {0};  // previous round polynomial, low to high (fused rounds)
    // sharded sumchecks: the local part has n variables, the whole sumcheck n + log2_ranks
    uint32_t log2_ranks = 0;
    bool partial = false;  // this rank holds some of the TERMS (whole tables): every round's sums are added over the ranks
    uint32_t global_round = 0;
    std::vector<dpb_term> terms_copy;
    dpb_sc* tail = nullptr;             // the last log2_ranks rounds, identical on every rank
    std::vector<dpb_mle*> tail_mles;
    void* tail_dev = nullptr;
    std::vector<MleDesc> h_desc;
    std::vector<FoldDesc> h_fold;
};

namespace dpb {

// the table MLE j presents in round i: where it lives and in which layout
static void table_at_round(const dpb_sc* sc, uint32_t j, uint32_t i, const void** ptr, int* dtype,
                           bool* active) {
    const MleTrack& t = sc->tr[j];
    const uint32_t first_active = t.padded ? 0 : sc->n - t.nv;
    if (i < first_active) {
        *ptr = t.orig;
        *dtype = t.dtype;
        *active = false;
        return;
    }
    *active = true;
    const uint32_t folds = i - first_active;
    if (folds == 0) {
        *ptr = t.orig;
        *dtype = t.dtype;
    } else {
        *ptr = t.buf[(folds - 1) & 1];
        *dtype = chal_dtype(t.dtype);
    }
}

// the term list in the layout the two-pass evaluation kernel reads
template <class F>
static void build_terms(const dpb_sc* sc, const dpb_term* terms, std::vector<uint8_t>& out) {
    typedef typename F::E E;
    std::vector<TermDev<F>> h(sc->n_terms);
    for (uint32_t t = 0; t < sc->n_terms; t++) {
        memcpy(&h[t].coeff, terms[t].coeff, sizeof(E));
        h[t].n_factors = terms[t].n_factors;
        h[t].coeff_is_one = F::is_one(h[t].coeff) ? 1u : 0u;
        for (int j = 0; j < DPB_MAX_FACTORS; j++) h[t].idx[j] = terms[t].idx[j];
    }
    out.assign((const uint8_t*)h.data(), (const uint8_t*)h.data() + h.size() * sizeof(TermDev<F>));
}

// entries a zero-padded table holds in round i (it keeps one entry once all its own variables are bound)
static uint64_t padded_entries(const MleTrack& t, uint32_t i) { return t.nv > i ? 1ull << (t.nv - i) : 1ull; }

template <class F, int D>
static void launch_eval_ranged(dpb_sc* sc, uint32_t round) {
    dpb_ctx* ctx = sc->ctx;
    const uint64_t tiles = sc->total_tiles[round];
    uint64_t blocks = std::min<uint64_t>(tiles ? tiles : 1, (uint64_t)ctx->sm_count * 8);
    if (blocks > ctx->max_blocks) blocks = ctx->max_blocks;
    const size_t prefix_bytes = ((size_t)sc->n_terms + 1) * 8;
    const bool in_smem = prefix_bytes <= 40 * 1024;
    sc_eval_ranged<F, D><<<(uint32_t)blocks, kThreads, in_smem ? prefix_bytes : 0, ctx->stream>>>(
        sc->d_desc + (size_t)round * sc->k, (const TermDev<F>*)sc->d_terms, sc->n_terms,
        sc->d_tile_prefix + (size_t)round * (sc->n_terms + 1), sc->d_term_pairs + (size_t)round * sc->n_terms,
        in_smem ? 1u : 0u, reduce_scratch<F>(ctx), (typename F::E*)ctx->round_out);
}

template <class F, int D>
static void launch_eval(dpb_sc* sc, uint32_t round, uint64_t n_pairs) {
    dpb_ctx* ctx = sc->ctx;
    // enough (pair, slice) items to fill the GPU once, at most one slice per term
    const uint64_t target = (uint64_t)ctx->sm_count * kThreads * 2;
    uint64_t n_slices = n_pairs >= target ? 1 : (target + n_pairs - 1) / n_pairs;
    if (n_slices > sc->n_terms) n_slices = sc->n_terms;
    sc_eval_generic<F, D><<<grid_for(ctx, n_pairs * n_slices, 4), kThreads, 0, ctx->stream>>>(
        sc->d_desc + (size_t)round * sc->k, (const TermDev<F>*)sc->d_terms, sc->n_terms, n_pairs, (uint32_t)n_slices,
        reduce_scratch<F>(ctx), (typename F::E*)ctx->round_out);
}

// The one-pass round over the segmented program (sc_round_seg): degrees 2..4.
template <class F, int D, bool SPLIT>
static int launch_seg(dpb_sc* sc, uint32_t round, uint64_t n_pairs, const typename F::E& r, const SplitEqArgs<F>& eq) {
    typedef typename F::E E;
    dpb_ctx* ctx = sc->ctx;
    const bool skip = round > 0;
    // rounds that do not fill the GPU with blocks of 256 run blocks of 128 or 64 on more SMs
    uint32_t threads = kThreads;
    while (threads > 64 && n_pairs < (uint64_t)ctx->sm_count * threads) threads /= 2;
    const size_t smem = sc->seg_smem / kThreads * threads;
    uint64_t blocks = (n_pairs + threads - 1) / threads;
    const uint64_t per_sm = std::max<uint64_t>(1, std::min<uint64_t>(2 * (kThreads / threads), (uint64_t)kOnePassMaxSmem / smem));
    if (blocks > (uint64_t)ctx->sm_count * per_sm) blocks = (uint64_t)ctx->sm_count * per_sm;
    if (blocks > ctx->max_blocks) blocks = ctx->max_blocks;
    const RoundTab* tabs = (SPLIT ? sc->d_rtab_eq : sc->d_rtab) + (size_t)round * sc->k;
    const typename F::FoldKey rk = F::fold_key(r);
    if (skip) {
        DPB_CUDA(cudaFuncSetAttribute(sc_round_seg<F, D, true, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kOnePassMaxSmem));
        sc_round_seg<F, D, true, SPLIT><<<(uint32_t)blocks, threads, smem, ctx->stream>>>(
            tabs, (const SegDesc*)sc->d_segs, sc->n_segs, (const ProgTerm<F>*)sc->d_seg_prog, rk, eq, n_pairs,
            sc->seg_inner_slot, reduce_scratch<F>(ctx), (E*)ctx->round_out);
    } else {
        DPB_CUDA(cudaFuncSetAttribute(sc_round_seg<F, D, false, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kOnePassMaxSmem));
        sc_round_seg<F, D, false, SPLIT><<<(uint32_t)blocks, threads, smem, ctx->stream>>>(
            tabs, (const SegDesc*)sc->d_segs, sc->n_segs, (const ProgTerm<F>*)sc->d_seg_prog, rk, eq, n_pairs,
            sc->seg_inner_slot, reduce_scratch<F>(ctx), (E*)ctx->round_out);
    }
    return DPB_OK;
}

template <class F, int D>
static int launch_one_pass(dpb_sc* sc, uint32_t round, uint64_t n_pairs, const typename F::E& r) {
    dpb_ctx* ctx = sc->ctx;
    if constexpr (D >= 2 && D <= 4) {
        if (sc->seg_ok) {
            SplitEqArgs<F> none;
            memset(&none, 0, sizeof none);
            return launch_seg<F, D, false>(sc, round, n_pairs, r, none);
        }
    }
    const bool skip = round > 0;
    if (skip)
        DPB_CUDA(cudaFuncSetAttribute(sc_round_generic<F, D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kOnePassMaxSmem));
    else
        DPB_CUDA(cudaFuncSetAttribute(sc_round_generic<F, D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kOnePassMaxSmem));
    uint64_t blocks = (n_pairs + sc->op_threads - 1) / sc->op_threads;
    const uint64_t cap = (uint64_t)ctx->sm_count * (kOnePassMaxSmem / sc->op_smem ? kOnePassMaxSmem / sc->op_smem : 1);
    if (blocks > cap) blocks = cap;
    if (blocks > ctx->max_blocks) blocks = ctx->max_blocks;
    const RoundTab* tabs = sc->d_rtab + (size_t)round * sc->k;
    const typename F::FoldKey rk = F::fold_key(r);
    if (skip)
        sc_round_generic<F, D, true><<<(uint32_t)blocks, sc->op_threads, sc->op_smem, ctx->stream>>>(
            tabs, sc->k, (const ProgGroup*)sc->d_groups, sc->n_groups, (const ProgTerm<F>*)sc->d_prog, rk, n_pairs,
            reduce_scratch<F>(ctx), (typename F::E*)ctx->round_out);
    else
        sc_round_generic<F, D, false><<<(uint32_t)blocks, sc->op_threads, sc->op_smem, ctx->stream>>>(
            tabs, sc->k, (const ProgGroup*)sc->d_groups, sc->n_groups, (const ProgTerm<F>*)sc->d_prog, rk, n_pairs,
            reduce_scratch<F>(ctx), (typename F::E*)ctx->round_out);
    return DPB_OK;
}

// Decides whether the large rounds can run in split-eq form and precomputes what they need.  Conditions: one-pass
// rounds, degree >= 2, at most 32 groups, every group led by an eq table (tagged by dpb_eq_table / dpb_eq_tables,
// full point, at most kMaxSplitEq of them) that no term uses as an inner factor, in every round the eq tables
// that move share their coordinate, and no coordinate is 0 or 1 (their inverses are needed).
template <class F>
static void plan_spliteq(dpb_sc* sc, dpb_mle* const* mles, const std::vector<ProgGroup>& groups,
                         const std::vector<ProgTerm<F>>& prog) {
    typedef typename F::E E;
    if (!sc->one_pass || sc->d < 2 || groups.size() > 32) return;
    std::vector<dpb_sc::EqLead> leads;
    std::vector<uint32_t> group_lead(groups.size());
    for (size_t g = 0; g < groups.size(); g++) {
        const uint32_t j = groups[g].outer;
        if (j == kNoOuter || mles[j]->eq_point.size() != (size_t)sc->tr[j].nv * sizeof(E) || sc->tr[j].padded) return;
        size_t at = leads.size();
        for (size_t q = 0; q < leads.size(); q++)
            if (leads[q].table == j) at = q;
        if (at == leads.size()) {
            if (leads.size() == (size_t)kMaxSplitEq) return;
            dpb_sc::EqLead l;
            l.table = j;
            l.vars = sc->tr[j].nv;
            l.first_active = sc->n - l.vars;
            l.q = mles[j]->eq_point;
            leads.push_back(l);
        }
        group_lead[g] = (uint32_t)at;
    }
    for (const auto& t : prog)
        for (uint32_t f = 0; f < t.n_factors; f++)
            for (const auto& l : leads)
                if (t.idx[f] == l.table) return;  // an eq table inside a product: not of the form eq * G
    // while a group's eq table does not move, nothing else in the group may: no factor with more variables
    for (size_t g = 0; g < groups.size(); g++)
        for (uint32_t t = groups[g].term_begin; t < groups[g].term_end; t++)
            for (uint32_t f = 0; f < prog[t].n_factors; f++)
                if (sc->tr[prog[t].idx[f]].nv > leads[group_lead[g]].vars) return;
    // per round: the shared coordinate of the eq tables that move
    const E one = F::one();
    std::vector<E> rq(sc->n, F::zero());
    for (uint32_t i = 0; i < sc->n; i++) {
        bool have = false;
        for (const auto& l : leads) {
            if (i < l.first_active) continue;
            E q;
            memcpy(&q, l.q.data() + (size_t)(i - l.first_active) * sizeof(E), sizeof(E));
            if (have && memcmp(&q, &rq[i], sizeof(E)) != 0) return;
            rq[i] = q;
            have = true;
        }
        if (!have) return;  // nothing moves in some round: leave it to the direct kernels
        if (F::is_zero(rq[i]) || F::is_zero(F::sub(one, rq[i]))) return;
    }
    // inverses: one field inversion for all of them (Montgomery's trick)
    std::vector<E> vals;  // the values to invert: per round q, per lead the prefix products of (1 - q_k)
    for (uint32_t i = 0; i < sc->n; i++) vals.push_back(rq[i]);
    for (auto& l : leads) {
        E zp = one;
        vals.push_back(zp);
        for (uint32_t k = 0; k < l.vars; k++) {
            E q;
            memcpy(&q, l.q.data() + (size_t)k * sizeof(E), sizeof(E));
            zp = F::mul(zp, F::sub(one, q));
            vals.push_back(zp);
        }
    }
    std::vector<E> pre(vals.size() + 1, one);
    for (size_t a = 0; a < vals.size(); a++) pre[a + 1] = F::mul(pre[a], vals[a]);
    E inv_all = F::inv(pre[vals.size()]);
    std::vector<E> inv(vals.size());
    for (size_t a = vals.size(); a-- > 0;) {
        inv[a] = F::mul(inv_all, pre[a]);
        inv_all = F::mul(inv_all, vals[a]);
    }
    sc->round_q.assign((const uint8_t*)rq.data(), (const uint8_t*)rq.data() + sc->n * sizeof(E));
    sc->round_inv_q.assign((const uint8_t*)inv.data(), (const uint8_t*)inv.data() + sc->n * sizeof(E));
    size_t at = sc->n;
    for (auto& l : leads) {
        l.inv_zp.assign((const uint8_t*)(inv.data() + at), (const uint8_t*)(inv.data() + at) + (l.vars + 1) * sizeof(E));
        at += l.vars + 1;
        memcpy(l.S, &one, sizeof(E));
        memcpy(l.S_prev, &one, sizeof(E));
    }
    // interpolation weights for H (degree d - 1, nodes 0..d-1), once per process and degree
    static E weights[7][7];
    static bool have_w[7] = {false, false, false, false, false, false, false};
    static std::mutex mu;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!have_w[sc->d]) {
            lagrange_weights<F>((int)sc->d - 1, weights[sc->d]);
            have_w[sc->d] = true;
        }
        memcpy(sc->lag_w_h, weights[sc->d], sc->d * sizeof(E));
    }
    sc->eq_leads = std::move(leads);
    sc->group_lead = std::move(group_lead);
    sc->spliteq = true;
}

// Host-side plan of the one-pass rounds and the resident kernel: the grouped term
// program, launch shapes and shared-memory layouts.  No device work.
template <class F>
static void plan_program(dpb_sc* sc, const dpb_term* terms, dpb_mle* const* mles, std::vector<uint8_t>& h_groups,
                         std::vector<uint8_t>& h_prog, std::vector<uint8_t>& h_segs, std::vector<uint8_t>& h_seg_prog) {
    typedef typename F::E E;
    if (sc->k > 4096) return;  // very many tables: the two-pass kernels run every round
    std::vector<ProgGroup> groups;
    std::vector<ProgTerm<F>> prog;
    std::vector<bool> is_eq(sc->k);
    for (uint32_t j = 0; j < sc->k; j++) is_eq[j] = mles[j]->eq_point.size() == (size_t)sc->tr[j].nv * sizeof(E);
    uint32_t mults = 0;
    std::vector<std::vector<ProgMono<F>>> group_monos;
    compile_program<F>(terms, sc->n_terms, sc->k, groups, prog, is_eq, &mults, &group_monos);
    // One thread walks the whole program per (pair, point) in the one-pass rounds and in the resident kernel; once
    // that chain of multiplications takes longer than two more launches, rounds too small to fill the GPU with
    // pairs are better spread over the terms (sc_fold_generic + sc_eval_generic with slices).
    sc->heavy = (uint64_t)mults * (sc->d + 1) >= 200u;
    sc->n_groups = (uint32_t)groups.size();
    sc->n_prog_terms = (uint32_t)prog.size();
    h_groups.assign((const uint8_t*)groups.data(), (const uint8_t*)groups.data() + groups.size() * sizeof(ProgGroup));
    h_prog.assign((const uint8_t*)prog.data(), (const uint8_t*)prog.data() + prog.size() * sizeof(ProgTerm<F>));
    sc->has_prog = true;
    // one-pass rounds: every thread keeps (value, difference) of every table in shared memory
    // block size: the one that keeps most warps on an SM, between the shared memory of the slots and the kernels'
    // registers (about 124 per thread: two blocks of 256 threads, four of 128); ties go to the larger block
    const size_t per_thread = (size_t)sc->k * 2 * sizeof(E);
    uint32_t threads = 0, best_warps = 0;
    for (uint32_t t = 256; t >= 64; t /= 2) {
        if (per_thread * t > (size_t)kOnePassMaxSmem) continue;
        const uint32_t by_smem = (uint32_t)((size_t)kOnePassMaxSmem / (per_thread * t)), by_regs = 512 / t;
        const uint32_t warps = std::min(by_smem, by_regs) * t / 32;
        if (warps > best_warps) {
            best_warps = warps;
            threads = t;
        }
    }
    if (threads >= 64) {
        sc->op_threads = threads;
        sc->op_smem = per_thread * threads;
        sc->one_pass = sc->fused_shape == kFusedNone;
    }
    // the same rounds over segments of the program, when it falls apart into independent parts over few tables
    // (also when the tables are too many for the unsegmented kernels' slots: the segments need few)
    if (sc->fused_shape == kFusedNone && sc->d >= 2 && sc->d <= 4 && !getenv("DPB_NO_SEGMENTS")) {
        std::vector<SegDesc> segs;
        std::vector<ProgTerm<F>> seg_prog;
        uint32_t widest = 0;
        if (compile_segments<F>(groups, group_monos, sc->k, segs, seg_prog, &widest)) {
            sc->seg_ok = true;
            sc->one_pass = true;
            sc->n_segs = (uint32_t)segs.size();
            sc->seg_inner_slot = 2 * widest;
            sc->seg_smem = (size_t)(2 * widest + sc->d + 1) * sizeof(E) * kThreads;
            h_segs.assign((const uint8_t*)segs.data(), (const uint8_t*)segs.data() + segs.size() * sizeof(SegDesc));
            h_seg_prog.assign((const uint8_t*)seg_prog.data(),
                              (const uint8_t*)seg_prog.data() + seg_prog.size() * sizeof(ProgTerm<F>));
        }
    }
    // interpolation weights per degree, computed once per process (field inversions are slow on the host)
    static E weights[7][7];
    static bool have[7] = {false, false, false, false, false, false, false};
    static std::mutex mu;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!have[sc->d]) {
            lagrange_weights<F>((int)sc->d, weights[sc->d]);
            have[sc->d] = true;
        }
        memcpy(sc->lag_w, weights[sc->d], (sc->d + 1) * sizeof(E));
    }
    if (sc->k <= kTailMaxTables) {
        // shared memory of the resident kernel: [program copy | round descriptors | slots or sum tree]
        const size_t prog_bytes = h_prog.size() + h_groups.size();
        sc->tail_prog_in_smem = prog_bytes <= (size_t)kTailProgBytes;
        size_t off = sc->tail_prog_in_smem ? prog_bytes : 0;
        off = (off + 15) & ~(size_t)15;
        off += 2 * (size_t)sc->k * sizeof(RoundTab);  // descriptors of the current and the next round
        off = (off + 15) & ~(size_t)15;
        sc->tail_slots_offset = (uint32_t)off;
        // pairs per round the kernel can take: two items per thread in the evaluation phase, and the slots must fit
        uint64_t max_pairs = 256;
        while (max_pairs * (sc->d + 1) > 2 * (uint64_t)kTailThreads) max_pairs >>= 1;
        const size_t per_pair = std::max<size_t>((size_t)sc->k * 2, sc->d + 1) * sizeof(E);
        while (max_pairs >= 1 && off + per_pair * max_pairs > (size_t)kOnePassMaxSmem) max_pairs >>= 1;
        if (max_pairs >= 1) {
            sc->tail_smem = off + per_pair * max_pairs;
            uint32_t i = 0;
            while (i < sc->n && (1ull << (sc->n - i - 1)) > max_pairs) i++;
            sc->tail_start = i;
        }
    }
    // split-eq form for the rounds before the resident kernel's; a sumcheck that is all "last rounds" skips the
    // planning (it costs a field inversion on the host)
    if (sc->tail_start > 0) plan_spliteq<F>(sc, mles, groups, prog);
}

// per-round descriptors of the one-pass kernels: which tables are bound inside the round's kernel
static void build_round_tabs(const dpb_sc* sc, std::vector<RoundTab>& rt) {
    rt.resize((size_t)sc->n * sc->k);
    for (uint32_t i = 0; i < sc->n; i++) {
        for (uint32_t j = 0; j < sc->k; j++) {
            const MleDesc& md = sc->h_desc[(size_t)i * sc->k + j];
            RoundTab& t = rt[(size_t)i * sc->k + j];
            t.in = md.ptr;
            t.out = nullptr;
            t.dtype_in = md.dtype;
            t.shift = md.shift;
            if (i >= 1) {
                const void* pptr;
                int pdt;
                bool pactive;
                table_at_round(sc, j, i - 1, &pptr, &pdt, &pactive);
                if (pactive) {
                    t.in = pptr;
                    t.dtype_in = pdt;
                    t.out = (void*)md.ptr;
                }
            }
        }
    }
}

// ---- split-eq rounds: host side ---------------------------------------------------

// eq(q, c) = q c + (1 - q)(1 - c)
template <class F>
static typename F::E eq_scalar(const typename F::E& q, const typename F::E& c) {
    const typename F::E one = F::one();
    return F::add(F::mul(q, c), F::mul(F::sub(one, q), F::sub(one, c)));
}

// Called at the start of round i >= 1 with the challenge that ended round i - 1.
template <class F>
static void spliteq_advance(dpb_sc* sc, uint32_t i, const typename F::E& r) {
    typedef typename F::E E;
    for (auto& l : sc->eq_leads) {
        memcpy(l.S_prev, l.S, sizeof(E));
        if (i - 1 < l.first_active) continue;
        E q, S;
        memcpy(&q, l.q.data() + (size_t)(i - 1 - l.first_active) * sizeof(E), sizeof(E));
        memcpy(&S, l.S, sizeof(E));
        S = F::mul(S, eq_scalar<F>(q, r));
        memcpy(l.S, &S, sizeof(E));
    }
}

// The large rounds of a logup layer from the layer's own formula (see sumcheck_hint_logup).
template <class F>
static int launch_logup(dpb_sc* sc, uint32_t round, uint64_t n_pairs, const typename F::E& r, const SplitEqArgs<F>& eq) {
    typedef typename F::E E;
    dpb_ctx* ctx = sc->ctx;
    const uint64_t per_sm = sizeof(E) == 16 ? 4 : 3;  // resident blocks: 126 registers per thread (Goldilocks), 168 (BN254)
    // blocks of 128 threads, of 64 when the pairs do not fill the GPU even then; and when they still do not, the
    // instances are cut into slices that run as blocks of their own
    uint32_t threads = 128;
    if (n_pairs < (uint64_t)ctx->sm_count * threads) threads = 64;
    uint64_t blocks_x = (n_pairs + threads - 1) / threads;
    const uint64_t room = (uint64_t)ctx->sm_count * per_sm * (128 / threads);
    if (blocks_x > room) blocks_x = room;
    uint32_t slices = 1;
    if (blocks_x < room) slices = (uint32_t)std::min<uint64_t>(sc->logup_n, room / blocks_x);
    const uint32_t inst_per_slice = (sc->logup_n + slices - 1) / slices;
    slices = (sc->logup_n + inst_per_slice - 1) / inst_per_slice;
    uint64_t blocks = blocks_x * slices;
    if (blocks > ctx->max_blocks) {
        slices = 1;
        blocks = blocks_x = std::min<uint64_t>(blocks_x, ctx->max_blocks);
    }
    const RoundTab* tabs = sc->d_rtab_eq + (size_t)round * sc->k;
    const typename F::FoldKey rk = F::fold_key(r);
    E lam;
    memcpy(&lam, sc->logup_lambda, sizeof(E));
    const typename F::FoldKey lamk = F::fold_key(lam);
    const LogupConsts<F>* consts = (const LogupConsts<F>*)sc->d_logup;
    const LogupInst* inst = (const LogupInst*)((const char*)sc->d_logup + (size_t)sc->logup_n * sizeof(LogupConsts<F>));
    const size_t smem = (size_t)sc->logup_n * (sizeof(LogupConsts<F>) + sizeof(LogupInst));
    if (round > 0)
        sc_round_logup<F, true><<<(uint32_t)blocks, threads, smem, ctx->stream>>>(
            tabs, inst, consts, sc->logup_n, rk, lamk, sc->logup_eq, eq.scale[0], eq.stride_log2[0], n_pairs,
            (uint32_t)blocks_x, slices == 1 ? sc->logup_n : inst_per_slice, reduce_scratch<F>(ctx), (E*)ctx->round_out);
    else
        sc_round_logup<F, false><<<(uint32_t)blocks, threads, smem, ctx->stream>>>(
            tabs, inst, consts, sc->logup_n, rk, lamk, sc->logup_eq, eq.scale[0], eq.stride_log2[0], n_pairs,
            (uint32_t)blocks_x, slices == 1 ? sc->logup_n : inst_per_slice, reduce_scratch<F>(ctx), (E*)ctx->round_out);
    return DPB_OK;
}

template <class F, int D>
static int launch_spliteq(dpb_sc* sc, uint32_t round, uint64_t n_pairs, const typename F::E& r) {
    typedef typename F::E E;
    dpb_ctx* ctx = sc->ctx;
    SplitEqArgs<F> eq;
    memset(&eq, 0, sizeof eq);
    for (size_t a = 0; a < sc->eq_leads.size(); a++) {
        const auto& l = sc->eq_leads[a];
        if (round < l.first_active) {
            for (size_t g = 0; g < sc->group_lead.size(); g++)
                if (sc->group_lead[g] == a) eq.const_groups |= 1u << g;
            continue;
        }
        const uint32_t ip = round - l.first_active;
        E S, iz;
        memcpy(&S, l.S, sizeof(E));
        memcpy(&iz, l.inv_zp.data() + (size_t)(ip + 1) * sizeof(E), sizeof(E));
        eq.table[eq.n_eq] = l.table;
        eq.stride_log2[eq.n_eq] = ip + 1;
        eq.scale[eq.n_eq] = F::mul(S, iz);
        eq.n_eq++;
    }
    if constexpr (D == 3) {
        if (sc->logup_ok && eq.n_eq == 1 && eq.const_groups == 0 && eq.table[0] == sc->logup_eq)
            return launch_logup<F>(sc, round, n_pairs, r, eq);
    }
    if constexpr (D >= 2 && D <= 4) {
        if (sc->seg_ok) return launch_seg<F, D, true>(sc, round, n_pairs, r, eq);
    }
    const bool skip = round > 0;
    if (skip)
        DPB_CUDA(cudaFuncSetAttribute(sc_round_spliteq<F, D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kOnePassMaxSmem));
    else
        DPB_CUDA(cudaFuncSetAttribute(sc_round_spliteq<F, D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kOnePassMaxSmem));
    uint64_t blocks = (n_pairs + sc->op_threads - 1) / sc->op_threads;
    const uint64_t cap = (uint64_t)ctx->sm_count * (kOnePassMaxSmem / sc->op_smem ? kOnePassMaxSmem / sc->op_smem : 1);
    if (blocks > cap) blocks = cap;
    if (blocks > ctx->max_blocks) blocks = ctx->max_blocks;
    const RoundTab* tabs = sc->d_rtab_eq + (size_t)round * sc->k;
    const typename F::FoldKey rk = F::fold_key(r);
    if (skip)
        sc_round_spliteq<F, D, true><<<(uint32_t)blocks, sc->op_threads, sc->op_smem, ctx->stream>>>(
            tabs, sc->k, (const ProgGroup*)sc->d_groups, sc->n_groups, (const ProgTerm<F>*)sc->d_prog, rk, eq, n_pairs,
            reduce_scratch<F>(ctx), (E*)ctx->round_out);
    else
        sc_round_spliteq<F, D, false><<<(uint32_t)blocks, sc->op_threads, sc->op_smem, ctx->stream>>>(
            tabs, sc->k, (const ProgGroup*)sc->d_groups, sc->n_groups, (const ProgTerm<F>*)sc->d_prog, rk, eq, n_pairs,
            reduce_scratch<F>(ctx), (E*)ctx->round_out);
    return DPB_OK;
}

// raw = H(0), [H(1)], .., H(d-1), C  ->  the round message s(0..d).  `claim` = s(0) + s(1), used after round 0.
template <class F>
static void spliteq_message(const dpb_sc* sc, uint32_t i, const typename F::E* raw, const typename F::E& claim,
                            typename F::E* out) {
    typedef typename F::E E;
    const uint32_t d = sc->d;
    E H[8];
    for (uint32_t x = 0; x < d; x++) H[x] = raw[x];
    const E C = raw[d], one = F::one();
    E q, inv_q;
    memcpy(&q, sc->round_q.data() + (size_t)i * sizeof(E), sizeof(E));
    memcpy(&inv_q, sc->round_inv_q.data() + (size_t)i * sizeof(E), sizeof(E));
    if (i > 0)  // s(0) + s(1) = (1 - q) H(0) + q H(1) + 2 C
        H[1] = F::mul(F::sub(F::sub(claim, F::add(C, C)), F::mul(F::sub(one, q), H[0])), inv_q);
    H[d] = lagrange_eval<F>((int)d - 1, H, (const E*)sc->lag_w_h, F::from_u64(d));
    const E slope = F::sub(F::add(q, q), one);  // (1 - q) + (2 q - 1) x
    E l = F::sub(one, q);
    for (uint32_t x = 0; x <= d; x++) {
        out[x] = F::add(F::mul(l, H[x]), C);
        l = F::add(l, slope);
    }
}

// The direct kernels (the resident one) are about to take over at round i: give every eq table that split-eq
// rounds left unbound the bound copy those kernels expect as their input, the table of round i - 1.
template <class F>
static int spliteq_materialize(dpb_sc* sc, uint32_t i) {
    typedef typename F::E E;
    dpb_ctx* ctx = sc->ctx;
    if (i == 0) return DPB_OK;
    for (const auto& l : sc->eq_leads) {
        if (i - 1 < l.first_active) continue;
        const uint32_t f = i - 1 - l.first_active;  // variables bound in the table of round i - 1
        if (f == 0) continue;                       // that table is the original
        const void* ptr;
        int dt;
        bool active;
        table_at_round(sc, l.table, i - 1, &ptr, &dt, &active);
        E S, iz;
        memcpy(&S, l.S_prev, sizeof(E));
        memcpy(&iz, l.inv_zp.data() + (size_t)f * sizeof(E), sizeof(E));
        const uint64_t n = 1ull << (l.vars - f);
        eq_materialize<F><<<grid_for(ctx, n), kThreads, 0, ctx->stream>>>(sc->tr[l.table].orig, sc->tr[l.table].dtype, f,
                                                                         F::mul(S, iz), n, (E*)ptr);
        DPB_CUDA(cudaGetLastError());
        ctx->sumcheck_launches++;
    }
    sc->eq_unbound = false;
    return DPB_OK;
}

// ---- resident last-rounds kernel: host side -------------------------------------


// Polls the mailbox until `ready` holds; bounded, and the stream is queried now and then so that a
// kernel that died or returned early surfaces as an error.
constexpr int kTailNoHost = 1;  // internal: the kernel found that launches block the host; fall back to launches
constexpr int kTailGaveUp = 2;  // internal: the kernel's wait for a challenge ran out and it returned

template <class Ready>
static int tail_wait_host(dpb_ctx* ctx, TailBox* box, Ready ready) {
    uint64_t spins = 0;
    std::chrono::steady_clock::time_point t0;
    while (!ready()) {
        if (box->status == 3) return kTailNoHost;
        if (box->status == 2) return kTailGaveUp;
        if ((++spins & 0xFFF) == 0) {
            cudaError_t e = cudaStreamQuery(ctx->tail_stream);
            if (e != cudaSuccess && e != cudaErrorNotReady)
                return fail(DPB_ECUDA, "resident round kernel: %s", cudaGetErrorString(e));
            if (e == cudaSuccess && box->status != 2 && box->status != 3 && !ready())
                return fail(DPB_ECUDA, "the resident round kernel returned without a result (%s)",
                            cudaGetErrorString(cudaGetLastError()));
            if (spins == 0x1000) t0 = std::chrono::steady_clock::now();
            else if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > 120.0)
                return fail(DPB_ETIMEOUT, "the resident round kernel did not answer within 120 s");
        }
    }
    std::atomic_thread_fence(std::memory_order_acquire);
    return DPB_OK;
}

template <class F, int D>
static int launch_tail(dpb_sc* sc, uint32_t round, const typename F::E& r) {
    dpb_ctx* ctx = sc->ctx;
    DPB_CUDA(cudaFuncSetAttribute(sc_tail_generic<F, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kOnePassMaxSmem));
    sc_tail_generic<F, D><<<1, kTailThreads, sc->tail_smem, ctx->tail_stream>>>(
        sc->d_rtab, sc->k, (const ProgGroup*)sc->d_groups, sc->n_groups, (const ProgTerm<F>*)sc->d_prog,
        sc->n_prog_terms, r, round, sc->n, (TailBox*)ctx->tail_box_dev, ctx->tail_wait_ns, sc->tail_prog_in_smem ? 1u : 0u,
        sc->tail_slots_offset);
    DPB_CUDA(cudaGetLastError());
    return DPB_OK;
}

// the challenge as chunks: data first, then the sequence numbers
template <class E>
static void tail_post(TailBox* box, const void* chal, uint32_t seq) {
    const uint64_t* w = (const uint64_t*)chal;
    constexpr int W8 = sizeof(E) / 8;
    for (int i = 0; i < W8; i++) ((volatile TailChunk*)box->chal)[i].data = w[i];
    std::atomic_thread_fence(std::memory_order_release);
    for (int i = 0; i < W8; i++) ((volatile TailChunk*)box->chal)[i].seq = seq;
}
// element `idx` of a chunk array, once every chunk of it carries `seq`
template <class E>
static bool tail_take(const TailChunk* base, uint32_t idx, uint32_t seq, E* out) {
    constexpr int W8 = sizeof(E) / 8;
    const volatile TailChunk* c = (const volatile TailChunk*)base + (size_t)idx * W8;
    uint64_t* w = (uint64_t*)out;
    for (int i = 0; i < W8; i++) {
        if (c[i].seq != seq) return false;
        std::atomic_thread_fence(std::memory_order_acquire);
        w[i] = c[i].data;
    }
    return true;
}

// Round i through the resident kernel: start it (first use) or post the challenge
// that ends round i - 1, then wait for the sums of round i.
// (Re)starts the resident kernel at round i; r is the challenge that ended round i - 1.
template <class F>
static int tail_start_kernel(dpb_sc* sc, uint32_t i, const typename F::E& r) {
    dpb_ctx* ctx = sc->ctx;
    TailBox* box = (TailBox*)ctx->tail_box_host;
    memset(box, 0, sizeof(TailBox));  // sequence numbers of an earlier run must not be mistaken for this one's
    std::atomic_thread_fence(std::memory_order_seq_cst);
    // the kernel runs on its own stream, after everything this context has queued so far
    DPB_CUDA(cudaEventRecord(ctx->tail_ev[0], ctx->stream));
    DPB_CUDA(cudaStreamWaitEvent(ctx->tail_stream, ctx->tail_ev[0], 0));
    int rc;
    switch (sc->d) {
        case 1: rc = launch_tail<F, 1>(sc, i, r); break;
        case 2: rc = launch_tail<F, 2>(sc, i, r); break;
        case 3: rc = launch_tail<F, 3>(sc, i, r); break;
        case 4: rc = launch_tail<F, 4>(sc, i, r); break;
        case 5: rc = launch_tail<F, 5>(sc, i, r); break;
        case 6: rc = launch_tail<F, 6>(sc, i, r); break;
        default: return fail(DPB_EINVAL, "degree %u not supported", sc->d);
    }
    if (rc != DPB_OK) return rc;
    // first sign of life, as soon as the launch call is back (the kernel waits 50 ms for it)
    ((volatile TailChunk*)&box->hello)->seq = 1;
    DPB_CUDA(cudaEventRecord(ctx->tail_ev[1], ctx->tail_stream));
    ctx->sumcheck_launches++;
    return DPB_OK;
}

// Round i through the resident kernel: start it (first use) or post the challenge that ends round i - 1, then
// wait for the sums of round i.  A kernel that gave up waiting for that challenge (the host was held up for longer
// than the kernel's limit, e.g. by a device-wide synchronisation elsewhere in the process) has left every table as
// round i - 1 made it, so it is started again at round i; only a second give-up in the same round is an error.
template <class F>
static int tail_round(dpb_sc* sc, uint32_t i, const typename F::E& r, typename F::E* raw) {
    typedef typename F::E E;
    dpb_ctx* ctx = sc->ctx;
    TailBox* box = (TailBox*)ctx->tail_box_host;
    const bool first = !sc->tail_active;
    if (first) {
        if (sc->eq_unbound) DPB_TRY(spliteq_materialize<F>(sc, i));
        DPB_TRY(tail_start_kernel<F>(sc, i, r));
        sc->tail_active = true;
        ctx->tail_owner = sc;
    } else {
        tail_post<E>(box, &r, i);
    }
    const uint32_t want = i + 1;
    for (int attempt = 0;; attempt++) {
        uint32_t x = 0;  // sums taken so far; the sum at 1 is not sent after round 0
        const int rc_wait = tail_wait_host(ctx, box, [&] {
            while (x <= sc->d) {
                if (i > 0 && x == 1) {
                    x++;
                    continue;
                }
                if (!tail_take<E>(box->evals, x, want, &raw[x])) return false;
                x++;
            }
            return true;
        });
        if (rc_wait == kTailNoHost) {
            // launches block this host thread (a profiler that serialises them, or blocking launches): the kernel
            // has left without touching anything; this context runs one launch per round from now on
            cudaStreamSynchronize(ctx->tail_stream);
            ctx->tail_enabled = false;
            sc->tail_active = false;
            ctx->tail_owner = nullptr;
            return rc_wait;
        }
        if (rc_wait == kTailGaveUp && !first && attempt == 0) {
            DPB_CUDA(cudaStreamSynchronize(ctx->tail_stream));  // it has returned; make that certain
            DPB_TRY(tail_start_kernel<F>(sc, i, r));
            continue;
        }
        if (rc_wait == kTailGaveUp)
            return fail(DPB_ETIMEOUT, "the resident round kernel gave up waiting for a challenge");
        return rc_wait;
    }
}

// Posts the last challenge, collects the final evaluations and releases the kernel's slot.
template <class F>
static int run_finish(dpb_sc* sc, const void* last_challenge, void* out);

template <class F>
static int tail_finish(dpb_sc* sc, const void* last_challenge, void* out) {
    typedef typename F::E E;
    dpb_ctx* ctx = sc->ctx;
    TailBox* box = (TailBox*)ctx->tail_box_host;
    tail_post<E>(box, last_challenge, sc->n);
    uint32_t j = 0;
    int rc = tail_wait_host(ctx, box, [&] {
        while (j < sc->k) {
            if (!tail_take<E>(box->finals, j, sc->n + 1, (E*)out + j)) return false;
            j++;
        }
        return true;
    });
    // later work of this context (frees, the next sumcheck) is ordered after the kernel's end
    cudaStreamWaitEvent(ctx->stream, ctx->tail_ev[1], 0);
    sc->tail_active = false;
    ctx->tail_owner = nullptr;
    if (rc == kTailGaveUp) {
        // the kernel left after the last round without the last challenge: its tables are in place, one small launch
        DPB_CUDA(cudaStreamSynchronize(ctx->tail_stream));
        return run_finish<F>(sc, last_challenge, out);
    }
    return rc;
}

// A sumcheck that is dropped before its last round: tell the kernel to leave and wait for it.
static void tail_abort(dpb_sc* sc) {
    dpb_ctx* ctx = sc->ctx;
    TailBox* box = (TailBox*)ctx->tail_box_host;
    for (int i = 0; i < 4; i++) ((volatile TailChunk*)box->chal)[i].seq = kTailAbort;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    cudaStreamSynchronize(ctx->tail_stream);  // bounded by the kernel's own wait limit
    sc->tail_active = false;
    ctx->tail_owner = nullptr;
}

// Fused product rounds (fused_v2.cuh).  The kernels leave SAMPLES of the round
// polynomial in the result buffer; run_round converts them.
template <int K>
static void launch_fused_gl(dpb_ctx* ctx, const MleDesc* desc, const FoldDesc* folds, uint32_t round, const Gl2& r,
                            uint64_t n_pairs) {
    V2Ptrs<K> ptrs;
    const ReduceScratch<GlFam> rs = reduce_scratch<GlFam>(ctx);
    Gl2* out = (Gl2*)ctx->round_out;
    const uint32_t grid = grid_for(ctx, n_pairs, 4);
    // staged kernels (fused_v4.cuh) once a launch has enough items per thread to pipeline
    const bool staged = n_pairs >= (uint64_t)grid * kStageThreads * 2;
    if (round == 0) {
        for (int j = 0; j < K; j++) {
            ptrs.in[j] = desc[j].ptr;
            ptrs.out[j] = nullptr;
        }
        const bool base = desc[0].dtype == DPB_GL_BASE;
        if (staged && base) {
            // three resident blocks per SM leave this kernel the registers it wants
            constexpr size_t sm = Stager<K, 1, 4>::bytes();
            const uint32_t grid3 = grid_for(ctx, n_pairs, 3);
            cudaFuncSetAttribute(v4_eval0_gl<K, true, 4, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
            v4_eval0_gl<K, true, 4, 3><<<grid3, kStageThreads, sm, ctx->stream>>>(ptrs, n_pairs, rs, out);
        } else if (staged) {
            constexpr size_t sm = Stager<K, 2, 3>::bytes();
            constexpr int minb = K <= 3 ? 2 : 1;
            cudaFuncSetAttribute(v4_eval0_gl<K, false, 3, minb>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
            v4_eval0_gl<K, false, 3, minb><<<grid, kStageThreads, sm, ctx->stream>>>(ptrs, n_pairs, rs, out);
        } else if (base) {
            v2_eval0<OpsGlBase, K><<<grid, kThreads, 0, ctx->stream>>>(ptrs, n_pairs, rs, out);
        } else {
            v2_eval0<OpsGlExt, K><<<grid, kThreads, 0, ctx->stream>>>(ptrs, n_pairs, rs, out);
        }
        return;
    }
    for (int j = 0; j < K; j++) {  // folds[] lists the tables in registration order (all are active)
        ptrs.in[j] = folds[j].in;
        ptrs.out[j] = folds[j].out;
    }
    GlChal c;
    c.r0 = r.c0;
    c.r1 = r.c1;
    c.r1x7 = gl_mul_small(r.c1, (uint32_t)GL_NONRES);
    const bool base = folds[0].dtype_in == DPB_GL_BASE;
    if (staged) {
        glw::Chal wc;
        wc.r0 = glw::make_w((uint32_t)c.r0, (uint32_t)(c.r0 >> 32));
        wc.r1 = glw::make_w((uint32_t)c.r1, (uint32_t)(c.r1 >> 32));
        wc.r1x7 = glw::make_w((uint32_t)c.r1x7, (uint32_t)(c.r1x7 >> 32));
        if (base) {
            constexpr size_t sm = Stager<K, 2, 3>::bytes();
            constexpr int minb = K <= 3 ? 2 : 1;
            cudaFuncSetAttribute(v4_fold_eval_gl<K, true, 3, minb>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
            v4_fold_eval_gl<K, true, 3, minb><<<grid, kStageThreads, sm, ctx->stream>>>(ptrs, wc, n_pairs, rs, out);
        } else {
            constexpr size_t sm = Stager<K, 4, 2>::bytes();
            constexpr int minb = K <= 3 ? 2 : 1;
            cudaFuncSetAttribute(v4_fold_eval_gl<K, false, 2, minb>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
            v4_fold_eval_gl<K, false, 2, minb><<<grid, kStageThreads, sm, ctx->stream>>>(ptrs, wc, n_pairs, rs, out);
        }
        return;
    }
    if (base) v2_fold_eval_gl<K, true, 1><<<grid, kThreads, 0, ctx->stream>>>(ptrs, c, n_pairs, rs, out);
    else v2_fold_eval_gl<K, false, 1><<<grid, kThreads, 0, ctx->stream>>>(ptrs, c, n_pairs, rs, out);
}

template <int K>
static void launch_fused_fr(dpb_ctx* ctx, const MleDesc* desc, const FoldDesc* folds, uint32_t round, const Fr& r,
                            uint64_t n_pairs) {
    V2Ptrs<K> ptrs;
    const ReduceScratch<FrFam> rs = reduce_scratch<FrFam>(ctx);
    Fr* out = (Fr*)ctx->round_out;
    const uint32_t grid = grid_for(ctx, n_pairs, 4);
    for (int j = 0; j < K; j++) {
        ptrs.in[j] = round == 0 ? desc[j].ptr : folds[j].in;
        ptrs.out[j] = round == 0 ? nullptr : folds[j].out;
    }
    // integer tables (DPB_FR_I32, K <= 3): round 0 in integer arithmetic, round 1 folds integers (fused_int.cuh)
    if constexpr (K <= 3) {
        if (round == 0 && desc[0].dtype == DPB_FR_I32) {
            v2_eval0_fr_i32<K><<<grid, kThreads, 0, ctx->stream>>>(ptrs, n_pairs, rs, out);
            return;
        }
        if (round > 0 && folds[0].dtype_in == DPB_FR_I32) {
            IntFoldKey key;
            int_fold_key(r, key);
            v2_fold_eval_fr_i32<K, 2><<<grid, kThreads, 0, ctx->stream>>>(ptrs, key, n_pairs, rs, out);
            return;
        }
    }
    // two resident blocks per SM: these kernels wait on their multiply chains, more warps hide that
    if (round == 0) {
        v2_eval0<OpsFr, K, 2><<<grid, kThreads, 0, ctx->stream>>>(ptrs, n_pairs, rs, out);
    } else {
        frw::FixedMul rk;  // the fold multiplies everything by this round's challenge: precomputed rows
        fr_fixed_table(r, rk);
        v2_fold_eval_fr<K, 2><<<grid, kThreads, 0, ctx->stream>>>(ptrs, rk, n_pairs, rs, out);
    }
}

static void launch_fused(dpb_ctx* ctx, const MleDesc* desc, const FoldDesc* folds, uint32_t k, uint32_t round,
                         const Gl2& r, uint64_t n_pairs) {
    if (k == 2) launch_fused_gl<2>(ctx, desc, folds, round, r, n_pairs);
    else if (k == 3) launch_fused_gl<3>(ctx, desc, folds, round, r, n_pairs);
    else launch_fused_gl<4>(ctx, desc, folds, round, r, n_pairs);
}
static void launch_fused(dpb_ctx* ctx, const MleDesc* desc, const FoldDesc* folds, uint32_t k, uint32_t round,
                         const Fr& r, uint64_t n_pairs) {
    if (k == 2) launch_fused_fr<2>(ctx, desc, folds, round, r, n_pairs);
    else if (k == 3) launch_fused_fr<3>(ctx, desc, folds, round, r, n_pairs);
    else launch_fused_fr<4>(ctx, desc, folds, round, r, n_pairs);
}

// Collects the sums of the round just launched from the chunk area in mapped host memory: every chunk carries
// the launch's sequence number once it has arrived.  The stream is queried now and then so that a failed launch
// surfaces, and the wait is bounded.
static int wait_round_chunks(dpb_ctx* ctx, size_t msg_bytes, void* out) {
    const unsigned int want = ctx->done_value;
    const volatile TailChunk* c = (const volatile TailChunk*)ctx->result_host;
    uint64_t* dst = (uint64_t*)out;
    uint64_t spins = 0;
    std::chrono::steady_clock::time_point t0;
    for (size_t w = 0; w < msg_bytes / 8; w++) {
        while (c[w].seq != want) {
            if ((++spins & 0xFFF) == 0) {
                cudaError_t e = cudaStreamQuery(ctx->stream);
                if (e != cudaSuccess && e != cudaErrorNotReady) return fail(DPB_ECUDA, "round kernel: %s", cudaGetErrorString(e));
                if (e == cudaSuccess && c[w].seq != want) {
                    // the stream drained without the result: the launch itself failed
                    e = cudaGetLastError();
                    if (c[w].seq == want) break;
                    return fail(DPB_ECUDA, "round kernel did not deliver its result (%s)", cudaGetErrorString(e));
                }
                if (spins == 0x1000) t0 = std::chrono::steady_clock::now();
                else if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > 120.0)
                    return fail(DPB_ETIMEOUT, "round kernel did not finish within 120 s");
            }
        }
        std::atomic_thread_fence(std::memory_order_acquire);
        dst[w] = c[w].data;
    }
    return DPB_OK;
}

constexpr uint64_t kSpreadPairs = 4096;  // rounds up to this size of a heavy program are spread over its terms
constexpr uint64_t kLogupMinPairs = 4096;  // rounds above this size of a hinted logup layer run sc_round_logup
constexpr uint64_t kSpreadLightPairs = 16384;  // and of any other program (measured: 14-15 % off a logup batch)

template <class F>
static int run_round(dpb_sc* sc, const void* prev_challenge, void* out_evals) {
    typedef typename F::E E;
    dpb_ctx* ctx = sc->ctx;
    const uint32_t i = sc->round;
    const uint64_t n_pairs = 1ull << (sc->n - i - 1);
    E r = F::zero();
    if (i > 0) memcpy(&r, prev_challenge, sizeof(E));

    // A sharded sumcheck publishes into this rank's slot of the exchange area (in-place all-gather).
    const size_t msg_bytes = (sc->d + 1) * sizeof(E);
    const bool sharded = sc->log2_ranks > 0 || sc->partial;
    const bool shared_xch = sharded && ctx->xch_host != nullptr;
    if (shared_xch) {
        // this rank's slot of the shared host segment: the kernel's last block writes the sums, then the sequence number
        ctx->xseq++;
        ctx->chunk_out_dev = (char*)ctx->xch_dev + xch_slot_offset(ctx->rank, ctx->xseq);
        ctx->round_out = nullptr;
        ctx->done_value = ctx->xseq;
    } else {
        ctx->round_out = sharded ? (void*)((char*)ctx->gather_dev + (size_t)ctx->rank * msg_bytes) : ctx->result_dev;
        // unsharded rounds signal completion through a flag in mapped host memory that the host polls
        ctx->done_seq++;
        ctx->done_value = ctx->done_seq;
        ctx->chunk_out_dev = sharded ? nullptr : ctx->result_dev;
    }
    if (sc->spliteq && i > 0) spliteq_advance<F>(sc, i, r);
    // the last rounds go to the resident kernel (one per context at a time; not while profiling per launch)
    bool use_tail = sc->tail_active || (sc->has_prog && ctx->tail_enabled && !sharded && !ctx->profile && !sc->heavy &&
                                        i >= sc->tail_start && ctx->tail_owner == nullptr);
    // Rounds too small to fill the GPU with one thread per pair run as a fold launch plus an evaluation spread over
    // (pair, slice of the term list) items: a thread's chain of dependent field products is what such a round
    // waits for, and the spread form makes it several times shorter.  Heavy programs: up to kSpreadPairs pairs;
    // every other program: between the resident kernel's rounds and kSpreadLightPairs.
    // a logup layer with its own round kernel spreads over instances inside that kernel instead
    // (down to kLogupMinPairs pairs; measured: a 36-instance batch of 2^18 rows 18.7 -> 17.0 ms, below that no gain)
    const bool logup_round = sc->logup_ok && sc->spliteq && !use_tail && n_pairs > kLogupMinPairs;
    const bool spread = !logup_round &&
                        ((sc->heavy && n_pairs <= kSpreadPairs) ||
                         (!use_tail && !sc->ranged && sc->has_prog && n_pairs <= kSpreadLightPairs)) &&
                        sc->fused_shape != kFusedProduct;
    if (spread && sc->eq_unbound) DPB_TRY(spliteq_materialize<F>(sc, i));
    E raw[kMaxAcc];
    if (use_tail) {
        const int rc = tail_round<F>(sc, i, r, raw);
        if (rc == kTailNoHost) use_tail = false;  // only possible right after the kernel's launch: nothing has run
        else if (rc != DPB_OK) return rc;
    }
    const bool profiled = ctx->profile && !use_tail;
    if (profiled) DPB_CUDA(cudaEventRecord(ctx->prof_ev[0], ctx->stream));
    bool done = false;
    if (use_tail) {
        // the sums are already in raw
    } else if (sc->fused_shape == kFusedProduct) {
        launch_fused(ctx, sc->h_desc.data() + (size_t)i * sc->k, i > 0 ? sc->h_fold.data() + (size_t)i * sc->k : nullptr,
                     sc->k, i, r, n_pairs);
        done = true;
    }
    bool one_pass = use_tail;
    bool split = false;
    if (!use_tail && !done && !spread && sc->spliteq) {
        int rc = DPB_OK;
        switch (sc->d) {
            case 2: rc = launch_spliteq<F, 2>(sc, i, n_pairs, r); break;
            case 3: rc = launch_spliteq<F, 3>(sc, i, n_pairs, r); break;
            case 4: rc = launch_spliteq<F, 4>(sc, i, n_pairs, r); break;
            case 5: rc = launch_spliteq<F, 5>(sc, i, n_pairs, r); break;
            case 6: rc = launch_spliteq<F, 6>(sc, i, n_pairs, r); break;
            default: return fail(DPB_EINVAL, "degree %u not supported", sc->d);
        }
        if (rc != DPB_OK) return rc;
        one_pass = split = true;
        sc->eq_unbound = true;
    }
    if (!use_tail && !done && !split && !spread && sc->one_pass) {
        int rc = DPB_OK;
        switch (sc->d) {
            case 1: rc = launch_one_pass<F, 1>(sc, i, n_pairs, r); break;
            case 2: rc = launch_one_pass<F, 2>(sc, i, n_pairs, r); break;
            case 3: rc = launch_one_pass<F, 3>(sc, i, n_pairs, r); break;
            case 4: rc = launch_one_pass<F, 4>(sc, i, n_pairs, r); break;
            case 5: rc = launch_one_pass<F, 5>(sc, i, n_pairs, r); break;
            case 6: rc = launch_one_pass<F, 6>(sc, i, n_pairs, r); break;
            default: return fail(DPB_EINVAL, "degree %u not supported", sc->d);
        }
        if (rc != DPB_OK) return rc;
        one_pass = true;
    }
    if (!done && !one_pass) {
        if (i > 0 && sc->n_fold[i] > 0) {
            dim3 grid(grid_for(ctx, sc->max_fold_out[i], 4), sc->n_fold[i]);
            sc_fold_generic<F><<<grid, kThreads, 0, ctx->stream>>>(sc->d_fold + (size_t)i * sc->k, F::fold_key(r));
        }
        if (sc->ranged) {
            switch (sc->d) {
                case 1: launch_eval_ranged<F, 1>(sc, i); break;
                case 2: launch_eval_ranged<F, 2>(sc, i); break;
                case 3: launch_eval_ranged<F, 3>(sc, i); break;
                case 4: launch_eval_ranged<F, 4>(sc, i); break;
                case 5: launch_eval_ranged<F, 5>(sc, i); break;
                case 6: launch_eval_ranged<F, 6>(sc, i); break;
                default: return fail(DPB_EINVAL, "degree %u not supported", sc->d);
            }
        } else {
            switch (sc->d) {
                case 1: launch_eval<F, 1>(sc, i, n_pairs); break;
                case 2: launch_eval<F, 2>(sc, i, n_pairs); break;
                case 3: launch_eval<F, 3>(sc, i, n_pairs); break;
                case 4: launch_eval<F, 4>(sc, i, n_pairs); break;
                case 5: launch_eval<F, 5>(sc, i, n_pairs); break;
                case 6: launch_eval<F, 6>(sc, i, n_pairs); break;
                default: return fail(DPB_EINVAL, "degree %u not supported", sc->d);
            }
        }
    }
    DPB_CUDA(cudaGetLastError());
    if (!use_tail) ctx->sumcheck_launches += (!done && !one_pass && i > 0 && sc->n_fold[i] > 0) ? 2 : 1;
    if (profiled) DPB_CUDA(cudaEventRecord(ctx->prof_ev[1], ctx->stream));
    if (use_tail) {
        // the sums are already in raw
    } else if (sharded) {
        // every rank's partial sums -> all hosts; add them mod p (NCCL has no modular sum)
        if (shared_xch) DPB_TRY(xch_collect(ctx, ctx->xseq, msg_bytes, ctx->gather_host, 60.0));
        else DPB_TRY(allgather_to_host(ctx, ctx->round_out, msg_bytes));
        const E* g = (const E*)ctx->gather_host;
        for (uint32_t x = 0; x <= sc->d; x++) {
            E tot = g[x];
            for (int q = 1; q < ctx->nranks; q++) tot = F::add(tot, g[(size_t)q * (sc->d + 1) + x]);
            raw[x] = tot;
        }
    } else {
        DPB_TRY(wait_round_chunks(ctx, msg_bytes, raw));
    }
    if (done) {
        // samples -> evaluations at 0..=d; P(1) of later rounds comes from the previous round's polynomial
        E* coeffs = (E*)sc->prev_coeffs;
        E claim = F::zero();
        if (i > 0) claim = eval_coeffs<F>((int)sc->d, coeffs, r);
        samples_to_evals<F>((int)sc->d, raw, i == 0, claim, (E*)out_evals, coeffs);
        memcpy(sc->prev_evals, out_evals, msg_bytes);
    } else {
        if (split) {
            // raw holds H at 0..d-1 (without 1 after round 0) and the constant part: rebuild the message
            E claim = F::zero(), msg[kMaxAcc];
            if (i > 0) claim = lagrange_eval<F>((int)sc->d, (const E*)sc->prev_evals, (const E*)sc->lag_w, r);
            spliteq_message<F>(sc, i, raw, claim, msg);
            memcpy(raw, msg, msg_bytes);
        } else if (one_pass && i > 0) {
            // s(1) = previous s(r) - s(0)
            const E claim = lagrange_eval<F>((int)sc->d, (const E*)sc->prev_evals, (const E*)sc->lag_w, r);
            raw[1] = F::sub(claim, raw[0]);
        }
        memcpy(out_evals, raw, msg_bytes);
        memcpy(sc->prev_evals, raw, msg_bytes);
    }
    if (profiled) {
        float ms = 0.f;
        DPB_CUDA(cudaEventSynchronize(ctx->prof_ev[1]));
        DPB_CUDA(cudaEventElapsedTime(&ms, ctx->prof_ev[0], ctx->prof_ev[1]));
        // minimum traffic of this round: every table read once, folded tables written once
        uint64_t bytes = 0;
        const char* name;
        const bool seg = sc->seg_ok && sc->d >= 2 && sc->d <= 4;
        if (i == 0) {
            for (uint32_t j = 0; j < sc->k; j++) bytes += dtype_size(sc->tr[j].dtype) << sc->tr[j].nv;
            name = done ? (sc->tr[0].dtype == DPB_GL_BASE ? "fused_eval0<base>"
                           : sc->tr[0].dtype == DPB_FR_I32 ? "fused_eval0<i32>" : "fused_eval0")
                        : split ? (sc->logup_ok && sc->d == 3 ? "sc_round_logup" : seg ? "sc_round_seg<spliteq>" : "sc_round_spliteq")
                        : one_pass ? (seg ? "sc_round_seg" : "sc_round_generic") : "sc_eval_generic";
        } else {
            const FoldDesc* fd = sc->h_fold.data() + (size_t)i * sc->k;
            for (uint32_t j = 0; j < sc->n_fold[i]; j++)
                bytes += fd[j].n_out * (2 * dtype_size(fd[j].dtype_in) + sizeof(E));
            for (uint32_t j = 0; j < sc->k; j++)
                if (sc->h_desc[(size_t)i * sc->k + j].shift >= 0) bytes += dtype_size(sc->tr[j].dtype) << sc->tr[j].nv;
            name = done ? (fd[0].dtype_in == DPB_GL_BASE ? "fused_fold_eval<base>"
                           : fd[0].dtype_in == DPB_FR_I32 ? "fused_fold_eval<i32>" : "fused_fold_eval")
                        : split ? (sc->logup_ok && sc->d == 3 ? "sc_round_logup" : seg ? "sc_round_seg<spliteq>" : "sc_round_spliteq")
                        : one_pass ? (seg ? "sc_round_seg" : "sc_round_generic") : "sc_fold_generic+sc_eval_generic";
        }
        bool found = false;
        for (auto& e : ctx->prof_log) {
            if (e.round == i && e.alg_bytes_per_launch == bytes && strcmp(e.kernel, name) == 0) {
                e.launches++;
                e.total_ms += ms;
                found = true;
                break;
            }
        }
        if (!found) {
            dpb_profile_entry e;
            memset(&e, 0, sizeof e);
            strncpy(e.kernel, name, sizeof(e.kernel) - 1);
            e.round = i;
            e.launches = 1;
            e.total_ms = ms;
            e.alg_bytes_per_launch = bytes;
            ctx->prof_log.push_back(e);
        }
    }
    return DPB_OK;
}

template <class F>
static int run_finish(dpb_sc* sc, const void* last_challenge, void* out) {
    typedef typename F::E E;
    dpb_ctx* ctx = sc->ctx;
    E r;
    memcpy(&r, last_challenge, sizeof(E));
    sc_final_evals<F><<<(sc->k + 127) / 128, 128, 0, ctx->stream>>>(
        sc->d_desc + (size_t)(sc->n - 1) * sc->k, sc->k, r, (E*)sc->d_final);
    DPB_CUDA(cudaGetLastError());
    ctx->sumcheck_launches++;
    DPB_CUDA(cudaMemcpyAsync(out, sc->d_final, sc->k * sizeof(E), cudaMemcpyDeviceToHost, ctx->stream));
    DPB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (sc->eq_unbound) {
        // split-eq rounds never bound the eq tables: their value at the point is the running product of eq(q_k, c_k)
        for (const auto& l : sc->eq_leads) {
            E q, S;
            memcpy(&q, l.q.data() + (size_t)(sc->n - 1 - l.first_active) * sizeof(E), sizeof(E));
            memcpy(&S, l.S, sizeof(E));
            ((E*)out)[l.table] = F::mul(S, eq_scalar<F>(q, r));
        }
    }
    return DPB_OK;
}

// Sharded sumcheck, first tail round: bind the last local variable, gather the
// one-entry shards from every rank and start the (replicated) tail sumcheck.
template <class F>
static int start_tail(dpb_sc* sc, const void* prev_challenge) {
    typedef typename F::E E;
    dpb_ctx* ctx = sc->ctx;
    const int G = ctx->nranks;
    const size_t bytes = sc->k * sizeof(E);
    E r;
    memcpy(&r, prev_challenge, sizeof(E));
    E* slot = (E*)((char*)ctx->gather_dev + (size_t)ctx->rank * bytes);
    sc_final_evals<F><<<(sc->k + 127) / 128, 128, 0, ctx->stream>>>(sc->d_desc + (size_t)(sc->n - 1) * sc->k, sc->k, r, slot);
    DPB_CUDA(cudaGetLastError());
    ctx->sumcheck_launches++;
    DPB_TRY(allgather_to_host(ctx, slot, bytes));
    // gathered[g][j] -> table j entry g (rank g owns the top-variable block g)
    const E* g = (const E*)ctx->gather_host;
    std::vector<E> stage((size_t)sc->k * G);
    for (uint32_t j = 0; j < sc->k; j++)
        for (int q = 0; q < G; q++) stage[(size_t)j * G + q] = g[(size_t)q * sc->k + j];
    DPB_TRY(device_alloc(ctx, stage.size() * sizeof(E), &sc->tail_dev));
    DPB_TRY(upload_small(ctx, sc->tail_dev, stage.data(), stage.size() * sizeof(E)));
    for (uint32_t j = 0; j < sc->k; j++) {
        dpb_mle* m = nullptr;
        DPB_TRY(dpb_mle_from_device(ctx, F::kChalDtype, (char*)sc->tail_dev + (size_t)j * G * sizeof(E), (uint64_t)G, &m));
        sc->tail_mles.push_back(m);
    }
    return dpb_sumcheck_begin(ctx, sc->log2_ranks, sc->tail_mles.data(), sc->k, sc->terms_copy.data(),
                              (uint32_t)sc->terms_copy.size(), &sc->tail);
}

}  // namespace dpb

extern "C" {

int dpb_sumcheck_begin(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k,
                       const dpb_term* terms, uint32_t n_terms, dpb_sc** out) {
    if (!ctx || !mles || !terms || !out) return fail(DPB_EINVAL, "null argument");
    if (num_vars < 1 || num_vars > 40) return fail(DPB_EINVAL, "num_vars %u out of range", num_vars);
    if (k < 1 || k > 65535) return fail(DPB_EINVAL, "table count %u out of range", k);
    if (n_terms < 1) return fail(DPB_EINVAL, "no terms");
    const bool gl = is_gl(mles[0] ? mles[0]->dtype : -1);
    uint32_t d = 0;
    for (uint32_t t = 0; t < n_terms; t++) {
        if (terms[t].n_factors > DPB_MAX_FACTORS)
            return fail(DPB_EINVAL, "term %u has %u factors (max %d)", t, terms[t].n_factors, DPB_MAX_FACTORS);
        for (uint32_t j = 0; j < terms[t].n_factors; j++)
            if (terms[t].idx[j] >= k) return fail(DPB_EINVAL, "term %u refers to table %u of %u", t, terms[t].idx[j], k);
        if (terms[t].n_factors > d) d = terms[t].n_factors;
    }
    if (d < 1 || d > 6) return fail(DPB_EINVAL, "degree %u outside 1..6", d);

    dpb_sc* sc = new (std::nothrow) dpb_sc();
    if (!sc) return fail(DPB_ENOMEM, "host allocation failed");
    sc->ctx = ctx;
    sc->gl = gl;
    sc->n = num_vars;
    sc->k = k;
    sc->d = d;
    sc->n_terms = n_terms;
    sc->tr.resize(k);
    const size_t es = gl ? 16 : 32;
    size_t slab_elems = 0;
    for (uint32_t j = 0; j < k; j++) {
        const dpb_mle* m = mles[j];
        if (!m || m->ctx != ctx || !valid_dtype(m->dtype) || is_gl(m->dtype) != gl) {
            delete sc;
            return fail(DPB_EINVAL, "table %u is null, foreign or of another field", j);
        }
        const uint32_t nv = log2u(m->len);
        if (nv < 1 || nv > num_vars) {
            delete sc;
            return fail(DPB_EINVAL, "table %u has %u variables, sumcheck has %u", j, nv, num_vars);
        }
        sc->tr[j].orig = m->ptr;
        sc->tr[j].dtype = m->dtype;
        sc->tr[j].nv = nv;
        sc->tr[j].padded = m->zero_pad && nv < num_vars;
        if (sc->tr[j].padded) sc->ranged = true;
        // a zero-padded table keeps folding (as one entry) after its own variables are bound: both buffers exist
        slab_elems += (1ull << (nv - 1)) + (nv >= 2 ? (1ull << (nv - 2)) : (sc->tr[j].padded ? 1 : 0));
    }
    sc->fused_shape = sc->ranged ? kFusedNone
                                 : detect_fused_shape(nullptr, sc->tr.size(), num_vars, terms, n_terms, gl,
                                                      [&](uint32_t j) { return sc->tr[j].nv; },
                                                      [&](uint32_t j) { return sc->tr[j].dtype; });
    // host-side plan, then ONE device allocation and ONE upload:
    // [fold buffers | table descriptors | fold descriptors | terms | final values | round tables | groups | program]
    std::vector<uint8_t> h_terms, h_groups, h_prog, h_segs, h_seg_prog;
    TracePhase t_plan("sumcheck.begin.plan");
    if (gl) {
        build_terms<GlFam>(sc, terms, h_terms);
        if (!sc->ranged) plan_program<GlFam>(sc, terms, mles, h_groups, h_prog, h_segs, h_seg_prog);
    } else {
        build_terms<FrFam>(sc, terms, h_terms);
        if (!sc->ranged) plan_program<FrFam>(sc, terms, mles, h_groups, h_prog, h_segs, h_seg_prog);
    }
    // ranged evaluation: per round and term, the pairs to visit and the tiles that cover them
    std::vector<uint64_t> h_tile_prefix, h_term_pairs;
    if (sc->ranged) {
        h_tile_prefix.resize((size_t)num_vars * (n_terms + 1));
        h_term_pairs.resize((size_t)num_vars * n_terms);
        sc->total_tiles.assign(num_vars, 0);
        for (uint32_t i = 0; i < num_vars; i++) {
            uint64_t run = 0;
            for (uint32_t t = 0; t < n_terms; t++) {
                uint64_t pairs = 1ull << (num_vars - i - 1);
                for (uint32_t j = 0; j < terms[t].n_factors; j++) {
                    const MleTrack& tk = sc->tr[terms[t].idx[j]];
                    if (!tk.padded) continue;
                    const uint64_t e = padded_entries(tk, i);
                    pairs = std::min(pairs, e >= 2 ? e / 2 : 1);
                }
                h_term_pairs[(size_t)i * n_terms + t] = pairs;
                h_tile_prefix[(size_t)i * (n_terms + 1) + t] = run;
                run += (pairs + kThreads - 1) / kThreads;
            }
            h_tile_prefix[(size_t)i * (n_terms + 1) + n_terms] = run;
            sc->total_tiles[i] = run;
        }
    }
    size_t off = (slab_elems * es + 255) & ~(size_t)255;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off = (off + bytes + 15) & ~(size_t)15;
        return o;
    };
    const size_t nk = (size_t)num_vars * k;
    const size_t o_desc = take(nk * sizeof(MleDesc)), o_fold = take(nk * sizeof(FoldDesc)), o_terms = take(h_terms.size()),
                 o_final = take(k * es), o_rtab = take(sc->has_prog ? nk * sizeof(RoundTab) : 0),
                 o_groups = take(h_groups.size()), o_prog = take(h_prog.size()),
                 o_tiles = take(h_tile_prefix.size() * 8), o_pairs = take(h_term_pairs.size() * 8),
                 o_rtab_eq = take(sc->spliteq ? nk * sizeof(RoundTab) : 0), o_segs = take(h_segs.size()),
                 o_seg_prog = take(h_seg_prog.size());
    t_plan.stop();
    TracePhase t_alloc("sumcheck.begin.alloc");
    // Sumchecks of one context run one after the other, each with one block of device memory for its fold buffers
    // and descriptors.  The context keeps the last block (up to kSlabCacheMax) and hands it to the next sumcheck that
    // fits: no trip through the allocator per tree level of a logup batch.
    int rc = DPB_OK;
    if (ctx->slab_cache && !ctx->slab_cache_busy && off <= ctx->slab_cache_bytes) {
        sc->slab = ctx->slab_cache;
        ctx->slab_cache_busy = true;
    } else {
        rc = device_alloc(ctx, off, &sc->slab);
        if (rc == DPB_OK && !ctx->slab_cache_busy && off <= kSlabCacheMax) {
            device_free(ctx, ctx->slab_cache);  // smaller than what was asked for (or absent)
            ctx->slab_cache = sc->slab;
            ctx->slab_cache_bytes = off;
            ctx->slab_cache_busy = true;
        }
    }
    t_alloc.stop();
    if (rc != DPB_OK) {
        delete sc;
        return rc;
    }
    TracePhase t_desc("sumcheck.begin.descriptors_upload");
    {
        char* base = (char*)sc->slab;
        sc->d_desc = (MleDesc*)(base + o_desc);
        sc->d_fold = (FoldDesc*)(base + o_fold);
        sc->d_terms = base + o_terms;
        sc->d_final = base + o_final;
        sc->d_rtab = (RoundTab*)(base + o_rtab);
        sc->d_groups = base + o_groups;
        sc->d_prog = base + o_prog;
        sc->d_rtab_eq = (RoundTab*)(base + o_rtab_eq);
        sc->d_segs = base + o_segs;
        sc->d_seg_prog = base + o_seg_prog;
        sc->d_tile_prefix = (uint64_t*)(base + o_tiles);
        sc->d_term_pairs = (uint64_t*)(base + o_pairs);
        // ping-pong fold buffers of every table, at the front of the block
        char* p = base;
        for (uint32_t j = 0; j < k; j++) {
            const uint32_t nv = sc->tr[j].nv;
            sc->tr[j].buf[0] = p;
            p += (es << (nv - 1));
            const bool second = nv >= 2 || sc->tr[j].padded;
            sc->tr[j].buf[1] = second ? p : nullptr;
            if (second) p += nv >= 2 ? (es << (nv - 2)) : es;
        }
    }
    // descriptors for every round
    sc->h_desc.resize((size_t)num_vars * k);
    sc->h_fold.resize((size_t)num_vars * k);
    sc->n_fold.assign(num_vars, 0);
    sc->max_fold_out.assign(num_vars, 0);
    for (uint32_t i = 0; i < num_vars; i++) {
        const uint32_t v = num_vars - i;
        for (uint32_t j = 0; j < k; j++) {
            const void* ptr;
            int dt;
            bool active;
            table_at_round(sc, j, i, &ptr, &dt, &active);
            MleDesc& md = sc->h_desc[(size_t)i * k + j];
            md.ptr = ptr;
            md.dtype = dt;
            md.shift = active ? -1 : (int32_t)(v - 1 - sc->tr[j].nv);
            md.limit = sc->tr[j].padded ? padded_entries(sc->tr[j], i) : kNoLimit;
            // fold that must run before round i: tables that were active in round i-1
            if (i >= 1) {
                const void* pptr;
                int pdt;
                bool pactive;
                table_at_round(sc, j, i - 1, &pptr, &pdt, &pactive);
                if (pactive) {
                    FoldDesc& fd = sc->h_fold[(size_t)i * k + sc->n_fold[i]];
                    fd.in = pptr;
                    fd.out = (void*)ptr;
                    fd.dtype_in = pdt;
                    fd.pad = 0;
                    fd.limit_in = kNoLimit;
                    if (sc->tr[j].padded) {
                        fd.limit_in = padded_entries(sc->tr[j], i - 1);
                        fd.n_out = padded_entries(sc->tr[j], i);
                    } else
                        fd.n_out = 1ull << (sc->tr[j].nv - (i - (num_vars - sc->tr[j].nv)));
                    if (fd.n_out > sc->max_fold_out[i]) sc->max_fold_out[i] = fd.n_out;
                    sc->n_fold[i]++;
                }
            }
        }
    }
    auto cleanup = [&](int code) {
        dpb_sumcheck_free(sc);
        return code;
    };
    {
        std::vector<uint8_t> blob(off - o_desc, 0);
        auto put = [&](size_t o, const void* src, size_t bytes) {
            if (bytes) memcpy(blob.data() + (o - o_desc), src, bytes);
        };
        put(o_desc, sc->h_desc.data(), nk * sizeof(MleDesc));
        put(o_fold, sc->h_fold.data(), nk * sizeof(FoldDesc));
        put(o_terms, h_terms.data(), h_terms.size());
        if (sc->has_prog) {
            std::vector<RoundTab> rt;
            build_round_tabs(sc, rt);
            put(o_rtab, rt.data(), rt.size() * sizeof(RoundTab));
            if (sc->spliteq) {
                // split-eq rounds read a leading eq table from its original, strided: no fold, marked constant
                for (uint32_t i = 0; i < num_vars; i++)
                    for (const auto& l : sc->eq_leads) {
                        if (i < l.first_active) continue;
                        RoundTab& t = rt[(size_t)i * k + l.table];
                        t.in = sc->tr[l.table].orig;
                        t.out = nullptr;
                        t.dtype_in = sc->tr[l.table].dtype;
                        t.shift = 0;
                    }
                put(o_rtab_eq, rt.data(), rt.size() * sizeof(RoundTab));
            }
        }
        put(o_groups, h_groups.data(), h_groups.size());
        put(o_prog, h_prog.data(), h_prog.size());
        put(o_segs, h_segs.data(), h_segs.size());
        put(o_seg_prog, h_seg_prog.data(), h_seg_prog.size());
        put(o_tiles, h_tile_prefix.data(), h_tile_prefix.size() * 8);
        put(o_pairs, h_term_pairs.data(), h_term_pairs.size() * 8);
        rc = upload_small(ctx, (char*)sc->slab + o_desc, blob.data(), blob.size());
        if (rc != DPB_OK) return cleanup(rc);
    }
    *out = sc;
    return DPB_OK;
}

uint32_t dpb_sumcheck_degree(const dpb_sc* sc) { return sc ? sc->d : 0; }

int dpb_sumcheck_begin_sharded(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k,
                               const dpb_term* terms, uint32_t n_terms, dpb_sc** out) {
    if (!ctx || !mles || !terms || !out) return fail(DPB_EINVAL, "null argument");
    uint32_t c = 0;
    while ((1 << c) < ctx->nranks) c++;
    if (c == 0) return dpb_sumcheck_begin(ctx, num_vars, mles, k, terms, n_terms, out);
    if (!ctx->nccl_comm) return fail(DPB_ESTATE, "the context has no communicator (dpb_comm_init)");
    if (num_vars <= c) return fail(DPB_EINVAL, "%u variables cannot be sharded over %d ranks", num_vars, ctx->nranks);
    const uint32_t n_loc = num_vars - c;
    for (uint32_t j = 0; j < k; j++)
        if (mles[j] && mles[j]->zero_pad) return fail(DPB_EINVAL, "zero-padded tables cannot be sharded (table %u)", j);
    for (uint32_t j = 0; j < k; j++)
        if (!mles[j] || mles[j]->len != (1ull << n_loc))
            return fail(DPB_EINVAL, "a sharded sumcheck needs every table to hold its 2^%u-entry shard (table %u)", n_loc, j);
    if ((size_t)k * ctx->nranks * 32 > ctx->result_bytes || (size_t)k * ctx->nranks * 32 > ctx->gather_bytes)
        return fail(DPB_EINVAL, "too many tables (%u) for the tail exchange", k);
    dpb_sc* sc = nullptr;
    DPB_TRY(dpb_sumcheck_begin(ctx, n_loc, mles, k, terms, n_terms, &sc));
    sc->log2_ranks = c;
    sc->spliteq = false;  // the shards of an eq table are not eq tables
    sc->terms_copy.assign(terms, terms + n_terms);
    *out = sc;
    return DPB_OK;
}

}  // extern "C"

namespace dpb {

template <class F>
static void hint_logup_impl(dpb_sc* sc, const LogupHintInst* inst, uint32_t n_inst, const void* lambda, uint32_t eq_table) {
    typedef typename F::E E;
    std::vector<LogupConsts<F>> consts(n_inst);
    std::vector<LogupInst> di(n_inst);
    memset(consts.data(), 0, consts.size() * sizeof(LogupConsts<F>));
    for (uint32_t i = 0; i < n_inst; i++) {
        E a, s, c;
        memcpy(&a, inst[i].alpha, sizeof(E));
        memcpy(&s, inst[i].sep, sizeof(E));
        memcpy(&c, inst[i].constant, sizeof(E));
        consts[i].alpha = F::fold_key(a);
        consts[i].sep = F::fold_key(s);
        consts[i].c = c;
        di[i].kind = (uint16_t)inst[i].kind;
        di[i].first = (uint16_t)inst[i].first;
        di[i].ncol = (uint16_t)inst[i].ncol;
        di[i].pad = 0;
    }
    const size_t bytes = n_inst * (sizeof(LogupConsts<F>) + sizeof(LogupInst));
    if (bytes > 96 * 1024) return;
    void* d = nullptr;
    if (device_alloc(sc->ctx, bytes, &d) != DPB_OK) return;
    std::vector<uint8_t> blob(bytes);
    memcpy(blob.data(), consts.data(), n_inst * sizeof(LogupConsts<F>));
    memcpy(blob.data() + n_inst * sizeof(LogupConsts<F>), di.data(), n_inst * sizeof(LogupInst));
    if (upload_small(sc->ctx, d, blob.data(), bytes) != DPB_OK) {
        device_free(sc->ctx, d);
        return;
    }
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(sc_round_logup<F, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        cudaFuncSetAttribute(sc_round_logup<F, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        attr_set = true;
    }
    sc->d_logup = d;
    sc->logup_n = n_inst;
    sc->logup_eq = eq_table;
    memcpy(sc->logup_lambda, lambda, sizeof(E));
    sc->logup_ok = true;
}

void sumcheck_hint_logup(dpb_sc* sc, const LogupHintInst* inst, uint32_t n_inst, const void* lambda, uint32_t eq_table) {
    if (!sc || !inst || !lambda || n_inst == 0 || n_inst > kLogupMaxInst || sc->logup_ok || getenv("DPB_NO_LOGUP_KERNEL")) return;
    // usable only by a degree-3 sumcheck in split-eq form whose one eq table is the hint's and whose other tables are
    // exactly the instances', in order
    if (!sc->spliteq || sc->d != 3 || sc->eq_leads.size() != 1 || sc->eq_leads[0].table != eq_table ||
        sc->eq_leads[0].first_active != 0 || sc->log2_ranks != 0)
        return;
    uint32_t next = 0;
    for (uint32_t i = 0; i < n_inst; i++) {
        const LogupHintInst& h = inst[i];
        if (h.first != next) return;
        if (h.kind == kLogupInner) next += 4;
        else if ((h.kind == kLogupLookup || h.kind == kLogupTable) && (h.ncol == 1 || h.ncol == 2))
            next += 2 * h.ncol + (h.kind == kLogupTable ? 2 : 0);
        else return;
    }
    if (next != eq_table || next + 1 != sc->k) return;
    if (sc->gl) hint_logup_impl<GlFam>(sc, inst, n_inst, lambda, eq_table);
    else hint_logup_impl<FrFam>(sc, inst, n_inst, lambda, eq_table);
}

}  // namespace dpb

extern "C" {

int dpb_sumcheck_begin_partial(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k,
                               const dpb_term* terms, uint32_t n_terms, dpb_sc** out) {
    if (!ctx || !mles || !terms || !out) return fail(DPB_EINVAL, "null argument");
    if (ctx->nranks <= 1) return dpb_sumcheck_begin(ctx, num_vars, mles, k, terms, n_terms, out);
    if (!ctx->nccl_comm) return fail(DPB_ESTATE, "the context has no communicator (dpb_comm_init)");
    dpb_sc* sc = nullptr;
    DPB_TRY(dpb_sumcheck_begin(ctx, num_vars, mles, k, terms, n_terms, &sc));
    sc->partial = true;
    *out = sc;
    return DPB_OK;
}

int dpb_sumcheck_round(dpb_sc* sc, const void* prev_challenge, void* out_evals, uint32_t* n_evals) {
    if (!sc || !out_evals) return fail(DPB_EINVAL, "null argument");
    const uint32_t total = sc->n + sc->log2_ranks;
    if (sc->finished || sc->global_round >= total) return fail(DPB_ESTATE, "all %u rounds already ran", total);
    if (sc->global_round == 0 && prev_challenge) return fail(DPB_ESTATE, "the first round takes no challenge");
    if (sc->global_round > 0 && !prev_challenge)
        return fail(DPB_ESTATE, "round %u needs the previous challenge", sc->global_round);
    int rc;
    if (sc->global_round < sc->n) {
        rc = sc->gl ? run_round<GlFam>(sc, prev_challenge, out_evals) : run_round<FrFam>(sc, prev_challenge, out_evals);
        if (rc == DPB_OK) sc->round++;
    } else if (sc->global_round == sc->n) {
        rc = sc->gl ? start_tail<GlFam>(sc, prev_challenge) : start_tail<FrFam>(sc, prev_challenge);
        if (rc == DPB_OK) rc = dpb_sumcheck_round(sc->tail, nullptr, out_evals, nullptr);
    } else {
        rc = dpb_sumcheck_round(sc->tail, prev_challenge, out_evals, nullptr);
    }
    if (rc != DPB_OK) return rc;
    if (n_evals) *n_evals = sc->d + 1;
    sc->global_round++;
    return DPB_OK;
}

int dpb_sumcheck_finish(dpb_sc* sc, const void* last_challenge, void* out_final_evals) {
    if (!sc || !last_challenge || !out_final_evals) return fail(DPB_EINVAL, "null argument");
    if (sc->finished) return fail(DPB_ESTATE, "already finished");
    const uint32_t total = sc->n + sc->log2_ranks;
    if (sc->global_round != total) return fail(DPB_ESTATE, "only %u of %u rounds ran", sc->global_round, total);
    int rc;
    if (sc->log2_ranks > 0) rc = dpb_sumcheck_finish(sc->tail, last_challenge, out_final_evals);
    else if (sc->tail_active) rc = sc->gl ? tail_finish<GlFam>(sc, last_challenge, out_final_evals)
                                          : tail_finish<FrFam>(sc, last_challenge, out_final_evals);
    else rc = sc->gl ? run_finish<GlFam>(sc, last_challenge, out_final_evals)
                     : run_finish<FrFam>(sc, last_challenge, out_final_evals);
    if (rc != DPB_OK) return rc;
    sc->finished = true;
    return DPB_OK;
}

void dpb_sumcheck_free(dpb_sc* sc) {
    if (!sc) return;
    if (sc->tail_active) tail_abort(sc);
    if (sc->tail) dpb_sumcheck_free(sc->tail);
    for (auto* m : sc->tail_mles) dpb_mle_free(m);
    device_free(sc->ctx, sc->tail_dev);
    device_free(sc->ctx, sc->d_logup);
    // the fold buffers and every descriptor array live in this one block
    if (sc->slab && sc->slab == sc->ctx->slab_cache) sc->ctx->slab_cache_busy = false;
    else device_free(sc->ctx, sc->slab);
    delete sc;
}

}  // extern "C"
