// C ABI of the host-side prover layer (include/dpb_prover.h): transcript,
// expression expansion, IOPProverState::prove and the batched logup prover.
// Exceptions of the C++ layer are caught here and turned into status codes.
#include "../../include/dpb_prover.h"

#include "common.cuh"
#include "host/claims.hpp"
#include "host/einsum.hpp"
#include "host/evals.hpp"
#include "host/logup.hpp"
#include "host/lookup.hpp"
#include "host/prover.hpp"
#include "host/transcript.hpp"

using namespace dpb;

struct dpb_transcript {
    bool gl;
    Blake3Transcript<GlFam>* g = nullptr;
    Blake3Transcript<FrFam>* f = nullptr;
    ~dpb_transcript() {
        delete g;
        delete f;
    }
};

struct dpb_logup_proof {
    std::vector<uint8_t> bytes;
};

struct dpb_einsum_proof {
    std::vector<uint8_t> bytes;
};

namespace {

template <class Fn>
int guarded(Fn&& fn) {
    try {
        return fn();
    } catch (const dp_crypto::Error& e) {
        return fail(e.code, "%s", e.what());
    } catch (const std::bad_alloc&) {
        return fail(DPB_ENOMEM, "host allocation failed");
    } catch (const std::exception& e) {
        return fail(DPB_EINVAL, "%s", e.what());
    }
}

template <class F>
dp_crypto::Expression<F> build_expr(const dpb_expr_node* nodes, uint32_t n) {
    typedef dp_crypto::Expression<F> X;
    typedef typename F::E E;
    std::vector<X> st;
    for (uint32_t i = 0; i < n; i++) {
        const dpb_expr_node& nd = nodes[i];
        E c0, c1;
        memcpy(&c0, nd.c0, sizeof(E));
        memcpy(&c1, nd.c1, sizeof(E));
        auto pop = [&]() {
            if (st.empty()) throw dp_crypto::Error(DPB_EINVAL, "malformed expression: stack underflow");
            X x = st.back();
            st.pop_back();
            return x;
        };
        switch (nd.op) {
            case DPB_EXPR_WITIN: st.push_back(X::WitIn((uint16_t)nd.a)); break;
            case DPB_EXPR_CONSTANT: st.push_back(X::Constant(c0)); break;
            case DPB_EXPR_CHALLENGE: st.push_back(X::Challenge((uint16_t)nd.a, nd.b, c0, c1)); break;
            case DPB_EXPR_ADD: { X r = pop(), l = pop(); st.push_back(l + r); break; }
            case DPB_EXPR_SUB: { X r = pop(), l = pop(); st.push_back(l - r); break; }
            case DPB_EXPR_MUL: { X r = pop(), l = pop(); st.push_back(l * r); break; }
            case DPB_EXPR_NEG: { X x = pop(); st.push_back(-x); break; }
            default: throw dp_crypto::Error(DPB_EINVAL, "malformed expression: unknown opcode");
        }
    }
    if (st.size() != 1) throw dp_crypto::Error(DPB_EINVAL, "malformed expression: it must leave one value");
    return st[0];
}

template <class F>
std::vector<typename F::E> elems(const void* p, uint32_t n) {
    std::vector<typename F::E> v(n);
    if (n) memcpy(v.data(), p, n * sizeof(typename F::E));
    return v;
}

template <class F>
int expr_to_terms_impl(const dpb_expr_node* nodes, uint32_t n_nodes, const void* challenges, uint32_t n_ch,
                       dpb_term* out, uint32_t cap, uint32_t* n_out) {
    auto e = build_expr<F>(nodes, n_nodes);
    dp_crypto::VirtualPolynomialsBuilder<F> b(1, 0);
    auto vp = b.to_virtual_polys({e}, elems<F>(challenges, n_ch));
    *n_out = (uint32_t)vp.terms.size();
    for (uint32_t i = 0; i < vp.terms.size() && i < cap; i++) out[i] = vp.terms[i];
    return DPB_OK;
}

template <class F, class T>
int prove_sumcheck_impl(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k, const dpb_term* terms,
                        uint32_t n_terms, T& tr, void* out_round_evals, uint32_t cap, void* out_point,
                        void* out_final, uint32_t* out_degree, bool sharded = false) {
    typedef typename F::E E;
    dp_crypto::VirtualPolynomials<F> vp;
    vp.num_vars = num_vars;
    vp.mles.assign(mles, mles + k);
    vp.terms.assign(terms, terms + n_terms);
    for (const auto& t : vp.terms) vp.max_degree = std::max(vp.max_degree, t.n_factors);
    if ((uint64_t)num_vars * (vp.max_degree + 1) > cap)
        return fail(DPB_EINVAL, "round-evaluation buffer holds %u elements, %llu needed", cap,
                    (unsigned long long)num_vars * (vp.max_degree + 1));
    auto res = dp_crypto::IOPProverState<F>::prove(ctx, vp, tr, sharded);
    E* o = (E*)out_round_evals;
    for (const auto& m : res.first.proofs)
        for (const auto& v : m.evaluations) *o++ = v;
    memcpy(out_point, res.second.collect_raw_challenges().data(), num_vars * sizeof(E));
    memcpy(out_final, res.second.get_mle_flatten_final_evaluations().data(), k * sizeof(E));
    if (out_degree) *out_degree = vp.max_degree;
    return DPB_OK;
}

// hadamard.rs:93-131
template <class F, class T>
int hadamard_impl(dpb_ctx* ctx, dpb_mle* v1, dpb_mle* v2, const void* point, uint32_t n, T& tr, void* out_evals,
                  void* out_point, void* out_claims) {
    typedef typename F::E E;
    typedef dp_crypto::Expression<F> X;
    if (dpb_mle_len(v1) != (1ull << n) || dpb_mle_len(v2) != (1ull << n))
        return fail(DPB_EINVAL, "claim point has %u coordinates but the tables have %llu and %llu entries", n,
                    (unsigned long long)dpb_mle_len(v1), (unsigned long long)dpb_mle_len(v2));
    dpb_mle* beta = nullptr;
    dp_crypto::check(dpb_eq_table(ctx, F::kChalDtype, point, n, &beta));
    struct G { dpb_mle* m; ~G() { dpb_mle_free(m); } } g{beta};
    dp_crypto::VirtualPolynomialsBuilder<F> b(1, n);
    X expr = X::Constant(F::one());
    for (dpb_mle* p : {v1, v2, beta}) expr = expr * b.lift(p);
    auto vp = b.to_virtual_polys({expr}, {});
    auto res = dp_crypto::IOPProverState<F>::prove(ctx, vp, tr);
    E* o = (E*)out_evals;
    for (const auto& m : res.first.proofs)
        for (const auto& v : m.evaluations) *o++ = v;
    memcpy(out_point, res.second.collect_raw_challenges().data(), n * sizeof(E));
    memcpy(out_claims, res.second.get_mle_flatten_final_evaluations().data(), 2 * sizeof(E));
    return DPB_OK;
}

// same_poly.rs:84-114
template <class F, class T>
int same_poly_impl(dpb_ctx* ctx, dpb_mle* poly, const void* points, uint32_t n_claims, uint32_t n, T& tr,
                   void* out_evals, void* out_point, void* out_eval) {
    typedef typename F::E E;
    typedef dp_crypto::Expression<F> X;
    if (dpb_mle_len(poly) != (1ull << n)) return fail(DPB_EINVAL, "invalid input len wrt to poly");
    if (n_claims == 0) return fail(DPB_EINVAL, "no claims");
    const std::vector<E> chal = tr.read_challenges(n_claims);
    std::vector<dpb_mle*> betas(n_claims, nullptr);
    dpb_mle* beta_owner = nullptr;
    struct G {
        std::vector<dpb_mle*>& v;
        dpb_mle*& owner;
        ~G() {
            for (auto* m : v) dpb_mle_free(m);
            dpb_mle_free(owner);
        }
    } g{betas, beta_owner};
    // one eq table per claim, all built in one call
    const std::vector<uint32_t> vars(n_claims, n);
    dp_crypto::check(dpb_eq_tables(ctx, F::kChalDtype, points, vars.data(), n_claims, &beta_owner, betas.data()));
    dp_crypto::VirtualPolynomialsBuilder<F> b(1, n);
    X poly_expr = b.lift(poly);
    X sum = X::Constant(F::zero());
    for (uint32_t i = 0; i < n_claims; i++)
        sum = sum + X::Challenge((uint16_t)i, 1, F::one(), F::zero()) * b.lift(betas[i]);
    auto vp = b.to_virtual_polys({poly_expr * sum}, chal);
    auto res = dp_crypto::IOPProverState<F>::prove(ctx, vp, tr);
    E* o = (E*)out_evals;
    for (const auto& m : res.first.proofs)
        for (const auto& v : m.evaluations) *o++ = v;
    memcpy(out_point, res.second.collect_raw_challenges().data(), n * sizeof(E));
    memcpy(out_eval, res.second.get_mle_flatten_final_evaluations().data(), sizeof(E));
    return DPB_OK;
}

// prover.rs:113-122, 140-255
template <class F, class T>
int claims_impl(dpb_ctx* ctx, const dpb_committed_poly* polys, uint32_t n_polys, T& tr, void* out_evals,
                uint32_t evals_room, void* out_point, uint32_t* out_num_vars, void* out_sc_evals, uint32_t sc_room,
                void* out_chal, dpb_mle** out_rlc) {
    typedef typename F::E E;
    using namespace zkml::poly_commit;
    std::vector<CommittedPoly<F>> in(n_polys);
    for (uint32_t i = 0; i < n_polys; i++) {
        const dpb_committed_poly& s = polys[i];
        if (!s.chunks || s.n_chunks == 0) return fail(DPB_EINVAL, "polynomial %u has no chunks", i);
        if (s.n_claims && (!s.claim_points || !s.claim_evals)) return fail(DPB_EINVAL, "polynomial %u has null claims", i);
        in[i].chunks.assign(s.chunks, s.chunks + s.n_chunks);
        for (auto* c : in[i].chunks)
            if (!c || c->ctx != ctx) return fail(DPB_EINVAL, "polynomial %u has a null or foreign chunk", i);
        if (s.n_chunks & (s.n_chunks - 1)) return fail(DPB_EINVAL, "polynomial %u: the chunk count must be a power of two", i);
        const size_t pt_len = in[i].num_vars_for_chunk() + in[i].batching_vars();
        for (uint32_t c = 0; c < s.n_claims; c++) {
            Claim<F> cl;
            cl.point.assign((const E*)s.claim_points + (size_t)c * pt_len, (const E*)s.claim_points + (size_t)(c + 1) * pt_len);
            memcpy(&cl.eval, (const E*)s.claim_evals + c, sizeof(E));
            in[i].claims.push_back(std::move(cl));
        }
    }
    auto proof = claims_batching_sumcheck<F>(ctx, in, tr);
    const size_t n = proof.max_num_vars;
    if (out_num_vars) *out_num_vars = (uint32_t)n;
    if (evals_room < n * 3) return fail(DPB_EINVAL, "room for %u round evaluations, %zu needed", evals_room, n * 3);
    if (sc_room < proof.sumcheck_evals.size())
        return fail(DPB_EINVAL, "room for %u evaluations, %zu needed", sc_room, proof.sumcheck_evals.size());
    E* o = (E*)out_evals;
    for (const auto& m : proof.sumcheck_proof.proofs)
        for (const auto& v : m.evaluations) *o++ = v;
    memcpy(out_point, proof.sumcheck_point.data(), n * sizeof(E));
    memcpy(out_sc_evals, proof.sumcheck_evals.data(), proof.sumcheck_evals.size() * sizeof(E));
    if (out_rlc) {
        const std::vector<E> ch = batching_rlc<F>(ctx, proof, tr, out_rlc);
        if (out_chal) memcpy(out_chal, ch.data(), ch.size() * sizeof(E));
    }
    return DPB_OK;
}

template <class F, class T>
int logup_impl(dpb_ctx* ctx, const dpb_logup_input* inputs, uint32_t n_inputs, T& tr, dpb_logup_proof** out,
               bool partial = false) {
    typedef typename F::E E;
    using namespace zkml::logup_gkr;
    std::vector<LogUpInput<F>> in;
    for (uint32_t i = 0; i < n_inputs; i++) {
        const dpb_logup_input& s = inputs[i];
        if (!s.columns || !s.constant_challenge || !s.column_separation_challenge)
            return fail(DPB_EINVAL, "input %u has a null field", i);
        std::vector<dpb_mle*> cols(s.columns, s.columns + s.n_columns);
        for (auto* c : cols)
            if (!c) return fail(DPB_EINVAL, "input %u has a null column", i);
        E cst, sep;
        memcpy(&cst, s.constant_challenge, sizeof(E));
        memcpy(&sep, s.column_separation_challenge, sizeof(E));
        if (s.kind == DPB_LOGUP_TABLE) in.push_back(LogUpInput<F>::new_table(cols, s.multiplicities, cst, sep));
        else if (s.kind == DPB_LOGUP_LOOKUP) in.push_back(LogUpInput<F>::new_lookup(cols, cst, sep, s.columns_per_instance));
        else return fail(DPB_EINVAL, "input %u has unknown kind %d", i, s.kind);
    }
    auto proof = new_batch_multiple_sizes_prove<F>(ctx, in, tr, partial);
    dpb_logup_proof* p = new dpb_logup_proof();
    p->bytes = proof.serialize();
    *out = p;
    return DPB_OK;
}

// einsum/prove.rs:48-335
template <class F, class T>
int einsum_impl(dpb_ctx* ctx, const dpb_einsum_operand* lhs, const dpb_einsum_operand* rhs, uint32_t n_rhs,
                dpb_mle* lhs_padded, T& tr, dpb_einsum_proof** out) {
    typedef typename F::E E;
    using namespace zkml::einsum;
    auto convert = [&](const dpb_einsum_operand& s, const char* side, uint32_t i) {
        if (!s.tensor || !s.shape || !s.axis_kind || s.rank == 0)
            throw dp_crypto::Error(DPB_EINVAL, std::string(side) + " operand " + std::to_string(i) + " has a null field");
        Operand<F> op;
        op.tensor = s.tensor;
        op.on_device = s.tensor_on_device != 0;
        op.shape.assign(s.shape, s.shape + s.rank);
        op.kind.assign(s.axis_kind, s.axis_kind + s.rank);
        op.points.resize(s.rank);
        for (uint32_t a = 0; a < s.rank; a++) {
            const uint32_t len = s.axis_point_len ? s.axis_point_len[a] : 0;
            if (op.kind[a] != DPB_AXIS_CONTRACTED && len) {
                if (!s.axis_points || !s.axis_points[a])
                    throw dp_crypto::Error(DPB_EINVAL, std::string(side) + " operand " + std::to_string(i) +
                                                           ": an axis has a point length but no point");
                op.points[a] = elems<F>(s.axis_points[a], len);
            }
            if (op.kind[a] != DPB_AXIS_CONTRACTED && (1ull << len) < op.shape[a])
                throw dp_crypto::Error(DPB_EINVAL, std::string(side) + " operand " + std::to_string(i) +
                                                       ": an outer or stacked axis needs ceil_log2(size) coordinates");
        }
        return op;
    };
    std::vector<Operand<F>> l, r;
    for (uint32_t i = 0; i < n_rhs; i++) l.push_back(convert(lhs[i], "left", i));
    for (uint32_t i = 0; i < n_rhs; i++) r.push_back(convert(rhs[i], "right", i));
    if (lhs_padded && lhs_padded->ctx != ctx) return fail(DPB_EINVAL, "the padded left tensor belongs to another context");
    const EinsumProof<F> pr = prove<F>(ctx, l, r, lhs_padded, tr);

    dpb_einsum_proof* p = new dpb_einsum_proof();
    auto& b = p->bytes;
    auto u32 = [&](uint64_t v) {
        const uint32_t x = (uint32_t)v;
        b.insert(b.end(), (const uint8_t*)&x, (const uint8_t*)&x + 4);
    };
    auto scal = [&](const E& v) {
        uint8_t c[32];
        dpb::to_canonical(v, c);
        b.insert(b.end(), c, c + dpb::canonical_size(v));
    };
    auto sumcheck = [&](const dp_crypto::IOPProof<F>& sp) {
        u32(sp.proofs.size());
        for (const auto& m : sp.proofs) {
            u32(m.evaluations.size());
            for (const auto& v : m.evaluations) scal(v);
        }
    };
    auto claim = [&](const std::vector<E>& pt, const E& ev) {
        u32(pt.size());
        for (const auto& v : pt) scal(v);
        scal(ev);
    };
    u32(n_rhs);
    u32(pr.stacking_coeffs[0].size());
    scal(pr.batching_challenge);
    for (const auto& cs : pr.stacking_coeffs)
        for (const auto& v : cs) scal(v);
    sumcheck(pr.sumcheck);
    u32(pr.point.size());
    for (const auto& v : pr.point) scal(v);
    u32(pr.evaluations.size());
    for (const auto& v : pr.evaluations) scal(v);
    for (uint32_t i = 0; i < n_rhs; i++) claim(pr.rhs_points[i], pr.rhs_evals[i]);
    claim(pr.lhs_point, pr.lhs_eval);
    u32(pr.aggregated ? 1 : 0);
    if (pr.aggregated) {
        scal(pr.input_batching_challenge);
        sumcheck(pr.aggregation);
    }
    *out = p;
    return DPB_OK;
}

// inputs/proving.rs:26-114
template <class F, class T>
int linking_impl(dpb_ctx* ctx, int variant, const dpb_chunking_info& ci, int64_t out_min, int64_t out_max,
                 const uint64_t* shape, uint32_t rank, dpb_mle* const* mles, uint32_t n_mles, const void* claim_point,
                 uint32_t n_claim, const void* logup_point, uint32_t n_logup, T& tr, void* out_evals, uint32_t cap,
                 void* out_point, void* out_evaluations, void* out_chal, uint32_t chal_cap, uint32_t* n_chal,
                 uint32_t* out_degree, dpb_mle* weight, void* out_weight_eval) {
    typedef typename F::E E;
    const std::vector<uint64_t> shp(shape, shape + rank);
    const std::vector<dpb_mle*> tabs(mles, mles + n_mles);
    for (auto* m : tabs)
        if (!m || m->ctx != ctx) return fail(DPB_EINVAL, "null or foreign witness table");
    if (weight && weight->ctx != ctx) return fail(DPB_EINVAL, "foreign weight table");
    const bool with_sum = variant == DPB_VARIANT_NORMALISATION_WITH_SUM;
    const auto v = with_sum ? zkml::lookup::LookupVariant::Normalisation : (zkml::lookup::LookupVariant)variant;
    auto res = zkml::lookup::prove_linking_sumcheck<F>(ctx, v, ci, out_min, out_max, shp, tabs, elems<F>(claim_point, n_claim),
                                                       elems<F>(logup_point, n_logup), tr, with_sum, weight);
    if (res.has_weight_eval && out_weight_eval) memcpy(out_weight_eval, &res.weight_eval, sizeof(E));
    const size_t n = res.sumcheck_point.size();
    if (n * (res.degree + 1) > cap)
        return fail(DPB_EINVAL, "round-evaluation buffer holds %u elements, %llu needed", cap, (unsigned long long)(n * (res.degree + 1)));
    if (res.batching_challenges.size() > chal_cap)
        return fail(DPB_EINVAL, "room for %u batching challenges, %llu needed", chal_cap, (unsigned long long)res.batching_challenges.size());
    E* o = (E*)out_evals;
    for (const auto& m : res.sumcheck_proof.proofs)
        for (const auto& v : m.evaluations) *o++ = v;
    memcpy(out_point, res.sumcheck_point.data(), n * sizeof(E));
    memcpy(out_evaluations, res.evaluations.data(), res.evaluations.size() * sizeof(E));
    memcpy(out_chal, res.batching_challenges.data(), res.batching_challenges.size() * sizeof(E));
    *n_chal = (uint32_t)res.batching_challenges.size();
    if (out_degree) *out_degree = res.degree;
    return DPB_OK;
}

}  // namespace

extern "C" {

int dpb_transcript_new(int family_dtype, const void* label, size_t label_len, dpb_transcript** out) {
    if (!out || (!label && label_len)) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    return guarded([&] {
        dpb_transcript* t = new dpb_transcript();
        t->gl = is_gl(family_dtype);
        if (t->gl) t->g = new Blake3Transcript<GlFam>(label, label_len);
        else t->f = new Blake3Transcript<FrFam>(label, label_len);
        *out = t;
        return DPB_OK;
    });
}

int dpb_transcript_clone(const dpb_transcript* t, dpb_transcript** out) {
    if (!t || !out) return fail(DPB_EINVAL, "null argument");
    return guarded([&] {
        dpb_transcript* c = new dpb_transcript();
        c->gl = t->gl;
        if (t->gl) c->g = new Blake3Transcript<GlFam>(*t->g);
        else c->f = new Blake3Transcript<FrFam>(*t->f);
        *out = c;
        return DPB_OK;
    });
}

void dpb_transcript_free(dpb_transcript* t) { delete t; }

int dpb_transcript_append_scalars(dpb_transcript* t, const void* scalars, uint32_t n) {
    if (!t || (!scalars && n)) return fail(DPB_EINVAL, "null argument");
    return guarded([&] {
        if (t->gl) t->g->append_scalars((const Gl2*)scalars, n);
        else t->f->append_scalars(elems<FrFam>(scalars, n));
        return DPB_OK;
    });
}

int dpb_transcript_append_and_sample(dpb_transcript* t, const void* label, size_t label_len, void* out) {
    if (!t || !out || (!label && label_len)) return fail(DPB_EINVAL, "null argument");
    return guarded([&] {
        if (t->gl) { Gl2 c = t->g->append_and_sample(label, label_len); memcpy(out, &c, sizeof c); }
        else { Fr c = t->f->append_and_sample(label, label_len); memcpy(out, &c, sizeof c); }
        return DPB_OK;
    });
}

int dpb_transcript_challenge_scalar(dpb_transcript* t, void* out) {
    if (!t || !out) return fail(DPB_EINVAL, "null argument");
    return guarded([&] {
        if (t->gl) { Gl2 c = t->g->challenge_scalar(); memcpy(out, &c, sizeof c); }
        else { Fr c = t->f->challenge_scalar(); memcpy(out, &c, sizeof c); }
        return DPB_OK;
    });
}

int dpb_transcript_state(const dpb_transcript* t, uint8_t out_state[32], uint32_t* out_round) {
    if (!t || !out_state) return fail(DPB_EINVAL, "null argument");
    memcpy(out_state, t->gl ? t->g->state() : t->f->state(), 32);
    if (out_round) *out_round = t->gl ? t->g->round() : t->f->round();
    return DPB_OK;
}

int dpb_expr_to_terms(int family_dtype, const dpb_expr_node* nodes, uint32_t n_nodes, const void* challenges,
                      uint32_t n_challenges, dpb_term* out, uint32_t cap, uint32_t* n_out) {
    if (!nodes || !n_out || (!out && cap) || (!challenges && n_challenges)) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    return guarded([&] {
        return is_gl(family_dtype)
                   ? expr_to_terms_impl<GlFam>(nodes, n_nodes, challenges, n_challenges, out, cap, n_out)
                   : expr_to_terms_impl<FrFam>(nodes, n_nodes, challenges, n_challenges, out, cap, n_out);
    });
}

int dpb_expr_eval(int family_dtype, const dpb_expr_node* nodes, uint32_t n_nodes, const void* wit_evals,
                  uint32_t n_wit, const void* challenges, uint32_t n_challenges, void* out) {
    if (!nodes || !out || (!wit_evals && n_wit) || (!challenges && n_challenges))
        return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    return guarded([&] {
        if (is_gl(family_dtype)) {
            Gl2 v = build_expr<GlFam>(nodes, n_nodes).evaluate(elems<GlFam>(wit_evals, n_wit), elems<GlFam>(challenges, n_challenges));
            memcpy(out, &v, sizeof v);
        } else {
            Fr v = build_expr<FrFam>(nodes, n_nodes).evaluate(elems<FrFam>(wit_evals, n_wit), elems<FrFam>(challenges, n_challenges));
            memcpy(out, &v, sizeof v);
        }
        return DPB_OK;
    });
}

int dpb_lookup_padding_evaluation(int family_dtype, const void* padding_value, const uint64_t* shape, uint32_t rank,
                                  const void* point, uint32_t n_point, void* out) {
    if (!padding_value || !shape || !out || (!point && n_point)) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    return guarded([&] {
        if (is_gl(family_dtype)) {
            Gl2 pv;
            memcpy(&pv, padding_value, sizeof pv);
            const Gl2 v = zkml::compute_lookup_padding_evaluation<GlFam>(pv, shape, rank, (const Gl2*)point, n_point);
            memcpy(out, &v, sizeof v);
        } else {
            Fr pv;
            memcpy(&pv, padding_value, sizeof pv);
            const Fr v = zkml::compute_lookup_padding_evaluation<FrFam>(pv, shape, rank, (const Fr*)point, n_point);
            memcpy(out, &v, sizeof v);
        }
        return DPB_OK;
    });
}

int dpb_scalar_inverse(int family_dtype, const void* a, void* out) {
    if (!a || !out) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    if (is_gl(family_dtype)) {
        Gl2 x;
        memcpy(&x, a, sizeof x);
        const Gl2 y = GlFam::is_zero(x) ? x : GlFam::inv(x);
        memcpy(out, &y, sizeof y);
    } else {
        Fr x;
        memcpy(&x, a, sizeof x);
        const Fr y = FrFam::inv(x);
        memcpy(out, &y, sizeof y);
    }
    return DPB_OK;
}

int dpb_bias_evaluation(int family_dtype, const uint64_t* output_shape, uint32_t rank, const uint8_t* axis_in_bias,
                        const uint32_t* bias_axis_position, const void* point, uint32_t n_point, const void* bias_eval,
                        void* out_eval, void* out_bias_point, uint32_t bias_point_cap, uint32_t* n_bias_point) {
    if (!output_shape || !axis_in_bias || !bias_eval || !out_eval || (!point && n_point))
        return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    return guarded([&] {
        auto run = [&](auto fam) {
            typedef decltype(fam) F;
            typedef typename F::E E;
            E be;
            memcpy(&be, bias_eval, sizeof be);
            std::vector<E> bp;
            const E v = zkml::compute_bias_evaluation<F>(output_shape, rank, axis_in_bias, bias_axis_position,
                                                         (const E*)point, n_point, be, bias_axis_position ? &bp : nullptr);
            memcpy(out_eval, &v, sizeof v);
            if (n_bias_point) *n_bias_point = (uint32_t)bp.size();
            if (out_bias_point && bias_axis_position) {
                if (bp.size() > bias_point_cap) throw dp_crypto::Error(DPB_EINVAL, "bias point buffer too small");
                if (!bp.empty()) memcpy(out_bias_point, bp.data(), bp.size() * sizeof(E));
            }
            return DPB_OK;
        };
        return is_gl(family_dtype) ? run(GlFam()) : run(FrFam());
    });
}

int dpb_prove_sumcheck(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k, const dpb_term* terms,
                       uint32_t n_terms, dpb_transcript* t, void* out_round_evals, uint32_t round_evals_cap,
                       void* out_point, void* out_final_evals, uint32_t* out_degree) {
    if (!ctx || !mles || !terms || !t || !out_round_evals || !out_point || !out_final_evals)
        return fail(DPB_EINVAL, "null argument");
    if (k == 0 || !mles[0]) return fail(DPB_EINVAL, "no tables");
    if (is_gl(mles[0]->dtype) != t->gl) return fail(DPB_EINVAL, "transcript and tables are of different fields");
    return guarded([&] {
        return t->gl ? prove_sumcheck_impl<GlFam>(ctx, num_vars, mles, k, terms, n_terms, *t->g, out_round_evals,
                                                  round_evals_cap, out_point, out_final_evals, out_degree)
                     : prove_sumcheck_impl<FrFam>(ctx, num_vars, mles, k, terms, n_terms, *t->f, out_round_evals,
                                                  round_evals_cap, out_point, out_final_evals, out_degree);
    });
}

int dpb_prove_sumcheck_sharded(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k,
                               const dpb_term* terms, uint32_t n_terms, dpb_transcript* t, void* out_round_evals,
                               uint32_t round_evals_cap, void* out_point, void* out_final_evals, uint32_t* out_degree) {
    if (!ctx || !mles || !terms || !t || !out_round_evals || !out_point || !out_final_evals)
        return fail(DPB_EINVAL, "null argument");
    if (k == 0 || !mles[0]) return fail(DPB_EINVAL, "no tables");
    if (is_gl(mles[0]->dtype) != t->gl) return fail(DPB_EINVAL, "transcript and tables are of different fields");
    return guarded([&] {
        return t->gl ? prove_sumcheck_impl<GlFam>(ctx, num_vars, mles, k, terms, n_terms, *t->g, out_round_evals,
                                                  round_evals_cap, out_point, out_final_evals, out_degree, true)
                     : prove_sumcheck_impl<FrFam>(ctx, num_vars, mles, k, terms, n_terms, *t->f, out_round_evals,
                                                  round_evals_cap, out_point, out_final_evals, out_degree, true);
    });
}

int dpb_hadamard_prove(dpb_ctx* ctx, dpb_mle* v1, dpb_mle* v2, const void* claim_point, uint32_t n,
                       dpb_transcript* t, void* out_round_evals, void* out_point, void* out_claims) {
    if (!ctx || !v1 || !v2 || !claim_point || !t || !out_round_evals || !out_point || !out_claims)
        return fail(DPB_EINVAL, "null argument");
    if (is_gl(v1->dtype) != t->gl || is_gl(v2->dtype) != t->gl)
        return fail(DPB_EINVAL, "transcript and tables are of different fields");
    return guarded([&] {
        return t->gl ? hadamard_impl<GlFam>(ctx, v1, v2, claim_point, n, *t->g, out_round_evals, out_point, out_claims)
                     : hadamard_impl<FrFam>(ctx, v1, v2, claim_point, n, *t->f, out_round_evals, out_point, out_claims);
    });
}

int dpb_same_poly_prove(dpb_ctx* ctx, dpb_mle* poly, const void* points, uint32_t n_claims, uint32_t n,
                        dpb_transcript* t, void* out_round_evals, void* out_point, void* out_eval) {
    if (!ctx || !poly || !points || !t || !out_round_evals || !out_point || !out_eval)
        return fail(DPB_EINVAL, "null argument");
    if (is_gl(poly->dtype) != t->gl) return fail(DPB_EINVAL, "transcript and table are of different fields");
    return guarded([&] {
        return t->gl ? same_poly_impl<GlFam>(ctx, poly, points, n_claims, n, *t->g, out_round_evals, out_point, out_eval)
                     : same_poly_impl<FrFam>(ctx, poly, points, n_claims, n, *t->f, out_round_evals, out_point, out_eval);
    });
}

int dpb_claims_batching_prove(dpb_ctx* ctx, const dpb_committed_poly* polys, uint32_t n_polys, dpb_transcript* t,
                              void* out_round_evals, uint32_t round_evals_cap, void* out_point,
                              uint32_t* out_num_vars, void* out_sumcheck_evals, uint32_t evals_cap,
                              void* out_rlc_challenges, dpb_mle** out_rlc) {
    if (!ctx || !polys || !t || !out_round_evals || !out_point || !out_sumcheck_evals) return fail(DPB_EINVAL, "null argument");
    if (n_polys == 0) return fail(DPB_EINVAL, "no committed polynomials");
    if (!polys[0].chunks || !polys[0].chunks[0]) return fail(DPB_EINVAL, "polynomial 0 has no chunks");
    if (is_gl(polys[0].chunks[0]->dtype) != t->gl) return fail(DPB_EINVAL, "transcript and tables are of different fields");
    return guarded([&] {
        return t->gl ? claims_impl<GlFam>(ctx, polys, n_polys, *t->g, out_round_evals, round_evals_cap, out_point,
                                          out_num_vars, out_sumcheck_evals, evals_cap, out_rlc_challenges, out_rlc)
                     : claims_impl<FrFam>(ctx, polys, n_polys, *t->f, out_round_evals, round_evals_cap, out_point,
                                          out_num_vars, out_sumcheck_evals, evals_cap, out_rlc_challenges, out_rlc);
    });
}

int dpb_logup_batch_prove(dpb_ctx* ctx, const dpb_logup_input* inputs, uint32_t n_inputs, dpb_transcript* t,
                          dpb_logup_proof** out) {
    if (!ctx || !t || !out || (!inputs && n_inputs)) return fail(DPB_EINVAL, "null argument");
    if (n_inputs == 0) return fail(DPB_EINVAL, "No inputs provided for LogUp");
    return guarded([&] {
        return t->gl ? logup_impl<GlFam>(ctx, inputs, n_inputs, *t->g, out)
                     : logup_impl<FrFam>(ctx, inputs, n_inputs, *t->f, out);
    });
}

int dpb_logup_batch_prove_partial(dpb_ctx* ctx, const dpb_logup_input* inputs, uint32_t n_inputs, dpb_transcript* t,
                                  dpb_logup_proof** out) {
    if (!ctx || !t || !out || (!inputs && n_inputs)) return fail(DPB_EINVAL, "null argument");
    if (n_inputs == 0) return fail(DPB_EINVAL, "No inputs provided for LogUp");
    return guarded([&] {
        return t->gl ? logup_impl<GlFam>(ctx, inputs, n_inputs, *t->g, out, true)
                     : logup_impl<FrFam>(ctx, inputs, n_inputs, *t->f, out, true);
    });
}

int dpb_logup_proof_serialize(const dpb_logup_proof* p, void* buf, size_t cap, size_t* len) {
    if (!p || !len || (!buf && cap)) return fail(DPB_EINVAL, "null argument");
    *len = p->bytes.size();
    if (cap >= p->bytes.size()) memcpy(buf, p->bytes.data(), p->bytes.size());
    return DPB_OK;
}

int dpb_einsum_prove(dpb_ctx* ctx, const dpb_einsum_operand* lhs_fixes, const dpb_einsum_operand* rhs, uint32_t n_rhs,
                     dpb_mle* lhs_padded, dpb_transcript* t, dpb_einsum_proof** out) {
    if (!ctx || !t || !out || !lhs_fixes || !rhs) return fail(DPB_EINVAL, "null argument");
    if (n_rhs == 0) return fail(DPB_EINVAL, "an einsum has at least one right tensor");
    return guarded([&] {
        return t->gl ? einsum_impl<GlFam>(ctx, lhs_fixes, rhs, n_rhs, lhs_padded, *t->g, out)
                     : einsum_impl<FrFam>(ctx, lhs_fixes, rhs, n_rhs, lhs_padded, *t->f, out);
    });
}

int dpb_einsum_proof_serialize(const dpb_einsum_proof* p, void* buf, size_t cap, size_t* len) {
    if (!p || !len || (!buf && cap)) return fail(DPB_EINVAL, "null argument");
    *len = p->bytes.size();
    if (cap >= p->bytes.size()) memcpy(buf, p->bytes.data(), p->bytes.size());
    return DPB_OK;
}

void dpb_einsum_proof_free(dpb_einsum_proof* p) { delete p; }

void dpb_logup_proof_free(dpb_logup_proof* p) { delete p; }

}  // extern "C"

extern "C" int dpb_lookup_linking_prove(dpb_ctx* ctx, int variant, const dpb_chunking_info* info, int64_t table_min_output,
                                        int64_t table_max_output, const uint64_t* shape, uint32_t rank, dpb_mle* const* mles,
                                        uint32_t n_mles, const void* last_claim_point, uint32_t n_claim_coords,
                                        const void* logup_point, uint32_t n_logup_coords, dpb_transcript* t,
                                        void* out_round_evals, uint32_t round_evals_cap, void* out_point,
                                        void* out_evaluations, void* out_batching_challenges, uint32_t chal_cap,
                                        uint32_t* out_n_challenges, uint32_t* out_degree, dpb_mle* weight,
                                        void* out_weight_eval) {
    if (!ctx || !info || !shape || !mles || !last_claim_point || !logup_point || !t || !out_round_evals || !out_point ||
        !out_evaluations || !out_batching_challenges || !out_n_challenges)
        return fail(DPB_EINVAL, "null argument");
    if (variant < DPB_VARIANT_STANDARD || variant > DPB_VARIANT_NORMALISATION_WITH_SUM)
        return fail(DPB_EINVAL, "unknown variant %d", variant);
    if (weight && !out_weight_eval) return fail(DPB_EINVAL, "a weight table needs room for its evaluation");
    if (rank < 1 || rank > 8) return fail(DPB_EINVAL, "rank %u outside 1..8", rank);
    for (uint32_t a = 0; a < rank; a++)
        if (shape[a] == 0) return fail(DPB_EINVAL, "axis %u is empty", a);
    if (info->n_value_chunks < 1 || info->n_value_chunks > 4 || info->n_zeroing_chunks > 4 || info->value_chunk_bits < 1 ||
        info->value_chunk_bits * info->n_value_chunks > 62 || info->table_sign < DPB_SIGN_POSITIVE || info->table_sign > DPB_SIGN_MIXED)
        return fail(DPB_EINVAL, "chunking info out of range");
    return guarded([&]() {
        return t->gl ? linking_impl<GlFam>(ctx, variant, *info, table_min_output, table_max_output, shape, rank, mles, n_mles,
                                           last_claim_point, n_claim_coords, logup_point, n_logup_coords, *t->g, out_round_evals,
                                           round_evals_cap, out_point, out_evaluations, out_batching_challenges, chal_cap,
                                           out_n_challenges, out_degree, weight, out_weight_eval)
                     : linking_impl<FrFam>(ctx, variant, *info, table_min_output, table_max_output, shape, rank, mles, n_mles,
                                           last_claim_point, n_claim_coords, logup_point, n_logup_coords, *t->f, out_round_evals,
                                           round_evals_cap, out_point, out_evaluations, out_batching_challenges, chal_cap,
                                           out_n_challenges, out_degree, weight, out_weight_eval);
    });
}
