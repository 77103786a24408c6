// Host side of the sumcheck prover, above the C ABI, with the names and
// argument meaning of the reference's dp-crypto API as zkml calls it:
//   Expression            zkml/src/lookup/logup_gkr/circuit.rs:245-284
//   VirtualPolynomialsBuilder::{new, new_with_mles, lift, to_virtual_polys}
//                         zkml/src/layers/hadamard.rs:108-114,
//                         zkml/src/layers/einsum/prove.rs:171-182
//   IOPProverState::prove, collect_raw_challenges,
//   get_mle_flatten_final_evaluations, IOPProof::extract_sum
//                         zkml/src/layers/hadamard.rs:115-130
//   eval_by_expr_with_instance
//                         zkml/src/lookup/logup_gkr/prover.rs:50-57
// The reference is Rust; no Rust toolchain is available to this build, so the
// host side is C++ and reaches the GPU only through the dpb_* C functions.
#pragma once
#include <algorithm>
#include <map>
#include <memory>
#include <stdexcept>
#include <vector>

#include "../../../include/dpb.h"
#include "../family.cuh"
#include "transcript.hpp"

namespace dp_crypto {

using dpb::FrFam;
using dpb::GlFam;

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};
inline void check(int rc) {
    if (rc != DPB_OK) throw Error(rc, dpb_last_error());
}

template <class F>
inline typename F::E pow_elem(typename F::E a, size_t e) {
    typename F::E r = F::one();
    while (e) {
        if (e & 1) r = F::mul(r, a);
        a = F::mul(a, a);
        e >>= 1;
    }
    return r;
}

template <class F>
inline bool elem_eq(const typename F::E& a, const typename F::E& b) {
    return memcmp(&a, &b, sizeof(typename F::E)) == 0;
}

// ---- Expression ---------------------------------------------------------------
template <class F>
class Expression {
   public:
    typedef typename F::E E;
    enum Kind { kWitIn, kConstant, kChallenge, kAdd, kMul, kNeg };
    struct Node {
        Kind kind;
        uint16_t id = 0;
        size_t pow = 0;
        E a, b;  // Constant: a; Challenge: a = scalar, b = offset
        std::shared_ptr<const Node> l, r;
    };
    // A monomial: its table ids in ascending order.  Ordered like a vector of ids (element by element, a prefix
    // before its extensions), which is the order the terms reach the sumcheck in.
    struct Mono {
        uint16_t n = 0;
        uint16_t id[DPB_MAX_FACTORS] = {0};
        bool operator<(const Mono& o) const {
            const uint16_t m = std::min(n, o.n);
            for (uint16_t i = 0; i < m; i++)
                if (id[i] != o.id[i]) return id[i] < o.id[i];
            return n < o.n;
        }
        bool operator==(const Mono& o) const { return n == o.n && std::equal(id, id + n, o.id); }
        size_t size() const { return n; }
        uint16_t operator[](size_t i) const { return id[i]; }
    };
    // Monomial form: (monomial, coefficient) sorted by monomial, no monomial twice, no zero coefficient.
    typedef std::vector<std::pair<Mono, E>> Terms;

    Expression() : n_(leaf(kConstant, 0, 0, F::zero(), F::zero())) {}
    static Expression ZERO() { return Constant(F::zero()); }
    static Expression ONE() { return Constant(F::one()); }
    static Expression WitIn(uint16_t id) { return Expression(leaf(kWitIn, id, 0, F::zero(), F::zero())); }
    static Expression Constant(const E& c) { return Expression(leaf(kConstant, 0, 0, c, F::zero())); }
    // scalar * challenge[id]^pow + offset
    static Expression Challenge(uint16_t id, size_t pow, const E& scalar, const E& offset) {
        return Expression(leaf(kChallenge, id, pow, scalar, offset));
    }
    Expression operator+(const Expression& o) const { return Expression(inner(kAdd, n_, o.n_)); }
    Expression operator*(const Expression& o) const { return Expression(inner(kMul, n_, o.n_)); }
    Expression operator-() const { return Expression(inner(kNeg, n_, nullptr)); }
    Expression operator-(const Expression& o) const { return *this + (-o); }

    // Monomial form under the given challenge values: {sorted table ids -> coefficient}.
    Terms to_terms(const std::vector<E>& challenges) const { return expand(*n_, challenges); }
    static void normalise_terms(Terms& t) { normalise(t); }

    // eval_by_expr_with_instance with witness values and challenges only.
    E evaluate(const std::vector<E>& wit_evals, const std::vector<E>& challenges) const {
        return eval(*n_, wit_evals, challenges);
    }

   private:
    explicit Expression(std::shared_ptr<const Node> n) : n_(std::move(n)) {}
    static std::shared_ptr<const Node> leaf(Kind k, uint16_t id, size_t pow, const E& a, const E& b) {
        auto n = std::make_shared<Node>();
        n->kind = k;
        n->id = id;
        n->pow = pow;
        n->a = a;
        n->b = b;
        return n;
    }
    static std::shared_ptr<const Node> inner(Kind k, std::shared_ptr<const Node> l, std::shared_ptr<const Node> r) {
        auto n = std::make_shared<Node>();
        n->kind = k;
        n->a = n->b = F::zero();
        n->l = std::move(l);
        n->r = std::move(r);
        return n;
    }
    static E challenge_value(const Node& n, const std::vector<E>& ch) {
        if (n.id >= ch.size()) throw Error(DPB_EINVAL, "expression refers to a challenge that was not supplied");
        return F::add(F::mul(n.a, pow_elem<F>(ch[n.id], n.pow)), n.b);
    }
    // sorts by monomial, adds up equal monomials, drops zeros
    static void normalise(Terms& t) {
        std::stable_sort(t.begin(), t.end(), [](const std::pair<Mono, E>& x, const std::pair<Mono, E>& y) { return x.first < y.first; });
        size_t w = 0;
        for (size_t r = 0; r < t.size();) {
            Mono m = t[r].first;
            E c = t[r].second;
            for (r++; r < t.size() && t[r].first == m; r++) c = F::add(c, t[r].second);
            if (!F::is_zero(c)) {
                t[w].first = m;
                t[w].second = c;
                w++;
            }
        }
        t.resize(w);
    }
    // two normalised lists -> their sum, normalised
    static Terms merge(const Terms& a, const Terms& b) {
        Terms out;
        out.reserve(a.size() + b.size());
        size_t i = 0, j = 0;
        while (i < a.size() || j < b.size()) {
            if (j == b.size() || (i < a.size() && a[i].first < b[j].first)) {
                out.push_back(a[i++]);
            } else if (i == a.size() || b[j].first < a[i].first) {
                out.push_back(b[j++]);
            } else {
                const E c = F::add(a[i].second, b[j].second);
                if (!F::is_zero(c)) out.emplace_back(a[i].first, c);
                i++;
                j++;
            }
        }
        return out;
    }
    static Terms expand(const Node& n, const std::vector<E>& ch) {
        Terms out;
        switch (n.kind) {
            case kWitIn: {
                Mono m;
                m.n = 1;
                m.id[0] = n.id;
                out.emplace_back(m, F::one());
                return out;
            }
            case kConstant: if (!F::is_zero(n.a)) out.emplace_back(Mono(), n.a); return out;
            case kChallenge: {
                const E v = challenge_value(n, ch);
                if (!F::is_zero(v)) out.emplace_back(Mono(), v);
                return out;
            }
            case kNeg: {
                out = expand(*n.l, ch);
                for (auto& kv : out) kv.second = F::neg(kv.second);
                return out;
            }
            case kAdd: return merge(expand(*n.l, ch), expand(*n.r, ch));
            case kMul: {
                const Terms a = expand(*n.l, ch), b = expand(*n.r, ch);
                out.reserve(a.size() * b.size());
                for (const auto& x : a)
                    for (const auto& y : b) {
                        if (x.first.n + y.first.n > DPB_MAX_FACTORS) throw Error(DPB_EINVAL, "product term has too many factors");
                        Mono m;
                        m.n = (uint16_t)(x.first.n + y.first.n);
                        std::merge(x.first.id, x.first.id + x.first.n, y.first.id, y.first.id + y.first.n, m.id);
                        out.emplace_back(m, F::mul(x.second, y.second));
                    }
                normalise(out);
                return out;
            }
        }
        return out;
    }
    static E eval(const Node& n, const std::vector<E>& w, const std::vector<E>& ch) {
        switch (n.kind) {
            case kWitIn:
                if (n.id >= w.size()) throw Error(DPB_EINVAL, "expression refers to a witness value that was not supplied");
                return w[n.id];
            case kConstant: return n.a;
            case kChallenge: return challenge_value(n, ch);
            case kNeg: return F::neg(eval(*n.l, w, ch));
            case kAdd: return F::add(eval(*n.l, w, ch), eval(*n.r, w, ch));
            case kMul: return F::mul(eval(*n.l, w, ch), eval(*n.r, w, ch));
        }
        return F::zero();
    }
    std::shared_ptr<const Node> n_;
};

// ---- VirtualPolynomials -------------------------------------------------------
template <class F>
struct VirtualPolynomials {
    uint32_t num_vars = 0;
    std::vector<dpb_mle*> mles;  // borrowed, registration order = WitIn id
    std::vector<dpb_term> terms;
    uint32_t max_degree = 0;
};

template <class F>
class VirtualPolynomialsBuilder {
   public:
    typedef typename F::E E;
    // num_threads is accepted for signature parity; the GPU needs no thread split.
    VirtualPolynomialsBuilder(size_t /*num_threads*/, uint32_t num_vars) : num_vars_(num_vars) {}
    static VirtualPolynomialsBuilder new_with_mles(size_t num_threads, uint32_t num_vars,
                                                   const std::vector<dpb_mle*>& mles) {
        VirtualPolynomialsBuilder b(num_threads, num_vars);
        b.mles_ = mles;
        return b;
    }
    // Registers a table (once) and returns the expression that stands for it.
    Expression<F> lift(dpb_mle* mle) {
        for (size_t i = 0; i < mles_.size(); i++)
            if (mles_[i] == mle) return Expression<F>::WitIn((uint16_t)i);
        mles_.push_back(mle);
        return Expression<F>::WitIn((uint16_t)(mles_.size() - 1));
    }
    VirtualPolynomials<F> to_virtual_polys(const std::vector<Expression<F>>& exprs,
                                           const std::vector<E>& challenges) const {
        typename Expression<F>::Terms all;
        for (const auto& e : exprs) {
            const auto t = e.to_terms(challenges);
            all.insert(all.end(), t.begin(), t.end());
        }
        Expression<F>::normalise_terms(all);
        VirtualPolynomials<F> vp;
        vp.num_vars = num_vars_;
        vp.mles = mles_;
        for (const auto& kv : all) {
            if (F::is_zero(kv.second)) continue;
            if (kv.first.size() > DPB_MAX_FACTORS) throw Error(DPB_EINVAL, "product term has too many factors");
            dpb_term t;
            memset(&t, 0, sizeof t);
            memcpy(t.coeff, &kv.second, sizeof(E));
            t.n_factors = (uint32_t)kv.first.size();
            for (size_t j = 0; j < kv.first.size(); j++) t.idx[j] = kv.first[j];
            vp.terms.push_back(t);
            vp.max_degree = std::max(vp.max_degree, t.n_factors);
        }
        return vp;
    }

   private:
    uint32_t num_vars_;
    std::vector<dpb_mle*> mles_;
};

// ---- IOPProof / IOPProverState --------------------------------------------------
template <class F>
struct IOPProverMessage {
    std::vector<typename F::E> evaluations;  // at 0..=max_degree
};

template <class F>
struct IOPProof {
    std::vector<IOPProverMessage<F>> proofs;
    typename F::E extract_sum() const {
        return F::add(proofs.at(0).evaluations.at(0), proofs.at(0).evaluations.at(1));
    }
};

constexpr const char* kRoundLabel = "sumcheck_round";

template <class F>
class IOPProverState {
   public:
    typedef typename F::E E;
    // Runs every round on the GPU behind `ctx`; the transcript is only touched here, on the host.
    template <class T>
    static std::pair<IOPProof<F>, IOPProverState> prove(dpb_ctx* ctx, const VirtualPolynomials<F>& vp,
                                                        T& transcript, int sharded = 0,
                                                        const std::vector<dpb::LogupHintInst>* logup_hint = nullptr,
                                                        const E* logup_lambda = nullptr, uint32_t logup_eq = 0) {
        if (vp.terms.empty()) throw Error(DPB_EINVAL, "virtual polynomial has no terms");
        IOPProverState st;
        IOPProof<F> proof;
        dpb_sc* sc = nullptr;
        dpb::TracePhase t_begin("sumcheck.begin");
        // sharded = 1: the tables are this rank's slices; 2: this rank's part of the terms over whole tables; every
        // rank runs this same loop
        check((sharded == 2 ? dpb_sumcheck_begin_partial : sharded ? dpb_sumcheck_begin_sharded : dpb_sumcheck_begin)(
            ctx, vp.num_vars, vp.mles.data(), (uint32_t)vp.mles.size(), vp.terms.data(), (uint32_t)vp.terms.size(), &sc));
        // the logup prover says what its layer looks like: the large rounds then run from the layer's formula
        if (logup_hint && logup_lambda && !logup_hint->empty())
            dpb::sumcheck_hint_logup(sc, logup_hint->data(), (uint32_t)logup_hint->size(), logup_lambda, logup_eq);
        t_begin.stop();
        dpb::TracePhase t_rounds("sumcheck.rounds");
        struct Guard {
            dpb_sc* s;
            ~Guard() { dpb_sumcheck_free(s); }
        } guard{sc};
        const uint32_t d = dpb_sumcheck_degree(sc);
        const E header[2] = {F::from_u64(vp.num_vars), F::from_u64(d)};
        transcript.append_scalars(header, 2);
        E r = F::zero();
        for (uint32_t i = 0; i < vp.num_vars; i++) {
            IOPProverMessage<F> msg;
            msg.evaluations.resize(d + 1);
            uint32_t n = 0;
            check(dpb_sumcheck_round(sc, i == 0 ? nullptr : &r, msg.evaluations.data(), &n));
            transcript.append_scalars(msg.evaluations);
            r = transcript.append_and_sample(kRoundLabel);
            st.challenges_.push_back(r);
            proof.proofs.push_back(std::move(msg));
        }
        t_rounds.stop();
        dpb::TracePhase t_finish("sumcheck.finish");
        st.final_evals_.resize(vp.mles.size());
        check(dpb_sumcheck_finish(sc, &r, st.final_evals_.data()));
        return {std::move(proof), std::move(st)};
    }
    // challenge j is the value of variable j
    const std::vector<E>& collect_raw_challenges() const { return challenges_; }
    // every registered table at the point, in registration order
    const std::vector<E>& get_mle_flatten_final_evaluations() const { return final_evals_; }

   private:
    std::vector<E> challenges_;
    std::vector<E> final_evals_;
};

}  // namespace dp_crypto
