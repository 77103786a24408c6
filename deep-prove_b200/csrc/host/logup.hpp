// Batched logup-GKR prover on the GPU, following the reference's in-repo code
// step for step:
//   LogUpInput, make_new_circuits     zkml/src/lookup/logup_gkr/structs.rs:138-272
//   LogUpCircuit                      zkml/src/lookup/logup_gkr/circuit.rs:503-600
//   layer_proving_info                zkml/src/lookup/logup_gkr/circuit.rs:231-412
//   new_batch_multiple_sizes_prove    zkml/src/lookup/logup_gkr/prover.rs:91-344
//   LogUpBatchProof                   zkml/src/lookup/logup_gkr/structs.rs:555-578
// Fraction trees are built and kept on the device (dpb_logup_build); each GKR
// step is one GPU sumcheck over borrowed views of a tree level.
#pragma once
#include <set>

#include "prover.hpp"

namespace zkml {
namespace logup_gkr {

using dp_crypto::check;
using dp_crypto::Error;
using dp_crypto::Expression;

enum class ProofType : uint32_t { Lookup = 0, Table = 1 };

template <class F>
struct Claim {
    std::vector<typename F::E> point;
    typename F::E eval;
};

template <class F>
struct LogUpInput {
    typedef typename F::E E;
    ProofType kind;
    std::vector<dpb_mle*> column_evals;  // borrowed device tables, equal power-of-two lengths
    dpb_mle* multiplicities = nullptr;   // tables only
    E constant_challenge;
    E column_separation_challenge;
    size_t columns_per_instance = 1;  // lookups only

    static void validate(const std::vector<dpb_mle*>& cols) {
        if (cols.empty()) throw Error(DPB_EINVAL, "No column evals were provided for Lookup input");
        const uint64_t n = dpb_mle_len(cols[0]);
        if (n == 0 || (n & (n - 1)))
            throw Error(DPB_EINVAL, "Need a power of two number of evaluations got: " + std::to_string(n));
        for (auto* c : cols)
            if (dpb_mle_len(c) != n) throw Error(DPB_EINVAL, "All sets of evaluations should be the same length");
    }
    static LogUpInput new_lookup(std::vector<dpb_mle*> cols, const E& constant, const E& sep, size_t per_instance) {
        validate(cols);
        if (per_instance == 0 || cols.size() % per_instance != 0)
            throw Error(DPB_EINVAL, "column count is not a multiple of columns_per_instance");
        LogUpInput in;
        in.kind = ProofType::Lookup;
        in.column_evals = std::move(cols);
        in.constant_challenge = constant;
        in.column_separation_challenge = sep;
        in.columns_per_instance = per_instance;
        return in;
    }
    static LogUpInput new_table(std::vector<dpb_mle*> cols, dpb_mle* mult, const E& constant, const E& sep) {
        validate(cols);
        if (!mult || dpb_mle_len(mult) != dpb_mle_len(cols[0]))
            throw Error(DPB_EINVAL, "Multiplicities length was not equal to column evaluations length");
        LogUpInput in;
        in.kind = ProofType::Table;
        in.column_evals = std::move(cols);
        in.multiplicities = mult;
        in.constant_challenge = constant;
        in.column_separation_challenge = sep;
        in.columns_per_instance = in.column_evals.size();
        return in;
    }
};

// One instance's fraction tree on the device plus what the prover needs to
// describe each of its layers to the sumcheck.
template <class F>
class LogUpCircuit {
   public:
    typedef typename F::E E;
    LogUpCircuit(dpb_ctx* ctx, ProofType kind, std::vector<dpb_mle*> cols, dpb_mle* mult, const E& constant,
                 const E& sep)
        : kind_(kind), cols_(std::move(cols)), mult_(mult), constant_(constant), sep_(sep) {
        m_ = 0;
        while ((1ull << m_) < dpb_mle_len(cols_[0])) m_++;
        check(dpb_logup_build(ctx, kind == ProofType::Table ? DPB_LOGUP_TABLE : DPB_LOGUP_LOOKUP, cols_.data(),
                              (uint32_t)cols_.size(), mult_, &constant_, &sep_, &tree_));
    }
    LogUpCircuit(const LogUpCircuit&) = delete;
    LogUpCircuit& operator=(const LogUpCircuit&) = delete;
    ~LogUpCircuit() {
        for (auto* v : views_) dpb_mle_free(v);
        dpb_logup_free(tree_);
    }
    size_t num_vars() const { return m_ - 1; }
    size_t denominator_column_count() const { return cols_.size(); }
    size_t final_eval_count() const { return 2 * cols_.size() + (kind_ == ProofType::Table ? 2 : 0); }
    std::vector<E> outputs() const {
        std::vector<E> o(4);
        check(dpb_logup_outputs(tree_, o.data()));
        return o;
    }
    const dpb_logup* tree() const { return tree_; }

    // Tables of the layer whose halves have `layer_vars` variables, in the
    // order layer_proving_info registers them.  Views stay alive with *this.
    std::vector<dpb_mle*> layer_mles(size_t layer_vars) {
        std::vector<dpb_mle*> out;
        const uint64_t half = 1ull << layer_vars;
        auto halves = [&](dpb_mle* t, std::vector<dpb_mle*>& lo, std::vector<dpb_mle*>& hi) {
            dpb_mle *a = nullptr, *b = nullptr;
            check(dpb_mle_view(t, 0, half, &a));
            views_.push_back(a);
            check(dpb_mle_view(t, half, half, &b));
            views_.push_back(b);
            lo.push_back(a);
            hi.push_back(b);
        };
        if (layer_vars == num_vars()) {
            std::vector<dpb_mle*> lo, hi;
            if (kind_ == ProofType::Table) {
                std::vector<dpb_mle*> nlo, nhi;
                halves(mult_, nlo, nhi);
                out.push_back(nlo[0]);
                out.push_back(nhi[0]);
            }
            for (auto* c : cols_) halves(c, lo, hi);
            out.insert(out.end(), lo.begin(), lo.end());
            out.insert(out.end(), hi.begin(), hi.end());
            return out;
        }
        dpb_mle* v[4];
        check(dpb_logup_level(tree_, (uint32_t)(m_ - 1 - layer_vars), v));
        for (auto* x : v) {
            views_.push_back(x);
            out.push_back(x);
        }
        return out;
    }

    struct LayerExprs {
        Expression<F> sumcheck, claim;
        uint16_t num_witnesses;
    };
    // circuit.rs:231-412.  Challenge ids: 0 = alpha, 1 = lambda, 2 = batching.
    LayerExprs layer_exprs(size_t layer_vars, size_t layer_count, uint16_t wit0) const {
        typedef Expression<F> X;
        const E one = F::one(), zero = F::zero();
        const uint16_t b = (uint16_t)(layer_count * 4);
        const X rho = X::Challenge(2, 1, one, zero), lam = X::Challenge(1, 1, one, zero);
        const X alpha_j = X::Challenge(0, layer_count, one, zero);
        X claim = alpha_j * (rho * (X::WitIn(b + 1) - X::WitIn(b)) + X::WitIn(b) +
                             lam * (rho * (X::WitIn(b + 3) - X::WitIn(b + 2)) + X::WitIn(b + 2)));
        if (layer_vars != num_vars()) {
            const X n_lo = X::WitIn(wit0), n_hi = X::WitIn(wit0 + 1), d_lo = X::WitIn(wit0 + 2),
                    d_hi = X::WitIn(wit0 + 3);
            return {alpha_j * (n_lo * d_hi + n_hi * d_lo + lam * d_lo * d_hi), claim, 4};
        }
        const uint16_t ncol = (uint16_t)cols_.size();
        const uint16_t first = wit0 + (kind_ == ProofType::Table ? 2 : 0);
        X d_lo = X::Constant(constant_), d_hi = X::Constant(constant_);
        E pw = one;
        for (uint16_t i = 0; i < ncol; i++) {
            d_lo = d_lo + X::Constant(pw) * X::WitIn(first + i);
            d_hi = d_hi + X::Constant(pw) * X::WitIn(first + ncol + i);
            pw = F::mul(pw, sep_);
        }
        if (kind_ == ProofType::Table)
            return {alpha_j * (X::WitIn(wit0) * d_hi + X::WitIn(wit0 + 1) * d_lo + lam * d_lo * d_hi), claim,
                    (uint16_t)(2 + 2 * ncol)};
        return {alpha_j * (-d_hi - d_lo + lam * d_lo * d_hi), claim, (uint16_t)(2 * ncol)};
    }

    // the input layer as sc_round_logup takes it (kinds 1 and 2 of dpb::LogupHintInst)
    dpb::LogupHintInst input_layer_hint(uint16_t wit0, const E& alpha_j) const {
        dpb::LogupHintInst h;
        memset(&h, 0, sizeof h);
        h.kind = kind_ == ProofType::Table ? 2 : 1;
        h.first = wit0;
        h.ncol = (uint32_t)cols_.size();
        memcpy(h.alpha, &alpha_j, sizeof(E));
        memcpy(h.constant, &constant_, sizeof(E));
        memcpy(h.sep, &sep_, sizeof(E));
        return h;
    }

    // circuit.rs:442-500
    std::vector<E> combine_final_evals(const E* evals, size_t n, const E& rho) const {
        if (n != final_eval_count()) throw Error(DPB_EINVAL, "wrong number of final evaluations");
        std::vector<E> out;
        const size_t ncol = cols_.size();
        auto comb = [&](const E& lo, const E& hi) { return F::add(F::mul(rho, F::sub(hi, lo)), lo); };
        if (kind_ == ProofType::Table) {
            out.push_back(comb(evals[0], evals[1]));
            evals += 2;
        }
        for (size_t i = 0; i < ncol; i++) out.push_back(comb(evals[i], evals[ncol + i]));
        return out;
    }

   private:
    ProofType kind_;
    std::vector<dpb_mle*> cols_;
    dpb_mle* mult_;
    E constant_, sep_;
    size_t m_;
    dpb_logup* tree_ = nullptr;
    std::vector<dpb_mle*> views_;
};

template <class F>
struct LogUpBatchProof {
    typedef typename F::E E;
    std::vector<dp_crypto::IOPProof<F>> sumcheck_proofs;
    std::vector<std::vector<E>> round_evaluations;
    std::vector<Claim<F>> output_claims;
    std::vector<std::vector<E>> circuit_outputs;
    ProofType proof_type;
    std::vector<size_t> num_vars_per_instance;
    std::vector<size_t> num_denominator_columns_per_instance;

    // structs.rs:587-597
    void fractional_outputs(std::vector<E>& num, std::vector<E>& den) const {
        for (const auto& e : circuit_outputs) {
            num.push_back(F::add(F::mul(e[0], e[3]), F::mul(e[1], e[2])));
            den.push_back(F::mul(e[2], e[3]));
        }
    }

    // Flat canonical encoding (u32 counts, canonical scalars) in the field order above.
    std::vector<uint8_t> serialize() const {
        std::vector<uint8_t> out;
        auto u32 = [&](uint64_t v) {
            const uint32_t x = (uint32_t)v;
            out.insert(out.end(), (const uint8_t*)&x, (const uint8_t*)&x + 4);
        };
        auto scal = [&](const E& v) {
            uint8_t b[32];
            dpb::to_canonical(v, b);
            out.insert(out.end(), b, b + dpb::canonical_size(v));
        };
        u32(sumcheck_proofs.size());
        for (const auto& p : sumcheck_proofs) {
            u32(p.proofs.size());
            for (const auto& m : p.proofs) {
                u32(m.evaluations.size());
                for (const auto& v : m.evaluations) scal(v);
            }
        }
        u32(round_evaluations.size());
        for (const auto& ev : round_evaluations) {
            u32(ev.size());
            for (const auto& v : ev) scal(v);
        }
        u32(output_claims.size());
        for (const auto& c : output_claims) {
            u32(c.point.size());
            for (const auto& v : c.point) scal(v);
            scal(c.eval);
        }
        u32(circuit_outputs.size());
        for (const auto& o : circuit_outputs) {
            u32(o.size());
            for (const auto& v : o) scal(v);
        }
        u32((uint32_t)proof_type);
        u32(num_vars_per_instance.size());
        for (auto v : num_vars_per_instance) u32(v);
        u32(num_denominator_columns_per_instance.size());
        for (auto v : num_denominator_columns_per_instance) u32(v);
        return out;
    }
};

// prover.rs:91-344.
// partial: the instances of the batch are spread over the ranks of ctx's communicator.  Every rank passes its own
// instances, of the same kinds, sizes and column counts on every rank; local instance i of rank g is instance
// i * G + g of the whole batch (so the batch stays ordered by size).  Each rank builds only its own trees and runs
// its own part of every layer's sumcheck (dpb_sumcheck_begin_partial adds the round sums over the ranks); the
// outputs and the final evaluations of each layer are gathered, every rank feeds the same transcript, and every
// rank returns the proof of the WHOLE batch.
template <class F, class T>
LogUpBatchProof<F> new_batch_multiple_sizes_prove(dpb_ctx* ctx, const std::vector<LogUpInput<F>>& input,
                                                  T& transcript, bool partial = false) {
    typedef typename F::E E;
    typedef Expression<F> X;
    const size_t G = partial ? (size_t)std::max(dpb_comm_size(ctx), 1) : 1;
    const size_t g_rank = G > 1 ? (size_t)dpb_comm_rank(ctx) : 0;
    partial = G > 1;
    // rank-order gather of equal-sized host vectors; out[q] = rank q's
    auto gather = [&](const std::vector<E>& mine) {
        std::vector<E> all(mine.size() * G);
        check(dpb::comm_allgather_host(ctx, mine.data(), mine.size() * sizeof(E), all.data()));
        return all;
    };
    if (input.empty()) throw Error(DPB_EINVAL, "No inputs provided for LogUp");
    const ProofType proof_type = input[0].kind;
    for (const auto& in : input)
        if (in.kind != proof_type) throw Error(DPB_EINVAL, "Not all proof types matched");

    // structs.rs:241-272
    dpb::TracePhase t_trees("logup.trees");
    std::vector<std::unique_ptr<LogUpCircuit<F>>> circuits;
    for (const auto& in : input) {
        if (in.kind == ProofType::Table) {
            circuits.emplace_back(new LogUpCircuit<F>(ctx, in.kind, in.column_evals, in.multiplicities,
                                                      in.constant_challenge, in.column_separation_challenge));
        } else {
            for (size_t i = 0; i < in.column_evals.size(); i += in.columns_per_instance) {
                std::vector<dpb_mle*> cols(in.column_evals.begin() + i,
                                           in.column_evals.begin() + i + in.columns_per_instance);
                circuits.emplace_back(new LogUpCircuit<F>(ctx, in.kind, cols, nullptr, in.constant_challenge,
                                                          in.column_separation_challenge));
            }
        }
    }
    size_t total_layers = 0;
    for (size_t i = 0; i < circuits.size(); i++) {
        if (i + 1 < circuits.size() && circuits[i]->num_vars() < circuits[i + 1]->num_vars())
            throw Error(DPB_EINVAL, "Circuits were not in decreasing size order");
        total_layers = std::max(total_layers, circuits[i]->num_vars());
    }
    std::set<size_t, std::greater<size_t>> sizes;
    for (const auto& c : circuits) sizes.insert(c->num_vars());

    LogUpBatchProof<F> proof;
    proof.proof_type = proof_type;
    t_trees.stop();
    {
        dpb::TracePhase t_out("logup.outputs");
        // every circuit's outputs (LogUpCircuit::outputs, circuit.rs:558-560) with one wait for the device
        std::vector<const dpb_logup*> trees;
        for (const auto& c : circuits) trees.push_back(c->tree());
        std::vector<E> flat(4 * trees.size());
        check(dpb_logup_outputs_batch(trees.data(), (uint32_t)trees.size(), flat.data()));
        if (partial) {
            // every rank must hold the same shapes: compare a signature before anything depends on it
            std::vector<E> sig;
            for (const auto& c : circuits)
                sig.push_back(F::from_u64(((uint64_t)c->num_vars() << 32) | ((uint64_t)c->denominator_column_count() << 1) |
                                          (c->final_eval_count() != 2 * c->denominator_column_count() ? 1u : 0u)));
            sig.push_back(F::from_u64(circuits.size()));
            const std::vector<E> sigs = gather(sig);
            for (size_t q = 0; q < G; q++)
                if (memcmp(sigs.data() + q * sig.size(), sig.data(), sig.size() * sizeof(E)) != 0)
                    throw Error(DPB_EINVAL, "the ranks of a partial logup batch must hold instances of the same shapes");
            const std::vector<E> all = gather(flat);
            for (size_t i = 0; i < trees.size(); i++)
                for (size_t q = 0; q < G; q++)
                    proof.circuit_outputs.emplace_back(all.begin() + q * flat.size() + 4 * i,
                                                       all.begin() + q * flat.size() + 4 * i + 4);
        } else {
            for (size_t i = 0; i < trees.size(); i++)
                proof.circuit_outputs.emplace_back(flat.begin() + 4 * i, flat.begin() + 4 * i + 4);
        }
    }

    const E count = F::from_u64(circuits.size() * G);
    transcript.append_scalars(&count, 1);
    for (const auto& o : proof.circuit_outputs) transcript.append_scalars(o);
    E rho = transcript.append_and_sample("initial_batching");
    E alpha = transcript.append_and_sample("initial_alpha");
    E lambda = transcript.append_and_sample("initial_lambda");
    std::vector<E> point{rho};

    for (size_t v = 1; v <= total_layers; v++) {
        const size_t remaining = total_layers - (v - 1);
        std::vector<E> wit_evals;
        if (!proof.round_evaluations.empty()) wit_evals = proof.round_evaluations.back();
        for (size_t i = 0; i < circuits.size(); i++)
            if (circuits[i]->num_vars() == remaining)
                for (size_t q = 0; q < G; q++)
                    wit_evals.insert(wit_evals.end(), proof.circuit_outputs[i * G + q].begin(),
                                     proof.circuit_outputs[i * G + q].end());
        if (wit_evals.empty())
            throw Error(DPB_EINVAL, "Proving failed: No previous evals and no evals for this number of variables");

        dpb::TracePhase t_expr("logup.layer_expressions");
        std::vector<dpb_mle*> mles;
        std::vector<dpb_mle*> eq_mles;
        std::vector<X> group_exprs;
        X claim_expr = X::ZERO();
        size_t layer_count = 0;
        uint16_t wit_off = 0;
        struct EqGuard {
            std::vector<dpb_mle*>& v;
            ~EqGuard() { for (auto* m : v) dpb_mle_free(m); }
        } eq_guard{eq_mles};
        // Every layer but the last is an inner layer of every instance it touches (an instance reaches its input
        // layer when one variable remains, all of them together).  Its expression is known in closed form,
        //   alpha_j * (n_lo d_hi + n_hi d_lo + lambda d_lo d_hi) * eq        (circuit.rs:231-296),
        // so the three product terms per instance and the claim are written down directly; only the last layer,
        // whose expression depends on the instances' columns, goes through the expression builder.
        const bool inner = remaining != 1;
        dp_crypto::VirtualPolynomials<F> vp;
        E current_claim = F::zero();
        std::vector<uint32_t> term_group;  // per direct term: the size group whose eq table closes it
        std::vector<dpb::LogupHintInst> hint;  // this rank's instances as the round kernel of a logup layer wants them
        E alpha_pow = F::one();            // alpha^layer_count
        for (size_t size : sizes) {
            if (size < remaining) continue;
            const E mult_e = F::from_u64(1ull << (total_layers - size));
            const X mult = X::Constant(mult_e);
            const size_t layer_vars = size - remaining + 1;
            X group = X::ZERO();
            for (auto& c : circuits) {
                if (c->num_vars() != size) continue;
                // the whole batch holds this instance once per rank, next to each other; only this rank's takes
                // part in its sumcheck, all of them in the claim
                for (size_t q = 0; q < G; q++) {
                    if (inner) {
                        const size_t b = layer_count * 4;
                        if (b + 3 >= wit_evals.size()) throw Error(DPB_EINVAL, "Proving failed: evaluations of the layer above are short");
                        const E &w0 = wit_evals[b], &w1 = wit_evals[b + 1], &w2 = wit_evals[b + 2], &w3 = wit_evals[b + 3];
                        const E num = F::add(F::mul(rho, F::sub(w1, w0)), w0), den = F::add(F::mul(rho, F::sub(w3, w2)), w2);
                        current_claim = F::add(current_claim, F::mul(mult_e, F::mul(alpha_pow, F::add(num, F::mul(lambda, den)))));
                        if (q == g_rank) {
                            auto lm = c->layer_mles(layer_vars);
                            mles.insert(mles.end(), lm.begin(), lm.end());
                            const E al = F::mul(alpha_pow, lambda);
                            const uint16_t w = wit_off;
                            auto term = [&](const E& coef, uint16_t x, uint16_t y) {
                                if (F::is_zero(coef)) return;
                                dpb_term t;
                                memset(&t, 0, sizeof t);
                                memcpy(t.coeff, &coef, sizeof(E));
                                t.n_factors = 3;
                                t.idx[0] = x;
                                t.idx[1] = y;
                                vp.terms.push_back(t);
                                term_group.push_back((uint32_t)group_exprs.size());
                            };
                            dpb::LogupHintInst h;
                            memset(&h, 0, sizeof h);
                            h.kind = 0;
                            h.first = w;
                            memcpy(h.alpha, &alpha_pow, sizeof(E));
                            hint.push_back(h);
                            term(alpha_pow, w, (uint16_t)(w + 3));       // n_lo d_hi
                            term(alpha_pow, (uint16_t)(w + 1), (uint16_t)(w + 2));  // n_hi d_lo
                            term(al, (uint16_t)(w + 2), (uint16_t)(w + 3));         // lambda d_lo d_hi
                            wit_off = (uint16_t)(wit_off + 4);
                        }
                        layer_count++;
                        alpha_pow = F::mul(alpha_pow, alpha);
                        continue;
                    }
                    auto le = c->layer_exprs(layer_vars, layer_count, wit_off);
                    if (q == g_rank) hint.push_back(c->input_layer_hint(wit_off, alpha_pow));
                    alpha_pow = F::mul(alpha_pow, alpha);
                    layer_count++;
                    claim_expr = claim_expr + mult * le.claim;
                    if (q != g_rank) continue;
                    auto lm = c->layer_mles(layer_vars);
                    mles.insert(mles.end(), lm.begin(), lm.end());
                    wit_off = (uint16_t)(wit_off + le.num_witnesses);
                    group = group + le.sumcheck;
                }
            }
            dpb_mle* eq = nullptr;
            {
                dpb::TracePhase t_eq("logup.eq_tables");
                check(dpb_eq_table(ctx, F::kChalDtype, point.data() + (point.size() - layer_vars), (uint32_t)layer_vars, &eq));
            }
            eq_mles.push_back(eq);
            group_exprs.push_back(group);
        }
        if (!inner) current_claim = claim_expr.evaluate(wit_evals, {alpha, lambda, rho});
        transcript.append_scalars(&current_claim, 1);

        std::vector<dpb_mle*> all(mles);
        all.insert(all.end(), eq_mles.begin(), eq_mles.end());
        if (inner) {
            if (vp.terms.empty()) throw Error(DPB_EINVAL, "virtual polynomial has no terms");
            for (size_t t = 0; t < vp.terms.size(); t++) vp.terms[t].idx[2] = (uint16_t)(wit_off + term_group[t]);
            vp.num_vars = (uint32_t)v;
            vp.mles = all;
            vp.max_degree = 3;
        } else {
            X full = X::ZERO();
            for (size_t i = 0; i < group_exprs.size(); i++) full = full + group_exprs[i] * X::WitIn((uint16_t)(wit_off + i));
            auto builder = dp_crypto::VirtualPolynomialsBuilder<F>::new_with_mles(1, (uint32_t)v, all);
            dpb::TracePhase t_expand("logup.expand_terms");
            vp = builder.to_virtual_polys({full}, {alpha, lambda});
        }
        t_expr.stop();
        // one size group: one eq table, right after the instances' tables
        const bool hinted = group_exprs.size() == 1;
        auto res = dp_crypto::IOPProverState<F>::prove(ctx, vp, transcript, partial ? 2 : 0, hinted ? &hint : nullptr, &lambda,
                                                       (uint32_t)wit_off);
        point = res.second.collect_raw_challenges();
        const auto& finals = res.second.get_mle_flatten_final_evaluations();
        std::vector<E> evals(finals.begin(), finals.begin() + wit_off);
        if (partial) {
            // the whole batch's evaluations: per instance of this layer (sizes in the order above), rank by rank
            const std::vector<E> all = gather(evals);
            std::vector<E> merged;
            merged.reserve(all.size());
            size_t at = 0;
            for (size_t size : sizes) {
                if (size < remaining) continue;
                const size_t layer_vars = size - remaining + 1;
                for (auto& c : circuits) {
                    if (c->num_vars() != size) continue;
                    const size_t n = layer_vars == c->num_vars() ? c->final_eval_count() : 4;
                    for (size_t q = 0; q < G; q++)
                        merged.insert(merged.end(), all.begin() + q * evals.size() + at, all.begin() + q * evals.size() + at + n);
                    at += n;
                }
            }
            evals.swap(merged);
        }

        rho = transcript.append_and_sample("logup_batching");
        if (v != total_layers) {
            alpha = transcript.append_and_sample("logup_alpha");
            lambda = transcript.append_and_sample("logup_lambda");
        }
        point.push_back(rho);
        proof.sumcheck_proofs.push_back(std::move(res.first));
        proof.round_evaluations.push_back(std::move(evals));
    }

    if (proof.round_evaluations.empty()) throw Error(DPB_EINVAL, "Proving failed: No round evaluations found");
    const auto& last = proof.round_evaluations.back();
    size_t skip = 0;
    for (const auto& c : circuits) {
        for (size_t q = 0; q < G; q++) {
            const size_t n = c->final_eval_count();
            if (skip + n > last.size()) throw Error(DPB_EINVAL, "final evaluations are short");
            auto ev = c->combine_final_evals(last.data() + skip, n, rho);
            skip += n;
            std::vector<E> pt(point.end() - (c->num_vars() + 1), point.end());
            for (const auto& e : ev) proof.output_claims.push_back({pt, e});
            proof.num_vars_per_instance.push_back(c->num_vars());
            proof.num_denominator_columns_per_instance.push_back(c->denominator_column_count());
        }
    }
    return proof;
}

}  // namespace logup_gkr
}  // namespace zkml
