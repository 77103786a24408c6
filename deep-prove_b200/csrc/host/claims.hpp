// Claim batching of the opening proof on the GPU, following the reference's
// in-repo code step for step:
//   ChunkedCommitment helpers, identity_eval, and build_sumcheck_expression's polynomial (summed in a form
//   that is linear-combined per claim first)   zkml/src/poly_commit/mod.rs:32-148, 184-192
//   CommitmentProver::claims_batching_sumcheck and the random linear combination
//   of the committed polynomials that CommitmentProver::prove builds before it
//   calls the commitment scheme        zkml/src/poly_commit/prover.rs:113-131, 140-255
// The commitment scheme itself (PCS::prove) is not part of this library.
#pragma once
#include "prover.hpp"

namespace zkml {
namespace poly_commit {

using dp_crypto::check;
using dp_crypto::Error;
using dp_crypto::Expression;

// mod.rs:184-192
template <class F>
typename F::E identity_eval(const typename F::E* r1, size_t n1, const typename F::E* r2, size_t n2) {
    typedef typename F::E E;
    E acc = F::one();
    const size_t n = std::min(n1, n2);
    for (size_t i = 0; i < n; i++) {
        const E a = r1[i], b = r2[i];
        acc = F::mul(acc, F::add(F::mul(a, b), F::mul(F::sub(F::one(), a), F::sub(F::one(), b))));
    }
    return acc;
}

template <class F>
struct Claim {
    std::vector<typename F::E> point;
    typename F::E eval;
};

// A committed polynomial as the tables of its M = 2^b chunks (all of one length) with the claims to batch.
template <class F>
struct CommittedPoly {
    typedef typename F::E E;
    std::vector<dpb_mle*> chunks;  // borrowed
    std::vector<Claim<F>> claims;

    size_t num_chunks() const { return chunks.size(); }
    size_t batching_vars() const {
        size_t b = 0;
        while ((1ull << b) < chunks.size()) b++;
        return b;
    }
    size_t num_vars_for_chunk() const {
        size_t m = 0;
        while ((1ull << m) < dpb_mle_len(chunks[0])) m++;
        return m;
    }
    // mod.rs:46-59: C_i = eq(bits of i, the last b coordinates of the point)
    std::vector<E> batching_coefficients_for_chunks(const std::vector<E>& point) const {
        const size_t b = batching_vars();
        std::vector<E> out;
        for (size_t i = 0; i < chunks.size(); i++) {
            std::vector<E> bits(b);
            for (size_t q = 0; q < b; q++) bits[q] = F::from_u64((i >> q) & 1);
            out.push_back(identity_eval<F>(point.data() + (point.size() - b), b, bits.data(), b));
        }
        return out;
    }
    void validate(size_t index) const {
        if (chunks.empty() || (chunks.size() & (chunks.size() - 1)))
            throw Error(DPB_EINVAL, "polynomial " + std::to_string(index) + ": the chunk count must be a power of two");
        const uint64_t len = dpb_mle_len(chunks[0]);
        if (len == 0 || (len & (len - 1)))
            throw Error(DPB_EINVAL, "polynomial " + std::to_string(index) + ": chunk length is not a power of two");
        for (auto* c : chunks)
            if (!c || dpb_mle_len(c) != len)
                throw Error(DPB_EINVAL, "polynomial " + std::to_string(index) + ": chunks differ in length");
        for (const auto& c : claims)
            if (c.point.size() != num_vars_for_chunk() + batching_vars())
                throw Error(DPB_EINVAL, "polynomial " + std::to_string(index) + ": a claim's point has the wrong length");
    }
};

template <class F>
struct ClaimsBatchingProof {
    typedef typename F::E E;
    dp_crypto::IOPProof<F> sumcheck_proof;
    std::vector<E> sumcheck_evals;  // the committed chunks at the point (of their zero-padded extensions)
    std::vector<E> sumcheck_point;
    size_t max_num_vars = 0;
    std::vector<dpb_mle*> committed_polys;  // borrowed, in sumcheck order
};

// prover.rs:140-255.  `polys` in the order the reference visits them: model commitments, then witness commitments.
template <class F, class T>
ClaimsBatchingProof<F> claims_batching_sumcheck(dpb_ctx* ctx, const std::vector<CommittedPoly<F>>& polys, T& transcript) {
    typedef typename F::E E;
    if (polys.empty()) throw Error(DPB_EINVAL, "no committed polynomials");
    ClaimsBatchingProof<F> out;
    std::vector<dpb_mle*> owned;  // eq tables and zero-padded views
    struct Guard {
        std::vector<dpb_mle*>& v;
        ~Guard() { for (auto* m : v) dpb_mle_free(m); }
    } guard{owned};
    std::vector<std::vector<std::vector<E>>> coeffs;
    std::vector<E> eq_points;       // the eq point of every claim, end to end
    std::vector<uint32_t> eq_vars;  // and its length
    size_t total_chunks = 0, total_claims = 0;
    for (size_t pi = 0; pi < polys.size(); pi++) {
        const auto& p = polys[pi];
        p.validate(pi);
        std::vector<std::vector<E>> per_claim;
        for (const auto& c : p.claims) {
            transcript.append_scalars(&c.eval, 1);
            // eq_point_per_chunk (mod.rs:61-69): the point without its last log2(chunks) coordinates
            eq_points.insert(eq_points.end(), c.point.begin(), c.point.begin() + p.num_vars_for_chunk());
            eq_vars.push_back((uint32_t)p.num_vars_for_chunk());
            per_claim.push_back(p.batching_coefficients_for_chunks(c.point));
        }
        total_claims += p.claims.size();
        total_chunks += p.num_chunks();
        coeffs.push_back(std::move(per_claim));
        out.committed_polys.insert(out.committed_polys.end(), p.chunks.begin(), p.chunks.end());
        out.max_num_vars = std::max(out.max_num_vars, p.num_vars_for_chunk());
    }
    if (total_chunks + total_claims > 65535) throw Error(DPB_EINVAL, "more than 65535 tables in one batching sumcheck");
    if (total_claims == 0) throw Error(DPB_EINVAL, "no claims to batch");
    // all eq tables in one call (one block of device memory, two launches)
    std::vector<dpb_mle*> eq_polys(total_claims, nullptr);
    dpb_mle* eq_owner = nullptr;
    check(dpb_eq_tables(ctx, F::kChalDtype, eq_points.data(), eq_vars.data(), (uint32_t)total_claims, &eq_owner,
                        eq_polys.data()));
    for (auto* m : eq_polys) owned.push_back(m);
    owned.push_back(eq_owner);  // freed last
    // The expression (build_sumcheck_expression, mod.rs:96-148) is  sum_t gamma^t (sum_c coef_{t,c} chunk_c) eq_t
    // over the claims t: LINEAR in the chunk tables.  The sumcheck therefore runs over one table per claim,
    // L_t = sum_c coef_{t,c} chunk_c (the chunk itself when the polynomial has one chunk), instead of over every
    // chunk: the same polynomial is summed, so the round messages are the same field elements, and the prover
    // binds and stores 2 tables per claim instead of (chunks + 1).  What the proof hands on, every chunk at the
    // sumcheck's point, comes from one pass over the chunks afterwards (dpb_mle_evaluate_many).
    std::vector<dpb_mle*> term_tables;
    for (size_t pi = 0; pi < polys.size(); pi++) {
        const auto& p = polys[pi];
        for (size_t i = 0; i < coeffs[pi].size(); i++) {
            if (coeffs[pi][i].size() != p.num_chunks()) throw Error(DPB_EINVAL, "wrong number of chunk challenges");
            if (p.num_chunks() == 1 && F::is_one(coeffs[pi][i][0])) {
                term_tables.push_back(p.chunks[0]);
                continue;
            }
            dpb_mle* l = nullptr;
            check(dpb_linear_combination(ctx, p.chunks.data(), coeffs[pi][i].data(), (uint32_t)p.num_chunks(), &l));
            owned.push_back(l);
            term_tables.push_back(l);
        }
    }
    typedef Expression<F> X;
    X expr = X::Constant(F::zero());
    for (size_t t = 0; t < total_claims; t++)
        expr = expr + X::Challenge(0, t, F::one(), F::zero()) * X::WitIn((uint16_t)t) * X::WitIn((uint16_t)(total_claims + t));
    // every table enters as a zero-padded view of max_num_vars variables (prover.rs:214-226)
    std::vector<dpb_mle*> views;
    auto add_view = [&](dpb_mle* m) {
        dpb_mle* v = nullptr;
        check(dpb_mle_zero_padded(m, &v));
        owned.push_back(v);
        views.push_back(v);
    };
    for (auto* m : term_tables) add_view(m);
    for (auto* m : eq_polys) add_view(m);
    const E challenge = transcript.append_and_sample("model_batching");
    auto builder = dp_crypto::VirtualPolynomialsBuilder<F>::new_with_mles(1, (uint32_t)out.max_num_vars, views);
    auto vp = builder.to_virtual_polys({expr}, {challenge});
    auto res = dp_crypto::IOPProverState<F>::prove(ctx, vp, transcript);
    out.sumcheck_point = res.second.collect_raw_challenges();
    out.sumcheck_proof = std::move(res.first);
    out.sumcheck_evals.resize(total_chunks);
    check(dpb_mle_evaluate_many(ctx, out.committed_polys.data(), (uint32_t)total_chunks, out.sumcheck_point.data(),
                                (uint32_t)out.max_num_vars, out.sumcheck_evals.data()));
    return out;
}

// prover.rs:113-122: point and evaluations into the transcript, one challenge per committed chunk, and the
// random linear combination the commitment scheme opens.  The caller owns *rlc.
template <class F, class T>
std::vector<typename F::E> batching_rlc(dpb_ctx* ctx, const ClaimsBatchingProof<F>& proof, T& transcript, dpb_mle** rlc) {
    typedef typename F::E E;
    transcript.append_scalars(proof.sumcheck_point);
    transcript.append_scalars(proof.sumcheck_evals);
    std::vector<E> challenges;
    for (size_t i = 0; i < proof.committed_polys.size(); i++) challenges.push_back(transcript.challenge_scalar());
    check(dpb_linear_combination(ctx, proof.committed_polys.data(), challenges.data(), (uint32_t)challenges.size(), rlc));
    return challenges;
}

}  // namespace poly_commit
}  // namespace zkml
