// The einsum layer prover above the axis fixing
// (EinSum::prove_internal, zkml/src/layers/einsum/prove.rs:48-335), without the
// axis mapping (the caller says which axis of which tensor is bound to which
// point) and without biases (a bias claim is an evaluation, prove.rs:190-213,
// dpb_bias_evaluation; it never touches the transcript).
//
// One left tensor, R right tensors, R outputs.  Output i fixes the left tensor
// at its own points (FixedAxesMapping::lhs_fixes, axis.rs:1043-1075) and the
// right tensor i at its points (rhs_fixes, axis.rs:1102-1140); the stacked axes
// give S tables per fix and the stacking coefficients
// prod_axes evals(point)[..size].  The sumcheck (op_info.rs:159-195) is
//   sum_i gamma^i sum_t coef_{i,t} * lhs_{i,t} * rhs_{i,t}
// over the contracted variables, gamma = append_and_sample("batching_challenge").
// With R > 1 the R claims on the left tensor are merged by a second sumcheck
// input * sum_i c^i eq_i over the padded left tensor (prove.rs:260-288),
// c = append_and_sample("input_batching_challenge").
#pragma once
#include "lookup.hpp"
#include "prover.hpp"

namespace zkml {
namespace einsum {

using dp_crypto::check;
using dp_crypto::Error;
using dp_crypto::Expression;

template <class F>
struct Operand {
    typedef typename F::E E;
    const int64_t* tensor;
    bool on_device;
    std::vector<uint64_t> shape;
    std::vector<uint8_t> kind;
    std::vector<std::vector<E>> points;  // per axis; empty for a contracted axis
};

template <class F>
struct EinsumProof {
    typedef typename F::E E;
    E batching_challenge;
    std::vector<std::vector<E>> stacking_coeffs;  // [R][S]
    dp_crypto::IOPProof<F> sumcheck;
    std::vector<E> point, evaluations;  // evaluations: lhs tables of every output, then rhs tables
    std::vector<std::vector<E>> rhs_points;
    std::vector<E> rhs_evals;
    bool aggregated = false;
    E input_batching_challenge;
    dp_crypto::IOPProof<F> aggregation;
    std::vector<E> lhs_point;
    E lhs_eval;
};

inline uint32_t ceil_log2(uint64_t x) {
    uint32_t n = 0;
    while ((1ull << n) < x) n++;
    return n;
}

// axis.rs:1052-1062: the first stacked axis is the slowest index
template <class F>
std::vector<typename F::E> stacking_coefficients(const Operand<F>& op) {
    typedef typename F::E E;
    std::vector<E> acc(1, F::one());
    for (size_t a = op.shape.size(); a-- > 0;) {
        if (op.kind[a] != DPB_AXIS_STACKED) continue;
        if ((1ull << op.points[a].size()) < op.shape[a])
            throw Error(DPB_EINVAL, "a stacked axis needs a point of ceil_log2(size) coordinates");
        const std::vector<E> beta = lookup::eq_evals<F>(op.points[a].data(), op.points[a].size());
        std::vector<E> next;
        next.reserve(acc.size() * op.shape[a]);
        for (uint64_t b = 0; b < op.shape[a]; b++)
            for (const E& x : acc) next.push_back(F::mul(x, beta[b]));
        acc.swap(next);
    }
    return acc;
}

// prove.rs:338-361
template <class F>
std::vector<typename F::E> reconstruct_full_point(const Operand<F>& op, const std::vector<typename F::E>& sc_point) {
    std::vector<typename F::E> out;
    size_t skip = 0;
    for (size_t a = op.shape.size(); a-- > 0;) {
        if (op.kind[a] == DPB_AXIS_CONTRACTED) {
            const uint32_t n = ceil_log2(op.shape[a]);
            if (skip + n > sc_point.size()) throw Error(DPB_EINVAL, "the sumcheck point is shorter than the contracted axes");
            out.insert(out.end(), sc_point.begin() + skip, sc_point.begin() + skip + n);
            skip += n;
        } else {
            out.insert(out.end(), op.points[a].begin(), op.points[a].end());
        }
    }
    return out;
}

template <class F>
struct FixedTables {
    dpb_mle* owner = nullptr;
    std::vector<dpb_mle*> views;
    FixedTables() = default;
    FixedTables(const FixedTables&) = delete;
    FixedTables& operator=(const FixedTables&) = delete;
    ~FixedTables() {
        for (auto* v : views) dpb_mle_free(v);
        dpb_mle_free(owner);
    }
    void fix(dpb_ctx* ctx, const Operand<F>& op) {
        const uint32_t rank = (uint32_t)op.shape.size();
        uint64_t S = 1;
        std::vector<const void*> pts(rank, nullptr);
        std::vector<uint32_t> lens(rank, 0);
        for (uint32_t a = 0; a < rank; a++) {
            if (op.kind[a] == DPB_AXIS_STACKED) S *= op.shape[a];
            if (op.kind[a] == DPB_AXIS_OUTER) {
                pts[a] = op.points[a].empty() ? nullptr : op.points[a].data();
                lens[a] = (uint32_t)op.points[a].size();
            }
        }
        views.assign(S, nullptr);
        uint32_t n = 0;
        check(dpb_einsum_fix_axes(ctx, F::kChalDtype, op.tensor, op.on_device ? 1 : 0, op.shape.data(), op.kind.data(),
                                  pts.data(), lens.data(), rank, &owner, views.data(), (uint32_t)S, &n));
        views.resize(n);
    }
};

template <class F, class T>
EinsumProof<F> prove(dpb_ctx* ctx, const std::vector<Operand<F>>& lhs, const std::vector<Operand<F>>& rhs,
                     dpb_mle* lhs_padded, T& transcript) {
    typedef typename F::E E;
    typedef Expression<F> X;
    const size_t R = rhs.size();
    if (R == 0 || lhs.size() != R) throw Error(DPB_EINVAL, "one fix of the left tensor per right tensor, at least one");
    EinsumProof<F> out;
    std::vector<FixedTables<F>> lt(R), rt(R);
    for (size_t i = 0; i < R; i++) {
        lt[i].fix(ctx, lhs[i]);
        out.stacking_coeffs.push_back(stacking_coefficients<F>(lhs[i]));
    }
    for (size_t i = 0; i < R; i++) rt[i].fix(ctx, rhs[i]);
    const size_t S = out.stacking_coeffs[0].size();
    for (size_t i = 0; i < R; i++)
        if (lt[i].views.size() != S || rt[i].views.size() != S || out.stacking_coeffs[i].size() != S)
            throw Error(DPB_EINVAL, "the stacked axes of all tensors must span the same number of tables");
    out.batching_challenge = transcript.append_and_sample("batching_challenge");

    std::vector<dpb_mle*> mles;
    for (size_t i = 0; i < R; i++) mles.insert(mles.end(), lt[i].views.begin(), lt[i].views.end());
    for (size_t i = 0; i < R; i++) mles.insert(mles.end(), rt[i].views.begin(), rt[i].views.end());
    const uint64_t len = dpb_mle_len(mles[0]);
    for (auto* m : mles)
        if (dpb_mle_len(m) != len) throw Error(DPB_EINVAL, "the contracted axes of all tensors must have the same sizes");
    const uint32_t num_vars = ceil_log2(len);

    // op_info.rs:159-195
    X expr = X::ZERO();
    for (size_t i = 0; i < R; i++) {
        const size_t off = i * S, roff = R * S + off;
        const auto& c = out.stacking_coeffs[i];
        X inner = X::Constant(c[0]) * X::WitIn((uint16_t)off) * X::WitIn((uint16_t)roff);
        for (size_t j = 1; j < S; j++)
            inner = X::Constant(c[j]) * X::WitIn((uint16_t)(off + j)) * X::WitIn((uint16_t)(roff + j)) + inner;
        expr = expr + X::Challenge(0, i, F::one(), F::zero()) * inner;
    }
    auto builder = dp_crypto::VirtualPolynomialsBuilder<F>::new_with_mles(1, num_vars, mles);
    auto vp = builder.to_virtual_polys({expr}, {out.batching_challenge});
    auto res = dp_crypto::IOPProverState<F>::prove(ctx, vp, transcript);
    out.sumcheck = std::move(res.first);
    out.point = res.second.collect_raw_challenges();
    out.evaluations = res.second.get_mle_flatten_final_evaluations();

    auto comb = [&](const std::vector<E>& c, const E* ev) {
        E acc = F::zero();
        for (size_t j = 0; j < c.size(); j++) acc = F::add(acc, F::mul(c[j], ev[j]));
        return acc;
    };
    for (size_t i = 0; i < R; i++) {
        out.rhs_points.push_back(reconstruct_full_point<F>(rhs[i], out.point));
        out.rhs_evals.push_back(comb(out.stacking_coeffs[i], out.evaluations.data() + R * S + i * S));
    }
    if (R == 1) {
        out.lhs_point = reconstruct_full_point<F>(lhs[0], out.point);
        out.lhs_eval = comb(out.stacking_coeffs[0], out.evaluations.data());
        return out;
    }

    // prove.rs:260-288
    if (!lhs_padded) throw Error(DPB_EINVAL, "several outputs: the padded left tensor is needed to merge its claims");
    const uint32_t nv = ceil_log2(dpb_mle_len(lhs_padded));
    std::vector<E> flat;
    for (size_t i = 0; i < R; i++) {
        const std::vector<E> p = reconstruct_full_point<F>(lhs[i], out.point);
        if (p.size() != nv) throw Error(DPB_EINVAL, "the padded left tensor does not have the variables of its claims");
        flat.insert(flat.end(), p.begin(), p.end());
    }
    std::vector<dpb_mle*> eqs(R, nullptr);
    dpb_mle* eq_owner = nullptr;
    struct G {
        std::vector<dpb_mle*>& v;
        dpb_mle*& owner;
        ~G() {
            for (auto* m : v) dpb_mle_free(m);
            dpb_mle_free(owner);
        }
    } guard{eqs, eq_owner};
    const std::vector<uint32_t> vars(R, nv);
    check(dpb_eq_tables(ctx, F::kChalDtype, flat.data(), vars.data(), (uint32_t)R, &eq_owner, eqs.data()));
    out.input_batching_challenge = transcript.append_and_sample("input_batching_challenge");
    X agg = X::ZERO();
    for (size_t i = 0; i < R; i++)
        agg = agg + X::WitIn(0) * X::WitIn((uint16_t)(i + 1)) * X::Challenge(0, i, F::one(), F::zero());
    std::vector<dpb_mle*> all{lhs_padded};
    all.insert(all.end(), eqs.begin(), eqs.end());
    auto b2 = dp_crypto::VirtualPolynomialsBuilder<F>::new_with_mles(1, nv, all);
    auto vp2 = b2.to_virtual_polys({agg}, {out.input_batching_challenge});
    auto res2 = dp_crypto::IOPProverState<F>::prove(ctx, vp2, transcript);
    out.aggregated = true;
    out.aggregation = std::move(res2.first);
    out.lhs_point = res2.second.collect_raw_challenges();
    out.lhs_eval = res2.second.get_mle_flatten_final_evaluations()[0];
    return out;
}

}  // namespace einsum
}  // namespace zkml
