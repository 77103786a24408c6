// The lookup linking sumcheck on the GPU, following the reference's in-repo code step for step:
//   LookupVariant::{build_full_sumcheck_expression, build_lookup_output_expressions,
//   sumcheck_expression_for_chunk} (all four variants), ValueExpression::new
//                                        zkml/src/lookup/operation/variant.rs:55-346, 363-379, 467-510
//   Shape::compute_eq_point_and_batching_challenges, split_point
//                                        zkml/src/shape.rs:475-496, 565-610
//   LookupVariant::build_eq_polys        zkml/src/lookup/operation/variant/proving.rs:225-253
//   LookupInputConfig::prove_linking_sumcheck
//                                        zkml/src/lookup/operation/inputs/proving.rs:26-114
#pragma once
#include "prover.hpp"

namespace zkml {
namespace lookup {

using dp_crypto::check;
using dp_crypto::Error;
using dp_crypto::Expression;

enum class LookupVariant { Standard = 0, GLU = 1, Softmax = 2, Normalisation = 3 };

template <class F>
typename F::E to_field(int64_t x) {
    // negative x -> p - |x| (zkml/src/quantization/mod.rs:220-267)
    const uint64_t mag = x < 0 ? (uint64_t)0 - (uint64_t)x : (uint64_t)x;
    const typename F::E a = F::from_u64(mag);
    return x < 0 ? F::neg(a) : a;
}

// dp_crypto::poly::eq::evals on the host, for the few coordinates of a tensor's leading dimensions
template <class F>
std::vector<typename F::E> eq_evals(const typename F::E* point, size_t m) {
    typedef typename F::E E;
    std::vector<E> out(1, F::one());
    for (size_t j = 0; j < m; j++) {
        const size_t half = out.size();
        out.resize(2 * half);
        for (size_t i = 0; i < half; i++) {
            const E hi = F::mul(out[i], point[j]);
            out[i + half] = hi;
            out[i] = F::sub(out[i], hi);
        }
    }
    return out;
}

template <class F>
struct LookupExpressions {
    Expression<F> value, prod_selector, clamping_expression, sum, squared_clamping_expression;
};

// variant.rs:73-226 with ValueExpression::new (variant.rs:467-510).  The witnesses of chunk c are its value chunk
// outputs followed by its zeroing chunk outputs; out_min / out_max are Table::min_output_value / max_output_value.
template <class F>
LookupExpressions<F> build_lookup_output_expressions(const dpb_chunking_info& ci, size_t current_chunk, int64_t out_min,
                                                     int64_t out_max) {
    typedef Expression<F> X;
    typedef typename F::E E;
    const E one = F::one(), zero = F::zero();
    const size_t nz = ci.n_zeroing_chunks, nv = ci.n_value_chunks, bits = ci.value_chunk_bits;
    const uint16_t offset = (uint16_t)(current_chunk * (nv + nz));
    X value, sum;
    uint16_t witness_offset;
    size_t sum_challenge_offset;
    if (nv == 1) {
        value = X::WitIn(offset);
        sum = X::WitIn(offset) * X::Challenge(0, 1, one, zero);
        witness_offset = offset + 1;
        sum_challenge_offset = 2;
    } else {
        value = X::Constant(F::neg(F::from_u64(1ull << (nv * bits - 1))));
        sum = X::ZERO();
        for (size_t idx = 0; idx < nv; idx++) {
            const X chunk = X::WitIn((uint16_t)(offset + idx));
            value = value + X::Constant(F::from_u64(1ull << (bits * idx))) * (chunk + X::Constant(F::from_u64(1ull << (bits - 1))));
            sum = sum + chunk * X::Challenge(0, idx + 1, one, zero);
        }
        witness_offset = (uint16_t)(offset + nv);
        sum_challenge_offset = 1 + nv;
    }
    X prod = X::ONE(), clamp, sq_clamp = X::ZERO();  // a squared clamping part exists only in the signed case
    if (ci.table_sign == DPB_SIGN_MIXED) {
        for (size_t idx = 0; idx + 1 < nz; idx++) {
            const X chunk = X::WitIn((uint16_t)(witness_offset + idx));
            prod = prod * chunk;
            sum = sum + chunk * X::Challenge(0, sum_challenge_offset + idx, one, zero);
        }
        E cmin, cmax;
        if (nv == 1) {
            cmin = to_field<F>(out_min);
            cmax = to_field<F>(out_max);
        } else {
            const size_t full = nv * bits;
            cmin = to_field<F>(-(1ll << (full - 1)));
            cmax = to_field<F>((1ll << (full - 1)) - 1);
        }
        if (nz != 0) {
            const X last = X::WitIn((uint16_t)(witness_offset - 1 + nz));
            const X lower = prod;
            const X one_minus_sq = X::ONE() - last * last;
            prod = prod * one_minus_sq;
            sum = sum + last * X::Challenge(0, sum_challenge_offset - 1 + nz, one, zero);
            const X half = X::Constant(F::inv(F::from_u64(2)));
            const X first = last * (last + X::ONE()) * half + (one_minus_sq - lower * one_minus_sq);
            const X second = last * (last - X::ONE()) * half;
            clamp = first * X::Constant(cmax) + second * X::Constant(cmin);
            sq_clamp = first * X::Constant(cmax) * X::Constant(cmax) + second * X::Constant(cmin) * X::Constant(cmin);
        } else {
            clamp = X::ZERO();
        }
    } else {
        for (size_t idx = 0; idx < nz; idx++) {
            const X chunk = X::WitIn((uint16_t)(witness_offset + idx));
            prod = prod * chunk;
            sum = sum + chunk * X::Challenge(0, sum_challenge_offset + idx, one, zero);
        }
        clamp = nz != 0 ? X::Constant(to_field<F>(ci.table_sign == DPB_SIGN_POSITIVE ? out_max : out_min)) : X::ONE();
    }
    return {value, prod, clamp, sum, sq_clamp};
}

// variant.rs:55-70, 229-346.  Normalisation: two more witnesses per chunk (its input and its scaling), the squared
// product expression under the third eq table, optionally the sum under it too and a weight table on the output.
template <class F>
Expression<F> build_full_sumcheck_expression(LookupVariant variant, size_t total_chunks, size_t final_dim_size,
                                             const dpb_chunking_info& ci, int64_t out_min, int64_t out_max,
                                             bool normalised_sum = false, bool has_weight = false) {
    typedef Expression<F> X;
    const size_t per = ci.n_value_chunks + ci.n_zeroing_chunks;
    const size_t total_out = total_chunks * per;
    const size_t extra = variant == LookupVariant::GLU ? 1 : variant == LookupVariant::Normalisation ? 2 : 0;
    const size_t total_wit = total_out + extra * total_chunks;
    if (total_wit + 4 > 0xffff) throw Error(DPB_EINVAL, "too many witness tables for 16-bit ids");
    size_t final_dim_log = 0;
    while ((1ull << final_dim_log) < final_dim_size) final_dim_log++;
    const X output_linking_eq = X::WitIn((uint16_t)total_wit), lookup_linking_eq = X::WitIn((uint16_t)(total_wit + 1));
    X acc = X::ZERO();
    for (size_t c = 0; c < total_chunks; c++) {
        const LookupExpressions<F> e = build_lookup_output_expressions<F>(ci, c, out_min, out_max);
        const X prod_expression = e.clamping_expression + e.prod_selector * e.value;
        if (variant == LookupVariant::Normalisation) {
            const X normalisation_eq = X::WitIn((uint16_t)(total_wit + 2));
            const typename F::E pow_two = F::from_u64(1ull << final_dim_log);
            const X prod_squared = e.squared_clamping_expression + e.prod_selector * e.value * e.value;
            const X lead = has_weight ? output_linking_eq * X::WitIn((uint16_t)(total_wit + 3)) : output_linking_eq;
            X out_part = lead * prod_expression;
            if (normalised_sum)
                out_part = out_part + X::Challenge((uint16_t)(1 + total_chunks), 2, pow_two, F::zero()) * (normalisation_eq * prod_expression);
            const X input = X::WitIn((uint16_t)(total_out + c)) * X::WitIn((uint16_t)(total_out + total_chunks + c));
            acc = acc + X::Challenge((uint16_t)(1 + c), 1, F::one(), F::zero()) *
                            (out_part + X::Challenge((uint16_t)(1 + total_chunks), 1, pow_two, F::zero()) * (normalisation_eq * prod_squared) +
                             lookup_linking_eq * (e.sum + X::Challenge((uint16_t)(2 + total_chunks), 1, F::one(), F::zero()) * input));
            continue;
        }
        X out_part = output_linking_eq * prod_expression;
        if (variant == LookupVariant::GLU) out_part = out_part * X::WitIn((uint16_t)(total_out + c));
        if (variant == LookupVariant::Softmax) {
            // the normalisation check rides on the same product expression through the third eq table
            const X normalisation_eq = X::WitIn((uint16_t)(total_wit + 2));
            const X sum_norm_challenge = X::Challenge((uint16_t)(1 + total_chunks), 1, F::from_u64(1ull << final_dim_log), F::zero());
            out_part = out_part + sum_norm_challenge * (normalisation_eq * prod_expression);
        }
        acc = acc + X::Challenge((uint16_t)(1 + c), 1, F::one(), F::zero()) * (out_part + lookup_linking_eq * e.sum);
    }
    return acc;
}

// shape.rs:565-610: (coordinates of the last two padded dimensions, one coefficient per slice over them)
template <class F>
std::pair<std::vector<typename F::E>, std::vector<typename F::E>> compute_eq_point_and_batching_challenges(
    const std::vector<uint64_t>& shape, const std::vector<typename F::E>& point) {
    typedef typename F::E E;
    std::vector<size_t> vars(shape.size());
    size_t total = 0;
    for (size_t i = 0; i < shape.size(); i++) {
        size_t v = 0;
        while ((1ull << v) < shape[i]) v++;
        vars[i] = v;
        total += v;
    }
    if (point.size() != total)
        throw Error(DPB_EINVAL, "Point length " + std::to_string(point.size()) + " does not match total variables " + std::to_string(total));
    const size_t skip = shape.size() > 2 ? shape.size() - 2 : 0;
    std::vector<E> eq_points, chal(1, F::one());
    size_t end = total;
    for (size_t i = 0; i < shape.size(); i++) {  // split_point: the first dimension takes the last coordinates
        const size_t start = end - vars[i];
        if (i < skip) {
            const std::vector<E> ev = eq_evals<F>(point.data() + start, vars[i]);
            std::vector<E> next;
            next.reserve(chal.size() * shape[i]);
            for (const E& c : chal)
                for (uint64_t j = 0; j < shape[i]; j++) next.push_back(F::mul(c, ev[j]));
            chal.swap(next);
        } else {
            std::vector<E> joined(point.begin() + start, point.begin() + end);
            joined.insert(joined.end(), eq_points.begin(), eq_points.end());
            eq_points.swap(joined);
        }
        end = start;
    }
    return {eq_points, chal};
}

template <class F>
struct LookupSumcheckProof {
    dp_crypto::IOPProof<F> sumcheck_proof;
    std::vector<typename F::E> evaluations;     // the witness tables at the sumcheck's point, eq tables left out
    std::vector<typename F::E> sumcheck_point;
    std::vector<typename F::E> batching_challenges;
    bool has_weight_eval = false;
    typename F::E weight_eval;                  // the weight table at the point, when one was given
    uint32_t degree = 0;
};

// inputs/proving.rs:26-114.  `mles` in the expression's order; weight_mle may be null.
template <class F, class T>
LookupSumcheckProof<F> prove_linking_sumcheck(dpb_ctx* ctx, LookupVariant variant, const dpb_chunking_info& ci, int64_t out_min,
                                              int64_t out_max, const std::vector<uint64_t>& unpadded_input_shape,
                                              const std::vector<dpb_mle*>& mles, const std::vector<typename F::E>& last_claim_point,
                                              const std::vector<typename F::E>& logup_point, T& transcript,
                                              bool normalised_sum = false, dpb_mle* weight_mle = nullptr) {
    typedef typename F::E E;
    auto pc = compute_eq_point_and_batching_challenges<F>(unpadded_input_shape, last_claim_point);
    const std::vector<E>& output_eq_point = pc.first;
    std::vector<E> batching = pc.second;
    const size_t total_chunks = batching.size();
    const size_t extra = variant == LookupVariant::GLU ? 1 : variant == LookupVariant::Normalisation ? 2 : 0;
    const size_t want = total_chunks * (ci.n_value_chunks + ci.n_zeroing_chunks + extra);
    if (weight_mle && variant != LookupVariant::Normalisation)
        throw Error(DPB_EINVAL, "only the normalisation variant's expression has a weight table");
    if (mles.size() != want)
        throw Error(DPB_EINVAL, "the expression has " + std::to_string(want) + " witness tables, " + std::to_string(mles.size()) + " given");
    if (logup_point.size() != output_eq_point.size())
        throw Error(DPB_EINVAL, "the logup point has " + std::to_string(logup_point.size()) + " coordinates, the slices " +
                                    std::to_string(output_eq_point.size()) + " variables");
    const E sum_challenge = transcript.append_and_sample("sum");
    batching.insert(batching.begin(), sum_challenge);
    // squeeze_sumcheck_challenges (variant.rs:363-379)
    const bool third_eq = variant == LookupVariant::Softmax || variant == LookupVariant::Normalisation;
    if (third_eq) batching.push_back(transcript.append_and_sample("normalisation"));
    if (variant == LookupVariant::Normalisation) batching.push_back(transcript.append_and_sample("input"));

    // build_eq_polys (variant/proving.rs:225-253): eq(output point), eq(logup point) and, for Softmax, eq of
    // (1/2, .., 1/2, the logup point's coordinates above the last dimension's); all in one call
    const uint32_t n = (uint32_t)output_eq_point.size();
    const uint32_t n_eq = third_eq ? 3 : 2;
    std::vector<E> pts(output_eq_point);
    pts.insert(pts.end(), logup_point.begin(), logup_point.end());
    if (third_eq) {
        size_t fdv = 0;
        while ((1ull << fdv) < unpadded_input_shape.back()) fdv++;
        const E half = F::inv(F::from_u64(2));
        for (size_t j = 0; j < n; j++) pts.push_back(j < fdv ? half : logup_point[j]);
    }
    const uint32_t nv[3] = {n, n, n};
    dpb_mle* eqs[3] = {nullptr, nullptr, nullptr};
    dpb_mle* eq_owner = nullptr;
    check(dpb_eq_tables(ctx, F::kChalDtype, pts.data(), nv, n_eq, &eq_owner, eqs));
    struct G {
        dpb_mle** v;
        dpb_mle*& owner;
        ~G() {
            for (int i = 0; i < 3; i++) dpb_mle_free(v[i]);
            dpb_mle_free(owner);
        }
    } g{eqs, eq_owner};
    std::vector<dpb_mle*> all(mles);
    for (uint32_t i = 0; i < n_eq; i++) all.push_back(eqs[i]);
    if (weight_mle) all.push_back(weight_mle);  // after the eq tables (inputs/proving.rs:66-68)
    const Expression<F> expression = build_full_sumcheck_expression<F>(variant, total_chunks, unpadded_input_shape.back(), ci,
                                                                       out_min, out_max, normalised_sum, weight_mle != nullptr);
    auto builder = dp_crypto::VirtualPolynomialsBuilder<F>::new_with_mles(1, n, all);
    auto vp = builder.to_virtual_polys({expression}, batching);
    auto res = dp_crypto::IOPProverState<F>::prove(ctx, vp, transcript);
    LookupSumcheckProof<F> out;
    out.sumcheck_proof = res.first;
    out.evaluations = res.second.get_mle_flatten_final_evaluations();
    if (weight_mle) {
        out.has_weight_eval = true;
        out.weight_eval = out.evaluations.back();
    }
    out.evaluations.resize(mles.size());  // drop the eq tables' (and the weight's) evaluations
    out.sumcheck_point = res.second.collect_raw_challenges();
    out.batching_challenges = batching;
    out.degree = vp.max_degree;
    return out;
}

}  // namespace lookup
}  // namespace zkml
