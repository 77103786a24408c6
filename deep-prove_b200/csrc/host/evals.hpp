// Closed-form evaluations the layer provers and verifiers use between sumchecks: the "less than" polynomial of a
// dimension, the evaluation of a lookup input's padding and of a broadcast bias.  Host arithmetic on a handful of
// field elements; restated from
//   eval_zeroifier_mle                       zkml/src/lib.rs:131-138
//   evaluate_dim_lt_poly                     zkml/src/lookup/operation/variant/verifying.rs:6-22
//   Shape::broadcasting_evaluation           zkml/src/shape.rs:516-562
//   compute_lookup_padding_evaluation        zkml/src/lookup/operation/mod.rs:289-340
//   AxesMapping::compute_bias_evaluation     zkml/src/layers/einsum/axis.rs:655-720
#pragma once
#include "prover.hpp"

namespace zkml {

using dp_crypto::Error;

inline uint32_t ceil_log2_sz(uint64_t x) {
    uint32_t l = 0;
    while ((1ull << l) < x) l++;
    return l;
}

// The MLE of the matrix with ones where column <= row at (column_point, row_point), coordinates little-endian.
template <class F>
typename F::E eval_zeroifier_mle(const typename F::E* column_point, const typename F::E* row_point, size_t n) {
    typedef typename F::E E;
    const E one = F::one();
    E acc = one;
    for (size_t i = 0; i < n; i++) {
        const E c = column_point[i], r = row_point[i];
        const E cr = F::mul(c, r);
        acc = F::add(F::mul(acc, F::add(F::sub(F::sub(one, c), r), F::add(cr, cr))), F::mul(F::sub(one, c), r));
    }
    return acc;
}

// lt(point, size): one on indices below `size`, zero on the padding, as a polynomial of the index bits
template <class F>
typename F::E dim_lt_eval(const typename F::E* point, size_t n, uint64_t size) {
    std::vector<typename F::E> bits(n);
    for (size_t b = 0; b < n; b++) bits[b] = F::from_u64(((size - 1) >> b) & 1);
    return eval_zeroifier_mle<F>(point, bits.data(), n);
}

template <class F>
typename F::E evaluate_dim_lt_poly(const typename F::E* point, size_t n, uint64_t size) {
    if (n != ceil_log2_sz(size))
        throw Error(DPB_EINVAL, "Row point length " + std::to_string(n) + " does not match unpadded seq len log2 " +
                                    std::to_string(ceil_log2_sz(size)));
    return dim_lt_eval<F>(point, n, size);
}

// `point`: the claim's point over the padded shape; dimension d owns the coordinates Shape::split_point gives it
// (the last dimension the first ones).  Returns offset and length of every dimension's slice.
inline void split_point_offsets(const uint64_t* shape, uint32_t rank, size_t n_point, std::vector<size_t>& off,
                                std::vector<size_t>& len) {
    size_t total = 0;
    for (uint32_t d = 0; d < rank; d++) total += ceil_log2_sz(shape[d]);
    if (total != n_point)
        throw Error(DPB_EINVAL, "Point length " + std::to_string(n_point) + " does not match total variables " +
                                    std::to_string(total));
    off.resize(rank);
    len.resize(rank);
    size_t end = n_point;
    for (uint32_t d = 0; d < rank; d++) {
        len[d] = ceil_log2_sz(shape[d]);
        off[d] = end - len[d];
        end = off[d];
    }
}

template <class F>
typename F::E compute_lookup_padding_evaluation(const typename F::E& padding_value, const uint64_t* shape, uint32_t rank,
                                                const typename F::E* point, size_t n_point) {
    typedef typename F::E E;
    if (rank == 0) throw Error(DPB_EINVAL, "Input tensor must have rank at least 1");
    std::vector<size_t> off, len;
    split_point_offsets(shape, rank, n_point, off, len);
    auto pow2 = [](uint64_t d) { return (d & (d - 1)) == 0; };
    const uint32_t lead = rank >= 2 ? rank - 2 : 0;
    bool all_pow2 = true;
    for (uint32_t d = lead; d < rank; d++) all_pow2 = all_pow2 && pow2(shape[d]);
    if (all_pow2) return F::zero();
    const E one = F::one();
    E leading = one;  // broadcasting_evaluation over the leading dimensions
    for (uint32_t d = 0; d < lead; d++) leading = F::mul(leading, dim_lt_eval<F>(point + off[d], len[d], shape[d]));
    const uint64_t second_last = rank >= 2 ? shape[rank - 2] : 1, last = shape[rank - 1];
    const E last_lt = pow2(last) ? F::zero()
                                 : F::sub(one, evaluate_dim_lt_poly<F>(point + off[rank - 1], len[rank - 1], last));
    E ev;
    if (second_last == 1 || pow2(second_last)) {
        ev = F::mul(leading, last_lt);
    } else {
        const E sl = evaluate_dim_lt_poly<F>(point + off[rank - 2], len[rank - 2], second_last);
        ev = F::mul(leading, F::add(F::mul(sl, last_lt), F::sub(one, sl)));
    }
    return F::mul(ev, padding_value);
}

// present[d] != 0: output dimension d is an axis of the bias.  Returns the broadcast evaluation; bias_point gets
// the bias's own evaluation point (its dimensions' slices, last dimension first) when bias_pos is given:
// bias_pos[d] = position of output dimension d in the bias tensor.
template <class F>
typename F::E compute_bias_evaluation(const uint64_t* out_shape, uint32_t rank, const uint8_t* present,
                                      const uint32_t* bias_pos, const typename F::E* point, size_t n_point,
                                      const typename F::E& bias_eval, std::vector<typename F::E>* bias_point) {
    typedef typename F::E E;
    std::vector<size_t> off, len;
    split_point_offsets(out_shape, rank, n_point, off, len);
    E ev = bias_eval;
    uint32_t bias_rank = 0;
    for (uint32_t d = 0; d < rank; d++) {
        if (!present[d]) ev = F::mul(ev, dim_lt_eval<F>(point + off[d], len[d], out_shape[d]));
        else bias_rank++;
    }
    if (bias_point && bias_pos) {
        std::vector<int> at(bias_rank, -1);
        for (uint32_t d = 0; d < rank; d++) {
            if (!present[d]) continue;
            if (bias_pos[d] >= bias_rank || at[bias_pos[d]] >= 0)
                throw Error(DPB_EINVAL, "Bias tensor does not have all its axes present in the output tensor");
            at[bias_pos[d]] = (int)d;
        }
        bias_point->clear();
        for (uint32_t b = bias_rank; b-- > 0;)
            bias_point->insert(bias_point->end(), point + off[at[b]], point + off[at[b]] + len[at[b]]);
    }
    return ev;
}

}  // namespace zkml
