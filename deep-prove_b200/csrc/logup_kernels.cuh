// logup-GKR fraction tree: one level per launch.
//
// A level holds a numerator and a denominator array.  The next level adds the
// fraction at index i to the one at i + half (the split is on the top
// variable): (n1/d1) + (n2/d2) = (n1*d2 + n2*d1) / (d1*d2), following
// LogUpLayer::next_layer (zkml/src/lookup/logup_gkr/circuit.rs:88-184) and
// Fraction's add (zkml/src/lookup/logup_gkr/structs.rs:48-58).
#pragma once
#include "family.cuh"

namespace dpb {

constexpr int kMaxLogupCols = 8;

template <class F>
struct LogupCols {
    const void* col[kMaxLogupCols];
    int32_t dtype[kMaxLogupCols];
    typename F::E sep_pow[kMaxLogupCols];  // sep^j, j = 0..
    typename F::E constant;
    uint32_t n_cols;
};

template <class F>
__device__ __forceinline__ typename F::E logup_denominator(const LogupCols<F>& c, uint64_t i) {
    typename F::E d = c.constant;
    for (uint32_t j = 0; j < c.n_cols; j++) {
        const typename F::E v = F::load(c.col[j], c.dtype[j], i);
        // sep^0 = 1: the first column is added as is (circuit.rs:162-171)
        d = F::add(d, j == 0 ? v : F::mul(c.sep_pow[j], v));
    }
    return d;
}

// First level of a lookup instance: numerators are all -1
// (circuit.rs:151-182).
template <class F>
__global__ void logup_initial_lookup(LogupCols<F> c, uint64_t half, typename F::E* __restrict__ num,
                                     typename F::E* __restrict__ den) {
    typedef typename F::E E;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < half; i += stride) {
        const E d1 = logup_denominator<F>(c, i);
        const E d2 = logup_denominator<F>(c, i + half);
        F::store(num, i, F::neg(F::add(d1, d2)));
        F::store(den, i, F::mul(d1, d2));
    }
}

// First level of a table instance: numerators are the multiplicities
// (circuit.rs:117-150).
template <class F>
__global__ void logup_initial_table(LogupCols<F> c, const void* __restrict__ mult, int mult_dtype,
                                    uint64_t half, typename F::E* __restrict__ num,
                                    typename F::E* __restrict__ den) {
    typedef typename F::E E;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < half; i += stride) {
        const E d1 = logup_denominator<F>(c, i);
        const E d2 = logup_denominator<F>(c, i + half);
        const E n1 = F::load(mult, mult_dtype, i);
        const E n2 = F::load(mult, mult_dtype, i + half);
        F::store(num, i, F::add(F::mul(n1, d2), F::mul(d1, n2)));
        F::store(den, i, F::mul(d1, d2));
    }
}

// Every later level (circuit.rs:97-116).
template <class F>
__global__ void logup_next_level(const typename F::E* __restrict__ num_in,
                                 const typename F::E* __restrict__ den_in, uint64_t half,
                                 typename F::E* __restrict__ num, typename F::E* __restrict__ den) {
    typedef typename F::E E;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < half; i += stride) {
        const E n1 = F::load(num_in, F::kChalDtype, i), n2 = F::load(num_in, F::kChalDtype, i + half);
        const E d1 = F::load(den_in, F::kChalDtype, i), d2 = F::load(den_in, F::kChalDtype, i + half);
        F::store(num, i, F::add(F::mul(n1, d2), F::mul(d1, n2)));
        F::store(den, i, F::mul(d1, d2));
    }
}

// The last levels of a tree in one block: level after level from `half` entries down to 2, each level's
// numerators and denominators stored right behind the previous level's (the tree's layout).  Launched once the
// levels are small enough that a launch per level costs more than the level.
template <class F>
__global__ void __launch_bounds__(kThreads)
    logup_small_levels(const typename F::E* num_in, const typename F::E* den_in, uint64_t half, typename F::E* num) {
    typedef typename F::E E;
    for (; half >= 2; half >>= 1) {
        E* den = num + half;
        for (uint64_t i = threadIdx.x; i < half; i += blockDim.x) {
            const E n1 = F::load(num_in, F::kChalDtype, i), n2 = F::load(num_in, F::kChalDtype, i + half);
            const E d1 = F::load(den_in, F::kChalDtype, i), d2 = F::load(den_in, F::kChalDtype, i + half);
            F::store(num, i, F::add(F::mul(n1, d2), F::mul(d1, n2)));
            F::store(den, i, F::mul(d1, d2));
        }
        __syncthreads();  // this level is complete (and visible to the block) before the next one reads it
        num_in = num;
        den_in = den;
        num = den + half;
    }
}

}  // namespace dpb
