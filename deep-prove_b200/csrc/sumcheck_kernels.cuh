// Sumcheck prover kernels: per-round evaluation of product terms over the
// remaining hypercube, and the fold that binds one variable.
//
// Round i of a sumcheck over n variables sees every table with n-i variables;
// entries 2p and 2p+1 differ in the variable being bound.  The round
// polynomial is returned as its evaluations at 0..=D.
#pragma once
#include "family.cuh"

namespace dpb {

// One registered table as a round sees it.
struct MleDesc {
    const void* ptr;
    int32_t dtype;   // storage layout of `ptr`
    int32_t shift;   // < 0: table has all remaining variables (entries 2p, 2p+1);
                     // >= 0: table is constant in this round, entry p >> shift
    uint64_t limit;  // entries the table really holds; entries from `limit` on read as zero
                     // (zero-padded tables); kNoLimit for every other table
};
constexpr uint64_t kNoLimit = ~0ull;

struct FoldDesc {
    const void* in;
    void* out;
    int32_t dtype_in;
    uint32_t pad;
    uint64_t n_out;
    uint64_t limit_in;  // entries `in` really holds (kNoLimit: all)
};

// entries 2p and 2p+1 of a table that reads as zero from `limit` on
template <class F>
__device__ __forceinline__ void load_pair_limited(const void* ptr, int dtype, uint64_t limit, uint64_t p,
                                                  typename F::E& a, typename F::E& b) {
    if (2 * p + 1 < limit) {
        F::load_pair(ptr, dtype, p, a, b);
    } else if (2 * p < limit) {
        a = F::load(ptr, dtype, 2 * p);
        b = F::zero();
    } else {
        a = F::zero();
        b = F::zero();
    }
}

template <class F>
struct TermDev {
    typename F::E coeff;
    uint32_t n_factors;
    uint32_t coeff_is_one;
    uint16_t idx[DPB_MAX_FACTORS];
};

// Scratch a round reduction needs: per-block partial sums and a ticket counter.
template <class F>
struct ReduceScratch {
    typename F::E* partials;  // [max_blocks][NACC]
    unsigned int* counter;    // zero between launches
    // Where the host polls for the result (mapped host memory), or nullptr.  The sums are then written there
    // instead of to `out`, as 16-byte chunks {8 bytes of data, done_value, pad}: a chunk arrives as one
    // transaction, so a host that sees done_value in every chunk of an element has the element, and the kernel
    // needs no system-wide fence (each costs more than a microsecond).
    void* chunk_out;
    unsigned int done_value;
};

// 16 bytes that travel as one transaction: 8 bytes of data and the sequence number that says which message
struct TailChunk {
    uint64_t data;
    uint32_t seq;
    uint32_t pad;
};
__device__ __forceinline__ void chunk_store(TailChunk* c, uint64_t data, uint32_t seq) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(c), "r"((uint32_t)data),
                 "r"((uint32_t)(data >> 32)), "r"(seq), "r"(0u)
                 : "memory");
}
// an element as chunks with one sequence number
template <class E>
__device__ __forceinline__ void chunks_store(TailChunk* c, const E& v, uint32_t seq) {
    const uint64_t* w = (const uint64_t*)&v;
#pragma unroll
    for (int i = 0; i < (int)(sizeof(E) / 8); i++) chunk_store(c + i, w[i], seq);
}

// the NACC sums of a launch go to the host's chunk area, or to `out`
template <class F, int NACC>
__device__ __forceinline__ void emit_result(const typename F::E (&v)[NACC], const ReduceScratch<F>& rs,
                                            typename F::E* out) {
    typedef typename F::E E;
    if (rs.chunk_out) {
#pragma unroll
        for (int i = 0; i < NACC; i++) chunks_store<E>((TailChunk*)rs.chunk_out + i * (sizeof(E) / 8), v[i], rs.done_value);
    } else {
#pragma unroll
        for (int i = 0; i < NACC; i++) out[i] = v[i];
    }
}

constexpr int kThreads = 256;
constexpr int kMaxWarps = kThreads / 32;

// Sums acc[] over the block; thread 0 ends up holding the totals.
template <class F, int NACC>
__device__ __forceinline__ void block_sum(typename F::E (&acc)[NACC]) {
    typedef typename F::E E;
    __shared__ E sm[NACC][kMaxWarps];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int i = 0; i < NACC; i++) acc[i] = F::add(acc[i], F::shfl_down(acc[i], off));
    }
    __syncthreads();  // protects sm[] when block_sum is called twice
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < NACC; i++) sm[i][warp] = acc[i];
    }
    __syncthreads();
    if (warp == 0) {
        const int nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
        for (int i = 0; i < NACC; i++) acc[i] = lane < nwarps ? sm[i][lane] : F::zero();
#pragma unroll
        for (int off = kMaxWarps / 2; off > 0; off >>= 1) {
#pragma unroll
            for (int i = 0; i < NACC; i++) acc[i] = F::add(acc[i], F::shfl_down(acc[i], off));
        }
    }
}

// Grid-wide sum of per-thread accumulators.  Every block publishes its partial
// sums; the block that draws the last ticket adds them up and writes NACC
// elements to `out` (device memory or mapped host memory).  The counter is
// left at zero for the next launch.
template <class F, int NACC>
__device__ __forceinline__ void grid_sum_publish(typename F::E (&acc)[NACC], ReduceScratch<F> rs,
                                                 typename F::E* out) {
    typedef typename F::E E;
    __shared__ bool is_last;
    block_sum<F, NACC>(acc);
    if (gridDim.x == 1) {
        if (threadIdx.x == 0) emit_result<F, NACC>(acc, rs, out);
        return;
    }
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < NACC; i++) rs.partials[(size_t)blockIdx.x * NACC + i] = acc[i];
        __threadfence();
        const unsigned int t = atomicAdd(rs.counter, 1u);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    E tot[NACC];
#pragma unroll
    for (int i = 0; i < NACC; i++) tot[i] = F::zero();
    const volatile uint64_t* pw = (const volatile uint64_t*)rs.partials;
    constexpr int W = sizeof(E) / 8;
    for (unsigned int b = threadIdx.x; b < gridDim.x; b += blockDim.x) {
#pragma unroll
        for (int i = 0; i < NACC; i++) {
            E v;
            uint64_t* vw = (uint64_t*)&v;
#pragma unroll
            for (int w = 0; w < W; w++) vw[w] = pw[((size_t)b * NACC + i) * W + w];
            tot[i] = F::add(tot[i], v);
        }
    }
    block_sum<F, NACC>(tot);
    if (threadIdx.x == 0) {
        emit_result<F, NACC>(tot, rs, out);
        *rs.counter = 0;
    }
}

// Generic round evaluation: any list of product terms over any tables.
// acc[x] = sum_p sum_t coeff_t * prod_j f_tj(x; p),  f(x; p) = f[2p] + x (f[2p+1] - f[2p]).
// Work items are (pair, slice): slice s of n_slices takes the terms s, s + n_slices, ..  A round with few pairs
// and many terms (a batch of many logup instances late in a sumcheck) is spread over the terms as well, instead
// of leaving one thread per pair to walk the whole list.
template <class F, int D>
__global__ void __launch_bounds__(kThreads)
    sc_eval_generic(const MleDesc* __restrict__ mles, const TermDev<F>* __restrict__ terms,
                    uint32_t n_terms, uint64_t n_pairs, uint32_t n_slices, ReduceScratch<F> rs,
                    typename F::E* out) {
    typedef typename F::E E;
    E acc[D + 1];
#pragma unroll
    for (int x = 0; x <= D; x++) acc[x] = F::zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t n_items = n_pairs * n_slices;
    for (uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; w < n_items; w += stride) {
        const uint64_t p = w % n_pairs;
        for (uint32_t t = (uint32_t)(w / n_pairs); t < n_terms; t += n_slices) {
            const TermDev<F>& tm = terms[t];
            E prod[D + 1];
            const uint32_t nf = tm.n_factors;
            for (uint32_t j = 0; j < nf; j++) {
                const MleDesc md = mles[tm.idx[j]];
                E f0, f1;
                if (md.shift < 0) {
                    load_pair_limited<F>(md.ptr, md.dtype, md.limit, p, f0, f1);
                } else {
                    f0 = F::load(md.ptr, md.dtype, p >> md.shift);
                    f1 = f0;
                }
                if (j == 0 && !tm.coeff_is_one) {
                    f0 = F::mul(f0, tm.coeff);
                    f1 = F::mul(f1, tm.coeff);
                }
                const E delta = F::sub(f1, f0);
                E val = f0;
#pragma unroll
                for (int x = 0; x <= D; x++) {
                    prod[x] = (j == 0) ? val : F::mul(prod[x], val);
                    if (x < D) val = F::add(val, delta);
                }
            }
            if (nf == 0) {
                // constant term: contributes coeff once per point of the pair (x-independent)
#pragma unroll
                for (int x = 0; x <= D; x++) acc[x] = F::add(acc[x], tm.coeff);
            } else {
#pragma unroll
                for (int x = 0; x <= D; x++) acc[x] = F::add(acc[x], prod[x]);
            }
        }
    }
    grid_sum_publish<F, D + 1>(acc, rs, out);
}

// Round evaluation when tables are zero-padded: a term is zero wherever one of
// its padded factors is, so each term is evaluated only over the pairs where all
// of them hold data (`term_pairs[t]`).  Work is cut into tiles of one block's
// width; `tile_prefix[t]` is the first tile of term t (n_terms + 1 entries), and a
// block finds the term of a tile by binary search.
template <class F, int D>
__global__ void __launch_bounds__(kThreads)
    sc_eval_ranged(const MleDesc* __restrict__ mles, const TermDev<F>* __restrict__ terms, uint32_t n_terms,
                   const uint64_t* __restrict__ tile_prefix_g, const uint64_t* __restrict__ term_pairs,
                   uint32_t prefix_in_smem, ReduceScratch<F> rs, typename F::E* out) {
    typedef typename F::E E;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint64_t* tile_prefix = tile_prefix_g;
    if (prefix_in_smem) {  // the search below runs per tile: keep its table on chip when it fits
        uint64_t* sp = (uint64_t*)smem_raw;
        for (uint32_t i = threadIdx.x; i <= n_terms; i += blockDim.x) sp[i] = tile_prefix_g[i];
        __syncthreads();
        tile_prefix = sp;
    }
    E acc[D + 1];
#pragma unroll
    for (int x = 0; x <= D; x++) acc[x] = F::zero();
    const uint64_t total_tiles = tile_prefix[n_terms];
    for (uint64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        uint32_t lo = 0, hi = n_terms;  // the term t with tile_prefix[t] <= tile < tile_prefix[t + 1]
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (tile_prefix[mid] <= tile) lo = mid;
            else hi = mid;
        }
        const uint32_t t = lo;
        const uint64_t p = (tile - tile_prefix[t]) * kThreads + threadIdx.x;
        if (p >= term_pairs[t]) continue;
        const TermDev<F>& tm = terms[t];
        const uint32_t nf = tm.n_factors;
        E prod[D + 1];
        for (uint32_t j = 0; j < nf; j++) {
            const MleDesc md = mles[tm.idx[j]];
            E f0, f1;
            if (md.shift < 0) {
                load_pair_limited<F>(md.ptr, md.dtype, md.limit, p, f0, f1);
            } else {
                f0 = F::load(md.ptr, md.dtype, p >> md.shift);
                f1 = f0;
            }
            if (j == 0 && !tm.coeff_is_one) {
                f0 = F::mul(f0, tm.coeff);
                f1 = F::mul(f1, tm.coeff);
            }
            const E delta = F::sub(f1, f0);
            E val = f0;
#pragma unroll
            for (int x = 0; x <= D; x++) {
                prod[x] = (j == 0) ? val : F::mul(prod[x], val);
                if (x < D) val = F::add(val, delta);
            }
        }
        if (nf == 0) {
#pragma unroll
            for (int x = 0; x <= D; x++) acc[x] = F::add(acc[x], tm.coeff);
        } else {
#pragma unroll
            for (int x = 0; x <= D; x++) acc[x] = F::add(acc[x], prod[x]);
        }
    }
    grid_sum_publish<F, D + 1>(acc, rs, out);
}

// Binds the lowest remaining variable of several tables in one launch:
// out[p] = in[2p] + r * (in[2p+1] - in[2p]).   blockIdx.y selects the table.
template <class F>
__global__ void __launch_bounds__(kThreads)
    sc_fold_generic(const FoldDesc* __restrict__ descs, typename F::FoldKey rk) {
    typedef typename F::E E;
    const FoldDesc d = descs[blockIdx.y];
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < d.n_out; p += stride) {
        E f0, f1;
        load_pair_limited<F>(d.in, d.dtype_in, d.limit_in, p, f0, f1);
        F::store(d.out, p, F::add(f0, F::mul_key(rk, F::sub(f1, f0))));
    }
}

// Last step of a sumcheck: every table has two entries left; bind the final
// variable and collect one value per table.
template <class F>
__global__ void sc_final_evals(const MleDesc* __restrict__ mles, uint32_t k, typename F::E r,
                               typename F::E* out) {
    typedef typename F::E E;
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= k) return;
    const MleDesc md = mles[j];
    E f0, f1;
    load_pair_limited<F>(md.ptr, md.dtype, md.limit, 0, f0, f1);
    out[j] = F::add(f0, F::mul(r, F::sub(f1, f0)));
    if (j == 0) __threadfence_system();
}

}  // namespace dpb
