// Partial evaluation (fix_high / fix_low): one pass binds up to five variables,
// out[j] = sum_l w[l] * in[index(j, l)] with the 2^g eq weights of those
// variables.  One thread per output entry runs the whole sum, so nothing is
// exchanged between threads, and because the weights are fixed for the launch
// the products take the cheap forms: Goldilocks accumulates the 128-bit
// products lazily and reduces once per output; BN254 multiplies through the
// precomputed rows of frw::mul_fixed.
#pragma once
#include "family.cuh"
#include "gl_words.cuh"
#include "sumcheck_kernels.cuh"

namespace dpb {

template <class F>
struct WSum;

template <>
struct WSum<GlFam> {
    struct Key {
        glw::W c0, c1, c1x7;  // the weight c0 + c1 X, and 7 c1
    };
    struct Acc {
        glw::A8 s0, s1;
    };
    // the block's threads fill keys[0..n) from the weights; the caller synchronises
    __device__ __forceinline__ static void make_keys_block(const Gl2* __restrict__ w, uint32_t n, Key* keys) {
        if (threadIdx.x < n) {
            const Gl2 v = w[threadIdx.x];
            Key k;
            k.c0 = glw::make_w((uint32_t)v.c0, (uint32_t)(v.c0 >> 32));
            k.c1 = glw::make_w((uint32_t)v.c1, (uint32_t)(v.c1 >> 32));
            k.c1x7 = glw::mul7(k.c1);
            keys[threadIdx.x] = k;
        }
    }
    __device__ __forceinline__ static Acc zero() {
        Acc a;
        a.s0 = a.s1 = glw::acc_zero();
        return a;
    }
    // acc += key * entry i
    __device__ __forceinline__ static void mac(Acc& a, const Key& k, const void* __restrict__ in, int dtype, uint64_t i) {
        if (dtype == DPB_GL_BASE) {
            const uint64_t x = ((const uint64_t*)in)[i];
            const glw::W xw = glw::make_w((uint32_t)x, (uint32_t)(x >> 32));
            glw::acc_mac(a.s0, xw, k.c0);
            glw::acc_mac(a.s1, xw, k.c1);
        } else if (dtype == DPB_GL_EXT) {
            const uint4 v = ((const uint4*)in)[i];
            const glw::W x0 = glw::make_w(v.x, v.y), x1 = glw::make_w(v.z, v.w);
            glw::acc_mac(a.s0, x0, k.c0);
            glw::acc_mac(a.s0, x1, k.c1x7);
            glw::acc_mac(a.s1, x0, k.c1);
            glw::acc_mac(a.s1, x1, k.c0);
        } else {  // integer tables: the base element the integer stands for
            const uint64_t x = GlFam::load(in, dtype, i).c0;
            const glw::W xw = glw::make_w((uint32_t)x, (uint32_t)(x >> 32));
            glw::acc_mac(a.s0, xw, k.c0);
            glw::acc_mac(a.s1, xw, k.c1);
        }
    }
    // acc += key0 * entry i + key1 * entry i + 1 of a base table, i even: one 16-byte load
    __device__ __forceinline__ static void mac_base_pair(Acc& a, const Key& k0, const Key& k1, const void* __restrict__ in,
                                                         uint64_t i) {
        const uint4 v = ((const uint4*)in)[i >> 1];
        const glw::W x0 = glw::make_w(v.x, v.y), x1 = glw::make_w(v.z, v.w);
        glw::acc_mac(a.s0, x0, k0.c0);
        glw::acc_mac(a.s1, x0, k0.c1);
        glw::acc_mac(a.s0, x1, k1.c0);
        glw::acc_mac(a.s1, x1, k1.c1);
    }
    static constexpr bool kBasePairs = true;
    __device__ __forceinline__ static Gl2 finish(const Acc& a) {
        return gl2_make(glw::to_u64(glw::canon(glw::acc_reduce(a.s0))), glw::to_u64(glw::canon(glw::acc_reduce(a.s1))));
    }
};

template <>
struct WSum<FrFam> {
    typedef frw::FixedMul Key;
    typedef Fr Acc;
    __device__ __forceinline__ static void make_keys_block(const Fr* __restrict__ w, uint32_t n, Key* keys) {
        for (uint32_t t = threadIdx.x; t < 8 * n; t += blockDim.x) fr_fixed_row(w[t >> 3], (int)(t & 7), keys[t >> 3].c[t & 7]);
    }
    __device__ __forceinline__ static Acc zero() { return fr_zero(); }
    __device__ __forceinline__ static void mac(Acc& a, const Key& k, const void* __restrict__ in, int dtype, uint64_t i) {
        a = fr_add(a, fr_mul_fixed(k, FrFam::load(in, dtype, i)));
    }
    __device__ __forceinline__ static void mac_base_pair(Acc&, const Key&, const Key&, const void*, uint64_t) {}
    static constexpr bool kBasePairs = false;
    __device__ __forceinline__ static Fr finish(const Acc& a) { return a; }
};

// Bottom g variables (g <= 5): out[j] = sum_{l < 2^g} w[l] * in[j * 2^g + l].
template <class F>
__global__ void __launch_bounds__(kThreads)
    fix_low_sum(const void* __restrict__ in, int dtype_in, const typename F::E* __restrict__ w, uint32_t g,
                uint64_t n_out, typename F::E* __restrict__ out) {
    __shared__ typename WSum<F>::Key keys[32];
    const uint32_t G = 1u << g;
    WSum<F>::make_keys_block(w, G, keys);
    __syncthreads();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_out; j += stride) {
        typename WSum<F>::Acc acc = WSum<F>::zero();
        if (WSum<F>::kBasePairs && dtype_in == DPB_GL_BASE) {  // G >= 2 entries of 8 bytes, read two at a time
            for (uint32_t l = 0; l < G; l += 2) WSum<F>::mac_base_pair(acc, keys[l], keys[l + 1], in, (j << g) + l);
        } else {
            for (uint32_t l = 0; l < G; l++) WSum<F>::mac(acc, keys[l], in, dtype_in, (j << g) + l);
        }
        F::store(out, j, WSum<F>::finish(acc));
    }
}

// Top g variables: out[j] = sum_{h < 2^g} w[h] * in[h * n_out + j].
template <class F>
__global__ void __launch_bounds__(kThreads)
    fix_high_sum(const void* __restrict__ in, int dtype_in, const typename F::E* __restrict__ w, uint32_t g,
                 uint64_t n_out, typename F::E* __restrict__ out) {
    __shared__ typename WSum<F>::Key keys[32];
    const uint32_t H = 1u << g;
    WSum<F>::make_keys_block(w, H, keys);
    __syncthreads();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_out; j += stride) {
        typename WSum<F>::Acc acc = WSum<F>::zero();
        for (uint32_t h = 0; h < H; h++) WSum<F>::mac(acc, keys[h], in, dtype_in, (uint64_t)h * n_out + j);
        F::store(out, j, WSum<F>::finish(acc));
    }
}

}  // namespace dpb
