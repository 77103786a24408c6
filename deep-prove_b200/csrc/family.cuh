// Field "families" the kernels are templated on.
//
// A family fixes the challenge/working element type E and how a table entry of
// a given storage layout is widened to E when it is loaded:
//   GlFam : E = Goldilocks quadratic extension (16 B); tables may hold base
//           elements (8 B) or extension elements (16 B).
//   FrFam : E = BN254 Fr in Montgomery form (32 B); tables hold E.
#pragma once
#include "../../include/dpb.h"
#include "field_bn254.cuh"
#include "field_gl.cuh"
#if defined(__CUDACC__)
#include "gl_words.cuh"
#endif

namespace dpb {

#if defined(__CUDACC__)
// canonical extension elements to and from the word-level form of gl_words.cuh
__device__ __forceinline__ glw::W2 gl2_words(const Gl2& a) {
    glw::W2 r;
    r.c0 = glw::make_w((uint32_t)a.c0, (uint32_t)(a.c0 >> 32));
    r.c1 = glw::make_w((uint32_t)a.c1, (uint32_t)(a.c1 >> 32));
    return r;
}
__device__ __forceinline__ Gl2 gl2_canonical(const glw::W2& a) {
    return gl2_make(glw::to_u64(glw::canon(a.c0)), glw::to_u64(glw::canon(a.c1)));
}
#endif

struct GlFam {
    typedef Gl2 E;
    static constexpr int kChalDtype = DPB_GL_EXT;
    DPB_HD static E zero() { return gl2_zero(); }
    DPB_HD static E one() { return gl2_one(); }
    // on the device the operations run on the word-level arithmetic; results are canonical either way
    DPB_HD static E add(const E& a, const E& b) {
#if defined(__CUDA_ARCH__)
        return gl2_canonical(glw::add_c(gl2_words(a), gl2_words(b)));
#else
        return gl2_add(a, b);
#endif
    }
    DPB_HD static E sub(const E& a, const E& b) {
#if defined(__CUDA_ARCH__)
        return gl2_canonical(glw::sub_c(gl2_words(a), gl2_words(b)));
#else
        return gl2_sub(a, b);
#endif
    }
    DPB_HD static E mul(const E& a, const E& b) {
#if defined(__CUDA_ARCH__)
        return gl2_canonical(glw::mul(gl2_words(a), gl2_words(b)));
#else
        return gl2_mul(a, b);
#endif
    }
    DPB_HD static E neg(const E& a) { return gl2_neg(a); }
    DPB_HD static bool is_one(const E& a) { return a.c0 == 1 && a.c1 == 0; }
    DPB_HD static bool is_zero(const E& a) { return a.c0 == 0 && a.c1 == 0; }
    DPB_HD static E from_u64(uint64_t x) { return gl2_make(x % GL_P, 0); }
    static E inv(const E& a) { return gl2_inv(a); }
    DPB_HD static size_t elem_size(int dtype) { return dtype == DPB_GL_BASE ? 8 : 16; }
#if defined(__CUDACC__)
    // What a launch needs to multiply many values by one challenge (the fold of a round).
    typedef Gl2 FoldKey;
    static FoldKey fold_key(const E& r) { return r; }
    __device__ __forceinline__ static E mul_key(const FoldKey& k, const E& a) { return mul(k, a); }
    // the same key, made by the threads of a block into *out (shared memory); the caller synchronises
    __device__ __forceinline__ static void fold_key_block(const E& r, FoldKey* out) {
        if (threadIdx.x == 0) *out = r;
    }
    // a signed integer as a canonical base element: negative x -> p - |x|
    __device__ __forceinline__ static uint64_t base_from_int(int64_t x) {
        return x < 0 ? GL_P - ((uint64_t)0 - (uint64_t)x) % GL_P : (uint64_t)x % GL_P;
    }
    __device__ __forceinline__ static E load(const void* p, int dtype, uint64_t i) {
        if (dtype == DPB_GL_BASE) return gl2_from_base(((const uint64_t*)p)[i]);
        if (dtype == DPB_GL_EXT) {
            const ulonglong2 v = ((const ulonglong2*)p)[i];
            return gl2_make(v.x, v.y);
        }
        if (dtype == DPB_GL_I32) return gl2_from_base(base_from_int(((const int32_t*)p)[i]));
        return gl2_from_base(base_from_int(((const int64_t*)p)[i]));
    }
    // entries 2i and 2i+1
    __device__ __forceinline__ static void load_pair(const void* p, int dtype, uint64_t i, E& a,
                                                     E& b) {
        if (dtype == DPB_GL_BASE) {
            const ulonglong2 v = ((const ulonglong2*)p)[i];
            a = gl2_from_base(v.x);
            b = gl2_from_base(v.y);
        } else if (dtype == DPB_GL_EXT) {
            const ulonglong2 v0 = ((const ulonglong2*)p)[2 * i];
            const ulonglong2 v1 = ((const ulonglong2*)p)[2 * i + 1];
            a = gl2_make(v0.x, v0.y);
            b = gl2_make(v1.x, v1.y);
        } else if (dtype == DPB_GL_I64) {
            const longlong2 v = ((const longlong2*)p)[i];
            a = gl2_from_base(base_from_int(v.x));
            b = gl2_from_base(base_from_int(v.y));
        } else {
            const int2 v = ((const int2*)p)[i];
            a = gl2_from_base(base_from_int(v.x));
            b = gl2_from_base(base_from_int(v.y));
        }
    }
    __device__ __forceinline__ static void store(void* p, uint64_t i, const E& v) {
        ((ulonglong2*)p)[i] = make_ulonglong2(v.c0, v.c1);
    }
    __device__ __forceinline__ static E shfl_down(const E& v, int off) {
        E r;
        r.c0 = __shfl_down_sync(0xffffffffu, (unsigned long long)v.c0, off);
        r.c1 = __shfl_down_sync(0xffffffffu, (unsigned long long)v.c1, off);
        return r;
    }
#endif
};

struct FrFam {
    typedef Fr E;
    static constexpr int kChalDtype = DPB_FR;
    DPB_HD static E zero() { return fr_zero(); }
    DPB_HD static E one() { return fr_one(); }
    DPB_HD static E add(const E& a, const E& b) { return fr_add(a, b); }
    DPB_HD static E sub(const E& a, const E& b) { return fr_sub(a, b); }
    DPB_HD static E mul(const E& a, const E& b) { return fr_mul(a, b); }
    DPB_HD static E neg(const E& a) { return fr_neg(a); }
    DPB_HD static bool is_one(const E& a) { return fr_eq(a, fr_one()); }
    DPB_HD static bool is_zero(const E& a) { return fr_is_zero(a); }
    DPB_HD static E from_u64(uint64_t x) { return fr_from_u64(x); }
    static E inv(const E& a) { return fr_inv(a); }
    DPB_HD static size_t elem_size(int) { return 32; }
#if defined(__CUDACC__)
    // The challenge as the eight precomputed rows of frw::mul_fixed: 80 wide multiply-adds per product instead of 128.
    typedef frw::FixedMul FoldKey;
    static FoldKey fold_key(const E& r) {
        FoldKey k;
        fr_fixed_table(r, k);
        return k;
    }
    __device__ __forceinline__ static E mul_key(const FoldKey& k, const E& a) { return fr_mul_fixed(k, a); }
    __device__ __forceinline__ static void fold_key_block(const E& r, FoldKey* out) {
        if (threadIdx.x < 8) fr_fixed_row(r, (int)threadIdx.x, out->c[threadIdx.x]);
    }
    __device__ __forceinline__ static E load(const void* p, int dtype, uint64_t i) {
        if (dtype == DPB_FR_I64) return fr_from_int_rows(((const int64_t*)p)[i]);
        if (dtype == DPB_FR_I32) return fr_from_int_rows((int64_t)((const int32_t*)p)[i]);
        const ulonglong2* q = (const ulonglong2*)p + 2 * i;
        const ulonglong2 a = q[0], b = q[1];
        E r;
        r.l[0] = a.x;
        r.l[1] = a.y;
        r.l[2] = b.x;
        r.l[3] = b.y;
        return r;
    }
    __device__ __forceinline__ static void load_pair(const void* p, int dtype, uint64_t i, E& a,
                                                     E& b) {
        a = load(p, dtype, 2 * i);
        b = load(p, dtype, 2 * i + 1);
    }
    __device__ __forceinline__ static void store(void* p, uint64_t i, const E& v) {
        ulonglong2* q = (ulonglong2*)p + 2 * i;
        q[0] = make_ulonglong2(v.l[0], v.l[1]);
        q[1] = make_ulonglong2(v.l[2], v.l[3]);
    }
    __device__ __forceinline__ static E shfl_down(const E& v, int off) {
        E r;
#pragma unroll
        for (int j = 0; j < 4; j++)
            r.l[j] = __shfl_down_sync(0xffffffffu, (unsigned long long)v.l[j], off);
        return r;
    }
#endif
};

}  // namespace dpb
