// Issue-rate probes: how many field products per second the integer pipes of
// this GPU deliver when nothing else (memory, reductions, host turn-arounds)
// is in the way.  The sumcheck kernels over BN254 are bound by these rates and
// not by HBM, so their roofline is quoted against what this file measures on
// the device the benchmark runs on.
//
// Each probe kernel runs chains of the SAME device functions the round kernels
// use (frw::mul, frw::mul_fixed, glw::acc_mac, glw::mul) on register operands:
// every thread advances kChains independent chains for `iters` steps, blocks
// fill every SM with the occupancy the round kernels have, and the result is
// stored so the work cannot be dropped.  A product's cost here is a lower
// bound on its cost inside a round kernel.
#include "common.cuh"
#include "field_bn254.cuh"
#include "gl_words.cuh"

namespace dpb {

constexpr int kProbeThreads = 256;
constexpr int kChains = 2;

__device__ __forceinline__ uint32_t probe_seed(uint32_t salt) {
    uint32_t x = (blockIdx.x * blockDim.x + threadIdx.x) * 0x9E3779B9u + salt * 0x85EBCA6Bu + 1u;
    x ^= x >> 15;
    x *= 0x2C1B3C6Du;
    x ^= x >> 12;
    return x;
}

// kind 0: 32x32->64 multiply-adds into a 64-bit accumulator (mad.lo.cc + madc.hi on one aligned word pair, the
// form every product routine here is built from); eight independent accumulators per thread
__global__ void __launch_bounds__(kProbeThreads) probe_wide_mad(uint32_t iters, uint32_t* out) {
    uint32_t lo[8], hi[8], a[8];
    const uint32_t m = probe_seed(7) | 1u;
#pragma unroll
    for (int c = 0; c < 8; c++) {
        lo[c] = probe_seed(c);
        hi[c] = probe_seed(c + 8);
        a[c] = probe_seed(c + 16);
    }
    for (uint32_t it = 0; it < iters; it++) {
#pragma unroll
        for (int c = 0; c < 8; c++)
            asm volatile("mad.lo.cc.u32 %0, %2, %3, %0; madc.hi.u32 %1, %2, %3, %1;"
                         : "+r"(lo[c]), "+r"(hi[c])
                         : "r"(a[c]), "r"(m));
    }
    uint32_t x = 0;
#pragma unroll
    for (int c = 0; c < 8; c++) x ^= lo[c] ^ hi[c];
    out[blockIdx.x * blockDim.x + threadIdx.x] = x;
}

// kind 1: BN254 Montgomery products; kind 2: products by a per-launch constant (precomputed rows)
template <bool FIXED>
__global__ void __launch_bounds__(kProbeThreads, 2) probe_fr(frw::FixedMul k, uint32_t iters, uint32_t* out) {
    frw::F8 a[kChains], b;
#pragma unroll
    for (int c = 0; c < kChains; c++) {
#pragma unroll
        for (int j = 0; j < 8; j++) a[c].w[j] = probe_seed(8 * c + j);
        a[c].w[7] &= 0x0fffffffu;  // below the modulus
    }
#pragma unroll
    for (int j = 0; j < 8; j++) b.w[j] = k.c[0][j];
    b.w[7] &= 0x0fffffffu;
    for (uint32_t it = 0; it < iters; it++) {
#pragma unroll
        for (int c = 0; c < kChains; c++) a[c] = FIXED ? frw::mul_fixed(a[c], k) : frw::mul(a[c], b);
    }
    uint32_t x = 0;
#pragma unroll
    for (int c = 0; c < kChains; c++)
#pragma unroll
        for (int j = 0; j < 8; j++) x ^= a[c].w[j];
    out[blockIdx.x * blockDim.x + threadIdx.x] = x;
}

// kind 3: Goldilocks lazy multiply-accumulates (four wide multiply-adds each);
// kind 4: full Goldilocks products (multiply and reduce)
template <bool FULL>
__global__ void __launch_bounds__(kProbeThreads, 2) probe_gl(uint32_t iters, uint32_t* out) {
    glw::W a[4], b[4];
    glw::A8 acc[4];
#pragma unroll
    for (int c = 0; c < 4; c++) {
        a[c] = glw::make_w(probe_seed(c), probe_seed(c + 4) & 0x7fffffffu);
        b[c] = glw::make_w(probe_seed(c + 8), probe_seed(c + 12) & 0x7fffffffu);
        acc[c] = glw::acc_zero();
    }
    for (uint32_t it = 0; it < iters; it++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            if (FULL) a[c] = glw::mul(a[c], b[c]);
            else {
                glw::acc_mac(acc[c], a[c], b[c]);
                a[c].lo ^= acc[c].e0;  // the next product depends on this one
            }
        }
    }
    uint32_t x = 0;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const glw::W r = glw::acc_reduce(acc[c]);
        x ^= a[c].lo ^ a[c].hi ^ r.lo ^ r.hi;
    }
    out[blockIdx.x * blockDim.x + threadIdx.x] = x;
}

}  // namespace dpb

using namespace dpb;

extern "C" int dpb_issue_rate_probe(dpb_ctx* ctx, int kind, uint32_t iters, double* ops_per_second, double* elapsed_ms) {
    if (!ctx || !ops_per_second) return fail(DPB_EINVAL, "null argument");
    if (kind < 0 || kind > 4) return fail(DPB_EINVAL, "unknown probe kind %d", kind);
    if (iters < 1 || iters > (1u << 20)) return fail(DPB_EINVAL, "iters %u outside 1..2^20", iters);
    const uint32_t blocks = (uint32_t)ctx->sm_count * 4;
    uint32_t* out = nullptr;
    DPB_TRY(device_alloc(ctx, (size_t)blocks * kProbeThreads * sizeof(uint32_t), (void**)&out));
    frw::FixedMul k;
    {
        Fr c;
        c.l[0] = 0x123456789abcdef1ull;
        c.l[1] = 0xfedcba9876543210ull;
        c.l[2] = 0x0f1e2d3c4b5a6978ull;
        c.l[3] = 0x1122334455667788ull;
        fr_fixed_table(c, k);
    }
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t err = cudaEventCreate(&e0);
    if (err == cudaSuccess) err = cudaEventCreate(&e1);
    double per_thread = 0;
    float ms = 0.f;
    for (int pass = 0; pass < 2 && err == cudaSuccess; pass++) {  // the first pass warms up
        if (pass == 1) err = cudaEventRecord(e0, ctx->stream);
        switch (kind) {
            case 0: probe_wide_mad<<<blocks, kProbeThreads, 0, ctx->stream>>>(iters, out); per_thread = 8.0; break;
            case 1: probe_fr<false><<<blocks, kProbeThreads, 0, ctx->stream>>>(k, iters, out); per_thread = kChains; break;
            case 2: probe_fr<true><<<blocks, kProbeThreads, 0, ctx->stream>>>(k, iters, out); per_thread = kChains; break;
            case 3: probe_gl<false><<<blocks, kProbeThreads, 0, ctx->stream>>>(iters, out); per_thread = 4.0; break;
            default: probe_gl<true><<<blocks, kProbeThreads, 0, ctx->stream>>>(iters, out); per_thread = 4.0; break;
        }
        if (err == cudaSuccess) err = cudaGetLastError();
    }
    if (err == cudaSuccess) err = cudaEventRecord(e1, ctx->stream);
    if (err == cudaSuccess) err = cudaEventSynchronize(e1);
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    device_free(ctx, out);
    if (err != cudaSuccess) return fail(DPB_ECUDA, "issue-rate probe: %s", cudaGetErrorString(err));
    *ops_per_second = (double)blocks * kProbeThreads * per_thread * iters / (ms * 1e-3);
    if (elapsed_ms) *elapsed_ms = ms;
    return DPB_OK;
}
