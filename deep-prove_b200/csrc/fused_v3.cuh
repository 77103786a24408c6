// Asynchronous staging of table entries for the fused Goldilocks rounds
// (fused_v4.cuh).  How table entries reach the registers: every thread streams the 16-byte chunks of its NEXT
// items from global to shared memory with cp.async while it works on the
// current item, so the integer pipes do not idle on HBM latency and the data in
// flight costs no registers.  Each thread only ever reads back the chunks it
// copied itself (chunk c of thread t lives at [c][t], stride 16 B across the
// warp: conflict-free 128-bit shared loads), so no block-wide barrier is
// needed: cp.async.wait_group orders a thread's own copies.
#pragma once
#include <type_traits>

#include "fused_v2.cuh"

namespace dpb {

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int kStageThreads = 256;

// Per-thread staging ring: STAGES slots of K tables x CH chunks of 16 bytes.
template <int K, int CH, int STAGES>
struct Stager {
    uint4* base;  // this block's shared memory
    __device__ __forceinline__ uint4* slot(int s, int j, int c) const {
        return base + (((size_t)s * K + j) * CH + c) * kStageThreads + threadIdx.x;
    }
    // item `p` of every table: CH consecutive chunks starting at chunk p * CH
    __device__ __forceinline__ void issue(int s, const void* const (&in)[K], uint64_t p, bool valid) const {
        if (valid) {
#pragma unroll
            for (int j = 0; j < K; j++) {
                const uint4* g = (const uint4*)in[j] + p * CH;
#pragma unroll
                for (int c = 0; c < CH; c++) cp_async16(slot(s, j, c), g + c);
            }
        }
        cp_async_commit();  // an empty group keeps the group count uniform
    }
    __device__ __forceinline__ uint4 get(int s, int j, int c) const { return *slot(s, j, c); }
    static constexpr size_t bytes() { return (size_t)STAGES * K * CH * kStageThreads * sizeof(uint4); }
};

}  // namespace dpb
