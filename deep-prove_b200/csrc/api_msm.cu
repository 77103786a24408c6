// C ABI: multi-scalar multiplication over BN254 G1, the arithmetic of the commitment scheme's commit
// (HyperKZG commits to a multilinear polynomial as sum_i evals[i] * G_i over the SRS's G1 points;
// CommittedPolynomial::batch_commit, zkml/src/poly_commit/context.rs:56-90, one MSM per chunk of at most 2^20
// evaluations).
//
// Bucket method (Pippenger) with windows of c bits:
//   1. msm_count      per scalar and window: which bucket it goes to (its c-bit digit; zero digits are skipped);
//                     a histogram of the (window, bucket) keys
//   2. msm_scan_*     exclusive prefix sums of the histogram: where every bucket's list starts
//   3. msm_scatter    the point indices, grouped by bucket
//   4. msm_buckets    one thread per bucket adds its points up (mixed Jacobian + affine additions); a bucket with
//                     more than 96 points (small integers crowd a wide window's low buckets) goes to a list that
//                     msm_heavy_plan / msm_heavy_chunks / msm_heavy_combine work off in chunks of 2048 points, one
//                     block per chunk
//   5. msm_reduce     per window sum_b b * B_b: a thread takes a run of 16 buckets (running sums from the top, plus
//                     the run's offset times its total), a block adds its 256 runs up in shared memory
//   6. host           the blocks' partial sums per window (a handful of points), the windows combined by c
//                     doublings each, one inversion for the affine result.
// Integer tables (DPB_FR_I32 / DPB_FR_I64) enter as magnitudes: a negative scalar adds the negated point, and only
// the one to four windows their bits reach are ever touched: committing to quantised tensors and 16-bit lookup
// columns costs a fraction of a commit to full-width scalars.
#include <vector>

#include "../../include/dpb_pcs.h"
#include "common.cuh"
#include "g1_bn254.cuh"

struct dpb_g1_bases {
    dpb_ctx* ctx = nullptr;
    uint64_t n = 0;
    dpb::G1Affine* dev = nullptr;
};

namespace dpb {

constexpr int kMsmRun = 16;         // buckets a reduction thread walks
constexpr int kMsmReduceThreads = 256;

struct MsmScalars {
    const void* ptr;
    int dtype;  // DPB_FR (Montgomery), DPB_FR_I32, DPB_FR_I64
};

// the scalar as a 256-bit magnitude (canonical integer below r) and a sign
__device__ __forceinline__ void msm_scalar(const MsmScalars& s, uint64_t i, uint64_t (&mag)[4], bool& neg) {
    neg = false;
    if (s.dtype == DPB_FR) {
        const Fr v = fr_from_mont(FrFam::load(s.ptr, DPB_FR, i));
        mag[0] = v.l[0];
        mag[1] = v.l[1];
        mag[2] = v.l[2];
        mag[3] = v.l[3];
        return;
    }
    const int64_t x = s.dtype == DPB_FR_I32 ? (int64_t)((const int32_t*)s.ptr)[i] : ((const int64_t*)s.ptr)[i];
    neg = x < 0;
    mag[0] = neg ? (uint64_t)0 - (uint64_t)x : (uint64_t)x;
    mag[1] = mag[2] = mag[3] = 0;
}
__device__ __forceinline__ uint32_t msm_digit(const uint64_t (&mag)[4], uint32_t w, uint32_t c) {
    const uint32_t bit = w * c, limb = bit >> 6, off = bit & 63;
    if (limb >= 4) return 0;
    uint64_t v = mag[limb] >> off;
    if (off + c > 64 && limb + 1 < 4) v |= mag[limb + 1] << (64 - off);
    return (uint32_t)(v & ((1ull << c) - 1));
}

// Lanes of a warp that hold the same key add their count with one atomic (a column of a few distinct values would
// otherwise send a million atomics to the same few counters).  Returns the lane's rank among them and, in every
// lane of the group, the value the leader's atomicAdd returned.
__device__ __forceinline__ uint32_t msm_group_add(uint32_t* counter, uint64_t key, bool take, unsigned active,
                                                  uint32_t& rank) {
    const unsigned peers = __match_any_sync(active, take ? key : ~0ull);
    const int leader = __ffs(peers) - 1;
    const unsigned lane = threadIdx.x & 31;
    rank = __popc(peers & ((1u << lane) - 1));
    uint32_t base = 0;
    if (take && (int)lane == leader) base = atomicAdd(counter, (uint32_t)__popc(peers));
    return __shfl_sync(peers, base, leader);
}

__global__ void __launch_bounds__(kThreads)
    msm_count(MsmScalars s, uint64_t n, uint32_t c, uint32_t windows, uint32_t* __restrict__ counts) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned active = __activemask();
        uint64_t mag[4];
        bool neg;
        msm_scalar(s, i, mag, neg);
        for (uint32_t w = 0; w < windows; w++) {
            const uint32_t d = msm_digit(mag, w, c);
            const size_t key = ((size_t)w << c) + d;
            uint32_t rank;
            msm_group_add(&counts[key], key, d != 0, active, rank);
        }
    }
}

// Exclusive scan of the histogram in three small launches: sums of tiles of 4096 counters, a scan of the tile sums
// by one block, and the scan inside every tile (all global accesses coalesced, the serial part in shared memory).
constexpr uint32_t kScanTile = 4096, kScanThreads = 256, kScanPer = kScanTile / kScanThreads;

__global__ void __launch_bounds__(kScanThreads)
    msm_scan_tile_sums(const uint32_t* __restrict__ counts, uint64_t n, uint32_t* __restrict__ tile_sums) {
    __shared__ uint32_t sh[kScanThreads];
    const uint64_t base = (uint64_t)blockIdx.x * kScanTile;
    uint32_t sum = 0;
    for (uint32_t j = 0; j < kScanPer; j++) {
        const uint64_t i = base + (uint64_t)j * kScanThreads + threadIdx.x;
        if (i < n) sum += counts[i];
    }
    sh[threadIdx.x] = sum;
    __syncthreads();
    for (uint32_t s = kScanThreads / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = sh[0];
}

// in place: tile_sums[t] becomes the sum of the tiles before t (n_tiles is at most a few thousand)
__global__ void __launch_bounds__(1024) msm_scan_tiles(uint32_t* __restrict__ tile_sums, uint32_t n_tiles) {
    __shared__ uint32_t part[1024];
    const uint32_t per = (n_tiles + blockDim.x - 1) / blockDim.x;
    const uint32_t lo = threadIdx.x * per, hi = lo + per < n_tiles ? lo + per : n_tiles;
    uint32_t sum = 0;
    for (uint32_t i = lo; i < hi; i++) sum += tile_sums[i];
    part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (uint32_t t = 0; t < blockDim.x; t++) {
            const uint32_t v = part[t];
            part[t] = run;
            run += v;
        }
    }
    __syncthreads();
    uint32_t run = part[threadIdx.x];
    for (uint32_t i = lo; i < hi; i++) {
        const uint32_t v = tile_sums[i];
        tile_sums[i] = run;
        run += v;
    }
}

__global__ void __launch_bounds__(kScanThreads)
    msm_scan_in_tiles(const uint32_t* __restrict__ counts, const uint32_t* __restrict__ tile_offsets, uint64_t n,
                      uint32_t* __restrict__ offsets) {
    __shared__ uint32_t vals[kScanTile];
    __shared__ uint32_t part[kScanThreads];
    const uint64_t base = (uint64_t)blockIdx.x * kScanTile;
    for (uint32_t j = 0; j < kScanPer; j++) {
        const uint32_t k = j * kScanThreads + threadIdx.x;
        vals[k] = base + k < n ? counts[base + k] : 0u;
    }
    __syncthreads();
    uint32_t sum = 0;
    for (uint32_t j = 0; j < kScanPer; j++) sum += vals[threadIdx.x * kScanPer + j];
    part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = tile_offsets[blockIdx.x];
        for (uint32_t t = 0; t < kScanThreads; t++) {
            const uint32_t v = part[t];
            part[t] = run;
            run += v;
        }
    }
    __syncthreads();
    uint32_t run = part[threadIdx.x];
    for (uint32_t j = 0; j < kScanPer; j++) {
        const uint32_t k = threadIdx.x * kScanPer + j;
        const uint32_t v = vals[k];
        vals[k] = run;
        run += v;
    }
    __syncthreads();
    for (uint32_t j = 0; j < kScanPer; j++) {
        const uint32_t k = j * kScanThreads + threadIdx.x;
        if (base + k < n) offsets[base + k] = vals[k];
    }
}

__global__ void __launch_bounds__(kThreads)
    msm_scatter(MsmScalars s, uint64_t n, uint32_t c, uint32_t windows, const uint32_t* __restrict__ offsets,
                uint32_t* __restrict__ cursor, uint32_t* __restrict__ items) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned active = __activemask();
        uint64_t mag[4];
        bool neg;
        msm_scalar(s, i, mag, neg);
        for (uint32_t w = 0; w < windows; w++) {
            const uint32_t d = msm_digit(mag, w, c);
            const size_t key = ((size_t)w << c) + d;
            uint32_t rank;
            const uint32_t at = msm_group_add(&cursor[key], key, d != 0, active, rank);
            if (d) items[offsets[key] + at + rank] = (uint32_t)i | (neg ? 0x80000000u : 0u);
        }
    }
}

constexpr uint32_t kMsmHeavy = 96;  // a bucket with more points than this is summed by a whole block

__global__ void __launch_bounds__(kThreads)
    msm_buckets(const G1Affine* __restrict__ bases, const uint32_t* __restrict__ offsets,
                const uint32_t* __restrict__ counts, const uint32_t* __restrict__ items, uint64_t n_keys,
                G1Jac* __restrict__ buckets, uint32_t* __restrict__ heavy_list, uint32_t* __restrict__ heavy_count) {
    const uint64_t key = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (key >= n_keys) return;
    const uint32_t lo = offsets[key], cnt = counts[key];
    if (cnt > kMsmHeavy) {  // skewed digits (small integers in a wide window): left to msm_heavy_buckets
        heavy_list[atomicAdd(heavy_count, 1u)] = (uint32_t)key;
        return;
    }
    G1Jac acc = g1_infinity();
    for (uint32_t j = 0; j < cnt; j++) {
        const uint32_t it = items[lo + j];
        G1Affine p = bases[it & 0x7fffffffu];
        if (it & 0x80000000u) p = g1_affine_neg(p);
        acc = g1_add_mixed(acc, p);
    }
    buckets[key] = acc;
}

// Heavy buckets are cut into chunks of kHeavyChunk points so that a bucket of a million points (16-bit values in a
// 13-bit window leave seven such buckets in the second window) is work for the whole GPU instead of one block.
// msm_heavy_plan: chunk_first[h] = number of chunks before heavy bucket h (one block; the list has at most
// n * windows / kMsmHeavy entries).
constexpr uint32_t kHeavyChunk = 2048;
__global__ void __launch_bounds__(1024)
    msm_heavy_plan(const uint32_t* __restrict__ counts, const uint32_t* __restrict__ heavy_list,
                   const uint32_t* __restrict__ heavy_count, uint32_t* __restrict__ chunk_first) {
    __shared__ uint32_t part[1024];
    const uint32_t n_heavy = *heavy_count;
    const uint32_t per = (n_heavy + blockDim.x - 1) / blockDim.x;
    const uint32_t lo = threadIdx.x * per < n_heavy ? threadIdx.x * per : n_heavy;
    const uint32_t hi = lo + per < n_heavy ? lo + per : n_heavy;
    uint32_t sum = 0;
    for (uint32_t h = lo; h < hi; h++) sum += (counts[heavy_list[h]] + kHeavyChunk - 1) / kHeavyChunk;
    part[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (uint32_t t = 0; t < blockDim.x; t++) {
            const uint32_t v = part[t];
            part[t] = run;
            run += v;
        }
        chunk_first[n_heavy] = run;  // total
    }
    __syncthreads();
    uint32_t run = part[threadIdx.x];
    for (uint32_t h = lo; h < hi; h++) {
        chunk_first[h] = run;
        run += (counts[heavy_list[h]] + kHeavyChunk - 1) / kHeavyChunk;
    }
}

// one block per chunk (grid-stride): every thread adds a strided share of the chunk's points, then a tree in shared
// memory; chunk_sums[g] = the chunk's sum
__global__ void __launch_bounds__(kMsmReduceThreads)
    msm_heavy_chunks(const G1Affine* __restrict__ bases, const uint32_t* __restrict__ offsets,
                     const uint32_t* __restrict__ counts, const uint32_t* __restrict__ items,
                     const uint32_t* __restrict__ heavy_list, const uint32_t* __restrict__ heavy_count,
                     const uint32_t* __restrict__ chunk_first, G1Jac* __restrict__ chunk_sums) {
    __shared__ G1Jac sh[kMsmReduceThreads];
    const uint32_t n_heavy = *heavy_count;
    const uint32_t total = chunk_first[n_heavy];
    for (uint32_t g = blockIdx.x; g < total; g += gridDim.x) {
        // the heavy bucket this chunk belongs to: last h with chunk_first[h] <= g
        uint32_t lo_h = 0, hi_h = n_heavy;
        while (hi_h - lo_h > 1) {
            const uint32_t mid = (lo_h + hi_h) >> 1;
            if (chunk_first[mid] <= g) lo_h = mid;
            else hi_h = mid;
        }
        const uint32_t key = heavy_list[lo_h];
        const uint32_t first = offsets[key] + (g - chunk_first[lo_h]) * kHeavyChunk;
        const uint32_t end_all = offsets[key] + counts[key];
        const uint32_t end = first + kHeavyChunk < end_all ? first + kHeavyChunk : end_all;
        G1Jac acc = g1_infinity();
        for (uint32_t j = first + threadIdx.x; j < end; j += blockDim.x) {
            const uint32_t it = items[j];
            G1Affine p = bases[it & 0x7fffffffu];
            if (it & 0x80000000u) p = g1_affine_neg(p);
            acc = g1_add_mixed(acc, p);
        }
        sh[threadIdx.x] = acc;
        __syncthreads();
        for (uint32_t s = kMsmReduceThreads / 2; s > 0; s >>= 1) {
            if (threadIdx.x < s) sh[threadIdx.x] = g1_add(sh[threadIdx.x], sh[threadIdx.x + s]);
            __syncthreads();
        }
        if (threadIdx.x == 0) chunk_sums[g] = sh[0];
        __syncthreads();
    }
}

// one block per heavy bucket (grid-stride): the sum of its chunks' sums
__global__ void __launch_bounds__(kMsmReduceThreads)
    msm_heavy_combine(const uint32_t* __restrict__ heavy_list, const uint32_t* __restrict__ heavy_count,
                      const uint32_t* __restrict__ chunk_first, const G1Jac* __restrict__ chunk_sums,
                      G1Jac* __restrict__ buckets) {
    __shared__ G1Jac sh[kMsmReduceThreads];
    const uint32_t n_heavy = *heavy_count;
    for (uint32_t h = blockIdx.x; h < n_heavy; h += gridDim.x) {
        const uint32_t first = chunk_first[h], end = chunk_first[h + 1];
        if (end - first == 1) {  // the usual case: a bucket of a few hundred points
            if (threadIdx.x == 0) buckets[heavy_list[h]] = chunk_sums[first];
            continue;
        }
        G1Jac acc = g1_infinity();
        for (uint32_t g = first + threadIdx.x; g < end; g += blockDim.x) acc = g1_add(acc, chunk_sums[g]);
        sh[threadIdx.x] = acc;
        __syncthreads();
        for (uint32_t s = kMsmReduceThreads / 2; s > 0; s >>= 1) {
            if (threadIdx.x < s) sh[threadIdx.x] = g1_add(sh[threadIdx.x], sh[threadIdx.x + s]);
            __syncthreads();
        }
        if (threadIdx.x == 0) buckets[heavy_list[h]] = sh[0];
        __syncthreads();
    }
}

// out[w * blocks_per_window + blk] = sum over the block's buckets b of b * B_b
__global__ void __launch_bounds__(kMsmReduceThreads)
    msm_reduce(const G1Jac* __restrict__ buckets, uint32_t c, uint32_t blocks_per_window, G1Jac* __restrict__ out) {
    __shared__ G1Jac sh[kMsmReduceThreads];
    const uint32_t w = blockIdx.x / blocks_per_window, blk = blockIdx.x % blocks_per_window;
    const uint64_t n_b = 1ull << c;
    const uint64_t run_id = (uint64_t)blk * kMsmReduceThreads + threadIdx.x;
    const uint64_t b_lo = run_id * kMsmRun;  // first bucket of this thread's run
    G1Jac total = g1_infinity();
    if (b_lo < n_b) {
        const uint64_t b_hi = b_lo + kMsmRun < n_b ? b_lo + kMsmRun : n_b;
        const G1Jac* B = buckets + ((size_t)w << c);
        G1Jac running = g1_infinity(), sum = g1_infinity();
        for (uint64_t b = b_hi; b-- > b_lo;) {  // sum = sum_b (b - b_lo + 1) B_b
            running = g1_add(running, B[b]);
            sum = g1_add(sum, running);
        }
        // sum_b b B_b = sum + (b_lo - 1) * running; bucket 0 is empty, so for b_lo = 0 the term (-1) * running
        // is cancelled by counting one copy less: walk it as sum - running
        if (b_lo == 0) {
            G1Jac neg = running;
            neg.Y = fq_neg(neg.Y);
            total = g1_add(sum, neg);
        } else {
            total = g1_add(sum, g1_mul_small(running, (uint32_t)(b_lo - 1)));
        }
    }
    sh[threadIdx.x] = total;
    __syncthreads();
    for (uint32_t s = kMsmReduceThreads / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) sh[threadIdx.x] = g1_add(sh[threadIdx.x], sh[threadIdx.x + s]);
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = sh[0];
}

__global__ void __launch_bounds__(kThreads) msm_bases_to_mont(G1Affine* p, uint64_t n, unsigned int* bad) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    G1Affine a = p[i];
    if (!g1_affine_is_infinity(a)) {
        if (fq_geq_q(a.x) || fq_geq_q(a.y)) {
            atomicAdd(bad, 1u);
            return;
        }
        a.x = fq_to_mont(a.x);
        a.y = fq_to_mont(a.y);
        if (!g1_affine_on_curve(a)) atomicAdd(bad, 1u);
    }
    p[i] = a;
}

// point i = (first + i) * G for the generator G = (1, 2): valid, distinct points for benchmarks and tests
__global__ void __launch_bounds__(kThreads) msm_synthetic_bases(G1Affine* out, uint64_t n, uint32_t first) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    G1Affine g;
    Fq one, two;
    one.l[0] = 1;
    two.l[0] = 2;
    one.l[1] = one.l[2] = one.l[3] = two.l[1] = two.l[2] = two.l[3] = 0;
    g.x = fq_to_mont(one);
    g.y = fq_to_mont(two);
    out[i] = g1_to_affine(g1_mul_small(g1_from_affine(g), first + (uint32_t)i));
}

static uint32_t msm_window_bits(uint64_t n) {
    uint32_t lg = 0;
    while ((1ull << lg) < n) lg++;
    if (lg >= 18) return 16;
    if (lg >= 14) return 13;
    if (lg >= 10) return 10;
    return 8;
}

constexpr uint32_t kMsmGroup = 16;               // commitments of a batch in flight together
constexpr size_t kMsmHostBytes = 1 << 20;         // pinned staging for their window sums

// One commitment: its layout in one block of device memory [counts | offsets | cursor | heavy count | items |
// heavy list | scan tiles | buckets | window sums | heavy chunk table | heavy chunk sums].
struct MsmJob {
    uint64_t n = 0;
    uint32_t c = 0, windows = 0, blocks_per_window = 0, n_tiles = 0;
    size_t n_keys = 0, n_partials = 0, host_off = 0;
    uint64_t max_heavy = 0, max_chunks = 0;
    size_t o_counts = 0, o_offsets = 0, o_cursor = 0, o_heavy_count = 0, o_items = 0, o_heavy = 0, o_tiles = 0, o_buckets = 0,
           o_part = 0, o_chunk_first = 0, o_chunk_sums = 0;
    void* slab = nullptr;
};

static int msm_plan(dpb_ctx* ctx, const dpb_g1_bases* bases, const dpb_mle* scalars, MsmJob& job) {
    if (scalars->dtype != DPB_FR && scalars->dtype != DPB_FR_I32 && scalars->dtype != DPB_FR_I64)
        return fail(DPB_EINVAL, "scalars must be a BN254 table (DPB_FR, DPB_FR_I32 or DPB_FR_I64), not dtype %d", scalars->dtype);
    const uint64_t n = scalars->len;
    if (n > bases->n)
        return fail(DPB_EINVAL, "%llu scalars but only %llu points", (unsigned long long)n, (unsigned long long)bases->n);
    job.n = n;
    job.c = msm_window_bits(n);
    const uint32_t scalar_bits = scalars->dtype == DPB_FR ? 254 : scalars->dtype == DPB_FR_I32 ? 32 : 64;
    job.windows = (scalar_bits + job.c - 1) / job.c;
    job.n_keys = (size_t)job.windows << job.c;
    const uint32_t runs = (uint32_t)(((1ull << job.c) + kMsmRun - 1) / kMsmRun);
    job.blocks_per_window = (runs + kMsmReduceThreads - 1) / kMsmReduceThreads;
    job.n_partials = (size_t)job.windows * job.blocks_per_window;
    job.n_tiles = (uint32_t)((job.n_keys + kScanTile - 1) / kScanTile);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off = (off + bytes + 255) & ~(size_t)255;
        return o;
    };
    job.o_counts = take(job.n_keys * 4);
    job.o_offsets = take(job.n_keys * 4);
    job.o_cursor = take(job.n_keys * 4);
    job.o_heavy_count = take(256);
    job.o_items = take((size_t)n * job.windows * 4);
    job.o_heavy = take(job.n_keys * 4);
    job.o_tiles = take((size_t)job.n_tiles * 4);
    job.o_buckets = take(job.n_keys * sizeof(G1Jac));
    job.o_part = take(job.n_partials * sizeof(G1Jac));
    // heavy buckets: at most n * windows / kMsmHeavy of them, cut into at most that many + n * windows / kHeavyChunk chunks
    job.max_heavy = (uint64_t)n * job.windows / kMsmHeavy + 1;
    if (job.max_heavy > job.n_keys) job.max_heavy = job.n_keys;
    job.max_chunks = job.max_heavy + (uint64_t)n * job.windows / kHeavyChunk + 1;
    job.o_chunk_first = take((job.max_heavy + 1) * 4);
    job.o_chunk_sums = take(job.max_chunks * sizeof(G1Jac));
    return device_alloc(ctx, off, &job.slab);
}

// every kernel of one commitment and the copy of its window sums to `h_part` (pinned), on stream `st`
static cudaError_t msm_launch(dpb_ctx* ctx, const dpb_g1_bases* bases, const dpb_mle* scalars, const MsmJob& job,
                              cudaStream_t st, G1Jac* h_part) {
    char* base = (char*)job.slab;
    uint32_t* counts = (uint32_t*)(base + job.o_counts);
    uint32_t* offsets = (uint32_t*)(base + job.o_offsets);
    uint32_t* cursor = (uint32_t*)(base + job.o_cursor);
    uint32_t* items = (uint32_t*)(base + job.o_items);
    uint32_t* heavy_list = (uint32_t*)(base + job.o_heavy);
    uint32_t* heavy_count = (uint32_t*)(base + job.o_heavy_count);
    uint32_t* tile_sums = (uint32_t*)(base + job.o_tiles);
    uint32_t* chunk_first = (uint32_t*)(base + job.o_chunk_first);
    G1Jac* chunk_sums = (G1Jac*)(base + job.o_chunk_sums);
    G1Jac* buckets = (G1Jac*)(base + job.o_buckets);
    G1Jac* partials = (G1Jac*)(base + job.o_part);
    MsmScalars s;
    s.ptr = scalars->ptr;
    s.dtype = scalars->dtype;
    const uint64_t n = job.n;
    const uint32_t c = job.c, windows = job.windows;
    const size_t n_keys = job.n_keys;
    cudaError_t e = cudaMemsetAsync(counts, 0, job.o_items - job.o_counts, st);  // counts, offsets, cursor, heavy count
    if (e != cudaSuccess) return e;
    msm_count<<<grid_for(ctx, n), kThreads, 0, st>>>(s, n, c, windows, counts);
    msm_scan_tile_sums<<<job.n_tiles, kScanThreads, 0, st>>>(counts, n_keys, tile_sums);
    msm_scan_tiles<<<1, 1024, 0, st>>>(tile_sums, job.n_tiles);
    msm_scan_in_tiles<<<job.n_tiles, kScanThreads, 0, st>>>(counts, tile_sums, n_keys, offsets);
    msm_scatter<<<grid_for(ctx, n), kThreads, 0, st>>>(s, n, c, windows, offsets, cursor, items);
    msm_buckets<<<(uint32_t)((n_keys + kThreads - 1) / kThreads), kThreads, 0, st>>>(
        bases->dev, offsets, counts, items, n_keys, buckets, heavy_list, heavy_count);
    const uint32_t cap = (uint32_t)ctx->sm_count * 16;  // idle blocks leave at once
    msm_heavy_plan<<<1, 1024, 0, st>>>(counts, heavy_list, heavy_count, chunk_first);
    msm_heavy_chunks<<<(uint32_t)(job.max_chunks < cap ? job.max_chunks : cap), kMsmReduceThreads, 0, st>>>(
        bases->dev, offsets, counts, items, heavy_list, heavy_count, chunk_first, chunk_sums);
    msm_heavy_combine<<<(uint32_t)(job.max_heavy < cap ? job.max_heavy : cap), kMsmReduceThreads, 0, st>>>(
        heavy_list, heavy_count, chunk_first, chunk_sums, buckets);
    msm_reduce<<<(uint32_t)job.n_partials, kMsmReduceThreads, 0, st>>>(buckets, c, job.blocks_per_window, partials);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return cudaMemcpyAsync(h_part, partials, job.n_partials * sizeof(G1Jac), cudaMemcpyDeviceToHost, st);
}

// host: windows from the top, total = 2^c * total + window sum; one inversion for the affine result
static void msm_finish(const MsmJob& job, const G1Jac* h_part, void* out_affine_xy) {
    G1Jac total = g1_infinity();
    for (uint32_t w = job.windows; w-- > 0;) {
        for (uint32_t d = 0; d < job.c; d++) total = g1_double(total);
        for (uint32_t k = 0; k < job.blocks_per_window; k++)
            total = g1_add(total, h_part[(size_t)w * job.blocks_per_window + k]);
    }
    const G1Affine a = g1_to_affine(total);
    Fq xy[2];
    if (g1_affine_is_infinity(a)) {
        xy[0] = xy[1] = fq_zero();
    } else {
        xy[0] = fq_from_mont(a.x);
        xy[1] = fq_from_mont(a.y);
    }
    memcpy(out_affine_xy, xy, sizeof xy);
}

static int msm_side_streams(dpb_ctx* ctx) {
    if (ctx->msm_stream[0]) return DPB_OK;
    for (int q = 0; q < dpb_ctx::kMsmStreams; q++) DPB_CUDA(cudaStreamCreateWithFlags(&ctx->msm_stream[q], cudaStreamNonBlocking));
    for (int q = 0; q <= dpb_ctx::kMsmStreams; q++) DPB_CUDA(cudaEventCreateWithFlags(&ctx->msm_ev[q], cudaEventDisableTiming));
    return DPB_OK;
}

}  // namespace dpb

using namespace dpb;

extern "C" {

int dpb_g1_bases_from_host(dpb_ctx* ctx, const void* affine_xy, uint64_t n, dpb_g1_bases** out) {
    if (!ctx || !affine_xy || !out) return fail(DPB_EINVAL, "null argument");
    if (n == 0 || n > (1ull << 31)) return fail(DPB_EINVAL, "number of points %llu outside 1..2^31", (unsigned long long)n);
    dpb_g1_bases* b = new (std::nothrow) dpb_g1_bases();
    if (!b) return fail(DPB_ENOMEM, "host allocation failed");
    b->ctx = ctx;
    b->n = n;
    void* p = nullptr;
    int rc = device_alloc(ctx, n * sizeof(G1Affine), &p);
    if (rc != DPB_OK) {
        delete b;
        return rc;
    }
    b->dev = (G1Affine*)p;
    unsigned int* bad = nullptr;
    rc = device_alloc(ctx, sizeof(unsigned int), (void**)&bad);
    unsigned int h_bad = 0;
    cudaError_t e = cudaSuccess;
    if (rc == DPB_OK) {
        e = cudaMemcpyAsync(p, affine_xy, n * sizeof(G1Affine), cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(bad, 0, sizeof(unsigned int), ctx->stream);
        if (e == cudaSuccess) {
            msm_bases_to_mont<<<(uint32_t)((n + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(b->dev, n, bad);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(&h_bad, bad, sizeof(unsigned int), cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    }
    device_free(ctx, bad);
    if (rc == DPB_OK && e != cudaSuccess) rc = fail(DPB_ECUDA, "uploading G1 points: %s", cudaGetErrorString(e));
    if (rc == DPB_OK && h_bad) rc = fail(DPB_EINVAL, "%u points are not on the curve or have coordinates >= q", h_bad);
    if (rc != DPB_OK) {
        device_free(ctx, p);
        delete b;
        return rc;
    }
    *out = b;
    return DPB_OK;
}

int dpb_g1_bases_synthetic(dpb_ctx* ctx, uint64_t n, uint32_t first_multiple, dpb_g1_bases** out) {
    if (!ctx || !out) return fail(DPB_EINVAL, "null argument");
    if (n == 0 || first_multiple == 0 || n + first_multiple > (1ull << 31))
        return fail(DPB_EINVAL, "multiples %u .. %llu of the generator are outside 1..2^31", first_multiple,
                    (unsigned long long)(n + first_multiple - 1));
    dpb_g1_bases* b = new (std::nothrow) dpb_g1_bases();
    if (!b) return fail(DPB_ENOMEM, "host allocation failed");
    b->ctx = ctx;
    b->n = n;
    void* p = nullptr;
    int rc = device_alloc(ctx, n * sizeof(G1Affine), &p);
    if (rc != DPB_OK) {
        delete b;
        return rc;
    }
    b->dev = (G1Affine*)p;
    msm_synthetic_bases<<<(uint32_t)((n + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>(b->dev, n, first_multiple);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        device_free(ctx, p);
        delete b;
        return fail(DPB_ECUDA, "synthetic bases: %s", cudaGetErrorString(e));
    }
    *out = b;
    return DPB_OK;
}

uint64_t dpb_g1_bases_len(const dpb_g1_bases* b) { return b ? b->n : 0; }

void dpb_g1_bases_free(dpb_g1_bases* b) {
    if (!b) return;
    device_free(b->ctx, b->dev);
    delete b;
}

int dpb_msm_g1(dpb_ctx* ctx, const dpb_g1_bases* bases, const dpb_mle* scalars, void* out_affine_xy) {
    dpb_mle* one[1] = {const_cast<dpb_mle*>(scalars)};
    if (!scalars) return fail(DPB_EINVAL, "null argument");
    return dpb_pcs_batch_commit(ctx, bases, one, 1, out_affine_xy);
}

int dpb_pcs_batch_commit(dpb_ctx* ctx, const dpb_g1_bases* bases, dpb_mle* const* polys, uint32_t n_polys,
                         void* out_affine_xy) {
    if (!ctx || !bases || !polys || !out_affine_xy) return fail(DPB_EINVAL, "null argument");
    if (bases->ctx != ctx) return fail(DPB_EINVAL, "the bases belong to another context");
    for (uint32_t i = 0; i < n_polys; i++) {
        if (!polys[i]) return fail(DPB_EINVAL, "polynomial %u is null", i);
        if (polys[i]->ctx != ctx) return fail(DPB_EINVAL, "polynomial %u belongs to another context", i);
    }
    if (n_polys > 1) DPB_TRY(msm_side_streams(ctx));
    // groups of commitments in flight together: their kernels are short chains of curve additions that leave most
    // of the GPU idle one at a time
    for (uint32_t first = 0; first < n_polys; first += kMsmGroup) {
        const uint32_t cnt = std::min<uint32_t>(kMsmGroup, n_polys - first);
        std::vector<MsmJob> jobs(cnt);
        int rc = DPB_OK;
        size_t host_off = 0;
        for (uint32_t j = 0; j < cnt && rc == DPB_OK; j++) {
            rc = msm_plan(ctx, bases, polys[first + j], jobs[j]);
            jobs[j].host_off = host_off;
            host_off += jobs[j].n_partials * sizeof(G1Jac);
        }
        if (rc == DPB_OK && host_off > kMsmHostBytes) rc = fail(DPB_EINVAL, "commitment staging of %zu bytes", host_off);
        cudaError_t e = cudaSuccess;
        if (rc == DPB_OK) {
            if (!ctx->msm_host) e = cudaHostAlloc(&ctx->msm_host, kMsmHostBytes, cudaHostAllocDefault);
            const bool side = cnt > 1;
            if (e == cudaSuccess && side) {
                // the side streams start after everything this context has queued (the scalars' producers included)
                e = cudaEventRecord(ctx->msm_ev[dpb_ctx::kMsmStreams], ctx->stream);
                for (int q = 0; q < dpb_ctx::kMsmStreams && e == cudaSuccess; q++)
                    e = cudaStreamWaitEvent(ctx->msm_stream[q], ctx->msm_ev[dpb_ctx::kMsmStreams], 0);
            }
            for (uint32_t j = 0; j < cnt && e == cudaSuccess; j++) {
                cudaStream_t st = side ? ctx->msm_stream[j % dpb_ctx::kMsmStreams] : ctx->stream;
                e = msm_launch(ctx, bases, polys[first + j], jobs[j], st, (G1Jac*)((char*)ctx->msm_host + jobs[j].host_off));
            }
            if (side) {
                // ... and this context's stream goes on after them (even when a launch failed: the slabs are freed below)
                for (int q = 0; q < dpb_ctx::kMsmStreams; q++) {
                    cudaEventRecord(ctx->msm_ev[q], ctx->msm_stream[q]);
                    cudaStreamWaitEvent(ctx->stream, ctx->msm_ev[q], 0);
                }
            }
            const cudaError_t es = cudaStreamSynchronize(ctx->stream);
            if (e == cudaSuccess) e = es;
        }
        for (auto& job : jobs) device_free(ctx, job.slab);
        if (rc != DPB_OK) return rc;
        if (e != cudaSuccess) return fail(DPB_ECUDA, "msm: %s", cudaGetErrorString(e));
        for (uint32_t j = 0; j < cnt; j++)
            msm_finish(jobs[j], (const G1Jac*)((const char*)ctx->msm_host + jobs[j].host_off),
                       (char*)out_affine_xy + (size_t)(first + j) * 64);
    }
    return DPB_OK;
}

}  // extern "C"
