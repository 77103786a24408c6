// Lookup witness generation on the device: the rescaled values of a layer's input are cut into shifted chunks,
// value chunks and zeroing chunks (ChunkingInfo::decompose_input, zkml/src/lookup/operation/decomposer.rs:252-312),
// the chunks are looked up (table_output, decomposer.rs:315-383), every column is written as a table of field
// elements (ChunkedInput::to_evals / ChunkedOutput::to_evals, decomposer.rs:71-87, 134-143) and the looked-up rows
// are counted per table (LookupOpWitness::get_counts, zkml/src/lookup/operation/mod.rs:193-267).
//
// One thread per padded entry: 8 bytes read, one field element written per column.  With BN254 the writes are
// 32 bytes per column and the kernel is bound by them, provided the conversion to Montgomery form is not a
// multiplication per entry: chunk values are small, so x*R mod r is put together from three 256-row tables in
// shared memory (x = x0 + 2^8 x1 + 2^16 x2) with two additions.
#pragma once
#include "family.cuh"

namespace dpb {

constexpr int kLookupCacheBits = 9;    // block-local (row, count) cache per table: 2^9 entries
constexpr int kLookupCache = 1 << kLookupCacheBits;
constexpr int kLookupProbes = 4;
constexpr uint32_t kLookupDirectBits = 13;  // a value table of at most 2^13 rows gets a full block-local histogram
constexpr uint32_t kLookupNoKey = 0xffffffffu;
constexpr int kLookupMaxChunks = 4;    // per kind: shifted, value, zeroing

struct LookupWitnessArgs {
    const int64_t* tensor;      // unpadded, row-major, n_slices x rows x cols
    uint64_t rows, cols;        // the last two dimensions
    uint32_t pcol_bits, p_bits; // log2 of the padded row length and of the padded slice
    uint64_t n_slices;
    int64_t fpm;                // fixed-point multiplier
    int64_t rc;                 // rounding constant 2^(right_shift - 1)
    int64_t pad_rescaled;       // padding_value * fpm + rc
    dpb_chunking_info ci;
    const int64_t* table_out;   // the value table's output column over min..=max inputs; null: output = input
    int64_t table_min;          // smallest input of the value table
    unsigned long long* counts[4];  // shift-check, value, zero-check, signed zero-check tables; null: not counted
    uint32_t n_in_per, n_out_per;   // columns per slice
    uint32_t value_in_column;       // value chunks are input columns (two-column value table)
    uint32_t direct_rows;           // rows of the block-local value histogram (0: none)
    int* error;                     // bit 0: a top zeroing chunk outside the signed zero-check table
};

// Block-local counters.  An atomic on one address in device memory takes tens of nanoseconds to come back, and
// lookups concentrate on few rows (zeroing chunks are nearly constant over a tensor, value chunks hit a table
// of a few thousand rows), so counting straight into device memory would take longer than writing the columns.
// Every table has a small open-addressed (row, count) cache per block; the value table, when small enough, a full
// histogram.  Both are added to device memory once, when the block ends; what the cache cannot hold goes to
// device memory directly (that is the spread-out case, where device atomics are fast).
struct LookupCache {
    uint32_t key[4][kLookupCache];
    uint32_t cnt[4][kLookupCache];
};

// Counts `bin` once per active lane; lanes of a warp that hit the same row add once.
__device__ __forceinline__ void lookup_count(unsigned long long* bins, LookupCache& cache, int h, uint32_t bin, bool active,
                                             uint32_t* direct = nullptr) {
    if (!bins) return;  // same for the whole grid
    const uint32_t key = active ? bin : kLookupNoKey;
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (!active) return;
    if ((int)(threadIdx.x & 31) != __ffs(peers) - 1) return;
    const uint32_t n = __popc(peers);
    if (direct) {
        atomicAdd(&direct[bin], n);
        return;
    }
    const uint32_t slot = (bin * 2654435761u) >> (32 - kLookupCacheBits);
    for (int p = 0; p < kLookupProbes; p++) {
        const uint32_t s = (slot + p) & (kLookupCache - 1);
        uint32_t k = *(volatile uint32_t*)&cache.key[h][s];
        if (k == kLookupNoKey) {
            k = atomicCAS(&cache.key[h][s], kLookupNoKey, bin);
            if (k == kLookupNoKey) k = bin;
        }
        if (k == bin) {
            atomicAdd(&cache.cnt[h][s], n);
            return;
        }
    }
    atomicAdd(&bins[bin], (unsigned long long)n);
}

// Signed small integer -> field element, per family.
template <class F>
struct SmallToField;

template <>
struct SmallToField<GlFam> {
    typedef uint64_t T;
    static constexpr int kDtype = DPB_GL_BASE;
    struct Shared {
        int unused;
    };
    __device__ static void init(Shared&) {}
    __device__ __forceinline__ static T conv(const Shared&, int64_t v) {
        // |v| < 2^63 < p: the magnitude is canonical (negative x -> p - |x|, zkml/src/quantization/mod.rs:220-267)
        return v < 0 ? GL_P - ((uint64_t)0 - (uint64_t)v) : (uint64_t)v;
    }
    __device__ __forceinline__ static void store(T* p, uint64_t i, T v) { p[i] = v; }
};

template <>
struct SmallToField<FrFam> {
    typedef Fr T;
    static constexpr int kDtype = DPB_FR;
    struct Shared {
        Fr row[3][256];  // row[j][k] = k * 2^(8 j) in Montgomery form
    };
    __device__ static void init(Shared& s) {
        for (uint32_t t = threadIdx.x; t < 3 * 256; t += blockDim.x)
            s.row[t >> 8][t & 255] = fr_from_u64((uint64_t)(t & 255) << (8 * (t >> 8)));
    }
    __device__ __forceinline__ static T conv(const Shared& s, int64_t v) {
        const uint64_t mag = v < 0 ? (uint64_t)0 - (uint64_t)v : (uint64_t)v;
        Fr a;
        if (mag < (1u << 24)) {
            a = s.row[0][mag & 255];
            if (mag >> 8) {
                a = fr_add(a, s.row[1][(mag >> 8) & 255]);
                if (mag >> 16) a = fr_add(a, s.row[2][mag >> 16]);
            }
        } else {
            a = fr_from_u64(mag);
        }
        return v < 0 ? fr_neg(a) : a;
    }
    __device__ __forceinline__ static void store(T* p, uint64_t i, const T& v) { FrFam::store(p, i, v); }
};

// Columns that stay integers (DPB_GL_I64 / DPB_FR_I64 tables): what the witness kernel writes is the chunk itself.
// Eight bytes per entry instead of 32 for BN254, and a commitment to such a column is a multi-scalar multiplication
// over one or two windows instead of sixteen (a negative chunk as a field element has all its bits set).
template <class F>
struct IntColumns {};
template <class F>
struct SmallToField<IntColumns<F>> {
    typedef int64_t T;
    static constexpr int kDtype = std::is_same<F, GlFam>::value ? DPB_GL_I64 : DPB_FR_I64;
    struct Shared {
        int unused;
    };
    __device__ static void init(Shared&) {}
    __device__ __forceinline__ static T conv(const Shared&, int64_t v) { return v; }
    __device__ __forceinline__ static void store(T* p, uint64_t i, T v) { p[i] = v; }
};

// Dynamic shared memory: [conversion tables | caches | value histogram (direct_rows words)].
template <class F>
size_t lookup_witness_smem(uint32_t direct_rows) {
    return sizeof(typename SmallToField<F>::Shared) + sizeof(LookupCache) + (size_t)direct_rows * 4;
}

template <class F>
__global__ void __launch_bounds__(512) lookup_witness_kernel(LookupWitnessArgs a, typename SmallToField<F>::T* __restrict__ in_cols,
                                                             typename SmallToField<F>::T* __restrict__ out_cols) {
    typedef SmallToField<F> Conv;
    typedef typename Conv::T T;
    extern __shared__ __align__(16) unsigned char smem[];
    typename Conv::Shared& conv = *reinterpret_cast<typename Conv::Shared*>(smem);
    LookupCache& hot = *reinterpret_cast<LookupCache*>(smem + sizeof(typename Conv::Shared));
    uint32_t* direct = a.direct_rows ? reinterpret_cast<uint32_t*>(smem + sizeof(typename Conv::Shared) + sizeof(LookupCache)) : nullptr;
    Conv::init(conv);
    for (uint32_t t = threadIdx.x; t < 4 * kLookupCache; t += blockDim.x) {
        (&hot.key[0][0])[t] = kLookupNoKey;
        (&hot.cnt[0][0])[t] = 0;
    }
    for (uint32_t t = threadIdx.x; t < a.direct_rows; t += blockDim.x) direct[t] = 0;
    __syncthreads();

    const dpb_chunking_info& ci = a.ci;
    const uint64_t total = a.n_slices << a.p_bits;
    const uint64_t slice_mask = (1ull << a.p_bits) - 1, col_mask = (1ull << a.pcol_bits) - 1;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const bool last_shift_partial = (ci.right_shift % 16) != 0;
    // g - lane is the same for a warp, so every lane of a warp makes the same number of trips
    for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g - (threadIdx.x & 31) < total; g += stride) {
        const bool active = g < total;
        const uint64_t slice = g >> a.p_bits, i = g & slice_mask;
        const uint64_t row = i >> a.pcol_bits, col = i & col_mask;
        int64_t x = a.pad_rescaled;
        if (active && row < a.rows && col < a.cols) x = a.tensor[(slice * a.rows + row) * a.cols + col] * a.fpm + a.rc;
        // the value after the offset is never negative for inputs inside the operation's range
        int64_t rem = ci.table_sign == DPB_SIGN_MIXED ? x + ci.offset : ci.table_sign == DPB_SIGN_POSITIVE ? x : -x;
        T* in = in_cols + ((slice * a.n_in_per) << a.p_bits) + i;
        T* out = out_cols + ((slice * a.n_out_per) << a.p_bits) + i;

        for (uint32_t s = 0; s < ci.n_shifted_chunks; s++) {
            int64_t chunk;
            if (s != ci.n_shifted_chunks - 1 || !last_shift_partial) {
                chunk = rem & 0xffff;
                rem >>= 16;
            } else {
                const uint32_t size = ci.right_shift % 16;
                chunk = (rem & ((1ll << size) - 1)) * ci.shifted_chunk_multiplier;
                rem >>= size;
            }
            if (active) Conv::store(in, 0, Conv::conv(conv, chunk));
            in += 1ull << a.p_bits;
            lookup_count(a.counts[0], hot, 0, (uint32_t)chunk, active);
        }
        const int64_t value_mask = (1ll << ci.value_chunk_bits) - 1;
        for (uint32_t s = 0; s < ci.n_value_chunks; s++) {
            const int64_t c = rem & value_mask;
            const int64_t v = ci.table_sign == DPB_SIGN_MIXED ? c - ci.value_chunk_offset : ci.table_sign == DPB_SIGN_POSITIVE ? c : -c;
            rem >>= ci.value_chunk_bits;
            const uint32_t bin = (uint32_t)(v - a.table_min);
            if (a.value_in_column) {
                if (active) Conv::store(in, 0, Conv::conv(conv, v));
                in += 1ull << a.p_bits;
            }
            if (active) Conv::store(out, 0, Conv::conv(conv, a.table_out ? a.table_out[bin] : v));
            out += 1ull << a.p_bits;
            lookup_count(a.counts[1], hot, 1, bin, active, direct);
        }
        for (uint32_t s = 0; s < ci.n_zeroing_chunks; s++) {
            const int64_t c = rem & 0xffff;
            rem >>= 16;
            if (s != ci.n_zeroing_chunks - 1 || ci.table_sign != DPB_SIGN_MIXED) {
                if (active) {
                    Conv::store(in, 0, Conv::conv(conv, c));
                    Conv::store(out, 0, Conv::conv(conv, c == 0 ? 1 : 0));
                }
                lookup_count(a.counts[2], hot, 2, (uint32_t)c, active);
            } else {
                const int64_t v = c - ci.top_zeroing_chunk_offset;
                const bool inside = v >= -32768 && v <= 32767;
                if (active && !inside) atomicOr(a.error, 1);
                if (active) {
                    Conv::store(in, 0, Conv::conv(conv, v));
                    Conv::store(out, 0, Conv::conv(conv, v > 0 ? 1 : v < 0 ? -1 : 0));
                }
                lookup_count(a.counts[3], hot, 3, (uint32_t)(v + 32768), active && inside);
            }
            in += 1ull << a.p_bits;
            out += 1ull << a.p_bits;
        }
    }
    __syncthreads();
    for (uint32_t t = threadIdx.x; t < 4 * kLookupCache; t += blockDim.x) {
        const uint32_t key = (&hot.key[0][0])[t], n = (&hot.cnt[0][0])[t];
        if (key != kLookupNoKey && n) atomicAdd(&a.counts[t / kLookupCache][key], (unsigned long long)n);
    }
    // start at a row that depends on the block, so that blocks ending together do not walk the table in step
    for (uint32_t t = threadIdx.x; t < a.direct_rows; t += blockDim.x) {
        const uint32_t r = (t + blockIdx.x * 97u) % a.direct_rows;
        if (direct[r]) atomicAdd(&a.counts[1][r], (unsigned long long)direct[r]);
    }
}

// multiplicity[i] = counts[i] as a field element (zkml/src/lookup/context.rs:313-371; the rows of these tables
// are distinct, their input column being a range, so no row's count is divided)
template <class F>
__global__ void lookup_multiplicities_kernel(const unsigned long long* __restrict__ counts, uint64_t n,
                                             typename SmallToField<F>::T* __restrict__ out) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t c = counts[i];
        if constexpr (std::is_same<F, FrFam>::value)
            FrFam::store(out, i, fr_from_u64(c));
        else
            out[i] = c >= GL_P ? c - GL_P : c;
    }
}

}  // namespace dpb
