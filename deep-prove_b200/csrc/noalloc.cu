// An entry point for callers that cannot allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a
// region that an outer runtime is capturing or replaying, under a memory
// manager that owns the whole device heap, or in a worker whose device memory
// budget was handed out up front.  For them dpb_product_round_noalloc computes
// the first sumcheck round of a product of tables (the same numbers
// dpb_sumcheck_begin + dpb_sumcheck_round produce) using only memory the
// caller passes in, plus a fixed scratch array that lives in this library's
// device image.
//
// The scratch array below is device memory reserved at load time on every GPU
// that loads the library (about 160 KiB, held until the process exits).  Its
// name is only a handle in host code: the address a kernel may use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
#include <mutex>

#include "common.cuh"
#include "fused_kernels.cuh"

namespace dpb {

constexpr uint32_t kNoallocMaxBlocks = 1024;
constexpr uint32_t kNoallocMaxTables = 4;
constexpr uint32_t kNoallocMaxLog2 = 30;  // tables of at most 2^30 entries
constexpr size_t kNoallocPartialBytes = (size_t)kNoallocMaxBlocks * (kNoallocMaxTables + 1) * sizeof(Fr);
constexpr size_t kNoallocCounterOffset = kNoallocPartialBytes;
constexpr size_t kNoallocScratchBytes = kNoallocPartialBytes + 256;

// per-block partial sums followed by the ticket counter
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoallocScratchBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_noalloc_mu;
static void* g_noalloc_ptr[kMaxDevices];  // device address of g_noalloc_scratch, per device

// Looks up (first call on the device) or returns the cached device address.
static int noalloc_scratch_for(int device, void** out) {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return fail(DPB_ECUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        g_noalloc_ptr[device] = p;
    }
    *out = g_noalloc_ptr[device];
    return DPB_OK;
}

template <class F, int K, bool BASE>
static void launch_noalloc(cudaStream_t s, const void* const* tables, uint64_t n_pairs, uint32_t grid, void* scratch,
                           void* out) {
    FusedPtrs<K> ptrs;
    for (int j = 0; j < K; j++) {
        ptrs.in[j] = tables[j];
        ptrs.out[j] = nullptr;
    }
    ReduceScratch<F> rs;
    rs.partials = (typename F::E*)scratch;
    rs.counter = (unsigned int*)((char*)scratch + kNoallocCounterOffset);
    rs.chunk_out = nullptr;
    rs.done_value = 0;
    fused_product_eval0<F, K, BASE><<<grid, kThreads, 0, s>>>(ptrs, n_pairs, rs, (typename F::E*)out);
}

template <class F, bool BASE>
static int dispatch_noalloc(cudaStream_t s, const void* const* tables, uint32_t k, uint64_t n_pairs, uint32_t grid,
                            void* scratch, void* out) {
    switch (k) {
        case 2: launch_noalloc<F, 2, BASE>(s, tables, n_pairs, grid, scratch, out); break;
        case 3: launch_noalloc<F, 3, BASE>(s, tables, n_pairs, grid, scratch, out); break;
        case 4: launch_noalloc<F, 4, BASE>(s, tables, n_pairs, grid, scratch, out); break;
        default: return fail(DPB_EINVAL, "table count %u outside 2..%u", k, kNoallocMaxTables);
    }
    return DPB_OK;
}

}  // namespace dpb

using namespace dpb;

extern "C" int dpb_product_round_noalloc(void* cuda_stream, int dtype, const void* const* tables_dev, uint32_t k,
                                         uint64_t len, void* out_evals_dev) {
    if (!tables_dev || !out_evals_dev) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(dtype)) return fail(DPB_EINVAL, "unknown dtype %d", dtype);
    if (is_int_dtype(dtype)) return fail(DPB_EINVAL, "this entry point takes field tables, not integer tables (dtype %d)", dtype);
    if (k < 2 || k > kNoallocMaxTables)
        return fail(DPB_EINVAL, "table count %u outside 2..%u", k, kNoallocMaxTables);
    if (!is_pow2(len) || len < 2) return fail(DPB_EINVAL, "length %llu is not a power of two >= 2", (unsigned long long)len);
    if (len > (1ull << kNoallocMaxLog2))
        return fail(DPB_EINVAL, "tables of %llu entries exceed this entry point's maximum of 2^%u",
                    (unsigned long long)len, kNoallocMaxLog2);
    for (uint32_t j = 0; j < k; j++)
        if (!tables_dev[j] || ((uintptr_t)tables_dev[j] & 15))
            return fail(DPB_EINVAL, "table %u is null or not 16-byte aligned", j);
    if ((uintptr_t)out_evals_dev & 15) return fail(DPB_EINVAL, "output is not 16-byte aligned");
    int device = -1;
    DPB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail(DPB_EINVAL, "device %d out of range", device);
    void* scratch = nullptr;
    DPB_TRY(noalloc_scratch_for(device, &scratch));
    cudaStream_t s = (cudaStream_t)cuda_stream;
    // the scratch array is per device: a stream of another GPU would run the kernel there with this GPU's address
    int stream_device = device;
    DPB_CUDA(cudaStreamGetDevice(s, &stream_device));
    if (stream_device != device)
        return fail(DPB_EINVAL, "the stream belongs to device %d but device %d is current", stream_device, device);
    // the ticket counter must start at zero even if an earlier call was cut short
    DPB_CUDA(cudaMemsetAsync((char*)scratch + kNoallocCounterOffset, 0, 256, s));
    const uint64_t n_pairs = len / 2;
    uint64_t blocks = (n_pairs + kThreads - 1) / kThreads;
    if (blocks > kNoallocMaxBlocks) blocks = kNoallocMaxBlocks;
    int rc;
    if (dtype == DPB_GL_BASE) rc = dispatch_noalloc<GlFam, true>(s, tables_dev, k, n_pairs, (uint32_t)blocks, scratch, out_evals_dev);
    else if (dtype == DPB_GL_EXT) rc = dispatch_noalloc<GlFam, false>(s, tables_dev, k, n_pairs, (uint32_t)blocks, scratch, out_evals_dev);
    else rc = dispatch_noalloc<FrFam, false>(s, tables_dev, k, n_pairs, (uint32_t)blocks, scratch, out_evals_dev);
    if (rc != DPB_OK) return rc;
    DPB_CUDA(cudaGetLastError());
    return DPB_OK;
}
