// mni_b200_add_bias_bwd_noalloc: the bias-add backward (copy of dy + column sums of dy) for
// callers that must not see this library allocate device memory.
//
// Who that is: a host runtime that owns the device's memory budget itself -- the reference's
// TensorStore hands out every buffer through its own caching allocator and assumes nobody else
// grows or frees device memory behind it -- and step loops that cannot afford cudaMalloc /
// cudaFree, which synchronise the whole device and so stall every stream of the process.  The
// regular entry point grows a library-owned scratch buffer on demand; this one never does.
//
// The column-sum kernels need a [slabs x n] block of partial sums.  Here that block lives in a
// fixed array in the library's device image (kNoAllocScratchBytes, 1 MiB): every GPU that loads
// the library carries it until the process exits, whether or not this entry point is used.
//
// Rules that follow from the shared array:
//   * Problems whose partial sums do not fit are refused with MNI_B200_ERR_WORKSPACE; nothing is
//     launched.  (1 MiB covers every n up to 262144 columns; typical bias widths need < 300 KiB.)
//   * All calls on a device use the same array, and it keeps whatever the previous call left in
//     it.  Nothing in it has to start at zero: the first kernel of a call writes every slot the
//     second kernel of that call reads, so stale contents are never observed.
//   * Two calls that run on the GPU at the same time (different streams, or different host
//     threads without ordering) write the same array and corrupt each other's sums.  Issue them
//     on one stream, or order them with events.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress) and caches it.  Make that first call during start-up, before any
//     stream capture is begun on that device.
#include "internal.h"

#include <mutex>

namespace {

constexpr size_t kNoAllocScratchBytes = 1u << 20;

// File-scope device array.  In host code this name is only a handle for the runtime's symbol
// lookup, never a device address: kernels get the pointer cudaGetSymbolAddress returns.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

struct NoAllocDevice {
    bool ready = false;
    float *scratch = nullptr;   // device address of g_noalloc_scratch on this device
    int sm_count = 0;
};
constexpr int kMaxDevices = 64;
NoAllocDevice g_state[kMaxDevices];
std::mutex g_state_mu;

// Per-device set-up, run with that device current.  No allocation: attribute queries and a
// symbol lookup only.
int noalloc_setup(NoAllocDevice **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return mni::fail(MNI_B200_ERR_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return mni::fail(MNI_B200_ERR_DEVICE, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_state_mu);
    NoAllocDevice &st = g_state[dev];
    if (!st.ready) {
        int major = 0, sms = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return mni::fail(MNI_B200_ERR_DEVICE, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        if (major != 10)
            return mni::fail(MNI_B200_ERR_DEVICE, "device %d is compute capability %d.x; this library only carries sm_100a code",
                             dev, major);
        float *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return mni::fail(MNI_B200_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        st.scratch = ptr;
        st.sm_count = sms;
        st.ready = true;
    }
    *out = &st;
    return MNI_B200_OK;
}

}  // namespace

extern "C" MNI_B200_API int mni_b200_add_bias_bwd_noalloc(const float *dy, float *d_y, float *dbias, int64_t rows,
                                                         int64_t n, uint32_t flags, void *stream) {
    if (rows < 0 || n < 0) return mni::fail(MNI_B200_ERR_ARG, "negative extent");
    if (!dy && rows * n > 0) return mni::fail(MNI_B200_ERR_ARG, "dy is null");
    NoAllocDevice *st = nullptr;
    int rc = noalloc_setup(&st);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool accumulate = (flags & MNI_B200_ACCUMULATE_DBIAS) != 0;
    size_t need = 0;
    if (dbias && n > 0 && rows > 0) {
        need = mni::colsum_partial_bytes(rows, n, st->sm_count);
        if (need > kNoAllocScratchBytes)
            return mni::fail(MNI_B200_ERR_WORKSPACE,
                             "add_bias_bwd_noalloc: %lld x %lld needs %zu bytes of partial sums, the built-in scratch "
                             "holds %zu; use mni_b200_add_bias_bwd for this size",
                             (long long)rows, (long long)n, need, kNoAllocScratchBytes);
    }
    if (d_y && d_y != dy) {
        rc = mni::launch_copy(dy, d_y, rows * n, s);
        if (rc) return rc;
    }
    if (!dbias || n == 0) return MNI_B200_OK;
    if (rows == 0) {
        if (!accumulate) MNI_CUDA(cudaMemsetAsync(dbias, 0, static_cast<size_t>(n) * sizeof(float), s));
        return MNI_B200_OK;
    }
    return mni::launch_colsum(dy, n, dbias, rows, n, accumulate, st->scratch, st->sm_count, s);
}
