// Column sums without any allocation: the same two-pass fixed-order reduction as
// volta_b200_colsum, but with its scratch partials in a buffer that is part of the library image.
//
// Who needs this: code that must not call the CUDA allocator at the point where it needs a
// bias gradient - a host thread inside a real-time or signal-like context where cudaMalloc's
// implicit device synchronisation and locking are unacceptable, a process that has handed all
// device memory to its own pool and has none left to give, or a plug-in whose host forbids
// allocator calls after start-up.  Such a caller still owns its input and output buffers; only
// the scratch comes from here.
#include <stdio.h>

#include <mutex>

#include "vb_common.cuh"

namespace {

// 1 Mi floats = 4 MiB of device memory on every GPU that loads this library, held until the
// process exits.  Enough for, e.g., 65536 x 4096 (77 824 floats) or 70000 x 130 (38 480).
constexpr long long kScratchFloats = 1LL << 20;
static __device__ __align__(256) float g_colsum_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
float *g_scratch_ptr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle; the kernels need its device address, which is
// looked up once per device with that device current.
cudaError_t scratch_for_current_device(float **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lk(g_mutex);
    if (!g_scratch_ptr[dev]) {
        float *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_colsum_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" int volta_b200_colsum_noalloc(float *out, const float *in, int64_t rows, int64_t cols, void *stream) {
    if (!out || !in || rows <= 0 || cols <= 0) return VB200_ERR_INVALID;
    const long long need = vb::colsum_chunks(rows, cols) * cols;
    if (need > kScratchFloats) {
        fprintf(stderr,
                "volta_b200_colsum_noalloc: a %lld x %lld input needs %lld scratch floats, the built-in scratch holds "
                "%lld; use volta_b200_colsum with caller-provided scratch\n",
                (long long)rows, (long long)cols, need, kScratchFloats);
        return VB200_ERR_TOO_LARGE;
    }
    float *scratch = nullptr;
    cudaError_t e = scratch_for_current_device(&scratch);
    if (e != cudaSuccess) {
        fprintf(stderr, "volta_b200_colsum_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
        return VB200_ERR_CUDA;
    }
    // Pass 1 writes every partial that pass 2 reads, so nothing in the scratch has to start at zero.
    e = vb::launch_colsum(out, in, rows, cols, scratch, (cudaStream_t)stream);
    return e == cudaSuccess ? VB200_OK : VB200_ERR_CUDA;
}
