// Allocation-free variant of the bias-gradient reduction.
//
// Who needs this: callers that must not allocate device memory when they call into the library --
// a host that hands out all GPU memory up front and forbids cudaMalloc afterwards (real-time and
// serving loops where an allocation may block or synchronise the device), code running where the
// CUDA allocator is off limits (inside a stream capture, or inside another framework's allocator
// callback), and embedders whose memory accounting must see every byte.  flstm_bias_grad sizes and
// cudaMallocs its partial-sum scratch on every call; this entry point keeps that scratch in a
// fixed array that is part of the loaded library image instead.
//
// The price: the array (kStaticBiasGradMaxCols x 32 partial sums, 2 MiB) is resident on every GPU
// that loads the library until the process exits, it bounds the supported width, and it is shared
// by every call, so two calls that may run on the GPU at the same time (different streams or
// threads) race on it.  Every partial sum is written before it is read within one call, so the
// array needs no clearing between calls even though it keeps the previous call's contents.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace {

constexpr size_t kStaticBiasGradMaxCols = 16384;  // 4H for H = 4096, the widest benchmark configuration
static __device__ __align__(256) float g_bias_grad_scratch[flstm_b200::simt::kColumnSumSplits * kStaticBiasGradMaxCols];

// In host code the array's name is only a handle for the runtime, not a device address: the address
// kernels may use is looked up once per device, with that device current.
std::mutex g_setup_mutex;
float *g_scratch_addr[64] = {};

int scratch_for_current_device(float **out) {
    using flstm_b200::set_error;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return set_error(FLSTM_ERR_UNSUPPORTED, "device index %d is not supported", dev);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev]) {
        float *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_bias_grad_scratch);
        if (e != cudaSuccess || !ptr)
            return set_error(FLSTM_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return FLSTM_OK;
}

}  // namespace

extern "C" int flstm_bias_grad_static(int dtype, const void *dg, size_t rows, size_t cols, int interleaved_h, float *db,
                                      void *stream) {
    using namespace flstm_b200;
    if (!dg || !db) return set_error(FLSTM_ERR_INVALID, "null pointer argument");
    if (dtype < FLSTM_DTYPE_F32 || dtype > FLSTM_DTYPE_BF16) return set_error(FLSTM_ERR_INVALID, "bad dtype %d", dtype);
    if (interleaved_h < 0 || (interleaved_h && (size_t)interleaved_h * 4 != cols) || (interleaved_h % 16))
        return set_error(FLSTM_ERR_INVALID, "interleaved_h must be 0 or cols/4 (a multiple of 16)");
    if (cols > kStaticBiasGradMaxCols)
        return set_error(FLSTM_ERR_UNSUPPORTED,
                         "flstm_bias_grad_static supports at most %zu columns (got %zu): its scratch is a fixed array; "
                         "use flstm_bias_grad for wider matrices",
                         kStaticBiasGradMaxCols, cols);
    if (rows == 0 || cols == 0) return FLSTM_OK;
    float *scratch = nullptr;
    FLSTM_TRY(scratch_for_current_device(&scratch));
    return simt::column_sum_two_pass(dtype, dg, rows, cols, scratch, db, interleaved_h, static_cast<cudaStream_t>(stream));
}
