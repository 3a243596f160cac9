// Shared device/host helpers: storage-type traits, status plumbing, activation math.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "flashlstm_b200/engine.h"

namespace flstm_b200 {

// ---------------------------------------------------------------- error plumbing
// The message of the last failure on this thread; flstm_last_error() returns it.
std::string &last_error_slot();
int set_error(int status, const char *fmt, ...);

#define FLSTM_CUDA_TRY(expr)                                                                  \
    do {                                                                                      \
        cudaError_t err__ = (expr);                                                           \
        if (err__ != cudaSuccess) {                                                           \
            return ::flstm_b200::set_error(FLSTM_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,    \
                                           cudaGetErrorString(err__), __FILE__, __LINE__);    \
        }                                                                                     \
    } while (0)

#define FLSTM_TRY(expr)                    \
    do {                                   \
        int st__ = (expr);                 \
        if (st__ != FLSTM_OK) return st__; \
    } while (0)

// ---------------------------------------------------------------- storage types
template <typename T>
struct Storage;
template <>
struct Storage<float> {
    static __device__ __forceinline__ float load(const float *p) { return *p; }
    static __device__ __forceinline__ void store(float *p, float v) { *p = v; }
};
template <>
struct Storage<__half> {
    static __device__ __forceinline__ float load(const __half *p) { return __half2float(*p); }
    static __device__ __forceinline__ void store(__half *p, float v) { *p = __float2half_rn(v); }
};
template <>
struct Storage<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};

template <typename T>
__device__ __forceinline__ float ld(const T *p) {
    return Storage<T>::load(p);
}
template <typename T>
__device__ __forceinline__ void st(T *p, float v) {
    Storage<T>::store(p, v);
}

inline size_t dtype_size(int dtype) { return dtype == FLSTM_DTYPE_F32 ? 4 : 2; }

// ---------------------------------------------------------------- activations (fp32)
// Accurate forms (expf / tanhf): the fp32 configuration is held to max-abs 2e-3 against
// torch, including weight gradients summed over T*B terms.
__device__ __forceinline__ float sigmoid_acc(float a) { return 1.0f / (1.0f + expf(-a)); }
__device__ __forceinline__ float tanh_acc(float a) { return tanhf(a); }

// Fast forms for the 16-bit paths: one MUFU.TANH; sigmoid(a) = 0.5*tanh(a/2) + 0.5.
// tanh.approx has ~2^-11 relative error, the size of an fp16 rounding step.
__device__ __forceinline__ float tanh_fast(float a) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(a));
    return y;
}
__device__ __forceinline__ float sigmoid_fast(float a) { return fmaf(0.5f, tanh_fast(0.5f * a), 0.5f); }

inline int ceil_div(size_t a, size_t b) { return static_cast<int>((a + b - 1) / b); }

// Opt-in dynamic shared memory above 48 KB.  cudaFuncSetAttribute acts on the CURRENT device only, so the
// largest limit set so far is remembered per (kernel, device); one process may drive several GPUs from
// several threads (engine.cu).  The limit of a kernel only ever grows: engines of different shapes share it.
cudaError_t ensure_smem_limit(const void *kernel, int bytes);
template <typename Kern>
inline cudaError_t ensure_smem_limit(Kern kernel, size_t bytes) {
    return ensure_smem_limit(reinterpret_cast<const void *>(kernel), static_cast<int>(bytes));
}

}  // namespace flstm_b200
