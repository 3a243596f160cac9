// Device helpers shared by the persistent recurrent kernels (tc_lstm_fwd.cu, tc_lstm_bwd.cu): the
// global-memory step barrier, cluster / distributed-shared-memory primitives and 16-bit conversions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "tc_common.cuh"

namespace flstm_b200 {
namespace tc {

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int *p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Named barrier that also ORs a predicate over its `threads` participants: every participant arrives whatever
// its own bounded waits returned, and all of them leave with the same verdict, so nobody is left at the barrier
// by threads that gave up earlier.
__device__ __forceinline__ bool named_barrier_or(int id, int threads, bool pred) {
    uint32_t out;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 p, %3, 0;\n"
        "barrier.cta.red.or.pred q, %1, %2, p;\n"
        "selp.u32 %0, 1, 0, q;\n"
        "}\n"
        : "=r"(out)
        : "r"(id), "r"(threads), "r"((uint32_t)pred)
        : "memory");
    return out != 0;
}
// 16 bytes into a cluster peer's (or this CTA's) shared memory; their arrival is counted on the mbarrier at
// `bar_addr` (same CTA as `addr`), so the data carries its own completion signal: the sender neither waits for
// the stores nor sends an arrive after them
__device__ __forceinline__ void st_async_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t bar_addr) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(bar_addr) : "memory");
}
// Bounded poll of a monotonic counter written by other CTAs; `code` goes to the error word on expiry.
__device__ __forceinline__ bool wait_counter(const unsigned int *ctr, unsigned int target, unsigned int *err_word,
                                             volatile uint32_t *abort_w, unsigned int code,
                                             unsigned long long limit_ns = kWaitLimitNs) {
    if (ld_acquire_gpu(ctr) >= target) return true;
    const unsigned long long t0 = global_timer_ns();
    uint32_t spins = 0;
    while (ld_acquire_gpu(ctr) < target) {
        if ((++spins & 63u) == 0) {
            if (*abort_w) return false;
            if (*reinterpret_cast<volatile unsigned int *>(err_word)) {
                *abort_w = 1;
                return false;
            }
            if (global_timer_ns() - t0 > limit_ns) {
                *abort_w = 1;
                atomicExch(err_word, code);
                return false;
            }
        }
    }
    return true;
}

template <bool BF16>
__device__ __forceinline__ float load16(const uint16_t *p) {
    if (BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(p));
    return __half2float(*reinterpret_cast<const __half *>(p));
}
template <bool BF16>
__device__ __forceinline__ uint16_t to16(float v) {
    if (BF16) {
        __nv_bfloat16 h = __float2bfloat16_rn(v);
        return *reinterpret_cast<uint16_t *>(&h);
    }
    __half h = __float2half_rn(v);
    return *reinterpret_cast<uint16_t *>(&h);
}

}  // namespace tc
}  // namespace flstm_b200
