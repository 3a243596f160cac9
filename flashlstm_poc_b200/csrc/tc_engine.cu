// Tensor-core (tcgen05 / TMEM / TMA) path of the engine.
#include "common.cuh"
#include "engine.h"
#include "kernels.h"
#include "tc_kernels.h"

namespace flstm_b200 {
namespace tc {

bool supported(const flstm_engine_config &) { return false; }
int init(Engine &) { return FLSTM_OK; }
void destroy(Engine &) {}
int on_capacity_change(Engine &) { return FLSTM_OK; }
int set_weights(Engine &, int, const float *, const float *, const float *, const float *, cudaStream_t) {
    return set_error(FLSTM_ERR_UNSUPPORTED, "tensor-core path not available");
}
int forward_layer(Engine &, int, size_t, const void *, void *, cudaStream_t) {
    return set_error(FLSTM_ERR_UNSUPPORTED, "tensor-core path not available");
}
int backward_layer(Engine &, int, size_t, const void *, const void *, const void *, const void *, void *, float *,
                   float *, cudaStream_t) {
    return set_error(FLSTM_ERR_UNSUPPORTED, "tensor-core path not available");
}


// A device word per device for the stand-alone entry points (never freed; 4 bytes).
static unsigned int *standalone_error_word() {
    static unsigned int *words[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!words[dev]) {
        if (cudaMalloc((void **)&words[dev], sizeof(unsigned int)) != cudaSuccess) return nullptr;
        cudaMemset(words[dev], 0, sizeof(unsigned int));
    }
    return words[dev];
}

int device_sm_count() {
    static int sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev] > 0 ? sms[dev] : 1;
}

}  // namespace tc
}  // namespace flstm_b200

extern "C" int flstm_tc_gemm(int dtype, int out_dtype, size_t M, size_t N, size_t K, const void *A, const void *B,
                             void *D, size_t ldd, const float *bias, int mn_major, void *stream) {
    using namespace flstm_b200;
    if (!A || !B || !D) return set_error(FLSTM_ERR_INVALID, "null pointer argument");
    unsigned int *err = tc::standalone_error_word();
    if (!err) return set_error(FLSTM_ERR_CUDA, "could not allocate the error word");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t lda = mn_major ? M : K, ldb = mn_major ? N : K;
    FLSTM_TRY(tc::gemm(dtype, out_dtype, M, N, K, A, lda, B, ldb, D, ldd, bias, mn_major != 0, err, tc::device_sm_count(), s));
    unsigned int h = 0;
    FLSTM_CUDA_TRY(cudaMemcpyAsync(&h, err, sizeof(h), cudaMemcpyDeviceToHost, s));
    FLSTM_CUDA_TRY(cudaStreamSynchronize(s));
    if (h) {
        cudaMemsetAsync(err, 0, sizeof(h), s);
        return set_error(FLSTM_ERR_TIMEOUT, "tensor-core GEMM: a bounded device-side wait expired");
    }
    return FLSTM_OK;
}
