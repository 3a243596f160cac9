// Tensor-core (tcgen05 / TMEM / TMA) path of the engine.
#include "common.cuh"
#include "engine.h"
#include "kernels.h"

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

}  // namespace tc
}  // namespace flstm_b200
