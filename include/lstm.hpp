/*
 * Streaming forward + backward v2 surface: the entry points bound by callers of the
 * reference's flashlstm_v2/include/lstm.hpp (its CPython extension
 * flashlstm_v2/python/flashlstm/_flashlstm_module.cpp:78-99,182-211 and the ctypes scripts
 * flashlstm_v2/scripts/validate_lstm_fwd.py:194-215, validate_lstm_bwd.py:333-363).
 *
 *   flstm::StreamingLstmForward   <- flashlstm_v2/include/lstm.hpp:43-70   (src/lstm_forward.cu:464)
 *   flstm::StreamingLstmBackward  <- flashlstm_v2/include/lstm.hpp:94-128  (src/lstm_backward.cu:643)
 *   flstm_StreamingLstmForward    <- flashlstm_v2/include/lstm.hpp:149-175(src/lstm_forward.cu:970)
 *   flstm_StreamingLstmBackward   <- flashlstm_v2/include/lstm.hpp:177-211(src/lstm_backward.cu:1253)
 *
 * Contract kept from the reference:
 *  - x, y, dY, dx and both checkpoint tensors are (pinned) HOST buffers; states, weights and
 *    gradients are DEVICE buffers.  Here a DEVICE pointer is also accepted for any of the
 *    host tensors (detected with cudaPointerGetAttributes) and is then used in place.
 *  - backward is stateless like the reference's: everything travels by pointer.  When it directly
 *    follows the forward of the same y tensor it consumes that forward's gate cache (and the weights
 *    that forward packed); otherwise, and always for sequences too long to stay on the device, it
 *    restores the state entering each segment from the CALLER'S h/c checkpoints and recomputes the
 *    segment (flashlstm_v2/src/lstm_backward.cu:496-523,975-1054).
 *  - x/y/dY/dx are fp16 (T,B,.); weights fp32 (4H,.) in gate order i,f,g,o; biases fp32 4H.
 *  - the "gate cache" is a pair of checkpoint tensors (ceil(T/R),B,H): entry k holds the h
 *    (resp. c) state ENTERING step k*R (entry 0 = h0/c0), stored as fp32 or fp16 according
 *    to the options (flashlstm_v2/src/lstm_forward.cu:727-783).
 *  - d_hn / d_cn may be null (zeros).  dW_ih, dW_hh, db_ih, db_hh are overwritten;
 *    db_ih == db_hh.  dh0/dc0 are fp32.
 *  - three distinct streams; recompute_interval >= 1; a zero-sized problem is a silent no-op;
 *    the call returns after all three streams have been synchronised.
 *  - NOTE the argument order: `options` follows the cache in the C++ functions and in the C
 *    forward, but is the LAST argument of the C backward.
 * Difference: the C++ functions throw std::runtime_error as the reference's do; the C
 * functions never abort the process (the reference's do, src/lstm_forward.cu:1029-1037) —
 * they record the failure, print it to stderr and return; query it with
 * flstm_last_error() / flstm_last_status() from include/flashlstm_b200/engine.h.
 */
#ifndef FLASHLSTM_V2_LSTM_HPP
#define FLASHLSTM_V2_LSTM_HPP

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>
#include <stddef.h>

#ifdef __cplusplus
namespace flstm {

enum class GateCacheDType : int { kFloat32 = 0, kFloat16 = 1 };

struct GateCacheHost {
    void *h_ptr;
    void *c_ptr;
};

struct StreamingLstmOptions {
    GateCacheDType h_dtype = GateCacheDType::kFloat32;
    GateCacheDType c_dtype = GateCacheDType::kFloat32;
};

void StreamingLstmForward(size_t time_steps, size_t batch_size, size_t input_size,
                          size_t hidden_size, size_t recompute_interval,
                          const __half *x_tensor_host, const __half *h0_device,
                          const __half *c0_device, const float *weights_ih,
                          const float *weights_hh, const float *bias_ih, const float *bias_hh,
                          __half *y_tensor_host, GateCacheHost gate_cache_host,
                          StreamingLstmOptions options, __half *hy_device, __half *cy_device,
                          cudaStream_t compute_stream, cudaStream_t h2d_stream,
                          cudaStream_t d2h_stream);

void StreamingLstmBackward(size_t time_steps, size_t batch_size, size_t input_size,
                           size_t hidden_size, size_t recompute_interval,
                           const __half *x_tensor_host, const __half *y_tensor_host,
                           GateCacheHost gate_cache_host, StreamingLstmOptions options,
                           const __half *dY_tensor_host, const __half *d_hn_device,
                           const __half *d_cn_device, const __half *h0_device,
                           const __half *c0_device, const float *weights_ih,
                           const float *weights_hh, const float *bias_ih, const float *bias_hh,
                           __half *dx_tensor_host, float *dW_ih, float *dW_hh, float *db_ih,
                           float *db_hh, float *dh0_out, float *dc0_out,
                           cudaStream_t compute_stream, cudaStream_t h2d_stream,
                           cudaStream_t d2h_stream);

}  // namespace flstm

extern "C" {
#endif

typedef enum { FLSTM_GATE_CACHE_FLOAT32 = 0, FLSTM_GATE_CACHE_FLOAT16 = 1 } flstm_GateCacheDType;

typedef struct {
    void *h_ptr;
    void *c_ptr;
} flstm_GateCacheHost;

typedef struct {
    flstm_GateCacheDType h_dtype;
    flstm_GateCacheDType c_dtype;
} flstm_StreamingLstmOptions;

void flstm_StreamingLstmForward(size_t time_steps, size_t batch_size, size_t input_size,
                                size_t hidden_size, size_t recompute_interval,
                                const __half *x_tensor_host, const __half *h0_device,
                                const __half *c0_device, const float *weights_ih,
                                const float *weights_hh, const float *bias_ih,
                                const float *bias_hh, __half *y_tensor_host,
                                flstm_GateCacheHost gate_cache_host,
                                const flstm_StreamingLstmOptions *options, __half *hy_device,
                                __half *cy_device, cudaStream_t compute_stream,
                                cudaStream_t h2d_stream, cudaStream_t d2h_stream);

void flstm_StreamingLstmBackward(size_t time_steps, size_t batch_size, size_t input_size,
                                 size_t hidden_size, size_t recompute_interval,
                                 const __half *x_tensor_host, const __half *y_tensor_host,
                                 flstm_GateCacheHost gate_cache_host,
                                 const __half *dY_tensor_host, const __half *d_hn_device,
                                 const __half *d_cn_device, const __half *h0_device,
                                 const __half *c0_device, const float *weights_ih,
                                 const float *weights_hh, const float *bias_ih,
                                 const float *bias_hh, __half *dx_tensor_host, float *dW_ih,
                                 float *dW_hh, float *db_ih, float *db_hh, float *dh0_out,
                                 float *dc0_out, cudaStream_t compute_stream,
                                 cudaStream_t h2d_stream, cudaStream_t d2h_stream,
                                 const flstm_StreamingLstmOptions *options);

/* Status of the last flstm_Streaming* call on this thread (a flstm_status value). */
int flstm_last_status(void);

/* Additions without a counterpart in the reference.
 * flstm_v2_set_weight_version: the reference converts and fuses the fp32 weights on every forward and every
 * backward call (flashlstm_v2/src/lstm_forward.cu:605, lstm_backward.cu:755), because the API passes bare
 * pointers and cannot know whether an optimiser has updated them in place.  A caller that can tell publishes a
 * non-zero version here and changes it whenever the weights change; calls then re-pack only when the version
 * or one of the four parameter pointers differs from the last packing.  Version 0 (the default) restores
 * "pack on every call".
 * flstm_v2_last_call_info: device bytes held by the context of the last flstm_Streaming* call on this thread
 * (engine workspace + staging) and whether it ran in streaming mode (the sequence processed in fixed-size
 * segments, footprint independent of T) or resident mode.  FLSTM_V2_DEVICE_BUDGET_BYTES caps the memory a
 * problem may take before streaming mode is chosen; FLSTM_V2_SEGMENT_STEPS fixes the segment length. */
void flstm_v2_set_weight_version(unsigned long long version);
void flstm_v2_last_call_info(size_t *device_bytes, int *streaming);

#ifdef __cplusplus
}
#endif
#endif /* FLASHLSTM_V2_LSTM_HPP */
