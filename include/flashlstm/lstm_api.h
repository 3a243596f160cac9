/*
 * Forward-only v1 surface: the five entry points a caller of the reference's
 * include/flashlstm/lstm_api.h:23-56 binds (python/test_lstm.py:44-84 does so with ctypes).
 * Names, argument order and meaning are the reference's; the implementation behind them is
 * the B200 engine (include/flashlstm_b200/engine.h).
 *
 *   lstm_create_buffers   <- include/flashlstm/lstm_api.h:23-29  (src/lstm.cu:675-858)
 *   lstm_destroy_buffers  <- include/flashlstm/lstm_api.h:31     (src/lstm.cu:860-867)
 *   lstm_set_execution_mode <- include/flashlstm/lstm_api.h:33 (src/lstm.cu:869-884)
 *   lstm_pack_weights     <- include/flashlstm/lstm_api.h:35-40  (src/lstm.cu:886-931)
 *   lstm_forward          <- include/flashlstm/lstm_api.h:43-56  (src/lstm.cu:1897-2148)
 *
 * Contract kept from the reference: every pointer is DEVICE fp32; x (T,B,I), weights
 * (4H,.) row-major in gate order i,f,g,o, biases 4H, h0/c0/hn/cn (B,H), output (T,B,H);
 * batch/input/hidden sizes are fixed at creation and re-validated on each call; seq_len may
 * differ per call (the workspace grows); precision must match the one given at creation;
 * weights must have been packed; the call is synchronous; the return value is 0 on success
 * or a cudaError_t value (cudaErrorInvalidValue for misuse) with a message on stderr.
 * Both precision modes compute with fp16 operands and fp32 accumulation here (ACC16 is
 * served by the more accurate mode).  The execution mode is accepted and recorded; the
 * recurrent part is one persistent kernel, so there is no per-step launch stream for a
 * graph to remove.  input_proj_chunk_size is accepted and advisory.
 */
#ifndef FLASHLSTM_LSTM_API_H
#define FLASHLSTM_LSTM_API_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    LSTM_COMPUTE_PRECISION_FP16_ACC32 = 0,
    LSTM_COMPUTE_PRECISION_FP16_ACC16 = 1
} lstm_compute_precision_t;

typedef enum {
    LSTM_EXECUTION_MODE_IMMEDIATE = 0,
    LSTM_EXECUTION_MODE_GRAPH = 1
} lstm_execution_mode_t;

/* Opaque handle; `impl` is owned by the library between create and destroy. */
typedef struct lstm_buffers {
    void *impl;
} lstm_buffers;

int lstm_create_buffers(lstm_compute_precision_t precision, size_t seq_len, size_t batch,
                        size_t input_size, size_t hidden_size, int input_proj_chunk_size,
                        lstm_buffers *buffers);

int lstm_destroy_buffers(lstm_buffers *buffers);

int lstm_set_execution_mode(lstm_buffers *buffers, lstm_execution_mode_t mode);

/* Not in the reference: how many lstm_forward calls on this handle were served by replaying the captured
 * graph of GRAPH mode (the first call with a new seq_len or new tensor addresses runs directly and records). */
unsigned long long lstm_graph_replays(const lstm_buffers *buffers);

int lstm_pack_weights(lstm_compute_precision_t precision, const float *weight_ih,
                      const float *weight_hh, size_t input_size, size_t hidden_size,
                      lstm_buffers *buffers);

int lstm_forward(const float *x, const float *b_ih, const float *b_hh, const float *h0,
                 const float *c0, float *output, float *hn, float *cn, size_t seq_len,
                 size_t batch, size_t input_size, size_t hidden_size,
                 const lstm_buffers *buffers, lstm_compute_precision_t precision);

#ifdef __cplusplus
}
#endif
#endif /* FLASHLSTM_LSTM_API_H */
