/*
 * Native engine C ABI of the B200 LSTM forward/backward engine.
 *
 * Everything crosses this boundary as plain pointers and sizes.  Pointers are DEVICE
 * pointers unless a comment says otherwise; `stream` arguments are cudaStream_t handles
 * passed as void* (NULL = the legacy default stream).  Every function returns a
 * flstm_status; the message of the last failure on the calling thread is available from
 * flstm_last_error().  No function aborts the process and none falls back to the CPU.
 *
 * The reference surfaces (include/flashlstm/lstm_api.h and include/lstm.hpp) are thin
 * shims over this handle API.  Compared with the reference's entry points
 * (include/flashlstm/lstm_api.h:23-56, flashlstm_v2/include/lstm.hpp:132-213) the handle
 * adds what those cannot express: stacked layers, BF16, device-resident I/O, a retained
 * gate cache for the backward pass and batch-sharded multi-GPU weight-gradient reduction.
 *
 * Semantics are torch.nn.LSTM's: gate row order i,f,g,o in every (4H, .) tensor; two
 * biases that are summed; seq-major contiguous (T,B,.) tensors; states shaped (L,B,H).
 */
#ifndef FLASHLSTM_B200_ENGINE_H
#define FLASHLSTM_B200_ENGINE_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    FLSTM_OK = 0,
    FLSTM_ERR_INVALID = 1,     /* bad argument / misuse                                   */
    FLSTM_ERR_CUDA = 2,        /* a CUDA runtime or driver call failed                    */
    FLSTM_ERR_TIMEOUT = 3,     /* a bounded device-side wait gave up (kernel returned)    */
    FLSTM_ERR_UNSUPPORTED = 4, /* shape / dtype not supported by the requested backend    */
    FLSTM_ERR_COMM = 5         /* communicator (NCCL) failure                             */
} flstm_status;

typedef enum {
    FLSTM_DTYPE_F32 = 0, /* fp32 storage, fp32 FMA arithmetic                             */
    FLSTM_DTYPE_F16 = 1, /* fp16 storage, fp32 accumulate, fp32 cell state                */
    FLSTM_DTYPE_BF16 = 2 /* bf16 storage, fp32 accumulate, fp32 cell state                */
} flstm_dtype;

typedef enum {
    FLSTM_BACKEND_AUTO = 0, /* tensor-core path when the shape allows it, else SIMT       */
    FLSTM_BACKEND_SIMT = 1, /* CUDA-core kernels: any shape, any dtype                    */
    FLSTM_BACKEND_TC = 2    /* tcgen05/TMEM + TMA kernels (16-bit dtypes, aligned shapes) */
} flstm_backend;

typedef struct {
    int dtype;          /* flstm_dtype: type of x, y, h0, c0, h_n, c_n, dY, d_hn, d_cn, dX */
    int layers;         /* >= 1                                                            */
    size_t batch;       /* per-GPU batch                                                   */
    size_t input_size;  /* I of layer 0 (upper layers consume H)                           */
    size_t hidden_size; /* H                                                               */
    size_t max_seq_len; /* workspace is sized for this T; a longer T grows it              */
    int training;       /* 1: forward keeps the gate cache + cell states for backward      */
    int backend;        /* flstm_backend                                                   */
} flstm_engine_config;

typedef struct flstm_engine flstm_engine;

/* Allocates the workspace on the CURRENT device.  Replaces the per-call cudaMalloc of
 * ~25 buffers in the reference (flashlstm_v2/src/lstm_forward.cu:555-645). */
int flstm_engine_create(const flstm_engine_config *config, flstm_engine **out);
int flstm_engine_destroy(flstm_engine *engine);

/* Snapshot + pack one layer's fp32 parameters (w_ih (4H,I_l), w_hh (4H,H), b_ih, b_hh (4H)).
 * Replaces pack_weights_kernel / FuseWeightsKernel / FuseBiasKernel
 * (src/kernels.cu:45-84, flashlstm_v2/src/lstm_forward.cu:180-217); done once per weight
 * update instead of on every forward and backward call. */
int flstm_engine_set_weights(flstm_engine *engine, int layer, const float *w_ih, const float *w_hh,
                             const float *b_ih, const float *b_hh, void *stream);

/* y (T,B,H), h_n/c_n (L,B,H) may be NULL when not wanted; h0/c0 NULL = zeros.
 * Asynchronous on `stream`.  In training mode x must stay valid and unchanged until the
 * matching flstm_engine_backward has been enqueued (it is re-read for dW_ih). */
int flstm_engine_forward(flstm_engine *engine, size_t seq_len, const void *x, const void *h0,
                         const void *c0, void *y, void *h_n, void *c_n, void *stream);

/* Consumes the cache of the LAST forward call.  dy (T,B,H); d_hn/d_cn (L,B,H) nullable;
 * dx (T,B,I) in the engine dtype, nullable; dh0/dc0 (L,B,H) fp32, nullable.  Weight and
 * bias gradients are written (not accumulated) into the engine's flat fp32 gradient buffer
 * (see flstm_engine_grad_ptrs).  With a communicator attached the flat buffer holds the
 * SUM over ranks when the call's work completes on `stream`. */
int flstm_engine_backward(flstm_engine *engine, size_t seq_len, const void *dy, const void *d_hn,
                          const void *d_cn, void *dx, float *dh0, float *dc0, void *stream);

/* The same work split into step ranges, so that a caller can overlap its own transfers with the
 * ranges already enqueued (what the reference's 32-step chunk pipeline does with pinned host
 * tensors, flashlstm_v2/src/lstm_forward.cu:673-940, lstm_backward.cu:899-1213).  x / y / dy / dx
 * are the base pointers of the WHOLE (T,B,.) tensors.  Forward ranges [t0,t1) must be contiguous and
 * ascending from 0; h_n / c_n are written by the range that ends at seq_len.  Backward ranges must
 * be contiguous and descending from seq_len; dX of a range is complete when the range's work is;
 * weight / bias gradients (and their allreduce), dh0 and dc0 are produced by the range with t0 == 0. */
int flstm_engine_forward_range(flstm_engine *engine, size_t seq_len, size_t t0, size_t t1, const void *x, const void *h0,
                               const void *c0, void *y, void *h_n, void *c_n, void *stream);
int flstm_engine_backward_range(flstm_engine *engine, size_t seq_len, size_t t0, size_t t1, const void *dy,
                                const void *d_hn, const void *d_cn, void *dx, float *dh0, float *dc0, void *stream);

/* Device pointers into the flat gradient buffer of one layer: dW_ih (4H,I_l), dW_hh (4H,H),
 * db (4H) (db_ih == db_hh == db, as in flashlstm_v2/src/lstm_backward.cu:1218-1231). */
int flstm_engine_grad_ptrs(flstm_engine *engine, int layer, float **dw_ih, float **dw_hh, float **db);
/* The whole flat buffer, layer after layer as [dW_ih | dW_hh | db]. */
int flstm_engine_grad_buffer(flstm_engine *engine, float **flat, size_t *count);

/* Post-activation gate cache of one layer from the last training forward: (T,B,4H) in the
 * engine dtype, plus the fp32 cell states (T+1,B,H) and the hidden states (T+1,B,H) whose
 * slot 0 is the initial state.  `gate_layout` is set to 0 when columns are in torch order
 * (g*H+u) and to 1 when they are tile-interleaved (((u/16)*4+g)*16 + u%16). */
int flstm_engine_cache_ptrs(flstm_engine *engine, int layer, void **gates, float **cells,
                            void **hiddens, int *gate_layout);

/* The cell state is fp32 inside the engine.  With this switch on, the c0 and c_n arguments of
 * flstm_engine_forward are fp32 (L,B,H) tensors instead of tensors in the engine dtype. */
int flstm_engine_set_cell_io_f32(flstm_engine *engine, int enabled);

/* Activation checkpoints instead of a full gate cache (the reference's recompute interval R,
 * flashlstm_v2/include/lstm.hpp:43-60, lstm_forward.cu:727-783, lstm_backward.cu:975-1054).  With
 * interval R > 0 the forward keeps only the h/c state entering every R-th step (plus each layer's output
 * sequence) and the backward re-runs the forward of one R-step segment at a time to rebuild its gates, so
 * the (T,B,4H) gate cache and dG shrink to (R,B,4H): 16 -> 2 bytes per (step, sequence, gate) at R = 8.
 * Outputs and state gradients are bit-identical to R = 0; weight gradients are summed segment by segment
 * (fp32) instead of in one pass.  Tensor-core backend only; whole-sequence calls only (no step ranges).
 * Call between sequences; it re-allocates the time-sized buffers.  flstm_engine_workspace_bytes returns
 * the bytes those buffers take now. */
int flstm_engine_set_recompute_interval(flstm_engine *engine, size_t interval);
size_t flstm_engine_workspace_bytes(const flstm_engine *engine);

/* Host streaming of sequences that do not fit the device (the reference keeps 2 x 32 steps of x / y / dY / dX on
 * the GPU and the rest in pinned host memory, flashlstm_v2/src/lstm_forward.cu:515,622-627,673-940,
 * lstm_backward.cu:496-523,899-1213).  The engine is created with max_seq_len = S and recompute interval S, so
 * its workspace holds ONE segment of S steps whatever the length of the sequence; the caller streams x, y, dY,
 * dX and the h/c checkpoints of the segment boundaries.
 *   forward : call flstm_engine_forward once per segment, in time order, with flstm_engine_set_cell_io_f32 on,
 *             feeding each call's h_n / c_n (fp32 cell state) to the next call as h0 / c0; the states entering a
 *             segment are its checkpoint.
 *   backward: call flstm_engine_backward_segment once per segment, LAST segment first.  x_seg / dy_seg / dx_seg
 *             are that segment's (steps,B,.) slices, h_in (L,B,H, engine dtype) and c_in (L,B,H, fp32) the
 *             checkpoint that entered it (NULL = zeros).  The engine re-runs the segment's forward from the
 *             checkpoint (rebuilding its gate cache), runs the BPTT over it and keeps the dh / dc carries for
 *             the next call; d_hn / d_cn are read by the call with last_in_time, dh0 / dc0 are written and the
 *             weight gradients are complete (and reduced over the ranks) after the call with first_in_time.
 * Results equal a single whole-sequence call up to the fp32 summation order of dW / db.  Tensor-core backend. */
int flstm_engine_backward_segment(flstm_engine *engine, size_t steps, int last_in_time, int first_in_time, const void *x_seg,
                                  const void *h_in, const float *c_in, const void *dy_seg, const void *d_hn, const void *d_cn,
                                  void *dx_seg, float *dh0, float *dc0, void *stream);

/* Which backend the engine resolved to (flstm_backend, never AUTO). */
int flstm_engine_backend(const flstm_engine *engine);

/* Batch-sharded data parallelism: one engine per GPU/process.  flstm_comm_unique_id fills a
 * 128-byte id on rank 0 (send it to the other ranks by any means); every rank then calls
 * flstm_engine_attach_comm.  The only collective is one sum-allreduce per layer over that
 * layer's slice of the flat gradient buffer, issued on an internal stream as soon as the
 * layer's weight-gradient kernels finish, so it overlaps the back-propagation of the layers
 * below it.  The reference has no multi-GPU path. */
int flstm_comm_unique_id(void *id128);
int flstm_engine_attach_comm(flstm_engine *engine, const void *id128, int rank, int world_size);

/* Host watchdog for a step: waits until everything enqueued on `stream` so far has finished, polling
 * without blocking in the driver, for at most `timeout_ms` milliseconds.  FLSTM_OK when the work is
 * done (a device-side wait that expired inside a kernel is reported here as FLSTM_ERR_TIMEOUT too).
 * When the deadline passes first the call returns FLSTM_ERR_TIMEOUT and, if a communicator is attached,
 * aborts it (ncclCommAbort) so that a collective a lost peer will never join cannot block this process;
 * backward then fails with FLSTM_ERR_COMM until flstm_engine_attach_comm is called again.
 * flstm_engine_abort_comm does the abort alone.  The reference has no counterpart (single GPU). */
int flstm_engine_wait(flstm_engine *engine, cudaStream_t stream, unsigned int timeout_ms);
int flstm_engine_abort_comm(flstm_engine *engine);

/* Every device-side wait of the persistent recurrent kernels (step barrier, mbarrier waits, cluster exchange)
 * gives up after a limit, 2 s unless set here (limit_us = 0 restores the default): the kernel raises an error
 * word, every role drains and the launch returns; the next call on the engine (or flstm_engine_wait) then
 * reports FLSTM_ERR_TIMEOUT and the engine stays usable.  The reference has no counterpart: its kernels never
 * wait on one another (flashlstm_v2/src/lstm_forward.cu:744-830 launches per step).
 * flstm_engine_selftest_missing_arrivals exercises that path without any fault: with arrivals = n > 0 every
 * step barrier of the following launches waits for n arrivals that no CTA makes, so the wait of the second
 * time step runs out after the limit.  Set a limit of a few milliseconds first; arrivals = 0 switches it off. */
int flstm_engine_set_wait_limit(flstm_engine *engine, unsigned long long limit_us);
int flstm_engine_selftest_missing_arrivals(flstm_engine *engine, unsigned int arrivals);

/* Per-phase device time of the last forward/backward pair in milliseconds (needs
 * flstm_engine_enable_timing(engine, 1); adds event records, no synchronisation).
 * out[0..5] = projection, recurrent forward, BPTT, weight-grad, input-grad, allreduce. */
int flstm_engine_enable_timing(flstm_engine *engine, int enabled);
int flstm_engine_phase_ms(flstm_engine *engine, float *out6);
/* Per-time-step profiling of the persistent kernels (tensor-core backend, layer 0): CTA 0 stamps
 * the SM clock at up to 16 points of each of the first `steps` time steps.  read_trace copies
 * 2 x steps x 16 values (forward kernel first, then BPTT) to host memory.  steps = 0 turns it off. */
int flstm_engine_enable_trace(flstm_engine *engine, int steps);
int flstm_engine_read_trace(flstm_engine *engine, long long *out_host, size_t count);
/* Number of kernels this library launched on behalf of `engine` since creation. */
unsigned long long flstm_engine_launch_count(const flstm_engine *engine);

/* How the tensor-core backend would lay a problem out on a GPU with `sm_count` SMs and `smem_limit`
 * bytes of opt-in shared memory per CTA (B200: 148, 232448): grids of the two persistent kernels,
 * batch tiling, TMA ring shape, whether the W_hh slices stay resident in shared memory; or, for wide
 * batches, the tile widths and K splits of the per-step GEMM launches.  Pure host
 * arithmetic (needs no device); FLSTM_ERR_UNSUPPORTED when the shape cannot be tiled. */
typedef struct {
    int fwd_batch_tile, fwd_row_tiles_per_cta, fwd_grid, fwd_batch_groups, fwd_tiles_per_group;
    int fwd_stages, fwd_chunks_per_stage, fwd_weights_resident, fwd_smem_bytes;
    int bwd_batch_tile, bwd_cluster_size, bwd_grid, bwd_batch_groups, bwd_tiles_per_group;
    int bwd_stages, bwd_chunks_per_stage, bwd_weights_resident, bwd_smem_bytes;
    /* wide batches run one GEMM launch per time step instead (then the fields above are zero) */
    int step_path, step_bn_fwd, step_bn_bwd, step_splits;
    int step_pair; /* the per-step GEMMs run on CTA pairs (256-sequence tiles, tcgen05 cta_group::2) */
    int fwd_pair;      /* persistent forward kernel: neighbouring row-tile CTAs form cta_group::2 pairs */
    int step_fwd_pair; /* wide batches: the all-steps forward kernel runs on CTA pairs (256-sequence tiles) */
} flstm_tc_plan_info;
int flstm_tc_plan(size_t batch, size_t hidden_size, int training, int sm_count, size_t smem_limit,
                  flstm_tc_plan_info *out);

/* The dense-contraction building block of the path on the tcgen05 tensor cores, exported for
 * unit tests and profiling: D[M,N] = A B^T (+ bias[N]) with f16/bf16 operands (`dtype`) and fp32
 * accumulation; D has dtype `out_dtype` (the operand dtype or FLSTM_DTYPE_F32) and row pitch ldd.
 *   layout 0: A is (M,K), B is (N,K), both row-major -- the input projection X W_ih^T
 *             (replaces the GEMMs of src/lstm_internal.h:48-68);
 *   layout 2: A is (M,K) row-major, B is stored (K,N) -- the input gradient dG W_ih, reading
 *             W_ih as it lies in memory (replaces flashlstm_v2/src/lstm_backward.cu:1159-1171);
 *   layout 1: A is stored (K,M), B is stored (K,N) -- the weight gradients dG^T [X|H], reduction
 *             dimension outermost (replaces flashlstm_v2/src/lstm_backward.cu:1112-1141); fp32 out.
 * Synchronous; returns FLSTM_ERR_TIMEOUT if a bounded device-side wait expired. */
int flstm_tc_gemm(int dtype, int out_dtype, size_t M, size_t N, size_t K, const void *A, const void *B,
                  void *D, size_t ldd, const float *bias, int layout, void *stream);

/* The bias-gradient reduction of the backward pass as a stand-alone call: db[c] = sum over `rows`
 * of dg[r][c] for a (rows, cols) matrix of dtype `dtype`, summed in a fixed order (two passes over
 * kernel-internal partial sums, so results are run-to-run identical).  With interleaved_h = H
 * (cols must be 4H) the columns are taken to be in the engine's tile-interleaved gate order and db
 * is written in torch order.  Replaces the ones-vector GEMV of
 * flashlstm_v2/src/lstm_backward.cu:1144-1156.  Allocates its scratch per call; synchronous. */
int flstm_bias_grad(int dtype, const void *dg, size_t rows, size_t cols, int interleaved_h, float *db, void *stream);

/* flstm_bias_grad without any allocation.  This entry point has no counterpart in the reference.
 * It is for callers that may not allocate device memory at call time: hosts that reserve all GPU
 * memory up front and forbid cudaMalloc in their serving or real-time loop (an allocation can block
 * or synchronise the device), code running where the CUDA allocator is off limits (during a stream
 * capture, inside another framework's allocator hooks), and embedders that must account for every
 * byte.  The partial sums live in a fixed 2 MiB array inside the library image, so:
 *   - cols may be at most 16384 (4H for H = 4096); wider input is rejected with
 *     FLSTM_ERR_UNSUPPORTED and a message naming the limit;
 *   - every GPU that loads the library holds the array until the process exits;
 *   - all calls share it: calls that may overlap on the GPU (different streams or threads) race and
 *     must be serialised by the caller.  Nothing needs clearing between calls.
 * The first call on each device looks up the array's device address (no allocation); make that
 * first call before starting a stream capture.  Asynchronous on `stream`; calls no cudaMalloc,
 * cudaFree or other allocating routine. */
int flstm_bias_grad_static(int dtype, const void *dg, size_t rows, size_t cols, int interleaved_h, float *db,
                           void *stream);

const char *flstm_last_error(void);
const char *flstm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASHLSTM_B200_ENGINE_H */
