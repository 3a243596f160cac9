// Internal C++ view of the engine handle (the C ABI in include/flashlstm_b200/engine.h wraps it).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <vector>

#include "flashlstm_b200/engine.h"

namespace flstm_b200 {

struct Comm;  // data-parallel communicator (comm.cu)

// Device-time accounting per phase with CUDA events; records only when enabled, never syncs
// until the totals are read.
enum Phase { PH_PROJ = 0, PH_RECUR_FWD, PH_BPTT, PH_WGRAD, PH_XGRAD, PH_ALLREDUCE, PH_COUNT };
struct PhaseTimer {
    bool enabled = false;
    std::vector<cudaEvent_t> pool;
    size_t used = 0;
    struct Span { int phase; size_t a, b; };
    std::vector<Span> spans;
    void reset() { used = 0; spans.clear(); }
    size_t mark(cudaStream_t s);
    void span(int phase, size_t a, size_t b) { if (enabled) spans.push_back({phase, a, b}); }
    int totals(float *out);
    ~PhaseTimer();
};

// Per-layer device buffers.  "T" below is the engine's storage type.
struct LayerBuffers {
    size_t in_size = 0;      // I_l
    void *w_ih = nullptr;    // T (4H, I_l)   SIMT: torch row order; TC: tile-interleaved rows
    void *w_hh = nullptr;    // T (4H, H)     same row order as w_ih
    float *bias = nullptr;   // fp32 (4H)     b_ih + b_hh, same order as the rows of w_ih
    void *gates = nullptr;   // T (Tcap, B, 4H)  input projection, overwritten by the gate cache
    void *hs = nullptr;      // T (Tcap+1, B, H) slot 0 = h0, slot t+1 = h_t
    float *cs = nullptr;     // fp32 (Tcap+1, B, H)
    void *dg = nullptr;      // T (Tcap, B, 4H)  pre-activation gradients (training)
    void *dx = nullptr;      // T (Tcap, B, I_l) gradient w.r.t. this layer's input (layers > 0)
    // activation-checkpoint mode (Engine::recompute > 0): the time-sized buffers above hold one segment
    void *y_all = nullptr;   // T (Tcap, B, H)  layers below the top: h_t for every step = the next layer's input
    void *ck_h = nullptr;    // T (K, B, H)     hidden state entering segment k
    float *ck_c = nullptr;   // fp32 (K, B, H)  cell state entering segment k
    float *dw_ih = nullptr;  // views into the flat gradient buffer
    float *dw_hh = nullptr;
    float *db = nullptr;
    size_t grad_offset = 0;  // element offset of this layer's [dW_ih | dW_hh | db] slice
    size_t grad_count = 0;
    bool weights_set = false;
};

struct Engine {
    flstm_engine_config cfg{};
    int backend = FLSTM_BACKEND_SIMT;
    int device = 0;
    size_t t_cap = 0;  // longest sequence the engine is currently sized for
    // Activation checkpoints (the reference's recompute interval R, flashlstm_v2/src/lstm_forward.cu:727-783,
    // lstm_backward.cu:975-1054): with recompute = R > 0 the forward keeps only the h/c state entering every
    // R-th step, and the backward re-runs the forward of one R-step segment at a time to rebuild its gate
    // cache.  gates / hs / cs / dg then span buf_steps = min(R, t_cap) steps instead of t_cap.
    size_t recompute = 0;
    size_t buf_steps = 0;
    size_t workspace_bytes = 0;  // bytes of the time-sized buffers currently allocated
    struct SegmentMode {
        bool active = false;         // the layer backward works on one segment with segment-local time indices
        bool final_segment = true;   // the segment that starts at t = 0: dh0/dc0 and the gradient allreduce follow it
        bool first_segment = true;   // the first one processed (the end of the sequence): weight gradients start from zero
        bool keep_gates = true;      // forward writes the activated gates back (off in the checkpointing forward pass)
    } seg;
    std::vector<LayerBuffers> layers;
    float *grads = nullptr;  // flat fp32: per layer [dW_ih | dW_hh | db]
    size_t grad_count = 0;
    float *dc_layers = nullptr;  // fp32 (L,B,H) cell-gradient carry, kept between backward ranges
    float *db_part = nullptr;  // TC: per batch-tile partial bias gradients
    unsigned int *sync_words = nullptr;  // TC: grid-barrier counters + error word
    size_t last_T = 0;       // sequence length of the last complete forward (0 = none)
    size_t fwd_progress = 0; // steps of the current forward already enqueued
    size_t bwd_progress = 0; // backward has been enqueued down to this step
    unsigned long long launches = 0;
    // Limit of every device-side wait of the persistent kernels in nanoseconds (0 = the kernels' 2 s default) and
    // the timeout self-test: a step barrier that waits for this many arrivals which nobody makes.
    unsigned long long wait_limit_ns = 0;
    unsigned int selftest_missing_arrivals = 0;
    bool cell_io_f32 = false;       // c0 / c_n cross the API as fp32 instead of the engine dtype
    const void *x_saved = nullptr;  // layer-0 input of the last forward (caller keeps it alive)
    PhaseTimer timer;
    Comm *comm = nullptr;
    bool comm_aborted = false;  // the watchdog gave up on a step: no collective until a new communicator is attached
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t comm_fork = nullptr, comm_join = nullptr;
    // second compute stream (created on first use): the two weight-gradient GEMMs of a layer run side by side on
    // disjoint halves of the SMs when that saves a round of tiles
    cudaStream_t aux_stream = nullptr;
    cudaEvent_t aux_fork = nullptr, aux_join = nullptr;
    int ensure_aux_stream();
    long long *trace = nullptr;  // device: [2 (fwd,bwd)][trace_steps][16] clock stamps of CTA 0
    int trace_steps = 0;
    void *tc_state = nullptr;  // tensor-core path: cached tensor maps etc. (tc_engine.cu)
    // CUDA-core path: persistent recurrent kernels when the shape fits (simt_persistent.cu)
    int simt_grid = 0;                       // 0: one launch per step
    unsigned int *simt_err_host = nullptr;   // pinned mirror of the error word
    int simt_check_error();
    float *simt_scratch = nullptr;           // split-K partial products of the weight-gradient GEMMs
    size_t simt_scratch_floats = 0;
    // Cross-layer wavefront (wide-batch path with stacked layers): layer l > 0 runs its time chunks on
    // lanes[l] one chunk behind layer l-1, so independent per-step kernels of different layers share the GPU.
    std::vector<cudaStream_t> lanes;        // lanes[0] is the caller's stream (not owned)
    std::vector<cudaEvent_t> lane_events;   // pool, reused call after call in stream order
    size_t lane_events_used = 0;
    // sum `count` floats of the flat gradient buffer at `offset` over the ranks, on the communication stream,
    // after everything enqueued on `from` so far (no-op without a communicator)
    int reduce_grads(size_t offset, size_t count, cudaStream_t from);
    int ensure_lanes(cudaStream_t s);
    cudaEvent_t next_lane_event();

    ~Engine();
    int allocate(size_t t_cap);
    void release_time_buffers();
    int ensure_capacity(size_t T);
    int set_weights(int layer, const float *w_ih, const float *w_hh, const float *b_ih, const float *b_hh,
                    cudaStream_t s);
    int forward(size_t T, const void *x, const void *h0, const void *c0, void *y, void *hn, void *cn,
                cudaStream_t s);
    int backward(size_t T, const void *dy, const void *dhn, const void *dcn, void *dx, float *dh0,
                 float *dc0, cudaStream_t s);
    int forward_range(size_t T, size_t t0, size_t t1, const void *x, const void *h0, const void *c0, void *y, void *hn,
                      void *cn, cudaStream_t s);
    int forward_checkpointed(size_t T, const void *x, const void *h0, const void *c0, void *y, void *hn, void *cn,
                             cudaStream_t s);
    int backward_checkpointed(size_t T, const void *dy, const void *dhn, const void *dcn, void *dx, float *dh0, float *dc0,
                              cudaStream_t s);
    int backward_segment(size_t n, bool last_in_time, bool first_in_time, const void *x_seg, const void *h_in,
                         const float *c_in, const void *dy_seg, const void *dhn, const void *dcn, void *dx_seg, float *dh0,
                         float *dc0, cudaStream_t s);
    int set_recompute(size_t R);
    int backward_range(size_t T, size_t t0, size_t t1, const void *dy, const void *dhn, const void *dcn, void *dx,
                       float *dh0, float *dc0, cudaStream_t s);
};

}  // namespace flstm_b200

// The opaque handle of the C ABI.
struct flstm_engine {
    flstm_b200::Engine impl;
};

namespace flstm_b200 {

// Tensor-core path entry points (tc_engine.cu).  `supported` decides AUTO resolution.
namespace tc {
bool supported(const flstm_engine_config &cfg);
int init(Engine &e);
void destroy(Engine &e);
int on_capacity_change(Engine &e);
int poll_error(Engine &e);  // reports (and clears) a device-side wait that expired in an earlier launch
int set_weights(Engine &e, int layer, const float *w_ih, const float *w_hh, const float *b_ih,
                const float *b_hh, cudaStream_t s);
int forward_layer(Engine &e, int layer, size_t t0, size_t t1, const void *x_l, void *y_out, cudaStream_t s);
// `dx_ready` (optional) is recorded on `s` once dx_l of the range is complete, before the weight gradients
int backward_layer(Engine &e, int layer, size_t T, size_t t0, size_t t1, const void *x_l, const void *dy_l,
                   const void *dhn_l, const void *dcn_l, void *dx_l, float *dh0_l, float *dc0_l, cudaStream_t s,
                   cudaEvent_t dx_ready = nullptr);
// steps per wavefront chunk for a range of n steps; 0 = no cross-layer wavefront for this engine
size_t wavefront_chunk(const Engine &e, size_t n);
}  // namespace tc

// Communicator (comm.cu): NCCL loaded at run time with dlopen.
int comm_unique_id(void *id128);
int comm_create(const void *id128, int rank, int world, Comm **out);
void comm_destroy(Comm *c);
void comm_abort(Comm *c);  // ncclCommAbort (falls back to destroy when the library lacks it), frees c
int comm_allreduce_sum_f32(Comm *c, float *buf, size_t count, cudaStream_t s);

}  // namespace flstm_b200
