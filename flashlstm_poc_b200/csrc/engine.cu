// Host orchestration of the engine: workspace lifetime, per-layer forward/backward
// scheduling, gradient buffer, data-parallel reduction and the C ABI.
//
// Role in the reference: src/lstm.cu (buffer object :192-319, forward entry :1897-2148) and the
// host loops of flashlstm_v2/src/lstm_forward.cu:464-966 / lstm_backward.cu:643-1250.  Unlike
// those, nothing is allocated, registered or re-packed per call: the handle owns a workspace
// sized at creation, weights are packed when they are set, and all work is enqueued
// asynchronously on the caller's stream.
#include "engine.h"

#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <thread>
#include <utility>

#include "common.cuh"
#include "kernels.h"

namespace flstm_b200 {

std::string &last_error_slot() {
    static thread_local std::string slot;
    return slot;
}

int set_error(int status, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_slot() = buf;
    return status;
}

cudaError_t ensure_smem_limit(const void *kernel, int bytes) {
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, int> limits;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    int &have = limits[{kernel, dev}];
    if (have >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) have = bytes;
    return e;
}

namespace {

template <typename P>
int dev_alloc(P **p, size_t bytes) {
    *p = nullptr;
    if (bytes == 0) return FLSTM_OK;
    void *raw = nullptr;
    cudaError_t e = cudaMalloc(&raw, bytes);
    if (e != cudaSuccess)
        return set_error(FLSTM_ERR_CUDA, "cudaMalloc(%zu bytes) failed: %s", bytes, cudaGetErrorString(e));
    *p = static_cast<P *>(raw);
    return FLSTM_OK;
}

template <typename P>
void dev_free(P *&p) {
    if (p) cudaFree(p);
    p = nullptr;
}

inline char *byte_ptr(void *p) { return static_cast<char *>(p); }
inline const char *byte_ptr(const void *p) { return static_cast<const char *>(p); }

}  // namespace

Engine::~Engine() {
    tc::destroy(*this);
    release_time_buffers();
    for (auto &l : layers) {
        dev_free(l.w_ih);
        dev_free(l.w_hh);
        dev_free(l.bias);
    }
    dev_free(grads);
    dev_free(dc_layers);
    dev_free(db_part);
    dev_free(sync_words);
    dev_free(trace);
    for (size_t i = 1; i < lanes.size(); ++i)
        if (lanes[i]) cudaStreamDestroy(lanes[i]);
    for (auto ev : lane_events) cudaEventDestroy(ev);
    if (simt_err_host) cudaFreeHost(simt_err_host);
    dev_free(simt_scratch);
    if (comm) comm_destroy(comm);
    if (comm_stream) cudaStreamDestroy(comm_stream);
    if (comm_fork) cudaEventDestroy(comm_fork);
    if (comm_join) cudaEventDestroy(comm_join);
    if (aux_stream) cudaStreamDestroy(aux_stream);
    if (aux_fork) cudaEventDestroy(aux_fork);
    if (aux_join) cudaEventDestroy(aux_join);
}

int Engine::ensure_aux_stream() {
    if (aux_stream) return FLSTM_OK;
    FLSTM_CUDA_TRY(cudaStreamCreateWithFlags(&aux_stream, cudaStreamNonBlocking));
    FLSTM_CUDA_TRY(cudaEventCreateWithFlags(&aux_fork, cudaEventDisableTiming));
    FLSTM_CUDA_TRY(cudaEventCreateWithFlags(&aux_join, cudaEventDisableTiming));
    return FLSTM_OK;
}

int Engine::reduce_grads(size_t offset, size_t count, cudaStream_t from) {
    if (!comm || count == 0) return FLSTM_OK;
    FLSTM_CUDA_TRY(cudaEventRecord(comm_fork, from));
    FLSTM_CUDA_TRY(cudaStreamWaitEvent(comm_stream, comm_fork, 0));
    size_t c0m = timer.mark(comm_stream);
    FLSTM_TRY(comm_allreduce_sum_f32(comm, grads + offset, count, comm_stream));
    size_t c1m = timer.mark(comm_stream);
    timer.span(PH_ALLREDUCE, c0m, c1m);
    return FLSTM_OK;
}

// A bounded wait that expired inside a persistent CUDA-core kernel is reported by the next call.
int Engine::simt_check_error() {
    if (simt_err_host && *simt_err_host) {
        const unsigned int code = *simt_err_host;
        *simt_err_host = 0;
        cudaMemset(sync_words, 0, sizeof(unsigned int));
        return set_error(FLSTM_ERR_TIMEOUT, "a bounded device-side wait expired in a persistent kernel (code %u)", code);
    }
    return FLSTM_OK;
}

int Engine::ensure_lanes(cudaStream_t s) {
    if (lanes.size() != layers.size()) {
        lanes.assign(layers.size(), nullptr);
        for (size_t i = 1; i < lanes.size(); ++i)
            FLSTM_CUDA_TRY(cudaStreamCreateWithFlags(&lanes[i], cudaStreamNonBlocking));
    }
    lanes[0] = s;
    lane_events_used = 0;
    return FLSTM_OK;
}

cudaEvent_t Engine::next_lane_event() {
    if (lane_events_used == lane_events.size()) {
        cudaEvent_t ev = nullptr;
        if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        lane_events.push_back(ev);
    }
    return lane_events[lane_events_used++];
}

void Engine::release_time_buffers() {
    for (auto &l : layers) {
        dev_free(l.gates);
        dev_free(l.hs);
        dev_free(l.cs);
        dev_free(l.dg);
        dev_free(l.dx);
        dev_free(l.y_all);
        dev_free(l.ck_h);
        dev_free(l.ck_c);
    }
    t_cap = 0;
    buf_steps = 0;
    workspace_bytes = 0;
}

int Engine::allocate(size_t cap) {
    const size_t B = cfg.batch, H = cfg.hidden_size, es = dtype_size(cfg.dtype);
    const bool tcp = backend == FLSTM_BACKEND_TC;
    const size_t bs = (recompute && recompute < cap) ? recompute : cap;  // steps the gate-sized buffers span
    const size_t segments = (cap + bs - 1) / bs;
    size_t total = 0;
    auto sized = [&](auto **p, size_t bytes) { total += bytes; return dev_alloc(p, bytes); };
    for (size_t li = 0; li < layers.size(); ++li) {
        auto &l = layers[li];
        FLSTM_TRY(sized(&l.gates, bs * B * 4 * H * es));
        FLSTM_TRY(sized(&l.hs, (bs + 1) * B * H * es));
        FLSTM_TRY(sized(&l.cs, (bs + 1) * B * H * sizeof(float)));
        if (cfg.training) {
            // with checkpoints one more slot: dG of the first step of the segment processed before
            FLSTM_TRY(sized(&l.dg, (bs + (recompute ? 1 : 0)) * B * 4 * H * es));
            if (li > 0) FLSTM_TRY(sized(&l.dx, cap * B * l.in_size * es));
        }
        if (recompute) {
            if (li + 1 < layers.size()) FLSTM_TRY(sized(&l.y_all, cap * B * H * es));
            FLSTM_TRY(sized(&l.ck_h, segments * B * H * es));
            FLSTM_TRY(sized(&l.ck_c, segments * B * H * sizeof(float)));
        }
    }
    t_cap = cap;
    buf_steps = bs;
    workspace_bytes = total;
    if (tcp) FLSTM_TRY(tc::on_capacity_change(*this));
    return FLSTM_OK;
}

int Engine::set_recompute(size_t R) {
    if (R && backend != FLSTM_BACKEND_TC)
        return set_error(FLSTM_ERR_UNSUPPORTED, "activation checkpoints need the tensor-core backend (f16/bf16, H %% 64 == 0)");
    if (R == recompute) return FLSTM_OK;
    FLSTM_CUDA_TRY(cudaDeviceSynchronize());
    const size_t cap = t_cap ? t_cap : 1;
    release_time_buffers();
    recompute = R;
    last_T = 0;
    return allocate(cap);
}

int Engine::ensure_capacity(size_t T) {
    if (T <= t_cap) return FLSTM_OK;
    // The reference grows its buffers when a call brings a longer sequence (src/lstm.cu:933-970).
    FLSTM_CUDA_TRY(cudaDeviceSynchronize());
    release_time_buffers();
    last_T = 0;
    return allocate(T);
}

int Engine::set_weights(int layer, const float *w_ih, const float *w_hh, const float *b_ih, const float *b_hh,
                        cudaStream_t s) {
    if (layer < 0 || layer >= (int)layers.size()) return set_error(FLSTM_ERR_INVALID, "layer %d out of range", layer);
    if (!w_ih || !w_hh || !b_ih || !b_hh) return set_error(FLSTM_ERR_INVALID, "null parameter pointer");
    auto &l = layers[layer];
    const size_t H = cfg.hidden_size;
    if (backend == FLSTM_BACKEND_TC) {
        FLSTM_TRY(tc::set_weights(*this, layer, w_ih, w_hh, b_ih, b_hh, s));
        launches += 5;
    } else {
        FLSTM_TRY(simt::convert(FLSTM_DTYPE_F32, w_ih, cfg.dtype, l.w_ih, 4 * H * l.in_size, s));
        FLSTM_TRY(simt::convert(FLSTM_DTYPE_F32, w_hh, cfg.dtype, l.w_hh, 4 * H * H, s));
        FLSTM_TRY(simt::bias_sum(b_ih, b_hh, l.bias, 4 * H, s));
        launches += 3;
    }
    l.weights_set = true;
    return FLSTM_OK;
}

int Engine::forward(size_t T, const void *x, const void *h0, const void *c0, void *y, void *hn, void *cn,
                    cudaStream_t s) {
    return forward_range(T, 0, T, x, h0, c0, y, hn, cn, s);
}

// Steps [t0, t1) of a T-step forward.  Ranges must be issued in ascending order starting at 0; x and
// y are the base pointers of the whole (T, B, .) tensors.  Splitting a sequence into ranges lets a
// caller overlap its own copies (host streaming) with the ranges already enqueued.
int Engine::forward_range(size_t T, size_t t0, size_t t1, const void *x, const void *h0, const void *c0, void *y,
                          void *hn, void *cn, cudaStream_t s) {
    const size_t B = cfg.batch, H = cfg.hidden_size, es = dtype_size(cfg.dtype);
    if (T == 0 || B == 0 || H == 0) return FLSTM_OK;  // zero-sized problem: silent no-op (lstm_forward.cu:493-495)
    if (!x) return set_error(FLSTM_ERR_INVALID, "x is null");
    if (t0 >= t1 || t1 > T) return set_error(FLSTM_ERR_INVALID, "bad step range [%zu, %zu) of %zu", t0, t1, T);
    if (recompute) {
        if (t0 != 0 || t1 != T)
            return set_error(FLSTM_ERR_UNSUPPORTED, "step ranges are not available with activation checkpoints");
        return forward_checkpointed(T, x, h0, c0, y, hn, cn, s);
    }
    const int L = (int)layers.size();
    const size_t slab = B * H;
    if (t0 == 0) {
        for (auto &l : layers)
            if (!l.weights_set) return set_error(FLSTM_ERR_INVALID, "weights have not been set for every layer");
        FLSTM_TRY(ensure_capacity(T));
        timer.reset();
        x_saved = x;
        last_T = 0;
        fwd_progress = 0;
    } else if (fwd_progress != t0) {
        return set_error(FLSTM_ERR_INVALID, "forward ranges must be contiguous and ascending (expected start %zu, got %zu)", fwd_progress, t0);
    }
    if (t0 == 0) {
        // initial state -> slot 0 of the state tensors
        for (int li = 0; li < L; ++li) {
            auto &l = layers[li];
            if (h0) FLSTM_CUDA_TRY(cudaMemcpyAsync(l.hs, byte_ptr(h0) + li * slab * es, slab * es, cudaMemcpyDeviceToDevice, s));
            else FLSTM_CUDA_TRY(cudaMemsetAsync(l.hs, 0, slab * es, s));
            const size_t ces = cell_io_f32 ? sizeof(float) : es;
            if (c0) { FLSTM_TRY(simt::convert(cell_io_f32 ? FLSTM_DTYPE_F32 : cfg.dtype, byte_ptr(c0) + li * slab * ces, FLSTM_DTYPE_F32, l.cs, slab, s)); ++launches; }
            else FLSTM_CUDA_TRY(cudaMemsetAsync(l.cs, 0, slab * sizeof(float), s));
        }
    }
    const size_t wave = backend == FLSTM_BACKEND_TC ? tc::wavefront_chunk(*this, t1 - t0) : 0;
    if (wave) {
        // Cross-layer wavefront: layer l works on time chunk k while layer l-1 is already on chunk k+1.
        FLSTM_TRY(ensure_lanes(s));
        cudaEvent_t fork = next_lane_event();
        if (!fork) return set_error(FLSTM_ERR_CUDA, "cudaEventCreate failed");
        FLSTM_CUDA_TRY(cudaEventRecord(fork, s));
        for (int li = 1; li < L; ++li) FLSTM_CUDA_TRY(cudaStreamWaitEvent(lanes[li], fork, 0));
        for (size_t c0s = t0; c0s < t1; c0s += wave) {
            const size_t c1s = c0s + wave < t1 ? c0s + wave : t1;
            cudaEvent_t prev = nullptr;
            for (int li = 0; li < L; ++li) {
                if (prev) FLSTM_CUDA_TRY(cudaStreamWaitEvent(lanes[li], prev, 0));
                const void *x_l = li == 0 ? x : byte_ptr(layers[li - 1].hs) + slab * es;
                FLSTM_TRY(tc::forward_layer(*this, li, c0s, c1s, x_l, (li == L - 1) ? y : nullptr, lanes[li]));
                if (li + 1 < L || c1s == t1) {
                    prev = next_lane_event();
                    if (!prev) return set_error(FLSTM_ERR_CUDA, "cudaEventCreate failed");
                    FLSTM_CUDA_TRY(cudaEventRecord(prev, lanes[li]));
                    if (c1s == t1 && li > 0) FLSTM_CUDA_TRY(cudaStreamWaitEvent(s, prev, 0));  // join
                }
            }
        }
    } else {
        for (int li = 0; li < L; ++li) {
            auto &l = layers[li];
            const void *x_l = li == 0 ? x : byte_ptr(layers[li - 1].hs) + slab * es;
            void *y_out = (li == L - 1) ? y : nullptr;
            if (backend == FLSTM_BACKEND_TC) {
                FLSTM_TRY(tc::forward_layer(*this, li, t0, t1, x_l, y_out, s));
            } else {
                // input projection for the steps of the range at once: P = X W_ih^T + (b_ih + b_hh)
                size_t m0 = timer.mark(s);
                FLSTM_TRY(simt::gemm(cfg.dtype, cfg.dtype, (t1 - t0) * B, 4 * H, l.in_size, byte_ptr(x_l) + t0 * B * l.in_size * es,
                                     l.in_size, true, l.w_ih, l.in_size, true, byte_ptr(l.gates) + t0 * B * 4 * H * es, 4 * H,
                                     l.bias, s));
                ++launches;
                size_t m1 = timer.mark(s);
                if (simt_grid) {
                    FLSTM_TRY(simt_check_error());
                    const size_t tiles = (size_t)simt::persistent_batch_tiles(B);
                    FLSTM_CUDA_TRY(cudaMemsetAsync(sync_words + 32, 0, tiles * sizeof(unsigned int), s));
                    simt::PersistentFwdParams pp{};
                    pp.w_hh = l.w_hh;
                    pp.hs = l.hs;
                    pp.cs = l.cs;
                    pp.gates = l.gates;
                    pp.y = y_out;
                    pp.counters = sync_words + 32;
                    pp.err = sync_words;
                    pp.B = (int)B;
                    pp.H = (int)H;
                    pp.t0 = (int)t0;
                    pp.T = (int)(t1 - t0);
                    pp.store_gates = 1;
                    pp.wait_ns = wait_limit_ns;
                    pp.extra_arrivals = selftest_missing_arrivals;
                    FLSTM_TRY(simt::persistent_forward(cfg.dtype, simt_grid, pp, s));
                    FLSTM_CUDA_TRY(cudaMemcpyAsync(simt_err_host, sync_words, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
                    ++launches;
                } else {
                    for (size_t t = t0; t < t1; ++t) {
                        FLSTM_TRY(simt::step_forward(cfg.dtype, B, H, byte_ptr(l.hs) + t * slab * es, l.w_hh,
                                                     byte_ptr(l.gates) + t * B * 4 * H * es, l.cs + t * slab,
                                                     l.cs + (t + 1) * slab, byte_ptr(l.hs) + (t + 1) * slab * es,
                                                     y_out ? byte_ptr(y_out) + t * slab * es : nullptr, s));
                    }
                    launches += t1 - t0;
                }
                size_t m2 = timer.mark(s);
                timer.span(PH_PROJ, m0, m1);
                timer.span(PH_RECUR_FWD, m1, m2);
            }
        }
    }
    if (t1 == T) {
        const size_t ces = cell_io_f32 ? sizeof(float) : es;
        for (int li = 0; li < L; ++li) {
            auto &l = layers[li];
            if (hn) FLSTM_CUDA_TRY(cudaMemcpyAsync(byte_ptr(hn) + li * slab * es, byte_ptr(l.hs) + T * slab * es, slab * es, cudaMemcpyDeviceToDevice, s));
            if (cn) { FLSTM_TRY(simt::convert(FLSTM_DTYPE_F32, l.cs + T * slab, cell_io_f32 ? FLSTM_DTYPE_F32 : cfg.dtype, byte_ptr(cn) + li * slab * ces, slab, s)); ++launches; }
        }
    }
    fwd_progress = t1;
    if (t1 == T) {
        last_T = T;
        bwd_progress = T;
    }
    return FLSTM_OK;
}

// Activation-checkpoint forward: segments of buf_steps steps run through the segment-sized buffers with
// segment-local time indices; the state entering each segment is kept, the gate cache is not written.
int Engine::forward_checkpointed(size_t T, const void *x, const void *h0, const void *c0, void *y, void *hn, void *cn,
                                 cudaStream_t s) {
    const size_t B = cfg.batch, H = cfg.hidden_size, es = dtype_size(cfg.dtype), slab = B * H;
    const int L = (int)layers.size();
    for (auto &l : layers)
        if (!l.weights_set) return set_error(FLSTM_ERR_INVALID, "weights have not been set for every layer");
    FLSTM_TRY(ensure_capacity(T));
    timer.reset();
    x_saved = x;
    last_T = 0;
    const size_t R = buf_steps, ces = cell_io_f32 ? sizeof(float) : es;
    struct Restore { Engine &e; ~Restore() { e.seg = SegmentMode{}; } } restore{*this};  // also on early error returns
    seg.keep_gates = false;
    int st = FLSTM_OK;
    for (int li = 0; li < L && st == FLSTM_OK; ++li) {
        auto &l = layers[li];
        if (h0) FLSTM_CUDA_TRY(cudaMemcpyAsync(l.hs, byte_ptr(h0) + li * slab * es, slab * es, cudaMemcpyDeviceToDevice, s));
        else FLSTM_CUDA_TRY(cudaMemsetAsync(l.hs, 0, slab * es, s));
        if (c0) { FLSTM_TRY(simt::convert(cell_io_f32 ? FLSTM_DTYPE_F32 : cfg.dtype, byte_ptr(c0) + li * slab * ces, FLSTM_DTYPE_F32, l.cs, slab, s)); ++launches; }
        else FLSTM_CUDA_TRY(cudaMemsetAsync(l.cs, 0, slab * sizeof(float), s));
        const void *x_l = li == 0 ? x : layers[li - 1].y_all;
        void *y_l = (li == L - 1) ? y : l.y_all;
        size_t k = 0;
        for (size_t seg0 = 0; seg0 < T && st == FLSTM_OK; seg0 += R, ++k) {
            const size_t n = T - seg0 < R ? T - seg0 : R;
            // checkpoint k: the state entering the segment (slot 0)
            FLSTM_CUDA_TRY(cudaMemcpyAsync(byte_ptr(l.ck_h) + k * slab * es, l.hs, slab * es, cudaMemcpyDeviceToDevice, s));
            FLSTM_CUDA_TRY(cudaMemcpyAsync(l.ck_c + k * slab, l.cs, slab * sizeof(float), cudaMemcpyDeviceToDevice, s));
            st = tc::forward_layer(*this, li, 0, n, byte_ptr(x_l) + seg0 * B * l.in_size * es,
                                   y_l ? byte_ptr(y_l) + seg0 * slab * es : nullptr, s);
            if (st != FLSTM_OK) break;
            // the state leaving the segment enters the next one
            FLSTM_CUDA_TRY(cudaMemcpyAsync(l.hs, byte_ptr(l.hs) + n * slab * es, slab * es, cudaMemcpyDeviceToDevice, s));
            FLSTM_CUDA_TRY(cudaMemcpyAsync(l.cs, l.cs + n * slab, slab * sizeof(float), cudaMemcpyDeviceToDevice, s));
        }
        if (st != FLSTM_OK) break;
        if (hn) FLSTM_CUDA_TRY(cudaMemcpyAsync(byte_ptr(hn) + li * slab * es, l.hs, slab * es, cudaMemcpyDeviceToDevice, s));
        if (cn) { FLSTM_TRY(simt::convert(FLSTM_DTYPE_F32, l.cs, cell_io_f32 ? FLSTM_DTYPE_F32 : cfg.dtype, byte_ptr(cn) + li * slab * ces, slab, s)); ++launches; }
    }
    seg.keep_gates = true;
    FLSTM_TRY(st);
    fwd_progress = T;
    last_T = T;
    bwd_progress = T;
    return FLSTM_OK;
}

// Activation-checkpoint backward: segments from the last to the first; per layer the forward of the segment
// is re-run from its checkpoint (rebuilding gates, h and c in the segment buffers), then the BPTT runs over
// it with the gradient carries (dc in dc_layers, dh as dG of the next step / partial sums) kept between
// segments, and the weight gradients accumulate segment by segment.
int Engine::backward_checkpointed(size_t T, const void *dy, const void *dhn, const void *dcn, void *dx, float *dh0,
                                  float *dc0, cudaStream_t s) {
    const size_t B = cfg.batch, H = cfg.hidden_size, es = dtype_size(cfg.dtype), slab = B * H;
    const int L = (int)layers.size();
    const size_t R = buf_steps, K = (T + R - 1) / R;
    struct Restore { Engine &e; ~Restore() { e.seg = SegmentMode{}; } } restore{*this};  // also on early error returns
    seg.active = true;
    int st = FLSTM_OK;
    for (size_t kk = K; kk-- > 0 && st == FLSTM_OK;) {
        const size_t seg0 = kk * R, n = T - seg0 < R ? T - seg0 : R;
        seg.final_segment = kk == 0;
        seg.first_segment = kk == K - 1;
        const size_t T_loc = (kk == K - 1) ? n : n + 1;  // slot n of dG then holds the step after the segment
        for (int li = L - 1; li >= 0 && st == FLSTM_OK; --li) {
            auto &l = layers[li];
            FLSTM_CUDA_TRY(cudaMemcpyAsync(l.hs, byte_ptr(l.ck_h) + kk * slab * es, slab * es, cudaMemcpyDeviceToDevice, s));
            FLSTM_CUDA_TRY(cudaMemcpyAsync(l.cs, l.ck_c + kk * slab, slab * sizeof(float), cudaMemcpyDeviceToDevice, s));
            const void *x_seg = li == 0 ? byte_ptr(x_saved) + seg0 * B * l.in_size * es
                                        : byte_ptr(layers[li - 1].y_all) + seg0 * slab * es;
            st = tc::forward_layer(*this, li, 0, n, x_seg, nullptr, s);  // recompute
            if (st != FLSTM_OK) break;
            const void *dy_seg = byte_ptr((li == L - 1) ? dy : layers[li + 1].dx) + seg0 * slab * es;
            void *dx_seg = li == 0 ? (dx ? byte_ptr(dx) + seg0 * B * l.in_size * es : nullptr) : byte_ptr(l.dx) + seg0 * slab * es;
            st = tc::backward_layer(*this, li, T_loc, 0, n, x_seg, dy_seg, dhn ? byte_ptr(dhn) + li * slab * es : nullptr,
                                    dcn ? byte_ptr(dcn) + li * slab * es : nullptr, dx_seg,
                                    (kk == 0 && dh0) ? dh0 + li * slab : nullptr, (kk == 0 && dc0) ? dc0 + li * slab : nullptr, s);
            if (st != FLSTM_OK) break;
            if (kk > 0)  // dG of the segment's first step: what the segment before it continues from
                FLSTM_CUDA_TRY(cudaMemcpyAsync(byte_ptr(l.dg) + R * B * 4 * H * es, l.dg, B * 4 * H * es, cudaMemcpyDeviceToDevice, s));
        }
    }
    seg = SegmentMode{};
    FLSTM_TRY(st);
    if (comm) {
        FLSTM_CUDA_TRY(cudaEventRecord(comm_join, comm_stream));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(s, comm_join, 0));
    }
    bwd_progress = 0;
    return FLSTM_OK;
}

int Engine::backward(size_t T, const void *dy, const void *dhn, const void *dcn, void *dx, float *dh0,
                     float *dc0, cudaStream_t s) {
    return backward_range(T, 0, T, dy, dhn, dcn, dx, dh0, dc0, s);
}

// One segment of a sequence that is streamed through the engine from outside (host streaming): the caller owns
// x, dY, dX and the h/c checkpoints, the engine holds one segment of gates / states / dG at a time.  Segments are
// passed from the LAST one to the FIRST.  Per layer the forward of the segment is re-run from the state that
// entered it (h_in 16-bit, c_in fp32, both (L,B,H)), then the BPTT runs over it with the gradient carries kept
// inside the engine between calls (dc in dc_layers, dh as dG of the following step in the extra dG slot / the
// partial sums of the wide-batch path); weight and bias gradients accumulate from call to call and are complete
// (and reduced over the ranks) after the call with `first_in_time`.
int Engine::backward_segment(size_t n, bool last_in_time, bool first_in_time, const void *x_seg, const void *h_in,
                             const float *c_in, const void *dy_seg, const void *dhn, const void *dcn, void *dx_seg,
                             float *dh0, float *dc0, cudaStream_t s) {
    const size_t B = cfg.batch, H = cfg.hidden_size, es = dtype_size(cfg.dtype), slab = B * H;
    const int L = (int)layers.size();
    if (!cfg.training) return set_error(FLSTM_ERR_INVALID, "engine was created with training = 0");
    if (backend != FLSTM_BACKEND_TC || !recompute)
        return set_error(FLSTM_ERR_UNSUPPORTED, "segment backward needs the tensor-core backend with a recompute interval set");
    if (n == 0 || n > buf_steps) return set_error(FLSTM_ERR_INVALID, "segment of %zu steps does not fit the %zu-step buffers", n, buf_steps);
    if (!x_seg || !dy_seg) return set_error(FLSTM_ERR_INVALID, "null pointer argument");
    if (comm_aborted) return set_error(FLSTM_ERR_COMM, "the communicator was aborted after a step missed its deadline; attach a new one");
    for (auto &l : layers)
        if (!l.weights_set) return set_error(FLSTM_ERR_INVALID, "weights have not been set for every layer");
    if (last_in_time) timer.reset();
    struct Restore { Engine &e; ~Restore() { e.seg = SegmentMode{}; } } restore{*this};
    seg.active = true;
    seg.first_segment = last_in_time;   // the first one processed: weight gradients start from zero
    seg.final_segment = first_in_time;  // the one that starts the sequence: dh0 / dc0 and the allreduce follow it
    seg.keep_gates = true;
    // recompute: rebuild gates, h and c of the segment, layer by layer, in the segment buffers
    for (int li = 0; li < L; ++li) {
        auto &l = layers[li];
        if (h_in) FLSTM_CUDA_TRY(cudaMemcpyAsync(l.hs, byte_ptr(h_in) + li * slab * es, slab * es, cudaMemcpyDeviceToDevice, s));
        else FLSTM_CUDA_TRY(cudaMemsetAsync(l.hs, 0, slab * es, s));
        if (c_in) FLSTM_CUDA_TRY(cudaMemcpyAsync(l.cs, c_in + li * slab, slab * sizeof(float), cudaMemcpyDeviceToDevice, s));
        else FLSTM_CUDA_TRY(cudaMemsetAsync(l.cs, 0, slab * sizeof(float), s));
        const void *x_l = li == 0 ? x_seg : byte_ptr(layers[li - 1].hs) + slab * es;
        FLSTM_TRY(tc::forward_layer(*this, li, 0, n, x_l, nullptr, s));
    }
    const size_t T_loc = last_in_time ? n : n + 1;  // slot n of dG then holds the step after the segment
    for (int li = L - 1; li >= 0; --li) {
        auto &l = layers[li];
        const void *x_l = li == 0 ? x_seg : byte_ptr(layers[li - 1].hs) + slab * es;
        const void *dy_l = (li == L - 1) ? dy_seg : layers[li + 1].dx;
        void *dx_l = li == 0 ? dx_seg : l.dx;
        FLSTM_TRY(tc::backward_layer(*this, li, T_loc, 0, n, x_l, dy_l, dhn ? byte_ptr(dhn) + li * slab * es : nullptr,
                                     dcn ? byte_ptr(dcn) + li * slab * es : nullptr, dx_l,
                                     (first_in_time && dh0) ? dh0 + li * slab : nullptr,
                                     (first_in_time && dc0) ? dc0 + li * slab : nullptr, s));
        if (!first_in_time)  // dG of the segment's first step: what the segment before it continues from
            FLSTM_CUDA_TRY(cudaMemcpyAsync(byte_ptr(l.dg) + buf_steps * B * 4 * H * es, l.dg, B * 4 * H * es,
                                           cudaMemcpyDeviceToDevice, s));
    }
    if (comm && first_in_time) {
        FLSTM_CUDA_TRY(cudaEventRecord(comm_join, comm_stream));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(s, comm_join, 0));
    }
    return FLSTM_OK;
}

// Time steps [t0, t1) of the backward pass, in reverse.  Ranges must be issued in descending order,
// the first one ending at T; dy and dx are base pointers of the whole tensors.  dX of a range is
// complete when the range's work is; the weight and bias gradients (and their allreduce) are formed
// by the last range (t0 == 0).
int Engine::backward_range(size_t T, size_t t0, size_t t1, const void *dy, const void *dhn, const void *dcn, void *dx,
                           float *dh0, float *dc0, cudaStream_t s) {
    const size_t B = cfg.batch, H = cfg.hidden_size, es = dtype_size(cfg.dtype);
    if (T == 0 || B == 0 || H == 0) return FLSTM_OK;
    if (!cfg.training) return set_error(FLSTM_ERR_INVALID, "engine was created with training = 0");
    if (comm_aborted) return set_error(FLSTM_ERR_COMM, "the communicator was aborted after a step missed its deadline; attach a new one");
    if (last_T != T) return set_error(FLSTM_ERR_INVALID, "backward(T=%zu) does not follow a forward of the same length (last T=%zu)", T, last_T);
    if (!dy) return set_error(FLSTM_ERR_INVALID, "dy is null");
    if (t0 >= t1 || t1 > T) return set_error(FLSTM_ERR_INVALID, "bad step range [%zu, %zu) of %zu", t0, t1, T);
    if (bwd_progress != t1) return set_error(FLSTM_ERR_INVALID, "backward ranges must be contiguous and descending (expected end %zu, got %zu)", bwd_progress, t1);
    if (recompute) {
        if (t0 != 0 || t1 != T)
            return set_error(FLSTM_ERR_UNSUPPORTED, "step ranges are not available with activation checkpoints");
        return backward_checkpointed(T, dy, dhn, dcn, dx, dh0, dc0, s);
    }
    const int L = (int)layers.size();
    const size_t slab = B * H;
    const size_t n = t1 - t0;  // steps in the range
    const size_t wave = backend == FLSTM_BACKEND_TC ? tc::wavefront_chunk(*this, n) : 0;
    if (wave) {
        // Cross-layer wavefront, descending in time: layer l takes chunk k as soon as layer l+1 has produced
        // its dX for that chunk; weight gradients of a layer follow its last chunk on the layer's own lane.
        FLSTM_TRY(ensure_lanes(s));
        cudaEvent_t fork = next_lane_event();
        if (!fork) return set_error(FLSTM_ERR_CUDA, "cudaEventCreate failed");
        FLSTM_CUDA_TRY(cudaEventRecord(fork, s));
        for (int li = 1; li < L; ++li) FLSTM_CUDA_TRY(cudaStreamWaitEvent(lanes[li], fork, 0));
        for (size_t c1s = t1; c1s > t0;) {
            const size_t c0s = (c1s - t0 > wave) ? c1s - wave : t0;
            cudaEvent_t above = nullptr;  // dX of this chunk from the layer above
            for (int li = L - 1; li >= 0; --li) {
                auto &l = layers[li];
                if (above) FLSTM_CUDA_TRY(cudaStreamWaitEvent(lanes[li], above, 0));
                const void *x_l = li == 0 ? x_saved : byte_ptr(layers[li - 1].hs) + slab * es;
                const void *dy_l = (li == L - 1) ? dy : layers[li + 1].dx;
                void *dx_l = li == 0 ? dx : l.dx;
                cudaEvent_t ready = nullptr;
                if (li > 0) {
                    ready = next_lane_event();
                    if (!ready) return set_error(FLSTM_ERR_CUDA, "cudaEventCreate failed");
                }
                FLSTM_TRY(tc::backward_layer(*this, li, T, c0s, c1s, x_l, dy_l, dhn ? byte_ptr(dhn) + li * slab * es : nullptr,
                                             dcn ? byte_ptr(dcn) + li * slab * es : nullptr, dx_l, dh0 ? dh0 + li * slab : nullptr,
                                             dc0 ? dc0 + li * slab : nullptr, lanes[li], ready));
                above = ready;
                if (c0s == t0 && li > 0) {  // join the lane after its last chunk of the range
                    cudaEvent_t done = next_lane_event();
                    if (!done) return set_error(FLSTM_ERR_CUDA, "cudaEventCreate failed");
                    FLSTM_CUDA_TRY(cudaEventRecord(done, lanes[li]));
                    FLSTM_CUDA_TRY(cudaStreamWaitEvent(s, done, 0));
                }
            }
            c1s = c0s;
        }
        if (comm && t0 == 0) {
            FLSTM_CUDA_TRY(cudaEventRecord(comm_join, comm_stream));
            FLSTM_CUDA_TRY(cudaStreamWaitEvent(s, comm_join, 0));
        }
        bwd_progress = t0;
        return FLSTM_OK;
    }
    for (int li = L - 1; li >= 0; --li) {
        auto &l = layers[li];
        const void *x_l = li == 0 ? x_saved : byte_ptr(layers[li - 1].hs) + slab * es;
        const void *dy_l = (li == L - 1) ? dy : layers[li + 1].dx;
        void *dx_l = li == 0 ? dx : l.dx;
        const void *dhn_l = dhn ? byte_ptr(dhn) + li * slab * es : nullptr;
        const void *dcn_l = dcn ? byte_ptr(dcn) + li * slab * es : nullptr;
        float *dh0_l = dh0 ? dh0 + li * slab : nullptr;
        float *dc0_l = dc0 ? dc0 + li * slab : nullptr;
        if (backend == FLSTM_BACKEND_TC) {
            FLSTM_TRY(tc::backward_layer(*this, li, T, t0, t1, x_l, dy_l, dhn_l, dcn_l, dx_l, dh0_l, dc0_l, s));
        } else {
            float *dc_l = dc_layers + li * slab;  // the carry survives between ranges, one per layer
            size_t m0 = timer.mark(s);
            if (t1 == T) {
                if (dcn_l) { FLSTM_TRY(simt::convert(cfg.dtype, dcn_l, FLSTM_DTYPE_F32, dc_l, slab, s)); ++launches; }
                else FLSTM_CUDA_TRY(cudaMemsetAsync(dc_l, 0, slab * sizeof(float), s));
            }
            if (simt_grid) {
                FLSTM_TRY(simt_check_error());
                const size_t tiles = (size_t)simt::persistent_batch_tiles(B);
                FLSTM_CUDA_TRY(cudaMemsetAsync(sync_words + 32, 0, tiles * sizeof(unsigned int), s));
                simt::PersistentBwdParams pp{};
                pp.w_hh = l.w_hh;
                pp.cs = l.cs;
                pp.gates = l.gates;
                pp.dg = l.dg;
                pp.dy = dy_l;
                pp.dhn = dhn_l;
                pp.dc = dc_l;
                pp.dh0 = dh0_l;
                pp.dc0 = dc0_l;
                pp.counters = sync_words + 32;
                pp.err = sync_words;
                pp.B = (int)B;
                pp.H = (int)H;
                pp.T = (int)T;
                pp.s0 = (int)(T - t1);
                pp.s1 = (int)(T - t0) + ((t0 == 0 && (dh0_l || dc0_l)) ? 1 : 0);  // the last range also forms dh0 / dc0
                pp.wait_ns = wait_limit_ns;
                pp.extra_arrivals = selftest_missing_arrivals;
                FLSTM_TRY(simt::persistent_backward(cfg.dtype, simt_grid, pp, s));
                FLSTM_CUDA_TRY(cudaMemcpyAsync(simt_err_host, sync_words, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
                ++launches;
            } else {
                for (size_t step = 0; step < n; ++step) {
                    size_t t = t1 - 1 - step;
                    const void *dg_next = (t == T - 1) ? nullptr : byte_ptr(l.dg) + (t + 1) * B * 4 * H * es;
                    FLSTM_TRY(simt::step_backward(cfg.dtype, B, H, dg_next, l.w_hh, dhn_l,
                                                  byte_ptr(dy_l) + t * slab * es,
                                                  byte_ptr(l.gates) + t * B * 4 * H * es, l.cs + (t + 1) * slab,
                                                  l.cs + t * slab, dc_l, byte_ptr(l.dg) + t * B * 4 * H * es, s));
                }
                launches += n;
            }
            size_t m1 = timer.mark(s), m2 = m1;
            if (t0 == 0) {
                if (!simt_grid) {
                    if (dh0_l) { FLSTM_TRY(simt::final_dh(cfg.dtype, B, H, l.dg, l.w_hh, dh0_l, s)); ++launches; }
                    if (dc0_l) FLSTM_CUDA_TRY(cudaMemcpyAsync(dc0_l, dc_l, slab * sizeof(float), cudaMemcpyDeviceToDevice, s));
                }
                // deferred parameter gradients over the whole sequence
                FLSTM_TRY(simt::gemm(cfg.dtype, FLSTM_DTYPE_F32, 4 * H, l.in_size, T * B, l.dg, 4 * H, false, x_l,
                                     l.in_size, false, l.dw_ih, l.in_size, nullptr, s, simt_scratch, simt_scratch_floats));
                FLSTM_TRY(simt::gemm(cfg.dtype, FLSTM_DTYPE_F32, 4 * H, H, T * B, l.dg, 4 * H, false, l.hs, H, false,
                                     l.dw_hh, H, nullptr, s, simt_scratch, simt_scratch_floats));
                FLSTM_TRY(simt::column_sum(cfg.dtype, l.dg, T * B, 4 * H, l.db, s));
                launches += 3;
                m2 = timer.mark(s);
            }
            if (dx_l) {
                FLSTM_TRY(simt::gemm(cfg.dtype, cfg.dtype, n * B, l.in_size, 4 * H, byte_ptr(l.dg) + t0 * B * 4 * H * es, 4 * H,
                                     true, l.w_ih, l.in_size, false, byte_ptr(dx_l) + t0 * B * l.in_size * es, l.in_size,
                                     nullptr, s));
                ++launches;
            }
            size_t m3 = timer.mark(s);
            timer.span(PH_BPTT, m0, m1);
            timer.span(PH_WGRAD, m1, m2);
            timer.span(PH_XGRAD, m2, m3);
        }
        // reduce this layer's gradients while the layers below keep back-propagating (the tensor-core path
        // starts its reductions itself, block by block, as the weight-gradient kernels finish)
        if (t0 == 0 && backend != FLSTM_BACKEND_TC) FLSTM_TRY(reduce_grads(l.grad_offset, l.grad_count, s));
    }
    if (comm && t0 == 0) {
        FLSTM_CUDA_TRY(cudaEventRecord(comm_join, comm_stream));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(s, comm_join, 0));
    }
    bwd_progress = t0;
    return FLSTM_OK;
}

}  // namespace flstm_b200

namespace flstm_b200 {

// ------------------------------------------------------------------ phase timer
size_t PhaseTimer::mark(cudaStream_t s) {
    if (!enabled) return 0;
    if (used == pool.size()) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) return 0;
        pool.push_back(e);
    }
    cudaEventRecord(pool[used], s);
    return used++;
}

int PhaseTimer::totals(float *out) {
    for (int i = 0; i < PH_COUNT; ++i) out[i] = 0.f;
    for (auto &sp : spans) {
        if (sp.a >= used || sp.b >= used) continue;
        if (cudaEventSynchronize(pool[sp.b]) != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "event sync failed");
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, pool[sp.a], pool[sp.b]) == cudaSuccess) out[sp.phase] += ms;
    }
    return FLSTM_OK;
}

PhaseTimer::~PhaseTimer() {
    for (auto e : pool) cudaEventDestroy(e);
}

}  // namespace flstm_b200

// ====================================================================== C ABI
using flstm_b200::Engine;
using flstm_b200::set_error;

namespace {
// Every entry point works on the engine's own device, whatever device is current on the calling thread,
// and leaves the caller's current device as it found it.
struct DeviceScope {
    int prev = -1;
    bool switched = false;
    explicit DeviceScope(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceScope() {
        if (switched) cudaSetDevice(prev);
    }
};
}  // namespace

extern "C" {

int flstm_engine_create(const flstm_engine_config *config, flstm_engine **out) {
    if (!config || !out) return set_error(FLSTM_ERR_INVALID, "null argument");
    *out = nullptr;
    if (config->dtype < FLSTM_DTYPE_F32 || config->dtype > FLSTM_DTYPE_BF16)
        return set_error(FLSTM_ERR_INVALID, "bad dtype %d", config->dtype);
    if (config->layers < 1 || config->layers > 64) return set_error(FLSTM_ERR_INVALID, "layers must be in [1,64]");
    if (config->batch == 0 || config->input_size == 0 || config->hidden_size == 0)
        return set_error(FLSTM_ERR_INVALID, "batch, input_size and hidden_size must be positive");
    if (config->backend < FLSTM_BACKEND_AUTO || config->backend > FLSTM_BACKEND_TC)
        return set_error(FLSTM_ERR_INVALID, "bad backend %d", config->backend);
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
        return set_error(FLSTM_ERR_CUDA, "no CUDA device: this library has no CPU path");
    flstm_engine *h = new (std::nothrow) flstm_engine();
    if (!h) return set_error(FLSTM_ERR_INVALID, "out of host memory");
    Engine &e = h->impl;
    e.cfg = *config;
    cudaGetDevice(&e.device);
    const bool tc_ok = flstm_b200::tc::supported(*config);
    if (config->backend == FLSTM_BACKEND_TC && !tc_ok) {
        delete h;
        return set_error(FLSTM_ERR_UNSUPPORTED,
                         "tensor-core backend needs a 16-bit dtype, hidden_size %% 64 == 0, input_size %% 64 == 0 and "
                         "batch %% 8 == 0 on an sm_100 device");
    }
    e.backend = (config->backend == FLSTM_BACKEND_AUTO) ? (tc_ok ? FLSTM_BACKEND_TC : FLSTM_BACKEND_SIMT) : config->backend;
    const size_t H = config->hidden_size, B = config->batch, es = flstm_b200::dtype_size(config->dtype);
    e.layers.resize(config->layers);
    size_t total = 0;
    for (int li = 0; li < config->layers; ++li) {
        auto &l = e.layers[li];
        l.in_size = li == 0 ? config->input_size : H;
        l.grad_offset = total;
        l.grad_count = 4 * H * l.in_size + 4 * H * H + 4 * H;
        total += l.grad_count;
    }
    e.grad_count = total;
    int st = FLSTM_OK;
    auto fail = [&](int code) { delete h; return code; };
    {
        void *raw = nullptr;
        if (cudaMalloc(&raw, total * sizeof(float)) != cudaSuccess) return fail(set_error(FLSTM_ERR_CUDA, "cudaMalloc of the gradient buffer failed"));
        e.grads = static_cast<float *>(raw);
        cudaMemset(raw, 0, total * sizeof(float));
        if (cudaMalloc(&raw, (size_t)config->layers * B * H * sizeof(float)) != cudaSuccess) return fail(set_error(FLSTM_ERR_CUDA, "cudaMalloc failed"));
        e.dc_layers = static_cast<float *>(raw);
    }
    for (auto &l : e.layers) {
        l.dw_ih = e.grads + l.grad_offset;
        l.dw_hh = l.dw_ih + 4 * H * l.in_size;
        l.db = l.dw_hh + 4 * H * H;
        void *raw = nullptr;
        if (cudaMalloc(&raw, 4 * H * l.in_size * es) != cudaSuccess) return fail(set_error(FLSTM_ERR_CUDA, "cudaMalloc failed"));
        l.w_ih = raw;
        if (cudaMalloc(&raw, 4 * H * H * es) != cudaSuccess) return fail(set_error(FLSTM_ERR_CUDA, "cudaMalloc failed"));
        l.w_hh = raw;
        if (cudaMalloc(&raw, 4 * H * sizeof(float)) != cudaSuccess) return fail(set_error(FLSTM_ERR_CUDA, "cudaMalloc failed"));
        l.bias = static_cast<float *>(raw);
    }
    if (e.backend == FLSTM_BACKEND_TC) {
        st = flstm_b200::tc::init(e);
        if (st != FLSTM_OK) return fail(st);
    } else {
        if (config->training) {
            // room for up to 8 partial products of the largest weight gradient, at most 64 MiB
            size_t widest = config->input_size > H ? config->input_size : H;
            size_t floats = 8 * 4 * H * widest;
            if (floats > (size_t)16 << 20) floats = (size_t)16 << 20;
            void *raw = nullptr;
            if (cudaMalloc(&raw, floats * sizeof(float)) == cudaSuccess) {
                e.simt_scratch = static_cast<float *>(raw);
                e.simt_scratch_floats = floats;
            } else {
                cudaGetLastError();  // the GEMMs then run unsplit
            }
        }
        int grid = 0;
        if (flstm_b200::simt::persistent_fits(config->dtype, B, H, config->training != 0, &grid)) {
            void *raw = nullptr;
            const size_t words = 32 + (size_t)flstm_b200::simt::persistent_batch_tiles(B);
            if (cudaMalloc(&raw, words * sizeof(unsigned int)) != cudaSuccess) return fail(set_error(FLSTM_ERR_CUDA, "cudaMalloc failed"));
            e.sync_words = static_cast<unsigned int *>(raw);
            cudaMemset(raw, 0, words * sizeof(unsigned int));
            if (cudaMallocHost(&raw, sizeof(unsigned int)) != cudaSuccess) return fail(set_error(FLSTM_ERR_CUDA, "cudaMallocHost failed"));
            e.simt_err_host = static_cast<unsigned int *>(raw);
            *e.simt_err_host = 0;
            e.simt_grid = grid;
        }
    }
    st = e.allocate(config->max_seq_len ? config->max_seq_len : 1);
    if (st != FLSTM_OK) return fail(st);
    *out = h;
    return FLSTM_OK;
}

int flstm_engine_destroy(flstm_engine *engine) {
    if (!engine) return FLSTM_OK;
    DeviceScope scope(engine->impl.device);
    cudaDeviceSynchronize();
    delete engine;
    return FLSTM_OK;
}

int flstm_engine_set_weights(flstm_engine *engine, int layer, const float *w_ih, const float *w_hh,
                             const float *b_ih, const float *b_hh, void *stream) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    DeviceScope scope(engine->impl.device);
    return engine->impl.set_weights(layer, w_ih, w_hh, b_ih, b_hh, static_cast<cudaStream_t>(stream));
}

int flstm_engine_forward(flstm_engine *engine, size_t seq_len, const void *x, const void *h0, const void *c0,
                         void *y, void *h_n, void *c_n, void *stream) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    DeviceScope scope(engine->impl.device);
    return engine->impl.forward(seq_len, x, h0, c0, y, h_n, c_n, static_cast<cudaStream_t>(stream));
}

int flstm_engine_backward(flstm_engine *engine, size_t seq_len, const void *dy, const void *d_hn,
                          const void *d_cn, void *dx, float *dh0, float *dc0, void *stream) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    DeviceScope scope(engine->impl.device);
    return engine->impl.backward(seq_len, dy, d_hn, d_cn, dx, dh0, dc0, static_cast<cudaStream_t>(stream));
}

int flstm_engine_forward_range(flstm_engine *engine, size_t seq_len, size_t t0, size_t t1, const void *x, const void *h0,
                               const void *c0, void *y, void *h_n, void *c_n, void *stream) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    DeviceScope scope(engine->impl.device);
    return engine->impl.forward_range(seq_len, t0, t1, x, h0, c0, y, h_n, c_n, static_cast<cudaStream_t>(stream));
}

int flstm_engine_backward_range(flstm_engine *engine, size_t seq_len, size_t t0, size_t t1, const void *dy,
                                const void *d_hn, const void *d_cn, void *dx, float *dh0, float *dc0, void *stream) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    DeviceScope scope(engine->impl.device);
    return engine->impl.backward_range(seq_len, t0, t1, dy, d_hn, d_cn, dx, dh0, dc0, static_cast<cudaStream_t>(stream));
}

int flstm_engine_backward_segment(flstm_engine *engine, size_t steps, int last_in_time, int first_in_time, const void *x_seg,
                                  const void *h_in, const float *c_in, const void *dy_seg, const void *d_hn, const void *d_cn,
                                  void *dx_seg, float *dh0, float *dc0, void *stream) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    DeviceScope scope(engine->impl.device);
    return engine->impl.backward_segment(steps, last_in_time != 0, first_in_time != 0, x_seg, h_in, c_in, dy_seg, d_hn, d_cn,
                                         dx_seg, dh0, dc0, static_cast<cudaStream_t>(stream));
}

int flstm_engine_grad_ptrs(flstm_engine *engine, int layer, float **dw_ih, float **dw_hh, float **db) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    if (layer < 0 || layer >= (int)engine->impl.layers.size()) return set_error(FLSTM_ERR_INVALID, "layer out of range");
    auto &l = engine->impl.layers[layer];
    if (dw_ih) *dw_ih = l.dw_ih;
    if (dw_hh) *dw_hh = l.dw_hh;
    if (db) *db = l.db;
    return FLSTM_OK;
}

int flstm_engine_grad_buffer(flstm_engine *engine, float **flat, size_t *count) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    if (flat) *flat = engine->impl.grads;
    if (count) *count = engine->impl.grad_count;
    return FLSTM_OK;
}

int flstm_engine_cache_ptrs(flstm_engine *engine, int layer, void **gates, float **cells, void **hiddens,
                            int *gate_layout) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    if (layer < 0 || layer >= (int)engine->impl.layers.size()) return set_error(FLSTM_ERR_INVALID, "layer out of range");
    auto &l = engine->impl.layers[layer];
    if (gates) *gates = l.gates;
    if (cells) *cells = l.cs;
    if (hiddens) *hiddens = l.hs;
    if (gate_layout) *gate_layout = engine->impl.backend == FLSTM_BACKEND_TC ? 1 : 0;
    return FLSTM_OK;
}

int flstm_engine_set_cell_io_f32(flstm_engine *engine, int enabled) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    engine->impl.cell_io_f32 = enabled != 0;
    return FLSTM_OK;
}

int flstm_engine_backend(const flstm_engine *engine) { return engine ? engine->impl.backend : -1; }

int flstm_comm_unique_id(void *id128) { return flstm_b200::comm_unique_id(id128); }

int flstm_engine_attach_comm(flstm_engine *engine, const void *id128, int rank, int world_size) {
    if (!engine || !id128) return set_error(FLSTM_ERR_INVALID, "null argument");
    Engine &e = engine->impl;
    if (e.comm) return set_error(FLSTM_ERR_INVALID, "a communicator is already attached");
    DeviceScope scope(e.device);
    int st = flstm_b200::comm_create(id128, rank, world_size, &e.comm);
    if (st != FLSTM_OK) return st;
    e.comm_aborted = false;
    if (!e.comm_stream &&
        (cudaStreamCreateWithFlags(&e.comm_stream, cudaStreamNonBlocking) != cudaSuccess ||
         cudaEventCreateWithFlags(&e.comm_fork, cudaEventDisableTiming) != cudaSuccess ||
         cudaEventCreateWithFlags(&e.comm_join, cudaEventDisableTiming) != cudaSuccess))
        return set_error(FLSTM_ERR_CUDA, "could not create the communication stream");
    return FLSTM_OK;
}

int flstm_engine_set_recompute_interval(flstm_engine *engine, size_t interval) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    DeviceScope scope(engine->impl.device);
    return engine->impl.set_recompute(interval);
}

size_t flstm_engine_workspace_bytes(const flstm_engine *engine) { return engine ? engine->impl.workspace_bytes : 0; }

int flstm_engine_abort_comm(flstm_engine *engine) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    Engine &e = engine->impl;
    if (e.comm) {
        flstm_b200::comm_abort(e.comm);
        e.comm = nullptr;
        e.comm_aborted = true;
    }
    return FLSTM_OK;
}

int flstm_engine_wait(flstm_engine *engine, cudaStream_t stream, unsigned int timeout_ms) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    Engine &e = engine->impl;
    DeviceScope scope(e.device);
    cudaEvent_t done = nullptr;
    FLSTM_CUDA_TRY(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
    cudaError_t err = cudaEventRecord(done, stream);
    const auto start = std::chrono::steady_clock::now();
    bool finished = false;
    while (err == cudaSuccess) {
        err = cudaEventQuery(done);
        if (err == cudaSuccess) { finished = true; break; }
        if (err != cudaErrorNotReady) break;
        err = cudaSuccess;
        const auto waited = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - start);
        if (waited.count() >= (long long)timeout_ms) break;
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    cudaEventDestroy(done);
    if (err != cudaSuccess && err != cudaErrorNotReady)
        return set_error(FLSTM_ERR_CUDA, "waiting for the step failed: %s", cudaGetErrorString(err));
    if (!finished) {
        const bool had_comm = e.comm != nullptr;
        flstm_engine_abort_comm(engine);
        return set_error(FLSTM_ERR_TIMEOUT, "the step did not finish within %u ms%s", timeout_ms,
                         had_comm ? "; the communicator was aborted" : "");
    }
    if (e.backend == FLSTM_BACKEND_TC) FLSTM_TRY(flstm_b200::tc::poll_error(e));
    else FLSTM_TRY(e.simt_check_error());
    return FLSTM_OK;
}

int flstm_engine_enable_trace(flstm_engine *engine, int steps) {
    if (!engine || steps < 0) return set_error(FLSTM_ERR_INVALID, "bad argument");
    Engine &e = engine->impl;
    DeviceScope scope(e.device);
    cudaDeviceSynchronize();
    if (e.trace) cudaFree(e.trace);
    e.trace = nullptr;
    e.trace_steps = 0;
    if (steps == 0) return FLSTM_OK;
    void *raw = nullptr;
    const size_t bytes = (size_t)2 * steps * 16 * sizeof(long long);
    if (cudaMalloc(&raw, bytes) != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "trace allocation failed");
    cudaMemset(raw, 0, bytes);
    e.trace = static_cast<long long *>(raw);
    e.trace_steps = steps;
    return FLSTM_OK;
}

int flstm_engine_read_trace(flstm_engine *engine, long long *out_host, size_t count) {
    if (!engine || !out_host) return set_error(FLSTM_ERR_INVALID, "null argument");
    Engine &e = engine->impl;
    DeviceScope scope(e.device);
    const size_t have = (size_t)2 * e.trace_steps * 16;
    if (!e.trace || count > have) return set_error(FLSTM_ERR_INVALID, "trace holds %zu values", have);
    if (cudaMemcpy(out_host, e.trace, count * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess)
        return set_error(FLSTM_ERR_CUDA, "trace copy failed");
    return FLSTM_OK;
}

int flstm_engine_enable_timing(flstm_engine *engine, int enabled) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    engine->impl.timer.enabled = enabled != 0;
    engine->impl.timer.reset();
    return FLSTM_OK;
}

int flstm_engine_phase_ms(flstm_engine *engine, float *out6) {
    if (!engine || !out6) return set_error(FLSTM_ERR_INVALID, "null argument");
    DeviceScope scope(engine->impl.device);
    return engine->impl.timer.totals(out6);
}

int flstm_engine_set_wait_limit(flstm_engine *engine, unsigned long long limit_us) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    engine->impl.wait_limit_ns = limit_us * 1000ull;
    return FLSTM_OK;
}

int flstm_engine_selftest_missing_arrivals(flstm_engine *engine, unsigned int arrivals) {
    if (!engine) return set_error(FLSTM_ERR_INVALID, "null engine");
    engine->impl.selftest_missing_arrivals = arrivals;
    return FLSTM_OK;
}

unsigned long long flstm_engine_launch_count(const flstm_engine *engine) {
    return engine ? engine->impl.launches : 0ull;
}

int flstm_bias_grad(int dtype, const void *dg, size_t rows, size_t cols, int interleaved_h, float *db, void *stream) {
    using namespace flstm_b200;
    if (!dg || !db) return set_error(FLSTM_ERR_INVALID, "null pointer argument");
    if (dtype < FLSTM_DTYPE_F32 || dtype > FLSTM_DTYPE_BF16) return set_error(FLSTM_ERR_INVALID, "bad dtype %d", dtype);
    if (interleaved_h < 0 || (interleaved_h && (size_t)interleaved_h * 4 != cols) || (interleaved_h % 16))
        return set_error(FLSTM_ERR_INVALID, "interleaved_h must be 0 or cols/4 (a multiple of 16)");
    if (rows == 0 || cols == 0) return FLSTM_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float *scratch = nullptr;
    FLSTM_CUDA_TRY(cudaMalloc((void **)&scratch, (size_t)simt::column_sum_scratch_floats(cols) * sizeof(float)));
    int st = simt::column_sum_two_pass(dtype, dg, rows, cols, scratch, db, interleaved_h, s);
    cudaError_t e = cudaStreamSynchronize(s);
    cudaFree(scratch);
    if (st != FLSTM_OK) return st;
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "bias gradient failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

const char *flstm_last_error(void) { return flstm_b200::last_error_slot().c_str(); }

const char *flstm_version(void) { return "flashlstm-b200 0.1 (sm_100a)"; }

}  // extern "C"
