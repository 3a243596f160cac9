// Streaming forward/backward v2 surface (include/lstm.hpp) as a shim over the engine.
//
// Mirrors flstm::StreamingLstmForward (flashlstm_v2/src/lstm_forward.cu:464-966) and
// flstm::StreamingLstmBackward (flashlstm_v2/src/lstm_backward.cu:643-1250) at the boundary:
// fp16 host tensors for x / y / dY / dx and the two checkpoint tensors, fp16 device states,
// fp32 device weights and gradients, three distinct streams, a synchronous call.
//
// Behind the boundary the design differs on purpose:
//  * the sequence is device resident (the largest benchmark configuration's activations fit
//    HBM many times over); host tensors move in chunks of whole time steps (about eight per
//    sequence) on the h2d / d2h streams, ordered against the compute stream with per-chunk events,
//    so that x / dY of the next chunk and y / checkpoints / dx of the previous chunk are in flight
//    while the projection GEMM and the persistent recurrence of the current chunk run (the role of
//    the reference's double-buffered 32-step chunk pipeline, lstm_forward.cu:673-940,
//    lstm_backward.cu:899-1213);
//  * a context per (device, B, I, H) owns the engine and the staging buffers, so a call
//    allocates nothing once the context exists (the reference cudaMallocs ~25 buffers and
//    registers the host tensors on every call, lstm_forward.cu:525-645);
//  * backward consumes the engine's post-activation gate cache when it still belongs to the
//    matching forward (same y tensor, same length, nothing in between); otherwise the cache is
//    rebuilt by running the forward recurrence again from x, h0, c0.  The cell state is never
//    reconstructed from y and o (the reference does, lstm_backward.cu:188-197).
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <stdexcept>
#include <tuple>
#include <vector>

#include "common.cuh"
#include "engine.h"
#include "kernels.h"
#include "lstm.hpp"

namespace {

using namespace flstm_b200;

struct V2Context {
    flstm_engine *engine = nullptr;
    size_t B = 0, I = 0, H = 0, t_cap = 0;
    void *x = nullptr, *y = nullptr, *dy = nullptr, *dx = nullptr;  // fp16 (T,B,.)
    void *chk_h = nullptr, *chk_c = nullptr;                        // up to fp32 (T,B,H)
    cudaEvent_t ev_in = nullptr, ev_compute = nullptr;
    std::vector<cudaEvent_t> ev_pool;  // per-chunk "input landed" / "compute done" events of the pipeline
    // identity of the forward whose cache the engine holds
    const void *fwd_y = nullptr;
    size_t fwd_T = 0;
    bool cache_valid = false;

    ~V2Context() {
        if (engine) flstm_engine_destroy(engine);
        release();
        if (ev_in) cudaEventDestroy(ev_in);
        if (ev_compute) cudaEventDestroy(ev_compute);
        for (auto e : ev_pool) cudaEventDestroy(e);
    }
    int event(size_t i, cudaEvent_t *out) {
        while (ev_pool.size() <= i) {
            cudaEvent_t e;
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess)
                return set_error(FLSTM_ERR_CUDA, "event creation failed");
            ev_pool.push_back(e);
        }
        *out = ev_pool[i];
        return FLSTM_OK;
    }
    void release() {
        for (void **p : {&x, &y, &dy, &dx, &chk_h, &chk_c}) {
            if (*p) cudaFree(*p);
            *p = nullptr;
        }
        t_cap = 0;
    }
    int reserve(size_t T) {
        if (T <= t_cap) return FLSTM_OK;
        cudaDeviceSynchronize();
        release();
        const size_t slab = B * H;
        if (cudaMalloc(&x, T * B * I * 2) != cudaSuccess || cudaMalloc(&y, T * slab * 2) != cudaSuccess ||
            cudaMalloc(&dy, T * slab * 2) != cudaSuccess || cudaMalloc(&dx, T * B * I * 2) != cudaSuccess ||
            cudaMalloc(&chk_h, T * slab * 4) != cudaSuccess || cudaMalloc(&chk_c, T * slab * 4) != cudaSuccess)
            return set_error(FLSTM_ERR_CUDA, "v2 staging allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
        t_cap = T;
        cache_valid = false;
        return FLSTM_OK;
    }
};

std::mutex g_mutex;
std::map<std::tuple<int, size_t, size_t, size_t>, V2Context *> g_contexts;
thread_local int g_last_status = FLSTM_OK;

int get_context(size_t T, size_t B, size_t I, size_t H, V2Context **out) {
    int dev = 0;
    FLSTM_CUDA_TRY(cudaGetDevice(&dev));
    auto key = std::make_tuple(dev, B, I, H);
    auto it = g_contexts.find(key);
    V2Context *c = nullptr;
    if (it == g_contexts.end()) {
        c = new V2Context();
        c->B = B;
        c->I = I;
        c->H = H;
        flstm_engine_config cfg{};
        cfg.dtype = FLSTM_DTYPE_F16;
        cfg.layers = 1;
        cfg.batch = B;
        cfg.input_size = I;
        cfg.hidden_size = H;
        cfg.max_seq_len = T;
        cfg.training = 1;
        cfg.backend = FLSTM_BACKEND_AUTO;
        int st = flstm_engine_create(&cfg, &c->engine);
        if (st != FLSTM_OK) {
            delete c;
            return st;
        }
        if (cudaEventCreateWithFlags(&c->ev_in, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&c->ev_compute, cudaEventDisableTiming) != cudaSuccess) {
            delete c;
            return set_error(FLSTM_ERR_CUDA, "event creation failed");
        }
        g_contexts[key] = c;
    } else {
        c = it->second;
    }
    FLSTM_TRY(c->reserve(T));
    *out = c;
    return FLSTM_OK;
}

// Host tensors move in chunks of whole time steps so that copies overlap the recurrence: about eight
// chunks per sequence, at least 16 steps each (the reference uses fixed 32-step chunks,
// flashlstm_v2/src/lstm_forward.cu:515).  FLSTM_STREAM_CHUNK overrides the number of steps.
size_t chunk_steps(size_t T) {
    if (const char *env = std::getenv("FLSTM_STREAM_CHUNK")) {
        const long v = std::atol(env);
        if (v > 0) return (size_t)v < T ? (size_t)v : T;
    }
    size_t n = (T + 7) / 8;
    if (n < 16) n = 16;
    return n < T ? n : T;
}

bool is_device_pointer(const void *p) {
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Brings a host (or device) tensor onto the device; returns the pointer kernels should read.
int stage_in(const void *src, void *staging, size_t bytes, cudaStream_t h2d, const void **dev) {
    if (is_device_pointer(src)) {
        *dev = src;
        return FLSTM_OK;
    }
    FLSTM_CUDA_TRY(cudaMemcpyAsync(staging, src, bytes, cudaMemcpyHostToDevice, h2d));
    *dev = staging;
    return FLSTM_OK;
}

int forward_impl(size_t T, size_t B, size_t I, size_t H, size_t R, const __half *x_host, const __half *h0,
                 const __half *c0, const float *w_ih, const float *w_hh, const float *b_ih, const float *b_hh,
                 __half *y_host, flstm_GateCacheHost cache, flstm_StreamingLstmOptions opt, __half *hy, __half *cy,
                 cudaStream_t sc, cudaStream_t sh, cudaStream_t sd) {
    if (T == 0 || B == 0 || I == 0 || H == 0) return FLSTM_OK;  // silent no-op (lstm_forward.cu:493-495)
    if (R == 0) return set_error(FLSTM_ERR_INVALID, "recompute_interval must be >= 1");
    if (sc == sh || sc == sd || sh == sd) return set_error(FLSTM_ERR_INVALID, "compute, h2d and d2h streams must be distinct");
    if (!x_host || !h0 || !c0 || !w_ih || !w_hh || !b_ih || !b_hh || !y_host || !hy || !cy)
        return set_error(FLSTM_ERR_INVALID, "null pointer argument");
    std::lock_guard<std::mutex> lock(g_mutex);
    V2Context *c = nullptr;
    FLSTM_TRY(get_context(T, B, I, H, &c));
    c->cache_valid = false;
    const size_t slab = B * H;
    const bool x_on_device = is_device_pointer(x_host), y_on_device = is_device_pointer(y_host);
    const void *x_dev = x_on_device ? (const void *)x_host : c->x;
    void *y_dev = y_on_device ? (void *)y_host : c->y;
    const size_t nchk = (T + R - 1) / R;
    const int hd = opt.h_dtype == FLSTM_GATE_CACHE_FLOAT16 ? FLSTM_DTYPE_F16 : FLSTM_DTYPE_F32;
    const int cd = opt.c_dtype == FLSTM_GATE_CACHE_FLOAT16 ? FLSTM_DTYPE_F16 : FLSTM_DTYPE_F32;
    const bool ch_dev = cache.h_ptr && is_device_pointer(cache.h_ptr);
    const bool cc_dev = cache.c_ptr && is_device_pointer(cache.c_ptr);
    char *chk_h_dev = static_cast<char *>(ch_dev ? cache.h_ptr : c->chk_h);
    char *chk_c_dev = static_cast<char *>(cc_dev ? cache.c_ptr : c->chk_c);
    void *hs = nullptr;
    float *cs = nullptr;
    FLSTM_TRY(flstm_engine_cache_ptrs(c->engine, 0, nullptr, &cs, &hs, nullptr));
    FLSTM_TRY(flstm_engine_set_weights(c->engine, 0, w_ih, w_hh, b_ih, b_hh, sc));

    // Chunk pipeline over the caller's three streams: x chunk k+1 travels host->device while chunk k
    // runs (projection GEMM + persistent recurrence over the chunk's steps), and y / checkpoint rows
    // of chunk k travel device->host while chunk k+1 runs.
    const size_t cs_steps = chunk_steps(T), nchunks = (T + cs_steps - 1) / cs_steps;
    if (!x_on_device) {
        for (size_t k = 0; k < nchunks; ++k) {
            const size_t t0 = k * cs_steps, t1 = (t0 + cs_steps < T) ? t0 + cs_steps : T;
            FLSTM_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(c->x) + t0 * B * I * 2,
                                           reinterpret_cast<const char *>(x_host) + t0 * B * I * 2, (t1 - t0) * B * I * 2,
                                           cudaMemcpyHostToDevice, sh));
            cudaEvent_t ev;
            FLSTM_TRY(c->event(2 * k, &ev));
            FLSTM_CUDA_TRY(cudaEventRecord(ev, sh));
        }
    }
    for (size_t k = 0; k < nchunks; ++k) {
        const size_t t0 = k * cs_steps, t1 = (t0 + cs_steps < T) ? t0 + cs_steps : T;
        cudaEvent_t ev_x, ev_done;
        FLSTM_TRY(c->event(2 * k, &ev_x));
        FLSTM_TRY(c->event(2 * k + 1, &ev_done));
        if (!x_on_device) FLSTM_CUDA_TRY(cudaStreamWaitEvent(sc, ev_x, 0));
        FLSTM_TRY(flstm_engine_forward_range(c->engine, T, t0, t1, x_dev, h0, c0, y_dev, hy, cy, sc));
        // checkpoints: entry e = state entering step e*R (entry 0 = h0 / c0); this chunk owns the
        // entries whose step lies in [t0, t1)
        const size_t e0 = (t0 + R - 1) / R, e1 = (t1 + R - 1) / R < nchk ? (t1 + R - 1) / R : nchk;
        if (e1 > e0) {
            if (cache.h_ptr)
                FLSTM_TRY(simt::gather_slabs(FLSTM_DTYPE_F16, static_cast<char *>(hs) + e0 * R * slab * 2, slab, R, e1 - e0, hd,
                                             chk_h_dev + e0 * slab * dtype_size(hd), sc));
            if (cache.c_ptr)
                FLSTM_TRY(simt::gather_slabs(FLSTM_DTYPE_F32, cs + e0 * R * slab, slab, R, e1 - e0, cd,
                                             chk_c_dev + e0 * slab * dtype_size(cd), sc));
        }
        FLSTM_CUDA_TRY(cudaEventRecord(ev_done, sc));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(sd, ev_done, 0));
        if (!y_on_device)
            FLSTM_CUDA_TRY(cudaMemcpyAsync(reinterpret_cast<char *>(y_host) + t0 * slab * 2, static_cast<char *>(c->y) + t0 * slab * 2,
                                           (t1 - t0) * slab * 2, cudaMemcpyDeviceToHost, sd));
        if (e1 > e0) {
            if (cache.h_ptr && !ch_dev)
                FLSTM_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(cache.h_ptr) + e0 * slab * dtype_size(hd),
                                               chk_h_dev + e0 * slab * dtype_size(hd), (e1 - e0) * slab * dtype_size(hd),
                                               cudaMemcpyDeviceToHost, sd));
            if (cache.c_ptr && !cc_dev)
                FLSTM_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(cache.c_ptr) + e0 * slab * dtype_size(cd),
                                               chk_c_dev + e0 * slab * dtype_size(cd), (e1 - e0) * slab * dtype_size(cd),
                                               cudaMemcpyDeviceToHost, sd));
        }
    }
    FLSTM_CUDA_TRY(cudaStreamSynchronize(sh));
    FLSTM_CUDA_TRY(cudaStreamSynchronize(sc));
    FLSTM_CUDA_TRY(cudaStreamSynchronize(sd));
    c->fwd_y = y_host;
    c->fwd_T = T;
    c->cache_valid = true;
    return FLSTM_OK;
}

int backward_impl(size_t T, size_t B, size_t I, size_t H, size_t R, const __half *x_host, const __half *y_host,
                  flstm_GateCacheHost cache, flstm_StreamingLstmOptions opt, const __half *dy_host,
                  const __half *d_hn, const __half *d_cn, const __half *h0, const __half *c0, const float *w_ih,
                  const float *w_hh, const float *b_ih, const float *b_hh, __half *dx_host, float *dw_ih,
                  float *dw_hh, float *db_ih, float *db_hh, float *dh0, float *dc0, cudaStream_t sc,
                  cudaStream_t sh, cudaStream_t sd) {
    (void)cache;
    (void)opt;
    if (T == 0 || B == 0 || I == 0 || H == 0) return FLSTM_OK;
    if (R == 0) return set_error(FLSTM_ERR_INVALID, "recompute_interval must be >= 1");
    if (sc == sh || sc == sd || sh == sd) return set_error(FLSTM_ERR_INVALID, "compute, h2d and d2h streams must be distinct");
    if (!x_host || !y_host || !dy_host || !h0 || !w_ih || !w_hh || !b_ih || !b_hh || !dx_host || !dw_ih || !dw_hh ||
        !db_ih || !db_hh || !dh0 || !dc0)
        return set_error(FLSTM_ERR_INVALID, "null pointer argument");
    std::lock_guard<std::mutex> lock(g_mutex);
    V2Context *c = nullptr;
    FLSTM_TRY(get_context(T, B, I, H, &c));
    const size_t slab = B * H;
    const bool have_cache = c->cache_valid && c->fwd_y == y_host && c->fwd_T == T;
    const bool dy_on_device = is_device_pointer(dy_host), dx_on_device = is_device_pointer(dx_host);
    const void *dy_dev = dy_on_device ? (const void *)dy_host : c->dy;
    void *dx_dev = dx_on_device ? (void *)dx_host : c->dx;
    const size_t cs_steps = chunk_steps(T), nchunks = (T + cs_steps - 1) / cs_steps;
    // dY chunks travel host->device in the order the reverse recurrence consumes them: last chunk first
    if (!dy_on_device) {
        for (size_t r = 0; r < nchunks; ++r) {
            const size_t k = nchunks - 1 - r;
            const size_t t0 = k * cs_steps, t1 = (t0 + cs_steps < T) ? t0 + cs_steps : T;
            FLSTM_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(c->dy) + t0 * slab * 2,
                                           reinterpret_cast<const char *>(dy_host) + t0 * slab * 2, (t1 - t0) * slab * 2,
                                           cudaMemcpyHostToDevice, sh));
            cudaEvent_t ev;
            FLSTM_TRY(c->event(2 * k, &ev));
            FLSTM_CUDA_TRY(cudaEventRecord(ev, sh));
        }
    }
    if (!have_cache) {
        // stateless call (another forward ran in between, or none did): rebuild the gate cache by
        // running the recurrence again from x, h0, c0.  With a live cache the forward's device copy
        // of x is still in place and nothing is recomputed.
        if (!c0) return set_error(FLSTM_ERR_INVALID, "c0 is null");
        const void *x_dev = nullptr;
        FLSTM_TRY(stage_in(x_host, c->x, T * B * I * 2, sh, &x_dev));
        FLSTM_CUDA_TRY(cudaEventRecord(c->ev_in, sh));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(sc, c->ev_in, 0));
        FLSTM_TRY(flstm_engine_set_weights(c->engine, 0, w_ih, w_hh, b_ih, b_hh, sc));
        FLSTM_TRY(flstm_engine_forward(c->engine, T, x_dev, h0, c0, nullptr, nullptr, nullptr, sc));
    }
    // reverse chunk pipeline: BPTT + dX GEMM of chunk k run while dY of chunk k-1 arrives and dX of
    // chunk k+1 leaves; the weight / bias gradients are formed over the whole sequence by the last chunk
    for (size_t r = 0; r < nchunks; ++r) {
        const size_t k = nchunks - 1 - r;
        const size_t t0 = k * cs_steps, t1 = (t0 + cs_steps < T) ? t0 + cs_steps : T;
        cudaEvent_t ev_dy, ev_done;
        FLSTM_TRY(c->event(2 * k, &ev_dy));
        FLSTM_TRY(c->event(2 * k + 1, &ev_done));
        if (!dy_on_device) FLSTM_CUDA_TRY(cudaStreamWaitEvent(sc, ev_dy, 0));
        FLSTM_TRY(flstm_engine_backward_range(c->engine, T, t0, t1, dy_dev, d_hn, d_cn, dx_dev, dh0, dc0, sc));
        FLSTM_CUDA_TRY(cudaEventRecord(ev_done, sc));
        if (!dx_on_device) {
            FLSTM_CUDA_TRY(cudaStreamWaitEvent(sd, ev_done, 0));
            FLSTM_CUDA_TRY(cudaMemcpyAsync(reinterpret_cast<char *>(dx_host) + t0 * B * I * 2,
                                           static_cast<char *>(c->dx) + t0 * B * I * 2, (t1 - t0) * B * I * 2,
                                           cudaMemcpyDeviceToHost, sd));
        }
    }
    float *g_ih = nullptr, *g_hh = nullptr, *g_b = nullptr;
    FLSTM_TRY(flstm_engine_grad_ptrs(c->engine, 0, &g_ih, &g_hh, &g_b));
    FLSTM_CUDA_TRY(cudaMemcpyAsync(dw_ih, g_ih, 4 * H * I * sizeof(float), cudaMemcpyDeviceToDevice, sc));
    FLSTM_CUDA_TRY(cudaMemcpyAsync(dw_hh, g_hh, 4 * H * H * sizeof(float), cudaMemcpyDeviceToDevice, sc));
    FLSTM_CUDA_TRY(cudaMemcpyAsync(db_ih, g_b, 4 * H * sizeof(float), cudaMemcpyDeviceToDevice, sc));
    FLSTM_CUDA_TRY(cudaMemcpyAsync(db_hh, g_b, 4 * H * sizeof(float), cudaMemcpyDeviceToDevice, sc));
    FLSTM_CUDA_TRY(cudaStreamSynchronize(sh));
    FLSTM_CUDA_TRY(cudaStreamSynchronize(sc));
    FLSTM_CUDA_TRY(cudaStreamSynchronize(sd));
    c->cache_valid = false;  // a cache is consumed once
    return FLSTM_OK;
}

void report(const char *fn, int st) {
    g_last_status = st;
    if (st != FLSTM_OK) std::fprintf(stderr, "%s failed: %s\n", fn, flstm_last_error());
}

}  // namespace

namespace flstm {

void StreamingLstmForward(size_t T, size_t B, size_t I, size_t H, size_t R, const __half *x_host, const __half *h0,
                          const __half *c0, const float *w_ih, const float *w_hh, const float *b_ih,
                          const float *b_hh, __half *y_host, GateCacheHost cache, StreamingLstmOptions options,
                          __half *hy, __half *cy, cudaStream_t sc, cudaStream_t sh, cudaStream_t sd) {
    flstm_GateCacheHost gc{cache.h_ptr, cache.c_ptr};
    flstm_StreamingLstmOptions o{(flstm_GateCacheDType)options.h_dtype, (flstm_GateCacheDType)options.c_dtype};
    int st = forward_impl(T, B, I, H, R, x_host, h0, c0, w_ih, w_hh, b_ih, b_hh, y_host, gc, o, hy, cy, sc, sh, sd);
    g_last_status = st;
    if (st != FLSTM_OK) throw std::runtime_error(flstm_last_error());
}

void StreamingLstmBackward(size_t T, size_t B, size_t I, size_t H, size_t R, const __half *x_host,
                           const __half *y_host, GateCacheHost cache, StreamingLstmOptions options,
                           const __half *dy_host, const __half *d_hn, const __half *d_cn, const __half *h0,
                           const __half *c0, const float *w_ih, const float *w_hh, const float *b_ih,
                           const float *b_hh, __half *dx_host, float *dw_ih, float *dw_hh, float *db_ih,
                           float *db_hh, float *dh0, float *dc0, cudaStream_t sc, cudaStream_t sh, cudaStream_t sd) {
    flstm_GateCacheHost gc{cache.h_ptr, cache.c_ptr};
    flstm_StreamingLstmOptions o{(flstm_GateCacheDType)options.h_dtype, (flstm_GateCacheDType)options.c_dtype};
    int st = backward_impl(T, B, I, H, R, x_host, y_host, gc, o, dy_host, d_hn, d_cn, h0, c0, w_ih, w_hh, b_ih, b_hh,
                           dx_host, dw_ih, dw_hh, db_ih, db_hh, dh0, dc0, sc, sh, sd);
    g_last_status = st;
    if (st != FLSTM_OK) throw std::runtime_error(flstm_last_error());
}

}  // namespace flstm

extern "C" {

void flstm_StreamingLstmForward(size_t T, size_t B, size_t I, size_t H, size_t R, const __half *x_host,
                                const __half *h0, const __half *c0, const float *w_ih, const float *w_hh,
                                const float *b_ih, const float *b_hh, __half *y_host, flstm_GateCacheHost cache,
                                const flstm_StreamingLstmOptions *options, __half *hy, __half *cy, cudaStream_t sc,
                                cudaStream_t sh, cudaStream_t sd) {
    flstm_StreamingLstmOptions o{FLSTM_GATE_CACHE_FLOAT32, FLSTM_GATE_CACHE_FLOAT32};
    if (options) o = *options;
    report("flstm_StreamingLstmForward",
           forward_impl(T, B, I, H, R, x_host, h0, c0, w_ih, w_hh, b_ih, b_hh, y_host, cache, o, hy, cy, sc, sh, sd));
}

void flstm_StreamingLstmBackward(size_t T, size_t B, size_t I, size_t H, size_t R, const __half *x_host,
                                 const __half *y_host, flstm_GateCacheHost cache, const __half *dy_host,
                                 const __half *d_hn, const __half *d_cn, const __half *h0, const __half *c0,
                                 const float *w_ih, const float *w_hh, const float *b_ih, const float *b_hh,
                                 __half *dx_host, float *dw_ih, float *dw_hh, float *db_ih, float *db_hh, float *dh0,
                                 float *dc0, cudaStream_t sc, cudaStream_t sh, cudaStream_t sd,
                                 const flstm_StreamingLstmOptions *options) {
    flstm_StreamingLstmOptions o{FLSTM_GATE_CACHE_FLOAT32, FLSTM_GATE_CACHE_FLOAT32};
    if (options) o = *options;
    report("flstm_StreamingLstmBackward",
           backward_impl(T, B, I, H, R, x_host, y_host, cache, o, dy_host, d_hn, d_cn, h0, c0, w_ih, w_hh, b_ih, b_hh,
                         dx_host, dw_ih, dw_hh, db_ih, db_hh, dh0, dc0, sc, sh, sd));
}

int flstm_last_status(void) { return g_last_status; }

}  // extern "C"
