// Streaming forward/backward v2 surface (include/lstm.hpp) as a shim over the engine.
//
// Mirrors flstm::StreamingLstmForward (flashlstm_v2/src/lstm_forward.cu:464-966) and
// flstm::StreamingLstmBackward (flashlstm_v2/src/lstm_backward.cu:643-1250) at the boundary:
// fp16 host tensors for x / y / dY / dx and the two checkpoint tensors, fp16 device states,
// fp32 device weights and gradients, three distinct streams, a synchronous call.
//
// Behind the boundary there are two modes, chosen per call from the device memory the problem would take
// (FLSTM_V2_DEVICE_BUDGET_BYTES, by default 60 % of the memory free when the context is created):
//  * RESIDENT (the sequence fits the budget): the whole sequence is staged on the device; host tensors move
//    in chunks of whole time steps (about eight per sequence) on the h2d / d2h streams, ordered against the
//    compute stream with per-chunk events, so that x / dY of the next chunk and y / checkpoints / dx of the
//    previous chunk are in flight while the projection GEMM and the persistent recurrence of the current
//    chunk run.  Backward consumes the engine's post-activation gate cache when it still belongs to the
//    matching forward (same y tensor, same length, nothing in between);
//  * STREAMING (it does not, or the backward call is stateless): the device holds ONE segment of S steps
//    (S a multiple of the recompute interval R) of gates, states and dG plus two staging slots per host
//    tensor, whatever T is -- the role of the reference's double-buffered 32-step chunk pipeline
//    (lstm_forward.cu:515,622-627,673-940, lstm_backward.cu:899-1213).  The forward runs segment after
//    segment, carrying h (fp16) and c (fp32) on the device and writing the caller's h/c checkpoints; the
//    backward walks the segments from the end, re-reads x and dY of a segment from the caller's tensors,
//    restores the state that entered it FROM THE CALLER'S CHECKPOINTS, re-runs the segment's forward to
//    rebuild its gates and runs the BPTT over it (lstm_backward.cu:496-523,975-1054).
// In both modes a context per (device, B, I, H) owns the engines and the staging buffers, so a call
// allocates nothing once the context exists (the reference cudaMallocs ~25 buffers and registers the host
// tensors on every call, lstm_forward.cu:525-645); at most four contexts are kept (least recently used
// goes first).  The cell state is never reconstructed from y and o (the reference does,
// lstm_backward.cu:188-197).  Packed weights are kept across calls while the caller says they have not
// changed (flstm_v2_set_weight_version); without that promise they are re-packed on every call, as the
// reference does (lstm_forward.cu:605).
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

constexpr size_t kMaxContexts = 4;

// Staging slots of the streaming mode: two of each, so that the copies of one segment overlap the work on another.
struct StreamSlots {
    void *x[2] = {}, *y[2] = {}, *dy[2] = {}, *dx[2] = {};  // fp16 (S,B,.)
    void *ck_raw_h[2] = {}, *ck_raw_c[2] = {};              // a checkpoint as the caller stores it (fp16 / fp32 slab)
    void *ck_h[2] = {};                                      // ... as the engine wants it: fp16 h
    float *ck_c[2] = {};                                     // ... fp32 c
    void *out_h[2] = {}, *out_c[2] = {};                     // checkpoints of one forward segment, the caller's dtype
    void *h_state[2] = {};                                   // carried between forward segments: fp16 h
    float *c_state[2] = {};                                  // ... fp32 c
};

struct V2Context {
    size_t B = 0, I = 0, H = 0;
    unsigned long long last_use = 0;
    size_t budget = 0;  // device bytes a problem may take in resident mode (and the streaming mode's target)
    // ---- resident mode
    flstm_engine *engine = nullptr;
    size_t t_cap = 0, chk_cap = 0, resident_staging_bytes = 0, slot_bytes = 0;
    void *x = nullptr, *y = nullptr, *dy = nullptr, *dx = nullptr;  // fp16 (T,B,.)
    void *chk_h = nullptr, *chk_c = nullptr;                        // up to fp32 (ceil(T/R),B,H)
    cudaEvent_t ev_in = nullptr;
    std::vector<cudaEvent_t> ev_pool;  // per-chunk events of the pipelines
    // identity of the forward whose cache the resident engine holds
    const void *fwd_y = nullptr;
    size_t fwd_T = 0;
    bool cache_valid = false;
    // ---- streaming mode
    flstm_engine *seg_engine = nullptr;
    size_t seg_steps = 0;
    StreamSlots slots;
    // ---- packed weights: what each engine was last given (pointers + the caller's version; 0 = no promise)
    struct Packed { const float *p[4] = {}; unsigned long long version = 0; } packed_resident, packed_seg;

    ~V2Context() {
        if (engine) flstm_engine_destroy(engine);
        if (seg_engine) flstm_engine_destroy(seg_engine);
        release_resident();
        release_slots();
        if (ev_in) cudaEventDestroy(ev_in);
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
    void release_resident() {
        for (void **p : {&x, &y, &dy, &dx, &chk_h, &chk_c}) {
            if (*p) cudaFree(*p);
            *p = nullptr;
        }
        t_cap = chk_cap = resident_staging_bytes = 0;
    }
    void release_slots() {
        auto drop = [](void *p) { if (p) cudaFree(p); };
        for (int i = 0; i < 2; ++i) {
            drop(slots.x[i]); drop(slots.y[i]); drop(slots.dy[i]); drop(slots.dx[i]);
            drop(slots.ck_raw_h[i]); drop(slots.ck_raw_c[i]); drop(slots.ck_h[i]); drop(slots.ck_c[i]);
            drop(slots.out_h[i]); drop(slots.out_c[i]); drop(slots.h_state[i]); drop(slots.c_state[i]);
        }
        slots = StreamSlots{};
        slot_bytes = 0;
    }
    // device bytes of the resident mode for a T-step sequence: staging + the engine's time-sized buffers
    size_t resident_bytes(size_t T, size_t R) const {
        const size_t slab = B * H, nchk = (T + R - 1) / R;
        return T * (2 * B * I * 2 + 2 * slab * 2) + nchk * slab * 8 + (T + 1) * slab * 22;
    }
    // ... of the streaming mode with S-step segments (two slots per host tensor + one segment in the engine)
    size_t streaming_bytes(size_t S, size_t R) const {
        const size_t slab = B * H;
        return 2 * S * (2 * B * I * 2 + 2 * slab * 2) + 2 * (S / R + 1) * slab * 8 + (S + 2) * slab * 22 + 16 * slab * 4;
    }
    int reserve_resident(size_t T, size_t R) {
        const size_t slab = B * H, nchk = (T + R - 1) / R;
        if (!engine) {
            flstm_engine_config cfg{};
            cfg.dtype = FLSTM_DTYPE_F16;
            cfg.layers = 1;
            cfg.batch = B;
            cfg.input_size = I;
            cfg.hidden_size = H;
            cfg.max_seq_len = T;
            cfg.training = 1;
            cfg.backend = FLSTM_BACKEND_AUTO;
            FLSTM_TRY(flstm_engine_create(&cfg, &engine));
            packed_resident = Packed{};
        }
        if (T > t_cap || nchk > chk_cap) {
            cudaDeviceSynchronize();
            release_resident();
            if (cudaMalloc(&x, T * B * I * 2) != cudaSuccess || cudaMalloc(&y, T * slab * 2) != cudaSuccess ||
                cudaMalloc(&dy, T * slab * 2) != cudaSuccess || cudaMalloc(&dx, T * B * I * 2) != cudaSuccess ||
                cudaMalloc(&chk_h, nchk * slab * 4) != cudaSuccess || cudaMalloc(&chk_c, nchk * slab * 4) != cudaSuccess)
                return set_error(FLSTM_ERR_CUDA, "v2 staging allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
            t_cap = T;
            chk_cap = nchk;
            resident_staging_bytes = T * (2 * B * I * 2 + 2 * slab * 2) + nchk * slab * 8;
            cache_valid = false;
        }
        return FLSTM_OK;
    }
    // Streaming needs the tensor-core backend (segment backward); returns FLSTM_ERR_UNSUPPORTED otherwise.
    int reserve_streaming(size_t S, size_t R) {
        if (seg_engine && seg_steps == S) return FLSTM_OK;
        cudaDeviceSynchronize();
        if (seg_engine) flstm_engine_destroy(seg_engine);
        seg_engine = nullptr;
        release_slots();
        seg_steps = 0;
        packed_seg = Packed{};
        flstm_engine_config cfg{};
        cfg.dtype = FLSTM_DTYPE_F16;
        cfg.layers = 1;
        cfg.batch = B;
        cfg.input_size = I;
        cfg.hidden_size = H;
        cfg.max_seq_len = S;
        cfg.training = 1;
        cfg.backend = FLSTM_BACKEND_AUTO;
        FLSTM_TRY(flstm_engine_create(&cfg, &seg_engine));
        if (flstm_engine_backend(seg_engine) != FLSTM_BACKEND_TC) {
            flstm_engine_destroy(seg_engine);
            seg_engine = nullptr;
            return set_error(FLSTM_ERR_UNSUPPORTED, "host streaming in segments needs the tensor-core backend (H %% 64 == 0, I %% 8 == 0)");
        }
        FLSTM_TRY(flstm_engine_set_recompute_interval(seg_engine, S));
        FLSTM_TRY(flstm_engine_set_cell_io_f32(seg_engine, 1));
        const size_t slab = B * H, ne = S / R + 1;
        bool ok = true;
        size_t total = 0;
        auto grab = [&](void **p, size_t bytes) { ok = ok && cudaMalloc(p, bytes) == cudaSuccess; total += bytes; };
        for (int i = 0; i < 2; ++i) {
            grab(&slots.x[i], S * B * I * 2);
            grab(&slots.y[i], S * slab * 2);
            grab(&slots.dy[i], S * slab * 2);
            grab(&slots.dx[i], S * B * I * 2);
            grab(&slots.ck_raw_h[i], slab * 4);
            grab(&slots.ck_raw_c[i], slab * 4);
            grab(&slots.ck_h[i], slab * 2);
            grab(reinterpret_cast<void **>(&slots.ck_c[i]), slab * 4);
            grab(&slots.out_h[i], ne * slab * 4);
            grab(&slots.out_c[i], ne * slab * 4);
            grab(&slots.h_state[i], slab * 2);
            grab(reinterpret_cast<void **>(&slots.c_state[i]), slab * 4);
        }
        if (!ok) {
            release_slots();
            return set_error(FLSTM_ERR_CUDA, "v2 streaming staging allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
        }
        seg_steps = S;
        slot_bytes = total;
        return FLSTM_OK;
    }
    // device bytes the context holds now (the engines' time-sized buffers + staging)
    size_t device_bytes() const {
        size_t n = resident_staging_bytes + slot_bytes;
        if (engine) n += flstm_engine_workspace_bytes(engine);
        if (seg_engine) n += flstm_engine_workspace_bytes(seg_engine);
        return n;
    }
};

std::mutex g_mutex;
std::map<std::tuple<int, size_t, size_t, size_t>, V2Context *> g_contexts;
unsigned long long g_use_counter = 0;
unsigned long long g_weight_version = 0;  // 0: the caller makes no promise, weights are re-packed on every call
thread_local int g_last_status = FLSTM_OK;
thread_local size_t g_last_device_bytes = 0;
thread_local int g_last_streaming = 0;

size_t device_budget() {
    if (const char *env = std::getenv("FLSTM_V2_DEVICE_BUDGET_BYTES")) {
        const long long v = std::atoll(env);
        if (v > 0) return (size_t)v;
    }
    size_t free_b = 0, total_b = 0;
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return (size_t)8 << 30;
    return free_b / 10 * 6;
}

int get_context(size_t B, size_t I, size_t H, V2Context **out) {
    int dev = 0;
    FLSTM_CUDA_TRY(cudaGetDevice(&dev));
    auto key = std::make_tuple(dev, B, I, H);
    auto it = g_contexts.find(key);
    V2Context *c = nullptr;
    if (it == g_contexts.end()) {
        if (g_contexts.size() >= kMaxContexts) {  // drop the least recently used shape
            auto victim = g_contexts.begin();
            for (auto j = g_contexts.begin(); j != g_contexts.end(); ++j)
                if (j->second->last_use < victim->second->last_use) victim = j;
            int vdev = std::get<0>(victim->first), cur = dev;
            cudaSetDevice(vdev);
            cudaDeviceSynchronize();
            delete victim->second;
            cudaSetDevice(cur);
            g_contexts.erase(victim);
        }
        c = new V2Context();
        c->B = B;
        c->I = I;
        c->H = H;
        if (cudaEventCreateWithFlags(&c->ev_in, cudaEventDisableTiming) != cudaSuccess) {
            delete c;
            return set_error(FLSTM_ERR_CUDA, "event creation failed");
        }
        g_contexts[key] = c;
    } else {
        c = it->second;
    }
    c->budget = device_budget() + c->device_bytes();  // what is free now plus what this context already holds
    if (const char *env = std::getenv("FLSTM_V2_DEVICE_BUDGET_BYTES"))
        if (std::atoll(env) > 0) c->budget = (size_t)std::atoll(env);
    c->last_use = ++g_use_counter;
    *out = c;
    return FLSTM_OK;
}

// Segment length of the streaming mode: the largest multiple of R that fits the budget, at most 512 steps and
// never less than R (a segment must start at a checkpoint).  FLSTM_V2_SEGMENT_STEPS overrides (rounded to R).
size_t pick_segment(const V2Context &c, size_t T, size_t R) {
    size_t S = R;
    if (const char *env = std::getenv("FLSTM_V2_SEGMENT_STEPS")) {
        const long v = std::atol(env);
        if (v > 0) S = ((size_t)v + R - 1) / R * R;
    } else {
        while (S + R <= 512 && c.streaming_bytes(S + R, R) <= c.budget) S += R;
    }
    const size_t t_round = (T + R - 1) / R * R;
    return S < t_round ? S : t_round;
}

// Weights are packed into an engine when they may have changed: always, unless the caller has published a
// version (flstm_v2_set_weight_version) and neither it nor the four pointers differ from the last packing.
int set_weights_cached(flstm_engine *e, V2Context::Packed &last, const float *w_ih, const float *w_hh, const float *b_ih,
                       const float *b_hh, cudaStream_t s) {
    const float *now[4] = {w_ih, w_hh, b_ih, b_hh};
    bool same = g_weight_version != 0 && last.version == g_weight_version;
    for (int i = 0; i < 4 && same; ++i) same = last.p[i] == now[i];
    if (same) return FLSTM_OK;
    FLSTM_TRY(flstm_engine_set_weights(e, 0, w_ih, w_hh, b_ih, b_hh, s));
    for (int i = 0; i < 4; ++i) last.p[i] = now[i];
    last.version = g_weight_version;
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

inline char *bytes(void *p) { return static_cast<char *>(p); }
inline const char *bytes(const void *p) { return static_cast<const char *>(p); }

// ------------------------------------------------------------------ streaming mode
// Forward over segments of S steps: x of segment k+1 (and k+2) travels to the device while segment k runs;
// y and the checkpoints of segment k travel back while segment k+1 runs.
int forward_streaming(V2Context *c, size_t T, size_t R, const __half *x_host, const __half *h0, const __half *c0,
                      const float *w_ih, const float *w_hh, const float *b_ih, const float *b_hh, __half *y_host,
                      flstm_GateCacheHost cache, int hd, int cd, __half *hy, __half *cy, cudaStream_t sc, cudaStream_t sh,
                      cudaStream_t sd) {
    const size_t B = c->B, I = c->I, H = c->H, slab = B * H, S = c->seg_steps, nseg = (T + S - 1) / S;
    StreamSlots &sl = c->slots;
    flstm_engine *e = c->seg_engine;
    FLSTM_TRY(set_weights_cached(e, c->packed_seg, w_ih, w_hh, b_ih, b_hh, sc));
    void *hs = nullptr;
    float *cs = nullptr;
    FLSTM_TRY(flstm_engine_cache_ptrs(e, 0, nullptr, &cs, &hs, nullptr));
    FLSTM_CUDA_TRY(cudaMemcpyAsync(sl.h_state[0], h0, slab * 2, cudaMemcpyDeviceToDevice, sc));
    FLSTM_TRY(simt::convert(FLSTM_DTYPE_F16, c0, FLSTM_DTYPE_F32, sl.c_state[0], slab, sc));
    auto seg_len = [&](size_t k) { return (k + 1) * S <= T ? S : T - k * S; };
    auto load_x = [&](size_t k) -> int {  // on the h2d stream, into slot k & 1
        cudaEvent_t ev;
        FLSTM_TRY(c->event(3 * k, &ev));
        FLSTM_CUDA_TRY(cudaMemcpyAsync(sl.x[k & 1], bytes(x_host) + k * S * B * I * 2, seg_len(k) * B * I * 2, cudaMemcpyDefault, sh));
        FLSTM_CUDA_TRY(cudaEventRecord(ev, sh));
        return FLSTM_OK;
    };
    for (size_t k = 0; k < nseg && k < 2; ++k) FLSTM_TRY(load_x(k));
    for (size_t k = 0; k < nseg; ++k) {
        const size_t t0 = k * S, n = seg_len(k), slot = k & 1;
        cudaEvent_t ev_x, ev_done, ev_out;
        FLSTM_TRY(c->event(3 * k, &ev_x));
        FLSTM_TRY(c->event(3 * k + 1, &ev_done));
        FLSTM_TRY(c->event(3 * k + 2, &ev_out));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(sc, ev_x, 0));
        if (k >= 2) {  // the y / checkpoint slots of segment k-2 must have left the device
            cudaEvent_t ev_prev;
            FLSTM_TRY(c->event(3 * (k - 2) + 2, &ev_prev));
            FLSTM_CUDA_TRY(cudaStreamWaitEvent(sc, ev_prev, 0));
        }
        FLSTM_TRY(flstm_engine_forward(e, n, sl.x[slot], sl.h_state[slot], sl.c_state[slot], sl.y[slot], sl.h_state[slot ^ 1],
                                       sl.c_state[slot ^ 1], sc));
        // checkpoints: entry e = state entering step e*R; this segment owns entries e0 .. e1-1.  Entry e0 is the
        // state that entered the segment (S is a multiple of R), the others sit in the engine's segment buffers.
        const size_t e0 = t0 / R, e1 = (t0 + n + R - 1) / R, ne = e1 - e0;
        if (cache.h_ptr) {
            FLSTM_TRY(simt::convert(FLSTM_DTYPE_F16, sl.h_state[slot], hd, sl.out_h[slot], slab, sc));
            if (ne > 1)
                FLSTM_TRY(simt::gather_slabs(FLSTM_DTYPE_F16, bytes(hs) + R * slab * 2, slab, R, ne - 1, hd,
                                             bytes(sl.out_h[slot]) + slab * dtype_size(hd), sc));
        }
        if (cache.c_ptr) {
            FLSTM_TRY(simt::convert(FLSTM_DTYPE_F32, sl.c_state[slot], cd, sl.out_c[slot], slab, sc));
            if (ne > 1)
                FLSTM_TRY(simt::gather_slabs(FLSTM_DTYPE_F32, cs + R * slab, slab, R, ne - 1, cd,
                                             bytes(sl.out_c[slot]) + slab * dtype_size(cd), sc));
        }
        FLSTM_CUDA_TRY(cudaEventRecord(ev_done, sc));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(sd, ev_done, 0));
        FLSTM_CUDA_TRY(cudaMemcpyAsync(bytes(y_host) + t0 * slab * 2, sl.y[slot], n * slab * 2, cudaMemcpyDefault, sd));
        if (cache.h_ptr)
            FLSTM_CUDA_TRY(cudaMemcpyAsync(bytes(cache.h_ptr) + e0 * slab * dtype_size(hd), sl.out_h[slot], ne * slab * dtype_size(hd),
                                           cudaMemcpyDefault, sd));
        if (cache.c_ptr)
            FLSTM_CUDA_TRY(cudaMemcpyAsync(bytes(cache.c_ptr) + e0 * slab * dtype_size(cd), sl.out_c[slot], ne * slab * dtype_size(cd),
                                           cudaMemcpyDefault, sd));
        FLSTM_CUDA_TRY(cudaEventRecord(ev_out, sd));
        if (k + 2 < nseg) {  // the x slot is free once segment k has run
            FLSTM_CUDA_TRY(cudaStreamWaitEvent(sh, ev_done, 0));
            FLSTM_TRY(load_x(k + 2));
        }
    }
    FLSTM_CUDA_TRY(cudaMemcpyAsync(hy, sl.h_state[nseg & 1], slab * 2, cudaMemcpyDeviceToDevice, sc));
    FLSTM_TRY(simt::convert(FLSTM_DTYPE_F32, sl.c_state[nseg & 1], FLSTM_DTYPE_F16, cy, slab, sc));
    return FLSTM_OK;
}

// Backward over the segments from the last to the first.  Per segment: x, dY and the checkpoint that entered it
// come from the caller's tensors, the engine re-runs the segment's forward and the BPTT, dX goes back.
int backward_streaming(V2Context *c, size_t T, size_t R, const __half *x_host, flstm_GateCacheHost cache, int hd, int cd,
                       const __half *dy_host, const __half *d_hn, const __half *d_cn, const __half *h0, const __half *c0,
                       const float *w_ih, const float *w_hh, const float *b_ih, const float *b_hh, __half *dx_host,
                       float *dh0, float *dc0, cudaStream_t sc, cudaStream_t sh, cudaStream_t sd) {
    const size_t B = c->B, I = c->I, H = c->H, slab = B * H, S = c->seg_steps, nseg = (T + S - 1) / S;
    StreamSlots &sl = c->slots;
    flstm_engine *e = c->seg_engine;
    if (nseg > 1 && (!cache.h_ptr || !cache.c_ptr))
        return set_error(FLSTM_ERR_INVALID, "a backward pass over %zu segments needs both checkpoint tensors", nseg);
    FLSTM_TRY(set_weights_cached(e, c->packed_seg, w_ih, w_hh, b_ih, b_hh, sc));
    auto seg_len = [&](size_t k) { return (k + 1) * S <= T ? S : T - k * S; };
    auto load = [&](size_t r) -> int {  // r-th segment from the end, on the h2d stream, into slot r & 1
        const size_t k = nseg - 1 - r, t0 = k * S, n = seg_len(k), slot = r & 1;
        cudaEvent_t ev;
        FLSTM_TRY(c->event(3 * r, &ev));
        FLSTM_CUDA_TRY(cudaMemcpyAsync(sl.x[slot], bytes(x_host) + t0 * B * I * 2, n * B * I * 2, cudaMemcpyDefault, sh));
        FLSTM_CUDA_TRY(cudaMemcpyAsync(sl.dy[slot], bytes(dy_host) + t0 * slab * 2, n * slab * 2, cudaMemcpyDefault, sh));
        if (k > 0 || !c0) {  // segment 0 starts from h0 / c0 themselves when the caller passed them
            const size_t en = t0 / R;
            FLSTM_CUDA_TRY(cudaMemcpyAsync(sl.ck_raw_h[slot], bytes(cache.h_ptr) + en * slab * dtype_size(hd), slab * dtype_size(hd),
                                           cudaMemcpyDefault, sh));
            FLSTM_CUDA_TRY(cudaMemcpyAsync(sl.ck_raw_c[slot], bytes(cache.c_ptr) + en * slab * dtype_size(cd), slab * dtype_size(cd),
                                           cudaMemcpyDefault, sh));
        }
        FLSTM_CUDA_TRY(cudaEventRecord(ev, sh));
        return FLSTM_OK;
    };
    if (!c0 && (!cache.h_ptr || !cache.c_ptr)) return set_error(FLSTM_ERR_INVALID, "c0 is null and there are no checkpoints");
    for (size_t r = 0; r < nseg && r < 2; ++r) FLSTM_TRY(load(r));
    for (size_t r = 0; r < nseg; ++r) {
        const size_t k = nseg - 1 - r, t0 = k * S, n = seg_len(k), slot = r & 1;
        cudaEvent_t ev_in, ev_done, ev_out;
        FLSTM_TRY(c->event(3 * r, &ev_in));
        FLSTM_TRY(c->event(3 * r + 1, &ev_done));
        FLSTM_TRY(c->event(3 * r + 2, &ev_out));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(sc, ev_in, 0));
        if (r >= 2) {  // the dX slot of two segments ago must have left the device
            cudaEvent_t ev_prev;
            FLSTM_TRY(c->event(3 * (r - 2) + 2, &ev_prev));
            FLSTM_CUDA_TRY(cudaStreamWaitEvent(sc, ev_prev, 0));
        }
        if (k > 0 || !c0) {
            FLSTM_TRY(simt::convert(hd, sl.ck_raw_h[slot], FLSTM_DTYPE_F16, sl.ck_h[slot], slab, sc));
            FLSTM_TRY(simt::convert(cd, sl.ck_raw_c[slot], FLSTM_DTYPE_F32, sl.ck_c[slot], slab, sc));
        } else {
            FLSTM_CUDA_TRY(cudaMemcpyAsync(sl.ck_h[slot], h0, slab * 2, cudaMemcpyDeviceToDevice, sc));
            FLSTM_TRY(simt::convert(FLSTM_DTYPE_F16, c0, FLSTM_DTYPE_F32, sl.ck_c[slot], slab, sc));
        }
        FLSTM_TRY(flstm_engine_backward_segment(e, n, r == 0, k == 0, sl.x[slot], sl.ck_h[slot], sl.ck_c[slot], sl.dy[slot], d_hn,
                                                d_cn, sl.dx[slot], dh0, dc0, sc));
        FLSTM_CUDA_TRY(cudaEventRecord(ev_done, sc));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(sd, ev_done, 0));
        FLSTM_CUDA_TRY(cudaMemcpyAsync(bytes(dx_host) + t0 * B * I * 2, sl.dx[slot], n * B * I * 2, cudaMemcpyDefault, sd));
        FLSTM_CUDA_TRY(cudaEventRecord(ev_out, sd));
        if (r + 2 < nseg) {
            FLSTM_CUDA_TRY(cudaStreamWaitEvent(sh, ev_done, 0));
            FLSTM_TRY(load(r + 2));
        }
    }
    return FLSTM_OK;
}

int copy_gradients_out(flstm_engine *e, size_t I, size_t H, float *dw_ih, float *dw_hh, float *db_ih, float *db_hh,
                       cudaStream_t sc) {
    float *g_ih = nullptr, *g_hh = nullptr, *g_b = nullptr;
    FLSTM_TRY(flstm_engine_grad_ptrs(e, 0, &g_ih, &g_hh, &g_b));
    FLSTM_CUDA_TRY(cudaMemcpyAsync(dw_ih, g_ih, 4 * H * I * sizeof(float), cudaMemcpyDeviceToDevice, sc));
    FLSTM_CUDA_TRY(cudaMemcpyAsync(dw_hh, g_hh, 4 * H * H * sizeof(float), cudaMemcpyDeviceToDevice, sc));
    FLSTM_CUDA_TRY(cudaMemcpyAsync(db_ih, g_b, 4 * H * sizeof(float), cudaMemcpyDeviceToDevice, sc));
    FLSTM_CUDA_TRY(cudaMemcpyAsync(db_hh, g_b, 4 * H * sizeof(float), cudaMemcpyDeviceToDevice, sc));
    return FLSTM_OK;
}

int sync_three(cudaStream_t sc, cudaStream_t sh, cudaStream_t sd) {
    FLSTM_CUDA_TRY(cudaStreamSynchronize(sh));
    FLSTM_CUDA_TRY(cudaStreamSynchronize(sc));
    FLSTM_CUDA_TRY(cudaStreamSynchronize(sd));
    return FLSTM_OK;
}

// Whether this call runs in streaming mode; reserves what the chosen mode needs.  `stateless_backward`: a backward
// call that cannot use the resident engine's gate cache consumes the caller's checkpoints segment by segment.
int choose_mode(V2Context *c, size_t T, size_t R, bool stateless_backward, bool *streaming) {
    const bool over_budget = c->resident_bytes(T, R) > c->budget;
    *streaming = false;
    if (over_budget || stateless_backward) {
        int st = c->reserve_streaming(pick_segment(*c, T, R), R);
        if (st == FLSTM_OK) {
            *streaming = true;
        } else if (st != FLSTM_ERR_UNSUPPORTED || over_budget) {
            return st;  // shapes the tensor-core path cannot tile stay resident while they fit
        }
    }
    if (!*streaming) FLSTM_TRY(c->reserve_resident(T, R));
    g_last_streaming = *streaming ? 1 : 0;
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
    FLSTM_TRY(get_context(B, I, H, &c));
    c->cache_valid = false;
    const int hd = opt.h_dtype == FLSTM_GATE_CACHE_FLOAT16 ? FLSTM_DTYPE_F16 : FLSTM_DTYPE_F32;
    const int cd = opt.c_dtype == FLSTM_GATE_CACHE_FLOAT16 ? FLSTM_DTYPE_F16 : FLSTM_DTYPE_F32;
    bool streaming = false;
    FLSTM_TRY(choose_mode(c, T, R, false, &streaming));
    g_last_device_bytes = c->device_bytes();
    if (streaming) {
        int st = forward_streaming(c, T, R, x_host, h0, c0, w_ih, w_hh, b_ih, b_hh, y_host, cache, hd, cd, hy, cy, sc, sh, sd);
        int sy = sync_three(sc, sh, sd);
        return st != FLSTM_OK ? st : sy;
    }
    const size_t slab = B * H;
    const bool x_on_device = is_device_pointer(x_host), y_on_device = is_device_pointer(y_host);
    const void *x_dev = x_on_device ? (const void *)x_host : c->x;
    void *y_dev = y_on_device ? (void *)y_host : c->y;
    const size_t nchk = (T + R - 1) / R;
    const bool ch_dev = cache.h_ptr && is_device_pointer(cache.h_ptr);
    const bool cc_dev = cache.c_ptr && is_device_pointer(cache.c_ptr);
    char *chk_h_dev = static_cast<char *>(ch_dev ? cache.h_ptr : c->chk_h);
    char *chk_c_dev = static_cast<char *>(cc_dev ? cache.c_ptr : c->chk_c);
    void *hs = nullptr;
    float *cs = nullptr;
    FLSTM_TRY(flstm_engine_cache_ptrs(c->engine, 0, nullptr, &cs, &hs, nullptr));
    FLSTM_TRY(set_weights_cached(c->engine, c->packed_resident, w_ih, w_hh, b_ih, b_hh, sc));

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
    FLSTM_TRY(sync_three(sc, sh, sd));
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
    if (T == 0 || B == 0 || I == 0 || H == 0) return FLSTM_OK;
    if (R == 0) return set_error(FLSTM_ERR_INVALID, "recompute_interval must be >= 1");
    if (sc == sh || sc == sd || sh == sd) return set_error(FLSTM_ERR_INVALID, "compute, h2d and d2h streams must be distinct");
    if (!x_host || !y_host || !dy_host || !h0 || !w_ih || !w_hh || !b_ih || !b_hh || !dx_host || !dw_ih || !dw_hh ||
        !db_ih || !db_hh || !dh0 || !dc0)
        return set_error(FLSTM_ERR_INVALID, "null pointer argument");
    std::lock_guard<std::mutex> lock(g_mutex);
    V2Context *c = nullptr;
    FLSTM_TRY(get_context(B, I, H, &c));
    const size_t slab = B * H;
    const int hd = opt.h_dtype == FLSTM_GATE_CACHE_FLOAT16 ? FLSTM_DTYPE_F16 : FLSTM_DTYPE_F32;
    const int cd = opt.c_dtype == FLSTM_GATE_CACHE_FLOAT16 ? FLSTM_DTYPE_F16 : FLSTM_DTYPE_F32;
    // the gate cache of the resident engine belongs to this backward when the forward of the same y tensor and
    // length ran last.  A backward that directly follows its forward uses the weights that forward packed.
    const bool have_cache = c->engine && c->cache_valid && c->fwd_y == y_host && c->fwd_T == T;
    const bool can_use_checkpoints = cache.h_ptr && cache.c_ptr;
    bool streaming = false;
    FLSTM_TRY(choose_mode(c, T, R, !have_cache && can_use_checkpoints, &streaming));
    g_last_device_bytes = c->device_bytes();
    if (streaming) {
        int st = backward_streaming(c, T, R, x_host, cache, hd, cd, dy_host, d_hn, d_cn, h0, c0, w_ih, w_hh, b_ih, b_hh, dx_host,
                                    dh0, dc0, sc, sh, sd);
        if (st == FLSTM_OK) st = copy_gradients_out(c->seg_engine, I, H, dw_ih, dw_hh, db_ih, db_hh, sc);
        int sy = sync_three(sc, sh, sd);
        return st != FLSTM_OK ? st : sy;
    }
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
        // stateless call without usable checkpoints (or on a shape the segment path cannot tile): rebuild the
        // gate cache by running the recurrence again from x, h0, c0
        if (!c0) return set_error(FLSTM_ERR_INVALID, "c0 is null");
        const void *x_dev = nullptr;
        FLSTM_TRY(stage_in(x_host, c->x, T * B * I * 2, sh, &x_dev));
        FLSTM_CUDA_TRY(cudaEventRecord(c->ev_in, sh));
        FLSTM_CUDA_TRY(cudaStreamWaitEvent(sc, c->ev_in, 0));
        FLSTM_TRY(set_weights_cached(c->engine, c->packed_resident, w_ih, w_hh, b_ih, b_hh, sc));
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
    FLSTM_TRY(copy_gradients_out(c->engine, I, H, dw_ih, dw_hh, db_ih, db_hh, sc));
    FLSTM_TRY(sync_three(sc, sh, sd));
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

void flstm_v2_set_weight_version(unsigned long long version) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_weight_version = version;
}

void flstm_v2_last_call_info(size_t *device_bytes, int *streaming) {
    if (device_bytes) *device_bytes = g_last_device_bytes;
    if (streaming) *streaming = g_last_streaming;
}

}  // extern "C"
