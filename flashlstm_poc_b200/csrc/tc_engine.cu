// Tensor-core (tcgen05 / TMEM / TMA) path of the engine: planning, tensor maps, weight packing in
// the tile-interleaved gate order, and the per-layer forward / backward schedules.
//
// Gate order.  Every 4H-indexed tensor of this path (rows of W_ih and W_hh, the bias, the columns
// of the projection / gate cache and of dG) uses the tile-interleaved order
//     index(g, u) = ((u / 16) * 4 + g) * 16 + u % 16
// so that the 64 rows a recurrent CTA owns are the four gates of 16 hidden units.  Weight and bias
// gradients are written back in torch order (g*H + u) by the GEMM epilogue / a small kernel.
#include <algorithm>
#include <cstdlib>
#include <vector>

#include "common.cuh"
#include "engine.h"
#include "kernels.h"
#include "tc_common.cuh"
#include "tc_kernels.h"

namespace flstm_b200 {
namespace tc {

namespace {

struct TcLayer {
    CUtensorMap tm_w;   // w_hh (4H, H), 64x64 boxes, 128B swizzle
    CUtensorMap tm_h;   // hs (Tcap+1, B, H), 1 x BT x 64 boxes, 128B swizzle
    CUtensorMap tm_g;   // gates (Tcap, B, 4H), 1 x BT x 64 boxes, no swizzle
    CUtensorMap tm_dg;  // dG (Tcap, B, 4H), 1 x BT x 64 boxes, 128B swizzle (BPTT operand)
    // wide-batch path (one GEMM launch per step)
    CUtensorMap tm_hs3;    // hs (Tcap+1, B, H), 1 x 128 x 64 boxes, 128B swizzle
    CUtensorMap tm_wstep;  // w_hh (4H, H), bn_fwd x 64 boxes, 128B swizzle
    CUtensorMap tm_dg3;    // dG (Tcap, B, 4H), 1 x 128 x 64 boxes, 128B swizzle
    CUtensorMap tm_g_ep, tm_c_ep, tm_h_ep;  // 32-row epilogue tiles of gates / cs / hs
};

struct TcState {
    int sms = 0;
    size_t smem_limit = 0;
    FwdPlan fwd{};
    BwdPlan bwd{};
    bool bwd_ok = false;
    StepPlan step{};
    float *dh_parts = nullptr;  // wide-batch path: fp32 (L, splits, B, H) partial sums of dG_t W_hh
    std::vector<TcLayer> layers;
    unsigned int *err_host = nullptr;  // pinned mirror of the device error word
};

TcState *state(Engine &e) { return static_cast<TcState *>(e.tc_state); }

__device__ __forceinline__ int interleaved_to_torch_row(int r, int H) {
    const int tile = r >> 6, g = (r >> 4) & 3, u = r & 15;
    return g * H + tile * 16 + u;
}

template <typename T>
__global__ void pack_rows_kernel(const float *__restrict__ w, int H, int K, T *__restrict__ out) {
    const size_t total = (size_t)4 * H * K;
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const int r = (int)(i / K), k = (int)(i % K);
        st(out + i, w[(size_t)interleaved_to_torch_row(r, H) * K + k]);
    }
}

__global__ void pack_bias_kernel(const float *__restrict__ a, const float *__restrict__ b, int H, float *__restrict__ out) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < 4 * H) {
        const int o = interleaved_to_torch_row(r, H);
        out[r] = a[o] + b[o];
    }
}

__global__ void unpermute_kernel(const float *__restrict__ in, int H, float *__restrict__ out) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < 4 * H) out[interleaved_to_torch_row(r, H)] = in[r];
}

int check_launch(const char *what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(err));
    return FLSTM_OK;
}

inline char *byte_ptr(void *p) { return static_cast<char *>(p); }
inline const char *byte_ptr(const void *p) { return static_cast<const char *>(p); }

}  // namespace

int pack_weights_interleaved(int dtype, const float *w, size_t H, size_t K, void *out, cudaStream_t s) {
    const size_t total = 4 * H * K;
    int grid = (int)((total + 255) / 256);
    if (grid > 148 * 16) grid = 148 * 16;
    if (dtype == FLSTM_DTYPE_F16) pack_rows_kernel<<<grid, 256, 0, s>>>(w, (int)H, (int)K, static_cast<__half *>(out));
    else pack_rows_kernel<<<grid, 256, 0, s>>>(w, (int)H, (int)K, static_cast<__nv_bfloat16 *>(out));
    return check_launch("pack_weights");
}

int pack_bias_interleaved(const float *b_ih, const float *b_hh, size_t H, float *out, cudaStream_t s) {
    pack_bias_kernel<<<(int)((4 * H + 255) / 256), 256, 0, s>>>(b_ih, b_hh, (int)H, out);
    return check_launch("pack_bias");
}

int unpermute_vector(const float *in, size_t H, float *out, cudaStream_t s) {
    unpermute_kernel<<<(int)((4 * H + 255) / 256), 256, 0, s>>>(in, (int)H, out);
    return check_launch("unpermute");
}

bool supported(const flstm_engine_config &cfg) {
    if (cfg.dtype != FLSTM_DTYPE_F16 && cfg.dtype != FLSTM_DTYPE_BF16) return false;
    if (cfg.hidden_size % 64 || cfg.input_size % 8) return false;
    const char *off = std::getenv("FLSTM_DISABLE_TC");
    if (off && off[0] == '1') return false;
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (major != 10) return false;
    int optin = 0;
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    StepPlan sp;
    if (plan_step((int)cfg.batch, (int)cfg.hidden_size, device_sm_count(), (size_t)optin, &sp) == FLSTM_OK && sp.use) return true;
    FwdPlan fp;
    if (plan_fwd((int)cfg.batch, (int)cfg.hidden_size, device_sm_count(), (size_t)optin, &fp) != FLSTM_OK) return false;
    if (cfg.training) {
        BwdPlan bp;
        if (plan_bwd((int)cfg.batch, (int)cfg.hidden_size, device_sm_count(), (size_t)optin, &bp) != FLSTM_OK) return false;
    }
    return true;
}

int init(Engine &e) {
    TcState *st = new TcState();
    e.tc_state = st;
    st->sms = device_sm_count();
    int optin = 0;
    FLSTM_CUDA_TRY(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, e.device));
    st->smem_limit = (size_t)optin;
    FLSTM_TRY(plan_step((int)e.cfg.batch, (int)e.cfg.hidden_size, st->sms, st->smem_limit, &st->step));
    void *raw = nullptr;
    if (st->step.use) {
        st->bwd_ok = e.cfg.training != 0;
        if (e.cfg.training) {
            const size_t n = e.layers.size() * (size_t)st->step.splits * e.cfg.batch * e.cfg.hidden_size;
            FLSTM_CUDA_TRY(cudaMalloc(&raw, n * sizeof(float)));
            st->dh_parts = static_cast<float *>(raw);
        }
    } else {
        FLSTM_TRY(plan_fwd((int)e.cfg.batch, (int)e.cfg.hidden_size, st->sms, st->smem_limit, &st->fwd));
        if (e.cfg.training) {
            FLSTM_TRY(plan_bwd((int)e.cfg.batch, (int)e.cfg.hidden_size, st->sms, st->smem_limit, &st->bwd));
            st->bwd_ok = true;
        }
    }
    st->layers.resize(e.layers.size());
    FLSTM_CUDA_TRY(cudaMalloc(&raw, 1024 * sizeof(unsigned int)));
    e.sync_words = static_cast<unsigned int *>(raw);
    FLSTM_CUDA_TRY(cudaMemset(raw, 0, 1024 * sizeof(unsigned int)));
    // one bias-gradient scratch per layer: with the cross-layer wavefront two layers may reduce at once
    FLSTM_CUDA_TRY(cudaMalloc(&raw, e.layers.size() * (size_t)simt::column_sum_scratch_floats(4 * e.cfg.hidden_size) * sizeof(float)));
    e.db_part = static_cast<float *>(raw);
    FLSTM_CUDA_TRY(cudaMallocHost(&raw, sizeof(unsigned int)));
    st->err_host = static_cast<unsigned int *>(raw);
    *st->err_host = 0;
    return FLSTM_OK;
}

void destroy(Engine &e) {
    TcState *st = state(e);
    if (!st) return;
    if (st->err_host) cudaFreeHost(st->err_host);
    if (st->dh_parts) cudaFree(st->dh_parts);
    delete st;
    e.tc_state = nullptr;
}

int on_capacity_change(Engine &e) {
    TcState *st = state(e);
    // time extent of the gate-sized buffers (one segment with activation checkpoints); dG has one slot more then
    const size_t B = e.cfg.batch, H = e.cfg.hidden_size, cap = e.buf_steps, dg_steps = cap + (e.recompute ? 1 : 0);
    for (size_t li = 0; li < e.layers.size(); ++li) {
        auto &l = e.layers[li];
        auto &t = st->layers[li];
        FLSTM_TRY(make_tensor_map_2d(&t.tm_w, l.w_hh, 4 * H, H, H, 64, 64, true));
        if (st->step.use) {
            FLSTM_TRY(make_tensor_map_3d(&t.tm_hs3, l.hs, cap + 1, B, H, H, B * H, 128, 64, true));
            FLSTM_TRY(make_tensor_map_2d(&t.tm_wstep, l.w_hh, 4 * H, H, H, (st->step.pair || st->step.fwd_pair) ? st->step.bn_fwd / 2 : st->step.bn_fwd, 64, true));
            FLSTM_TRY(make_tensor_map_3d_tile(&t.tm_g_ep, l.gates, 2, cap, B, 4 * H, 32, 64));
            FLSTM_TRY(make_tensor_map_3d_tile(&t.tm_c_ep, l.cs, 4, cap + 1, B, H, 32, 16));
            FLSTM_TRY(make_tensor_map_3d_tile(&t.tm_h_ep, l.hs, 2, cap + 1, B, H, 32, 16));
            if (e.cfg.training && l.dg)
                FLSTM_TRY(make_tensor_map_3d(&t.tm_dg3, l.dg, dg_steps, B, 4 * H, 4 * H, B * 4 * H, 128, 64, true));
            continue;
        }
        FLSTM_TRY(make_tensor_map_chunked(&t.tm_h, l.hs, cap + 1, B, H, st->fwd.pair ? st->fwd.BT / 2 : st->fwd.BT, st->fwd.ch));
        FLSTM_TRY(make_tensor_map_3d(&t.tm_g, l.gates, cap, B, 4 * H, 4 * H, B * 4 * H, st->fwd.BT, 64, false));
        if (e.cfg.training && l.dg)
            FLSTM_TRY(make_tensor_map_chunked(&t.tm_dg, l.dg, dg_steps, B, 4 * H, st->bwd.BT, st->bwd.ch));
    }
    return FLSTM_OK;
}

int set_weights(Engine &e, int layer, const float *w_ih, const float *w_hh, const float *b_ih, const float *b_hh,
                cudaStream_t s) {
    auto &l = e.layers[layer];
    const size_t H = e.cfg.hidden_size;
    FLSTM_TRY(pack_weights_interleaved(e.cfg.dtype, w_ih, H, l.in_size, l.w_ih, s));
    FLSTM_TRY(pack_weights_interleaved(e.cfg.dtype, w_hh, H, H, l.w_hh, s));
    FLSTM_TRY(pack_bias_interleaved(b_ih, b_hh, H, l.bias, s));
    return FLSTM_OK;
}

// Deferred error reporting: the device error word is mirrored into pinned host memory after each
// layer; a non-zero mirror fails the NEXT call (and flstm_engine_synchronize reports it at once).
static int check_async_error(Engine &e) {
    TcState *st = state(e);
    if (st && *st->err_host) {
        const unsigned int code = *st->err_host;
        *st->err_host = 0;
        cudaMemset(e.sync_words, 0, sizeof(unsigned int));
        return set_error(FLSTM_ERR_TIMEOUT, "a bounded device-side wait expired in a persistent kernel (code %u)", code);
    }
    return FLSTM_OK;
}

int poll_error(Engine &e) { return check_async_error(e); }

int forward_layer(Engine &e, int li, size_t t0, size_t t1, const void *x_l, void *y_out, cudaStream_t s) {
    TcState *st = state(e);
    FLSTM_TRY(check_async_error(e));
    auto &l = e.layers[li];
    auto &t = st->layers[li];
    const size_t B = e.cfg.batch, H = e.cfg.hidden_size, es = dtype_size(e.cfg.dtype), n = t1 - t0;
    unsigned int *err = e.sync_words;
    size_t m0 = e.timer.mark(s);
    // P = X W_ih^T + (b_ih + b_hh) for the steps of the range, 16-bit, columns tile-interleaved
    FLSTM_TRY(gemm(e.cfg.dtype, e.cfg.dtype, n * B, 4 * H, l.in_size, byte_ptr(x_l) + t0 * B * l.in_size * es, l.in_size, false,
                   l.w_ih, l.in_size, false, byte_ptr(l.gates) + t0 * B * 4 * H * es, 4 * H, l.bias, 0, err, st->sms, s));
    size_t m1 = e.timer.mark(s);
    if (st->step.use) {
        CUtensorMap tm_y;
        if (y_out) FLSTM_TRY(make_tensor_map_3d_tile(&tm_y, y_out, 2, t1, B, H, 32, 16));
        const StepFwdMaps maps{&t.tm_hs3, &t.tm_wstep, &t.tm_g_ep, &t.tm_c_ep, &t.tm_h_ep, y_out ? &tm_y : nullptr};
        // one cooperative launch for the whole range, unless layers run concurrently on their own streams (the
        // cross-layer wavefront): two cooperative grids that each need most of the machine must not be in flight
        // at once, each could hold SMs the other is waiting for
        if (st->step.fwd_persistent && wavefront_chunk(e, (size_t)-1) == 0) {
            FLSTM_CUDA_TRY(cudaMemsetAsync(e.sync_words + 1, 0, sizeof(unsigned int), s));
            WideFwdParams wp{};
            wp.err = err;
            wp.counter = e.sync_words + 1;
            wp.t0 = (int)t0;
            wp.nsteps = (int)n;
            wp.B = (int)B;
            wp.H = (int)H;
            wp.store_gates = (e.cfg.training && e.seg.keep_gates) ? 1 : 0;
            wp.wait_ns = e.wait_limit_ns;
            wp.extra_arrivals = e.selftest_missing_arrivals;
            FLSTM_TRY(lstm_wide_forward(e.cfg.dtype, st->step, maps, wp, st->sms, s));
            size_t m2 = e.timer.mark(s);
            e.timer.span(PH_PROJ, m0, m1);
            e.timer.span(PH_RECUR_FWD, m1, m2);
            e.launches += 2;
            FLSTM_CUDA_TRY(cudaMemcpyAsync(st->err_host, err, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
            return FLSTM_OK;
        }
        for (size_t step = t0; step < t1; ++step) {
            StepFwdParams sp{};
            sp.err = err;
            sp.t = (int)step;
            sp.B = (int)B;
            sp.H = (int)H;
            sp.store_gates = (e.cfg.training && e.seg.keep_gates) ? 1 : 0;
            FLSTM_TRY(lstm_step_forward(e.cfg.dtype, st->step, maps, sp, st->sms, s));
        }
        size_t m2 = e.timer.mark(s);
        e.timer.span(PH_PROJ, m0, m1);
        e.timer.span(PH_RECUR_FWD, m1, m2);
        e.launches += 1 + n;
        FLSTM_CUDA_TRY(cudaMemcpyAsync(st->err_host, err, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
        return FLSTM_OK;
    }
    FLSTM_CUDA_TRY(cudaMemsetAsync(e.sync_words + 1, 0, (size_t)st->fwd.ngroups * sizeof(unsigned int), s));
    FwdParams p{};
    p.cs = l.cs;
    p.hs = l.hs;
    p.y = y_out;
    p.gates = l.gates;
    p.counters = e.sync_words + 1;
    p.err = err;
    p.T = (int)n;
    p.t0 = (int)t0;
    p.B = (int)B;
    p.H = (int)H;
    p.store_gates = (e.cfg.training && e.seg.keep_gates) ? 1 : 0;
    p.trace = (li == 0 && t0 == 0) ? e.trace : nullptr;
    p.trace_steps = e.trace_steps;
    p.wait_ns = e.wait_limit_ns;
    p.extra_arrivals = e.selftest_missing_arrivals;
    FLSTM_TRY(lstm_forward_persistent(e.cfg.dtype, st->fwd, t.tm_w, t.tm_h, t.tm_g, p, s));
    size_t m2 = e.timer.mark(s);
    e.timer.span(PH_PROJ, m0, m1);
    e.timer.span(PH_RECUR_FWD, m1, m2);
    e.launches += 2;
    FLSTM_CUDA_TRY(cudaMemcpyAsync(st->err_host, err, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
    return FLSTM_OK;
}

// Wide-batch BPTT over the steps [t0, t1), descending: per step one pointwise kernel (dG_t, cell-gradient
// carry) and one split-K GEMM (the fp32 partial sums of dG_t W_hh that step t-1 adds to its dy).
static int backward_steps(Engine &e, int li, size_t T, size_t t0, size_t t1, const void *dy_l, const void *dhn_l,
                          const void *dcn_l, float *dh0_l, float *dc0_l, bool finalize, cudaStream_t s) {
    TcState *st = state(e);
    auto &l = e.layers[li];
    auto &t = st->layers[li];
    const size_t B = e.cfg.batch, H = e.cfg.hidden_size, es = dtype_size(e.cfg.dtype), slab = B * H;
    const int splits = st->step.splits;
    float *parts = st->dh_parts + (size_t)li * splits * slab;
    float *dc = e.dc_layers + (size_t)li * slab;
    if (t1 == T) {
        // gradients entering the last step: dh_n in partial buffer 0, dc_n in the carry
        if (dhn_l) { FLSTM_TRY(simt::convert(e.cfg.dtype, dhn_l, FLSTM_DTYPE_F32, parts, slab, s)); ++e.launches; }
        else FLSTM_CUDA_TRY(cudaMemsetAsync(parts, 0, slab * sizeof(float), s));
        if (dcn_l) { FLSTM_TRY(simt::convert(e.cfg.dtype, dcn_l, FLSTM_DTYPE_F32, dc, slab, s)); ++e.launches; }
        else FLSTM_CUDA_TRY(cudaMemsetAsync(dc, 0, slab * sizeof(float), s));
    }
    for (size_t step = t1; step-- > t0;) {
        const int nparts = (step == T - 1) ? 1 : splits;
        FLSTM_TRY(lstm_step_backward_pointwise(e.cfg.dtype, byte_ptr(l.gates) + step * B * 4 * H * es, l.cs + (step + 1) * slab,
                                               l.cs + step * slab, byte_ptr(dy_l) + step * slab * es, parts, nparts, dc,
                                               byte_ptr(l.dg) + step * B * 4 * H * es, (int)B, (int)H, s));
        ++e.launches;
        if (step > 0 || dh0_l || !finalize) {  // the product at step 0 is dh0, or the carry into the segment before
            FLSTM_TRY(lstm_step_backward_gemm(e.cfg.dtype, st->step, t.tm_dg3, t.tm_w, (int)step, (int)B, (int)H, parts,
                                              e.sync_words, st->sms, s));
            ++e.launches;
        }
    }
    if (t0 == 0 && finalize) {
        if (dh0_l) { FLSTM_TRY(sum_parts(parts, splits, slab, dh0_l, s)); ++e.launches; }
        if (dc0_l) FLSTM_CUDA_TRY(cudaMemcpyAsync(dc0_l, dc, slab * sizeof(float), cudaMemcpyDeviceToDevice, s));
    }
    return FLSTM_OK;
}

// Opt-in (FLSTM_WAVE_CHUNK=<steps per chunk>): measured neutral on configs 3 and 5, which already run at the
// board's power cap -- the overlap only lowers the SM clock (1.9 -> 1.6 GHz) -- so the default stays the
// layer-by-layer schedule.
size_t wavefront_chunk(const Engine &e, size_t n) {
    TcState *st = static_cast<TcState *>(e.tc_state);
    if (!st || !st->step.use || e.layers.size() < 2 || e.timer.enabled) return 0;
    const char *env = std::getenv("FLSTM_WAVE_CHUNK");
    if (!env) return 0;
    const long v = std::atol(env);
    if (v <= 0) return 0;
    return (size_t)v < n ? (size_t)v : 0;  // a single chunk is the plain layer-by-layer schedule
}

int backward_layer(Engine &e, int li, size_t T, size_t t0, size_t t1, const void *x_l, const void *dy_l, const void *dhn_l,
                   const void *dcn_l, void *dx_l, float *dh0_l, float *dc0_l, cudaStream_t s, cudaEvent_t dx_ready) {
    TcState *st = state(e);
    FLSTM_TRY(check_async_error(e));
    if (!st->bwd_ok) return set_error(FLSTM_ERR_UNSUPPORTED, "tensor-core backward is not planned for this engine");
    auto &l = e.layers[li];
    auto &t = st->layers[li];
    const size_t B = e.cfg.batch, H = e.cfg.hidden_size, es = dtype_size(e.cfg.dtype), n = t1 - t0;
    unsigned int *err = e.sync_words;
    size_t m0 = e.timer.mark(s);
    // with activation checkpoints `T` and the range are segment-local; only the segment that starts the sequence
    // finishes the recurrence (dh0 / dc0) and the layer's gradients
    const bool finalize = t0 == 0 && (!e.seg.active || e.seg.final_segment);
    if (st->step.use) FLSTM_TRY(backward_steps(e, li, T, t0, t1, dy_l, dhn_l, dcn_l, dh0_l, dc0_l, finalize, s));
    else {
    FLSTM_CUDA_TRY(cudaMemsetAsync(e.sync_words + 1, 0, (size_t)st->bwd.ngroups * sizeof(unsigned int), s));
    BwdParams p{};
    p.cs = l.cs;
    p.gates = l.gates;
    p.dg = l.dg;
    p.dy = dy_l;
    p.dhn = dhn_l;
    p.dcn = dcn_l;
    p.dh0 = dh0_l;
    p.dc0 = dc0_l;
    p.dc = e.dc_layers + (size_t)li * B * H;
    p.trace = (li == 0 && e.trace && t1 == T) ? e.trace + (size_t)e.trace_steps * 16 : nullptr;
    p.trace_steps = e.trace_steps;
    p.counters = e.sync_words + 1;
    p.err = err;
    p.T = (int)T;
    p.s0 = (int)(T - t1);
    p.s1 = (int)(T - t0) + (finalize ? 1 : 0);  // the last range also runs the iteration that writes dh0 / dc0
    p.B = (int)B;
    p.H = (int)H;
    p.wait_ns = e.wait_limit_ns;
    p.extra_arrivals = e.selftest_missing_arrivals;
    FLSTM_TRY(lstm_backward_persistent(e.cfg.dtype, st->bwd, t.tm_w, t.tm_dg, p, s));
    e.launches += 1;
    }
    size_t m1 = e.timer.mark(s);
    auto input_grad = [&]() -> int {
        if (!dx_l) return FLSTM_OK;
        // dX = dG W_ih for the steps of the range: W_ih (rows tile-interleaved, like dG's columns) is read as stored
        FLSTM_TRY(gemm(e.cfg.dtype, e.cfg.dtype, n * B, l.in_size, 4 * H, byte_ptr(l.dg) + t0 * B * 4 * H * es, 4 * H, false,
                       l.w_ih, l.in_size, true, byte_ptr(dx_l) + t0 * B * l.in_size * es, l.in_size, nullptr, 0, err, st->sms,
                       s));
        ++e.launches;
        return FLSTM_OK;
    };
    auto weight_grads = [&]() -> int {
        if (t0 != 0) return FLSTM_OK;
        // dW = dG^T [X | H_prev] over the whole sequence: both operands read as stored (reduction dim
        // T*B outermost); rows of the product are written back in torch gate order.  With a communicator
        // each block of the layer's gradients starts its allreduce as soon as it is complete.
        // With activation checkpoints the sum runs segment by segment (the n steps in the buffers now),
        // accumulating from the second segment on, and the allreduce follows the last one.
        const size_t steps = e.seg.active ? n : T;
        const bool acc = e.seg.active && !e.seg.first_segment, last = !e.seg.active || e.seg.final_segment;
        const size_t n_ih = 4 * H * l.in_size;
        // Opt-in (FLSTM_DW_SIDE_BY_SIDE=1, without a communicator): the two GEMMs run SIDE BY SIDE, each on its share of
        // the SMs.  Their 128 x 256 tiles run for milliseconds (K = T*B), so a last, partly filled round of tiles is
        // expensive -- config 3: 512 tiles each, 4 + 4 rounds on 148 SMs one after the other, 7 rounds on 74 + 74 SMs.
        // Measured: the phase drops from 27.7 to 26.0 ms, the whole step does not (122.2 against 120.7 ms): the board
        // is at its power cap in this phase, and SMs that idle through a partial round let the others clock higher.
        const size_t tiles_ih = ((4 * H + 127) / 128) * ((l.in_size + 255) / 256), tiles_hh = ((4 * H + 127) / 128) * ((H + 255) / 256);
        int sms_ih = (int)((size_t)st->sms * tiles_ih / (tiles_ih + tiles_hh));
        if (sms_ih < 1) sms_ih = 1;
        if (sms_ih > st->sms - 1) sms_ih = st->sms - 1;
        const int sms_hh = st->sms - sms_ih;
        auto rounds = [](size_t tiles, int sms) { return (tiles + sms - 1) / sms; };
        const size_t seq_rounds = rounds(tiles_ih, st->sms) + rounds(tiles_hh, st->sms);
        // a round = the time of one tile, whatever the number of CTAs working
        const size_t par_rounds = std::max(rounds(tiles_ih, sms_ih), rounds(tiles_hh, sms_hh));
        const char *sbs = std::getenv("FLSTM_DW_SIDE_BY_SIDE");
        const bool side_by_side = !e.comm && st->sms >= 2 && sbs && sbs[0] == '1' && par_rounds < seq_rounds;
        if (side_by_side) {
            FLSTM_TRY(e.ensure_aux_stream());
            FLSTM_CUDA_TRY(cudaEventRecord(e.aux_fork, s));
            FLSTM_CUDA_TRY(cudaStreamWaitEvent(e.aux_stream, e.aux_fork, 0));
            FLSTM_TRY(gemm(e.cfg.dtype, FLSTM_DTYPE_F32, 4 * H, H, steps * B, l.dg, 4 * H, true, l.hs, H, true, l.dw_hh, H,
                           nullptr, (int)H, err, sms_hh, e.aux_stream, acc));
            FLSTM_TRY(gemm(e.cfg.dtype, FLSTM_DTYPE_F32, 4 * H, l.in_size, steps * B, l.dg, 4 * H, true, x_l, l.in_size, true,
                           l.dw_ih, l.in_size, nullptr, (int)H, err, sms_ih, s, acc));
            FLSTM_CUDA_TRY(cudaEventRecord(e.aux_join, e.aux_stream));
            FLSTM_CUDA_TRY(cudaStreamWaitEvent(s, e.aux_join, 0));
        } else {
            FLSTM_TRY(gemm(e.cfg.dtype, FLSTM_DTYPE_F32, 4 * H, l.in_size, steps * B, l.dg, 4 * H, true, x_l, l.in_size, true,
                           l.dw_ih, l.in_size, nullptr, (int)H, err, st->sms, s, acc));
            if (last) FLSTM_TRY(e.reduce_grads(l.grad_offset, n_ih, s));
            FLSTM_TRY(gemm(e.cfg.dtype, FLSTM_DTYPE_F32, 4 * H, H, steps * B, l.dg, 4 * H, true, l.hs, H, true, l.dw_hh, H,
                           nullptr, (int)H, err, st->sms, s, acc));
        }
        FLSTM_TRY(simt::column_sum_two_pass(e.cfg.dtype, l.dg, steps * B, 4 * H,
                                            e.db_part + (size_t)li * simt::column_sum_scratch_floats(4 * H), l.db, (int)H, s,
                                            acc));
        if (last) FLSTM_TRY(e.reduce_grads(l.grad_offset + n_ih, l.grad_count - n_ih, s));
        e.launches += 4;
        return FLSTM_OK;
    };
    size_t m2, m3;
    if (dx_ready) {
        // wavefront: the layer below waits for dX of this range, so it goes first
        FLSTM_TRY(input_grad());
        FLSTM_CUDA_TRY(cudaEventRecord(dx_ready, s));
        m2 = e.timer.mark(s);
        FLSTM_TRY(weight_grads());
        m3 = e.timer.mark(s);
        e.timer.span(PH_XGRAD, m1, m2);
        e.timer.span(PH_WGRAD, m2, m3);
    } else {
        // weight gradients first: their allreduce then hides behind the input-gradient GEMM
        FLSTM_TRY(weight_grads());
        m2 = e.timer.mark(s);
        FLSTM_TRY(input_grad());
        m3 = e.timer.mark(s);
        e.timer.span(PH_WGRAD, m1, m2);
        e.timer.span(PH_XGRAD, m2, m3);
    }
    e.timer.span(PH_BPTT, m0, m1);
    FLSTM_CUDA_TRY(cudaMemcpyAsync(st->err_host, err, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
    return FLSTM_OK;
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

extern "C" int flstm_tc_plan(size_t batch, size_t hidden_size, int training, int sm_count, size_t smem_limit,
                             flstm_tc_plan_info *out) {
    using namespace flstm_b200;
    if (!out || sm_count < 1) return set_error(FLSTM_ERR_INVALID, "bad argument");
    *out = flstm_tc_plan_info{};
    tc::StepPlan sp{};
    FLSTM_TRY(tc::plan_step((int)batch, (int)hidden_size, sm_count, smem_limit, &sp));
    out->step_path = sp.use ? 1 : 0;
    out->step_bn_fwd = sp.bn_fwd;
    out->step_bn_bwd = sp.bn_bwd;
    out->step_splits = sp.splits;
    out->step_pair = sp.pair ? 1 : 0;
    out->step_fwd_pair = sp.fwd_pair ? 1 : 0;
    if (sp.use) return FLSTM_OK;
    tc::FwdPlan f{};
    FLSTM_TRY(tc::plan_fwd((int)batch, (int)hidden_size, sm_count, smem_limit, &f));
    out->fwd_batch_tile = f.BT;
    out->fwd_pair = f.pair ? 1 : 0;
    out->fwd_row_tiles_per_cta = f.rt;
    out->fwd_grid = f.grid;
    out->fwd_batch_groups = f.ngroups;
    out->fwd_tiles_per_group = f.nt;
    out->fwd_stages = f.stages;
    out->fwd_chunks_per_stage = f.ch;
    out->fwd_weights_resident = f.resident ? 1 : 0;
    out->fwd_smem_bytes = f.smem_bytes;
    if (training) {
        tc::BwdPlan b{};
        FLSTM_TRY(tc::plan_bwd((int)batch, (int)hidden_size, sm_count, smem_limit, &b, /*check_device=*/false));
        out->bwd_batch_tile = b.BT;
        out->bwd_cluster_size = b.KS;
        out->bwd_grid = b.grid;
        out->bwd_batch_groups = b.ngroups;
        out->bwd_tiles_per_group = b.nt;
        out->bwd_stages = b.stages;
        out->bwd_chunks_per_stage = b.ch;
        out->bwd_weights_resident = b.resident ? 1 : 0;
        out->bwd_smem_bytes = b.smem_bytes;
    }
    return FLSTM_OK;
}

extern "C" int flstm_tc_gemm(int dtype, int out_dtype, size_t M, size_t N, size_t K, const void *A, const void *B,
                             void *D, size_t ldd, const float *bias, int layout, void *stream) {
    using namespace flstm_b200;
    if (!A || !B || !D) return set_error(FLSTM_ERR_INVALID, "null pointer argument");
    if (layout < 0 || layout > 2) return set_error(FLSTM_ERR_INVALID, "layout must be 0, 1 or 2");
    unsigned int *err = tc::standalone_error_word();
    if (!err) return set_error(FLSTM_ERR_CUDA, "could not allocate the error word");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool a_mn = layout == 1, b_mn = layout >= 1;
    const size_t lda = a_mn ? M : K, ldb = b_mn ? N : K;
    FLSTM_TRY(tc::gemm(dtype, out_dtype, M, N, K, A, lda, a_mn, B, ldb, b_mn, D, ldd, bias, 0, err,
                       tc::device_sm_count(), s));
    unsigned int h = 0;
    FLSTM_CUDA_TRY(cudaMemcpyAsync(&h, err, sizeof(h), cudaMemcpyDeviceToHost, s));
    FLSTM_CUDA_TRY(cudaStreamSynchronize(s));
    if (h) {
        cudaMemsetAsync(err, 0, sizeof(h), s);
        return set_error(FLSTM_ERR_TIMEOUT, "tensor-core GEMM: a bounded device-side wait expired");
    }
    return FLSTM_OK;
}
