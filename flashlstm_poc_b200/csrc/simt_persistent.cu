// Persistent CUDA-core (fp32 FMA) recurrent kernels: one cooperative launch runs all the time steps of a
// layer, like the tensor-core kernels do, for the configurations that must stay in fp32 arithmetic
// (configuration 1: fp32, H = 256, B = 32, held to max-abs 2e-3 including dW) and for shapes the tensor path
// cannot tile.  A CTA owns 8 hidden units x 8 sequences for the whole sequence: its slice of W_hh stays in
// shared memory as fp32, four lanes share one (sequence, unit) pair (the four gates forward, four slices of
// the 4H-long sum backward), and the CTAs of a batch tile meet at a monotonic counter in global memory once
// per step (bounded wait, one release per CTA).  When the slices do not fit shared memory or the grid cannot
// be co-resident the engine falls back to one launch per step (simt_kernels.cu).
//
// Replaces, for the fp32 path, the same reference code as the tensor-core recurrent kernels: the per-step
// launches of src/lstm.cu:1241-1337 / src/kernels.cu:86-164 and flashlstm_v2/src/lstm_backward.cu:806-1110.
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"
#include "tc_recurrent.cuh"

namespace flstm_b200 {
namespace simt {

namespace {

constexpr int PB = 8, PU = 8;  // sequences x hidden units per CTA
constexpr int kThreads = 256;

using tc::wait_counter;
using tc::red_release_gpu_add;

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
persistent_forward_kernel(PersistentFwdParams p) {
    extern __shared__ float smem[];
    const int H = p.H, B = p.B, HS = H + 1;
    float *ws = smem;                 // [4 * PU][H + 1], row = unit * 4 + gate
    float *hs = ws + 4 * PU * HS;     // [PB][H + 1]
    __shared__ volatile uint32_t abort_w;
    const int tid = threadIdx.x;
    const int g = tid & 3, ul = (tid >> 2) % PU, bl = tid / (4 * PU);
    const int unit_tiles = (H + PU - 1) / PU;
    const int ut = blockIdx.x % unit_tiles, bt = blockIdx.x / unit_tiles;
    const int u0 = ut * PU, b0 = bt * PB;
    const T *w_hh = static_cast<const T *>(p.w_hh);
    T *hs_g = static_cast<T *>(p.hs), *gates = static_cast<T *>(p.gates), *y = static_cast<T *>(p.y);
    unsigned int *counter = p.counters + bt;
    if (tid == 0) abort_w = 0;
    for (int e = tid; e < 4 * PU * H; e += kThreads) {
        const int k = e % H, r = e / H, u = r >> 2, gg = r & 3;
        ws[r * HS + k] = (u0 + u < H) ? ld(w_hh + ((size_t)gg * H + u0 + u) * H + k) : 0.f;
    }
    __syncthreads();
    const size_t slab = (size_t)B * H, G = (size_t)4 * H;
    const int b = b0 + bl, u = u0 + ul;
    const bool owner = g == 0 && b < B && u < H;
    float c_keep = owner ? p.cs[(size_t)p.t0 * slab + (size_t)b * H + u] : 0.f;
    for (int tt = 0; tt < p.T; ++tt) {
        const int t = p.t0 + tt;
        if (tt > 0) {
            // h_{t-1} of this batch tile is complete when each of its unit_tiles CTAs has arrived tt times
            if (tid == 0 && !wait_counter(counter, (unsigned)unit_tiles * (unsigned)tt + p.extra_arrivals, p.err, &abort_w, 5u,
                                          p.wait_ns ? p.wait_ns : tc::kWaitLimitNs))
                abort_w = 1;
            __syncthreads();
            if (abort_w) break;
        }
        const T *h_prev = hs_g + (size_t)t * slab;
        for (int e = tid; e < PB * H; e += kThreads) {
            const int bb = e / H, k = e % H;
            hs[bb * HS + k] = (b0 + bb < B) ? ld(h_prev + (size_t)(b0 + bb) * H + k) : 0.f;
        }
        __syncthreads();
        const float *hrow = hs + bl * HS, *wrow = ws + (ul * 4 + g) * HS;
        float acc = 0.f;
#pragma unroll 8
        for (int k = 0; k < H; ++k) acc = fmaf(hrow[k], wrow[k], acc);
        const int base = (tid & 31) & ~3;
        const float s_i = __shfl_sync(0xffffffffu, acc, base), s_f = __shfl_sync(0xffffffffu, acc, base + 1);
        const float s_g = __shfl_sync(0xffffffffu, acc, base + 2), s_o = __shfl_sync(0xffffffffu, acc, base + 3);
        if (owner) {
            T *row = gates + ((size_t)t * B + b) * G;
            const float gi = sigmoid_acc(s_i + ld(row + u)), gf = sigmoid_acc(s_f + ld(row + H + u));
            const float gg = tanh_acc(s_g + ld(row + 2 * H + u)), go = sigmoid_acc(s_o + ld(row + 3 * H + u));
            const size_t idx = (size_t)b * H + u;
            const float c = fmaf(gf, c_keep, gi * gg);
            const float h = go * tanh_acc(c);
            c_keep = c;
            st(hs_g + (size_t)(t + 1) * slab + idx, h);  // first: it is what the other CTAs wait for
            p.cs[(size_t)(t + 1) * slab + idx] = c;
            if (y) st(y + (size_t)t * slab + idx, h);
            if (p.store_gates) {
                st(row + u, gi);
                st(row + H + u, gf);
                st(row + 2 * H + u, gg);
                st(row + 3 * H + u, go);
            }
        }
        __syncthreads();  // every store of the CTA is ordered before thread 0's release; hs may be overwritten
        if (tid == 0) red_release_gpu_add(counter, 1u);
    }
    if (tid == 0 && abort_w) atomicCAS(p.err, 0u, 1u);
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
persistent_backward_kernel(PersistentBwdParams p) {
    extern __shared__ float smem[];
    const int H = p.H, B = p.B, G = 4 * H, GS = G + 1;
    float *ws = smem;                  // [4H][PU + 1]: the CTA's columns of W_hh
    float *ds = ws + (size_t)G * (PU + 1);  // [PB][4H + 1]: dG_{t+1} of the CTA's sequences
    __shared__ volatile uint32_t abort_w;
    const int tid = threadIdx.x;
    const int q = tid & 3, ul = (tid >> 2) % PU, bl = tid / (4 * PU);
    const int unit_tiles = (H + PU - 1) / PU;
    const int ut = blockIdx.x % unit_tiles, bt = blockIdx.x / unit_tiles;
    const int u0 = ut * PU, b0 = bt * PB;
    const T *w_hh = static_cast<const T *>(p.w_hh);
    const T *gates = static_cast<const T *>(p.gates), *dy = static_cast<const T *>(p.dy);
    const T *dhn = static_cast<const T *>(p.dhn);
    T *dg = static_cast<T *>(p.dg);
    unsigned int *counter = p.counters + bt;
    if (tid == 0) abort_w = 0;
    for (int e = tid; e < G * PU; e += kThreads) {
        const int uu = e % PU, k = e / PU;
        ws[k * (PU + 1) + uu] = (u0 + uu < H) ? ld(w_hh + (size_t)k * H + u0 + uu) : 0.f;
    }
    __syncthreads();
    const size_t slab = (size_t)B * H;
    const int b = b0 + bl, u = u0 + ul;
    const bool owner = q == 0 && b < B && u < H;
    const size_t idx = (size_t)b * H + u;
    float dc_keep = owner ? p.dc[idx] : 0.f;  // carry entering this launch (the host seeds it from dc_n or zero)
    // reverse iterations [s0, s1): iteration s handles time t = T-1-s; s == T only forms dh0 / dc0
    for (int s = p.s0; s < p.s1; ++s) {
        const int t = p.T - 1 - s;
        float acc = 0.f;
        if (s > 0) {
            if (s > p.s0) {
                if (tid == 0 && !wait_counter(counter, (unsigned)unit_tiles * (unsigned)(s - p.s0) + p.extra_arrivals, p.err, &abort_w,
                                              6u, p.wait_ns ? p.wait_ns : tc::kWaitLimitNs))
                    abort_w = 1;
                __syncthreads();
                if (abort_w) break;
            }
            const T *dg_next = dg + (size_t)(t + 1) * B * G;
            for (int e = tid; e < PB * G; e += kThreads) {
                const int bb = e / G, k = e % G;
                ds[bb * GS + k] = (b0 + bb < B) ? ld(dg_next + (size_t)(b0 + bb) * G + k) : 0.f;
            }
            __syncthreads();
            const float *drow = ds + bl * GS;
#pragma unroll 8
            for (int k = q; k < G; k += 4) acc = fmaf(drow[k], ws[k * (PU + 1) + ul], acc);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        }
        if (owner) {
            if (t < 0) {
                if (p.dh0) p.dh0[idx] = acc;
                if (p.dc0) p.dc0[idx] = dc_keep;
            } else {
                float dh = acc + ld(dy + (size_t)t * slab + idx);
                if (s == 0 && dhn) dh += ld(dhn + idx);
                const T *grow = gates + ((size_t)t * B + b) * G;
                const float gi = ld(grow + u), gf = ld(grow + H + u), gg = ld(grow + 2 * H + u), go = ld(grow + 3 * H + u);
                const float tcv = tanh_acc(p.cs[(size_t)(t + 1) * slab + idx]);
                const float d_o = dh * tcv;
                const float dcv = dc_keep + dh * go * (1.f - tcv * tcv);
                const float cprev = p.cs[(size_t)t * slab + idx];
                T *drow_out = dg + ((size_t)t * B + b) * G;
                st(drow_out + u, dcv * gg * gi * (1.f - gi));
                st(drow_out + H + u, dcv * cprev * gf * (1.f - gf));
                st(drow_out + 2 * H + u, dcv * gi * (1.f - gg * gg));
                st(drow_out + 3 * H + u, d_o * go * (1.f - go));
                dc_keep = dcv * gf;
            }
        }
        if (t < 0) break;
        __syncthreads();  // stores ordered before thread 0's release; ds may be overwritten
        if (tid == 0) red_release_gpu_add(counter, 1u);
    }
    if (owner) p.dc[idx] = dc_keep;  // a later launch continues the recurrence from here
    if (tid == 0 && abort_w) atomicCAS(p.err, 0u, 1u);
}

template <typename Kern>
bool raise_smem_limit(Kern kern, size_t smem) {
    if (ensure_smem_limit(kern, smem) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return true;
}

template <typename Kern>
int coop_launch(Kern kern, int grid, size_t smem, cudaStream_t s, void *params, const char *what) {
    if (!raise_smem_limit(kern, smem)) return set_error(FLSTM_ERR_CUDA, "%s: cannot reserve %zu bytes of shared memory", what, smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs must be co-resident: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void *args[] = {params};
    cudaError_t e = cudaLaunchKernelExC(&cfg, reinterpret_cast<const void *>(kern), args);
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
    return FLSTM_OK;
}

size_t fwd_smem(int H) { return (size_t)(4 * PU + PB) * (H + 1) * sizeof(float); }
size_t bwd_smem(int H) { return ((size_t)4 * H * (PU + 1) + (size_t)PB * (4 * H + 1)) * sizeof(float); }

template <typename T>
bool fits_t(int B, int H, bool training, int *grid) {
    int dev = 0, sms = 0, optin = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const int g = ((H + PU - 1) / PU) * ((B + PB - 1) / PB);
    auto check = [&](auto kern, size_t smem) {
        if (smem > (size_t)optin || !raise_smem_limit(kern, smem)) return false;
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem) != cudaSuccess) return false;
        return per_sm * sms >= g;
    };
    if (!check(persistent_forward_kernel<T>, fwd_smem(H))) { cudaGetLastError(); return false; }
    if (training && !check(persistent_backward_kernel<T>, bwd_smem(H))) { cudaGetLastError(); return false; }
    *grid = g;
    return true;
}

}  // namespace

int persistent_batch_tiles(size_t B) { return (int)((B + PB - 1) / PB); }

bool persistent_fits(int dtype, size_t B, size_t H, bool training, int *grid) {
    if (const char *env = std::getenv("FLSTM_SIMT_PERSISTENT"))
        if (env[0] == '0') return false;
    switch (dtype) {
        case FLSTM_DTYPE_F32: return fits_t<float>((int)B, (int)H, training, grid);
        case FLSTM_DTYPE_F16: return fits_t<__half>((int)B, (int)H, training, grid);
        case FLSTM_DTYPE_BF16: return fits_t<__nv_bfloat16>((int)B, (int)H, training, grid);
    }
    return false;
}

int persistent_forward(int dtype, int grid, PersistentFwdParams p, cudaStream_t s) {
    const size_t smem = fwd_smem(p.H);
    switch (dtype) {
        case FLSTM_DTYPE_F32: return coop_launch(persistent_forward_kernel<float>, grid, smem, s, &p, "persistent fp32 forward");
        case FLSTM_DTYPE_F16: return coop_launch(persistent_forward_kernel<__half>, grid, smem, s, &p, "persistent fp32 forward");
        case FLSTM_DTYPE_BF16: return coop_launch(persistent_forward_kernel<__nv_bfloat16>, grid, smem, s, &p, "persistent fp32 forward");
    }
    return set_error(FLSTM_ERR_INVALID, "persistent_forward: bad dtype %d", dtype);
}

int persistent_backward(int dtype, int grid, PersistentBwdParams p, cudaStream_t s) {
    const size_t smem = bwd_smem(p.H);
    switch (dtype) {
        case FLSTM_DTYPE_F32: return coop_launch(persistent_backward_kernel<float>, grid, smem, s, &p, "persistent fp32 BPTT");
        case FLSTM_DTYPE_F16: return coop_launch(persistent_backward_kernel<__half>, grid, smem, s, &p, "persistent fp32 BPTT");
        case FLSTM_DTYPE_BF16: return coop_launch(persistent_backward_kernel<__nv_bfloat16>, grid, smem, s, &p, "persistent fp32 BPTT");
    }
    return set_error(FLSTM_ERR_INVALID, "persistent_backward: bad dtype %d", dtype);
}

}  // namespace simt
}  // namespace flstm_b200
