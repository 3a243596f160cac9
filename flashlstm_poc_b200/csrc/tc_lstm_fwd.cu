// Persistent recurrent forward kernel: ONE launch runs all T time steps of one layer.
//
// Work split.  The 4H gate rows are stored tile-interleaved: row tile j (64 rows) holds the four
// gates i,f,g,o of hidden units [16j, 16j+16).  A CTA owns `rt` consecutive row tiles and a group
// of batch tiles (BT = 32 or 64 sequences each); its slice of W_hh stays in shared memory for the
// whole sequence when it fits (W_RESIDENT), otherwise it is streamed through the TMA ring from L2.
//
// Per step and (row tile, batch tile):
//   producer warp : TMA-loads the P_t tile (input projection + bias, 16-bit), waits on the grid
//                   barrier for h_{t-1}, then streams h_{t-1} (BT x 64 chunks) through the ring
//   MMA warp      : tcgen05.mma M=64 (gate rows) x N=BT (batch) x K=16, accumulating over K = H into TMEM
//   4 epilogue warps: tcgen05.ld -> + P_t -> sigmoid/tanh -> exchange through shared memory so that
//                   one thread sees i,f,g,o of its (unit, sequence) pair -> c_t (fp32), h_t (16-bit);
//                   the activated gates overwrite the P_t tile in shared memory and go back to the
//                   same place in global memory with one TMA store: that is the FP16/BF16 gate cache
// Steps are separated by a per-batch-group barrier in global memory (release add / acquire poll).
// Every wait is bounded; a timeout raises the error word and every CTA drains and returns.
//
// Replaces, per step, the reference's ScaleAndPackColumnsKernel + GemmTN + ForwardPointwiseKernel
// launches (flashlstm_v2/src/lstm_forward.cu:744-830) and v1's GEMM + lstm_pointwise_kernel pair
// (src/lstm.cu:1241-1337, src/kernels.cu:86-164).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "tc_common.cuh"
#include "tc_kernels.h"

namespace flstm_b200 {
namespace tc {

namespace {

constexpr int kFwdThreads = 192;  // 4 epilogue warps + producer warp + MMA warp
constexpr int kChunkBytesW = 64 * 64 * 2;

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int *p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Bounded poll of a monotonic counter written by other CTAs.
__device__ __forceinline__ bool wait_counter(const unsigned int *ctr, unsigned int target, unsigned int *err_word,
                                             volatile uint32_t *abort_w) {
    if (ld_acquire_gpu(ctr) >= target) return true;
    const unsigned long long t0 = global_timer_ns();
    uint32_t spins = 0;
    while (ld_acquire_gpu(ctr) < target) {
        if ((++spins & 63u) == 0) {
            if (*abort_w) return false;
            if (*reinterpret_cast<volatile unsigned int *>(err_word)) {
                *abort_w = 1;
                return false;
            }
            if (global_timer_ns() - t0 > kWaitLimitNs) {
                *abort_w = 1;
                atomicExch(err_word, 2u);
                return false;
            }
        }
    }
    return true;
}

template <bool BF16>
__device__ __forceinline__ float load16(const uint16_t *p) {
    if (BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(p));
    return __half2float(*reinterpret_cast<const __half *>(p));
}
template <bool BF16>
__device__ __forceinline__ uint16_t to16(float v) {
    if (BF16) {
        __nv_bfloat16 h = __float2bfloat16_rn(v);
        return *reinterpret_cast<uint16_t *>(&h);
    }
    __half h = __float2half_rn(v);
    return *reinterpret_cast<uint16_t *>(&h);
}

}  // namespace

struct FwdSmemLayout {
    int w_bytes, ring_stage_bytes, stages, p_bytes, ex_bytes, total;
};

__host__ __device__ inline FwdSmemLayout fwd_smem_layout(int BT, int H, int rt, bool resident, int stages) {
    FwdSmemLayout l;
    const int kc = H / 64;
    l.w_bytes = resident ? rt * kc * kChunkBytesW : 0;
    l.ring_stage_bytes = BT * 128 + (resident ? 0 : kChunkBytesW);
    l.stages = stages;
    l.p_bytes = 2 * BT * 128;
    l.ex_bytes = 2 * 64 * (BT + 1) * 4;
    l.total = l.w_bytes + stages * l.ring_stage_bytes + l.p_bytes + l.ex_bytes + 1024 /*align*/ + 512 /*barriers*/;
    return l;
}

template <int BT, bool W_RESIDENT, bool BF16>
__global__ void __launch_bounds__(kFwdThreads, 1)
lstm_fwd_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_h,
                const __grid_constant__ CUtensorMap tm_g, FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int KC = p.H / 64;
    const FwdSmemLayout L = fwd_smem_layout(BT, p.H, p.rt, W_RESIDENT, p.stages);
    uint8_t *s_w = smem;                                   // resident W slice: rt*KC chunks of 8 KB
    uint8_t *s_ring = s_w + L.w_bytes;                     // stages x [h chunk | (W chunk)]
    uint8_t *s_p = s_ring + L.stages * L.ring_stage_bytes;  // 2 P/gate tiles, BT rows x 128 B, not swizzled
    float *s_ex = reinterpret_cast<float *>(s_p + L.p_bytes);  // 2 x [64][BT+1] activated gates (fp32)
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(s_ex) + L.ex_bytes);
    uint64_t *full = bars, *empty = bars + L.stages;
    uint64_t *tfull = empty + L.stages, *tempty = tfull + 2;
    uint64_t *pfull = tempty + 2, *pempty = pfull + 2;
    uint64_t *wbar = pempty + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(wbar + 1);
    volatile uint32_t *abort_w = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ng = blockIdx.x / p.cta_rows;        // batch group
    const int jr = blockIdx.x % p.cta_rows;        // first row tile = jr * rt
    unsigned int *counter = p.counters + ng;
    constexpr int kTmemCols = (2 * BT < 32) ? 32 : 2 * BT;

    if (threadIdx.x == 0) {
        for (int i = 0; i < L.stages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], 4);
            mbar_init(&pfull[i], 1);
            mbar_init(&pempty[i], 1);
        }
        mbar_init(wbar, 1);
        *abort_w = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_h);
        tma_prefetch_desc(&tm_g);
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int nt_count = p.nt;  // batch tiles per group
    const int items_per_step = p.rt * nt_count;

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        if (elect_one()) {
            bool ok = true;
            if (W_RESIDENT) {
                mbar_expect_tx(wbar, (uint32_t)(p.rt * KC * kChunkBytesW));
                for (int r = 0; r < p.rt; ++r)
                    for (int kc = 0; kc < KC; ++kc)
                        tma_load_2d(s_w + (r * KC + kc) * kChunkBytesW, &tm_w, kc * 64, (jr * p.rt + r) * 64, wbar);
            }
            int stage = 0;
            uint32_t phase = 0, wi = 0;
            for (int t = 0; t < p.T && ok; ++t) {
                bool first = true;
                for (int r = 0; r < p.rt && ok; ++r) {
                    const int j = jr * p.rt + r;
                    for (int n = 0; n < nt_count && ok; ++n, ++wi) {
                        const int b0 = (ng * nt_count + n) * BT;
                        const int pb = wi & 1;
                        ok = mbar_wait(&pempty[pb], ((wi >> 1) & 1) ^ 1, abort_w);
                        if (!ok) break;
                        mbar_expect_tx(&pfull[pb], BT * 128);
                        tma_load_3d(s_p + pb * BT * 128, &tm_g, j * 64, b0, t, &pfull[pb]);
                        if (first && t > 0) {
                            // h_{t-1} of this batch group is complete when every CTA of the group has
                            // arrived t times (4 epilogue warps each)
                            ok = wait_counter(counter, (unsigned)(p.cta_rows * 4) * (unsigned)t, p.err, abort_w);
                            if (!ok) break;
                            fence_proxy_async_all();
                        }
                        first = false;
                        for (int kc = 0; kc < KC; ++kc) {
                            ok = mbar_wait(&empty[stage], phase ^ 1, abort_w);
                            if (!ok) break;
                            uint8_t *sh = s_ring + stage * L.ring_stage_bytes;
                            mbar_expect_tx(&full[stage], (uint32_t)L.ring_stage_bytes);
                            tma_load_3d(sh, &tm_h, kc * 64, b0, t, &full[stage]);
                            if (!W_RESIDENT) tma_load_2d(sh + BT * 128, &tm_w, kc * 64, j * 64, &full[stage]);
                            if (++stage == L.stages) { stage = 0; phase ^= 1; }
                        }
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            bool ok = true;
            if (W_RESIDENT) ok = mbar_wait(wbar, 0, abort_w);
            int stage = 0;
            uint32_t phase = 0, wi = 0;
            const uint32_t total_items = (uint32_t)p.T * items_per_step;
            for (uint32_t it = 0; it < total_items && ok; ++it, ++wi) {
                const int r = (it % items_per_step) / nt_count;
                const int buf = wi & 1;
                ok = mbar_wait(&tempty[buf], ((wi >> 1) & 1) ^ 1, abort_w);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BT;
                for (int kc = 0; kc < KC; ++kc) {
                    ok = mbar_wait(&full[stage], phase, abort_w);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t h_base = smem_u32(s_ring + stage * L.ring_stage_bytes);
                    const uint32_t w_base = W_RESIDENT ? smem_u32(s_w + (r * KC + kc) * kChunkBytesW) : h_base + BT * 128;
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_f16(d_tmem, umma_desc_kmajor_sw128(w_base + k * 32), umma_desc_kmajor_sw128(h_base + k * 32),
                                 p.idesc, (kc | k) != 0);
                    umma_commit(&empty[stage]);
                    if (++stage == L.stages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&tfull[buf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (128 threads)
        const int tid = threadIdx.x;         // 0..127
        const int u = tid & 15, nb = tid >> 4;  // phase-B ownership: unit u, sequences nb + 8*i
        constexpr int PAIRS = BT / 8;
        float c_keep[PAIRS];
        const bool keep_c = items_per_step == 1;
        const size_t slab = (size_t)p.B * p.H;
        uint16_t *hs = static_cast<uint16_t *>(p.hs);
        uint16_t *y = static_cast<uint16_t *>(p.y);
        uint32_t wi = 0;
        bool ok = true;
        for (int t = 0; t < p.T && ok; ++t) {
            for (int r = 0; r < p.rt && ok; ++r) {
                const int j = jr * p.rt + r;
                for (int n = 0; n < nt_count && ok; ++n, ++wi) {
                    const int b0 = (ng * nt_count + n) * BT;
                    const int buf = wi & 1, pb = wi & 1;
                    // the previous item's gate-cache store must have read its tile before the tile is reused
                    if (tid == 0 && wi > 0) {
                        if (p.store_gates) tma_store_wait_read<0>();
                        mbar_arrive(&pempty[(wi - 1) & 1]);
                    }
                    // cell state entering this step (own writes of the previous step, or registers)
                    float c_prev[PAIRS];
#pragma unroll
                    for (int i = 0; i < PAIRS; ++i) {
                        const int b = b0 + nb + 8 * i;
                        if (keep_c && t > 0) c_prev[i] = c_keep[i];
                        else c_prev[i] = (b < p.B) ? p.cs[(size_t)t * slab + (size_t)b * p.H + j * 16 + u] : 0.f;
                    }
                    ok = mbar_wait(&tfull[buf], (wi >> 1) & 1, abort_w);
                    if (!ok) break;
                    tcgen05_fence_after();
                    ok = mbar_wait(&pfull[pb], (wi >> 1) & 1, abort_w);
                    if (!ok) break;
                    uint16_t *ptile = reinterpret_cast<uint16_t *>(s_p + pb * BT * 128);
                    float *ex = s_ex + (wi & 1) * 64 * (BT + 1);
                    // phase A: lanes 0..15 of warp g hold gate g of units 0..15 for all BT sequences
#pragma unroll
                    for (int c0 = 0; c0 < BT; c0 += 32) {
                        uint32_t acc[32];
                        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BT + c0, acc);
                        tmem_ld_wait();
                        if (lane < 16) {
                            const int col = warp * 16 + lane;
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const int nn = c0 + i;
                                const float pre = __uint_as_float(acc[i]) + load16<BF16>(ptile + nn * 64 + col);
                                const float a = (warp == 2) ? tanh_fast(pre) : sigmoid_fast(pre);
                                ptile[nn * 64 + col] = to16<BF16>(a);
                                ex[col * (BT + 1) + nn] = a;
                            }
                        }
                    }
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tempty[buf]);
                    fence_proxy_async_smem();  // tile writes -> visible to the TMA store
                    named_barrier_sync(1, 128);
                    if (tid == 0 && p.store_gates) {
                        tma_store_3d(&tm_g, ptile, j * 64, b0, t);
                        tma_store_commit();
                    }
                    // phase B: one thread per (unit, sequence) pair
#pragma unroll
                    for (int i = 0; i < PAIRS; ++i) {
                        const int nn = nb + 8 * i, b = b0 + nn;
                        const float gi = ex[(0 * 16 + u) * (BT + 1) + nn], gf = ex[(1 * 16 + u) * (BT + 1) + nn];
                        const float gg = ex[(2 * 16 + u) * (BT + 1) + nn], go = ex[(3 * 16 + u) * (BT + 1) + nn];
                        const float c = fmaf(gf, c_prev[i], gi * gg);
                        const float h = go * tanh_fast(c);
                        c_keep[i] = c;
                        if (b < p.B) {
                            const size_t idx = (size_t)b * p.H + j * 16 + u;
                            p.cs[(size_t)(t + 1) * slab + idx] = c;
                            const uint16_t h16 = to16<BF16>(h);
                            hs[(size_t)(t + 1) * slab + idx] = h16;
                            if (y) y[(size_t)t * slab + idx] = h16;
                        }
                    }
                }
            }
            if (!ok) break;
            // publish h_t: generic-proxy stores -> visible to other CTAs' TMA loads
            fence_proxy_async_all();
            __threadfence();
            __syncwarp();
            if (lane == 0) red_release_gpu_add(counter, 1u);
        }
        if (tid == 0) tma_store_wait_all<0>();
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem_base, kTmemCols);
    if (threadIdx.x == 0 && *abort_w) atomicCAS(p.err, 0u, 1u);
}

// ------------------------------------------------------------------ host launcher
template <int BT, bool RES, bool BF16>
static int launch_fwd(const CUtensorMap &tw, const CUtensorMap &th, const CUtensorMap &tg, const FwdParams &p, int grid,
                      int smem_bytes, cudaStream_t s) {
    auto kern = lstm_fwd_kernel<BT, RES, BF16>;
    static int configured = 0;
    if (configured < smem_bytes) {
        FLSTM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        configured = smem_bytes;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kFwdThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs must be co-resident: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, th, tg, p);
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "recurrent forward launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

int plan_fwd(int B, int H, int sms, size_t smem_limit, FwdPlan *plan) {
    if (H % 64 != 0 || H < 64) return set_error(FLSTM_ERR_UNSUPPORTED, "hidden size must be a multiple of 64");
    const int R = H / 16;  // row tiles
    int rt = 1;
    while (R / rt > sms || R % rt) ++rt;
    const int cta_rows = R / rt;
    const int BT = (B >= 128) ? 64 : 32;
    const int tiles = (B + BT - 1) / BT;
    int ngroups = sms / cta_rows;
    if (ngroups > tiles) ngroups = tiles;
    if (ngroups < 1) ngroups = 1;
    const int nt = (tiles + ngroups - 1) / ngroups;
    ngroups = (tiles + nt - 1) / nt;
    // resident weights if the slice plus a useful ring fits
    bool resident = true;
    int stages = 8;
    FwdSmemLayout l = fwd_smem_layout(BT, H, rt, true, stages);
    while ((size_t)l.total > smem_limit && stages > 4) l = fwd_smem_layout(BT, H, rt, true, --stages);
    if ((size_t)l.total > smem_limit) {
        resident = false;
        stages = 12;
        l = fwd_smem_layout(BT, H, rt, false, stages);
        while ((size_t)l.total > smem_limit && stages > 2) l = fwd_smem_layout(BT, H, rt, false, --stages);
        if ((size_t)l.total > smem_limit) return set_error(FLSTM_ERR_UNSUPPORTED, "recurrent kernel does not fit shared memory");
    }
    plan->BT = BT;
    plan->rt = rt;
    plan->cta_rows = cta_rows;
    plan->ngroups = ngroups;
    plan->nt = nt;
    plan->stages = stages;
    plan->resident = resident;
    plan->smem_bytes = l.total;
    plan->grid = cta_rows * ngroups;
    return FLSTM_OK;
}

int lstm_forward_persistent(int dtype, const FwdPlan &plan, const CUtensorMap &tm_w, const CUtensorMap &tm_h,
                            const CUtensorMap &tm_g, FwdParams p, cudaStream_t s) {
    const bool bf16 = dtype == FLSTM_DTYPE_BF16;
    p.rt = plan.rt;
    p.cta_rows = plan.cta_rows;
    p.nt = plan.nt;
    p.stages = plan.stages;
    p.idesc = umma_idesc_f16(64, plan.BT, bf16 ? 1 : 0, 0, 0);
#define FLSTM_FWD_CASE(BT_, RES_)                                                                              \
    if (plan.BT == BT_ && plan.resident == RES_)                                                               \
        return bf16 ? launch_fwd<BT_, RES_, true>(tm_w, tm_h, tm_g, p, plan.grid, plan.smem_bytes, s)          \
                    : launch_fwd<BT_, RES_, false>(tm_w, tm_h, tm_g, p, plan.grid, plan.smem_bytes, s);
    FLSTM_FWD_CASE(32, true)
    FLSTM_FWD_CASE(32, false)
    FLSTM_FWD_CASE(64, true)
    FLSTM_FWD_CASE(64, false)
#undef FLSTM_FWD_CASE
    return set_error(FLSTM_ERR_UNSUPPORTED, "no recurrent forward kernel for this plan");
}

}  // namespace tc
}  // namespace flstm_b200
