// Wide-batch recurrent path: one tcgen05 GEMM launch per time step instead of a persistent kernel.
//
// The persistent kernels (tc_lstm_fwd.cu, tc_lstm_bwd.cu) give every CTA a 64-row slice of W_hh and
// make it read ALL of h_{t-1} (dG_t) every step.  That is the right trade while the batch is a few
// tiles; from a few hundred sequences on, re-reading the activations by every row-slice CTA costs
// more L2 bandwidth than the step barrier saves.  Here a step is a plain output-tiled GEMM
//     forward :  S[B,4H]  = h_{t-1}[B,H]  W_hh^T         (+ fused gate / cell / hidden update epilogue)
//     backward:  dh[B,H]  = dG_t[B,4H]    W_hh           (split along K = 4H into fp32 partial sums)
// with the batch on the UMMA M axis (128 sequences per tile), so each operand byte is read once
// per 128 or 256 output columns.  With the tile-interleaved gate order, 64 consecutive columns of S
// are the four gates of 16 hidden units: the thread that owns a batch row (one TMEM lane) holds
// everything the pointwise update of those units needs, and the epilogue goes straight from TMEM
// registers to global memory.  The backward pointwise step (dG_t from dh, dc and the gate cache)
// is a small HBM-bound SIMT kernel between two GEMM launches.
//
//   warp 0   TMA producer, warp 1 UMMA issuer, warps 2-5 epilogue (same roles as tc_gemm.cu)
//
// Replaces, for large batches, the same reference code as the persistent kernels: the per-step
// recurrent launches of flashlstm_v2/src/lstm_forward.cu:744-830 and lstm_backward.cu:806-1110.
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "tc_common.cuh"
#include "tc_kernels.h"

namespace flstm_b200 {
namespace tc {

namespace {

constexpr int BM = 128, BK = 64;
constexpr int kStepThreads = 192;

template <int BN>
struct StepShape {
    static constexpr int kStages = (BN == 256) ? 4 : 6;
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

enum Epilogue { EPI_LSTM_FWD = 0, EPI_F32_PARTS = 1 };

struct StepArgs {
    int M, N, K;       // M = batch, N = output columns, K = contraction length
    int a_z;           // time coordinate of the A operand in its (steps, batch, width) tensor map
    int splits;        // K splits (EPI_F32_PARTS): split s writes parts + s*M*N
    uint32_t idesc;
    unsigned int *err;
    // EPI_F32_PARTS
    float *parts;
    // EPI_LSTM_FWD: all pointers already at time step t
    void *gates_t;        // 16-bit (B,4H): projection in, activated gates out
    const float *c_prev;  // fp32 (B,H)
    float *c_out;         // fp32 (B,H)
    void *h_out;          // 16-bit (B,H)
    void *y_out;          // 16-bit (B,H) or null
    int H;
    int store_gates;
};

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    if (BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w));
    return __half22float2(*reinterpret_cast<const __half2 *>(&w));
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    if (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

// The LSTM cell update of 16 hidden units of one sequence.  acc[0..63]: recurrent sums, gate-major
// (i,f,g,o) x 16 units, exactly the 64 columns of one unit group.
template <bool BF16>
__device__ __forceinline__ void lstm_cell_16(const uint32_t (&acc)[64], const StepArgs &a, int b, int group) {
    const size_t G = (size_t)4 * a.H;
    uint16_t *grow = static_cast<uint16_t *>(a.gates_t) + (size_t)b * G + (size_t)group * 64;
    const size_t sidx = (size_t)b * a.H + (size_t)group * 16;
#pragma unroll
    for (int ub = 0; ub < 2; ++ub) {  // 8 units at a time
        uint4 pv[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) pv[g] = *reinterpret_cast<const uint4 *>(grow + g * 16 + ub * 8);
        const float4 c0 = *reinterpret_cast<const float4 *>(a.c_prev + sidx + ub * 8);
        const float4 c1 = *reinterpret_cast<const float4 *>(a.c_prev + sidx + ub * 8 + 4);
        const float cp[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        float cn[8], hn[8], act[4][8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint32_t w[4] = {pv[g].x, pv[g].y, pv[g].z, pv[g].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 pp = unpack2<BF16>(w[k]);
                act[g][2 * k] = __uint_as_float(acc[g * 16 + ub * 8 + 2 * k]) + pp.x;
                act[g][2 * k + 1] = __uint_as_float(acc[g * 16 + ub * 8 + 2 * k + 1]) + pp.y;
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float gi = sigmoid_fast(act[0][u]), gf = sigmoid_fast(act[1][u]);
            const float gg = tanh_fast(act[2][u]), go = sigmoid_fast(act[3][u]);
            const float c = fmaf(gf, cp[u], gi * gg);
            cn[u] = c;
            hn[u] = go * tanh_fast(c);
            act[0][u] = gi; act[1][u] = gf; act[2][u] = gg; act[3][u] = go;
        }
        const uint4 hv = make_uint4(pack2<BF16>(hn[0], hn[1]), pack2<BF16>(hn[2], hn[3]), pack2<BF16>(hn[4], hn[5]),
                                    pack2<BF16>(hn[6], hn[7]));
        *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(a.h_out) + sidx + ub * 8) = hv;
        if (a.y_out) *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(a.y_out) + sidx + ub * 8) = hv;
        *reinterpret_cast<float4 *>(a.c_out + sidx + ub * 8) = make_float4(cn[0], cn[1], cn[2], cn[3]);
        *reinterpret_cast<float4 *>(a.c_out + sidx + ub * 8 + 4) = make_float4(cn[4], cn[5], cn[6], cn[7]);
        if (a.store_gates) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
                *reinterpret_cast<uint4 *>(grow + g * 16 + ub * 8) =
                    make_uint4(pack2<BF16>(act[g][0], act[g][1]), pack2<BF16>(act[g][2], act[g][3]),
                               pack2<BF16>(act[g][4], act[g][5]), pack2<BF16>(act[g][6], act[g][7]));
        }
    }
}

// A: (steps, M, K) K-major through a 3-D map with 128 x 64 boxes.  B: K-major (N, K) with BN x 64 boxes
// (forward: W_hh rows = gate columns) or MN-major, stored (K, N), 64 x 64 boxes (backward: W_hh as stored).
template <int BN, int EPI, bool B_MN, bool BF16>
__global__ void __launch_bounds__(kStepThreads, 1)
step_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const StepArgs a) {
    using S = StepShape<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + S::kStages * S::kStageBytes);
    uint64_t *full = bars, *empty = bars + S::kStages;
    uint64_t *tfull = bars + 2 * S::kStages, *tempty = tfull + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + 2);
    volatile uint32_t *abort_w = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < S::kStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], 4);
        }
        *abort_w = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, S::kTmemCols);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_m = (a.M + BM - 1) / BM, num_n = a.N / BN;
    const int kblocks = a.K / BK, kper = kblocks / a.splits;
    const int tiles = num_m * num_n * a.splits;
    // tile -> (split, m, n): n fastest, so CTAs that run together share the A tile in L2

    if (warp == 0) {
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
                const int ks = tile / (num_m * num_n), mn = tile % (num_m * num_n);
                const int m0 = (mn / num_n) * BM, n0 = (mn % num_n) * BN;
                bool ok = true;
                for (int kb = ks * kper; kb < (ks + 1) * kper && ok; ++kb) {
                    ok = mbar_wait(&empty[stage], phase ^ 1, abort_w);
                    if (!ok) break;
                    uint8_t *sa = smem + stage * S::kStageBytes, *sb = sa + S::kABytes;
                    mbar_expect_tx(&full[stage], S::kStageBytes);
                    tma_load_3d(sa, &tm_a, kb * BK, m0, a.a_z, &full[stage]);
                    if (!B_MN) {
                        tma_load_2d(sb, &tm_b, kb * BK, n0, &full[stage]);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tm_b, n0 + j * 64, kb * BK, &full[stage]);
                    }
                    if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                const uint32_t bphase = (it >> 1) & 1;
                if (!mbar_wait(&tempty[buf], bphase ^ 1, abort_w)) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                bool ok = true;
                for (int kb = 0; kb < kper; ++kb) {
                    ok = mbar_wait(&full[stage], phase, abort_w);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t a_base = smem_u32(smem + stage * S::kStageBytes), b_base = a_base + S::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t da = umma_desc_kmajor_sw128(a_base + k * 32);
                        const uint64_t db = B_MN ? umma_desc_mnmajor_sw128(b_base + k * 2048, 8192)
                                                 : umma_desc_kmajor_sw128(b_base + k * 32);
                        umma_f16(d_tmem, da, db, a.idesc, (kb | k) != 0);
                    }
                    umma_commit(&empty[stage]);
                    if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&tfull[buf]);
            }
        }
    } else {
        const int q = warp & 3;  // TMEM lane quadrant this warp may access
        int it = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            const uint32_t bphase = (it >> 1) & 1;
            const int ks = tile / (num_m * num_n), mn = tile % (num_m * num_n);
            const int m0 = (mn / num_n) * BM, n0 = (mn % num_n) * BN;
            if (!mbar_wait(&tfull[buf], bphase, abort_w)) break;
            tcgen05_fence_after();
            const int row = m0 + q * 32 + lane;  // sequence index
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            if (EPI == EPI_LSTM_FWD) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 64) {
                    uint32_t acc[64];
                    tmem_ld_32x32b_x32(t_row + c, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
                    tmem_ld_32x32b_x32(t_row + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
                    tmem_ld_wait();
                    if (row < a.M) lstm_cell_16<BF16>(acc, a, row, (n0 + c) >> 6);
                }
            } else {
                float *dst = a.parts + ((size_t)ks * a.M + row) * a.N + n0;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t acc[32];
                    tmem_ld_32x32b_x32(t_row + c, acc);
                    tmem_ld_wait();
                    if (row < a.M) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            reinterpret_cast<float4 *>(dst + c)[i] =
                                make_float4(__uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]),
                                            __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[buf]);
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, S::kTmemCols);
    if (threadIdx.x == 0 && *abort_w) atomicExch(a.err, 1u);
}

// Pointwise backward of one time step for 8 hidden units of one sequence per thread:
//   dh = dy_t + sum of the fp32 partial products dG_{t+1} W_hh;  dc, dG_t as in the persistent BPTT kernel.
template <bool BF16>
__global__ void __launch_bounds__(256)
step_bwd_pointwise_kernel(const uint16_t *__restrict__ gates_t, const float *__restrict__ c_t,
                          const float *__restrict__ c_prev, const uint16_t *__restrict__ dy_t,
                          const float *__restrict__ parts, int nparts, float *__restrict__ dc,
                          uint16_t *__restrict__ dg_t, int B, int H) {
    const int octets = H >> 3;
    const size_t total = (size_t)B * octets, slab = (size_t)B * H;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int b = (int)(i / octets), U0 = (int)(i % octets) * 8;
        const size_t sidx = (size_t)b * H + U0;
        // columns of the four gates of units U0..U0+7 in the tile-interleaved order
        const size_t gcol = (size_t)b * 4 * H + (size_t)(U0 >> 4) * 64 + (U0 & 15);
        float gate[4][8], ct[8], cp[8], dh[8], dcv[8];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint4 v = *reinterpret_cast<const uint4 *>(gates_t + gcol + g * 16);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = unpack2<BF16>(w[k]);
                gate[g][2 * k] = f.x;
                gate[g][2 * k + 1] = f.y;
            }
        }
        {
            const uint4 v = *reinterpret_cast<const uint4 *>(dy_t + sidx);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = unpack2<BF16>(w[k]);
                dh[2 * k] = f.x;
                dh[2 * k + 1] = f.y;
            }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float4 a = *reinterpret_cast<const float4 *>(c_t + sidx + 4 * h);
            const float4 p = *reinterpret_cast<const float4 *>(c_prev + sidx + 4 * h);
            const float4 d = *reinterpret_cast<const float4 *>(dc + sidx + 4 * h);
            ct[4 * h] = a.x; ct[4 * h + 1] = a.y; ct[4 * h + 2] = a.z; ct[4 * h + 3] = a.w;
            cp[4 * h] = p.x; cp[4 * h + 1] = p.y; cp[4 * h + 2] = p.z; cp[4 * h + 3] = p.w;
            dcv[4 * h] = d.x; dcv[4 * h + 1] = d.y; dcv[4 * h + 2] = d.z; dcv[4 * h + 3] = d.w;
        }
        {
            float rec[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int s = 0; s < nparts; ++s) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float4 r = *reinterpret_cast<const float4 *>(parts + (size_t)s * slab + sidx + 4 * h);
                    rec[4 * h] += r.x; rec[4 * h + 1] += r.y; rec[4 * h + 2] += r.z; rec[4 * h + 3] += r.w;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) dh[u] += rec[u];
        }
        float da[4][8], dcp[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float gi = gate[0][u], gf = gate[1][u], gg = gate[2][u], go = gate[3][u];
            const float tc = tanh_fast(ct[u]);
            const float d_o = dh[u] * tc;
            const float dcu = dcv[u] + dh[u] * go * (1.f - tc * tc);
            da[0][u] = dcu * gg * gi * (1.f - gi);
            da[1][u] = dcu * cp[u] * gf * (1.f - gf);
            da[2][u] = dcu * gi * (1.f - gg * gg);
            da[3][u] = d_o * go * (1.f - go);
            dcp[u] = dcu * gf;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h)
            *reinterpret_cast<float4 *>(dc + sidx + 4 * h) = make_float4(dcp[4 * h], dcp[4 * h + 1], dcp[4 * h + 2], dcp[4 * h + 3]);
#pragma unroll
        for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4 *>(dg_t + gcol + g * 16) =
                make_uint4(pack2<BF16>(da[g][0], da[g][1]), pack2<BF16>(da[g][2], da[g][3]),
                           pack2<BF16>(da[g][4], da[g][5]), pack2<BF16>(da[g][6], da[g][7]));
    }
}

// out = sum of the fp32 partial buffers (the gradient w.r.t. h0 after the last backward step)
__global__ void sum_parts_kernel(const float *__restrict__ parts, int nparts, size_t n, float *__restrict__ out) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < nparts; ++s) v += parts[(size_t)s * n + i];
        out[i] = v;
    }
}

template <int BN, int EPI, bool B_MN, bool BF16>
int launch_step(const CUtensorMap &ta, const CUtensorMap &tb, const StepArgs &a, int sms, cudaStream_t s) {
    using S = StepShape<BN>;
    auto kern = step_kernel<BN, EPI, B_MN, BF16>;
    static bool configured = false;  // per instantiation
    if (!configured) {
        FLSTM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kSmemBytes));
        configured = true;
    }
    const int tiles = ((a.M + BM - 1) / BM) * (a.N / BN) * a.splits;
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, kStepThreads, S::kSmemBytes, s>>>(ta, tb, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "step kernel launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

// Cost model for the tile width: rounds of the persistent tile loop times the shared-memory-bound
// cost of one K step (a 128 x BN x 16 UMMA reads 4 KB + BN*32 B of operands).
int pick_bn(int m_tiles, int N, int splits, int sms) {
    if (N % 256) return 128;
    const int t128 = m_tiles * (N / 128) * splits, t256 = m_tiles * (N / 256) * splits;
    const int cost128 = ((t128 + sms - 1) / sms) * 2, cost256 = ((t256 + sms - 1) / sms) * 3;
    return cost256 < cost128 ? 256 : 128;
}

}  // namespace

int plan_step(int B, int H, int sms, StepPlan *plan) {
    *plan = StepPlan{};
    if (H % 64 != 0 || H < 64) return set_error(FLSTM_ERR_UNSUPPORTED, "hidden size must be a multiple of 64");
    int min_batch = 256;
    if (const char *env = std::getenv("FLSTM_STEP_MIN_BATCH")) min_batch = std::atoi(env);
    plan->use = min_batch > 0 && B >= min_batch && H % 128 == 0;  // the backward tiles are 128 or 256 units wide
    const int m_tiles = (B + BM - 1) / BM;
    plan->bn_fwd = pick_bn(m_tiles, 4 * H, 1, sms);
    // backward: K = 4H is long and N = H short; split K until the tiles fill the machine
    int splits = 1;
    while (splits < 8 && m_tiles * (H / 128) * splits * 2 <= sms && ((4 * H / BK) % (splits * 2)) == 0) splits *= 2;
    plan->splits = splits;
    plan->bn_bwd = pick_bn(m_tiles, H, splits, sms);
    return FLSTM_OK;
}

int lstm_step_forward(int dtype, const StepPlan &plan, const CUtensorMap &tm_hs, const CUtensorMap &tm_w,
                      const StepFwdParams &p, int sms, cudaStream_t s) {
    const bool bf16 = dtype == FLSTM_DTYPE_BF16;
    StepArgs a{};
    a.M = p.B;
    a.N = 4 * p.H;
    a.K = p.H;
    a.a_z = p.t;
    a.splits = 1;
    a.idesc = umma_idesc_f16(BM, plan.bn_fwd, bf16 ? 1 : 0, 0, 0);
    a.err = p.err;
    a.gates_t = p.gates_t;
    a.c_prev = p.c_prev;
    a.c_out = p.c_out;
    a.h_out = p.h_out;
    a.y_out = p.y_out;
    a.H = p.H;
    a.store_gates = p.store_gates;
    if (plan.bn_fwd == 256)
        return bf16 ? launch_step<256, EPI_LSTM_FWD, false, true>(tm_hs, tm_w, a, sms, s)
                    : launch_step<256, EPI_LSTM_FWD, false, false>(tm_hs, tm_w, a, sms, s);
    return bf16 ? launch_step<128, EPI_LSTM_FWD, false, true>(tm_hs, tm_w, a, sms, s)
                : launch_step<128, EPI_LSTM_FWD, false, false>(tm_hs, tm_w, a, sms, s);
}

int lstm_step_backward_gemm(int dtype, const StepPlan &plan, const CUtensorMap &tm_dg, const CUtensorMap &tm_w64, int t,
                            int B, int H, float *parts, unsigned int *err, int sms, cudaStream_t s) {
    const bool bf16 = dtype == FLSTM_DTYPE_BF16;
    StepArgs a{};
    a.M = B;
    a.N = H;
    a.K = 4 * H;
    a.a_z = t;
    a.splits = plan.splits;
    a.idesc = umma_idesc_f16(BM, plan.bn_bwd, bf16 ? 1 : 0, 0, 1);
    a.err = err;
    a.parts = parts;
    a.H = H;
    if (plan.bn_bwd == 256) return launch_step<256, EPI_F32_PARTS, true, false>(tm_dg, tm_w64, a, sms, s);
    return launch_step<128, EPI_F32_PARTS, true, false>(tm_dg, tm_w64, a, sms, s);
}

int lstm_step_backward_pointwise(int dtype, const void *gates_t, const float *c_t, const float *c_prev, const void *dy_t,
                                 const float *parts, int nparts, float *dc, void *dg_t, int B, int H, cudaStream_t s) {
    const size_t total = (size_t)B * (H / 8);
    int grid = (int)((total + 255) / 256);
    if (grid > 148 * 8) grid = 148 * 8;
    if (dtype == FLSTM_DTYPE_BF16)
        step_bwd_pointwise_kernel<true><<<grid, 256, 0, s>>>(static_cast<const uint16_t *>(gates_t), c_t, c_prev,
                                                             static_cast<const uint16_t *>(dy_t), parts, nparts, dc,
                                                             static_cast<uint16_t *>(dg_t), B, H);
    else
        step_bwd_pointwise_kernel<false><<<grid, 256, 0, s>>>(static_cast<const uint16_t *>(gates_t), c_t, c_prev,
                                                              static_cast<const uint16_t *>(dy_t), parts, nparts, dc,
                                                              static_cast<uint16_t *>(dg_t), B, H);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "step pointwise launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

int sum_parts(const float *parts, int nparts, size_t n, float *out, cudaStream_t s) {
    int grid = (int)((n + 255) / 256);
    if (grid > 148 * 8) grid = 148 * 8;
    sum_parts_kernel<<<grid, 256, 0, s>>>(parts, nparts, n, out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "sum_parts launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

}  // namespace tc
}  // namespace flstm_b200
