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
#include <utility>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "tc_common.cuh"
#include "tc_kernels.h"
#include "tc_recurrent.cuh"

namespace flstm_b200 {
namespace tc {

namespace {

constexpr int BM = 128, BK = 64;
constexpr int kStepThreads = 192;

enum Epilogue { EPI_LSTM_FWD = 0, EPI_F32_PARTS = 1 };

// Staging tiles of one forward-epilogue warp (32 sequences x one group of 16 hidden units), all filled and
// drained by TMA: 2 x [32 x 128 B] projection in / gates out, 2 x [32 x 64 B] cell state in / out,
// [32 x 32 B] hidden state out.
constexpr int kEpiPBytes = 32 * 128, kEpiCBytes = 32 * 64, kEpiHBytes = 32 * 32;
constexpr int kEpiWarpBytes = 2 * kEpiPBytes + 2 * kEpiCBytes + kEpiHBytes;  // 13312, a multiple of 1024

// PAIR: a cluster of two CTAs works on a 256 x BN tile (tcgen05 cta_group::2): each CTA stages 128 rows of A and
// BN / 2 rows of B per K block and gets its own 128 accumulator rows, so the shared-memory traffic per FLOP -- what
// bounds the lone-CTA 128 x 128 tile at half of the tensor rate -- drops by a quarter (BN = 128) or a third (256).
template <int BN, int EPI, bool PAIR>
struct StepShape {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = (PAIR ? BN / 2 : BN) * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kEpiBytes = (EPI == EPI_LSTM_FWD) ? 4 * kEpiWarpBytes : 0;
    static constexpr int kStages = PAIR ? ((227 * 1024 - kEpiBytes - 2048) / kStageBytes > 8 ? 8 : (227 * 1024 - kEpiBytes - 2048) / kStageBytes)
                                        : ((EPI == EPI_LSTM_FWD) ? ((BN == 256) ? 3 : (BN == 128) ? 5 : 6) : ((BN == 256) ? 4 : 6));
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct StepArgs {
    int M, N, K;       // M = batch, N = output columns, K = contraction length
    int a_z;           // time coordinate of the A operand in its (steps, batch, width) tensor map
    int splits;        // K splits (EPI_F32_PARTS): split s writes parts + s*M*N
    uint32_t idesc;
    unsigned int *err;
    // EPI_F32_PARTS
    float *parts;
    // EPI_LSTM_FWD
    int t;             // time step: projection / gate cache and y at slot t, states read at slot t, written at t+1
    int has_y;         // also store h_t into the caller's y
    int store_gates;   // write the activated gates back (the gate cache)
    int early;         // fetch the first weight blocks ahead of the previous kernel's completion (FLSTM_PDL_EARLY=0: off)
};

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Kernels of the per-step chain start while the previous one drains (programmatic dependent launch); each
// waits for its predecessor with griddepcontrol.wait before touching what that one wrote.  FLSTM_PDL=0 turns it off.
// FLSTM_PDL_EARLY=0 keeps every global access behind that wait (no weight blocks / forward-pass operands fetched
// ahead of it).
bool pdl_early_enabled() {
    const char *env = std::getenv("FLSTM_PDL_EARLY");
    return !(env && env[0] == '0');
}
bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *env = std::getenv("FLSTM_PDL");
        on = (env && env[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// `cluster` > 1 launches the grid as clusters of that many CTAs (the CTA pairs of cta_group::2).
template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kern)(KArgs...), int grid, int block, size_t smem, cudaStream_t s, int cluster,
                           Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (cluster > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = cluster;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

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

// The LSTM cell update of 16 hidden units of one sequence from the staged tiles.  acc[0..63]: recurrent
// sums, gate-major (i,f,g,o) x 16 units (the 64 columns of one unit group).  r: row of the warp's
// 32-sequence block.  TMA wrote the tiles with the swizzle of their row size: 16-byte chunk j of row r sits at
// chunk j ^ (r & 7) (128 B rows), j ^ ((r >> 1) & 3) (64 B rows), j ^ ((r >> 2) & 1) (32 B rows).
// Outputs overwrite the inputs in place (gates over the projection, c_t over c_{t-1}).
template <bool BF16>
__device__ __forceinline__ void lstm_cell_16(const uint32_t (&acc)[64], uint8_t *sP, uint8_t *sC, uint8_t *sH, int r,
                                             int store_gates) {
    uint8_t *prow = sP + r * 128, *crow = sC + r * 64, *hrow = sH + r * 32;
    const int xp = r & 7, xc = (r >> 1) & 3, xh = (r >> 2) & 1;
#pragma unroll
    for (int ub = 0; ub < 2; ++ub) {  // 8 units at a time
        uint4 pv[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) pv[g] = *reinterpret_cast<const uint4 *>(prow + (((g * 2 + ub) ^ xp) << 4));
        const float4 c0 = *reinterpret_cast<const float4 *>(crow + (((ub * 2) ^ xc) << 4));
        const float4 c1 = *reinterpret_cast<const float4 *>(crow + (((ub * 2 + 1) ^ xc) << 4));
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
        *reinterpret_cast<uint4 *>(hrow + ((ub ^ xh) << 4)) =
            make_uint4(pack2<BF16>(hn[0], hn[1]), pack2<BF16>(hn[2], hn[3]), pack2<BF16>(hn[4], hn[5]), pack2<BF16>(hn[6], hn[7]));
        *reinterpret_cast<float4 *>(crow + (((ub * 2) ^ xc) << 4)) = make_float4(cn[0], cn[1], cn[2], cn[3]);
        *reinterpret_cast<float4 *>(crow + (((ub * 2 + 1) ^ xc) << 4)) = make_float4(cn[4], cn[5], cn[6], cn[7]);
        if (store_gates) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
                *reinterpret_cast<uint4 *>(prow + (((g * 2 + ub) ^ xp) << 4)) =
                    make_uint4(pack2<BF16>(act[g][0], act[g][1]), pack2<BF16>(act[g][2], act[g][3]),
                               pack2<BF16>(act[g][4], act[g][5]), pack2<BF16>(act[g][6], act[g][7]));
        }
    }
}

// A: (steps, M, K) K-major through a 3-D map with 128 x 64 boxes.  B: K-major (N, K) with BN x 64 boxes
// (forward: W_hh rows = gate columns) or MN-major, stored (K, N), 64 x 64 boxes (backward: W_hh as stored).
// Forward epilogue maps (make_tensor_map_3d_tile, 32-row boxes): tm_g gates (T,B,4H) 64 columns wide, tm_c cell
// states (T+1,B,H) fp32 16 wide, tm_h hidden states (T+1,B,H) 16 wide, tm_y the caller's y (T,B,H) 16 wide.
template <int BN, int EPI, bool B_MN, bool BF16, bool PAIR>
__global__ void __launch_bounds__(kStepThreads, 1)
step_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
            const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_c,
            const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_y, const StepArgs a) {
    using S = StepShape<BN, EPI, PAIR>;
    constexpr int BNB = PAIR ? BN / 2 : BN;  // rows of B this CTA stages per K block
    constexpr int BMT = PAIR ? 2 * BM : BM;  // rows of a tile (both CTAs of a pair)
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *epi = smem + S::kStages * S::kStageBytes;  // 1024-aligned: stage sizes are multiples of 1024
    uint64_t *bars = reinterpret_cast<uint64_t *>(epi + S::kEpiBytes);
    uint64_t *full = bars, *empty = bars + S::kStages;
    uint64_t *tfull = bars + 2 * S::kStages, *tempty = tfull + 2;
    uint64_t *ldbars = tempty + 2;  // 2 per epilogue warp
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(ldbars + 8);
    volatile uint32_t *abort_w = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = rank == 0;
    // tiles are dealt to CTAs (lone) or to CTA pairs
    const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    // The next kernel of the chain may be scheduled as soon as CTAs of this grid retire (it is never
    // co-resident with one: both need most of the SM's shared memory); it still waits for this whole grid.
    grid_launch_dependents();
    if (threadIdx.x == 0) {
        for (int i = 0; i < S::kStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], PAIR ? 8 : 4);  // PAIR: the leader's barrier takes both CTAs' epilogue warps
        }
        for (int i = 0; i < 8; ++i) mbar_init(&ldbars[i], 1);
        *abort_w = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (EPI == EPI_LSTM_FWD) {
            tma_prefetch_desc(&tm_g);
            tma_prefetch_desc(&tm_c);
            tma_prefetch_desc(&tm_h);
        }
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(tmem_slot, S::kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, S::kTmemCols);
            tmem_relinquish();
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // both CTAs' barriers and tensor memory exist before anything crosses the pair
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Launched with programmatic stream serialization: everything above overlapped the tail of the previous
    // step's kernel; its results (h, c, dG, partial sums) may be touched only from here on.  The producer warp
    // waits a little later: W_hh does not change along the chain, so it first fetches the weight blocks of its
    // first ring stages.
    if (warp != 0) grid_dependency_wait();

    const int num_m = (a.M + BMT - 1) / BMT, num_n = a.N / BN;
    const int kblocks = a.K / BK, kper = kblocks / a.splits;
    const int tiles = num_m * num_n * a.splits;
    // tile -> (split, m, n): n fastest, so CTAs that run together share the A tile in L2

    if (warp == 0) {
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            const uint32_t full0 = PAIR ? map_to_rank(smem_u32(full), 0) : 0u;  // the leader's "operands landed" barriers
            auto load_b_block = [&](uint8_t *sb, int kb, int n0, uint64_t *bar) {  // lone CTAs
                if (!B_MN) {
                    tma_load_2d(sb, &tm_b, kb * BK, n0, bar);
                } else {
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tm_b, n0 + j * 64, kb * BK, bar);
                }
            };
            // weight blocks of the first tile's first K blocks, ahead of the previous kernel's completion
            int npre = 0;
            if (a.early && worker < tiles) {
                const int ks = worker / (num_m * num_n), n0 = ((worker % (num_m * num_n)) % num_n) * BN + (int)rank * BNB;
                npre = kper < S::kStages ? kper : S::kStages;
                for (int b = 0; b < npre; ++b) {
                    uint8_t *sb = smem + b * S::kStageBytes + S::kABytes;
                    const int kb = ks * kper + b;
                    if (PAIR) {
                        const uint32_t bar = full0 + 8u * (uint32_t)b;
                        if (leader) mbar_expect_tx(&full[b], 2 * S::kStageBytes);
                        if (!B_MN) {
                            tma_load_2d_pair(sb, &tm_b, kb * BK, n0, bar);
                        } else {
#pragma unroll
                            for (int j = 0; j < BNB / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tm_b, n0 + j * 64, kb * BK, bar);
                        }
                    } else {
                        mbar_expect_tx(&full[b], S::kStageBytes);
                        load_b_block(sb, kb, n0, &full[b]);
                    }
                }
            }
            grid_dependency_wait();
            for (int tile = worker; tile < tiles; tile += workers) {
                const int ks = tile / (num_m * num_n), mn = tile % (num_m * num_n);
                const int m0 = (mn / num_n) * BMT + (int)rank * BM, n0 = (mn % num_n) * BN + (int)rank * BNB;
                bool ok = true;
                for (int kb = ks * kper; kb < (ks + 1) * kper && ok; ++kb) {
                    uint8_t *sa = smem + stage * S::kStageBytes, *sb = sa + S::kABytes;
                    if (tile == worker && kb - ks * kper < npre) {  // the weights of this stage are already on their way
                        if (PAIR) tma_load_3d_pair(sa, &tm_a, kb * BK, m0, a.a_z, full0 + 8u * (uint32_t)stage);
                        else tma_load_3d(sa, &tm_a, kb * BK, m0, a.a_z, &full[stage]);
                        if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                        continue;
                    }
                    ok = mbar_wait(&empty[stage], phase ^ 1, abort_w);
                    if (!ok) break;
                    if (PAIR) {
                        // each CTA fetches its own halves; the bytes of both are counted on the leader's barrier
                        const uint32_t bar = full0 + 8u * (uint32_t)stage;
                        if (leader) mbar_expect_tx(&full[stage], 2 * S::kStageBytes);
                        tma_load_3d_pair(sa, &tm_a, kb * BK, m0, a.a_z, bar);
                        if (!B_MN) {
                            tma_load_2d_pair(sb, &tm_b, kb * BK, n0, bar);
                        } else {
#pragma unroll
                            for (int j = 0; j < BNB / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tm_b, n0 + j * 64, kb * BK, bar);
                        }
                    } else {
                        mbar_expect_tx(&full[stage], S::kStageBytes);
                        tma_load_3d(sa, &tm_a, kb * BK, m0, a.a_z, &full[stage]);
                        load_b_block(sb, kb, n0, &full[stage]);
                    }
                    if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (leader && elect_one()) {  // in a pair only the leader issues UMMAs; they write both CTAs' accumulators
            const uint32_t empty_l = smem_u32(empty), tfull_l = smem_u32(tfull);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            for (int tile = worker; tile < tiles; tile += workers, ++it) {
                const int buf = it & 1;
                const uint32_t bphase = (it >> 1) & 1;
                if (!(PAIR ? mbar_wait_cluster(&tempty[buf], bphase ^ 1, abort_w) : mbar_wait(&tempty[buf], bphase ^ 1, abort_w))) break;
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
                        if (PAIR) umma_f16_pair(d_tmem, da, db, a.idesc, (kb | k) != 0);
                        else umma_f16(d_tmem, da, db, a.idesc, (kb | k) != 0);
                    }
                    if (PAIR) {  // the stage may be refilled in both CTAs once these UMMAs have read it
                        umma_commit_pair_both(empty_l + 8u * (uint32_t)stage);
                    } else {
                        umma_commit(&empty[stage]);
                    }
                    if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (PAIR) {
                    umma_commit_pair_both(tfull_l + 8u * (uint32_t)buf);
                } else {
                    umma_commit(&tfull[buf]);
                }
            }
        }
    } else {
        const int q = warp & 3;  // TMEM lane quadrant this warp may access
        const uint32_t tempty0 = PAIR ? map_to_rank(smem_u32(tempty), 0) : 0u;
        // this warp is done with accumulator `b`: tell the UMMA issuer (in a pair: the leader's barrier)
        auto release_accumulator = [&](int b) {
            if (PAIR) mbar_arrive_cluster_relaxed(tempty0 + 8u * (uint32_t)b);
            else mbar_arrive(&tempty[b]);
        };
        if (EPI == EPI_LSTM_FWD) {
            // Items = (tile, 64-column unit group) pairs in order.  Lane 0 keeps the loads of the next item in
            // flight while the warp works on the current one; outputs leave through TMA stores from the same tiles.
            constexpr int kGroups = BN / 64;
            uint8_t *wb = epi + q * kEpiWarpBytes;
            uint8_t *sH = wb + 2 * kEpiPBytes + 2 * kEpiCBytes;
            uint64_t *ldbar = ldbars + q * 2;
            const int my_tiles = (tiles > worker) ? (tiles - worker + workers - 1) / workers : 0;
            const int items = my_tiles * kGroups;
            auto item_coords = [&](int idx, int &row0, int &col0) {
                const int tl = worker + (idx / kGroups) * workers;
                row0 = (tl / num_n) * BMT + (int)rank * BM + q * 32;
                col0 = (tl % num_n) * BN + (idx % kGroups) * 64;
            };
            auto issue_loads = [&](int idx) {  // one lane
                int row0, col0;
                item_coords(idx, row0, col0);
                if (row0 >= a.M) return;  // nothing of this block is a real sequence
                const int buf = idx & 1;
                mbar_expect_tx(&ldbar[buf], kEpiPBytes + kEpiCBytes);
                tma_load_3d(wb + buf * kEpiPBytes, &tm_g, col0, row0, a.t, &ldbar[buf]);
                tma_load_3d(wb + 2 * kEpiPBytes + buf * kEpiCBytes, &tm_c, col0 >> 2, row0, a.t, &ldbar[buf]);
            };
            if (lane == 0 && items > 0) issue_loads(0);
            uint32_t ldphase = 0;  // bit b: parity of the next completion of ldbar[b]
            int item = 0, it = 0;
            bool ok = true;
            for (int tile = worker; tile < tiles && ok; tile += workers, ++it) {
                const int tbuf = it & 1;
                if (!mbar_wait(&tfull[tbuf], (it >> 1) & 1, abort_w)) break;
                tcgen05_fence_after();
                const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + tbuf * BN;
#pragma unroll 1
                for (int g = 0; g < kGroups; ++g, ++item) {
                    const int buf = item & 1;
                    int row0, col0;
                    item_coords(item, row0, col0);
                    if (lane == 0) {
                        tma_store_wait_read<0>();  // earlier stores have read the other buffers and sH
                        if (item + 1 < items) issue_loads(item + 1);
                    }
                    __syncwarp();
                    uint32_t acc[64];
                    tmem_ld_32x32b_x32(t_row + g * 64, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
                    tmem_ld_32x32b_x32(t_row + g * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
                    tmem_ld_wait();
                    if (g == kGroups - 1) {  // the accumulator is in registers: hand it back to the UMMA warp
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) release_accumulator(tbuf);
                    }
                    if (row0 >= a.M) continue;
                    ok = mbar_wait(&ldbar[buf], (ldphase >> buf) & 1u, abort_w);
                    if (!ok) break;
                    ldphase ^= 1u << buf;
                    uint8_t *sP = wb + buf * kEpiPBytes, *sC = wb + 2 * kEpiPBytes + buf * kEpiCBytes;
                    lstm_cell_16<BF16>(acc, sP, sC, sH, lane, a.store_gates);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (a.store_gates) tma_store_3d(&tm_g, sP, col0, row0, a.t);
                        tma_store_3d(&tm_c, sC, col0 >> 2, row0, a.t + 1);
                        tma_store_3d(&tm_h, sH, col0 >> 2, row0, a.t + 1);
                        if (a.has_y) tma_store_3d(&tm_y, sH, col0 >> 2, row0, a.t);
                        tma_store_commit();
                    }
                }
            }
            if (lane == 0) tma_store_wait_all<0>();
        } else {
            int it = 0;
            for (int tile = worker; tile < tiles; tile += workers, ++it) {
                const int buf = it & 1;
                const int ks = tile / (num_m * num_n), mn = tile % (num_m * num_n);
                const int m0 = (mn / num_n) * BMT + (int)rank * BM, n0 = (mn % num_n) * BN;
                if (!mbar_wait(&tfull[buf], (it >> 1) & 1, abort_w)) break;
                tcgen05_fence_after();
                const int row = m0 + q * 32 + lane;  // sequence index
                const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
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
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) release_accumulator(buf);
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) {
        cluster_sync_all();  // the peer's shared and tensor memory stay valid until the leader's last UMMA is consumed
        if (warp == 1) tmem_dealloc_pair(tmem_base, S::kTmemCols);
    } else if (warp == 1) {
        tmem_dealloc(tmem_base, S::kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_w) atomicExch(a.err, 1u);
}

// ------------------------------------------------------------------ all time steps in one launch
// The forward step GEMM as a persistent kernel: ONE cooperative launch runs the steps [t0, t0 + nsteps) of a layer.
// A kernel boundary per step costs more than the step's UMMAs (the per-step launches spend two thirds of their
// time on dependency resolution, pipeline fill and drain); here a CTA keeps its output tiles for the whole range,
// the steps are separated by a counter barrier in global memory (release add by every CTA once its h_t tiles
// are stored, acquire poll by the producers), and what does not depend on the recurrence is fetched ahead of
// the barrier: the W_hh blocks of the first ring stages and the projection / cell-state tiles of the epilogue.
//   warp 0   producer: per step, W_hh blocks for the free stages -> wait for h_{t-1} -> h blocks -> the rest
//   warp 1   UMMA issuer (as in step_kernel), warps 2-5 fused LSTM epilogue (as in step_kernel)
// Every wait is bounded; the four epilogue warps agree on failure at the named barrier that precedes the
// release (barrier.cta.red.or), so none of them is left behind.
struct WideFwdArgs {
    int M, N, K;       // batch, 4H, H
    int t0, nsteps;    // first absolute time step and number of steps of this launch
    uint32_t idesc;
    unsigned int *err;
    unsigned int *counter;        // step barrier, zeroed before the launch
    int has_y, store_gates;
    unsigned long long wait_ns;   // limit of every wait (0 = the 2 s default)
    unsigned int extra_arrivals;  // self-test of the timeout path: arrivals nobody makes
};

template <int BN, bool BF16, bool PAIR>
__global__ void __launch_bounds__(kStepThreads, 1)
wide_fwd_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ CUtensorMap tm_c,
                const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_y, const WideFwdArgs a) {
    using S = StepShape<BN, EPI_LSTM_FWD, PAIR>;
    constexpr int BNB = PAIR ? BN / 2 : BN;  // rows of W_hh this CTA stages per K block
    constexpr int BMT = PAIR ? 2 * BM : BM;  // sequences of a tile (both CTAs of a pair)
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *epi = smem + S::kStages * S::kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(epi + S::kEpiBytes);
    uint64_t *full = bars, *empty = bars + S::kStages;
    uint64_t *tfull = bars + 2 * S::kStages, *tempty = tfull + 2;
    uint64_t *ldbars = tempty + 2;  // 2 per epilogue warp
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(ldbars + 8);
    volatile uint32_t *abort_w = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = rank == 0;
    // tiles are dealt to CTAs (lone) or to CTA pairs
    const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const unsigned long long wait_ns = a.wait_ns ? a.wait_ns : kWaitLimitNs;
    if (threadIdx.x == 0) {
        for (int i = 0; i < S::kStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], PAIR ? 8 : 4);  // PAIR: the leader's barrier takes both CTAs' epilogue warps
        }
        for (int i = 0; i < 8; ++i) mbar_init(&ldbars[i], 1);
        *abort_w = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        tma_prefetch_desc(&tm_g);
        tma_prefetch_desc(&tm_c);
        tma_prefetch_desc(&tm_h);
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(tmem_slot, S::kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, S::kTmemCols);
            tmem_relinquish();
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // both CTAs' barriers and tensor memory exist before anything crosses the pair
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the barriers this CTA's operand copies complete: its own, or (PAIR) the leader's at the same offsets
    const uint32_t full_c = PAIR ? map_to_rank(smem_u32(full), 0) : smem_u32(full);
    const uint32_t stage_tx = (PAIR ? 2u : 1u) * (uint32_t)S::kStageBytes;
    auto load_a = [&](void *dst, int x, int y, int z, uint32_t bar) {
        if (PAIR) tma_load_3d_pair(dst, &tm_a, x, y, z, bar);
        else tma_load_3d_addr(dst, &tm_a, x, y, z, bar);
    };
    auto load_b = [&](void *dst, int x, int y, uint32_t bar) {
        if (PAIR) tma_load_2d_pair(dst, &tm_b, x, y, bar);
        else tma_load_2d_addr(dst, &tm_b, x, y, bar);
    };

    const int num_m = (a.M + BMT - 1) / BMT, num_n = a.N / BN;
    const int tiles = num_m * num_n, kblocks = a.K / BK;
    const int my_tiles = (tiles > worker) ? (tiles - worker + workers - 1) / workers : 0;
    // k-blocks a CTA streams per step, in order: tile after tile
    const int blocks_per_step = my_tiles * kblocks;

    if (warp == 0) {
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t issued = 0, parity = 0;  // the last copy started into every stage (drained on the way out)
            bool ok = true;
            auto coords = [&](int blk, int &m0, int &n0, int &kb) {
                const int tile = worker + (blk / kblocks) * workers;
                m0 = (tile / num_n) * BMT + (int)rank * BM;
                n0 = (tile % num_n) * BN + (int)rank * BNB;
                kb = blk % kblocks;
            };
            for (int tt = 0; tt < a.nsteps && ok; ++tt) {
                const int t = a.t0 + tt;
                // 1. W_hh blocks of as many k-blocks as the ring takes, before h_{t-1} is known to be complete
                const int npre = blocks_per_step < S::kStages ? blocks_per_step : S::kStages;
                int pre_stage[S::kStages];
                for (int b = 0; b < npre && ok; ++b) {
                    int m0, n0, kb;
                    coords(b, m0, n0, kb);
                    ok = mbar_wait(&empty[stage], phase ^ 1, abort_w, wait_ns);
                    if (!ok) break;
                    uint8_t *sb = smem + stage * S::kStageBytes + S::kABytes;
                    if (leader) mbar_expect_tx(&full[stage], stage_tx);
                    issued |= 1u << stage;
                    parity = (parity & ~(1u << stage)) | (phase << stage);
                    load_b(sb, kb * BK, n0, full_c + 8u * (uint32_t)stage);
                    pre_stage[b] = stage;
                    if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                // 2. h_{t-1} is complete when every CTA has arrived tt times in this launch
                if (tt > 0) {
                    ok = wait_counter(a.counter, gridDim.x * (unsigned)tt + a.extra_arrivals, a.err, abort_w, 7u, wait_ns);
                    if (!ok) break;
                    fence_proxy_async_global();
                }
                for (int b = 0; b < npre; ++b) {
                    int m0, n0, kb;
                    coords(b, m0, n0, kb);
                    load_a(smem + pre_stage[b] * S::kStageBytes, kb * BK, m0, t, full_c + 8u * (uint32_t)pre_stage[b]);
                }
                // 3. the rest of the step
                for (int b = npre; b < blocks_per_step && ok; ++b) {
                    int m0, n0, kb;
                    coords(b, m0, n0, kb);
                    ok = mbar_wait(&empty[stage], phase ^ 1, abort_w, wait_ns);
                    if (!ok) break;
                    uint8_t *sa = smem + stage * S::kStageBytes, *sb = sa + S::kABytes;
                    if (leader) mbar_expect_tx(&full[stage], stage_tx);
                    issued |= 1u << stage;
                    parity = (parity & ~(1u << stage)) | (phase << stage);
                    load_a(sa, kb * BK, m0, t, full_c + 8u * (uint32_t)stage);
                    load_b(sb, kb * BK, n0, full_c + 8u * (uint32_t)stage);
                    if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                }
            }
            // way out: every copy this thread started has landed before the CTA exits.  A stage whose W_hh block was
            // fetched ahead of a barrier that then failed never gets its h block: that wait runs into its limit.
            // (PAIR: the peer's copies complete the LEADER's barriers, which it cannot wait on; after a normal run the
            // UMMAs have consumed them all, after an abort the whole CTA lingers before it leaves)
            for (int i = 0; i < S::kStages && leader; ++i)
                if (issued >> i & 1u) mbar_drain(&full[i], parity >> i & 1u, ok ? wait_ns : kAbortDrainNs);
        }
    } else if (warp == 1) {
        if (leader && elect_one()) {
            const uint32_t empty_l = smem_u32(empty), tfull_l = smem_u32(tfull);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0, last_commit = -1;
            bool ok = true;
            for (int tt = 0; tt < a.nsteps && ok; ++tt) {
                for (int i = 0; i < my_tiles && ok; ++i, ++it) {
                    const int buf = it & 1;
                    ok = PAIR ? mbar_wait_cluster(&tempty[buf], ((it >> 1) & 1) ^ 1, abort_w, wait_ns)
                              : mbar_wait(&tempty[buf], ((it >> 1) & 1) ^ 1, abort_w, wait_ns);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * BN;
                    for (int kb = 0; kb < kblocks; ++kb) {
                        ok = mbar_wait(&full[stage], phase, abort_w, wait_ns);
                        if (!ok) break;
                        tcgen05_fence_after();
                        const uint32_t a_base = smem_u32(smem + stage * S::kStageBytes), b_base = a_base + S::kABytes;
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k) {
                            if (PAIR)
                                umma_f16_pair(d_tmem, umma_desc_kmajor_sw128(a_base + k * 32),
                                              umma_desc_kmajor_sw128(b_base + k * 32), a.idesc, (kb | k) != 0);
                            else
                                umma_f16(d_tmem, umma_desc_kmajor_sw128(a_base + k * 32),
                                         umma_desc_kmajor_sw128(b_base + k * 32), a.idesc, (kb | k) != 0);
                        }
                        if (PAIR) umma_commit_pair_both(empty_l + 8u * (uint32_t)stage);
                        else umma_commit(&empty[stage]);
                        if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                    }
                    if (!ok) break;
                    if (PAIR) umma_commit_pair_both(tfull_l + 8u * (uint32_t)buf);
                    else umma_commit(&tfull[buf]);
                    last_commit = it;
                }
            }
            if (last_commit >= 0) mbar_drain(&tfull[last_commit & 1], (uint32_t)(last_commit >> 1) & 1u, wait_ns);
        }
    } else {
        const int q = warp & 3;  // TMEM lane quadrant this warp may access
        constexpr int kGroups = BN / 64;
        uint8_t *wb = epi + q * kEpiWarpBytes;
        uint8_t *sH = wb + 2 * kEpiPBytes + 2 * kEpiCBytes;
        uint64_t *ldbar = ldbars + q * 2;
        const int items_per_step = my_tiles * kGroups;
        const uint32_t tempty_c = PAIR ? map_to_rank(smem_u32(tempty), 0) : 0u;
        auto item_coords = [&](int idx, int &row0, int &col0) {  // idx within a step
            const int tl = worker + (idx / kGroups) * workers;
            row0 = (tl / num_n) * BMT + (int)rank * BM + q * 32;
            col0 = (tl % num_n) * BN + (idx % kGroups) * 64;
        };
        // Items (tile, 64-column unit group) are numbered through the whole launch: item n stages its tiles in
        // buffer n & 1, and lane 0 keeps the loads of item n + 1 in flight while the warp works on item n.
        auto issue_loads = [&](int idx, int t, int buf) {  // one lane; idx = item within its step
            int row0, col0;
            item_coords(idx, row0, col0);
            if (row0 >= a.M) return;  // nothing of this block is a real sequence
            mbar_expect_tx(&ldbar[buf], kEpiPBytes + kEpiCBytes);
            tma_load_3d(wb + buf * kEpiPBytes, &tm_g, col0, row0, t, &ldbar[buf]);
            tma_load_3d(wb + 2 * kEpiPBytes + buf * kEpiCBytes, &tm_c, col0 >> 2, row0, t, &ldbar[buf]);
        };
        if (lane == 0 && items_per_step > 0) issue_loads(0, a.t0, 0);
        uint32_t ldphase = 0;  // bit b: parity of the next completion of ldbar[b]
        int it = 0, gitem = 0;
        bool ok = true;
        for (int tt = 0; tt < a.nsteps && ok; ++tt) {
            const int t = a.t0 + tt;
            bool good = true;  // warp-uniform: every wait of this step returned in time
            int item = 0;
            for (int i = 0; i < my_tiles; ++i, ++it) {
                const int tbuf = it & 1;
                if (good) good = __all_sync(0xffffffffu, mbar_wait(&tfull[tbuf], (it >> 1) & 1, abort_w, wait_ns));
                tcgen05_fence_after();
                const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + tbuf * BN;
#pragma unroll 1
                for (int g = 0; g < kGroups; ++g, ++item, ++gitem) {
                    const int buf = gitem & 1;
                    int row0, col0;
                    item_coords(item, row0, col0);
                    if (lane == 0 && good) {
                        tma_store_wait_read<0>();  // earlier stores have read the other buffer and sH
                        // the next item of THIS step; the first item of the next step waits for this step's own
                        // stores to complete (its cell-state tile is one of them), see the end of the step
                        if (item + 1 < items_per_step) issue_loads(item + 1, t, (gitem + 1) & 1);
                    }
                    __syncwarp();
                    uint32_t acc[64];
                    if (good) {
                        tmem_ld_32x32b_x32(t_row + g * 64, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
                        tmem_ld_32x32b_x32(t_row + g * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
                        tmem_ld_wait();
                    }
                    if (g == kGroups - 1) {  // the accumulator is in registers: hand it back to the UMMA warp
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (PAIR) mbar_arrive_cluster_relaxed(tempty_c + 8u * (uint32_t)tbuf);
                            else mbar_arrive(&tempty[tbuf]);
                        }
                    }
                    if (row0 >= a.M || !good) continue;
                    good = __all_sync(0xffffffffu, mbar_wait(&ldbar[buf], (ldphase >> buf) & 1u, abort_w, wait_ns));
                    if (!good) continue;
                    ldphase ^= 1u << buf;
                    uint8_t *sP = wb + buf * kEpiPBytes, *sC = wb + 2 * kEpiPBytes + buf * kEpiCBytes;
                    lstm_cell_16<BF16>(acc, sP, sC, sH, lane, a.store_gates);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (a.store_gates) tma_store_3d(&tm_g, sP, col0, row0, t);
                        tma_store_3d(&tm_c, sC, col0 >> 2, row0, t + 1);
                        tma_store_3d(&tm_h, sH, col0 >> 2, row0, t + 1);
                        if (a.has_y) tma_store_3d(&tm_y, sH, col0 >> 2, row0, t);
                        tma_store_commit();
                    }
                }
            }
            // h_t, c_t of this warp's rows are in global memory before the CTA arrives at the step barrier
            if (lane == 0) tma_store_wait_all<0>();
            __syncwarp();
            if (named_barrier_or(1, 128, !good)) {
                ok = false;
                break;
            }
            if (warp == 2 && lane == 0) {
                fence_proxy_async_global();  // the tiles were written through the async proxy
                red_release_gpu_add(a.counter, 1u);
            }
            if (lane == 0 && tt + 1 < a.nsteps && items_per_step > 0) issue_loads(0, t + 1, gitem & 1);
        }
        if (lane == 0) tma_store_wait_all<0>();
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) {
        // after an abort this CTA's own copies may still be landing on barriers it cannot see (the leader's)
        if (*abort_w) {
            const unsigned long long t0 = global_timer_ns();
            while (global_timer_ns() - t0 < kAbortDrainNs) {}
        }
        cluster_sync_all();  // the peer's shared and tensor memory stay valid until the leader's last UMMA is consumed
        if (warp == 1) tmem_dealloc_pair(tmem_base, S::kTmemCols);
    } else if (warp == 1) {
        tmem_dealloc(tmem_base, S::kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_w) atomicCAS(a.err, 0u, 1u);
}

// Pointwise backward of one time step for 4 hidden units of one sequence per thread:
//   dh = dy_t + sum of the fp32 partial products dG_{t+1} W_hh;  dc, dG_t as in the persistent BPTT kernel.
template <bool BF16>
__global__ void __launch_bounds__(256)
step_bwd_pointwise_kernel(const uint16_t *__restrict__ gates_t, const float *__restrict__ c_t,
                          const float *__restrict__ c_prev, const uint16_t *__restrict__ dy_t,
                          const float *__restrict__ parts, int nparts, float *__restrict__ dc,
                          uint16_t *__restrict__ dg_t, int B, int H, int early) {
    const int quads = H >> 2;
    const size_t total = (size_t)B * quads, slab = (size_t)B * H;
    // The split-K GEMM that follows may start its prologue and fetch its first weight blocks while this kernel
    // runs; it waits for this whole grid before it touches dG_t.
    if (early) grid_launch_dependents();
    else grid_dependency_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int b = (int)(i / quads), U0 = (int)(i % quads) * 4;
        const size_t sidx = (size_t)b * H + U0;
        // columns of the four gates of units U0..U0+3 in the tile-interleaved order
        const size_t gcol = (size_t)b * 4 * H + (size_t)(U0 >> 4) * 64 + (U0 & 15);
        float gate[4][4], dh[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint2 v = *reinterpret_cast<const uint2 *>(gates_t + gcol + g * 16);
            const float2 lo = unpack2<BF16>(v.x), hi = unpack2<BF16>(v.y);
            gate[g][0] = lo.x; gate[g][1] = lo.y; gate[g][2] = hi.x; gate[g][3] = hi.y;
        }
        {
            const uint2 v = *reinterpret_cast<const uint2 *>(dy_t + sidx);
            const float2 lo = unpack2<BF16>(v.x), hi = unpack2<BF16>(v.y);
            dh[0] = lo.x; dh[1] = lo.y; dh[2] = hi.x; dh[3] = hi.y;
        }
        const float4 ctv = *reinterpret_cast<const float4 *>(c_t + sidx);
        const float4 cpv = *reinterpret_cast<const float4 *>(c_prev + sidx);
        // everything above was written by the forward pass; the partial sums and the cell-gradient carry come from
        // the kernels right before this one in the chain
        if (early) grid_dependency_wait();
        const float4 dcv4 = *reinterpret_cast<const float4 *>(dc + sidx);
        const float ct[4] = {ctv.x, ctv.y, ctv.z, ctv.w}, cp[4] = {cpv.x, cpv.y, cpv.z, cpv.w};
        const float dcin[4] = {dcv4.x, dcv4.y, dcv4.z, dcv4.w};
        for (int s = 0; s < nparts; ++s) {
            const float4 r = *reinterpret_cast<const float4 *>(parts + (size_t)s * slab + sidx);
            dh[0] += r.x; dh[1] += r.y; dh[2] += r.z; dh[3] += r.w;
        }
        float da[4][4], dcp[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float gi = gate[0][u], gf = gate[1][u], gg = gate[2][u], go = gate[3][u];
            const float tc = tanh_fast(ct[u]);
            const float d_o = dh[u] * tc;
            const float dcu = dcin[u] + dh[u] * go * (1.f - tc * tc);
            da[0][u] = dcu * gg * gi * (1.f - gi);
            da[1][u] = dcu * cp[u] * gf * (1.f - gf);
            da[2][u] = dcu * gi * (1.f - gg * gg);
            da[3][u] = d_o * go * (1.f - go);
            dcp[u] = dcu * gf;
        }
        *reinterpret_cast<float4 *>(dc + sidx) = make_float4(dcp[0], dcp[1], dcp[2], dcp[3]);
#pragma unroll
        for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint2 *>(dg_t + gcol + g * 16) =
                make_uint2(pack2<BF16>(da[g][0], da[g][1]), pack2<BF16>(da[g][2], da[g][3]));
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

struct EpilogueMaps {
    const CUtensorMap *g, *c, *h, *y;
};

template <int BN, int EPI, bool B_MN, bool BF16, bool PAIR>
int launch_step_one(const CUtensorMap &ta, const CUtensorMap &tb, const EpilogueMaps &em, const StepArgs &a, int sms,
                    cudaStream_t s) {
    using S = StepShape<BN, EPI, PAIR>;
    auto kern = step_kernel<BN, EPI, B_MN, BF16, PAIR>;
    FLSTM_CUDA_TRY(ensure_smem_limit(kern, (size_t)S::kSmemBytes));
    const int rows = PAIR ? 2 * BM : BM;
    const int tiles = ((a.M + rows - 1) / rows) * (a.N / BN) * a.splits;
    const int workers = PAIR ? sms / 2 : sms;
    const int grid = (tiles < workers ? tiles : workers) * (PAIR ? 2 : 1);
    cudaError_t e = launch_chained(kern, grid, kStepThreads, S::kSmemBytes, s, PAIR ? 2 : 1, ta, tb, *em.g, *em.c, *em.h,
                                   *em.y, a);
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "step kernel launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

template <int BN, int EPI, bool B_MN, bool BF16>
int launch_step(bool pair, const CUtensorMap &ta, const CUtensorMap &tb, const EpilogueMaps &em, const StepArgs &a, int sms,
                cudaStream_t s) {
    return pair ? launch_step_one<BN, EPI, B_MN, BF16, true>(ta, tb, em, a, sms, s)
                : launch_step_one<BN, EPI, B_MN, BF16, false>(ta, tb, em, a, sms, s);
}

// Cost model for the tile width: rounds of the persistent tile loop times the shared-memory-bound
// cost of one K step (a 128 x BN x 16 UMMA reads 4 KB + BN*32 B of operands).  For CTA pairs (m_tiles counts
// 256-row tiles, sms / 2 workers) a K block of a 256 x 128 tile costs 3/8 and of a 256 x 256 tile 4/8 of what a
// lone 128 x 256 tile costs: each CTA stages 24 KB resp. 32 KB instead of 48 KB.
int pick_bn(int m_tiles, int N, int splits, int sms, bool pair = false, bool allow64 = false) {
    if (N % 256) return 128;
    const int workers = pair ? sms / 2 : sms;
    const int t128 = m_tiles * (N / 128) * splits, t256 = m_tiles * (N / 256) * splits;
    const int cost128 = ((t128 + workers - 1) / workers) * (pair ? 3 : 2), cost256 = ((t256 + workers - 1) / workers) * (pair ? 4 : 3);
    // 64-wide tiles (forward, lone CTAs) when 128-wide ones leave half of the SMs without a tile: a CTA then takes
    // in 128 + 64 operand rows per K block instead of 128 + 128 (cost 1.5 on the scale above)
    if (allow64 && !pair && 2 * t128 <= workers && cost128 <= cost256) return 64;
    return cost256 < cost128 ? 256 : 128;
}

// FLSTM_STEP_PAIR=1 turns the CTA-pair tiles on (off by default until measured)
bool step_pair_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *env = std::getenv("FLSTM_STEP_PAIR");
        on = (env && env[0] == '1') ? 1 : 0;
    }
    return on == 1;
}

}  // namespace

int plan_step(int B, int H, int sms, size_t smem_limit, StepPlan *plan) {
    *plan = StepPlan{};
    if (H % 64 != 0 || H < 64) return set_error(FLSTM_ERR_UNSUPPORTED, "hidden size must be a multiple of 64");
    // Measured crossover (H = 1024 / 2048 / 4096, B = 8..2048): the persistent kernels win exactly while every
    // CTA has a single batch tile per step; with two or more tiles per CTA the per-step GEMM launches win.
    // FLSTM_STEP_MIN_BATCH=n replaces the rule by "B >= n" (0: never).
    bool use;
    if (const char *env = std::getenv("FLSTM_STEP_MIN_BATCH")) {
        const int min_batch = std::atoi(env);
        use = min_batch > 0 && B >= min_batch;
    } else {
        FwdPlan fp{};
        use = plan_fwd(B, H, sms, smem_limit, &fp) != FLSTM_OK || fp.nt > 1;
    }
    plan->use = use && H % 128 == 0;  // the backward tiles are 128 or 256 units wide
    // from 256 sequences on a tile is 256 rows on a CTA pair (cta_group::2)
    plan->pair = B >= 2 * BM && sms >= 2 && step_pair_enabled();
    // FLSTM_STEP_BWD_PAIR=1: only the backward split-K GEMM on CTA pairs (the forward keeps its all-steps kernel)
    const char *bp = std::getenv("FLSTM_STEP_BWD_PAIR");
    plan->bwd_pair = plan->pair || (B >= 2 * BM && sms >= 2 && bp && bp[0] == '1');
    const int rows = plan->pair ? 2 * BM : BM;
    const int m_tiles = (B + rows - 1) / rows;
    plan->bn_fwd = pick_bn(m_tiles, 4 * H, 1, sms, plan->pair, true);
    // backward: K = 4H is long and N = H short; split K until the tiles fill the machine
    const int rows_b = plan->bwd_pair ? 2 * BM : BM, workers_b = plan->bwd_pair ? sms / 2 : sms;
    const int m_tiles_b = (B + rows_b - 1) / rows_b;
    int splits = 1;
    while (splits < 8 && m_tiles_b * (H / 128) * splits * 2 <= workers_b && ((4 * H / BK) % (splits * 2)) == 0) splits *= 2;
    plan->splits = splits;
    plan->bn_bwd = pick_bn(m_tiles_b, H, splits, sms, plan->bwd_pair);
    size_t need_fwd, need_bwd;
    if (plan->pair) {
        need_fwd = plan->bn_fwd == 256 ? StepShape<256, EPI_LSTM_FWD, true>::kSmemBytes : StepShape<128, EPI_LSTM_FWD, true>::kSmemBytes;
    } else {
        need_fwd = plan->bn_fwd == 256 ? StepShape<256, EPI_LSTM_FWD, false>::kSmemBytes
                   : plan->bn_fwd == 128 ? StepShape<128, EPI_LSTM_FWD, false>::kSmemBytes
                                         : StepShape<64, EPI_LSTM_FWD, false>::kSmemBytes;
    }
    if (plan->bwd_pair)
        need_bwd = plan->bn_bwd == 256 ? StepShape<256, EPI_F32_PARTS, true>::kSmemBytes : StepShape<128, EPI_F32_PARTS, true>::kSmemBytes;
    else
        need_bwd = plan->bn_bwd == 256 ? StepShape<256, EPI_F32_PARTS, false>::kSmemBytes : StepShape<128, EPI_F32_PARTS, false>::kSmemBytes;
    if (need_fwd > smem_limit || need_bwd > smem_limit) plan->use = false;  // the step kernels do not fit this device
    // forward: all steps of a range in one cooperative launch; FLSTM_WIDE_PERSIST=0 = one launch per step
    const char *wp = std::getenv("FLSTM_WIDE_PERSIST");
    plan->fwd_persistent = plan->use && !plan->pair && !(wp && wp[0] == '0');
    // ... on CTA pairs from 256 sequences on (the forward tile width is then chosen for pairs; FLSTM_WIDE_PAIR=0 keeps
    // lone CTAs).  Measured forward phases, lone -> pairs: config 3 33.5-35.0 -> 31.9-32.1 ms, config 5 26.7 -> 24.6 ms.
    const char *wpair = std::getenv("FLSTM_WIDE_PAIR");
    const char *wave = std::getenv("FLSTM_WAVE_CHUNK");  // the cross-layer wavefront launches per step (lone CTAs)
    plan->fwd_pair = plan->fwd_persistent && B >= 2 * BM && sms >= 2 && !(wpair && wpair[0] == '0') &&
                     !(wave && std::atoi(wave) > 0);
    if (plan->fwd_pair) {
        plan->bn_fwd = pick_bn((B + 2 * BM - 1) / (2 * BM), 4 * H, 1, sms, true);
        const size_t need = plan->bn_fwd == 256 ? StepShape<256, EPI_LSTM_FWD, true>::kSmemBytes : StepShape<128, EPI_LSTM_FWD, true>::kSmemBytes;
        if (need > smem_limit) {
            plan->fwd_pair = false;
            plan->bn_fwd = pick_bn(m_tiles, 4 * H, 1, sms, plan->pair, true);
        }
    }
    return FLSTM_OK;
}

int lstm_step_forward(int dtype, const StepPlan &plan, const StepFwdMaps &m, const StepFwdParams &p, int sms,
                      cudaStream_t s) {
    const bool bf16 = dtype == FLSTM_DTYPE_BF16;
    StepArgs a{};
    a.early = pdl_early_enabled() ? 1 : 0;
    a.M = p.B;
    a.N = 4 * p.H;
    a.K = p.H;
    a.a_z = p.t;
    a.splits = 1;
    a.idesc = umma_idesc_f16(plan.pair ? 2 * BM : BM, plan.bn_fwd, bf16 ? 1 : 0, 0, 0);
    a.err = p.err;
    a.t = p.t;
    a.has_y = m.y ? 1 : 0;
    a.store_gates = p.store_gates;
    const EpilogueMaps em{m.gates, m.cs, m.hs_out, m.y ? m.y : m.hs_out};
    if (plan.bn_fwd == 256)
        return bf16 ? launch_step<256, EPI_LSTM_FWD, false, true>(plan.pair, *m.hs, *m.w, em, a, sms, s)
                    : launch_step<256, EPI_LSTM_FWD, false, false>(plan.pair, *m.hs, *m.w, em, a, sms, s);
    if (plan.bn_fwd == 64)  // lone CTAs only (the planner never pairs 64-wide tiles)
        return bf16 ? launch_step_one<64, EPI_LSTM_FWD, false, true, false>(*m.hs, *m.w, em, a, sms, s)
                    : launch_step_one<64, EPI_LSTM_FWD, false, false, false>(*m.hs, *m.w, em, a, sms, s);
    return bf16 ? launch_step<128, EPI_LSTM_FWD, false, true>(plan.pair, *m.hs, *m.w, em, a, sms, s)
                : launch_step<128, EPI_LSTM_FWD, false, false>(plan.pair, *m.hs, *m.w, em, a, sms, s);
}

template <int BN, bool BF16, bool PAIR>
static int launch_wide_fwd(const StepFwdMaps &m, const WideFwdArgs &a, int sms, cudaStream_t s) {
    using S = StepShape<BN, EPI_LSTM_FWD, PAIR>;
    auto kern = wide_fwd_kernel<BN, BF16, PAIR>;
    FLSTM_CUDA_TRY(ensure_smem_limit(kern, (size_t)S::kSmemBytes));
    const int rows = PAIR ? 2 * BM : BM, workers = PAIR ? sms / 2 : sms;
    const int tiles = ((a.M + rows - 1) / rows) * (a.N / BN);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((tiles < workers ? tiles : workers) * (PAIR ? 2 : 1));
    cfg.blockDim = dim3(kStepThreads);
    cfg.dynamicSmemBytes = S::kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;  // the CTAs wait on one another: all of them must be resident
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;  // PAIR: clusters of two
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = PAIR ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, *m.hs, *m.w, *m.gates, *m.cs, *m.hs_out, m.y ? *m.y : *m.hs_out, a);
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "wide-batch forward launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

int lstm_wide_forward(int dtype, const StepPlan &plan, const StepFwdMaps &m, const WideFwdParams &p, int sms, cudaStream_t s) {
    const bool bf16 = dtype == FLSTM_DTYPE_BF16;
    WideFwdArgs a{};
    a.M = p.B;
    a.N = 4 * p.H;
    a.K = p.H;
    a.t0 = p.t0;
    a.nsteps = p.nsteps;
    a.idesc = umma_idesc_f16(plan.fwd_pair ? 2 * BM : BM, plan.bn_fwd, bf16 ? 1 : 0, 0, 0);
    a.err = p.err;
    a.counter = p.counter;
    a.has_y = m.y ? 1 : 0;
    a.store_gates = p.store_gates;
    a.wait_ns = p.wait_ns;
    a.extra_arrivals = p.extra_arrivals;
    if (plan.fwd_pair) {
        if (plan.bn_fwd == 256)
            return bf16 ? launch_wide_fwd<256, true, true>(m, a, sms, s) : launch_wide_fwd<256, false, true>(m, a, sms, s);
        return bf16 ? launch_wide_fwd<128, true, true>(m, a, sms, s) : launch_wide_fwd<128, false, true>(m, a, sms, s);
    }
    if (plan.bn_fwd == 256)
        return bf16 ? launch_wide_fwd<256, true, false>(m, a, sms, s) : launch_wide_fwd<256, false, false>(m, a, sms, s);
    if (plan.bn_fwd == 64)
        return bf16 ? launch_wide_fwd<64, true, false>(m, a, sms, s) : launch_wide_fwd<64, false, false>(m, a, sms, s);
    return bf16 ? launch_wide_fwd<128, true, false>(m, a, sms, s) : launch_wide_fwd<128, false, false>(m, a, sms, s);
}

int lstm_step_backward_gemm(int dtype, const StepPlan &plan, const CUtensorMap &tm_dg, const CUtensorMap &tm_w64, int t,
                            int B, int H, float *parts, unsigned int *err, int sms, cudaStream_t s) {
    const bool bf16 = dtype == FLSTM_DTYPE_BF16;
    StepArgs a{};
    a.early = pdl_early_enabled() ? 1 : 0;
    a.M = B;
    a.N = H;
    a.K = 4 * H;
    a.a_z = t;
    a.splits = plan.splits;
    a.idesc = umma_idesc_f16(plan.bwd_pair ? 2 * BM : BM, plan.bn_bwd, bf16 ? 1 : 0, 0, 1);
    a.err = err;
    a.parts = parts;
    const EpilogueMaps em{&tm_dg, &tm_dg, &tm_dg, &tm_dg};  // unused by this epilogue
    if (plan.bn_bwd == 256) return launch_step<256, EPI_F32_PARTS, true, false>(plan.bwd_pair, tm_dg, tm_w64, em, a, sms, s);
    return launch_step<128, EPI_F32_PARTS, true, false>(plan.bwd_pair, tm_dg, tm_w64, em, a, sms, s);
}

int lstm_step_backward_pointwise(int dtype, const void *gates_t, const float *c_t, const float *c_prev, const void *dy_t,
                                 const float *parts, int nparts, float *dc, void *dg_t, int B, int H, cudaStream_t s) {
    const size_t total = (size_t)B * (H / 4);
    int grid = (int)((total + 255) / 256);
    if (grid > 148 * 16) grid = 148 * 16;
    const uint16_t *g16 = static_cast<const uint16_t *>(gates_t), *dy16 = static_cast<const uint16_t *>(dy_t);
    uint16_t *dg16 = static_cast<uint16_t *>(dg_t);
    cudaError_t e = dtype == FLSTM_DTYPE_BF16
                        ? launch_chained(step_bwd_pointwise_kernel<true>, grid, 256, 0, s, 1, g16, c_t, c_prev, dy16, parts, nparts, dc, dg16, B, H, pdl_early_enabled() ? 1 : 0)
                        : launch_chained(step_bwd_pointwise_kernel<false>, grid, 256, 0, s, 1, g16, c_t, c_prev, dy16, parts, nparts, dc, dg16, B, H, pdl_early_enabled() ? 1 : 0);
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
