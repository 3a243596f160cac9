// Persistent recurrent forward kernel: ONE launch runs all T time steps of one layer.
//
// Work split.  The 4H gate rows are stored tile-interleaved: row tile j (64 rows) holds the four
// gates i,f,g,o of hidden units [16j, 16j+16).  A CTA owns `rt` consecutive row tiles and a group
// of batch tiles (BT = 32, 64 or 128 sequences each); its slice of W_hh stays in shared memory for the
// whole sequence when it fits (W_RESIDENT), otherwise it is streamed through the TMA ring from L2 (the chunks of a
// step's first ring stages ahead of the step barrier).  Neighbouring row-tile CTAs normally work as a CTA PAIR
// (template parameter PAIR, see the kernel): one UMMA of M = 128 over both, each CTA staging half of the h tile.
//
// Per step and (row tile, batch tile):
//   producer warp : TMA-loads the P_t tile (input projection + bias, 16-bit), waits on the grid
//                   barrier for h_{t-1}, then streams h_{t-1} (BT x 64 chunks) through the ring
//   MMA warp      : tcgen05.mma M=64 (gate rows; M=128 over a pair) x N=BT (batch) x K=16, accumulating over K = H
//                   into TMEM
//   4 epilogue warps: tcgen05.ld -> exchange through shared memory so that one thread sees all four
//                   gate sums of its (unit, sequence) pair -> + P_t -> sigmoid/tanh -> c_t (fp32),
//                   h_t (16-bit).  h_t is stored and published first; the cell state and the activated
//                   gates (the FP16/BF16 gate cache, written over P_t in global memory) follow
// Steps are separated by a per-batch-group barrier in global memory (release add / acquire poll).
// Every wait is bounded (FwdParams::wait_ns, 2 s by default); a timeout raises the CTA's abort word and the
// global error word, and every role leaves:
//   * the producer and MMA threads run their loops alone and simply break; on the way out the producer waits
//     (bounded) for every TMA copy it started and the MMA thread for its last committed UMMAs;
//   * the 256 epilogue threads never leave between their waits and the named barrier that follows: the barrier
//     ORs "my wait failed" over all of them (barrier.cta.red.or), so they continue or break TOGETHER and nobody is
//     left at a bar.sync; no wait lies between that barrier and the release barrier of the same step;
//   * all 320 threads meet at the final __syncthreads (a pair also at a final barrier.cluster, which each CTA reaches
//     on its own once its bounded waits have returned), after which the tensor memory is freed.
// Other CTAs learn of an abort through the global error word, which their counter polls read.
//
// Replaces, per step, the reference's ScaleAndPackColumnsKernel + GemmTN + ForwardPointwiseKernel
// launches (flashlstm_v2/src/lstm_forward.cu:744-830) and v1's GEMM + lstm_pointwise_kernel pair
// (src/lstm.cu:1241-1337, src/kernels.cu:86-164).
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "tc_common.cuh"
#include "tc_kernels.h"
#include "tc_recurrent.cuh"

namespace flstm_b200 {
namespace tc {

namespace {

constexpr int kFwdThreads = 320;  // warps 0-3 epilogue (TMEM readers), 4 producer, 5 MMA, 6-9 pointwise helpers
constexpr int kFwdEpilogueThreads = 256;
constexpr int kChunkBytesW = 64 * 64 * 2;

}  // namespace

struct FwdSmemLayout {
    int w_bytes, ring_stage_bytes, stages, p_bytes, ex_bytes, total;
};

// One ring stage holds `ch` consecutive 64-wide K chunks of an h tile (and of W when streamed).
// pair: the CTA is one half of a CTA pair (cta_group::2) and stages only its BT/2 sequences of every h chunk.
__host__ __device__ inline FwdSmemLayout fwd_smem_layout(int BT, int H, int rt, bool resident, int stages, int ch,
                                                         bool pair = false) {
    FwdSmemLayout l;
    const int kc = H / 64;
    l.w_bytes = resident ? rt * kc * kChunkBytesW : 0;
    l.ring_stage_bytes = ch * ((pair ? BT / 2 : BT) * 128 + (resident ? 0 : kChunkBytesW));
    l.stages = stages;
    l.p_bytes = 2 * BT * 128;
    l.ex_bytes = 2 * 64 * (BT + 4) * 4;
    l.total = l.w_bytes + stages * l.ring_stage_bytes + l.p_bytes + l.ex_bytes + 1024 /*align*/ + 512 /*barriers*/;
    return l;
}

// PAIR: two CTAs with neighbouring row tiles (ranks 0 and 1 of a cluster) run ONE tcgen05.mma.cta_group::2 of
// M = 128: each keeps its own 64 rows of W_hh, but stages only HALF of the h tile (BT/2 sequences) -- the UMMA reads
// the other half from the peer's shared memory -- so a step pulls half as many h bytes through L2 into every SM.
// Only the leader (rank 0) issues UMMAs; both CTAs' loads are counted on the leader's barriers, its commits
// signal both CTAs.  Each CTA finds its 64 x BT accumulator in its own tensor memory, sequences [0, BT/2) in lanes
// 0-63 and [BT/2, BT) in lanes 64-127 (BT/2 columns).  Nothing is multicast.
template <int BT, bool W_RESIDENT, bool BF16, bool PAIR>
__global__ void __launch_bounds__(kFwdThreads, 1)
lstm_fwd_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_h,
                const __grid_constant__ CUtensorMap tm_g, FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int EXS = BT + 4;  // row stride of the exchange buffer (floats), keeps float4 alignment
    const int KC = p.H / 64, CH = p.ch, NLOAD = KC / CH;
    const FwdSmemLayout L = fwd_smem_layout(BT, p.H, p.rt, W_RESIDENT, p.stages, CH, PAIR);
    constexpr int BTH = PAIR ? BT / 2 : BT;  // sequences of an h chunk this CTA stages
    uint8_t *s_w = smem;                                   // resident W slice: rt*KC chunks of 8 KB
    uint8_t *s_ring = s_w + L.w_bytes;                     // stages x [CH h chunks | (CH W chunks)]
    uint8_t *s_p = s_ring + L.stages * L.ring_stage_bytes;  // 2 P tiles, BT rows x 128 B, not swizzled
    float *s_ex = reinterpret_cast<float *>(s_p + L.p_bytes);  // 2 x [64][EXS] gate pre-activations (fp32)
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
    constexpr int kAccCols = PAIR ? BT / 2 : BT;  // tensor-memory columns of one accumulator
    constexpr int kTmemCols = (2 * kAccCols < 32) ? 32 : 2 * kAccCols;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < L.stages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], PAIR ? 8 : 4);  // the epilogue warps of both CTAs report to the leader
            mbar_init(&pfull[i], 1);
            mbar_init(&pempty[i], kFwdEpilogueThreads / 32);
        }
        mbar_init(wbar, 1);
        *abort_w = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_h);
        tma_prefetch_desc(&tm_g);
    }
    if (warp == 5) {
        if (PAIR) {
            tmem_alloc_pair(tmem_slot, kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, kTmemCols);
            tmem_relinquish();
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // both CTAs' barriers and tensor memory exist before anything crosses the pair
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // barriers the loads of this CTA complete: its own, or (PAIR) the leader's at the same offsets
    const uint32_t full_c = PAIR ? map_to_rank(smem_u32(full), 0) : smem_u32(full);
    const uint32_t wbar_c = PAIR ? map_to_rank(smem_u32(wbar), 0) : smem_u32(wbar);
    const uint32_t tempty_c = PAIR ? map_to_rank(smem_u32(tempty), 0) : smem_u32(tempty);
    const uint32_t stage_tx = (PAIR ? 2u : 1u) * (uint32_t)L.ring_stage_bytes;
    auto load_w = [&](void *dst, int x, int y, uint32_t bar) {  // a W_hh chunk
        if (PAIR) tma_load_2d_pair(dst, &tm_w, x, y, bar);
        else tma_load_2d_addr(dst, &tm_w, x, y, bar);
    };
    auto load_h = [&](void *dst, int b0, int chunk0, int t, uint32_t bar) {  // CH chunks of this CTA's part of an h tile
        if (PAIR) tma_load_4d_pair(dst, &tm_h, 0, b0 + (int)rank * BTH, chunk0, t, bar);
        else tma_load_4d_addr(dst, &tm_h, 0, b0, chunk0, t, bar);
    };

    const unsigned long long wait_ns = p.wait_ns ? p.wait_ns : kWaitLimitNs;
    const int nt_count = p.nt;  // batch tiles per group
    const int items_per_step = p.rt * nt_count;
    const bool tracing = p.trace != nullptr && blockIdx.x == 0;
#define FLSTM_STAMP(step, slot)                                                     \
    do {                                                                            \
        if (tracing && (step) < p.trace_steps) p.trace[(step) * 16 + (slot)] = clock64(); \
    } while (0)

    if (warp == 4) {
        // ------------------------------------------------------------ producer
        if (elect_one()) {
            bool ok = true;
            if (W_RESIDENT) {
                if (leader) mbar_expect_tx(wbar, (PAIR ? 2u : 1u) * (uint32_t)(p.rt * KC * kChunkBytesW));
                for (int r = 0; r < p.rt; ++r)
                    for (int kc = 0; kc < KC; ++kc)
                        load_w(s_w + (r * KC + kc) * kChunkBytesW, kc * 64, (jr * p.rt + r) * 64, wbar_c);
            }
            int stage = 0;
            uint32_t phase = 0, wi = 0;
            // what was issued last into every ring stage / P buffer, so that nothing is left in flight at exit
            uint32_t ring_issued = 0, ring_parity = 0, p_issued = 0, p_parity = 0;
            for (int tt = 0; tt < p.T && ok; ++tt) {
                const int t = p.t0 + tt;  // absolute time step; this launch runs steps [t0, t0 + T)
                bool first = true;
                for (int r = 0; r < p.rt && ok; ++r) {
                    const int j = jr * p.rt + r;
                    for (int n = 0; n < nt_count && ok; ++n, ++wi) {
                        const int b0 = (ng * nt_count + n) * BT;
                        const int pb = wi & 1;
                        ok = mbar_wait(&pempty[pb], ((wi >> 1) & 1) ^ 1, abort_w, wait_ns);
                        if (!ok) break;
                        mbar_expect_tx(&pfull[pb], BT * 128);
                        tma_load_3d(s_p + pb * BT * 128, &tm_g, j * 64, b0, t, &pfull[pb]);
                        p_issued |= 1u << pb;
                        p_parity = (p_parity & ~(1u << pb)) | (((wi >> 1) & 1u) << pb);
                        // Streamed weights: the W_hh chunks of a step's first loads do not depend on h_{t-1}, so they
                        // go into the ring AHEAD of the step barrier (the stage's byte count covers both copies; the
                        // h chunks follow once the barrier has been passed).
                        int npre = 0;
                        int pre_stage[kMaxRingStages];
                        if (!W_RESIDENT && first && tt > 0) {
                            npre = NLOAD < L.stages ? NLOAD : L.stages;
                            for (int ld = 0; ld < npre; ++ld) {
                                ok = mbar_wait(&empty[stage], phase ^ 1, abort_w, wait_ns);
                                if (!ok) break;
                                uint8_t *sh = s_ring + stage * L.ring_stage_bytes;
                                if (leader) mbar_expect_tx(&full[stage], stage_tx);
                                ring_issued |= 1u << stage;
                                ring_parity = (ring_parity & ~(1u << stage)) | (phase << stage);
                                for (int c = 0; c < CH; ++c)
                                    load_w(sh + CH * BTH * 128 + c * kChunkBytesW, (ld * CH + c) * 64, j * 64,
                                           full_c + 8u * (uint32_t)stage);
                                pre_stage[ld] = stage;
                                if (++stage == L.stages) { stage = 0; phase ^= 1; }
                            }
                            if (!ok) break;
                        }
                        if (first && tt > 0) {
                            // h_{t-1} of this batch group is complete when every CTA of the group has
                            // arrived tt times in this launch (once per step each); the state a launch
                            // starts from was completed by the previous launch.  p.extra_arrivals is 0 except in
                            // the self-test of the timeout path, where it asks for arrivals that nobody makes.
                            ok = wait_counter(counter, (unsigned)(p.cta_rows) * (unsigned)tt + p.extra_arrivals, p.err,
                                              abort_w, 2u, wait_ns);
                            if (!ok) break;
                            fence_proxy_async_global();
                        }
                        if (first) FLSTM_STAMP(tt, 0);
                        first = false;
                        for (int ld = 0; ld < npre; ++ld)
                            load_h(s_ring + pre_stage[ld] * L.ring_stage_bytes, b0, ld * CH, t,
                                   full_c + 8u * (uint32_t)pre_stage[ld]);
                        for (int ld = npre; ld < NLOAD; ++ld) {
                            ok = mbar_wait(&empty[stage], phase ^ 1, abort_w, wait_ns);
                            if (!ok) break;
                            uint8_t *sh = s_ring + stage * L.ring_stage_bytes;
                            if (leader) mbar_expect_tx(&full[stage], stage_tx);
                            ring_issued |= 1u << stage;
                            ring_parity = (ring_parity & ~(1u << stage)) | (phase << stage);
                            // CH chunks of the h tile with one copy: (x, row, chunk, step)
                            load_h(sh, b0, ld * CH, t, full_c + 8u * (uint32_t)stage);
                            if (!W_RESIDENT)
                                for (int c = 0; c < CH; ++c)
                                    load_w(sh + CH * BTH * 128 + c * kChunkBytesW, (ld * CH + c) * 64, j * 64,
                                           full_c + 8u * (uint32_t)stage);
                            if (++stage == L.stages) { stage = 0; phase ^= 1; }
                        }
                        FLSTM_STAMP(tt, 1);
                    }
                }
            }
            // Way out (normal or aborted): every copy this thread started must have landed before the CTA
            // exits.  After a normal run the consumers have already waited for all of them, so this costs nothing.
            // (a stage whose W_hh chunks went ahead of a barrier that then failed never gets its h chunks: after an
            // abort the wait for it is cut short, long after the chunks that were started have landed)
            // (PAIR: the peer's copies complete the LEADER's barriers, which it cannot wait on; after a normal run
            // the UMMAs have consumed them all, after an abort the whole CTA lingers before it leaves, see below)
            if (W_RESIDENT && leader) mbar_drain(wbar, 0, wait_ns);
            for (int i = 0; i < L.stages && leader; ++i)
                if (ring_issued >> i & 1u) mbar_drain(&full[i], ring_parity >> i & 1u, ok ? wait_ns : kAbortDrainNs);
            for (int i = 0; i < 2; ++i)
                if (p_issued >> i & 1u) mbar_drain(&pfull[i], p_parity >> i & 1u, wait_ns);
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer (PAIR: the leader's only)
        if (leader && elect_one()) {
            bool ok = true;
            if (W_RESIDENT) ok = mbar_wait(wbar, 0, abort_w, wait_ns);
            int stage = 0;
            uint32_t phase = 0, wi = 0;
            const uint32_t s_w_u32 = smem_u32(s_w), idesc = p.idesc;
            const uint32_t empty_l = smem_u32(empty), tfull_l = smem_u32(tfull);
            const uint32_t total_items = (uint32_t)p.T * items_per_step;
            int last_commit = -1;
            for (uint32_t it = 0; it < total_items && ok; ++it, ++wi) {
                const int r = (it % items_per_step) / nt_count;
                const int buf = wi & 1;
                ok = PAIR ? mbar_wait_cluster(&tempty[buf], ((wi >> 1) & 1) ^ 1, abort_w, wait_ns)
                          : mbar_wait(&tempty[buf], ((wi >> 1) & 1) ^ 1, abort_w, wait_ns);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * kAccCols;
                for (int ld = 0; ld < NLOAD; ++ld) {
                    ok = mbar_wait(&full[stage], phase, abort_w, wait_ns);
                    if (!ok) break;
                    if (ld == 0) FLSTM_STAMP((int)(it / items_per_step), 2);
                    if (ld == NLOAD - 1) FLSTM_STAMP((int)(it / items_per_step), 3);
                    tcgen05_fence_after();
                    const uint32_t st_base = smem_u32(s_ring + stage * L.ring_stage_bytes);
                    for (int c = 0; c < CH; ++c) {
                        const int kc = ld * CH + c;
                        const uint32_t h_base = st_base + c * BTH * 128;
                        const uint32_t w_base = W_RESIDENT ? s_w_u32 + (uint32_t)(r * KC + kc) * kChunkBytesW
                                                           : st_base + CH * BTH * 128 + c * kChunkBytesW;
                        // one descriptor per chunk; the three further K steps of 16 elements advance the
                        // start-address field by 32 bytes (2 in descriptor units)
                        const uint64_t dw = umma_desc_kmajor_sw128(w_base), dh = umma_desc_kmajor_sw128(h_base);
                        if (PAIR) {
                            umma_f16_pair(d_tmem, dw, dh, idesc, kc != 0);
                            umma_f16_pair(d_tmem, dw + 2, dh + 2, idesc, 1u);
                            umma_f16_pair(d_tmem, dw + 4, dh + 4, idesc, 1u);
                            umma_f16_pair(d_tmem, dw + 6, dh + 6, idesc, 1u);
                        } else {
                            if (kc == 0) umma_f16_imm<false>(d_tmem, dw, dh, idesc);
                            else umma_f16_imm<true>(d_tmem, dw, dh, idesc);
                            umma_f16_imm<true>(d_tmem, dw + 2, dh + 2, idesc);
                            umma_f16_imm<true>(d_tmem, dw + 4, dh + 4, idesc);
                            umma_f16_imm<true>(d_tmem, dw + 6, dh + 6, idesc);
                        }
                    }
                    // the stage may be refilled (PAIR: in both CTAs) once these UMMAs have read it
                    if (PAIR) umma_commit_pair_both(empty_l + 8u * (uint32_t)stage);
                    else umma_commit(&empty[stage]);
                    if (++stage == L.stages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (PAIR) umma_commit_pair_both(tfull_l + 8u * (uint32_t)buf);
                else umma_commit(&tfull[buf]);
                last_commit = (int)wi;
                FLSTM_STAMP((int)(it / items_per_step), 4);
            }
            // the tensor memory is freed at the end of the kernel: the last committed batch of UMMAs must be done
            if (last_commit >= 0) mbar_drain(&tfull[last_commit & 1], (uint32_t)(last_commit >> 1) & 1u, wait_ns);
        }
    } else {
        // ------------------------------------------------------------ epilogue (256 threads)
        // Warps 0-3 own the TMEM lane quadrants and move the accumulator to shared memory (phase A); the
        // pointwise update (phase B) is spread over them and the four helper warps 6-9.
        const int tid = warp < 4 ? threadIdx.x : threadIdx.x - 64;  // 0..255
        const int u = tid & 15, nb = tid >> 4;  // phase-B ownership: unit u, sequences nb + 16*i
        constexpr int PAIRS = BT / 16;
        float c_keep[PAIRS];
        const bool keep_c = items_per_step == 1;
        const size_t slab = (size_t)p.B * p.H;
        const size_t G = (size_t)4 * p.H;
        uint16_t *hs = static_cast<uint16_t *>(p.hs);
        uint16_t *y = static_cast<uint16_t *>(p.y);
        uint16_t *gates = static_cast<uint16_t *>(p.gates);
        uint32_t wi = 0;
        bool ok = true;
        for (int tt = 0; tt < p.T && ok; ++tt) {
            const int t = p.t0 + tt;
            for (int r = 0; r < p.rt && ok; ++r) {
                const int j = jr * p.rt + r;
                for (int n = 0; n < nt_count && ok; ++n, ++wi) {
                    const int b0 = (ng * nt_count + n) * BT;
                    const int buf = wi & 1, pb = wi & 1;
                    const bool last_item = (r == p.rt - 1) && (n == nt_count - 1);
                    // cell state entering this step (own writes of the previous step, or registers)
                    float c_prev[PAIRS];
#pragma unroll
                    for (int i = 0; i < PAIRS; ++i) {
                        const int b = b0 + nb + 16 * i;
                        if (keep_c && tt > 0) c_prev[i] = c_keep[i];
                        else c_prev[i] = (b < p.B) ? p.cs[(size_t)t * slab + (size_t)b * p.H + j * 16 + u] : 0.f;
                    }
                    // No thread leaves between here and the named barrier below, whatever its waits return: the
                    // barrier ORs the failures, so that all 256 threads go on or give up together.
                    bool good = mbar_wait(&tfull[buf], (wi >> 1) & 1, abort_w, wait_ns);
                    if (tid == 0) FLSTM_STAMP(tt, 5);
                    tcgen05_fence_after();
                    float *ex = s_ex + (wi & 1) * 64 * EXS;
                    // phase A (warps 0-3): lanes 0..15 of warp g hold the recurrent sums of gate g, units 0..15,
                    // all BT sequences; they go to shared memory as they are
                    if (warp < 4 && !PAIR) {
#pragma unroll
                        for (int c0 = 0; c0 < BT; c0 += 32) {
                            uint32_t acc[32];
                            tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BT + c0, acc);
                            tmem_ld_wait();
                            if (lane < 16) {
                                float4 *dst = reinterpret_cast<float4 *>(ex + (warp * 16 + lane) * EXS + c0);
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    dst[i] = make_float4(__uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]),
                                                         __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
                            }
                        }
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tempty[buf]);
                    }
                    if (warp < 4 && PAIR) {
                        // M = 128 over the pair: lane quadrant w holds rows 32 (w & 1) + lane of this CTA's 64 and
                        // the sequences [(w >> 1) BT/2, +BT/2); every lane carries a row
                        const int row = 32 * (warp & 1) + lane, seq0 = (warp >> 1) * (BT / 2);
                        constexpr int W16 = (BT / 2 < 32) ? 16 : 32;  // columns per tensor-memory load
#pragma unroll
                        for (int c0 = 0; c0 < BT / 2; c0 += W16) {
                            uint32_t acc[W16];
                            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * kAccCols + c0;
                            if (W16 == 16) tmem_ld_32x32b_x16(taddr, *reinterpret_cast<uint32_t(*)[16]>(&acc[0]));
                            else tmem_ld_32x32b_x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
                            tmem_ld_wait();
                            float4 *dst = reinterpret_cast<float4 *>(ex + row * EXS + seq0 + c0);
#pragma unroll
                            for (int i = 0; i < W16 / 4; ++i)
                                dst[i] = make_float4(__uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]),
                                                     __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
                        }
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster_relaxed(tempty_c + 8u * (uint32_t)buf);
                    }
                    if (good) good = mbar_wait(&pfull[pb], (wi >> 1) & 1, abort_w, wait_ns);
                    if (named_barrier_or(1, kFwdEpilogueThreads, !good)) {
                        ok = false;
                        break;
                    }
                    if (tid == 0) FLSTM_STAMP(tt, 6);
                    // phase B: one thread per (unit, sequence) pair does the whole pointwise update
                    const uint16_t *ptile = reinterpret_cast<const uint16_t *>(s_p + pb * BT * 128);
                    float act[PAIRS][4];
                    uint16_t h16[PAIRS];
#pragma unroll
                    for (int i = 0; i < PAIRS; ++i) {
                        const int nn = nb + 16 * i;
                        const float ai = ex[(0 * 16 + u) * EXS + nn] + load16<BF16>(ptile + nn * 64 + 0 * 16 + u);
                        const float af = ex[(1 * 16 + u) * EXS + nn] + load16<BF16>(ptile + nn * 64 + 1 * 16 + u);
                        const float ag = ex[(2 * 16 + u) * EXS + nn] + load16<BF16>(ptile + nn * 64 + 2 * 16 + u);
                        const float ao = ex[(3 * 16 + u) * EXS + nn] + load16<BF16>(ptile + nn * 64 + 3 * 16 + u);
                        const float gi = sigmoid_fast(ai), gf = sigmoid_fast(af), gg = tanh_fast(ag), go = sigmoid_fast(ao);
                        const float c = fmaf(gf, c_prev[i], gi * gg);
                        const float h = go * tanh_fast(c);
                        c_keep[i] = c;
                        act[i][0] = gi; act[i][1] = gf; act[i][2] = gg; act[i][3] = go;
                        h16[i] = to16<BF16>(h);
                        // h_t first: it is what the other CTAs wait for
                        if (b0 + nn < p.B) hs[(size_t)(t + 1) * slab + (size_t)(b0 + nn) * p.H + j * 16 + u] = h16[i];
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&pempty[pb]);  // this warp is done with the P tile
                    if (last_item) {
                        if (tid == 0) FLSTM_STAMP(tt, 7);
                        // publish h_t: after the named barrier thread 0's release is cumulative over every epilogue
                        // warp's stores.  The generic->async proxy fence sits on the consumer side, between its
                        // acquire of the counter and its TMA loads.
                        // ONE arrival per CTA: the arrivals of a step serialise on the counter's address in L2, and
                        // one per epilogue warp cost every step about a thousand cycles more
                        named_barrier_sync(2, kFwdEpilogueThreads);
                        if (tid == 0) red_release_gpu_add(counter, 1u);
                        if (tid == 0) FLSTM_STAMP(tt, 8);
                    }
                    // everything nobody waits for: cell state, gate cache, the caller's y
#pragma unroll
                    for (int i = 0; i < PAIRS; ++i) {
                        const int b = b0 + nb + 16 * i;
                        if (b >= p.B) continue;
                        const size_t idx = (size_t)b * p.H + j * 16 + u;
                        p.cs[(size_t)(t + 1) * slab + idx] = c_keep[i];
                        if (y) y[(size_t)t * slab + idx] = h16[i];
                        if (p.store_gates) {
                            uint16_t *grow = gates + ((size_t)t * p.B + b) * G + (size_t)j * 64 + u;
                            grow[0] = to16<BF16>(act[i][0]);
                            grow[16] = to16<BF16>(act[i][1]);
                            grow[32] = to16<BF16>(act[i][2]);
                            grow[48] = to16<BF16>(act[i][3]);
                        }
                    }
                }
            }
        }
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
        if (warp == 5) tmem_dealloc_pair(tmem_base, kTmemCols);
    } else if (warp == 5) {
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_w) atomicCAS(p.err, 0u, 1u);
}

// ------------------------------------------------------------------ host launcher
template <int BT, bool RES, bool BF16, bool PAIR>
static int launch_fwd(const CUtensorMap &tw, const CUtensorMap &th, const CUtensorMap &tg, const FwdParams &p, int grid,
                      int smem_bytes, cudaStream_t s) {
    auto kern = lstm_fwd_kernel<BT, RES, BF16, PAIR>;
    FLSTM_CUDA_TRY(ensure_smem_limit(kern, (size_t)smem_bytes));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kFwdThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs must be co-resident: they wait on one another
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;  // PAIR: neighbouring row tiles form a cluster of two
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = PAIR ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, th, tg, p);
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "recurrent forward launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

// FLSTM_FWD_PAIR=0: no CTA pairs in the forward kernel
static int fwd_pair_mode() {
    const char *env = std::getenv("FLSTM_FWD_PAIR");
    return (env && env[0] == '0') ? 0 : 1;
}

// FLSTM_BT64=0 keeps 32-wide batch tiles for 33..64 sequences (two tiles per CTA when H >= 2048)
bool wide_tile_enabled() {
    const char *env = std::getenv("FLSTM_BT64");
    return !(env && env[0] == '0');
}

bool wider_tile_enabled() {
    const char *env = std::getenv("FLSTM_BT128");
    return !(env && env[0] == '0');
}

int plan_fwd(int B, int H, int sms, size_t smem_limit, FwdPlan *plan) {
    if (H % 64 != 0 || H < 64) return set_error(FLSTM_ERR_UNSUPPORTED, "hidden size must be a multiple of 64");
    const int R = H / 16;  // row tiles
    int rt = 1;
    while (R / rt > sms || R % rt) ++rt;
    const int cta_rows = R / rt;
    // 32 sequences per batch tile while every batch group then gets its own set of CTAs; when the row tiles
    // alone fill the machine (H = 2048) a CTA would take two 32-wide tiles per step and stream its W_hh slice
    // twice, so 33..64 sequences become ONE 64-wide tile (the UMMA costs the same at N = 32 and N = 64), and
    // 65..128 sequences per batch group ONE 128-wide tile.
    // Measured at B = 64, H = 2048, L = 2, T = 1024 (fwd+bwd): 46.5 ms against 55.6 ms on the per-step path.  With
    // two row tiles per CTA (H = 4096) the per-step path stays ahead (75.6 against 88.6 ms), so the rule stops there.
    int BT = (B >= 128) ? 64 : 32;
    int tiles = 0, ngroups = 0, nt = 0;
    auto split = [&](int bt) {
        tiles = (B + bt - 1) / bt;
        ngroups = sms / cta_rows;
        if (ngroups > tiles) ngroups = tiles;
        if (ngroups < 1) ngroups = 1;
        nt = (tiles + ngroups - 1) / ngroups;
        ngroups = (tiles + nt - 1) / nt;
    };
    split(BT);
    if (nt > 1 && rt == 1) {
        // the narrowest wider tile that leaves every CTA a single batch tile per step
        const int max_groups = sms / cta_rows < 1 ? 1 : sms / cta_rows;
        const int first = BT == 32 ? 64 : 128;
        bool found = false;
        for (int bt = first; bt <= 128 && !found; bt *= 2) {
            if (bt == 64 && !(max_groups == 1 && wide_tile_enabled())) continue;
            // 128-wide tiles pay when two or more batch groups work side by side (H <= 1024); measured at
            // H = 2048, B = 128 the per-step path stays ahead over forward + backward (79.8 against 82.2 ms)
            if (bt == 128 && !(max_groups >= 2 && wider_tile_enabled())) continue;
            split(bt);
            if (nt == 1 && ngroups == max_groups) {  // and no batch group's CTAs are left idle
                BT = bt;
                found = true;
            }
        }
        if (!found) split(BT);
    }
    // CTA pairs (each CTA stages half of the h tile) need an even number of row-tile CTAs per batch group: the two
    // CTAs of a pair share a batch tile.  Measured forward phases, lone CTAs -> pairs: config 2 2.05 -> 1.83 ms;
    // config 3 at 16 / 32 / 64 sequences per GPU 12.7 -> 10.6 / 13.1 -> 10.9 / 15.7 -> 12.4 ms; config 5 at 256
    // sequences 8.3 -> 7.3 ms; config 4 (two row tiles per CTA, HBM-bound) 47.7 -> 47.1 ms.
    const bool pair = cta_rows % 2 == 0 && fwd_pair_mode() != 0;
    // One TMA copy brings `ch` 64-wide K chunks of an h tile; the ring holds a whole tile when it can.
    // The W_hh slice stays resident if it fits next to a ring of at least two stages.
    const int kc = H / 64;
    // measured on config 2: one 64 KB copy per step beats 2, 4, 8 or 16 smaller ones (TMA issue cost
    // outweighs the longer exposed UMMA tail), so a stage takes up to 16 chunks
    // (measured: the streamed-weight and multi-tile regimes need several smaller stages in flight instead)
    int ch16 = 16;
    while (kc % ch16) --ch16;
    const bool one_tile_resident = nt == 1 && (size_t)fwd_smem_layout(BT, H, rt, true, kc / ch16, ch16, pair).total <= smem_limit;
    int ch = one_tile_resident ? 16 : 4;
    if (const char *env = std::getenv("FLSTM_CH")) ch = std::atoi(env) > 0 ? std::atoi(env) : ch;
    while (kc % ch) --ch;
    bool resident = true;
    int stages = kc / ch;
    FwdSmemLayout l = fwd_smem_layout(BT, H, rt, true, stages, ch, pair);
    while ((size_t)l.total > smem_limit && stages > 2) l = fwd_smem_layout(BT, H, rt, true, --stages, ch, pair);
    if ((size_t)l.total > smem_limit || (stages < 2 && kc / ch >= 2)) {
        resident = false;
        stages = kc / ch < 4 ? kc / ch : 4;
        l = fwd_smem_layout(BT, H, rt, false, stages, ch, pair);
        while ((size_t)l.total > smem_limit && stages > 1) l = fwd_smem_layout(BT, H, rt, false, --stages, ch, pair);
        // a single stage cannot overlap the copy with the UMMAs: rather two stages of half the chunks
        while (stages < 2 && ch > 1 && kc / (ch / 2) >= 2) {
            ch /= 2;
            stages = 2;
            l = fwd_smem_layout(BT, H, rt, false, stages, ch, pair);
            if ((size_t)l.total > smem_limit) stages = 1;
        }
        l = fwd_smem_layout(BT, H, rt, false, stages, ch, pair);
        while ((size_t)l.total > smem_limit && ch > 1) {
            --ch;
            while (kc % ch) --ch;
            l = fwd_smem_layout(BT, H, rt, false, stages, ch, pair);
        }
        if ((size_t)l.total > smem_limit) return set_error(FLSTM_ERR_UNSUPPORTED, "recurrent kernel does not fit shared memory");
    }
    plan->ch = ch;
    plan->pair = pair;
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
    p.ch = plan.ch;
    p.idesc = umma_idesc_f16(plan.pair ? 128 : 64, plan.BT, bf16 ? 1 : 0, 0, 0);
#define FLSTM_FWD_CASE(BT_, RES_)                                                                                  \
    if (plan.BT == BT_ && plan.resident == RES_) {                                                                 \
        if (plan.pair)                                                                                             \
            return bf16 ? launch_fwd<BT_, RES_, true, true>(tm_w, tm_h, tm_g, p, plan.grid, plan.smem_bytes, s)    \
                        : launch_fwd<BT_, RES_, false, true>(tm_w, tm_h, tm_g, p, plan.grid, plan.smem_bytes, s);  \
        return bf16 ? launch_fwd<BT_, RES_, true, false>(tm_w, tm_h, tm_g, p, plan.grid, plan.smem_bytes, s)       \
                    : launch_fwd<BT_, RES_, false, false>(tm_w, tm_h, tm_g, p, plan.grid, plan.smem_bytes, s);     \
    }
    FLSTM_FWD_CASE(32, true)
    FLSTM_FWD_CASE(32, false)
    FLSTM_FWD_CASE(64, true)
    FLSTM_FWD_CASE(64, false)
    FLSTM_FWD_CASE(128, true)
    FLSTM_FWD_CASE(128, false)
#undef FLSTM_FWD_CASE
    return set_error(FLSTM_ERR_UNSUPPORTED, "no recurrent forward kernel for this plan");
}

}  // namespace tc
}  // namespace flstm_b200
