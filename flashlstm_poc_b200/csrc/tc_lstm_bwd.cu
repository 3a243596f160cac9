// Persistent BPTT kernel: ONE launch runs the whole reverse recurrence of one layer.
//
// Per reverse step the recurrence needs dh_{t} = dY_t + dG_{t+1} W_hh, a contraction over K = 4H.
// Work split: a cluster of KS CTAs owns 64 hidden units (unit tile j); CTA kq of the cluster
// contracts over its quarter (1/KS) of K with its slice of W_hh resident in shared memory (read as
// stored, i.e. as an MN-major UMMA operand), the KS partial results are reduce-scattered through
// distributed shared memory (st.shared::cluster + a remote mbarrier arrive), and every CTA then runs
// the fused pointwise backward for its 64/KS units:
//   producer warp : waits on the grid barrier for dG_{t+1}, streams it (BT x 64 chunks) via TMA
//   MMA warp      : tcgen05.mma M=64 (hidden units) x N=BT (batch) x K=16 into TMEM
//   4 epilogue warps: tcgen05.ld -> partials to the owner CTA's shared memory -> sum -> gate cache,
//                   c_t, c_{t-1}, dY_t (prefetched before the wait) -> dG_t (16-bit, tile-interleaved),
//                   dc carry in registers -> publish dG_t (release add on the group's counter)
// The cell state is READ from the forward's cache; it is never reconstructed from y and o as the
// reference does (flashlstm_v2/src/lstm_backward.cu:188-197).
//
// Every wait is bounded (BwdParams::wait_ns, 2 s by default) and the way out after a timeout is the forward
// kernel's: the producer and MMA threads break out of their loops and wait (bounded) for the copies / UMMAs
// they started; the 256 epilogue threads stay together because the named barrier after their waits ORs the
// failures (barrier.cta.red.or) and no wait lies between it and the release barrier of the step; everybody
// meets at the final __syncthreads and the cluster barrier (each CTA gets there on its own: its waits for a
// peer's partial sums are bounded too), then the tensor memory is freed.
//
// Replaces, per step, BackwardPointwiseKernel + GemmNN (flashlstm_v2/src/lstm_backward.cu:158-227,
// 1057-1101) and the whole recompute loop (:991-1054), which the gate cache makes unnecessary.
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

constexpr int kBwdThreads = 320;  // warps 0-3 epilogue (TMEM readers), 4 producer, 5 MMA, 6-9 pointwise helpers
constexpr int kBwdEpilogueThreads = 256;
constexpr int kChunkBytesW = 64 * 64 * 2;

struct PairIn {
    float gi, gf, gg, go, ct, cp, dy;
};

}  // namespace

struct BwdSmemLayout {
    int w_bytes, ring_stage_bytes, stages, red_bytes, total;
};

__host__ __device__ inline BwdSmemLayout bwd_smem_layout(int BT, int H, int KS, bool resident, int stages, int ch) {
    BwdSmemLayout l;
    const int kc_per = (H / 16) / KS;  // 64-wide K chunks this CTA contracts over
    l.w_bytes = resident ? kc_per * kChunkBytesW : 0;
    l.ring_stage_bytes = ch * (BT * 128 + (resident ? 0 : kChunkBytesW));
    l.stages = stages;
    l.red_bytes = 2 * KS * (64 / KS) * (BT + 4) * 4;  // 2 x [KS sources][64/KS units][BT+4]
    l.total = l.w_bytes + stages * l.ring_stage_bytes + l.red_bytes + 1024 + 512;
    return l;
}

template <int BT, int KS, bool W_RESIDENT, bool BF16>
__global__ void __launch_bounds__(kBwdThreads, 1)
lstm_bwd_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_dg, BwdParams p) {
    constexpr int UPO = 64 / KS;            // units this CTA owns after the reduce-scatter
    constexpr int UQ = UPO / 16;            // 16-unit groups per owner
    constexpr int PAIRS = UQ * (BT / 16);   // (unit, sequence) pairs per epilogue thread
    constexpr bool PREFETCH = PAIRS <= 8;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int RS = BT + 4;  // row stride of the reduce buffer (floats), keeps float4 alignment
    const int KCper = (p.H / 16) / KS, CH = p.ch, NLOAD = KCper / CH;
    const BwdSmemLayout L = bwd_smem_layout(BT, p.H, KS, W_RESIDENT, p.stages, CH);
    uint8_t *s_w = smem;
    uint8_t *s_ring = s_w + L.w_bytes;
    float *s_red = reinterpret_cast<float *>(s_ring + L.stages * L.ring_stage_bytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(s_red) + L.red_bytes);
    uint64_t *full = bars, *empty = bars + L.stages;
    uint64_t *tfull = empty + L.stages, *tempty = tfull + 2;
    uint64_t *rbar = tempty + 2;  // [2] reduce-scatter arrival barriers (64 arrivals each)
    uint64_t *wbar = rbar + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(wbar + 1);
    volatile uint32_t *abort_w = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kq = (KS > 1) ? (int)cluster_ctarank() : 0;
    const int cl = blockIdx.x / KS;          // cluster index
    const int ng = cl / p.jt;                // batch group
    const int j = cl % p.jt;                 // unit tile: hidden units [64j, 64j+64)
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
            // split K: the remote partials count themselves in (st.async), one expect_tx arrival announces their
            // bytes, and the UPO lanes that hold this CTA's own rows arrive after their plain stores
            mbar_init(&rbar[i], KS > 1 ? 1 + UPO : 64);
        }
        mbar_init(wbar, 1);
        *abort_w = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_dg);
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    if (KS > 1) cluster_sync_all();  // every CTA's barriers exist before any remote arrive
    const uint32_t tmem_base = *tmem_slot;
    const unsigned long long wait_ns = p.wait_ns ? p.wait_ns : kWaitLimitNs;
    const int nt_count = p.nt;
    const int c_first = kq * KCper;  // first K chunk (= forward row tile) of this CTA
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
                mbar_expect_tx(wbar, (uint32_t)(KCper * kChunkBytesW));
                for (int c = 0; c < KCper; ++c)
                    tma_load_2d(s_w + c * kChunkBytesW, &tm_w, j * 64, (c_first + c) * 64, wbar);
            }
            int stage = 0;
            uint32_t phase = 0;
            uint32_t ring_issued = 0, ring_parity = 0;  // the last copy started into every ring stage
            // this launch runs reverse iterations [s0, s1); iteration s handles time t = T-1-s and, for
            // s >= 1, first contracts dG_{t+1}, which iteration s-1 produced (in this launch: wait for
            // the group's counter; in the previous launch: already complete).  p.extra_arrivals is 0 except in
            // the self-test of the timeout path, where it asks for arrivals that nobody makes.
            for (int s = (p.s0 > 1 ? p.s0 : 1); s < p.s1 && ok; ++s) {
                const int t_src = p.T - s;  // dG_{t+1} with t = T-1-s
                // Streamed weights: the W_hh chunks of the iteration's first loads do not depend on dG_{t+1}, so they
                // go into the ring AHEAD of the step barrier (the stage's byte count covers both copies; the dG
                // chunks follow once the barrier has been passed).
                int npre = 0;
                int pre_stage[kMaxRingStages];
                if (!W_RESIDENT && s > p.s0) {
                    npre = NLOAD < L.stages ? NLOAD : L.stages;
                    for (int ld = 0; ld < npre; ++ld) {
                        ok = mbar_wait(&empty[stage], phase ^ 1, abort_w, wait_ns);
                        if (!ok) break;
                        uint8_t *sd = s_ring + stage * L.ring_stage_bytes;
                        mbar_expect_tx(&full[stage], (uint32_t)L.ring_stage_bytes);
                        ring_issued |= 1u << stage;
                        ring_parity = (ring_parity & ~(1u << stage)) | (phase << stage);
                        for (int c = 0; c < CH; ++c)
                            tma_load_2d(sd + CH * BT * 128 + c * kChunkBytesW, &tm_w, j * 64, (c_first + ld * CH + c) * 64,
                                        &full[stage]);
                        pre_stage[ld] = stage;
                        if (++stage == L.stages) { stage = 0; phase ^= 1; }
                    }
                    if (!ok) break;
                }
                if (s > p.s0)
                    ok = wait_counter(counter, (unsigned)(p.jt * KS) * (unsigned)(s - p.s0) + p.extra_arrivals, p.err, abort_w,
                                      3u, wait_ns);
                if (!ok) break;
                fence_proxy_async_global();
                FLSTM_STAMP(s - p.s0, 0);
                for (int n = 0; n < nt_count && ok; ++n) {
                    const int b0 = (ng * nt_count + n) * BT;
                    const int skip = n == 0 ? npre : 0;
                    for (int ld = 0; ld < skip; ++ld)
                        tma_load_4d(s_ring + pre_stage[ld] * L.ring_stage_bytes, &tm_dg, 0, b0, c_first + ld * CH, t_src,
                                    &full[pre_stage[ld]]);
                    for (int ld = skip; ld < NLOAD; ++ld) {
                        ok = mbar_wait(&empty[stage], phase ^ 1, abort_w, wait_ns);
                        if (!ok) break;
                        uint8_t *sd = s_ring + stage * L.ring_stage_bytes;
                        mbar_expect_tx(&full[stage], (uint32_t)L.ring_stage_bytes);
                        ring_issued |= 1u << stage;
                        ring_parity = (ring_parity & ~(1u << stage)) | (phase << stage);
                        // CH chunks of the dG tile with one copy: (x, row, chunk, step)
                        tma_load_4d(sd, &tm_dg, 0, b0, c_first + ld * CH, t_src, &full[stage]);
                        if (!W_RESIDENT)
                            for (int c = 0; c < CH; ++c)
                                tma_load_2d(sd + CH * BT * 128 + c * kChunkBytesW, &tm_w, j * 64,
                                            (c_first + ld * CH + c) * 64, &full[stage]);
                        if (++stage == L.stages) { stage = 0; phase ^= 1; }
                    }
                }
                FLSTM_STAMP(s - p.s0, 1);
            }
            // way out (normal or aborted): every copy this thread started must have landed before the CTA exits
            // (a stage whose W_hh chunks went ahead of a barrier that then failed never gets its dG chunks: after an
            // abort the wait for it is cut short, long after the chunks that were started have landed)
            if (W_RESIDENT) mbar_drain(wbar, 0, wait_ns);
            for (int i = 0; i < L.stages; ++i)
                if (ring_issued >> i & 1u) mbar_drain(&full[i], ring_parity >> i & 1u, ok ? wait_ns : kAbortDrainNs);
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            bool ok = true;
            if (W_RESIDENT) ok = mbar_wait(wbar, 0, abort_w, wait_ns);
            int stage = 0;
            uint32_t phase = 0;
            const uint32_t s_w_u32 = smem_u32(s_w), idesc = p.idesc;
            const uint32_t items = (uint32_t)(p.s1 - (p.s0 > 1 ? p.s0 : 1)) * nt_count;
            int last_commit = -1;
            for (uint32_t wi = 0; wi < items && ok; ++wi) {
                const int buf = wi & 1;
                ok = mbar_wait(&tempty[buf], ((wi >> 1) & 1) ^ 1, abort_w, wait_ns);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BT;
                for (int ld = 0; ld < NLOAD; ++ld) {
                    ok = mbar_wait(&full[stage], phase, abort_w, wait_ns);
                    if (!ok) break;
                    if (ld == 0) FLSTM_STAMP((int)(wi / nt_count) + 1 - (p.s0 > 0 ? 1 : 0), 2);
                    if (ld == NLOAD - 1) FLSTM_STAMP((int)(wi / nt_count) + 1 - (p.s0 > 0 ? 1 : 0), 3);
                    tcgen05_fence_after();
                    const uint32_t st_base = smem_u32(s_ring + stage * L.ring_stage_bytes);
                    for (int c = 0; c < CH; ++c) {
                        const int kc = ld * CH + c;
                        const uint32_t dg_base = st_base + c * BT * 128;
                        const uint32_t w_base = W_RESIDENT ? s_w_u32 + (uint32_t)kc * kChunkBytesW
                                                           : st_base + CH * BT * 128 + c * kChunkBytesW;
                        // K steps of 16: +2048 bytes on the MN-major W slice, +32 bytes on the K-major dG tile
                        const uint64_t dw = umma_desc_mnmajor_sw128(w_base, 8192), dd = umma_desc_kmajor_sw128(dg_base);
                        if (kc == 0) umma_f16_imm<false>(d_tmem, dw, dd, idesc);
                        else umma_f16_imm<true>(d_tmem, dw, dd, idesc);
                        umma_f16_imm<true>(d_tmem, dw + 128, dd + 2, idesc);
                        umma_f16_imm<true>(d_tmem, dw + 256, dd + 4, idesc);
                        umma_f16_imm<true>(d_tmem, dw + 384, dd + 6, idesc);
                    }
                    umma_commit(&empty[stage]);
                    if (++stage == L.stages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&tfull[buf]);
                last_commit = (int)wi;
                FLSTM_STAMP((int)(wi / nt_count) + 1 - (p.s0 > 0 ? 1 : 0), 4);
            }
            // the tensor memory is freed at the end of the kernel: the last committed batch of UMMAs must be done
            if (last_commit >= 0) mbar_drain(&tfull[last_commit & 1], (uint32_t)(last_commit >> 1) & 1u, wait_ns);
        }
    } else {
        // ------------------------------------------------------------ epilogue (256 threads)
        // Warps 0-3 own the TMEM lane quadrants: they read the accumulator and scatter the partial sums (phase A).
        // The reduction of the partials and the pointwise backward are spread over them and helper warps 6-9.
        const int tid = warp < 4 ? threadIdx.x : threadIdx.x - 64;  // 0..255
        const int u16 = tid & 15, nb = tid >> 4;  // unit u16 (+16q), sequences nb + 16*i
        const size_t slab = (size_t)p.B * p.H;
        const size_t G = (size_t)4 * p.H;
        const uint16_t *gates = static_cast<const uint16_t *>(p.gates);
        const uint16_t *dy = static_cast<const uint16_t *>(p.dy);
        const uint16_t *dhn = static_cast<const uint16_t *>(p.dhn);
        const uint16_t *dcn = static_cast<const uint16_t *>(p.dcn);
        uint16_t *dg = static_cast<uint16_t *>(p.dg);
        const bool keep_dc = nt_count == 1;
        float dc_keep[PAIRS];
        const uint32_t red_local = smem_u32(s_red);
        const uint32_t rbar_local = smem_u32(rbar);
        uint32_t wi = 0;  // MMA item counter (iterations s >= 1)
        bool ok = true;
        for (int s = p.s0; s < p.s1 && ok; ++s) {
            const int t = p.T - 1 - s;  // time step whose dG is produced (t = -1: only dh0 / dc0)
            for (int n = 0; n < nt_count && ok; ++n) {
                const int b0 = (ng * nt_count + n) * BT;
                PairIn in[PAIRS];
                float dc_in[PAIRS];
                auto unit_of = [&](int q) { return j * 64 + kq * UPO + q * 16 + u16; };
                auto load_pair = [&](int q, int i, PairIn &v) {
                    const int b = b0 + nb + 16 * i, U = unit_of(q);
                    if (b < p.B && t >= 0) {
                        const uint16_t *grow = gates + ((size_t)t * p.B + b) * G + (size_t)(U >> 4) * 64 + (U & 15);
                        v.gi = load16<BF16>(grow);
                        v.gf = load16<BF16>(grow + 16);
                        v.gg = load16<BF16>(grow + 32);
                        v.go = load16<BF16>(grow + 48);
                        const size_t idx = (size_t)b * p.H + U;
                        v.ct = p.cs[(size_t)(t + 1) * slab + idx];
                        v.cp = p.cs[(size_t)t * slab + idx];
                        v.dy = load16<BF16>(dy + (size_t)t * slab + idx);
                    } else {
                        v = PairIn{0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    }
                };
                // cell-gradient carry entering this step
#pragma unroll
                for (int q = 0; q < UQ; ++q)
#pragma unroll
                    for (int i = 0; i < BT / 16; ++i) {
                        const int k = q * (BT / 16) + i;
                        const int b = b0 + nb + 16 * i;
                        const size_t idx = (size_t)b * p.H + unit_of(q);
                        if (s == 0) dc_in[k] = (dcn && b < p.B) ? load16<BF16>(dcn + idx) : 0.f;
                        else if (keep_dc && s > p.s0) dc_in[k] = dc_keep[k];
                        else dc_in[k] = (b < p.B) ? p.dc[idx] : 0.f;
                        if (PREFETCH) load_pair(q, i, in[k]);
                    }
                // dh contribution from the step above: reduce-scattered partial products
                float dh_in[PAIRS];
                if (s == 0) {
#pragma unroll
                    for (int q = 0; q < UQ; ++q)
#pragma unroll
                        for (int i = 0; i < BT / 16; ++i) {
                            const int b = b0 + nb + 16 * i;
                            dh_in[q * (BT / 16) + i] = (dhn && b < p.B) ? load16<BF16>(dhn + (size_t)b * p.H + unit_of(q)) : 0.f;
                        }
                } else {
                    const int buf = wi & 1, rb = wi & 1;
                    // No thread leaves between here and the named barrier below, whatever its waits return: the
                    // barrier ORs the failures, so that all 256 threads go on or give up together.  A warp sends
                    // its partial sums only if all of its lanes saw the accumulator complete.
                    bool good = __all_sync(0xffffffffu, mbar_wait(&tfull[buf], (wi >> 1) & 1, abort_w, wait_ns));
                    if (tid == 0) FLSTM_STAMP(s - p.s0, 5);
                    tcgen05_fence_after();
                    if (warp < 4 && good) {
                        // phase A (warps 0-3): lanes 0..15 of warp w hold units 16w+lane of the tile, all BT sequences
#pragma unroll
                        for (int c0 = 0; c0 < BT; c0 += 32) {
                            uint32_t acc[32];
                            tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BT + c0, acc);
                            tmem_ld_wait();
                            if (lane < 16) {
                                const int row = warp * 16 + lane;        // unit within the tile
                                const uint32_t owner = row / UPO, lu = row % UPO;
                                const uint32_t off = (uint32_t)(((rb * KS + kq) * UPO + lu) * RS + c0) * 4u;
                                if (KS > 1 && owner != (uint32_t)kq) {
                                    const uint32_t dst = map_to_rank(red_local + off, owner);
                                    const uint32_t bar = map_to_rank(rbar_local + rb * 8, owner);
#pragma unroll
                                    for (int i = 0; i < 8; ++i)
                                        st_async_v4(dst + 16 * i, acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3], bar);
                                } else {
                                    float4 *dst = reinterpret_cast<float4 *>(s_red + off / 4);
#pragma unroll
                                    for (int i = 0; i < 8; ++i)
                                        dst[i] = make_float4(__uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]),
                                                             __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
                                }
                            }
                        }
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tempty[buf]);
                        if (KS > 1) {
                            // this CTA receives UPO rows of BT fp32 partials from each of the other KS-1 CTAs; its own
                            // rows were stored directly by the lanes that hold them
                            if (tid == 0) mbar_expect_tx(&rbar[rb], (uint32_t)((KS - 1) * UPO * BT * 4));
                            if (lane < 16 && (uint32_t)((warp * 16 + lane) / UPO) == (uint32_t)kq) mbar_arrive(&rbar[rb]);
                        } else if (lane < 16) {
                            mbar_arrive(&rbar[rb]);
                        }
                    }
                    if (tid == 0) FLSTM_STAMP(s - p.s0, 9);
                    if (good) good = mbar_wait_cluster(&rbar[rb], (wi >> 1) & 1, abort_w, wait_ns);
                    if (tid == 0) FLSTM_STAMP(s - p.s0, 10);
                    const float *red = s_red + (size_t)rb * KS * UPO * RS;
#pragma unroll
                    for (int q = 0; q < UQ; ++q)
#pragma unroll
                        for (int i = 0; i < BT / 16; ++i) {
                            const int lu = q * 16 + u16, nn = nb + 16 * i;
                            float acc = 0.f;
#pragma unroll
                            for (int src = 0; src < KS; ++src) acc += red[(src * UPO + lu) * RS + nn];
                            dh_in[q * (BT / 16) + i] = acc;
                        }
                    // every warp has read this item's partials before any warp sends the next item's
                    if (named_barrier_or(1, kBwdEpilogueThreads, !good)) {
                        ok = false;
                        break;
                    }
                    if (tid == 0) FLSTM_STAMP(s - p.s0, 6);
                    ++wi;
                }
                // fused pointwise backward for the owned (unit, sequence) pairs
#pragma unroll
                for (int q = 0; q < UQ; ++q)
#pragma unroll
                    for (int i = 0; i < BT / 16; ++i) {
                        const int k = q * (BT / 16) + i;
                        const int b = b0 + nb + 16 * i, U = unit_of(q);
                        if (b >= p.B) continue;
                        const size_t idx = (size_t)b * p.H + U;
                        if (t < 0) {
                            if (p.dh0) p.dh0[idx] = dh_in[k];
                            if (p.dc0) p.dc0[idx] = dc_in[k];
                            continue;
                        }
                        PairIn v;
                        if (PREFETCH) v = in[k];
                        else load_pair(q, i, v);
                        const float dh = v.dy + dh_in[k];
                        const float tc = tanh_fast(v.ct);
                        const float d_o = dh * tc;
                        const float dcv = dc_in[k] + dh * v.go * (1.f - tc * tc);
                        const float dai = dcv * v.gg * v.gi * (1.f - v.gi);
                        const float daf = dcv * v.cp * v.gf * (1.f - v.gf);
                        const float dag = dcv * v.gi * (1.f - v.gg * v.gg);
                        const float dao = d_o * v.go * (1.f - v.go);
                        const float dcp = dcv * v.gf;
                        if (keep_dc) dc_keep[k] = dcp;
                        else p.dc[idx] = dcp;
                        uint16_t *drow = dg + ((size_t)t * p.B + b) * G + (size_t)(U >> 4) * 64 + (U & 15);
                        drow[0] = to16<BF16>(dai);
                        drow[16] = to16<BF16>(daf);
                        drow[32] = to16<BF16>(dag);
                        drow[48] = to16<BF16>(dao);
                    }
            }
            if (!ok) break;
            if (t >= 0) {
                if (tid == 0) FLSTM_STAMP(s - p.s0, 7);
                // publish dG_t (release, cumulative over the warp's stores); the generic->async proxy fence
                // is on the consumer side, after its acquire and before its TMA loads
                // ONE arrival per CTA (see the forward kernel): after the named barrier thread 0's release is
                // cumulative over every epilogue warp's stores
                named_barrier_sync(2, kBwdEpilogueThreads);
                if (tid == 0) red_release_gpu_add(counter, 1u);
                if (tid == 0) FLSTM_STAMP(s - p.s0, 8);
            }
        }
        // a later launch continues the recurrence: leave the cell-gradient carry where it will look for it
        if (ok && keep_dc && p.s1 <= p.T) {
            const int b0 = ng * nt_count * BT;
#pragma unroll
            for (int q = 0; q < UQ; ++q)
#pragma unroll
                for (int i = 0; i < BT / 16; ++i) {
                    const int b = b0 + nb + 16 * i;
                    if (b < p.B) p.dc[(size_t)b * p.H + j * 64 + kq * UPO + q * 16 + u16] = dc_keep[q * (BT / 16) + i];
                }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (KS > 1) {
        cluster_sync_all();  // nobody leaves while a peer may still send into its shared memory
        if (*abort_w) {
            // after an abort this CTA may not have waited for partial sums that a peer sent before it reached the
            // barrier above: give those asynchronous stores time to land before the shared memory is released
            const unsigned long long t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 20000ull) {}
        }
    }
    if (warp == 5) tmem_dealloc(tmem_base, kTmemCols);
    if (threadIdx.x == 0 && *abort_w) atomicCAS(p.err, 0u, 1u);
}

// ------------------------------------------------------------------ host side
template <int BT, int KS, bool RES, bool BF16>
static int launch_bwd(const CUtensorMap &tw, const CUtensorMap &tdg, const BwdParams &p, int grid, int smem_bytes,
                      cudaStream_t s) {
    auto kern = lstm_bwd_kernel<BT, KS, RES, BF16>;
    FLSTM_CUDA_TRY(ensure_smem_limit(kern, (size_t)smem_bytes));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kBwdThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeCooperative;  // co-residency: CTAs wait on one another
    attr[na].val.cooperative = 1;
    ++na;
    if (KS > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = KS;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tdg, p);
    if (KS > 1 && (e == cudaErrorNotSupported || e == cudaErrorInvalidValue)) {
        // a driver that refuses the cooperative and cluster attributes TOGETHER: the planner has already proved
        // with cudaOccupancyMaxActiveClusters that every cluster of this grid is resident at once (plan_bwd fails
        // otherwise), so the cluster attribute alone gives the same guarantee.  Any other error is reported.
        cudaGetLastError();
        cfg.attrs = attr + 1;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, kern, tw, tdg, p);
    }
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "BPTT launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

template <int BT, int KS, bool RES>
static int max_clusters(int smem_bytes, int grid) {
    auto kern = lstm_bwd_kernel<BT, KS, RES, false>;
    if (ensure_smem_limit(kern, (size_t)smem_bytes) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kBwdThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = KS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return n;
}

static int query_clusters(const BwdPlan &pl) {
#define FLSTM_BWD_Q(BT_, KS_, RES_) \
    if (pl.BT == BT_ && pl.KS == KS_ && pl.resident == RES_) return max_clusters<BT_, KS_, RES_>(pl.smem_bytes, pl.grid);
    FLSTM_BWD_Q(32, 2, true) FLSTM_BWD_Q(32, 2, false) FLSTM_BWD_Q(32, 4, true) FLSTM_BWD_Q(32, 4, false)
    FLSTM_BWD_Q(64, 2, true) FLSTM_BWD_Q(64, 2, false) FLSTM_BWD_Q(64, 4, true) FLSTM_BWD_Q(64, 4, false)
    FLSTM_BWD_Q(128, 4, true) FLSTM_BWD_Q(128, 4, false)
#undef FLSTM_BWD_Q
    return -1;
}

int plan_bwd(int B, int H, int sms, size_t smem_limit, BwdPlan *plan, bool check_device) {
    if (H % 64 != 0 || H < 64) return set_error(FLSTM_ERR_UNSUPPORTED, "hidden size must be a multiple of 64");
    const int jt = H / 64, kc_total = H / 16;
    // split K = 4H so that a CTA's slice of W_hh (kc_total/KS chunks of 8 KB) can stay resident
    int KS = 1;
    while (KS < 4 && ((kc_total / KS) * kChunkBytesW > 128 * 1024 || jt * KS * 2 <= sms / 2) && (kc_total % (KS * 2) == 0) &&
           jt * KS * 2 <= sms)
        KS *= 2;
    if (jt * KS > sms) return set_error(FLSTM_ERR_UNSUPPORTED, "hidden size too large for the persistent BPTT kernel");
    // batch tile width as in plan_fwd: 33..64 sequences are one 64-wide tile when a CTA would otherwise take two
    int BT = (B >= 128) ? 64 : 32;
    int tiles = 0, ngroups = 0, nt = 0;
    auto split = [&](int bt) {
        tiles = (B + bt - 1) / bt;
        ngroups = sms / (jt * KS);
        if (ngroups > tiles) ngroups = tiles;
        if (ngroups < 1) ngroups = 1;
        nt = (tiles + ngroups - 1) / ngroups;
        ngroups = (tiles + nt - 1) / nt;
    };
    split(BT);
    if (nt > 1) {
        const int max_groups = sms / (jt * KS) < 1 ? 1 : sms / (jt * KS);
        const int first = BT == 32 ? 64 : 128;
        bool found = false;
        for (int bt = first; bt <= 128 && !found; bt *= 2) {
            if (bt == 64 && !(max_groups == 1 && wide_tile_enabled())) continue;
            // 128-wide tiles exist for clusters of 4 only, and pay when two or more batch groups work side by side
            if (bt == 128 && !(KS == 4 && max_groups >= 2 && wider_tile_enabled())) continue;
            split(bt);
            if (nt == 1 && ngroups == max_groups) {  // and no batch group's CTAs are left idle
                BT = bt;
                found = true;
            }
        }
        if (!found) split(BT);
    }
    const int kc_per = kc_total / KS;
    // measured on config 2: one 64 KB copy per step beats 2, 4, 8 or 16 smaller ones (TMA issue cost
    // outweighs the longer exposed UMMA tail), so a stage takes up to 16 chunks
    // (measured: the streamed-weight and multi-tile regimes need several smaller stages in flight instead)
    int ch16 = 16;
    while (kc_per % ch16) --ch16;
    const bool one_tile_resident = nt == 1 && (size_t)bwd_smem_layout(BT, H, KS, true, kc_per / ch16, ch16).total <= smem_limit;
    int ch = one_tile_resident ? 16 : 4;
    if (const char *env = std::getenv("FLSTM_CH")) ch = std::atoi(env) > 0 ? std::atoi(env) : ch;
    while (kc_per % ch) --ch;
    bool resident = true;
    int stages = kc_per / ch;
    BwdSmemLayout l = bwd_smem_layout(BT, H, KS, true, stages, ch);
    while ((size_t)l.total > smem_limit && stages > 2) l = bwd_smem_layout(BT, H, KS, true, --stages, ch);
    if ((size_t)l.total > smem_limit || (stages < 2 && kc_per / ch >= 2)) {
        resident = false;
        stages = kc_per / ch < 4 ? kc_per / ch : 4;
        l = bwd_smem_layout(BT, H, KS, false, stages, ch);
        while ((size_t)l.total > smem_limit && stages > 1) l = bwd_smem_layout(BT, H, KS, false, --stages, ch);
        // a single stage cannot overlap the copy with the UMMAs: rather two stages of half the chunks
        while (stages < 2 && ch > 1 && kc_per / (ch / 2) >= 2) {
            ch /= 2;
            stages = 2;
            l = bwd_smem_layout(BT, H, KS, false, stages, ch);
            if ((size_t)l.total > smem_limit) stages = 1;
        }
        l = bwd_smem_layout(BT, H, KS, false, stages, ch);
        while ((size_t)l.total > smem_limit && ch > 1) {
            --ch;
            while (kc_per % ch) --ch;
            l = bwd_smem_layout(BT, H, KS, false, stages, ch);
        }
        if ((size_t)l.total > smem_limit) return set_error(FLSTM_ERR_UNSUPPORTED, "BPTT kernel does not fit shared memory");
    }
    plan->ch = ch;
    plan->BT = BT;
    plan->KS = KS;
    plan->jt = jt;
    plan->ngroups = ngroups;
    plan->nt = nt;
    plan->stages = stages;
    plan->resident = resident;
    plan->smem_bytes = l.total;
    plan->grid = jt * KS * ngroups;
    if (KS > 1 && check_device) {
        // The CTAs wait on one another, so every cluster must be resident at once: shrink the number of batch
        // groups until the occupancy query says so.  A failed query or a grid that still does not fit is a
        // planning error (the caller falls back to another path); it is never left to the bounded waits.
        for (;;) {
            const int fit = query_clusters(*plan);
            if (fit < 0)
                return set_error(FLSTM_ERR_UNSUPPORTED, "BPTT planning: the cluster occupancy query failed (clusters of %d CTAs, %d bytes of shared memory)", KS, plan->smem_bytes);
            if (fit * KS >= plan->grid) break;
            if (plan->ngroups == 1)
                return set_error(FLSTM_ERR_UNSUPPORTED, "BPTT planning: %d clusters of %d CTAs are needed at once, the device holds %d", plan->grid / KS, KS, fit);
            plan->ngroups -= 1;
            plan->nt = (tiles + plan->ngroups - 1) / plan->ngroups;
            plan->ngroups = (tiles + plan->nt - 1) / plan->nt;
            plan->grid = jt * KS * plan->ngroups;
        }
    }
    return FLSTM_OK;
}

int lstm_backward_persistent(int dtype, const BwdPlan &plan, const CUtensorMap &tm_w, const CUtensorMap &tm_dg,
                             BwdParams p, cudaStream_t s) {
    const bool bf16 = dtype == FLSTM_DTYPE_BF16;
    p.jt = plan.jt;
    p.nt = plan.nt;
    p.stages = plan.stages;
    p.ch = plan.ch;
    p.idesc = umma_idesc_f16(64, plan.BT, bf16 ? 1 : 0, /*A MN-major*/ 1, /*B K-major*/ 0);
#define FLSTM_BWD_CASE(BT_, KS_, RES_)                                                                         \
    if (plan.BT == BT_ && plan.KS == KS_ && plan.resident == RES_)                                             \
        return bf16 ? launch_bwd<BT_, KS_, RES_, true>(tm_w, tm_dg, p, plan.grid, plan.smem_bytes, s)          \
                    : launch_bwd<BT_, KS_, RES_, false>(tm_w, tm_dg, p, plan.grid, plan.smem_bytes, s);
    FLSTM_BWD_CASE(32, 1, true) FLSTM_BWD_CASE(32, 1, false) FLSTM_BWD_CASE(32, 2, true) FLSTM_BWD_CASE(32, 2, false)
    FLSTM_BWD_CASE(32, 4, true) FLSTM_BWD_CASE(32, 4, false) FLSTM_BWD_CASE(64, 1, true) FLSTM_BWD_CASE(64, 1, false)
    FLSTM_BWD_CASE(64, 2, true) FLSTM_BWD_CASE(64, 2, false) FLSTM_BWD_CASE(64, 4, true) FLSTM_BWD_CASE(64, 4, false)
    FLSTM_BWD_CASE(128, 4, true) FLSTM_BWD_CASE(128, 4, false)
#undef FLSTM_BWD_CASE
    return set_error(FLSTM_ERR_UNSUPPORTED, "no BPTT kernel for this plan");
}

}  // namespace tc
}  // namespace flstm_b200
