// Dense contractions on the 5th-generation tensor cores: D[M,N] = A * B^T (+ bias) with 16-bit
// operands and fp32 accumulation in TMEM.
//
//   warp 0   TMA producer: cp.async.bulk.tensor tiles -> shared-memory ring (mbarrier full/empty)
//   warp 1   UMMA issuer : one elected thread issues tcgen05.mma (128 x BN x 16) from shared memory
//                          descriptors into one of two TMEM accumulators; tcgen05.commit releases
//                          ring slots and publishes finished accumulators
//   warps 2-5 epilogue   : tcgen05.ld TMEM -> registers -> (bias, convert) -> global, overlapping the
//                          next tile's main loop through the second accumulator
// The grid is persistent (one CTA per SM, static round-robin over output tiles).
//
// Two tile shapes.  gemm_kernel: one CTA per 128 x BN tile (BN 128 / 256).  gemm_pair_kernel: a cluster of two
// CTAs per 256 x 256 tile (tcgen05 cta_group::2): each CTA stages 128 rows of A and 128 rows of B per K block
// (32 KB instead of the 48 KB a lone CTA needs for 128 x 256) and the pair's UMMA reads both halves of B, so the
// shared-memory traffic per FLOP -- what bounds the one-CTA kernel at about 2/3 of the tensor peak -- drops by a
// third, and so does the L2 traffic.  Every CTA loads its own halves with plain TMA copies (nothing is multicast).
// The pair kernel is used for K-major A with K >= 2048, M >= 256 and N a multiple of 256 (FLSTM_GEMM_PAIR=0 turns it
// off, =2 takes it whenever M >= 256 and N % 256 == 0).
//
// Used for (shapes at the benchmark configurations, per layer):
//   input projection  P[T*B,4H]  = X[T*B,I] W_ih^T + b      (K-major x K-major, 16-bit out)
//   input gradient    dX[T*B,I]  = dG[T*B,4H] W_ih          (K-major x K-major via W_ih^T, 16-bit out)
//   weight gradients  dW[4H,I|H] = dG^T [X|H_prev]          (MN-major x MN-major: both operands are read
//                                                            as stored, reduction dim T*B outermost; fp32 out)
// These replace the reference's CUTLASS mma.sync instantiations (src/lstm_internal.h:48-68,
// flashlstm_v2/src/gemm.cu:208-359) and its per-32-step chunked dW/dX GEMMs with beta=1
// (flashlstm_v2/src/lstm_backward.cu:1112-1171).
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
constexpr int kGemmThreads = 192;

template <int BN>
struct GemmShape {
    static constexpr int kStages = (BN == 256) ? 4 : 6;
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    // 16-bit outputs leave through TMA: each epilogue warp stages [32 rows x 128 B] tiles, double-buffered
    static constexpr int kOutTileBytes = 32 * 128;
    static constexpr int kOutBytes = 4 * 2 * kOutTileBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kOutBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

enum OutMode { OUT_F16 = 0, OUT_BF16 = 1, OUT_F32 = 2 };

template <int MODE>
__device__ __forceinline__ void store_row32(void *dst_row, int col0, const uint32_t (&acc)[32], const float *bias,
                                            int n_valid, bool accumulate = false) {
    // dst_row: start of this thread's output row; writes columns [col0, col0+32) clipped to n_valid
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]);
    if (bias) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < n_valid) v[i] += __ldg(bias + col0 + i);
    }
    if (MODE == OUT_F32) {
        float *p = static_cast<float *>(dst_row) + col0;
        if (n_valid >= 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                if (accumulate) {  // D += A B^T: partial products of successive K ranges (sequence segments)
                    const float4 old = reinterpret_cast<const float4 *>(p)[i];
                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                reinterpret_cast<float4 *>(p)[i] = o;
            }
        } else {
            for (int i = 0; i < 32 && i < n_valid; ++i) p[i] = accumulate ? p[i] + v[i] : v[i];
        }
    } else {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (MODE == OUT_F16) {
                __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                packed[i] = *reinterpret_cast<uint32_t *>(&h);
            } else {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                packed[i] = *reinterpret_cast<uint32_t *>(&h);
            }
        }
        uint16_t *p = static_cast<uint16_t *>(dst_row) + col0;
        if (n_valid >= 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4 *>(p)[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        } else {
            for (int i = 0; i < 32 && i < n_valid; ++i)
                p[i] = (i & 1) ? (uint16_t)(packed[i >> 1] >> 16) : (uint16_t)(packed[i >> 1] & 0xFFFF);
        }
    }
}

// 64 accumulator columns of one output row -> 16-bit, into row r of a [32 x 128 B] staging tile laid out
// the way a 128B-swizzled TMA store expects it (16-byte chunk j of row r at chunk j ^ (r & 7)).
template <int MODE>
__device__ __forceinline__ void stage_row64(uint8_t *tile, int r, const uint32_t (&acc)[64], const float *bias, int col0,
                                            int n_valid) {
    uint8_t *row = tile + r * 128;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc[8 * j + i]);
        if (bias) {
            if (n_valid >= 64) {
                const float4 b0 = __ldg(reinterpret_cast<const float4 *>(bias + col0 + 8 * j));
                const float4 b1 = __ldg(reinterpret_cast<const float4 *>(bias + col0 + 8 * j + 4));
                v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (8 * j + i < n_valid) v[i] += __ldg(bias + col0 + 8 * j + i);
            }
        }
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (MODE == OUT_F16) {
                __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t *>(&h);
            } else {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t *>(&h);
            }
        }
        *reinterpret_cast<uint4 *>(row + ((j ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// Output rows may be written through the inverse of the tile-interleaved gate order: row
// r' = ((u/16)*4 + g)*16 + u%16 of the product goes to row g*H + u of D (unperm_h = H, else 0).
__device__ __forceinline__ int unpermute_gate_row(int r, int H) {
    const int tile = r >> 6, g = (r >> 4) & 3, u = r & 15;
    return g * H + tile * 16 + u;
}

// TMA_OUT (16-bit outputs with a 16-byte aligned D and row pitch): tm_d maps D as (M, N) with 32 x 64 boxes.
template <int BN, int MODE, bool HAS_BIAS, bool A_MN, bool B_MN, bool TMA_OUT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
            const __grid_constant__ CUtensorMap tm_d, void *__restrict__ D,
            size_t ldd, const float *__restrict__ bias, int M, int N, int K, uint32_t idesc, int unperm_h,
            unsigned int *__restrict__ err_word, int accumulate) {
    using S = GemmShape<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *s_out = smem + S::kStages * S::kStageBytes;  // 1024-aligned: stage sizes are multiples of 1024
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_out + S::kOutBytes);
    uint64_t *full = bars, *empty = bars + S::kStages;
    uint64_t *tfull = bars + 2 * S::kStages, *tempty = tfull + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + 2);
    volatile uint32_t *abort_w = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        if (TMA_OUT) tma_prefetch_desc(&tm_d);
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

    const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN;
    const int tiles = num_m * num_n, kblocks = (K + BK - 1) / BK;

    if (warp == 0) {
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
                const int m0 = (tile / num_n) * BM, n0 = (tile % num_n) * BN;
                bool ok = true;
                for (int kb = 0; kb < kblocks && ok; ++kb) {
                    ok = mbar_wait(&empty[stage], phase ^ 1, abort_w);
                    if (!ok) break;
                    uint8_t *sa = smem + stage * S::kStageBytes, *sb = sa + S::kABytes;
                    mbar_expect_tx(&full[stage], S::kStageBytes);
                    if (!A_MN) {
                        tma_load_2d(sa, &tm_a, kb * BK, m0, &full[stage]);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tm_a, m0 + j * 64, kb * BK, &full[stage]);
                    }
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
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait(&full[stage], phase, abort_w);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t a_base = smem_u32(smem + stage * S::kStageBytes), b_base = a_base + S::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t da = A_MN ? umma_desc_mnmajor_sw128(a_base + k * 2048, 8192)
                                                 : umma_desc_kmajor_sw128(a_base + k * 32);
                        const uint64_t db = B_MN ? umma_desc_mnmajor_sw128(b_base + k * 2048, 8192)
                                                 : umma_desc_kmajor_sw128(b_base + k * 32);
                        umma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
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
        int it = 0, out_idx = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            const uint32_t bphase = (it >> 1) & 1;
            const int m0 = (tile / num_n) * BM, n0 = (tile % num_n) * BN;
            if (!mbar_wait(&tfull[buf], bphase, abort_w)) break;
            tcgen05_fence_after();
            const int row = m0 + q * 32 + lane;
            if (TMA_OUT) {
                const int row0 = m0 + q * 32;
#pragma unroll 1
                for (int c = 0; c < BN; c += 64) {
                    uint32_t acc[64];
                    tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
                    tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
                    tmem_ld_wait();
                    if (c + 64 >= BN) {  // accumulator drained: the UMMA warp may start the tile after next
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tempty[buf]);
                    }
                    const int n_valid = N - (n0 + c);
                    if (row0 >= M || n_valid <= 0) continue;
                    uint8_t *tile = s_out + (q * 2 + (out_idx & 1)) * S::kOutTileBytes;
                    if (lane == 0) tma_store_wait_read<1>();  // the store that last used this buffer has read it
                    __syncwarp();
                    stage_row64<MODE>(tile, lane, acc, HAS_BIAS ? bias : nullptr, n0 + c, n_valid);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tm_d, tile, n0 + c, row0);
                        tma_store_commit();
                    }
                    ++out_idx;
                }
                continue;
            }
            const size_t esz = (MODE == OUT_F32) ? 4 : 2;
            const int out_row = (unperm_h && row < M) ? unpermute_gate_row(row, unperm_h) : row;
            char *dst_row = static_cast<char *>(D) + (size_t)out_row * ldd * esz;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t acc[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c, acc);
                tmem_ld_wait();
                const int n_valid = N - (n0 + c);
                if (row < M && n_valid > 0)
                    store_row32<MODE>(dst_row, n0 + c, acc, HAS_BIAS ? bias : nullptr, n_valid, MODE == OUT_F32 && accumulate);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[buf]);
        }
        if (TMA_OUT && lane == 0) tma_store_wait_all<0>();
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, S::kTmemCols);
    if (threadIdx.x == 0 && *abort_w) atomicExch(err_word, 1u);
}

// ------------------------------------------------------------------ CTA-pair kernel (256 x 256 tiles)
struct PairShape {
    static constexpr int kBN = 256;         // tile width; each CTA stages kBN / 2 rows of B
    static constexpr int kStages = 6;
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = (kBN / 2) * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;  // per CTA
    static constexpr int kTmemCols = 2 * kBN;
    static constexpr int kOutTileBytes = 32 * 128;
    static constexpr int kOutBytes = 4 * 2 * kOutTileBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kOutBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// Roles as in gemm_kernel, in both CTAs of the pair, except that only the leader's warp 1 issues UMMAs.
// Barriers (same offsets in both CTAs):
//   full[s]   leader only: 1 arrival (its expect_tx) + the bytes of BOTH CTAs' loads of stage s
//   empty[s]  each CTA: 1 arrival = the leader's commit after the UMMAs that read stage s
//   tfull[b]  each CTA: 1 arrival = the leader's commit after the last UMMA of a tile (accumulator b complete)
//   tempty[b] leader only: 8 arrivals = the four epilogue warps of both CTAs have drained accumulator b
template <int MODE, bool HAS_BIAS, bool A_MN, bool B_MN, bool TMA_OUT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_d, void *__restrict__ D, size_t ldd,
                 const float *__restrict__ bias, int M, int N, int K, uint32_t idesc, int unperm_h,
                 unsigned int *__restrict__ err_word, int accumulate) {
    using S = PairShape;
    constexpr int BN = S::kBN, BNH = S::kBN / 2;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *s_out = smem + S::kStages * S::kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_out + S::kOutBytes);
    uint64_t *full = bars, *empty = bars + S::kStages;
    uint64_t *tfull = bars + 2 * S::kStages, *tempty = tfull + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + 2);
    volatile uint32_t *abort_w = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    if (threadIdx.x == 0) {
        if (TMA_OUT) tma_prefetch_desc(&tm_d);
        for (int i = 0; i < S::kStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], 8);
        }
        *abort_w = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, S::kTmemCols);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers and tensor memory exist before anything crosses the pair
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_m = (M + 2 * BM - 1) / (2 * BM), num_n = N / BN;
    const int tiles = num_m * num_n, kblocks = (K + BK - 1) / BK;

    if (warp == 0) {
        if (elect_one()) {
            const uint32_t full0 = map_to_rank(smem_u32(full), 0);  // the leader's "operands landed" barriers
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = pair; tile < tiles; tile += npairs) {
                const int m0 = (tile / num_n) * 2 * BM + (int)rank * BM, n0 = (tile % num_n) * BN + (int)rank * BNH;
                bool ok = true;
                for (int kb = 0; kb < kblocks && ok; ++kb) {
                    ok = mbar_wait(&empty[stage], phase ^ 1, abort_w);
                    if (!ok) break;
                    uint8_t *sa = smem + stage * S::kStageBytes, *sb = sa + S::kABytes;
                    const uint32_t bar = full0 + 8u * (uint32_t)stage;
                    if (leader) mbar_expect_tx(&full[stage], 2 * S::kStageBytes);
                    if (!A_MN) {
                        tma_load_2d_pair(sa, &tm_a, kb * BK, m0, bar);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tm_a, m0 + j * 64, kb * BK, bar);
                    }
                    if (!B_MN) {
                        tma_load_2d_pair(sb, &tm_b, kb * BK, n0, bar);
                    } else {
#pragma unroll
                        for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tm_b, n0 + j * 64, kb * BK, bar);
                    }
                    if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (leader && elect_one()) {
            const uint32_t empty_l = smem_u32(empty), tfull_l = smem_u32(tfull);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            for (int tile = pair; tile < tiles; tile += npairs, ++it) {
                const int buf = it & 1;
                const uint32_t bphase = (it >> 1) & 1;
                if (!mbar_wait_cluster(&tempty[buf], bphase ^ 1, abort_w)) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                bool ok = true;
                for (int kb = 0; kb < kblocks; ++kb) {
                    ok = mbar_wait(&full[stage], phase, abort_w);
                    if (!ok) break;
                    tcgen05_fence_after();
                    const uint32_t a_base = smem_u32(smem + stage * S::kStageBytes), b_base = a_base + S::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t da = A_MN ? umma_desc_mnmajor_sw128(a_base + k * 2048, 8192)
                                                 : umma_desc_kmajor_sw128(a_base + k * 32);
                        const uint64_t db = B_MN ? umma_desc_mnmajor_sw128(b_base + k * 2048, 8192)
                                                 : umma_desc_kmajor_sw128(b_base + k * 32);
                        umma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0);
                    }
                    // the stage may be refilled in both CTAs once these UMMAs have read it
                    umma_commit_pair_both(empty_l + 8u * (uint32_t)stage);
                    if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair_both(tfull_l + 8u * (uint32_t)buf);
            }
        }
    } else {
        const int q = warp & 3;  // TMEM lane quadrant this warp may access
        const uint32_t tempty0 = map_to_rank(smem_u32(tempty), 0);
        int it = 0, out_idx = 0;
        for (int tile = pair; tile < tiles; tile += npairs, ++it) {
            const int buf = it & 1;
            const uint32_t bphase = (it >> 1) & 1;
            const int m0 = (tile / num_n) * 2 * BM + (int)rank * BM, n0 = (tile % num_n) * BN;
            if (!mbar_wait(&tfull[buf], bphase, abort_w)) break;
            tcgen05_fence_after();
            const int row = m0 + q * 32 + lane;
            if (TMA_OUT) {
                const int row0 = m0 + q * 32;
#pragma unroll 1
                for (int c = 0; c < BN; c += 64) {
                    uint32_t acc[64];
                    tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
                    tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
                    tmem_ld_wait();
                    if (c + 64 >= BN) {  // accumulator drained: the leader may start the tile after next
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8u * (uint32_t)buf);
                    }
                    const int n_valid = N - (n0 + c);
                    if (row0 >= M || n_valid <= 0) continue;
                    uint8_t *tile_s = s_out + (q * 2 + (out_idx & 1)) * S::kOutTileBytes;
                    if (lane == 0) tma_store_wait_read<1>();  // the store that last used this buffer has read it
                    __syncwarp();
                    stage_row64<MODE>(tile_s, lane, acc, HAS_BIAS ? bias : nullptr, n0 + c, n_valid);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tm_d, tile_s, n0 + c, row0);
                        tma_store_commit();
                    }
                    ++out_idx;
                }
                continue;
            }
            const size_t esz = (MODE == OUT_F32) ? 4 : 2;
            const int out_row = (unperm_h && row < M) ? unpermute_gate_row(row, unperm_h) : row;
            char *dst_row = static_cast<char *>(D) + (size_t)out_row * ldd * esz;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t acc[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c, acc);
                tmem_ld_wait();
                const int n_valid = N - (n0 + c);
                if (row < M && n_valid > 0)
                    store_row32<MODE>(dst_row, n0 + c, acc, HAS_BIAS ? bias : nullptr, n_valid, MODE == OUT_F32 && accumulate);
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8u * (uint32_t)buf);
        }
        if (TMA_OUT && lane == 0) tma_store_wait_all<0>();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's shared and tensor memory stay valid until the leader's last UMMA is consumed
    if (warp == 1) tmem_dealloc_pair(tmem_base, S::kTmemCols);
    if (threadIdx.x == 0 && *abort_w) atomicExch(err_word, 1u);
}

struct GemmArgs {
    CUtensorMap ta, tb, td;
    bool tma_out;
    void *D;
    size_t ldd;
    const float *bias;
    int M, N, K;
    uint32_t idesc;
    int unperm_h;
    unsigned int *err;
    int sms;
    int accumulate;
    cudaStream_t s;
    bool pair;  // 256 x 256 tiles on CTA pairs (gemm_pair_kernel)
};

// FLSTM_GEMM_PAIR: 0 = never, 2 = whenever the shape allows (tests), otherwise by the measured rule in gemm().
// Read on every call, so a test can switch it inside one process.
bool pair_enabled() {
    const char *env = std::getenv("FLSTM_GEMM_PAIR");
    return !(env && env[0] == '0');
}
bool pair_forced() {
    const char *env = std::getenv("FLSTM_GEMM_PAIR");
    return env && env[0] == '2';
}

template <int BN, int MODE, bool HAS_BIAS, bool A_MN, bool B_MN, bool TMA_OUT>
int launch_one(const GemmArgs &g) {
    using S = GemmShape<BN>;
    auto kern = gemm_kernel<BN, MODE, HAS_BIAS, A_MN, B_MN, TMA_OUT>;
    FLSTM_CUDA_TRY(ensure_smem_limit(kern, (size_t)S::kSmemBytes));
    const int tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
    const int grid = tiles < g.sms ? tiles : g.sms;
    kern<<<grid, kGemmThreads, S::kSmemBytes, g.s>>>(g.ta, g.tb, g.td, g.D, g.ldd, g.bias, g.M, g.N, g.K, g.idesc,
                                                    g.unperm_h, g.err, g.accumulate);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "tc gemm launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

template <int MODE, bool HAS_BIAS, bool A_MN, bool B_MN, bool TMA_OUT>
int launch_pair_one(const GemmArgs &g) {
    using S = PairShape;
    auto kern = gemm_pair_kernel<MODE, HAS_BIAS, A_MN, B_MN, TMA_OUT>;
    FLSTM_CUDA_TRY(ensure_smem_limit(kern, (size_t)S::kSmemBytes));
    const int tiles = ((g.M + 2 * BM - 1) / (2 * BM)) * (g.N / S::kBN);
    const int pairs = tiles < g.sms / 2 ? tiles : g.sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = S::kSmemBytes;
    cfg.stream = g.s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, g.ta, g.tb, g.td, g.D, g.ldd, g.bias, g.M, g.N, g.K, g.idesc, g.unperm_h,
                                       g.err, g.accumulate);
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "tc pair gemm launch failed: %s", cudaGetErrorString(e));
    return FLSTM_OK;
}

template <int MODE, bool HAS_BIAS, bool A_MN, bool B_MN>
int launch_pair(const GemmArgs &g) {
    if (MODE != OUT_F32 && g.tma_out) return launch_pair_one<MODE, HAS_BIAS, A_MN, B_MN, (MODE != OUT_F32)>(g);
    return launch_pair_one<MODE, HAS_BIAS, A_MN, B_MN, false>(g);
}

template <int BN, int MODE, bool HAS_BIAS, bool A_MN, bool B_MN>
int launch(const GemmArgs &g) {
    if (g.pair) return launch_pair<MODE, HAS_BIAS, A_MN, B_MN>(g);
    if (MODE != OUT_F32 && g.tma_out) return launch_one<BN, MODE, HAS_BIAS, A_MN, B_MN, (MODE != OUT_F32)>(g);
    return launch_one<BN, MODE, HAS_BIAS, A_MN, B_MN, false>(g);
}

template <int BN>
int dispatch(int out_dtype, bool a_mn, bool b_mn, const GemmArgs &g) {
    const bool has_bias = g.bias != nullptr;
    if (a_mn && b_mn) {
        if (out_dtype != FLSTM_DTYPE_F32 || has_bias)
            return set_error(FLSTM_ERR_UNSUPPORTED, "MN-major x MN-major is instantiated for fp32 output without bias");
        return launch<BN, OUT_F32, false, true, true>(g);
    }
    if (a_mn) return set_error(FLSTM_ERR_UNSUPPORTED, "MN-major A with K-major B is not instantiated");
    if (b_mn) {
        if (has_bias) return set_error(FLSTM_ERR_UNSUPPORTED, "bias with an MN-major B is not instantiated");
        switch (out_dtype) {
            case FLSTM_DTYPE_F32: return launch<BN, OUT_F32, false, false, true>(g);
            case FLSTM_DTYPE_F16: return launch<BN, OUT_F16, false, false, true>(g);
            case FLSTM_DTYPE_BF16: return launch<BN, OUT_BF16, false, false, true>(g);
        }
        return set_error(FLSTM_ERR_INVALID, "bad output dtype");
    }
    switch (out_dtype) {
        case FLSTM_DTYPE_F32:
            if (has_bias) return set_error(FLSTM_ERR_UNSUPPORTED, "bias with fp32 output is not instantiated");
            return launch<BN, OUT_F32, false, false, false>(g);
        case FLSTM_DTYPE_F16:
            return has_bias ? launch<BN, OUT_F16, true, false, false>(g) : launch<BN, OUT_F16, false, false, false>(g);
        case FLSTM_DTYPE_BF16:
            return has_bias ? launch<BN, OUT_BF16, true, false, false>(g) : launch<BN, OUT_BF16, false, false, false>(g);
    }
    return set_error(FLSTM_ERR_INVALID, "bad output dtype");
}

}  // namespace

int gemm(int dtype, int out_dtype, size_t M, size_t N, size_t K, const void *A, size_t lda, bool a_mn, const void *B,
         size_t ldb, bool b_mn, void *D, size_t ldd, const float *bias, int unperm_h, unsigned int *err_word, int sms,
         cudaStream_t s, bool accumulate) {
    if (accumulate && out_dtype != FLSTM_DTYPE_F32)
        return set_error(FLSTM_ERR_UNSUPPORTED, "accumulating GEMM output must be fp32");
    if (dtype != FLSTM_DTYPE_F16 && dtype != FLSTM_DTYPE_BF16)
        return set_error(FLSTM_ERR_UNSUPPORTED, "tensor-core GEMM operands must be f16 or bf16");
    if (M == 0 || N == 0 || K == 0) return FLSTM_OK;
    if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
        return set_error(FLSTM_ERR_UNSUPPORTED, "tensor-core GEMM needs 16-byte aligned operands and row pitches");
    const int BN = (N > 128) ? 256 : 128;
    GemmArgs g{};
    // measured on B200 (bf16) inside the engine's step: pairs win for K-major A from K = 2048 on (config 3:
    // projection 1465 -> 1529, input gradient 1507 -> 1540 TFLOP/s; 8192^3 1159 -> 1377).  With K = 1024 and the
    // bias epilogue (every projection) they lose (config 5: 12.8 -> 20.5 ms per step, 1351 -> 790 TFLOP/s in
    // isolation; without a bias the same shape gains, 1036 -> 1275), and the MN-major weight-gradient form is
    // neutral in isolation (1158 -> 1205) and 2 % slower inside the step, so both stay on lone CTAs.
    g.pair = pair_enabled() && !a_mn && K >= 2048 && M >= 256 && N % 256 == 0 && sms >= 2;
    if (pair_forced()) g.pair = M >= 256 && N % 256 == 0 && sms >= 2;
    // K-major: (rows, K) with K contiguous, box rows x 64.  MN-major: stored (K, rows), 64 x 64 boxes.
    if (!a_mn) FLSTM_TRY(make_tensor_map_2d(&g.ta, A, M, K, lda, BM, BK, true));
    else FLSTM_TRY(make_tensor_map_2d(&g.ta, A, K, M, lda, BK, 64, true));
    if (!b_mn) FLSTM_TRY(make_tensor_map_2d(&g.tb, B, N, K, ldb, g.pair ? 128 : BN, BK, true));
    else FLSTM_TRY(make_tensor_map_2d(&g.tb, B, K, N, ldb, BK, 64, true));
    // 16-bit outputs go out through TMA when D can be described by a tensor map
    g.tma_out = out_dtype != FLSTM_DTYPE_F32 && unperm_h == 0 && N >= 64 && (ldd % 8) == 0 &&
                (reinterpret_cast<uintptr_t>(D) & 15) == 0 && (reinterpret_cast<uintptr_t>(bias) & 15) == 0;
    if (const char *env = std::getenv("FLSTM_GEMM_TMA_OUT")) g.tma_out = g.tma_out && env[0] != '0';
    if (g.tma_out) FLSTM_TRY(make_tensor_map_2d(&g.td, D, M, N, ldd, 32, 64, true));
    else g.td = g.ta;  // unused
    g.D = D;
    g.ldd = ldd;
    g.bias = bias;
    g.M = (int)M;
    g.N = (int)N;
    g.K = (int)K;
    g.idesc = umma_idesc_f16(g.pair ? 2 * BM : BM, BN, dtype == FLSTM_DTYPE_BF16 ? 1 : 0, a_mn ? 1 : 0, b_mn ? 1 : 0);
    g.unperm_h = unperm_h;
    g.err = err_word;
    g.sms = sms;
    g.accumulate = accumulate ? 1 : 0;
    g.s = s;
    return BN == 256 ? dispatch<256>(out_dtype, a_mn, b_mn, g) : dispatch<128>(out_dtype, a_mn, b_mn, g);
}

// ------------------------------------------------------------------ tensor-map encoding (host)
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

}  // namespace

int make_tensor_map_2d(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint64_t row_pitch_elems,
                       uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(FLSTM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_pitch_elems * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(FLSTM_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a %llux%llu tensor, pitch %llu, box %ux%u",
                         (int)r, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)row_pitch_elems,
                         box_rows, box_cols);
    return FLSTM_OK;
}

int make_tensor_map_3d(CUtensorMap *out, const void *base, uint64_t d2, uint64_t rows, uint64_t cols,
                       uint64_t row_pitch_elems, uint64_t d2_pitch_elems, uint32_t box_rows, uint32_t box_cols,
                       bool swizzle128) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(FLSTM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {cols, rows, d2};
    cuuint64_t strides[2] = {row_pitch_elems * 2, d2_pitch_elems * 2};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(FLSTM_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed (%d)", (int)r);
    return FLSTM_OK;
}

int make_tensor_map_3d_tile(CUtensorMap *out, const void *base, int elem_bytes, uint64_t d2, uint64_t rows, uint64_t cols,
                            uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(FLSTM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const uint32_t inner = box_cols * elem_bytes;
    if (elem_bytes != 2 && elem_bytes != 4) return set_error(FLSTM_ERR_INVALID, "tensor map element size must be 2 or 4");
    if (inner != 32 && inner != 64 && inner != 128) return set_error(FLSTM_ERR_INVALID, "tile rows must be 32, 64 or 128 bytes");
    cuuint64_t dims[3] = {cols, rows, d2};
    cuuint64_t strides[2] = {cols * elem_bytes, rows * cols * elem_bytes};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle sw = inner == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : inner == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    CUresult r = fn(out, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(FLSTM_ERR_CUDA, "cuTensorMapEncodeTiled (3-D tile) failed (%d)", (int)r);
    return FLSTM_OK;
}

int make_tensor_map_chunked(CUtensorMap *out, const void *base, uint64_t steps, uint64_t rows, uint64_t width,
                            uint32_t box_rows, uint32_t chunks) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return set_error(FLSTM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {64, rows, width / 64, steps};
    cuuint64_t strides[3] = {width * 2, 128, rows * width * 2};
    cuuint32_t box[4] = {64, box_rows, chunks, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(FLSTM_ERR_CUDA, "cuTensorMapEncodeTiled (chunked) failed (%d)", (int)r);
    return FLSTM_OK;
}

}  // namespace tc
}  // namespace flstm_b200
