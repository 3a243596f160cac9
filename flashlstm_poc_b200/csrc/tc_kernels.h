// Host-side launchers of the tensor-core path kernels (tc_*.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace flstm_b200 {
namespace tc {

// D[M,N] (row pitch ldd, dtype out_dtype) = A B^T (+ bias[N]), fp32 accumulation in TMEM.
//   a_mn == false: A is (M,K) row-major with pitch lda;  a_mn == true: A is stored (K,M) with pitch lda.
//   b_mn == false: B is (N,K) row-major with pitch ldb;  b_mn == true: B is stored (K,N) with pitch ldb.
//   unperm_h != 0: output rows are written through the inverse tile-interleaved gate order (H = unperm_h).
// `err_word` is a device word the kernel sets to 1 if a bounded wait expired.
int gemm(int dtype, int out_dtype, size_t M, size_t N, size_t K, const void *A, size_t lda, bool a_mn, const void *B,
         size_t ldb, bool b_mn, void *D, size_t ldd, const float *bias, int unperm_h, unsigned int *err_word, int sms,
         cudaStream_t s, bool accumulate = false);  // accumulate (fp32 output only): D += A B^T

int device_sm_count();

// ------------------------------------------------------------------ persistent recurrent forward
struct FwdPlan {
    int BT;        // sequences per batch tile (UMMA N): 32, 64 or 128
    int rt;        // row tiles (64 gate rows = 16 hidden units x 4 gates) per CTA
    int cta_rows;  // CTAs along the row-tile axis = (H/16) / rt
    int ngroups;   // batch groups (each with its own step barrier)
    int nt;        // batch tiles per group
    int stages;    // TMA ring depth
    int ch;        // 64-wide K chunks per ring stage (one TMA copy each)
    bool resident; // W_hh slice stays in shared memory for the whole sequence
    bool pair;     // neighbouring row-tile CTAs form cta_group::2 pairs; the h map then has BT/2 rows per box
    int smem_bytes;
    int grid;
};

struct FwdParams {
    float *cs;            // fp32 (T+1, B, H) cell states, slot 0 = c0
    void *hs;             // 16-bit (T+1, B, H) hidden states, slot 0 = h0
    void *y;              // optional 16-bit (T, B, H) copy of h_t for the caller
    void *gates;          // 16-bit (T, B, 4H): holds P on entry, the activated gates on exit
    unsigned int *counters;  // one step counter per batch group, zeroed before the launch
    unsigned int *err;    // error word: non-zero after a bounded wait expired
    int T, B, H;          // T = number of steps this launch runs
    int t0;               // first (absolute) time step of this launch; the state of step t0 is in slot t0 of hs/cs
    int store_gates;      // write the activated gates back (the gate cache)
    long long *trace;     // optional: CTA 0 stamps clock64() at 16 points of each of the first trace_steps steps
    int trace_steps;
    unsigned long long wait_ns;   // limit of every device-side wait (0 = the 2 s default)
    unsigned int extra_arrivals;  // self-test of the timeout path: the step barrier waits for this many arrivals nobody makes
    // filled by the launcher from the plan
    int rt, cta_rows, nt, stages, ch;
    uint32_t idesc;
};

int plan_fwd(int B, int H, int sms, size_t smem_limit, FwdPlan *plan);
bool wide_tile_enabled();   // 33..64 sequences as one 64-wide batch tile when a CTA would otherwise take two
bool wider_tile_enabled();  // 65..128 sequences as one 128-wide batch tile likewise
// tm_w: W_hh rows tile-interleaved (4H, H), box 64x64, 128B swizzle.  tm_h: hidden states as a
// chunked map (make_tensor_map_chunked) with box rows BT (BT/2 for plan.pair) and plan.ch chunks.  tm_g: projection as
// (T, B, 4H), box 1 x BT x 64, no swizzle.
int lstm_forward_persistent(int dtype, const FwdPlan &plan, const CUtensorMap &tm_w, const CUtensorMap &tm_h,
                            const CUtensorMap &tm_g, FwdParams p, cudaStream_t s);

// ------------------------------------------------------------------ persistent BPTT
struct BwdPlan {
    int BT;        // sequences per batch tile
    int KS;        // cluster size: CTAs that split the K = 4H contraction of one 64-unit tile
    int jt;        // unit tiles = H / 64
    int ngroups, nt, stages;
    int ch;        // 64-wide K chunks per ring stage (one TMA copy each)
    bool resident;
    int smem_bytes;
    int grid;
};

struct BwdParams {
    const float *cs;      // fp32 (T+1, B, H) cell states from the forward
    const void *gates;    // 16-bit (T, B, 4H) post-activation gate cache, tile-interleaved columns
    void *dg;             // 16-bit (T, B, 4H) pre-activation gradients (written), same column order
    const void *dy;       // 16-bit (T, B, H)
    const void *dhn;      // 16-bit (B, H) or null
    const void *dcn;      // 16-bit (B, H) or null
    float *dh0, *dc0;     // fp32 (B, H) or null
    float *dc;            // fp32 (B, H) scratch for the cell-gradient carry (used when nt > 1)
    unsigned int *counters;
    unsigned int *err;
    long long *trace;     // optional per-step clock64() stamps of CTA 0 (see FwdParams)
    int trace_steps;
    int T, B, H;          // T = length of the whole sequence
    int s0, s1;           // reverse iterations [s0, s1) of this launch; iteration s is time T-1-s, s == T writes dh0/dc0
    unsigned long long wait_ns;   // limit of every device-side wait (0 = the 2 s default)
    unsigned int extra_arrivals;  // self-test of the timeout path (see FwdParams)
    int jt, nt, stages, ch;
    uint32_t idesc;
};

// check_device: verify with the occupancy query of the CURRENT device that all clusters of the grid are resident
// at once (shrinking the number of batch groups if need be) and fail when they are not; false = host arithmetic only.
int plan_bwd(int B, int H, int sms, size_t smem_limit, BwdPlan *plan, bool check_device = true);
// tm_w: the same map as the forward's (W_hh rows tile-interleaved, 64x64 boxes): the BPTT reads the
// slice as an MN-major operand.  tm_dg: dG as a chunked map (make_tensor_map_chunked) of width 4H
// with box rows BT and plan.ch chunks.
int lstm_backward_persistent(int dtype, const BwdPlan &plan, const CUtensorMap &tm_w, const CUtensorMap &tm_dg,
                             BwdParams p, cudaStream_t s);

// ------------------------------------------------------------------ wide-batch path: one GEMM launch per step
struct StepPlan {
    bool use;     // the engine takes this path instead of the persistent kernels
    int bn_fwd;   // output-tile width of the forward step GEMM (gate columns): 64, 128 or 256
    int bn_bwd;   // output-tile width of the backward step GEMM (hidden units): 128 or 256
    int splits;   // K = 4H splits of the backward step GEMM (fp32 partial sums, added by the pointwise kernel)
    bool pair;    // tiles of 256 sequences on CTA pairs (cta_group::2); the forward W_hh map then has bn_fwd / 2 rows per box
    bool bwd_pair;        // the backward split-K GEMM runs on CTA pairs (256-sequence tiles)
    bool fwd_persistent;  // forward: one cooperative launch per range of steps (lstm_wide_forward) instead of one per step
    bool fwd_pair;        // that launch runs on CTA pairs (256-sequence tiles); the forward W_hh map has bn_fwd / 2 rows per box
};

struct StepFwdParams {
    unsigned int *err;
    int t;            // absolute time step: h_{t-1} / c_{t-1} in slot t of the state tensors, results in slot t+1
    int B, H;
    int store_gates;  // overwrite the projection with the activated gates (the gate cache)
};

// Tensor maps of the forward step kernel.  Operands: hs (T+1, B, H) as a 3-D map with 1 x 128 x 64 boxes and
// W_hh (rows tile-interleaved, (4H, H)) with plan.bn_fwd x 64 boxes (plan.bn_fwd / 2 x 64 for CTA pairs), both 128B-swizzled.  Epilogue tiles
// (make_tensor_map_3d_tile, 32-row boxes): gates (T, B, 4H) 64 columns wide, cs (T+1, B, H) fp32 16 wide,
// hs_out (T+1, B, H) 16 wide, y = the caller's (T, B, H) output 16 wide or null.
struct StepFwdMaps {
    const CUtensorMap *hs, *w, *gates, *cs, *hs_out, *y;
};

// All steps [t0, t0 + nsteps) of the forward step GEMM in ONE cooperative launch: the CTAs keep their output tiles,
// a counter barrier in global memory separates the steps (same tensor maps as lstm_step_forward).
struct WideFwdParams {
    unsigned int *err;
    unsigned int *counter;  // zeroed before the launch
    int t0, nsteps;
    int B, H;
    int store_gates;
    unsigned long long wait_ns;
    unsigned int extra_arrivals;
};
int lstm_wide_forward(int dtype, const StepPlan &plan, const StepFwdMaps &m, const WideFwdParams &p, int sms, cudaStream_t s);

int plan_step(int B, int H, int sms, size_t smem_limit, StepPlan *plan);
int lstm_step_forward(int dtype, const StepPlan &plan, const StepFwdMaps &m, const StepFwdParams &p, int sms,
                      cudaStream_t s);
// parts[s] (B,H) fp32 = dG_t[:, K slice s] W_hh[K slice s, :].  tm_dg: dG (T, B, 4H) as a 3-D map, box
// 1 x 128 x 64, 128B swizzle.  tm_w64: W_hh (4H, H) with 64 x 64 boxes (read as an MN-major operand).
int lstm_step_backward_gemm(int dtype, const StepPlan &plan, const CUtensorMap &tm_dg, const CUtensorMap &tm_w64, int t,
                            int B, int H, float *parts, unsigned int *err, int sms, cudaStream_t s);
// dG_t and the cell-gradient carry from dh = dy_t + sum(parts[0..nparts)), the gate cache and the cell states.
int lstm_step_backward_pointwise(int dtype, const void *gates_t, const float *c_t, const float *c_prev, const void *dy_t,
                                 const float *parts, int nparts, float *dc, void *dg_t, int B, int H, cudaStream_t s);
int sum_parts(const float *parts, int nparts, size_t n, float *out, cudaStream_t s);

// fp32 (4H, K) torch-ordered rows -> 16-bit tile-interleaved rows; bias likewise (b_ih + b_hh)
int pack_weights_interleaved(int dtype, const float *w, size_t H, size_t K, void *out, cudaStream_t s);
int pack_bias_interleaved(const float *b_ih, const float *b_hh, size_t H, float *out, cudaStream_t s);
// out[g*H + u] = in[tile-interleaved index of (g,u)]
int unpermute_vector(const float *in, size_t H, float *out, cudaStream_t s);

}  // namespace tc
}  // namespace flstm_b200
