// Host-side launchers of every kernel in the library.  All launches are asynchronous on the
// given stream and return a flstm_status.  `dtype` is a flstm_dtype value.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>

namespace flstm_b200 {

// ------------------------------------------------------------------ generic (any shape)
namespace simt {

// dst[i] = (TOut) src[i]
int convert(int src_dtype, const void *src, int dst_dtype, void *dst, size_t n, cudaStream_t s);
// out = b_ih + b_hh (fp32, n entries)
int bias_sum(const float *b_ih, const float *b_hh, float *out, size_t n, cudaStream_t s);
// strided gather of whole (B,H) slabs: dst[k] = (dst dtype) src[k*stride_slabs] for k < count
int gather_slabs(int src_dtype, const void *src, size_t slab_elems, size_t stride_slabs, size_t count,
                 int dst_dtype, void *dst, cudaStream_t s);

// C[M,N] (row-major, ldc) = sum_k A(m,k) B(k,n) (+ bias[n]); fp32 accumulation.
//   a_kcontig: A(m,k) = A[m*lda + k]   else A(m,k) = A[k*lda + m]
//   b_kcontig: B(k,n) = B[n*ldb + k]   else B(k,n) = B[k*ldb + n]
// With a scratch buffer (fp32 C, no bias) long contractions with few output tiles are split along K into
// partial products that a second kernel adds in a fixed order.
int gemm(int ab_dtype, int c_dtype, size_t M, size_t N, size_t K, const void *A, size_t lda,
         bool a_kcontig, const void *B, size_t ldb, bool b_kcontig, void *C, size_t ldc,
         const float *bias, cudaStream_t s, float *scratch = nullptr, size_t scratch_floats = 0);

// One forward time step: gates = p_t + h_prev W_hh^T, activations, cell/hidden update.
// p_t (B,4H) holds the input projection (bias included) and is overwritten with the
// post-activation gates i,f,g,o (the gate cache).  y_t is optional.
int step_forward(int dtype, size_t B, size_t H, const void *h_prev, const void *w_hh, void *p_t,
                 const float *c_prev, float *c_next, void *h_next, void *y_t, cudaStream_t s);

// One backward time step (reverse order): dh = dy_t + dg_next W_hh (or + dh_init at the last
// step, where dg_next == nullptr), then the fused pointwise backward -> dg_t, dc (in/out).
int step_backward(int dtype, size_t B, size_t H, const void *dg_next, const void *w_hh,
                  const void *dh_init, const void *dy_t, const void *gates_t, const float *c_t,
                  const float *c_prev, float *dc, void *dg_t, cudaStream_t s);
// dh0 (fp32) = dg_0 W_hh
int final_dh(int dtype, size_t B, size_t H, const void *dg0, const void *w_hh, float *dh0, cudaStream_t s);

// ---- persistent fp32 recurrent kernels (simt_persistent.cu): one cooperative launch per layer and range
struct PersistentFwdParams {
    const void *w_hh;        // (4H, H) engine dtype, torch row order
    void *hs;                // (T+1, B, H) engine dtype; slot t0 holds the state the launch starts from
    float *cs;               // (T+1, B, H) fp32
    void *gates;             // (T, B, 4H): projection in, activated gates out (when store_gates)
    void *y;                 // optional (T, B, H) copy of h_t
    unsigned int *counters;  // one per batch tile of 8 sequences, zeroed before the launch
    unsigned int *err;       // error word (a bounded wait expired)
    int B, H;
    int t0, T;               // first step and number of steps of this launch
    int store_gates;
    unsigned long long wait_ns;   // limit of the step-barrier wait (0 = the 2 s default)
    unsigned int extra_arrivals;  // self-test of the timeout path: wait for this many arrivals nobody makes
};
struct PersistentBwdParams {
    const void *w_hh;
    const float *cs;
    const void *gates;
    void *dg;                // (T, B, 4H): written; dG_{t+1} is read back for the next iteration
    const void *dy;          // (T, B, H)
    const void *dhn;         // (B, H) or null: added at the last time step
    float *dc;               // (B, H) fp32 cell-gradient carry: read at launch start, written at its end
    float *dh0, *dc0;        // (B, H) fp32 or null, written by the iteration s == T
    unsigned int *counters, *err;
    int B, H;
    int T;                   // length of the whole sequence
    int s0, s1;              // reverse iterations [s0, s1): iteration s is time T-1-s
    unsigned long long wait_ns;   // as in PersistentFwdParams
    unsigned int extra_arrivals;
};
// whether the shape fits (shared memory for the W_hh slices, all CTAs co-resident); grid = CTAs to launch
bool persistent_fits(int dtype, size_t B, size_t H, bool training, int *grid);
int persistent_batch_tiles(size_t B);
int persistent_forward(int dtype, int grid, PersistentFwdParams p, cudaStream_t s);
int persistent_backward(int dtype, int grid, PersistentBwdParams p, cudaStream_t s);

// out[n] = sum_r dg[r, n] over R rows (deterministic order)
int column_sum(int dtype, const void *dg, size_t R, size_t N, float *out, cudaStream_t s);

// Two-pass form for tall matrices: `scratch` holds kColumnSumSplits x N fp32 partial sums (every
// entry is overwritten, nothing needs clearing).  unperm_h != 0 writes `out` in torch gate order
// from tile-interleaved columns (H = unperm_h).
constexpr int kColumnSumSplits = 32;
int column_sum_scratch_floats(size_t N);
// accumulate: out += column sums (segment-by-segment bias gradients)
int column_sum_two_pass(int dtype, const void *dg, size_t R, size_t N, float *scratch, float *out, int unperm_h,
                        cudaStream_t s, bool accumulate = false);

}  // namespace simt
}  // namespace flstm_b200
