// CUDA-core (SIMT) kernels: the generic path of the engine.  Any shape, any storage type,
// fp32 arithmetic with true FMA (no TF32), so the fp32 configuration meets its max-abs bound.
// The tensor-core path (tc_*.cu) replaces these kernels when the shape is tile-aligned.
//
// What each kernel replaces in the reference:
//   convert / bias_sum        <- HalfToFloatKernel, FloatToHalfKernel, FuseBiasKernel
//                                (flashlstm_v2/src/lstm_forward.cu:164-217), combine_bias_kernel
//                                (src/kernels.cu:45-55)
//   gemm                      <- the CUTLASS GemmTN/NN/NT wrappers (flashlstm_v2/src/gemm.cu:208-359)
//   step_forward              <- per-step GEMM + ForwardPointwiseKernel
//                                (flashlstm_v2/src/lstm_forward.cu:322-405,785-797), fused into one launch
//   step_backward / final_dh  <- BackwardPointwiseKernel + GemmNN dh
//                                (flashlstm_v2/src/lstm_backward.cu:158-227,1084-1096), fused; the cell
//                                state is read from the cache instead of being reconstructed
//   column_sum                <- the ones-vector GEMV for db (flashlstm_v2/src/lstm_backward.cu:1144-1156)
#include "common.cuh"
#include "kernels.h"

namespace flstm_b200 {
namespace simt {

namespace {

template <typename TI, typename TO>
__global__ void convert_kernel(const TI *__restrict__ src, TO *__restrict__ dst, size_t n) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) st(dst + i, ld(src + i));
}

__global__ void bias_sum_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                float *__restrict__ out, size_t n) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}

template <typename TI, typename TO>
__global__ void gather_slabs_kernel(const TI *__restrict__ src, size_t slab, size_t stride_slabs,
                                    size_t count, TO *__restrict__ dst) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    size_t total = slab * count;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        size_t k = i / slab, e = i % slab;
        st(dst + i, ld(src + k * stride_slabs * slab + e));
    }
}

// ---------------------------------------------------------------- tiled fp32-accumulate GEMM
constexpr int BM = 64, BN = 64, BK = 16;

template <typename TAB, typename TC, bool A_KC, bool B_KC>
__global__ void __launch_bounds__(256)
gemm_kernel(int M, int N, int K_total, const TAB *__restrict__ A, size_t lda, const TAB *__restrict__ B,
            size_t ldb, TC *__restrict__ C, size_t ldc, const float *__restrict__ bias, int k_per_split,
            size_t c_split_stride) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    // split K: block z contracts over [z * k_per_split, ...) and writes its own partial product
    const int kz0 = blockIdx.z * k_per_split;
    const int K = (kz0 + k_per_split < K_total) ? kz0 + k_per_split : K_total;
    C += (size_t)blockIdx.z * c_split_stride;
    float acc[4][4] = {};
    for (int k0 = kz0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int e = tid + i * 256;
            int m, k;
            if (A_KC) { m = e / BK; k = e % BK; } else { k = e / BM; m = e % BM; }
            int gm = m0 + m, gk = k0 + k;
            float v = 0.f;
            if (gm < M && gk < K) v = A_KC ? ld(A + (size_t)gm * lda + gk) : ld(A + (size_t)gk * lda + gm);
            As[k][m] = v;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int e = tid + i * 256;
            int n, k;
            if (B_KC) { n = e / BK; k = e % BK; } else { k = e / BN; n = e % BN; }
            int gn = n0 + n, gk = k0 + k;
            float v = 0.f;
            if (gn < N && gk < K) v = B_KC ? ld(B + (size_t)gn * ldb + gk) : ld(B + (size_t)gk * ldb + gn);
            Bs[k][n] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j] + (bias ? bias[gn] : 0.f);
            st(C + (size_t)gm * ldc + gn, v);
        }
    }
}

// ---------------------------------------------------------------- fused forward step
// CTA tile: 8 sequences x 8 hidden units; four consecutive lanes hold the four gate sums of one
// (sequence, unit) pair, so a launch has (H/8) x (B/8) CTAs (128 for H = 256, B = 32: every SM has one) and
// a thread's dot product is H long.  Lane 0 of each quad gathers the gates and does the pointwise update.
constexpr int SB = 8, SU = 8, SK = 64;

template <typename T>
__global__ void __launch_bounds__(256)
step_forward_kernel(int B, int H, const T *__restrict__ h_prev, const T *__restrict__ w_hh,
                    T *__restrict__ p_t, const float *__restrict__ c_prev, float *__restrict__ c_next,
                    T *__restrict__ h_next, T *__restrict__ y_t) {
    __shared__ float hs[SB][SK + 1];
    __shared__ float ws[4 * SU][SK + 1];  // row = unit * 4 + gate
    const int tid = threadIdx.x;
    const int g = tid & 3, ul = (tid >> 2) % SU, bl = tid / (4 * SU);
    const int u0 = blockIdx.x * SU, b0 = blockIdx.y * SB;
    float acc = 0.f;
    for (int k0 = 0; k0 < H; k0 += SK) {
        for (int e = tid; e < SB * SK; e += 256) {
            int b = e / SK, k = e % SK;
            hs[b][k] = (b0 + b < B && k0 + k < H) ? ld(h_prev + (size_t)(b0 + b) * H + k0 + k) : 0.f;
        }
        for (int e = tid; e < 4 * SU * SK; e += 256) {
            int k = e % SK, r = e / SK, u = r >> 2, gg = r & 3;
            ws[r][k] = (u0 + u < H && k0 + k < H) ? ld(w_hh + ((size_t)gg * H + u0 + u) * H + k0 + k) : 0.f;
        }
        __syncthreads();
        const float *hrow = hs[bl], *wrow = ws[ul * 4 + g];
#pragma unroll 16
        for (int k = 0; k < SK; ++k) acc = fmaf(hrow[k], wrow[k], acc);
        __syncthreads();
    }
    // the quad's four gate sums -> its first lane
    const unsigned full = 0xffffffffu;
    const int base = (tid & 31) & ~3;
    const float s_i = __shfl_sync(full, acc, base), s_f = __shfl_sync(full, acc, base + 1);
    const float s_g = __shfl_sync(full, acc, base + 2), s_o = __shfl_sync(full, acc, base + 3);
    const int b = b0 + bl, u = u0 + ul;
    if (g != 0 || b >= B || u >= H) return;
    T *row = p_t + (size_t)b * 4 * H;
    float ai = s_i + ld(row + u);
    float af = s_f + ld(row + H + u);
    float ag = s_g + ld(row + 2 * H + u);
    float ao = s_o + ld(row + 3 * H + u);
    float gi = sigmoid_acc(ai), gf = sigmoid_acc(af), gg = tanh_acc(ag), go = sigmoid_acc(ao);
    size_t idx = (size_t)b * H + u;
    float c = fmaf(gf, c_prev[idx], gi * gg);
    float h = go * tanh_acc(c);
    st(row + u, gi);
    st(row + H + u, gf);
    st(row + 2 * H + u, gg);
    st(row + 3 * H + u, go);
    c_next[idx] = c;
    st(h_next + idx, h);
    if (y_t) st(y_t + idx, h);
}

// ---------------------------------------------------------------- fused backward step
// dh[b,u] = dy_t[b,u] + sum_k dg_next[b,k] w_hh[k,u]  (k over 4H), then pointwise backward.
// Same 8 x 8 tile; the four lanes of a quad split the 4H-long sum (k = lane, lane + 4, ...) and add up with
// shuffles.  When FINAL, only the matrix product is formed and written to dh_out (fp32).
template <typename T, bool FINAL>
__global__ void __launch_bounds__(256)
step_backward_kernel(int B, int H, const T *__restrict__ dg_next, const T *__restrict__ w_hh,
                     const T *__restrict__ dh_init, const T *__restrict__ dy_t,
                     const T *__restrict__ gates_t, const float *__restrict__ c_t,
                     const float *__restrict__ c_prev, float *__restrict__ dc, T *__restrict__ dg_t,
                     float *__restrict__ dh_out) {
    constexpr int BK2 = 128;
    __shared__ float ds[SB][BK2 + 1];
    __shared__ float ws[BK2][SU + 1];
    const int tid = threadIdx.x;
    const int q = tid & 3, ul = (tid >> 2) % SU, bl = tid / (4 * SU);
    const int u0 = blockIdx.x * SU, b0 = blockIdx.y * SB;
    const int G = 4 * H;
    float acc = 0.f;
    if (dg_next) {
        for (int k0 = 0; k0 < G; k0 += BK2) {
            for (int e = tid; e < SB * BK2; e += 256) {
                int b = e / BK2, k = e % BK2;
                ds[b][k] = (b0 + b < B && k0 + k < G) ? ld(dg_next + (size_t)(b0 + b) * G + k0 + k) : 0.f;
            }
            for (int e = tid; e < BK2 * SU; e += 256) {
                int u = e % SU, k = e / SU;
                ws[k][u] = (u0 + u < H && k0 + k < G) ? ld(w_hh + (size_t)(k0 + k) * H + u0 + u) : 0.f;
            }
            __syncthreads();
#pragma unroll 8
            for (int k = q; k < BK2; k += 4) acc = fmaf(ds[bl][k], ws[k][ul], acc);
            __syncthreads();
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    }
    const int b = b0 + bl, u = u0 + ul;
    if (q != 0 || b >= B || u >= H) return;
    const size_t idx = (size_t)b * H + u;
    if (FINAL) {
        dh_out[idx] = acc;
        return;
    }
    float dh = acc + ld(dy_t + idx);
    if (!dg_next && dh_init) dh += ld(dh_init + idx);
    const T *grow = gates_t + (size_t)b * G;
    float gi = ld(grow + u), gf = ld(grow + H + u), gg = ld(grow + 2 * H + u), go = ld(grow + 3 * H + u);
    float tc = tanh_acc(c_t[idx]);
    float d_o = dh * tc;
    float dcv = dc[idx] + dh * go * (1.f - tc * tc);
    float dai = dcv * gg * gi * (1.f - gi);
    float daf = dcv * c_prev[idx] * gf * (1.f - gf);
    float dag = dcv * gi * (1.f - gg * gg);
    float dao = d_o * go * (1.f - go);
    dc[idx] = dcv * gf;
    T *drow = dg_t + (size_t)b * G;
    st(drow + u, dai);
    st(drow + H + u, daf);
    st(drow + 2 * H + u, dag);
    st(drow + 3 * H + u, dao);
}

// ---------------------------------------------------------------- column sum (bias gradient)
template <typename T>
__global__ void __launch_bounds__(256)
column_sum_kernel(const T *__restrict__ dg, size_t R, size_t N, float *__restrict__ out) {
    __shared__ float part[8][33];
    const int cl = threadIdx.x % 32, rl = threadIdx.x / 32;
    const size_t col = (size_t)blockIdx.x * 32 + cl;
    float s = 0.f;
    if (col < N)
        for (size_t r = rl; r < R; r += 8) s += ld(dg + r * N + col);
    part[rl][cl] = s;
    __syncthreads();
    if (rl == 0 && col < N) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += part[i][cl];
        out[col] = t;
    }
}

// Two-pass form for tall matrices: pass 1 sums a slice of the rows per block into
// partial[split][col]; pass 2 adds the splits in a fixed order (deterministic).
template <typename T>
__global__ void __launch_bounds__(256)
column_sum_partial_kernel(const T *__restrict__ dg, size_t R, size_t N, int splits, float *__restrict__ partial) {
    __shared__ float part[8][33];
    const int cl = threadIdx.x % 32, rl = threadIdx.x / 32;
    const size_t col = (size_t)blockIdx.x * 32 + cl;
    const size_t rows_per = (R + splits - 1) / splits;
    const size_t r0 = (size_t)blockIdx.y * rows_per;
    const size_t r1 = r0 + rows_per < R ? r0 + rows_per : R;
    float s = 0.f;
    if (col < N)
        for (size_t r = r0 + rl; r < r1; r += 8) s += ld(dg + r * N + col);
    part[rl][cl] = s;
    __syncthreads();
    if (rl == 0 && col < N) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += part[i][cl];
        partial[(size_t)blockIdx.y * N + col] = t;
    }
}

__global__ void column_sum_final_kernel(const float *__restrict__ partial, size_t N, int splits, float *__restrict__ out,
                                        int unperm_h, int accumulate) {
    const size_t col = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (col >= N) return;
    float t = 0.f;
    for (int s = 0; s < splits; ++s) t += partial[(size_t)s * N + col];
    size_t o = col;
    if (unperm_h) {  // tile-interleaved gate order -> torch order
        const int r = (int)col, tile = r >> 6, g = (r >> 4) & 3, u = r & 15;
        o = (size_t)g * unperm_h + tile * 16 + u;
    }
    out[o] = accumulate ? out[o] + t : t;
}

inline int grid_1d(size_t n, int block = 256, int cap = 148 * 16) {
    size_t g = (n + block - 1) / block;
    if (g < 1) g = 1;
    return (int)(g > (size_t)cap ? cap : g);
}

inline int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FLSTM_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
    return FLSTM_OK;
}

template <typename TI>
int convert_from(const TI *src, int dst_dtype, void *dst, size_t n, cudaStream_t s) {
    int g = grid_1d(n);
    switch (dst_dtype) {
        case FLSTM_DTYPE_F32: convert_kernel<<<g, 256, 0, s>>>(src, (float *)dst, n); break;
        case FLSTM_DTYPE_F16: convert_kernel<<<g, 256, 0, s>>>(src, (__half *)dst, n); break;
        case FLSTM_DTYPE_BF16: convert_kernel<<<g, 256, 0, s>>>(src, (__nv_bfloat16 *)dst, n); break;
        default: return set_error(FLSTM_ERR_INVALID, "convert: bad dtype %d", dst_dtype);
    }
    return check_launch("convert");
}

template <typename TI>
int gather_from(const TI *src, size_t slab, size_t stride, size_t count, int dst_dtype, void *dst, cudaStream_t s) {
    int g = grid_1d(slab * count);
    switch (dst_dtype) {
        case FLSTM_DTYPE_F32: gather_slabs_kernel<<<g, 256, 0, s>>>(src, slab, stride, count, (float *)dst); break;
        case FLSTM_DTYPE_F16: gather_slabs_kernel<<<g, 256, 0, s>>>(src, slab, stride, count, (__half *)dst); break;
        case FLSTM_DTYPE_BF16: gather_slabs_kernel<<<g, 256, 0, s>>>(src, slab, stride, count, (__nv_bfloat16 *)dst); break;
        default: return set_error(FLSTM_ERR_INVALID, "gather: bad dtype %d", dst_dtype);
    }
    return check_launch("gather_slabs");
}

__global__ void sum_splits_kernel(const float *__restrict__ parts, int splits, size_t M, size_t N, float *__restrict__ C,
                                  size_t ldc) {
    const size_t total = M * N;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int z = 0; z < splits; ++z) v += parts[(size_t)z * total + i];  // fixed order: deterministic
        C[(i / N) * ldc + i % N] = v;
    }
}

template <typename TAB, typename TC>
int gemm_typed(size_t M, size_t N, size_t K, const TAB *A, size_t lda, bool akc, const TAB *B, size_t ldb,
               bool bkc, TC *C, size_t ldc, const float *bias, cudaStream_t s, int splits = 1, float *parts = nullptr) {
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM), splits);
    const int kper = splits > 1 ? (int)(((K + splits - 1) / splits + BK - 1) / BK * BK) : (int)K;
    TC *out = C;
    size_t out_ld = ldc, stride = 0;
    if (splits > 1) {  // partial products go to the scratch buffer (only instantiated for fp32 C)
        out = reinterpret_cast<TC *>(parts);
        out_ld = N;
        stride = M * N;
    }
    if (akc && bkc) gemm_kernel<TAB, TC, true, true><<<grid, 256, 0, s>>>((int)M, (int)N, (int)K, A, lda, B, ldb, out, out_ld, bias, kper, stride);
    else if (akc && !bkc) gemm_kernel<TAB, TC, true, false><<<grid, 256, 0, s>>>((int)M, (int)N, (int)K, A, lda, B, ldb, out, out_ld, bias, kper, stride);
    else if (!akc && bkc) gemm_kernel<TAB, TC, false, true><<<grid, 256, 0, s>>>((int)M, (int)N, (int)K, A, lda, B, ldb, out, out_ld, bias, kper, stride);
    else gemm_kernel<TAB, TC, false, false><<<grid, 256, 0, s>>>((int)M, (int)N, (int)K, A, lda, B, ldb, out, out_ld, bias, kper, stride);
    FLSTM_TRY(check_launch("gemm"));
    if (splits > 1) {
        sum_splits_kernel<<<grid_1d(M * N), 256, 0, s>>>(parts, splits, M, N, reinterpret_cast<float *>(C), ldc);
        return check_launch("gemm split sum");
    }
    return FLSTM_OK;
}

template <typename TAB>
int gemm_ab(int c_dtype, size_t M, size_t N, size_t K, const TAB *A, size_t lda, bool akc, const TAB *B,
            size_t ldb, bool bkc, void *C, size_t ldc, const float *bias, cudaStream_t s, float *scratch,
            size_t scratch_floats) {
    if (c_dtype == FLSTM_DTYPE_F32) {
        // long contractions with few output tiles (the weight gradients): split K over grid.z into the scratch
        // buffer, then add the partial products in a fixed order
        int splits = 1;
        const size_t tiles = (size_t)ceil_div(N, BN) * ceil_div(M, BM);
        if (scratch && !bias && K >= 1024 && tiles < 148) {
            while (splits < 8 && tiles * splits * 2 <= 296 && K / (splits * 2) >= 256 &&
                   (size_t)(splits * 2) * M * N <= scratch_floats)
                splits *= 2;
        }
        return gemm_typed(M, N, K, A, lda, akc, B, ldb, bkc, (float *)C, ldc, bias, s, splits, scratch);
    }
    // a 16-bit C has the same type as A and B
    return gemm_typed(M, N, K, A, lda, akc, B, ldb, bkc, (TAB *)C, ldc, bias, s);
}

}  // namespace

int convert(int src_dtype, const void *src, int dst_dtype, void *dst, size_t n, cudaStream_t s) {
    if (n == 0) return FLSTM_OK;
    switch (src_dtype) {
        case FLSTM_DTYPE_F32: return convert_from((const float *)src, dst_dtype, dst, n, s);
        case FLSTM_DTYPE_F16: return convert_from((const __half *)src, dst_dtype, dst, n, s);
        case FLSTM_DTYPE_BF16: return convert_from((const __nv_bfloat16 *)src, dst_dtype, dst, n, s);
    }
    return set_error(FLSTM_ERR_INVALID, "convert: bad dtype %d", src_dtype);
}

int bias_sum(const float *b_ih, const float *b_hh, float *out, size_t n, cudaStream_t s) {
    if (n == 0) return FLSTM_OK;
    bias_sum_kernel<<<ceil_div(n, 256), 256, 0, s>>>(b_ih, b_hh, out, n);
    return check_launch("bias_sum");
}

int gather_slabs(int src_dtype, const void *src, size_t slab, size_t stride, size_t count, int dst_dtype,
                 void *dst, cudaStream_t s) {
    if (slab * count == 0) return FLSTM_OK;
    switch (src_dtype) {
        case FLSTM_DTYPE_F32: return gather_from((const float *)src, slab, stride, count, dst_dtype, dst, s);
        case FLSTM_DTYPE_F16: return gather_from((const __half *)src, slab, stride, count, dst_dtype, dst, s);
        case FLSTM_DTYPE_BF16: return gather_from((const __nv_bfloat16 *)src, slab, stride, count, dst_dtype, dst, s);
    }
    return set_error(FLSTM_ERR_INVALID, "gather: bad dtype %d", src_dtype);
}

int gemm(int ab_dtype, int c_dtype, size_t M, size_t N, size_t K, const void *A, size_t lda, bool akc,
         const void *B, size_t ldb, bool bkc, void *C, size_t ldc, const float *bias, cudaStream_t s, float *scratch,
         size_t scratch_floats) {
    if (M == 0 || N == 0) return FLSTM_OK;
    if (c_dtype != FLSTM_DTYPE_F32 && c_dtype != ab_dtype)
        return set_error(FLSTM_ERR_INVALID, "gemm: C dtype must be f32 or the operand dtype");
    switch (ab_dtype) {
        case FLSTM_DTYPE_F32: return gemm_ab(c_dtype, M, N, K, (const float *)A, lda, akc, (const float *)B, ldb, bkc, C, ldc, bias, s, scratch, scratch_floats);
        case FLSTM_DTYPE_F16: return gemm_ab(c_dtype, M, N, K, (const __half *)A, lda, akc, (const __half *)B, ldb, bkc, C, ldc, bias, s, scratch, scratch_floats);
        case FLSTM_DTYPE_BF16: return gemm_ab(c_dtype, M, N, K, (const __nv_bfloat16 *)A, lda, akc, (const __nv_bfloat16 *)B, ldb, bkc, C, ldc, bias, s, scratch, scratch_floats);
    }
    return set_error(FLSTM_ERR_INVALID, "gemm: bad dtype %d", ab_dtype);
}

template <typename T>
static int step_forward_t(size_t B, size_t H, const void *h_prev, const void *w_hh, void *p_t,
                          const float *c_prev, float *c_next, void *h_next, void *y_t, cudaStream_t s) {
    dim3 grid(ceil_div(H, SU), ceil_div(B, SB));
    step_forward_kernel<T><<<grid, 256, 0, s>>>((int)B, (int)H, (const T *)h_prev, (const T *)w_hh, (T *)p_t,
                                               c_prev, c_next, (T *)h_next, (T *)y_t);
    return check_launch("step_forward");
}

int step_forward(int dtype, size_t B, size_t H, const void *h_prev, const void *w_hh, void *p_t,
                 const float *c_prev, float *c_next, void *h_next, void *y_t, cudaStream_t s) {
    switch (dtype) {
        case FLSTM_DTYPE_F32: return step_forward_t<float>(B, H, h_prev, w_hh, p_t, c_prev, c_next, h_next, y_t, s);
        case FLSTM_DTYPE_F16: return step_forward_t<__half>(B, H, h_prev, w_hh, p_t, c_prev, c_next, h_next, y_t, s);
        case FLSTM_DTYPE_BF16: return step_forward_t<__nv_bfloat16>(B, H, h_prev, w_hh, p_t, c_prev, c_next, h_next, y_t, s);
    }
    return set_error(FLSTM_ERR_INVALID, "step_forward: bad dtype %d", dtype);
}

template <typename T>
static int step_backward_t(size_t B, size_t H, const void *dg_next, const void *w_hh, const void *dh_init,
                           const void *dy_t, const void *gates_t, const float *c_t, const float *c_prev,
                           float *dc, void *dg_t, float *dh_out, bool final, cudaStream_t s) {
    dim3 grid(ceil_div(H, SU), ceil_div(B, SB));
    if (final)
        step_backward_kernel<T, true><<<grid, 256, 0, s>>>((int)B, (int)H, (const T *)dg_next, (const T *)w_hh,
                                                          nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                                          nullptr, dh_out);
    else
        step_backward_kernel<T, false><<<grid, 256, 0, s>>>((int)B, (int)H, (const T *)dg_next, (const T *)w_hh,
                                                           (const T *)dh_init, (const T *)dy_t,
                                                           (const T *)gates_t, c_t, c_prev, dc, (T *)dg_t, nullptr);
    return check_launch("step_backward");
}

int step_backward(int dtype, size_t B, size_t H, const void *dg_next, const void *w_hh, const void *dh_init,
                  const void *dy_t, const void *gates_t, const float *c_t, const float *c_prev, float *dc,
                  void *dg_t, cudaStream_t s) {
    switch (dtype) {
        case FLSTM_DTYPE_F32: return step_backward_t<float>(B, H, dg_next, w_hh, dh_init, dy_t, gates_t, c_t, c_prev, dc, dg_t, nullptr, false, s);
        case FLSTM_DTYPE_F16: return step_backward_t<__half>(B, H, dg_next, w_hh, dh_init, dy_t, gates_t, c_t, c_prev, dc, dg_t, nullptr, false, s);
        case FLSTM_DTYPE_BF16: return step_backward_t<__nv_bfloat16>(B, H, dg_next, w_hh, dh_init, dy_t, gates_t, c_t, c_prev, dc, dg_t, nullptr, false, s);
    }
    return set_error(FLSTM_ERR_INVALID, "step_backward: bad dtype %d", dtype);
}

int final_dh(int dtype, size_t B, size_t H, const void *dg0, const void *w_hh, float *dh0, cudaStream_t s) {
    switch (dtype) {
        case FLSTM_DTYPE_F32: return step_backward_t<float>(B, H, dg0, w_hh, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, dh0, true, s);
        case FLSTM_DTYPE_F16: return step_backward_t<__half>(B, H, dg0, w_hh, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, dh0, true, s);
        case FLSTM_DTYPE_BF16: return step_backward_t<__nv_bfloat16>(B, H, dg0, w_hh, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, dh0, true, s);
    }
    return set_error(FLSTM_ERR_INVALID, "final_dh: bad dtype %d", dtype);
}

int column_sum(int dtype, const void *dg, size_t R, size_t N, float *out, cudaStream_t s) {
    if (N == 0) return FLSTM_OK;
    int grid = ceil_div(N, 32);
    switch (dtype) {
        case FLSTM_DTYPE_F32: column_sum_kernel<<<grid, 256, 0, s>>>((const float *)dg, R, N, out); break;
        case FLSTM_DTYPE_F16: column_sum_kernel<<<grid, 256, 0, s>>>((const __half *)dg, R, N, out); break;
        case FLSTM_DTYPE_BF16: column_sum_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16 *)dg, R, N, out); break;
        default: return set_error(FLSTM_ERR_INVALID, "column_sum: bad dtype %d", dtype);
    }
    return check_launch("column_sum");
}

int column_sum_scratch_floats(size_t N) { return (int)(kColumnSumSplits * N); }

int column_sum_two_pass(int dtype, const void *dg, size_t R, size_t N, float *scratch, float *out, int unperm_h,
                        cudaStream_t s, bool accumulate) {
    if (N == 0) return FLSTM_OK;
    dim3 grid(ceil_div(N, 32), kColumnSumSplits);
    switch (dtype) {
        case FLSTM_DTYPE_F32: column_sum_partial_kernel<<<grid, 256, 0, s>>>((const float *)dg, R, N, kColumnSumSplits, scratch); break;
        case FLSTM_DTYPE_F16: column_sum_partial_kernel<<<grid, 256, 0, s>>>((const __half *)dg, R, N, kColumnSumSplits, scratch); break;
        case FLSTM_DTYPE_BF16: column_sum_partial_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16 *)dg, R, N, kColumnSumSplits, scratch); break;
        default: return set_error(FLSTM_ERR_INVALID, "column_sum: bad dtype %d", dtype);
    }
    FLSTM_TRY(check_launch("column_sum_partial"));
    column_sum_final_kernel<<<ceil_div(N, 256), 256, 0, s>>>(scratch, N, kColumnSumSplits, out, unperm_h, accumulate ? 1 : 0);
    return check_launch("column_sum_final");
}

}  // namespace simt
}  // namespace flstm_b200
