// Forward-only v1 surface (include/flashlstm/lstm_api.h) as a shim over the engine.
//
// Mirrors the behaviour of the reference's entry points in src/lstm.cu: creation :675-858,
// destroy :860-867, execution mode :869-884, weight packing :886-931, forward :1897-2148.
// Kept: fp32 device I/O, sizes fixed at creation and re-validated per call (:1915-1917),
// precision must match (:897,1915), weights must be packed first (:1918), a longer sequence
// grows the workspace (:933-970), the handle owns a non-blocking stream (:851) and the call is
// synchronous (:2081,2146); failures return a cudaError_t value and print to stderr.
#include <cstdio>
#include <new>

#include "common.cuh"
#include "engine.h"
#include "flashlstm/lstm_api.h"
#include "kernels.h"

namespace {

using namespace flstm_b200;

struct V1Handle {
    flstm_engine *engine = nullptr;
    int precision = 0;
    int mode = LSTM_EXECUTION_MODE_GRAPH;
    int chunk = 0;
    size_t B = 0, I = 0, H = 0, t_cap = 0;
    bool packed = false;
    cudaStream_t stream = nullptr;
    // staging in the engine's 16-bit type
    void *x16 = nullptr, *y16 = nullptr, *st16 = nullptr;  // st16: h0, hn (2 slabs)
    float *w_ih = nullptr, *w_hh = nullptr;                // packed-weight snapshot (fp32)
};

int fail(int cuda_code, const char *what) {
    std::fprintf(stderr, "flashlstm: %s: %s\n", what, flstm_last_error());
    return cuda_code;
}

int misuse(const char *what) {
    std::fprintf(stderr, "flashlstm: %s\n", what);
    return (int)cudaErrorInvalidValue;
}

int to_cuda_code(int st) {
    switch (st) {
        case FLSTM_OK: return 0;
        case FLSTM_ERR_INVALID: return (int)cudaErrorInvalidValue;
        case FLSTM_ERR_UNSUPPORTED: return (int)cudaErrorNotSupported;
        default: return (int)cudaErrorUnknown;
    }
}

void free_staging(V1Handle *h) {
    if (h->x16) cudaFree(h->x16);
    if (h->y16) cudaFree(h->y16);
    h->x16 = h->y16 = nullptr;
}

int alloc_staging(V1Handle *h, size_t T) {
    free_staging(h);
    if (cudaMalloc(&h->x16, T * h->B * h->I * 2) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
    if (cudaMalloc(&h->y16, T * h->B * h->H * 2) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
    h->t_cap = T;
    return 0;
}

}  // namespace

extern "C" {

int lstm_create_buffers(lstm_compute_precision_t precision, size_t seq_len, size_t batch, size_t input_size,
                        size_t hidden_size, int input_proj_chunk_size, lstm_buffers *buffers) {
    if (!buffers) return misuse("lstm_create_buffers: buffers is null");
    buffers->impl = nullptr;
    if (precision != LSTM_COMPUTE_PRECISION_FP16_ACC32 && precision != LSTM_COMPUTE_PRECISION_FP16_ACC16)
        return misuse("lstm_create_buffers: unknown precision");
    if (seq_len == 0 || batch == 0 || input_size == 0 || hidden_size == 0 || input_proj_chunk_size < 0)
        return misuse("lstm_create_buffers: sizes must be positive");
    V1Handle *h = new (std::nothrow) V1Handle();
    if (!h) return (int)cudaErrorMemoryAllocation;
    h->precision = precision;
    h->chunk = input_proj_chunk_size;
    h->B = batch;
    h->I = input_size;
    h->H = hidden_size;
    flstm_engine_config cfg{};
    cfg.dtype = FLSTM_DTYPE_F16;
    cfg.layers = 1;
    cfg.batch = batch;
    cfg.input_size = input_size;
    cfg.hidden_size = hidden_size;
    cfg.max_seq_len = seq_len;
    cfg.training = 0;
    cfg.backend = FLSTM_BACKEND_AUTO;
    int st = flstm_engine_create(&cfg, &h->engine);
    if (st != FLSTM_OK) {
        delete h;
        return fail(to_cuda_code(st), "lstm_create_buffers");
    }
    flstm_engine_set_cell_io_f32(h->engine, 1);
    bool ok = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaMalloc(&h->st16, 2 * batch * hidden_size * 2) == cudaSuccess &&
              cudaMalloc((void **)&h->w_ih, 4 * hidden_size * input_size * sizeof(float)) == cudaSuccess &&
              cudaMalloc((void **)&h->w_hh, 4 * hidden_size * hidden_size * sizeof(float)) == cudaSuccess &&
              alloc_staging(h, seq_len) == 0;
    if (!ok) {
        lstm_buffers tmp{h};
        lstm_destroy_buffers(&tmp);
        return misuse("lstm_create_buffers: device allocation failed"), (int)cudaErrorMemoryAllocation;
    }
    buffers->impl = h;
    return 0;
}

int lstm_destroy_buffers(lstm_buffers *buffers) {
    if (!buffers || !buffers->impl) return 0;
    V1Handle *h = static_cast<V1Handle *>(buffers->impl);
    if (h->stream) cudaStreamSynchronize(h->stream);
    flstm_engine_destroy(h->engine);
    free_staging(h);
    if (h->st16) cudaFree(h->st16);
    if (h->w_ih) cudaFree(h->w_ih);
    if (h->w_hh) cudaFree(h->w_hh);
    if (h->stream) cudaStreamDestroy(h->stream);
    delete h;
    buffers->impl = nullptr;
    return 0;
}

int lstm_set_execution_mode(lstm_buffers *buffers, lstm_execution_mode_t mode) {
    if (!buffers || !buffers->impl) return misuse("lstm_set_execution_mode: handle is null");
    if (mode != LSTM_EXECUTION_MODE_IMMEDIATE && mode != LSTM_EXECUTION_MODE_GRAPH)
        return misuse("lstm_set_execution_mode: unknown mode");
    static_cast<V1Handle *>(buffers->impl)->mode = mode;
    return 0;
}

int lstm_pack_weights(lstm_compute_precision_t precision, const float *weight_ih, const float *weight_hh,
                      size_t input_size, size_t hidden_size, lstm_buffers *buffers) {
    if (!buffers || !buffers->impl) return misuse("lstm_pack_weights: handle is null");
    V1Handle *h = static_cast<V1Handle *>(buffers->impl);
    if (!weight_ih || !weight_hh) return misuse("lstm_pack_weights: weight pointer is null");
    if ((int)precision != h->precision) return misuse("lstm_pack_weights: precision differs from the handle's");
    if (input_size != h->I || hidden_size != h->H) return misuse("lstm_pack_weights: sizes differ from the handle's");
    // The biases arrive with lstm_forward (as in the reference), so the snapshot is kept in fp32
    // here and the engine packs weights and biases together on the next forward call.
    if (cudaMemcpyAsync(h->w_ih, weight_ih, 4 * h->H * h->I * sizeof(float), cudaMemcpyDeviceToDevice, h->stream) != cudaSuccess ||
        cudaMemcpyAsync(h->w_hh, weight_hh, 4 * h->H * h->H * sizeof(float), cudaMemcpyDeviceToDevice, h->stream) != cudaSuccess ||
        cudaStreamSynchronize(h->stream) != cudaSuccess) {
        std::fprintf(stderr, "flashlstm: lstm_pack_weights: copy failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return (int)cudaErrorUnknown;
    }
    h->packed = true;
    return 0;
}

int lstm_forward(const float *x, const float *b_ih, const float *b_hh, const float *h0, const float *c0,
                 float *output, float *hn, float *cn, size_t seq_len, size_t batch, size_t input_size,
                 size_t hidden_size, const lstm_buffers *buffers, lstm_compute_precision_t precision) {
    if (!buffers || !buffers->impl) return misuse("lstm_forward: handle is null");
    V1Handle *h = static_cast<V1Handle *>(buffers->impl);
    if ((int)precision != h->precision) return misuse("lstm_forward: precision differs from the handle's");
    if (batch != h->B || input_size != h->I || hidden_size != h->H)
        return misuse("lstm_forward: batch/input/hidden size differs from the handle's");
    if (!h->packed) return misuse("lstm_forward: weights have not been packed");
    if (!x || !b_ih || !b_hh || !h0 || !c0 || !output || !hn || !cn) return misuse("lstm_forward: null pointer argument");
    if (seq_len == 0) return misuse("lstm_forward: seq_len must be positive");
    if (seq_len > h->t_cap && alloc_staging(h, seq_len) != 0) return misuse("lstm_forward: could not grow the staging buffers");
    cudaStream_t s = h->stream;
    const size_t slab = h->B * h->H;
    char *st16 = static_cast<char *>(h->st16);
    int st = flstm_engine_set_weights(h->engine, 0, h->w_ih, h->w_hh, b_ih, b_hh, s);
    if (st == FLSTM_OK) st = simt::convert(FLSTM_DTYPE_F32, x, FLSTM_DTYPE_F16, h->x16, seq_len * h->B * h->I, s);
    if (st == FLSTM_OK) st = simt::convert(FLSTM_DTYPE_F32, h0, FLSTM_DTYPE_F16, st16, slab, s);
    // the cell state crosses in fp32 both ways (the reference keeps c in fp32 throughout)
    if (st == FLSTM_OK)
        st = flstm_engine_forward(h->engine, seq_len, h->x16, st16, c0, h->y16, st16 + slab * 2, cn, s);
    if (st == FLSTM_OK) st = simt::convert(FLSTM_DTYPE_F16, h->y16, FLSTM_DTYPE_F32, output, seq_len * slab, s);
    if (st == FLSTM_OK) st = simt::convert(FLSTM_DTYPE_F16, st16 + slab * 2, FLSTM_DTYPE_F32, hn, slab, s);
    if (st != FLSTM_OK) return fail(to_cuda_code(st), "lstm_forward");
    cudaError_t ce = cudaStreamSynchronize(s);
    if (ce != cudaSuccess) {
        std::fprintf(stderr, "flashlstm: lstm_forward: %s\n", cudaGetErrorString(ce));
        return (int)ce;
    }
    return 0;
}

}  // extern "C"
