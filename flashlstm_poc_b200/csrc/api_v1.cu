// Forward-only v1 surface (include/flashlstm/lstm_api.h) as a shim over the engine.
//
// Mirrors the behaviour of the reference's entry points in src/lstm.cu: creation :675-858,
// destroy :860-867, execution mode :869-884, weight packing :886-931, forward :1897-2148.
// Kept: fp32 device I/O, sizes fixed at creation and re-validated per call (:1915-1917),
// precision must match (:897,1915), weights must be packed first (:1918), a longer sequence
// grows the workspace (:933-970), the handle owns a non-blocking stream (:851) and the call is
// synchronous (:2081,2146); failures return a cudaError_t value and print to stderr.
//
// Execution mode (:869-884).  IMMEDIATE enqueues the kernels of a call directly.  GRAPH (the default, as the
// reference forces it, src/lstm.cu:23,1922-1924) replays a captured CUDA graph of the whole call -- input
// conversion, weight packing, projection GEMM, persistent recurrence, output conversion: the first call with a
// new sequence length or new tensor addresses runs directly and then records its graph (the reference rebuilds
// its graph when T changes, :2085-2087, and stages the tensors into owned buffers to keep node pointers valid,
// :1950-2040; here the addresses are part of the graph's key instead, so nothing is copied twice).
// input_proj_chunk_size (:144-153,1204-1239): 0 projects the whole sequence with one GEMM; n > 0 runs the
// sequence in ranges of n steps, each with its own projection GEMM followed by the recurrence over the range.
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
    // GRAPH mode: the captured call and what it was captured for
    cudaGraphExec_t graph_exec = nullptr;
    size_t graph_T = 0;
    const void *graph_ptrs[8] = {};
    unsigned long long graph_replays = 0;
};

void drop_graph(V1Handle *h) {
    if (h->graph_exec) cudaGraphExecDestroy(h->graph_exec);
    h->graph_exec = nullptr;
    h->graph_T = 0;
}

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
    drop_graph(h);  // its nodes point into the old staging buffers
    free_staging(h);
    if (cudaMalloc(&h->x16, T * h->B * h->I * 2) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
    if (cudaMalloc(&h->y16, T * h->B * h->H * 2) != cudaSuccess) return (int)cudaErrorMemoryAllocation;
    h->t_cap = T;
    return 0;
}

// Everything one call enqueues on the handle's stream: fp32 -> fp16 staging, weight packing (the biases arrive
// with this call), the forward pass in ranges of `chunk` steps, fp16 -> fp32 results.
int enqueue_forward(V1Handle *h, const float *x, const float *b_ih, const float *b_hh, const float *h0, const float *c0,
                    float *output, float *hn, float *cn, size_t T, cudaStream_t s) {
    const size_t slab = h->B * h->H;
    char *st16 = static_cast<char *>(h->st16);
    FLSTM_TRY(flstm_engine_set_weights(h->engine, 0, h->w_ih, h->w_hh, b_ih, b_hh, s));
    FLSTM_TRY(simt::convert(FLSTM_DTYPE_F32, x, FLSTM_DTYPE_F16, h->x16, T * h->B * h->I, s));
    FLSTM_TRY(simt::convert(FLSTM_DTYPE_F32, h0, FLSTM_DTYPE_F16, st16, slab, s));
    // the cell state crosses in fp32 both ways (the reference keeps c in fp32 throughout)
    const size_t step = (h->chunk > 0 && (size_t)h->chunk < T) ? (size_t)h->chunk : T;
    for (size_t t0 = 0; t0 < T; t0 += step) {
        const size_t t1 = t0 + step < T ? t0 + step : T;
        FLSTM_TRY(flstm_engine_forward_range(h->engine, T, t0, t1, h->x16, st16, c0, h->y16, st16 + slab * 2, cn, s));
    }
    FLSTM_TRY(simt::convert(FLSTM_DTYPE_F16, h->y16, FLSTM_DTYPE_F32, output, T * slab, s));
    FLSTM_TRY(simt::convert(FLSTM_DTYPE_F16, st16 + slab * 2, FLSTM_DTYPE_F32, hn, slab, s));
    return FLSTM_OK;
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
    drop_graph(h);
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

// Number of lstm_forward calls on this handle that were served by replaying the captured graph
// (diagnostics and tests; no counterpart in the reference).
unsigned long long lstm_graph_replays(const lstm_buffers *buffers) {
    return (buffers && buffers->impl) ? static_cast<const V1Handle *>(buffers->impl)->graph_replays : 0ull;
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
    const void *ptrs[8] = {x, b_ih, b_hh, h0, c0, output, hn, cn};
    auto finish = [&]() -> int {
        cudaError_t ce = cudaStreamSynchronize(s);
        if (ce != cudaSuccess) {
            std::fprintf(stderr, "flashlstm: lstm_forward: %s\n", cudaGetErrorString(ce));
            return (int)ce;
        }
        return 0;
    };
    if (h->mode == LSTM_EXECUTION_MODE_GRAPH && h->graph_exec && h->graph_T == seq_len) {
        bool same = true;
        for (int i = 0; i < 8; ++i) same = same && h->graph_ptrs[i] == ptrs[i];
        if (same) {
            cudaError_t ce = cudaGraphLaunch(h->graph_exec, s);
            if (ce != cudaSuccess) {
                std::fprintf(stderr, "flashlstm: lstm_forward: graph launch failed: %s\n", cudaGetErrorString(ce));
                return (int)ce;
            }
            ++h->graph_replays;
            return finish();
        }
    }
    int st = enqueue_forward(h, x, b_ih, b_hh, h0, c0, output, hn, cn, seq_len, s);
    if (st != FLSTM_OK) return fail(to_cuda_code(st), "lstm_forward");
    int rc = finish();
    if (rc != 0 || h->mode != LSTM_EXECUTION_MODE_GRAPH) return rc;
    // record this call for the next one with the same length and tensors; a capture that fails leaves the
    // handle on direct launches
    drop_graph(h);
    cudaGraph_t graph = nullptr;
    if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    st = enqueue_forward(h, x, b_ih, b_hh, h0, c0, output, hn, cn, seq_len, s);
    cudaError_t ce = cudaStreamEndCapture(s, &graph);
    if (st == FLSTM_OK && ce == cudaSuccess && graph && cudaGraphInstantiate(&h->graph_exec, graph, 0) == cudaSuccess) {
        h->graph_T = seq_len;
        for (int i = 0; i < 8; ++i) h->graph_ptrs[i] = ptrs[i];
    } else {
        cudaGetLastError();
        h->graph_exec = nullptr;
    }
    if (graph) cudaGraphDestroy(graph);
    return 0;
}

}  // extern "C"
