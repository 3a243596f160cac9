// CPython extension `_flashlstm`: the two functions the reference's Python package imports
// (flashlstm_v2/python/flashlstm/_flashlstm_module.cpp:217-239).  Arguments are raw addresses
// and stream handles passed as unsigned integers, in the reference's order
// (:41-65 forward, 22 values; :137-169 backward, 30 values); 0 means null.  The GIL is
// released around the native call.  Unlike the reference, a failure raises RuntimeError.
#include <Python.h>

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstdint>

#include "flashlstm_b200/engine.h"
#include "lstm.hpp"

namespace {

template <typename P>
P as_ptr(unsigned long long v) {
    return reinterpret_cast<P>(static_cast<uintptr_t>(v));
}

bool parse_values(PyObject *args, unsigned long long *out, Py_ssize_t want, const char *fn) {
    if (!PyTuple_Check(args) || PyTuple_GET_SIZE(args) != want) {
        PyErr_Format(PyExc_TypeError, "%s expects %zd integer arguments", fn, want);
        return false;
    }
    for (Py_ssize_t i = 0; i < want; ++i) {
        PyObject *item = PyTuple_GET_ITEM(args, i);
        unsigned long long v = PyLong_AsUnsignedLongLongMask(item);
        if (v == (unsigned long long)-1 && PyErr_Occurred()) return false;
        out[i] = v;
    }
    return true;
}

PyObject *raise_if_failed() {
    if (flstm_last_status() != FLSTM_OK) {
        PyErr_SetString(PyExc_RuntimeError, flstm_last_error());
        return nullptr;
    }
    Py_RETURN_NONE;
}

PyObject *py_forward(PyObject *, PyObject *args) {
    unsigned long long v[22];
    if (!parse_values(args, v, 22, "streaming_lstm_forward")) return nullptr;
    flstm_GateCacheHost cache{as_ptr<void *>(v[13]), as_ptr<void *>(v[14])};
    flstm_StreamingLstmOptions opt{static_cast<flstm_GateCacheDType>(v[15]), static_cast<flstm_GateCacheDType>(v[16])};
    Py_BEGIN_ALLOW_THREADS
    flstm_StreamingLstmForward(v[0], v[1], v[2], v[3], v[4], as_ptr<const __half *>(v[5]), as_ptr<const __half *>(v[6]),
                               as_ptr<const __half *>(v[7]), as_ptr<const float *>(v[8]), as_ptr<const float *>(v[9]),
                               as_ptr<const float *>(v[10]), as_ptr<const float *>(v[11]), as_ptr<__half *>(v[12]),
                               cache, &opt, as_ptr<__half *>(v[17]), as_ptr<__half *>(v[18]),
                               as_ptr<cudaStream_t>(v[19]), as_ptr<cudaStream_t>(v[20]), as_ptr<cudaStream_t>(v[21]));
    Py_END_ALLOW_THREADS
    return raise_if_failed();
}

PyObject *py_backward(PyObject *, PyObject *args) {
    unsigned long long v[30];
    if (!parse_values(args, v, 30, "streaming_lstm_backward")) return nullptr;
    flstm_GateCacheHost cache{as_ptr<void *>(v[7]), as_ptr<void *>(v[8])};
    flstm_StreamingLstmOptions opt{static_cast<flstm_GateCacheDType>(v[9]), static_cast<flstm_GateCacheDType>(v[10])};
    Py_BEGIN_ALLOW_THREADS
    flstm_StreamingLstmBackward(
        v[0], v[1], v[2], v[3], v[4], as_ptr<const __half *>(v[5]), as_ptr<const __half *>(v[6]), cache,
        as_ptr<const __half *>(v[11]), as_ptr<const __half *>(v[12]), as_ptr<const __half *>(v[13]),
        as_ptr<const __half *>(v[14]), as_ptr<const __half *>(v[15]), as_ptr<const float *>(v[16]),
        as_ptr<const float *>(v[17]), as_ptr<const float *>(v[18]), as_ptr<const float *>(v[19]),
        as_ptr<__half *>(v[20]), as_ptr<float *>(v[21]), as_ptr<float *>(v[22]), as_ptr<float *>(v[23]),
        as_ptr<float *>(v[24]), as_ptr<float *>(v[25]), as_ptr<float *>(v[26]), as_ptr<cudaStream_t>(v[27]),
        as_ptr<cudaStream_t>(v[28]), as_ptr<cudaStream_t>(v[29]), &opt);
    Py_END_ALLOW_THREADS
    return raise_if_failed();
}

PyMethodDef kMethods[] = {
    {"streaming_lstm_forward", py_forward, METH_VARARGS,
     "streaming_lstm_forward(T,B,I,H,R, x_host,h0,c0, W_ih,W_hh,b_ih,b_hh, y_host, cache_h,cache_c, "
     "cache_h_dtype,cache_c_dtype, hy,cy, compute_stream,h2d_stream,d2h_stream) -> None"},
    {"streaming_lstm_backward", py_backward, METH_VARARGS,
     "streaming_lstm_backward(T,B,I,H,R, x,y, cache_h,cache_c,h_dtype,c_dtype, dY,d_hn,d_cn, h0,c0, "
     "W_ih,W_hh,b_ih,b_hh, dx, dW_ih,dW_hh,db_ih,db_hh, dh0,dc0, compute,h2d,d2h) -> None"},
    {nullptr, nullptr, 0, nullptr},
};

PyModuleDef kModule = {PyModuleDef_HEAD_INIT, "_flashlstm", "B200 LSTM streaming forward/backward bindings", -1, kMethods,
                       nullptr, nullptr, nullptr, nullptr};

}  // namespace

PyMODINIT_FUNC PyInit__flashlstm(void) { return PyModule_Create(&kModule); }
