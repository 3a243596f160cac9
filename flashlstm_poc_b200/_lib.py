"""ctypes binding of the C-ABI library (include/flashlstm_b200/engine.h, include/flashlstm/lstm_api.h,
include/lstm.hpp).  The library is the product; there is no Python or CPU fallback: if it is
missing or cannot be loaded, importing this module fails loudly."""

from __future__ import annotations

import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libflashlstm_b200.so")

# every symbol the public headers declare; tests check that each one is exported
ENGINE_SYMBOLS = [
    "flstm_engine_create", "flstm_engine_destroy", "flstm_engine_set_weights", "flstm_engine_forward",
    "flstm_engine_backward", "flstm_engine_forward_range", "flstm_engine_backward_range", "flstm_engine_grad_ptrs", "flstm_engine_grad_buffer", "flstm_engine_cache_ptrs",
    "flstm_engine_set_cell_io_f32", "flstm_engine_backend", "flstm_comm_unique_id", "flstm_engine_attach_comm",
    "flstm_engine_enable_timing", "flstm_engine_phase_ms", "flstm_engine_launch_count", "flstm_tc_gemm",
    "flstm_engine_enable_trace", "flstm_engine_read_trace", "flstm_bias_grad", "flstm_tc_plan", "flstm_engine_wait", "flstm_engine_abort_comm",
                  "flstm_engine_set_recompute_interval", "flstm_engine_workspace_bytes",
    "flstm_bias_grad_static", "flstm_engine_set_wait_limit", "flstm_engine_selftest_missing_arrivals",
    "flstm_engine_backward_segment",
    "flstm_last_error",
    "flstm_version",
]
V1_SYMBOLS = ["lstm_create_buffers", "lstm_destroy_buffers", "lstm_set_execution_mode", "lstm_pack_weights",
              "lstm_forward", "lstm_graph_replays"]
V2_SYMBOLS = ["flstm_StreamingLstmForward", "flstm_StreamingLstmBackward", "flstm_last_status",
              "flstm_v2_set_weight_version", "flstm_v2_last_call_info"]

STATUS_NAMES = {0: "OK", 1: "INVALID", 2: "CUDA", 3: "TIMEOUT", 4: "UNSUPPORTED", 5: "COMM"}
DTYPE_CODES = {"f32": 0, "f16": 1, "bf16": 2}
BACKEND_CODES = {"auto": 0, "simt": 1, "tc": 2}
BACKEND_NAMES = {v: k for k, v in BACKEND_CODES.items()}


class EngineConfig(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int), ("layers", ctypes.c_int), ("batch", ctypes.c_size_t),
        ("input_size", ctypes.c_size_t), ("hidden_size", ctypes.c_size_t), ("max_seq_len", ctypes.c_size_t),
        ("training", ctypes.c_int), ("backend", ctypes.c_int),
    ]


class TcPlanInfo(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "fwd_batch_tile", "fwd_row_tiles_per_cta", "fwd_grid", "fwd_batch_groups", "fwd_tiles_per_group",
        "fwd_stages", "fwd_chunks_per_stage", "fwd_weights_resident", "fwd_smem_bytes",
        "bwd_batch_tile", "bwd_cluster_size", "bwd_grid", "bwd_batch_groups", "bwd_tiles_per_group",
        "bwd_stages", "bwd_chunks_per_stage", "bwd_weights_resident", "bwd_smem_bytes",
        "step_path", "step_bn_fwd", "step_bn_bwd", "step_splits", "step_pair", "fwd_pair", "step_fwd_pair")]


class LstmBuffers(ctypes.Structure):
    _fields_ = [("impl", ctypes.c_void_p)]


class GateCacheHost(ctypes.Structure):
    _fields_ = [("h_ptr", ctypes.c_void_p), ("c_ptr", ctypes.c_void_p)]


class StreamingLstmOptions(ctypes.Structure):
    _fields_ = [("h_dtype", ctypes.c_int), ("c_dtype", ctypes.c_int)]


class FlashLstmError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"flashlstm-b200 [{STATUS_NAMES.get(status, status)}]: {message}")
        self.status = status


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m flashlstm_poc_b200._build` "
            "(needs nvcc with sm_100a support). There is no CPU fallback."
        )
    lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.flstm_engine_create.argtypes = [ctypes.POINTER(EngineConfig), ctypes.POINTER(vp)]
    lib.flstm_engine_destroy.argtypes = [vp]
    lib.flstm_engine_set_weights.argtypes = [vp, ci, vp, vp, vp, vp, vp]
    lib.flstm_engine_forward.argtypes = [vp, sz, vp, vp, vp, vp, vp, vp, vp]
    lib.flstm_engine_backward.argtypes = [vp, sz, vp, vp, vp, vp, vp, vp, vp]
    lib.flstm_engine_forward_range.argtypes = [vp, sz, sz, sz, vp, vp, vp, vp, vp, vp, vp]
    lib.flstm_engine_backward_range.argtypes = [vp, sz, sz, sz, vp, vp, vp, vp, vp, vp, vp]
    lib.flstm_engine_grad_ptrs.argtypes = [vp, ci, ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp)]
    lib.flstm_engine_grad_buffer.argtypes = [vp, ctypes.POINTER(vp), ctypes.POINTER(sz)]
    lib.flstm_engine_cache_ptrs.argtypes = [vp, ci, ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp),
                                            ctypes.POINTER(ci)]
    lib.flstm_engine_set_cell_io_f32.argtypes = [vp, ci]
    lib.flstm_engine_backend.argtypes = [vp]
    lib.flstm_comm_unique_id.argtypes = [vp]
    lib.flstm_engine_attach_comm.argtypes = [vp, vp, ci, ci]
    lib.flstm_engine_enable_timing.argtypes = [vp, ci]
    lib.flstm_engine_phase_ms.argtypes = [vp, ctypes.POINTER(ctypes.c_float)]
    lib.flstm_engine_launch_count.argtypes = [vp]
    lib.flstm_engine_launch_count.restype = ctypes.c_ulonglong
    lib.flstm_engine_enable_trace.argtypes = [vp, ci]
    lib.flstm_engine_read_trace.argtypes = [vp, vp, sz]
    lib.flstm_tc_plan.argtypes = [sz, sz, ci, ci, sz, ctypes.POINTER(TcPlanInfo)]
    lib.flstm_engine_wait.argtypes = [vp, vp, ctypes.c_uint]
    lib.flstm_engine_abort_comm.argtypes = [vp]
    lib.flstm_engine_backward_segment.argtypes = [vp, sz, ci, ci] + [vp] * 10
    lib.flstm_engine_set_wait_limit.argtypes = [vp, ctypes.c_ulonglong]
    lib.flstm_engine_selftest_missing_arrivals.argtypes = [vp, ctypes.c_uint]
    lib.flstm_engine_set_recompute_interval.argtypes = [vp, sz]
    lib.flstm_engine_workspace_bytes.argtypes = [vp]
    lib.flstm_engine_workspace_bytes.restype = sz
    lib.flstm_bias_grad.argtypes = [ci, vp, sz, sz, ci, vp, vp]
    lib.flstm_bias_grad_static.argtypes = [ci, vp, sz, sz, ci, vp, vp]
    lib.flstm_tc_gemm.argtypes = [ci, ci, sz, sz, sz, vp, vp, vp, sz, vp, ci, vp]
    lib.flstm_last_error.restype = ctypes.c_char_p
    lib.flstm_version.restype = ctypes.c_char_p
    # v1 surface
    lib.lstm_create_buffers.argtypes = [ci, sz, sz, sz, sz, ci, ctypes.POINTER(LstmBuffers)]
    lib.lstm_destroy_buffers.argtypes = [ctypes.POINTER(LstmBuffers)]
    lib.lstm_set_execution_mode.argtypes = [ctypes.POINTER(LstmBuffers), ci]
    lib.lstm_pack_weights.argtypes = [ci, vp, vp, sz, sz, ctypes.POINTER(LstmBuffers)]
    lib.lstm_forward.argtypes = [vp] * 8 + [sz] * 4 + [ctypes.POINTER(LstmBuffers), ci]
    lib.lstm_graph_replays.argtypes = [ctypes.POINTER(LstmBuffers)]
    lib.lstm_graph_replays.restype = ctypes.c_ulonglong
    # v2 surface
    lib.flstm_StreamingLstmForward.argtypes = [sz] * 5 + [vp] * 8 + [GateCacheHost, ctypes.POINTER(StreamingLstmOptions)] + [vp] * 5
    lib.flstm_StreamingLstmForward.restype = None
    lib.flstm_StreamingLstmBackward.argtypes = [sz] * 5 + [vp, vp, GateCacheHost] + [vp] * 19 + [ctypes.POINTER(StreamingLstmOptions)]
    lib.flstm_StreamingLstmBackward.restype = None
    lib.flstm_last_status.restype = ci
    lib.flstm_v2_set_weight_version.argtypes = [ctypes.c_ulonglong]
    lib.flstm_v2_set_weight_version.restype = None
    lib.flstm_v2_last_call_info.argtypes = [ctypes.POINTER(sz), ctypes.POINTER(ci)]
    lib.flstm_v2_last_call_info.restype = None
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        raise FlashLstmError(status, load().flstm_last_error().decode())
