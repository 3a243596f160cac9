"""Python handle over the native engine (include/flashlstm_b200/engine.h): torch tensors in,
device pointers across the C ABI.  PyTorch is used for device memory and streams only."""

from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import BACKEND_CODES, BACKEND_NAMES, DTYPE_CODES, EngineConfig, check

TORCH_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
DTYPE_OF_TORCH = {v: k for k, v in TORCH_DTYPES.items()}
PHASES = ("projection", "recurrent_fwd", "bptt", "weight_grad", "input_grad", "allreduce")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class Engine:
    """One LSTM stack on one GPU.  x (T,B,I), states (L,B,H), all in the engine dtype."""

    def __init__(self, dtype: str, layers: int, batch: int, input_size: int, hidden_size: int, max_seq_len: int,
                 training: bool = True, backend: str = "auto", device: Optional[torch.device] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("flashlstm-b200 needs a CUDA device: there is no CPU fallback")
        self.lib = _lib.load()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.dtype, self.layers, self.batch = dtype, layers, batch
        self.input_size, self.hidden_size, self.training = input_size, hidden_size, training
        self.torch_dtype = TORCH_DTYPES[dtype]
        cfg = EngineConfig(DTYPE_CODES[dtype], layers, batch, input_size, hidden_size, max_seq_len,
                           1 if training else 0, BACKEND_CODES[backend])
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(self.lib.flstm_engine_create(ctypes.byref(cfg), ctypes.byref(handle)))
        self._h = handle
        self._saved_x = None

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.lib.flstm_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def backend(self) -> str:
        return BACKEND_NAMES[self.lib.flstm_engine_backend(self._h)]

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _check_tensor(self, t: torch.Tensor, shape: Tuple[int, ...], name: str, dtype=None) -> torch.Tensor:
        dtype = dtype or self.torch_dtype
        if t.device != self.device:
            raise ValueError(f"{name} must be on {self.device}, got {t.device}")
        if t.dtype != dtype:
            raise ValueError(f"{name} must have dtype {dtype}, got {t.dtype}")
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
        return t if t.is_contiguous() else t.contiguous()

    def set_weights(self, layer: int, w_ih: torch.Tensor, w_hh: torch.Tensor, b_ih: torch.Tensor,
                    b_hh: torch.Tensor) -> None:
        H = self.hidden_size
        I = self.input_size if layer == 0 else H
        w_ih = self._check_tensor(w_ih.detach(), (4 * H, I), "w_ih", torch.float32)
        w_hh = self._check_tensor(w_hh.detach(), (4 * H, H), "w_hh", torch.float32)
        b_ih = self._check_tensor(b_ih.detach(), (4 * H,), "b_ih", torch.float32)
        b_hh = self._check_tensor(b_hh.detach(), (4 * H,), "b_hh", torch.float32)
        check(self.lib.flstm_engine_set_weights(self._h, layer, w_ih.data_ptr(), w_hh.data_ptr(), b_ih.data_ptr(),
                                                b_hh.data_ptr(), self._stream()))

    def forward(self, x: torch.Tensor, h0: Optional[torch.Tensor] = None, c0: Optional[torch.Tensor] = None,
                want_states: bool = True):
        T = x.shape[0]
        L, B, H = self.layers, self.batch, self.hidden_size
        x = self._check_tensor(x, (T, B, self.input_size), "x")
        if h0 is not None:
            h0 = self._check_tensor(h0, (L, B, H), "h0")
        if c0 is not None:
            c0 = self._check_tensor(c0, (L, B, H), "c0")
        y = torch.empty((T, B, H), dtype=self.torch_dtype, device=self.device)
        hn = torch.empty((L, B, H), dtype=self.torch_dtype, device=self.device) if want_states else None
        cn = torch.empty((L, B, H), dtype=self.torch_dtype, device=self.device) if want_states else None
        check(self.lib.flstm_engine_forward(self._h, T, x.data_ptr(), _ptr(h0), _ptr(c0), y.data_ptr(), _ptr(hn),
                                            _ptr(cn), self._stream()))
        self._saved_x = x  # re-read by backward for dW_ih
        return y, hn, cn

    def backward(self, dy: torch.Tensor, dhn: Optional[torch.Tensor] = None, dcn: Optional[torch.Tensor] = None,
                 want_dx: bool = True, want_dstates: bool = True):
        T = dy.shape[0]
        L, B, H = self.layers, self.batch, self.hidden_size
        dy = self._check_tensor(dy, (T, B, H), "dy")
        if dhn is not None:
            dhn = self._check_tensor(dhn, (L, B, H), "dhn")
        if dcn is not None:
            dcn = self._check_tensor(dcn, (L, B, H), "dcn")
        dx = torch.empty((T, B, self.input_size), dtype=self.torch_dtype, device=self.device) if want_dx else None
        dh0 = torch.empty((L, B, H), dtype=torch.float32, device=self.device) if want_dstates else None
        dc0 = torch.empty((L, B, H), dtype=torch.float32, device=self.device) if want_dstates else None
        check(self.lib.flstm_engine_backward(self._h, T, dy.data_ptr(), _ptr(dhn), _ptr(dcn), _ptr(dx), _ptr(dh0),
                                             _ptr(dc0), self._stream()))
        return dx, dh0, dc0

    # ---- raw-pointer forms for callers that own all buffers (benchmark, CUDA-graph capture)
    def forward_into(self, T: int, x, h0, c0, y, hn, cn) -> None:
        check(self.lib.flstm_engine_forward(self._h, T, x.data_ptr(), _ptr(h0), _ptr(c0), _ptr(y), _ptr(hn),
                                            _ptr(cn), self._stream()))

    def backward_into(self, T: int, dy, dhn, dcn, dx, dh0, dc0) -> None:
        check(self.lib.flstm_engine_backward(self._h, T, dy.data_ptr(), _ptr(dhn), _ptr(dcn), _ptr(dx), _ptr(dh0),
                                             _ptr(dc0), self._stream()))

    def forward_range_into(self, T: int, t0: int, t1: int, x, h0, c0, y, hn, cn) -> None:
        """Steps [t0, t1) of a T-step forward; ranges ascending from 0 (see flstm_engine_forward_range)."""
        check(self.lib.flstm_engine_forward_range(self._h, T, t0, t1, x.data_ptr(), _ptr(h0), _ptr(c0), _ptr(y), _ptr(hn),
                                                  _ptr(cn), self._stream()))

    def backward_range_into(self, T: int, t0: int, t1: int, dy, dhn, dcn, dx, dh0, dc0) -> None:
        """Steps [t0, t1) of the backward pass; ranges descending from T (see flstm_engine_backward_range)."""
        check(self.lib.flstm_engine_backward_range(self._h, T, t0, t1, dy.data_ptr(), _ptr(dhn), _ptr(dcn), _ptr(dx),
                                                   _ptr(dh0), _ptr(dc0), self._stream()))

    def backward_segment_into(self, steps: int, last_in_time: bool, first_in_time: bool, x_seg, h_in, c_in, dy_seg, dhn, dcn,
                              dx_seg, dh0, dc0) -> None:
        """One segment of a sequence streamed through a segment-sized engine, last segment first
        (see flstm_engine_backward_segment): h_in (L,B,H) engine dtype and c_in (L,B,H) fp32 are the states
        that entered the segment."""
        check(self.lib.flstm_engine_backward_segment(self._h, steps, int(last_in_time), int(first_in_time), x_seg.data_ptr(),
                                                     _ptr(h_in), _ptr(c_in), dy_seg.data_ptr(), _ptr(dhn), _ptr(dcn),
                                                     _ptr(dx_seg), _ptr(dh0), _ptr(dc0), self._stream()))

    def set_cell_io_f32(self, on: bool = True) -> None:
        """c0 / c_n cross the API as fp32 (the engine's own cell-state precision) instead of the engine dtype."""
        check(self.lib.flstm_engine_set_cell_io_f32(self._h, 1 if on else 0))

    def capture_step(self, x, h0, c0, y, hn, cn, dy=None, dx=None, dh0=None, dc0=None) -> "torch.cuda.CUDAGraph":
        """Capture one forward (+ backward when dy is given) over the given, caller-owned tensors into a
        CUDA graph: the projection GEMM, the persistent recurrent kernels (cooperative launches), the
        gradient GEMMs and, with a communicator attached, the per-layer allreduce all become graph nodes.
        Replay with graph.replay(); the tensors keep their addresses, only their contents may change."""
        T = x.shape[0]
        # run once eagerly so lazy one-time set-up (function attributes, NCCL channels) is not captured
        self.forward_into(T, x, h0, c0, y, hn, cn)
        if dy is not None:
            self.backward_into(T, dy, None, None, dx, dh0, dc0)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.forward_into(T, x, h0, c0, y, hn, cn)
            if dy is not None:
                self.backward_into(T, dy, None, None, dx, dh0, dc0)
        return graph

    def _wrap(self, ptr: int, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """A torch view over engine-owned device memory (valid while the engine lives)."""
        n = 1
        for s in shape:
            n *= s

        class _Holder:
            pass

        holder = _Holder()
        holder.__cuda_array_interface__ = {
            "shape": tuple(shape), "typestr": {torch.float32: "<f4", torch.float16: "<f2", torch.bfloat16: "<u2"}[dtype],
            "data": (ptr, False), "version": 3,
        }
        t = torch.as_tensor(holder, device=self.device)
        if dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        t._flstm_owner = self
        return t

    def grads(self, layer: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Views of dW_ih (4H,I_l), dW_hh (4H,H), db (4H) in the flat fp32 gradient buffer."""
        a, b, c = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        check(self.lib.flstm_engine_grad_ptrs(self._h, layer, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)))
        H = self.hidden_size
        I = self.input_size if layer == 0 else H
        return (self._wrap(a.value, (4 * H, I), torch.float32), self._wrap(b.value, (4 * H, H), torch.float32),
                self._wrap(c.value, (4 * H,), torch.float32))

    def grad_buffer(self) -> torch.Tensor:
        p, n = ctypes.c_void_p(), ctypes.c_size_t()
        check(self.lib.flstm_engine_grad_buffer(self._h, ctypes.byref(p), ctypes.byref(n)))
        return self._wrap(p.value, (n.value,), torch.float32)

    def gate_cache(self, layer: int, T: int) -> torch.Tensor:
        """Post-activation gates (T,B,4H) of the last training forward, returned in torch column
        order (g*H+u) whatever the engine's internal layout."""
        g, c, h, layout = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int()
        check(self.lib.flstm_engine_cache_ptrs(self._h, layer, ctypes.byref(g), ctypes.byref(c), ctypes.byref(h),
                                               ctypes.byref(layout)))
        B, H = self.batch, self.hidden_size
        raw = self._wrap(g.value, (T, B, 4 * H), self.torch_dtype)
        if layout.value == 0:
            return raw.clone()
        # tile-interleaved: column ((u/16)*4 + g)*16 + u%16
        return raw.view(T, B, H // 16, 4, 16).permute(0, 1, 3, 2, 4).reshape(T, B, 4 * H).contiguous()

    def cell_states(self, layer: int, T: int) -> torch.Tensor:
        g, c, h, layout = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int()
        check(self.lib.flstm_engine_cache_ptrs(self._h, layer, ctypes.byref(g), ctypes.byref(c), ctypes.byref(h),
                                               ctypes.byref(layout)))
        return self._wrap(c.value, (T + 1, self.batch, self.hidden_size), torch.float32)

    def attach_comm(self, unique_id: bytes, rank: int, world_size: int) -> None:
        buf = ctypes.create_string_buffer(unique_id, 128)
        with torch.cuda.device(self.device):
            check(self.lib.flstm_engine_attach_comm(self._h, buf, rank, world_size))

    def set_recompute_interval(self, interval: int) -> None:
        """Activation checkpoints: keep h/c every `interval` steps and rebuild the gate cache segment by segment in
        backward (0 = keep the full gate cache).  Re-allocates the time-sized buffers."""
        with torch.cuda.device(self.device):
            check(self.lib.flstm_engine_set_recompute_interval(self._h, int(interval)))

    @property
    def workspace_bytes(self) -> int:
        return int(self.lib.flstm_engine_workspace_bytes(self._h))

    def wait(self, timeout_s: float, stream: Optional[torch.cuda.Stream] = None) -> None:
        """Host watchdog: block until the work enqueued so far on `stream` has finished, at most `timeout_s`
        seconds.  Raises FlashLstmError (TIMEOUT) past the deadline, after aborting an attached communicator."""
        with torch.cuda.device(self.device):
            s = stream if stream is not None else torch.cuda.current_stream()
            check(self.lib.flstm_engine_wait(self._h, s.cuda_stream, max(0, int(timeout_s * 1000))))

    def set_wait_limit(self, microseconds: int) -> None:
        """Limit of every device-side wait of the persistent kernels (0 = the 2 s default)."""
        check(self.lib.flstm_engine_set_wait_limit(self._h, int(microseconds)))

    def selftest_missing_arrivals(self, arrivals: int) -> None:
        """Timeout self-test: every step barrier of the following launches waits for `arrivals` arrivals that no
        CTA makes, so the second time step's wait runs out after the limit and the launch returns with the
        error word set (the next call raises TIMEOUT).  0 switches it off."""
        check(self.lib.flstm_engine_selftest_missing_arrivals(self._h, int(arrivals)))

    def abort_comm(self) -> None:
        check(self.lib.flstm_engine_abort_comm(self._h))

    @property
    def config_key(self) -> tuple:
        """What every rank of a data-parallel group must agree on (the per-rank batch may not differ either:
        the weight-gradient allreduce assumes equal shards)."""
        return (self.dtype, self.layers, self.batch, self.input_size, self.hidden_size, bool(self.training))

    @staticmethod
    def new_unique_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        check(_lib.load().flstm_comm_unique_id(buf))
        return buf.raw

    def enable_timing(self, on: bool = True) -> None:
        check(self.lib.flstm_engine_enable_timing(self._h, 1 if on else 0))

    def phase_ms(self) -> dict:
        out = (ctypes.c_float * 6)()
        check(self.lib.flstm_engine_phase_ms(self._h, out))
        return dict(zip(PHASES, [float(v) for v in out]))

    @property
    def launch_count(self) -> int:
        return int(self.lib.flstm_engine_launch_count(self._h))
