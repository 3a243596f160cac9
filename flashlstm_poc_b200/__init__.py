"""flashlstm_poc_b200: a B200-native (sm_100a) LSTM forward/backward engine behind the operator
surface of flashlstm_poc.  The CUDA library is the product; importing the operator modules
fails loudly when it has not been built (`python -m flashlstm_poc_b200._build`)."""

from .workloads import WORKLOADS, Workload, make_inputs  # noqa: F401

__all__ = ["WORKLOADS", "Workload", "make_inputs", "Engine", "LSTM", "StreamingLSTM", "streaming_lstm",
           "streaming_lstm_forward", "streaming_lstm_backward", "GateCache"]

_LAZY = {
    "Engine": ("engine", "Engine"),
    "LSTM": ("lstm", "LSTM"),
    "StreamingLSTM": ("streaming_lstm", "StreamingLSTM"),
    "streaming_lstm": ("streaming_lstm", "streaming_lstm"),
    "GateCache": ("streaming_lstm", "GateCache"),
    "streaming_lstm_forward": ("_flashlstm", "streaming_lstm_forward"),
    "streaming_lstm_backward": ("_flashlstm", "streaming_lstm_backward"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        mod, attr = _LAZY[name]
        value = getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
        globals()[name] = value  # the function wins over the submodule of the same name
        return value
    raise AttributeError(name)
