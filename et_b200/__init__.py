"""B200-native E.T. encoder hot path: ctypes binding of the C-ABI library `libet_b200.so`.

The library holds hand-written sm_100a CUDA kernels and the host-side C++ that mirrors the
reference's Linear/encoder objects. There is no CPU fallback: every op raises if the library is
missing or a call fails. torch is used only to own device memory and streams.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# ET_B200_LIB points the binding at another build of the library (e.g. a profiling build)
LIB_PATH = os.environ.get("ET_B200_LIB") or os.path.join(_HERE, "libet_b200.so")
INCLUDE_DIR = os.path.join(os.path.dirname(_HERE), "include")

_lib = None


class EtError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"et_b200 status {code}: {text}")
        self.code = code


def lib():
    """Loads the C-ABI library (built in-tree by et_b200/build.py); raises if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EtError(-1, f"{LIB_PATH} is missing: run `python et_b200/build.py` (needs nvcc)")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.et_last_error.restype = ctypes.c_char_p
    return _lib


def check(code):
    if code != 0:
        raise EtError(code, lib().et_last_error().decode("utf-8", "replace"))


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array / None as c_void_p."""
    if t is None:
        return ctypes.c_void_p(0)
    if hasattr(t, "data_ptr"):
        return ctypes.c_void_p(t.data_ptr())
    return ctypes.c_void_p(t.ctypes.data)


def stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


from .ops import *  # noqa: E402,F401
