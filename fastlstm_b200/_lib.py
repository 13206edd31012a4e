"""ctypes binding of libfastlstm_b200.so (the C ABI in include/fastlstm_b200.h).

There is no fallback: if the library is missing or cannot be loaded, importing
an operator raises.  Build it with `python -m fastlstm_b200.build`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int32, c_size_t, c_void_p, POINTER, Structure

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libfastlstm_b200.so")

ABI_VERSION = 1
F32, F16, BF16 = 0, 1, 2
DTYPE_CODE = {"fp32": F32, "fp16": F16, "bf16": BF16}
PHASE_FWD, PHASE_BWD, PHASE_FWD_OP = 0, 1, 2
FLAG_FORCE_GENERIC = 1
FLAG_INFERENCE = 8
FLAG_NO_FUSED = 32        # blstm_fwd: keep tiny sizes on projection + recurrence
FLAG_NO_CLUSTER = 16      # forward: keep small hidden sizes on the general kernel
FLAG_HALF_DEVICE = 128    # recurrences: plan for half of the SMs (two persistent kernels side by side)
FLAG_TEST_NO_ARRIVE = 4   # test hook: no CTA signals step completion (every wait runs out)

OK = 0
E_WAIT_TIMEOUT = 6
E_TOO_LARGE = 8


class Desc(Structure):
    _fields_ = [("dtype", c_int32), ("seq_len", c_int32), ("batch", c_int32),
                ("input_size", c_int32), ("hidden_size", c_int32), ("flags", c_int32),
                ("wait_limit_us", c_int32), ("reserved", c_int32)]


# name -> (restype, argtypes); every symbol include/fastlstm_b200.h declares
P = c_void_p
DP = POINTER(Desc)
SIGNATURES = {
    "blstm_abi_version": (c_int, []),
    "blstm_strerror": (c_char_p, [c_int]),
    "blstm_last_cuda_error": (c_char_p, []),
    "blstm_device_check": (c_int, [c_int]),
    "blstm_workspace_bytes": (c_size_t, [DP, c_int]),
    "blstm_plan_name": (c_char_p, [DP, c_int]),
    "blstm_plan_detail": (c_int, [DP, c_int, ctypes.c_char_p, c_size_t]),
    "blstm_input_projection": (c_int, [DP, P, P, P, P, P, P]),
    "blstm_fwd_recurrence": (c_int, [DP, P, P, P, P, P, c_size_t, P]),
    "blstm_fwd": (c_int, [DP, P, P, P, P, P, P, P, P, P, P, P, c_size_t, P]),
    "blstm_bwd_recurrence": (c_int, [DP, P, P, P, P, P, P, P, P, P, P, P, c_size_t, P]),
    "blstm_dgrad_input": (c_int, [DP, P, P, P, P, c_size_t, P]),
    "blstm_wgrad": (c_int, [DP, P, P, P, P, P, P, c_size_t, P]),
    "blstm_bias_grad": (c_int, [DP, P, P, P, c_size_t, P]),
    "blstm_bwd": (c_int, [DP] + [P] * 17 + [c_size_t, P]),
    "blstm_read_status": (c_int, [P, POINTER(c_int32), P]),
    "blstm_launch_count": (ctypes.c_ulonglong, []),
    "blstm_fwd_recurrence_static": (c_int, [DP, P, P, P, P, P]),
    "blstm_static_scratch_capacity": (c_size_t, []),
    "blstm_static_scratch_status": (c_int, [POINTER(c_int32), P]),
}

_lib = None


def load():
    """Load the shared library once; raise (never fall back) when unavailable."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} not found: the CUDA library is required (there is no CPU or "
            "PyTorch fallback). Build it with `python -m fastlstm_b200.build`.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.blstm_abi_version() != ABI_VERSION:
        raise RuntimeError("libfastlstm_b200.so ABI version mismatch; rebuild the library")
    _lib = lib
    return lib


def strerror(code: int) -> str:
    lib = load()
    msg = lib.blstm_strerror(code).decode()
    if code == 4:
        msg += ": " + lib.blstm_last_cuda_error().decode()
    return msg


class BlstmError(RuntimeError):
    def __init__(self, code, where=""):
        self.code = code
        super().__init__(f"fastlstm_b200 {where}: [{code}] {strerror(code)}")


def check(code: int, where: str = ""):
    if code != OK:
        raise BlstmError(code, where)
