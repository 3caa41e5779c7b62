"""ctypes binding of libqfa_sm100a.so (the C ABI declared in include/qfa.h).

There is no fallback: if the shared library is missing or cannot be loaded, every
operator of this package raises.  Build it with `python -m quant_flash_attn_b200.build`.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libqfa_sm100a.so")

QFA_F16, QFA_BF16 = 0, 1
QFA_MODE_REF, QFA_MODE_INT8 = 0, 1

c_i64x3 = C.c_int64 * 3


class QfaQuantTensor(C.Structure):
    _fields_ = [("codes", C.c_void_p), ("stride", c_i64x3), ("scale", C.c_void_p),
                ("zp", C.c_void_p), ("rowsum", C.c_void_p)]


class QfaQuantJob(C.Structure):
    _fields_ = [("x", C.c_void_p), ("codes", C.c_void_p), ("scale_f16", C.c_void_p), ("zp", C.c_void_p),
                ("rowsum_or_null", C.c_void_p), ("dequant_or_null", C.c_void_p),
                ("Z", C.c_int64), ("H", C.c_int64), ("M", C.c_int64), ("D", C.c_int64),
                ("sx_z", C.c_int64), ("sx_h", C.c_int64), ("sx_m", C.c_int64), ("sx_k", C.c_int64),
                ("centered_or_null", C.c_void_p)]


class QfaFwdArgs(C.Structure):
    _fields_ = [("mode", C.c_int32), ("dtype", C.c_int32), ("causal", C.c_int32), ("sm_scale", C.c_float),
                ("B", C.c_int64), ("H", C.c_int64), ("Sq", C.c_int64), ("Skv", C.c_int64), ("D", C.c_int64),
                ("q", C.c_void_p), ("q_stride", c_i64x3),
                ("qq", QfaQuantTensor), ("k", QfaQuantTensor), ("v", QfaQuantTensor),
                ("v_hat", C.c_void_p), ("o", C.c_void_p), ("o_stride", c_i64x3),
                ("lse", C.c_void_p), ("lse_stride", C.c_int64), ("status", C.c_void_p), ("Hkv", C.c_int64),
                ("k_ctr", C.c_void_p)]


class QfaBwdArgs(C.Structure):
    _fields_ = [("mode", C.c_int32), ("dtype", C.c_int32), ("causal", C.c_int32), ("dkv_fused", C.c_int32),
                ("sm_scale", C.c_float),
                ("B", C.c_int64), ("H", C.c_int64), ("Sq", C.c_int64), ("Skv", C.c_int64), ("D", C.c_int64),
                ("q", C.c_void_p), ("q_stride", c_i64x3),
                ("qq", QfaQuantTensor), ("k", QfaQuantTensor), ("v", QfaQuantTensor),
                ("d_o", C.c_void_p), ("do_stride", c_i64x3),
                ("lse", C.c_void_p), ("delta", C.c_void_p), ("lse_stride", C.c_int64),
                ("dq", C.c_void_p), ("dq_stride", c_i64x3),
                ("dk", C.c_void_p), ("dk_stride", c_i64x3),
                ("dv", C.c_void_p), ("dv_stride", c_i64x3),
                ("dq_accum", C.c_void_p), ("status", C.c_void_p),
                ("q_hat", C.c_void_p), ("k_hat", C.c_void_p), ("v_hat", C.c_void_p)]


# name -> (restype, argtypes); every symbol include/qfa.h declares
_I64 = C.c_int64
SIGNATURES = {
    "qfa_quant_per_token": (C.c_int, [C.c_void_p] * 5 + [_I64] * 8 + [C.c_int, C.c_void_p]),
    "qfa_quant_dequant_per_token": (C.c_int, [C.c_void_p] * 6 + [_I64] * 8 + [C.c_int, C.c_void_p]),
    "qfa_center_per_token": (C.c_int, [C.c_void_p] * 3 + [_I64] * 7 + [C.c_void_p]),
    "qfa_quant_batch_per_token": (C.c_int, [C.POINTER(QfaQuantJob), C.c_int, C.c_int, C.c_void_p]),
    "qfa_dequant_per_token": (C.c_int, [C.c_void_p] * 4 + [_I64] * 7 + [C.c_int, C.c_void_p]),
    "qfa_attn_fwd": (C.c_int, [C.POINTER(QfaFwdArgs), C.c_void_p]),
    "qfa_attn_bwd_delta": (C.c_int, [C.c_void_p, C.POINTER(c_i64x3), C.c_void_p, C.POINTER(c_i64x3), C.c_void_p,
                                     _I64, _I64, _I64, _I64, _I64, C.c_int, C.c_void_p]),
    "qfa_attn_bwd": (C.c_int, [C.POINTER(QfaBwdArgs), C.c_void_p]),
    "qfa_attn_bwd_static_scratch": (C.c_int, [C.POINTER(QfaBwdArgs), C.c_void_p]),
    "qfa_static_scratch_capacity": (C.c_int64, []),
    "qfa_selftest_wait_timeout": (C.c_int, [C.c_uint64, C.c_void_p, C.c_void_p]),
    "qfa_probe_mma_rate": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double), C.c_void_p, C.c_void_p]),
    "qfa_strerror": (C.c_char_p, [C.c_int]),
    "qfa_last_cuda_error": (C.c_char_p, []),
    "qfa_version": (C.c_int, []),
    "qfa_launch_count": (C.c_int64, []),
}

_lib = None
_lock = threading.Lock()


def load():
    """Loads the shared library once; raises RuntimeError with build instructions if absent."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: the CUDA library is required (there is no CPU or PyTorch fallback). "
                "Build it with `python -m quant_flash_attn_b200.build`.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the export is missing
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        lib = load()
        msg = lib.qfa_strerror(rc).decode()
        if rc == -8:
            msg += ": " + lib.qfa_last_cuda_error().decode()
        raise RuntimeError(f"{what} failed: {msg} (code {rc})")


def launch_count() -> int:
    return int(load().qfa_launch_count())


# ----------------------------------------------------------------------------------------------- kernel status
# Every attention launch gets a status word.  It lives in pinned HOST memory, which the GPU writes directly
# (pinned memory is mapped into the device's address space), so it can be read back without a device
# synchronisation: each operator looks at it before its next launch on that device, and
# `raise_if_kernel_status(device, synchronize=True)` checks it on demand.
_status_words = {}


def status_word(device):
    """The (1,) int32 pinned host tensor that kernels launched on `device` report into."""
    import torch
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        with _lock:
            t = _status_words.get(idx)
            if t is None:
                t = torch.zeros(1, dtype=torch.int32).pin_memory()
                _status_words[idx] = t
    return t


def raise_if_kernel_status(device, synchronize: bool = False):
    """Raises if a kernel launched earlier on `device` reported a status (a bounded wait that ran out); the word
    is cleared, so the error is reported once.  With `synchronize` the device is synchronised first, so every
    launch made so far is covered."""
    import torch
    if synchronize:
        torch.cuda.synchronize(device)
    t = status_word(device)
    code = int(t[0])
    if code:
        t.zero_()
        raise RuntimeError(f"a qfa kernel on {torch.device(device)} reported status {code}: "
                           f"{load().qfa_strerror(code).decode()}; its outputs are not valid")
