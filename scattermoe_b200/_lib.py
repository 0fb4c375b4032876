"""ctypes binding of the C-ABI library (include/scattermoe_b200.h).

The library is the only implementation: there is no PyTorch or CPU fallback. If it cannot be loaded the
import of any op fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p

import torch

from . import build as _build

_lock = threading.Lock()
_lib = None

ABI_VERSION = 4          # SMOE_ABI_VERSION of include/scattermoe_b200.h this binding was written against

SMOE_OK = 0
SMOE_ERR_BAD_ARG = 1
SMOE_ERR_UNSUPPORTED = 2

FLAG_ALLOW_TF32 = 1
FLAG_FORCE_SIMT = 2
FLAG_FORCE_TC = 4
FLAG_GATHER_ROWS = 8

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}

_P, _I64, _I32 = c_void_p, c_int64, c_int32

# name -> argtypes; every symbol declared in include/scattermoe_b200.h
SIGNATURES = {
    "smoe_version": ([], c_int32),
    "smoe_last_error": ([], c_char_p),
    "smoe_last_path_was_tensor_core": ([], c_int32),
    "smoe_sort_count_workspace_bytes": ([_I64, _I32], c_size_t),
    "smoe_sort_count": ([_P, _I64, _I32, _P, _P, _P, _P, c_size_t, _P], c_int32),
    "smoe_sort_count_static_capacity": ([], c_int64),
    "smoe_sort_count_static": ([_P, _I64, _I32, _P, _P, _P, _P], c_int32),
    "smoe_route_topk_workspace_bytes": ([_I64, _I32, _I32], c_size_t),
    "smoe_route_topk": ([_P, _I64, _I32, _I64, _I32, _I32, _I32, _I32, _P, _P, _P, _P, _P, _P, _P, c_size_t, _P], c_int32),
    "smoe_offsets_from_sorted": ([_P, _I64, _I32, _P, _P], c_int32),
    "smoe_scatter2scatter": ([_P, _I64, _I64, _I64,          # X
                              _P, _I64, _I64, _I64,          # W
                              _P, _I64, _I64,                # bias
                              _P, _I64, _I64,                # Y
                              _P, _P, _P,                    # index tensors
                              _I64, _I32, _I32, _I32, _I32,  # R K N E fan_out
                              _I32, _I32, _I32, _I32,        # x_grouped y_grouped dtype flags
                              _P, _P], c_int32),
    "smoe_group_bwd_w": ([_P, _I64, _I64,                    # DY
                          _P, _I64, _I64, _I64,              # X
                          _P, _P, _I32,                      # offsets, gather idx, fan_out
                          _P, _I64, _I64, _I64,              # DW
                          _P, _I64, _I64,                    # Db
                          _I64, _I32, _I32, _I32, _I32, _I32,  # R K N E dtype flags
                          _P, _P], c_int32),
    "smoe_group": ([_P, _I64, _I64, _I64, _P, _P, _I32, _P, _I64, _I64, _I64, _I32, _I32, _P], c_int32),
    "smoe_topk_reduce": ([_P, _I64, _P, _I64, _I64, _P, _I64, _I64, _I32, _I32, _I32, _P], c_int32),
    "smoe_gate_grad": ([_P, _I64, _P, _I64, _P, _I64, _I64, _I64, _I32, _I32, _I32, _P], c_int32),
    "smoe_activation_forward": ([_P, _I64, _P, _I64, _I64, _P, _I32, _I32, _I32, c_float, c_float, _I32, _P], c_int32),
    "smoe_activation_backward": ([_P, _I64, _P, _I64, _P, _I64, _I64, _P, _I32, _I32, _I32, c_float, c_float, _I32, _P],
                                 c_int32),
    "smoe_scatter2scatter_act": ([_P, _I64, _I64, _I64, _P, _I64, _I64, _I64, _P, _I64, _I64, _P, _I64, _I64, _P, _I64,
                                  _P, _P, _P, _I64, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, c_float, c_float,
                                  _P, _P, _P], c_int32),
    "smoe_scatter2scatter_act_bwd": ([_P, _I64, _I64, _P, _I64, _I64, _I64, _P, _I64, _P, _I64, _P, _I64, _I32, _I32, _I32,
                                      _I32, _I32, _I32, _I32, c_float, c_float, _P, _P, _P, _P, _P], c_int32),
    "smoe_act_bwd_partial_lines": ([_I32], c_int32),
    "smoe_gate_grad_from_partials": ([_P, _I32, _I64, _P, _P, _I32, _P], c_int32),
    "smoe_single2scatter": ([_P, _I64, _I64, _I64, _P, _I64, _I64, _I64, _P, _I64, _I64, _P, _I32, _I32, _I32, _I32, _I32, _P],
                            c_int32),
    "smoe_ep_dispatch": ([_P, _I64, _I64, _P, _P, _P, _P, _P, _I32, _P, _I64, _I64, _P, _I32, _I64, _I32, _I32, _I32, _I32,
                          _P], c_int32),
    "smoe_ep_plan_rows": ([_P, _I32, _I32, _I32, _P, _P, _P], c_int32),
    "smoe_ep_return": ([_P, _I64, _P, _P, _I64, _P, _I64, _I64, _I32, _I32, _I32, _I32, _I32, _P], c_int32),
    "smoe_scatter2scatter_to_peers": ([_P, _I64, _I64, _I64, _P, _I64, _I64, _I64, _P, _P, _P, _I64, _I64, _I32, _I32,
                                       _I32, _I32, _I32, _I32, _I32, _P, _P], c_int32),
    "smoe_ep_barrier": ([_P, _I32, _I32, _I32, _I64, _P, _P], c_int32),
    "smoe_ep_tokmeta_ints": ([_I32], c_int32),
    "smoe_ep_plan_tokens": ([_P, _P, _I64, _I32, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I32, _I32, _I32, _I32,
                             _P], c_int32),
    "smoe_ep_dispatch_meta": ([_P, _P, _P, _P, _P, _P, _I32, _P, _I64, _I32, _I64, _I32, _I32, _I32, _P], c_int32),
    "smoe_ep_expand": ([_P, _I64, _I64, _P, _P, _I64, _I32, _P, _I64, _P, _I64, _P, _I64, _I32, _I32, _I32, _P], c_int32),
    "smoe_ep_combine": ([_P, _I64, _I64, _P, _P, _I64, _P, _I32, _P, _I64, _I64, _I32, _I32, _I32, _I32, _I32, _P], c_int32),
    "smoe_ep_sum_parts": ([_P, _I64, _P, _I32, _P, _I64, _I64, _I32, _I32, _P], c_int32),
    "smoe_status_poison": ([_P, _P, _I64, _P], c_int32),
}


def library_path() -> str:
    return _build.LIB_PATH


def load():
    """Load (building first if the shared object is absent) and return the ctypes library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.LIB_PATH
        if not os.path.exists(path):
            try:
                _build.build()
            except Exception as e:  # no nvcc, or a compile error
                raise ImportError(
                    "scattermoe_b200: the CUDA library %s is missing and could not be built (%s). "
                    "Run `python -m scattermoe_b200.build`; there is no fallback implementation." % (path, e)
                ) from e
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise ImportError("scattermoe_b200: cannot load %s: %s" % (path, e)) from e
        for name, (argtypes, restype) in SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as e:
                raise ImportError("scattermoe_b200: %s does not export %s (stale build?)" % (path, name)) from e
            fn.argtypes = argtypes
            fn.restype = restype
        if lib.smoe_version() != ABI_VERSION:
            raise ImportError("scattermoe_b200: %s has ABI version %d, this package needs %d (stale build: run "
                              "`python -m scattermoe_b200.build --force`)" % (path, lib.smoe_version(), ABI_VERSION))
        _lib = lib
        return _lib


def last_error() -> str:
    msg = load().smoe_last_error()
    return msg.decode() if msg else ""


def check(rc: int, what: str):
    """Turn a non-zero status into the exception class the reference would raise for the same mistake:
    AssertionError for shape contract violations (the reference only has `assert`s, ops.py:124-125, :132,
    :380), RuntimeError for everything else."""
    if rc == SMOE_OK:
        return
    msg = "%s failed (status %d): %s" % (what, rc, last_error())
    if rc == SMOE_ERR_BAD_ARG:
        raise AssertionError(msg)
    raise RuntimeError(msg)


def on_device(t: torch.Tensor) -> bool:
    """True for tensors the kernels can take. One predicate for every "is this a GPU tensor" branch of the package,
    so that host-only tests can trace those branches with stand-in tensors."""
    return t.is_cuda


def require_cuda(t: torch.Tensor, name: str):
    if not on_device(t):
        raise RuntimeError(
            "scattermoe_b200: `%s` is on %s; this package runs on CUDA (sm_100a) only and has no CPU path"
            % (name, t.device))


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_status_words = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] the tensor-core kernels write when one of their bounded waits gives up."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = t
    return t


def check_device_status(device=None):
    """Synchronise and raise if a kernel reported a timed-out wait since the last check."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    t = status_word(device)
    vals = t.tolist()
    if vals[0] != 0:
        t.zero_()
        raise RuntimeError("scattermoe_b200: a kernel gave up waiting on the device (status %s)" % (vals,))
