"""ctypes binding of ``libvsa_b200.so`` (declared in ``include/vsa_b200.h``).

The library is built in-tree by ``python -m cudnn_vsa_b200.build``.  There is no fallback:
if the shared object is missing or an entry point fails, a ``RuntimeError`` says so.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int32, c_int64, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libvsa_b200.so"

_P, _I32, _I64, _F = c_void_p, c_int32, c_int64, c_float

# name -> (restype, argtypes); mirrors include/vsa_b200.h one to one.
SIGNATURES = {
    "vsa_abi_version": (_I32, []),
    "vsa_row_gather": (_I32, [_P, _P, _P, _I64, _I64, _P]),
    "vsa_row_scatter": (_I32, [_P, _P, _P, _I64, _I64, _P]),
    "vsa_slots_pool": (_I32, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I32, _P]),
    "vsa_slots_pool_strided": (_I32, [_P, _P, _P, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I32, _P]),
    "vsa_route_scratch_bytes": (_I64, [_I64, _I64, _I32]),
    "vsa_route": (_I32, [_P, _P, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _P, _I64, _I32, _P,
                         _I64, _P]),
    "vsa_selftest_wait_timeout": (_I32, [_P, _I64, _P]),
    "vsa_route_static": (_I32, [_P, _P, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _P, _I64, _I32, _P]),
    "vsa_fine_fwd": (_I32, [_P, _P, _P, _I64, _I64, _I32, _P, _P, _I64, _I64, _I32, _P, _F, _P, _P, _P, _P,
                            _P, _P, _P, _I64, _P, _P]),
    "vsa_fine_fwd_strided": (_I32, [_P, _P, _P, _I64, _I64, _I32, _P, _P, _I64, _I64, _I32, _P, _F, _P, _P, _P, _P,
                                    _P, _I64, _I64, _P, _P, _I64, _P, _P]),
    "vsa_fine_fwd_running": (_I32, [_P, _P, _P, _I64, _I64, _I32, _P, _P, _I64, _I64, _I32, _P, _F, _P, _P, _P, _P]),
    "vsa_fine_fwd_running_range": (_I32, [_P, _P, _P, _I64, _I64, _I32, _P, _P, _I64, _I64, _I32, _I32, _P, _F, _P,
                                          _P, _P, _P]),
    "vsa_merge_bwd": (_I32, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I32, _P]),
    "vsa_merge_bwd_strided": (_I32, [_P, _P, _I64, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I32, _P]),
    "vsa_kv_mask_words": (_I64, [_I64]),
    "vsa_fine_bwd": (_I32, [_P, _P, _P, _P, _I64, _I64, _I32, _P, _P, _I64, _I64, _I32, _P, _P, _F, _P, _P,
                            _P, _P, _P, _P, _I64, _I64, _P, _P, _P, _P, _P, _I32, _P, _P, _P, _P, _P, _I32,
                            _I32, _P, _P]),
    "vsa_fine_bwd_strided": (_I32, [_P, _P, _P, _P, _I64, _I64, _I32, _P, _P, _I64, _I64, _I32, _P, _P, _F, _P, _P,
                                    _P, _P, _P, _P, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _P, _I32, _P, _P, _I32,
                                    _P, _P]),
    "vsa_fine_bwd_range": (_I32, [_P, _P, _P, _P, _I64, _I64, _I32, _P, _P, _P, _I64, _I64, _I32, _I32, _P, _P, _F,
                                  _P, _P, _P, _I32, _I32, _P, _P, _P, _I32, _I32, _P, _P]),
    "vsa_list_bounds": (_I32, [_P, _P, _I64, _I32, _I32, _I32, _P, _P]),
    "vsa_partition_indices": (_I32, [_P, _P, _P, _P, _P, _I64, _I32, _I32, _I32, _I32, _I64, _I64, _P]),
    "vsa_merge_partial": (_I32, [_P, _P, _P, _P, _I64, _I32, _P]),
    "vsa_gate_merge": (_I32, [_P, _P, _P, _P, _P, _P, _P, _I64, _I32, _I64, _P]),
    "vsa_grad_finish": (_I32, [_P, _P, _P, _I32, _P, _P, _P, _I64, _I32, _I64, _P]),
}

_STATUS = {1: "bad argument", 2: "CUDA error", 3: "cuTensorMapEncodeTiled unavailable",
           4: "tensor map rejected", 5: "size beyond a documented limit",
           6: "the request does not fit the library's 16 MiB built-in scratch array"}

_lib = None

# Kernels launched by this process through `call` (the benchmark reports the count per step).
LAUNCHES = 0

# Per-entry-point device timing, off by default: while a `trace()` block is active every `call`
# is bracketed by two CUDA events on the current stream (`mark` brackets host-side regions such
# as a stream join the same way).
_TRACE = None


class trace:
    """``with _cabi.trace() as t: step()`` then ``t.summary()`` gives milliseconds and call counts
    per entry point, measured on the device between events recorded around each call."""

    def __enter__(self):
        global _TRACE
        self.records, self._outer = [], _TRACE
        _TRACE = self
        return self

    def __exit__(self, *exc):
        global _TRACE
        _TRACE = self._outer

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, start, stop in self.records:
            entry = out.setdefault(name, {"ms": 0.0, "calls": 0})
            entry["ms"] += start.elapsed_time(stop)
            entry["calls"] += 1
        return out


class mark:
    """Brackets a region of the current stream under ``name`` when a trace is active."""

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        self.start = None
        if _TRACE is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()

    def __exit__(self, *exc):
        if self.start is not None and _TRACE is not None:
            stop = torch.cuda.Event(enable_timing=True)
            stop.record()
            _TRACE.records.append((self.name, self.start, stop))


def load():
    """Return the loaded library, raising if it was not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m cudnn_vsa_b200.build` "
                "(the VSA path has no fallback implementation)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = lib
    return _lib


def ptr(tensor):
    """Device address of a tensor (``None`` passes a null pointer)."""
    return None if tensor is None else c_void_p(tensor.data_ptr())


def stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def call(name, *args, launches=1):
    """Invoke an int-returning entry point and raise on a nonzero status.

    ``launches`` is the number of kernels the call enqueues (one for most entry points).
    """
    global LAUNCHES
    if _TRACE is not None:
        with mark(name):
            rc = getattr(load(), name)(*args)
    else:
        rc = getattr(load(), name)(*args)
    LAUNCHES += launches
    if rc != 0:
        detail = _STATUS.get(rc, "unknown status")
        if rc == 2:
            detail += f" ({torch.cuda.get_device_name()}; check that the device is sm_100)"
        raise RuntimeError(f"{name} failed with status {rc}: {detail}")
