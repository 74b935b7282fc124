"""Python entries to the gradient-compression kernels (``csrc/kernels/compress.cu``): the f16 wire and the
sparse serializer of the reference (comms/src/handles/compressor.rs:71-118, comms/src/sparse/protocol.rs:33-144)."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_declared = False


def _fn():
    global _declared
    lib = _lib.load()
    if not _declared:
        vp, ll, cf, ull, ci, cu = C.c_void_p, C.c_longlong, C.c_float, C.c_ulonglong, C.c_int, C.c_uint
        lib.ono_sparse_threshold.argtypes = [vp, ll, cf, ull, vp, vp]
        lib.ono_sparse_mask.argtypes = [vp, ll, vp, vp, vp, vp]
        lib.ono_sparse_compact.argtypes = [vp, ll, vp, vp, vp, vp, cu, vp, ci, vp]
        lib.ono_sparse_lift.argtypes = [vp, ll, vp, vp, vp, cu, vp]
        for f in (lib.ono_sparse_threshold, lib.ono_sparse_mask, lib.ono_sparse_compact, lib.ono_sparse_lift):
            f.restype = ci
        _declared = True
    return lib


def sparse_threshold(x: torch.Tensor, r: float, seed: int, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """Device scalar: the magnitude above which entries of ``x`` are sent (keep ratio ``r`` of the largest)."""
    out = torch.empty(1, device=x.device) if out is None else out
    _lib.check(_fn().ono_sparse_threshold(x.data_ptr(), x.numel(), float(r), int(seed) & (2**64 - 1), out.data_ptr(),
                                          _lib.stream_ptr(stream)), "ono_sparse_threshold")
    return out


def wire_mask(residual: torch.Tensor, wire: torch.Tensor, thr: torch.Tensor | None = None, sent: torch.Tensor | None = None,
              stream=None) -> None:
    """``wire`` = f16-rounded entries that are sent (all of them without ``thr``); they are zeroed in ``residual``."""
    _lib.check(_fn().ono_sparse_mask(residual.data_ptr(), residual.numel(), None if thr is None else thr.data_ptr(),
                                     wire.data_ptr(), None if sent is None else sent.data_ptr(), _lib.stream_ptr(stream)),
               "ono_sparse_mask")


def sparse_compact(x: torch.Tensor, thr: torch.Tensor, capacity: int, zero_sent: bool = True, stream=None):
    """Returns (idx uint32-as-int32 tensor, f16 values, count tensor) of the entries with |x| >= thr, ascending."""
    n = x.numel()
    scratch = torch.empty((n + 1023) // 1024, device=x.device, dtype=torch.int32)
    idx = torch.empty(capacity, device=x.device, dtype=torch.int32)
    val = torch.empty(capacity, device=x.device, dtype=torch.float16)
    count = torch.zeros(1, device=x.device, dtype=torch.int32)
    _lib.check(_fn().ono_sparse_compact(x.data_ptr(), n, thr.data_ptr(), scratch.data_ptr(), idx.data_ptr(), val.data_ptr(),
                                        capacity, count.data_ptr(), int(zero_sent), _lib.stream_ptr(stream)), "ono_sparse_compact")
    return idx, val, count


def sparse_lift(acc: torch.Tensor, idx: torch.Tensor, val: torch.Tensor, count: torch.Tensor, stream=None) -> None:
    """``acc[idx[i]] += val[i]`` for the first ``count`` pairs."""
    _lib.check(_fn().ono_sparse_lift(acc.data_ptr(), acc.numel(), idx.data_ptr(), val.data_ptr(), count.data_ptr(), idx.numel(),
                                     _lib.stream_ptr(stream)), "ono_sparse_lift")
