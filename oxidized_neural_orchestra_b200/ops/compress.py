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
        lib.ono_sparse_mask.argtypes = [vp, ll, vp, vp, vp, ci, vp, vp]
        lib.ono_sparse_lift_range.argtypes = [vp, ll, ll, vp, vp, vp, cu, vp, ci, vp, vp]
        lib.ono_sparse_lift_range.restype = ci
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


def wire_mask(residual: torch.Tensor, wire: torch.Tensor | None = None, thr: torch.Tensor | None = None,
              sent: torch.Tensor | None = None, wire16: torch.Tensor | None = None, stream=None) -> None:
    """The entries that are sent (all of them without ``thr``) go to ``wire`` (f32, rounded through f16) and / or ``wire16``
    (float16 or bfloat16: the buffer peers read over NVLink) and are zeroed in ``residual``; the rest stays as residual."""
    if wire is None and wire16 is None:
        raise ValueError("wire_mask needs a wire buffer")
    _lib.check(_fn().ono_sparse_mask(residual.data_ptr(), residual.numel(), None if thr is None else thr.data_ptr(),
                                     None if wire is None else wire.data_ptr(), None if wire16 is None else wire16.data_ptr(),
                                     int(wire16 is not None and wire16.dtype == torch.float16),
                                     None if sent is None else sent.data_ptr(), _lib.stream_ptr(stream)), "ono_sparse_mask")


def sparse_compact(x: torch.Tensor, thr: torch.Tensor, capacity: int, zero_sent: bool = True, stream=None, out=None,
                   scratch: torch.Tensor | None = None):
    """Returns (idx uint32-as-int32 tensor, f16 values, count tensor) of the entries with |x| >= thr, ascending.
    ``out=(idx, val, count)`` writes into existing buffers (e.g. regions of this rank's window that peers read)."""
    n = x.numel()
    if scratch is None:
        scratch = torch.empty((n + 1023) // 1024, device=x.device, dtype=torch.int32)
    if out is not None:
        idx, val, count = out
        capacity = idx.numel()
    else:
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


def sparse_lift_range(acc: torch.Tensor, begin: int, end: int, idx_ptr: int, val_ptr: int, count_ptr: int, capacity: int,
                      dense16_ptr: int, dense_f16: bool, bytes_out: torch.Tensor | None = None, stream=None) -> None:
    """One sender's contribution to the owned range ``[begin, end)`` of the local accumulator ``acc``: the part of the
    sender's ascending (index, f16) list inside the range, or that range of its dense 16-bit wire if its selection did
    not fit the list. The sender's buffers are given as addresses (they may be a peer GPU's window)."""
    _lib.check(_fn().ono_sparse_lift_range(acc.data_ptr(), begin, end, idx_ptr, val_ptr, count_ptr, capacity, dense16_ptr,
                                           int(dense_f16), None if bytes_out is None else bytes_out.data_ptr(),
                                           _lib.stream_ptr(stream)), "ono_sparse_lift_range")
