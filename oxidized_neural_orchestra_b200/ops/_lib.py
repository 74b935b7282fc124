"""ctypes view of ``libono_kernels.so`` (the sm_100a kernel library built in-tree).

The library is loaded lazily. On a machine with a GPU a missing library is an error, never a
silent fallback: the ops in this package raise if they cannot reach their CUDA kernels.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libono_kernels.so"
_lib = None


class OnoEpilogue(C.Structure):
    _fields_ = [
        ("out_f32", C.c_void_p), ("outT_f32", C.c_void_p), ("out_bf16", C.c_void_p),
        ("outT_bf16", C.c_void_p), ("pre_f32", C.c_void_p), ("pre_bf16", C.c_void_p),
        ("bias", C.c_void_p), ("aux_f32", C.c_void_p), ("aux_bf16", C.c_void_p),
        ("ld_out", C.c_int), ("ld_outT", C.c_int), ("ld_aux", C.c_int),
        ("act", C.c_int), ("act_param", C.c_float), ("dact", C.c_int), ("dact_param", C.c_float),
        ("relu_quirk", C.c_int), ("alpha", C.c_float), ("beta", C.c_float),
    ]


class OnoGemm(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("lda", C.c_int), ("ldb", C.c_int), ("dtype", C.c_int), ("a_major", C.c_int),
        ("b_major", C.c_int), ("bn", C.c_int), ("max_ctas", C.c_int), ("epi", OnoEpilogue),
        ("status", C.c_void_p),
    ]


def lib_path() -> Path:
    return _LIB_PATH


def load():
    """Return the loaded kernel library, raising if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: run `python -m oxidized_neural_orchestra_b200.build`")
        _lib = C.CDLL(str(_LIB_PATH))
        _lib.ono_last_error.restype = C.c_char_p
        _lib.ono_gemm.argtypes = [C.POINTER(OnoGemm), C.c_void_p]
        _lib.ono_gemm.restype = C.c_int
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().ono_last_error().decode()
        raise RuntimeError(f"{what} failed (rc={rc}): {msg}")


def stream_ptr(stream=None) -> int:
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream
