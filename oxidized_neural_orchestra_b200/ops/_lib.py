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
        ("bias", C.c_void_p), ("bias_bf16", C.c_void_p), ("aux_f32", C.c_void_p), ("aux_bf16", C.c_void_p),
        ("ld_out", C.c_int), ("ld_outT", C.c_int), ("ld_aux", C.c_int),
        ("act", C.c_int), ("act_param", C.c_float), ("dact", C.c_int), ("dact_param", C.c_float),
        ("relu_quirk", C.c_int), ("alpha", C.c_float), ("beta", C.c_float), ("reduce_out", C.c_int),
        ("out16_f16", C.c_int),
    ]


class OnoApply(C.Structure):
    _fields_ = [
        ("p", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p), ("p_bf16", C.c_void_p), ("ld", C.c_int),
        ("kind", C.c_int), ("lr", C.c_float), ("mu", C.c_float), ("b1", C.c_float), ("b2", C.c_float),
        ("eps", C.c_float), ("grad_scale", C.c_float), ("adam_pows", C.c_void_p),
    ]


class OnoGemm(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
        ("lda", C.c_int), ("ldb", C.c_int), ("dtype", C.c_int), ("a_major", C.c_int),
        ("b_major", C.c_int), ("bn", C.c_int), ("max_ctas", C.c_int), ("split_k", C.c_int), ("pair", C.c_int), ("epi", OnoEpilogue),
        ("status", C.c_void_p), ("apply", OnoApply), ("gate", C.c_void_p), ("gate_target", C.c_void_p),
        ("gate_stride", C.c_int), ("gate_mask", C.c_uint), ("timeout_ns", C.c_ulonglong), ("workspace", C.c_void_p), ("workspace_elems", C.c_longlong),
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
        _declare(_lib)
    return _lib


def _declare(lib) -> None:
    vp, ci, cf, ll, ull = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_ulonglong
    sigs = {
        "ono_loss": [C.POINTER(OnoLoss), vp],
        "ono_colsum": [vp, ci, ci, ci, ci, vp, cf, vp],
        "ono_softmax": [C.POINTER(OnoSoftmax), vp],
        "ono_optim": [C.POINTER(OnoOptim), vp],
        "ono_adam_tick": [vp, cf, cf, vp],
        "ono_local_sgd": [vp, vp, vp, ll, cf, vp, vp],
        "ono_sumsq": [vp, ll, vp, vp],
        "ono_init": [vp, ll, ull, ull, ci, cf, cf, vp],
        "ono_rows": [C.POINTER(OnoRows), vp],
        "ono_sync_step": [C.POINTER(OnoSync), vp],
        "ono_sync_step_emulated": [C.POINTER(OnoSync), vp],
        "ono_ps_async_step": [C.POINTER(OnoPsAsync), vp],
        "ono_ring_allreduce": [C.POINTER(OnoRing), vp],
        "ono_ring_allreduce_emulated": [vp, vp],
        "ono_pingpong": [ci, vp, vp, ci, C.c_uint, vp, vp, vp],
        "ono_push_add": [vp, vp, ll, vp],
        "ono_cast16": [vp, vp, ll, ci, vp],
        "ono_copy_async": [vp, vp, ll, vp],
        "ono_stage_pull": [C.POINTER(OnoStagePull), vp],
        "ono_stage_signal": [C.POINTER(vp), ci, ci, ci, vp, vp],
        "ono_stage_tick": [vp, vp],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ci
    lib.ono_num_sms.restype = ci
    lib.ono_sizeof.argtypes = [ci]
    lib.ono_sizeof.restype = ci
    for i, st in enumerate((OnoGemm, OnoLoss, OnoOptim, OnoRows, OnoSync, OnoPsAsync, OnoRing, OnoStagePull, OnoRingEmu)):
        if lib.ono_sizeof(i) != C.sizeof(st):
            raise RuntimeError(f"ABI mismatch for {st.__name__}: C {lib.ono_sizeof(i)} vs ctypes {C.sizeof(st)}")


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().ono_last_error().decode()
        raise RuntimeError(f"{what} failed (rc={rc}): {msg}")


def stream_ptr(stream=None) -> int:
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


# --------------------------------------------------------------------------------------------
# Structures of the elementwise and collective entry points (field order mirrors ono_kernels.h).
# --------------------------------------------------------------------------------------------
MAX_RANKS = 8
MAX_RANGES = 16


class OnoLoss(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("y", C.c_void_p), ("aux", C.c_void_p),
        ("B", C.c_int), ("C", C.c_int), ("ld", C.c_int), ("ldy", C.c_int),
        ("kind", C.c_int), ("softmax", C.c_int),
        ("dact", C.c_int), ("dact_param", C.c_float), ("relu_quirk", C.c_int),
        ("eps", C.c_float),
        ("probs", C.c_void_p), ("d_f32", C.c_void_p), ("dT_f32", C.c_void_p),
        ("d_bf16", C.c_void_p), ("dT_bf16", C.c_void_p),
        ("ld_d", C.c_int), ("ld_dT", C.c_int),
        ("loss_sum", C.c_void_p), ("correct", C.c_void_p),
    ]


class OnoSoftmax(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("ld_x", C.c_int), ("p_f32", C.c_void_p), ("p_bf16", C.c_void_p), ("ld_p", C.c_int),
        ("B", C.c_int), ("C", C.c_int), ("backward", C.c_int),
        ("out_f32", C.c_void_p), ("out_bf16", C.c_void_p), ("outT_f32", C.c_void_p), ("outT_bf16", C.c_void_p),
        ("ld_out", C.c_int), ("ld_outT", C.c_int),
    ]


class OnoOptim(C.Structure):
    _fields_ = [
        ("p", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
        ("n", C.c_longlong), ("kind", C.c_int),
        ("lr", C.c_float), ("mu", C.c_float), ("b1", C.c_float), ("b2", C.c_float), ("eps", C.c_float),
        ("grad_scale", C.c_float), ("adam_pows", C.c_void_p), ("p_bf16", C.c_void_p),
        ("zero_grad", C.c_int),
    ]


class OnoRows(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("ld_src", C.c_int), ("idx", C.c_void_p), ("R", C.c_int), ("W", C.c_int),
        ("dst_f32", C.c_void_p), ("dstT_f32", C.c_void_p), ("dst_bf16", C.c_void_p),
        ("dstT_bf16", C.c_void_p), ("ld_dst", C.c_int), ("ld_dstT", C.c_int),
    ]


class OnoRange(C.Structure):
    _fields_ = [("begin", C.c_longlong), ("end", C.c_longlong)]


STAGE_BUCKETS = 64


class OnoStagePull(C.Structure):
    _fields_ = [
        ("nranks", C.c_int), ("rank", C.c_int), ("nblocks", C.c_int), ("bucket", C.c_int),
        ("src", C.c_void_p * MAX_RANKS), ("dst", C.c_void_p * MAX_RANKS),
        ("n_ranges", C.c_int), ("ranges", OnoRange * MAX_RANGES),
        ("ready", C.c_void_p), ("step", C.c_void_p),
        ("status", C.c_void_p), ("timeout_ns", C.c_ulonglong),
    ]


class OnoSyncLocal(C.Structure):
    _fields_ = [
        ("p_master", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p), ("state_off", C.c_longlong),
        ("adam_pows", C.c_void_p), ("epoch", C.c_void_p), ("sumsq", C.c_void_p), ("status", C.c_void_p),
        ("fwd", C.c_void_p), ("n_ranges", C.c_int), ("ranges", OnoRange * MAX_RANGES),
    ]


class OnoSync(C.Structure):
    _fields_ = [
        ("nranks", C.c_int), ("rank", C.c_int), ("algo", C.c_int), ("nblocks", C.c_int),
        ("n", C.c_longlong),
        ("g", C.c_void_p * MAX_RANKS), ("p_out_f32", C.c_void_p * MAX_RANKS),
        ("p_out_bf16", C.c_void_p * MAX_RANKS), ("flags", C.c_void_p * MAX_RANKS),
        ("g_mc", C.c_void_p), ("p_mc_f32", C.c_void_p), ("p_mc_bf16", C.c_void_p),
        ("worker_mask", C.c_uint), ("member_mask", C.c_uint), ("live_mask", C.c_void_p),
        ("n_workers", C.c_int),
        ("kind", C.c_int), ("lr", C.c_float), ("mu", C.c_float), ("b1", C.c_float), ("b2", C.c_float),
        ("eps", C.c_float),
        ("divide", C.c_int), ("zero_grad", C.c_int), ("g_dtype", C.c_int), ("timeout_ns", C.c_ulonglong),
        ("loc", OnoSyncLocal * MAX_RANKS),
    ]


class OnoPsAsync(C.Structure):
    _fields_ = [
        ("nranks", C.c_int), ("rank", C.c_int), ("nblocks", C.c_int),
        ("g", C.c_void_p), ("p_local_f32", C.c_void_p), ("p_local_bf16", C.c_void_p),
        ("master", C.c_void_p * MAX_RANKS), ("m", C.c_void_p * MAX_RANKS), ("v", C.c_void_p * MAX_RANKS),
        ("state_off", C.c_longlong * MAX_RANKS), ("locks", C.c_void_p * MAX_RANKS),
        ("n_ranges", C.c_int * MAX_RANKS), ("ranges", (OnoRange * MAX_RANGES) * MAX_RANKS),
        ("n_workers", C.c_int), ("divide", C.c_int),
        ("kind", C.c_int), ("lr", C.c_float), ("mu", C.c_float), ("b1", C.c_float), ("b2", C.c_float),
        ("eps", C.c_float), ("adam_pows", C.c_void_p),
        ("status", C.c_void_p), ("timeout_ns", C.c_ulonglong),
    ]


class OnoRing(C.Structure):
    _fields_ = [
        ("nranks", C.c_int), ("rank", C.c_int), ("nblocks", C.c_int), ("n", C.c_longlong),
        ("g", C.c_void_p), ("acc", C.c_void_p * MAX_RANKS), ("flags", C.c_void_p * MAX_RANKS),
        ("epoch", C.c_void_p),
        ("p", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p), ("adam_pows", C.c_void_p),
        ("p_bf16", C.c_void_p),
        ("kind", C.c_int), ("lr", C.c_float), ("mu", C.c_float), ("b1", C.c_float), ("b2", C.c_float),
        ("eps", C.c_float),
        ("status", C.c_void_p), ("timeout_ns", C.c_ulonglong),
    ]


class OnoRingEmu(C.Structure):
    _fields_ = [
        ("nranks", C.c_int), ("nblocks", C.c_int), ("n", C.c_longlong),
        ("g", C.c_void_p * MAX_RANKS), ("acc", C.c_void_p * MAX_RANKS), ("flags", C.c_void_p * MAX_RANKS),
        ("epoch", C.c_void_p * MAX_RANKS), ("p", C.c_void_p * MAX_RANKS), ("m", C.c_void_p * MAX_RANKS),
        ("v", C.c_void_p * MAX_RANKS), ("p_bf16", C.c_void_p * MAX_RANKS), ("adam_pows", C.c_void_p),
        ("kind", C.c_int), ("lr", C.c_float), ("mu", C.c_float), ("b1", C.c_float), ("b2", C.c_float), ("eps", C.c_float),
        ("status", C.c_void_p), ("timeout_ns", C.c_ulonglong),
    ]
