"""Python entries to the convolution / pooling gather-scatter kernels (``csrc/kernels/conv.cu``).

Image activations are pixel-major 2-D tensors ``[B*H*W, ld]`` (channels contiguous). The convolution
itself is ``cols @ K^T`` on the tcgen05 GEMM; these kernels build ``cols`` (im2col), fold the column
gradient back (col2im), pool, and convert to and from the flattened NCHW rows dense layers use.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .gemm import ACT


class OnoConvGeom(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("B", "C", "H", "W", "K", "S", "P", "OH", "OW")]


_declared = False


def _fn():
    global _declared
    lib = _lib.load()
    if not _declared:
        vp, ci, cf, ll = C.c_void_p, C.c_int, C.c_float, C.c_longlong
        G = C.POINTER(OnoConvGeom)
        lib.ono_im2col.argtypes = [G, ci, vp, ci, vp, ci, vp, ci, vp]
        lib.ono_col2im.argtypes = [G, ci, vp, ci, vp, ci, ci, cf, ci, vp, ci, vp, ci, vp]
        lib.ono_pool_fwd.argtypes = [G, ci, vp, ci, vp, ci, vp, ci, vp, ci, cf, vp]
        lib.ono_pool_bwd.argtypes = [G, ci, vp, ci, vp, ci, vp, ci, cf, ci, vp, ci, vp]
        lib.ono_nchw_flat.argtypes = [ci, ci, ci, ci, ci, vp, ci, vp, ci, vp, ci, vp, ci, ci, cf, ci, vp]
        lib.ono_finish_delta.argtypes = [ci, ll, ci, vp, ci, vp, ci, ci, cf, ci, vp, ci, vp, ci, vp]
        lib.ono_conv1_fwd.argtypes = [G, ci, ci, vp, ci, vp, vp, ci, cf, vp, ci, vp]
        lib.ono_conv1_wgrad.argtypes = [G, ci, ci, vp, ci, vp, ci, vp, vp, cf, vp]
        lib.ono_conv1_fwd.restype = lib.ono_conv1_wgrad.restype = ci
        lib.ono_conv_kperm.argtypes = [ci, ci, ci, ci, ci, vp, ci, vp, ci, vp, ci, cf, vp]
        lib.ono_conv_kperm.restype = ci
        for f in (lib.ono_im2col, lib.ono_col2im, lib.ono_pool_fwd, lib.ono_pool_bwd, lib.ono_nchw_flat, lib.ono_finish_delta):
            f.restype = ci
        _declared = True
    return lib


def geom(B, C_, H, W, K, S, P) -> OnoConvGeom:
    g = OnoConvGeom()
    g.B, g.C, g.H, g.W, g.K, g.S, g.P = B, C_, H, W, K, S, P
    g.OH = (H + 2 * P - K) // S + 1
    g.OW = (W + 2 * P - K) // S + 1
    return g


def _dt(t: torch.Tensor) -> int:
    return 0 if t.dtype == torch.float32 else 1


def _p(t):
    return None if t is None else t.data_ptr()


def _ld(t):
    return 0 if t is None else t.stride(0)


def im2col(g, x, cols, cols_t=None, stream=None):
    lib = _fn()
    _lib.check(lib.ono_im2col(C.byref(g), _dt(x), x.data_ptr(), x.stride(0), cols.data_ptr(), cols.stride(0), _p(cols_t),
                              _ld(cols_t), _lib.stream_ptr(stream)), "ono_im2col")


def col2im(g, dcols, dx, dx_t=None, aux=None, dact=None, dact_param=0.0, relu_quirk=False, stream=None):
    lib = _fn()
    _lib.check(lib.ono_col2im(C.byref(g), _dt(dcols), dcols.data_ptr(), dcols.stride(0), _p(aux), _ld(aux), ACT[dact],
                              dact_param, int(relu_quirk), dx.data_ptr(), dx.stride(0), _p(dx_t), _ld(dx_t),
                              _lib.stream_ptr(stream)), "ono_col2im")


def pool_fwd(g, x, y, arg, y_t=None, act=None, act_param=0.0, stream=None):
    lib = _fn()
    _lib.check(lib.ono_pool_fwd(C.byref(g), _dt(x), x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), _p(y_t), _ld(y_t),
                                arg.data_ptr(), ACT[act], act_param, _lib.stream_ptr(stream)), "ono_pool_fwd")


def pool_bwd(g, d, y, arg, dx_f32, act=None, act_param=0.0, relu_quirk=False, stream=None):
    lib = _fn()
    _lib.check(lib.ono_pool_bwd(C.byref(g), _dt(d), d.data_ptr(), d.stride(0), y.data_ptr(), y.stride(0), arg.data_ptr(),
                                ACT[act], act_param, int(relu_quirk), dx_f32.data_ptr(), dx_f32.stride(0),
                                _lib.stream_ptr(stream)), "ono_pool_bwd")


def nchw_flat(B, C_, HW, to_flat, img, flat, out_t=None, aux=None, dact=None, dact_param=0.0, relu_quirk=False, stream=None):
    lib = _fn()
    _lib.check(lib.ono_nchw_flat(_dt(img), B, C_, HW, int(to_flat), img.data_ptr(), img.stride(0), flat.data_ptr(),
                                 flat.stride(0), _p(out_t), _ld(out_t), _p(aux), _ld(aux), ACT[dact], dact_param,
                                 int(relu_quirk), _lib.stream_ptr(stream)), "ono_nchw_flat")


def finish_delta(rows, C_, src_f32, dst, dst_t=None, aux=None, dact=None, dact_param=0.0, relu_quirk=False, stream=None):
    lib = _fn()
    _lib.check(lib.ono_finish_delta(_dt(dst), rows, C_, src_f32.data_ptr(), src_f32.stride(0), _p(aux), _ld(aux), ACT[dact],
                                    dact_param, int(relu_quirk), dst.data_ptr(), dst.stride(0), _p(dst_t), _ld(dst_t),
                                    _lib.stream_ptr(stream)), "ono_finish_delta")


def kernel_to_operand(F, C_, K, params_f32, dst, dst_t=None, stream=None):
    """K[F][C][k][k] (flat f32 parameters) -> GEMM operand rows in (ky, kx, c) order, plus its transpose."""
    lib = _fn()
    _lib.check(lib.ono_conv_kperm(F, C_, K, 0, _dt(dst), params_f32.data_ptr(), 0, dst.data_ptr(), dst.stride(0), _p(dst_t),
                                  _ld(dst_t), 0.0, _lib.stream_ptr(stream)), "ono_conv_kperm")


def operand_grad_to_kernel(F, C_, K, src_f32, grads_f32, beta=0.0, stream=None):
    """f32 weight gradient in operand order [F][(ky, kx, c)] -> parameter order K[F][C][k][k], dst = beta*dst + src."""
    lib = _fn()
    _lib.check(lib.ono_conv_kperm(F, C_, K, 1, 0, src_f32.data_ptr(), src_f32.stride(0), grads_f32.data_ptr(), 0, None, 0,
                                  float(beta), _lib.stream_ptr(stream)), "ono_conv_kperm")


def conv1_fwd(g, F, x, kparams_f32, bias_f32, y, act=None, act_param=0.0, stream=None):
    """Direct forward of a convolution with one input channel: y = act(conv(x, K) + b), K given in parameter order."""
    lib = _fn()
    _lib.check(lib.ono_conv1_fwd(C.byref(g), F, _dt(x), x.data_ptr(), x.stride(0), kparams_f32.data_ptr(), _p(bias_f32), ACT[act],
                                 act_param, y.data_ptr(), y.stride(0), _lib.stream_ptr(stream)), "ono_conv1_fwd")


def conv1_wgrad(g, F, x, dy, gk_f32, gb_f32, beta=0.0, stream=None):
    """Weight and bias gradient of a one-input-channel convolution, written in parameter order (g = beta*g + d)."""
    lib = _fn()
    _lib.check(lib.ono_conv1_wgrad(C.byref(g), F, _dt(x), x.data_ptr(), x.stride(0), dy.data_ptr(), dy.stride(0), gk_f32.data_ptr(),
                                   gb_f32.data_ptr(), float(beta), _lib.stream_ptr(stream)), "ono_conv1_wgrad")
