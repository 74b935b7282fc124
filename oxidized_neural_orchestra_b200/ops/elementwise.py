"""Python entries to the bandwidth-bound CUDA kernels (``csrc/kernels/elementwise.cu``).

Each function launches exactly one kernel on the current (or given) stream and returns nothing;
they are graph-capturable. Reference semantics are cited in the CUDA source.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .gemm import ACT

OPT_KIND = {"sgd": 0, "gradient_descent": 0, "momentum": 1, "gradient_descent_with_momentum": 1, "adam": 2}
INIT_KIND = {"uniform": 0, "uniform_inclusive": 1, "normal": 2}


def _p(t):
    return None if t is None else t.data_ptr()


def _need_cuda(t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise RuntimeError("this op runs on CUDA only (no CPU fallback on this path)")


def loss_backward(a: torch.Tensor, y: torch.Tensor, *, kind: str, softmax: bool, loss_sum: torch.Tensor,
                  d: torch.Tensor | None = None, d_t: torch.Tensor | None = None,
                  d_bf16: torch.Tensor | None = None, d_t_bf16: torch.Tensor | None = None,
                  probs: torch.Tensor | None = None, correct: torch.Tensor | None = None,
                  dact: str | None = None, dact_param: float = 0.0, relu_quirk: bool = False,
                  aux: torch.Tensor | None = None, eps: float = 1.1920929e-07, stream=None) -> None:
    """Fused (softmax +) loss + gradient w.r.t. the last layer's pre-activation.

    ``loss_sum`` (float64[1]) is incremented by the batch loss; ``correct`` (int32[1]) by the number
    of rows whose arg-max matches the label's.
    """
    _need_cuda(a)
    lib = _lib.load()
    l = _lib.OnoLoss()
    l.a, l.y, l.aux = a.data_ptr(), y.data_ptr(), _p(aux)
    l.B, l.C = a.shape
    l.ld, l.ldy = a.stride(0), y.stride(0)
    l.kind = {"mse": 0, "cross_entropy": 1}[kind]
    l.softmax = int(softmax)
    l.dact, l.dact_param, l.relu_quirk = ACT[dact], dact_param, int(relu_quirk)
    l.eps = eps
    l.probs = _p(probs)
    l.d_f32, l.dT_f32, l.d_bf16, l.dT_bf16 = _p(d), _p(d_t), _p(d_bf16), _p(d_t_bf16)
    rows = [t for t in (d, d_bf16) if t is not None]
    cols = [t for t in (d_t, d_t_bf16) if t is not None]
    l.ld_d = rows[0].stride(0) if rows else 0
    l.ld_dT = cols[0].stride(0) if cols else 0
    l.loss_sum, l.correct = _p(loss_sum), _p(correct)
    _lib.check(lib.ono_loss(C.byref(l), _lib.stream_ptr(stream)), "ono_loss")


def softmax_layer(x: torch.Tensor, *, p: torch.Tensor | None = None, out: torch.Tensor | None = None,
                  out_t: torch.Tensor | None = None, stream=None) -> None:
    """Softmax as a layer activation. Forward (``p`` is None): ``out = softmax(x)`` row-wise. Backward: ``x`` is the gradient
    w.r.t. the softmax output, ``p`` the stored output (f32 or bf16), ``out = p * (x - sum_k p_k x_k)``
    (arch/layers/softmax.rs:44-64). ``out`` / ``out_t`` (transposed copy) may be f32 or bf16; ``x`` is f32."""
    _need_cuda(x)
    a = _lib.OnoSoftmax()
    a.x, a.ld_x = x.data_ptr(), x.stride(0)
    a.B, a.C = x.shape
    a.backward = int(p is not None)
    if p is not None:
        if p.dtype == torch.float32:
            a.p_f32 = p.data_ptr()
        else:
            a.p_bf16 = p.data_ptr()
        a.ld_p = p.stride(0)
    if out is not None:
        if out.dtype == torch.float32:
            a.out_f32 = out.data_ptr()
        else:
            a.out_bf16 = out.data_ptr()
        a.ld_out = out.stride(0)
    if out_t is not None:
        if out_t.dtype == torch.float32:
            a.outT_f32 = out_t.data_ptr()
        else:
            a.outT_bf16 = out_t.data_ptr()
        a.ld_outT = out_t.stride(0)
    _lib.check(_lib.load().ono_softmax(C.byref(a), _lib.stream_ptr(stream)), "ono_softmax")


def colsum(d: torch.Tensor, out: torch.Tensor, beta: float = 0.0, stream=None) -> None:
    """``out[n] = beta*out[n] + sum_m d[m, n]`` (bias gradient)."""
    _need_cuda(d)
    lib = _lib.load()
    dt = 0 if d.dtype == torch.float32 else 1
    _lib.check(lib.ono_colsum(d.data_ptr(), dt, d.shape[0], d.shape[1], d.stride(0), out.data_ptr(), beta,
                              _lib.stream_ptr(stream)), "ono_colsum")


def push_add(src: torch.Tensor, dst: torch.Tensor, stream=None) -> None:
    """``dst += src`` with reply-free reductions; ``dst`` may be a view of a peer GPU's window."""
    _need_cuda(src)
    lib = _lib.load()
    _lib.check(lib.ono_push_add(src.data_ptr(), dst.data_ptr(), src.numel(), _lib.stream_ptr(stream)), "ono_push_add")


def cast16(src: torch.Tensor, dst: torch.Tensor, f16: bool = False, stream=None) -> None:
    """``dst[i] = bf16(src[i])`` (IEEE f16 with ``f16=True``); ``dst`` may be a view of a peer GPU's window."""
    _need_cuda(src)
    if dst.numel() != src.numel() or dst.element_size() != 2 or src.dtype != torch.float32:
        raise ValueError("cast16 needs an f32 source and a 16-bit destination of the same length")
    _lib.check(_lib.load().ono_cast16(src.data_ptr(), dst.data_ptr(), src.numel(), int(f16), _lib.stream_ptr(stream)),
               "ono_cast16")


def optim_step(p: torch.Tensor, g: torch.Tensor, *, kind: str, lr: float, mu: float = 0.0, b1: float = 0.9,
               b2: float = 0.999, eps: float = 1e-8, m: torch.Tensor | None = None,
               v: torch.Tensor | None = None, adam_pows: torch.Tensor | None = None,
               grad_scale: float = 1.0, p_bf16: torch.Tensor | None = None, zero_grad: bool = False,
               stream=None) -> None:
    """SGD / momentum / Adam on a flat f32 buffer (one kernel)."""
    _need_cuda(p)
    lib = _lib.load()
    o = _lib.OnoOptim()
    o.p, o.g, o.m, o.v = p.data_ptr(), g.data_ptr(), _p(m), _p(v)
    o.n = p.numel()
    o.kind = OPT_KIND[kind]
    o.lr, o.mu, o.b1, o.b2, o.eps = lr, mu, b1, b2, eps
    o.grad_scale = grad_scale
    o.adam_pows = _p(adam_pows)
    o.p_bf16 = _p(p_bf16)
    o.zero_grad = int(zero_grad)
    _lib.check(lib.ono_optim(C.byref(o), _lib.stream_ptr(stream)), "ono_optim")


def adam_tick(pows: torch.Tensor, b1: float, b2: float, stream=None) -> None:
    """Advance the running products ``{b1^t, b2^t}`` kept in device memory (graph friendly)."""
    _lib.check(_lib.load().ono_adam_tick(pows.data_ptr(), b1, b2, _lib.stream_ptr(stream)), "ono_adam_tick")


def local_sgd(p: torch.Tensor, g: torch.Tensor, r: torch.Tensor, lr: float,
              p_bf16: torch.Tensor | None = None, stream=None) -> None:
    """Round cadence: ``p -= lr*g ; r += g`` (machine_learning/src/arch/sequential.rs:129-141)."""
    _need_cuda(p)
    _lib.check(_lib.load().ono_local_sgd(p.data_ptr(), g.data_ptr(), r.data_ptr(), p.numel(), lr, _p(p_bf16),
                                         _lib.stream_ptr(stream)), "ono_local_sgd")


def sumsq(x: torch.Tensor, out: torch.Tensor, stream=None) -> None:
    """``out[0] += sum(x*x)`` with a float64 accumulator."""
    _need_cuda(x)
    _lib.check(_lib.load().ono_sumsq(x.data_ptr(), x.numel(), out.data_ptr(), _lib.stream_ptr(stream)), "ono_sumsq")


def philox_init(out: torch.Tensor, *, seed: int, index_offset: int, kind: str, a: float, b: float,
                stream=None) -> None:
    """Fill ``out`` with counter-based samples: element i uses counter ``index_offset + i``."""
    _need_cuda(out)
    _lib.check(_lib.load().ono_init(out.data_ptr(), out.numel(), index_offset, seed & (2**64 - 1),
                                    INIT_KIND[kind], a, b, _lib.stream_ptr(stream)), "ono_init")


def rows(src: torch.Tensor, *, idx: torch.Tensor | None = None, n_rows: int | None = None,
         dst: torch.Tensor | None = None, dst_t: torch.Tensor | None = None,
         dst_bf16: torch.Tensor | None = None, dst_t_bf16: torch.Tensor | None = None, stream=None) -> None:
    """Gather rows (optionally by int32 ``idx``), cast and/or transpose in one pass.

    ``src`` may be a pinned host tensor: under unified addressing the kernel then reads the selected rows straight out of
    host memory over PCIe (the host-to-device copy and the gather are one pass; ``idx`` and the outputs are on the GPU)."""
    if not src.is_cuda and not src.is_pinned():
        raise RuntimeError("rows() needs a CUDA tensor or a pinned host tensor as its source")
    lib = _lib.load()
    r = _lib.OnoRows()
    r.src, r.ld_src = src.data_ptr(), src.stride(0)
    r.idx = _p(idx)
    r.R = n_rows if n_rows is not None else (idx.numel() if idx is not None else src.shape[0])
    r.W = src.shape[1]
    r.dst_f32, r.dstT_f32, r.dst_bf16, r.dstT_bf16 = _p(dst), _p(dst_t), _p(dst_bf16), _p(dst_t_bf16)
    rr = [t for t in (dst, dst_bf16) if t is not None]
    cc = [t for t in (dst_t, dst_t_bf16) if t is not None]
    r.ld_dst = rr[0].stride(0) if rr else 0
    r.ld_dstT = cc[0].stride(0) if cc else 0
    _lib.check(lib.ono_rows(C.byref(r), _lib.stream_ptr(stream)), "ono_rows")
