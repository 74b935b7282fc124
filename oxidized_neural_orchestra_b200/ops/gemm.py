"""Python entry to the tcgen05 GEMM (``csrc/kernels/gemm_tcgen05.cu``).

``gemm(a, b, ...)`` computes ``D[M,N] = A[M,K] @ B[K,N]`` on the 5th-generation tensor cores with
f32 accumulation in TMEM and a fused epilogue (bias, activation, activation derivative, row-major
and transposed outputs in f32/bf16). Operands are described the way the hardware sees them:

* ``a``: ``[M, K]`` (K contiguous, "K-major") or, with ``a_mn_major=True``, ``[K, M]``
* ``b``: ``[N, K]`` (K contiguous)              or, with ``b_mn_major=True``, ``[K, N]``

MN-major operands: bf16, and f32/tf32 (128-byte swizzle on 32-byte units). f32 tensors run as tf32 tiles straight from the f32 storage.
This mirrors the three GEMMs of the reference's Dense layer
(machine_learning/src/arch/layers/dense.rs:36-64): forward ``X·W``, ``d·Wᵀ`` and ``Xᵀ·d``.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

ACT = {"none": 0, None: 0, "relu": 1, "sigmoid": 2, "tanh": 3, "gelu": 4}


def _ptr(t):
    return None if t is None else t.data_ptr()


# CTAs a GEMM may use when the caller gives no limit (0 = one per SM). The rank runtime lowers it while gradient
# buckets are synchronised during backward, so that the communication kernels find free SMs.
DEFAULT_MAX_CTAS = 0
# CTA pairs (256-row tiles) for GEMMs whose caller does not choose. "auto": pairs for bf16 tiles (measured three times,
# alternating, on the 8 x 8192 MLP step: 4.64 / 4.67 / 4.66 ms with pairs against 4.78 / 4.78 / 4.78 ms without; the gain comes
# from the short-K weight-gradient GEMMs), single CTAs for tf32 tiles; "1": wherever the shape allows; "0": never.
DEFAULT_PAIR = __import__("os").environ.get("ONO_GEMM_PAIR", "auto")

# Split-K workspaces, one per (device, stream): GEMMs on different streams may overlap on the device, so each stream
# gets its own slabs. 8 Mi floats hold e.g. 148 slabs of a 64 x 576 weight gradient or 49 of a 342 x 128 product.
WORKSPACE_ELEMS = 8 << 20
_workspaces: dict = {}


def _workspace(device: torch.device, stream) -> torch.Tensor | None:
    s = stream if stream is not None else torch.cuda.current_stream(device)
    key = (device.index, s.cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            return None      # never allocate inside a capture; the library's static buffer serves this call
        ws = torch.empty(WORKSPACE_ELEMS, dtype=torch.float32, device=device)
        _workspaces[key] = ws
    return ws


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
         out: torch.Tensor | None = None, out_t: torch.Tensor | None = None,
         out_bf16: torch.Tensor | None = None, out_t_bf16: torch.Tensor | None = None,
         pre: torch.Tensor | None = None, bias: torch.Tensor | None = None,
         act: str | None = None, act_param: float = 0.0,
         aux: torch.Tensor | None = None, dact: str | None = None, dact_param: float = 0.0,
         relu_quirk: bool = False, alpha: float = 1.0, beta: float = 0.0, bn: int = 0,
         max_ctas: int = 0, split_k: int = 0, pair: int = 0, reduce_out: bool = False, out_f16: torch.Tensor | None = None,
         apply: dict | None = None, gate: tuple | None = None, timeout_ns: int = 0, status: torch.Tensor | None = None,
         stream=None) -> None:
    """Launch one GEMM. All tensors must be 2-D, on the current CUDA device, with unit inner stride.

    ``split_k``: 0 lets the library decide (a shape with a handful of output tiles and a long reduction, e.g. 342 x 128 x
    3136, is split over the SMs), ``> 1`` asks for that many splits, 1 keeps the call single-pass. Every split stores its
    partial product into its own slab of a per-stream workspace and a small finishing kernel adds the slabs in order and
    applies the whole epilogue, so the result is the same to the bit from run to run.

    ``out_f16``: like ``out_bf16`` but the values are IEEE f16 (a 16-bit gradient wire in the reference's format). Either
    16-bit output may be a view of a peer GPU's window: aligned tiles then leave through TMA stores over NVLink.

    ``gate``: ``(flags, target, stride, mask)``: the kernel loads no operand before ``flags[i * stride] >= target[0]`` for every
    bit ``i`` of ``mask`` (int32 device tensors; a bounded wait: on a timeout ``status`` becomes non-zero and the kernel returns
    without output). Used to queue a layer's GEMM while its weights are still arriving from their owners.

    ``apply``: optimizer applied by the epilogue to the tile it has just computed (the weight gradient of a layer this
    rank owns outright), which is then never written to memory: ``dict(p=, m=, v=, p_bf16=, kind=, lr=, mu=, b1=, b2=,
    eps=, grad_scale=, adam_pows=)`` with ``p``/``m``/``v``/``p_bf16`` shaped like the result."""
    if not a.is_cuda:
        raise RuntimeError("ono gemm needs CUDA tensors (there is no CPU fallback on this path)")
    lib = _lib.load()
    if a.dtype != b.dtype or a.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("a and b must both be float32 (tf32 tiles) or bfloat16")
    if out_f16 is not None:
        if out_bf16 is not None or out_f16.dtype != torch.float16:
            raise ValueError("out_f16 must be float16 and excludes out_bf16")
        out_bf16 = out_f16
    for t in (a, b, out, out_t, out_bf16, out_t_bf16, pre, aux):
        if t is not None and (t.dim() != 2 or t.stride(1) != 1):
            raise ValueError("tensors must be 2-D with unit inner stride")
    if a_mn_major:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn_major:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    g = _lib.OnoGemm()
    g.A, g.B = a.data_ptr(), b.data_ptr()
    g.M, g.N, g.K = M, N, K
    g.lda, g.ldb = a.stride(0), b.stride(0)
    g.dtype = 0 if a.dtype == torch.float32 else 1
    g.a_major, g.b_major = int(a_mn_major), int(b_mn_major)
    g.epi.reduce_out = int(reduce_out)
    g.epi.out16_f16 = int(out_f16 is not None)
    if split_k != 1 and apply is None and not reduce_out:
        ws = _workspace(a.device, stream)
        if ws is not None:
            g.workspace, g.workspace_elems = ws.data_ptr(), ws.numel()
    if apply is not None:
        ap, pm = g.apply, apply["p"]
        if pm.dim() != 2 or pm.stride(1) != 1 or tuple(pm.shape) != (M, N) or pm.dtype != torch.float32:
            raise ValueError("apply['p'] must be an f32 [M, N] matrix with unit inner stride")
        ap.p, ap.ld = pm.data_ptr(), pm.stride(0)
        for k in ("m", "v", "p_bf16"):
            t = apply.get(k)
            if t is not None and (t.stride(0) != pm.stride(0) or tuple(t.shape) != (M, N)):
                raise ValueError(f"apply[{k!r}] must share the shape and leading dimension of apply['p']")
        ap.m, ap.v, ap.p_bf16 = _ptr(apply.get("m")), _ptr(apply.get("v")), _ptr(apply.get("p_bf16"))
        ap.kind = {"sgd": 0, "momentum": 1, "adam": 2}[apply["kind"]]
        ap.lr, ap.mu = apply["lr"], apply.get("mu", 0.0)
        ap.b1, ap.b2, ap.eps = apply.get("b1", 0.9), apply.get("b2", 0.999), apply.get("eps", 1e-8)
        ap.grad_scale = apply.get("grad_scale", 1.0)
        ap.adam_pows = _ptr(apply.get("adam_pows"))
    if pair == 0:
        if DEFAULT_PAIR == "auto":
            pair = 1 if (a.dtype == torch.bfloat16 and M >= 256 and not reduce_out) else -1
        else:
            pair = 1 if DEFAULT_PAIR == "1" else -1
    g.bn, g.max_ctas, g.split_k, g.pair = bn, max_ctas or DEFAULT_MAX_CTAS, split_k, pair
    e = g.epi
    ld_out = ld_out_t = 0
    for t in (out, out_bf16, pre):
        if t is not None:
            if ld_out and t.stride(0) != ld_out:
                raise ValueError("row-major outputs must share one leading dimension")
            ld_out = t.stride(0)
    for t in (out_t, out_t_bf16):
        if t is not None:
            if ld_out_t and t.stride(0) != ld_out_t:
                raise ValueError("transposed outputs must share one leading dimension")
            ld_out_t = t.stride(0)
    if out is not None and out.dtype != torch.float32:
        raise TypeError("out must be float32")
    e.out_f32, e.outT_f32 = _ptr(out), _ptr(out_t)
    e.out_bf16, e.outT_bf16 = _ptr(out_bf16), _ptr(out_t_bf16)
    if pre is not None:
        if pre.dtype == torch.float32:
            e.pre_f32 = pre.data_ptr()
        else:
            e.pre_bf16 = pre.data_ptr()
    if bias is not None and bias.dtype == torch.bfloat16:
        e.bias_bf16 = bias.data_ptr()
    else:
        e.bias = _ptr(bias)
    if aux is not None:
        if aux.dtype == torch.float32:
            e.aux_f32 = aux.data_ptr()
        else:
            e.aux_bf16 = aux.data_ptr()
        e.ld_aux = aux.stride(0)
    e.ld_out, e.ld_outT = ld_out, ld_out_t
    e.act, e.act_param = ACT[act], act_param
    e.dact, e.dact_param = ACT[dact], dact_param
    e.relu_quirk = int(relu_quirk)
    e.alpha, e.beta = alpha, beta
    g.status = _ptr(status)
    g.timeout_ns = timeout_ns
    if gate is not None:
        flags, target, stride, mask = gate
        g.gate, g.gate_target, g.gate_stride, g.gate_mask = flags.data_ptr(), target.data_ptr(), stride, mask
    _lib.check(lib.ono_gemm(C.byref(g), _lib.stream_ptr(stream)), "ono_gemm")
