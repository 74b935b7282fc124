"""GPU training engine: explicit forward/backward over flat f32 parameters in HBM.

The engine is the B200 counterpart of the reference's ``Sequential`` + ``ParamManager``
(machine_learning/src/arch/sequential.rs:43-148, machine_learning/src/param_manager.rs:61-198):

* parameters and gradients are two flat f32 vectors in the reference's external layout
  (per layer ``W[in,out]`` row-major then ``b[out]``; conv ``K[F][C][k][k]`` then ``b[F]``), so that
  collectives, optimizers and the safetensors export all work on the same buffer;
* layers are views (offset tables) into those vectors;
* every GEMM runs on the tcgen05 kernel; operands the tensor cores cannot address directly from the
  flat vector (wrong major-ness for tf32, unaligned rows, bf16 tiles) are "compute copies" that
  ``refresh()`` regenerates after each parameter update;
* there is no autograd: each layer contributes explicit forward, dgrad and wgrad launches, and a
  whole mini-batch step is a fixed kernel sequence that can be captured in a CUDA graph.

Tile dtype ``tf32`` keeps every tensor in f32 and uses K-major operands only (transposed copies are
written by the producing epilogue); ``bf16`` keeps bf16 activations/deltas and uses MN-major
operands, so no transposed copies exist.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..ops import elementwise as ew
from ..ops.gemm import gemm


def _up(n: int, m: int = 16) -> int:
    return (n + m - 1) // m * m


@dataclass
class LayerPlan:
    kind: str                       # dense | conv | pool
    in_features: int
    out_features: int
    act: str | None = None
    act_param: float = 0.0
    w_off: int = 0                  # offset of W in the flat vector
    b_off: int = 0                  # offset of b
    n_params: int = 0
    extra: dict = field(default_factory=dict)


def layer_param_count(spec: dict) -> int:
    if spec["kind"] == "dense":
        return (spec["in"] + 1) * spec["out"]
    if spec["kind"] == "conv":
        f, c, k = spec["kernel_dim"]
        return f * c * k * k + f
    return 0


class GpuEngine:
    """Forward/backward of a dense network for one fixed maximum batch size on one GPU."""

    def __init__(self, layers: list[dict], *, batch_size: int, tile_dtype: str, loss: str,
                 params: torch.Tensor, grads: torch.Tensor, params_bf16: torch.Tensor | None = None,
                 leaky_relu_exact: bool = True, device=None, bias_from_shadow: bool = False,
                 input_grad: bool = False, final: bool = True):
        self.bias_from_shadow = bias_from_shadow
        # final = False: a dense block in the middle of a network (convolutions follow). Its last layer then writes its
        # activation into ``out_act`` like any inner layer, and backward starts from ``d[-1]``, which whoever consumes
        # ``out_act`` fills with the gradient w.r.t. that layer's pre-activation.
        self.final = final
        self.input_grad = input_grad  # also produce d[0], the gradient w.r.t. the input batch
        self.max_ctas = 0             # CTAs a GEMM of this engine may use (0 = one per SM); lowered while other kernels need SMs
        self.push = None              # weight-gradient tiles added into the owners' f32 accumulators (see backward)
        self.wire16 = None            # weight-gradient tiles stored as 16-bit values into the owners' slabs
        self.apply_plan = None        # optimizer applied by the weight-gradient GEMM's epilogue, per layer
        self.gates = None             # per layer: flags its forward GEMM waits on before it loads the layer's weights
        if tile_dtype not in ("tf32", "bf16"):
            raise ValueError("tile_dtype must be 'tf32' or 'bf16'")
        self.dev = device or params.device
        if self.dev.type != "cuda":
            raise RuntimeError("GpuEngine needs a CUDA device; CPU runs use the C++ oracle engine")
        self.bf16 = tile_dtype == "bf16"
        self.B = batch_size
        self.ldB = _up(batch_size)
        self.loss = loss
        self.relu_quirk = not leaky_relu_exact
        self.params, self.grads, self.params_bf16 = params, grads, params_bf16
        self.plans: list[LayerPlan] = []
        off = 0
        for sp in layers:
            if sp["kind"] != "dense":
                raise NotImplementedError("GpuEngine handles dense layers; see ConvEngine for conv/pool")
            act = sp.get("act")
            pl = LayerPlan("dense", sp["in"], sp["out"], act[0] if act else None, act[1] if act else 0.0)
            pl.w_off, pl.b_off = off, off + sp["in"] * sp["out"]
            pl.n_params = (sp["in"] + 1) * sp["out"]
            off += pl.n_params
            self.plans.append(pl)
        self.n_params = off
        if params.numel() < off or grads.numel() < off:
            raise ValueError("flat parameter/gradient buffers are too small")
        # softmax on the last layer is fused into the loss kernel; on any other layer it is a row-wise pass of its own
        # after the GEMM (forward) and before the next GEMM's operand is formed (Jacobian-vector product in backward)
        self.softmax_last = self.final and self.plans[-1].act == "softmax"
        if not self.final and self.plans[-1].act in ("softmax", "gelu"):
            raise NotImplementedError("a dense layer followed by a convolution needs a relu / sigmoid / tanh / linear activation")
        self._alloc()

    # ------------------------------------------------------------------------------------------
    def _alloc(self) -> None:
        dev, B, ldB = self.dev, self.B, self.ldB
        cd = torch.bfloat16 if self.bf16 else torch.float32
        f32 = torch.float32
        z = lambda r, c, dt: torch.zeros(r, c, device=dev, dtype=dt)
        L = self.plans
        feats = [L[0].in_features] + [p.out_features for p in L]
        self.lds = [_up(f) for f in feats]
        # activations a[0] = input batch, a[l+1] = output of layer l
        self.a = [z(B, self.lds[i], cd) for i in range(len(feats) - 1)]
        self.logits = z(B, self.lds[-1], f32)
        self.d = [z(B, self.lds[0], cd) if self.input_grad else None] + [z(B, self.lds[i], cd) for i in range(1, len(feats))]
        self.zpre = [None] * len(feats)
        self.soft_tmp = [None] * len(feats)       # f32 scratch of an inner softmax layer: pre-activations, then d/d(output)
        for l, pl in enumerate(L):
            if pl.act == "gelu":
                self.zpre[l + 1] = z(B, self.lds[l + 1], cd)
            if pl.act == "softmax" and l < len(L) - 1:
                self.soft_tmp[l + 1] = z(B, self.lds[l + 1], f32)
        # MN-major operands let every GEMM read activations, deltas and weights as they are stored. bf16 always does;
        # for tf32 the MN-major tiles (32-element rows, twelve small TMA boxes per stage) measured slower than K-major
        # tiles fed from transposed compute copies (wide MLP step 1.20 ms against 1.13 ms), so it is opt-in: ONO_TF32_MN=1
        import os
        self.mn = self.bf16 or os.environ.get("ONO_TF32_MN", "0") == "1"
        self.at = self.dt = None
        if not self.mn:
            self.at = [z(feats[i], ldB, f32) for i in range(len(feats) - 1)]
            self.dt = [None] + [z(feats[i], ldB, f32) for i in range(1, len(feats))]
        self.out_act = None if self.final else z(B, self.lds[-1], cd)
        self.ybuf = z(B, _up(feats[-1]), f32)
        self.loss_sum = torch.zeros(1, device=dev, dtype=torch.float64)
        self.correct = torch.zeros(1, device=dev, dtype=torch.int32)
        self.status = torch.zeros(1, device=dev, dtype=torch.int32)
        # weight operands
        self.w_k, self.w_t, self.w_copy_needed, self.gw_tmp = [], [], [], []
        for pl in L:
            i, o = pl.in_features, pl.out_features
            esz_mult = 8 if self.bf16 else 4
            flat = self.params_bf16 if self.bf16 else self.params
            direct = flat is not None and o % esz_mult == 0 and pl.w_off % esz_mult == 0 and \
                (flat.data_ptr() + pl.w_off * flat.element_size()) % 16 == 0
            if direct:
                self.w_k.append(flat[pl.w_off:pl.w_off + i * o].view(i, o))
                self.w_copy_needed.append(False)
            else:
                self.w_k.append(z(i, _up(o), cd)[:, :o])
                self.w_copy_needed.append(True)
            self.w_t.append(None if self.mn else z(o, _up(i), f32)[:, :i])
            g_direct = o % 4 == 0 and pl.w_off % 4 == 0 and (self.grads.data_ptr() + 4 * pl.w_off) % 16 == 0
            self.gw_tmp.append(None if g_direct else z(i, _up(o), f32)[:, :o])

    def _gemm(self, *args, **kw) -> None:
        gemm(*args, max_ctas=self.max_ctas, **kw)

    def w_view(self, l: int) -> torch.Tensor:
        pl = self.plans[l]
        return self.params[pl.w_off:pl.w_off + pl.in_features * pl.out_features].view(pl.in_features, pl.out_features)

    @property
    def needs_f32_params(self) -> bool:
        """False when every operand the engine reads comes from the bf16 shadow (weights used in place
        and biases read as bf16): then only the owner of a range needs its f32 master."""
        return not (self.bf16 and self.bias_from_shadow and self.params_bf16 is not None
                    and not any(self.w_copy_needed))

    def b_view(self, l: int) -> torch.Tensor:
        pl = self.plans[l]
        if not self.needs_f32_params:
            return self.params_bf16[pl.b_off:pl.b_off + pl.out_features]
        return self.params[pl.b_off:pl.b_off + pl.out_features]

    def gw_view(self, l: int) -> torch.Tensor:
        pl = self.plans[l]
        return self.grads[pl.w_off:pl.w_off + pl.in_features * pl.out_features].view(pl.in_features, pl.out_features)

    def gb_view(self, l: int) -> torch.Tensor:
        pl = self.plans[l]
        return self.grads[pl.b_off:pl.b_off + pl.out_features]

    # ------------------------------------------------------------------------------------------
    def refresh(self, stream=None) -> int:
        """Regenerate the compute copies of the weights from the f32 master. Returns #launches."""
        n = 0
        for l in range(len(self.plans)):
            w = self.w_view(l)
            if self.bf16:
                if self.w_copy_needed[l]:
                    ew.rows(w, dst_bf16=self.w_k[l], stream=stream)
                    n += 1
            elif self.mn:
                if self.w_copy_needed[l]:
                    ew.rows(w, dst=self.w_k[l], stream=stream)
                    n += 1
            else:
                if self.w_copy_needed[l]:
                    ew.rows(w, dst=self.w_k[l], dst_t=self.w_t[l], stream=stream)
                else:
                    ew.rows(w, dst_t=self.w_t[l], stream=stream)
                n += 1
        return n

    def load_batch(self, x: torch.Tensor, y: torch.Tensor, nrows: int, idx: torch.Tensor | None = None,
                   stream=None) -> int:
        """Stage ``x[idx]`` (f32, [rows, in]) as the first GEMM's A operand and ``y[idx]`` as the labels."""
        if self.bf16:
            ew.rows(x, idx=idx, n_rows=nrows, dst_bf16=self.a[0], stream=stream)
        elif self.mn:
            ew.rows(x, idx=idx, n_rows=nrows, dst=self.a[0], stream=stream)
        else:
            ew.rows(x, idx=idx, n_rows=nrows, dst=self.a[0], dst_t=self.at[0], stream=stream)
        ew.rows(y, idx=idx, n_rows=nrows, dst=self.ybuf, stream=stream)
        return 2

    def forward(self, nrows: int, stream=None) -> int:
        L, n = self.plans, 0
        for l, pl in enumerate(L):
            last = l == len(L) - 1 and self.final
            a_in = self.a[l][:nrows, :pl.in_features]
            inner_softmax = pl.act == "softmax" and not last
            act = None if (pl.act == "softmax") else pl.act
            kw = dict(bias=self.b_view(l), act=act, act_param=pl.act_param, status=self.status, stream=stream)
            if self.gates is not None and self.gates.get(l) is not None:
                kw["gate"] = self.gates[l]      # the layer's weights may still be arriving from their owners
                kw["timeout_ns"] = 10_000_000_000   # the same patience as the fused kernel's barriers: a rank may start late
            if inner_softmax:
                o = pl.out_features
                kw["out"] = self.soft_tmp[l + 1][:nrows, :o]
                if self.mn:
                    self._gemm(a_in, self.w_k[l], b_mn_major=True, **kw)
                else:
                    self._gemm(a_in, self.w_t[l], **kw)
                ew.softmax_layer(self.soft_tmp[l + 1][:nrows, :o], out=self.a[l + 1][:nrows, :o],
                                 out_t=None if self.mn else self.at[l + 1][:, :nrows], stream=stream)
                n += 2
                continue
            if last:
                kw["out"] = self.logits[:nrows, :pl.out_features]
            elif l == len(L) - 1:      # a block in the middle of a network: the activation goes to whoever follows
                kw["out_bf16" if self.bf16 else "out"] = self.out_act[:nrows, :pl.out_features]
            elif self.bf16:
                kw["out_bf16"] = self.a[l + 1][:nrows, :pl.out_features]
                if self.zpre[l + 1] is not None:
                    kw["pre"] = self.zpre[l + 1][:nrows, :pl.out_features]
            else:
                kw["out"] = self.a[l + 1][:nrows, :pl.out_features]
                if not self.mn:
                    kw["out_t"] = self.at[l + 1][:, :nrows]
                if self.zpre[l + 1] is not None:
                    kw["pre"] = self.zpre[l + 1][:nrows, :pl.out_features]
            if self.mn:
                self._gemm(a_in, self.w_k[l], b_mn_major=True, **kw)
            else:
                self._gemm(a_in, self.w_t[l], **kw)
            n += 1
        return n

    def loss_backward(self, nrows: int, stream=None) -> int:
        y = self.ybuf
        pl = self.plans[-1]
        C = pl.out_features
        lg = self.logits[:nrows, :C]
        kw = dict(kind=self.loss, softmax=self.softmax_last, loss_sum=self.loss_sum, correct=self.correct,
                  stream=stream)
        if not self.softmax_last and pl.act is not None:
            kw.update(dact=pl.act, dact_param=pl.act_param, relu_quirk=self.relu_quirk)
        if self.bf16:
            kw["d_bf16"] = self.d[-1][:nrows, :C]
        else:
            kw["d"] = self.d[-1][:nrows, :C]
            if not self.mn:
                kw["d_t"] = self.dt[-1][:, :nrows]
        ew.loss_backward(lg, y[:nrows, :C], **kw)
        return 1

    def backward(self, nrows: int, accumulate: bool = False, stream=None, after_layer=None) -> int:
        """dgrad + wgrad + bias-grad for every layer; gradients land in the flat gradient vector.

        Per layer the input gradient is computed first, so that nothing reads the layer's weights once
        its own gradient is complete: ``after_layer(l)`` may then start synchronising (and overwriting)
        that layer's parameters while the layers below are still running."""
        L, n = self.plans, 0
        beta = 1.0 if accumulate else 0.0
        push, wire, app = self.push, self.wire16, self.apply_plan
        if (push is not None or wire is not None or app is not None) and accumulate:
            raise RuntimeError("pushed / fused weight gradients cannot accumulate over several batches")
        for l in range(len(L) - 1, -1, -1):
            pl = L[l]
            i, o = pl.in_features, pl.out_features
            d_out = self.d[l + 1][:nrows, :o]
            if l > 0 or self.input_grad:
                # dgrad through the previous layer's activation: d_{l} = (d_{l+1} W^T) * act'(a_l);
                # for l = 0 this is the raw gradient w.r.t. the input batch (whoever produced the
                # batch applies its own activation derivative)
                prev = L[l - 1] if l > 0 else LayerPlan("input", 0, i)
                stored = self.zpre[l] if prev.act == "gelu" else self.a[l]
                kw = dict(status=self.status, stream=stream)
                if prev.act == "softmax":
                    # the GEMM leaves d/d(softmax output) in f32; the Jacobian-vector product needs whole rows
                    tmp = self.soft_tmp[l][:nrows, :i]
                    self._gemm(d_out, self.w_k[l], out=tmp, **kw)
                    ew.softmax_layer(tmp, p=self.a[l][:nrows, :i], out=self.d[l][:nrows, :i],
                                     out_t=None if (self.mn or l == 0) else self.dt[l][:, :nrows], stream=stream)
                    n += 2
                elif prev.act is not None:
                    kw.update(aux=stored[:nrows, :i], dact=prev.act, dact_param=prev.act_param,
                              relu_quirk=self.relu_quirk)
                if prev.act == "softmax":
                    pass
                elif self.bf16:
                    self._gemm(d_out, self.w_k[l], out_bf16=self.d[l][:nrows, :i], **kw)
                elif self.mn:
                    self._gemm(d_out, self.w_k[l], out=self.d[l][:nrows, :i], **kw)
                else:
                    self._gemm(d_out, self.w_k[l], out=self.d[l][:nrows, :i],
                               out_t=self.dt[l][:, :nrows] if l > 0 else None, **kw)
                if prev.act != "softmax":
                    n += 1

            def wgrad(r0, r1, **out_kw):     # rows [r0, r1) of dW = A_l^T d
                if self.mn:
                    self._gemm(self.a[l][:nrows, r0:r1], d_out, a_mn_major=True, b_mn_major=True, status=self.status,
                               stream=stream, **out_kw)
                else:
                    self._gemm(self.at[l][r0:r1, :nrows], self.dt[l + 1][:, :nrows], status=self.status, stream=stream,
                               **out_kw)

            if wire is not None:
                # 16-bit gradient wire. "staged": dW leaves the epilogue as bf16 / f16 into this rank's own 16-bit
                # gradient vector (TMA stores to local memory); the caller's after_layer hook then ships the ranges other
                # ranks own with copy-engine transfers while backward goes on. "direct": the epilogue's TMA stores go
                # straight into the slab the owner of those rows keeps for this rank (its window over NVLink).
                k16 = "out_f16" if wire["f16"] else "out_bf16"
                pieces = wire["w"][l]
                if pieces is not None:
                    for r0, r1, dst in pieces:
                        wgrad(r0, r1, **{k16: dst})
                        n += 1
                else:
                    tgt = self.gw_tmp[l] if self.gw_tmp[l] is not None else self.gw_view(l)
                    wgrad(0, i, out=tgt)
                    n += 1
                    if self.gw_tmp[l] is not None:
                        ew.rows(tgt, dst=self.gw_view(l), stream=stream)
                        n += 1
                ew.colsum(d_out, self.gb_view(l), beta=0.0, stream=stream)
                n += 1
                for src, dst in wire["cast"][l]:
                    ew.cast16(src, dst, f16=wire["f16"], stream=stream)
                    n += 1
                if after_layer is not None:
                    n += after_layer(l) or 0
                continue
            if app is not None and app.get(l) is not None:
                # this rank owns the whole layer: the epilogue applies the optimizer to the tile it has just
                # computed (master, state, bf16 shadow); the weight gradient itself is never stored
                wgrad(0, i, apply=app[l])
                ew.colsum(d_out, self.gb_view(l), beta=0.0, stream=stream)
                n += 2
                if after_layer is not None:
                    n += after_layer(l) or 0
                continue
            if push is not None:
                # weight gradient tiles are added straight into the accumulator of the rank that owns those rows (its
                # window, over NVLink): the reduce-scatter happens inside the GEMM epilogue, tile by tile
                for r0, r1, dst in push["w"][l]:
                    wgrad(r0, r1, out=dst, reduce_out=True)
                    n += 1
                ew.colsum(d_out, self.gb_view(l), beta=0.0, stream=stream)
                ew.push_add(self.gb_view(l), push["b"][l], stream=stream)
                n += 2
                if after_layer is not None:
                    n += after_layer(l) or 0
                continue
            # wgrad: dW[in,out] = A_{l}^T d
            tgt = self.gw_tmp[l] if self.gw_tmp[l] is not None else self.gw_view(l)
            wbeta = beta if self.gw_tmp[l] is None else 0.0
            wgrad(0, i, out=tgt, beta=wbeta)
            n += 1
            if self.gw_tmp[l] is not None:
                if accumulate:
                    self.gw_view(l).add_(tgt)
                else:
                    ew.rows(tgt, dst=self.gw_view(l), stream=stream)
                n += 1
            ew.colsum(d_out, self.gb_view(l), beta=beta, stream=stream)
            n += 1
            if after_layer is not None:
                n += after_layer(l) or 0
        return n

    def step(self, x: torch.Tensor, y: torch.Tensor, nrows: int, idx=None, accumulate=False, stream=None,
             after_layer=None) -> int:
        """load -> forward -> loss -> backward. Returns the number of kernels launched."""
        n = self.load_batch(x, y, nrows, idx, stream)
        n += self.forward(nrows, stream)
        n += self.loss_backward(nrows, stream)
        n += self.backward(nrows, accumulate, stream, after_layer)
        return n
