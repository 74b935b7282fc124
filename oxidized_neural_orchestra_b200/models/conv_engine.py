"""Convolution / pooling layers ahead of the dense stack on the GPU.

The reference runs ``Conv2d`` as per-sample im2col + GEMM and ``MaxPooling`` as a scalar window scan
(machine_learning/src/arch/layers/conv/conv2d.rs:61-190, arch/layers/max_pooling.rs:47-157). Here a
convolution is one batched tcgen05 GEMM ``cols[B*oh*ow, C*k*k] @ K[F, C*k*k]^T`` with bias and activation
in its epilogue, the weight gradient a split-K GEMM over all output pixels of the batch, the input
gradient a GEMM followed by a gather-form col2im. Columns are ordered (ky, kx, c) - channels fastest - so
that the gathers read and write contiguous runs; the kernel tensor ``K[F][C][k][k]`` is permuted into that
order at every parameter refresh and the weight gradient is permuted back into the flat gradient vector. Image activations are pixel-major ``[B*H*W, ld]``; the flattened
NCHW order dense layers expect is restored by one conversion kernel at the conv -> dense boundary.

``ConvNetEngine`` covers ``(conv | max_pooling)* dense+`` - every model of the reference's benchmarks. ``StagedEngine``
chains such units for any other order the configuration accepts (dense layers before convolutions, several conv / dense
alternations): a dense block in the middle hands its activation rows to the next unit's convolutions and receives the
gradient w.r.t. its last pre-activation back from them.
"""
from __future__ import annotations

import torch

from ..ops import conv as cv
from ..ops import elementwise as ew
from ..ops.gemm import gemm
from .engine import GpuEngine, _up


class ConvNetEngine:
    """``ConvFront`` + the dense ``GpuEngine``, with the interface the rank runtime uses."""

    def __init__(self, layers: list[dict], *, batch_size: int, tile_dtype: str, loss: str, params: torch.Tensor,
                 grads: torch.Tensor, params_bf16: torch.Tensor | None = None, leaky_relu_exact: bool = True,
                 bias_from_shadow: bool = False, first: bool = True, prev_act=None, final: bool = True):
        # first = False: this unit follows a dense block. Its input arrives as activation rows of that block (not as a
        # batch), and backward also produces the gradient w.r.t. that block's last pre-activation (``prev_act`` is that
        # layer's activation: its derivative is applied from the stored activation, like between two layers).
        self.first, self.prev_act = first, prev_act
        nfront = 0
        while nfront < len(layers) and layers[nfront]["kind"] != "dense":
            nfront += 1
        if nfront == len(layers):
            raise NotImplementedError("a model needs at least one dense layer after its conv/pool layers on the GPU")
        if any(l["kind"] != "dense" for l in layers[nfront:]):
            raise NotImplementedError("conv/pool layers after a dense layer are not supported on the GPU engine")
        self.bf16 = tile_dtype == "bf16"
        self.dev = params.device
        self.sms = torch.cuda.get_device_properties(self.dev).multi_processor_count
        # tf32 weight gradients read dy and the columns in place as MN-major operands (no transposed copies of either);
        # ONO_CONV_TF32_T=1 brings back the K-major operands with their transposed copies
        self.wgrad_t = tile_dtype != "bf16" and __import__("os").environ.get("ONO_CONV_TF32_T", "0") == "1"
        self.B = batch_size
        self.relu_quirk = not leaky_relu_exact
        self.params, self.grads, self.params_bf16 = params, grads, params_bf16
        self.T = torch.bfloat16 if self.bf16 else torch.float32
        off = 0
        self.front = []
        for sp in layers[:nfront]:
            c, h, w = sp["input_dim"]
            d = dict(sp)
            if sp["kind"] == "conv":
                f, _, k = sp["kernel_dim"]
                d.update(C=c, H=h, W=w, F=f, K=k, off=off, n=f * c * k * k + f)
                off += d["n"]
            else:
                d.update(C=c, H=h, W=w, F=c, K=sp["filter_size"], off=off, n=0)
            d["S"], d["P"] = sp["stride"], sp["padding"]
            d["OH"] = (h + 2 * d["P"] - d["K"]) // d["S"] + 1
            d["OW"] = (w + 2 * d["P"] - d["K"]) // d["S"] + 1
            self.front.append(d)
        self.front_params = off
        last = self.front[-1]
        dense_layers = layers[nfront:]
        assert dense_layers[0]["in"] == last["F"] * last["OH"] * last["OW"]
        self.dense = GpuEngine(dense_layers, batch_size=batch_size, tile_dtype=tile_dtype, loss=loss,
                               params=params[off:], grads=grads[off:],
                               params_bf16=None if params_bf16 is None else params_bf16[off:],
                               leaky_relu_exact=leaky_relu_exact, bias_from_shadow=False, input_grad=True, final=final)
        self.n_params = off + self.dense.n_params
        self.loss_sum, self.correct, self.status = self.dense.loss_sum, self.dense.correct, self.dense.status
        self._alloc()

    # the f32 master is read for the (small) kernel tensors and biases of the front
    needs_f32_params = True

    def _alloc(self):
        B, T, dev = self.B, self.T, self.dev
        z = lambda r, c, dt=T: torch.zeros(r, c, device=dev, dtype=dt)
        for j, d in enumerate(self.front):
            Min, Mout = B * d["H"] * d["W"], B * d["OH"] * d["OW"]
            d["y"] = z(Mout, _up(d["F"]))
            d["dy"] = z(Mout, _up(d["F"]))
            if d["kind"] == "conv":
                ckk = d["C"] * d["K"] * d["K"]
                d["ckk"] = ckk
                # first layer with one input channel: direct CUDA-core kernels (K = k*k is too short for the tensor cores)
                d["direct"] = j == 0 and self.first and d["C"] == 1 and d["K"] <= 5 and d["F"] <= 128
                if d["direct"]:
                    continue
                d["cols"] = z(Mout, _up(ckk))
                d["dcols"] = z(Mout, _up(ckk)) if (j > 0 or not self.first) else None
                d["gk_tmp"] = z(d["F"], _up(ckk), torch.float32)
                if self.wgrad_t:
                    d["colsT"] = z(ckk, _up(Mout))
                    d["dyT"] = z(d["F"], _up(Mout))
                if not self.bf16:
                    d["kt"] = z(ckk, _up(d["F"]))                     # K^T for dgrad
                # the kernel tensor as a GEMM operand: rows in (ky, kx, c) order, rebuilt at every refresh
                d["kop"] = z(d["F"], _up(ckk))[:, :ckk]
            else:
                d["arg"] = torch.zeros(Mout, d["C"], device=dev, dtype=torch.int32)
                d["dx32"] = z(Min, _up(d["C"]), torch.float32)
        c0 = self.front[0]
        self.x0 = z(B * c0["H"] * c0["W"], _up(c0["C"]))      # pixel-major input batch
        self.xflat = z(B, _up(c0["C"] * c0["H"] * c0["W"]))   # the batch as rows, in the tile dtype
        self.in_stub = None
        if not self.first:
            # stands in for "the layer below the first one": its output is this unit's input, its gradient buffer receives
            # d(loss)/d(pre-activation of the dense layer that produced the input), pixel-major
            self.dx0 = z(B * c0["H"] * c0["W"], _up(c0["C"]))
            self.in_stub = {"kind": "conv", "y": self.x0, "dy": self.dx0, "act": self.prev_act, "direct": True}

    def _k_view(self, d):
        return self.params[d["off"]:d["off"] + d["F"] * d["ckk"]].view(d["F"], d["ckk"])

    def _kb_view(self, d):
        return self.params[d["off"] + d["F"] * d["ckk"]:d["off"] + d["n"]]

    def refresh(self, stream=None) -> int:
        n = 0
        for d in self.front:
            if d["kind"] != "conv" or d.get("direct"):
                continue
            cv.kernel_to_operand(d["F"], d["C"], d["K"], self._k_view(d), d["kop"],
                                 None if self.bf16 else d["kt"][:, :d["F"]], stream=stream)
            n += 1
        return n + self.dense.refresh(stream)

    def _act(self, d):
        a = d.get("act")
        return (a[0], a[1]) if a else (None, 0.0)

    def forward_front(self, x: torch.Tensor | None, nrows: int, stream=None, from_rows: torch.Tensor | None = None) -> int:
        """``x``: the f32 batch (first unit), or ``from_rows``: activation rows of the dense block below, in the tile dtype."""
        n = 0
        c0 = self.front[0]
        xin = c0["C"] * c0["H"] * c0["W"]
        if from_rows is None:
            if self.bf16:
                ew.rows(x, n_rows=nrows, dst_bf16=self.xflat, stream=stream)
            else:
                ew.rows(x, n_rows=nrows, dst=self.xflat, stream=stream)
            n += 1
            from_rows = self.xflat
        hw = c0["H"] * c0["W"]
        cv.nchw_flat(nrows, c0["C"], hw, False, self.x0, from_rows[:, :xin], stream=stream)
        n += 1
        cur = self.x0
        for d in self.front:
            Mout = nrows * d["OH"] * d["OW"]
            g = cv.geom(nrows, d["C"], d["H"], d["W"], d["K"], d["S"], d["P"])
            act, ap = self._act(d)
            if d["kind"] == "conv" and d.get("direct"):
                cv.conv1_fwd(g, d["F"], cur, self._k_view(d), self._kb_view(d), d["y"], act=act, act_param=ap, stream=stream)
                n += 1
            elif d["kind"] == "conv":
                cv.im2col(g, cur, d["cols"], d["colsT"] if self.wgrad_t else None, stream=stream)
                kw = dict(bias=self._kb_view(d), act=act, act_param=ap, status=self.status, stream=stream)
                if self.bf16:
                    kw["out_bf16"] = d["y"][:Mout, :d["F"]]
                else:
                    kw["out"] = d["y"][:Mout, :d["F"]]
                gemm(d["cols"][:Mout, :d["ckk"]], d["kop"], **kw)
                n += 2
            else:
                cv.pool_fwd(g, cur, d["y"], d["arg"], act=act, act_param=ap, stream=stream)
                n += 1
            cur = d["y"]
        last = self.front[-1]
        de = self.dense
        cv.nchw_flat(nrows, last["F"], last["OH"] * last["OW"], True, last["y"], de.a[0],
                     out_t=None if de.at is None else de.at[0], stream=stream)
        return n + 1

    def backward_front(self, nrows: int, accumulate: bool, stream=None, grad_rows: torch.Tensor | None = None,
                       grad_rows_t: torch.Tensor | None = None) -> int:
        """``grad_rows`` (units after the first): where the gradient w.r.t. the last pre-activation of the dense block below
        goes, as rows in the tile dtype (``grad_rows_t``: its transposed copy for K-major tf32 operands)."""
        n = 0
        de = self.dense
        last = self.front[-1]
        act, ap = self._act(last) if last["kind"] == "conv" else (None, 0.0)
        want_t = self.wgrad_t and last["kind"] == "conv" and not last.get("direct")
        cv.nchw_flat(nrows, last["F"], last["OH"] * last["OW"], False, last["dy"], de.d[0],
                     out_t=last["dyT"] if want_t else None, aux=last["y"], dact=act, dact_param=ap,
                     relu_quirk=self.relu_quirk, stream=stream)
        n += 1
        for j in range(len(self.front) - 1, -1, -1):
            d = self.front[j]
            prev = self.front[j - 1] if j > 0 else self.in_stub
            Mout, Min = nrows * d["OH"] * d["OW"], nrows * d["H"] * d["W"]
            g = cv.geom(nrows, d["C"], d["H"], d["W"], d["K"], d["S"], d["P"])
            pact, pap = (self._act(prev) if (prev is not None and prev["kind"] == "conv") else (None, 0.0))
            prev_t = prev is not None and prev["kind"] == "conv" and self.wgrad_t and not prev.get("direct")
            if d["kind"] == "conv" and d.get("direct"):
                F, ckk = d["F"], d["ckk"]
                cv.conv1_wgrad(g, F, self.x0, d["dy"], self.grads[d["off"]:d["off"] + F * ckk],
                               self.grads[d["off"] + F * ckk:d["off"] + d["n"]], beta=1.0 if accumulate else 0.0, stream=stream)
                n += 1
            elif d["kind"] == "conv":
                F, ckk = d["F"], d["ckk"]
                dy = d["dy"][:Mout, :F]
                if prev is not None:
                    if self.bf16:
                        gemm(dy, d["kop"], b_mn_major=True, out_bf16=d["dcols"][:Mout, :ckk], status=self.status, stream=stream)
                    else:
                        gemm(dy, d["kt"][:, :F], out=d["dcols"][:Mout, :ckk], status=self.status, stream=stream)
                    cv.col2im(g, d["dcols"], prev["dy"], prev["dyT"] if prev_t else None, aux=prev["y"], dact=pact,
                              dact_param=pap, relu_quirk=self.relu_quirk, stream=stream)
                    n += 2
                # weight gradient: K = every output pixel of the batch, tiny output -> split-K
                tmp = d["gk_tmp"]
                # one work unit per SM: every split writes its partial product into a slab of its own and a finishing pass
                # adds the slabs in order (run-to-run deterministic), so more splits than SMs only add slabs
                kb = -(-Mout // (64 if self.bf16 else 32))
                tiles = -(-F // 128) * (1 if ckk <= 128 else -(-ckk // 128))
                split = max(1, min(kb, -(-self.sms // tiles)))
                if not self.wgrad_t:
                    gemm(dy, d["cols"][:Mout, :ckk], a_mn_major=True, b_mn_major=True, out=tmp[:, :ckk], split_k=split,
                         status=self.status, stream=stream)
                else:
                    gemm(d["dyT"][:, :Mout], d["colsT"][:, :Mout], out=tmp[:, :ckk], split_k=split, status=self.status,
                         stream=stream)
                gk = self.grads[d["off"]:d["off"] + F * ckk]
                cv.operand_grad_to_kernel(F, d["C"], d["K"], tmp[:, :ckk], gk, beta=1.0 if accumulate else 0.0, stream=stream)
                ew.colsum(dy, self.grads[d["off"] + F * ckk:d["off"] + d["n"]], beta=1.0 if accumulate else 0.0, stream=stream)
                n += 4      # split GEMM + finishing pass, permutation, bias column sums
            else:
                if prev is None:
                    continue
                act, ap = self._act(d)
                d["dx32"].zero_()
                cv.pool_bwd(g, d["dy"], d["y"], d["arg"], d["dx32"], act=act, act_param=ap, relu_quirk=self.relu_quirk,
                            stream=stream)
                cv.finish_delta(Min, d["C"], d["dx32"], prev["dy"], prev["dyT"] if prev_t else None, aux=prev["y"],
                                dact=pact, dact_param=pap, relu_quirk=self.relu_quirk, stream=stream)
                n += 3
        if self.in_stub is not None:
            c0 = self.front[0]
            xin = c0["C"] * c0["H"] * c0["W"]
            cv.nchw_flat(nrows, c0["C"], c0["H"] * c0["W"], True, self.dx0, grad_rows[:, :xin],
                         out_t=None if grad_rows_t is None else grad_rows_t, stream=stream)
            n += 1
        return n

    def step(self, x, y, nrows, idx=None, accumulate=False, stream=None, after_layer=None) -> int:
        if idx is not None:
            raise NotImplementedError("index gather is done by the batch feeder for conv models")
        de = self.dense
        n = self.forward_front(x, nrows, stream)
        ew.rows(y, n_rows=nrows, dst=de.ybuf, stream=stream)
        n += 1
        n += de.forward(nrows, stream)
        n += de.loss_backward(nrows, stream)
        n += de.backward(nrows, accumulate, stream)
        n += self.backward_front(nrows, accumulate, stream)
        return n


def _units(layers: list[dict]) -> list[tuple[list[dict], list[dict]]]:
    """Split a layer list into (conv/pool run, dense run) units; a model must end with a dense layer."""
    out, i = [], 0
    while i < len(layers):
        front, dense = [], []
        while i < len(layers) and layers[i]["kind"] != "dense":
            front.append(layers[i]); i += 1
        while i < len(layers) and layers[i]["kind"] == "dense":
            dense.append(layers[i]); i += 1
        if not dense:
            raise NotImplementedError("a model needs a dense layer after its last conv/pool layer on the GPU")
        out.append((front, dense))
    return out


class StagedEngine:
    """Units of ``(conv | pool)* dense+`` chained in any order the model asks for (machine_learning/src/arch/layer.rs:10-19
    puts no order on the layer kinds). Every unit but the last ends in a dense block whose activation rows feed the next
    unit's convolutions."""

    needs_f32_params = True

    def __init__(self, layers: list[dict], *, batch_size: int, tile_dtype: str, loss: str, params: torch.Tensor,
                 grads: torch.Tensor, params_bf16: torch.Tensor | None = None, leaky_relu_exact: bool = True,
                 bias_from_shadow: bool = False):
        units = _units(layers)
        self.B, self.max_ctas = batch_size, 0
        self.units, off = [], 0
        kw = dict(batch_size=batch_size, tile_dtype=tile_dtype, loss=loss, leaky_relu_exact=leaky_relu_exact)
        for k, (front, dense) in enumerate(units):
            final = k == len(units) - 1
            pb = None if params_bf16 is None else params_bf16[off:]
            if front:
                prev_act = units[k - 1][1][-1].get("act") if k > 0 else None
                u = ConvNetEngine(front + dense, params=params[off:], grads=grads[off:], params_bf16=pb, first=k == 0,
                                  prev_act=prev_act, final=final, **kw)
            else:           # only the first unit can be dense-only
                u = GpuEngine(dense, params=params[off:], grads=grads[off:], params_bf16=pb, bias_from_shadow=False, final=final,
                              **kw)
            off += u.n_params
            self.units.append(u)
        self.n_params = off
        last = self._dense(self.units[-1])
        self.loss_sum, self.correct, self.status = last.loss_sum, last.correct, last.status
        for u in self.units:        # one status word for every GEMM of the model
            u.status = self.status
            if isinstance(u, ConvNetEngine):
                u.dense.status = self.status

    @staticmethod
    def _dense(u) -> GpuEngine:
        return u.dense if isinstance(u, ConvNetEngine) else u

    def refresh(self, stream=None) -> int:
        return sum(u.refresh(stream) for u in self.units)

    def step(self, x, y, nrows, idx=None, accumulate=False, stream=None, after_layer=None) -> int:
        if idx is not None:
            raise NotImplementedError("index gather is done by the batch feeder for conv models")
        last = self._dense(self.units[-1])
        ew.rows(y, n_rows=nrows, dst=last.ybuf, stream=stream)
        n, rows_in = 1, None
        for k, u in enumerate(self.units):
            if isinstance(u, ConvNetEngine):
                n += u.forward_front(x if k == 0 else None, nrows, stream, from_rows=rows_in)
                n += u.dense.forward(nrows, stream)
            else:
                if u.bf16:
                    ew.rows(x, n_rows=nrows, dst_bf16=u.a[0], stream=stream)
                elif u.mn:
                    ew.rows(x, n_rows=nrows, dst=u.a[0], stream=stream)
                else:
                    ew.rows(x, n_rows=nrows, dst=u.a[0], dst_t=u.at[0], stream=stream)
                n += 1 + u.forward(nrows, stream)
            rows_in = self._dense(u).out_act
        n += last.loss_backward(nrows, stream)
        for k in range(len(self.units) - 1, -1, -1):
            u = self.units[k]
            if isinstance(u, ConvNetEngine):
                n += u.dense.backward(nrows, accumulate, stream)
                below = self._dense(self.units[k - 1]) if k > 0 else None
                n += u.backward_front(nrows, accumulate, stream,
                                      grad_rows=None if below is None else below.d[-1],
                                      grad_rows_t=None if (below is None or below.dt is None) else below.dt[-1])
            else:
                n += u.backward(nrows, accumulate, stream)
        return n


def make_engine(layers: list[dict], **kw):
    """The engine for a layer list: dense-only, one conv/pool front followed by dense layers, or chained units."""
    if all(l["kind"] == "dense" for l in layers):
        return GpuEngine(layers, **kw)
    if len(_units(layers)) == 1:
        return ConvNetEngine(layers, **kw)
    return StagedEngine(layers, **kw)
