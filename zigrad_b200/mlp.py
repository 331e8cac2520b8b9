"""MLP training step on the device interface.

Restates what the reference's MNIST example does above the device boundary
(``examples/mnist/src/model.zig:17-111`` for the model,
``examples/mnist/src/main-simple.zig:61-71`` for the loop, and the autograd
backward order of ``src/graph.zig:55-85`` / ``src/ndtensor.zig:780-796,
1092-1136``) as a fixed sequence of device ops over preallocated buffers, so
that the whole step can be captured once into a CUDA graph
(``CudaDevice.capture``) and replayed.

Two op sequences produce the same tensors:

* ``fused=False`` -- exactly the device calls the reference issues: per layer
  ``bmm_acc`` (beta 0), ``add`` (bias, in place), ``relu_fwd`` (in place); the
  loss; then per layer ``relu_inplace_bwd``, zero fill + ``unbroadcast``
  (alpha = beta = 1) for the bias gradient, zero fill + ``bmm_acc`` (beta 1)
  for dX and dW; then the optimizer.
* ``fused=True``  -- one zero fill of the flat gradient buffer, ``linear`` ops
  with bias / ReLU / ReLU-mask epilogues, bias gradients taken from the loss
  kernel (last layer) and from the dX GEMM epilogues (hidden layers): 10 kernel
  launches + 1 memset for the three-layer model.  When the last two layers have
  the widths the ``mlp_tail`` op is built for (128 -> 64 -> at most 16 classes:
  the MNIST model), ``step()`` replaces everything between the first layer's
  forward GEMM and the weight gradients by that one op; with plain SGD and no
  reduction between backward and update the weight updates then ride in the
  gradient GEMMs' epilogues (``fuse_update``): 6 launches per step (forward
  GEMM, tail, three independent weight-gradient GEMMs, the biases' update).

Parameters, gradients and optimizer state live in flat buffers in attach
order (W0, b0, W1, b1, ...), which is what a data-parallel step all-reduces
(one buffer) and what the multi-tensor optimizer kernels consume.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import numpy as np

from . import opspec
from .abi import BF16, SINGLE
from .device import CudaDevice, DeviceSlice


def kaiming_uniform(dims: Sequence[int], seed: int):
    """Seeded U(+-sqrt(6/fan_in)) weights and zero biases (synthetic stand-in
    for the reference's initialiser, examples/mnist/src/model.zig:75-87; the
    same host arrays are uploaded to every backend under comparison)."""
    g = np.random.Generator(np.random.PCG64(seed))
    Ws, bs = [], []
    for fan_in, fan_out in zip(dims[:-1], dims[1:]):
        bound = np.sqrt(6.0 / fan_in)
        Ws.append(g.uniform(-bound, bound, (fan_out, fan_in)).astype(np.float32))
        bs.append(np.zeros(fan_out, np.float32))
    return Ws, bs


def split_sm_shares(sms: int, tiles0: int, tiles1: int, k_slabs: int):
    """Shares of `sms` SMs for two split-K GEMMs that run side by side, the first on the critical
    path.  Both are grids of (output tiles x K ranges) CTAs, one CTA per SM, and a CTA's time goes
    with the 32-deep k-slabs of its range: the first gets as many K ranges as leave the second a
    range at most 1.3 times as long.  Returns (SMs of the first, SMs of the second) or None."""
    best = None
    for s0 in range(1, sms // tiles0 + 1):
        s1 = (sms - tiles0 * s0) // tiles1
        if s1 < 1:
            break
        if -(-k_slabs // s1) <= 1.3 * -(-k_slabs // s0):
            best = (tiles0 * s0, tiles1 * s1)
    return best


class MlpTrainer:
    def __init__(self, dev: CudaDevice, dims: Sequence[int], batch: int, weights, biases, opt: str = "sgd",
                 lr: float = 0.01, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, clip: bool = False,
                 max_norm: float = 10.0, delta: float = 1e-6, fused: bool = True, loss_div: Optional[int] = None,
                 index_labels: bool = False, bf16: bool = False, pad_logits: bool = True, zero_grads_in_update: bool = False,
                 tail: Optional[bool] = None, fuse_update: bool = True, update_by_layer: bool = False):
        self.dev, self.dims, self.B, self.L = dev, [int(d) for d in dims], int(batch), len(dims) - 1
        self.opt, self.lr, self.beta1, self.beta2, self.eps = opt, lr, beta1, beta2, eps
        self.clip, self.max_norm, self.delta = clip, max_norm, delta
        self.fused, self.index_labels, self.bf16 = fused, index_labels, bf16
        self.loss_div = float(loss_div if loss_div is not None else batch)
        self.t = 0  # Adam's optimizer-wide counter (advances once per tensor per step)
        if bf16 and not fused:
            raise ValueError("the bf16 path exists only as fused ops")
        # SGD only: the update kernel clears the gradients it applied, so the next step needs no
        # zero_grad launch (the gradients are then not readable after step())
        if zero_grads_in_update and not (fused and opt == "sgd"):
            raise ValueError("zero_grads_in_update needs the fused ops and SGD")
        self.zero_grads_in_update, self._grads_clear = bool(zero_grads_in_update), False
        # the fused middle of the step (opspec.mlp_tail): on by default wherever the library has a kernel for the widths
        can_tail = (fused and not bf16 and self.L >= 3 and
                    dev.mlp_tail_supported(SINGLE, self.dims[-3], self.dims[-2], self.dims[-1]))
        if tail and not can_tail:
            raise ValueError("no mlp_tail kernel for the widths %s" % self.dims[-3:])
        self.tail = can_tail if tail is None else bool(tail)
        self._dw_shares = None
        self.update_by_layer = bool(update_by_layer)
        # the tail path applies plain SGD from inside the backward pass (see _forward_backward_tail) unless told not to
        self.fuse_update = bool(fuse_update) and self.tail
        # flat parameter layout, attach order
        self.segments, off = [], 0
        for l in range(self.L):
            for n in (self.dims[l + 1] * self.dims[l], self.dims[l + 1]):
                self.segments.append((off, n))
                off += n
        self.n_params = off
        d = dev
        self.params = d.mem_cache_alloc(SINGLE, off)
        self.grads = d.mem_cache_alloc(SINGLE, off)
        self.norms = d.mem_cache_alloc(SINGLE, len(self.segments))
        flat = np.concatenate([np.concatenate([np.asarray(w, np.float32).ravel(), np.asarray(b, np.float32).ravel()])
                               for w, b in zip(weights, biases)])
        d.mem_transfer_htod(flat, self.params)
        d.mem_fill(self.grads, 0.0)
        if opt == "adam":
            self.m, self.v = d.mem_cache_alloc(SINGLE, off), d.mem_cache_alloc(SINGLE, off)
            d.mem_fill(self.m, 0.0)
            d.mem_fill(self.v, 0.0)
            # tensor updates done so far, kept on the device so that a captured step keeps counting on replay
            self.t_dev = d.from_numpy(np.zeros(1, np.uint64))
        self.W = [self.params.view(self.segments[2 * l][0], self.segments[2 * l][1]) for l in range(self.L)]
        self.b = [self.params.view(self.segments[2 * l + 1][0], self.segments[2 * l + 1][1]) for l in range(self.L)]
        self.dW = [self.grads.view(self.segments[2 * l][0], self.segments[2 * l][1]) for l in range(self.L)]
        self.db = [self.grads.view(self.segments[2 * l + 1][0], self.segments[2 * l + 1][1]) for l in range(self.L)]
        # activations and their gradients.  bf16 mode: hidden activations and all
        # backward operands are bf16, logits / loss / parameter gradients fp32.
        act_t = BF16 if bf16 else SINGLE
        # Row stride of the logits and their gradient: padded to a multiple of 4
        # floats in the fused path so that the skinny last-layer GEMMs (n, k or m
        # = number of classes) satisfy TMA's 16-byte stride rule and run on the
        # tensor cores; the reference op sequence keeps them contiguous.
        C = self.dims[-1]
        self.ld_out = (C + 3) // 4 * 4 if (fused and pad_logits) else C
        self.ld = [self.dims[l + 1] if l + 1 < self.L else self.ld_out for l in range(self.L)]
        self.act = [d.mem_cache_alloc(act_t if l + 1 < self.L else SINGLE, self.B * self.ld[l]) for l in range(self.L)]
        self.dact = [d.mem_cache_alloc(act_t if l + 1 < self.L else SINGLE, self.B * self.ld[l]) for l in range(self.L)]
        if self.ld_out != C:
            d.mem_fill(self.act[-1], 0.0)
            d.mem_fill(self.dact[-1], 0.0)
        self.loss = d.mem_cache_alloc(SINGLE, 1)
        if bf16:
            self.params_bf16 = d.mem_cache_alloc(BF16, off)
            d.cast(self.params, self.params_bf16)
            self.Wb = [self.params_bf16.view(self.segments[2 * l][0], self.segments[2 * l][1]) for l in range(self.L)]
            self.dlogits_bf16 = d.mem_cache_alloc(BF16, self.B * self.ld_out)
        d.sync()

    # ------------------------------------------------------------------ pieces
    def forward(self, X: DeviceSlice):
        d, B = self.dev, self.B
        inp = X
        if self.fused:
            # zero_grad (model.zig:57-62) as ONE fill of the flat gradient buffer; the
            # weight-gradient GEMMs then accumulate with beta = 1 as the reference does
            # (kept on the main stream: as a side branch joined after the forward pass it
            # cost more in extra graph dependencies than the 2.5 us it hides).  With
            # zero_grads_in_update the previous step's SGD kernel has cleared them already.
            if not self._grads_clear:
                d.mem_fill(self.grads, 0.0)
            self._grads_clear = False
        for l in range(self.L):
            K, N = self.dims[l], self.dims[l + 1]
            last = l + 1 == self.L
            if self.fused:
                W = self.Wb[l] if self.bf16 else self.W[l]
                d.dispatch(opspec.linear(inp, W, self.act[l], B, N, K, False, True, K, K, self.ld[l], 1.0, 0.0,
                                         "bias" if last else "bias_relu", self.b[l]))
            else:
                d.dispatch(opspec.bmm_acc(inp, self.W[l], self.act[l], (1, B, K), (1, K, N), (1, B, N), False, True, K, K, N, 1.0, 0.0))
                d.dispatch(opspec.add(self.b[l], self.act[l], self.act[l]))
                if not last:
                    d.dispatch(opspec.relu_fwd(self.act[l], self.act[l]))
            inp = self.act[l]
        return self.act[-1]

    def loss_and_grad(self, T: DeviceSlice):
        d, B, C = self.dev, self.B, self.dims[-1]
        if not self.fused:
            d.mem_fill(self.dact[-1], 0.0)  # ensure_grad(0), then `+=`
        if self.fused:  # the bias gradient of the last layer comes out of the same pass
            d.dispatch(opspec.softmax_ce(self.act[-1], T, B, C, self.loss, self.dact[-1], self.loss_div, accumulate=False,
                                         ld=self.ld_out, bias_grad=self.db[-1]))
        else:
            d.dispatch(opspec.softmax_ce(self.act[-1], T, B, C, self.loss, self.dact[-1], self.loss_div, accumulate=True))

    def backward(self, X: DeviceSlice, last_bias_done: bool = True, on_layer_grads: Optional[Callable[[int], None]] = None,
                 update_by_layer: bool = False):
        """Backward from dact[L-1].  `last_bias_done`: the bias gradient of the last
        layer was already produced by the loss kernel (fused path); pass False when
        dact[L-1] comes from elsewhere (e.g. the DQN's gather backward).
        `on_layer_grads(l)` (fused path) is called on the side stream right after
        layer l's weight gradient has been issued there -- dW[l] and db[l] are then
        final in stream order, so a data-parallel caller can start reducing that
        layer's slice of the gradient buffer while the backward pass goes on.
        `update_by_layer` (fused path, Adam): the optimizer step rides on the backward
        pass, a layer at a time.  Layer l's tensors are updated on a second side stream
        once its weight gradient (first side stream) and its dX product (main stream, the
        last reader of W[l]) have been issued, so the memory-bound update runs beside the
        tensor-bound GEMMs of the layers below.  Same arithmetic per element as one update
        over all tensors (zg_adam_step_part keeps every tensor's position in the step
        count); the caller must not call update() for this step.  Off by default: on the
        wide MLP the update then competes with the persistent GEMMs for memory bandwidth
        and the step got slower (2.39 ms against 2.27 ms with one update after the join)."""
        d, B = self.dev, self.B
        if self.fused and not last_bias_done:
            if self.ld_out != self.dims[-1]:
                raise ValueError("an external output gradient needs unpadded logits (pad_logits=False)")
            d.dispatch(opspec.unbroadcast(self.dact[-1], [B, self.dims[-1]], self.db[-1], [self.dims[-1]], None, 1.0, 0.0))
        for l in range(self.L - 1, -1, -1):
            K, N = self.dims[l], self.dims[l + 1]
            a_in = X if l == 0 else self.act[l - 1]
            dy = self.dact[l]
            if self.fused:
                ldy = self.ld[l]
                if l + 1 == self.L:
                    if self.bf16:  # fp32 dlogits -> bf16 operand of the backward GEMMs
                        d.cast(dy, self.dlogits_bf16)
                        dy = self.dlogits_bf16
                # bias gradients: db[L-1] came out of the loss kernel; db[l-1] is the
                # column sum of the masked dX that this layer's dX GEMM stores
                # (added by its epilogue into the zero-filled gradient buffer)
                # The weight gradient does not feed the dX chain: it goes to the side
                # stream (a parallel branch of a captured step), forked here where dY
                # is ready, and runs next to this layer's dX GEMM.
                with d.branch():
                    d.dispatch(opspec.linear(dy, a_in, self.dW[l], N, K, B, True, False, ldy, K, K, 1.0, 1.0))
                    if on_layer_grads is not None:
                        on_layer_grads(l)
                if l > 0:  # dX = dY . W, zeroed where the previous activation is <= 0
                    W = self.Wb[l] if self.bf16 else self.W[l]
                    d.dispatch(opspec.linear(dy, W, self.dact[l - 1], B, K, N, False, False, ldy, K, K, 1.0, 0.0,
                                             "relu_mask", None, self.act[l - 1], colsum=self.db[l - 1]))
                if update_by_layer:
                    with d.branch(1, after=(0,)):
                        self._adam_layer(l, last=(l == 0))
            else:
                if l + 1 < self.L:
                    d.dispatch(opspec.relu_inplace_bwd(self.act[l], dy))
                d.mem_fill(self.db[l], 0.0)
                d.dispatch(opspec.unbroadcast(dy, [B, N], self.db[l], [N], None, 1.0, 1.0))
                if l > 0:
                    d.mem_fill(self.dact[l - 1], 0.0)
                    d.dispatch(opspec.bmm_acc(dy, self.W[l], self.dact[l - 1], (1, B, N), (1, N, K), (1, B, K), False, False, N, K, K, 1.0, 1.0))
                d.mem_fill(self.dW[l], 0.0)
                d.dispatch(opspec.bmm_acc(dy, a_in, self.dW[l], (1, N, B), (1, B, K), (1, N, K), True, False, N, K, K, 1.0, 1.0))
        if self.fused:
            d.join()  # the weight gradients are complete before anything that follows on the main stream

    def _adam_layer(self, l: int, last: bool):
        """Adam over the two tensors of layer l: the segment list keeps every tensor (the others
        empty) so that the per-tensor step counts are those of one update over the whole model;
        the device counter is advanced by the last call of the step."""
        segs = [(off, n if j in (2 * l, 2 * l + 1) else 0) for j, (off, n) in enumerate(self.segments)]
        self.dev.dispatch(opspec.adam(self.params, self.grads, self.m, self.v, segs, self.t + 1, self.lr, self.beta1,
                                      self.beta2, self.eps, self.clip, self.max_norm, self.delta, self.norms,
                                      self.params_bf16 if self.bf16 else None, self.t_dev, advance_counter=last))
        if last:
            self.t += len(self.segments)  # host mirror (eager steps only; read_t() is the truth)

    def update(self):
        d = self.dev
        if self.opt == "sgd":
            d.dispatch(opspec.sgd(self.params, self.grads, self.segments, self.lr, self.clip, self.max_norm, self.delta, self.norms,
                                  self.zero_grads_in_update))
            self._grads_clear = self.zero_grads_in_update
        elif self.opt == "adam":
            d.dispatch(opspec.adam(self.params, self.grads, self.m, self.v, self.segments, self.t + 1, self.lr, self.beta1,
                                   self.beta2, self.eps, self.clip, self.max_norm, self.delta, self.norms,
                                   self.params_bf16 if self.bf16 else None, self.t_dev))
            self.t += len(self.segments)  # host mirror (eager steps only; read_t() is the truth)
        elif self.opt != "none":
            raise ValueError(self.opt)

    # -------------------------------------------------------------------- step
    def layer_grads(self, l: int) -> DeviceSlice:
        """The contiguous slice [dW_l ; db_l] of the flat gradient buffer."""
        off = self.segments[2 * l][0]
        return self.grads.view(off, self.segments[2 * l][1] + self.segments[2 * l + 1][1])

    def _forward_backward_tail(self, X: DeviceSlice, T: DeviceSlice, fuse_update: bool = False):
        """forward, loss and backward with the last two layers, the loss and the
        dX chain down to dact[L-3] done by one mlp_tail op.

        ``fuse_update`` (plain SGD, no all-reduce in between): the update rides on the
        backward pass instead of following it.  For layer 0 and the two tail layers nothing
        reads the weights any more once their gradient runs, so
        * with ``zero_grads_in_update`` (the gradients are not kept past the step) the
          weight-gradient GEMM accumulates straight into the weights,
          W += (-lr) * dY^T X (alpha = -lr, beta = 1, C = W): no gradient tensor, no update launch;
        * otherwise each weight gradient is followed, on its own stream, by the SGD update
          of that one tensor.
        The biases, whose gradients the tail op has finished, are updated behind the last
        layer's product; no update waits for the join of all streams.  The weights of the
        layers in between are still read by the dX products and are updated after the join."""
        d, B, L = self.dev, self.B, self.L
        if not self._grads_clear:
            d.mem_fill(self.grads, 0.0)
        self._grads_clear = False

        in_gemm = fuse_update and self.zero_grads_in_update
        nlr = -float(np.float32(self.lr))  # lr cast f64 -> f32, then negated (optim.zig:103)

        def target(l):  # (C, alpha) of layer l's weight-gradient product
            return (self.W[l], nlr) if in_gemm and l in (0, L - 2, L - 1) else (self.dW[l], 1.0)

        def update(segs):
            if in_gemm:
                segs = [sg for sg in segs if sg not in [self.segments[2 * l] for l in (0, L - 2, L - 1)]]
            if fuse_update and segs:
                d.dispatch(opspec.sgd(self.params, self.grads, segs, self.lr, False, self.max_norm, self.delta, self.norms,
                                      self.zero_grads_in_update))

        weight, bias = (lambda l: self.segments[2 * l]), (lambda l: self.segments[2 * l + 1])
        inp = X
        for l in range(L - 2):  # the layers in front of the tail
            K, N = self.dims[l], self.dims[l + 1]
            d.dispatch(opspec.linear(inp, self.W[l], self.act[l], B, N, K, False, True, K, K, self.ld[l], 1.0, 0.0, "bias_relu", self.b[l]))
            inp = self.act[l]
        h1, h2, C = self.dims[L - 2], self.dims[L - 1], self.dims[L]
        d.dispatch(opspec.mlp_tail(self.act[L - 3], self.W[L - 2], self.b[L - 2], self.W[L - 1], self.b[L - 1], T, B, h1, h2, C,
                                   self.ld_out, self.loss_div, self.act[L - 2], self.act[L - 1], self.loss, self.dact[L - 1],
                                   self.dact[L - 2], self.dact[L - 3], self.db[L - 1], self.db[L - 2], self.db[L - 3],
                                   weights_ready=L - 2 >= 1))
        # the weight gradients of the two tail layers are independent of each other and of everything that follows:
        # one side stream each.
        # With one layer in front of the tail, its weight gradient (main stream) runs beside the two of the tail:
        # the SMs are shared out by output tiles so that the three split-K grids fit in one wave together.
        share = self._dw_sm_shares() if L == 3 else {}
        with d.branch(0):
            Cw, a = target(L - 2)
            d.dispatch(opspec.linear(self.dact[L - 2], self.act[L - 3], Cw, h2, h1, B, True, False, h2, h1, h1, a, 1.0,
                                     sm_budget=share.get(L - 2, 0)))
            update([weight(L - 2)])
        with d.branch(1):
            Cw, a = target(L - 1)
            d.dispatch(opspec.linear(self.dact[L - 1], self.act[L - 2], Cw, C, h2, B, True, False, self.ld_out, h2, h2, a, 1.0))
            # the tail op wrote the bias gradients of its two layers and of the layer in front of it
            update([weight(L - 1)] + [bias(l) for l in (L - 3, L - 2, L - 1)])
        for l in range(L - 3, -1, -1):
            K, N = self.dims[l], self.dims[l + 1]
            a_in = X if l == 0 else self.act[l - 1]
            if l == 0:  # nothing else is left on the main stream: the largest weight gradient runs there
                Cw, a = target(0)
                d.dispatch(opspec.linear(self.dact[l], a_in, Cw, N, K, B, True, False, N, K, K, a, 1.0, sm_budget=share.get(0, 0)))
                update([weight(0)])
            else:
                with d.branch(0):
                    d.dispatch(opspec.linear(self.dact[l], a_in, self.dW[l], N, K, B, True, False, N, K, K, 1.0, 1.0))
                d.dispatch(opspec.linear(self.dact[l], self.W[l], self.dact[l - 1], B, K, N, False, False, N, K, K, 1.0, 0.0,
                                         "relu_mask", None, self.act[l - 1], colsum=self.db[l - 1]))
        d.join()
        if fuse_update:
            # what did not ride on the backward pass: the weights the dX products read and the biases in front of them
            update([weight(l) for l in range(1, L - 2)] + [bias(l) for l in range(L - 3)])
            self._grads_clear = self.zero_grads_in_update

    def _dw_sm_shares(self) -> dict:
        """SMs for each tensor-core weight-gradient GEMM of a three-layer step (layers 0 and 1; the last
        layer's output is a few rows and goes to a small FFMA kernel that fits beside the others)."""
        if self._dw_shares is None:
            t0, t1 = (-(-self.dims[l + 1] // 128) * -(-self.dims[l] // 128) for l in (0, 1))
            best = split_sm_shares(self.dev.sm_count(), t0, t1, -(-self.B // 32))
            self._dw_shares = {0: best[0], 1: best[1]} if best else {}
        return self._dw_shares

    def step(self, X: DeviceSlice, T: DeviceSlice, allreduce: Optional[Callable[[DeviceSlice], None]] = None):
        """forward + loss + backward [+ gradient all-reduce] + update, all
        asynchronous on the device stream.  The loss stays in ``self.loss``."""
        if self.tail:
            fuse = self.fuse_update and allreduce is None and self.opt == "sgd" and not self.clip
            self._forward_backward_tail(X, T, fuse_update=fuse)
            if fuse:
                return
        else:
            by_layer = self.update_by_layer and self.fused and self.opt == "adam" and allreduce is None
            self.forward(X)
            self.loss_and_grad(T)
            self.backward(X, update_by_layer=by_layer)
            if by_layer:
                return
        if allreduce is not None:
            fused = getattr(allreduce, "reduce_and_sgd", None)
            if fused is not None and self.opt == "sgd" and not self.clip:
                if self.zero_grads_in_update:
                    fused(self.grads, self.params, self.lr, True)  # reduction, update and zero_grad in one kernel
                    self._grads_clear = True
                else:
                    fused(self.grads, self.params, self.lr)  # reduction and update in one kernel
                return
            allreduce(self.grads)
        self.update()

    def read_loss(self) -> float:
        return float(self.dev.to_numpy(self.loss)[0])

    def read_t(self) -> int:
        """Adam's counter as the device holds it (tensor updates done so far)."""
        return int(self.dev.to_numpy(self.t_dev)[0]) if self.opt == "adam" else 0

    # ------------------------------------------------------------- inspection
    def act_numpy(self, l: int, grad: bool = False) -> np.ndarray:
        """Activation (or its gradient) of layer l as a [B, dims[l+1]] fp32 array
        (row padding of the logits stripped, bf16 widened)."""
        s = (self.dact if grad else self.act)[l]
        a = self.dev.to_numpy(s)
        if s.dtype == BF16:
            a = (a.astype(np.uint32) << 16).view(np.float32)
        return a.reshape(self.B, self.ld[l])[:, :self.dims[l + 1]].copy()

    def get_params(self):
        flat = self.dev.to_numpy(self.params)
        return self._split(flat)

    def get_grads(self):
        return self._split(self.dev.to_numpy(self.grads))

    def _split(self, flat):
        Ws, bs = [], []
        for l in range(self.L):
            o, n = self.segments[2 * l]
            Ws.append(flat[o:o + n].reshape(self.dims[l + 1], self.dims[l]).copy())
            o, n = self.segments[2 * l + 1]
            bs.append(flat[o:o + n].copy())
        return Ws, bs

    def free(self):
        d = self.dev
        d.sync()
        for s in [self.params, self.grads, self.norms, self.loss] + self.act + self.dact:
            d.mem_cache_free(s)
        if self.opt == "adam":
            d.mem_cache_free(self.m)
            d.mem_cache_free(self.v)
            d.mem_cache_free(self.t_dev)
        if self.bf16:
            d.mem_cache_free(self.params_bf16)
            d.mem_cache_free(self.dlogits_bf16)
