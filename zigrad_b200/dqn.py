"""DQN update step on the device interface.

Restates ``DQNAgent.train`` + ``updateTargetNetwork`` of the reference
(``examples/dqn/src/dqn_agent.zig:111-228``; that example still targets the
library's removed Model/Layer API and loops over host memory, marked there as
"illegal in the incoming device api") as a fixed sequence of device ops:

  target net forward (no grad) -> clamp +-100 -> max over dim 1
  targets = r + gamma * max * (1 - done) -> clamp
  policy net forward -> clamp in place -> gather by action
  smooth-L1 (beta 1) -> gather backward (scatter_add) -> backward -> Adam (clip on)
  soft target update: target = (1 - tau) * target + tau * policy

Every tensor is tiny (batch 256, 4-128-128-2), so the step is launch-latency
bound; it is meant to be captured into ONE CUDA graph and replayed.
"""
from __future__ import annotations

import numpy as np

from . import opspec
from .abi import SINGLE
from .device import USIZE, CudaDevice, DeviceSlice
from .mlp import MlpTrainer


class DqnTrainer:
    def __init__(self, dev: CudaDevice, dims, batch: int, weights, biases, lr: float = 1e-4, gamma: float = 0.99,
                 tau: float = 0.005, q_clip: float = 100.0):
        self.dev, self.B, self.C = dev, int(batch), int(dims[-1])
        self.gamma, self.tau, self.q_clip = gamma, tau, q_clip
        # policy net: Adam with the library's default clipping; target net: forward only
        self.policy = MlpTrainer(dev, dims, batch, weights, biases, "adam", lr=lr, clip=True, fused=True, pad_logits=False)
        self.target = MlpTrainer(dev, dims, batch, weights, biases, "none", fused=True, pad_logits=False)
        d, B = dev, self.B
        self.maxq = d.mem_cache_alloc(SINGLE, B)
        self.tmp = d.mem_cache_alloc(SINGLE, B)
        self.targets = d.mem_cache_alloc(SINGLE, B)
        self.q = d.mem_cache_alloc(SINGLE, B)
        self.dq = d.mem_cache_alloc(SINGLE, B)
        self.offsets = d.mem_cache_alloc(USIZE, B)
        self.gamma_s = d.from_numpy(np.array([gamma], np.float32))
        self.one_s = d.from_numpy(np.array([1.0], np.float32))
        self.loss = d.mem_cache_alloc(SINGLE, 1)

    def step(self, states: DeviceSlice, actions: DeviceSlice, next_states: DeviceSlice, rewards: DeviceSlice,
             dones: DeviceSlice):
        d, B, C, qc = self.dev, self.B, self.C, self.q_clip
        pol, tgt = self.policy, self.target
        # ---- targets (gradients disabled in the reference): a chain of small kernels that does not depend
        # on the policy net, so it runs on a side stream beside the policy forward
        with d.branch(1):
            qn = tgt.forward(next_states)
            d.dispatch(opspec.clamp_fwd(qn, qn, -qc, qc))
            d.dispatch(opspec.max_along(qn, [B, C], self.maxq, [B, 1], 1))
            d.dispatch(opspec.mul(self.maxq, self.gamma_s, self.tmp))          # gamma * max
            d.dispatch(opspec.sub(self.one_s, dones, self.targets))            # 1 - done
            d.dispatch(opspec.mul(self.tmp, self.targets, self.tmp))           # masked
            d.dispatch(opspec.add(rewards, self.tmp, self.targets))            # r + ...
            d.dispatch(opspec.clamp_fwd(self.targets, self.targets, -qc, qc))
            # the two zero fills the loss and the gather backward accumulate into (ensure_grad(0))
            d.mem_fill(self.dq, 0.0)
            d.mem_fill(pol.dact[-1], 0.0)
        # ---- policy forward, clamp outside the graph, gather by action
        q_all = pol.forward(states)
        d.dispatch(opspec.clamp_fwd(q_all, q_all, -qc, qc))
        d.gather_rows(q_all, actions, B, C, self.q, self.offsets)
        d.join()  # the targets and the cleared gradients are ready
        # ---- loss and its gradient w.r.t. the gathered values
        d.dispatch(opspec.smooth_l1(self.q, self.targets, 1.0, self.loss, self.dq))
        # ---- gather backward: scatter into a zero gradient of all Q values
        d.dispatch(opspec.scatter_add(self.dq, self.offsets, pol.dact[-1]))
        pol.backward(states, last_bias_done=False)
        pol.update()
        # ---- soft update of the target parameters (one kernel over the flat buffer)
        d.soft_update(pol.params, tgt.params, self.tau)

    def read_loss(self) -> float:
        return float(self.dev.to_numpy(self.loss)[0])

    def free(self):
        d = self.dev
        d.sync()
        for s in (self.maxq, self.tmp, self.targets, self.q, self.dq, self.offsets, self.gamma_s, self.one_s, self.loss):
            d.mem_cache_free(s)
        self.policy.free()
        self.target.free()
