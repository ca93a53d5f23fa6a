"""CPU restatement of the reference's optimizer step and schedule (TEST INFRASTRUCTURE ONLY).

onecycle_point : optim.h:18-44 (PyTorch-compatible OneCycleLR multiplier and inverse-cycled momentum).
Optimizer.step : cuda/optim.cuh:66-118 — global-norm clip, then
    * "mantissa" AdamW on embedding, head and norms (decay on the head only), bias
      correction with the *current* beta1 (cuda/optim.cuh:93-105);
    * Muon on the hidden matrices (cuda/optim.cuh:16-65): Nesterov momentum, BF16
      Frobenius normalisation, `ns_steps` BF16 Newton-Schulz iterations with
      (3.4445, -4.775, 2.0315), lr*sqrt(max(1, rows/cols)), decoupled decay.
  ``hidden="adamw"`` sends the hidden matrices through AdamW with decay instead (the
  scaled architecture's plain-AdamW configuration; tied embedding counts as the head).
All arithmetic is float32 like the device code; weights are exact FP32 masters.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from .model import Arch, specification, is_norm, is_hidden_matrix

f32 = np.float32


@dataclass
class OneCycle:
    total_steps: int = 0
    warmup_fraction: float = 0.30
    initial_lr_fraction: float = 0.04
    final_lr_fraction: float = 0.000004
    low_momentum: float = 0.85
    high_momentum: float = 0.95


def onecycle_point(s: OneCycle, step: int):
    ok = (s.total_steps >= 1 and 0 <= step < s.total_steps and 0 < s.warmup_fraction < 1
          and 0 < s.initial_lr_fraction < 1 and 0 < s.final_lr_fraction <= s.initial_lr_fraction
          and 0 <= s.low_momentum < 1 and s.low_momentum <= s.high_momentum < 1)
    if not ok:
        raise ValueError("Invalid OneCycle schedule or step")
    warmup_steps = s.warmup_fraction * s.total_steps - 1
    if warmup_steps == 0:
        raise ValueError("OneCycle warmup must span at least two steps")
    warming = step <= warmup_steps
    fraction = step / warmup_steps if warming else (step - warmup_steps) / (s.total_steps - 1 - warmup_steps)
    mix = lambda a, b: b + (a - b) * 0.5 * (1 + math.cos(math.pi * fraction))
    if warming:
        return f32(mix(s.initial_lr_fraction, 1.0)), f32(mix(s.high_momentum, s.low_momentum))
    return f32(mix(1.0, s.final_lr_fraction)), f32(mix(s.low_momentum, s.high_momentum))


def _bf16(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().float().numpy()


@dataclass
class Hyper:
    learning_rate: float = 0.0006
    muon_lr: float = 0.02
    beta1: float = 0.9
    beta2: float = 0.95
    momentum: float = 0.95
    weight_decay: float = 0.1
    epsilon: float = 1e-8
    clip: float = 1.0
    ns_steps: int = 5


class Optimizer:
    def __init__(self, arch: Arch, hyper: Hyper, weights: np.ndarray, hidden: str = "muon",
                 schedule: OneCycle | None = None):
        self.arch, self.h, self.hidden, self.schedule = arch, hyper, hidden, schedule
        self.w = np.array(weights, dtype=np.float32)
        self.m = np.zeros_like(self.w)
        self.v = np.zeros_like(self.w)
        self.step_index = 0
        self.entries = []
        offset = 0
        for name, shape in specification(arch):
            n = int(np.prod(shape))
            self.entries.append((name, shape, offset, n))
            offset += n

    def step(self, gradient: np.ndarray) -> None:
        h = self.h
        g = np.asarray(gradient, dtype=np.float32)
        clip = f32(1)
        if h.clip > 0:
            norm = np.sqrt(np.sum(g.astype(np.float64) ** 2)).astype(np.float32)
            clip = min(f32(1), f32(h.clip) / (norm + f32(1e-6)))
        multiplier, beta1, momentum = f32(1), f32(h.beta1), f32(h.momentum)
        if self.schedule is not None:
            multiplier, rate = onecycle_point(self.schedule, self.step_index)
            beta1 = momentum = rate
        lr = f32(h.learning_rate) * multiplier
        muon_lr = f32(h.muon_lr) * multiplier
        t = f32(self.step_index + 1)
        bc1 = f32(1) - f32(beta1) ** t
        bc2 = f32(1) - f32(h.beta2) ** t
        for name, shape, o, n in self.entries:
            sl = slice(o, o + n)
            gi = g[sl] * clip
            hidden = is_hidden_matrix(name.split(".")[-1], shape)
            if hidden and self.hidden == "muon":
                self._muon(sl, shape, gi, muon_lr, momentum)
                continue
            tied_head = self.arch.tied and name == "embedding"
            decay = name == "head" or tied_head or (hidden and self.hidden == "adamw")
            m = self.m[sl] + (f32(1) - beta1) * (gi - self.m[sl])
            v = f32(h.beta2) * self.v[sl] + (f32(1) - f32(h.beta2)) * gi * gi
            self.m[sl], self.v[sl] = m, v
            w = self.w[sl] * (f32(1) - lr * f32(h.weight_decay if decay else 0))
            self.w[sl] = w - (lr / bc1) * m / (np.sqrt(v) / np.sqrt(bc2) + f32(h.epsilon))
        self.step_index += 1

    def _muon(self, sl, shape, g, lr, mu):
        h = self.h
        rows, cols = shape
        m = self.m[sl] + (f32(1) - mu) * (g - self.m[sl])
        self.m[sl] = m
        x = _bf16(g + mu * (m - g)).reshape(rows, cols)
        if rows > cols:
            x = x.T.copy()
        norm = max(_bf16(np.sqrt(np.sum(x * x, dtype=np.float32))[None])[0], _bf16(np.array([1e-7]))[0])
        x = _bf16(x / norm)
        for _ in range(h.ns_steps):
            a = _bf16(x @ x.T)
            b = _bf16(f32(-4.775) * a + f32(2.0315) * (a @ a))
            x = _bf16(f32(3.4445) * x + b @ x)
        if rows > cols:
            x = x.T
        adjusted = lr * f32(math.sqrt(max(1.0, rows / cols)))
        w = self.w[sl].reshape(rows, cols) * (f32(1) - lr * f32(h.weight_decay))
        self.w[sl] = (w - adjusted * x).reshape(-1).astype(np.float32)
