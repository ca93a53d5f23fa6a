"""CPU restatement of the byte-level GPT step (TEST INFRASTRUCTURE ONLY — see oracle/__init__.py).

Two architectures share one code path:

* ``Arch.reference(depth)`` — the reference's own model: width 16, 4 heads of 4,
  RMSNorm (eps 1e-6, FP32 scale), hard arg-max attention gated by GELU(top score),
  partial RoPE (first pair of every head, 1 rad per position), SwiGLU hidden 48,
  untied 256-way head.  Follows tests/reference.py:6-81 op by op, with its sizes
  made parameters.  cuda/model.cuh:7-59 is the device code both restate.
* ``Arch.gpt(...)`` — the scaled architecture: pre-LayerNorm (eps 1e-5, FP32 scale and
  bias), causal softmax attention with scale 1/sqrt(d_head), GELU (erf) MLP, tied
  embedding/head, no positional parameters.  It keeps the reference's numeric
  conventions: BF16 compute weights are the FP32 master *truncated* to 16 bits with a
  straight-through gradient (tests/reference.py:14-21), norm math in FP32 then BF16
  (tests/reference.py:53-54), BF16 activations between ops, FP32 logits
  (tests/reference.py:81), mean cross-entropy over batch x context (tests/verify.py:26-27).
  Softmax attention rounds where a fused kernel has to: the unnormalised probabilities
  exp(s - rowmax) go to BF16 for the product with V (they are a tensor-core operand), their FP32
  sum divides the result afterwards.

``fp32=True`` switches every rounding off (weights untruncated, FP32 activations): the
check mode whose tolerance is 1e-5.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
from torch.nn import functional as F


@dataclass(frozen=True)
class Arch:
    depth: int = 4
    width: int = 16
    heads: int = 4
    hidden: int = 48
    norm: str = "rms"          # "rms" | "ln"
    attention: str = "argmax"  # "argmax" | "softmax"
    mlp: str = "swiglu"        # "swiglu" | "gelu"
    tied: bool = False
    rope: str = "partial"      # "partial" | "none"
    vocab: int = 256

    @staticmethod
    def reference(depth: int = 4) -> "Arch":
        return Arch(depth=depth)

    @staticmethod
    def gpt(depth: int, width: int, heads: int, hidden: int | None = None) -> "Arch":
        return Arch(depth=depth, width=width, heads=heads, hidden=hidden or 4 * width,
                    norm="ln", attention="softmax", mlp="gelu", tied=True, rope="none")

    @property
    def d_head(self) -> int:
        return self.width // self.heads


def specification(arch: Arch):
    """Flat parameter order: the reference's (model.h:12-37, tests/reference.py:6-13) with
    sizes from ``arch``; LayerNorm adds a bias right after each scale, a GELU MLP has no
    ``up`` matrix, a tied model has no ``head``."""
    w, hd = arch.width, arch.hidden
    norm = lambda name: [(name + "w", (w,))] + ([(name + "b", (w,))] if arch.norm == "ln" else [])
    entries = [("embedding", (arch.vocab, w))]
    for l in range(arch.depth):
        layer = norm("ln1") + [("qkv", (3 * w, w)), ("attention", (w, w))] + norm("ln2")
        layer += [("gate", (hd, w))]
        if arch.mlp == "swiglu":
            layer += [("up", (hd, w))]
        layer += [("projection", (w, hd))]
        entries += [(f"{l}.{name}", shape) for name, shape in layer]
    entries += norm("final")
    if not arch.tied:
        entries.append(("head", (arch.vocab, w)))
    return entries


def parameter_count(arch: Arch) -> int:
    return sum(int(np.prod(shape)) for _, shape in specification(arch))


def is_norm(name: str) -> bool:
    return name.endswith(("ln1w", "ln2w", "finalw", "ln1b", "ln2b", "finalb"))


def is_hidden_matrix(name: str, shape) -> bool:
    """Matrices the reference hands to Muon (tests/verify.py:55-56): every 2-D tensor
    except embedding and head."""
    return len(shape) == 2 and name not in ("embedding", "head")


class _Truncate(torch.autograd.Function):
    """FP32 -> BF16 by dropping the low 16 bits; gradient passes through in FP32."""

    @staticmethod
    def forward(ctx, x):
        return (x.contiguous().view(torch.int32) & -65536).view(torch.float32).to(torch.bfloat16)

    @staticmethod
    def backward(ctx, grad):
        return grad.float()


class Model:
    def __init__(self, arch: Arch, seed: int = 42, scale: float = 0.02, fp32: bool = False):
        self.arch, self.fp32 = arch, fp32
        generator = torch.Generator().manual_seed(seed)
        self.params = {}
        for name, shape in specification(arch):
            if name.endswith("w") and is_norm(name):
                value = torch.ones(shape)
            elif len(shape) == 1:
                value = torch.zeros(shape)
            else:
                value = torch.randn(shape, generator=generator) * scale
                if name.endswith(("attention", "projection")):
                    value /= math.sqrt(2 * arch.depth)
            self.params[name] = torch.nn.Parameter(value)

    def flat(self) -> np.ndarray:
        return torch.cat([p.detach().flatten() for p in self.params.values()]).numpy().copy()

    def load(self, flat) -> None:
        offset = 0
        with torch.no_grad():
            for p in self.params.values():
                p.copy_(torch.as_tensor(np.asarray(flat[offset:offset + p.numel()])).reshape(p.shape))
                offset += p.numel()
        assert offset == len(flat)

    def flat_grad(self) -> np.ndarray:
        return torch.cat([p.grad.flatten() for p in self.params.values()]).numpy().copy()

    def zero_grad(self) -> None:
        for p in self.params.values():
            p.grad = None

    # -- forward ---------------------------------------------------------------------
    def forward(self, x: torch.Tensor, trace: dict | None = None) -> torch.Tensor:
        """x: int64 [B, T] bytes -> FP32 logits [B, T, 256].  ``trace``, when given, receives every
        layer's intermediate activations as FP32 arrays [B*T, features] under "<layer>.<name>"."""
        a, p = self.arch, self.params

        def keep(name, t):
            if trace is not None:
                trace[name] = t.detach().float().reshape(-1, t.shape[-1]).numpy()

        act = (lambda t: t.float()) if self.fp32 else (lambda t: t.bfloat16())
        if self.fp32:
            q = {n: v for n, v in p.items() if not is_norm(n)}
        else:
            q = {n: _Truncate.apply(v) for n, v in p.items() if not is_norm(n)}
        B, T = x.shape
        H, D, W = a.heads, a.d_head, a.width

        def norm(t, name):
            if a.norm == "rms":
                return act(F.rms_norm(t.float(), (W,), p[name + "w"], eps=1e-6))
            return act(F.layer_norm(t.float(), (W,), p[name + "w"], p[name + "b"], eps=1e-5))

        def linear(t, name):
            return F.linear(t, q[name])

        h = F.embedding(x, q["embedding"])
        positions = torch.arange(T, dtype=torch.float64)
        cos, sin = torch.cos(positions).float()[:, None], torch.sin(positions).float()[:, None]

        def rope(t):  # t: [B, H, T, D]; rotate dims (0, 1) of every head by `pos` radians
            t = t.float()
            x0, x1 = t[..., 0:1], t[..., 1:2]
            return act(torch.cat((x0 * cos - x1 * sin, x0 * sin + x1 * cos, t[..., 2:]), -1))

        mask = torch.ones(T, T, dtype=torch.bool).tril()
        for l in range(a.depth):
            s = f"{l}."
            keep(s + "x", h)
            n1 = norm(h, s + "ln1")
            keep(s + "normed1", n1)
            packed = linear(n1, s + "qkv")
            keep(s + "qkv", packed)
            query, key, value = [t.reshape(B, T, H, D).transpose(1, 2) for t in packed.split(W, -1)]
            if a.rope == "partial":
                query, key = rope(query), rope(key)
            scores = query.float() @ key.float().transpose(-1, -2)
            if a.attention == "argmax":
                top, index = scores.masked_fill(~mask, -1e30).max(-1, keepdim=True)
                selected = value.gather(2, index.expand(-1, -1, -1, D))
                out = act(selected.float() * F.gelu(top))
            else:
                scaled = (scores / math.sqrt(D)).masked_fill(~mask, float("-inf"))
                if self.fp32:
                    out = torch.softmax(scaled, -1) @ value.float()
                else:
                    unnormalised = torch.exp(scaled - scaled.max(-1, keepdim=True).values)
                    out = act((act(unnormalised).float() @ value.float()) / unnormalised.sum(-1, keepdim=True))
            out = out.transpose(1, 2).reshape(B, T, W)
            keep(s + "attended", out)
            h = h + linear(out, s + "attention")
            keep(s + "middle", h)
            n2 = norm(h, s + "ln2")
            keep(s + "normed2", n2)
            if a.mlp == "swiglu":
                # one packed projection = one BF16 input-gradient rounding (tests/reference.py:77-79)
                gate, up = F.linear(n2, torch.cat((q[s + "gate"], q[s + "up"]))).split(a.hidden, -1)
                middle = F.silu(gate) * up
            else:
                middle = act(F.gelu(linear(n2, s + "gate").float()))
            keep(s + "activated", middle)
            h = h + linear(middle, s + "projection")
        keep("final_x", h)
        final = norm(h, "final")
        keep("final_normed", final)
        head = q["embedding"] if a.tied else q["head"]
        return F.linear(final, head).float()

    # -- one evaluation the way tg_batch reports it -------------------------------------
    def batch(self, x: np.ndarray, y: np.ndarray, backward: bool = True, divisor: int | None = None):
        """Returns (logits [B,T,256], flat gradient of the mean loss or None, per-position
        mean loss [T]) — the three outputs of tg_batch (cuda/runtime.cu:291-320).
        ``divisor`` replaces B*T in the mean (data-parallel shards pass the global count)."""
        self.zero_grad()
        tx, ty = torch.as_tensor(x.astype(np.int64)), torch.as_tensor(y.astype(np.int64))
        logits = self.forward(tx)
        loss = F.cross_entropy(logits.flatten(0, 1), ty.flatten(), reduction="none").reshape(tx.shape)
        grad = None
        if backward:
            (loss.sum() / (divisor or loss.numel())).backward()
            grad = self.flat_grad()
        return logits.detach().numpy(), grad, loss.detach().mean(0).numpy()
