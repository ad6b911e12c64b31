"""Counter-based dropout RNG shared by the CUDA kernels and their PyTorch oracles.

A dropout mask is a pure function of ``(seed, stream, element index)``: the kernels recompute it
in the backward pass instead of storing it, and a captured CUDA graph stays valid across steps
because ``seed`` is read from device memory (the step counter is folded into it each step).

``keep(idx) = (mix(seed, stream, idx) >> 8) * 2^-24 >= p``.  ``mix`` is two rounds of a
murmur3-style finaliser; the same integer arithmetic is reproduced below with int64 tensors masked
to 32 bits, so CPU tests can compare kernel outputs bit-for-bit in the mask.
"""
from __future__ import annotations

import torch

_M32 = 0xFFFFFFFF


def _mul32(x: torch.Tensor, c: int) -> torch.Tensor:
    # 32x32 -> low 32 bits without overflowing int64: split the constant in two 16-bit halves
    lo = (x * (c & 0xFFFF)) & _M32
    hi = ((x * (c >> 16)) & 0xFFFF) << 16
    return (lo + hi) & _M32


def mix32(seed, stream: int, idx: torch.Tensor) -> torch.Tensor:
    """idx: int64 tensor of non-negative element indices (< 2^32).  ``seed`` is a Python int or an int64 tensor
    (one element, on ``idx``'s device): the tensor form keeps the whole computation on the device, so it can be
    recorded into a CUDA graph and follow the device-resident seed from step to step."""
    x = (_mul32(idx & _M32, 0x9E3779B1) + (seed & _M32)) & _M32
    x = x ^ (x >> 16)
    x = _mul32(x, 0x85EBCA6B)
    x = x ^ (x >> 13)
    x = _mul32(x, 0xC2B2AE35)
    x = x ^ (x >> 16)
    x = (x + ((stream * 0x27D4EB2F) & _M32)) & _M32
    x = x ^ (x >> 15)
    x = _mul32(x, 0x2C1B3C6D)
    x = x ^ (x >> 12)
    x = _mul32(x, 0x297A2D39)
    x = x ^ (x >> 15)
    return x


def keep_mask(seed, stream: int, shape, p: float, device="cpu") -> torch.Tensor:
    """Boolean keep-mask of ``shape`` (row-major element index), True = element survives.  ``seed``: int or
    one-element integer tensor (see :func:`mix32`)."""
    n = 1
    for s in shape:
        n *= int(s)
    if p <= 0.0:
        return torch.ones(shape, dtype=torch.bool, device=device)
    idx = torch.arange(n, dtype=torch.int64, device=device)
    seed = seed.to(torch.int64).reshape(()) if torch.is_tensor(seed) else int(seed)
    u = (mix32(seed, int(stream), idx) >> 8).to(torch.float32) * (1.0 / 16777216.0)
    return (u >= p).view(*shape)


class DropoutRNG:
    """Host-side handle: base seed plus a per-step counter; ``stream`` ids name the call sites."""

    def __init__(self, seed: int):
        self.base_seed = int(seed) & _M32
        self.step = 0

    def seed_for_step(self) -> int:
        return (self.base_seed + 0x632BE5AB * (self.step + 1)) & _M32

    def advance(self) -> None:
        self.step += 1

    def state_dict(self) -> dict:
        return {"base_seed": self.base_seed, "step": self.step}

    def load_state_dict(self, sd: dict) -> None:
        self.base_seed = int(sd["base_seed"])
        self.step = int(sd["step"])
