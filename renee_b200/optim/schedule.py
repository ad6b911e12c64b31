"""Half-cosine learning-rate schedule with linear warm-up.

Parity: the reference builds ``transformers.get_cosine_schedule_with_warmup`` for both optimizers
and steps it every iteration (dl_base.py:241-242, 376-377, 395-397).  The multiplier is
``step / warmup`` during warm-up and ``max(0, 0.5 (1 + cos(pi * progress)))`` afterwards, with
``progress = (step - warmup) / (total - warmup)``.

The same closed form is evaluated on the device by the fused optimizer kernels (they read the
step counter from device memory), which keeps a captured CUDA graph of the training step valid
for every step.
"""
from __future__ import annotations

import math


def cosine_warmup_multiplier(step: int, warmup_steps: int, total_steps: int) -> float:
    if step < warmup_steps:
        return float(step) / float(max(1, warmup_steps))
    progress = float(step - warmup_steps) / float(max(1, total_steps - warmup_steps))
    return max(0.0, 0.5 * (1.0 + math.cos(math.pi * progress)))


class CosineWarmupSchedule:
    """Stateful wrapper with ``state_dict``/``load_state_dict`` (the reference checkpoints both
    scheduler states, dl_base.py:423-424)."""

    def __init__(self, base_lr: float, warmup_steps: int, total_steps: int):
        self.base_lr = float(base_lr)
        self.warmup_steps = int(warmup_steps)
        self.total_steps = int(total_steps)
        self.last_step = 0

    def multiplier(self, step: int | None = None) -> float:
        return cosine_warmup_multiplier(self.last_step if step is None else step, self.warmup_steps, self.total_steps)

    def lr(self, step: int | None = None) -> float:
        return self.base_lr * self.multiplier(step)

    def step(self) -> float:
        self.last_step += 1
        return self.lr()

    def state_dict(self) -> dict:
        return {"base_lr": self.base_lr, "warmup_steps": self.warmup_steps,
                "total_steps": self.total_steps, "last_step": self.last_step}

    def load_state_dict(self, sd: dict) -> None:
        self.base_lr = float(sd["base_lr"])
        self.warmup_steps = int(sd["warmup_steps"])
        self.total_steps = int(sd["total_steps"])
        self.last_step = int(sd["last_step"])
