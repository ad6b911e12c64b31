"""Device-resident hyper-parameter block and loss-scale state machine.

A captured CUDA graph bakes kernel arguments, so everything that changes from step to step lives
in one small fp32 device tensor that the kernels read:

* slots ``[0, 8)`` are written by the host once per step (one 32-byte pinned H2D copy): the two
  learning rates of the cosine schedule and the dropout seed;
* slots ``[8, 16)`` are owned by the device: loss scale, its inverse, the found-inf flag raised by
  the gradient all-reduce / unscale kernel, the growth tracker and the count of Adam steps actually
  taken.

The loss-scale state machine reproduces ``torch.cuda.amp.GradScaler`` as the reference uses it
(dl_base.py:158, 372-374): init ``2**12`` with ``--fp16xfc`` else ``2**16``, growth ×2 every 2000
clean steps, back-off ×0.5 and the encoder step skipped when a non-finite gradient is found.  Only
the encoder-input gradient is scaled (split loss scaling, dl_base.py:598-608); the classifier
update is never scaled.
"""
from __future__ import annotations

import torch


class HP:
    LR_XFC = 0
    LR_ENC = 1
    SEED = 2           # int32 bits
    # device-owned
    SCALE = 8
    INV_SCALE = 9
    FOUND_INF = 10
    TRACKER = 11
    ADAM_STEP = 12     # number of optimizer steps taken so far (+1 = step used for bias correction)
    SIZE = 16
    HOST_SLOTS = 8


class HyperParams:
    def __init__(self, device, init_scale: float = 2.0 ** 16, enabled: bool = True,
                 growth_factor: float = 2.0, backoff_factor: float = 0.5, growth_interval: int = 2000):
        self.device = torch.device(device)
        self.enabled = bool(enabled)
        self.growth_factor = float(growth_factor)
        self.backoff_factor = float(backoff_factor)
        self.growth_interval = int(growth_interval)
        self.buf = torch.zeros(HP.SIZE, dtype=torch.float32, device=self.device)
        scale = float(init_scale) if enabled else 1.0
        self.buf[HP.SCALE] = scale
        self.buf[HP.INV_SCALE] = 1.0 / scale
        # The host block is copied asynchronously; the CPU may already be preparing a later step when
        # the copy engine reads it, so each step gets its own pinned slot from a ring.
        self._ring = torch.zeros(self.RING, HP.HOST_SLOTS, dtype=torch.float32)
        if self.device.type == "cuda":
            self._ring = self._ring.pin_memory()
        self._slot = 0
        self.host = self._ring[0]

    # -- host-written part -------------------------------------------------------------------
    RING = 512

    def set_step(self, lr_xfc: float, lr_enc: float, seed: int) -> None:
        self._slot = (self._slot + 1) % self.RING
        self.host = self._ring[self._slot]
        self.host[HP.LR_XFC] = lr_xfc
        self.host[HP.LR_ENC] = lr_enc
        self.host.view(torch.int32)[HP.SEED] = int(seed) - (1 << 32) if int(seed) >= (1 << 31) else int(seed)

    def upload(self) -> None:
        self.buf[: HP.HOST_SLOTS].copy_(self.host, non_blocking=True)

    def seed_tensor(self) -> torch.Tensor:
        return self.buf.view(torch.int32)[HP.SEED: HP.SEED + 1]

    # -- device-owned part -------------------------------------------------------------------
    def update_scale(self) -> None:
        """End-of-step transition (runs on the device; no host synchronisation)."""
        if self.buf.is_cuda:
            from ..ops import cuda as cu
            cu.scaler_update(self.buf, self.enabled, self.growth_factor, self.backoff_factor, self.growth_interval)
            return
        b = self.buf
        if float(b[HP.FOUND_INF]) != 0.0:
            if self.enabled:
                b[HP.SCALE] *= self.backoff_factor
            b[HP.TRACKER] = 0.0
        else:
            b[HP.ADAM_STEP] += 1.0
            b[HP.TRACKER] += 1.0
            if self.enabled and float(b[HP.TRACKER]) >= self.growth_interval:
                b[HP.SCALE] *= self.growth_factor
                b[HP.TRACKER] = 0.0
        b[HP.INV_SCALE] = 1.0 / b[HP.SCALE]
        b[HP.FOUND_INF] = 0.0

    def get_scale(self) -> float:
        return float(self.buf[HP.SCALE])

    def state_dict(self) -> dict:
        b = self.buf.detach().cpu()
        return {"scale": float(b[HP.SCALE]), "growth_factor": self.growth_factor,
                "backoff_factor": self.backoff_factor, "growth_interval": self.growth_interval,
                "_growth_tracker": int(b[HP.TRACKER]), "adam_step": int(b[HP.ADAM_STEP]), "enabled": self.enabled}

    def load_state_dict(self, sd: dict) -> None:
        if not sd:
            return
        self.buf[HP.SCALE] = float(sd["scale"])
        self.buf[HP.INV_SCALE] = 1.0 / float(sd["scale"])
        self.buf[HP.TRACKER] = float(sd.get("_growth_tracker", 0))
        self.buf[HP.ADAM_STEP] = float(sd.get("adam_step", 0))
        self.growth_factor = float(sd.get("growth_factor", self.growth_factor))
        self.backoff_factor = float(sd.get("backoff_factor", self.backoff_factor))
        self.growth_interval = int(sd.get("growth_interval", self.growth_interval))
