"""Warm-up + decay learning-rate schedule as a pure function of the step.

Shapes (reference: aspec/training/lr_scheduler.py:35-163): linear warm-up ``init_lr -> max_lr`` over
``warmup_steps``; then ``constant`` | ``linear`` | ``cosine`` | ``inverse-square-root`` | ``WSD`` (stable,
then a final decay of ``wsd_decay_steps`` shaped linear / cosine / exponential ``2 * 0.5^r - 1`` /
minus-sqrt) down to ``min_lr``; beyond ``total_steps`` the rate stays at ``min_lr``.

The schedule object holds only ``last_step``; ``state_dict`` is therefore tiny and a resumed run
reproduces the same rates exactly.
"""
from __future__ import annotations

import math
from typing import Optional

DECAY_STYLES = ("constant", "linear", "cosine", "inverse-square-root", "WSD")
WSD_STYLES = ("linear", "cosine", "exponential", "minus_sqrt")


def lr_at_step(step: int, *, max_lr: float, total_steps: int, warmup_steps: int = 0, min_lr: float = 0.0,
               init_lr: float = 0.0, decay_style: str = "cosine", wsd_decay_steps: Optional[int] = None,
               wsd_decay_style: Optional[str] = None) -> float:
    if warmup_steps > 0 and step <= warmup_steps:
        return init_lr + (max_lr - init_lr) * step / warmup_steps
    if decay_style == "constant":
        return max_lr
    if step > total_steps:
        return min_lr
    if decay_style == "inverse-square-root":
        return max(min_lr, max_lr * max(warmup_steps, 1) ** 0.5 / max(step, 1) ** 0.5)
    ratio = min(max((step - warmup_steps) / float(total_steps - warmup_steps), 0.0), 1.0)
    if decay_style == "linear":
        coeff = 1.0 - ratio
    elif decay_style == "cosine":
        coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
    elif decay_style == "WSD":
        start = total_steps - wsd_decay_steps
        if step <= start:
            coeff = 1.0
        else:
            r = (step - start) / float(wsd_decay_steps)
            coeff = {"linear": 1.0 - r, "cosine": 0.5 * (math.cos(math.pi * r) + 1.0),
                     "exponential": 2.0 * 0.5 ** r - 1.0, "minus_sqrt": 1.0 - math.sqrt(r)}[wsd_decay_style]
    else:
        raise ValueError(f"Unknown decay style: {decay_style}")
    return min_lr + coeff * (max_lr - min_lr)


class LRSchedulerWithWarmup:
    """Drives ``optimizer.lr`` (any object with an ``lr`` attribute or torch ``param_groups``)."""

    def __init__(self, optimizer, max_lr: float, total_steps: int, warmup_steps: int = 0,
                 min_lr: float = 0.0, init_lr: float = 0.0, decay_style: str = "cosine",
                 wsd_decay_steps: Optional[int] = None, wsd_decay_style: Optional[str] = None,
                 last_epoch: int = -1):
        self.max_lr, self.min_lr, self.init_lr = float(max_lr), float(min_lr), float(init_lr)
        self.warmup_steps, self.total_steps = int(warmup_steps), int(total_steps)
        self.decay_style, self.wsd_decay_steps, self.wsd_decay_style = decay_style, wsd_decay_steps, wsd_decay_style
        if self.min_lr < 0.0:
            raise ValueError(f"min_lr must be non-negative, got {self.min_lr}")
        if self.max_lr < self.min_lr:
            raise ValueError(f"max_lr must be >= min_lr, got max_lr={self.max_lr}, min_lr={self.min_lr}")
        if self.init_lr > self.max_lr:
            raise ValueError(f"init_lr must be <= max_lr, got init_lr={self.init_lr}, max_lr={self.max_lr}")
        if self.total_steps <= 0:
            raise ValueError(f"total_steps must be positive, got {self.total_steps}")
        if self.warmup_steps < 0 or self.warmup_steps >= self.total_steps:
            raise ValueError("warmup_steps must be in [0, total_steps), got "
                             f"warmup_steps={self.warmup_steps}, total_steps={self.total_steps}")
        if decay_style not in DECAY_STYLES:
            raise ValueError(f"Unknown decay style: {decay_style}")
        if decay_style == "WSD":
            if wsd_decay_steps is None or not 0 < wsd_decay_steps <= self.total_steps:
                raise ValueError("WSD decay requires wsd_decay_steps in (0, total_steps]")
            if wsd_decay_style not in WSD_STYLES:
                raise ValueError(f"Unknown WSD decay style: {wsd_decay_style}")
        self.optimizer = optimizer
        self.last_epoch = last_epoch
        self.step()

    def current_lr(self) -> float:
        return lr_at_step(self.last_epoch, max_lr=self.max_lr, total_steps=self.total_steps,
                          warmup_steps=self.warmup_steps, min_lr=self.min_lr, init_lr=self.init_lr,
                          decay_style=self.decay_style, wsd_decay_steps=self.wsd_decay_steps,
                          wsd_decay_style=self.wsd_decay_style)

    def step(self) -> None:
        self.last_epoch += 1
        lr = self.current_lr()
        if hasattr(self.optimizer, "param_groups"):
            for g in self.optimizer.param_groups:
                g["lr"] = lr
        if hasattr(self.optimizer, "lr"):
            self.optimizer.lr = lr

    def get_last_lr(self):
        return [self.current_lr()]

    def state_dict(self) -> dict:
        return {"last_epoch": self.last_epoch}

    def load_state_dict(self, state: dict) -> None:
        self.last_epoch = int(state["last_epoch"])
        lr = self.current_lr()
        if hasattr(self.optimizer, "param_groups"):
            for g in self.optimizer.param_groups:
                g["lr"] = lr
        if hasattr(self.optimizer, "lr"):
            self.optimizer.lr = lr


def get_lr_scheduler(optimizer, max_lr, total_steps, warmup_steps=0, min_lr=0.0, init_lr=0.0,
                     decay_style="cosine", wsd_decay_steps=None, wsd_decay_style=None, last_epoch=-1):
    return LRSchedulerWithWarmup(optimizer, max_lr, total_steps, warmup_steps, min_lr, init_lr, decay_style,
                                 wsd_decay_steps, wsd_decay_style, last_epoch)
