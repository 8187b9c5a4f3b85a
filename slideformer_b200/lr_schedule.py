"""Learning-rate schedule of the reference's training script: linear warm-up, then cosine decay
to zero (scripts/main_real.py:186-196), applied through `update_learning_rate` before each step.
"""
from __future__ import annotations

import math


def warmup_cosine_lr(global_step: int, learning_rate: float, warmup_steps: int, total_steps: int) -> float:
    """lr for `global_step` (0-based): learning_rate * step / max(1, warmup) during warm-up, then
    learning_rate * 0.5 * (1 + cos(pi * progress)) with progress = (step - warmup) / max(1, total - warmup)."""
    if global_step < warmup_steps:
        return learning_rate * (global_step / max(1, warmup_steps))
    progress = (global_step - warmup_steps) / max(1, (total_steps - warmup_steps))
    return learning_rate * 0.5 * (1.0 + math.cos(math.pi * progress))


class WarmupCosine:
    """Drives anything with `update_learning_rate(lr)` (LayerAdam, SlideFormerOffloader)."""

    def __init__(self, target, learning_rate: float, warmup_steps: int, total_steps: int):
        self.target, self.learning_rate = target, float(learning_rate)
        self.warmup_steps, self.total_steps = int(warmup_steps), int(total_steps)
        self.global_step = 0

    def step(self) -> float:
        """Set the lr for the step about to run and advance the counter; returns that lr."""
        lr = warmup_cosine_lr(self.global_step, self.learning_rate, self.warmup_steps, self.total_steps)
        self.target.update_learning_rate(lr)
        self.global_step += 1
        return lr
