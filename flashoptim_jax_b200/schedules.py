"""Learning-rate schedules that a capturable step can evaluate on the device.

`warmup_cosine` restates `make_warmup_cosine_schedule` of the reference's examples
(examples/example_utils.py:94-103).  The object is callable on the host like the reference's closure
(`schedule(count)`, count zero-based), and `flash_*(capturable=True)` hands it to the device
(`fo_step_scalars_schedule`), where the same fp32 formula runs on the device counter.
"""

from __future__ import annotations

from typing import Any, Tuple

import numpy as np

F32 = np.float32
FO_SCHEDULE_WARMUP_COSINE = 1


class DeviceSchedule:
    """A schedule with a device twin: `kind` and three fp32 parameters."""

    kind: int = 0

    def device_params(self) -> Tuple[float, float, float]:
        raise NotImplementedError

    def __call__(self, count: Any) -> float:
        raise NotImplementedError


class WarmupCosine(DeviceSchedule):
    """Linear warm-up over `warmup_steps`, then cosine decay to zero at `total_steps`."""

    kind = FO_SCHEDULE_WARMUP_COSINE

    def __init__(self, total_steps: int, warmup_steps: int, peak_lr: float):
        self.total_steps, self.warmup_steps, self.peak_lr = int(total_steps), int(warmup_steps), float(peak_lr)

    def device_params(self) -> Tuple[float, float, float]:
        return float(self.total_steps), float(self.warmup_steps), self.peak_lr

    def __call__(self, count: Any) -> float:
        step = F32(int(count))
        total, warmup, peak = F32(self.total_steps), F32(self.warmup_steps), F32(self.peak_lr)
        if warmup > 0 and step < warmup:
            return float(F32(F32(peak * F32(step + F32(1.0))) / warmup))
        span = max(F32(1.0), F32(total - warmup))
        progress = min(max(F32(F32(step - warmup) / span), F32(0.0)), F32(1.0))
        c = F32(np.cos(np.float64(F32(F32(np.pi) * progress))))  # the cosine in float64, rounded once
        return float(F32(F32(np.float64(peak) * 0.5) * F32(F32(1.0) + c)))

    def __hash__(self) -> int:
        return hash((self.kind, self.total_steps, self.warmup_steps, self.peak_lr))

    def __eq__(self, other: Any) -> bool:
        return isinstance(other, WarmupCosine) and self.device_params() == other.device_params()


def warmup_cosine(total_steps: int, warmup_steps: int, peak_lr: float) -> WarmupCosine:
    return WarmupCosine(total_steps, warmup_steps, peak_lr)
