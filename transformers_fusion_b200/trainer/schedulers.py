"""Learning-rate schedules.

The five optimizer-embedded schedules of the reference (CONSTANT, COSINE, LINEAR, WARMUP_COSINE,
COSINE_RESTART with an lr floor of 1e-8: src/trainer/optimizer.cpp:57-90) and its 14 scheduler classes
(src/trainer/scheduler.cpp, include/quant/scheduler.h): LinearDecay, CosineDecay, Exponential, Step,
ReduceLROnPlateau, OneCycle, Warmup, Sequential, Chained, CosineWarmupRestart, Poly, MultiStep,
LinearWarmupDecay, Cyclic.  Every scheduler is a callable ``lr = sched(step)`` (ReduceLROnPlateau also
takes the monitored metric through ``observe``)."""
from __future__ import annotations

import math
from typing import List, Sequence

LR_FLOOR = 1e-8


def schedule_lr(kind: str, base_lr: float, step: int, total_steps: int, warmup_steps: int = 0, min_ratio: float = 0.0,
                restart_period: int = 0) -> float:
    kind = kind.upper()
    total = max(1, total_steps)
    if kind == "CONSTANT":
        lr = base_lr
    elif kind == "LINEAR":
        lr = base_lr * max(min_ratio, 1.0 - step / total)
    elif kind == "COSINE":
        lr = base_lr * (min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * min(1.0, step / total))))
    elif kind == "WARMUP_COSINE":
        if warmup_steps > 0 and step < warmup_steps:
            lr = base_lr * (step + 1) / warmup_steps
        else:
            p = min(1.0, (step - warmup_steps) / max(1, total - warmup_steps))
            lr = base_lr * (min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * p)))
    elif kind == "COSINE_RESTART":
        period = restart_period or max(1, total // 4)
        lr = base_lr * (min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * (step % period) / period)))
    else:
        raise ValueError(kind)
    return max(lr, LR_FLOOR)


class Scheduler:
    def __init__(self, base_lr: float):
        self.base_lr = base_lr

    def get_lr(self, step: int) -> float:
        """The reference's spelling of a call (include/quant/scheduler.h:11); the value is remembered as ``last_lr``."""
        self.last_lr = float(self(step))
        return self.last_lr

    def get_last_lr(self) -> float:
        return getattr(self, "last_lr", self.base_lr)

    def __call__(self, step: int) -> float:
        raise NotImplementedError


class LinearDecay(Scheduler):
    def __init__(self, base_lr, total_steps, end_lr=0.0):
        super().__init__(base_lr)
        self.total, self.end = max(1, total_steps), end_lr

    def __call__(self, step):
        p = min(1.0, step / self.total)
        return max(self.base_lr + (self.end - self.base_lr) * p, LR_FLOOR)


class CosineDecay(Scheduler):
    def __init__(self, base_lr, total_steps, min_lr=0.0):
        super().__init__(base_lr)
        self.total, self.min = max(1, total_steps), min_lr

    def __call__(self, step):
        p = min(1.0, step / self.total)
        return max(self.min + (self.base_lr - self.min) * 0.5 * (1 + math.cos(math.pi * p)), LR_FLOOR)


class Exponential(Scheduler):
    def __init__(self, base_lr, gamma=0.999):
        super().__init__(base_lr)
        self.gamma = gamma

    def __call__(self, step):
        return max(self.base_lr * self.gamma ** step, LR_FLOOR)


class Step(Scheduler):
    def __init__(self, base_lr, step_size, gamma=0.1):
        super().__init__(base_lr)
        self.size, self.gamma = max(1, step_size), gamma

    def __call__(self, step):
        return max(self.base_lr * self.gamma ** (step // self.size), LR_FLOOR)


class MultiStep(Scheduler):
    def __init__(self, base_lr, milestones: Sequence[int], gamma=0.1):
        super().__init__(base_lr)
        self.milestones, self.gamma = sorted(milestones), gamma

    def __call__(self, step):
        return max(self.base_lr * self.gamma ** sum(1 for m in self.milestones if step >= m), LR_FLOOR)


class Poly(Scheduler):
    def __init__(self, base_lr, total_steps, power=2.0, end_lr=0.0):
        super().__init__(base_lr)
        self.total, self.power, self.end = max(1, total_steps), power, end_lr

    def __call__(self, step):
        p = min(1.0, step / self.total)
        return max((self.base_lr - self.end) * (1 - p) ** self.power + self.end, LR_FLOOR)


class Warmup(Scheduler):
    def __init__(self, base_lr, warmup_steps):
        super().__init__(base_lr)
        self.warm = max(1, warmup_steps)

    def __call__(self, step):
        return max(self.base_lr * min(1.0, (step + 1) / self.warm), LR_FLOOR)


class LinearWarmupDecay(Scheduler):
    def __init__(self, base_lr, warmup_steps, total_steps, end_lr=0.0):
        super().__init__(base_lr)
        self.warm, self.total, self.end = max(1, warmup_steps), max(2, total_steps), end_lr

    def __call__(self, step):
        if step < self.warm:
            return max(self.base_lr * (step + 1) / self.warm, LR_FLOOR)
        p = min(1.0, (step - self.warm) / max(1, self.total - self.warm))
        return max(self.base_lr + (self.end - self.base_lr) * p, LR_FLOOR)


class CosineWarmupRestart(Scheduler):
    def __init__(self, base_lr, warmup_steps, period, min_lr=0.0, t_mult=1.0):
        super().__init__(base_lr)
        self.warm, self.period, self.min, self.t_mult = warmup_steps, max(1, period), min_lr, t_mult

    def __call__(self, step):
        if step < self.warm:
            return max(self.base_lr * (step + 1) / max(1, self.warm), LR_FLOOR)
        s, period = step - self.warm, float(self.period)
        while s >= period:
            s -= period
            period *= self.t_mult
        return max(self.min + (self.base_lr - self.min) * 0.5 * (1 + math.cos(math.pi * s / period)), LR_FLOOR)


class OneCycle(Scheduler):
    def __init__(self, max_lr, total_steps, pct_start=0.3, div_factor=25.0, final_div=1e4):
        super().__init__(max_lr)
        self.total, self.pct, self.init, self.final = max(2, total_steps), pct_start, max_lr / div_factor, max_lr / final_div

    def __call__(self, step):
        up = self.pct * self.total
        if step < up:
            return max(self.init + (self.base_lr - self.init) * step / max(1.0, up), LR_FLOOR)
        p = min(1.0, (step - up) / max(1.0, self.total - up))
        return max(self.final + (self.base_lr - self.final) * 0.5 * (1 + math.cos(math.pi * p)), LR_FLOOR)


class Cyclic(Scheduler):
    def __init__(self, base_lr, max_lr, step_size_up=2000, mode="triangular", gamma=1.0):
        super().__init__(base_lr)
        self.max, self.up, self.mode, self.gamma = max_lr, max(1, step_size_up), mode, gamma

    def __call__(self, step):
        cycle = math.floor(1 + step / (2 * self.up))
        x = abs(step / self.up - 2 * cycle + 1)
        amp = (self.max - self.base_lr) * max(0.0, 1 - x)
        if self.mode == "triangular2":
            amp /= 2 ** (cycle - 1)
        elif self.mode == "exp_range":
            amp *= self.gamma ** step
        return max(self.base_lr + amp, LR_FLOOR)


class ReduceLROnPlateau(Scheduler):
    def __init__(self, base_lr, factor=0.5, patience=10, min_lr=LR_FLOOR, threshold=1e-4):
        super().__init__(base_lr)
        self.factor, self.patience, self.min, self.threshold = factor, patience, min_lr, threshold
        self.best, self.bad, self.lr = float("inf"), 0, base_lr

    def observe(self, metric: float):
        if metric < self.best - self.threshold:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
            if self.bad > self.patience:
                self.lr = max(self.lr * self.factor, self.min)
                self.bad = 0
        return self.lr

    def __call__(self, step):
        return self.lr


class Sequential(Scheduler):
    """Runs schedulers one after another; ``milestones[i]`` is the step at which scheduler i+1 takes over."""

    def __init__(self, schedulers: List[Scheduler], milestones: Sequence[int]):
        super().__init__(schedulers[0].base_lr)
        self.s, self.m = schedulers, list(milestones)

    def __call__(self, step):
        i = sum(1 for m in self.m if step >= m)
        start = self.m[i - 1] if i else 0
        return self.s[i](step - start)


class Chained(Scheduler):
    """Multiplies the relative factors of several schedulers."""

    def __init__(self, schedulers: List[Scheduler]):
        super().__init__(schedulers[0].base_lr)
        self.s = schedulers

    def __call__(self, step):
        lr = self.base_lr
        for s in self.s:
            lr *= s(step) / s.base_lr
        return max(lr, LR_FLOOR)


ALL = {c.__name__: c for c in (LinearDecay, CosineDecay, Exponential, Step, ReduceLROnPlateau, OneCycle, Warmup,
                               Sequential, Chained, CosineWarmupRestart, Poly, MultiStep, LinearWarmupDecay, Cyclic)}


class Constant(Scheduler):
    def __call__(self, step):
        return self.base_lr


class Lambda(Scheduler):
    """``fn(step)`` is the rate (not a multiplier), as in the reference's LambdaScheduler (include/quant/scheduler.h:120-128)."""

    def __init__(self, fn, base_lr: float = 0.0):
        super().__init__(base_lr)
        self.fn = fn

    def __call__(self, step):
        return float(self.fn(step))


# the reference's class names (include/quant/scheduler.h)
LRScheduler = Scheduler
ConstantScheduler = Constant
LambdaScheduler = Lambda
LinearDecayScheduler = LinearDecay
CosineDecayScheduler = CosineDecay
ExponentialDecayScheduler = Exponential
StepDecayScheduler = Step
MultiStepDecay = MultiStep
PolyScheduler = Poly
WarmupScheduler = Warmup
OneCycleScheduler = OneCycle
CyclicLR = Cyclic
ReduceLROnPlateauScheduler = ReduceLROnPlateau
SequentialScheduler = Sequential
ChainedScheduler = Chained
