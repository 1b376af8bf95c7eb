"""Learning-rate schedulers (crates/axonml-optim/src/lr_scheduler.rs:15-451).  Every scheduler
implements the reference's ``LRScheduler`` trait: ``step(optimizer)``, ``get_last_lr()``,
``get_step()``; the optimizer may also be bound at construction, in which case ``step()`` needs
no argument."""
from __future__ import annotations

import math


class LRScheduler:
    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.base_lr = optimizer.get_lr()
        self.last_lr = self.base_lr
        self.current_step = 0

    def _lr(self, step: int) -> float:  # pragma: no cover - abstract
        raise NotImplementedError

    def step(self, optimizer=None) -> None:
        opt = optimizer or self.optimizer
        self.current_step += 1
        self.last_lr = self._lr(self.current_step)
        opt.set_lr(self.last_lr)

    def get_last_lr(self) -> float: return self.last_lr
    def get_step(self) -> int: return self.current_step

    def state_dict(self) -> dict:
        return {k: v for k, v in self.__dict__.items() if k != "optimizer"}

    def load_state_dict(self, sd: dict) -> None:
        self.__dict__.update(sd)


class StepLR(LRScheduler):
    def __init__(self, optimizer, step_size: int, gamma: float = 0.1):
        super().__init__(optimizer)
        self.step_size, self.gamma = step_size, gamma

    @classmethod
    def new(cls, optimizer, step_size, gamma): return cls(optimizer, step_size, gamma)

    def _lr(self, step): return self.base_lr * self.gamma ** (step // self.step_size)


class MultiStepLR(LRScheduler):
    def __init__(self, optimizer, milestones, gamma: float = 0.1):
        super().__init__(optimizer)
        self.milestones, self.gamma = sorted(milestones), gamma

    @classmethod
    def new(cls, optimizer, milestones, gamma): return cls(optimizer, milestones, gamma)

    def _lr(self, step):
        return self.base_lr * self.gamma ** sum(1 for m in self.milestones if step >= m)


class ExponentialLR(LRScheduler):
    def __init__(self, optimizer, gamma: float):
        super().__init__(optimizer)
        self.gamma = gamma

    @classmethod
    def new(cls, optimizer, gamma): return cls(optimizer, gamma)

    def _lr(self, step): return self.base_lr * self.gamma ** step


class CosineAnnealingLR(LRScheduler):
    def __init__(self, optimizer, t_max: int, eta_min: float = 0.0):
        super().__init__(optimizer)
        self.t_max, self.eta_min = t_max, eta_min

    @classmethod
    def new(cls, optimizer, t_max): return cls(optimizer, t_max)

    @classmethod
    def with_eta_min(cls, optimizer, t_max, eta_min): return cls(optimizer, t_max, eta_min)

    def _lr(self, step):
        t = min(step, self.t_max)
        return self.eta_min + (self.base_lr - self.eta_min) * (1 + math.cos(math.pi * t / self.t_max)) / 2


class ReduceLROnPlateau(LRScheduler):
    def __init__(self, optimizer, mode: str = "min", factor: float = 0.1, patience: int = 10,
                 threshold: float = 1e-4, min_lr: float = 0.0):
        super().__init__(optimizer)
        self.mode, self.factor, self.patience = mode, factor, patience
        self.threshold, self.min_lr = threshold, min_lr
        self.best = None
        self.num_bad = 0

    @classmethod
    def new(cls, optimizer): return cls(optimizer)

    @classmethod
    def with_options(cls, optimizer, mode, factor, patience, threshold, min_lr):
        return cls(optimizer, mode, factor, patience, threshold, min_lr)

    def step_with_metric(self, optimizer_or_metric, metric=None) -> None:
        if metric is None:
            opt, metric = self.optimizer, optimizer_or_metric
        else:
            opt = optimizer_or_metric
        self.current_step += 1
        better = (self.best is None or
                  (metric < self.best - self.threshold if self.mode == "min" else metric > self.best + self.threshold))
        if better:
            self.best, self.num_bad = metric, 0
        else:
            self.num_bad += 1
            if self.num_bad > self.patience:
                self.last_lr = max(opt.get_lr() * self.factor, self.min_lr)
                opt.set_lr(self.last_lr)
                self.num_bad = 0

    def step(self, optimizer=None) -> None:
        self.current_step += 1


class OneCycleLR(LRScheduler):
    """Cosine warm-up from max_lr/div_factor to max_lr over pct_start of the run, then cosine
    decay to initial/final_div_factor."""

    def __init__(self, optimizer, max_lr: float, total_steps: int, pct_start: float = 0.3,
                 div_factor: float = 25.0, final_div_factor: float = 1e4):
        super().__init__(optimizer)
        self.max_lr, self.total_steps, self.pct_start = max_lr, total_steps, pct_start
        self.initial_lr = max_lr / div_factor
        self.min_lr = self.initial_lr / final_div_factor
        self.last_lr = self.initial_lr
        optimizer.set_lr(self.initial_lr)

    @classmethod
    def new(cls, optimizer, max_lr, total_steps): return cls(optimizer, max_lr, total_steps)

    @classmethod
    def with_options(cls, optimizer, max_lr, total_steps, pct_start, div_factor, final_div_factor):
        return cls(optimizer, max_lr, total_steps, pct_start, div_factor, final_div_factor)

    def _lr(self, step):
        up = max(1, int(self.pct_start * self.total_steps))
        if step <= up:
            return self.initial_lr + (self.max_lr - self.initial_lr) * (1 - math.cos(math.pi * step / up)) / 2
        t = min(step - up, self.total_steps - up) / max(1, self.total_steps - up)
        return self.min_lr + (self.max_lr - self.min_lr) * (1 + math.cos(math.pi * t)) / 2


class WarmupLR(LRScheduler):
    def __init__(self, optimizer, warmup_steps: int):
        super().__init__(optimizer)
        self.warmup_steps = warmup_steps

    @classmethod
    def new(cls, optimizer, warmup_steps): return cls(optimizer, warmup_steps)

    def _lr(self, step):
        return self.base_lr * min(1.0, step / max(1, self.warmup_steps))
