"""Training utilities (crates/axonml/src/trainer.rs:30-478): ``TrainingConfig`` builder,
``TrainingState``, ``TrainingMetrics``, ``Callback``, ``EarlyStopping``, ``ProgressLogger``,
``TrainingHistory``, ``clip_grad_norm``, ``compute_accuracy`` - plus a real ``Trainer.fit`` (the
reference documents one but does not implement it, trainer.rs:10-13)."""
from __future__ import annotations

import dataclasses
import time

import torch

from .optim import clip_grad_norm as _clip


class TrainingConfig:
    def __init__(self):
        self._epochs, self._batch_size, self._lr = 10, 32, 1e-3
        self._clip, self._accum, self._log_every, self._amp, self._seed = None, 1, 100, False, None

    @classmethod
    def new(cls): return cls()
    def epochs(self, n): self._epochs = n; return self
    def batch_size(self, n): self._batch_size = n; return self
    def learning_rate(self, lr): self._lr = lr; return self
    def gradient_clip_norm(self, m): self._clip = m; return self
    def gradient_accumulation_steps(self, n): self._accum = n; return self
    def log_every(self, n): self._log_every = n; return self
    def mixed_precision(self, flag): self._amp = flag; return self
    def seed(self, s): self._seed = s; return self


@dataclasses.dataclass
class TrainingState:
    epoch: int = 0
    global_step: int = 0
    train_losses: list = dataclasses.field(default_factory=list)
    val_losses: list = dataclasses.field(default_factory=list)
    best_val_loss: float | None = None
    should_stop: bool = False

    @classmethod
    def new(cls): return cls()
    def current_epoch(self) -> int: return self.epoch
    def avg_train_loss(self) -> float: return sum(self.train_losses) / len(self.train_losses) if self.train_losses else 0.0
    def last_val_loss(self): return self.val_losses[-1] if self.val_losses else None


class TrainingMetrics:
    def __init__(self, loss: float):
        self.loss, self.accuracy, self.extra = float(loss), None, {}

    @classmethod
    def new(cls, loss): return cls(loss)
    def with_accuracy(self, a): self.accuracy = float(a); return self
    def with_metric(self, name, value): self.extra[name] = float(value); return self


class Callback:
    def on_train_begin(self, state): pass
    def on_train_end(self, state): pass
    def on_epoch_begin(self, epoch, state): pass
    def on_epoch_end(self, epoch, metrics, state) -> bool: return True      # False stops training
    def on_batch_end(self, step, metrics, state): pass


class EarlyStopping(Callback):
    def __init__(self, patience: int):
        self.patience, self._delta, self._mode = patience, 0.0, "min"
        self.best, self.bad = None, 0

    @classmethod
    def new(cls, patience): return cls(patience)
    def min_delta(self, d): self._delta = d; return self
    def mode(self, m): self._mode = m; return self

    def on_epoch_end(self, epoch, metrics, state) -> bool:
        v = metrics.extra.get("val_loss", metrics.loss)
        better = self.best is None or (v < self.best - self._delta if self._mode == "min" else v > self.best + self._delta)
        if better:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
        return self.bad < self.patience


class ProgressLogger(Callback):
    def __init__(self, log_every: int = 100, sink=print):
        self.log_every, self.sink, self._t0 = log_every, sink, time.time()

    @classmethod
    def new(cls, log_every): return cls(log_every)

    def on_batch_end(self, step, metrics, state):
        if self.log_every and step % self.log_every == 0:
            self.sink(f"step {step}: loss {metrics.loss:.4f}" + (f" acc {metrics.accuracy:.4f}" if metrics.accuracy is not None else ""))

    def on_epoch_end(self, epoch, metrics, state) -> bool:
        self.sink(f"epoch {epoch}: loss {metrics.loss:.4f} ({time.time() - self._t0:.1f}s)")
        return True


@dataclasses.dataclass
class TrainingHistory:
    train_loss: list = dataclasses.field(default_factory=list)
    val_loss: list = dataclasses.field(default_factory=list)
    train_acc: list = dataclasses.field(default_factory=list)
    val_acc: list = dataclasses.field(default_factory=list)
    lr: list = dataclasses.field(default_factory=list)

    @classmethod
    def new(cls): return cls()
    def best_train_loss(self): return min(self.train_loss) if self.train_loss else None
    def best_val_loss(self): return min(self.val_loss) if self.val_loss else None


def clip_grad_norm(parameters, max_norm: float) -> float:
    return float(_clip(list(parameters), max_norm))


def compute_accuracy(predictions: torch.Tensor, targets: torch.Tensor) -> float:
    """Fraction of rows whose argmax equals the target (class index, or one-hot row)."""
    pred = predictions.argmax(-1)
    tgt = targets.argmax(-1) if targets.dim() == predictions.dim() else targets.long()
    return float((pred == tgt).float().mean())


class Trainer:
    def __init__(self, model, optimizer, loss_fn, config: TrainingConfig | None = None, callbacks=None,
                 scheduler=None, device=None):
        self.model, self.optimizer, self.loss_fn = model, optimizer, loss_fn
        self.config, self.callbacks, self.scheduler = config or TrainingConfig(), list(callbacks or []), scheduler
        self.device = device
        self.state, self.history = TrainingState(), TrainingHistory()
        self.scaler = None

    def _to(self, t):
        return t.to(self.device, non_blocking=True) if self.device is not None else t

    def evaluate(self, loader) -> TrainingMetrics:
        self.model.eval()
        tot, acc, n = 0.0, 0.0, 0
        with torch.no_grad():
            for b in loader:
                x, y = self._to(b.data), self._to(b.targets)
                out = self.model(x)
                tot += float(self.loss_fn(out, y)) * b.size
                if out.dim() == 2:
                    acc += compute_accuracy(out, y) * b.size
                n += b.size
        self.model.train()
        return TrainingMetrics(tot / max(n, 1)).with_accuracy(acc / max(n, 1))

    def fit(self, train_loader, val_loader=None) -> TrainingHistory:
        cfg = self.config
        if cfg._seed is not None:
            torch.manual_seed(cfg._seed)
        if cfg._amp and self.scaler is None:
            from .optim import GradScaler
            self.scaler = GradScaler()
        for cb in self.callbacks:
            cb.on_train_begin(self.state)
        self.model.train()
        for epoch in range(cfg._epochs):
            self.state.epoch = epoch
            for cb in self.callbacks:
                cb.on_epoch_begin(epoch, self.state)
            run, cnt = 0.0, 0
            self.optimizer.zero_grad()
            for i, b in enumerate(train_loader):
                x, y = self._to(b.data), self._to(b.targets)
                if cfg._amp:
                    from .autograd import autocast
                    with autocast():
                        loss = self.loss_fn(self.model(x), y) / cfg._accum
                    self.scaler.scale(loss).backward()
                else:
                    loss = self.loss_fn(self.model(x), y) / cfg._accum
                    loss.backward()
                if (i + 1) % cfg._accum == 0:
                    if cfg._clip is not None:
                        if self.scaler is not None:
                            self.scaler.unscale_(self.optimizer)
                        clip_grad_norm(self.optimizer.parameters(), cfg._clip)
                    if self.scaler is not None:
                        self.scaler.step(self.optimizer)
                        self.scaler.update()
                    else:
                        self.optimizer.step()
                    self.optimizer.zero_grad()
                    self.state.global_step += 1
                lv = float(loss.detach()) * cfg._accum
                run, cnt = run + lv, cnt + 1
                self.state.train_losses.append(lv)
                m = TrainingMetrics(lv)
                for cb in self.callbacks:
                    cb.on_batch_end(self.state.global_step, m, self.state)
            metrics = TrainingMetrics(run / max(cnt, 1))
            self.history.train_loss.append(metrics.loss)
            self.history.lr.append(self.optimizer.get_lr())
            if val_loader is not None:
                vm = self.evaluate(val_loader)
                metrics.with_metric("val_loss", vm.loss)
                self.history.val_loss.append(vm.loss)
                self.history.val_acc.append(vm.accuracy)
                self.state.val_losses.append(vm.loss)
            if self.scheduler is not None:
                self.scheduler.step(self.optimizer)
            keep = all([cb.on_epoch_end(epoch, metrics, self.state) is not False for cb in self.callbacks])
            if not keep:
                self.state.should_stop = True
                break
        for cb in self.callbacks:
            cb.on_train_end(self.state)
        return self.history
