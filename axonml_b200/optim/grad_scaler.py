"""GradScaler (crates/axonml-optim/src/grad_scaler.rs:46-277): initial scale 65536, x2 after
``growth_interval`` (2000) clean steps, x0.5 on overflow, clamped to [1, f32::MAX/2].

Two usage shapes are supported: the reference's slice API (``scale_loss(float)``,
``unscale_grads(list/tensor) -> bool``, ``update()``) and the optimizer-driven loop
``scaler.scale(loss).backward(); scaler.step(optimizer); scaler.update()``.  On CUDA the scale
and the found-inf flag live in device memory and the optimizer kernels read them, so a training
step has no host synchronisation."""
from __future__ import annotations

import dataclasses

import torch

from ..ops import optim as O

_F32_MAX_HALF = 3.4028234663852886e38 / 2


@dataclasses.dataclass
class GradScalerState:
    scale: float
    growth_tracker: int


class GradScaler:
    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0,
                 backoff_factor: float = 0.5, growth_interval: int = 2000, enabled: bool = True):
        self._scale = float(init_scale)
        self._growth_factor, self._backoff_factor = growth_factor, backoff_factor
        self._growth_interval = growth_interval
        self._enabled = enabled
        self._growth_tracker = 0
        self._found_inf = False
        # device-resident mirrors (created lazily per device)
        self._dev = None
        self._scale_t = None
        self._inv_scale_t = None
        self._found_inf_t = None
        self._pending_device_update = False

    @classmethod
    def new(cls): return cls()

    @classmethod
    def with_scale(cls, init_scale: float): return cls(init_scale)

    @classmethod
    def with_options(cls, init_scale, growth_factor, backoff_factor, growth_interval):
        return cls(init_scale, growth_factor, backoff_factor, growth_interval)

    def growth_factor(self, f): self._growth_factor = f; return self
    def backoff_factor(self, f): self._backoff_factor = f; return self
    def growth_interval(self, n): self._growth_interval = n; return self
    def enabled(self, flag): self._enabled = flag; return self

    # ---- reference accessors
    def get_scale(self) -> float:
        self._sync_from_device()
        return self._scale

    def set_scale(self, s: float) -> None:
        self._scale = float(s)
        self._push_to_device()

    def is_enabled(self) -> bool: return self._enabled
    def set_enabled(self, flag: bool) -> None: self._enabled = flag

    def found_inf(self) -> bool:
        if self._pending_device_update:
            return bool(self._found_inf_t.item())
        return self._found_inf

    def set_found_inf(self, flag: bool) -> None: self._found_inf = bool(flag)

    def scale_loss(self, loss):
        """Multiplies a float or a tensor loss by the current scale."""
        if not self._enabled:
            return loss
        if torch.is_tensor(loss) and loss.is_cuda:
            self._ensure_device(loss.device)
            return loss * self._scale_t.to(loss.dtype)[0]
        return loss * self._scale

    scale = scale_loss

    def unscale_grads(self, grads) -> bool:
        """In-place ``g /= scale`` on a tensor or list of tensors (or a list of floats); returns
        True when every value is finite and records found_inf otherwise."""
        if not self._enabled:
            return True
        inv = 1.0 / self._scale
        if isinstance(grads, (list, tuple)) and grads and not torch.is_tensor(grads[0]):
            ok = True
            for i, g in enumerate(grads):
                grads[i] = g * inv
                if grads[i] != grads[i] or abs(grads[i]) == float("inf"):
                    ok = False
            self._found_inf = not ok
            return ok
        ts = [grads] if torch.is_tensor(grads) else list(grads)
        ok = True
        for g in ts:
            g.mul_(inv)
            if not bool(torch.isfinite(g).all()):
                ok = False
        self._found_inf = not ok
        return ok

    def check_grads(self, grads) -> bool:
        ts = [grads] if torch.is_tensor(grads) else list(grads)
        ok = all(bool(torch.isfinite(torch.as_tensor(g)).all()) for g in ts)
        self._found_inf = not ok
        return ok

    # ---- optimizer-driven loop
    def unscale_(self, optimizer) -> None:
        """Unscales ``optimizer``'s gradients in place and records overflow on the device."""
        if not self._enabled:
            return
        grads = [p.grad for p in optimizer.parameters() if p.grad is not None]
        if not grads:
            return
        if grads[0].is_cuda:
            self._ensure_device(grads[0].device)
            by = {}
            for g in grads:
                by.setdefault(g.dtype, []).append(g)
            for gl in by.values():
                if O.supported(gl, gl):
                    O.multi_tensor("unscale_check", None, gl, inv_scale=self._inv_scale_t,
                                   norms=self._found_inf_t)
                else:
                    for g in gl:
                        g.mul_(self._inv_scale_t.to(g.dtype)[0])
                        self._found_inf_t.logical_or_(~torch.isfinite(g).all())
            self._unscaled = True
        else:
            self.unscale_grads(grads)
            self._unscaled = True

    def step(self, optimizer) -> None:
        """Runs ``optimizer.step()`` unless the gradients overflowed.  If ``unscale_`` was not
        called, unscaling and the overflow check are fused into the optimizer kernels."""
        if not self._enabled:
            optimizer.step()
            return
        grads = [p.grad for p in optimizer.parameters() if p.grad is not None]
        on_cuda = bool(grads) and grads[0].is_cuda
        if on_cuda:
            self._ensure_device(grads[0].device)
            if not getattr(self, "_unscaled", False):
                self.unscale_(optimizer)
            optimizer._inv_scale = None
            optimizer._found_inf = self._found_inf_t
            try:
                optimizer.step()
            finally:
                optimizer._found_inf = None
            self._pending_device_update = True
        else:
            if not getattr(self, "_unscaled", False):
                self.unscale_grads(grads)
            if not self._found_inf:
                optimizer.step()
        self._unscaled = False

    def update(self) -> None:
        """Adjusts the scale after a step (grad_scaler.rs:230-252)."""
        if not self._enabled:
            return
        if self._pending_device_update:
            # device-side update: no host sync
            f = self._found_inf_t
            grow = (self._growth_tracker_t + 1 >= self._growth_interval) & (f == 0)
            new_scale = torch.where(f != 0, self._scale_t * self._backoff_factor,
                                    torch.where(grow, self._scale_t * self._growth_factor, self._scale_t))
            self._scale_t.copy_(new_scale.clamp(1.0, _F32_MAX_HALF))
            self._growth_tracker_t.copy_(torch.where((f != 0) | grow, torch.zeros_like(self._growth_tracker_t),
                                                     self._growth_tracker_t + 1))
            self._inv_scale_t.copy_(1.0 / self._scale_t)
            self._found_inf_t.zero_()
            self._pending_device_update = False
            self._device_is_truth = True
            return
        if self._found_inf:
            self._scale = max(self._scale * self._backoff_factor, 1.0)
            self._growth_tracker = 0
        else:
            self._growth_tracker += 1
            if self._growth_tracker >= self._growth_interval:
                self._scale = min(self._scale * self._growth_factor, _F32_MAX_HALF)
                self._growth_tracker = 0
        self._found_inf = False
        self._push_to_device()

    def state_dict(self) -> GradScalerState:
        self._sync_from_device()
        return GradScalerState(self._scale, self._growth_tracker)

    def load_state_dict(self, state) -> None:
        if isinstance(state, dict):
            state = GradScalerState(state["scale"], state["growth_tracker"])
        self._scale, self._growth_tracker = float(state.scale), int(state.growth_tracker)
        self._push_to_device()

    # ---- device mirrors
    def _ensure_device(self, dev) -> None:
        if self._dev == dev:
            return
        self._dev = dev
        self._scale_t = torch.full((1,), self._scale, dtype=torch.float32, device=dev)
        self._inv_scale_t = torch.full((1,), 1.0 / self._scale, dtype=torch.float32, device=dev)
        self._found_inf_t = torch.zeros(1, dtype=torch.int32, device=dev)
        self._growth_tracker_t = torch.full((1,), self._growth_tracker, dtype=torch.int32, device=dev)
        self._device_is_truth = False

    def _push_to_device(self) -> None:
        if self._dev is not None:
            self._scale_t.fill_(self._scale)
            self._inv_scale_t.fill_(1.0 / self._scale)
            self._growth_tracker_t.fill_(self._growth_tracker)
            self._device_is_truth = False

    def _sync_from_device(self) -> None:
        if self._dev is not None and getattr(self, "_device_is_truth", False):
            self._scale = float(self._scale_t.item())
            self._growth_tracker = int(self._growth_tracker_t.item())
            self._device_is_truth = False
            if self._pending_device_update:
                self._found_inf = bool(self._found_inf_t.item())
