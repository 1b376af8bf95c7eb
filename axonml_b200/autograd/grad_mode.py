"""Thread-local gradient modes (crates/axonml-autograd/src/no_grad.rs:133-220)."""
import torch

no_grad = torch.no_grad
enable_grad = torch.enable_grad
inference_mode = torch.inference_mode
set_grad_enabled_context = torch.set_grad_enabled
is_grad_enabled = torch.is_grad_enabled
is_inference_mode = torch.is_inference_mode_enabled


class NoGradGuard:
    """Gradient recording is off from construction until ``drop()`` (or the end of a ``with``
    block); the previous mode comes back afterwards (no_grad.rs: ``NoGradGuard::new`` + Drop)."""

    def __init__(self):
        self._prev = torch.is_grad_enabled()
        self._live = True
        torch.set_grad_enabled(False)

    @classmethod
    def new(cls): return cls()

    def drop(self) -> None:
        if self._live:
            torch.set_grad_enabled(self._prev)
            self._live = False

    def __enter__(self): return self
    def __exit__(self, *exc): self.drop()
    def __del__(self): self.drop()


class EnableGradGuard(NoGradGuard):
    """Gradient recording is on until ``drop()``, inside a region where it was off (no_grad.rs:93-125)."""

    def __init__(self):
        self._prev = torch.is_grad_enabled()
        self._live = True
        torch.set_grad_enabled(True)


class InferenceModeGuard:
    """Inference mode (no recording, no version counters) until ``drop()`` (no_grad.rs:186-220)."""

    def __init__(self):
        self._cm = torch.inference_mode()
        self._cm.__enter__()
        self._live = True

    @classmethod
    def new(cls): return cls()

    def drop(self) -> None:
        if self._live:
            self._live = False
            self._cm.__exit__(None, None, None)

    def __enter__(self): return self
    def __exit__(self, *exc): self.drop()
