"""Training checkpoints (crates/axonml-serialize/src/checkpoint.rs:16-272): ``TrainingState``,
``Checkpoint`` and ``CheckpointBuilder``; bincode layout in field order ``model_state,
optimizer_state, training_state, rng_state, config, axonml_version, timestamp``.  Unlike the
reference, optimizers expose their state, so ``optimizer_state`` is populated (Adam moments, step
counters, GradScaler scale are stored as tensors in the optimizer StateDict)."""
from __future__ import annotations

import dataclasses
import struct
import time

import torch

from .state_dict import StateDict, TensorData


@dataclasses.dataclass
class TrainingState:
    epoch: int = 0
    step: int = 0
    global_step: int = 0
    best_metric: float | None = None
    best_metric_name: str | None = None
    loss_history: list = dataclasses.field(default_factory=list)
    val_loss_history: list = dataclasses.field(default_factory=list)
    lr_history: list = dataclasses.field(default_factory=list)
    custom_metrics: dict = dataclasses.field(default_factory=dict)

    @classmethod
    def new(cls): return cls()

    def record_loss(self, loss: float) -> None:
        self.loss_history.append(float(loss))
        if len(self.loss_history) > 1000:          # checkpoint.rs:45-51
            self.loss_history.pop(0)

    def record_val_loss(self, loss: float) -> None: self.val_loss_history.append(float(loss))
    def record_lr(self, lr: float) -> None: self.lr_history.append(float(lr))
    def record_metric(self, name: str, value: float) -> None:
        self.custom_metrics.setdefault(name, []).append(float(value))

    def update_best(self, name: str, value: float, higher_is_better: bool) -> bool:
        better = (self.best_metric is None or
                  (value > self.best_metric if higher_is_better else value < self.best_metric))
        if better:
            self.best_metric, self.best_metric_name = float(value), name
        return better

    def avg_loss(self, n: int):
        if not self.loss_history:
            return None
        tail = self.loss_history[-n:]
        return sum(tail) / len(tail)

    def next_epoch(self) -> None:
        self.epoch += 1
        self.step = 0

    def next_step(self) -> None:
        self.step += 1
        self.global_step += 1


@dataclasses.dataclass
class Checkpoint:
    model_state: StateDict
    optimizer_state: StateDict
    training_state: TrainingState
    rng_state: bytes | None = None
    config: dict = dataclasses.field(default_factory=dict)
    axonml_version: str = "0.2.8"
    timestamp: str = ""

    @staticmethod
    def builder() -> "CheckpointBuilder": return CheckpointBuilder()
    def epoch(self) -> int: return self.training_state.epoch
    def global_step(self) -> int: return self.training_state.global_step
    def best_metric(self): return self.training_state.best_metric


class CheckpointBuilder:
    def __init__(self):
        self._model, self._opt = StateDict(), StateDict()
        self._ts, self._rng, self._cfg = TrainingState(), None, {}

    @classmethod
    def new(cls): return cls()
    def model_state(self, sd: StateDict): self._model = sd; return self
    def optimizer_state(self, sd: StateDict): self._opt = sd; return self
    def training_state(self, ts: TrainingState): self._ts = ts; return self
    def rng_state(self, b: bytes): self._rng = bytes(b); return self
    def config(self, key: str, value: str): self._cfg[key] = str(value); return self
    def epoch(self, e: int): self._ts.epoch = e; return self
    def global_step(self, s: int): self._ts.global_step = s; return self

    def build(self) -> Checkpoint:
        return Checkpoint(self._model, self._opt, self._ts, self._rng, dict(self._cfg), "0.2.8",
                          str(int(time.time())))


# ------------------------------------------------------------------ optimizer <-> StateDict
def optimizer_to_state_dict(optimizer) -> StateDict:
    sd = StateDict()
    st = optimizer.state_dict()
    sd.set_metadata("lr", repr(st["lr"]))
    sd.set_metadata("step", str(st["step"]))
    for k, v in st.get("hyper", {}).items():
        sd.set_metadata("hyper." + k, repr(v))
    for i, tensors in st["state"].items():
        for name, t in tensors.items():
            if torch.is_tensor(t):
                sd.insert(f"{i}.{name}", TensorData.from_tensor(t))
            else:
                sd.set_metadata(f"flag.{i}.{name}", repr(t))
    return sd


def optimizer_from_state_dict(optimizer, sd: StateDict) -> None:
    import ast
    state: dict = {}
    for k, e in sd.entries():
        i, name = k.split(".", 1)
        state.setdefault(int(i), {})[name] = e.data.to_tensor().clone()
    hyper = {}
    for k, v in sd.metadata.items():
        if k.startswith("hyper."):
            hyper[k[6:]] = ast.literal_eval(v)
        elif k.startswith("flag."):
            _, i, name = k.split(".", 2)
            state.setdefault(int(i), {})[name] = ast.literal_eval(v)
    optimizer.load_state_dict({"lr": float(sd.metadata.get("lr", optimizer.get_lr())),
                               "step": int(sd.metadata.get("step", 0)), "state": state, "hyper": hyper})


# ------------------------------------------------------------------ bincode of Checkpoint
def encode_checkpoint(ck: Checkpoint) -> bytes:
    import ctypes
    from . import codec
    lib = codec._lib()
    w = lib.ax_bc_writer_new()
    W = ctypes.c_void_p(w)
    u64 = ctypes.c_uint64

    def wstr(s):
        b = s.encode()
        lib.ax_bc_write_str(W, b, u64(len(b)))

    def wvec(v):
        lib.ax_bc_write_u64(W, u64(len(v)))
        for x in v:
            lib.ax_bc_write_f32(W, ctypes.c_float(x))
    try:
        codec._write_state_dict(lib, w, ck.model_state)
        codec._write_state_dict(lib, w, ck.optimizer_state)
        ts = ck.training_state
        for v in (ts.epoch, ts.step, ts.global_step):
            lib.ax_bc_write_u64(W, u64(v))
        if ts.best_metric is None:
            lib.ax_bc_write_u8(W, ctypes.c_uint8(0))
        else:
            lib.ax_bc_write_u8(W, ctypes.c_uint8(1))
            lib.ax_bc_write_f32(W, ctypes.c_float(ts.best_metric))
        if ts.best_metric_name is None:
            lib.ax_bc_write_u8(W, ctypes.c_uint8(0))
        else:
            lib.ax_bc_write_u8(W, ctypes.c_uint8(1))
            wstr(ts.best_metric_name)
        wvec(ts.loss_history); wvec(ts.val_loss_history); wvec(ts.lr_history)
        lib.ax_bc_write_u64(W, u64(len(ts.custom_metrics)))
        for k, v in ts.custom_metrics.items():
            wstr(k); wvec(v)
        if ck.rng_state is None:
            lib.ax_bc_write_u8(W, ctypes.c_uint8(0))
        else:
            lib.ax_bc_write_u8(W, ctypes.c_uint8(1))
            lib.ax_bc_write_u64(W, u64(len(ck.rng_state)))
            lib.ax_bc_write_raw(W, ck.rng_state, u64(len(ck.rng_state)))
        codec._write_map(lib, w, ck.config)
        wstr(ck.axonml_version); wstr(ck.timestamp)
        return codec._writer_bytes(lib, w)
    finally:
        lib.ax_bc_writer_free(W)


def decode_checkpoint(data: bytes) -> Checkpoint:
    from . import codec
    model, pos = codec.decode_state_dict(data, 0)
    opt, pos = codec.decode_state_dict(data, pos)
    buf = memoryview(data)

    def u64():
        nonlocal pos
        v = struct.unpack_from("<Q", buf, pos)[0]; pos += 8
        return v

    def u8():
        nonlocal pos
        v = buf[pos]; pos += 1
        return v

    def f32():
        nonlocal pos
        v = struct.unpack_from("<f", buf, pos)[0]; pos += 4
        return v

    def rstr():
        nonlocal pos
        s, pos = codec._read_str(buf, pos)
        return s

    def vec():
        n = u64()
        return [f32() for _ in range(n)]
    ts = TrainingState(u64(), u64(), u64())
    ts.best_metric = f32() if u8() else None
    ts.best_metric_name = rstr() if u8() else None
    ts.loss_history, ts.val_loss_history, ts.lr_history = vec(), vec(), vec()
    for _ in range(u64()):
        k = rstr()
        ts.custom_metrics[k] = vec()
    rng = None
    if u8():
        n = u64()
        rng = bytes(buf[pos:pos + n]); pos += n
    cfg, pos = codec._read_map(buf, pos + 8, struct.unpack_from("<Q", buf, pos)[0])
    version = rstr()
    stamp = rstr()
    return Checkpoint(model, opt, ts, rng, cfg, version, stamp)
