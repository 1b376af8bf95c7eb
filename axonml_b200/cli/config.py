"""Project file ``axonml.toml`` (crates/axonml-cli/src/config.rs:19-340): ``ProjectConfig`` with the
``project``, ``training``, ``model`` and ``data`` tables of the reference, plus ``[distributed]``
and ``[precision]`` for the multi-GPU paths.  Precedence used by the commands: command-line flag >
``--config`` file > ``./axonml.toml`` > defaults (train.rs:101-157)."""
from __future__ import annotations

import dataclasses
import os
import tomllib
from dataclasses import dataclass, field


@dataclass
class OptimizerConfig:
    name: str = "adam"
    weight_decay: float = 0.0
    momentum: float = 0.9
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    nesterov: bool = False


@dataclass
class SchedulerConfig:
    name: str = "none"
    step_size: int = 10
    gamma: float = 0.1
    milestones: list = field(default_factory=list)
    t_max: int = 100
    eta_min: float = 0.0
    warmup_epochs: int = 0


@dataclass
class TrainingSection:
    epochs: int = 10
    batch_size: int = 32
    learning_rate: float = 1e-3
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    device: str = "auto"
    seed: int = 42
    checkpoint_frequency: int = 1
    output_dir: str = "./output"
    num_workers: int = 0
    gradient_clip: float = 0.0
    mixed_precision: bool = False


@dataclass
class ModelSection:
    architecture: str = "mlp"
    path: str = ""
    input_size: list = field(default_factory=lambda: [784])
    num_classes: int = 10
    hidden_sizes: list = field(default_factory=lambda: [256, 128])
    dropout: float = 0.0
    pretrained: bool = False


@dataclass
class DataSection:
    train_path: str = ""
    val_path: str = ""
    test_path: str = ""
    format: str = "synthetic-mnist"
    val_split: float = 0.1
    augmentation: bool = False
    shuffle: bool = True
    normalize: bool = True
    mean: list = field(default_factory=lambda: [0.1307])
    std: list = field(default_factory=lambda: [0.3081])


@dataclass
class DistributedSection:
    dp: int = 1
    tp: int = 1
    pp: int = 1
    fsdp: str = "none"            # none | full_shard | shard_grad_op | no_shard | hybrid_shard
    bucket_mb: int = 25
    microbatches: int = 1
    timeout_s: float = 300.0


@dataclass
class PrecisionSection:
    dtype: str = "fp32"           # fp32 | bf16
    loss_scale: float = 65536.0


@dataclass
class ProjectSection:
    name: str = "axonml-project"
    version: str = "0.1.0"
    description: str = ""
    author: str = ""


@dataclass
class ProjectConfig:
    project: ProjectSection = field(default_factory=ProjectSection)
    training: TrainingSection = field(default_factory=TrainingSection)
    model: ModelSection = field(default_factory=ModelSection)
    data: DataSection = field(default_factory=DataSection)
    distributed: DistributedSection = field(default_factory=DistributedSection)
    precision: PrecisionSection = field(default_factory=PrecisionSection)

    # ------------------------------------------------------------------ load / save
    @classmethod
    def from_dict(cls, d: dict) -> "ProjectConfig":
        def build(tp, src):
            kw = {}
            for f in dataclasses.fields(tp):
                if f.name not in src:
                    continue
                v = src[f.name]
                sub = f.default_factory if f.default_factory is not dataclasses.MISSING else None
                if isinstance(v, dict) and sub is not None and dataclasses.is_dataclass(sub):
                    kw[f.name] = build(sub, v)
                else:
                    kw[f.name] = v
            return tp(**kw)
        return build(cls, d)

    @classmethod
    def load(cls, path: str) -> "ProjectConfig":
        with open(path, "rb") as f:
            return cls.from_dict(tomllib.load(f))

    @classmethod
    def resolve(cls, explicit: str | None = None) -> "ProjectConfig":
        """``--config`` file, else ``./axonml.toml``, else defaults."""
        if explicit:
            return cls.load(explicit)
        if os.path.exists("axonml.toml"):
            return cls.load("axonml.toml")
        return cls()

    def to_toml(self) -> str:
        def emit(v):
            if isinstance(v, bool):
                return "true" if v else "false"
            if isinstance(v, (int, float)):
                return repr(v)
            if isinstance(v, str):
                return '"' + v.replace("\\", "\\\\").replace('"', '\\"') + '"'
            if isinstance(v, (list, tuple)):
                return "[" + ", ".join(emit(x) for x in v) + "]"
            raise TypeError(type(v))

        lines = []

        def table(name, obj):
            lines.append(f"[{name}]")
            subs = []
            for f in dataclasses.fields(obj):
                v = getattr(obj, f.name)
                if dataclasses.is_dataclass(v):
                    subs.append((f"{name}.{f.name}", v))
                else:
                    lines.append(f"{f.name} = {emit(v)}")
            lines.append("")
            for n, o in subs:
                table(n, o)

        for f in dataclasses.fields(self):
            table(f.name, getattr(self, f.name))
        return "\n".join(lines)

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.to_toml())

    def validate(self) -> list:
        """Returns a list of problems (empty when the file is usable)."""
        errs = []
        t = self.training
        if t.epochs <= 0: errs.append("training.epochs must be positive")
        if t.batch_size <= 0: errs.append("training.batch_size must be positive")
        if t.learning_rate <= 0: errs.append("training.learning_rate must be positive")
        if t.optimizer.name.lower() not in ("sgd", "adam", "adamw", "rmsprop", "lamb"):
            errs.append(f"unknown optimizer {t.optimizer.name!r}")
        if self.model.architecture.lower() not in ("mlp", "simplecnn", "cnn", "lenet", "resnet18", "resnet34"):
            errs.append(f"unknown architecture {self.model.architecture!r}")
        if not 0.0 <= self.data.val_split < 1.0: errs.append("data.val_split must be in [0, 1)")
        d = self.distributed
        if min(d.dp, d.tp, d.pp) < 1: errs.append("distributed sizes must be >= 1")
        if self.precision.dtype not in ("fp32", "bf16"): errs.append("precision.dtype must be fp32 or bf16")
        return errs
