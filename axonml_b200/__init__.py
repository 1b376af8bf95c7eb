"""axonml_b200: a Blackwell-native deep-learning framework with AxonML's API surface.

Sub-packages are imported on first attribute access (``axonml_b200.nn`` etc.), so importing the
package is cheap and does not load the CUDA library.  ``prelude()`` returns the names the
reference's ``axonml::prelude`` re-exports (crates/axonml/src/lib.rs)."""
import importlib

__version__ = "0.1.0"

_SUBPACKAGES = ("core", "tensor", "autograd", "nn", "optim", "data", "vision", "text", "audio", "llm", "parallel",
                "serialize", "quant", "fusion", "jit", "profile", "onnx", "hub", "server", "cli", "trainer", "benchmark",
                "ops", "integrations", "utils")
_ALIASES = {"distributed": "parallel"}           # the reference's crate name


def __getattr__(name):
    target = _ALIASES.get(name, name)
    if target in _SUBPACKAGES:
        mod = importlib.import_module(f"{__name__}.{target}")
        globals()[name] = mod
        return mod
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def version() -> str:
    return __version__


def features() -> str:
    """Comma-separated list of what this installation can use (the reference prints its cargo
    features, crates/axonml/src/lib.rs)."""
    import torch
    f = ["core", "nn", "optim", "data", "vision", "text", "audio", "llm", "distributed", "serialize", "onnx", "quant",
         "fusion", "jit", "profile", "server", "cli"]
    if torch.cuda.is_available():
        f.append("cuda")
        from . import _native
        if _native.is_blackwell():
            f.append("sm_100a-kernels")
    return ", ".join(f)


def prelude() -> dict:
    """Names of the reference's prelude: tensor constructors, Variable, layers, losses,
    optimizers, data loading and the trainer helpers."""
    from . import autograd, data, nn, optim, tensor, trainer
    out = {}
    for mod, names in ((tensor, ("Tensor", "zeros", "ones", "rand", "randn", "arange", "linspace", "eye", "full")),
                       (autograd, ("Variable", "no_grad", "backward")),
                       (nn, ("Module", "Parameter", "Sequential", "Linear", "Conv2d", "BatchNorm2d", "LayerNorm", "Dropout",
                             "ReLU", "Sigmoid", "Tanh", "GELU", "Softmax", "Embedding", "LSTM", "GRU", "MultiHeadAttention",
                             "CrossEntropyLoss", "MSELoss", "BCELoss", "L1Loss")),
                       (optim, ("Optimizer", "SGD", "Adam", "AdamW", "RMSprop", "LAMB", "GradScaler", "StepLR",
                                "CosineAnnealingLR", "OneCycleLR")),
                       (data, ("Dataset", "DataLoader", "TensorDataset", "random_split")),
                       (trainer, ("Trainer", "TrainingConfig", "TrainingState", "TrainingMetrics", "EarlyStopping",
                                  "ProgressLogger", "clip_grad_norm", "compute_accuracy"))):
        for n in names:
            if hasattr(mod, n):
                out[n] = getattr(mod, n)
    return out
