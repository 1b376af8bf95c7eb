"""axonml_b200: a Blackwell-native deep-learning framework with AxonML's API surface.

Sub-packages are imported on first attribute access (``axonml_b200.nn`` etc.), so importing the
package is cheap and does not load the CUDA library.  ``prelude()`` returns the names the
reference's ``axonml::prelude`` re-exports (crates/axonml/src/lib.rs)."""
import importlib

__version__ = "0.1.0"

_SUBPACKAGES = ("core", "tensor", "autograd", "nn", "optim", "data", "vision", "text", "audio", "llm", "parallel",
                "serialize", "quant", "fusion", "jit", "profile", "onnx", "hub", "server", "cli", "tui", "trainer", "benchmark",
                "ops", "integrations", "utils")
_ALIASES = {"distributed": "parallel"}           # the reference's crate name

# names the reference's umbrella crate re-exports at its root (crates/axonml/src/lib.rs:235-273)
_ROOT_NAMES = {
    "trainer": ("Trainer", "Callback", "EarlyStopping", "ProgressLogger", "TrainingConfig", "TrainingHistory", "TrainingMetrics",
                "TrainingState", "clip_grad_norm", "compute_accuracy"),
    "hub": ("ModelCategory", "UnifiedModelInfo", "compare_benchmarks", "list_all_models", "models_by_category",
            "models_by_max_params", "models_by_max_size_mb", "recommended_models", "search_models"),
    "benchmark": ("BenchmarkResult", "MemorySnapshot", "ThroughputConfig", "ThroughputResult", "benchmark_model",
                  "benchmark_model_named", "compare_models", "throughput_test", "warmup_model", "print_throughput_results",
                  "print_memory_profile", "profile_model_memory"),
}
_ROOT_LOOKUP = {n: mod for mod, names in _ROOT_NAMES.items() for n in names}


def __getattr__(name):
    target = _ALIASES.get(name, name)
    if target in _SUBPACKAGES:
        mod = importlib.import_module(f"{__name__}.{target}")
        globals()[name] = mod
        return mod
    if name in _ROOT_LOOKUP:
        value = getattr(importlib.import_module(f"{__name__}.{_ROOT_LOOKUP[name]}"), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(set(globals()) | set(_SUBPACKAGES) | set(_ALIASES) | set(_ROOT_LOOKUP))


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
    """The names of the reference's ``axonml::prelude`` (crates/axonml/src/lib.rs:287-366), plus
    the trainer helpers: ``globals().update(axonml_b200.prelude())`` is ``use axonml::prelude::*``."""
    from . import audio, autograd, core, data, jit, llm, nn, optim, parallel, profile, tensor, text, trainer, vision
    groups = (
        (core, ("DType", "Device", "Error")),
        (tensor, ("Tensor", "zeros", "ones", "rand", "randn", "arange", "linspace", "eye", "full")),
        (autograd, ("Variable", "no_grad", "backward")),
        (nn, ("AvgPool2d", "BCELoss", "BatchNorm1d", "BatchNorm2d", "Conv2d", "CrossEntropyLoss", "Dropout", "Embedding", "L1Loss",
              "LayerNorm", "LeakyReLU", "Linear", "MSELoss", "MaxPool2d", "Module", "MultiHeadAttention", "Parameter", "ReLU",
              "Sequential", "SiLU", "Sigmoid", "Softmax", "Tanh", "GELU", "GRU", "LSTM", "RNN")),
        (optim, ("Adam", "AdamW", "CosineAnnealingLR", "ExponentialLR", "LRScheduler", "Optimizer", "RMSprop", "StepLR", "SGD", "LAMB",
                 "GradScaler", "OneCycleLR")),
        (data, ("DataLoader", "Dataset", "RandomSampler", "SequentialSampler", "Transform", "TensorDataset", "random_split")),
        (vision, ("CenterCrop", "ImageNormalize", "LeNet", "RandomHorizontalFlip", "Resize", "SimpleCNN", "SyntheticCIFAR", "SyntheticMNIST")),
        (text, ("BasicBPETokenizer", "CharTokenizer", "LanguageModelDataset", "SyntheticSentimentDataset", "TextDataset", "Tokenizer",
                "Vocab", "WhitespaceTokenizer")),
        (audio, ("AddNoise", "MelSpectrogram", "NormalizeAudio", "Resample", "SyntheticCommandDataset", "SyntheticMusicDataset", "MFCC")),
        (parallel, ("all_reduce_mean", "all_reduce_sum", "barrier", "broadcast", "DistributedDataParallel", "ProcessGroup", "World", "DDP")),
        (profile, ("Bottleneck", "BottleneckAnalyzer", "ComputeProfiler", "MemoryProfiler", "ProfileGuard", "ProfileReport", "Profiler",
                   "TimelineProfiler")),
        (llm, ("Bert", "BertConfig", "BertForMaskedLM", "BertForSequenceClassification", "GPT2Config", "GPT2LMHead", "GenerationConfig",
               "TextGenerator", "GPT2")),
        (jit, ("trace", "CompiledFunction", "Graph", "JitCompiler", "TracedValue")),
        (trainer, ("Trainer", "TrainingConfig", "TrainingState", "TrainingMetrics", "EarlyStopping", "ProgressLogger", "clip_grad_norm",
                   "compute_accuracy")),
    )
    out = {}
    for mod, names in groups:
        for n in names:
            if hasattr(mod, n):
                out[n] = getattr(mod, n)
    out["JitOptimizer"] = jit.Optimizer if hasattr(jit, "Optimizer") else None
    if out["JitOptimizer"] is None:
        del out["JitOptimizer"]
    return out
