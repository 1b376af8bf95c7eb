"""Catalogue of well-known datasets for ``axonml dataset list/info/search`` and the server's
built-in dataset route (crates/axonml-cli/src/commands/dataset.rs:38-118: MNIST, Fashion-MNIST,
CIFAR-10/100, Iris, Wine Quality, Breast Cancer; sources builtin / kaggle / uci / data.gov).
``loader`` names the class of this package that reads the files once they are on disk;
``synthetic`` names the generator that stands in for them when they are not."""
from __future__ import annotations

BUILTIN_DATASETS = [
    {"id": "mnist", "name": "MNIST Handwritten Digits", "type": "image", "task": "classification", "samples": 70000,
     "classes": 10, "shape": [1, 28, 28], "size_mb": 11.6, "source": "builtin", "loader": "vision.datasets.MNIST",
     "synthetic": "vision.datasets.SyntheticMNIST", "files": ["train-images-idx3-ubyte", "train-labels-idx1-ubyte",
                                                              "t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte"]},
    {"id": "fashion-mnist", "name": "Fashion MNIST", "type": "image", "task": "classification", "samples": 70000,
     "classes": 10, "shape": [1, 28, 28], "size_mb": 30.9, "source": "builtin", "loader": "vision.datasets.FashionMNIST",
     "synthetic": "vision.datasets.SyntheticMNIST", "files": ["train-images-idx3-ubyte", "train-labels-idx1-ubyte"]},
    {"id": "cifar-10", "name": "CIFAR-10", "type": "image", "task": "classification", "samples": 60000, "classes": 10,
     "shape": [3, 32, 32], "size_mb": 170.0, "source": "builtin", "loader": "vision.datasets.CIFAR10",
     "synthetic": "vision.datasets.SyntheticCIFAR", "files": ["data_batch_1.bin", "test_batch.bin"]},
    {"id": "cifar-100", "name": "CIFAR-100", "type": "image", "task": "classification", "samples": 60000, "classes": 100,
     "shape": [3, 32, 32], "size_mb": 169.0, "source": "builtin", "loader": "vision.datasets.CIFAR100",
     "synthetic": "vision.datasets.SyntheticCIFAR", "files": ["train.bin", "test.bin"]},
    {"id": "iris", "name": "Iris Flower Dataset", "type": "tabular", "task": "classification", "samples": 150, "classes": 3,
     "shape": [4], "size_mb": 0.005, "source": "uci", "loader": "data.datasets.CSVDataset", "synthetic": None,
     "files": ["iris.csv"]},
    {"id": "wine-quality", "name": "Wine Quality Dataset", "type": "tabular", "task": "regression", "samples": 6497,
     "classes": None, "shape": [11], "size_mb": 0.4, "source": "uci", "loader": "data.datasets.CSVDataset",
     "synthetic": None, "files": ["winequality-red.csv", "winequality-white.csv"]},
    {"id": "breast-cancer", "name": "Breast Cancer Wisconsin", "type": "tabular", "task": "classification", "samples": 569,
     "classes": 2, "shape": [30], "size_mb": 0.12, "source": "uci", "loader": "data.datasets.CSVDataset", "synthetic": None,
     "files": ["wdbc.csv"]},
]

SOURCES = [
    {"id": "builtin", "name": "Built-in", "description": "datasets this package reads from their original file formats"},
    {"id": "kaggle", "name": "Kaggle", "description": "community datasets (needs credentials and network: axonml kaggle login)"},
    {"id": "uci", "name": "UCI ML Repository", "description": "classic tabular datasets"},
    {"id": "data.gov", "name": "data.gov", "description": "US government open data"},
]


def list_datasets(source: str | None = None) -> list[dict]:
    return [d for d in BUILTIN_DATASETS if source in (None, "all", d["source"])]


def get_dataset_info(dataset_id: str) -> dict | None:
    key = dataset_id.lower().replace("_", "-")
    aliases = {"cifar10": "cifar-10", "cifar100": "cifar-100", "fashionmnist": "fashion-mnist"}
    key = aliases.get(key, key)
    return next((d for d in BUILTIN_DATASETS if d["id"] == key), None)


def search_datasets(query: str, source: str | None = None, limit: int = 10) -> list[dict]:
    q = query.lower()
    hits = [d for d in list_datasets(source) if q in d["id"] or q in d["name"].lower() or q in d["type"] or q in (d["task"] or "")]
    return hits[:limit]
