"""Vision datasets (crates/axonml-vision/src/datasets): MNIST / FashionMNIST from IDX files,
CIFAR-10/100 from the binary batches, and deterministic synthetic stand-ins.  Targets are class
indices (the reference returns one-hot rows that its own CrossEntropyLoss cannot consume)."""
from __future__ import annotations

import gzip
import os
import struct

import numpy as np
import torch

from ..data.dataset import Dataset


def read_idx(path) -> np.ndarray:
    op = gzip.open if str(path).endswith(".gz") else open
    with op(path, "rb") as f:
        zero, dtype, nd = struct.unpack(">HBB", f.read(4))
        shape = struct.unpack(">" + "I" * nd, f.read(4 * nd))
        dt = {8: np.uint8, 9: np.int8, 11: ">i2", 12: ">i4", 13: ">f4", 14: ">f8"}[dtype]
        return np.frombuffer(f.read(), dtype=dt).reshape(shape)


class MNIST(Dataset):
    FILES = {True: ("train-images-idx3-ubyte", "train-labels-idx1-ubyte"), False: ("t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte")}

    def __init__(self, root: str, train: bool = True):
        img, lab = self.FILES[train]
        def find(n):
            for c in (n, n + ".gz"):
                if os.path.exists(os.path.join(root, c)):
                    return os.path.join(root, c)
            raise FileNotFoundError(os.path.join(root, n))
        self.images = torch.from_numpy(read_idx(find(img)).copy()).float().div_(255.0).unsqueeze(1)
        self.labels = torch.from_numpy(read_idx(find(lab)).copy()).long()
        self.train = train

    CLASSES = [str(d) for d in range(10)]

    @classmethod
    def new(cls, root, train=True): return cls(root, train)
    def len(self) -> int: return self.images.shape[0]
    def get(self, i): return self.images[i], self.labels[i]
    def is_train(self) -> bool: return self.train
    def num_classes(self) -> int: return 10
    def image_size(self) -> tuple: return (28, 28)
    @classmethod
    def class_names(cls) -> list: return list(cls.CLASSES)


class FashionMNIST(MNIST):
    CLASSES = ["T-shirt/top", "Trouser", "Pullover", "Dress", "Coat", "Sandal", "Shirt", "Sneaker", "Bag", "Ankle boot"]


class CIFAR10(Dataset):
    NUM_FINE, REC = 10, 3073

    def __init__(self, root: str, train: bool = True):
        files = [f"data_batch_{i}.bin" for i in range(1, 6)] if train else ["test_batch.bin"]
        raw = np.concatenate([np.fromfile(os.path.join(root, f), dtype=np.uint8) for f in files]).reshape(-1, self.REC)
        self.labels = torch.from_numpy(raw[:, self.REC - 3073].astype(np.int64))
        self.images = torch.from_numpy(raw[:, -3072:].copy()).float().div_(255.0).view(-1, 3, 32, 32)
        self.train = train

    CLASSES = ["airplane", "automobile", "bird", "cat", "deer", "dog", "frog", "horse", "ship", "truck"]

    @classmethod
    def new(cls, root, train=True): return cls(root, train)
    def len(self) -> int: return self.images.shape[0]
    def get(self, i): return self.images[i], self.labels[i]
    def is_train(self) -> bool: return self.train
    def num_classes(self) -> int: return self.NUM_FINE
    def image_size(self) -> tuple: return (3, 32, 32)
    @classmethod
    def class_names(cls) -> list: return list(cls.CLASSES)


class CIFAR100(CIFAR10):
    NUM_FINE, REC = 100, 3074

    def __init__(self, root: str, train: bool = True):
        raw = np.fromfile(os.path.join(root, "train.bin" if train else "test.bin"), dtype=np.uint8).reshape(-1, self.REC)
        self.coarse_labels = torch.from_numpy(raw[:, 0].astype(np.int64))        # the 20 superclasses
        self.labels = torch.from_numpy(raw[:, 1].astype(np.int64))
        self.images = torch.from_numpy(raw[:, 2:].copy()).float().div_(255.0).view(-1, 3, 32, 32)
        self.train = train

    CLASSES = None                                    # the 100 fine names are not part of the binary files

    @classmethod
    def class_names(cls): return None
    def num_fine_classes(self) -> int: return 100
    def num_coarse_classes(self) -> int: return 20

    def get_with_coarse(self, i: int):
        """``(image, fine label, coarse label)``, or ``None`` past the end."""
        if not 0 <= i < self.len():
            return None
        return self.images[i], self.labels[i], self.coarse_labels[i]


class _SyntheticImages(Dataset):
    def __init__(self, n, shape, classes, seed):
        self.n, self.shape, self.classes, self.seed = n, shape, classes, seed

    def len(self) -> int: return self.n
    def num_classes(self) -> int: return self.classes

    def get(self, i):
        if not 0 <= i < self.n:
            raise IndexError(f"index {i} out of range for a dataset of {self.n} samples")
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        label = i % self.classes
        img = torch.rand(self.shape, generator=g) * 0.3
        c, h, w = self.shape
        r = (label * 2 + 2) % (h - 4)
        img[:, r:r + 4, :] += 0.6           # a class-dependent bright band makes the task learnable
        return img.clamp_(0, 1), torch.tensor(label, dtype=torch.long)


class SyntheticMNIST(_SyntheticImages):
    def __init__(self, num_samples: int = 1000, seed: int = 42): super().__init__(num_samples, (1, 28, 28), 10, seed)
    @classmethod
    def new(cls, num_samples=1000): return cls(num_samples)
    # sizes of the reference's presets (mnist.rs:285-299)
    @classmethod
    def small(cls): return cls(100)
    @classmethod
    def train(cls): return cls(60000)
    @classmethod
    def test(cls): return cls(10000)


class SyntheticCIFAR(_SyntheticImages):
    def __init__(self, num_samples: int = 1000, num_classes: int = 10, seed: int = 42): super().__init__(num_samples, (3, 32, 32), num_classes, seed)
    @classmethod
    def new(cls, num_samples=1000): return cls(num_samples)
    @classmethod
    def cifar10(cls, size: int): return cls(size, 10)
    @classmethod
    def cifar100(cls, size: int): return cls(size, 100)
    @classmethod
    def small(cls): return cls(100, 10)
    @classmethod
    def train(cls): return cls(50000, 10)
    @classmethod
    def test(cls): return cls(10000, 10)
    def class_names(self):
        """The CIFAR-10 names for a ten-class set, ``None`` otherwise."""
        return CIFAR10.class_names() if self.classes == 10 else None


class SyntheticImageNet(_SyntheticImages):
    """N(0,1) 3x224x224 images with uniform random labels in [0, 1000) (benchmark input shape)."""

    def __init__(self, num_samples: int = 1024, seed: int = 0): super().__init__(num_samples, (3, 224, 224), 1000, seed)

    def get(self, i):
        if not 0 <= i < self.n:
            raise IndexError(f"index {i} out of range for a dataset of {self.n} samples")
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        return torch.randn(self.shape, generator=g), torch.randint(0, 1000, (), generator=g)


def write_idx(path, array: np.ndarray) -> None:
    """Writes a uint8 array in IDX format (the inverse of ``read_idx``)."""
    a = np.ascontiguousarray(array, dtype=np.uint8)
    with open(path, "wb") as f:
        f.write(struct.pack(">HBB", 0, 8, a.ndim))
        f.write(struct.pack(">" + "I" * a.ndim, *a.shape))
        f.write(a.tobytes())


def write_synthetic_idx(root: str, shape, classes: int, samples: int = 2048, seed: int = 42) -> int:
    """A stand-in for MNIST-style data in the original file layout (train and t10k image/label IDX
    files), generated from the synthetic dataset, so that ``MNIST(root)`` reads it.  Only
    single-channel shapes have an IDX layout; others are written channel-first as 4-D IDX."""
    os.makedirs(root, exist_ok=True)
    c, h, w = shape
    ds = _SyntheticImages(samples, (c, h, w), classes, seed)
    imgs = np.zeros((samples, h, w) if c == 1 else (samples, c, h, w), dtype=np.uint8)
    labels = np.zeros((samples,), dtype=np.uint8)
    for i in range(samples):
        x, y = ds.get(i)
        imgs[i] = (x[0] if c == 1 else x).mul(255).round().to(torch.uint8).numpy()
        labels[i] = int(y)
    n_test = max(samples // 8, 1)
    write_idx(os.path.join(root, "train-images-idx3-ubyte"), imgs[:-n_test])
    write_idx(os.path.join(root, "train-labels-idx1-ubyte"), labels[:-n_test])
    write_idx(os.path.join(root, "t10k-images-idx3-ubyte"), imgs[-n_test:])
    write_idx(os.path.join(root, "t10k-labels-idx1-ubyte"), labels[-n_test:])
    return samples
