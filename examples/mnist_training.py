"""MNIST classification with an MLP (the reference's crates/axonml/examples/mnist_training.rs).
Reads the IDX files from ``--data`` when they exist, else trains on the synthetic stand-in.

    python examples/mnist_training.py [--data ./data/mnist] [--epochs 2] [--device cuda]
"""
import argparse
import os
import time

import torch

from axonml_b200 import nn, optim
from axonml_b200.data import DataLoader
from axonml_b200.trainer import compute_accuracy
from axonml_b200.vision.datasets import MNIST, SyntheticMNIST


def main(argv=None) -> float:
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default="./data/mnist")
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--samples", type=int, default=2048, help="size of the synthetic set when the files are absent")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    have = os.path.exists(os.path.join(a.data, "train-images-idx3-ubyte"))
    train = MNIST(a.data, train=True) if have else SyntheticMNIST(a.samples)
    test = MNIST(a.data, train=False) if have else SyntheticMNIST(a.samples // 4, seed=7)
    print(f"dataset: {'MNIST files' if have else 'synthetic MNIST'}; {train.len()} training / {test.len()} test samples")
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 128), nn.ReLU(), nn.Linear(128, 10)).to(a.device)
    opt = optim.Adam(list(model.parameters()), 1e-3)
    crit = nn.CrossEntropyLoss()
    acc = 0.0
    for epoch in range(a.epochs):
        t0, total, n = time.time(), 0.0, 0
        for b in DataLoader(train, a.batch_size, shuffle=True):
            x, y = b.data.to(a.device).reshape(b.data.shape[0], -1), b.targets.to(a.device)
            opt.zero_grad()
            loss = crit(model(x), y)
            loss.backward()
            opt.step()
            total, n = total + float(loss.detach()), n + 1
        hit = tot = 0
        with torch.no_grad():
            for b in DataLoader(test, 256):
                x, y = b.data.to(a.device).reshape(b.data.shape[0], -1), b.targets.to(a.device)
                hit += compute_accuracy(model(x), y) * y.numel()
                tot += y.numel()
        acc = hit / max(tot, 1)
        print(f"epoch {epoch + 1}/{a.epochs}: loss {total / max(n, 1):.4f}  test accuracy {acc:.4f}  ({time.time() - t0:.1f}s)")
    return acc


if __name__ == "__main__":
    main()
