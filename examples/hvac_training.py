"""Training pipeline for the HVAC failure predictor (the reference's
crates/axonml/examples/hvac_training.rs): synthetic sensor traces of normal operation with injected
pump, pressure and temperature failures, sliding windows with labels at three horizons, AdamW,
per-epoch validation accuracy, checkpoint in the ``.axonml`` format.

    python examples/hvac_training.py [--epochs 3] [--device cuda]
"""
import argparse
import math
import os

import torch

from axonml_b200 import nn, optim
from axonml_b200.data import DataLoader, TensorDataset
from axonml_b200.serialize import save_state_dict
from axonml_b200.serialize.state_dict import StateDict

try:
    from hvac_model import HvacConfig, HvacPredictor
except ImportError:  # run as a module from the repository root
    from examples.hvac_model import HvacConfig, HvacPredictor

HORIZONS = (5, 15, 30)          # minutes ahead == samples ahead (one sample per minute)


class HvacDataGenerator:
    """28 normalised features: 6 pump currents, 4 loop pressures, 6 temperatures, 6 valve positions,
    2 VFD speeds, 4 status bits (the grouping of the reference's generator)."""

    def __init__(self, seed: int = 0):
        self.g = torch.Generator().manual_seed(seed)

    def normal(self, n: int) -> torch.Tensor:
        t = torch.arange(n, dtype=torch.float32)
        base = torch.tensor([0.5] * 6 + [0.83, 0.38, 0.5, 0.5] + [0.64, 0.55, 0.35, 0.35, 0.5, 0.5] + [0.6] * 6 + [0.5, 0.5]
                            + [0.0] * 4)
        daily = 0.05 * torch.sin(2 * math.pi * t / 1440.0).unsqueeze(1)
        x = base.unsqueeze(0) + daily + 0.01 * torch.randn(n, 28, generator=self.g)
        x[:, 24:] = 0.0
        return x.clamp(0, 1)

    def inject(self, x: torch.Tensor, kind: int, start: int) -> torch.Tensor:
        """Labels per sample (0 = normal).  kind 1-6 pump current decay, 7-10 pressure low/high, 11-13 temperature."""
        n = x.shape[0]
        labels = torch.zeros(n, dtype=torch.long)
        ramp = torch.clamp((torch.arange(n) - start).float(), min=0) * 0.01
        if 1 <= kind <= 6:
            x[:, kind - 1] = (x[:, kind - 1] - ramp).clamp(0, 1)
            labels[x[:, kind - 1] < 0.3] = kind
        elif 7 <= kind <= 10:
            col, sign = 6 + (kind - 7) // 2 * 2, (-1.0 if (kind - 7) % 2 == 0 else 1.0)
            x[:, col] = (x[:, col] + sign * ramp).clamp(0, 1)
            labels[(x[:, col] - (0.83 if col == 6 else 0.5)).abs() > 0.2] = kind
        else:
            col = 10 + (kind - 11)
            x[:, col] = (x[:, col] + ramp).clamp(0, 1)
            labels[ramp > 0.2] = kind
        labels[:start] = 0
        return labels

    def dataset(self, scenarios: int, length: int, seq_len: int, stride: int = 10):
        xs, ys = [], []
        for s in range(scenarios):
            x = self.normal(length)
            kind = s % 14                       # 0 = a purely normal trace
            labels = self.inject(x, kind, length // 3) if kind else torch.zeros(length, dtype=torch.long)
            last = length - seq_len - max(HORIZONS)
            for t0 in range(0, last, stride):
                xs.append(x[t0:t0 + seq_len])
                ys.append(torch.stack([labels[t0 + seq_len - 1 + h] for h in HORIZONS]))
        return torch.stack(xs), torch.stack(ys)


def evaluate(model, loader, device):
    model.eval()
    hit = torch.zeros(3)
    tot = 0
    with torch.no_grad():
        for b in loader:
            outs = model(b.data.to(device))
            y = b.targets.to(device)
            for i, o in enumerate(outs):
                hit[i] += float((o.argmax(-1) == y[:, i]).sum())
            tot += y.shape[0]
    model.train()
    return (hit / max(tot, 1)).tolist()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--epochs", type=int, default=3)
    ap.add_argument("--scenarios", type=int, default=28)
    ap.add_argument("--length", type=int, default=400)
    ap.add_argument("--seq-len", type=int, default=60)
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--output", default="output/hvac_model.axonml")
    a = ap.parse_args(argv)
    torch.manual_seed(0)
    x, y = HvacDataGenerator(0).dataset(a.scenarios, a.length, a.seq_len)
    n_val = max(len(x) // 5, 1)
    perm = torch.randperm(len(x))
    tr, va = perm[n_val:], perm[:n_val]
    print(f"{len(tr)} training windows, {len(va)} validation windows, {int((y[:, 0] > 0).sum())} windows end in a failure")
    train = DataLoader(TensorDataset(x[tr], y[tr]), a.batch_size, shuffle=True)
    val = DataLoader(TensorDataset(x[va], y[va]), 128)
    model = HvacPredictor(HvacConfig(seq_len=a.seq_len)).to(a.device)
    opt = optim.AdamW(list(model.parameters()), 1e-3, weight_decay=0.01)
    crit = nn.CrossEntropyLoss()
    accs = [0.0, 0.0, 0.0]
    for epoch in range(a.epochs):
        total, n = 0.0, 0
        for b in train:
            xb, yb = b.data.to(a.device), b.targets.to(a.device)
            opt.zero_grad()
            outs = model(xb)
            loss = sum(crit(o, yb[:, i]) for i, o in enumerate(outs)) / 3.0
            loss.backward()
            optim.clip_grad_norm(list(model.parameters()), 1.0)
            opt.step()
            total, n = total + float(loss.detach()), n + 1
        accs = evaluate(model, val, a.device)
        print(f"epoch {epoch + 1}/{a.epochs}: loss {total / max(n, 1):.4f}  val accuracy 5/15/30 min: "
              + " / ".join(f"{v:.3f}" for v in accs))
    os.makedirs(os.path.dirname(a.output) or ".", exist_ok=True)
    save_state_dict(StateDict.from_module(model), a.output)
    print(f"saved {a.output}")
    return accs


if __name__ == "__main__":
    main()
