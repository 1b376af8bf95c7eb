"""XOR with a 2-4-1 sigmoid MLP and Adam (the reference's crates/axonml/examples/simple_training.rs).

    python examples/simple_training.py
"""
import torch

import axonml_b200 as axonml
from axonml_b200 import nn, optim


def main(epochs: int = 1000) -> float:
    print("=== AxonML - simple training example ===\n")
    print("version :", axonml.version())
    print("features:", axonml.features(), "\n")
    inputs = torch.tensor([[0.0, 0.0], [0.0, 1.0], [1.0, 0.0], [1.0, 1.0]])
    targets = torch.tensor([[0.0], [1.0], [1.0], [0.0]])
    torch.manual_seed(0)
    l1, l2 = nn.Linear(2, 4), nn.Linear(4, 1)
    opt = optim.Adam(list(l1.parameters()) + list(l2.parameters()), 0.1)
    loss_value = 0.0
    for epoch in range(epochs):
        total = 0.0
        for x, y in zip(inputs, targets):
            out = torch.sigmoid(l2(torch.sigmoid(l1(x.unsqueeze(0)))))
            loss = ((out - y.unsqueeze(0)) ** 2).sum()
            total += float(loss.detach())
            loss.backward()
            opt.step()
            opt.zero_grad()
        loss_value = total / 4
        if epoch % 200 == 0 or epoch == epochs - 1:
            print(f"   epoch {epoch}: loss = {loss_value:.6f}")
    print("\ntrained model:")
    with torch.no_grad():
        for x, y in zip(inputs, targets):
            p = float(torch.sigmoid(l2(torch.sigmoid(l1(x.unsqueeze(0))))))
            print(f"   input {x.tolist()} -> {p:.4f} (rounded {round(p)}) | expected {int(y)}")
    return loss_value


if __name__ == "__main__":
    main()
