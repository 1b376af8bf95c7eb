"""HVAC multi-horizon failure predictor (the reference's crates/axonml/examples/hvac_model.rs):
Linear(28 -> 128) + LayerNorm + ReLU, a 2-layer GRU, mean pooling over time, and three heads
(5, 15 and 30 minute horizons), each Linear(128 -> 128) -> ReLU -> Linear(128 -> 64) -> ReLU ->
Linear(64 -> 20).

    python examples/hvac_model.py
"""
from dataclasses import dataclass

import torch

from axonml_b200 import nn

FAILURE_TYPES = ["normal", "pump_failure_hw_5", "pump_failure_hw_6", "pump_failure_cw_3", "pump_failure_cw_4",
                 "pump_failure_2pipe_a", "pump_failure_2pipe_b", "pressure_low_hw", "pressure_high_hw", "pressure_low_cw",
                 "pressure_high_cw", "temp_anomaly_hw_supply", "temp_anomaly_cw_supply", "temp_anomaly_space",
                 "valve_stuck_1_3", "valve_stuck_2_3", "vfd_fault", "sensor_drift", "chiller_fault", "interlock_violation"]


@dataclass
class HvacConfig:
    num_features: int = 28
    seq_len: int = 120
    hidden_size: int = 128
    num_layers: int = 2
    num_classes: int = 20
    dropout: float = 0.1


class PredictionHead(nn.Module):
    def __init__(self, hidden: int, classes: int, dropout: float):
        super().__init__()
        self.fc1, self.fc2, self.fc3 = nn.Linear(hidden, hidden), nn.Linear(hidden, 64), nn.Linear(64, classes)
        self.drop = nn.Dropout(dropout)

    def forward(self, x):
        x = self.drop(torch.relu(self.fc1(x)))
        return self.fc3(torch.relu(self.fc2(x)))


class HvacPredictor(nn.Module):
    def __init__(self, cfg: HvacConfig | None = None):
        super().__init__()
        self.cfg = cfg or HvacConfig()
        c = self.cfg
        self.input_proj = nn.Linear(c.num_features, c.hidden_size)
        self.input_norm = nn.LayerNorm(c.hidden_size)
        self.gru = nn.GRU(c.hidden_size, c.hidden_size, c.num_layers, batch_first=True)
        self.head_5min = PredictionHead(c.hidden_size, c.num_classes, c.dropout)
        self.head_15min = PredictionHead(c.hidden_size, c.num_classes, c.dropout)
        self.head_30min = PredictionHead(c.hidden_size, c.num_classes, c.dropout)

    def forward(self, x):
        """x: [batch, seq_len, num_features] -> three [batch, num_classes] logit tensors."""
        h = torch.relu(self.input_norm(self.input_proj(x)))
        out = self.gru(h)
        seq = out[0] if isinstance(out, tuple) else out
        pooled = seq.mean(dim=1)
        return self.head_5min(pooled), self.head_15min(pooled), self.head_30min(pooled)

    def predict(self, x):
        with torch.no_grad():
            return tuple(torch.softmax(l, -1) for l in self.forward(x))


def main():
    torch.manual_seed(0)
    model = HvacPredictor().eval()
    n = sum(p.numel() for p in model.parameters())
    print(f"HvacPredictor: {n:,} parameters")
    x = torch.rand(2, model.cfg.seq_len, model.cfg.num_features)
    for name, p in zip(("5 min", "15 min", "30 min"), model.predict(x)):
        top = int(p[0].argmax())
        print(f"  {name:6s}: shape {tuple(p.shape)}, row sums {p.sum(-1).tolist()}, top class {FAILURE_TYPES[top]} ({float(p[0, top]):.3f})")
    return model


if __name__ == "__main__":
    main()
