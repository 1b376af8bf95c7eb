"""Inference with the trained HVAC predictor (the reference's
crates/axonml/examples/hvac_inference.rs): loads the ``.axonml`` checkpoint written by
``hvac_training.py``, builds one window of nominal sensor readings and prints the three horizons.

    python examples/hvac_inference.py [output/hvac_model.axonml]
"""
import sys

import torch

from axonml_b200.serialize import load_state_dict

try:
    from hvac_model import FAILURE_TYPES, HvacConfig, HvacPredictor
except ImportError:
    from examples.hvac_model import FAILURE_TYPES, HvacConfig, HvacPredictor


def nominal_window(seq_len: int) -> torch.Tensor:
    row = [25.0 / 50.0] * 6 + [(180 - 80) / 120, (55 - 40) / 40, (135 - 115) / 40, (95 - 70) / 50,
                               (70 + 20) / 140, (72 - 50) / 40, (72 - 65) / 20, (72 - 65) / 20, 0.5, 0.5] + [0.6] * 6 \
        + [0.5, 0.5, 0.0, 0.0, 0.0, 0.0]
    return torch.tensor(row).repeat(seq_len, 1).unsqueeze(0)


def main(path: str = "output/hvac_model.axonml", seq_len: int = 60):
    model = HvacPredictor(HvacConfig(seq_len=seq_len)).eval()
    try:
        load_state_dict(path).load_into(model, strict=False)
        print(f"loaded {path}")
    except FileNotFoundError:
        print(f"{path} not found: using untrained weights (run hvac_training.py first)")
    x = nominal_window(seq_len)
    print("input shape:", tuple(x.shape))
    out = {}
    for name, p in zip(("5 min", "15 min", "30 min"), model.predict(x)):
        top = torch.topk(p[0], 3)
        out[name] = [(FAILURE_TYPES[int(i)], float(v)) for v, i in zip(top.values, top.indices)]
        print(f"  {name:6s}: " + ", ".join(f"{n} {v:.3f}" for n, v in out[name]))
    return out


if __name__ == "__main__":
    main(*sys.argv[1:2])
