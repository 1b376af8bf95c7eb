"""A small LLaMA trained on sequences that are sharded over the ranks (context parallel).

Every rank holds the whole model and one slice of every sequence; attention exchanges q/k/v with
all-to-alls (form "ulysses"), gathers K/V ("allgather") or passes them around the ring ("ring").
The loss each rank returns is scaled so that the mean over the ranks is the loss of the whole
sequence, and DDP over the same ranks averages the gradients accordingly.

    python examples/context_parallel_llama.py                       # one process: plain attention
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \\
        examples/context_parallel_llama.py --form ring
"""
import argparse

import torch

from axonml_b200 import optim
from axonml_b200.llm import LLaMAConfig, LLaMAForCausalLM
from axonml_b200.parallel import DDP, ProcessGroup
from axonml_b200.parallel.backend import init_from_env


def main(form: str = "ulysses", steps: int = 20, seq_len: int = 64) -> float:
    pg = ProcessGroup(init_from_env())
    dev = pg.backend().device()
    torch.manual_seed(0)                                   # same weights and data on every rank
    cfg = LLaMAConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=seq_len)
    model = LLaMAForCausalLM(cfg).to(dev).enable_context_parallel(pg, form)
    ddp = DDP(model, pg)
    opt = optim.AdamW(list(model.parameters()), 3e-3)
    ids = (torch.arange(seq_len).repeat(4, 1) * 7 + torch.arange(4)[:, None]) % cfg.vocab_size   # learnable pattern
    ids = ids.to(dev)
    loss_value = 0.0
    for step in range(steps):
        loss, _ = model.forward_with_loss(ids)
        loss.backward()
        ddp.sync_gradients()
        opt.step()
        opt.zero_grad()
        t = loss.detach().clone()
        pg.backend().all_reduce(t)
        loss_value = float(t) / pg.world_size()
        if pg.rank() == 0 and (step % 5 == 0 or step == steps - 1):
            print(f"step {step:3d}  loss {loss_value:.4f}  ({pg.world_size()} rank(s), form {form})")
    return loss_value


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--form", default="ulysses", choices=["ulysses", "allgather", "ring"])
    ap.add_argument("--steps", type=int, default=20)
    a = ap.parse_args()
    main(a.form, a.steps)
