"""Text generation (crates/axonml-llm/src/generation.rs:11-395): ``GenerationConfig`` with its
presets, ``TextGenerator`` (repetition penalty -> temperature -> top-k -> top-p -> sample or
argmax) and ``BeamSearch``.  Sampling is real (the reference's ``generate`` is always greedy)."""
from __future__ import annotations

import dataclasses

import torch


@dataclasses.dataclass
class GenerationConfig:
    max_new_tokens: int = 50
    temperature: float = 1.0
    top_k: int | None = None
    top_p: float | None = None
    repetition_penalty: float = 1.0
    eos_token_ids: list = dataclasses.field(default_factory=list)
    pad_token_id: int | None = None
    do_sample: bool = True
    num_beams: int = 1
    length_penalty: float = 1.0
    early_stopping: bool = False

    @classmethod
    def greedy(cls, max_new_tokens: int = 50): return cls(max_new_tokens=max_new_tokens, do_sample=False)
    @classmethod
    def sampling(cls, max_new_tokens: int = 50, temperature: float = 1.0):
        return cls(max_new_tokens=max_new_tokens, temperature=temperature)
    @classmethod
    def top_k_sampling(cls, max_new_tokens: int, k: int, temperature: float = 1.0):
        return cls(max_new_tokens=max_new_tokens, top_k=k, temperature=temperature)
    @classmethod
    def nucleus_sampling(cls, max_new_tokens: int, p: float, temperature: float = 1.0):
        return cls(max_new_tokens=max_new_tokens, top_p=p, temperature=temperature)
    @classmethod
    def beam_search(cls, max_new_tokens: int, num_beams: int):
        return cls(max_new_tokens=max_new_tokens, num_beams=num_beams, do_sample=False)

    # chainable setters (generation.rs:105-121)
    def with_max_tokens(self, max_new_tokens: int):
        self.max_new_tokens = int(max_new_tokens)
        return self

    def with_eos_token(self, eos_token_id: int):
        self.eos_token_ids = list(self.eos_token_ids) + [int(eos_token_id)]
        return self

    def with_repetition_penalty(self, penalty: float):
        self.repetition_penalty = float(penalty)
        return self


class TextGenerator:
    def __init__(self, config: GenerationConfig | None = None):
        self.config = config or GenerationConfig()

    @classmethod
    def new(cls, config): return cls(config)

    # ---- the steps of the pipeline, each on ``logits [B, V]`` (or ``[V]``), returning new logits
    def apply_repetition_penalty(self, logits: torch.Tensor, generated) -> torch.Tensor:
        """Scores of tokens already generated are divided by the penalty when positive and
        multiplied when negative (generation.rs:145-158)."""
        pen = self.config.repetition_penalty
        if pen == 1.0 or generated is None:
            return logits
        gen = torch.as_tensor(generated, device=logits.device).long()
        if gen.numel() == 0:
            return logits
        flat = logits.dim() == 1
        lg = (logits.unsqueeze(0) if flat else logits).clone()
        gen = gen.reshape(lg.shape[0], -1)
        score = torch.gather(lg, 1, gen)
        lg.scatter_(1, gen, torch.where(score > 0, score / pen, score * pen))
        return lg[0] if flat else lg

    def apply_temperature(self, logits: torch.Tensor) -> torch.Tensor:
        t = self.config.temperature
        return logits / t if t != 1.0 and t > 0 else logits

    def apply_top_k(self, logits: torch.Tensor) -> torch.Tensor:
        """Everything below the k-th largest logit becomes -inf."""
        k = self.config.top_k
        if k is None or not 0 < k < logits.shape[-1]:
            return logits
        kth = torch.topk(logits, k, dim=-1).values[..., -1:]
        return logits.masked_fill(logits < kth, float("-inf"))

    def apply_top_p(self, logits: torch.Tensor) -> torch.Tensor:
        """Keeps the smallest set of most likely tokens whose probabilities sum to at least p."""
        p = self.config.top_p
        if p is None or not 0.0 < p < 1.0:
            return logits
        sl, si = torch.sort(logits, descending=True, dim=-1)
        probs = torch.softmax(sl, -1)
        sl = sl.masked_fill(probs.cumsum(-1) - probs > p, float("-inf"))
        return torch.full_like(logits, float("-inf")).scatter(-1, si, sl)

    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        return logits.argmax(-1)

    def process_logits(self, logits: torch.Tensor, generated: torch.Tensor | None = None) -> torch.Tensor:
        """Repetition penalty -> temperature -> top-k -> top-p on fp32 logits (generation.rs:258-270)."""
        logits = self.apply_repetition_penalty(logits.float(), generated)
        return self.apply_top_p(self.apply_top_k(self.apply_temperature(logits)))

    def get_next_token(self, logits, generated=None):
        """Next token for one sequence: ``logits [V]`` and the tokens generated so far -> int."""
        lg = torch.as_tensor(logits, dtype=torch.float32).reshape(1, -1)
        gen = None if generated is None else torch.as_tensor(generated).reshape(1, -1)
        return int(self.sample(lg, gen)[0])

    def should_stop(self, token: int) -> bool:
        return int(token) in self.config.eos_token_ids

    def sample(self, logits: torch.Tensor, generated=None) -> torch.Tensor:
        logits = self.process_logits(logits, generated)
        if self.config.do_sample:
            return torch.multinomial(torch.softmax(logits, -1), 1).squeeze(-1)
        return logits.argmax(-1)

    @torch.no_grad()
    def generate(self, model, ids: torch.Tensor) -> torch.Tensor:
        """Autoregressive decode with the model's KV cache when it offers one."""
        c = self.config
        if c.num_beams > 1:
            return BeamSearch(c.num_beams, c.length_penalty, c.early_stopping).search(model, ids, c)
        caches = model.create_kv_cache(ids.shape[0], ids.shape[1] + c.max_new_tokens) if hasattr(model, "create_kv_cache") else None
        out = ids
        done = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
        step_in, pos0 = ids, 0
        for _ in range(c.max_new_tokens):
            if caches is not None:
                logits = model(step_in, caches, pos0) if _takes_pos(model) else model(step_in, caches)
                pos0 += step_in.shape[1]
            else:
                logits = model(out)
            nxt = self.sample(logits[:, -1], out)
            if c.eos_token_ids:
                if c.pad_token_id is not None:
                    nxt = torch.where(done, torch.full_like(nxt, c.pad_token_id), nxt)
                done = done | torch.isin(nxt, torch.tensor(c.eos_token_ids, device=nxt.device))
            out = torch.cat([out, nxt[:, None]], dim=1)
            step_in = nxt[:, None]
            if c.eos_token_ids and bool(done.all()):
                break
        return out


def _takes_pos(model) -> bool:
    import inspect
    try:
        return "pos0" in inspect.signature(model.forward).parameters
    except (TypeError, ValueError):
        return False


@dataclasses.dataclass
class Beam:
    """One hypothesis of a beam search (generation.rs:279-303): its tokens, the sum of the
    log-probabilities of the generated ones, and whether it has produced an end token."""
    tokens: list
    score: float = 0.0
    finished: bool = False

    @classmethod
    def new(cls, initial_tokens): return cls(list(initial_tokens))

    def normalized_score(self, length_penalty: float) -> float:
        return self.score / (len(self.tokens) ** length_penalty)

    def extended(self, token: int, log_prob: float, finished: bool) -> "Beam":
        return Beam(self.tokens + [int(token)], self.score + float(log_prob), finished)


class BeamSearch:
    """Beam search as separate steps (generation.rs:306-395) -- ``init_beams``, ``expand_beams``,
    ``should_stop``, ``best_sequence`` -- and ``search``, which drives them with a model."""

    def __init__(self, num_beams: int, length_penalty: float = 1.0, early_stopping: bool = False, eos_token_ids=()):
        self.num_beams, self.length_penalty, self.early_stopping = num_beams, length_penalty, early_stopping
        self.eos_token_ids = [int(t) for t in eos_token_ids]

    @classmethod
    def new(cls, num_beams, length_penalty, early_stopping, eos_token_ids): return cls(num_beams, length_penalty, early_stopping, eos_token_ids)

    def init_beams(self, input_ids) -> list:
        return [Beam.new(torch.as_tensor(input_ids).reshape(-1).tolist())]

    def expand_beams(self, beams, next_token_logits) -> list:
        """One step: every live beam is extended by its ``2 * num_beams`` best tokens (scores are
        added as given: pass log-probabilities), finished beams are carried over, and the
        ``num_beams`` candidates with the best length-normalised score are kept."""
        eos = set(self.eos_token_ids)
        cand = []
        for beam, logits in zip(beams, next_token_logits):
            if beam.finished:
                cand.append(beam)
                continue
            lp = torch.as_tensor(logits, dtype=torch.float32).reshape(-1)
            top = torch.topk(lp, min(2 * self.num_beams, lp.numel()))
            for v, i in zip(top.values.tolist(), top.indices.tolist()):
                cand.append(beam.extended(i, v, i in eos))
        cand.sort(key=lambda b: b.normalized_score(self.length_penalty), reverse=True)
        return cand[:self.num_beams]

    def should_stop(self, beams) -> bool:
        return self.early_stopping and all(b.finished for b in beams)

    def best_sequence(self, beams):
        """Tokens of the best finished beam; of the first beam when none has finished; None without beams."""
        done = [b for b in beams if b.finished]
        if done:
            return list(max(done, key=lambda b: b.normalized_score(self.length_penalty)).tokens)
        return list(beams[0].tokens) if beams else None

    @torch.no_grad()
    def search(self, model, ids: torch.Tensor, config: GenerationConfig) -> torch.Tensor:
        """Beam search for batch size 1 (as in the reference); returns the best sequence."""
        if not self.eos_token_ids:
            self.eos_token_ids = [int(t) for t in config.eos_token_ids]
        beams = self.init_beams(ids[:1])
        for _ in range(config.max_new_tokens):
            live = [b for b in beams if not b.finished]
            if not live:
                break
            batch = torch.tensor([b.tokens for b in live], device=ids.device)      # live beams have equal lengths
            lps = torch.log_softmax(model(batch)[:, -1].float(), -1)
            it = iter(lps)
            beams = self.expand_beams(beams, [None if b.finished else next(it) for b in beams])
            if all(b.finished for b in beams) or (self.early_stopping and beams[0].finished):
                break
        return torch.tensor([self.best_sequence(beams)], device=ids.device)
