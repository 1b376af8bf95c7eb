"""Tensor-parallel (Megatron style, sequence-parallel) LLaMA for training on one NVSwitch box.

Same architecture and arithmetic as ``llm/llama.py`` (crates/axonml-llm/src/llama.rs), with every
weight matrix split over the tensor-parallel group the way the reference's ColumnParallelLinear /
RowParallelLinear split theirs (crates/axonml-distributed/src/fsdp.rs:414-600):

* the residual stream is sharded along tokens (rank r holds tokens ``[r*T/W, (r+1)*T/W)``);
* q|k|v and gate|up are column-parallel: ``all-gather(tokens) -> GEMM`` in one fused kernel;
* o_proj and down_proj are row-parallel: ``GEMM -> reduce-scatter(tokens)`` in one fused kernel;
* the embedding table and the LM head are split along the vocabulary (padded to a multiple of
  ``128 * W`` rows so that the fused GEMM tiles divide it); the loss is computed from the local
  logit slice with two small all-reduces (``vocab_parallel_cross_entropy``);
* RMSNorm weights are replicated; their gradients are summed over the group by
  ``sync_replicated_grads()``.

``from_full_state_dict`` / ``full_state_dict`` convert from and to the HuggingFace layout of the
unsharded model, so checkpoints stay interchangeable.
"""
from __future__ import annotations

import torch

from .. import nn
from ..nn.module import Parameter
from ..ops import elementwise as E
from ..ops import misc as Mi
from ..ops.attention import sdpa_packed
from ..parallel import fused_gemm
from ..parallel import tensor_parallel as TP
from ..parallel.backend import ReduceOp
from .config import LLaMAConfig


def padded_vocab(vocab_size: int, world: int) -> int:
    unit = 128 * world
    return (vocab_size + unit - 1) // unit * unit


class TPDecoderLayer(nn.Module):
    def __init__(self, cfg: LLaMAConfig, pg, device=None, dtype=torch.bfloat16):
        super().__init__()
        W = pg.world_size()
        self.pg = pg
        self.hd = cfg.head_dim()
        if cfg.num_attention_heads % W or cfg.num_key_value_heads % W or cfg.intermediate_size % W:
            raise ValueError("heads, kv heads and the FFN width must be divisible by the tensor-parallel size")
        self.nh, self.nkv, self.inter = cfg.num_attention_heads // W, cfg.num_key_value_heads // W, cfg.intermediate_size // W
        H = cfg.hidden_size
        mk = lambda r, c: Parameter(torch.empty(r, c, device=device, dtype=dtype).normal_(0.0, 0.02))
        self.input_layernorm = nn.RMSNorm(H, cfg.rms_norm_eps, device=device, dtype=dtype)
        self.post_attention_layernorm = nn.RMSNorm(H, cfg.rms_norm_eps, device=device, dtype=dtype)
        self.wqkv = mk((self.nh + 2 * self.nkv) * self.hd, H)     # local q heads | k heads | v heads
        self.wo = mk(H, self.nh * self.hd)
        self.wgu = mk(2 * self.inter, H)                          # local gate rows | up rows
        self.wdown = mk(H, self.inter)

    def forward(self, delta, residual, B: int, S: int, cos, sin):
        if residual is None:
            a, residual = self.input_layernorm(delta), delta
        else:
            a, residual = self.input_layernorm(delta, residual=residual)
        qkv = fused_gemm.all_gather_linear(a, self.wqkv, pg=self.pg)              # [B*S, (nh+2nkv)*hd]
        packed = qkv.view(B, S, self.nh + 2 * self.nkv, self.hd)
        packed = Mi.rope(packed, cos, sin, seq_len=S, pos0=0, rot_heads=self.nh + self.nkv)
        o = sdpa_packed(packed, self.nh, self.nkv, causal=True)
        attn = fused_gemm.linear_reduce_scatter(o.reshape(B * S, self.nh * self.hd), self.wo, pg=self.pg)
        m, residual = self.post_attention_layernorm(attn, residual=residual)
        gu = fused_gemm.all_gather_linear(m, self.wgu, pg=self.pg)
        return fused_gemm.linear_reduce_scatter(E.swiglu(gu), self.wdown, pg=self.pg), residual


class TPLLaMAForCausalLM(nn.Module):
    def __init__(self, cfg: LLaMAConfig, pg, device=None, dtype=torch.bfloat16, layers=None,
                 first_stage: bool = True, last_stage: bool = True):
        """``layers``: range of decoder layers held by this pipeline stage (default: all)."""
        super().__init__()
        self.cfg, self.pg = cfg, pg
        W, r = pg.world_size(), pg.rank()
        self.vocab_p = padded_vocab(cfg.vocab_size, W)
        self.v_local = self.vocab_p // W
        self.v_start = r * self.v_local
        H = cfg.hidden_size
        self.first_stage, self.last_stage = first_stage, last_stage
        if first_stage:
            self.embed = Parameter(torch.empty(self.v_local, H, device=device, dtype=dtype).normal_(0.0, 0.02))
        idx = list(layers) if layers is not None else list(range(cfg.num_hidden_layers))
        self.layer_ids = idx
        self.layers = nn.ModuleList([TPDecoderLayer(cfg, pg, device, dtype) for _ in idx])
        if last_stage:
            self.norm = nn.RMSNorm(H, cfg.rms_norm_eps, device=device, dtype=dtype)
            self.lm_head = Parameter(torch.empty(self.v_local, H, device=device, dtype=dtype).normal_(0.0, 0.02))
        cos, sin = Mi.rope_tables(cfg.max_position_embeddings, cfg.head_dim(), cfg.rope_theta)
        self.register_buffer("cos", cos.to(device), persistent=False)
        self.register_buffer("sin", sin.to(device), persistent=False)

    # ------------------------------------------------------------------ pieces (pipeline stages call these)
    def embed_tokens(self, ids):
        """ids [B, S] (identical on every rank) -> this rank's token shard of the embeddings [T/W, H]."""
        flat = ids.reshape(-1)
        local = flat - self.v_start
        local = local.masked_fill((local < 0) | (local >= self.v_local), -1)      # gather kernel: id < 0 -> zeros
        part = Mi.embedding(local, self.embed)
        return TP.reduce_scatter_tokens(part, self.pg)

    def run_layers(self, x_local, B: int, S: int, residual=None):
        delta = x_local
        for layer in self.layers:
            delta, residual = layer(delta, residual, B, S, self.cos, self.sin)
        return delta, residual

    def loss_from_hidden(self, delta, residual, labels):
        h, _ = self.norm(delta, residual=residual)
        logits = fused_gemm.all_gather_linear(h, self.lm_head, pg=self.pg)         # [B*S, V/W]
        tgt = torch.full_like(labels, -100)
        tgt[:, :-1] = labels[:, 1:]
        return TP.vocab_parallel_cross_entropy(logits, tgt.reshape(-1), self.pg, self.v_start,
                                               valid_vocab=self.cfg.vocab_size)

    def forward_with_loss(self, ids, labels=None):
        B, S = ids.shape
        labels = ids if labels is None else labels
        delta, residual = self.run_layers(self.embed_tokens(ids), B, S)
        return self.loss_from_hidden(delta, residual, labels)

    forward = forward_with_loss

    # ------------------------------------------------------------------ replicated parameters
    def replicated_parameters(self):
        out = []
        for layer in self.layers:
            out += [layer.input_layernorm.weight, layer.post_attention_layernorm.weight]
        if self.last_stage:
            out.append(self.norm.weight)
        return out

    def sync_replicated_grads(self) -> None:
        """Every rank saw only its token shard: sum the RMSNorm weight gradients over the group
        (one flat all-reduce)."""
        if self.pg.world_size() == 1:
            return
        ps = [p for p in self.replicated_parameters() if p.grad is not None]
        if not ps:
            return
        flat = torch.cat([p.grad.reshape(-1).float() for p in ps])
        self.pg.backend().all_reduce(flat, ReduceOp.Sum)
        off = 0
        for p in ps:
            n = p.grad.numel()
            p.grad.copy_(flat[off:off + n].view_as(p.grad))
            off += n

    # ------------------------------------------------------------------ checkpoints in the unsharded layout
    def load_full_state_dict(self, sd: dict) -> None:
        """``sd``: HuggingFace-named tensors of the unsharded model (as ``LLaMAForCausalLM`` has)."""
        W, r = self.pg.world_size(), self.pg.rank()
        cfg = self.cfg
        hd = cfg.head_dim()

        def rows(w, per_rank):
            return w[r * per_rank:(r + 1) * per_rank]

        def vocab_rows(w):
            out = torch.zeros(self.v_local, w.shape[1], dtype=w.dtype)
            lo, hi = self.v_start, min(self.v_start + self.v_local, w.shape[0])
            if hi > lo:
                out[:hi - lo] = w[lo:hi]
            return out

        with torch.no_grad():
            if self.first_stage:
                self.embed.copy_(vocab_rows(sd["model.embed_tokens.weight"]))
            for layer, i in zip(self.layers, self.layer_ids):
                p = f"model.layers.{i}."
                q = rows(sd[p + "self_attn.q_proj.weight"], layer.nh * hd)
                k = rows(sd[p + "self_attn.k_proj.weight"], layer.nkv * hd)
                v = rows(sd[p + "self_attn.v_proj.weight"], layer.nkv * hd)
                layer.wqkv.copy_(torch.cat([q, k, v], 0))
                wo = sd[p + "self_attn.o_proj.weight"]
                layer.wo.copy_(wo[:, r * layer.nh * hd:(r + 1) * layer.nh * hd])
                g = rows(sd[p + "mlp.gate_proj.weight"], layer.inter)
                u = rows(sd[p + "mlp.up_proj.weight"], layer.inter)
                layer.wgu.copy_(torch.cat([g, u], 0))
                wd = sd[p + "mlp.down_proj.weight"]
                layer.wdown.copy_(wd[:, r * layer.inter:(r + 1) * layer.inter])
                layer.input_layernorm.weight.copy_(sd[p + "input_layernorm.weight"])
                layer.post_attention_layernorm.weight.copy_(sd[p + "post_attention_layernorm.weight"])
            if self.last_stage:
                self.norm.weight.copy_(sd["model.norm.weight"])
                self.lm_head.copy_(vocab_rows(sd["lm_head.weight"]))

    def full_state_dict(self) -> dict:
        """Gathers the shards back into the unsharded HuggingFace layout (every rank gets it)."""
        pg, W = self.pg, self.pg.world_size()
        cfg, hd = self.cfg, self.cfg.head_dim()

        def gather(t):
            t = t.detach().contiguous()
            if W == 1:
                return [t]
            out = torch.empty((W,) + tuple(t.shape), dtype=t.dtype, device=t.device)
            pg.backend().all_gather(t, out)
            return list(out.unbind(0))

        sd = {}
        if self.first_stage:
            sd["model.embed_tokens.weight"] = torch.cat(gather(self.embed), 0)[:cfg.vocab_size]
        for layer, i in zip(self.layers, self.layer_ids):
            p = f"model.layers.{i}."
            nq, nk = layer.nh * hd, layer.nkv * hd
            parts = gather(layer.wqkv)
            sd[p + "self_attn.q_proj.weight"] = torch.cat([t[:nq] for t in parts], 0)
            sd[p + "self_attn.k_proj.weight"] = torch.cat([t[nq:nq + nk] for t in parts], 0)
            sd[p + "self_attn.v_proj.weight"] = torch.cat([t[nq + nk:] for t in parts], 0)
            sd[p + "self_attn.o_proj.weight"] = torch.cat(gather(layer.wo), 1)
            parts = gather(layer.wgu)
            sd[p + "mlp.gate_proj.weight"] = torch.cat([t[:layer.inter] for t in parts], 0)
            sd[p + "mlp.up_proj.weight"] = torch.cat([t[layer.inter:] for t in parts], 0)
            sd[p + "mlp.down_proj.weight"] = torch.cat(gather(layer.wdown), 1)
            sd[p + "input_layernorm.weight"] = layer.input_layernorm.weight.detach().clone()
            sd[p + "post_attention_layernorm.weight"] = layer.post_attention_layernorm.weight.detach().clone()
        if self.last_stage:
            sd["model.norm.weight"] = self.norm.weight.detach().clone()
            sd["lm_head.weight"] = torch.cat(gather(self.lm_head), 0)[:cfg.vocab_size]
        return sd


class TPPipelineStage(nn.Module):
    """One pipeline stage of the tensor-parallel model as a plain module: the first stage maps token
    ids to the packed ``[2, T/W, H]`` pair (delta, residual) of this rank's token shard, later
    stages map such a pair to the next one.  Ranks with the same tensor-parallel index in
    consecutive stages exchange exactly this tensor, so nothing is sent twice."""

    def __init__(self, model: TPLLaMAForCausalLM, seq_len: int):
        super().__init__()
        self.model, self.seq_len = model, seq_len

    def forward(self, x):
        m = self.model
        if m.first_stage:
            B, S = x.shape
            delta, residual = m.run_layers(m.embed_tokens(x), B, S)
        else:
            tl = x.shape[1]
            B = tl * m.pg.world_size() // self.seq_len
            delta, residual = m.run_layers(x[0], B, self.seq_len, residual=x[1])
        return torch.stack([delta, residual])

    def loss(self, y, labels):
        return self.model.loss_from_hidden(y[0], y[1], labels)


class TPPipelineChunks(nn.Module):
    """The model chunks a rank holds under the interleaved schedule (virtual stages ``s``, ``s +
    pp``, ...) behind the interface of a single ``TPPipelineStage``: ``loss`` belongs to the chunk
    that ends the model, parameter helpers cover all chunks."""

    def __init__(self, chunks):
        super().__init__()
        self.chunks = nn.ModuleList(chunks)

    @property
    def model(self):
        """Callers written for a single stage use ``stage.model``."""
        return self

    @property
    def last_stage(self) -> bool:
        return any(c.model.last_stage for c in self.chunks)

    def loss(self, y, labels):
        return next(c for c in self.chunks if c.model.last_stage).loss(y, labels)

    def sync_replicated_grads(self) -> None:
        for c in self.chunks:
            c.model.sync_replicated_grads()

    def load_full_state_dict(self, sd: dict) -> None:
        for c in self.chunks:
            c.model.load_full_state_dict(sd)

    def full_state_dict(self) -> dict:
        out = {}
        for c in self.chunks:
            out.update(c.model.full_state_dict())
        return out


def build_tp_pp(cfg: LLaMAConfig, world, tp: int, pp: int, seq_len: int, device=None, dtype=torch.bfloat16,
                num_microbatches: int = 8, chunks: int = 1):
    """Lays ``tp * pp`` ranks out as ``pp`` consecutive tensor-parallel groups (stage s = ranks
    ``[s*tp, (s+1)*tp)``) and returns ``(pipeline, stage_module, tp_group)`` for the calling rank.
    ``world``: a ``parallel.World``.  Every rank creates every sub-group (required by the
    process-group rendezvous) and keeps the ones it belongs to.

    ``chunks > 1`` selects the interleaved 1F1B schedule: the layers are cut into ``pp * chunks``
    virtual stages and pipeline rank ``s`` holds stages ``s, s + pp, ...`` (a smaller bubble for
    more, smaller transfers); the returned module is then a ``TPPipelineChunks``."""
    from ..parallel.pipeline import Pipeline, PipelineSchedule, PipelineStage
    rank = world.rank()
    if world.world_size() != tp * pp:
        raise ValueError("world size must be tp * pp")
    my_stage, my_tp = rank // tp, rank % tp
    tp_groups = [world.new_group(list(range(s * tp, (s + 1) * tp))) for s in range(pp)]
    pp_groups = [world.new_group([s * tp + t for s in range(pp)]) for t in range(tp)]
    tp_pg, pp_pg = tp_groups[my_stage], pp_groups[my_tp]
    if chunks > 1:
        n_stages = pp * chunks
        if cfg.num_hidden_layers < n_stages:
            raise ValueError(f"{cfg.num_hidden_layers} layers cannot fill {n_stages} virtual stages")
        per = cfg.num_hidden_layers // n_stages
        mine = {}
        for sid in range(my_stage, n_stages, pp):
            layers = range(sid * per, cfg.num_hidden_layers if sid == n_stages - 1 else (sid + 1) * per)
            model = TPLLaMAForCausalLM(cfg, tp_pg, device=device, dtype=dtype, layers=layers,
                                       first_stage=sid == 0, last_stage=sid == n_stages - 1)
            mine[sid] = TPPipelineStage(model, seq_len)
        stages = [PipelineStage(mine.get(sid), sid, sid % pp) for sid in range(n_stages)]
        pipe = Pipeline(stages, pp_pg, PipelineSchedule.InterleavedOneFOneB, num_microbatches)
        return pipe, TPPipelineChunks([mine[sid] for sid in sorted(mine)]), tp_pg
    per = cfg.num_hidden_layers // pp
    layers = range(my_stage * per, cfg.num_hidden_layers if my_stage == pp - 1 else (my_stage + 1) * per)
    model = TPLLaMAForCausalLM(cfg, tp_pg, device=device, dtype=dtype, layers=layers,
                               first_stage=my_stage == 0, last_stage=my_stage == pp - 1)
    stage = TPPipelineStage(model, seq_len)
    stages = [PipelineStage(stage if s == my_stage else None, s, s) for s in range(pp)]
    pipe = Pipeline(stages, pp_pg, PipelineSchedule.OneFOneBSchedule, num_microbatches)
    return pipe, stage, tp_pg
