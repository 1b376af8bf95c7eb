"""Context (sequence) parallel attention, DeepSpeed-Ulysses style.

Activations are sharded along the sequence: every rank holds ``[B, S/W, H, D]``.  Attention needs
the whole sequence, so q, k and v are exchanged with one all-to-all each into ``[B, S, H/W, D]``
(whole sequence, a slice of the heads), attention runs locally on the flash-attention kernel, and
a fourth all-to-all brings the output back to the sequence sharding.  Every all-to-all moves
``1/W`` of the tensor per peer, so the traffic per rank is independent of ``W``; over NVSwitch
every peer is at full bandwidth.  The exchanges are autograd functions whose backward is the
opposite exchange.

The reference has no sequence or context parallelism (its blockwise attention,
crates/axonml-llm/src/attention.rs:836-943, is single-device); this module is what lets a
sequence longer than one GPU's activation memory train with the same attention kernel.

Requirements: ``S`` sharded contiguously in rank order, ``Hq % W == 0``; K/V heads that do not
divide by ``W`` (grouped-query attention with few KV heads) are repeated up to ``Hq`` first.

``allgather_kv_attention`` is the second form, for grouped-query models whose K/V are small: the
queries stay sharded, K and V are all-gathered along the sequence (backward: reduce-scatter) and
every rank attends from its own queries to the keys up to its last token - the kernels' causal
mask is aligned to the end of the key range, so the slice ``K[:, :(rank + 1) * s]`` is all that
is needed.  No restriction on the head counts; with a causal mask the last rank does the most
work (contiguous sharding, no zigzag).

``ring_attention`` is the third form, for sequences whose K/V do not fit one GPU even once: the
K/V slices travel around the ring (``Backend.sendrecv``), every rank attends from its queries to
the slice it currently holds and merges the partial results with their log-sum-exp.  The block
products are torch expressions (differentiable; the shifts are autograd functions whose backward
shifts the gradient the other way), not the flash kernels, which do not return a differentiable
log-sum-exp."""
from __future__ import annotations

import torch

from ..ops import attention as A
from .process_group import ProcessGroup


def _exchange(pg: ProcessGroup, send: torch.Tensor) -> torch.Tensor:
    recv = torch.empty_like(send)
    pg.backend().all_to_all(send, recv)
    return recv


def _seq_to_heads(x: torch.Tensor, pg: ProcessGroup) -> torch.Tensor:
    """[B, s, H, D] (sequence shard, all heads) -> [B, W*s, H/W, D] (whole sequence, head slice)."""
    W = pg.world_size()
    B, s, H, D = x.shape
    h = H // W
    send = x.reshape(B, s, W, h, D).permute(2, 0, 1, 3, 4).contiguous()      # [W, B, s, h, D]
    recv = _exchange(pg, send)                                                # recv[j]: rank j's tokens
    return recv.permute(1, 0, 2, 3, 4).reshape(B, W * s, h, D)


def _heads_to_seq(x: torch.Tensor, pg: ProcessGroup) -> torch.Tensor:
    """[B, W*s, h, D] -> [B, s, W*h, D]: the inverse exchange."""
    W = pg.world_size()
    B, S, h, D = x.shape
    s = S // W
    send = x.reshape(B, W, s, h, D).permute(1, 0, 2, 3, 4).contiguous()      # [W, B, s, h, D]
    recv = _exchange(pg, send)                                                # recv[j]: head slice j
    return recv.permute(1, 2, 0, 3, 4).reshape(B, s, W * h, D)


class _SeqToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return _seq_to_heads(x, pg)

    @staticmethod
    def backward(ctx, g):
        return _heads_to_seq(g.contiguous(), ctx.pg), None


class _HeadsToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return _heads_to_seq(x, pg)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_heads(g.contiguous(), ctx.pg), None


def shard_sequence(x: torch.Tensor, pg: ProcessGroup, dim: int = 1) -> torch.Tensor:
    """This rank's contiguous slice of ``x`` along ``dim``."""
    W, r = pg.world_size(), pg.rank()
    if x.shape[dim] % W:
        raise ValueError(f"sequence length {x.shape[dim]} is not divisible by the group size {W}")
    return x.chunk(W, dim=dim)[r]


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pg: ProcessGroup, causal: bool = True,
                      scale: float | None = None) -> torch.Tensor:
    """q ``[B, S/W, Hq, D]``, k/v ``[B, S/W, Hkv, D]`` (this rank's tokens) -> ``[B, S/W, Hq, D]``."""
    W = pg.world_size()
    if W == 1:
        return A.sdpa(q, k, v, causal=causal, scale=scale)
    Hq, Hkv = q.shape[2], k.shape[2]
    if Hq % W:
        raise ValueError(f"{Hq} query heads cannot be split over {W} ranks")
    if Hkv % W:
        rep = Hq // Hkv
        k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
    qh, kh, vh = (_SeqToHeads.apply(t, pg) for t in (q, k, v))
    o = A.sdpa(qh, kh, vh, causal=causal, scale=scale)
    return _HeadsToSeq.apply(o.contiguous(), pg)


class _AllGatherSeq(torch.autograd.Function):
    """[B, s, H, D] -> [B, W*s, H, D]; backward sums the gradients of every rank's copy and keeps
    this rank's slice (reduce-scatter)."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        W = pg.world_size()
        xt = x.transpose(0, 1).contiguous()
        full = torch.empty((W * xt.shape[0],) + tuple(xt.shape[1:]), dtype=x.dtype, device=x.device)
        pg.backend().all_gather(xt, full)
        return full.transpose(0, 1)

    @staticmethod
    def backward(ctx, g):
        from .backend import ReduceOp
        W = ctx.pg.world_size()
        gt = g.transpose(0, 1).contiguous()
        mine = torch.empty((gt.shape[0] // W,) + tuple(gt.shape[1:]), dtype=g.dtype, device=g.device)
        ctx.pg.backend().reduce_scatter(gt, mine, ReduceOp.Sum)
        return mine.transpose(0, 1), None


def allgather_kv_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pg: ProcessGroup, causal: bool = True,
                           scale: float | None = None) -> torch.Tensor:
    """q ``[B, S/W, Hq, D]``, k/v ``[B, S/W, Hkv, D]`` (this rank's tokens) -> ``[B, S/W, Hq, D]``."""
    W, r = pg.world_size(), pg.rank()
    if W == 1:
        return A.sdpa(q, k, v, causal=causal, scale=scale)
    s = q.shape[1]
    K, V = _AllGatherSeq.apply(k, pg), _AllGatherSeq.apply(v, pg)
    if causal:
        K, V = K[:, :(r + 1) * s], V[:, :(r + 1) * s]
    return A.sdpa(q, K, V, causal=causal, scale=scale)


class _RingShift(torch.autograd.Function):
    """Every rank sends ``x`` to the next rank and receives the previous rank's; backward sends the
    gradient to the previous rank and receives the next rank's."""

    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        W, r = pg.world_size(), pg.rank()
        out = torch.empty_like(x)
        pg.backend().sendrecv(x.contiguous(), (r + 1) % W, out, (r - 1) % W)
        return out

    @staticmethod
    def backward(ctx, g):
        W, r = ctx.pg.world_size(), ctx.pg.rank()
        out = torch.empty_like(g)
        ctx.pg.backend().sendrecv(g.contiguous(), (r - 1) % W, out, (r + 1) % W)
        return out, None


def _block_attention(q, k, v, scale, diagonal: bool):
    """Partial attention of q [B,s,Hq,D] against one K/V slice -> (o [B,Hq,s,D] fp32, lse [B,Hq,s])."""
    Hq, Hkv = q.shape[2], k.shape[2]
    qf, kf, vf = (t.float().permute(0, 2, 1, 3) for t in (q, k, v))
    if Hkv != Hq:
        kf, vf = kf.repeat_interleave(Hq // Hkv, dim=1), vf.repeat_interleave(Hq // Hkv, dim=1)
    sc = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if diagonal:
        s = sc.shape[-1]
        sc = sc.masked_fill(~torch.ones(s, s, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    lse = torch.logsumexp(sc, dim=-1)
    return torch.matmul(torch.exp(sc - lse.unsqueeze(-1)), vf), lse


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pg: ProcessGroup, causal: bool = True,
                   scale: float | None = None) -> torch.Tensor:
    """q ``[B, S/W, Hq, D]``, k/v ``[B, S/W, Hkv, D]`` (this rank's tokens) -> ``[B, S/W, Hq, D]``."""
    W, r = pg.world_size(), pg.rank()
    if W == 1:
        return A.sdpa(q, k, v, causal=causal, scale=scale)
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    o = lse = None
    kv = torch.stack([k, v])
    for t in range(W):
        src = (r - t) % W                                   # owner of the slice held in this step
        if not causal or src <= r:
            ob, lb = _block_attention(q, kv[0], kv[1], scale, diagonal=causal and src == r)
            if o is None:
                o, lse = ob, lb
            else:
                new = torch.logaddexp(lse, lb)
                o = o * torch.exp(lse - new).unsqueeze(-1) + ob * torch.exp(lb - new).unsqueeze(-1)
                lse = new
        elif o is not None:
            # a slice this rank does not attend to must stay in the graph, or this rank's backward
            # would skip the ring shift its neighbours wait for
            o = o + kv.float().sum() * 0.0
        if t + 1 < W:
            kv = _RingShift.apply(kv, pg)
    return o.permute(0, 2, 1, 3).to(q.dtype)


def attention_fn(form: str):
    """The context-parallel attention function called ``form``: "ulysses", "allgather" or "ring"."""
    fns = {"ulysses": ulysses_attention, "allgather": allgather_kv_attention, "ring": ring_attention}
    if form not in fns:
        raise ValueError(f"unknown context-parallel form {form!r} (one of {sorted(fns)})")
    return fns[form]


class UlyssesAttention(torch.nn.Module):
    """Drop-in attention core for sequence-sharded activations (see module docstring)."""

    def __init__(self, process_group: ProcessGroup, causal: bool = True):
        super().__init__()
        self.pg, self.causal = process_group, causal

    def forward(self, q, k, v, scale: float | None = None):
        return ulysses_attention(q, k, v, self.pg, self.causal, scale)
