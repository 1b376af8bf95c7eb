"""Tensor parallelism (Megatron style) with optional sequence parallelism.

Reference API (crates/axonml-distributed/src/fsdp.rs:414-600): ``ColumnParallelLinear(in, out,
bias, pg, gather_output)`` holds ``weight[out/world, in]``; ``RowParallelLinear(in, out, bias, pg,
input_is_parallel)`` holds ``weight[out, in/world]`` and adds its bias after the reduction.  The
reference stacks gathered outputs on a new leading dim and wraps the weights as constants, so they
never train (fsdp.rs:465-481, :575); here outputs are concatenated on the feature dim and every
collective has the matching backward (all-reduce <-> identity, all-gather <-> reduce-scatter).

With ``sequence_parallel=True`` activations between the two layers of a block are sharded along the
token dim: the column layer all-gathers tokens in front of its GEMM and the row layer
reduce-scatters its output, which is what the fused all-gather->GEMM and GEMM->reduce-scatter
kernels implement in one launch each.
"""
from __future__ import annotations

import torch

from ..nn import init
from ..nn.module import Module, Parameter
from ..ops.linear import linear
from .backend import ReduceOp
from .process_group import ProcessGroup


def _all_reduce(t, pg):
    if pg.world_size() > 1:
        t = t.contiguous()
        pg.backend().all_reduce(t, ReduceOp.Sum)
    return t


def _all_gather_dim(t, pg, dim):
    w = pg.world_size()
    if w == 1:
        return t
    t = t.contiguous()
    out = torch.empty((w,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    pg.backend().all_gather(t, out)
    return torch.cat(list(out.unbind(0)), dim=dim)


def _reduce_scatter_dim0(t, pg):
    w = pg.world_size()
    if w == 1:
        return t
    t = t.contiguous()
    out = torch.empty((t.shape[0] // w,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    pg.backend().reduce_scatter(t, out, ReduceOp.Sum)
    return out


class _CopyToTP(torch.autograd.Function):          # fwd identity, bwd all-reduce
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g.clone(), ctx.pg), None


class _ReduceFromTP(torch.autograd.Function):      # fwd all-reduce, bwd identity
    @staticmethod
    def forward(ctx, x, pg):
        return _all_reduce(x.clone(), pg)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherLastDim(torch.autograd.Function):     # fwd all-gather(features), bwd take own slice
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return _all_gather_dim(x, pg, -1)

    @staticmethod
    def backward(ctx, g):
        w, r = ctx.pg.world_size(), ctx.pg.rank()
        n = g.shape[-1] // w
        return g[..., r * n:(r + 1) * n].contiguous(), None


class _ScatterLastDim(torch.autograd.Function):    # fwd take own slice, bwd all-gather
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        w, r = pg.world_size(), pg.rank()
        n = x.shape[-1] // w
        return x[..., r * n:(r + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.pg, -1), None


class _AllGatherTokens(torch.autograd.Function):   # fwd all-gather(dim 0), bwd reduce-scatter
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return _all_gather_dim(x, pg, 0)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_dim0(g, ctx.pg), None


class _ReduceScatterTokens(torch.autograd.Function):  # fwd reduce-scatter(dim 0), bwd all-gather
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        return _reduce_scatter_dim0(x, pg)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim(g, ctx.pg, 0), None


def copy_to_tensor_parallel(x, pg): return _CopyToTP.apply(x, pg)
def reduce_from_tensor_parallel(x, pg): return _ReduceFromTP.apply(x, pg)
def gather_from_tensor_parallel(x, pg): return _GatherLastDim.apply(x, pg)
def scatter_to_tensor_parallel(x, pg): return _ScatterLastDim.apply(x, pg)
def all_gather_tokens(x, pg): return _AllGatherTokens.apply(x, pg)
def reduce_scatter_tokens(x, pg): return _ReduceScatterTokens.apply(x, pg)


class ColumnParallelLinear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 process_group: ProcessGroup | None = None, gather_output: bool = False,
                 sequence_parallel: bool = False, activation: str | None = None, device=None, dtype=None):
        super().__init__()
        self.pg = process_group or ProcessGroup.mock()
        w = self.pg.world_size()
        if out_features % w:
            raise ValueError("out_features must be divisible by the tensor-parallel size")
        self.in_features, self.out_features, self.local_out = in_features, out_features, out_features // w
        self.gather_output, self.sequence_parallel = gather_output, sequence_parallel
        self.activation = activation or "none"
        self.weight = Parameter(init.kaiming_uniform(self.local_out, in_features).to(device=device, dtype=dtype or torch.float32))
        if bias:
            self.bias = Parameter(torch.zeros(self.local_out, device=device, dtype=dtype or torch.float32))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def new(cls, in_features, out_features, bias, process_group, gather_output=False):
        return cls(in_features, out_features, bias, process_group, gather_output)

    def forward(self, x):
        if self.sequence_parallel:
            from . import fused_gemm
            y = fused_gemm.all_gather_linear(x, self.weight, self.bias, self.activation, self.pg)
        else:
            y = linear(copy_to_tensor_parallel(x, self.pg), self.weight, self.bias, self.activation)
        return gather_from_tensor_parallel(y, self.pg) if self.gather_output else y


class RowParallelLinear(Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 process_group: ProcessGroup | None = None, input_is_parallel: bool = True,
                 sequence_parallel: bool = False, device=None, dtype=None):
        super().__init__()
        self.pg = process_group or ProcessGroup.mock()
        w = self.pg.world_size()
        if in_features % w:
            raise ValueError("in_features must be divisible by the tensor-parallel size")
        self.in_features, self.out_features, self.local_in = in_features, out_features, in_features // w
        self.input_is_parallel, self.sequence_parallel = input_is_parallel, sequence_parallel
        self.weight = Parameter(init.kaiming_uniform(out_features, self.local_in).to(device=device, dtype=dtype or torch.float32))
        if bias:
            self.bias = Parameter(torch.zeros(out_features, device=device, dtype=dtype or torch.float32))
        else:
            self.register_parameter("bias", None)

    @classmethod
    def new(cls, in_features, out_features, bias, process_group, input_is_parallel=True):
        return cls(in_features, out_features, bias, process_group, input_is_parallel)

    def forward(self, x):
        if not self.input_is_parallel:
            x = scatter_to_tensor_parallel(x, self.pg)
        if self.sequence_parallel:
            from . import fused_gemm
            y = fused_gemm.linear_reduce_scatter(x, self.weight, self.pg)
        else:
            y = reduce_from_tensor_parallel(linear(x, self.weight), self.pg)
        if self.bias is not None:       # added once, after the reduction (fsdp.rs:579-590)
            y = y + self.bias.to(y.dtype)
        return y


class VocabParallelEmbedding(Module):
    """Embedding table split along the vocabulary; out-of-range ids contribute zeros and the partial
    results are all-reduced."""

    def __init__(self, num_embeddings: int, embedding_dim: int, process_group: ProcessGroup | None = None,
                 device=None, dtype=None):
        super().__init__()
        self.pg = process_group or ProcessGroup.mock()
        w, r = self.pg.world_size(), self.pg.rank()
        self.per = (num_embeddings + w - 1) // w
        self.lo, self.hi = r * self.per, min((r + 1) * self.per, num_embeddings)
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = Parameter(torch.randn(self.per, embedding_dim).mul_(0.02).to(device=device, dtype=dtype or torch.float32))

    def forward(self, ids):
        from ..ops import misc as Mi
        local = ids - self.lo
        mask = (ids < self.lo) | (ids >= self.hi)
        local = local.masked_fill(mask, -1)           # the gather kernel writes zeros for id < 0
        out = Mi.embedding(local, self.weight)
        return reduce_from_tensor_parallel(out, self.pg)


def _vp_kernel_ok(logits) -> bool:
    from .. import _native as N
    return (logits.is_cuda and N.have_gpu() and logits.dtype in (torch.bfloat16, torch.float32)
            and logits.dim() == 2 and logits.stride(1) == 1)


class _VocabParallelCE(torch.autograd.Function):
    """Mean cross-entropy from a vocabulary slice of the logits.  On a GPU two kernels of
    ``csrc/kernels/softmax_ce.cu`` do the work (per-row max / sum-exp / target logit of the slice,
    then (softmax - onehot) * scale in place of the logits' gradient) around ONE small all-gather of
    the row statistics; elsewhere rows are processed in chunks of torch ops so that the fp32
    temporaries stay small next to the (large) bf16 logits."""

    CHUNK = 4096

    @staticmethod
    def forward(ctx, logits, target, pg, vocab_start, ignore_index, valid_vocab):
        T, V = logits.shape
        dev = logits.device
        n_valid_cols = V if valid_vocab is None else max(0, min(V, valid_vocab - vocab_start))
        ctx.kernel = _vp_kernel_ok(logits)
        if ctx.kernel:
            from .. import _native as N
            local_t = (target - vocab_start).contiguous()
            # targets on another rank get a negative marker; rows to ignore keep ignore_index
            off = -1 if ignore_index != -1 else -2
            local_t = torch.where((local_t >= 0) & (local_t < n_valid_cols), local_t, torch.full_like(local_t, off))
            valid = target != ignore_index
            local_t = torch.where(valid, local_t, torch.full_like(local_t, ignore_index)).contiguous()
            stats = torch.empty(T, 4, dtype=torch.float32, device=dev)
            N.check(N.cuda().ax_vp_ce_stats(1 if logits.dtype == torch.bfloat16 else 0, N.ptr(logits), N.ptr(local_t),
                                            N.ptr(stats), T, n_valid_cols, N.c_int64(logits.stride(0)), N.stream_ptr()),
                    "ax_vp_ce_stats")
            W = pg.world_size()
            if W > 1:
                allst = torch.empty(W, T, 4, dtype=torch.float32, device=dev)
                pg.backend().all_gather(stats, allst)
            else:
                allst = stats.unsqueeze(0)
            m = allst[..., 0].max(dim=0).values
            s = (allst[..., 1] * (allst[..., 0] - m).exp()).sum(0)
            picked = allst[..., 2].sum(0)
            lse = m + s.log()
            count = valid.sum().clamp_min(1).float()
            loss = torch.where(valid, lse - picked, torch.zeros_like(lse)).sum() / count
            ctx.save_for_backward(logits, lse.contiguous(), local_t, count)
            ctx.n_valid_cols, ctx.ignore_index = n_valid_cols, ignore_index
            return loss
        m = torch.empty(T, dtype=torch.float32, device=dev)
        for i in range(0, T, _VocabParallelCE.CHUNK):
            blk = logits[i:i + _VocabParallelCE.CHUNK, :n_valid_cols]
            m[i:i + blk.shape[0]] = blk.max(dim=-1).values.float() if n_valid_cols else float("-inf")
        if pg.world_size() > 1:
            pg.backend().all_reduce(m, ReduceOp.Max)
        s = torch.empty(T, dtype=torch.float32, device=dev)
        picked = torch.zeros(T, dtype=torch.float32, device=dev)
        local_t = target - vocab_start
        mine = (local_t >= 0) & (local_t < n_valid_cols)
        for i in range(0, T, _VocabParallelCE.CHUNK):
            blk = logits[i:i + _VocabParallelCE.CHUNK, :n_valid_cols].float()
            j = i + blk.shape[0]
            s[i:j] = (blk - m[i:j, None]).exp().sum(-1)
            idx = local_t[i:j].clamp(0, max(n_valid_cols - 1, 0)).unsqueeze(-1)
            if n_valid_cols:
                picked[i:j] = torch.where(mine[i:j], torch.gather(blk, -1, idx).squeeze(-1), picked[i:j])
        both = torch.stack([s, picked])
        if pg.world_size() > 1:
            pg.backend().all_reduce(both, ReduceOp.Sum)
        s, picked = both[0], both[1]
        lse = m + s.log()
        valid = target != ignore_index
        count = valid.sum().clamp_min(1).float()
        loss = torch.where(valid, lse - picked, torch.zeros_like(lse)).sum() / count
        ctx.save_for_backward(logits, lse, local_t, mine & valid, valid, count)
        ctx.n_valid_cols = n_valid_cols
        return loss

    @staticmethod
    def backward(ctx, g):
        if ctx.kernel:
            from .. import _native as N
            logits, lse, local_t, count = ctx.saved_tensors
            T, V = logits.shape
            grad = torch.empty_like(logits)
            scale = (g / count).float().reshape(1).contiguous()
            N.check(N.cuda().ax_vp_ce_bwd(1 if logits.dtype == torch.bfloat16 else 0, N.ptr(logits), N.ptr(local_t),
                                          N.ptr(lse), N.ptr(scale), N.c_float(1.0), N.ptr(grad), T, ctx.n_valid_cols, V,
                                          N.c_int64(logits.stride(0)), N.c_int64(ctx.ignore_index), N.stream_ptr()),
                    "ax_vp_ce_bwd")
            return grad, None, None, None, None, None
        logits, lse, local_t, hit, valid, count = ctx.saved_tensors
        T, V = logits.shape
        nv = ctx.n_valid_cols
        grad = torch.zeros_like(logits)
        scale = (g / count).float()
        for i in range(0, T, _VocabParallelCE.CHUNK):
            blk = logits[i:i + _VocabParallelCE.CHUNK, :nv].float()
            j = i + blk.shape[0]
            p = (blk - lse[i:j, None]).exp()
            rows = torch.nonzero(hit[i:j]).squeeze(-1)
            if rows.numel():
                p[rows, local_t[i:j][rows]] -= 1.0
            p *= (valid[i:j].float() * scale)[:, None]
            grad[i:j, :nv] = p.to(logits.dtype)
        return grad, None, None, None, None, None


def vocab_parallel_cross_entropy(local_logits: torch.Tensor, target: torch.Tensor, pg: ProcessGroup,
                                 vocab_start: int, ignore_index: int = -100,
                                 valid_vocab: int | None = None) -> torch.Tensor:
    """Mean cross-entropy over logits whose class dim is split across ranks: the row maxima and
    the sum-exp / target-logit pairs are combined with two small all-reduces, so the full logits
    are never gathered.  ``valid_vocab``: size of the real vocabulary when the split one was
    padded (columns beyond it are ignored)."""
    return _VocabParallelCE.apply(local_logits, target, pg, vocab_start, ignore_index, valid_vocab)
