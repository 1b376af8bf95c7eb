"""Sparse COO / CSR tensors (crates/axonml-tensor/src/sparse.rs:33-534): construction from dense,
``coalesce``, ``to_dense``, ``matvec``, ``matmul_dense``, format conversion."""
from __future__ import annotations

import torch


class SparseCOO:
    def __init__(self, indices: torch.Tensor, values: torch.Tensor, shape):
        self.indices, self.values, self.shape = indices.long(), values, tuple(shape)

    @classmethod
    def from_dense(cls, dense: torch.Tensor, threshold: float = 0.0):
        mask = dense.abs() > threshold
        idx = mask.nonzero().t().contiguous()
        return cls(idx, dense[mask], dense.shape)

    @classmethod
    def from_triplets(cls, rows, cols, values, shape):
        return cls(torch.tensor([rows, cols]), torch.as_tensor(values, dtype=torch.float32), shape)

    def nnz(self) -> int: return self.values.numel()
    def density(self) -> float:
        n = 1
        for s in self.shape:
            n *= s
        return self.nnz() / max(n, 1)

    def coalesce(self) -> "SparseCOO":
        t = torch.sparse_coo_tensor(self.indices, self.values, self.shape).coalesce()
        return SparseCOO(t.indices(), t.values(), self.shape)

    def to_dense(self) -> torch.Tensor:
        return torch.sparse_coo_tensor(self.indices, self.values, self.shape).to_dense()

    def to_csr(self) -> "SparseCSR":
        c = self.coalesce()
        rows, cols = c.indices[0], c.indices[1]
        crow = torch.zeros(self.shape[0] + 1, dtype=torch.long)
        crow[1:] = torch.bincount(rows, minlength=self.shape[0]).cumsum(0)
        return SparseCSR(crow, cols, c.values, self.shape)

    def matvec(self, x: torch.Tensor) -> torch.Tensor: return self.to_csr().matvec(x)
    def matmul_dense(self, b: torch.Tensor) -> torch.Tensor: return self.to_csr().matmul_dense(b)
    def transpose(self) -> "SparseCOO":
        return SparseCOO(self.indices.flip(0), self.values, (self.shape[1], self.shape[0]))


class SparseCSR:
    def __init__(self, crow: torch.Tensor, cols: torch.Tensor, values: torch.Tensor, shape):
        self.crow, self.cols, self.values, self.shape = crow.long(), cols.long(), values, tuple(shape)

    @classmethod
    def from_dense(cls, dense: torch.Tensor, threshold: float = 0.0):
        return SparseCOO.from_dense(dense, threshold).to_csr()

    def nnz(self) -> int: return self.values.numel()

    def _t(self):
        return torch.sparse_csr_tensor(self.crow, self.cols, self.values, self.shape)

    def to_dense(self) -> torch.Tensor: return self._t().to_dense()
    def matvec(self, x: torch.Tensor) -> torch.Tensor: return (self._t() @ x.reshape(-1, 1)).reshape(-1)
    def matmul_dense(self, b: torch.Tensor) -> torch.Tensor: return self._t() @ b

    def to_coo(self) -> SparseCOO:
        rows = torch.repeat_interleave(torch.arange(self.shape[0]), self.crow[1:] - self.crow[:-1])
        return SparseCOO(torch.stack([rows, self.cols]), self.values, self.shape)

    def row(self, i: int):
        a, b = int(self.crow[i]), int(self.crow[i + 1])
        return self.cols[a:b], self.values[a:b]
