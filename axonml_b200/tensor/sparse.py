"""Sparse COO / CSR tensors (crates/axonml-tensor/src/sparse.rs:33-534): construction from dense,
``coalesce``, ``to_dense``, ``matvec``, ``matmul_dense``, format conversion."""
from __future__ import annotations

import enum

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

    @classmethod
    def from_coo_2d(cls, rows, cols, values, shape):
        """Matrix from parallel row / column / value lists (sparse.rs ``from_coo_2d``)."""
        return cls.from_triplets(rows, cols, values, shape)

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
    def nrows(self) -> int: return self.shape[0]
    def ncols(self) -> int: return self.shape[1]

    def density(self) -> float:
        n = self.shape[0] * self.shape[1]
        return self.nnz() / n if n else 0.0

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


class SparseFormat(enum.Enum):
    """Storage layouts a sparse tensor can take (sparse.rs:33-40)."""
    COO = "coo"
    CSR = "csr"
    CSC = "csc"


class SparseTensor:
    """Either layout behind one interface (sparse.rs:399-534): built from coordinates, a dense
    tensor, an identity or a diagonal; ``matvec`` / ``matmul`` always run on the CSR form."""

    def __init__(self, inner):
        if not isinstance(inner, (SparseCOO, SparseCSR)):
            raise TypeError("SparseTensor wraps a SparseCOO or a SparseCSR")
        self.inner = inner

    @classmethod
    def from_coo(cls, indices, values, shape):
        """``indices`` = one list of positions per dimension (row list, column list)."""
        idx = torch.as_tensor(indices, dtype=torch.long).reshape(len(indices), -1)
        return cls(SparseCOO(idx, torch.as_tensor(values, dtype=torch.float32), tuple(shape)))

    @classmethod
    def from_coords(cls, coords, values, shape):
        """``coords`` = (row, column) pairs."""
        rows = [int(r) for r, _ in coords]
        cols = [int(c) for _, c in coords]
        return cls(SparseCOO.from_triplets(rows, cols, values, tuple(shape)))

    @classmethod
    def from_dense(cls, tensor: torch.Tensor, threshold: float = 0.0):
        return cls(SparseCOO.from_dense(tensor, threshold))

    @classmethod
    def eye(cls, n: int):
        r = list(range(n))
        return cls(SparseCOO.from_triplets(r, r, [1.0] * n, (n, n)))

    @classmethod
    def diag(cls, values):
        v = [float(x) for x in values]
        r = list(range(len(v)))
        return cls(SparseCOO.from_triplets(r, r, v, (len(v), len(v))))

    def format(self) -> SparseFormat:
        return SparseFormat.COO if isinstance(self.inner, SparseCOO) else SparseFormat.CSR

    def nnz(self) -> int: return self.inner.nnz()
    def shape(self) -> tuple: return tuple(self.inner.shape)

    def density(self) -> float:
        n = 1
        for s in self.inner.shape:
            n *= s
        return self.nnz() / n if n else 0.0

    def to_dense(self) -> torch.Tensor: return self.inner.to_dense()
    def to_csr(self) -> SparseCSR: return self.inner if isinstance(self.inner, SparseCSR) else self.inner.to_csr()
    def to_coo(self) -> SparseCOO: return self.inner if isinstance(self.inner, SparseCOO) else self.inner.to_coo()
    def as_format(self, fmt: SparseFormat) -> "SparseTensor":
        if fmt is SparseFormat.CSC:
            raise NotImplementedError("CSC is a declared format without a container, as in the reference")
        return SparseTensor(self.to_coo() if fmt is SparseFormat.COO else self.to_csr())

    def matvec(self, x) -> torch.Tensor:
        return self.to_csr().matvec(torch.as_tensor(x, dtype=torch.float32))

    def matmul(self, dense: torch.Tensor) -> torch.Tensor:
        return self.to_csr().matmul_dense(dense)

    def mul_scalar(self, scalar: float) -> "SparseTensor":
        i = self.inner
        if isinstance(i, SparseCOO):
            return SparseTensor(SparseCOO(i.indices, i.values * scalar, i.shape))
        return SparseTensor(SparseCSR(i.crow, i.cols, i.values * scalar, i.shape))
