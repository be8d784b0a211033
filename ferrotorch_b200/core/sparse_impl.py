"""Sparse containers with their own storage (index and value tensors) and their own algorithms: coalescing by sort + segment sum,
COO <-> CSR <-> CSC conversion by counting and stable sorting, sparse x dense products by gather + ``index_add``, transposes and sums.
Everything is expressed on dense tensor operations, so it runs on any device and is differentiable with respect to the stored values and
the dense operand.

Reference parity: ferrotorch-core/src/sparse.rs:99-2192 (SparseTensor :99, CooTensor :771, CsrTensor :1075, CscTensor :1692 and their
conversions, ``spmm``, ``add``, ``coalesce``, ``t``).
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch

from ..errors import InvalidArgument, ShapeMismatch


def _segment_starts(sorted_keys: torch.Tensor) -> torch.Tensor:
    """True at the first element of every run of equal keys."""
    first = torch.ones_like(sorted_keys, dtype=torch.bool)
    if sorted_keys.numel() > 1:
        first[1:] = sorted_keys[1:] != sorted_keys[:-1]
    return first


def _ptrs(sorted_major: torch.Tensor, n: int) -> torch.Tensor:
    """Compressed pointers [n + 1] of a sorted index vector: ptr[i] = number of entries with index < i."""
    counts = torch.zeros(n, dtype=torch.int64, device=sorted_major.device)
    if sorted_major.numel():
        counts.index_add_(0, sorted_major, torch.ones_like(sorted_major))
    return torch.cat([counts.new_zeros(1), counts.cumsum(0)])


def _expand_ptrs(ptrs: torch.Tensor, nnz: int) -> torch.Tensor:
    """Inverse of ``_ptrs``: the major index of every stored entry."""
    n = ptrs.numel() - 1
    return torch.repeat_interleave(torch.arange(n, device=ptrs.device), ptrs[1:] - ptrs[:-1], output_size=nnz)


class SparseTensor:
    """COO tensor of any rank: ``indices`` [ndim, nnz] (int64) and ``values`` [nnz]. Duplicate coordinates are allowed until ``coalesce``
    sums them; the constructor coalesces by default, as the two-dimensional ``CooTensor`` alias always has."""

    def __init__(self, indices: torch.Tensor, values: torch.Tensor, shape: Sequence[int], coalesce: bool = True):
        indices = torch.as_tensor(indices, dtype=torch.int64)
        values = torch.as_tensor(values)
        shape = tuple(int(s) for s in shape)
        if indices.dim() != 2 or indices.shape[0] != len(shape):
            raise ShapeMismatch(f"sparse indices must be [ndim = {len(shape)}, nnz], got {tuple(indices.shape)}")
        if values.dim() != 1 or values.shape[0] != indices.shape[1]:
            raise ShapeMismatch(f"sparse values must be [nnz = {indices.shape[1]}], got {tuple(values.shape)}")
        if indices.numel():
            top = indices.amax(1)
            if bool((indices < 0).any()) or any(int(t) >= s for t, s in zip(top, shape)):
                raise InvalidArgument("sparse index out of range")
        self._indices, self._values, self._shape, self._coalesced = indices.to(values.device), values, shape, False
        if coalesce:
            c = self.coalesce()
            self._indices, self._values, self._coalesced = c._indices, c._values, True

    # ---- construction / views
    @classmethod
    def _raw(cls, indices, values, shape, coalesced):
        obj = cls.__new__(cls)
        obj._indices, obj._values, obj._shape, obj._coalesced = indices, values, tuple(shape), coalesced
        return obj

    @classmethod
    def from_dense(cls, d: torch.Tensor, threshold: float = 0.0) -> "SparseTensor":
        """Keeps the entries whose magnitude exceeds ``threshold`` (row-major order, hence coalesced)."""
        keep = d.abs() > threshold
        idx = keep.nonzero().t().contiguous()
        return cls._raw(idx, d[keep], d.shape, True)

    def indices(self) -> torch.Tensor:
        return self._indices

    def values(self) -> torch.Tensor:
        return self._values

    def shape(self) -> Tuple[int, ...]:
        return self._shape

    def ndim(self) -> int:
        return len(self._shape)

    def nnz(self) -> int:
        return int(self._values.shape[0])

    def is_coalesced(self) -> bool:
        return self._coalesced

    def nrows(self) -> int:
        return self._shape[0]

    def ncols(self) -> int:
        return self._shape[-1]

    def row_indices(self) -> torch.Tensor:
        return self._indices[0]

    def col_indices(self) -> torch.Tensor:
        return self._indices[-1]

    def to_torch(self) -> torch.Tensor:
        """The same data as a sparse tensor of the substrate (for interoperation)."""
        return torch.sparse_coo_tensor(self._indices, self._values, self._shape, is_coalesced=self._coalesced)

    # ---- algorithms
    def _linear(self) -> torch.Tensor:
        lin = torch.zeros(self.nnz(), dtype=torch.int64, device=self._indices.device)
        for d, s in enumerate(self._shape):
            lin = lin * s + self._indices[d]
        return lin

    def coalesce(self) -> "SparseTensor":
        """Sorted coordinates (row-major), duplicates summed."""
        if self._coalesced:
            return self
        if self.nnz() == 0:
            return self._raw(self._indices, self._values, self._shape, True)
        lin = self._linear()
        order = torch.argsort(lin, stable=True)
        lin_s = lin[order]
        first = _segment_starts(lin_s)
        seg = first.cumsum(0) - 1
        vals = torch.zeros(int(seg[-1]) + 1, dtype=self._values.dtype, device=self._values.device).index_add(0, seg, self._values[order])
        return self._raw(self._indices[:, order][:, first], vals, self._shape, True)

    def to_dense(self) -> torch.Tensor:
        out = torch.zeros(self._shape, dtype=self._values.dtype, device=self._values.device)
        if self.nnz():
            out = out.reshape(-1).index_add(0, self._linear(), self._values).reshape(self._shape)
        return out

    def to_dense_on(self, device) -> torch.Tensor:
        return self.to(device).to_dense()

    def to(self, device) -> "SparseTensor":
        return self._raw(self._indices.to(device), self._values.to(device), self._shape, self._coalesced)

    def spmm(self, dense: torch.Tensor) -> torch.Tensor:
        """[m, k] sparse times [k, n] (or [k]) dense: each stored entry scales a gathered row of the dense operand, rows are summed by index."""
        if self.ndim() != 2:
            raise InvalidArgument("spmm needs a two-dimensional sparse tensor")
        vec = dense.dim() == 1
        dm = dense.unsqueeze(-1) if vec else dense
        if dm.dim() != 2 or dm.shape[0] != self._shape[1]:
            raise ShapeMismatch(f"spmm: {self._shape} x {tuple(dense.shape)}")
        dt = torch.promote_types(self._values.dtype, dm.dtype)
        contrib = self._values.to(dt).unsqueeze(-1) * dm.to(dt).index_select(0, self._indices[1])
        out = torch.zeros(self._shape[0], dm.shape[1], dtype=dt, device=dm.device).index_add(0, self._indices[0], contrib)
        return out.squeeze(-1) if vec else out

    matmul = spmm

    def mul_scalar(self, s: float) -> "SparseTensor":
        return self._raw(self._indices, self._values * s, self._shape, self._coalesced)

    def add(self, other: "SparseTensor") -> "SparseTensor":
        if self._shape != other._shape:
            raise ShapeMismatch(f"sparse add: {self._shape} and {other._shape}")
        dt = torch.promote_types(self._values.dtype, other._values.dtype)
        both = self._raw(torch.cat([self._indices, other._indices.to(self._indices.device)], 1),
                         torch.cat([self._values.to(dt), other._values.to(dt).to(self._values.device)]), self._shape, False)
        return both.coalesce()

    def t(self) -> "SparseTensor":
        """Two-dimensional transpose (coalesced, so the result is sorted for its own row-major order)."""
        if self.ndim() != 2:
            raise InvalidArgument("t() needs a two-dimensional sparse tensor")
        return self._raw(self._indices.flip(0), self._values, (self._shape[1], self._shape[0]), False).coalesce()

    transpose = t

    # ---- conversions
    def to_csr(self) -> "CsrTensor":
        return CsrTensor.from_coo(self)

    def to_csc(self) -> "CscTensor":
        return CscTensor.from_csr(self.to_csr())

    @classmethod
    def from_csr(cls, csr: "CsrTensor") -> "SparseTensor":
        rows = _expand_ptrs(csr._ptrs, csr.nnz())
        return cls._raw(torch.stack([rows, csr._minor]), csr._values, csr._shape, True)

    def __repr__(self):
        return f"{type(self).__name__}(shape={self._shape}, nnz={self.nnz()}, dtype={self._values.dtype})"


CooTensor = SparseTensor


class _Compressed:
    """Shared body of CSR and CSC: ``ptrs`` [major + 1], ``minor`` [nnz] sorted within each major slice, ``values`` [nnz]."""
    _major_is_row = True

    def __init__(self, ptrs, minor=None, values=None, shape=None):
        if minor is None:                                   # a compressed sparse tensor of the substrate
            t = ptrs
            if self._major_is_row:
                ptrs, minor, values = t.crow_indices(), t.col_indices(), t.values()
            else:
                ptrs, minor, values = t.ccol_indices(), t.row_indices(), t.values()
            shape = tuple(t.shape)
        ptrs, minor = torch.as_tensor(ptrs, dtype=torch.int64), torch.as_tensor(minor, dtype=torch.int64)
        values = torch.as_tensor(values)
        shape = tuple(int(s) for s in shape)
        n_major = shape[0] if self._major_is_row else shape[1]
        n_minor = shape[1] if self._major_is_row else shape[0]
        if len(shape) != 2 or ptrs.shape != (n_major + 1,) or minor.shape != values.shape or minor.dim() != 1:
            raise ShapeMismatch("compressed sparse tensor: pointer / index / value shapes do not fit the matrix shape")
        if int(ptrs[0]) != 0 or int(ptrs[-1]) != minor.shape[0] or bool((ptrs[1:] < ptrs[:-1]).any()):
            raise InvalidArgument("compressed sparse tensor: pointers must start at 0, end at nnz and never decrease")
        if minor.numel() and (int(minor.min()) < 0 or int(minor.max()) >= n_minor):
            raise InvalidArgument("compressed sparse tensor: index out of range")
        self._ptrs, self._minor, self._values, self._shape = ptrs, minor, values, shape

    def nnz(self) -> int:
        return int(self._values.shape[0])

    def nrows(self) -> int:
        return self._shape[0]

    def ncols(self) -> int:
        return self._shape[1]

    def shape(self) -> Tuple[int, int]:
        return self._shape

    def values(self) -> torch.Tensor:
        return self._values

    def _coords(self) -> Tuple[torch.Tensor, torch.Tensor]:
        major = _expand_ptrs(self._ptrs, self.nnz())
        return (major, self._minor) if self._major_is_row else (self._minor, major)

    def to_dense(self) -> torch.Tensor:
        rows, cols = self._coords()
        out = torch.zeros(self._shape[0] * self._shape[1], dtype=self._values.dtype, device=self._values.device)
        return out.index_add(0, rows * self._shape[1] + cols, self._values).reshape(self._shape)

    def to_dense_on(self, device) -> torch.Tensor:
        return self.to_dense().to(device)

    def matmul(self, dense: torch.Tensor) -> torch.Tensor:
        rows, cols = self._coords()
        return SparseTensor._raw(torch.stack([rows, cols]), self._values, self._shape, False).spmm(dense)

    def __repr__(self):
        return f"{type(self).__name__}(shape={self._shape}, nnz={self.nnz()}, dtype={self._values.dtype})"


class CsrTensor(_Compressed):
    _major_is_row = True

    @classmethod
    def from_coo(cls, coo: SparseTensor) -> "CsrTensor":
        if coo.ndim() != 2:
            raise InvalidArgument("CSR needs a two-dimensional tensor")
        c = coo.coalesce()
        return cls(_ptrs(c._indices[0], c._shape[0]), c._indices[1], c._values, c._shape)

    @classmethod
    def from_dense(cls, d: torch.Tensor, threshold: float = 0.0) -> "CsrTensor":
        return cls.from_coo(SparseTensor.from_dense(d, threshold))

    def crow_indices(self) -> torch.Tensor:
        return self._ptrs

    row_ptrs = crow_indices

    def col_indices(self) -> torch.Tensor:
        return self._minor

    def to_coo(self) -> SparseTensor:
        return SparseTensor.from_csr(self)

    def to_csc(self) -> "CscTensor":
        return CscTensor.from_csr(self)

    def to_torch(self) -> torch.Tensor:
        return torch.sparse_csr_tensor(self._ptrs, self._minor, self._values, self._shape)


class CscTensor(_Compressed):
    _major_is_row = False

    @classmethod
    def from_csr(cls, csr: CsrTensor) -> "CscTensor":
        rows = _expand_ptrs(csr._ptrs, csr.nnz())
        order = torch.argsort(csr._minor, stable=True)      # by column; the stable sort keeps the rows ascending inside a column
        return cls(_ptrs(csr._minor[order], csr._shape[1]), rows[order], csr._values[order], csr._shape)

    @classmethod
    def from_dense(cls, d: torch.Tensor, threshold: float = 0.0) -> "CscTensor":
        return cls.from_csr(CsrTensor.from_dense(d, threshold))

    def ccol_indices(self) -> torch.Tensor:
        return self._ptrs

    col_ptrs = ccol_indices

    def row_indices(self) -> torch.Tensor:
        return self._minor

    def to_csr(self) -> CsrTensor:
        cols = _expand_ptrs(self._ptrs, self.nnz())
        order = torch.argsort(self._minor, stable=True)
        return CsrTensor(_ptrs(self._minor[order], self._shape[0]), cols[order], self._values[order], self._shape)

    def to_torch(self) -> torch.Tensor:
        return torch.sparse_csc_tensor(self._ptrs, self._minor, self._values, self._shape)
