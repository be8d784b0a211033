"""Sparse containers with own storage: coalescing, conversions between COO / CSR / CSC, products with dense operands, sums, transposes and
gradients, against dense algebra and the substrate's sparse tensors."""
import pytest
import torch

from ferrotorch_b200 import core as C


def _rand_sparse(m, n, density=0.3, seed=0, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(m, n, generator=g, dtype=dtype) * (torch.rand(m, n, generator=g) < density)


def test_coalescing_sums_duplicates_and_sorts_row_major():
    idx = torch.tensor([[1, 0, 1, 0, 2], [2, 1, 2, 1, 0]])
    s = C.SparseTensor(idx, torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0]), (3, 3))
    assert s.is_coalesced() and s.nnz() == 3
    assert s.indices().tolist() == [[0, 1, 2], [1, 2, 0]] and s.values().tolist() == [6.0, 4.0, 5.0]
    raw = C.SparseTensor(idx, torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0]), (3, 3), coalesce=False)
    assert not raw.is_coalesced() and raw.nnz() == 5 and torch.equal(raw.to_dense(), s.to_dense())
    ref = torch.sparse_coo_tensor(idx, torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0]), (3, 3)).coalesce()
    assert torch.equal(s.indices(), ref.indices()) and torch.equal(s.values(), ref.values())
    assert torch.equal(s.to_torch().to_dense(), ref.to_dense())
    empty = C.SparseTensor(torch.zeros(2, 0, dtype=torch.long), torch.zeros(0), (4, 5))
    assert empty.nnz() == 0 and torch.equal(empty.to_dense(), torch.zeros(4, 5)) and empty.to_csr().crow_indices().tolist() == [0] * 5
    t3 = C.SparseTensor(torch.tensor([[0, 1, 0], [1, 0, 1], [2, 2, 2]]), torch.tensor([1.0, 2.0, 3.0]), (2, 2, 3))
    assert t3.ndim() == 3 and t3.nnz() == 2 and float(t3.to_dense()[0, 1, 2]) == 4.0
    for bad in (lambda: C.SparseTensor(torch.tensor([[0], [5]]), torch.ones(1), (2, 3)), lambda: C.SparseTensor(torch.tensor([[0, 1]]), torch.ones(2), (2, 3)),
                lambda: C.SparseTensor(torch.tensor([[0], [1]]), torch.ones(2), (2, 3)), lambda: t3.spmm(torch.ones(3, 2)), lambda: t3.t()):
        with pytest.raises(Exception):
            bad()


@pytest.mark.parametrize("m,n", [(5, 6), (1, 7), (8, 1), (12, 12)])
def test_conversions_products_sums_and_transposes_match_dense_algebra(m, n):
    d = _rand_sparse(m, n, seed=m * n)
    rhs, vec = torch.randn(n, 3, dtype=torch.float64), torch.randn(n, dtype=torch.float64)
    coo = C.SparseTensor.from_dense(d)
    assert coo.nnz() == int((d != 0).sum()) and torch.equal(coo.to_dense(), d) and (coo.nrows(), coo.ncols()) == (m, n)
    assert torch.allclose(coo.spmm(rhs), d @ rhs) and torch.allclose(coo.matmul(vec), d @ vec)
    csr, ref = coo.to_csr(), d.to_sparse_csr()
    assert torch.equal(csr.crow_indices(), ref.crow_indices()) and torch.equal(csr.col_indices(), ref.col_indices()) and torch.equal(csr.values(), ref.values())
    assert torch.equal(csr.to_dense(), d) and torch.allclose(csr.matmul(rhs), d @ rhs) and torch.equal(csr.to_torch().to_dense(), d)
    csc, refc = csr.to_csc(), d.to_sparse_csc()
    assert torch.equal(csc.ccol_indices(), refc.ccol_indices()) and torch.equal(csc.row_indices(), refc.row_indices()) and torch.equal(csc.values(), refc.values())
    assert torch.equal(csc.to_dense(), d) and torch.allclose(csc.matmul(rhs), d @ rhs)
    back = csc.to_csr()
    assert torch.equal(back.crow_indices(), csr.crow_indices()) and torch.equal(back.col_indices(), csr.col_indices()) and torch.equal(back.values(), csr.values())
    assert torch.equal(C.SparseTensor.from_csr(csr).indices(), coo.indices()) and torch.equal(csr.to_coo().to_dense(), d)
    assert torch.equal(C.CsrTensor(ref).to_dense(), d) and torch.equal(C.CscTensor(refc).to_dense(), d)        # from the substrate's compressed tensors
    other = C.SparseTensor.from_dense(_rand_sparse(m, n, seed=99))
    assert torch.allclose(coo.add(other).to_dense(), d + other.to_dense()) and coo.add(other).is_coalesced()
    assert torch.equal(coo.t().to_dense(), d.t()) and coo.t().is_coalesced() and torch.equal(coo.mul_scalar(-2.0).to_dense(), -2.0 * d)
    assert torch.equal(C.SparseTensor.from_dense(d, threshold=0.5).to_dense(), torch.where(d.abs() > 0.5, d, torch.zeros_like(d)))
    assert torch.equal(coo.to_dense_on("cpu"), d)
    with pytest.raises(Exception):
        coo.add(C.SparseTensor.from_dense(torch.ones(m + 1, n)))


def test_products_are_differentiable_in_values_and_dense_operand():
    d = _rand_sparse(6, 5, seed=3)
    coo = C.SparseTensor.from_dense(d)
    vals = coo.values().clone().requires_grad_()
    rhs = torch.randn(5, 4, dtype=torch.float64, requires_grad=True)
    w = torch.randn(6, 4, dtype=torch.float64)
    out = C.SparseTensor(coo.indices(), vals, (6, 5), coalesce=False).spmm(rhs)
    gv, gr = torch.autograd.grad((out * w).sum(), (vals, rhs))
    dd = d.clone().requires_grad_()
    rr = rhs.detach().clone().requires_grad_()
    gd, gr2 = torch.autograd.grad(((dd @ rr) * w).sum(), (dd, rr))
    assert torch.allclose(gr, gr2) and torch.allclose(gv, gd[d != 0])
    with pytest.raises(Exception):
        C.CsrTensor(torch.tensor([0, 2, 1]), torch.tensor([0, 1]), torch.ones(2), (2, 2))
    with pytest.raises(Exception):
        C.CsrTensor(torch.tensor([0, 1, 2]), torch.tensor([0, 5]), torch.ones(2), (2, 2))
