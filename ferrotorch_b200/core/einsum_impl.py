"""Einstein summation written out: parse the equation, take diagonals of repeated subscripts, sum subscripts that occur in one operand
only, then contract the operands pairwise as batched matrix products (permute -> reshape -> ``bmm`` -> reshape).

Reference parity: ferrotorch-core/src/einsum.rs:1517 (``einsum``) and :1543 (``einsum_differentiable``): explicit and implicit output,
ellipsis, repeated subscripts, any number of operands. Gradients come from the differentiable primitives it is composed of.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

from ..errors import InvalidArgument

_ELL = "…"                                  # stands for one broadcast dimension of an ellipsis after expansion (upper-case letters are used up)


def _parse(equation: str, operands: Sequence[torch.Tensor]) -> Tuple[List[List[str]], List[str]]:
    eq = equation.replace(" ", "")
    lhs, arrow, rhs = eq.partition("->")
    terms = lhs.split(",")
    if len(terms) != len(operands):
        raise InvalidArgument(f"einsum: {len(terms)} subscript lists for {len(operands)} operands")
    n_ell = 0
    for term, op in zip(terms, operands):
        if term.count("...") > 1 or ("." in term.replace("...", "")):
            raise InvalidArgument(f"einsum: malformed ellipsis in '{term}'")
        named = len(term.replace("...", ""))
        if "..." in term:
            if op.dim() < named:
                raise InvalidArgument(f"einsum: operand has {op.dim()} dims, subscripts '{term}' name {named}")
            n_ell = max(n_ell, op.dim() - named)
        elif op.dim() != named:
            raise InvalidArgument(f"einsum: operand has {op.dim()} dims, subscripts '{term}' name {named}")
    ell = [f"{_ELL}{k}" for k in range(n_ell)]
    ins: List[List[str]] = []
    for term, op in zip(terms, operands):
        if "..." in term:
            a, _, b = term.partition("...")
            k = op.dim() - len(a) - len(b)
            ins.append(list(a) + ell[n_ell - k:] + list(b))
        else:
            ins.append(list(term))
    for sub in ins:
        for c in sub:
            if len(c) == 1 and not c.isalpha():
                raise InvalidArgument(f"einsum: invalid subscript '{c}'")
    if arrow:
        if "..." in rhs:
            a, _, b = rhs.partition("...")
            out = list(a) + ell + list(b)
        else:
            out = list(rhs)
        if len(set(out)) != len(out):
            raise InvalidArgument("einsum: a subscript appears twice in the output")
        seen = {c for sub in ins for c in sub}
        for c in out:
            if c not in seen:
                raise InvalidArgument(f"einsum: output subscript '{c}' does not appear in an input")
    else:
        counts: Dict[str, int] = {}
        for sub in ins:
            for c in sub:
                counts[c] = counts.get(c, 0) + 1
        out = ell + sorted(c for c, k in counts.items() if k == 1 and not c.startswith(_ELL))
    return ins, out


def _diagonalise(t: torch.Tensor, sub: List[str]) -> Tuple[torch.Tensor, List[str]]:
    """Repeated subscripts within one operand select its diagonal along those dims."""
    while len(set(sub)) != len(sub):
        c = next(c for c in sub if sub.count(c) > 1)
        i = sub.index(c)
        j = sub.index(c, i + 1)
        if t.shape[i] != t.shape[j]:
            raise InvalidArgument(f"einsum: subscript '{c}' has sizes {t.shape[i]} and {t.shape[j]} in one operand")
        t = torch.diagonal(t, dim1=i, dim2=j)                # the diagonal becomes the last dim
        sub = [s for k, s in enumerate(sub) if k not in (i, j)] + [c]
    return t, sub


def _contract(a: torch.Tensor, sa: List[str], b: torch.Tensor, sb: List[str], keep: set) -> Tuple[torch.Tensor, List[str]]:
    """One pairwise contraction. Subscripts in both and in ``keep`` are batch dims, in both and not kept are summed, the rest are free."""
    sizes: Dict[str, int] = {}
    for t, s in ((a, sa), (b, sb)):
        for c, n in zip(s, t.shape):
            if sizes.get(c, n) != n and 1 not in (sizes.get(c, n), n):
                raise InvalidArgument(f"einsum: subscript '{c}' has sizes {sizes[c]} and {n}")
            sizes[c] = max(sizes.get(c, 1), n)
    a = a.expand([sizes[c] for c in sa])
    b = b.expand([sizes[c] for c in sb])
    batch = [c for c in sa if c in sb and c in keep]
    summed = [c for c in sa if c in sb and c not in keep]
    free_a = [c for c in sa if c not in sb]
    free_b = [c for c in sb if c not in sa]

    def prod(cs):
        n = 1
        for c in cs:
            n *= sizes[c]
        return n
    A = a.permute([sa.index(c) for c in batch + free_a + summed]).reshape(prod(batch), prod(free_a), prod(summed))
    B = b.permute([sb.index(c) for c in batch + summed + free_b]).reshape(prod(batch), prod(summed), prod(free_b))
    out = torch.bmm(A, B).reshape([sizes[c] for c in batch + free_a + free_b])
    return out, batch + free_a + free_b


def einsum(equation: str, *operands) -> torch.Tensor:
    if len(operands) == 1 and isinstance(operands[0], (list, tuple)):
        operands = tuple(operands[0])
    if not operands:
        raise InvalidArgument("einsum needs at least one operand")
    dt = operands[0].dtype
    for t in operands[1:]:
        dt = torch.promote_types(dt, t.dtype)
    ops = [t.to(dt) for t in operands]
    ins, out = _parse(equation, ops)
    work: List[Tuple[torch.Tensor, List[str]]] = []
    for t, sub in zip(ops, ins):
        t, sub = _diagonalise(t, sub)
        work.append((t, sub))
    # a subscript of a single operand that the output does not want is summed before any product
    for k, (t, sub) in enumerate(work):
        others = {c for j, (_, s) in enumerate(work) if j != k for c in s}
        drop = [i for i, c in enumerate(sub) if c not in out and c not in others]
        if drop:
            t = t.sum(dim=drop)
            sub = [c for i, c in enumerate(sub) if i not in drop]
        work[k] = (t, sub)
    t, sub = work[0]
    for k in range(1, len(work)):
        later = {c for _, s in work[k + 1:] for c in s}
        use_matmul = t.is_floating_point() or t.is_complex()
        if use_matmul:
            t, sub = _contract(t, sub, work[k][0], work[k][1], set(out) | later)
        else:                                                # integer operands: broadcast product and sum (bmm is for floating types)
            u, su = work[k]
            allc = sub + [c for c in su if c not in sub]
            ta = t.permute([sub.index(c) for c in allc if c in sub]).reshape([t.shape[sub.index(c)] if c in sub else 1 for c in allc])
            tb = u.permute([su.index(c) for c in allc if c in su]).reshape([u.shape[su.index(c)] if c in su else 1 for c in allc])
            prod = ta * tb
            dead = [i for i, c in enumerate(allc) if c not in out and c not in later]
            t = prod.sum(dim=dead) if dead else prod
            sub = [c for i, c in enumerate(allc) if i not in dead]
    extra = [i for i, c in enumerate(sub) if c not in out]
    if extra:
        t = t.sum(dim=extra)
        sub = [c for i, c in enumerate(sub) if i not in extra]
    return t.permute([sub.index(c) for c in out]) if out != sub else t
