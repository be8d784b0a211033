"""Graph optimisation passes: constant folding, dead-code elimination, common-subexpression elimination, algebraic simplification,
DAG fusion of elementwise regions and a liveness-based memory plan.

Reference parity: ferrotorch-jit/src/{optimize.rs (const fold / DCE), dag_fusion.rs:92 (find_fusion_groups), fusion.rs:281,
memory_plan.rs}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Set, Tuple

import torch

from .ir import ELEMENTWISE, IrGraph, IrNode
from .interpreter import eval_node

_FOLD_LIMIT = 1 << 20          # never materialise folded constants above this many elements


def dead_code_elimination(g: IrGraph) -> int:
    live: Set[int] = set(g.outputs)
    removed = 0
    for n in reversed(g.topo_order()):
        if any(o in live for o in n.outputs):
            live.update(n.inputs)
        else:
            for o in n.outputs:
                g.values.pop(o, None)
            del g.nodes[n.id]
            removed += 1
    for c in [c for c in g.constants if c not in live and c not in g.outputs]:
        del g.constants[c]
        g.values.pop(c, None)
    return removed


def constant_folding(g: IrGraph) -> int:
    folded = 0
    for n in g.topo_order():
        if n.op in ("opaque", "dropout", "fused") or not n.inputs:
            continue
        if any(i in g.constants and g.constants[i].requires_grad for i in n.inputs):
            continue                                   # a trainable parameter changes between calls: nothing computed from it is a constant
        if all(i in g.constants for i in n.inputs) and all(g.values[o].numel() <= _FOLD_LIMIT for o in n.outputs):
            out = eval_node(n, [g.constants[i] for i in n.inputs], g)
            outs = out if isinstance(out, (tuple, list)) else [out]
            for vid, t in zip(n.outputs, outs):
                g.constants[vid] = t
                g.values[vid].producer = None
            del g.nodes[n.id]
            folded += 1
    return folded


def _key(g: IrGraph, n: IrNode):
    if n.op in ("opaque", "dropout"):
        return None
    return (n.op, tuple(n.inputs), tuple(sorted((k, str(v)) for k, v in n.attrs.items())))


def common_subexpression_elimination(g: IrGraph) -> int:
    seen: Dict[Tuple, IrNode] = {}
    rename: Dict[int, int] = {}
    removed = 0
    for n in g.topo_order():
        n.inputs = [rename.get(i, i) for i in n.inputs]
        k = _key(g, n)
        if k is None:
            continue
        if k in seen:
            for a, b in zip(n.outputs, seen[k].outputs):
                rename[a] = b
                g.values.pop(a, None)
            del g.nodes[n.id]
            removed += 1
        else:
            seen[k] = n
    g.outputs = [rename.get(o, o) for o in g.outputs]
    return removed


def _const_scalar(g: IrGraph, vid: int) -> Optional[float]:
    c = g.constants.get(vid)
    if c is not None and c.numel() == 1:
        return float(c)
    return None


def algebraic_simplification(g: IrGraph) -> int:
    """x*1, x/1, x+0, x-0, x**1, neg(neg(x)), cast to the same dtype -> x (only when shapes and dtypes are unchanged)."""
    rename: Dict[int, int] = {}
    changed = 0
    for n in g.topo_order():
        n.inputs = [rename.get(i, i) for i in n.inputs]
        tgt = None
        if n.op in ("mul", "div", "pow") and _const_scalar(g, n.inputs[1]) == 1.0:
            tgt = n.inputs[0]
        elif n.op == "mul" and _const_scalar(g, n.inputs[0]) == 1.0:
            tgt = n.inputs[1]
        elif n.op in ("add", "sub") and _const_scalar(g, n.inputs[1]) == 0.0:
            tgt = n.inputs[0]
        elif n.op == "add" and _const_scalar(g, n.inputs[0]) == 0.0:
            tgt = n.inputs[1]
        elif n.op == "neg":
            p = g.values[n.inputs[0]].producer
            if p is not None and p in g.nodes and g.nodes[p].op == "neg":
                tgt = g.nodes[p].inputs[0]
        elif n.op == "cast" and g.values[n.inputs[0]].dtype == n.attrs["dtype"]:
            tgt = n.inputs[0]
        if tgt is not None:
            o, t = g.values[n.outputs[0]], g.values[tgt]
            if o.shape == t.shape and o.dtype == t.dtype:
                rename[n.outputs[0]] = tgt
                del g.nodes[n.id]
                g.values.pop(n.outputs[0], None)
                changed += 1
    g.outputs = [rename.get(o, o) for o in g.outputs]
    return changed


# ----------------------------------------------------------------------------------------------------------------------
# DAG fusion
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class FusionGroup:
    nodes: List[int]
    inputs: List[int] = field(default_factory=list)
    outputs: List[int] = field(default_factory=list)
    shape: Tuple[int, ...] = ()


def _fusable(g: IrGraph, n: IrNode) -> bool:
    if n.op not in ELEMENTWISE:
        return False
    return all(isinstance(s, int) for s in g.values[n.outputs[0]].shape)


def find_fusion_groups(g: IrGraph, min_size: int = 2) -> List[FusionGroup]:
    """DAG fusion: elementwise nodes with equal output shapes are merged along producer->consumer edges (union-find over groups).
    Two groups may merge only if no path from the earlier to the later one passes through a node outside both -- such a path would make
    the fused node depend on itself."""
    order = g.topo_order()
    pos = {n.id: i for i, n in enumerate(order)}
    parent: Dict[int, int] = {}

    def find(x: int) -> int:
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    members: Dict[int, List[int]] = {}
    for n in order:
        if _fusable(g, n):
            parent[n.id] = n.id
            members[n.id] = [n.id]

    def producers(nid: int) -> List[int]:
        return [g.values[i].producer for i in g.nodes[nid].inputs if g.values[i].producer is not None and g.values[i].producer in g.nodes]

    def path_through_outside(ga: int, gb: int) -> bool:
        """True if some member of gb reaches a member of ga through at least one node outside both groups."""
        lo = min(pos[m] for m in members[ga])
        seen: Set[int] = set()
        stack = [(p, False) for m in members[gb] for p in producers(m)]
        while stack:
            nid, outside = stack.pop()
            in_a = nid in parent and find(nid) == ga
            in_b = nid in parent and find(nid) == gb
            if in_a:
                if outside:
                    return True
                continue
            if pos[nid] < lo or (nid, outside) in seen:
                continue
            seen.add((nid, outside))
            for p in producers(nid):
                stack.append((p, outside or not in_b))
        return False

    for n in order:
        if n.id not in parent:
            continue
        shape = g.values[n.outputs[0]].shape
        for p in producers(n.id):
            if p not in parent:
                continue
            ga, gb = find(p), find(n.id)
            if ga == gb or g.values[g.nodes[p].outputs[0]].shape != shape:
                continue
            if path_through_outside(ga, gb):
                continue
            parent[gb] = ga
            members[ga] += members.pop(gb)
    users = g.users()
    out: List[FusionGroup] = []
    for gid, mem in members.items():
        if len(mem) < min_size:
            continue
        mem = sorted(mem, key=lambda m: pos[m])
        mset = set(mem)
        produced = {o for m in mem for o in g.nodes[m].outputs}
        ins, outs = [], []
        for m in mem:
            for i in g.nodes[m].inputs:
                if i not in produced and i not in ins:
                    ins.append(i)
        for o in sorted(produced):
            if o in g.outputs or any(u not in mset for u in users.get(o, [])):
                outs.append(o)
        out.append(FusionGroup(mem, ins, outs, g.values[g.nodes[mem[0]].outputs[0]].shape))
    return out


def fuse_elementwise(g: IrGraph, min_size: int = 2) -> int:
    """Replaces every fusion group by one ``fused`` node whose ``body`` attribute is the sub-graph."""
    n_fused = 0
    for grp in find_fusion_groups(g, min_size):
        body = IrGraph()
        ren: Dict[int, int] = {}
        ext_inputs = []
        for i in grp.inputs:
            v = g.values[i]
            if i in g.constants and g.constants[i].numel() == 1 and g.constants[i].device.type == "cpu":
                ren[i] = body.add_constant(g.constants[i].reshape(())).id     # scalar literals are inlined into the kernel
            else:
                ren[i] = body.add_input(v.shape, v.dtype).id
                ext_inputs.append(i)
        for nid in grp.nodes:
            n = g.nodes[nid]
            bn = body.add_node(n.op, [ren[i] for i in n.inputs], [(g.values[o].shape, g.values[o].dtype) for o in n.outputs], **n.attrs)
            for a, b in zip(n.outputs, bn.outputs):
                ren[a] = b
        body.set_outputs([ren[o] for o in grp.outputs])
        body.single_output = False
        fn = g.add_node("fused", ext_inputs, [(g.values[o].shape, g.values[o].dtype) for o in grp.outputs], body=body, size=len(grp.nodes))
        # rewire: the new node's outputs take over the old value ids
        for old, new in zip(grp.outputs, list(fn.outputs)):
            g.values.pop(new)
            g.values[old].producer = fn.id
        fn.outputs = list(grp.outputs)
        for nid in grp.nodes:
            for o in g.nodes[nid].outputs:
                if o not in grp.outputs:
                    g.values.pop(o, None)
            del g.nodes[nid]
        n_fused += 1
    return n_fused


# ----------------------------------------------------------------------------------------------------------------------
# memory plan
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class MemoryPlan:
    slot_of: Dict[int, int]
    slot_bytes: List[int]
    naive_bytes: int

    @property
    def planned_bytes(self) -> int:
        return sum(self.slot_bytes)


_ITEM = {"f32": 4, "f64": 8, "bf16": 2, "f16": 2, "i64": 8, "i32": 4, "bool": 1, "u8": 1, "i8": 1, "i16": 2}


def plan_memory(g: IrGraph) -> MemoryPlan:
    """Linear-scan buffer reuse over the topological order: a value's slot is released after its last use, graph outputs are pinned."""
    order = g.topo_order()
    last_use: Dict[int, int] = {}
    for i, n in enumerate(order):
        for v in n.inputs:
            last_use[v] = i
    free: List[Tuple[int, int]] = []          # (bytes, slot)
    slot_of: Dict[int, int] = {}
    slot_bytes: List[int] = []
    naive = 0
    alias_ops = {"reshape", "permute", "transpose", "expand", "unsqueeze", "squeeze", "slice", "select"}
    for i, n in enumerate(order):
        for o in n.outputs:
            v = g.values[o]
            if n.op in alias_ops:
                continue
            nbytes = v.numel() * _ITEM[v.dtype]
            naive += nbytes
            best = None
            for k, (fb, fs) in enumerate(free):
                if fb >= nbytes and (best is None or fb < free[best][0]):
                    best = k
            if best is not None and o not in g.outputs:
                _, s = free.pop(best)
            else:
                s = len(slot_bytes)
                slot_bytes.append(nbytes)
            slot_of[o] = s
        for v in set(n.inputs):
            if last_use.get(v) == i and v in slot_of and v not in g.outputs:
                # views may still alias this slot: only release when no alias op consumed it
                if not any(g.nodes[u].op in alias_ops for u in g.users().get(v, []) if u in g.nodes):
                    free.append((slot_bytes[slot_of[v]], slot_of[v]))
    return MemoryPlan(slot_of, slot_bytes, naive)


def fuse_reductions(g: IrGraph) -> int:
    """A sum / mean / amax / amin over the last dimension whose only producer is a fused elementwise region (and which is the only consumer of that
    value) is folded into the region: the node becomes ``fused_reduce`` (outputs: the reduced value first, then the region's other outputs)."""
    users = g.users()
    n_done = 0
    for r in list(g.topo_order()):
        if r.id not in g.nodes or r.op not in ("sum", "mean", "amax", "amin"):
            continue
        src = r.inputs[0]
        v = g.values[src]
        if tuple(r.attrs["dims"]) != (len(v.shape) - 1,) or len(v.shape) < 1:
            continue
        pid = v.producer
        if pid is None or pid not in g.nodes or g.nodes[pid].op != "fused" or src in g.outputs or users.get(src, []) != [r.id]:
            continue
        f = g.nodes[pid]
        idx = f.outputs.index(src)
        rest = [o for o in f.outputs if o != src]
        node = g.add_node("fused_reduce", f.inputs, [(g.values[r.outputs[0]].shape, g.values[r.outputs[0]].dtype)] + [(g.values[o].shape, g.values[o].dtype) for o in rest],
                          body=f.attrs["body"], red_op=r.op, red_index=idx, keepdim=bool(r.attrs.get("keepdim", False)), size=f.attrs.get("size", 0) + 1)
        for new in list(node.outputs):
            g.values.pop(new)
        node.outputs = [r.outputs[0]] + rest
        for o in node.outputs:
            g.values[o].producer = node.id
        g.values.pop(src, None)
        del g.nodes[f.id], g.nodes[r.id]
        users = g.users()
        n_done += 1
    return n_done


def optimize(g: IrGraph, fuse: bool = True) -> Dict[str, int]:
    stats = {"folded": constant_folding(g), "simplified": algebraic_simplification(g), "cse": common_subexpression_elimination(g),
             "dce": dead_code_elimination(g)}
    stats["fused_groups"] = fuse_elementwise(g) if fuse else 0
    stats["fused_reductions"] = fuse_reductions(g) if fuse else 0
    g.validate()
    return stats
