"""Graph convolution network (Kipf & Welling GCN) over an edge list with segment scatter-add aggregation.

Reference parity: ferrotorch-graph/src/{graph.rs:17, gcn.rs:65,290, loader.rs:57}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from .. import nn
from ..errors import InvalidArgument


@dataclass
class Graph:
    """Directed edge list ``edge_index [2, E]`` (source row 0, target row 1) over ``num_nodes`` nodes."""
    edge_index: torch.Tensor
    num_nodes: int

    def __post_init__(self):
        if self.edge_index.dim() != 2 or self.edge_index.shape[0] != 2:
            raise InvalidArgument("edge_index must be [2, E]")
        if self.edge_index.numel() and int(self.edge_index.max()) >= self.num_nodes:
            raise InvalidArgument("edge references a node outside the graph")

    def with_self_loops(self) -> "Graph":
        loops = torch.arange(self.num_nodes, device=self.edge_index.device)
        return Graph(torch.cat([self.edge_index, torch.stack([loops, loops])], 1), self.num_nodes)

    def degree(self) -> torch.Tensor:
        return torch.zeros(self.num_nodes, device=self.edge_index.device).index_add_(0, self.edge_index[1], torch.ones(self.edge_index.shape[1], device=self.edge_index.device))

    def gcn_norm(self):
        """Symmetric normalisation ``D^-1/2 (A + I) D^-1/2`` as per-edge weights."""
        g = self.with_self_loops()
        d = g.degree().pow(-0.5)
        d[torch.isinf(d)] = 0
        return g, d[g.edge_index[0]] * d[g.edge_index[1]]


def scatter_add_segments(src: torch.Tensor, index: torch.Tensor, num_segments: int) -> torch.Tensor:
    return torch.zeros(num_segments, *src.shape[1:], device=src.device, dtype=src.dtype).index_add_(0, index, src)


class GcnConv(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.lin = nn.Linear(in_features, out_features, bias=False)
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self._cache = None

    def forward(self, x, graph: Graph):
        if self._cache is None or self._cache[0] is not graph:
            self._cache = (graph, *graph.gcn_norm())
        _, g, w = self._cache
        h = self.lin(x)
        out = scatter_add_segments(h[g.edge_index[0]] * w[:, None].to(h.dtype), g.edge_index[1], g.num_nodes)
        return out + self.bias if self.bias is not None else out


class GcnNet(nn.Module):
    """Two-layer GCN: conv -> ReLU -> dropout -> conv (Cora: 1433 -> 16 -> 7)."""

    def __init__(self, in_features: int = 1433, hidden: int = 16, num_classes: int = 7, dropout: float = 0.5):
        super().__init__()
        self.conv1, self.conv2, self.p = GcnConv(in_features, hidden), GcnConv(hidden, num_classes), dropout

    def forward(self, x, graph: Graph):
        h = F.dropout(F.relu(self.conv1(x, graph)), self.p, self.training)
        return self.conv2(h, graph)


def load_gcn_net(path: str, in_features=1433, hidden=16, num_classes=7) -> GcnNet:
    """Loads PyG-style names (``conv1.lin.weight``, ``conv1.bias`` ...) from a safetensors file."""
    from ..serialize import load_safetensors
    m = GcnNet(in_features, hidden, num_classes)
    m.load_state_dict(load_safetensors(path), strict=True)
    return m
