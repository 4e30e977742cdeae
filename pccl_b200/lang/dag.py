"""Directed graph used for the op DAG and the device topology of a collective program.

Capability parity with the reference's ``DirectedGraph`` (pccl/lang/utils/graph.py:17-134):
node/edge insertion and removal, predecessor/successor queries, acyclicity, topological order
and undirected connected components.  The design differs on purpose:

* nodes are keyed by the id the caller supplies (the reference auto-numbers and ignores the id it
  is given, graph.py:23-27, which breaks topologies whose device ids are not 0..n-1);
* adjacency is kept in insertion-ordered dicts, so every traversal is deterministic and O(V+E);
* ordering uses Kahn's algorithm (iterative; no recursion limit on long ring programs);
* ``reachability()`` returns per-node ancestor bitsets, which the static race check needs.
"""
from __future__ import annotations

from typing import Any, Dict, Hashable, Iterable, List, Optional


class DirectedGraph:
    def __init__(self) -> None:
        self._succ: Dict[Hashable, Dict[Hashable, Any]] = {}
        self._pred: Dict[Hashable, Dict[Hashable, Any]] = {}
        self._data: Dict[Hashable, Any] = {}
        self._auto = 0

    # -- construction -------------------------------------------------------------------------
    def add_node(self, node_id: Optional[Hashable] = None, data: Any = None) -> Hashable:
        """Insert ``node_id`` (or a fresh integer id when None).  Re-adding is a no-op."""
        if node_id is None:
            while self._auto in self._succ:
                self._auto += 1
            node_id = self._auto
        if node_id not in self._succ:
            self._succ[node_id] = {}
            self._pred[node_id] = {}
        if data is not None or node_id not in self._data:
            self._data[node_id] = data
        return node_id

    def add_edge(self, src: Hashable, dst: Hashable, data: Any = None) -> None:
        if src not in self._succ or dst not in self._succ:
            raise ValueError(f"edge ({src!r} -> {dst!r}) names an unknown node")
        self._succ[src][dst] = data
        self._pred[dst][src] = data

    def remove_edge(self, src: Hashable, dst: Hashable) -> bool:
        if src in self._succ and dst in self._succ[src]:
            del self._succ[src][dst]
            del self._pred[dst][src]
            return True
        return False

    # -- queries ------------------------------------------------------------------------------
    def __contains__(self, node_id: Hashable) -> bool:
        return node_id in self._succ

    def __len__(self) -> int:
        return len(self._succ)

    @property
    def nodes(self) -> List[Hashable]:
        return list(self._succ)

    def get_node(self, node_id: Hashable) -> Any:
        return self._data.get(node_id)

    def get_edges(self) -> List[tuple]:
        return [(s, d) for s, ds in self._succ.items() for d in ds]

    def num_edges(self) -> int:
        return sum(len(d) for d in self._succ.values())

    def get_successors(self, node_id: Hashable) -> List[Hashable]:
        return list(self._succ.get(node_id, ()))

    def get_predecessors(self, node_id: Hashable) -> List[Hashable]:
        return list(self._pred.get(node_id, ()))

    def in_degree(self, node_id: Hashable) -> int:
        return len(self._pred[node_id])

    # -- algorithms ---------------------------------------------------------------------------
    def topological_sort(self) -> List[Hashable]:
        """Kahn's algorithm; ties resolve in insertion order.  Raises ValueError on a cycle."""
        indeg = {n: len(p) for n, p in self._pred.items()}
        ready = [n for n, d in indeg.items() if d == 0]
        order: List[Hashable] = []
        head = 0
        while head < len(ready):
            n = ready[head]
            head += 1
            order.append(n)
            for m in self._succ[n]:
                indeg[m] -= 1
                if indeg[m] == 0:
                    ready.append(m)
        if len(order) != len(self._succ):
            raise ValueError("graph has a cycle")
        return order

    def is_acyclic(self) -> bool:
        try:
            self.topological_sort()
            return True
        except ValueError:
            return False

    def get_connected_components(self) -> List[List[Hashable]]:
        """Components of the graph with edge direction ignored."""
        seen = set()
        comps: List[List[Hashable]] = []
        for root in self._succ:
            if root in seen:
                continue
            comp, stack = [], [root]
            seen.add(root)
            while stack:
                n = stack.pop()
                comp.append(n)
                for m in list(self._succ[n]) + list(self._pred[n]):
                    if m not in seen:
                        seen.add(m)
                        stack.append(m)
            comps.append(comp)
        return comps

    def reachability(self) -> Dict[Hashable, int]:
        """For every node, a bitset (python int) of its strict ancestors.

        Bit ``i`` refers to the i-th node in topological order (also returned under key
        ``"__index__"`` as a dict).  Two nodes are ordered iff one is an ancestor of the other.
        """
        order = self.topological_sort()
        index = {n: i for i, n in enumerate(order)}
        anc: Dict[Hashable, int] = {}
        for n in order:
            bits = 0
            for p in self._pred[n]:
                bits |= anc[p] | (1 << index[p])
            anc[n] = bits
        anc["__index__"] = index  # type: ignore[assignment]
        return anc

    def critical_path(self, weight: Optional[Dict[Hashable, float]] = None) -> float:
        """Longest weighted path (node weights, default 1) — a lower bound on schedule steps."""
        best: Dict[Hashable, float] = {}
        for n in self.topological_sort():
            w = 1.0 if weight is None else float(weight.get(n, 0.0))
            best[n] = w + max((best[p] for p in self._pred[n]), default=0.0)
        return max(best.values(), default=0.0)

    def subgraph(self, keep: Iterable[Hashable]) -> "DirectedGraph":
        keep = set(keep)
        g = DirectedGraph()
        for n in self._succ:
            if n in keep:
                g.add_node(n, self._data.get(n))
        for s, ds in self._succ.items():
            if s in keep:
                for d, data in ds.items():
                    if d in keep:
                        g.add_edge(s, d, data)
        return g
