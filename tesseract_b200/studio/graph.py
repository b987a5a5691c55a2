"""Block graph of the visual builder: typed nodes wired port to port, saved as ``.tsb`` JSON
(studio/core/include/tesseract/studio/BlockGraph.hpp:15-106, studio/core/src/BlockGraph.cpp). The text form is
stable: ``from_tsb(g.to_tsb()).to_tsb() == g.to_tsb()``.
"""
from __future__ import annotations

import enum
import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class PortType(enum.Enum):
    Tensor = "tensor"
    Model = "model"
    Params = "params"          # a parameter list feeding an optimizer
    Optimizer = "optimizer"
    Loss = "loss"
    Tokenizer = "tokenizer"
    Dataset = "dataset"
    Scalar = "scalar"          # a numeric / string config value
    Any = "any"

    @staticmethod
    def from_string(s: str) -> "PortType":
        try:
            return PortType(s)
        except ValueError:
            raise ValueError(f"unknown port type '{s}'") from None


@dataclass
class Endpoint:
    node: int = -1
    port: str = ""


@dataclass
class Edge:
    src: Endpoint      # an output port
    dst: Endpoint      # an input port


@dataclass
class Node:
    id: int = -1
    kind: str = ""                                   # catalog key, e.g. "Linear", "LoadLlama", "Adam"
    params: Dict[str, Any] = field(default_factory=dict)
    x: float = 0.0                                   # canvas position (UI only)
    y: float = 0.0

    def param_int(self, key: str, default: int = 0) -> int:
        v = self.params.get(key, default)
        try:
            return int(v)
        except (TypeError, ValueError):
            return default

    def param_num(self, key: str, default: float = 0.0) -> float:
        v = self.params.get(key, default)
        try:
            return float(v)
        except (TypeError, ValueError):
            return default

    def param_bool(self, key: str, default: bool = False) -> bool:
        v = self.params.get(key, default)
        return bool(v) if isinstance(v, (bool, int)) else default

    def param_str(self, key: str, default: str = "") -> str:
        v = self.params.get(key, default)
        return v if isinstance(v, str) else default


class BlockGraph:
    def __init__(self, name: str = "untitled", device: str = "cpu"):
        self.name = name
        self.device = device        # "cpu" | "cuda"
        self.nodes: List[Node] = []
        self.edges: List[Edge] = []
        self._next_id = 1

    def add_node(self, kind: str, params: Optional[Dict[str, Any]] = None, x: float = 0.0, y: float = 0.0) -> int:
        nid = self._next_id
        self._next_id += 1
        self.nodes.append(Node(nid, kind, dict(params or {}), float(x), float(y)))
        return nid

    def find_node(self, nid: int) -> Optional[Node]:
        for n in self.nodes:
            if n.id == nid:
                return n
        return None

    def connect(self, from_node: int, from_port: str, to_node: int, to_port: str) -> None:
        """An input port holds one wire: connecting it again replaces the old one."""
        self.edges = [e for e in self.edges if not (e.dst.node == to_node and e.dst.port == to_port)]
        self.edges.append(Edge(Endpoint(from_node, from_port), Endpoint(to_node, to_port)))

    def incoming(self, node: int, port: str) -> Optional[Edge]:
        for e in self.edges:
            if e.dst.node == node and e.dst.port == port:
                return e
        return None

    def outgoing(self, node: int, port: str) -> List[Edge]:
        return [e for e in self.edges if e.src.node == node and e.src.port == port]

    def topo_order(self) -> List[int]:
        """Node ids, producers first (ties by id). Raises ``ValueError`` on a cycle."""
        ids = sorted(n.id for n in self.nodes)
        indeg = {i: 0 for i in ids}
        for e in self.edges:
            if e.src.node in indeg and e.dst.node in indeg:
                indeg[e.dst.node] += 1
        ready = [i for i in ids if indeg[i] == 0]
        order: List[int] = []
        while ready:
            n = ready.pop(0)
            order.append(n)
            for e in self.edges:
                if e.src.node == n and e.dst.node in indeg:
                    indeg[e.dst.node] -= 1
                    if indeg[e.dst.node] == 0:
                        ready.append(e.dst.node)
                        ready.sort()
        if len(order) != len(ids):
            raise ValueError("the block graph has a cycle")
        return order

    # ---- .tsb ---------------------------------------------------------------------------------------------------
    def to_json(self) -> Dict[str, Any]:
        return {
            "format": "tsb", "version": 1, "name": self.name, "device": self.device,
            "nodes": [{"id": n.id, "kind": n.kind, "params": n.params, "x": n.x, "y": n.y} for n in self.nodes],
            "edges": [{"from": {"node": e.src.node, "port": e.src.port}, "to": {"node": e.dst.node, "port": e.dst.port}}
                      for e in self.edges],
        }

    @staticmethod
    def from_json(j: Dict[str, Any]) -> "BlockGraph":
        if not isinstance(j, dict) or "nodes" not in j:
            raise ValueError("not a .tsb document: no 'nodes'")
        g = BlockGraph(str(j.get("name", "untitled")), str(j.get("device", "cpu")))
        for n in j.get("nodes", []):
            g.nodes.append(Node(int(n["id"]), str(n["kind"]), dict(n.get("params", {})), float(n.get("x", 0.0)),
                                float(n.get("y", 0.0))))
        for e in j.get("edges", []):
            g.edges.append(Edge(Endpoint(int(e["from"]["node"]), str(e["from"]["port"])),
                                Endpoint(int(e["to"]["node"]), str(e["to"]["port"]))))
        g._next_id = max([n.id for n in g.nodes], default=0) + 1
        return g

    def to_tsb(self, indent: int = 2) -> str:
        return json.dumps(self.to_json(), indent=indent, sort_keys=False, ensure_ascii=False)

    @staticmethod
    def from_tsb(text: str) -> "BlockGraph":
        return BlockGraph.from_json(json.loads(text))

    def copy(self) -> "BlockGraph":
        return BlockGraph.from_json(json.loads(json.dumps(self.to_json())))
