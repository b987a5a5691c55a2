"""Static checks of a block graph before it runs: unknown kinds, wires between ports of different types, required
inputs left open, cycles (errors), and shape inference along the tensor wires with a warning where a layer's
declared width disagrees with what reaches it (studio/core/src/Analysis.cpp:40-209).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .catalog import BlockCatalog
from .graph import BlockGraph, Node, PortType


@dataclass
class Diagnostic:
    severity: str          # "error" | "warning"
    node: int              # -1: graph level
    message: str


@dataclass
class AnalysisResult:
    ok: bool = True
    diagnostics: List[Diagnostic] = field(default_factory=list)
    out_shapes: Dict[int, List[int]] = field(default_factory=dict)

    def to_json(self) -> Dict[str, Any]:
        return {"ok": self.ok,
                "diagnostics": [{"severity": d.severity, "node": d.node, "message": d.message} for d in self.diagnostics],
                "shapes": {str(k): list(v) for k, v in sorted(self.out_shapes.items())}}


_LAST_DIM_PARAM = {"Linear": "in_features", "RMSNorm": "dim", "LayerNorm": "dim", "FeedForward": "d_model",
                   "MultiHeadAttention": "d_model", "TransformerBlock": "d_model"}


def _propagate(n: Node, shape: List[int], diags: List[Diagnostic]) -> List[int]:
    key = _LAST_DIM_PARAM.get(n.kind)
    if key is not None and shape and shape[-1] != n.param_int(key):
        diags.append(Diagnostic("warning", n.id, f"{n.kind}: {key} expects last dim {n.param_int(key)} but got {shape}"))
    if n.kind == "Linear":
        return shape[:-1] + [n.param_int("out_features")] if shape else shape
    if n.kind == "Embedding":
        return shape + [n.param_int("embedding_dim")]
    return list(shape)


def analyze(g: BlockGraph) -> AnalysisResult:
    r = AnalysisResult()
    cat = BlockCatalog.instance()
    d = r.diagnostics
    for n in g.nodes:
        if cat.find(n.kind) is None:
            d.append(Diagnostic("error", n.id, f"unknown block kind '{n.kind}'"))
    for e in g.edges:
        fn, tn = g.find_node(e.src.node), g.find_node(e.dst.node)
        if fn is None or tn is None:
            d.append(Diagnostic("error", -1, "edge references a missing node"))
            continue
        fs, ts = cat.find(fn.kind), cat.find(tn.kind)
        if fs is None or ts is None:
            continue
        fp, tp = fs.output(e.src.port), ts.input(e.dst.port)
        if fp is None:
            d.append(Diagnostic("error", fn.id, f"no output port '{e.src.port}'"))
            continue
        if tp is None:
            d.append(Diagnostic("error", tn.id, f"no input port '{e.dst.port}'"))
            continue
        if fp.type != tp.type and PortType.Any not in (fp.type, tp.type):
            d.append(Diagnostic("error", tn.id, f"type mismatch: {fn.kind}.{fp.name} ({fp.type.value}) -> "
                                                f"{tn.kind}.{tp.name} ({tp.type.value})"))
    for n in g.nodes:
        spec = cat.find(n.kind)
        if spec is None:
            continue
        for p in spec.inputs:
            optional = n.kind == "Generate" and p.name == "tokenizer"
            if not optional and g.incoming(n.id, p.name) is None:
                d.append(Diagnostic("error", n.id, f"{n.kind}: input '{p.name}' is not connected"))
    order: List[int] = []
    try:
        order = g.topo_order()
    except ValueError as ex:
        d.append(Diagnostic("error", -1, str(ex)))

    def shape_from(node: int, port: str) -> Optional[List[int]]:
        e = g.incoming(node, port)
        return r.out_shapes.get(e.src.node) if e is not None else None

    for nid in order:
        n = g.find_node(nid)
        if n.kind == "Input":
            r.out_shapes[nid] = [n.param_int("batch", 32), n.param_int("features", 8)]
        elif n.kind == "TensorConst":
            r.out_shapes[nid] = [n.param_int("rows", 2), n.param_int("cols", 3)]
        elif n.kind in ("TAdd", "TSub", "TMul", "TMatMul"):
            sa, sb = shape_from(nid, "a"), shape_from(nid, "b")
            if sa is None or sb is None:
                continue
            if n.kind == "TMatMul":
                if len(sa) == 2 and len(sb) == 2:
                    if sa[-1] != sb[0]:
                        d.append(Diagnostic("warning", nid, f"MatMul inner dims disagree: {sa} . {sb}"))
                    r.out_shapes[nid] = [sa[0], sb[1]]
            else:
                if sa != sb:
                    d.append(Diagnostic("warning", nid, f"{n.kind}: shapes differ {sa} vs {sb}"))
                r.out_shapes[nid] = list(sa)
        else:
            s = shape_from(nid, "in")
            if s is not None:
                r.out_shapes[nid] = _propagate(n, s, d)
    r.ok = not any(x.severity == "error" for x in d)
    return r
