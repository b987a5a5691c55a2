"""Graph capture and replay: ``GraphScope`` records the ops executed inside it into a small ``Graph`` (nodes with
a kind, inputs, outputs and attributes) and ``run`` re-executes a graph on new inputs -- the role of the
reference's C++ graph IR (include/tesseract/graph/GraphScope.hpp:42-102, src/graph/Interpreter.cpp:105-168).

Capture is built on ``torch.fx`` symbolic tracing of a module or function (the idiomatic torch stand-in for the
reference's per-op ``graph::maybe_record`` hook); node kinds are normalised to the reference's op names where one
exists (``matmul``, ``add``, ``rms_norm`` ...). ``build_backward`` returns a callable that evaluates the graph's
gradient with autograd (the reference transforms the graph itself, src/graph/Autograd.cpp). The MLIR dialect, its
passes and the JIT engines of the reference (src/ir) are not part of this framework.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.fx as fx

_KIND = {"linear": "matmul", "matmul": "matmul", "add": "add", "sub": "sub", "mul": "mul", "truediv": "div",
         "relu": "relu", "sigmoid": "sigmoid", "tanh": "tanh", "softmax": "softmax", "reshape": "reshape",
         "view": "reshape", "permute": "permute", "transpose": "transpose", "cat": "cat", "exp": "exp", "log": "log",
         "sum": "sum", "mean": "mean", "neg": "neg", "sqrt": "sqrt"}


@dataclass
class Node:
    kind: str
    name: str
    inputs: List[str]
    attrs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class Graph:
    nodes: List[Node]
    inputs: List[str]
    outputs: List[str]
    module: fx.GraphModule

    def op_kinds(self) -> List[str]:
        return [n.kind for n in self.nodes]

    def __len__(self) -> int:
        return len(self.nodes)


class GraphScope:
    """``with GraphScope() as g: g.trace(fn_or_module)`` -> ``g.graph``. Thread-local nesting is not needed: the
    trace is explicit."""

    def __init__(self):
        self.graph: Optional[Graph] = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False

    def trace(self, target: Callable) -> Graph:
        gm = fx.symbolic_trace(target)
        nodes, inputs, outputs = [], [], []
        for n in gm.graph.nodes:
            if n.op == "placeholder":
                inputs.append(n.name)
            elif n.op == "output":
                outs = n.args[0] if isinstance(n.args[0], (tuple, list)) else [n.args[0]]
                outputs = [getattr(o, "name", str(o)) for o in outs]
            elif n.op in ("call_function", "call_method", "call_module"):
                raw = n.target if isinstance(n.target, str) else getattr(n.target, "__name__", str(n.target))
                if n.op == "call_module":
                    raw = type(gm.get_submodule(n.target)).__name__.lower()
                kind = _KIND.get(raw, raw)
                ins = [a.name for a in n.all_input_nodes]
                nodes.append(Node(kind, n.name, ins, {k: v for k, v in n.kwargs.items() if not isinstance(v, fx.Node)}))
        self.graph = Graph(nodes, inputs, outputs, gm)
        return self.graph


def run(graph: Graph, *inputs):
    """Interpret the captured graph on new inputs."""
    return fx.Interpreter(graph.module).run(*inputs)


def build_backward(graph: Graph) -> Callable:
    """Returns ``f(*inputs, grad_output=None) -> list of input gradients`` for a single-output graph."""

    def backward(*inputs, grad_output=None):
        xs = [x.detach().clone().requires_grad_(x.is_floating_point()) for x in inputs]
        y = run(graph, *xs)
        if grad_output is None:
            grad_output = torch.ones_like(y)
        need = [x for x in xs if x.requires_grad]
        grads = torch.autograd.grad(y, need, grad_output, allow_unused=True)
        it = iter(grads)
        return [next(it) if x.requires_grad else None for x in xs]

    return backward


__all__ = ["Graph", "GraphScope", "Node", "run", "build_backward"]
