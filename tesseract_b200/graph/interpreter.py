"""Graph interpreter: ``run(g, bindings)`` walks the ops in order and dispatches each to the eager op of the same
name, under no-grad, and returns the tensors of ``g.outputs`` (src/graph/Interpreter.cpp:105-228). It also runs the
backward-extended graphs of ``build_backward`` (``relu_backward``, ``cross_entropy_with_logits_backward``,
``reduce_to_shape``), which is what graph-mode training is built on.

``GraphExecutor`` is the replay form for a GPU: bindings live in static buffers, the whole op list is captured once
into a CUDA graph, and each call copies the new inputs in and launches the graph -- one launch per step instead
of one per op. On a CPU it interprets.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from .ir import Graph, Op, ValueId
from .scope import is_recording


def _need(attrs, key, kind):
    if key not in attrs:
        raise KeyError(f"graph.run: op '{kind}' is missing its '{key}' attribute")
    return attrs[key]


def _reduce(fn, is_max=False):
    def k(op: Op, x):
        if "dim" not in op.attrs:
            return fn(x)
        out = fn(x, int(op.attrs["dim"]), bool(op.attrs.get("keepdim", False)))
        return out[0] if is_max else out
    return k


def reduce_to_shape(x: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
    """The adjoint of broadcasting: sums ``x`` over the axes that broadcasting ``shape`` to ``x.shape`` expanded."""
    shape = tuple(shape)
    if tuple(x.shape) == shape:
        return x
    lead = x.dim() - len(shape)
    if lead < 0:
        raise ValueError(f"reduce_to_shape: target {shape} has more dims than the source {tuple(x.shape)}")
    if lead:
        x = x.sum(dim=tuple(range(lead)))
    dims = tuple(i for i, s in enumerate(shape) if s == 1 and x.shape[i] != 1)
    if dims:
        x = x.sum(dim=dims, keepdim=True)
    if tuple(x.shape) != shape:
        raise ValueError(f"reduce_to_shape: {tuple(x.shape)} does not reduce to {shape}")
    return x


def _ce_backward(op: Op, logits, targets, grad):
    # (softmax - one_hot) * grad / n, built in place on the softmax buffer
    n = logits.shape[0]
    p = torch.softmax(logits.float(), dim=-1)
    p.scatter_add_(1, targets.view(-1, 1), p.new_full((n, 1), -1.0))
    p.mul_(grad.float() / n)
    return p if p.dtype == logits.dtype else p.to(logits.dtype)


_KERNELS: Dict[str, Callable] = {
    "add": lambda op, a, b: a + b,
    "sub": lambda op, a, b: a - b,
    "mul": lambda op, a, b: a * b,
    "div": lambda op, a, b: a / b,
    "neg": lambda op, x: -x,
    "matmul": lambda op, a, b: torch.matmul(a, b),
    "sum": _reduce(torch.sum),
    "mean": _reduce(torch.mean),
    "max": _reduce(torch.max, is_max=True),
    "relu": lambda op, x: torch.relu(x),
    "sigmoid": lambda op, x: torch.sigmoid(x),
    "tanh": lambda op, x: torch.tanh(x),
    "exp": lambda op, x: torch.exp(x),
    "log": lambda op, x: torch.log(x),
    "sqrt": lambda op, x: torch.sqrt(x),
    "softmax": lambda op, x: torch.softmax(x, int(_need(op.attrs, "dim", op.kind))),
    "view": lambda op, x: x.view(list(_need(op.attrs, "shape", op.kind))),
    "reshape": lambda op, x: x.reshape(list(_need(op.attrs, "shape", op.kind))),
    "permute": lambda op, x: x.permute(list(_need(op.attrs, "axes", op.kind))),
    "transpose": lambda op, x: x.transpose(int(_need(op.attrs, "dim_a", op.kind)), int(_need(op.attrs, "dim_b", op.kind))),
    "contiguous": lambda op, x: x.contiguous(),
    "clone": lambda op, x: x.clone(),
    "broadcast_to": lambda op, x: x.broadcast_to(list(_need(op.attrs, "shape", op.kind))),
    "reduce_to_shape": lambda op, x: reduce_to_shape(x, _need(op.attrs, "shape", op.kind)),
    "cross_entropy_with_logits": lambda op, logits, targets: F.cross_entropy(logits, targets),
    "relu_backward": lambda op, grad, x: torch.ops.aten.threshold_backward(grad, x, 0.0),
    "fused_linear": lambda op, x, w, b: F.linear(x, w, b),         # produced by plan(), never recorded
    "matmul_tn": lambda op, a, b: torch.mm(a.t(), b),              # likewise
    "cross_entropy_with_logits_backward": _ce_backward,
}


def supported_ops() -> List[str]:
    return sorted(k for k in _KERNELS if k not in ("fused_linear", "matmul_tn"))


def _check_bindings(g: Graph, env: Dict[ValueId, torch.Tensor]) -> None:
    for role, ids in (("input", g.inputs), ("param", g.params), ("constant", g.constants)):
        for vid in ids:
            if vid not in env:
                if role == "constant" and vid in g.constant_data:
                    env[vid] = g.constant_data[vid]
                    continue
                v = g.value(vid)
                raise KeyError(f"graph.run: {role} %{v.name or vid} has no tensor bound")
            v, t = g.value(vid), env[vid]
            if tuple(t.shape) != v.shape or t.dtype != v.dtype:
                raise ValueError(f"graph.run: {role} %{v.name or vid} is declared {v.shape} {v.dtype} but the bound "
                                 f"tensor is {tuple(t.shape)} {t.dtype}")


def _live(ops: Sequence[Op], outputs: Sequence[ValueId]) -> List[Op]:
    """The ops whose results reach ``outputs`` (a backward-extended graph also carries the gradient of its inputs,
    which graph-mode training never reads: the largest matmul of an MLP step)."""
    needed = set(outputs)
    keep: List[Op] = []
    for op in reversed(ops):
        if any(o in needed for o in op.outputs):
            keep.append(op)
            needed.update(op.inputs)
    keep.reverse()
    return keep


def _is_2d_transpose(op: Optional[Op], g: Graph) -> bool:
    if op is None or op.kind != "transpose" or len(g.value(op.inputs[0]).shape) != 2:
        return False
    return {int(op.attrs.get("dim_a", -9)), int(op.attrs.get("dim_b", -9))} in ({0, 1}, {-1, -2}, {0, -1}, {1, -2})


def plan(g: Graph) -> List[Op]:
    """The op list the interpreter actually walks: dead ops removed and two peepholes applied (the reference does this
    kind of clean-up in its lowering passes, src/ir/passes/): ``add(matmul(x, transpose(W)), broadcast_to(bias))``
    whose intermediates have no other reader becomes one ``fused_linear``; the result is cached on the graph."""
    key = (len(g.ops), tuple(g.outputs))
    cached = getattr(g, "_plan_cache", None)
    if cached is not None and cached[0] == key:
        return cached[1]
    ops = _live(g.ops, g.outputs)
    uses: Dict[ValueId, int] = {}
    for op in ops:
        for i in op.inputs:
            uses[i] = uses.get(i, 0) + 1
    for o in g.outputs:
        uses[o] = uses.get(o, 0) + 1
    producer = {op.outputs[0]: op for op in ops}
    folded = set()
    rewritten: List[Op] = []
    for op in ops:
        if op.kind == "add" and len(op.inputs) == 2:
            for a, b in (op.inputs, op.inputs[::-1]):
                pm, pb = producer.get(a), producer.get(b)
                if (pm is None or pb is None or pm.kind != "matmul" or pb.kind != "broadcast_to"
                        or uses.get(a) != 1 or uses.get(b) != 1):
                    continue
                x, t = pm.inputs
                pt = producer.get(t)
                bias = pb.inputs[0]
                out_shape = g.value(op.outputs[0]).shape
                if (_is_2d_transpose(pt, g) and len(g.value(x).shape) == 2 and len(g.value(bias).shape) == 1
                        and g.value(bias).shape[0] == out_shape[-1] and g.value(a).shape == out_shape):
                    folded.update((id(pm), id(pb)))
                    op = Op("fused_linear", [x, pt.inputs[0], bias], list(op.outputs), {})
                    break
        elif _is_2d_transpose(op, g):
            # transpose(matmul(transpose(a), b)) = matmul(transpose(b), a): the weight gradient of a Linear comes out
            # in the parameter's own layout, contiguous, instead of as a transposed view
            pm = producer.get(op.inputs[0])
            if pm is not None and pm.kind == "matmul" and uses.get(op.inputs[0]) == 1:
                pt = producer.get(pm.inputs[0])
                if _is_2d_transpose(pt, g) and len(g.value(pm.inputs[1]).shape) == 2:
                    folded.add(id(pm))
                    op = Op("matmul_tn", [pm.inputs[1], pt.inputs[0]], list(op.outputs), {})
        rewritten.append(op)
    final = _live([op for op in rewritten if id(op) not in folded], g.outputs)
    g._plan_cache = (key, final)
    return final


def _execute(g: Graph, env: Dict[ValueId, torch.Tensor]) -> List[torch.Tensor]:
    for op in plan(g):
        kernel = _KERNELS.get(op.kind)
        if kernel is None:
            raise NotImplementedError(f"graph.run: no kernel for op kind '{op.kind}'")
        try:
            args = [env[i] for i in op.inputs]
        except KeyError as e:
            raise KeyError(f"graph.run: op '{op.kind}' reads value %{e.args[0]} before it is defined") from None
        out = kernel(op, *args)
        env[op.outputs[0]] = out
    return [env[o] for o in g.outputs]


def run(g: Graph, bindings: Dict[ValueId, torch.Tensor]) -> List[torch.Tensor]:
    """Returns one tensor per ``g.outputs`` entry. Every input and param (and every constant that was not created
    while recording) needs a binding whose shape and dtype match the declared value. Not callable from inside a live
    ``GraphScope``."""
    if is_recording():
        raise RuntimeError("graph.run: called inside a live GraphScope")
    env = dict(bindings)
    _check_bindings(g, env)
    with torch.no_grad():
        return _execute(g, env)


class GraphExecutor:
    """Replays ``g`` with fixed shapes. ``bindings`` gives the initial tensors of all inputs / params / constants;
    they are copied into buffers owned by the executor. ``__call__(updates)`` copies the given tensors over their
    buffers and runs the graph; the returned tensors are the executor's output buffers (valid until the next call).
    ``buffer(vid)`` exposes a static buffer; the bindings named in ``share`` are not copied but used in place, so
    parameters that an optimizer updates in place are seen by the next call.

    With ``cuda_graph=True`` (the default when the buffers are on a GPU) the op list is captured once, after
    ``warmup`` eager runs on a side stream, and each call is one graph launch.
    """

    def __init__(self, g: Graph, bindings: Dict[ValueId, torch.Tensor], cuda_graph: Optional[bool] = None, warmup: int = 2,
                 share: Sequence[ValueId] = ()):
        if is_recording():
            raise RuntimeError("GraphExecutor: built inside a live GraphScope")
        self.graph = g
        env = dict(bindings)
        _check_bindings(g, env)
        shared = set(share)      # these bindings are used in place (parameters that an optimizer updates in place)
        self._static = {vid: env[vid].detach() if vid in shared else env[vid].detach().clone()
                        for vid in list(g.inputs) + list(g.params) + list(g.constants)}
        on_gpu = any(t.is_cuda for t in self._static.values())
        self.cuda_graph = on_gpu if cuda_graph is None else bool(cuda_graph)
        if self.cuda_graph and not on_gpu:
            raise ValueError("GraphExecutor: cuda_graph=True needs the bindings on a CUDA device")
        self._captured = None
        self._outputs: List[torch.Tensor] = []
        if self.cuda_graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side), torch.no_grad():
                for _ in range(max(1, warmup)):
                    _execute(g, dict(self._static))
            torch.cuda.current_stream().wait_stream(side)
            self._captured = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._captured), torch.no_grad():
                self._outputs = _execute(g, dict(self._static))

    def buffer(self, vid: ValueId) -> torch.Tensor:
        return self._static[vid]

    def __call__(self, updates: Optional[Dict[ValueId, torch.Tensor]] = None) -> List[torch.Tensor]:
        for vid, t in (updates or {}).items():
            self._static[vid].copy_(t, non_blocking=True)
        if self._captured is not None:
            self._captured.replay()
            return self._outputs
        with torch.no_grad():
            self._outputs = _execute(self.graph, dict(self._static))
        return self._outputs
