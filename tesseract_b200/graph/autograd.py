"""Reverse-mode differentiation as a graph transform: ``build_backward(g)`` appends the backward ops to ``g`` itself
(src/graph/Autograd.cpp, contract in include/tesseract/graph/Autograd.hpp:12-31).

On return ``g`` has one new input per original output (its cotangent, same shape / dtype / device) and one new
output per param, in ``g.params`` order (plus one per entry of ``wrt`` when given). A param that the forward graph
never uses gets a zero gradient, emitted as ``sub(p, p)``. The rule table covers the reference's set (add, sub,
mul, neg, matmul, sum, mean, transpose, broadcast_to, relu, cross_entropy_with_logits) and the rest of the
interpreter's differentiable ops (div, sigmoid, tanh, exp, log, softmax, reshape / view, permute, contiguous,
clone, reduce_to_shape). ``max`` has no rule, as in the reference's tape (src/ops/cpu/Reduction.cpp:338-346).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch

from .ir import Graph, Op, ValueId, ValueKind


@dataclass
class BackwardResult:
    cotangents: List[ValueId]
    dparams: List[ValueId]
    dinputs: List[ValueId] = field(default_factory=list)


class _Builder:
    def __init__(self, g: Graph):
        self.g = g
        self.grad: Dict[ValueId, ValueId] = {}

    # ---- emitters ----------------------------------------------------------------------------------------------
    def emit(self, kind: str, ins: Sequence[ValueId], shape, like: ValueId, attrs=None) -> ValueId:
        v = self.g.value(like)
        out = self.g.new_value(shape, v.dtype, v.device)
        self.g.add_op(kind, list(ins), [out], attrs)
        return out

    def shape(self, vid: ValueId):
        return self.g.value(vid).shape

    def binary(self, kind: str, a: ValueId, b: ValueId) -> ValueId:
        shape = torch.broadcast_shapes(self.shape(a), self.shape(b))
        return self.emit(kind, [a, b], shape, a)

    def unary(self, kind: str, x: ValueId) -> ValueId:
        return self.emit(kind, [x], self.shape(x), x)

    def transpose(self, x: ValueId, a: int, b: int) -> ValueId:
        s = list(self.shape(x))
        s[a], s[b] = s[b], s[a]
        return self.emit("transpose", [x], s, x, {"dim_a": a, "dim_b": b})

    def reshape(self, x: ValueId, shape) -> ValueId:
        if tuple(shape) == self.shape(x):
            return x
        return self.emit("reshape", [x], shape, x, {"shape": [int(s) for s in shape]})

    def broadcast_to(self, x: ValueId, shape) -> ValueId:
        if tuple(shape) == self.shape(x):
            return x
        return self.emit("broadcast_to", [x], shape, x, {"shape": [int(s) for s in shape]})

    def reduce_to(self, x: ValueId, shape) -> ValueId:
        if tuple(shape) == self.shape(x):
            return x
        return self.emit("reduce_to_shape", [x], shape, x, {"shape": [int(s) for s in shape]})

    def scalar(self, value: float, like: ValueId) -> ValueId:
        v = self.g.value(like)
        return self.g.add_constant((), v.dtype, v.device, data=torch.tensor(value, dtype=v.dtype, device=v.device))

    def matmul(self, a: ValueId, b: ValueId) -> ValueId:
        sa, sb = self.shape(a), self.shape(b)
        batch = torch.broadcast_shapes(sa[:-2], sb[:-2])
        return self.emit("matmul", [a, b], tuple(batch) + (sa[-2], sb[-1]), a)

    # ---- accumulation ------------------------------------------------------------------------------------------
    def accumulate(self, vid: ValueId, g: ValueId) -> None:
        if not self.g.value(vid).dtype.is_floating_point:
            return
        g = self.reduce_to(g, self.shape(vid))
        self.grad[vid] = g if vid not in self.grad else self.binary("add", self.grad[vid], g)


def _r_add(b: _Builder, op: Op, g: ValueId):
    b.accumulate(op.inputs[0], g)
    b.accumulate(op.inputs[1], g)


def _r_sub(b, op, g):
    b.accumulate(op.inputs[0], g)
    b.accumulate(op.inputs[1], b.unary("neg", g))


def _r_mul(b, op, g):
    x, y = op.inputs
    b.accumulate(x, b.binary("mul", g, y))
    b.accumulate(y, b.binary("mul", g, x))


def _r_div(b, op, g):
    x, y = op.inputs
    b.accumulate(x, b.binary("div", g, y))
    q = b.binary("div", op.outputs[0], y)           # x / y^2
    b.accumulate(y, b.unary("neg", b.binary("mul", g, q)))


def _r_neg(b, op, g):
    b.accumulate(op.inputs[0], b.unary("neg", g))


def _r_matmul(b, op, g):
    x, w = op.inputs
    sx, sw = b.shape(x), b.shape(w)
    if len(sx) < 2 or len(sw) < 2:
        raise NotImplementedError("build_backward: matmul of a 1-D operand has no rule")
    wt = b.transpose(w, len(sw) - 2, len(sw) - 1)
    b.accumulate(x, b.matmul(g, wt))
    if len(sw) == 2 and len(sx) > 2:                # [.., M, K] @ [K, N]: fold the batch into the rows
        x2 = b.reshape(x, (_prod(sx[:-1]), sx[-1]))
        g2 = b.reshape(g, (_prod(sx[:-1]), sw[-1]))
        b.accumulate(w, b.matmul(b.transpose(x2, 0, 1), g2))
    else:
        xt = b.transpose(x, len(sx) - 2, len(sx) - 1)
        b.accumulate(w, b.matmul(xt, g))


def _prod(xs) -> int:
    n = 1
    for x in xs:
        n *= int(x)
    return n


def _reduce_cotangent(b, op, g) -> ValueId:
    """Brings the cotangent of a sum / mean back to the input's shape."""
    x = op.inputs[0]
    sx = b.shape(x)
    if "dim" in op.attrs and not op.attrs.get("keepdim", False):
        keep = list(sx)
        keep[int(op.attrs["dim"])] = 1
        g = b.reshape(g, keep)
    return b.broadcast_to(g, sx)


def _r_sum(b, op, g):
    b.accumulate(op.inputs[0], _reduce_cotangent(b, op, g))


def _r_mean(b, op, g):
    x = op.inputs[0]
    sx = b.shape(x)
    n = sx[int(op.attrs["dim"])] if "dim" in op.attrs else _prod(sx)
    full = _reduce_cotangent(b, op, g)
    b.accumulate(x, b.binary("mul", full, b.scalar(1.0 / max(n, 1), x)))


def _r_transpose(b, op, g):
    b.accumulate(op.inputs[0], b.transpose(g, int(op.attrs["dim_a"]), int(op.attrs["dim_b"])))


def _r_permute(b, op, g):
    axes = [int(a) for a in op.attrs["axes"]]
    inv = [0] * len(axes)
    for i, a in enumerate(axes):
        inv[a] = i
    x = op.inputs[0]
    b.accumulate(x, b.emit("permute", [g], b.shape(x), x, {"axes": inv}))


def _r_reshape(b, op, g):
    x = op.inputs[0]
    b.accumulate(x, b.reshape(g, b.shape(x)))


def _r_identity(b, op, g):
    b.accumulate(op.inputs[0], g)


def _r_broadcast_to(b, op, g):
    x = op.inputs[0]
    b.accumulate(x, b.reduce_to(g, b.shape(x)))


def _r_reduce_to_shape(b, op, g):
    x = op.inputs[0]
    b.accumulate(x, b.broadcast_to(g, b.shape(x)))


def _r_relu(b, op, g):
    x = op.inputs[0]
    b.accumulate(x, b.emit("relu_backward", [g, x], b.shape(x), x))


def _r_sigmoid(b, op, g):
    y = op.outputs[0]
    b.accumulate(op.inputs[0], b.binary("mul", g, b.binary("sub", y, b.binary("mul", y, y))))


def _r_tanh(b, op, g):
    y = op.outputs[0]
    b.accumulate(op.inputs[0], b.binary("sub", g, b.binary("mul", g, b.binary("mul", y, y))))


def _r_exp(b, op, g):
    b.accumulate(op.inputs[0], b.binary("mul", g, op.outputs[0]))


def _r_log(b, op, g):
    b.accumulate(op.inputs[0], b.binary("div", g, op.inputs[0]))


def _r_softmax(b, op, g):
    x, y = op.inputs[0], op.outputs[0]
    d = int(op.attrs["dim"])
    gy = b.binary("mul", g, y)
    keep = list(b.shape(x))
    keep[d] = 1
    s = b.emit("sum", [gy], keep, x, {"dim": d, "keepdim": True})
    b.accumulate(x, b.binary("mul", y, b.binary("sub", g, b.broadcast_to(s, b.shape(x)))))


def _r_cross_entropy(b, op, g):
    logits, targets = op.inputs
    b.accumulate(logits, b.emit("cross_entropy_with_logits_backward", [logits, targets, g], b.shape(logits), logits))


_RULES: Dict[str, Callable] = {
    "add": _r_add, "sub": _r_sub, "mul": _r_mul, "div": _r_div, "neg": _r_neg, "matmul": _r_matmul,
    "sum": _r_sum, "mean": _r_mean, "transpose": _r_transpose, "permute": _r_permute, "reshape": _r_reshape,
    "view": _r_reshape, "contiguous": _r_identity, "clone": _r_identity, "broadcast_to": _r_broadcast_to,
    "reduce_to_shape": _r_reduce_to_shape, "relu": _r_relu, "sigmoid": _r_sigmoid, "tanh": _r_tanh, "exp": _r_exp,
    "log": _r_log, "softmax": _r_softmax, "cross_entropy_with_logits": _r_cross_entropy,
}


def differentiable_ops() -> List[str]:
    return sorted(_RULES)


def build_backward(g: Graph, wrt: Optional[Sequence[ValueId]] = None) -> BackwardResult:
    """Extends ``g`` in place with its backward pass and returns the new value ids."""
    forward_ops = list(g.ops)
    outputs = list(g.outputs)
    if not outputs:
        raise ValueError("build_backward: the graph has no outputs")
    b = _Builder(g)
    cotangents = []
    for i, o in enumerate(outputs):
        v = g.value(o)
        ct = g.add_input(v.shape, v.dtype, v.device, f"ct{i}")
        cotangents.append(ct)
        b.grad[o] = ct if o not in b.grad else b.binary("add", b.grad[o], ct)
    for op in reversed(forward_ops):
        gy = b.grad.get(op.outputs[0])
        if gy is None:
            continue                                   # this op does not reach any output
        rule = _RULES.get(op.kind)
        if rule is None:
            raise NotImplementedError(f"build_backward: op '{op.kind}' has no backward rule")
        rule(b, op, gy)

    def grad_of(vid: ValueId) -> ValueId:
        if vid in b.grad:
            return b.grad[vid]
        return b.emit("sub", [vid, vid], b.shape(vid), vid)      # zero gradient placeholder

    dparams = [grad_of(p) for p in g.params]
    dinputs = [grad_of(i) for i in (wrt or [])]
    for vid in dparams + dinputs:
        g.mark_output(vid)
    return BackwardResult(cotangents, dparams, dinputs)
