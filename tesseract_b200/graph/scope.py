"""``GraphScope``: while one is live on a thread, every tensor op executed eagerly is also appended to its ``Graph``
(the reference's ``graph::maybe_record`` hook called from every op entry point,
include/tesseract/graph/GraphScope.hpp:42-102, src/graph/GraphScope.cpp). Here the hook is a
``TorchFunctionMode``: torch hands every public tensor function to it, the scope runs the function, and records
the matching dialect op. ``torch.nn.functional.linear`` is decomposed the way the reference's ``Linear`` runs
(``matmul(x, transpose(W))`` then a broadcast add of the bias, src/nn/Linear.cpp:63-83), so the recorded graph
only holds ops that the interpreter and the backward transform know.

Tensors are keyed by identity and pinned for the life of the scope, so an id is never reused for another tensor.
"""
from __future__ import annotations

import threading
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F
from torch.overrides import TorchFunctionMode

from .ir import Graph, ValueId, ValueKind, kInvalidValueId

_tls = threading.local()


def active_scope() -> Optional["GraphScope"]:
    return getattr(_tls, "scope", None)


def is_recording() -> bool:
    return active_scope() is not None


def _norm_dim(dim: int, rank: int) -> int:
    return dim + rank if dim < 0 else dim


class _Recorder(TorchFunctionMode):
    def __init__(self, scope: "GraphScope"):
        super().__init__()
        self.scope = scope

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        handler = _HANDLERS.get(func)
        if handler is not None:
            return handler(self.scope, *args, **kwargs)
        out = func(*args, **kwargs)
        if isinstance(out, torch.Tensor) and func not in _PASSTHROUGH:
            touched = [a for a in list(args) + list(kwargs.values())
                       if isinstance(a, torch.Tensor) and id(a) in self.scope.value_of]
            if touched:
                name = getattr(func, "__qualname__", None) or getattr(func, "__name__", str(func))
                raise NotImplementedError(f"GraphScope: '{name}' has no graph op; the scope records only ops that the "
                                          "interpreter can replay")
        return out


class GraphScope:
    """``with GraphScope() as scope:`` ... run eager code ... ``scope.mark_output(y)``; the result is ``scope.graph``.
    Nesting is rejected, as in the reference (tests/graph/test_graph_smoke.cpp:119)."""

    def __init__(self):
        self.graph = Graph()
        self.value_of: Dict[int, ValueId] = {}
        self.pinned: List[torch.Tensor] = []
        self._mode: Optional[_Recorder] = None

    def __enter__(self) -> "GraphScope":
        if active_scope() is not None:
            raise RuntimeError("GraphScope: a scope is already recording on this thread; scopes do not nest")
        _tls.scope = self
        self._mode = _Recorder(self)
        self._mode.__enter__()
        return self

    def __exit__(self, *exc):
        self._mode.__exit__(*exc)
        self._mode = None
        _tls.scope = None
        return False

    # ---- bindings ----------------------------------------------------------------------------------------------
    def _bind(self, t: torch.Tensor, kind: ValueKind, name: str) -> ValueId:
        key = id(t)
        if key in self.value_of:
            return self.value_of[key]      # the kind of an already bound tensor is not upgraded
        g = self.graph
        if kind == ValueKind.PARAM:
            vid = g.add_param(t.shape, t.dtype, t.device, name)
        elif kind == ValueKind.CONSTANT:
            vid = g.add_constant(t.shape, t.dtype, t.device, name, data=t.detach())
        elif kind == ValueKind.INPUT:
            vid = g.add_input(t.shape, t.dtype, t.device, name)
        else:
            vid = g.new_value(t.shape, t.dtype, t.device, kind, name)
        self.value_of[key] = vid
        self.pinned.append(t)
        return vid

    def bind_input(self, t: torch.Tensor, name: str = "") -> ValueId:
        return self._bind(t, ValueKind.INPUT, name)

    def bind_param(self, t: torch.Tensor, name: str = "") -> ValueId:
        return self._bind(t, ValueKind.PARAM, name)

    def bind_constant(self, t: torch.Tensor, name: str = "") -> ValueId:
        return self._bind(t, ValueKind.CONSTANT, name)

    def bind_module(self, module: torch.nn.Module, prefix: str = "") -> Dict[str, ValueId]:
        """Binds every parameter of ``module`` as a graph param under its dotted name."""
        return {n: self.bind_param(p, prefix + n.replace(".", "_")) for n, p in module.named_parameters()}

    def value_id_of(self, t: torch.Tensor) -> ValueId:
        return self.value_of.get(id(t), kInvalidValueId)

    def ensure_value(self, t: torch.Tensor, kind: ValueKind = ValueKind.INPUT) -> ValueId:
        return self._bind(t, kind, "")

    def mark_output(self, t: torch.Tensor) -> None:
        vid = self.value_id_of(t)
        if vid == kInvalidValueId:
            raise ValueError("GraphScope.mark_output: the tensor was not produced or bound inside this scope")
        self.graph.mark_output(vid)

    def record(self, kind: str, inputs: Sequence[torch.Tensor], outputs: Sequence[torch.Tensor], attrs=None) -> int:
        ins = [self.ensure_value(t) for t in inputs]
        outs = [self._bind(t, ValueKind.INTERMEDIATE, "") for t in outputs]
        return self.graph.add_op(kind, ins, outs, attrs)

    def trace(self, fn: Callable, *example_inputs: torch.Tensor, names: Optional[Sequence[str]] = None) -> Graph:
        """Runs ``fn`` on the example inputs inside this (entered) scope: inputs are bound in order, the parameters
        of a module are bound as params, and the result (a tensor or a sequence of tensors) becomes the outputs."""
        if active_scope() is not self:
            raise RuntimeError("GraphScope.trace: enter the scope first (with GraphScope() as scope: ...)")
        for i, x in enumerate(example_inputs):
            self.bind_input(x, names[i] if names else "")
        if isinstance(fn, torch.nn.Module):
            self.bind_module(fn)
        out = fn(*example_inputs)
        for y in (out if isinstance(out, (tuple, list)) else (out,)):
            self.mark_output(y)
        return self.graph


def maybe_record(kind: str, inputs, outputs, attrs=None) -> int:
    """Module-level hook for hand-written ops: records into the active scope, or returns -1 outside one."""
    s = active_scope()
    return -1 if s is None else s.record(kind, inputs, outputs, attrs)


# ---- handlers: run the op with recording off (torch disables the mode inside its handler), then record ----------

def _as_tensor_like(scope: GraphScope, x, like: torch.Tensor) -> torch.Tensor:
    """A python scalar operand becomes a 0-d constant of the other operand's dtype and device."""
    if isinstance(x, torch.Tensor):
        return x
    t = torch.tensor(x, dtype=like.dtype if like.is_floating_point() or not isinstance(x, float) else torch.float32,
                     device=like.device)
    scope.bind_constant(t)
    return t


def _binary(kind: str, fn):
    def h(scope, a, b, **kw):
        if kw.get("alpha", 1) != 1:
            raise NotImplementedError(f"GraphScope: {kind} with alpha != 1 has no graph op")
        like = a if isinstance(a, torch.Tensor) else b
        a, b = _as_tensor_like(scope, a, like), _as_tensor_like(scope, b, like)
        out = fn(a, b)
        scope.record(kind, [a, b], [out])
        return out
    return h


def _rbinary(kind: str, fn):
    def h(scope, a, b):
        return _binary(kind, fn)(scope, b, a)
    return h


def _unary(kind: str, fn):
    def h(scope, x, **kw):
        if kw.get("inplace"):
            raise NotImplementedError(f"GraphScope: in-place {kind} has no graph op")
        out = fn(x)
        scope.record(kind, [x], [out])
        return out
    return h


def _reduce(kind: str, fn):
    def h(scope, x, dim=None, keepdim=False, **kw):
        if kw.get("dtype") is not None:
            raise NotImplementedError(f"GraphScope: {kind} with a dtype argument has no graph op")
        if dim is None:
            out = fn(x)
            scope.record(kind, [x], [out])
            return out
        if isinstance(dim, (tuple, list)):
            if len(dim) != 1:
                raise NotImplementedError(f"GraphScope: {kind} over several dims has no graph op")
            dim = dim[0]
        d = _norm_dim(int(dim), x.dim())
        out = fn(x, d, keepdim)
        res = out[0] if kind == "max" else out       # torch.max(x, dim) returns (values, indices)
        scope.record(kind, [x], [res], {"dim": d, "keepdim": bool(keepdim)})
        return out
    return h


def _h_matmul(scope, a, b):
    out = torch.matmul(a, b)
    scope.record("matmul", [a, b], [out])
    return out


def _h_linear(scope, x, w, bias=None):
    wt = w.transpose(0, 1)
    scope.record("transpose", [w], [wt], {"dim_a": 0, "dim_b": 1})
    y = torch.matmul(x, wt)
    scope.record("matmul", [x, wt], [y])
    if bias is None:
        return y
    bb = bias.broadcast_to(y.shape)
    scope.record("broadcast_to", [bias], [bb], {"shape": list(y.shape)})
    out = y + bb
    scope.record("add", [y, bb], [out])
    return out


def _h_softmax(scope, x, dim=-1, **kw):
    if kw.get("dtype") is not None:
        raise NotImplementedError("GraphScope: softmax with a dtype argument has no graph op")
    d = _norm_dim(int(dim), x.dim())
    out = torch.softmax(x, d)
    scope.record("softmax", [x], [out], {"dim": d})
    return out


def _shape_arg(args) -> List[int]:
    if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)):
        return [int(s) for s in args[0]]
    return [int(s) for s in args]


def _h_reshape(kind: str):
    def h(scope, x, *shape):
        out = x.reshape(_shape_arg(shape)) if kind == "reshape" else x.view(_shape_arg(shape))
        scope.record(kind, [x], [out], {"shape": list(out.shape)})
        return out
    return h


def _h_flatten(scope, x, start_dim=0, end_dim=-1):
    out = torch.flatten(x, start_dim, end_dim)
    scope.record("reshape", [x], [out], {"shape": list(out.shape)})
    return out


def _h_permute(scope, x, *axes):
    ax = [_norm_dim(a, x.dim()) for a in _shape_arg(axes)]
    out = x.permute(ax)
    scope.record("permute", [x], [out], {"axes": ax})
    return out


def _h_transpose(scope, x, dim_a, dim_b):
    a, b = _norm_dim(int(dim_a), x.dim()), _norm_dim(int(dim_b), x.dim())
    out = x.transpose(a, b)
    scope.record("transpose", [x], [out], {"dim_a": a, "dim_b": b})
    return out


def _h_t(scope, x):
    if x.dim() != 2:
        raise NotImplementedError("GraphScope: Tensor.t() of a tensor that is not 2-D has no graph op")
    return _h_transpose(scope, x, 0, 1)


def _h_broadcast(scope, x, *shape):
    target = _shape_arg(shape)
    full = [x.shape[i - (len(target) - x.dim())] if s == -1 else s for i, s in enumerate(target)]
    out = x.broadcast_to(full)
    scope.record("broadcast_to", [x], [out], {"shape": list(out.shape)})
    return out


def _h_cross_entropy(scope, logits, targets, **kw):
    extra = {k: v for k, v in kw.items() if v is not None}
    if extra.get("reduction", "mean") != "mean" or extra.get("label_smoothing", 0.0) != 0.0 or "weight" in extra \
            or extra.get("ignore_index", -100) != -100:
        raise NotImplementedError("GraphScope: cross_entropy records only the mean over rows with integer targets")
    if logits.dim() != 2 or targets.dtype != torch.int64:
        raise NotImplementedError("GraphScope: cross_entropy_with_logits wants [N, C] logits and int64 targets")
    out = F.cross_entropy(logits, targets)
    scope.record("cross_entropy_with_logits", [logits, targets], [out])
    return out


_T = torch.Tensor
_HANDLERS = {}
for _fns, _h in (
    ((torch.add, _T.add, _T.__add__), _binary("add", torch.add)),
    ((_T.__radd__,), _rbinary("add", torch.add)),
    ((torch.sub, _T.sub, _T.__sub__), _binary("sub", torch.sub)),
    ((_T.__rsub__,), _rbinary("sub", torch.sub)),
    ((torch.mul, _T.mul, _T.__mul__), _binary("mul", torch.mul)),
    ((_T.__rmul__,), _rbinary("mul", torch.mul)),
    ((torch.div, _T.div, _T.__truediv__, torch.true_divide, _T.true_divide), _binary("div", torch.true_divide)),
    ((_T.__rtruediv__,), _rbinary("div", torch.true_divide)),
    ((torch.neg, _T.neg, _T.__neg__, torch.negative), _unary("neg", torch.neg)),
    ((torch.relu, _T.relu, F.relu), _unary("relu", torch.relu)),
    ((torch.sigmoid, _T.sigmoid, F.sigmoid), _unary("sigmoid", torch.sigmoid)),
    ((torch.tanh, _T.tanh, F.tanh), _unary("tanh", torch.tanh)),
    ((torch.exp, _T.exp), _unary("exp", torch.exp)),
    ((torch.log, _T.log), _unary("log", torch.log)),
    ((torch.clone, _T.clone), _unary("clone", torch.clone)),
    ((_T.contiguous,), _unary("contiguous", lambda x: x.contiguous())),
    ((torch.sum, _T.sum), _reduce("sum", torch.sum)),
    ((torch.mean, _T.mean), _reduce("mean", torch.mean)),
    ((torch.max, _T.max, torch.amax, _T.amax), None),
    ((torch.matmul, _T.matmul, _T.__matmul__, torch.mm, _T.mm), _h_matmul),
    ((F.linear,), _h_linear),
    ((torch.softmax, _T.softmax, F.softmax), _h_softmax),
    ((torch.reshape, _T.reshape), _h_reshape("reshape")),
    ((_T.view,), _h_reshape("view")),
    ((torch.flatten, _T.flatten), _h_flatten),
    ((torch.permute, _T.permute), _h_permute),
    ((torch.transpose, _T.transpose), _h_transpose),
    ((_T.t, torch.t), _h_t),
    ((torch.broadcast_to, _T.broadcast_to, _T.expand), _h_broadcast),
    ((F.cross_entropy,), _h_cross_entropy),
):
    for _f in _fns:
        if _h is not None:
            _HANDLERS[_f] = _h


def _h_max(scope, x, dim=None, keepdim=False):
    if isinstance(dim, torch.Tensor):
        raise NotImplementedError("GraphScope: elementwise max of two tensors has no graph op")
    return _reduce("max", torch.max)(scope, x, dim, keepdim)


def _h_amax(scope, x, dim=None, keepdim=False):
    if dim is None:
        return _reduce("max", torch.max)(scope, x)
    d = _norm_dim(int(dim if not isinstance(dim, (tuple, list)) else dim[0]), x.dim())
    out = torch.amax(x, d, keepdim)
    scope.record("max", [x], [out], {"dim": d, "keepdim": bool(keepdim)})
    return out


_HANDLERS[torch.max] = _HANDLERS[_T.max] = _h_max
_HANDLERS[torch.amax] = _HANDLERS[_T.amax] = _h_amax

def _alias(fn):
    """Functions whose result is the same value (detach, a no-op conversion): the result shares the ValueId."""
    def h(scope, x, *a, **kw):
        out = fn(x, *a, **kw)
        vid = scope.value_id_of(x)
        if vid != kInvalidValueId and out is not x:
            if out.dtype != x.dtype or out.device != x.device:
                raise NotImplementedError("GraphScope: dtype / device conversions of recorded values have no graph op")
            scope.value_of[id(out)] = vid
            scope.pinned.append(out)
        return out
    return h


for _f in (_T.detach, _T.to, _T.float, _T.double, _T.cpu, _T.cuda, _T.type_as, _T.requires_grad_):
    _HANDLERS[_f] = _alias(_f)

#: tensor-returning functions that build fresh tensors (no data flow from recorded values)
_PASSTHROUGH = {torch.zeros_like, torch.ones_like, torch.empty_like, _T.new_zeros, _T.new_ones, _T.new_empty,
                _T.new_full, torch.tensor, torch.as_tensor, _T.grad.__get__}
