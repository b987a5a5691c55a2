"""SSA graph IR: ``Graph`` is a list of ``Op``s over ``Value``s. Values carry (shape, dtype, device) metadata and a
stable integer id; they hold no storage. Op mnemonics are the names of the reference's ``tesseract`` dialect
(``add``, ``matmul``, ``reshape`` ...), so a graph prints and round-trips under those names.

Reference: include/tesseract/graph/Graph.hpp:26-98, include/tesseract/graph/Value.hpp:29-58, src/graph/Graph.cpp.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

ValueId = int
kInvalidValueId = -1

#: attribute values are: int, float, bool, str, list of int (the reference's ``Attr`` variant)
Attr = Any


class ValueKind(enum.IntEnum):
    INTERMEDIATE = 0
    INPUT = 1
    PARAM = 2       # graph-level input that accumulates a gradient in ``build_backward``
    CONSTANT = 3


@dataclass
class Value:
    id: ValueId
    shape: Tuple[int, ...]
    dtype: torch.dtype
    device: torch.device
    kind: ValueKind = ValueKind.INTERMEDIATE
    name: str = ""


@dataclass
class Op:
    kind: str
    inputs: List[ValueId]
    outputs: List[ValueId]
    attrs: Dict[str, Attr] = field(default_factory=dict)


_DTYPE_NAMES = {torch.float32: "f32", torch.float64: "f64", torch.float16: "f16", torch.bfloat16: "bf16",
                torch.int64: "i64", torch.int32: "i32", torch.int8: "i8", torch.uint8: "ui8", torch.bool: "i1"}
_DTYPE_OF_NAME = {v: k for k, v in _DTYPE_NAMES.items()}


def dtype_name(dt: torch.dtype) -> str:
    try:
        return _DTYPE_NAMES[dt]
    except KeyError:
        raise NotImplementedError(f"graph IR: no element type name for {dt}") from None


def dtype_of_name(name: str) -> torch.dtype:
    try:
        return _DTYPE_OF_NAME[name]
    except KeyError:
        raise ValueError(f"graph IR: unknown element type '{name}'") from None


class Graph:
    def __init__(self):
        self._values: List[Value] = []
        self._ops: List[Op] = []
        self._inputs: List[ValueId] = []
        self._outputs: List[ValueId] = []
        self._params: List[ValueId] = []
        self._constants: List[ValueId] = []
        #: tensors of constants created while recording (python scalars, literal tensors); ``run`` binds them
        #: when the caller does not
        self.constant_data: Dict[ValueId, torch.Tensor] = {}

    # ---- construction ------------------------------------------------------------------------------------------
    def new_value(self, shape: Sequence[int], dtype: torch.dtype, device, kind: ValueKind = ValueKind.INTERMEDIATE,
                  name: str = "") -> ValueId:
        vid = len(self._values)
        self._values.append(Value(vid, tuple(int(s) for s in shape), dtype, torch.device(device), kind, name))
        return vid

    def add_input(self, shape, dtype, device, name: str = "") -> ValueId:
        vid = self.new_value(shape, dtype, device, ValueKind.INPUT, name)
        self._inputs.append(vid)
        return vid

    def add_param(self, shape, dtype, device, name: str = "") -> ValueId:
        vid = self.new_value(shape, dtype, device, ValueKind.PARAM, name)
        self._params.append(vid)
        return vid

    def add_constant(self, shape, dtype, device, name: str = "", data: Optional[torch.Tensor] = None) -> ValueId:
        vid = self.new_value(shape, dtype, device, ValueKind.CONSTANT, name)
        self._constants.append(vid)
        if data is not None:
            self.constant_data[vid] = data
        return vid

    def mark_output(self, vid: ValueId) -> None:
        self.value(vid)
        self._outputs.append(vid)

    def add_op(self, kind: str, inputs: Sequence[ValueId], outputs: Sequence[ValueId],
               attrs: Optional[Dict[str, Attr]] = None) -> int:
        for v in list(inputs) + list(outputs):
            self.value(v)
        self._ops.append(Op(kind, list(inputs), list(outputs), dict(attrs or {})))
        return len(self._ops) - 1

    # ---- accessors ---------------------------------------------------------------------------------------------
    @property
    def values(self) -> List[Value]:
        return self._values

    @property
    def ops(self) -> List[Op]:
        return self._ops

    @property
    def inputs(self) -> List[ValueId]:
        return self._inputs

    @property
    def outputs(self) -> List[ValueId]:
        return self._outputs

    @property
    def params(self) -> List[ValueId]:
        return self._params

    @property
    def constants(self) -> List[ValueId]:
        return self._constants

    def value(self, vid: ValueId) -> Value:
        if not (0 <= vid < len(self._values)):
            raise IndexError(f"graph IR: value id {vid} out of range (graph has {len(self._values)} values)")
        return self._values[vid]

    def num_values(self) -> int:
        return len(self._values)

    def num_ops(self) -> int:
        return len(self._ops)

    def __len__(self) -> int:
        return len(self._ops)

    def op_kinds(self) -> List[str]:
        return [o.kind for o in self._ops]

    # ---- printing ----------------------------------------------------------------------------------------------
    def _type_str(self, vid: ValueId) -> str:
        v = self._values[vid]
        dims = "x".join(str(d) for d in v.shape)
        return f"tensor<{dims + 'x' if dims else ''}{dtype_name(v.dtype)}>"

    def _ref(self, vid: ValueId) -> str:
        v = self._values[vid]
        return f"%{v.name}" if v.name else f"%{vid}"

    def to_string(self) -> str:
        """Stable, human-readable listing (close to MLIR's look, not its grammar)."""
        lines = ["graph {"]
        for title, ids in (("input", self._inputs), ("param", self._params), ("const", self._constants)):
            for vid in ids:
                lines.append(f"  {title} {self._ref(vid)} : {self._type_str(vid)}")
        for op in self._ops:
            outs = ", ".join(self._ref(o) for o in op.outputs)
            ins = ", ".join(self._ref(i) for i in op.inputs)
            attrs = ""
            if op.attrs:
                attrs = " {" + ", ".join(f"{k} = {op.attrs[k]!r}" for k in sorted(op.attrs)) + "}"
            types = ", ".join(self._type_str(o) for o in op.outputs)
            lines.append(f"  {outs} = {op.kind}({ins}){attrs} : {types}")
        lines.append("  return " + ", ".join(self._ref(o) for o in self._outputs))
        lines.append("}")
        return "\n".join(lines)

    __str__ = to_string
