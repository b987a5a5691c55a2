"""Text form of a ``Graph`` in MLIR's generic operation syntax under the ``tesseract`` dialect namespace
(op names as in src/ir/TesseractOps.td:30-456): one ``func.func @main`` whose arguments are the graph's inputs,
params and constants in that order, one ``"tesseract.<kind>"(...)`` line per op, one ``return``. ``parse_mlir``
reads that form back, so a graph round-trips through text; the dialect definition, its passes and the JIT engines
of the reference (src/ir) are not part of this framework -- the generic syntax needs none of them to be well formed.
"""
from __future__ import annotations

import re
from typing import Dict, List, Tuple

import torch

from .ir import Graph, ValueId, ValueKind, dtype_name, dtype_of_name

_ROLE_ATTR = {ValueKind.INPUT: "input", ValueKind.PARAM: "param", ValueKind.CONSTANT: "constant"}


def _type(g: Graph, vid: ValueId) -> str:
    v = g.value(vid)
    dims = "".join(f"{d}x" for d in v.shape)
    return f"tensor<{dims}{dtype_name(v.dtype)}>"


def _attr(v) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return f"{v} : i64"
    if isinstance(v, float):
        return f"{v!r} : f64"
    if isinstance(v, str):
        return '"' + v.replace("\\", "\\\\").replace('"', '\\"') + '"'
    if isinstance(v, (list, tuple)):
        return "array<i64" + (": " + ", ".join(str(int(x)) for x in v) if len(v) else "") + ">"
    raise TypeError(f"emit_mlir: attribute value {v!r} has no MLIR form")


def emit_mlir(g: Graph) -> str:
    args = list(g.inputs) + list(g.params) + list(g.constants)
    name: Dict[ValueId, str] = {vid: f"%arg{i}" for i, vid in enumerate(args)}
    sig = ", ".join(f'{name[vid]}: {_type(g, vid)} {{tesseract.role = "{_ROLE_ATTR[g.value(vid).kind]}"'
                    + (f', tesseract.name = "{g.value(vid).name}"' if g.value(vid).name else "") + "}" for vid in args)
    res = ", ".join(_type(g, o) for o in g.outputs)
    lines = ["module {", f"  func.func @main({sig}) -> ({res}) {{"]
    n = 0
    for op in g.ops:
        for o in op.outputs:
            name[o] = f"%{n}"
            n += 1
        outs = ", ".join(name[o] for o in op.outputs)
        try:
            ins = ", ".join(name[i] for i in op.inputs)
        except KeyError as e:
            raise ValueError(f"emit_mlir: op '{op.kind}' uses value {e.args[0]} that is neither an argument nor defined "
                             "by an earlier op") from None
        attrs = ""
        if op.attrs:
            attrs = " {" + ", ".join(f"{k} = {_attr(op.attrs[k])}" for k in sorted(op.attrs)) + "}"
        in_t = ", ".join(_type(g, i) for i in op.inputs)
        out_t = ", ".join(_type(g, o) for o in op.outputs)
        out_t = out_t if len(op.outputs) == 1 else f"({out_t})"
        lines.append(f'    {outs} = "tesseract.{op.kind}"({ins}){attrs} : ({in_t}) -> {out_t}')
    lines.append("    return " + ", ".join(name[o] for o in g.outputs) + " : " + res)
    lines += ["  }", "}"]
    return "\n".join(lines) + "\n"


_TENSOR = re.compile(r"tensor<((?:\d+x)*)([a-z0-9]+)>")
_ARG = re.compile(r"(%arg\d+): (tensor<[^>]*>) \{([^}]*)\}")
_OP = re.compile(r'^\s*((?:%\d+(?:, )?)+) = "tesseract\.([a-z_0-9]+)"\(([^)]*)\)(?: \{(.*)\})? : \((.*)\) -> (.*)$')


def _parse_type(text: str) -> Tuple[Tuple[int, ...], torch.dtype]:
    m = _TENSOR.fullmatch(text.strip())
    if not m:
        raise ValueError(f"parse_mlir: cannot read the type '{text}'")
    dims = tuple(int(d) for d in m.group(1).split("x") if d)
    return dims, dtype_of_name(m.group(2))


def _split_top(text: str) -> List[str]:
    """Splits on commas that are outside <...> and quotes."""
    parts, depth, cur, quoted = [], 0, "", False
    for ch in text:
        if ch == '"':
            quoted = not quoted
        if not quoted:
            if ch == "<":
                depth += 1
            elif ch == ">":
                depth -= 1
            elif ch == "," and depth == 0:
                parts.append(cur.strip())
                cur = ""
                continue
        cur += ch
    if cur.strip():
        parts.append(cur.strip())
    return parts


def _parse_attr(text: str):
    text = text.strip()
    if text in ("true", "false"):
        return text == "true"
    if text.startswith('"'):
        return text[1:-1].replace('\\"', '"').replace("\\\\", "\\")
    if text.startswith("array<i64"):
        body = text[len("array<i64"):-1].lstrip(":").strip()
        return [int(x) for x in body.split(",")] if body else []
    value, _, ty = text.rpartition(" : ")
    return int(value) if ty == "i64" else float(value)


def parse_mlir(text: str, device="cpu") -> Graph:
    """Reads the form that ``emit_mlir`` writes. Constants come back without their data."""
    g = Graph()
    ids: Dict[str, ValueId] = {}
    lines = text.splitlines()
    head = next((l for l in lines if "func.func @main" in l), None)
    if head is None:
        raise ValueError("parse_mlir: no func.func @main")
    for m in _ARG.finditer(head):
        shape, dt = _parse_type(m.group(2))
        meta = dict(re.findall(r'tesseract\.(\w+) = "([^"]*)"', m.group(3)))
        add = {"input": g.add_input, "param": g.add_param, "constant": g.add_constant}[meta.get("role", "input")]
        ids[m.group(1)] = add(shape, dt, device, meta.get("name", ""))
    for line in lines:
        s = line.strip()
        if s.startswith("return"):
            names = s[len("return"):].split(" : ")[0]
            for nme in names.split(","):
                g.mark_output(ids[nme.strip()])
            continue
        m = _OP.match(line)
        if not m:
            continue
        outs = [o.strip() for o in m.group(1).split(",")]
        ins = [i.strip() for i in m.group(3).split(",") if i.strip()]
        attrs = {}
        if m.group(4):
            for item in _split_top(m.group(4)):
                k, _, v = item.partition(" = ")
                attrs[k.strip()] = _parse_attr(v)
        out_types = m.group(6).strip()
        out_types = _split_top(out_types[1:-1]) if out_types.startswith("(") else [out_types]
        out_ids = []
        for o, t in zip(outs, out_types):
            shape, dt = _parse_type(t)
            ids[o] = g.new_value(shape, dt, device)
            out_ids.append(ids[o])
        g.add_op(m.group(2), [ids[i] for i in ins], out_ids, attrs)
    return g
