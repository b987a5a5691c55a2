"""Source generation from a block graph (studio/core/include/tesseract/studio/Codegen.hpp:10-33,
studio/core/src/Codegen.cpp): ``generate_python`` writes a runnable script against the ``tesseract`` Python
frontend, ``generate_ir`` lowers the forward pass to ``tesseract``-dialect text by recording it through the graph
IR, and every generated source carries the graph itself as an embedded ``.tsb`` block, so ``extract_tsb`` turns
the script back into the graph (the builder is bidirectional). The reference also emits C++ against its own C++
API; this framework has no C++ frontend, so ``generate_cpp`` is not offered.
"""
from __future__ import annotations

import json
import re
from typing import List, Optional

import torch

from .executor import build_layer, layer_chain
from .graph import BlockGraph, Node

_BEGIN, _END = "# ---- tsb begin ----", "# ---- tsb end ----"


def _embed(g: BlockGraph) -> str:
    body = "\n".join("# " + line for line in g.to_tsb().splitlines())
    return f"{_BEGIN}\n{body}\n{_END}\n"


def extract_tsb(source: str) -> Optional[BlockGraph]:
    m = re.search(re.escape(_BEGIN) + r"\n(.*?)\n" + re.escape(_END), source, re.S)
    if not m:
        return None
    text = "\n".join(line[2:] if line.startswith("# ") else line.lstrip("#") for line in m.group(1).splitlines())
    try:
        return BlockGraph.from_tsb(text)
    except (ValueError, KeyError, json.JSONDecodeError):
        return None


def _first(g: BlockGraph, kind: str) -> Optional[Node]:
    return next((n for n in g.nodes if n.kind == kind), None)


def _src(g: BlockGraph, node: Node, port: str) -> Optional[Node]:
    e = g.incoming(node.id, port)
    return g.find_node(e.src.node) if e is not None else None


def _py_layer(n: Node) -> str:
    p = n.params
    if n.kind == "Linear":
        return f"ts.nn.Linear({n.param_int('in_features', 8)}, {n.param_int('out_features', 32)}, bias={n.param_bool('bias', True)})"
    if n.kind in ("ReLU", "Sigmoid", "Tanh"):
        return f"ts.nn.{n.kind}()"
    if n.kind == "Embedding":
        return f"ts.nn.Embedding({n.param_int('num_embeddings', 1000)}, {n.param_int('embedding_dim', 32)})"
    args = ", ".join(f"{k}={p[k]!r}" for k in sorted(p))
    return f"tsb.nn.{n.kind}({args})      # tesseract_b200.nn (not in the compact frontend)"


def generate_python(g: BlockGraph) -> str:
    out: List[str] = ['"""Generated from the block graph \'%s\'. Edit the graph, not this file: the block at the end '
                      'holds it."""' % g.name,
                      "import numpy as np", "import tesseract as ts", "import tesseract_b200 as tsb", ""]
    loop, gen, inspect = _first(g, "TrainLoop"), _first(g, "Generate"), _first(g, "TensorInspect")
    if loop is not None:
        model, data, opt = _src(g, loop, "model"), _src(g, loop, "data"), _src(g, loop, "optimizer")
        layers = layer_chain(g, model) if model is not None and model.kind == "SequentialModel" else []
        out.append("model = ts.nn.Sequential([")
        out += [f"    {_py_layer(l)}," for l in layers]
        out.append("])")
        if data is not None and data.kind == "SyntheticClassification":
            out += [f"rng = np.random.default_rng({data.param_int('seed', 0)})",
                    f"N, F, C = {data.param_int('samples', 256)}, {data.param_int('features', 8)}, {data.param_int('classes', 3)}",
                    "centres = rng.normal(size=(C, F)) * 3.0", "y = np.arange(N) % C",
                    "x = (centres[y] + 0.5 * rng.normal(size=(N, F))).astype(np.float32)"]
        elif data is not None:
            out += [f"table = np.loadtxt({data.param_str('path', 'data.csv')!r}, delimiter=',', skiprows=0)",
                    f"col = {data.param_int('label_col', -1)} % table.shape[1]",
                    "y = table[:, col].astype(np.int64)", "x = np.delete(table, col, axis=1).astype(np.float32)"]
        if opt is not None and opt.kind == "Adam":
            out.append(f"opt = ts.optim.Adam(model.parameters(), lr={opt.param_num('lr', 1e-3)}, beta1={opt.param_num('beta1', 0.9)}, "
                       f"beta2={opt.param_num('beta2', 0.999)}, eps={opt.param_num('eps', 1e-8)})")
        elif opt is not None:
            out.append(f"opt = ts.optim.SGD(model.parameters(), lr={opt.param_num('lr', 0.1)}, momentum={opt.param_num('momentum', 0.0)})")
        bs = loop.param_int("batch_size", 32)
        out += [f"for epoch in range({loop.param_int('epochs', 30)}):",
                f"    for i in range(0, len(x), {bs}):",
                f"        xb, yb = ts.Tensor(x[i:i + {bs}]), ts.Tensor(y[i:i + {bs}].astype(np.int64))",
                "        opt.zero_grad()",
                "        loss = ts.ops.cross_entropy(model(xb), yb)",
                "        loss.backward()",
                "        opt.step()",
                "    print(epoch, loss.item())"]
    elif gen is not None:
        model = _src(g, gen, "model")
        if model is not None and model.kind == "LoadMamba":
            fields = ", ".join(f"{k}={model.param_int(k)}" for k in ("vocab_size", "hidden_size", "num_hidden_layers", "d_state",
                                                                     "d_conv", "expand"))
            out += [f"model = ts.models.MambaModel(ts.models.MambaConfig({fields}))",
                    f"cfg = ts.models.MambaGenerateConfig(max_new_tokens={gen.param_int('max_new_tokens', 16)})"]
        elif model is not None:
            out.append("config = ts.models.LlamaConfig()")
            for k in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                      "intermediate_size", "max_position_embeddings", "num_experts", "num_experts_per_tok"):
                out.append(f"config.{k} = {model.param_int(k)}")
            md = model.param_str("model_dir", "")
            out.append(f"model = ts.models.LlamaModel.from_pretrained({md + '/model.safetensors'!r}, config)" if md
                       else "model = ts.models.LlamaModel(config)")
            out += [f"cfg = ts.models.LlamaGenerateConfig(max_new_tokens={gen.param_int('max_new_tokens', 16)}, "
                    f"do_sample={gen.param_bool('do_sample', False)}, seed={gen.param_int('seed', 0)})"]
        ids = [int(p) for p in gen.param_str("prompt_ids", "1, 2, 3").split(",") if p.strip()]
        out += [f"print(model.generate({ids!r}, cfg))"]
    elif inspect is not None:
        names = {}
        for nid in g.topo_order():
            n = g.find_node(nid)
            if n.kind == "TensorConst":
                names[nid] = f"t{nid}"
                out += [f"t{nid} = ts.Tensor(np.random.default_rng({n.param_int('seed', 0)}).normal(size=({n.param_int('rows', 2)}, "
                        f"{n.param_int('cols', 3)})).astype(np.float32) * {n.param_num('scale', 1.0)})",
                        f"t{nid}.requires_grad = True"]
            elif n.kind in ("TAdd", "TSub", "TMul", "TMatMul"):
                a, b = names[g.incoming(nid, "a").src.node], names[g.incoming(nid, "b").src.node]
                op = {"TAdd": "+", "TSub": "-", "TMul": "*", "TMatMul": "@"}[n.kind]
                names[nid] = f"t{nid}"
                out.append(f"t{nid} = {a} {op} {b}")
            elif n.kind in ("TReLU", "TSigmoid", "TTanh", "TExp"):
                fn = {"TReLU": "ts.ops.relu", "TSigmoid": "ts.ops.sigmoid", "TTanh": "ts.ops.tanh", "TExp": "ts.ops.exp"}[n.kind]
                names[nid] = f"t{nid}"
                out.append(f"t{nid} = {fn}({names[g.incoming(nid, 'in').src.node]})")
        res = names.get(g.incoming(inspect.id, "in").src.node, "None")
        out.append(f"print({res})")
    out += ["", _embed(g)]
    return "\n".join(out)


def _forward_module(g: BlockGraph):
    """-> (module, example input) of the layer chain, or of the tensor expression under a TensorInspect."""
    seq = _first(g, "SequentialModel")
    if seq is not None:
        layers = layer_chain(g, seq)
        mod = torch.nn.Sequential(*[build_layer(l, "cpu") for l in layers])
        first = g.incoming(layers[0].id, "in") if layers else g.incoming(seq.id, "in")
        src = g.find_node(first.src.node) if first is not None else None
        batch = src.param_int("batch", 32) if src is not None and src.kind == "Input" else 32
        feats = src.param_int("features", 8) if src is not None and src.kind == "Input" else 8
        return mod, [torch.zeros(batch, feats)], ["x"]
    return None, [], []


def generate_ir(g: BlockGraph) -> str:
    """``func.func @forward`` in the ``tesseract`` dialect for the graph's forward pass."""
    from ..graph import GraphScope, emit_mlir
    mod, inputs, names = _forward_module(g)
    with GraphScope() as scope:
        if mod is not None:
            scope.trace(mod, *inputs, names=names)
        else:
            inspect = _first(g, "TensorInspect")
            if inspect is None:
                raise ValueError("generate_ir: the graph has neither a SequentialModel nor a TensorInspect block")
            vals = {}
            ops = {"TAdd": torch.add, "TSub": torch.sub, "TMul": torch.mul, "TMatMul": torch.matmul, "TReLU": torch.relu,
                   "TSigmoid": torch.sigmoid, "TTanh": torch.tanh, "TExp": torch.exp}
            for nid in g.topo_order():
                n = g.find_node(nid)
                if n.kind == "TensorConst":
                    vals[nid] = torch.zeros(n.param_int("rows", 2), n.param_int("cols", 3))
                    scope.bind_param(vals[nid], f"t{nid}")
                elif n.kind in ops:
                    ports = ("a", "b") if g.incoming(nid, "a") is not None else ("in",)
                    vals[nid] = ops[n.kind](*[vals[g.incoming(nid, p).src.node] for p in ports])
            scope.mark_output(vals[g.incoming(inspect.id, "in").src.node])
    return emit_mlir(scope.graph).replace("func.func @main", "func.func @forward")
