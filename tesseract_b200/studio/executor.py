"""Runs a block graph: the sink block decides the mode -- ``TrainLoop`` trains the wired model on the wired
dataset, ``Generate`` decodes from a Llama / Mamba block, ``TensorInspect`` evaluates a tensor expression and
backpropagates to its leaves. Progress goes to an event sink as ``RunEvent(type, data)`` with types ``log``,
``loss``, ``metric``, ``token``, ``text``, ``tensor``, ``done``, ``error``; the summary of the ``done`` event is also
the return value (studio/core/include/tesseract/studio/Executor.hpp:12-43, studio/core/src/Executor.cpp).
Cancellation is cooperative: ``RunOptions.cancel`` is a ``threading.Event`` polled between steps.
"""
from __future__ import annotations

import csv
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch

from .analysis import analyze
from .graph import BlockGraph, Node


@dataclass
class RunEvent:
    type: str
    data: Dict[str, Any]


EventSink = Callable[[RunEvent], None]


@dataclass
class RunOptions:
    device: str = "cpu"                          # "cpu" | "cuda" | "cuda:N"
    cancel: Optional[threading.Event] = None


class _Cancelled(Exception):
    pass


def _device(opt: RunOptions) -> torch.device:
    if opt.device.startswith("cuda"):
        if not torch.cuda.is_available():
            raise RuntimeError("device 'cuda' requested but no CUDA device is visible")
        return torch.device(opt.device)
    if opt.device != "cpu":
        raise ValueError(f"unknown device '{opt.device}'")
    return torch.device("cpu")


# ---- building blocks -----------------------------------------------------------------------------------------------
def build_layer(n: Node, device, dtype=torch.float32) -> torch.nn.Module:
    from .. import nn as tnn
    k = n.kind
    if k == "Linear":
        return tnn.Linear(n.param_int("in_features", 8), n.param_int("out_features", 32), n.param_bool("bias", True), dtype, device)
    if k == "ReLU":
        return tnn.ReLU()
    if k == "Sigmoid":
        return tnn.Sigmoid()
    if k == "Tanh":
        return tnn.Tanh()
    if k == "RMSNorm":
        return tnn.RMSNorm(n.param_int("dim", 32), n.param_num("eps", 1e-5), dtype, device)
    if k == "LayerNorm":
        return tnn.LayerNorm(n.param_int("dim", 32), n.param_num("eps", 1e-5), dtype, device)
    if k == "Embedding":
        return tnn.Embedding(n.param_int("num_embeddings", 1000), n.param_int("embedding_dim", 32), dtype, device)
    if k == "FeedForward":
        return tnn.FeedForward(n.param_int("d_model", 32), n.param_int("d_ff", 64), dtype, device)
    if k == "MultiHeadAttention":
        return tnn.MultiHeadAttention(n.param_int("d_model", 32), n.param_int("num_heads", 4), n.param_int("num_kv_heads", 0),
                                      dtype=dtype, device=device)
    if k == "TransformerBlock":
        return tnn.TransformerBlock(n.param_int("d_model", 32), n.param_int("num_heads", 4), n.param_int("d_ff", 64),
                                    n.param_int("num_kv_heads", 0), dtype=dtype, device=device)
    raise ValueError(f"block '{k}' is not a layer")


def layer_chain(g: BlockGraph, seq_node: Node) -> List[Node]:
    """The layers feeding a SequentialModel, first layer first (walks the `in` wires back to an Input block)."""
    chain: List[Node] = []
    cur = g.incoming(seq_node.id, "in")
    seen = set()
    while cur is not None:
        n = g.find_node(cur.src.node)
        if n is None or n.id in seen:
            break
        seen.add(n.id)
        if n.kind == "Input":
            break
        chain.append(n)
        cur = g.incoming(n.id, "in")
    chain.reverse()
    return chain


def build_model(g: BlockGraph, n: Node, device) -> torch.nn.Module:
    if n.kind == "SequentialModel":
        from .. import nn as tnn
        return tnn.Sequential(*[build_layer(l, device) for l in layer_chain(g, n)])
    if n.kind == "LoadLlama":
        from ..models import LlamaConfig, LlamaModel
        import os
        dtype = torch.float16 if n.param_bool("fp16", False) else torch.float32
        model_dir = n.param_str("model_dir", "")
        if model_dir:
            cfg = LlamaConfig.from_json(open(os.path.join(model_dir, "config.json")).read())
            cfg.dtype = dtype
            return LlamaModel.from_pretrained(os.path.join(model_dir, "model.safetensors"), cfg, device=device)
        cfg = LlamaConfig(vocab_size=n.param_int("vocab_size", 256), hidden_size=n.param_int("hidden_size", 64),
                          num_hidden_layers=n.param_int("num_hidden_layers", 2),
                          num_attention_heads=n.param_int("num_attention_heads", 4),
                          num_key_value_heads=n.param_int("num_key_value_heads", 4),
                          intermediate_size=n.param_int("intermediate_size", 128),
                          max_position_embeddings=n.param_int("max_position_embeddings", 512),
                          num_experts=n.param_int("num_experts", 0),
                          num_experts_per_tok=n.param_int("num_experts_per_tok", 0), dtype=dtype)
        return LlamaModel(cfg, device=device, init_std=0.02, seed=0)
    if n.kind == "LoadMamba":
        from ..models.mamba import MambaConfig, MambaModel
        torch.manual_seed(0)
        return MambaModel(MambaConfig(vocab_size=n.param_int("vocab_size", 256), hidden_size=n.param_int("hidden_size", 64),
                                      num_hidden_layers=n.param_int("num_hidden_layers", 2), d_state=n.param_int("d_state", 16),
                                      d_conv=n.param_int("d_conv", 4), expand=n.param_int("expand", 2)), device=device)
    raise ValueError(f"block '{n.kind}' does not produce a model")


def build_dataset(n: Node):
    """-> (features [N, F] fp32, labels [N] int64, classes)."""
    if n.kind == "SyntheticClassification":
        N, F, C = n.param_int("samples", 256), n.param_int("features", 8), n.param_int("classes", 3)
        gen = torch.Generator().manual_seed(n.param_int("seed", 0))
        centres = torch.randn(C, F, generator=gen) * 3.0
        y = torch.arange(N) % C
        x = centres[y] + 0.5 * torch.randn(N, F, generator=gen)
        perm = torch.randperm(N, generator=gen)
        return x[perm], y[perm], C
    if n.kind == "CsvDataset":
        rows = []
        with open(n.param_str("path", "data.csv"), newline="") as f:
            for rec in csv.reader(f):
                try:
                    rows.append([float(v) for v in rec])
                except ValueError:
                    continue                      # a header line
        if not rows:
            raise ValueError("CsvDataset: no numeric rows")
        t = torch.tensor(rows, dtype=torch.float32)
        col = n.param_int("label_col", -1)
        col = col if col >= 0 else t.shape[1] - 1
        y = t[:, col].long()
        x = torch.cat([t[:, :col], t[:, col + 1:]], dim=1)
        return x, y, int(y.max()) + 1
    raise ValueError(f"block '{n.kind}' does not produce a dataset")


def build_optimizer(n: Node, params):
    from .. import optim
    if n.kind == "SGD":
        return optim.SGD(params, lr=n.param_num("lr", 0.1), momentum=n.param_num("momentum", 0.0))
    if n.kind == "Adam":
        return optim.Adam(params, lr=n.param_num("lr", 1e-3), beta1=n.param_num("beta1", 0.9), beta2=n.param_num("beta2", 0.999),
                          eps=n.param_num("eps", 1e-8))
    raise ValueError(f"block '{n.kind}' is not an optimizer")


# ---- modes ---------------------------------------------------------------------------------------------------------
class Executor:
    @staticmethod
    def run(g: BlockGraph, sink: Optional[EventSink] = None, opt: Optional[RunOptions] = None) -> Dict[str, Any]:
        opt = opt or RunOptions(device=g.device)
        sink = sink or (lambda e: None)

        def emit(kind: str, **data):
            sink(RunEvent(kind, data))

        def finish(summary: Dict[str, Any]) -> Dict[str, Any]:
            emit("done", **summary)
            return summary

        a = analyze(g)
        for d in a.diagnostics:
            emit("log", level=d.severity, node=d.node, message=d.message)
        if not a.ok:
            emit("error", message="validation failed")
            return finish({"ok": False, "reason": "validation failed"})
        try:
            dev = _device(opt)
            for kind, mode in (("TrainLoop", _run_train), ("Generate", _run_generate), ("TensorInspect", _run_tensor)):
                sinks = [n for n in g.nodes if n.kind == kind]
                if sinks:
                    return finish(mode(g, sinks[0], emit, dev, opt))
            emit("error", message="the graph has no TrainLoop, Generate or TensorInspect block to run")
            return finish({"ok": False, "reason": "no sink"})
        except _Cancelled:
            return finish({"ok": False, "reason": "cancelled"})
        except Exception as ex:  # a failing run reports, it does not take the host application down
            emit("error", message=f"{type(ex).__name__}: {ex}")
            return finish({"ok": False, "reason": str(ex)})


def _check_cancel(opt: RunOptions) -> None:
    if opt.cancel is not None and opt.cancel.is_set():
        raise _Cancelled()


def _src(g: BlockGraph, node: Node, port: str) -> Node:
    e = g.incoming(node.id, port)
    return g.find_node(e.src.node)


def _run_train(g, loop: Node, emit, dev, opt) -> Dict[str, Any]:
    model = build_model(g, _src(g, loop, "model"), dev)
    x, y, classes = build_dataset(_src(g, loop, "data"))
    x, y = x.to(dev), y.to(dev)
    optimizer = build_optimizer(_src(g, loop, "optimizer"), list(model.parameters()))
    epochs, bs = max(1, loop.param_int("epochs", 30)), max(1, loop.param_int("batch_size", 32))
    emit("log", level="info", node=loop.id,
         message=f"training {sum(p.numel() for p in model.parameters())} parameters on {x.shape[0]} samples, "
                 f"{classes} classes, {epochs} epochs, batch {bs}, device {dev}")
    step, last_loss, last_acc = 0, 0.0, 0.0
    model.train()
    for ep in range(epochs):
        ep_loss = ep_acc = 0.0
        batches = 0
        for i in range(0, x.shape[0], bs):
            _check_cancel(opt)
            xb, yb = x[i:i + bs], y[i:i + bs]
            optimizer.zero_grad()
            logits = model(xb)
            loss = torch.nn.functional.cross_entropy(logits.float(), yb)
            loss.backward()
            optimizer.step()
            last_loss = float(loss.detach())
            last_acc = float((logits.argmax(-1) == yb).float().mean())
            ep_loss += last_loss
            ep_acc += last_acc
            batches += 1
            step += 1
            emit("loss", step=step, epoch=ep, loss=last_loss, acc=last_acc)
        emit("metric", epoch=ep, loss=ep_loss / max(1, batches), acc=ep_acc / max(1, batches))
    model.eval()
    with torch.no_grad():
        final_acc = float((model(x).argmax(-1) == y).float().mean())
    return {"ok": True, "mode": "train", "final_loss": last_loss, "final_acc": final_acc, "steps": step}


def _run_generate(g, gen: Node, emit, dev, opt) -> Dict[str, Any]:
    model = build_model(g, _src(g, gen, "model"), dev).eval()
    tok = None
    if g.incoming(gen.id, "tokenizer") is not None:
        from ..io.tokenizer import BpeTokenizer
        tok = BpeTokenizer.from_file(_src(g, gen, "tokenizer").param_str("path", "tokenizer.json"))
    vocab = model.config.vocab_size
    text = gen.param_str("prompt", "")
    if tok is not None and text:
        prompt = [int(i) for i in tok.encode(text)]
    else:
        prompt = [int(p) for p in gen.param_str("prompt_ids", "1, 2, 3").replace(";", ",").split(",") if p.strip()]
    if not prompt:
        raise ValueError("Generate: empty prompt")
    if any(i < 0 or i >= vocab for i in prompt):
        raise ValueError(f"Generate: a prompt id is outside [0, {vocab})")
    from ..models.sampler import SamplingParams
    sampling = SamplingParams(temperature=gen.param_num("temperature", 1.0), top_k=gen.param_int("top_k", 0),
                              top_p=gen.param_num("top_p", 1.0))
    common = dict(max_new_tokens=gen.param_int("max_new_tokens", 16), do_sample=gen.param_bool("do_sample", False),
                  seed=gen.param_int("seed", 0), sampling=sampling)
    if type(model).__name__ == "MambaModel":
        from ..models.mamba import MambaGenerateConfig
        cfg = MambaGenerateConfig(**common)
    else:
        from ..models import GenerateConfig
        cfg = GenerateConfig(eos_token_id=-1, **common)
    _check_cancel(opt)
    with torch.no_grad():
        out = [int(t) for t in model.generate(prompt, cfg)]
    for i in range(len(prompt), len(out)):
        data = {"index": i - len(prompt), "id": out[i]}
        if tok is not None:
            data["text"] = tok.decode([out[i]])
        emit("token", **data)
    if tok is not None:
        emit("text", text=tok.decode(out))
    return {"ok": True, "mode": "generate", "prompt_len": len(prompt), "generated": len(out) - len(prompt), "ids": out}


def _tensor_event(emit, role: str, node: int, label: str, t: Optional[torch.Tensor], limit: int = 64) -> None:
    if t is None:
        emit("tensor", role=role, node=node, label=label, shape=[], values=[], numel=0)
        return
    flat = t.detach().float().reshape(-1).cpu()
    emit("tensor", role=role, node=node, label=label, shape=list(t.shape), values=[float(v) for v in flat[:limit]],
         numel=int(flat.numel()))


def _make_leaf(n: Node, dev) -> torch.Tensor:
    rows, cols = max(1, n.param_int("rows", 2)), max(1, n.param_int("cols", 3))
    init, scale = n.param_str("init", "randn"), n.param_num("scale", 1.0)
    if init == "zeros":
        t = torch.zeros(rows, cols)
    elif init == "ones":
        t = torch.ones(rows, cols)
    elif init == "arange":
        t = torch.arange(rows * cols, dtype=torch.float32).view(rows, cols)
    elif init == "eye":
        t = torch.eye(rows, cols)
    else:
        t = torch.randn(rows, cols, generator=torch.Generator().manual_seed(n.param_int("seed", 0)))
    return (t * scale).to(dev).requires_grad_(True)


_TENSOR_OPS = {"TAdd": torch.add, "TSub": torch.sub, "TMul": torch.mul, "TMatMul": torch.matmul, "TReLU": torch.relu,
               "TSigmoid": torch.sigmoid, "TTanh": torch.tanh, "TExp": torch.exp}


def _run_tensor(g, inspect: Node, emit, dev, opt) -> Dict[str, Any]:
    values: Dict[int, torch.Tensor] = {}
    leaves: List[Node] = []
    for nid in g.topo_order():
        _check_cancel(opt)
        n = g.find_node(nid)
        if n.kind == "TensorConst":
            values[nid] = _make_leaf(n, dev)
            leaves.append(n)
        elif n.kind in _TENSOR_OPS:
            ports = ("a", "b") if g.incoming(nid, "a") is not None else ("in",)
            args = [values[g.incoming(nid, p).src.node] for p in ports]
            values[nid] = _TENSOR_OPS[n.kind](*args)
    result = values[g.incoming(inspect.id, "in").src.node]
    # only the leaves that the inspected value depends on are reported
    for leaf in leaves:
        _tensor_event(emit, "value", leaf.id, f"TensorConst #{leaf.id}", values[leaf.id])
    _tensor_event(emit, "result", inspect.id, "result", result)
    did_backward = False
    if inspect.param_bool("backward", True) and result.requires_grad:
        result.sum().backward()
        did_backward = True
        for leaf in leaves:
            _tensor_event(emit, "grad", leaf.id, f"d sum(out) / d #{leaf.id}", values[leaf.id].grad)
    return {"ok": True, "mode": "tensor", "backward": did_backward, "leaves": len(leaves)}
