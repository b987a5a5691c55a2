"""Block palette: every block kind with its typed ports and its parameter schema
(studio/core/include/tesseract/studio/BlockCatalog.hpp:12-66; the kinds, ports, parameter names and defaults of
studio/core/src/BlockCatalog.cpp:40-210, so a ``.tsb`` file written by either side opens in the other).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .graph import PortType

PT = PortType


@dataclass
class ParamSpec:
    name: str
    type: str                      # "int" | "float" | "bool" | "string" | "enum"
    default: Any
    label: str
    options: List[str] = field(default_factory=list)


@dataclass
class PortSpec:
    name: str
    type: PortType


@dataclass
class BlockSpec:
    kind: str
    category: str
    label: str
    summary: str
    inputs: List[PortSpec]
    outputs: List[PortSpec]
    params: List[ParamSpec]

    def input(self, name: str) -> Optional[PortSpec]:
        return next((p for p in self.inputs if p.name == name), None)

    def output(self, name: str) -> Optional[PortSpec]:
        return next((p for p in self.outputs if p.name == name), None)


def _pi(name, default, label):
    return ParamSpec(name, "int", int(default), label)


def _pf(name, default, label):
    return ParamSpec(name, "float", float(default), label)


def _pb(name, default, label):
    return ParamSpec(name, "bool", bool(default), label)


def _ps(name, default, label):
    return ParamSpec(name, "string", str(default), label)


def _pe(name, default, label, options):
    return ParamSpec(name, "enum", str(default), label, list(options))


def _port(name, t):
    return PortSpec(name, t)


def _unary(kind, category, label, summary, params=()):
    return BlockSpec(kind, category, label, summary, [_port("in", PT.Tensor)], [_port("out", PT.Tensor)], list(params))


def _binary(kind, label, summary):
    return BlockSpec(kind, "Tensor", label, summary, [_port("a", PT.Tensor), _port("b", PT.Tensor)],
                     [_port("out", PT.Tensor)], [])


def _build() -> List[BlockSpec]:
    s: List[BlockSpec] = []
    # ---- Data
    s.append(BlockSpec("Input", "Data", "Input", "Input tensor [batch, features].", [], [_port("out", PT.Tensor)],
                       [_pi("batch", 32, "Batch size"), _pi("features", 8, "Features")]))
    s.append(BlockSpec("SyntheticClassification", "Data", "Synthetic classification",
                       "Gaussian-mixture classification set (in-memory).", [], [_port("data", PT.Dataset)],
                       [_pi("samples", 256, "Samples"), _pi("features", 8, "Features"), _pi("classes", 3, "Classes"),
                        _pi("seed", 0, "Seed")]))
    s.append(BlockSpec("CsvDataset", "Data", "CSV dataset", "Numeric CSV; one column is the integer class label.", [],
                       [_port("data", PT.Dataset)],
                       [_ps("path", "data.csv", "CSV path"), _pi("label_col", -1, "Label column (-1 = last)")]))
    # ---- Layers
    s.append(_unary("Linear", "Layers", "Linear", "Affine: y = x W^T + b.",
                    [_pi("in_features", 8, "In features"), _pi("out_features", 32, "Out features"), _pb("bias", True, "Bias")]))
    s.append(_unary("ReLU", "Layers", "ReLU", "max(0, x)."))
    s.append(_unary("Sigmoid", "Layers", "Sigmoid", "1 / (1 + e^-x)."))
    s.append(_unary("Tanh", "Layers", "Tanh", "Hyperbolic tangent."))
    s.append(_unary("RMSNorm", "Layers", "RMSNorm", "Llama RMS normalization.",
                    [_pi("dim", 32, "Normalized dim"), _pf("eps", 1e-5, "Eps")]))
    s.append(_unary("LayerNorm", "Layers", "LayerNorm", "Standard LayerNorm.",
                    [_pi("dim", 32, "Normalized dim"), _pf("eps", 1e-5, "Eps"), _pb("bias", True, "Bias")]))
    s.append(_unary("Embedding", "Layers", "Embedding", "Lookup table [num_embeddings, dim].",
                    [_pi("num_embeddings", 1000, "Vocab"), _pi("embedding_dim", 32, "Embedding dim")]))
    s.append(_unary("FeedForward", "Layers", "FeedForward (SwiGLU)", "Llama SwiGLU MLP.",
                    [_pi("d_model", 32, "d_model"), _pi("d_ff", 64, "d_ff"), _pb("bias", False, "Bias")]))
    s.append(_unary("MultiHeadAttention", "Layers", "Multi-head attention", "Causal MHA / GQA over [B, S, D].",
                    [_pi("d_model", 32, "d_model"), _pi("num_heads", 4, "Heads"), _pi("num_kv_heads", 0, "KV heads (0=MHA)"),
                     _pb("causal", True, "Causal")]))
    s.append(_unary("TransformerBlock", "Layers", "Transformer block", "Pre-norm attention + SwiGLU + residuals.",
                    [_pi("d_model", 32, "d_model"), _pi("num_heads", 4, "Heads"), _pi("d_ff", 64, "d_ff"),
                     _pi("num_kv_heads", 0, "KV heads"), _pb("causal", True, "Causal")]))
    # ---- Tensor playground
    s.append(BlockSpec("TensorConst", "Tensor", "Tensor", "A leaf tensor (requires_grad).", [], [_port("out", PT.Tensor)],
                       [_pi("rows", 2, "Rows"), _pi("cols", 3, "Cols"),
                        _pe("init", "randn", "Init", ["randn", "zeros", "ones", "arange", "eye"]),
                        _pf("scale", 1.0, "Scale"), _pi("seed", 0, "Seed")]))
    s.append(_binary("TAdd", "Add (a + b)", "Element-wise add."))
    s.append(_binary("TSub", "Sub (a - b)", "Element-wise subtract."))
    s.append(_binary("TMul", "Mul (a * b)", "Element-wise multiply."))
    s.append(_binary("TMatMul", "MatMul (a . b)", "Matrix product."))
    s.append(_unary("TReLU", "Tensor", "ReLU(x)", "max(0, x)."))
    s.append(_unary("TSigmoid", "Tensor", "Sigmoid(x)", "1/(1+e^-x)."))
    s.append(_unary("TTanh", "Tensor", "Tanh(x)", "Hyperbolic tangent."))
    s.append(_unary("TExp", "Tensor", "Exp(x)", "e^x."))
    s.append(BlockSpec("TensorInspect", "Tensor", "Inspect / backward",
                       "Evaluate `in`; show shape + values, optionally run autograd backward and show leaf gradients.",
                       [_port("in", PT.Tensor)], [], [_pb("backward", True, "Run backward (d sum(out) / d leaf)")]))
    # ---- Model
    s.append(BlockSpec("SequentialModel", "Model", "Sequential model", "Assemble the layer chain feeding `in` into a model.",
                       [_port("in", PT.Tensor)], [_port("model", PT.Model)], []))
    s.append(BlockSpec("LoadLlama", "Model", "Llama model", "Build/load a Llama (set model_dir to load HF weights).", [],
                       [_port("model", PT.Model)],
                       [_ps("model_dir", "", "HF model dir (blank = random init)"), _pi("vocab_size", 256, "Vocab"),
                        _pi("hidden_size", 64, "Hidden"), _pi("num_hidden_layers", 2, "Layers"),
                        _pi("num_attention_heads", 4, "Heads"), _pi("num_key_value_heads", 4, "KV heads"),
                        _pi("intermediate_size", 128, "Intermediate"), _pi("max_position_embeddings", 512, "Max pos"),
                        _pi("num_experts", 0, "Experts (0=dense)"), _pi("num_experts_per_tok", 0, "Experts/token"),
                        _pb("fp16", False, "FP16")]))
    s.append(BlockSpec("LoadMamba", "Model", "Mamba model", "Build a Mamba (SSM) model.", [], [_port("model", PT.Model)],
                       [_pi("vocab_size", 256, "Vocab"), _pi("hidden_size", 64, "Hidden"), _pi("num_hidden_layers", 2, "Layers"),
                        _pi("d_state", 16, "d_state"), _pi("d_conv", 4, "d_conv"), _pi("expand", 2, "Expand")]))
    # ---- Loss / optimizers / tokenizer
    s.append(BlockSpec("CrossEntropyLoss", "Loss", "Cross-entropy loss", "Softmax cross-entropy with integer targets.", [],
                       [_port("loss", PT.Loss)], []))
    s.append(BlockSpec("SGD", "Optimizer", "SGD", "Stochastic gradient descent (+ momentum).", [_port("model", PT.Model)],
                       [_port("opt", PT.Optimizer)], [_pf("lr", 0.1, "Learning rate"), _pf("momentum", 0.0, "Momentum")]))
    s.append(BlockSpec("Adam", "Optimizer", "Adam", "Adam optimizer.", [_port("model", PT.Model)], [_port("opt", PT.Optimizer)],
                       [_pf("lr", 1e-3, "Learning rate"), _pf("beta1", 0.9, "Beta1"), _pf("beta2", 0.999, "Beta2"),
                        _pf("eps", 1e-8, "Eps")]))
    s.append(BlockSpec("BpeTokenizer", "Tokenizer", "BPE tokenizer", "Load a tokenizer.json (byte-level BPE).", [],
                       [_port("tokenizer", PT.Tokenizer)], [_ps("path", "tokenizer.json", "tokenizer.json path")]))
    # ---- sinks
    s.append(BlockSpec("TrainLoop", "Train", "Train loop", "Train `model` on `data` with `optimizer` minimizing `loss`.",
                       [_port("model", PT.Model), _port("data", PT.Dataset), _port("optimizer", PT.Optimizer),
                        _port("loss", PT.Loss)], [], [_pi("epochs", 30, "Epochs"), _pi("batch_size", 32, "Batch size")]))
    s.append(BlockSpec("Generate", "Inference", "Generate", "Autoregressively generate tokens from `model`.",
                       [_port("model", PT.Model), _port("tokenizer", PT.Tokenizer)], [],
                       [_ps("prompt", "", "Prompt text (needs tokenizer)"), _ps("prompt_ids", "1, 2, 3", "or prompt ids (comma-sep)"),
                        _pi("max_new_tokens", 16, "Max new tokens"), _pb("do_sample", False, "Sample"),
                        _pf("temperature", 1.0, "Temperature"), _pi("top_k", 0, "Top-k"), _pf("top_p", 1.0, "Top-p"),
                        _pi("seed", 0, "Seed")]))
    return s


class BlockCatalog:
    _instance: Optional["BlockCatalog"] = None

    def __init__(self):
        self._specs = _build()
        self._by_kind = {b.kind: b for b in self._specs}

    @classmethod
    def instance(cls) -> "BlockCatalog":
        if cls._instance is None:
            cls._instance = BlockCatalog()
        return cls._instance

    def find(self, kind: str) -> Optional[BlockSpec]:
        return self._by_kind.get(kind)

    def specs(self) -> List[BlockSpec]:
        return self._specs

    def default_params(self, kind: str) -> Dict[str, Any]:
        spec = self.find(kind)
        return {p.name: p.default for p in spec.params} if spec else {}

    def to_json(self) -> List[Dict[str, Any]]:
        """The palette as the UI reads it."""
        out = []
        for b in self._specs:
            out.append({"kind": b.kind, "category": b.category, "label": b.label, "summary": b.summary,
                        "inputs": [{"name": p.name, "type": p.type.value} for p in b.inputs],
                        "outputs": [{"name": p.name, "type": p.type.value} for p in b.outputs],
                        "params": [{"name": p.name, "type": p.type, "default": p.default, "label": p.label,
                                    **({"options": p.options} if p.options else {})} for p in b.params]})
        return out
