"""``tesseract._core``: the reference's pybind surface (python/_core.cpp:102-360) re-created over torch, plus the
C++-only classes of the reference (RMSNorm, MultiHeadAttention, FeedForward, TransformerBlock, MoEFeedForward,
Mamba, KV caches, scheduler, speculative / structured / disaggregated decoding, quantisation, distributed) under
their C++ names.

``Tensor`` is a thin value handle over ``torch.Tensor`` with the reference's method set: ``shape`` is a list,
``dtype`` a ``DType``, ``grad()`` a method returning None when unset, ``numpy()`` / ``item()`` / ``backward()``;
modules accept and return ``Tensor``.
"""
from __future__ import annotations

import enum
from types import SimpleNamespace
from typing import Optional

import numpy as np
import torch

import tesseract_b200 as _tb
from tesseract_b200 import io as _io
from tesseract_b200 import models as _models
from tesseract_b200 import nn as _nn
from tesseract_b200 import ops as _ops
from tesseract_b200 import optim as _optim


class DType(enum.Enum):
    float32 = "float32"
    float64 = "float64"
    int64 = "int64"
    int32 = "int32"
    float16 = "float16"
    bfloat16 = "bfloat16"
    bool = "bool"
    int8 = "int8"
    uint8 = "uint8"

    @property
    def torch(self) -> torch.dtype:
        return getattr(torch, self.value)

    @staticmethod
    def of(dt: torch.dtype) -> "DType":
        return DType(str(dt).replace("torch.", ""))


class Device:
    def __init__(self, dev: torch.device):
        self._dev = torch.device(dev)

    @staticmethod
    def cpu() -> "Device":
        return Device(torch.device("cpu"))

    @staticmethod
    def cuda(index: int = 0) -> "Device":
        return Device(torch.device("cuda", index))

    def is_cpu(self) -> bool:
        return self._dev.type == "cpu"

    def is_cuda(self) -> bool:
        return self._dev.type == "cuda"

    def __repr__(self) -> str:
        return f"Device({self._dev})"

    def __eq__(self, other) -> bool:
        return isinstance(other, Device) and self._dev == other._dev


def _unwrap(x):
    return x.t if isinstance(x, Tensor) else x


def _wrap(x):
    return Tensor._from_torch(x) if isinstance(x, torch.Tensor) else x


class Tensor:
    __slots__ = ("t",)

    def __init__(self, array=None):
        if array is None:
            self.t = torch.empty(0)
        elif isinstance(array, torch.Tensor):
            self.t = array
        else:
            a = np.asarray(array)
            if a.dtype not in (np.float32, np.float64, np.int64, np.int32):
                raise TypeError(f"Tensor: unsupported numpy dtype {a.dtype}")
            self.t = torch.from_numpy(np.ascontiguousarray(a)).clone()

    @classmethod
    def _from_torch(cls, t: torch.Tensor) -> "Tensor":
        o = cls.__new__(cls)
        o.t = t
        return o

    # factories
    @staticmethod
    def from_numpy(a) -> "Tensor":
        return Tensor(a)

    @staticmethod
    def zeros(shape, dtype: DType = DType.float32) -> "Tensor":
        return Tensor._from_torch(torch.zeros(list(shape), dtype=dtype.torch))

    @staticmethod
    def ones(shape, dtype: DType = DType.float32) -> "Tensor":
        return Tensor._from_torch(torch.ones(list(shape), dtype=dtype.torch))

    @staticmethod
    def full(shape, value, dtype: DType = DType.float32) -> "Tensor":
        return Tensor._from_torch(torch.full(list(shape), value, dtype=dtype.torch))

    # properties
    @property
    def shape(self):
        return list(self.t.shape)

    @property
    def dtype(self) -> DType:
        return DType.of(self.t.dtype)

    @property
    def ndim(self) -> int:
        return self.t.dim()

    @property
    def numel(self) -> int:
        return self.t.numel()

    @property
    def device(self) -> Device:
        return Device(self.t.device)

    @property
    def requires_grad(self) -> bool:
        return self.t.requires_grad

    @requires_grad.setter
    def requires_grad(self, flag: bool) -> None:
        self.t.requires_grad_(bool(flag))

    def grad(self) -> Optional["Tensor"]:
        return None if self.t.grad is None else Tensor._from_torch(self.t.grad)

    def backward(self, grad: Optional["Tensor"] = None) -> None:
        if grad is None and self.t.numel() != 1:
            raise RuntimeError("backward: a gradient is required for a non-scalar root")
        self.t.backward(_unwrap(grad))

    def numpy(self) -> np.ndarray:
        return self.t.detach().cpu().numpy()

    def item(self):
        if self.t.numel() != 1:
            raise RuntimeError("item(): tensor has more than one element")
        return self.t.item()

    def reshape(self, shape) -> "Tensor":
        return Tensor._from_torch(self.t.reshape(list(shape)))

    def to(self, device) -> "Tensor":
        dev = device._dev if isinstance(device, Device) else device
        return Tensor._from_torch(self.t.to(dev))

    def matmul(self, other) -> "Tensor":
        return ops.matmul(self, other)

    def __add__(self, o):
        return ops.add(self, o)

    def __sub__(self, o):
        return ops.sub(self, o)

    def __mul__(self, o):
        return ops.mul(self, o)

    def __matmul__(self, o):
        return ops.matmul(self, o)

    def __repr__(self) -> str:
        return f"Tensor(shape={self.shape}, dtype={self.dtype.value}, device={self.t.device})"


def backward(root: Tensor, grad: Optional[Tensor] = None) -> None:
    root.backward(grad)


def _check_same(a, b, what):
    if a.t.device != b.t.device:
        raise RuntimeError(f"{what}: tensors are on different devices")
    if a.t.dtype != b.t.dtype:
        raise TypeError(f"{what}: dtype mismatch ({a.t.dtype} vs {b.t.dtype})")


def _binary(name, fn):
    def op(a: Tensor, b: Tensor) -> Tensor:
        _check_same(a, b, name)
        return _wrap(fn(a.t, b.t))
    op.__name__ = name
    return op


def _matmul(a: Tensor, b: Tensor) -> Tensor:
    _check_same(a, b, "matmul")
    if a.t.dim() < 2 or b.t.dim() < 2:
        raise ValueError("matmul: both operands must have rank >= 2")
    if a.t.shape[-1] != b.t.shape[-2]:
        raise ValueError(f"matmul: inner dimensions differ ({a.t.shape[-1]} vs {b.t.shape[-2]})")
    if a.t.is_cuda and a.t.dtype == torch.bfloat16 and a.t.dim() == 2 and b.t.dim() == 2:
        return _wrap(_LinearNN.apply(a.t, b.t))
    if (not a.t.is_cuda and a.t.dtype == torch.float32 and b.t.dtype == torch.float32 and a.t.dim() == 2
            and b.t.dim() == 2):
        from tesseract_b200.ops import cpu_gemm
        if cpu_gemm.native_selected():          # TESSERACT_CPU_GEMM=native: the host runtime's GEMM, with autograd
            return _wrap(cpu_gemm.matmul(a.t, b.t))
    return _wrap(a.t @ b.t)


class _LinearNN(torch.autograd.Function):
    """a [M, K] @ b [K, N] on the tcgen05 kernel (b is the N-major operand)."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return _ops.gemm_bf16(a.contiguous(), b.contiguous(), b_mn=True)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        g = g.contiguous()
        da = _ops.gemm_bf16(g, b.contiguous())                              # g [M,N] @ b[K,N]^T
        db = _ops.gemm_bf16(a.contiguous(), g, a_mn=True, b_mn=True)        # a^T @ g
        return da, db


def _cross_entropy(logits: Tensor, targets: Tensor) -> Tensor:
    lt = logits.t
    if lt.dim() > 2:
        lt = lt.reshape(-1, lt.shape[-1])
    return _wrap(_ops.cross_entropy(lt, targets.t.reshape(-1)))


ops = SimpleNamespace(
    add=_binary("add", torch.add), sub=_binary("sub", torch.sub), mul=_binary("mul", torch.mul),
    div=_binary("div", torch.div), matmul=_matmul,
    relu=lambda x: _wrap(torch.relu(x.t)), sigmoid=lambda x: _wrap(torch.sigmoid(x.t)),
    tanh=lambda x: _wrap(torch.tanh(x.t)), exp=lambda x: _wrap(torch.exp(x.t)), log=lambda x: _wrap(torch.log(x.t)),
    sqrt=lambda x: _wrap(torch.sqrt(x.t)), neg=lambda x: _wrap(torch.neg(x.t)),
    softmax=lambda x, dim=-1: _wrap(torch.softmax(x.t, dim)), log_softmax=lambda x, dim=-1: _wrap(torch.log_softmax(x.t, dim)),
    sum=lambda x, dim=None, keepdim=False: _wrap(x.t.sum() if dim is None else x.t.sum(dim, keepdim)),
    mean=lambda x, dim=None, keepdim=False: _wrap(x.t.mean() if dim is None else x.t.mean(dim, keepdim)),
    cross_entropy=_cross_entropy,
    rms_norm=lambda x, w, eps=1e-5: _wrap(_ops.rms_norm(x.t, w.t, eps)),
    swiglu_silu_gate=lambda g, u: _wrap(_ops.swiglu_silu_gate(g.t, u.t)),
    attention=lambda q, k, v, causal=False: _wrap(_ops.attention_ref(q.t, k.t, v.t, causal=causal)),
)


class _ModuleHandle:
    """Wraps a torch module so that it consumes / produces ``Tensor`` handles."""

    def __init__(self, mod: torch.nn.Module):
        self._m = mod

    def forward(self, *args):
        return _wrap(self._m(*[_unwrap(a) for a in args]))

    __call__ = forward

    def parameters(self):
        return [Tensor._from_torch(p) for p in self._m.parameters()]

    def named_parameters(self):
        return [(n, Tensor._from_torch(p)) for n, p in self._m.named_parameters()]

    def zero_grad(self):
        self._m.zero_grad(set_to_none=True)

    def train(self, on: bool = True):
        self._m.train(on)
        return self

    def eval(self):
        self._m.eval()
        return self

    def to(self, device):
        self._m.to(device._dev if isinstance(device, Device) else device)
        return self

    @property
    def module(self) -> torch.nn.Module:
        return self._m


def _handle_class(name, factory, extra=None):
    def __init__(self, *a, **k):
        k = {kk: (vv.torch if isinstance(vv, DType) else vv) for kk, vv in k.items()}
        a = [(x.torch if isinstance(x, DType) else x) for x in a]
        _ModuleHandle.__init__(self, factory(*a, **k))
    ns = {"__init__": __init__}
    if extra:
        ns.update(extra)
    return type(name, (_ModuleHandle,), ns)


def _seq_factory(mods=()):
    return _nn.Sequential([m._m if isinstance(m, _ModuleHandle) else m for m in mods])


def _seq_add(self, m):
    self._m.append(m._m if isinstance(m, _ModuleHandle) else m)
    return self


nn = SimpleNamespace(
    Module=_ModuleHandle,
    Linear=_handle_class("Linear", _nn.Linear, {"weight": lambda self: Tensor._from_torch(self._m.weight),
                                                "bias": lambda self: _wrap(self._m.bias)}),
    Embedding=_handle_class("Embedding", _nn.Embedding, {"weight": lambda self: Tensor._from_torch(self._m.weight)}),
    ReLU=_handle_class("ReLU", _nn.ReLU), Sigmoid=_handle_class("Sigmoid", _nn.Sigmoid),
    Tanh=_handle_class("Tanh", _nn.Tanh),
    Sequential=_handle_class("Sequential", _seq_factory, {"add": _seq_add}),
    RMSNorm=_handle_class("RMSNorm", _nn.RMSNorm), LayerNorm=_handle_class("LayerNorm", _nn.LayerNorm),
    MultiHeadAttention=_handle_class("MultiHeadAttention", _nn.MultiHeadAttention),
    FeedForward=_handle_class("FeedForward", _nn.FeedForward),
    TransformerBlock=_handle_class("TransformerBlock", _nn.TransformerBlock),
    CrossEntropyLoss=_handle_class("CrossEntropyLoss", _nn.CrossEntropyLoss),
)


def _params_of(params):
    return [p.t if isinstance(p, Tensor) else p for p in params]


class _SGD(_optim.SGD):
    def __init__(self, params, lr, momentum=0.0):
        super().__init__(_params_of(params), lr, momentum)


class _Adam(_optim.Adam):
    def __init__(self, params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8):
        super().__init__(_params_of(params), lr, beta1, beta2, eps)


optim = SimpleNamespace(SGD=_SGD, Adam=_Adam)


class _LlamaModel(_ModuleHandle):
    def __init__(self, config):
        super().__init__(_models.LlamaModel(config))

    @staticmethod
    def from_pretrained(path, config):
        h = _LlamaModel.__new__(_LlamaModel)
        _ModuleHandle.__init__(h, _models.LlamaModel.from_pretrained(path, config))
        return h

    def generate(self, prompt_ids, cfg=None):
        return self._m.generate(prompt_ids, cfg)

    def config(self):
        return self._m.config


def _late_models():
    from tesseract_b200.models.mamba import MambaConfig, MambaGenerateConfig, MambaModel

    class _MambaModel(_ModuleHandle):
        def __init__(self, config):
            super().__init__(MambaModel(config))

        def generate(self, prompt_ids, cfg=None):
            return self._m.generate(prompt_ids, cfg)

        def config(self):
            return self._m.config

    return MambaConfig, MambaGenerateConfig, _MambaModel


_MambaConfig, _MambaGenerateConfig, _MambaModelH = _late_models()

models = SimpleNamespace(
    SamplingParams=_models.SamplingParams, LlamaConfig=_models.LlamaConfig,
    LlamaGenerateConfig=_models.GenerateConfig, LlamaModel=_LlamaModel,
    MambaConfig=_MambaConfig, MambaGenerateConfig=_MambaGenerateConfig, MambaModel=_MambaModelH,
    Sampler=_models.Sampler,
)

io = SimpleNamespace(
    Tokenizer=_io.Tokenizer, WhitespaceTokenizerConfig=_io.WhitespaceTokenizerConfig,
    WhitespaceTokenizer=_io.WhitespaceTokenizer, BpeTokenizer=_io.BpeTokenizer, SafeTensors=_io.SafeTensors,
)

__all__ = ["DType", "Device", "Tensor", "backward", "ops", "nn", "optim", "models", "io"]
