"""Graph-mode training step: the forward pass and the loss of a module are recorded once, the backward pass is
appended by ``build_backward``, and every later step replays that one graph (the ``graph`` engine of the
reference's examples/mnist.cpp; parity with the eager tape is what tests/graph/test_graph_train_parity.cpp:270
checks). On a GPU the replay is a single CUDA-graph launch.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .autograd import build_backward
from .interpreter import GraphExecutor
from .scope import GraphScope


class GraphTrainStep:
    """``step = GraphTrainStep(model, loss_fn, x0, y0)``; ``loss = step(x, y)`` writes ``p.grad`` of every parameter
    (overwriting it) and returns the loss. Shapes are fixed by the example batch. Parameters are shared with the
    module, so any optimizer that updates them in place works between steps."""

    def __init__(self, model: torch.nn.Module, loss_fn: Callable, example_x: torch.Tensor, example_y: torch.Tensor,
                 cuda_graph: Optional[bool] = None):
        self.model = model
        self.params = [p for _, p in model.named_parameters()]
        with GraphScope() as scope:
            self.x_id = scope.bind_input(example_x, "x")
            self.y_id = scope.bind_input(example_y, "y")
            ids = scope.bind_module(model)
            loss = loss_fn(model(example_x), example_y)
            scope.mark_output(loss)
        self.graph = scope.graph
        self.forward_ops = self.graph.num_ops()
        res = build_backward(self.graph)
        self.param_ids = [ids[n] for n, _ in model.named_parameters()]
        assert self.param_ids == list(self.graph.params)
        bindings = {self.x_id: example_x, self.y_id: example_y, res.cotangents[0]: torch.ones_like(loss)}
        bindings.update({vid: p.data for vid, p in zip(self.param_ids, self.params)})
        self.executor = GraphExecutor(self.graph, bindings, cuda_graph=cuda_graph, share=self.param_ids)

    def __call__(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        outs = self.executor({self.x_id: x, self.y_id: y})
        loss, grads = outs[0], outs[1:]
        for p, g in zip(self.params, grads):
            # CUDA-graph outputs are static buffers, interpreted outputs are fresh tensors: either way they are handed
            # out as they are (a transposed view is made contiguous first: optimizers update it in place)
            p.grad = g if g.is_contiguous() else g.contiguous()
        return loss
