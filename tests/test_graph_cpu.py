"""Graph IR on CPU: capture, interpreter, backward transform, text round trip, graph-mode training parity.
Mirrors the reference's tests/graph/{test_graph_smoke,test_graph_autograd,test_graph_mnist_mode,
test_graph_train_parity}.cpp."""
import pytest
import torch
import torch.nn.functional as F

from tesseract_b200.graph import (Graph, GraphExecutor, GraphScope, GraphTrainStep, ValueKind, build_backward,
                                  differentiable_ops, emit_mlir, is_recording, parse_mlir, run, supported_ops)


def test_scope_captures_binary_elementwise_ops():
    a, b = torch.randn(2, 3), torch.randn(2, 3)
    with GraphScope() as s:
        assert is_recording()
        s.bind_input(a, "a")
        s.bind_input(b, "b")
        c = a + b
        d = c * a
        e = d - b
        f = e / 2.0
        s.mark_output(f)
    assert not is_recording()
    g = s.graph
    assert g.op_kinds() == ["add", "mul", "sub", "div"]
    assert len(g.inputs) == 2 and len(g.constants) == 1 and len(g.outputs) == 1
    assert g.value(g.ops[0].outputs[0]).shape == (2, 3)
    a2, b2 = torch.randn(2, 3), torch.randn(2, 3)
    (out,) = run(g, {g.inputs[0]: a2, g.inputs[1]: b2})
    assert torch.equal(out, ((a2 + b2) * a2 - b2) / 2.0)


def test_scope_records_matmul_relu_chain_and_view_family():
    x, w = torch.randn(4, 6), torch.randn(6, 5)
    with GraphScope() as s:
        y = torch.relu(x @ w)
        z = y.reshape(2, 10).transpose(0, 1).contiguous().view(5, 4).permute(1, 0)
        r = z.sum(dim=1, keepdim=True).broadcast_to(4, 5).mean()
        s.mark_output(r)
    g = s.graph
    assert g.op_kinds() == ["matmul", "relu", "reshape", "transpose", "contiguous", "view", "permute", "sum",
                            "broadcast_to", "mean"]
    kinds = {o.kind: o for o in g.ops}
    assert kinds["reshape"].attrs == {"shape": [2, 10]}
    assert kinds["transpose"].attrs == {"dim_a": 0, "dim_b": 1}
    assert kinds["permute"].attrs == {"axes": [1, 0]}
    assert kinds["sum"].attrs == {"dim": 1, "keepdim": True}
    assert kinds["mean"].attrs == {}
    assert [g.value(i).kind for i in g.inputs] == [ValueKind.INPUT, ValueKind.INPUT]     # lazily bound operands
    (out,) = run(g, {g.inputs[0]: x, g.inputs[1]: w})
    assert torch.allclose(out, r)


def test_scope_captures_linear_and_rejects_nesting_and_unknown_ops():
    lin = torch.nn.Linear(8, 3)
    x = torch.randn(5, 8)
    with GraphScope() as s:
        g = s.trace(lin, x, names=["x"])
        with pytest.raises(RuntimeError, match="do not nest"):
            with GraphScope():
                pass
        with pytest.raises(NotImplementedError, match="no graph op"):
            torch.cumsum(lin(x), dim=0)
        with pytest.raises(RuntimeError, match="live GraphScope"):
            run(g, {})
    assert g.op_kinds()[:4] == ["transpose", "matmul", "broadcast_to", "add"]
    assert [g.value(p).name for p in g.params] == ["weight", "bias"]
    text = g.to_string()
    assert text == g.to_string() and "matmul" in text and "param %weight : tensor<3x8xf32>" in text
    with pytest.raises(KeyError, match="no tensor bound"):
        run(g, {g.inputs[0]: x})
    with pytest.raises(ValueError, match="declared"):
        run(g, {g.inputs[0]: x[:, :4], g.params[0]: lin.weight, g.params[1]: lin.bias})


def _eager_grads(fn, params, *xs):
    for p in params:
        p.grad = None
    fn(*xs).backward()
    return [p.grad.clone() for p in params]


def test_backward_matches_eager_tape_on_add_sum():
    p = torch.randn(3, 4, requires_grad=True)
    x = torch.randn(3, 4)
    with GraphScope() as s:
        s.bind_input(x, "x")
        s.bind_param(p, "p")
        unused = torch.randn(2, requires_grad=True)
        s.bind_param(unused, "unused")
        y = (x + p).sum()
        s.mark_output(y)
    g = s.graph
    res = build_backward(g)
    assert len(res.cotangents) == 1 and len(res.dparams) == 2 and g.inputs[-1] == res.cotangents[0]
    out = run(g, {g.inputs[0]: x, g.params[0]: p.detach(), g.params[1]: unused.detach(),
                  res.cotangents[0]: torch.tensor(1.0)})
    assert torch.allclose(out[0], (x + p).sum())
    assert torch.equal(out[1], torch.ones(3, 4)) and torch.equal(out[2], torch.zeros(2))


def test_backward_matches_eager_tape_on_linear_relu_ce():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(10, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    x, y = torch.randn(6, 10), torch.randint(0, 4, (6,))
    step = GraphTrainStep(model, F.cross_entropy, x, y)
    assert "cross_entropy_with_logits_backward" in step.graph.op_kinds() and "relu_backward" in step.graph.op_kinds()
    for _ in range(2):
        x, y = torch.randn(6, 10), torch.randint(0, 4, (6,))
        loss = step(x, y)
        got = [p.grad.clone() for p in model.parameters()]
        want = _eager_grads(lambda a, b: F.cross_entropy(model(a), b), list(model.parameters()), x, y)
        assert torch.allclose(loss, F.cross_entropy(model(x), y), atol=1e-6)
        for a, b in zip(got, want):
            assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.parametrize("name", ["div", "sigmoid", "tanh", "exp_log", "softmax", "mean_dim", "permute", "batched_matmul"])
def test_backward_rules_against_autograd(name):
    torch.manual_seed(3)
    p = torch.randn(2, 3, 4, dtype=torch.float64, requires_grad=True)
    q = torch.rand(3, 4, dtype=torch.float64).add(0.5).requires_grad_()
    w = torch.randn(4, 5, dtype=torch.float64, requires_grad=True)
    fns = {
        "div": lambda: (p / q).sum() + (1.0 / q).sum(),
        "sigmoid": lambda: (torch.sigmoid(p) * q).sum(),
        "tanh": lambda: torch.tanh(p * 0.5).mean(),
        "exp_log": lambda: (torch.exp(p * 0.1) + torch.log(q)).sum(),
        "softmax": lambda: (torch.softmax(p, dim=-1) * q).sum(),
        "mean_dim": lambda: (p.mean(dim=1) * 2.0).sum(dim=0).sum(),
        "permute": lambda: (p.permute(2, 0, 1).reshape(4, 6).t().clone() * 2.0).sum(),
        "batched_matmul": lambda: (p @ w).tanh().sum(),
    }
    fn = fns[name]
    params = [p, q, w]
    with GraphScope() as s:
        for i, t in enumerate(params):
            s.bind_param(t, "pqw"[i])
        out = fn()
        s.mark_output(out)
    g = s.graph
    res = build_backward(g)
    outs = run(g, {g.params[0]: p.detach(), g.params[1]: q.detach(), g.params[2]: w.detach(),
                   res.cotangents[0]: torch.ones((), dtype=torch.float64)})
    for t in params:
        t.grad = None
    fn().backward()
    for got, t in zip(outs[1:], params):
        want = t.grad if t.grad is not None else torch.zeros_like(t)
        assert torch.allclose(got, want, atol=1e-10), name
    assert set(g.op_kinds()) <= set(supported_ops())


def test_max_has_no_backward_rule_and_rule_tables_are_consistent():
    p = torch.randn(3, 4, requires_grad=True)
    with GraphScope() as s:
        s.bind_param(p, "p")
        s.mark_output(p.max())
    with pytest.raises(NotImplementedError, match="no backward rule"):
        build_backward(s.graph)
    assert set(differentiable_ops()) <= set(supported_ops())


def _mlp():
    torch.manual_seed(1)
    return torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(64, 32), torch.nn.ReLU(), torch.nn.Linear(32, 10))


def test_mnist_mode_graph_round_trips_through_text():
    model = _mlp()
    x, y = torch.randn(8, 1, 8, 8), torch.randint(0, 10, (8,))
    step = GraphTrainStep(model, F.cross_entropy, x, y)
    g = step.graph
    text = emit_mlir(g)
    assert text.count('"tesseract.') == g.num_ops() and "func.func @main" in text
    assert '"tesseract.cross_entropy_with_logits"' in text and "tensor<8x10xf32>" in text
    g2 = parse_mlir(text)
    assert g2.op_kinds() == g.op_kinds() and [o.attrs for o in g2.ops] == [o.attrs for o in g.ops]
    assert emit_mlir(g2) == text
    # the parsed graph runs: bind by argument order (inputs, params, constants)
    src = list(g.inputs) + list(g.params) + list(g.constants)
    dst = list(g2.inputs) + list(g2.params) + list(g2.constants)
    env = {step.x_id: x, step.y_id: y, g.inputs[-1]: torch.tensor(1.0)}
    env.update({vid: p.detach() for vid, p in zip(g.params, model.parameters())})
    env.update({vid: g.constant_data[vid] for vid in g.constants})
    a = run(g, env)
    b = run(g2, {d: env[s_] for s_, d in zip(src, dst)})
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    # every forward op that reaches the loss got a backward rule: all params receive a real gradient
    assert all(torch.count_nonzero(t) > 0 for t in a[1:])


def test_graph_mode_training_reproduces_eager_loss_curve():
    xs = torch.randn(12, 16, 1, 8, 8, generator=torch.Generator().manual_seed(5))
    ys = torch.randint(0, 10, (12, 16), generator=torch.Generator().manual_seed(6))
    curves = {}
    for engine in ("eager", "graph"):
        model = _mlp()
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
        step = GraphTrainStep(model, F.cross_entropy, xs[0], ys[0]) if engine == "graph" else None
        losses = []
        for x, y in zip(xs, ys):
            if step is None:
                opt.zero_grad()
                loss = F.cross_entropy(model(x), y)
                loss.backward()
            else:
                loss = step(x, y)
            opt.step()
            losses.append(float(loss))
        curves[engine] = losses
    assert curves["graph"][-1] < curves["graph"][0]
    assert torch.allclose(torch.tensor(curves["graph"]), torch.tensor(curves["eager"]), atol=1e-5)


def test_executor_on_cpu_interprets_and_shares_params():
    w = torch.ones(2, 2)
    g = Graph()
    x = g.add_input((2, 2), torch.float32, "cpu", "x")
    p = g.add_param((2, 2), torch.float32, "cpu", "w")
    o = g.new_value((2, 2), torch.float32, "cpu")
    g.add_op("matmul", [x, p], [o])
    g.mark_output(o)
    ex = GraphExecutor(g, {x: torch.eye(2), p: w}, share=[p])
    assert not ex.cuda_graph and torch.equal(ex()[0], torch.ones(2, 2))
    w.mul_(3.0)
    assert torch.equal(ex({x: 2 * torch.eye(2)})[0], 6 * torch.ones(2, 2))
    with pytest.raises(ValueError, match="needs the bindings on a CUDA device"):
        GraphExecutor(g, {x: torch.eye(2), p: w}, cuda_graph=True)


def test_execution_plan_drops_dead_ops_and_fuses_linear_layers():
    """The interpreter's plan: the gradient of the input batch never reaches an output and is dropped, a Linear layer
    runs as one fused op, the weight gradient comes out contiguous in the parameter's layout -- and the results equal
    autograd's."""
    import torch.nn.functional as F
    from tesseract_b200.graph import GraphTrainStep
    from tesseract_b200.graph.interpreter import plan
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(36, 16), torch.nn.ReLU(), torch.nn.Linear(16, 5))
    x, y = torch.rand(7, 1, 6, 6), torch.randint(0, 5, (7,))
    step = GraphTrainStep(model, F.cross_entropy, x, y, cuda_graph=False)
    kinds = [op.kind for op in plan(step.graph)]
    assert kinds.count("fused_linear") == 2 and kinds.count("matmul_tn") == 2
    assert len(kinds) < step.graph.num_ops()
    assert kinds.count("matmul") == 1                       # only the hidden activation's gradient is left
    assert set(step.graph.op_kinds()) <= set(supported_ops())   # the IR itself is untouched
    loss = step(x, y)
    got = [p.grad.clone() for p in model.parameters()]
    assert all(g.is_contiguous() for g in got)
    for p in model.parameters():
        p.grad = None
    ref = F.cross_entropy(model(x), y)
    ref.backward()
    assert torch.allclose(loss, ref.detach(), atol=1e-6)
    for g, p in zip(got, model.parameters()):
        assert torch.allclose(g, p.grad, atol=1e-5)
