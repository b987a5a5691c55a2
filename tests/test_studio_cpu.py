"""Visual-builder core on CPU (mirrors the reference's studio/core/tests/test_studio.cpp)."""
import threading

from tesseract_b200.studio import (BlockCatalog, BlockGraph, Executor, RunOptions, analyze, extract_tsb, generate_ir,
                                   generate_python)


def make_mlp_graph(epochs=30):
    g = BlockGraph("mlp")
    cat = BlockCatalog.instance()
    inp = g.add_node("Input", {"batch": 32, "features": 8})
    l1 = g.add_node("Linear", {"in_features": 8, "out_features": 32, "bias": True})
    act = g.add_node("ReLU")
    l2 = g.add_node("Linear", {"in_features": 32, "out_features": 3, "bias": True})
    seq = g.add_node("SequentialModel")
    ds = g.add_node("SyntheticClassification", cat.default_params("SyntheticClassification"))
    loss = g.add_node("CrossEntropyLoss")
    opt = g.add_node("Adam", {"lr": 0.01})
    loop = g.add_node("TrainLoop", {"epochs": epochs, "batch_size": 32})
    g.connect(inp, "out", l1, "in")
    g.connect(l1, "out", act, "in")
    g.connect(act, "out", l2, "in")
    g.connect(l2, "out", seq, "in")
    g.connect(seq, "model", opt, "model")
    g.connect(seq, "model", loop, "model")
    g.connect(ds, "data", loop, "data")
    g.connect(opt, "opt", loop, "optimizer")
    g.connect(loss, "loss", loop, "loss")
    return g


def make_tensor_graph():
    g = BlockGraph("tensor")
    a = g.add_node("TensorConst", {"rows": 3, "cols": 4, "init": "randn", "seed": 1})
    b = g.add_node("TensorConst", {"rows": 4, "cols": 2, "init": "arange", "scale": 0.1})
    mm = g.add_node("TMatMul")
    th = g.add_node("TTanh")
    ins = g.add_node("TensorInspect", {"backward": True})
    g.connect(a, "out", mm, "a")
    g.connect(b, "out", mm, "b")
    g.connect(mm, "out", th, "in")
    g.connect(th, "out", ins, "in")
    return g


def make_llama_graph():
    g = BlockGraph("llama")
    m = g.add_node("LoadLlama", BlockCatalog.instance().default_params("LoadLlama"))
    gen = g.add_node("Generate", {"prompt_ids": "1, 2, 3", "max_new_tokens": 6})
    g.connect(m, "model", gen, "model")
    return g


def run_collect(g, opt=None):
    events = []
    summary = Executor.run(g, events.append, opt)
    return events, summary


def test_tsb_is_bidirectional_and_catalog_has_core_kinds():
    g = make_mlp_graph()
    tsb = g.to_tsb()
    g2 = BlockGraph.from_tsb(tsb)
    assert len(g2.nodes) == len(g.nodes) and len(g2.edges) == len(g.edges) and g2.to_tsb() == tsb
    assert g2.add_node("ReLU") == max(n.id for n in g.nodes) + 1
    cat = BlockCatalog.instance()
    for kind in ("Linear", "TrainLoop", "LoadLlama", "Generate", "TensorConst", "TMatMul", "TensorInspect"):
        assert cat.find(kind) is not None
    assert len(cat.to_json()) >= 15 and cat.find("Nope") is None
    assert cat.default_params("Adam") == {"lr": 1e-3, "beta1": 0.9, "beta2": 0.999, "eps": 1e-8}


def test_analysis_validates_and_flags():
    g = make_mlp_graph()
    a = analyze(g)
    assert a.ok and any(s == [32, 3] for s in a.out_shapes.values())
    bad = g.copy()
    bad.edges = [e for e in bad.edges if e.dst.port != "data"]
    b = analyze(bad)
    assert not b.ok and any("'data' is not connected" in d.message for d in b.diagnostics)
    bad = g.copy()
    ds = next(n.id for n in bad.nodes if n.kind == "SyntheticClassification")
    bad.connect(ds, "data", bad.nodes[1].id, "in")
    b = analyze(bad)
    assert not b.ok and any("type mismatch" in d.message for d in b.diagnostics)
    bad = g.copy()
    bad.nodes[3].params["in_features"] = 16                      # wrong width: a warning, not an error
    b = analyze(bad)
    assert b.ok and any(d.severity == "warning" and "in_features expects last dim 16" in d.message for d in b.diagnostics)
    bad = g.copy()
    bad.add_node("Mystery")
    bad.connect(bad.nodes[2].id, "out", bad.nodes[1].id, "in")   # ReLU -> first Linear: a cycle
    b = analyze(bad)
    msgs = " | ".join(d.message for d in b.diagnostics)
    assert not b.ok and "unknown block kind 'Mystery'" in msgs and "cycle" in msgs
    t = analyze(make_tensor_graph())
    assert t.ok and [3, 2] in t.out_shapes.values()
    assert set(t.to_json()) == {"ok", "diagnostics", "shapes"}


def test_codegen_round_trips_and_lowers_to_the_dialect():
    g = make_mlp_graph()
    py = generate_python(g)
    assert "ts.nn.Sequential" in py and "ts.ops.cross_entropy" in py and "ts.optim.Adam" in py
    compile(py, "<generated>", "exec")
    back = extract_tsb(py)
    assert back is not None and len(back.nodes) == len(g.nodes) and back.to_tsb() == g.to_tsb()
    assert extract_tsb("print('no graph here')") is None
    for other in (make_tensor_graph(), make_llama_graph()):
        src = generate_python(other)
        compile(src, "<generated>", "exec")
        assert extract_tsb(src).to_tsb() == other.to_tsb()
    ir = generate_ir(g)
    assert "tesseract.matmul" in ir and "tesseract.relu" in ir and "func.func @forward" in ir
    tir = generate_ir(make_tensor_graph())
    assert "tesseract.matmul" in tir and "tensor<3x2xf32>" in tir and "tesseract.tanh" in tir


def test_executor_trains_an_mlp():
    events, summary = run_collect(make_mlp_graph(60))
    losses = [e.data["loss"] for e in events if e.type == "loss"]
    done = [e for e in events if e.type == "done"]
    assert len(done) == 1 and done[0].data == summary and summary["ok"] and summary["mode"] == "train"
    assert len(losses) > 10 and losses[-1] < losses[0] and summary["final_acc"] > 0.8
    assert sum(1 for e in events if e.type == "metric") == 60


def test_executor_evaluates_a_tensor_graph_and_backprops():
    events, summary = run_collect(make_tensor_graph())
    results = [e for e in events if e.type == "tensor" and e.data["role"] == "result"]
    grads = [e for e in events if e.type == "tensor" and e.data["role"] == "grad"]
    assert summary == {"ok": True, "mode": "tensor", "backward": True, "leaves": 2}
    assert len(results) == 1 and results[0].data["shape"] == [3, 2] and results[0].data["numel"] == 6
    assert len(grads) == 2 and grads[0].data["shape"] == [3, 4] and grads[1].data["shape"] == [4, 2]


def test_executor_generates_from_llama_and_mamba_blocks():
    events, summary = run_collect(make_llama_graph())
    assert summary["ok"] and summary["generated"] == 6 and summary["prompt_len"] == 3
    assert sum(1 for e in events if e.type == "token") == 6 and summary["ids"][:3] == [1, 2, 3]
    g = BlockGraph("mamba")
    m = g.add_node("LoadMamba", BlockCatalog.instance().default_params("LoadMamba"))
    gen = g.add_node("Generate", {"prompt_ids": "4, 5", "max_new_tokens": 3})
    g.connect(m, "model", gen, "model")
    events, summary = run_collect(g)
    assert summary["ok"] and summary["generated"] == 3


def test_executor_reports_failures_and_cancellation():
    g = make_mlp_graph()
    g.edges = [e for e in g.edges if e.dst.port != "optimizer"]
    events, summary = run_collect(g)
    assert summary == {"ok": False, "reason": "validation failed"} and any(e.type == "error" for e in events)
    lone = BlockGraph()
    lone.add_node("Input")
    assert run_collect(lone)[1]["reason"] == "no sink"
    bad = make_llama_graph()
    bad.nodes[1].params["prompt_ids"] = "999999"
    assert "outside" in run_collect(bad)[1]["reason"]
    cancel = threading.Event()
    cancel.set()
    assert run_collect(make_mlp_graph(), RunOptions(cancel=cancel))[1] == {"ok": False, "reason": "cancelled"}
    assert "no CUDA device" in run_collect(make_mlp_graph(), RunOptions(device="cuda"))[1]["reason"] \
        or __import__("torch").cuda.is_available()


def test_generated_scripts_run():
    for g in (make_mlp_graph(2), make_tensor_graph(), make_llama_graph()):
        exec(compile(generate_python(g), f"<generated {g.name}>", "exec"), {})


def test_http_api_serves_catalog_analysis_codegen_and_streams_a_run():
    import json
    import urllib.error
    import urllib.request
    from tesseract_b200.studio.server import StudioServer
    srv = StudioServer(("127.0.0.1", 0))
    port = srv.server_address[1]
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    try:
        base = f"http://127.0.0.1:{port}"

        def post(path, body):
            req = urllib.request.Request(base + path, data=body.encode(), method="POST")
            with urllib.request.urlopen(req, timeout=60) as r:
                return r.read().decode()

        assert "<textarea" in urllib.request.urlopen(base + "/", timeout=10).read().decode()
        kinds = [b["kind"] for b in json.loads(urllib.request.urlopen(base + "/api/catalog", timeout=10).read())]
        assert "TrainLoop" in kinds and "LoadLlama" in kinds
        tsb = make_mlp_graph(3).to_tsb()
        assert json.loads(post("/api/analyze", tsb))["ok"] is True
        src = json.loads(post("/api/codegen?target=python", tsb))["source"]
        assert "ts.nn.Sequential" in src
        assert "tesseract.matmul" in json.loads(post("/api/codegen?target=ir", tsb))["source"]
        back = json.loads(post("/api/import", json.dumps({"source": src})))
        assert len(back["nodes"]) == 9
        events = [json.loads(l) for l in post("/api/run", tsb).splitlines() if l.strip()]
        assert events[-1]["type"] == "done" and events[-1]["data"]["ok"] and events[-1]["data"]["steps"] == 24
        assert sum(1 for e in events if e["type"] == "metric") == 3
        for path, body, code in (("/api/analyze", "not json", 400), ("/api/codegen?target=cobol", tsb, 400), ("/api/nope", tsb, 404)):
            try:
                post(path, body)
                raise AssertionError("expected an HTTP error")
            except urllib.error.HTTPError as e:
                assert e.code == code
    finally:
        srv.shutdown()
        srv.server_close()
