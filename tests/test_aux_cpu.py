"""Auxiliary subsystems on CPU: failure detection (host-injected faults only), checkpoints, metrics, graph capture."""
import json

import pytest
import torch

from tesseract_b200.graph import GraphScope, build_backward, run
from tesseract_b200.models import LlamaConfig, LlamaModel
from tesseract_b200.training import TrainConfig, Trainer
from tesseract_b200.utils import checkpoint, env, metrics
from tesseract_b200.utils.watchdog import DictStore, RankLost, RankWatchdog


def test_watchdog_detects_silent_never_joined_and_failed_ranks():
    store, now = DictStore(), [0.0]
    clock = lambda: now[0]
    a = RankWatchdog(store, 0, 3, timeout_s=5.0, clock=clock)
    b = RankWatchdog(store, 1, 3, timeout_s=5.0, clock=clock)
    a.check()                      # rank 2 has not joined yet: tolerated until the timeout
    now[0] = 3.0
    b.beat(); a.step()
    now[0] = 6.0
    b.beat()
    with pytest.raises(RankLost) as e:   # rank 2 never joined
        a.check()
    assert e.value.rank == 2 and "never joined" in e.value.reason
    c = RankWatchdog(store, 2, 3, timeout_s=5.0, clock=clock)
    a._seen.clear(); a.check()
    now[0] = 20.0
    c.beat()
    with pytest.raises(RankLost) as e:   # rank 1 stopped beating
        a.check()
    assert e.value.rank == 1
    b.beat()
    c.report_failure("ValueError: injected on the host")
    with pytest.raises(RankLost) as e:   # rank 2 raised and told the others before their next launch
        a.check()
    assert e.value.rank == 2 and "injected" in e.value.reason


def test_checkpoint_roundtrip_and_resume(tmp_path):
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                      intermediate_size=64, max_position_embeddings=32)
    torch.manual_seed(0)
    batch = torch.randint(0, 64, (2, 17))
    m1 = LlamaModel(cfg, init_std=0.1, seed=1)
    t1 = Trainer(m1, TrainConfig(lr=1e-2, micro_batch=2))
    for _ in range(3):
        t1.train_step(batch)
    path = str(tmp_path / "ckpt.tsrct")
    checkpoint.save_checkpoint(path, m1, t1)
    man = json.load(open(path + "/manifest.json"))
    assert man["format"] == "tsrct" and man["step"] == 3 and man["config"]["hidden_size"] == 32
    after = [t1.train_step(batch) for _ in range(2)]
    m2 = LlamaModel(cfg, init_std=0.1, seed=99)
    t2 = Trainer(m2, TrainConfig(lr=1e-2, micro_batch=2))
    checkpoint.load_checkpoint(path, m2, t2)
    assert t2.steps_done == 3
    resumed = [t2.train_step(batch) for _ in range(2)]
    assert resumed == pytest.approx(after, abs=1e-6)


def test_metrics_and_env(tmp_path):
    p = str(tmp_path / "m.jsonl")
    log = metrics.MetricsLogger(p)
    log.log(step=1, tok_s=123.0)
    line = log.bench_line("decode", tok_s=10, ttft_ms=1.5)
    log.close()
    rec = json.loads(open(p).read().strip())
    assert rec["step"] == 1 and line.startswith("[bench] decode tok_s=10")
    assert metrics.percentile([5, 1, 3], 50) == 3
    assert env.get("TESSERACT_GEMM") in ("tcgen05", "cublas") and "TESSERACT_TP_COMM" in env.describe()


def test_graph_capture_run_and_backward():
    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = torch.nn.Linear(4, 8), torch.nn.Linear(8, 2)

        def forward(self, x):
            return self.b(torch.relu(self.a(x))) + 1.0

    m = MLP()
    x = torch.randn(3, 4)
    with GraphScope() as scope:
        g = scope.trace(m, x, names=["x"])
    assert [k for k in g.op_kinds() if k in ("matmul", "relu")] == ["matmul", "relu", "matmul"] and g.op_kinds()[-1] == "add"
    assert [g.value(i).name for i in g.inputs] == ["x"] and len(g.params) == 4
    x2 = torch.randn(3, 4)
    env = {g.inputs[0]: x2}
    env.update({vid: p.detach() for vid, p in zip(g.params, m.parameters())})
    assert torch.allclose(run(g, env)[0], m(x2))
    res = build_backward(g, wrt=[g.inputs[0]])
    env[res.cotangents[0]] = torch.ones(3, 2)
    gx = run(g, env)[-1]
    xr = x2.clone().requires_grad_()
    m(xr).sum().backward()
    assert torch.allclose(gx, xr.grad, atol=1e-6)


def test_decode_gemm_plan():
    """The decode GEMM planner: one wave of cluster CTAs for small outputs, the persistent GEMM once the tiles
    fill the GPU, atomics only on request."""
    from tesseract_b200.ops.gemm import plan_decode_gemm
    for M in (1, 64, 256):
        kind, s = plan_decode_gemm(M, 4096, 4096)                  # o_proj: 32 or 64 tiles
        assert kind == "cluster" and s in (1, 2, 4, 8)
        tiles = ((M + 127) // 128) * 32
        assert tiles * s <= 148 and (s == 8 or tiles * s * 2 > 148 or 64 // (s * 2) < 8)
    assert plan_decode_gemm(64, 28672, 4096) == ("plain", 0)       # gate_up: 224 tiles already fill the GPU
    assert plan_decode_gemm(256, 128256, 4096) == ("plain", 0)     # lm_head
    assert plan_decode_gemm(64, 4096, 512)[0] == "cluster" and plan_decode_gemm(64, 4096, 512)[1] == 1   # 8 k-blocks
    kind, s = plan_decode_gemm(64, 6144, 4096, mode="simple")
    assert kind == "atomic" and 2 <= s <= 16
    assert plan_decode_gemm(64, 28672, 4096, mode="simple") == ("plain", 0)


def test_every_environment_variable_read_by_the_code_is_registered():
    import os
    import re
    from tesseract_b200.utils import env
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    used = set()
    for base in ("tesseract_b200", "benchmarks", "examples"):
        for d, _, files in os.walk(os.path.join(root, base)):
            for f in files:
                if f.endswith((".py", ".cu", ".cuh", ".cpp", ".hpp")):
                    text = open(os.path.join(d, f), errors="replace").read()
                    used |= set(re.findall(r'(?:getenv\(|environ\.get\(|environ\[)\s*"(TESSERACT_[A-Z0-9_]+)"', text))
    used |= set(re.findall(r'environ\.get\(\s*"(TESSERACT_[A-Z0-9_]+)"', open(os.path.join(root, "bench.py")).read()))
    missing = sorted(used - set(env.REGISTRY))
    assert not missing, f"not in utils/env.py: {missing}"
    assert "TESSERACT_SWIGLU" in used and len(used) >= 12


def test_trainer_writes_metrics_and_stops_on_a_lost_peer(tmp_path):
    """The instrumented Trainer: one metrics record per step; a peer's posted error or silence raises RankLost on the
    host BEFORE the step launches anything (the step counter does not move); its own exception reaches the store."""
    import json

    from tesseract_b200.models import LlamaConfig, LlamaModel
    from tesseract_b200.training import TrainConfig, Trainer
    from tesseract_b200.utils.metrics import MetricsLogger
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                      intermediate_size=48, max_position_embeddings=16)
    trainer = Trainer(LlamaModel(cfg, init_std=0.02, seed=0), TrainConfig(lr=1e-3))
    now = [0.0]
    store = DictStore()
    me = RankWatchdog(store, 0, 2, timeout_s=5.0, clock=lambda: now[0])
    peer = RankWatchdog(store, 1, 2, timeout_s=5.0, clock=lambda: now[0])
    path = tmp_path / "m.jsonl"
    trainer.instrument(metrics=MetricsLogger(str(path)), watchdog=me, nvtx_ranges=True)
    batch = torch.randint(0, 64, (2, 9))
    for _ in range(2):
        peer.beat()
        trainer.train_step(batch)
    recs = [json.loads(line) for line in path.read_text().splitlines()]
    assert [r["step"] for r in recs] == [1, 2] and all(r["step_ms"] > 0 and r["tokens_per_s_rank"] > 0 for r in recs)
    now[0] = 10.0                                    # the peer has been silent for longer than the timeout
    with pytest.raises(RankLost, match="no heartbeat"):
        trainer.train_step(batch)
    assert trainer.steps_done == 2
    peer.beat()
    peer.report_failure("ValueError: boom")
    with pytest.raises(RankLost, match="boom"):
        trainer.train_step(batch)
    # this rank's own failure is posted for the others
    with pytest.raises(Exception):
        trainer.watchdog = RankWatchdog(DictStore(), 0, 1)
        trainer.train_step(torch.randint(0, 64, (2, 40)))        # longer than max_position_embeddings
    assert trainer.watchdog.store.get("tsb/hb/error/0")
