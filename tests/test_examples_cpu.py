"""The example command lines run end to end on CPU (the reference ships the same three as C++ binaries and drives
them from ctest: examples/llama_train.cpp, llama_generate.cpp, llama_serve.cpp)."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=300):
    return subprocess.run([sys.executable, *args], cwd=os.path.join(ROOT, "examples"), capture_output=True, text=True,
                          timeout=timeout)


def test_llama_train_converges_below_gate(tmp_path):
    r = _run("llama_train.py", "--steps", "60", "--lr", "3e-3", "--target-loss", "0.5", "--save", str(tmp_path / "ck"))
    assert r.returncode == 0, r.stdout + r.stderr
    assert "loss" in r.stdout and (tmp_path / "ck").exists()
    r = _run("llama_train.py", "--steps", "2", "--target-loss", "0.001")
    assert r.returncode == 1 and "FAILED" in r.stderr


def test_llama_generate_greedy_sampled_and_constrained():
    r = _run("llama_generate.py", "--model", "tiny", "--prompt", "hi", "--max-new-tokens", "5", "--no-stream")
    assert r.returncode == 0 and "5 new tokens" in r.stderr
    r2 = _run("llama_generate.py", "--model", "tiny", "--prompt", "hi", "--max-new-tokens", "5", "--no-stream")
    assert r2.stdout == r.stdout                                   # greedy decoding is deterministic
    r = _run("llama_generate.py", "--model", "tiny", "--prompt", "12", "--max-new-tokens", "6", "--grammar-regex",
             "[0-9]+", "--sample", "--top-p", "0.9", "--seed", "3", "--kv-int8", "--no-stream")
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip().isdigit() and len(r.stdout.strip()) == 8
    assert _run("llama_generate.py").returncode == 1               # no model given


def test_llama_serve_finishes_every_request():
    r = _run("llama_serve.py", "--model", "tiny", "--prompts", "a|bb|ccc", "--max-new-tokens", "4", "--max-batch", "2")
    assert r.returncode == 0, r.stderr
    assert r.stdout.count("done at step") == 3 and "3 requests, 12 tokens" in r.stdout


def test_mnist_graph_mode_matches_eager():
    """Graph-mode training replays one recorded graph; with the same seed it follows the eager run step for step
    (examples/mnist.cpp --mode graph; tests/graph/test_graph_train_parity.cpp)."""
    outs = {}
    for mode in ("eager", "graph"):
        r = _run("mnist.py", "--synthetic", "--mode", mode, "--max-steps", "40", "--seed", "1")
        assert r.returncode == 0, r.stderr
        outs[mode] = [l for l in r.stdout.splitlines() if l.startswith("epoch 1")][0]
    field = lambda line, key: float(line.split(key + "=")[1].split()[0])      # noqa: E731
    assert abs(field(outs["eager"], "loss") - field(outs["graph"], "loss")) < 1e-3
    assert field(outs["graph"], "test_acc") > 0.9
    r = _run("mnist.py", "--synthetic", "--mode", "graph", "--max-steps", "1", "--dump-ir")
    assert '"tesseract.cross_entropy_with_logits_backward"' in r.stdout and "func.func @main" in r.stdout
    assert _run("mnist.py").returncode != 0                                   # neither a directory nor --synthetic
    assert _run("mnist.py", "--synthetic", "--mode", "graph", "--engine", "mlir").returncode != 0


def test_llama_forward_and_infer():
    r = _run("llama_forward.py", "--backward")
    assert r.returncode == 0, r.stderr
    assert "finite  = 2048 / 2048" in r.stdout and "backward: sum(||grad||)" in r.stdout
    r = _run("llama_infer.py", "--synthetic", "--batch", "2", "--seq", "8", "--topk", "3")
    assert r.returncode == 0, r.stderr
    assert "logits.shape = [2, 8, 512]" in r.stdout and r.stdout.count("  id=") == 3
    r = _run("llama_infer.py", "--synthetic", "--prompt", "hey", "--generate", "--max-new-tokens", "4")
    assert r.returncode == 0 and "generated 4 tokens" in r.stdout
    assert _run("llama_infer.py").returncode != 0
