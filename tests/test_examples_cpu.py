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
