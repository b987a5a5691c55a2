#!/usr/bin/env python
"""CPU-side benchmarks with the shapes of the reference's informational CPU benches (benchmarks/bench_matmul.cpp,
bench_python_overhead.cpp + bench/external/python_overhead.py, bench_graph_vs_eager.cpp, bench_moe_sparse.cpp):

* ``matmul``           native fp32 GEMM of the host runtime (csrc/host/gemm_f32.cpp) at 128^3 .. 1024^3, beside torch's
                       library GEMM on the same cores;
* ``python_overhead``  per-call cost of the drop-in ``tesseract._core`` frontend over the tensor library underneath it
                       (add / matmul / Linear forward on small and real-size operands);
* ``graph_vs_eager``   one training step of the MNIST MLP: eager autograd against the recorded graph with its
                       backward pass appended as a graph transform and interpreted (tesseract_b200/graph);
* ``moe_sparse``       sparse top-k MoE forward against all experts on every token.

No GPU is used. One JSON line per measurement; ``--case`` selects (repeatable).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np  # noqa: E402
import torch  # noqa: E402


def best_of(fn, iters: int, reps: int = 5) -> float:
    """Seconds per call: the best of ``reps`` batches of ``iters`` calls (after one warm-up call)."""
    fn()
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        best = min(best, (time.perf_counter() - t0) / iters)
    return best


def out(**kw):
    print(json.dumps(kw), flush=True)


def case_matmul():
    from tesseract_b200 import _native
    host = _native.host()
    for n in (128, 256, 512, 1024):
        a = np.random.default_rng(n).standard_normal((n, n)).astype(np.float32)
        b = np.random.default_rng(n + 1).standard_normal((n, n)).astype(np.float32)
        ta, tb = torch.from_numpy(a), torch.from_numpy(b)
        iters = max(10, int(4e9 / (2 * n ** 3)))
        rec = {"case": "matmul", "n": n, "threads_available": torch.get_num_threads()}
        if host is not None:
            s = best_of(lambda: host.gemm_f32(a, b, False, 0), iters)
            rec["native_gflops"] = round(2 * n ** 3 / s / 1e9, 1)
            rec["native_threads"] = int(host.gemm_num_threads(n, n, n, 0))
        s = best_of(lambda: ta @ tb, iters)
        rec["torch_gflops"] = round(2 * n ** 3 / s / 1e9, 1)
        out(**rec)


def case_python_overhead():
    import tesseract as ts
    from tesseract import _core
    for n in (8, 64, 512):
        a_np = np.random.default_rng(0).standard_normal((n, n)).astype(np.float32)
        a, b = _core.Tensor(a_np), _core.Tensor(a_np.copy())
        ta, tb = torch.from_numpy(a_np), torch.from_numpy(a_np.copy())
        iters = 2000 if n <= 64 else 200
        for name, f_core, f_torch in (("add", lambda: _core.ops.add(a, b), lambda: torch.add(ta, tb)),
                                      ("matmul", lambda: _core.ops.matmul(a, b), lambda: torch.matmul(ta, tb))):
            s_core, s_torch = best_of(f_core, iters), best_of(f_torch, iters)
            out(case="python_overhead", op=name, n=n, frontend_us=round(s_core * 1e6, 2), library_us=round(s_torch * 1e6, 2),
                overhead_us=round((s_core - s_torch) * 1e6, 2), overhead_pct=round(100 * (s_core - s_torch) / s_torch, 1))
    lin = _core.nn.Linear(256, 256)
    x = _core.Tensor(np.random.default_rng(1).standard_normal((32, 256)).astype(np.float32))
    tl = torch.nn.Linear(256, 256)
    tx = torch.randn(32, 256)
    with torch.no_grad():
        s_core, s_torch = best_of(lambda: lin(x), 2000), best_of(lambda: tl(tx), 2000)
    out(case="python_overhead", op="linear_32x256x256", frontend_us=round(s_core * 1e6, 2),
        library_us=round(s_torch * 1e6, 2), overhead_us=round((s_core - s_torch) * 1e6, 2))
    assert ts.__version__


def case_graph_vs_eager():
    import torch.nn.functional as F
    from tesseract_b200.graph import GraphTrainStep
    for hidden, batch in ((128, 64), (512, 128)):
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, hidden), torch.nn.ReLU(),
                                    torch.nn.Linear(hidden, 10))
        x, y = torch.rand(batch, 1, 28, 28), torch.randint(0, 10, (batch,))
        step = GraphTrainStep(model, F.cross_entropy, x, y, cuda_graph=False)

        def eager():
            for p in model.parameters():
                p.grad = None
            F.cross_entropy(model(x), y).backward()

        s_eager, s_graph = best_of(eager, 200), best_of(lambda: step(x, y), 200)
        out(case="graph_vs_eager", hidden=hidden, batch=batch, forward_ops=step.forward_ops,
            total_ops=step.graph.num_ops(), eager_us=round(s_eager * 1e6, 1), graph_us=round(s_graph * 1e6, 1),
            graph_over_eager=round(s_graph / s_eager, 2))


def case_moe_sparse():
    from tesseract_b200.nn.moe import MoEFeedForward
    # the last shape is the one the reference publishes (docs/design/moe-sparse.md:41-47: 300 ms sparse, 644 ms dense)
    for (T, D, F_, E, k) in ((512, 256, 512, 8, 2), (2048, 256, 512, 8, 2), (2048, 256, 512, 16, 1),
                             (4096, 512, 1024, 8, 2)):
        torch.manual_seed(0)
        moe = MoEFeedForward(D, F_, num_experts=E, num_experts_per_tok=k)
        x = torch.randn(1, T, D)
        with torch.no_grad():
            s_sparse = best_of(lambda: moe(x), 5, reps=3)
            s_dense = best_of(lambda: moe.forward_dense_reference(x), 5, reps=3)
            err = (moe(x) - moe.forward_dense_reference(x)).abs().max().item()
        out(case="moe_sparse", tokens=T, hidden=D, ffn=F_, experts=E, top_k=k, sparse_ms=round(s_sparse * 1e3, 2),
            dense_ms=round(s_dense * 1e3, 2), speedup=round(s_dense / s_sparse, 2), max_abs_diff=round(err, 6))


def case_mamba_vs_llama():
    """Decode-step latency against context length (the reference's bench_mamba_vs_llama_scaling: d = 256, 4 layers;
    docs/design/mamba-scaling.md:41-47 reports Mamba flat at 12.4 ms and Llama 14.6 -> 27.3 ms for 128 -> 2048)."""
    from tesseract_b200.models import LlamaConfig, LlamaModel
    from tesseract_b200.models.mamba import MambaConfig, MambaModel
    torch.manual_seed(0)
    lcfg = LlamaConfig(vocab_size=32000, hidden_size=256, num_hidden_layers=4, num_attention_heads=8,
                       num_key_value_heads=8, intermediate_size=688, max_position_embeddings=4096, dtype=torch.float32)
    llama = LlamaModel(lcfg)
    mamba = MambaModel(MambaConfig(vocab_size=32000, hidden_size=256, num_hidden_layers=4))
    tok = torch.tensor([[5]])
    with torch.no_grad():
        for L in (128, 512, 2048):
            caches = llama.make_kv_caches(1, L + 64)
            llama.forward_step(torch.randint(0, 32000, (1, L)), caches)          # fill the context
            s_llama = best_of(lambda: (llama.forward_step(tok, caches), [c.set_current_len(L) for c in caches])[0], 20, reps=3)
            states = mamba.make_state_caches(1)
            for t in torch.randint(0, 32000, (8,)).tolist():                     # the recurrent state has no length
                mamba.forward_step(torch.tensor([[t]]), states)
            s_mamba = best_of(lambda: mamba.forward_step(tok, states), 20, reps=3)
            out(case="mamba_vs_llama", context=L, llama_ms=round(s_llama * 1e3, 3), mamba_ms=round(s_mamba * 1e3, 3))


CASES = {"mamba_vs_llama": case_mamba_vs_llama, "matmul": case_matmul, "python_overhead": case_python_overhead, "graph_vs_eager": case_graph_vs_eager,
         "moe_sparse": case_moe_sparse}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--case", action="append", choices=sorted(CASES), help="repeatable; default: all")
    a = ap.parse_args()
    for name in (a.case or sorted(CASES)):
        CASES[name]()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
