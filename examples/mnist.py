"""MNIST two-layer MLP trainer in eager mode or graph mode (the reference's examples/mnist.cpp:380-470 command
line). Graph mode records forward + loss once, appends the backward pass as a graph transform and replays that
graph every step (one CUDA-graph launch per step on a GPU); ``--dump-ir`` prints the graph as ``tesseract``-dialect
text. The data directory holds the four IDX files; with ``--synthetic`` (or when the files are absent and
``--synthetic-if-missing`` is given) ten noisy class prototypes of the same shape stand in.

    python examples/mnist.py data/mnist --mode graph --epochs 1 --max-steps 50
    python examples/mnist.py --synthetic --mode graph --dump-ir
"""
from __future__ import annotations

import argparse
import os
import struct
import time

import _common  # noqa: F401  (puts the repository root on sys.path)
import torch
import torch.nn.functional as F

from tesseract_b200.graph import GraphTrainStep, emit_mlir


def load_idx_images(path: str) -> torch.Tensor:
    with open(path, "rb") as f:
        magic, n, rows, cols = struct.unpack(">IIII", f.read(16))
        if magic != 2051:
            raise SystemExit(f"error: {path} is not an IDX3 image file (magic {magic})")
        data = torch.frombuffer(bytearray(f.read(n * rows * cols)), dtype=torch.uint8)
    return data.reshape(n, 1, rows, cols).float().div_(255.0)


def load_idx_labels(path: str) -> torch.Tensor:
    with open(path, "rb") as f:
        magic, n = struct.unpack(">II", f.read(8))
        if magic != 2049:
            raise SystemExit(f"error: {path} is not an IDX1 label file (magic {magic})")
        data = torch.frombuffer(bytearray(f.read(n)), dtype=torch.uint8)
    return data.long()


def synthetic_digits(n_train: int = 8192, n_test: int = 1024, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    protos = torch.rand(10, 1, 28, 28, generator=g)

    def draw(n):
        y = torch.randint(0, 10, (n,), generator=g)
        x = (protos[y] + 0.35 * torch.randn(n, 1, 28, 28, generator=g)).clamp_(0.0, 1.0)
        return x, y
    return (*draw(n_train), *draw(n_test))


def evaluate(model, x, y, batch: int) -> float:
    hit = 0
    with torch.no_grad():
        for i in range(0, x.shape[0], batch):
            hit += int((model(x[i:i + batch]).argmax(-1) == y[i:i + batch]).sum())
    return hit / max(1, x.shape[0])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("data_dir", nargs="?", default="")
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--max-steps", type=int, default=0, help="cap on batches per epoch (<= 0: unlimited)")
    ap.add_argument("--mode", default="eager", choices=["eager", "graph"])
    ap.add_argument("--engine", default="interp", help="graph engine: interp (the MLIR JIT engine is not built)")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--dump-ir", action="store_true")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--synthetic-if-missing", action="store_true")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    if args.engine != "interp":
        raise SystemExit(f"error: --engine '{args.engine}' is not available; only 'interp' is built")
    dev = _common.pick_device(args.device)

    files = ["train-images-idx3-ubyte", "train-labels-idx1-ubyte", "t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte"]
    have = bool(args.data_dir) and all(os.path.exists(os.path.join(args.data_dir, f)) for f in files)
    if args.synthetic or (not have and args.synthetic_if_missing):
        print("data: synthetic digits (10 noisy prototypes, 28x28)")
        train_x, train_y, test_x, test_y = synthetic_digits(seed=args.seed)
    elif have:
        print(f"Loading MNIST from {args.data_dir} ...")
        train_x, test_x = (load_idx_images(os.path.join(args.data_dir, files[i])) for i in (0, 2))
        train_y, test_y = (load_idx_labels(os.path.join(args.data_dir, files[i])) for i in (1, 3))
    else:
        raise SystemExit("error: give the MNIST directory (four IDX files) or --synthetic")
    train_x, train_y, test_x, test_y = (t.to(dev) for t in (train_x, train_y, test_x, test_y))
    print(f"train: {tuple(train_x.shape)}  test: {tuple(test_x.shape)}")

    torch.manual_seed(args.seed)
    model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, 128), torch.nn.ReLU(),
                                torch.nn.Linear(128, 10)).to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=args.lr)
    B = args.batch
    step = None
    if args.mode == "graph":
        step = GraphTrainStep(model, F.cross_entropy, train_x[:B], train_y[:B])
        print(f"graph: {step.forward_ops} forward ops, {step.graph.num_ops()} with backward, "
              f"{'CUDA-graph replay' if step.executor.cuda_graph else 'interpreter'}")
        if args.dump_ir:
            print(emit_mlir(step.graph))

    n_batches = train_x.shape[0] // B
    for epoch in range(args.epochs):
        perm = torch.randperm(train_x.shape[0], device=dev, generator=None)
        t0, total, count = time.perf_counter(), 0.0, 0
        for b in range(n_batches):
            if 0 < args.max_steps <= b:
                break
            idx = perm[b * B:(b + 1) * B]
            x, y = train_x[idx], train_y[idx]
            if step is None:
                opt.zero_grad(set_to_none=True)
                loss = F.cross_entropy(model(x), y)
                loss.backward()
            else:
                loss = step(x, y)
            opt.step()
            total += float(loss.detach())
            count += 1
        acc = evaluate(model, test_x, test_y, 1024)
        print(f"epoch {epoch + 1}  mode={args.mode}  steps={count}  loss={total / max(1, count):.4f}  "
              f"test_acc={acc:.4f}  time={time.perf_counter() - t0:.2f}s")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
