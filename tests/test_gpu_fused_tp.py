"""Fused TP kernels. On one GPU the ranks of a group are emulated by launching each rank's kernel in turn over
buffers that all live on that GPU, in an order in which no launch waits for a later one (the gather kernel is
split into its push half and its multiply half for that; the barrier kernel is not used here). With >= 2 GPUs
the real peer-memory path runs in child processes."""
import ctypes
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr_array(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("world,rpr,N,K,b_mn", [(1, 256, 512, 256, False), (4, 128, 256, 192, False),
                                                 (2, 256, 384, 512, True), (8, 128, 4096, 512, False)])
def test_gemm_rs_emulated_ranks(world, rpr, N, K, b_mn):
    from tesseract_b200 import _native
    from tesseract_b200.parallel import fused_tp  # noqa: F401 (registers the signatures)
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    M = rpr * world
    g = torch.Generator(device=dev).manual_seed(world * 100 + N)
    xs = [torch.randn(M, K, device=dev, generator=g).bfloat16() for _ in range(world)]
    ws = [(torch.randn(N, K, device=dev, generator=g) * 0.1).bfloat16() for _ in range(world)]
    staging = [torch.full((world, rpr, N), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
    pa = _ptr_array(staging)
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(world):
        w_in = ws[r].t().contiguous() if b_mn else ws[r]
        _native.check(lib.tsb_gemm_rs(xs[r].data_ptr(), w_in.data_ptr(), pa, M, N, K, xs[r].stride(0), w_in.stride(0),
                                      int(b_mn), rpr, r, world, stream), "tsb_gemm_rs")
    torch.cuda.synchronize()
    assert _native.read_status(stream) == 0
    total = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    for r in range(world):
        assert torch.isfinite(staging[r].float()).all(), "a staging slot was not written"
        out = torch.empty(rpr, N, device=dev, dtype=torch.bfloat16)
        _native.check(lib.tsb_reduce_slots(staging[r].data_ptr(), out.data_ptr(), world, rpr * N, stream), "reduce")
        assert _rel(out, total[r * rpr:(r + 1) * rpr]) < 1e-2
        for src in range(world):  # each slot holds exactly that source rank's partial product
            part = xs[src][r * rpr:(r + 1) * rpr].float() @ ws[src].float().t()
            assert _rel(staging[r][src], part) < 1e-2


@pytest.mark.parametrize("world,rpr,N,K,b_mn,keep", [(1, 256, 512, 256, False, True), (4, 128, 256, 512, False, True),
                                                      (2, 512, 768, 1024, True, False),
                                                      (8, 128, 3584, 4096, False, True), (8, 256, 768, 4096, False, False)])
def test_ag_gemm_emulated_ranks(world, rpr, N, K, b_mn, keep):
    """Pass 1 runs only the push half of every rank's kernel (shards land in every rank's buffer, counters rise),
    pass 2 only the multiply half, so no launch ever waits for a later one."""
    from tesseract_b200 import _native
    from tesseract_b200.parallel import fused_tp  # noqa: F401
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    M = rpr * world
    g = torch.Generator(device=dev).manual_seed(world * 7 + K)
    stream = torch.cuda.current_stream().cuda_stream
    nsub = 2 if (rpr // 128) % 2 == 0 else 1
    lands = [torch.full((M, K), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
    flags = [torch.zeros(world * nsub, dtype=torch.int32, device=dev) for _ in range(world)]
    pl, pf = _ptr_array(lands), _ptr_array(flags)
    ws = [(torch.randn(N, K, device=dev, generator=g) * 0.1).bfloat16() for _ in range(world)]
    w_ins = [w.t().contiguous() if b_mn else w for w in ws]
    for call in (1, 2):   # the counters keep counting across calls; the data changes
        shards = [torch.randn(rpr, K, device=dev, generator=g).bfloat16() for _ in range(world)]
        full = torch.cat(shards)
        x_fulls = [torch.full((M, K), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
        ys = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(world)]
        for mask in (1, 2):
            for r in range(world):
                _native.check(lib.tsb_gemm_ag(shards[r].data_ptr(), pl, pf, x_fulls[r].data_ptr() if keep else None,
                                              w_ins[r].data_ptr(), ys[r].data_ptr(), call, nsub, mask, M, N,
                                              K, w_ins[r].stride(0), ys[r].stride(0), int(b_mn), rpr, r, world, None,
                                              stream), "tsb_gemm_ag")
            torch.cuda.synchronize()
            assert _native.read_status(stream) == 0
        for r in range(world):
            assert torch.equal(lands[r], full), "landing buffer differs from the concatenated shards"
            if keep:
                assert torch.equal(x_fulls[r], full), "kept activations differ from the concatenated shards"
            assert _rel(ys[r], full.float() @ ws[r].float().t()) < 1e-2
    for r in range(world):
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        assert int(flags[r].min()) == 2 * sms and int(flags[r].max()) == 2 * sms


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0", TESSERACT_TP_FUSED_MIN_AG="0", TESSERACT_TP_FUSED_MIN_RS="0")
    try:
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from tesseract_b200 import _native
        from tesseract_b200.models import LlamaConfig
        from tesseract_b200.parallel.fused_tp import FusedTP
        from tesseract_b200.parallel.tp_layers import TPContext, ag_matmul, matmul_rs
        fused = FusedTP(dist.group.WORLD, rank, world, dev)
        ctx_f = TPContext(dist.group.WORLD, rank, world, impl="fused", fused=fused)
        ctx_n = TPContext(dist.group.WORLD, rank, world, impl="nccl")
        g = torch.Generator(device=dev).manual_seed(11 + rank)
        errs = []
        for it in range(3):
            x = torch.randn(256 * world, 512, device=dev, generator=g).bfloat16()
            w = (torch.randn(1024, 512, device=dev, generator=g) * 0.05).bfloat16()
            a, b = matmul_rs(ctx_f, x, w), matmul_rs(ctx_n, x, w)
            errs.append(((a.float() - b.float()).norm() / b.float().norm()).item())
            xl = torch.randn(256, 512, device=dev, generator=g).bfloat16()
            (ya, xa), (yb, xb) = ag_matmul(ctx_f, xl, w), ag_matmul(ctx_n, xl, w)
            assert torch.equal(xa, xb)
            errs.append(((ya.float() - yb.float()).norm() / yb.float().norm()).item())
        torch.cuda.synchronize()
        status = _native.read_status(torch.cuda.current_stream().cuda_stream)
        # one optimizer step of a small TP+SP Llama: fused communication vs NCCL
        from tesseract_b200.parallel import build_parallel_trainer
        from tesseract_b200.training import TrainConfig
        cfg = LlamaConfig(vocab_size=1024, hidden_size=512, num_hidden_layers=2, num_attention_heads=8,
                          num_key_value_heads=4, intermediate_size=1024, max_position_embeddings=256,
                          dtype=torch.bfloat16)
        losses = {}
        for impl in ("fused", "nccl"):
            os.environ["TESSERACT_TP_COMM"] = impl
            trainer, plan = build_parallel_trainer(cfg, TrainConfig(lr=1e-3, micro_batch=2), world, rank, dev, "tp", seed=3)
            batch = torch.randint(0, 1024, (2, 257), generator=torch.Generator().manual_seed(5)).pin_memory()
            losses[impl] = (trainer.train_step(batch), trainer.train_step(batch), plan["fused_comm"])
        # expert parallelism: grouped-GEMM experts on each rank's share, rows exchanged with NCCL all-to-alls
        import copy
        from tesseract_b200.nn.moe import MoEFeedForward
        from tesseract_b200.parallel.expert import ExpertParallel
        torch.manual_seed(21)
        full = MoEFeedForward(256, 384, num_experts=2 * world, num_experts_per_tok=2, dtype=torch.bfloat16, device=dev)
        sharded = copy.deepcopy(full)
        fused_l = copy.deepcopy(full)
        ExpertParallel(dist.group.WORLD, rank, world).shard_(sharded)
        xe = torch.randn(200 + 8 * rank, 256, device=dev, generator=g).bfloat16()
        xa, xb = xe.clone().requires_grad_(True), xe.clone().requires_grad_(True)
        ya, yb = full(xa), sharded(xb)
        ge = torch.randn_like(ya)
        ya.backward(ge)
        yb.backward(ge)
        ep_errs = [((ya.float() - yb.float()).norm() / ya.float().norm()).item(),
                   ((xa.grad.float() - xb.grad.float()).norm() / xa.grad.float().norm()).item()]
        errs += ep_errs
        # the same layer with the device-side exchange over peer memory (no NCCL, no host read of the counts)
        from tesseract_b200.parallel.expert import FusedExpertParallel
        fep = FusedExpertParallel(dist.group.WORLD, rank, world, dev, 256, 2 * world, 2, max_tokens=512)
        fep.shard_(fused_l)
        for it in range(3):                                          # several calls: buffers and tags are reused
            # result rows returned by the down projection's own epilogue (peer stores), then by the separate kernel
            fep.scatter_epilogue = it != 1
            xc = xe.clone().requires_grad_(True)
            yc = fused_l(xc)
            yc.backward(ge)
            errs += [((ya.float() - yc.float()).norm() / ya.float().norm()).item(),
                     ((xa.grad.float() - xc.grad.float()).norm() / xa.grad.float().norm()).item()]
        for ge_i in range(2 * world):                                # expert weight gradients: same order everywhere
            for name in ("gate_proj", "up_proj", "down_proj"):
                wfull = getattr(full.experts[ge_i], name).weight
                want = torch.zeros_like(wfull, dtype=torch.float32) if wfull.grad is None else wfull.grad.float().clone()
                dist.all_reduce(want)
                el_ = 2
                if ge_i // el_ == rank:
                    got = getattr(fused_l.experts[ge_i - rank * el_], name).weight.grad.float()
                    # three backward passes accumulated into .grad
                    errs.append(((got / 3 - want).norm() / want.norm().clamp_min(1e-6)).item())
        assert fep.calls == 3
        status |= _native.read_status(torch.cuda.current_stream().cuda_stream)
        # tensor-parallel serving: sharded engine (one-shot all-reduce kernel inside the decode CUDA graph) against
        # the single-GPU engine on the same seeded model and requests
        from tesseract_b200.models import GenerateConfig, LlamaModel
        from tesseract_b200.models.scheduler import EngineConfig
        from tesseract_b200.serving import ServingEngine, TPServe
        from tesseract_b200.parallel.fused_tp import SymmAllReduce
        ar = SymmAllReduce(dist.group.WORLD, rank, world, dev, 64 * 512)
        for it in range(4):                                            # both buffers, several epochs
            part = torch.randn(64, 512, device=dev, generator=g).bfloat16()
            ar.input_view(64, 512).copy_(part)
            got = ar.reduce(64, 512)
            want = part.float().clone()
            dist.all_reduce(want)
            errs.append(((got.float() - want).norm() / want.norm()).item())
        scfg = LlamaConfig(vocab_size=2048, hidden_size=64 * 4 * world, num_hidden_layers=2, num_attention_heads=4 * world,
                           num_key_value_heads=world, intermediate_size=1024, max_position_embeddings=256,
                           dtype=torch.bfloat16)            # head_dim 64 at every world size
        ecfg = EngineConfig(block_size=16, num_blocks=256, max_seq_len=256, max_batch_size=8)
        prompts = [[(7 * i + j) % 2048 for j in range(20 + 9 * i)] for i in range(5)]
        outs = {}
        for mode in ("single", "tp"):
            m = LlamaModel(scfg, device=dev, init_std=0.05, seed=9)
            tp = TPServe(dist.group.WORLD, rank, world, dev, scfg.hidden_size) if mode == "tp" else None
            eng = ServingEngine(m, ecfg, tp=tp)
            ids = [eng.add_request(p, GenerateConfig(max_new_tokens=12)) for p in prompts]
            eng.run()
            outs[mode] = [eng.result(i)[len(p):] for i, p in zip(ids, prompts)]
            if tp is not None:     # greedy tensor-parallel serving: the LM head is split by vocabulary rows
                assert eng.vocab_shard == 2048 // world and eng.w_head.shape[0] == 2048 // world
                assert tp.head_ar.calls > 0
        flat = torch.tensor([t for o in outs["tp"] for t in o], device=dev)
        lo, hi = flat.clone(), flat.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert torch.equal(lo, hi), "tensor-parallel ranks picked different tokens"
        same = sum(a == b for x, y in zip(outs["single"], outs["tp"]) for a, b in zip(x, y))
        agree = same / sum(len(x) for x in outs["single"])
        assert all(x[0] == y[0] for x, y in zip(outs["single"], outs["tp"])), "first tokens differ from the single-GPU engine"
        assert agree > 0.6, agree
        status |= _native.read_status(torch.cuda.current_stream().cuda_stream)
        # data-parallel gradient all-reduce: the two-shot peer-memory kernel against NCCL on the same buffers, then two
        # optimizer steps of a small replicated model with either collective
        from tesseract_b200.parallel.fused_tp import SymmGradAllReduce, SymmetricMemory
        n = 3 * 1024 * 1024 + 128
        sm = SymmetricMemory(dist.group.WORLD, rank, world, n * 2, dev)
        gar = SymmGradAllReduce(sm)
        view = sm.local[:n * 2].view(torch.bfloat16)
        for it in range(3):
            data = torch.randn(n, device=dev, generator=g).bfloat16()
            view.copy_(data)
            lo_e, hi_e = 1024 * it, n - 128 * it                     # different ranges of the same buffer
            want = data[lo_e:hi_e].float().clone()
            dist.all_reduce(want)
            torch.cuda.synchronize()
            dist.barrier()
            gar.all_reduce_(lo_e * 2, hi_e - lo_e, torch.bfloat16, scale=1.0 / world)
            got = view[lo_e:hi_e].float() * world
            errs.append(((got - want).norm() / want.norm()).item())
            same_bits = view[lo_e:hi_e].view(torch.int16).to(torch.int64).sum()
            a1, a2 = same_bits.clone(), same_bits.clone()
            dist.all_reduce(a1, op=dist.ReduceOp.MIN)
            dist.all_reduce(a2, op=dist.ReduceOp.MAX)
            assert int(a1) == int(a2), "ranks hold different reduced gradients"
            if lo_e > 0:
                assert torch.equal(view[:lo_e], data[:lo_e])        # outside the range: untouched
        dp_losses = {}
        for comm in ("symm", "nccl"):
            os.environ["TESSERACT_DP_COMM"] = comm
            trainer, plan = build_parallel_trainer(cfg, TrainConfig(lr=1e-3, micro_batch=1), world, rank, dev, "dp", seed=3)
            assert plan["dp_comm"] == ("symm-twoshot" if comm == "symm" else "nccl")
            batch = torch.randint(0, 1024, (2, 257), generator=torch.Generator().manual_seed(50 + rank)).pin_memory()
            dp_losses[comm] = (trainer.train_step(batch), trainer.train_step(batch))
            if comm == "symm":
                assert trainer.grad_reducer.symm.calls > 0 and trainer.grad_reducer.overlapped_bytes > 0
        losses["dp"] = dp_losses
        status |= _native.read_status(torch.cuda.current_stream().cuda_stream)
        dist.barrier()
        q.put((rank, None, (errs, status, losses)))
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc(), None))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_tp_matches_nccl_on_real_peers():
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    try:
        for p in procs:
            p.start()
        results = [q.get(timeout=300) for _ in range(world)]
        for p in procs:
            p.join(timeout=60)
    finally:
        # a rank that raised leaves its peers inside a collective: never leave children holding GPUs behind
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=30)
    bad = [r for r in results if r[1] is not None]
    assert not bad, bad[0][1]
    for _, _, (errs, status, losses) in results:
        assert status == 0
        assert max(errs) < 3e-2, errs
        assert losses["fused"][2] is True and losses["nccl"][2] is False
        assert abs(losses["fused"][0] - losses["nccl"][0]) < 2e-2
        assert losses["fused"][1] < losses["fused"][0]
        dp = losses["dp"]
        assert abs(dp["symm"][0] - dp["nccl"][0]) < 1e-3 and abs(dp["symm"][1] - dp["nccl"][1]) < 2e-2
        assert dp["symm"][1] < dp["symm"][0]


def test_barrier_wait_runs_out_and_reports_through_the_status_word():
    """A rank whose peer never signals: the barrier kernel gives up after its (here: short) limit, records the
    flag-timeout code, returns, and the context stays usable -- nothing traps or hangs. The "peer" is a second
    flag pad on the same GPU that nothing ever writes."""
    import ctypes

    from tesseract_b200 import _native
    from tesseract_b200.parallel import fused_tp  # noqa: F401  (registers the signatures)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _native.read_status(stream)                                 # clear
    pads = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]
    arr = (ctypes.c_void_p * 2)(*[p.data_ptr() for p in pads])
    limit = 100_000_000                                         # about 50 ms of SM clock
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _native.check(_native.lib().tsb_symm_barrier_limit(arr, 0, 2, 1, limit, stream), "tsb_symm_barrier_limit")
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 2000.0
    assert int(pads[0][0]) == 1 and int(pads[1][0]) == 1        # this rank did announce itself to both pads
    assert _native.read_status(stream) == 2                     # kStatusFlagTimeout
    assert _native.read_status(stream) == 0                     # reading clears it
    # the next launches work: the same barrier with the peer's slot already signalled passes at once
    pads[0][1] = 2
    _native.check(_native.lib().tsb_symm_barrier_limit(arr, 0, 2, 2, limit, stream), "tsb_symm_barrier_limit")
    x = torch.randn(256, 256, device=dev, dtype=torch.bfloat16)
    from tesseract_b200.ops.gemm import gemm_bf16
    y = gemm_bf16(x, x)
    torch.cuda.synchronize()
    assert _native.read_status(stream) == 0
    assert torch.isfinite(y.float()).all()


def test_twoshot_allreduce_emulated_ranks_on_one_gpu():
    """The gradient all-reduce kernel with every rank's buffer on ONE GPU: the ranks run one after the other, phase by
    phase (start barrier with the peers' flags already written, reduce + broadcast, end barrier), which gives what
    concurrent ranks give because a vector is read and rewritten by its owning rank only."""
    import ctypes

    from tesseract_b200 import _native
    from tesseract_b200.parallel import fused_tp  # noqa: F401
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _native.read_status(stream)
    for world, n, dtype in ((4, 8 * 1000 + 8 * 3, torch.bfloat16), (8, 4 * 515, torch.float32), (2, 8 * 4096, torch.bfloat16)):
        g = torch.Generator(device=dev).manual_seed(world)
        bufs = [torch.randn(n, device=dev, generator=g).to(dtype) for _ in range(world)]
        want = torch.stack([b.float() for b in bufs]).sum(0) / world
        flags = [torch.zeros(32, dtype=torch.int32, device=dev) for _ in range(world)]
        states = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(world)]
        parr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
        farr = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
        code = 1 if dtype == torch.bfloat16 else 0
        for phase in (1, 2, 4):
            for r in range(world):
                flags[r][:world] = 1                 # the peers' "ready" flags, as concurrent ranks would have set them
                if phase == 4:                       # ... and their "done" flags
                    flags[r][16:16 + world] = 1
                _native.check(_native.lib().tsb_allreduce_twoshot(parr, farr, states[r].data_ptr(), n, code, r, world, 1,
                                                                  1.0 / world, 7, phase, 200_000_000, stream),
                              "tsb_allreduce_twoshot")
        torch.cuda.synchronize()
        assert _native.read_status(stream) == 0
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-6
        for b in bufs:
            assert torch.equal(b, bufs[0])           # every rank ends with the same bits
            assert (b.float() - want).abs().max() <= tol * want.abs().max()
        assert all(int(f[:world].min()) == 1 for f in flags)
    # a start barrier whose peer never arrives runs out and reports
    flags = [torch.zeros(32, dtype=torch.int32, device=dev) for _ in range(2)]
    state = torch.zeros(2, dtype=torch.int32, device=dev)
    bufs = [torch.ones(64, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    parr = (ctypes.c_void_p * 2)(*[b.data_ptr() for b in bufs])
    farr = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
    _native.check(_native.lib().tsb_allreduce_twoshot(parr, farr, state.data_ptr(), 64, 1, 0, 2, 1, 1.0, 4, 7, 50_000_000,
                                                      stream), "tsb_allreduce_twoshot")
    torch.cuda.synchronize()
    assert _native.read_status(stream) == 2
    assert torch.equal(bufs[0], torch.ones_like(bufs[0]))       # nothing was reduced
