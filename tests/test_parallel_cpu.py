"""Parallel layers without a cluster: the in-process simulation backend (TP=1 vs TP=2/3 parity, forward and
backward) and real multi-process runs over gloo CPU ranks (TP+SP Llama vs dense, DP gradient reducer,
rank-local collectives)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tesseract_b200.nn import Linear
from tesseract_b200.parallel import ColumnParallelLinear, RowParallelLinear, SimCommBackend


def test_column_parallel_matches_dense_exactly():
    torch.manual_seed(0)
    dense = Linear(12, 18, bias=True)
    x = torch.randn(5, 12, requires_grad=True)
    for world in (2, 3):
        col = ColumnParallelLinear.from_dense(dense, SimCommBackend(world))
        assert [n for n, _ in col.named_parameters()][:2] == ["shard.0.weight", "shard.0.bias"]
        y = col(x)
        assert torch.equal(y, dense(x))
        g = torch.randn_like(y)
        y.backward(g)
        xg = x.grad.clone()
        x.grad = None
        dense.zero_grad()
        dense(x).backward(g)
        wg = torch.cat([p.grad for p in col.weight_shards])
        assert torch.allclose(wg, dense.weight.grad, atol=0) and torch.allclose(xg, x.grad, atol=1e-6)
        x.grad = None


def test_row_parallel_and_megatron_mlp():
    torch.manual_seed(1)
    up, down = Linear(8, 24, bias=False), Linear(24, 8, bias=True)
    x = torch.randn(4, 8, requires_grad=True)
    ref = down(torch.relu(up(x)))
    for world in (2, 3):
        comm = SimCommBackend(world)
        col = ColumnParallelLinear.from_dense(up, comm)
        row = RowParallelLinear.from_dense(down, comm)
        shards = [torch.relu(s) for s in col.forward_shards(x)]
        y = row.forward_shards(shards)
        assert (y - ref).abs().max() < 1e-5
        y.sum().backward()
        wg = torch.cat([p.grad for p in row.weight_shards], dim=1)
        down.zero_grad(); up.zero_grad()
        xg = x.grad.clone(); x.grad = None
        down(torch.relu(up(x))).sum().backward()
        assert (wg - down.weight.grad).abs().max() < 1e-5 and (row.bias.grad - down.bias.grad).abs().max() < 1e-5
        assert (xg - x.grad).abs().max() < 1e-5
        x.grad = None
    with pytest.raises(ValueError):
        RowParallelLinear(10, 4, SimCommBackend(3))
    with pytest.raises(ValueError):
        row.forward_shards([x])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run_ranks(fn, world, *args):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q) + args) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    bad = [r for r in results if r[1] is not None]
    assert not bad, bad[0][1]
    return {r[0]: r[2] for r in results}


def _entry(fn, rank, world, port, q, *args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(2)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        out = fn(rank, world, *args)
        dist.barrier()
        q.put((rank, None, out))
    except Exception:  # pragma: no cover - reported to the parent
        import traceback
        q.put((rank, traceback.format_exc(), None))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _tp_llama_worker(rank, world):
    from tesseract_b200.models import LlamaConfig, LlamaModel
    from tesseract_b200.parallel.tp_layers import TPContext
    from tesseract_b200.parallel.tp_model import TPLlamaModel
    from tesseract_b200.optim import ParamArena
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, intermediate_size=688, max_position_embeddings=128, rope_theta=10000.0)
    dense = LlamaModel(cfg, init_std=0.02, seed=7)
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, 512, (4, 128), generator=g)
    tgt = torch.randint(0, 512, (4, 128), generator=g)
    ref_loss = dense.loss(tok, tgt)
    ref_loss.backward()
    tp = TPContext(dist.group.WORLD, rank, world, impl="nccl")
    model = TPLlamaModel(cfg, tp)
    model.load_dense_state_dict(dense.hf_state_dict())
    ParamArena.from_module(model)
    loss = model.loss(tok, tgt)
    loss.backward()
    model.sync_replicated_grads()
    assert abs(loss.item() - ref_loss.item()) < 1e-5, (loss.item(), ref_loss.item())
    worst = 0.0
    dgrads = dict(dense.named_parameters())
    for name, p in model.named_parameters():
        want = model._shard_of(name, dgrads[name].grad)
        worst = max(worst, (p.main_grad - want).abs().max().item())
    assert worst < 1e-5, worst
    full = model.gather_dense_state_dict()
    for k, v in dense.hf_state_dict().items():
        assert torch.equal(full[k], v), k
    return worst


def test_tp_sp_llama_matches_dense_over_gloo_ranks():
    _run_ranks(_tp_llama_worker, 2)


def _dp_worker(rank, world):
    from tesseract_b200.models import LlamaConfig
    from tesseract_b200.parallel import build_parallel_trainer
    from tesseract_b200.training import TrainConfig
    cfg = LlamaConfig(vocab_size=64, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                      intermediate_size=128, max_position_embeddings=32)
    out = {}
    for mode in ("dp", "tp"):
        trainer, plan = build_parallel_trainer(cfg, TrainConfig(lr=1e-3, micro_batch=1), world, rank, "cpu", mode, seed=5)
        g = torch.Generator().manual_seed(100 + plan["dp_rank"])
        batch = torch.randint(0, 64, (2, 17), generator=g)
        l0 = trainer.train_step(batch)
        l1 = trainer.train_step(batch)
        assert l1 < l0
        flat = trainer.arena.flat.clone()
        if mode == "dp":
            gathered = [torch.empty_like(flat) for _ in range(world)]
            dist.all_gather(gathered, flat)
            assert all(torch.equal(gathered[0], t) for t in gathered), "replicas diverged"
            assert trainer.grad_reducer.overlapped_bytes > 0
        out[mode] = (l0, l1, plan["name"])
    return out


def test_dp_reducer_and_tp_trainer_over_gloo_ranks():
    res = _run_ranks(_dp_worker, 2)
    assert res[0]["dp"][2] == "dp2" and res[0]["tp"][2] == "tp2+sp"
    assert abs(res[0]["tp"][0] - res[1]["tp"][0]) < 1e-6


def _collectives_worker(rank, world):
    from tesseract_b200.parallel import NcclCommBackend
    c = NcclCommBackend()
    x = torch.full((2, 3), float(rank + 1))
    assert torch.equal(c.all_reduce_sum(x), torch.full((2, 3), float(sum(range(1, world + 1)))))
    g = c.all_gather(x, dim=-1)
    assert g.shape == (2, 3 * world) and float(g[0, -1]) == world
    rs = c.reduce_scatter(torch.arange(world * 2, dtype=torch.float32).view(world * 2, 1))
    assert torch.equal(rs, world * torch.arange(rank * 2, rank * 2 + 2, dtype=torch.float32).view(2, 1))
    a2a = c.all_to_all(torch.arange(world, dtype=torch.float32).view(world, 1) + 10 * rank)
    assert torch.equal(a2a.view(-1), torch.tensor([10.0 * r + rank for r in range(world)]))
    return True


def test_rank_local_collectives_over_gloo():
    _run_ranks(_collectives_worker, 3)


def _ep_worker(rank, world):
    import copy
    from tesseract_b200.nn.moe import MoEFeedForward
    from tesseract_b200.parallel.expert import ExpertParallel
    torch.manual_seed(7)
    full = MoEFeedForward(16, 24, num_experts=4, num_experts_per_tok=2)          # same weights on every rank
    sharded = copy.deepcopy(full)
    ep = ExpertParallel(dist.group.WORLD, rank, world)
    ep.shard_(sharded)
    assert len(sharded.experts) == 4 // world
    x = torch.randn(9 + rank, 16, generator=torch.Generator().manual_seed(100 + rank))   # different tokens per rank
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya, yb = full(xa), sharded(xb)
    assert torch.allclose(ya, yb, atol=1e-5), (ya - yb).abs().max()
    g = torch.randn_like(ya)
    ya.backward(g)
    yb.backward(g)
    assert torch.allclose(xa.grad, xb.grad, atol=1e-5)
    assert torch.allclose(full.gate.weight.grad, sharded.gate.weight.grad, atol=1e-5)
    el = 4 // world
    for ge in range(4):                                                          # same collective order on every rank
        for name in ("gate_proj", "up_proj", "down_proj"):
            w = getattr(full.experts[ge], name).weight
            want = torch.zeros_like(w) if w.grad is None else w.grad.clone()
            dist.all_reduce(want)                                                # tokens of every rank reach this expert
            if ge // el == rank:
                got = getattr(sharded.experts[ge - rank * el], name).weight.grad
                assert torch.allclose(got, want, atol=1e-5), name
    assert ep.stats["rows_sent"] == (9 + rank) * 2
    return True


def test_expert_parallel_matches_single_process_over_gloo_ranks():
    assert all(_run_ranks(_ep_worker, 2).values())


def _zero_worker(rank, world):
    from tesseract_b200.models import LlamaConfig
    from tesseract_b200.parallel import ShardedAdam, build_parallel_trainer
    from tesseract_b200.training import TrainConfig
    cfg = LlamaConfig(vocab_size=64, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                      intermediate_size=128, max_position_embeddings=32)
    flats, losses = {}, {}
    for stage in (0, 1):
        tc = TrainConfig(lr=1e-3, micro_batch=1, max_grad_norm=1.0, weight_decay=0.01, zero_stage=stage)
        trainer, plan = build_parallel_trainer(cfg, tc, world, rank, "cpu", "dp", seed=5)
        g = torch.Generator().manual_seed(100 + plan["dp_rank"])
        batch = torch.randint(0, 64, (2, 17), generator=g)
        losses[stage] = [trainer.train_step(batch) for _ in range(3)]
        flats[stage] = trainer.arena.flat.clone()
        if stage == 1:
            assert isinstance(trainer.opt, ShardedAdam)
            full = 2 * 4 * trainer.arena.numel
            assert trainer.opt.state_bytes() <= full // world + 2 * 4 * 64
            sd = trainer.opt.state_dict()
            assert sd["flat_m"].numel() == trainer.opt.end - trainer.opt.begin
            trainer.opt.load_state_dict(sd)
            gathered = [torch.empty_like(flats[1]) for _ in range(world)]
            dist.all_gather(gathered, flats[1])
            assert all(torch.equal(gathered[0], t) for t in gathered), "replicas diverged"
    assert torch.equal(flats[0], flats[1]), float((flats[0] - flats[1]).abs().max())
    assert losses[0] == losses[1]
    return True


def test_zero1_sharded_adam_matches_replicated_adam_over_gloo_ranks():
    from tesseract_b200.parallel import shard_ranges
    for numel, world in ((1000, 3), (64, 4), (130, 2), (5, 8)):
        r = shard_ranges(numel, world)
        assert r[0][0] == 0 and r[-1][1] == numel and all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(a % 64 == 0 for a, _ in r if a < numel)
    _run_ranks(_zero_worker, 3)


def _replica_worker(rank, world):
    from tesseract_b200.serving import make_replica_plan, split_requests
    plan = make_replica_plan(world, rank, 2)
    assert (plan.replicas, plan.replica, plan.tp_rank) == (world // 2, rank // 2, rank % 2)
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=plan.group)                        # the group holds exactly this replica's two ranks
    assert t.item() == 4 * plan.replica + 1
    mine = split_requests(list(range(10)), plan)
    assert mine == [i for i in range(10) if i % plan.replicas == plan.replica]
    return plan.is_leader


def test_serving_replica_plan_over_gloo_ranks():
    from tesseract_b200.serving import default_tp, make_replica_plan, split_requests
    solo = make_replica_plan(1, 0, 1)
    assert solo.replicas == 1 and solo.group is None and split_requests([3, 4], solo) == [3, 4]
    assert [default_tp(w) for w in (1, 2, 4, 8)] == [1, 1, 1, 1]
    with pytest.raises(ValueError):
        make_replica_plan(8, 0, 3)
    leaders = _run_ranks(_replica_worker, 4)
    assert leaders == {0: True, 1: False, 2: True, 3: False}


def _ep_model_worker(rank, world):
    from tesseract_b200.models import LlamaConfig, LlamaModel
    from tesseract_b200.parallel.ep_model import EPMoELlama
    cfg = LlamaConfig(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, intermediate_size=48, max_position_embeddings=32, rope_theta=10000.0,
                      num_experts=4, num_experts_per_tok=2)
    full = LlamaModel(cfg, init_std=0.05, seed=11)                         # every expert, same on every rank
    g = torch.Generator().manual_seed(5)
    tok = torch.randint(0, 128, (world, 2, 16), generator=g)               # [rank, micro-batch, seq]
    tgt = torch.randint(0, 128, (world, 2, 16), generator=g)
    ref = sum(full.loss(tok[r, m:m + 1], tgt[r, m:m + 1]) for r in range(world) for m in range(2)) / (2 * world)
    ref.backward()
    ep = EPMoELlama(cfg, dist.group.WORLD, rank, world, None, max_tokens=16, exchange="nccl")
    ep.load_full_state_dict(full.state_dict())
    ep.zero_grad()
    mine = sum(ep.forward_backward(tok[rank, m:m + 1], tgt[rank, m:m + 1], scale=1.0 / (2 * world)) for m in range(2))
    ep.reduce_replicated_grads()
    total = mine.clone()
    dist.all_reduce(total)
    assert abs(total.item() / (2 * world) - ref.item()) < 1e-5
    want = dict(full.named_parameters())
    el = cfg.num_experts // world
    worst = 0.0
    for name, p in ep.model.named_parameters():
        parts = name.split(".")
        if "experts" in parts:
            at = parts.index("experts")
            parts[at + 1] = str(int(parts[at + 1]) + rank * el)
            got = p.grad
        else:
            got = p.main_grad
        w = want[".".join(parts)].grad
        w = torch.zeros_like(got) if w is None else w
        got = torch.zeros_like(w) if got is None else got
        d = (got - w).abs().max().item()
        if d > 2e-5: print('BAD', rank, name, d, w.abs().max().item(), flush=True)
        worst = max(worst, d)
    assert worst < 2e-5, worst
    # one decode step through caches equals the full model's
    caches, fcaches = ep.make_kv_caches(1, 32), full.make_kv_caches(1, 32)
    a = ep.decode_step(tok[rank, :1, :5], caches)
    b = full.forward_step(tok[rank, :1, :5], fcaches)
    assert (a - b).abs().max() < 1e-4
    return worst


def test_expert_parallel_moe_llama_matches_full_model_over_gloo_ranks():
    _run_ranks(_ep_model_worker, 2)
