"""The one-node launcher on CPU ranks (gloo): results in rank order, a failing rank's traceback in the parent, the
skip code, a rank that exits without a word, and the command-line form. Failures are made on the host only."""
import os
import subprocess
import sys

import pytest
import torch

from tesseract_b200.parallel.launch import LaunchError, LaunchSkipped, Skip, launch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _sum_ranks(rank, world, offset):
    import torch.distributed as dist
    t = torch.tensor([float(rank + offset)])
    dist.all_reduce(t)
    assert os.environ["MASTER_ADDR"] == "127.0.0.1" and int(os.environ["RANK"]) == rank
    return (rank, float(t))


def _rank1_raises(rank, world):
    if rank == 1:
        raise ValueError("boom on the host")
    return rank


def _rank0_skips(rank, world):
    if rank == 0:
        raise Skip("needs more GPUs than this node has")
    return rank


def _rank1_vanishes(rank, world):
    if rank == 1:
        os._exit(3)                 # leaves between steps, nothing in flight
    return rank


def test_launch_returns_results_in_rank_order():
    assert launch(_sum_ranks, 3, 10, backend="gloo") == [(0, 33.0), (1, 33.0), (2, 33.0)]


def test_launch_reports_the_failing_rank_skip_and_silent_death():
    with pytest.raises(LaunchError) as e:
        launch(_rank1_raises, 2, backend="gloo")
    assert e.value.rank == 1 and "boom on the host" in e.value.detail and "ValueError" in e.value.detail
    with pytest.raises(LaunchSkipped, match="needs more GPUs"):
        launch(_rank0_skips, 2, backend="gloo")
    with pytest.raises(LaunchError) as e:
        launch(_rank1_vanishes, 2, backend="gloo")
    assert e.value.rank == 1 and "code 3" in e.value.detail
    with pytest.raises(ValueError):
        launch(_sum_ranks, 2, 0, backend="mpi")


def test_command_line_form_runs_a_torchrun_style_script(tmp_path):
    script = tmp_path / "job.py"
    script.write_text(
        "import os, sys, torch, torch.distributed as dist\n"
        "dist.init_process_group('gloo')\n"
        "t = torch.ones(1) * (dist.get_rank() + 1)\n"
        "dist.all_reduce(t)\n"
        "open(sys.argv[1] + os.environ['RANK'], 'w').write(str(float(t)))\n"
        "dist.destroy_process_group()\n"
        "sys.exit(0)\n")
    r = subprocess.run([sys.executable, "-m", "tesseract_b200.parallel.launch", "--nproc", "2", "--backend", "gloo", str(script),
                        str(tmp_path / "out")], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert (tmp_path / "out0").read_text() == "3.0" and (tmp_path / "out1").read_text() == "3.0"
    bad = tmp_path / "bad.py"
    bad.write_text("import sys\nsys.exit(77)\n")
    r = subprocess.run([sys.executable, "-m", "tesseract_b200.parallel.launch", "--nproc", "2", "--backend", "gloo", str(bad)],
                       cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 77


def _peer_learns_of_a_failure(rank, world, out_path):
    """Rank 1 fails on the host between steps; rank 0 learns of it from the job's store (the launcher posts the
    failing rank's exception there) at its next watchdog step, before it would enter a collective."""
    import time

    import torch.distributed as dist

    from tesseract_b200.parallel.launch import job_watchdog
    from tesseract_b200.utils.watchdog import RankLost
    wd = job_watchdog(timeout_s=30.0)
    assert wd is not None and wd.world == world
    dist.barrier()
    if rank == 1:
        raise RuntimeError("rank 1 gives up between steps")
    try:
        for _ in range(3000):
            wd.step()
            time.sleep(0.005)
    except RankLost as e:
        with open(out_path, "w") as f:
            f.write(f"{e.rank}|{e.reason}")
        return "lost"
    return "never noticed"


def test_watchdog_over_the_job_store_tells_peers_of_a_failed_rank(tmp_path):
    out = tmp_path / "seen.txt"
    with pytest.raises(LaunchError) as e:
        launch(_peer_learns_of_a_failure, 2, str(out), backend="gloo")
    assert e.value.rank == 1 and "gives up between steps" in e.value.detail
    assert out.exists(), "rank 0 did not learn of the failure before the launcher took it down"
    rank, reason = out.read_text().split("|", 1)
    assert rank == "1" and "RuntimeError" in reason and "gives up between steps" in reason
