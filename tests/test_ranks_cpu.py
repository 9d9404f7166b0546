"""The multi-process plumbing of the benchmark (one process per GPU, replicas only) run as
two `gloo` ranks on the CPU: sharding of independent units, the barrier, the max-over-ranks
time, and the rule that only rank 0 reports."""
import json
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_shard_units_partitions_exactly(pkg):
    for n_units in (0, 1, 7, 8, 9, 148, 1000):
        for world in (1, 2, 3, 4, 8):
            seen = []
            sizes = []
            for r in range(world):
                sh = pkg.ranks.shard_units(n_units, r, world)
                seen.extend(sh)
                sizes.append(len(sh))
            assert seen == list(range(n_units))
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        pkg.ranks.shard_units(4, 2, 2)


def test_rank_info_from_env(pkg):
    info = pkg.ranks.RankInfo.from_env({"RANK": "3", "WORLD_SIZE": "8", "LOCAL_RANK": "3"})
    assert (info.rank, info.world, info.local_rank) == (3, 8, 3)
    assert pkg.ranks.RankInfo.from_env({}).world == 1


WORKER = textwrap.dedent("""
    import json, os, sys, time
    sys.path.insert(0, {root!r})
    import __graft_entry__ as graft
    pkg = graft.import_package()
    info = pkg.ranks.RankInfo.from_env()
    ranks = pkg.ranks.Ranks(info, backend="gloo")
    units = pkg.ranks.shard_units(11, info.rank, info.world)
    ranks.barrier()
    t = 0.010 * (info.rank + 1)          # rank 1 is the slow one
    time.sleep(t)
    ranks.barrier()
    slowest = ranks.max_over_ranks(t)
    total = ranks.sum_over_ranks(len(units))
    if ranks.is_root:
        print(json.dumps({{"slowest": slowest, "units": total, "world": info.world,
                          "rate": pkg.ranks.whole_job_rate(total, slowest)}}))
    ranks.close()
""")


@pytest.mark.timeout(180)
def test_two_gloo_ranks_line_up_and_root_reports(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
         "--master-port", "29731", str(script)],
        capture_output=True, text=True, env=env, timeout=170)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout            # rank 0 alone reports
    out = json.loads(lines[0])
    assert out["world"] == 2 and out["units"] == 11
    assert abs(out["slowest"] - 0.020) < 1e-9    # the max over ranks, not rank 0's own time
    assert abs(out["rate"] - 11 / 0.020) < 1e-6


@pytest.mark.timeout(300)
def test_reference_arm_other_ranks_exit_quietly():
    """`bench.py --impl reference` under two ranks: rank 0 prints the line, rank 1 exits 0
    without work (no GPU needed: the arm times the CPU oracle)."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
         "--master-port", "29733", str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1"],
        capture_output=True, text=True, env=env, timeout=290, cwd=str(ROOT))
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and out["metric"] == "decode_tokens_per_s" and out["value"] > 0
    assert out["cpu_baseline"]["kind"] == "port" and out["e2e"]["h2d_bytes_per_step"] == 0
