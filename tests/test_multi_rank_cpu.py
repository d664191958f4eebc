"""World-size-2 run of the multi-GPU host logic on CPU ranks (gloo)."""
import os
import subprocess
import sys

from tests.util import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, json
sys.path.insert(0, %r)
import torch.distributed as dist
from mongoose_b200 import multi, synthetic
rank, world, local = multi.rank_env()
dist.init_process_group("gloo")
ms = [100.0, 7.0] if rank == 0 else [80.0, 9.0]
mx = multi.reduce_max(ms, dist)
dist.barrier()
seqs = multi.sequences_for_rank(7, rank, world)
prompt = synthetic.prompt_ids(rank, 4, 1000).tolist()
mine = {"rank": rank, "max": mx, "seqs": seqs, "prompt": prompt,
        "rate": multi.aggregate_rate(world, 200, mx[0])}
everyone = [None] * world
dist.all_gather_object(everyone, mine)          # one writer: lines of two ranks on one pipe can interleave
if rank == 0:
    print("RESULTS " + json.dumps(everyone), flush=True)
dist.destroy_process_group()
""" % ROOT


def test_two_ranks_agree_on_max_time_and_split_sequences(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", str(free_port()), str(script)],
                         capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    found = [l for l in out.stdout.splitlines() if l.startswith("RESULTS ")]
    assert len(found) == 1, out.stdout[-1000:]
    lines = json.loads(found[0][len("RESULTS "):])
    assert len(lines) == 2
    by = {l["rank"]: l for l in lines}
    for r in (0, 1):
        assert by[r]["max"] == [100.0, 9.0]
        assert abs(by[r]["rate"] - 2 * 200 / 0.1) < 1e-9          # whole-job rate uses the slowest rank
    assert by[0]["seqs"] == [0, 2, 4, 6] and by[1]["seqs"] == [1, 3, 5]
    assert by[0]["prompt"] != by[1]["prompt"]                        # each rank decodes its own sequence


def test_single_process_defaults():
    from mongoose_b200 import multi
    assert multi.reduce_max([3.0, 4.0]) == [3.0, 4.0]
    assert multi.sequences_for_rank(5, 0, 1) == [0, 1, 2, 3, 4]
    assert multi.aggregate_rate(8, 200, 50.0) == 8 * 200 / 0.05
