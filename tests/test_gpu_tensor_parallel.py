"""Tensor-parallel decode on 2 (and 4) GPUs of one node against the CPU oracle.

Each rank is a child process with its own GPU (tests/tp_worker.py, launched by torchrun); the ranks
exchange partial sums through NCCL inside the C library.  Skipped where fewer GPUs are visible.
No rank leaves mid-step and nothing here is expected to fail on the device.
"""
import json
import os
import subprocess
import sys

import pytest

from tests.util import free_port

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = 1e-4   # relative to max|y|, the same bound as the single-GPU engine tests


# Which cases run on how many ranks (a CPU test checks that each has a partition for that many ranks:
# four Q heads cannot be dealt to eight ranks).
RANK_CASES = {
    2: ["tiny", "tiny-bias-ragged", "tiny-q4", "hd128-gqa", "tiny-kv1", "kv1-uneven", "qwen7b-width-2L"],
    4: ["tiny", "tiny-bias-ragged", "hd128-gqa", "gqa-28-4"],
    8: ["gqa-28-4"],
}


def run_ranks(world, cases, nccl_exchange=False, kernels_path=False, timeout=300):
    assert all(c in RANK_CASES[world] for c in cases), (world, cases)
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, {torch.cuda.device_count()} visible")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MG_TP_NCCL="1" if nccl_exchange else "0",
               MG_TP_MEGA="0" if kernels_path else "1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
                          os.path.join(ROOT, "tests", "tp_worker.py"), *cases],
                         capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-3000:])
    found = [l for l in out.stdout.splitlines() if l.startswith("TP_RESULTS ")]
    assert len(found) == 1, (out.stdout[-1500:], out.stderr[-3000:])
    lines = json.loads(found[0][len("TP_RESULTS "):])
    assert len(lines) == world
    return sorted(lines, key=lambda l: l["rank"])


def check(lines, cases, n_new=24, nccl_exchange=False, persistent=True):
    for name in cases:
        assert all(l["results"][name]["nccl_exchange"] == nccl_exchange for l in lines), "unexpected exchange path"
        assert all(l["results"][name]["persistent"] == persistent for l in lines), "unexpected kernel path"
        toks = lines[0]["results"][name]["tokens"]
        for l in lines:
            r = l["results"][name]
            assert r["logits_err"] <= TOL and r["hidden_err"] <= TOL and r["token_logits_err"] <= TOL, (name, r)
            assert r["exact"] + r["ties"] == n_new, (name, r)
            assert r["tokens"] == toks, f"{name}: ranks disagree on the greedy tokens"
            assert r["launches"] > 0


def test_two_ranks_match_the_oracle():
    """The persistent kernel on every rank, partial sums and argmax keys exchanged inside it (peer
    stores into mapped receive buffers)."""
    cases = ["tiny", "tiny-bias-ragged", "tiny-q4", "hd128-gqa", "tiny-kv1"]
    check(run_ranks(2, cases), cases)


def test_two_ranks_on_the_phase_kernels_match_the_oracle():
    """The graph of per-phase kernels with the exchange fused into their prologues / epilogues."""
    cases = ["tiny", "tiny-bias-ragged", "tiny-q4", "hd128-gqa", "tiny-kv1"]
    check(run_ranks(2, cases, kernels_path=True), cases, persistent=False)


def test_two_ranks_with_nccl_exchange_match_the_oracle():
    """The same with ncclAllReduce between the kernels (MG_TP_NCCL=1)."""
    cases = ["tiny", "hd128-gqa"]
    check(run_ranks(2, cases, nccl_exchange=True), cases, nccl_exchange=True, persistent=False)


def test_two_ranks_share_a_kv_head_and_split_its_q_heads_unevenly():
    """What eight ranks do with 28 Q / 4 KV heads (4 + 3 Q heads of a KV head held twice), on two."""
    cases = ["kv1-uneven"]
    check(run_ranks(2, cases), cases)
    check(run_ranks(2, cases, kernels_path=True), cases, persistent=False)


def test_four_ranks_with_replicated_kv_heads_match_the_oracle():
    # 2 KV heads over 4 ranks: every KV head is held by two ranks that split its Q heads
    cases = ["tiny", "tiny-bias-ragged", "hd128-gqa"]
    check(run_ranks(4, cases), cases)


def test_eight_ranks_split_the_q_groups_of_shared_kv_heads():
    """28 Q heads over 4 KV heads on 8 ranks: consecutive ranks share a KV head and take 4 + 3 of its Q heads."""
    cases = ["gqa-28-4"]
    check(run_ranks(8, cases), cases)


def test_two_ranks_on_7b_class_widths():
    """Real 7B-class layer shapes (dim 3584, head_dim 128, FFN 18944) split over two ranks."""
    cases = ["qwen7b-width-2L"]
    check(run_ranks(2, cases, timeout=900), cases)


def test_four_ranks_on_the_7b_head_geometry():
    cases = ["gqa-28-4"]
    check(run_ranks(4, cases), cases)
