"""Tensor-parallel partition tables (mg_tp_partition): host arithmetic, no GPU.

The ranks' parts must tile the model: Q heads and FFN features exactly once, vocabulary rows
exactly once, every Q head served by a KV head its rank holds, no quantization block split.
"""
import os
import subprocess
import sys

from tests.util import free_port

import pytest

from mongoose_b200 import configs as mc
from mongoose_b200 import multi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def check_tiling(cfg, size):
    parts = [multi.tp_partition(cfg, r, size) for r in range(size)]
    group = cfg.n_heads // cfg.n_kv_heads
    q_seen, f_seen, v_seen = [], [], []
    for p in parts:
        q0, q1 = p["q_heads"]
        kv0, kv1 = p["kv_heads"]
        assert q1 > q0 and kv1 > kv0
        for h in range(q0, q1):
            assert kv0 <= h // group < kv1          # the KV head of every local Q head is local
        # local head -> local KV head must be the kernel's mapping (local index // local group)
        lg = (q1 - q0) // (kv1 - kv0)
        assert (q1 - q0) % (kv1 - kv0) == 0
        for h in range(q0, q1):
            assert (h - q0) // lg + kv0 == h // group
        f0, f1 = p["ffn"]
        assert f0 % 32 == 0 and f1 % 32 == 0 and f1 > f0
        q_seen += list(range(q0, q1))
        f_seen.append((f0, f1))
        v_seen.append(p["vocab"])
    assert q_seen == list(range(cfg.n_heads))
    assert f_seen[0][0] == 0 and f_seen[-1][1] == cfg.ffn_dim
    assert all(f_seen[i][1] == f_seen[i + 1][0] for i in range(size - 1))
    assert v_seen[0][0] == 0 and v_seen[-1][1] == cfg.vocab
    assert all(v_seen[i][1] == v_seen[i + 1][0] for i in range(size - 1))
    stride = -(-cfg.vocab // size)
    assert all(v[0] == min(cfg.vocab, r * stride) for r, v in enumerate(v_seen))
    return parts


@pytest.mark.parametrize("size", [1, 2, 4, 8])
def test_7b_partitions_tile_the_model(size):
    parts = check_tiling(mc.QWEN25_7B, size)
    if size == 8:
        # 4 KV heads over 8 ranks: each KV head on two ranks that take 4 + 3 of its 7 Q heads
        assert [p["q_heads"][1] - p["q_heads"][0] for p in parts] == [4, 3] * 4
        assert [p["kv_heads"] for p in parts] == [(k, k + 1) for k in range(4) for _ in range(2)]
        assert parts[0]["ffn"] == (0, 2368) and parts[0]["vocab"] == (0, 19008)


@pytest.mark.parametrize("size", [2, 4])
def test_tinyllama_partitions(size):
    check_tiling(mc.TINYLLAMA_11B, size)


def test_qwen05b_two_ranks_and_ragged_vocab():
    parts = check_tiling(mc.QWEN25_05B, 2)
    assert parts[0]["q_heads"] == (0, 7) and parts[1]["kv_heads"] == (1, 2)
    odd = mc.TINY.with_(name="ragged", vocab=1001)
    parts = check_tiling(odd, 2)
    assert parts[0]["vocab"] == (0, 501) and parts[1]["vocab"] == (501, 1001)


def test_unsplittable_head_counts_are_refused():
    with pytest.raises(ValueError):
        multi.tp_partition(mc.QWEN25_05B, 0, 3)      # 2 KV heads and 3 ranks: neither divides the other
    with pytest.raises(ValueError):
        multi.tp_partition(mc.QWEN25_7B, 0, 3)
    with pytest.raises(ValueError):
        multi.tp_partition(mc.QWEN25_7B, 2, 2)


WORKER = r"""
import os, sys, json
sys.path.insert(0, %r)
import torch.distributed as dist
from mongoose_b200 import multi, configs as mc
rank, world, local = multi.rank_env()
dist.init_process_group("gloo")
mine = multi.tp_partition(mc.QWEN25_7B, rank, world)
parts = [None] * world
dist.all_gather_object(parts, mine)
box = [os.urandom(128) if rank == 0 else None]
dist.broadcast_object_list(box, src=0)
everyone = [None] * world
dist.all_gather_object(everyone, {"rank": rank, "parts": parts, "id": box[0].hex()})
if rank == 0:
    print("RESULTS " + json.dumps(everyone), flush=True)
dist.destroy_process_group()
""" % ROOT


def test_two_gloo_ranks_agree_on_the_partition_and_the_id(tmp_path):
    script = tmp_path / "tp_worker.py"
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
    a, b = sorted(lines, key=lambda l: l["rank"])
    assert a["parts"] == b["parts"] and a["id"] == b["id"] and len(a["id"]) == 256
    assert a["parts"][0]["q_heads"] == [0, 14] and a["parts"][1]["q_heads"] == [14, 28]
    assert a["parts"][0]["kv_heads"] == [0, 2] and a["parts"][1]["ffn"] == [9472, 18944]


# -- the split itself, restated with the CPU oracle ---------------------------------------------
@pytest.mark.parametrize("fmt", [mc.FMT_Q8_0, mc.FMT_Q4_0], ids=["q8_0", "q4_0"])
@pytest.mark.parametrize("size", [2, 4])
def test_sharded_layer_equals_the_unsplit_layer_on_the_oracle(fmt, size):
    """One transformer layer's matvecs computed shard by shard from slices of the UNSPLIT quantized
    tensors (rows for q/k/v/gate/up, block-aligned columns for wo/down) and summed over ranks equal
    the unsplit computation: the partition never cuts a quantization block and every Q head finds its
    KV head on its rank."""
    import numpy as np
    from oracle import oracle as O
    cfg = mc.TINY.with_(name="tp-oracle", dim=256, n_heads=8, n_kv_heads=2, head_dim=32, ffn_dim=352)
    hd, dim, kvd, ffn = cfg.head_dim, cfg.dim, cfg.kv_dim, cfg.ffn_dim
    rng = np.random.default_rng(11)
    W = {n: (0.05 * rng.standard_normal(s)).astype(np.float32)
         for n, s in (("q", (dim, dim)), ("k", (kvd, dim)), ("v", (kvd, dim)), ("o", (dim, dim)),
                      ("g", (ffn, dim)), ("u", (ffn, dim)), ("d", (dim, ffn)))}
    B = {n: O.quantize(fmt, w) for n, w in W.items()}
    bb = {mc.FMT_Q8_0: 34, mc.FMT_Q4_0: 18}[fmt]

    def cols(blocks, k0, k1):          # raw blocks of columns [k0, k1) of every row
        assert k0 % 32 == 0 and k1 % 32 == 0
        return np.ascontiguousarray(blocks[:, k0 // 32 * bb:k1 // 32 * bb])

    x = rng.standard_normal(dim).astype(np.float32)
    attn = rng.standard_normal(dim).astype(np.float32)          # stands in for the attention output
    q_full = O.matvec(fmt, B["q"], x, dim, dim)
    k_full = O.matvec(fmt, B["k"], x, kvd, dim)
    o_full = O.matvec(fmt, B["o"], attn, dim, dim)
    g_full = O.matvec(fmt, B["g"], x, ffn, dim)
    u_full = O.matvec(fmt, B["u"], x, ffn, dim)
    mid = O.silu_gate_mul(g_full, u_full)
    d_full = O.matvec(fmt, B["d"], mid, dim, ffn)

    q_parts, o_sum, d_sum = [], np.zeros(dim, np.float64), np.zeros(dim, np.float64)
    group = cfg.n_heads // cfg.n_kv_heads
    for r in range(size):
        p = multi.tp_partition(cfg, r, size)
        (q0, q1), (kv0, kv1), (f0, f1) = p["q_heads"], p["kv_heads"], p["ffn"]
        # row splits reproduce the unsplit rows bit for bit
        q_r = O.matvec(fmt, np.ascontiguousarray(B["q"][q0 * hd:q1 * hd]), x, (q1 - q0) * hd, dim)
        k_r = O.matvec(fmt, np.ascontiguousarray(B["k"][kv0 * hd:kv1 * hd]), x, (kv1 - kv0) * hd, dim)
        assert np.array_equal(q_r, q_full[q0 * hd:q1 * hd]) and np.array_equal(k_r, k_full[kv0 * hd:kv1 * hd])
        assert all(kv0 <= h // group < kv1 for h in range(q0, q1))
        q_parts.append(q_r)
        # column splits give partial sums
        o_sum += O.matvec(fmt, cols(B["o"], q0 * hd, q1 * hd), attn[q0 * hd:q1 * hd], dim, (q1 - q0) * hd)
        g_r = O.matvec(fmt, np.ascontiguousarray(B["g"][f0:f1]), x, f1 - f0, dim)
        u_r = O.matvec(fmt, np.ascontiguousarray(B["u"][f0:f1]), x, f1 - f0, dim)
        mid_r = O.silu_gate_mul(g_r, u_r)
        assert np.array_equal(mid_r, mid[f0:f1])
        d_sum += O.matvec(fmt, cols(B["d"], f0, f1), mid_r, dim, f1 - f0)
    assert np.array_equal(np.concatenate(q_parts), q_full)
    for got, want in ((o_sum, o_full), (d_sum, d_full)):
        assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max()


def test_every_gpu_test_case_has_a_partition_for_its_rank_count():
    """The multi-GPU tests name (ranks, model) pairs; a pair without a partition would only show on
    a box with that many GPUs."""
    from mongoose_b200 import multi
    from tests import tp_worker
    from tests.test_gpu_tensor_parallel import RANK_CASES
    for world, names in RANK_CASES.items():
        for name in names:
            cfg, _ = tp_worker.CASES[name]
            for rank in range(world):
                part = multi.tp_partition(cfg, rank, world)
                assert part["q_heads"][1] > part["q_heads"][0], (world, name, rank, part)
