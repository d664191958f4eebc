"""One tensor-parallel rank of the GPU parity test (launched by torchrun from
test_gpu_tensor_parallel.py; not collected by pytest).

Every rank builds the same seeded model, hands the FULL tensors to its engine (which keeps its
shard) and to a CPU oracle, and compares: logits of PartialStep/StepToken within 1e-4 relative,
greedy tokens identical (ties by the oracle's own logits excepted).  Rank 0 prints every rank's
results as one JSON line.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch                                   # noqa: E402
import torch.distributed as dist               # noqa: E402

from mongoose_b200 import configs as mc        # noqa: E402
from mongoose_b200 import multi                # noqa: E402
from mongoose_b200.fused_infer import CUDAFusedInference   # noqa: E402
from oracle import gen                         # noqa: E402
from oracle import oracle as O                 # noqa: E402
from tests.util import fill_models, greedy_parity, rel_err   # noqa: E402

CASES = {
    "tiny": (mc.TINY, False),
    "tiny-bias-ragged": (mc.TINY.with_(name="tiny-ragged", vocab=1001), True),
    "tiny-q4": (mc.TINY_Q4, False),
    # one KV head for four Q heads: with two ranks the KV head (rows, bias, cache) is held by both
    "tiny-kv1": (mc.TINY.with_(name="tiny-kv1", n_kv_heads=1), True),
    # one KV head held by both of two ranks, which take 2 + 1 of its three Q heads (and 192 + 160 FFN
    # features): the mechanism of the 8-rank 28 Q / 4 KV split - a replicated KV head, ranks with
    # different numbers of Q heads - on two GPUs
    "kv1-uneven": (mc.TINY.with_(name="kv1-uneven", dim=96, n_heads=3, n_kv_heads=1, head_dim=32, ffn_dim=352), True),
    "hd128-gqa": (mc.TINY.with_(name="hd128-gqa", dim=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn_dim=1184,
                               vocab=1500, n_layers=2), True),
    # the 7B-class head geometry on a small model: 28 Q heads over 4 KV heads; with 8 ranks every KV head is
    # held by two ranks that take 4 + 3 of its Q heads
    "gqa-28-4": (mc.TINY.with_(name="gqa-28-4", dim=896, n_heads=28, n_kv_heads=4, head_dim=32, ffn_dim=1024,
                              vocab=1608, n_layers=2), True),
    # real 7B-class widths (head_dim 128, FFN 18944), two layers and a cut vocabulary
    "qwen7b-width-2L": (mc.QWEN25_7B.with_(name="qwen7b-width-2L", n_layers=2, vocab=4000, max_seq=48), False),
}


def progress(msg):
    """Progress lines on stderr when TP_WORKER_VERBOSE=1 (which step a stuck run had reached)."""
    if os.environ.get("TP_WORKER_VERBOSE") == "1":
        print(f"[tp_worker rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


def main():
    rank, world, local = multi.rank_env()
    dist.init_process_group("gloo")
    torch.cuda.set_device(local)
    results = {}
    for name in sys.argv[1:]:
        cfg, bias = CASES[name]
        tp_id = multi.share_unique_id(dist, rank)
        eng = CUDAFusedInference(cfg, device=local, tp_rank=rank, tp_size=world, tp_id=tp_id)
        om = O.OracleModel(cfg)
        note = eng._lib.mg_last_error(eng._h).decode()      # says so when the exchange goes through NCCL
        fill_models(cfg, seed=3, jitter=0.1, engine=eng, oracle_model=om, raw_slots=True, bias=bias)
        progress(f"{name}: weights set")
        eng.BuildFusedDispatch()
        progress(f"{name}: built: {eng._lib.mg_last_error(eng._h).decode()!r}")
        persistent = "persistent kernel not used" not in eng._lib.mg_last_error(eng._h).decode()
        rng = np.random.default_rng(5)
        worst = 0.0
        logits = np.empty(cfg.vocab, np.float32)
        hid = np.empty(cfg.dim, np.float32)
        # hidden-state input, every layer and the head in one call; then layer ranges
        for pos in range(5):
            h = rng.standard_normal(cfg.dim).astype(np.float32)
            eng.PartialStep(h, pos, 0, cfg.n_layers, None, logits)
            progress(f"{name}: PartialStep pos {pos} done")
            _, want = om.step(h, pos, 0, cfg.n_layers)
            worst = max(worst, rel_err(logits, want))
        eng.ResetKV(); om.reset_kv()
        h = rng.standard_normal(cfg.dim).astype(np.float32)
        eng.PartialStep(h, 0, 0, 1, hid, None)
        want_h, _ = om.step(h, 0, 0, 1, want_logits=False)
        worst_hidden = rel_err(hid, want_h)
        progress(f"{name}: layer-range step done, logits err {worst:.2e}, hidden err {worst_hidden:.2e}")
        # token input with logits
        eng.ResetKV(); om.reset_kv()
        tok_err = 0.0
        t = 7
        for pos in range(4):
            nxt = eng.StepToken(t, pos, logits)
            want = om.step_token(t, pos)
            tok_err = max(tok_err, rel_err(logits, want))
            assert nxt == int(np.argmax(logits)), "argmax over ranks differs from the gathered logits"
            t = nxt
        progress(f"{name}: StepToken loop done")
        # greedy generation
        eng.ResetKV()
        prompt = gen.prompt_ids(0, 6, cfg.vocab)
        n_new = 24
        toks = eng.Generate(prompt, n_new)
        progress(f"{name}: Generate done")
        exact, ties, _ = greedy_parity(toks, om, prompt, n_new)
        results[name] = {"logits_err": worst, "hidden_err": worst_hidden, "token_logits_err": tok_err,
                         "exact": exact, "ties": len(ties), "tokens": [int(x) for x in toks],
                         "launches": eng.LaunchCount(),
                         "nccl_exchange": "ncclAllReduce" in note, "persistent": persistent}
        eng.close(); om.close()
        dist.barrier()
    # one writer: lines of several ranks on a shared pipe can interleave
    everyone = [None] * world
    dist.all_gather_object(everyone, {"rank": rank, "world": world, "results": results})
    if rank == 0:
        print("TP_RESULTS " + json.dumps(everyone), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
