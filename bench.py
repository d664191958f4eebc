#!/usr/bin/env python
"""Decode benchmark for the fused quantized decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Workload (default): Qwen2.5-0.5B architecture, random-init, Q8_0 (block 32, fp16 scales), fp16 KV,
batch 1: a 32-token prompt fed one position at a time, then K greedy decode steps.  A "step" is one
decode token.  Prints ONE JSON line.

  value     tokens/s with everything resident in HBM: K greedy steps enqueued back to back
            (argmax fed back on the device), timed with CUDA events on the engine's stream.
  e2e       tokens/s through the reference-facing call PartialStep(hiddenIn, pos, 0, L, nil, logitsOut)
            with pinned HOST buffers: each step uploads the hidden vector and downloads the logits.
  roofline  the decode step as a whole (it is one graph launch): algorithmic bytes per token
            (quantized weights + fp16 KV read at the mean context) / step time, against the measured
            HBM copy peak in MEASURED_PEAKS.json.

With N > 1 (launched under torchrun, one rank per GPU) every rank decodes its own independent
sequence on its own replica of the weights: no data-path collective, weak scaling.

--impl reference times the CPU port of the reference's pure-Go engine (oracle/oracle.c,
oracle_cpu_engine_step_token) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from mongoose_b200 import configs as mc  # noqa: E402
from mongoose_b200 import multi  # noqa: E402
from mongoose_b200 import synthetic  # noqa: E402

PROMPT_LEN = 32
# DRAM bytes per decoded token (dram__bytes_read.sum + dram__bytes_write.sum of mega_decode_kernel from one
# ncu capture of a 3-token launch, divided by 3).
NCU_TRAFFIC_PER_TOKEN = {"qwen2.5-0.5b-q8_0-b1": 634.1e6}
# The one number the reference publishes for this metric: Qwen2.5-0.5B, batch 1, 200 tokens, "CUDA Q8
# fused matvec" (per-row INT8 weights) on an RTX 5090: 234.0 tok/s (README.md:55-60 of the reference).
PUBLISHED_TOK_S = {"qwen2.5-0.5b-q8_0-b1": 234.0}
WORKLOADS = {
    "qwen2.5-0.5b-q8_0-b1": mc.QWEN25_05B,
    "qwen2.5-0.5b-q4_0-b1": mc.QWEN25_05B_Q4,
    "tiny-q8_0-b1": mc.TINY,
    "qwen2.5-7b-q8_0-b1": mc.QWEN25_7B,
    # one sequence, the model split over all ranks (tensor parallel; needs --gpus 2, 4 or 8);
    # on one GPU it is the same as qwen2.5-7b-q8_0-b1
    "qwen2.5-7b-q8_0-tp": mc.QWEN25_7B,
    "tiny-q8_0-tp": mc.TINY,
    # 7B-class layer shapes with few layers and a cut vocabulary: loads in seconds (smoke runs of the exchange)
    "qwen2.5-7b-width-4l-q8_0-tp": mc.QWEN25_7B.with_(name="qwen2.5-7b-width-4l", n_layers=4, vocab=16000),
    # 64 independent sequences (512-token prompt + 512 decode steps each in the full configuration),
    # sequence i on GPU i mod G, each decoded with batch-1 semantics as the reference would (one
    # engine pass per token); select sizes with --sequences / --prompt-len / --steps
    "tinyllama-1.1b-q8_0-seqs": mc.TINYLLAMA_11B,
    # the single-op configuration: one Q8_0 dequant-matvec, W 4864 x 896 in raw 34-byte blocks
    "q8_0-matvec-4864x896": None,
}
FMT_NAME = {mc.FMT_Q8_0: "q8_0", mc.FMT_Q4_0: "q4_0", mc.FMT_F16: "f16"}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="qwen2.5-0.5b-q8_0-b1", choices=sorted(WORKLOADS))
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN)
    ap.add_argument("--sequences", type=int, default=8, help="sequences of the *-seqs workload (full config: 64)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--cpu-steps", type=int, default=0, help="steps of the CPU baseline sample (0 = auto)")
    ap.add_argument("--no-legs", action="store_true",
                    help="skip the two partitioned configurations that ride in the same line (tensor-parallel 7B-class "
                         "layers over the ranks, independent TinyLlama sequences sharded over the ranks)")
    return ap.parse_args()


def algorithmic_bytes_per_token(cfg, first_pos: int, steps: int) -> float:
    """Quantized weight bytes + fp16 KV bytes read at the mean context of the timed window."""
    mean_ctx = first_pos + 1 + (steps - 1) / 2.0      # positions attended to, averaged over the window
    return mc.weight_bytes_per_token(cfg) + mc.kv_bytes_per_position(cfg) * mean_ctx


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.windows = []          # [begin, end] pairs: the timed regions

    # nvidia-smi needs a few hundred ms to come up, longer than a short timed region: start it
    # early (start), then bracket every timed region (begin / end; the device-resident loop and the
    # host-buffer loop are both bracketed); stop() keeps the samples whose timestamps fall inside a
    # bracket.  A query takes nvidia-smi 20-100 ms, so a bracket of 80 ms can fall between two
    # samples: the brackets are then widened step by step (and the line says by how much).
    def begin(self):
        import datetime
        self.windows.append([datetime.datetime.now(), None])

    def end(self):
        import datetime
        self.windows[-1][1] = datetime.datetime.now()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f")
                rows.append((ts, float(f[1]), float(f[2]), float(f[3]), f[5:9]))
            except ValueError:
                continue
        windows = [w for w in self.windows if w[1] is not None]
        picked, used_slack = rows if not windows else [], None
        for slack_ms in (25, 100, 300, 1000):
            if picked or not windows:
                break
            slack = datetime.timedelta(milliseconds=slack_ms)
            picked = [r for r in rows if any(w[0] - slack <= r[0] <= w[1] + slack for w in windows)]
            used_slack = slack_ms
        sm = [r[1] for r in picked]
        mx = [r[2] for r in picked]
        power = [r[3] for r in picked]
        reasons = set()
        for r in picked:
            for n, v in zip(names, r[4]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        res = {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
               "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}
        if used_slack is not None and used_slack > 25:
            res["window"] = f"timed regions widened by {used_slack} ms (nvidia-smi answered slower than they are long)"
        return res


# ---------------------------------------------------------------------------
# CPU baseline (the only place this file touches oracle/)
# ---------------------------------------------------------------------------
def cpu_baseline_run(cfg, max_steps: int, nthreads: int, budget_s: float = 25.0, seed: int = 0, prompt_len: int = 2):
    """Times decode tokens of the CPU-engine port on a freshly generated model: `prompt_len` prompt
    tokens through the same path (untimed; the first pages the weights in), then as many tokens as
    fit in about `budget_s` seconds (at most max_steps).
    Returns (tok_per_s, seconds, threads, steps)."""
    from oracle import oracle as O
    om = O.OracleModel(cfg)
    for idx, kind, rows, cols, fmt in synthetic.model_slots(cfg):
        if kind == "norm":
            om.set_weight(idx, synthetic.norm_vector(seed, idx, cols), 0)
        else:
            om.set_weight(idx, O.quantize(fmt, synthetic.tensor_f32(seed, idx, rows, cols)), fmt)
    prompt = synthetic.prompt_ids(seed, max(prompt_len, 2), cfg.vocab)
    # the thread count is passed to the OpenMP region explicitly: launchers such as torchrun export
    # OMP_NUM_THREADS=1, which must not silently turn the all-cores arm into a single-threaded one
    nthreads = max(1, nthreads)
    logits, probe = None, 0.0
    for pos in range(max(prompt_len, 2)):
        t0 = time.perf_counter()
        logits = om.cpu_engine_step_token(int(prompt[pos]), pos, nthreads)
        probe = time.perf_counter() - t0
    first = max(prompt_len, 2)
    steps = max(1, min(max_steps, cfg.max_seq - first, int(budget_s / max(probe, 1e-4))))
    tok = int(np.argmax(logits))
    t0 = time.perf_counter()
    for i in range(steps):
        logits = om.cpu_engine_step_token(tok, first + i, nthreads)
        tok = int(np.argmax(logits))
    dt = time.perf_counter() - t0
    om.close()
    return steps / dt, dt, nthreads, steps


def reference_gpu_kernels(cfg, steps: int, context: int):
    """The reference's own CUDA kernels (kernels/mongoose.cu built unmodified for this GPU) chained in
    the op order of its PartialStep on its per-row INT8 weights and fp32 KV: one token's 410 launches
    are captured in a CUDA graph once and replayed, so the figure is the device-side time of the
    reference's path with every host cost removed.  None where the library or a GPU is missing."""
    try:
        import torch
        from oracle import oracle as O
        from oracle import ref_chain
        if not torch.cuda.is_available() or not os.path.exists(ref_chain.REF_LIB):
            return None
        lib = ref_chain.load()
        cfg = cfg.with_(max_seq=context + 1)
        weights, norms = ref_chain.synthetic_model(cfg, seed=0)
        cos, sin = O.rope_tables(cfg.max_seq, cfg.head_dim, cfg.rope_theta)
        chain = ref_chain.RefChain(torch, cfg, weights, norms, cos, sin)
        del weights
        s = torch.cuda.Stream()
        chain.hidden.normal_()
        with torch.cuda.stream(s):
            chain.enqueue(lib, context, 0, cfg.n_layers, True, stream=s.cuda_stream)     # warm-up, eager
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            chain.enqueue(lib, context, 0, cfg.n_layers, True, stream=s.cuda_stream)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            g.replay()
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / steps
        return {"value": 1e3 / ms, "unit": "tok/s", "ms_per_step": ms, "launches_per_token": cfg.n_layers * 17 + 2,
                "how": f"kernels/mongoose.cu (sm_100 build) in PartialStep order, per-row INT8 weights, fp32 KV, context {context}, "
                       f"one CUDA graph per token replayed {steps} times (no host launch cost)"}
    except Exception as ex:
        return {"unavailable": f"{type(ex).__name__}: {ex}"[:200]}


def run_reference_arm(args, cfg, rank):
    """The reference's CPU implementation of the path, timed on the host cores (rank 0 only: one host
    run whatever the number of GPUs)."""
    if rank != 0:
        return
    ncores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    cfg = cfg.with_(max_seq=max(cfg.max_seq, PROMPT_LEN + args.steps + 2))
    tps, dt, threads, sample = cpu_baseline_run(cfg, args.steps, ncores, budget_s=40.0, prompt_len=PROMPT_LEN)
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": tps, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / tps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": FMT_NAME[cfg.layer_fmt], "data": "synthetic",
        "config": {"workload": args.workload, "prompt_len": PROMPT_LEN, "batch": 1,
                   "note": "one run on the host cores at every N: the CPU engine has no multi-GPU form"},
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"{sample} decode tokens ({dt:.1f} s) after the {PROMPT_LEN}-token prompt, rows split over "
                                   f"{threads} OpenMP threads (the Go engine itself is single-threaded)"},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    gpu = reference_gpu_kernels(cfg, max(args.steps, 20), PROMPT_LEN + 100)
    if gpu is not None:
        line["reference_gpu_kernels"] = gpu
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# B200 arm
# ---------------------------------------------------------------------------
def run_b200_arm(args, cfg, rank, world, local_rank):
    import torch
    from mongoose_b200.fused_infer import CUDAFusedInference

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for this path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    K, W = args.steps, max(args.warmup, 3)
    cfg = cfg.with_(max_seq=max(cfg.max_seq, PROMPT_LEN + K))
    tp = args.workload.endswith("-tp") and world > 1    # one sequence over all ranks, else one per rank
    if tp:
        eng = CUDAFusedInference(cfg, device=local_rank, tp_rank=rank, tp_size=world,
                                 tp_id=multi.share_unique_id(dist, rank))
    else:
        eng = CUDAFusedInference(cfg, device=local_rank)
    seed = 0                                            # same weights on every replica
    synthetic.load_engine(eng, cfg, seed=seed)          # under tensor parallelism each rank keeps its part
    eng.BuildFusedDispatch()
    prompt = synthetic.prompt_ids(0 if tp else rank, PROMPT_LEN, cfg.vocab)   # replicas decode their own sequence
    stream = torch.cuda.ExternalStream(eng.stream, device=local_rank)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def feed_prompt():
        """The prompt goes through the decode path one position at a time (the reference has no
        batched prefill); the last prompt step yields the first generated token."""
        eng.ResetKV()
        tok = -1
        for pos, t in enumerate(prompt):
            tok = eng.StepToken(int(t), pos)
        eng.SetCursor(tok, PROMPT_LEN)
        return PROMPT_LEN

    sampler = ClockSampler(local_rank)
    sampler.start()                                     # comes up during the warm-up

    # ---- warm-up: W greedy steps on the same graph, then start over ----
    feed_prompt()
    eng.EnqueueGreedy(min(W, cfg.max_seq - PROMPT_LEN))
    eng.Sync()

    # ---- timed: device-resident greedy decode ----
    first_pos = feed_prompt()
    launches0 = eng.LaunchCount()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.begin()
    ev0.record(stream)
    eng.EnqueueGreedy(K)
    ev1.record(stream)
    eng.Sync()
    sampler.end()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = eng.LaunchCount() - launches0
    tok_last, pos_last = eng.GetCursor()
    assert pos_last == first_pos + K, (pos_last, first_pos, K)

    # ---- e2e: PartialStep with pinned host buffers (hidden in, logits out) ----
    # The token sequence is the one just generated, so no host-side sampling sits in the timed loop;
    # the caller-side embedding rows (dequantized lm_head rows) are prepared beforehand.
    e2e_s, e2e_last_tok = float("nan"), -1
    gen_tokens = eng.Generate(prompt, K)                # g0 .. g(K-1): the inputs of the K decode steps
    if not args.no_e2e:
        seq = np.concatenate([prompt, gen_tokens])
        head_idx = cfg.n_layers * 12 + 1
        hid = torch.empty((len(seq), cfg.dim), dtype=torch.float32).pin_memory()
        for i, t in enumerate(seq):
            hid[i] = torch.from_numpy(eng.DequantRows(head_idx, int(t), 1, cfg.dim)[0])
        logits_host = torch.empty(cfg.vocab, dtype=torch.float32).pin_memory()
        eng.ResetKV()
        for i in range(PROMPT_LEN):
            eng.PartialStep(hid[i], i, 0, cfg.n_layers, None, logits_host)
        barrier()
        sampler.begin()
        t0 = time.perf_counter()
        for i in range(PROMPT_LEN, PROMPT_LEN + K):
            eng.PartialStep(hid[i], i, 0, cfg.n_layers, None, logits_host)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        sampler.end()
        e2e_last_tok = int(torch.argmax(logits_host))
        barrier()
    clocks = sampler.stop()

    # max over ranks
    ms_max, e2e_ms_max = multi.reduce_max([ms, e2e_s * 1e3], dist, device="cuda")
    eng.close()
    eng = None
    legs = {}
    if not args.no_legs and not tp and args.workload == "qwen2.5-0.5b-q8_0-b1":
        for name, fn in (("tp", run_tp_leg), ("seqs", run_seqs_leg)):
            try:
                legs[name] = fn(torch, dist, rank, world, local_rank)
            except Exception as ex:                 # a leg must not take the headline number down with it
                legs[name] = {"error": f"{type(ex).__name__}: {ex}"[:300]}

    if rank == 0:
        jobs = 1 if tp else world                                   # sequences decoded side by side
        tps = multi.aggregate_rate(jobs, K, ms_max)
        bytes_tok = algorithmic_bytes_per_token(cfg, first_pos, K) / (world if tp else 1)
        peak, peak_src = measured_peak_gbs()
        achieved = bytes_tok * (K / (ms_max / 1e3)) / 1e9          # per GPU
        line = {
            "metric": "decode_tokens_per_s", "value": tps, "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_max / K, "higher_is_better": True, "scaling": "strong" if tp else "weak",
            "vs_baseline": (tps / PUBLISHED_TOK_S[args.workload] if args.workload in PUBLISHED_TOK_S else None),
            "dtype": FMT_NAME[cfg.layer_fmt], "data": "synthetic",
            "config": {"workload": args.workload, "prompt_len": PROMPT_LEN, "batch": 1,
                       "published_baseline": ("234.0 tok/s: the reference's README figure for this model and batch "
                                              "on one RTX 5090 with per-row INT8 weights"
                                              if args.workload in PUBLISHED_TOK_S else None),
                       "parallelism": (f"tensor parallel x{world} (partial sums exchanged " +
                                        ("by ncclAllReduce)" if os.environ.get("MG_TP_NCCL") == "1" else
                                         "inside the kernels over peer memory)") if tp else
                                       f"replicas x{world}" if world > 1 else "single GPU"),
                       "l2": "inputs larger than L2 (weights streamed per token: %d MB)" %
                             (mc.weight_bytes_per_token(cfg) // 2 ** 20),
                       "timing": "CUDA events on the engine stream, max over ranks"},
            "e2e": {"value": multi.aggregate_rate(jobs, K, e2e_ms_max), "unit": "tok/s",
                    "h2d_bytes_per_step": cfg.dim * 4 + 8, "d2h_bytes_per_step": cfg.vocab * 4,
                    "api": "PartialStep(hiddenIn, pos, 0, L, nil, logitsOut) with pinned host buffers (the logits cross PCIe as stores of the kernel into logitsOut)",
                    "last_token_matches_device_loop": bool(e2e_last_tok == tok_last)},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_PER_TOKEN.get(args.workload),
                         "traffic_unit": "bytes per token (one launch decodes all timed tokens)", "peak_source": peak_src,
                         "kernel": ("whole decode step (mega_decode_kernel: one persistent launch for all timed tokens)"
                                    if launches == 1 else "whole decode step (graph of fused phase kernels)"),
                         "algorithmic_bytes_per_token": bytes_tok, "frac_of_8TBs": achieved / 8000.0},
            "clocks": clocks,
            "tokens_tail": [int(x) for x in gen_tokens[-4:]],
        }
        if world == 1 and not args.no_cpu_baseline:
            ctps, cdt, cth, n = cpu_baseline_run(cfg.with_(max_seq=64), args.cpu_steps or 60, 1, budget_s=15.0)
            line["cpu_baseline"] = {"value": ctps, "unit": "tok/s", "cores": cth, "kind": "port",
                                    "sample": f"{n} decode tokens of the same model (after a 2-token prompt) on the "
                                              f"single-threaded CPU-engine port ({cdt:.1f} s)"}
        if legs:
            line["legs"] = legs
        print(json.dumps(line), flush=True)
    if eng is not None:
        eng.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# The two configurations that partition work over the GPUs ride in the same line as "legs"
# ---------------------------------------------------------------------------
TP_LEG_CFG = mc.QWEN25_7B.with_(name="qwen2.5-7b-width-4l", n_layers=4, vocab=16000, max_seq=PROMPT_LEN + 64)
SEQ_LEG_CFG = mc.TINYLLAMA_11B


def run_tp_leg(torch, dist, rank, world, local_rank, steps=48):
    """One sequence, 7B-class layer shapes (4 layers, cut vocabulary: loads in seconds) split over all
    ranks by rows / columns; the partial sums are exchanged inside the persistent kernel over peer
    memory.  Strong scaling: tokens/s of the one sequence."""
    from mongoose_b200.fused_infer import CUDAFusedInference
    cfg = TP_LEG_CFG
    kw = {}
    if world > 1:
        kw = dict(tp_rank=rank, tp_size=world, tp_id=multi.share_unique_id(dist, rank))
    # A rank whose engine fails must still meet the others in every collective below, or they would
    # wait for it: engine work sits in guarded sections, the collectives run unconditionally.
    err, eng, note, stream, ms, tok_last = None, None, "", None, 0.0, -1
    try:
        eng = CUDAFusedInference(cfg, device=local_rank, **kw)
        synthetic.load_engine(eng, cfg, seed=0)
        eng.BuildFusedDispatch()
        note = eng._lib.mg_last_error(eng._h).decode()
        prompt = synthetic.prompt_ids(0, PROMPT_LEN, cfg.vocab)
        stream = torch.cuda.ExternalStream(eng.stream, device=local_rank)

        def feed():
            eng.ResetKV()
            tok = -1
            for pos, t in enumerate(prompt):
                tok = eng.StepToken(int(t), pos)
            eng.SetCursor(tok, PROMPT_LEN)

        feed()
        eng.EnqueueGreedy(8)
        eng.Sync()
        feed()
        torch.cuda.synchronize()
    except Exception as ex:
        err = ex
    if dist is not None:
        dist.barrier()
    if err is None:
        try:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record(stream)
            eng.EnqueueGreedy(steps)
            ev1.record(stream)
            eng.Sync()
            ms = ev0.elapsed_time(ev1)
            tok_last, _ = eng.GetCursor()
        except Exception as ex:
            err = ex
    ms, failed = multi.reduce_max([ms, 0.0 if err is None else 1.0], dist, device="cuda")
    if eng is not None:
        eng.close()
    if err is not None:
        raise err
    if failed:
        raise RuntimeError("the tensor-parallel leg failed on another rank")
    bytes_tok = (mc.weight_bytes_per_token(cfg) + mc.kv_bytes_per_position(cfg) * (PROMPT_LEN + steps / 2.0)) / world
    peak, _ = measured_peak_gbs()
    return {"workload": f"{cfg.name}-q8_0 tensor parallel x{world}", "value": steps / (ms / 1e3), "unit": "tok/s",
            "ms_per_step": ms / steps, "scaling": "strong", "steps": steps,
            "exchange": ("none (one GPU)" if world == 1 else
                         "inside the persistent kernel: peer stores of tagged partial sums" if "not used" not in note
                         else note),
            "roofline_frac_per_gpu": bytes_tok * (steps / (ms / 1e3)) / 1e9 / peak, "last_token": int(tok_last)}


def run_seqs_leg(torch, dist, rank, world, local_rank, sequences=16, prompt_len=32, steps=96):
    """Independent TinyLlama-1.1B sequences, sequence i on GPU i mod G, no communication; every
    sequence is decoded with batch-1 semantics (prompt through the decode path).  Strong scaling."""
    from mongoose_b200.fused_infer import CUDAFusedInference
    cfg = SEQ_LEG_CFG.with_(max_seq=prompt_len + steps)
    mine = multi.sequences_for_rank(sequences, rank, world)
    # (guarded sections + unconditional collectives, as in the tensor-parallel leg)
    err, eng, ms, tails = None, None, 0.0, []
    try:
        eng = CUDAFusedInference(cfg, device=local_rank)
        synthetic.load_engine(eng, cfg, seed=0)
        eng.BuildFusedDispatch()
        stream = torch.cuda.ExternalStream(eng.stream, device=local_rank)
        for _ in range(3):
            eng.StepToken(1, 0)
        torch.cuda.synchronize()
    except Exception as ex:
        err = ex
    if dist is not None:
        dist.barrier()
    if err is None:
        try:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record(stream)
            for sidx in mine:
                eng.ResetKV()
                tails.append(int(eng.Generate(synthetic.prompt_ids(sidx, prompt_len, cfg.vocab), steps)[-1]))
            ev1.record(stream)
            torch.cuda.synchronize()
            ms = ev0.elapsed_time(ev1)
        except Exception as ex:
            err = ex
    ms, failed = multi.reduce_max([ms, 0.0 if err is None else 1.0], dist, device="cuda")
    if eng is not None:
        eng.close()
    if err is not None:
        raise err
    if failed:
        raise RuntimeError("the sequences leg failed on another rank")
    tokens_total = sequences * (prompt_len + steps - 1)
    return {"workload": f"tinyllama-1.1b-q8_0, {sequences} sequences x ({prompt_len} prompt + {steps} decode), i mod {world}",
            "value": tokens_total / (ms / 1e3), "unit": "tok/s", "scaling": "strong", "sequences_per_gpu": len(mine),
            "batch": "1 per sequence", "tail": tails[:2]}


def run_sequences_arm(args, cfg, rank, world, local_rank):
    """Independent sequences sharded over the GPUs (sequence i on rank i mod G), no communication.
    A step is one decoded token of one sequence; value counts prompt and generated tokens alike,
    because the prompt goes through the same decode path."""
    import torch
    from mongoose_b200.fused_infer import CUDAFusedInference
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    P, K = args.prompt_len, args.steps
    cfg = cfg.with_(max_seq=P + K)
    eng = CUDAFusedInference(cfg, device=local_rank)
    synthetic.load_engine(eng, cfg, seed=0)
    eng.BuildFusedDispatch()
    mine = multi.sequences_for_rank(args.sequences, rank, world)
    stream = torch.cuda.ExternalStream(eng.stream, device=local_rank)
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        eng.StepToken(1, 0)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sampler.begin()
    launches0 = eng.LaunchCount()
    ev0.record(stream)
    tails = []
    for sidx in mine:
        eng.ResetKV()
        toks = eng.Generate(synthetic.prompt_ids(sidx, P, cfg.vocab), K)
        tails.append(int(toks[-1]))
    ev1.record(stream)
    torch.cuda.synchronize()
    sampler.end()
    if dist is not None:
        dist.barrier()
    clocks = sampler.stop()
    ms_max, = multi.reduce_max([ev0.elapsed_time(ev1)], dist, device="cuda")
    if rank == 0:
        tokens_total = args.sequences * (P + K - 1)
        tps = tokens_total / (ms_max / 1e3)
        per_gpu_seq = len(mine)
        bytes_tok = mc.weight_bytes_per_token(cfg) + mc.kv_bytes_per_position(cfg) * (P + K) / 2.0
        peak, peak_src = measured_peak_gbs()
        achieved = bytes_tok * (per_gpu_seq * (P + K - 1)) / (ms_max / 1e3) / 1e9
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": tps, "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_max / max(1, per_gpu_seq * (P + K - 1)),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": FMT_NAME[cfg.layer_fmt],
            "data": "synthetic",
            "config": {"workload": args.workload, "sequences": args.sequences, "prompt_len": P, "decode_steps": K,
                       "batch": "1 per sequence, sequences sharded i mod G", "l2": "inputs larger than L2"},
            "gpu_launches": int(eng.LaunchCount() - launches0),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": peak_src, "kernel": "whole decode step",
                         "algorithmic_bytes_per_token": bytes_tok},
            "clocks": clocks, "tokens_tail": tails[:4]}), flush=True)
    eng.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# The single-op configuration: one Q8_0 dequant-matvec, W 4864 x 896
# ---------------------------------------------------------------------------
def run_matvec_workload(args):
    """y = W x through the drop-in symbol mongoose_q8_0_matvec (raw 34-byte blocks, caller-owned).
    Two figures: HBM (a ring of 64 distinct copies of W, 296 MB > 2 x L2, so every launch streams
    its weights from DRAM) and L2-hot (the same copy every launch).  A step is one matvec.
    Beside it: the reference's CPU engine semantics (dequantize, naive triple loop, one thread)."""
    import torch
    from mongoose_b200 import kernels as K
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for this path")
    N, Kd, copies = 4864, 896, 64
    blocks, x = synthetic.single_matvec_case(0, N, Kd)
    wbytes = blocks.size
    ring = torch.from_numpy(np.ascontiguousarray(blocks)).cuda().repeat(copies, 1, 1)      # [copies, N, row bytes]
    dx = torch.from_numpy(x).cuda()
    out = torch.empty(N, device="cuda")
    steps, warm = max(args.steps, 64), max(args.warmup, 3)

    # one CUDA graph of `copies` launches (one per ring copy, or all on copy 0), replayed: the host's
    # launch rate (several microseconds per call from Python) stays out of the figure
    side = torch.cuda.Stream()
    K.KQ8_0Matvec(dx, ring[0], out, N, Kd, stream=side)           # first call outside any capture
    side.synchronize()
    graphs = {}
    for hot in (False, True):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(copies):
                K.KQ8_0Matvec(dx, ring[0 if hot else i], out, N, Kd, stream=side)
        graphs[hot] = g

    def timed(n, hot):
        reps = max(1, n // copies)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(reps):
            graphs[hot].replay()
        ev1.record()
        torch.cuda.synchronize()
        return ev0.elapsed_time(ev1) / (reps * copies)

    sampler = ClockSampler(0)
    sampler.start()
    t_up = time.perf_counter()
    while time.perf_counter() - t_up < 0.8:              # warm-up under load while nvidia-smi comes up
        timed(max(warm, 1) * copies, False)
    sampler.begin()
    ms_hbm = timed(steps, False)
    ms_hot = timed(steps, True)
    sampler.end()
    clocks = sampler.stop()
    y = out.cpu().numpy()
    # end to end: host x in, host y out, through the same call
    xh = torch.from_numpy(x).pin_memory()
    yh = torch.empty(N).pin_memory()
    t0 = time.perf_counter()
    for i in range(steps):
        dx.copy_(xh, non_blocking=True)
        K.KQ8_0Matvec(dx, ring[i % copies], out, N, Kd, stream=torch.cuda.current_stream())
        yh.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    peak, peak_src = measured_peak_gbs()
    alg = wbytes + Kd * 4 + N * 4
    line = {"metric": "q8_0_matvec_per_s", "value": 1e3 / ms_hbm, "unit": "matvec/s", "n_gpus": 1, "steps": steps,
            "warmup": warm, "ms_per_step": ms_hbm, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "q8_0", "data": "synthetic",
            "config": {"workload": args.workload, "N": N, "K": Kd, "l2": f"ring of {copies} copies of W ({copies * wbytes >> 20} MB)",
                       "timing": "CUDA events around replays of a CUDA graph of 64 launches"},
            "e2e": {"value": 1e3 / e2e_ms, "unit": "matvec/s", "h2d_bytes_per_step": Kd * 4, "d2h_bytes_per_step": N * 4,
                    "api": "mongoose_q8_0_matvec with pinned host x / y"},
            "gpu_launches": steps,
            "roofline": {"bound": "hbm", "achieved": alg / (ms_hbm * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / (ms_hbm * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": peak_src,
                         "kernel": "raw_block_matvec_kernel", "algorithmic_bytes_per_launch": alg,
                         "l2_hot_GBs": alg / (ms_hot * 1e-3) / 1e9, "l2_hot_us": ms_hot * 1e3},
            "clocks": clocks, "checksum": float(np.abs(y).sum())}
    if not args.no_cpu_baseline:
        from oracle import oracle as O
        O.cpu_engine_matvec(O.FMT_Q8_0, blocks, x, N, Kd, 1)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            O.cpu_engine_matvec(O.FMT_Q8_0, blocks, x, N, Kd, 1)
            reps += 1
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": reps / dt, "unit": "matvec/s", "cores": 1, "kind": "port",
                                "sample": f"{reps} matvecs in {dt:.1f} s: dequantize + the CPU engine's naive loop, one thread"}
    print(json.dumps(line), flush=True)


def main():
    global PROMPT_LEN
    args = parse_args()
    PROMPT_LEN = args.prompt_len
    rank, world, local_rank = multi.rank_env()
    cfg = WORKLOADS[args.workload]
    if args.workload == "q8_0-matvec-4864x896":
        if rank == 0 and args.impl != "reference":
            run_matvec_workload(args)
        elif rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the single-op workload times its CPU side inside the main arm (cpu_baseline)"}))
        return
    if args.impl == "reference":
        run_reference_arm(args, cfg, rank)
        return
    if args.workload.endswith("-seqs"):
        run_sequences_arm(args, cfg, rank, world, local_rank)
        return
    run_b200_arm(args, cfg, rank, world, local_rank)


def _one_line_stdout():
    """Libraries (NCCL's version banner, for one) write to file descriptor 1.  The contract is ONE
    JSON line on stdout, so everything written to fd 1 while the benchmark runs goes to stderr and
    only what this module prints through `print` reaches the real stdout."""
    sys.stdout.flush()
    real = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real, "w", buffering=1)


if __name__ == "__main__":
    _one_line_stdout()
    main()
