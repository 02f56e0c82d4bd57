#!/usr/bin/env python
"""Batch-1 greedy decode benchmark on the Qwen2.5-3B-shaped Q4_K_M model (BASELINE configuration 2).

One step = one pass of the hot path over one batch of synthetic input: starting from a
32-token prompt already in the KV cache, decode 256 tokens greedily with the on-device
token loop.  Weights are random N(0, 0.02) quantised on the device (no model files are
available); norm weights are ones; ctx 4096.  `value` is tokens per second with everything
resident in HBM (CUDA events around the kernels); `e2e` is the same count of tokens over
the wall-clock time of the C-ABI call that takes its scalars from host memory and returns
the tokens to host memory.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

N > 1 runs N independent replicas (one process per GPU under torchrun): the decode loop
of this model has no unit to shard without a per-layer exchange, which costs more than a
layer's HBM time at this size.  `--impl reference` times the CPU restatement of the
reference algorithm (the reference has no CPU path of its own for these kernels) on all
host cores, on a bounded sample of the same workload.

`--workload` selects one of the other BASELINE configurations instead (same JSON line, other
`config.workload`): `3b-long` (16384-token prompt, ctx 32768, 512 decoded tokens), `hybrid-4b`
(Gated-DeltaNet hybrid, 64-token prompt), `32b-tp` (Qwen2.5-32B shape, 128-token prompt; under
torchrun the N ranks form ONE tensor-parallel engine: strong scaling, the value is not
multiplied by N).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN, N_DECODE, CTX = 32, 256, 4096
# name -> (config attribute of taraference_b200.synth, prompt tokens, decoded tokens per step, ctx, description)
WORKLOADS = {
    "3b": ("QWEN25_3B", 32, 256, 4096,
           "qwen2.5-3b-shape Q4_K_M, batch-1 greedy decode, 32-token prompt, 256 decoded tokens per step, ctx 4096 "
           "(BASELINE configuration 2)"),
    "3b-long": ("QWEN25_3B", 16384, 512, 32768,
                "qwen2.5-3b-shape Q4_K_M, long-context flash-decode: 16384-token prompt in the fp16 KV cache, 512 decoded "
                "tokens per step at positions 16384..16895, ctx 32768 (BASELINE configuration 3)"),
    "3b-prompt": ("QWEN25_3B", 2048, 64, 4096,
                  "qwen2.5-3b-shape Q4_K_M, 2048-token prompt through the chunk kernels (the `prefill` object), then 64 "
                  "decoded tokens per step at positions 2048..2111"),
    "hybrid-4b": ("QWEN35_4B", 64, 256, 4096,
                  "qwen3.5-4b-style hybrid Q4_K_M (3 Gated-DeltaNet layers : 1 gated full-attention layer), 64-token prompt, "
                  "256 decoded tokens per step (BASELINE configuration 4)"),
    "32b-tp": ("QWEN25_32B", 128, 256, 4096,
               "qwen2.5-32b-shape Q4_K_M, tensor-parallel over the ranks of the job, 128-token prompt, 256 decoded tokens "
               "per step (BASELINE configuration 5)"),
}
METRIC, UNIT = "batch1_decode_tokens_per_s", "tok/s"
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one gate+up launch, from the ncu capture
# summarised in profiles/ffn_gate_up_qwen25_3b.md
GATE_UP_DRAM_TRAFFIC_BYTES = 25437184


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle samples taken while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def aggregate_over_ranks(dev_ms_total: float, wall_s_total: float, tokens_per_rank: int, world: int, dist=None,
                         device="cpu"):
    """Whole-job numbers from per-rank timings: every rank decodes `tokens_per_rank` tokens on its own
    replica; the job takes as long as its slowest rank (MAX over ranks), and the value counts all tokens."""
    import torch
    if world > 1:
        t = torch.tensor([dev_ms_total, wall_s_total], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms_total, wall_s_total = float(t[0]), float(t[1])
    tokens_all = tokens_per_rank * world
    return {"value": tokens_all / (dev_ms_total / 1000.0), "e2e": tokens_all / wall_s_total,
            "dev_ms": dev_ms_total, "wall_s": wall_s_total, "tokens": tokens_all}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def cpu_port_tokens_per_s(host_tensors, cfg, prompt, first, n_tokens: int, threads: int):
    """Times the CPU restatement (oracle/) on n_tokens decode steps after the prompt.  Checker code
    used as a reported baseline only."""
    from oracle import oracle as O
    O.set_threads(threads)
    om = O.OracleModel(cfg, host_tensors, PROMPT_LEN + n_tokens + 1)
    # fill the prompt rows of the cache cheaply: only what attention needs, one pass per token
    for i, t in enumerate(prompt):
        om.decode_token(i, int(t))
    t0 = time.perf_counter()
    om.decode_greedy(PROMPT_LEN, int(first), n_tokens)
    dt = time.perf_counter() - t0
    O.set_threads(1)
    return n_tokens / dt, dt


def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference algorithm on the host cores (CPU restatement)."""
    if rank != 0:
        return
    from oracle import oracle as O
    from taraference_b200 import synth as S  # numpy only: this process never maps the CUDA library
    cfg = dict(S.QWEN25_3B)
    threads = O.max_threads()
    # same tensor plan, quantisation mix and block value distributions as the GPU arm; the bytes come from numpy
    # (the time of a CPU pass over the weights does not depend on their values)
    host = S.random_model(cfg, seed=0)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg["n_vocab"], PROMPT_LEN)
    O.set_threads(threads)
    om = O.OracleModel(cfg, host, CTX)
    sample = 2  # tokens per step: a bounded sample of the 256-token workload
    pos = 0
    for t in prompt:  # the workload's whole prompt goes into the cache first, one decode step per token
        om.decode_token(pos, int(t))
        pos += 1
    tok = int(prompt[-1])
    times = []
    for step in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        toks, _, _ = om.decode_greedy(pos, tok, sample)
        dt = time.perf_counter() - t0
        pos += sample
        tok = int(toks[-1])
        if step >= args.warmup:
            times.append(dt)
    total = float(np.sum(times))
    value = sample * len(times) / total
    covered = sample * (args.warmup + args.steps)
    loaded = sorted({ln.split()[-1].split("/")[-1] for ln in open("/proc/self/maps") if ln.rstrip().endswith(".so") and
                     ("oracle" in ln or "tarafer" in ln)})
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000 * total / len(times),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
            "data": "synthetic",
            "config": {"workload": "qwen2.5-3b-shape Q4_K_M batch-1 greedy decode, CPU restatement of the reference "
                                   "kernels' arithmetic (the reference has no CPU implementation of this path)",
                       "prompt_tokens": PROMPT_LEN, "decode_tokens_per_step": sample,
                       "tokens_covered": f"positions {PROMPT_LEN}..{PROMPT_LEN + covered - 1}: the first {covered} of the "
                                         f"workload's {N_DECODE} decoded tokens ({len(times) * sample} of them timed)"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"{sample} decode tokens per step, {len(times)} timed steps after a {PROMPT_LEN}-token "
                                       f"prompt ({covered} of the workload's {N_DECODE} decoded tokens), OpenMP over {threads} threads"},
            "native_so_loaded": loaded,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def reference_kernels_on_gpu(cfg, host, prompt_len: int):
    """The reference's own kernels (compiled unmodified, its launch shapes) replayed from a CUDA graph of
    one decode step at a mid-run position: what its token costs on this GPU without its host loop."""
    import torch
    try:
        from oracle import ref_gpu
        if not ref_gpu.available():
            return None
        rm = ref_gpu.RefModel(cfg, host, prompt_len + N_DECODE + 1)
        pos = prompt_len + N_DECODE // 2
        rm.decode_token(pos, 17)  # warm-up, loads modules
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        before = ref_gpu.kernels().launches
        with torch.cuda.graph(g):
            rm.decode_token(pos, 17)
        nodes = ref_gpu.kernels().launches - before
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        reps = 32
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1000 / reps
        return {"us_per_token": us, "tokens_per_s": 1e6 / us, "kernel_nodes": nodes,
                "note": "reference .cu compiled unmodified with its NVRTC options for sm_100, its launch shapes, one "
                        "CUDA graph per token, no argmax readback"}
    except Exception as exc:  # the comparison is informative; never fail the bench for it
        return {"error": repr(exc)[:200]}


def gate_up_roofline(E, S, cfg, peak_gbs, peak_kind):
    """Average duration of the fused gate+up kernel (the largest per-layer read) over distinct weight
    sets that together exceed L2, with CUDA events on the launching stream."""
    import torch
    from taraference_b200 import synth_gpu
    K, FF = cfg["n_embd"], cfg["n_ff"]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(123)
    sets = []
    for _ in range(10):  # 10 x 25.4 MB = 254 MB > 126 MB L2
        g = synth_gpu.quantized_matrix(S.Q4_K, K, FF, gen)
        u = synth_gpu.quantized_matrix(S.Q4_K, K, FF, gen)
        sets.append((E.GpuMat(S.Q4_K, K, FF, g), E.GpuMat(S.Q4_K, K, FF, u)))
        del g, u
    x = torch.randn(K, device="cuda")
    nw = torch.ones(K, device="cuda")
    h = torch.zeros(FF, device="cuda")
    for mg, mu in sets:
        E.op_ffn_gate_up(mg, mu, x, h, nw, 1e-6)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rounds = 20
    a.record()
    for _ in range(rounds):
        for mg, mu in sets:
            E.op_ffn_gate_up(mg, mu, x, h, nw, 1e-6)
    b.record()
    torch.cuda.synchronize()
    us = a.elapsed_time(b) * 1000 / (rounds * len(sets))
    alg = 2 * FF * (K // 256) * 144 + 2 * K * 4 + FF * 4  # both matrices + x + norm weights + h
    for mg, mu in sets:
        mg.free(), mu.free()
    ach = alg / us * 1e-3
    return {"bound": "hbm", "kernel": "k_gemv<BlockQ4,EpiSilu> (RMSNorm+Q8+gate/up+SiLU*mul, 11008x2048 Q4_K x2)",
            "achieved": ach, "peak": peak_gbs, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": ach / peak_gbs,
            "traffic": GATE_UP_DRAM_TRAFFIC_BYTES, "algorithmic_bytes_per_launch": alg, "us_per_launch": us,
            "note": "back-to-back launches on one stream: includes the launch gap"}


def attention_roofline(E, cfg, n_keys, peak_gbs, peak_kind):
    """Stand-alone split-KV attention at n_keys keys: CUDA events over 120 launches that rotate through 12 K/V buffer
    pairs (more than L2 holds), and the reference's attn_flash_partial + attn_flash_reduce on the same cache."""
    import torch
    H, Hkv, hd = cfg["n_head"], cfg["n_kv"], cfg["head_dim"]
    rng = np.random.default_rng(0)
    base_k = rng.normal(0, 1, (n_keys + 8, Hkv * hd)).astype(np.float16).view(np.int16)
    base_v = rng.normal(0, 1, (n_keys + 8, Hkv * hd)).astype(np.float16).view(np.int16)
    nbuf = 12
    kcs = [torch.from_numpy(base_k).cuda().clone() for _ in range(nbuf)]
    vcs = [torch.from_numpy(base_v).cuda().clone() for _ in range(nbuf)]
    q = torch.randn(H * hd, device="cuda")
    out = torch.zeros(H * hd, device="cuda")

    def timed(fn, reps=120):
        for i in range(nbuf):
            fn(i)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for r in range(reps):
            fn(r % nbuf)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1000 / reps

    us = timed(lambda i: E.op_attention(q, kcs[i], vcs[i], out, H, Hkv, hd, n_keys - 1))
    ref_us = None
    try:
        from oracle import ref_gpu
        if ref_gpu.available():
            ref_us = timed(lambda i: ref_gpu.attention(q, kcs[i], vcs[i], H, Hkv, hd, n_keys - 1), reps=36)
    except Exception:  # the comparison is informative only
        ref_us = None
    alg = 2 * n_keys * Hkv * hd * 2 + 2 * H * hd * 4  # K and V rows once, q in, out
    ach = alg / us * 1e-3
    return {"bound": "hbm", "kernel": f"k_attn_decode<{hd}> (split-KV flash-decode, {n_keys} keys, {H} query / {Hkv} KV heads)",
            "achieved": ach, "peak": peak_gbs, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": ach / peak_gbs,
            "traffic": None, "algorithmic_bytes_per_launch": alg, "us_per_launch": us,
            "reference_attn_flash_us_per_launch": ref_us,
            "note": "back-to-back launches on one stream over 12 rotating K/V buffers (208 MB); includes the launch gap; the "
                    "reference figure is its attn_flash_partial + attn_flash_reduce launched through the driver API"}


def tensor_parallel_32b(rank, world, local, dist, steps: int = 8, warmup: int = 3):
    """BASELINE configuration 5 as a side measurement of the default run: the Qwen2.5-32B shape with the
    job's ranks as ONE tensor-parallel engine (a single GPU at N = 1).  All ranks call this."""
    import torch
    from taraference_b200 import synth as S, synth_gpu
    cfg_name, prompt_len, n_decode, ctx, text = WORKLOADS["32b-tp"]
    cfg = dict(getattr(S, cfg_name))
    t_build = time.perf_counter()
    build_cfg = dict(cfg, tp_rank=rank, tp_size=world) if world > 1 else cfg
    model, _ = synth_gpu.build_model(build_cfg, seed=0, device=local, context_length=ctx)
    if world > 1:
        from taraference_b200 import tp as TP
        TP.connect(model, dist)
    kv = model.alloc_kv(ctx)
    t_build = time.perf_counter() - t_build
    prompt = np.random.default_rng(0).integers(0, cfg["n_vocab"], prompt_len)
    first = model.forward_greedy(prompt, kv)
    last_tokens = []

    def timed_us_per_token():
        dev = []
        for i in range(warmup + steps):
            kv.len = prompt_len
            if world > 1:
                dist.barrier()
            toks = model.decode_burst(first, n_decode, kv)
            assert len(toks) == n_decode
            last_tokens[:] = [int(t) for t in toks]
            if i >= warmup:
                dev.append(model.last_device_ms())
        total = float(np.sum(dev))
        if world > 1:
            t = torch.tensor([total], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total = float(t[0])
        return total * 1000 / (n_decode * steps)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    us = timed_us_per_token()
    clocks = sampler.stop() if rank == 0 else None
    tp_tokens = list(last_tokens)
    # every rank must have emitted the same tokens
    ranks_agree = True
    if world > 1:
        mine = torch.tensor([first] + tp_tokens, dtype=torch.int64, device="cuda")
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        ranks_agree = all(bool(torch.equal(everyone[0], t)) for t in everyone)
    nccl = None
    if world > 1:
        # comparison baseline: the same engine with ncclAllReduce between kernels instead of the in-kernel exchange
        try:
            TP.use_nccl(model, dist)
            us_nccl = timed_us_per_token()
            nccl = {"tokens_per_s": 1e6 / us_nccl, "us_per_token": us_nccl,
                    "what": "row-parallel partial sums and the argmax through ncclAllReduce nodes in the same CUDA graph"}
        except Exception as exc:  # the baseline is informative only
            nccl = {"error": repr(exc)[:200]}
    kv.free()
    model.destroy()
    # the same bytes on ONE GPU (rank 0), fed the tensor-parallel engine's own tokens: its greedy choice must be the
    # token the tensor-parallel engine emitted wherever its top-2 margin is not small.  "Small" is set by what two
    # correct implementations show at this depth: after 36 layers the reference's own two FFN kernels move the logits
    # by 4.7e-2 of the largest logit (tests/test_engine_gpu.py, full-depth test), so a margin below 0.2 of the largest
    # logit decides nothing at 64 layers.
    check = {"ranks_agree": ranks_agree, "compared_with_one_gpu": 0, "equal": 0, "mismatches_within_margin": 0,
             "mismatches_beyond_margin": 0, "margin_gate": "0.2 x largest logit of the position"}
    if world > 1:
        n_cmp = 48
        counts = [0, 0, 0]
        if rank == 0:
            single, _ = synth_gpu.build_model(cfg, seed=0, device=local, context_length=ctx)
            kv1 = single.alloc_kv(ctx)
            single.forward_greedy(prompt, kv1)
            fed = [int(first)] + tp_tokens[:n_cmp - 1]
            for i, t in enumerate(fed):
                nxt = single.forward_greedy([t], kv1)
                if nxt == tp_tokens[i]:
                    counts[0] += 1
                    continue
                lg = single.current_logits()
                top = np.sort(lg)[-2:]
                counts[1 if float(top[1] - top[0]) <= 0.2 * float(np.abs(lg).max()) else 2] += 1
            kv1.free()
            single.destroy()
        flag = torch.tensor(counts, dtype=torch.int64, device="cuda")
        dist.broadcast(flag, src=0)
        check["compared_with_one_gpu"] = n_cmp
        check["equal"], check["mismatches_within_margin"], check["mismatches_beyond_margin"] = (int(v) for v in flag)
    tokens_match = bool(check["ranks_agree"] and check["mismatches_beyond_margin"] == 0)
    wbytes = synth_gpu.weight_bytes(cfg) + synth_gpu.kv_bytes_per_position(cfg) * (prompt_len + n_decode / 2)
    return {"workload": text, "parallelism": f"tp{world}" if world > 1 else "single GPU", "scaling": "strong",
            "tokens_per_s": 1e6 / us, "us_per_token": us, "steps": steps, "warmup": warmup,
            "tokens_match": tokens_match, "tokens_check": check, "clocks": clocks,
            "aggregate_weight_kv_gbs": wbytes / us * 1e-3, "build_s": t_build, "nccl_allreduce_baseline": nccl,
            "timing": "CUDA events around each 256-token burst, max over ranks"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-reference-gpu", action="store_true")
    ap.add_argument("--workload", default="3b", choices=sorted(WORKLOADS))
    ap.add_argument("--skip-32b", action="store_true",
                    help="default workload only: leave out the 32B-shape tensor-parallel side measurement")
    ap.add_argument("--share-of", type=int, default=1,
                    help="32b-tp workload on ONE GPU: run the slice of the model a rank of an N-way tensor-parallel engine holds "
                         "(heads, FFN rows and vocabulary divided by N) as an ordinary engine, i.e. a rank's work without any "
                         "exchange; the difference to the tensor-parallel figure at N ranks is what the exchange costs")
    ap.add_argument("--roofline-only", action="store_true",
                    help="time only the fused gate+up kernel over 254 MB of weights (the small case used for ncu)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode library has no CPU fallback")
    from taraference_b200 import engine as E, synth as S, synth_gpu
    if args.roofline_only:
        peak, peak_kind = measured_peaks()
        torch.cuda.set_device(local)
        print(json.dumps({"roofline": gate_up_roofline(E, S, dict(S.QWEN25_3B), peak, peak_kind)}), flush=True)
        return
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    warmup = max(args.warmup, 3)
    cfg_name, PROMPT_LEN, N_DECODE, CTX, workload_text = WORKLOADS[args.workload]
    cfg = dict(getattr(S, cfg_name))
    if args.share_of > 1:
        if args.workload != "32b-tp" or world != 1:
            raise SystemExit("--share-of applies to --workload 32b-tp on one GPU")
        n = args.share_of
        blocks = (cfg["n_ff"] // 256 + n - 1) // n  # the larger FFN slice of the plan (e.g. 14 of 13/14 blocks at n = 8)
        heads = cfg["n_head"] // n
        heads += heads % 2  # the stand-alone engine wants whole 256-element blocks of attention width (128-wide heads in pairs)
        cfg.update(n_head=heads, n_kv=max(1, cfg["n_kv"] // n), n_ff=256 * blocks,
                   n_vocab=(cfg["n_vocab"] // n + 1) // 2 * 2)
        workload_text += f" -- the 1/{n} slice of one rank, run alone on one GPU without exchange"
    tp = world if args.workload == "32b-tp" else 1   # the ranks form one engine instead of N replicas
    main_workload = args.workload == "3b"
    want_host = main_workload and rank == 0 and world == 1 and not (args.skip_cpu_baseline and args.skip_reference_gpu)
    build_cfg = dict(cfg, tp_rank=rank, tp_size=tp) if tp > 1 else cfg
    model, host = synth_gpu.build_model(build_cfg, seed=0, device=local, context_length=CTX, keep_host=want_host)
    if tp > 1:
        from taraference_b200 import tp as TP
        TP.connect(model, dist)
    kv = model.alloc_kv(CTX)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg["n_vocab"], PROMPT_LEN)
    first = model.forward_greedy(prompt, kv)  # prefill once; every step restarts from this cache state
    prefill = {"tokens": int(PROMPT_LEN), "device_ms": model.last_device_ms(),
               "tokens_per_s": PROMPT_LEN / max(model.last_device_ms(), 1e-9) * 1e3, "chunk_tokens": model.prefill_chunk(),
               "what": "tfr_forward_greedy over the whole prompt: chunks of chunk_tokens through the batched kernels "
                       "(0: one decode step per token), the last token as a decode step with the head"}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step():
        # every step restarts at the end of the prompt; a hybrid model's recurrent state simply carries on
        # (its cost does not depend on the content)
        kv.len = PROMPT_LEN
        t0 = time.perf_counter()
        toks = model.decode_burst(first, N_DECODE, kv)
        wall = time.perf_counter() - t0
        assert len(toks) == N_DECODE
        return model.last_device_ms(), wall, toks

    for _ in range(warmup):
        one_step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    launches0 = model.launch_count()
    dev_ms, walls = [], []
    t_all = time.perf_counter()
    for _ in range(args.steps):
        d, w, toks = one_step()
        dev_ms.append(d)
        walls.append(w)
    barrier()
    wall_all = time.perf_counter() - t_all
    clocks = sampler.stop() if rank == 0 else None
    launches = model.launch_count() - launches0
    agg = aggregate_over_ranks(float(np.sum(dev_ms)), float(np.sum(walls)), N_DECODE * args.steps, world,
                               dist if world > 1 else None, "cuda")
    if tp > 1:  # one engine: every rank emitted the same tokens
        agg["value"], agg["e2e"], agg["tokens"] = agg["value"] / world, agg["e2e"] / world, agg["tokens"] // world
    dev_total, wall_total, value, e2e_value = agg["dev_ms"], agg["wall_s"], agg["value"], agg["e2e"]

    # per-token host round-trip through forward_greedy (the reference's call pattern), rank 0 only
    per_token_api = None
    if tp > 1 or rank == 0:  # a tensor-parallel engine needs every rank in every call
        kv.len = PROMPT_LEN
        t, t0 = first, time.perf_counter()
        for _ in range(64):
            t = model.forward_greedy([t], kv)
        per_token_api = 64 / (time.perf_counter() - t0)

    verify = None
    if main_workload and rank == 0 and tp == 1:
        # one-pass verification batch (forward_greedy_all, 9 tokens as the reference's MAX_VERIFY_TOKENS)
        vt = [int(t) for t in rng.integers(0, cfg["n_vocab"], 9)]
        kv.len = PROMPT_LEN
        model.forward_greedy_all(vt, kv)
        kv.len = PROMPT_LEN
        model.forward_greedy_all(vt, kv)
        v_us = model.last_device_ms() * 1000
        step_us = float(np.sum(dev_ms)) * 1000 / (N_DECODE * args.steps)
        verify = {"tokens": 9, "device_us": v_us, "decode_steps_equivalent": v_us / step_us, "chunk_tokens": model.prefill_chunk()}
    attn_roof = None
    if args.workload == "3b-long" and rank == 0:
        peak_a, kind_a = measured_peaks()
        attn_roof = attention_roofline(E, cfg, PROMPT_LEN + N_DECODE, peak_a, kind_a)
    tp32 = None
    if main_workload and not args.skip_32b:
        kv.free()
        model.destroy()
        kv = model = None
        tp32 = tensor_parallel_32b(rank, world, local, dist if world > 1 else None, steps=max(args.steps, 1))
    if rank == 0:
        peak, peak_kind = measured_peaks()
        wbytes = synth_gpu.weight_bytes(cfg)
        kvb = synth_gpu.kv_bytes_per_position(cfg)
        bytes_per_token = wbytes + kvb * (PROMPT_LEN + N_DECODE / 2) + synth_gpu.recurrent_state_bytes(cfg)
        us_tok = dev_total * 1000 / (N_DECODE * args.steps)
        token_gbs = bytes_per_token / us_tok * 1e-3
        roof = gate_up_roofline(E, S, dict(S.QWEN25_3B), peak, peak_kind) if main_workload else attn_roof
        cpu = None
        if want_host and not args.skip_cpu_baseline:
            from oracle import oracle as O
            th = O.max_threads()
            v, dt = cpu_port_tokens_per_s(host, cfg, prompt[:4], int(prompt[4]), 4, th)
            cpu = {"value": v, "unit": UNIT, "cores": th, "kind": "port",
                   "sample": f"4 decode tokens after a 4-token prefix ({dt:.1f} s), OpenMP over {th} threads"}
        ref_gpu_info = None
        if want_host and not args.skip_reference_gpu:
            ref_gpu_info = reference_kernels_on_gpu(cfg, host, PROMPT_LEN)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": dev_total / args.steps, "higher_is_better": True, "scaling": "strong" if tp > 1 else "weak",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": workload_text,
                       "weights": "N(0,0.02) quantised on device; Q6_K token_embd/attn_v/ffn_down, Q4_K elsewhere",
                       "l2": f"each token streams {wbytes / 1e9:.2f} GB of weights, far beyond the 126 MB L2",
                       "parallelism": f"tp{tp} (in-kernel all-reduce over NVLink peer memory)" if tp > 1 else
                                      ("replicas" if world > 1 else "single GPU"),
                       "timing": "CUDA events on the engine's stream around each 256-token burst; max over ranks"},
            "us_per_token": us_tok,
            "token_roofline": {"bytes_per_token": bytes_per_token, "achieved_gbs": token_gbs,
                               "frac_of_8TBs_nominal": token_gbs / NOMINAL_HBM_GBS,
                               f"frac_of_{peak_kind}_copy_peak": token_gbs / peak, "peak_gbs": peak},
            "roofline": roof, "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 64, "d2h_bytes_per_step": 4 * N_DECODE + 96,
                    "call": "tfr_decode_burst: scalars from pinned host memory, tokens back to host memory",
                    "per_token_forward_greedy_tok_s": per_token_api},
            "gpu_launches": int(launches), "clocks": clocks, "reference_kernels_same_gpu": ref_gpu_info,
            "wall_s_timed_region": wall_all, "prefill": prefill, "verify_batch": verify, "tensor_parallel_32b": tp32,
        }
        print(json.dumps(line), flush=True)
    if model is not None:
        kv.free()
        model.destroy()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
