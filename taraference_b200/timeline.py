"""In-kernel timeline of one decode step (profiling aid).

Thread 0 of every CTA of the matrix-vector and attention kernels stores the GPU's nanosecond timer at
fixed points when a buffer is registered with tfr_debug_set_timeline.  This module runs a few layers of
a model shape, records one step and prints, per kernel of the step, the earliest and latest time over
the CTAs at which each point was passed:

    python -m taraference_b200.timeline --layers 3 --prompt 32

Columns of the matrix-vector kernels: kernel entry | weight tiles requested | grid-dependency wait
returned | activation vector in shared memory | RMSNorm done | Q8 quantisation done | block dots done
(after the CTA barrier) | epilogue done.  Attention kernels: entry | wait returned | q loaded | scores
of the last tile | softmax of the last tile | value phase done | cluster merge midpoint | done.
The timer ticks every 256 ns or finer depending on the GPU; read differences of a microsecond or more.

    python -m taraference_b200.timeline --path loop --layers 12 --prompt 32

records the persistent decode loop instead (one cooperative kernel for the whole burst): thread 0 of every CTA marks
14 points per layer of one decode step in the middle of a burst — layer start, then for each of the four matrix-vector
phases "activation quantised" and "dots, row sums and epilogue done", the grid barrier after each phase, and the
attention phase — and the table gives the earliest and latest CTA per point, relative to the layer's start.
"""
from __future__ import annotations

import argparse

import numpy as np

GEMV_POINTS = (0, 1, 3, 2, 6, 7, 4, 5)
ATTN_POINTS = (0, 1, 4, 6, 7, 2, 3, 5)
SLOTS = 160  # CTAs per launch the probe has room for


def record(model, kv, token: int, n_launches: int):
    """One decode step with the probe on; returns times [launch][cta][point] in ns (0 = not passed)."""
    import torch

    from . import _lib
    lib = _lib.lib()
    buf = torch.zeros(n_launches * SLOTS * 8, dtype=torch.int64, device="cuda")
    lib.tfr_debug_set_timeline(buf.data_ptr())
    try:
        for _ in range(3):  # the last repetition is the warm one that is reported
            buf.zero_()
            torch.cuda.synchronize()
            model.forward_greedy([token], kv)
            torch.cuda.synchronize()
            kv.len = kv.len - 1
    finally:
        lib.tfr_debug_set_timeline(0)
    return buf.cpu().numpy().reshape(n_launches, SLOTS, 8).astype(np.float64)


def render(times, attention_launches=()) -> str:
    t0 = times[times > 0].min()
    lines = []
    for k in range(times.shape[0]):
        t = times[k]
        if not (t > 0).any():
            continue
        cols = []
        for p in (ATTN_POINTS if k in attention_launches else GEMV_POINTS):
            v = t[:, p][t[:, p] > 0]
            cols.append(f"{(v.min() - t0) / 1000:7.2f}/{(v.max() - t0) / 1000:7.2f}" if len(v) else "       -       ")
        lines.append(f"{k:3d} {'attn' if k in attention_launches else 'gemv'} " + " | ".join(cols))
    return "\n".join(lines)


LOOP_POINTS = ("start", "qkv act", "qkv gemv", "barrier", "attention", "barrier(s)", "o act", "o gemv", "barrier", "gate/up act",
               "gate/up gemv", "barrier", "down act", "down gemv")


def record_loop(model, kv, first: int, layers: int, burst: int):
    """A burst through the persistent loop with the probe on its middle step; times [point][cta] in ns."""
    import torch
    pts = len(LOOP_POINTS) * layers + 3
    buf = torch.zeros(pts * model.sm_count, dtype=torch.int64, device="cuda")
    start = kv.len
    model.decode_burst(first, burst, kv)  # warm
    kv.len = start
    model.set_loop_timeline(buf, burst // 2, pts)
    try:
        model.decode_burst(first, burst, kv)
    finally:
        model.set_loop_timeline(None, -1, 0)
    us_per_token = model.last_device_ms() * 1000 / burst
    return buf.cpu().numpy().reshape(pts, model.sm_count).astype(np.float64), us_per_token


def render_loop(t, layers: int) -> str:
    n = len(LOOP_POINTS)
    lines = []
    for li in sorted({min(1, layers - 1), layers - 1}):
        base = t[n * li].min()
        lines.append(f"layer {li}: microseconds from the layer's first mark, earliest / latest CTA")
        for k, name in enumerate(LOOP_POINTS):
            row = t[n * li + k]
            lines.append(f"   {name:14s} {(row.min() - base) / 1e3:7.2f} {(row.max() - base) / 1e3:7.2f}")
        nxt = t[n * (li + 1)]
        lines.append(f"   {'layer end':14s} {(nxt.min() - base) / 1e3:7.2f} {(nxt.max() - base) / 1e3:7.2f}")
    hb = t[n * layers].min()
    for k, name in enumerate(("head start", "head done", "step barrier")):
        row = t[n * layers + k]
        lines.append(f"   {name:14s} {(row.min() - hb) / 1e3:7.2f} {(row.max() - hb) / 1e3:7.2f}")
    lines.append(f"   step total {(t[n * layers + 2].max() - t[0].min()) / 1e3:.1f} us")
    return "\n".join(lines)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shape", default="QWEN25_3B", help="name of a shape in taraference_b200.synth")
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--prompt", type=int, default=32, help="positions in the cache before the recorded step")
    ap.add_argument("--path", default="chained", choices=["chained", "loop"], help="chained kernels or the persistent loop")
    ap.add_argument("--burst", type=int, default=64, help="loop path: decode steps of the recorded burst")
    args = ap.parse_args()
    from . import _lib
    _lib.use_aids_build()  # the probes are compiled into the instrumented build only
    from . import synth as S, synth_gpu
    cfg = dict(getattr(S, args.shape), n_layer=args.layers)
    model, _ = synth_gpu.build_model(cfg, seed=0)
    kv = model.alloc_kv(max(4096, args.prompt + 64))
    rng = np.random.default_rng(0)
    if args.path == "loop":
        model.set_decode_path(model.PATH_LOOP)
        tok = model.forward_greedy(rng.integers(0, cfg["n_vocab"], args.prompt), kv)
        t, us = record_loop(model, kv, tok, args.layers, args.burst)
        print(f"{args.shape}, {args.layers} layers, persistent loop, {args.burst}-step burst from position {args.prompt}: "
              f"{us:.1f} us per token")
        print(render_loop(t, args.layers))
        kv.free()
        model.destroy()
        return
    tok = model.forward_greedy(rng.integers(0, cfg["n_vocab"], args.prompt), kv)
    tok = int(model.decode_burst(tok, 8, kv)[-1])
    n_launches = (8 if S.is_hybrid(cfg) else 5) * args.layers + 4
    times = record(model, kv, tok, n_launches)
    attn = tuple(range(1, n_launches, 5)) if not S.is_hybrid(cfg) else ()
    print(f"{args.shape}, {args.layers} layers, position {kv.len}: min/max over CTAs in microseconds")
    print(render(times, attn))
    kv.free()
    model.destroy()


if __name__ == "__main__":
    main()
