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


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shape", default="QWEN25_3B", help="name of a shape in taraference_b200.synth")
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--prompt", type=int, default=32, help="positions in the cache before the recorded step")
    args = ap.parse_args()
    from . import synth as S, synth_gpu
    cfg = dict(getattr(S, args.shape), n_layer=args.layers)
    model, _ = synth_gpu.build_model(cfg, seed=0)
    kv = model.alloc_kv(max(4096, args.prompt + 64))
    rng = np.random.default_rng(0)
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
