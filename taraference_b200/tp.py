"""Host-side plumbing of tensor parallelism: one process per GPU, torch.distributed as the
side channel.  The data path never goes through it: the ranks' kernels exchange partial sums
through NVLink peer memory by themselves (csrc/tfr_tp.cuh); this module only hands the 64-byte
CUDA IPC handles of the exchange buffers around once, and merges logits for callers that ask.

The split itself (which rows / K blocks a rank keeps) is decided inside the library from
tp_rank / tp_size; shard_plan mirrors that arithmetic for planning and for the tests.
"""
from __future__ import annotations

import numpy as np


def shard_plan(cfg: dict, rank: int, tp: int) -> dict:
    """The slice of a dense model that rank `rank` of `tp` keeps (mirrors TpPlan in csrc/tfr_engine.cu).

    Q/K/V rows go with whole heads (a KV head stays with the query heads it serves); the FFN
    width is cut on 256-element block borders, unevenly when the block count does not divide;
    attn_output keeps the K blocks that cover the rank's heads (a border block is shared with
    the neighbour: the rank's activation is zero outside its own heads); the vocabulary head
    is cut by rows."""
    H, Hkv, hd, FF, V = (cfg[k] for k in ("n_head", "n_kv", "head_dim", "n_ff", "n_vocab"))
    if tp < 1 or not 0 <= rank < tp:
        raise ValueError("bad rank / tp")
    if H % tp or Hkv % tp:
        raise ValueError(f"tp={tp} does not divide {H} query / {Hkv} KV heads")
    if FF // 256 < tp:
        raise ValueError("FFN narrower than one block per rank")
    nq, nkv = H // tp * hd, Hkv // tp * hd
    q_lo = rank * nq
    b0, b1 = q_lo // 256, (q_lo + nq + 255) // 256
    nbf = FF // 256
    f0, f1 = nbf * rank // tp, nbf * (rank + 1) // tp
    return dict(q_rows=(q_lo, q_lo + nq), kv_rows=(rank * nkv, rank * nkv + nkv), wo_blocks=(b0, b1),
                attn_offset=q_lo - b0 * 256, attn_width=(b1 - b0) * 256, ff_rows=(f0 * 256, f1 * 256),
                ff_blocks=(f0, f1), vocab_rows=(V * rank // tp, V * (rank + 1) // tp))


def connect(model, dist) -> None:
    """All ranks call this after finalize_load: gathers the exchange-buffer handles in rank order
    and maps the peers.  `dist` is an initialised torch.distributed (any backend)."""
    handles = [None] * dist.get_world_size()
    dist.all_gather_object(handles, model.tp_ipc_handle())
    model.tp_attach_ipc(handles)
    dist.barrier()


def use_nccl(model, dist, on: bool = True) -> None:
    """Comparison baseline for measurements: the same engine with ncclAllReduce between kernels instead
    of the in-kernel exchange.  All ranks call this."""
    from . import engine as E
    if not on:
        model.tp_use_nccl(None)
        return
    box = [E.nccl_unique_id() if dist.get_rank() == 0 else None]
    dist.broadcast_object_list(box, src=0)
    model.tp_use_nccl(box[0])
    dist.barrier()


def gather_logits(model, dist) -> np.ndarray:
    """Full logits on every rank from the ranks' vocabulary slices (host side, not a hot path)."""
    parts = [None] * dist.get_world_size()
    a, b = model.tp_vocab_range()
    dist.all_gather_object(parts, (a, b, model.current_logits()[a:b]))
    out = np.zeros(model.cfg["n_vocab"], np.float32)
    for lo, hi, v in parts:
        out[lo:hi] = v
    return out
