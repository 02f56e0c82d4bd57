"""Tensor-parallel split arithmetic on CPU: the shard plan, and a two-rank gloo run in which
every rank computes its share of the row-/column-parallel products with the CPU oracle and the
partial sums meet in an all-reduce — the same exchange the kernels do over NVLink."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from taraference_b200 import synth as S  # noqa: E402
from taraference_b200 import tp as TP  # noqa: E402

TP_TEST = dict(arch="qwen2", n_layer=1, n_embd=512, n_head=12, n_kv=4, head_dim=64, n_ff=1280, n_vocab=1001,
               rope_theta=1e6, eps=1e-6, tied=False, qkv_bias=True)


@pytest.mark.parametrize("cfg,tps", [(S.QWEN25_32B, (1, 2, 4, 8)), (TP_TEST, (1, 2, 4))])
def test_shard_plans_tile_the_model(cfg, tps):
    H, Hkv, hd, FF, V = (cfg[k] for k in ("n_head", "n_kv", "head_dim", "n_ff", "n_vocab"))
    for tp in tps:
        plans = [TP.shard_plan(cfg, r, tp) for r in range(tp)]
        for key, total in (("q_rows", H * hd), ("kv_rows", Hkv * hd), ("ff_rows", FF), ("vocab_rows", V)):
            assert plans[0][key][0] == 0 and plans[-1][key][1] == total
            for a, b in zip(plans, plans[1:]):
                assert a[key][1] == b[key][0], (key, tp)
        for p in plans:
            lo, hi = p["q_rows"]
            b0, b1 = p["wo_blocks"]
            assert b0 * 256 <= lo and hi <= b1 * 256 and p["attn_offset"] == lo - b0 * 256
            assert p["attn_width"] == (b1 - b0) * 256 and p["attn_offset"] % 32 == 0
            assert (lo // hd) // (H // Hkv) == p["kv_rows"][0] // hd     # a KV head stays with its query heads
            assert p["ff_rows"] == (p["ff_blocks"][0] * 256, p["ff_blocks"][1] * 256)
        sizes = [p["ff_blocks"][1] - p["ff_blocks"][0] for p in plans]
        assert max(sizes) - min(sizes) <= 1


def test_shard_plan_rejects_bad_splits():
    with pytest.raises(ValueError):
        TP.shard_plan(S.QWEN25_3B, 0, 4)       # 2 KV heads over 4 ranks
    with pytest.raises(ValueError):
        TP.shard_plan(S.QWEN25_32B, 8, 8)


def _k_slice(raw, wtype, K, N, b0, b1):
    blk = S.BLOCK_BYTES[wtype]
    return np.ascontiguousarray(raw.reshape(N, K // 256, blk)[:, b0:b1]).reshape(-1)


def _row_slice(raw, wtype, K, N, r0, r1):
    blk = S.BLOCK_BYTES[wtype]
    return np.ascontiguousarray(raw.reshape(N, (K // 256) * blk)[r0:r1]).reshape(-1)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    from oracle import oracle as O
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = TP_TEST
    tens = S.make_model(cfg, seed=21)           # every rank sees the same full tensors
    plan = TP.shard_plan(cfg, rank, world)
    rng = np.random.default_rng(5)
    K, nq, FF = cfg["n_embd"], cfg["n_head"] * cfg["head_dim"], cfg["n_ff"]
    attn = rng.normal(0, 1, nq).astype(np.float32)   # full attention output, identical on all ranks
    xn = rng.normal(0, 1, K).astype(np.float32)
    res = {}
    # row-parallel attn_output: K blocks covering the rank's heads, activation zero outside them
    t, Kw, Nw, raw = tens["blk.0.attn_output.weight"]
    b0, b1 = plan["wo_blocks"]
    lo, hi = plan["q_rows"]
    act = np.zeros(plan["attn_width"], np.float32)
    act[plan["attn_offset"]:plan["attn_offset"] + hi - lo] = attn[lo:hi]
    part = O.gemv(O.mat(t, _k_slice(raw, t, Kw, Nw, b0, b1), (b1 - b0) * 256, Nw), act)
    red = torch.from_numpy(part.copy())
    dist.all_reduce(red)
    res["wo"] = (red.numpy(), O.gemv(O.mat(t, raw, Kw, Nw), attn))
    # column-parallel gate/up feeding the row-parallel down projection
    r0, r1 = plan["ff_rows"]
    f0, f1 = plan["ff_blocks"]
    tg, _, _, rg = tens["blk.0.ffn_gate.weight"]
    tu, _, _, ru = tens["blk.0.ffn_up.weight"]
    td, _, _, rd = tens["blk.0.ffn_down.weight"]
    h_loc = O.ffn_gate_up(O.mat(tg, _row_slice(rg, tg, K, FF, r0, r1), K, r1 - r0),
                          O.mat(tu, _row_slice(ru, tu, K, FF, r0, r1), K, r1 - r0), xn)
    part = O.gemv(O.mat(td, _k_slice(rd, td, FF, K, f0, f1), (f1 - f0) * 256, K), h_loc)
    red = torch.from_numpy(part.copy())
    dist.all_reduce(red)
    h_full = O.ffn_gate_up(O.mat(tg, rg, K, FF), O.mat(tu, ru, K, FF), xn)
    res["ffn"] = (red.numpy(), O.gemv(O.mat(td, rd, FF, K), h_full))
    res["h_slice_exact"] = bool(np.array_equal(h_loc, h_full[r0:r1]))
    # vocabulary-parallel head: (logit, index) maximum over ranks
    th, _, V, rh = tens["output.weight"]
    v0, v1 = plan["vocab_rows"]
    loc = O.gemv(O.mat(th, _row_slice(rh, th, K, V, v0, v1), K, v1 - v0), xn)
    best = torch.tensor([float(loc.max()), float(-(v0 + int(loc.argmax())))], dtype=torch.float64)
    gathered = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, best)
    win = max(gathered, key=lambda g: (g[0].item(), g[1].item()))
    full = O.gemv(O.mat(th, rh, K, V), xn)
    res["argmax"] = (int(-win[1].item()), int(full.argmax()))
    res["logit_slice_exact"] = bool(np.array_equal(loc, full[v0:v1]))
    dist.barrier()
    out[rank] = res
    dist.destroy_process_group()


def test_two_rank_split_sums_to_the_single_rank_result():
    world = 2
    port = 31000 + os.getpid() % 2000
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    for rank in range(world):
        r = out[rank]
        for key in ("wo", "ffn"):
            got, want = r[key]
            # identical int8 activations and integer dots on both sides: only the fp32 order of the
            # cross-rank sum differs
            assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max(), key
        assert r["h_slice_exact"] and r["logit_slice_exact"]
        assert r["argmax"][0] == r["argmax"][1]
    assert np.array_equal(out[0]["wo"][0], out[1]["wo"][0])   # every rank holds the same reduced vector
