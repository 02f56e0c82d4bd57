"""Tensor-parallel decode through the C ABI.

The two-rank tests need two GPUs (one process per GPU, NVLink peer memory) and skip otherwise;
the bounded-wait test runs on one GPU: it gives a rank a peer buffer that nobody ever writes.
"""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]

from taraference_b200 import synth as S  # noqa: E402

# 12 query / 4 KV heads of 64: at tp=2 a rank's heads cover 384 elements, so the attn_output
# slices share a border block; 5 FFN blocks split 2 + 3; the odd vocabulary splits 500 + 501
TP_CFG = dict(arch="qwen2", n_layer=3, n_embd=512, n_head=12, n_kv=4, head_dim=64, n_ff=1280, n_vocab=1001,
              rope_theta=1e6, eps=1e-6, tied=False, qkv_bias=True)
PROMPT = [5, 17, 3, 250, 9]


def _rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def _worker(rank, world, port, out, graph):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    from taraference_b200 import engine as E, tp as TP
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tens = S.make_model(TP_CFG, seed=4)
    m = E.CudaModel.load_with(dict(TP_CFG, tp_rank=rank, tp_size=world), tens, device=rank)
    m.set_cuda_graph(graph)
    TP.connect(m, dist)
    kv = m.alloc_kv(64)
    K, L = TP_CFG["n_embd"], TP_CFG["n_layer"]
    m.debug_read("layer_x", L * K)
    first = m.forward_greedy(PROMPT[:1], kv)
    lx0 = m.debug_read("layer_x", L * K).reshape(L, K)
    nxt = m.forward_greedy(PROMPT[1:], kv)
    logits = TP.gather_logits(m, dist)
    toks = m.decode_burst(nxt, 20, kv)
    x = m.debug_read("x", K)
    res = dict(first=first, nxt=nxt, toks=toks, x=x, lx0=lx0, logits=logits, kv_len=kv.len,
               kv_bytes=kv.bytes_per_token(), vocab=m.tp_vocab_range())
    dist.barrier()
    # the comparison mode (ncclAllReduce between kernels) must give the same tokens: with two ranks the sum
    # a + b has one order only
    try:
        TP.use_nccl(m, dist)
        kv.clear()
        n2 = m.forward_greedy(PROMPT, kv)
        res["nccl"] = dict(nxt=n2, toks=m.decode_burst(n2, 20, kv), x=m.debug_read("x", K))
        TP.use_nccl(m, dist, on=False)
        kv.clear()
        n3 = m.forward_greedy(PROMPT, kv)
        res["back"] = dict(nxt=n3, toks=m.decode_burst(n3, 20, kv))
    except E.TfrError as exc:
        res["nccl"] = dict(error=str(exc))
    dist.barrier()
    if rank == 0:
        # the same model on one GPU, and the CPU oracle
        m1 = E.CudaModel.load_with(TP_CFG, tens, device=0)
        kv1 = m1.alloc_kv(64)
        m1.debug_read("layer_x", L * K)
        f1 = m1.forward_greedy(PROMPT[:1], kv1)
        res["single_lx0"] = m1.debug_read("layer_x", L * K).reshape(L, K)
        n1 = m1.forward_greedy(PROMPT[1:], kv1)
        res["single"] = dict(first=f1, nxt=n1, logits=m1.current_logits(), toks=m1.decode_burst(n1, 20, kv1),
                             kv_bytes=kv1.bytes_per_token())
        from oracle import oracle as O
        om = O.OracleModel(TP_CFG, tens, 64)
        for i, t in enumerate(PROMPT):
            ol = om.decode_token(i, t)
        otoks, omarg, _ = om.decode_greedy(len(PROMPT), nxt, 20)
        res["oracle"] = dict(logits=ol, toks=otoks, margins=omarg)
        kv1.free()
        m1.destroy()
    dist.barrier()
    out[rank] = res
    kv.free()
    m.destroy()
    dist.destroy_process_group()


@pytest.mark.parametrize("graph", [True, False], ids=["graph", "plain"])
def test_two_ranks_match_single_gpu_and_oracle(cuda_lib, graph):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from test_engine_gpu import margin_gated_equal
    world = 2
    port = 33000 + os.getpid() % 2000
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out, graph), nprocs=world, join=True)
    r0, r1 = out[0], out[1]
    # the replicated residual stream and every emitted token are bit-identical across ranks
    assert np.array_equal(r0["x"], r1["x"]) and np.array_equal(r0["lx0"], r1["lx0"])
    assert r0["first"] == r1["first"] and r0["nxt"] == r1["nxt"] and np.array_equal(r0["toks"], r1["toks"])
    assert r0["kv_len"] == r1["kv_len"] == len(PROMPT) + 20 and len(r0["toks"]) == 20
    assert r0["vocab"] == (0, 500) and r1["vocab"] == (500, 1001)
    s, o = r0["single"], r0["oracle"]
    assert r0["kv_bytes"] * 2 == s["kv_bytes"]
    # first token, layer by layer against the single-GPU engine: the same integer dots, another fp32 order
    le = np.array([_rel(r0["lx0"][li], r0["single_lx0"][li]) for li in range(TP_CFG["n_layer"])])
    assert le[0] < 2e-6 and le.max() < 1e-2, le
    assert _rel(r0["logits"], s["logits"]) < 5e-2 and _rel(r0["logits"], o["logits"]) < 5e-2
    assert r0["first"] == s["first"]
    assert margin_gated_equal(r0["toks"], o["toks"], o["margins"]), (r0["toks"], o["toks"], o["margins"])
    if "error" in r0["nccl"]:
        assert "libnccl" in r0["nccl"]["error"], r0["nccl"]   # only a missing library excuses the baseline
    else:
        for r in (r0, r1):
            assert r["nccl"]["nxt"] == r["nxt"] and np.array_equal(r["nccl"]["toks"], r["toks"])
            assert np.array_equal(r["nccl"]["x"], r["x"])
            assert r["back"]["nxt"] == r["nxt"] and np.array_equal(r["back"]["toks"], r["toks"])


def test_missing_peer_ends_in_an_error_not_a_hang(cuda_lib):
    """One GPU: rank 0 of 2 is connected to a peer buffer that nothing ever writes.  The bounded
    wait of the first all-reduce runs out, the burst ends and the call reports the failure."""
    import time
    from taraference_b200 import engine as E
    tens = S.make_model(TP_CFG, seed=4)
    m = E.CudaModel.load_with(dict(TP_CFG, tp_rank=0, tp_size=2), tens)
    kv = m.alloc_kv(16)
    with pytest.raises(E.TfrError, match="not connected"):
        m.forward_greedy([1], kv)
    # leaving the NCCL comparison mode needs the peers' buffers: refused while they were never connected
    with pytest.raises(E.TfrError, match="never connected"):
        m.tp_use_nccl(None)
    fake_peer = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    m.tp_attach_pointers([m.tp_local_pointer(), fake_peer.data_ptr()])
    t0 = time.time()
    with pytest.raises(E.TfrError, match="peer rank did not deliver"):
        m.decode_burst(1, 4, kv)
    assert time.time() - t0 < 30
    torch.cuda.synchronize()  # the context is still usable
    assert int(torch.ones(4, device="cuda").sum().item()) == 4
    kv.free()
    m.destroy()


def test_tp_config_errors(cuda_lib):
    from taraference_b200 import engine as E
    m = E.CudaModel(0)
    with pytest.raises(E.TfrError, match="does not divide"):
        m.set_config(dict(S.QWEN25_3B, tp_rank=0, tp_size=4))
    with pytest.raises(E.TfrError, match="tp_rank"):
        m.set_config(dict(TP_CFG, tp_rank=2, tp_size=2))
    with pytest.raises(E.TfrError, match="dense"):
        m.set_config(dict(S.TINY_HYBRID, tp_rank=0, tp_size=2))
    m.destroy()


def test_one_process_drives_two_gpus_through_attached_pointers(cuda_lib):
    """Two engines on two GPUs in ONE process, wired with tfr_tp_local_pointer / tfr_tp_attach_pointers (no IPC
    handles, no process group).  Every forward call needs both ranks at the same time, so each engine is driven
    by its own host thread.  The ranks must emit identical tokens, equal to the single-GPU engine's wherever that
    engine's margin is large."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import threading
    from taraference_b200 import engine as E
    from test_engine_gpu import margin_gated_equal
    tens = S.make_model(TP_CFG, seed=4)
    models = [E.CudaModel.load_with(dict(TP_CFG, tp_rank=r, tp_size=2), tens, device=r) for r in range(2)]
    with pytest.raises(E.TfrError, match="not connected"):
        kv_bad = models[0].alloc_kv(8)
        try:
            models[0].forward_greedy([1], kv_bad)
        finally:
            kv_bad.free()
    bases = [m.tp_local_pointer() for m in models]
    for m in models:
        m.tp_attach_pointers(bases)
    kvs = [m.alloc_kv(64) for m in models]
    results = [None, None]

    def run(r):
        try:
            torch.cuda.set_device(r)
            nxt = models[r].forward_greedy(PROMPT, kvs[r])
            toks = models[r].decode_burst(nxt, 20, kvs[r])
            results[r] = (nxt, [int(t) for t in toks], models[r].debug_read("x", TP_CFG["n_embd"]))
        except Exception as exc:  # surfaced by the assertions below
            results[r] = exc

    threads = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in threads), "a rank did not return"
    for r in results:
        assert not isinstance(r, Exception), r
    assert results[0][0] == results[1][0] and results[0][1] == results[1][1]
    assert np.array_equal(results[0][2], results[1][2])  # the replicated residual stream, bit for bit
    torch.cuda.set_device(0)
    single = E.CudaModel.load_with(TP_CFG, tens, device=0)
    kv1 = single.alloc_kv(64)
    n1 = single.forward_greedy(PROMPT, kv1)
    margins, want, t = [], [], n1
    for _ in range(20):
        t = single.forward_greedy([t], kv1)
        top = np.sort(single.current_logits())[-2:]
        want.append(t)
        margins.append(float(top[1] - top[0]))
    if results[0][0] == n1:
        assert margin_gated_equal(results[0][1], want, margins), (results[0][1], want, margins)
    kv1.free()
    single.destroy()
    for kv in kvs:
        kv.free()
    for m in models:
        m.destroy()
