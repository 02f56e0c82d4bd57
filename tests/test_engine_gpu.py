"""Whole-model parity of the decode engine through the C ABI (needs a B200)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from taraference_b200 import synth as S  # noqa: E402

SMALL = dict(arch="qwen2", n_layer=3, n_embd=512, n_head=8, n_kv=2, head_dim=64, n_ff=1024, n_vocab=1000,
             rope_theta=1e6, eps=1e-6, tied=True, qkv_bias=True)
SMALL_128 = dict(arch="qwen2", n_layer=2, n_embd=1024, n_head=8, n_kv=1, head_dim=128, n_ff=2816, n_vocab=2000,
                 rope_theta=1e6, eps=1e-6, tied=False, qkv_bias=True)


@pytest.fixture(scope="module")
def E(cuda_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from taraference_b200 import engine
    return engine


def _rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def margin_gated_equal(toks, ref_toks, ref_margins, gate=1e-2):
    """Greedy tokens must agree up to (and including) the first position where the checker's
    top-2 logit gap is below the gate; after a legitimate divergence the sequences differ."""
    for i, (a, b) in enumerate(zip(toks, ref_toks)):
        if a != b:
            return ref_margins[i] <= gate
    return True


@pytest.mark.parametrize("cfg", [S.TINY_DENSE, SMALL, SMALL_128], ids=["tiny", "small64", "small128"])
def test_logits_and_tokens_vs_cpu_oracle(E, oracle, cfg):
    tens = S.make_dense_model(cfg, seed=3)
    om = oracle.OracleModel(cfg, tens, 64)
    m = E.CudaModel.load_with(cfg, tens)
    kv = m.alloc_kv(64)
    prompt = [5, 17, 3, 250, 9]
    nxt = m.forward_greedy(prompt, kv)
    assert kv.len == 5
    for i, t in enumerate(prompt):
        ologits = om.decode_token(i, t)
    glogits = m.current_logits()
    assert _rel(glogits, ologits) < 1e-3, _rel(glogits, ologits)
    assert nxt == int(np.argmax(ologits)) or np.sort(ologits)[-1] - np.sort(ologits)[-2] < 1e-2
    toks = m.decode_burst(nxt, 20, kv)
    otoks, omarg, _ = om.decode_greedy(5, nxt, 20)
    assert len(toks) == 20 and kv.len == 25
    assert margin_gated_equal(toks, otoks, omarg), (toks, otoks, omarg)
    kv.free()
    m.destroy()


@pytest.mark.parametrize("cfg", [S.TINY_DENSE, SMALL_128], ids=["tiny", "small128"])
def test_logits_vs_reference_kernels(E, cfg):
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("reference cubin not present")
    tens = S.make_dense_model(cfg, seed=4)
    rm = ref_gpu.RefModel(cfg, tens, 64)
    m = E.CudaModel.load_with(cfg, tens)
    kv = m.alloc_kv(64)
    prompt = [1, 2, 3, 4, 5, 6, 7]
    nxt = m.forward_greedy(prompt, kv)
    for i, t in enumerate(prompt):
        rlogits = rm.decode_token(i, t)
    rl = rlogits.cpu().numpy()
    gl = m.current_logits()
    assert _rel(gl, rl) < 1e-3, _rel(gl, rl)
    rtoks, rmarg, _ = rm.decode_greedy(7, nxt, 12)
    toks = m.decode_burst(nxt, 12, kv)
    assert margin_gated_equal(toks, rtoks, rmarg), (toks, rtoks, rmarg)
    kv.free()
    m.destroy()


def test_burst_equals_token_by_token_and_graph_equals_eager(E):
    cfg = SMALL
    tens = S.make_dense_model(cfg, seed=5)
    m = E.CudaModel.load_with(cfg, tens)
    kv = m.alloc_kv(128)
    first = m.forward_greedy([11, 12, 13], kv)
    burst = m.decode_burst(first, 24, kv)
    logits_graph = m.current_logits()
    assert m.graph_active()
    # token by token through forward_greedy (one host round-trip per token, reference style)
    kv.len = 3
    t, single = first, []
    for _ in range(24):
        t = m.forward_greedy([t], kv)
        single.append(t)
    assert list(burst) == single
    # eager launches instead of graph replay
    m.set_cuda_graph(False)
    kv.len = 3
    eager = m.decode_burst(first, 24, kv)
    assert not m.graph_active()
    assert list(burst) == list(eager)
    assert np.array_equal(logits_graph, m.current_logits())
    # a second cache forces a re-capture and still agrees
    m.set_cuda_graph(True)
    kv2 = m.alloc_kv(40)
    f2 = m.forward_greedy([11, 12, 13], kv2)
    assert f2 == first and list(m.decode_burst(f2, 24, kv2)) == list(burst)
    assert m.launch_count() > 0
    kv.free(), kv2.free()
    m.destroy()


def test_stop_ids_context_limit_and_errors(E):
    cfg = S.TINY_DENSE
    tens = S.make_dense_model(cfg, seed=6)
    m = E.CudaModel.load_with(cfg, tens)
    kv = m.alloc_kv(16)
    with pytest.raises(E.TfrError, match="empty tokens"):
        m.forward_greedy([], kv)
    with pytest.raises(E.TfrError, match="context full"):
        m.forward_greedy(list(range(17)), kv)
    with pytest.raises(E.TfrError, match="out of range"):
        m.forward_greedy([cfg["n_vocab"]], kv)
    first = m.forward_greedy([1, 2, 3], kv)
    free_run = m.decode_burst(first, 13, kv)
    assert len(free_run) == 13 and kv.len == 16
    with pytest.raises(E.TfrError, match="context full"):
        m.decode_burst(1, 1, kv)
    # stop id: the burst ends right after emitting it
    kv.len = 3
    stop = int(free_run[4])
    cut = m.decode_burst(first, 13, kv, stop_ids=[stop])
    k = list(free_run).index(stop)
    assert list(cut) == list(free_run[: k + 1]) and kv.len == 3 + k + 1
    # asking for more than the cache holds is clipped to the capacity
    kv.len = 10
    assert len(m.decode_burst(first, 100, kv)) == 6 and kv.len == 16
    kv.clear()
    assert kv.len == 0 and kv.bytes_per_token() == cfg["n_layer"] * cfg["n_kv"] * cfg["head_dim"] * 4
    kv.free()
    m.destroy()


def test_missing_tensor_is_reported(E):
    cfg = S.TINY_DENSE
    tens = S.make_dense_model(cfg, seed=7)
    del tens["blk.1.ffn_down.weight"]
    with pytest.raises(E.TfrError, match="missing tensor blk.1.ffn_down.weight"):
        E.CudaModel.load_with(cfg, tens)


def test_full_size_3b_layer_shapes_vs_oracle(E, oracle):
    """Two layers at the Qwen2.5-3B shape with the full vocabulary head, device-generated weights,
    the same bytes fed to the CPU oracle: logits within 1e-3, greedy tokens margin-gated."""
    from taraference_b200 import synth_gpu
    cfg = dict(S.QWEN25_3B, n_layer=2)
    m, host = synth_gpu.build_dense_model(cfg, seed=0, keep_host=True)
    kv = m.alloc_kv(64)
    prompt = [100, 2000, 30000, 151000]
    nxt = m.forward_greedy(prompt, kv)
    oracle.set_threads(oracle.max_threads())
    om = oracle.OracleModel(cfg, host, 64)
    for i, t in enumerate(prompt):
        ologits = om.decode_token(i, t)
    gl = m.current_logits()
    assert _rel(gl, ologits) < 1e-3, _rel(gl, ologits)
    toks = m.decode_burst(nxt, 6, kv)
    otoks, omarg, _ = om.decode_greedy(4, nxt, 6)
    oracle.set_threads(1)
    assert margin_gated_equal(toks, otoks, omarg), (toks, otoks, omarg)
    kv.free()
    m.destroy()
