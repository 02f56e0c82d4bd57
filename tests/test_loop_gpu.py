"""The persistent decode loop (one cooperative kernel per call) against the chained-kernel schedule, the CPU
oracle and the reference's kernels, through the C ABI (needs a B200)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from taraference_b200 import synth as S  # noqa: E402
from tests.test_engine_gpu import SMALL, SMALL_128, TF_TYPICAL, TF_WORST, _rel, margin_gated_equal, teacher_forced_errors  # noqa: E402

# K = 768 gives rows of three blocks (a row never fills a warp task), FF = 1280 five: the general row-sum route
ODD = dict(arch="qwen2", n_layer=2, n_embd=768, n_head=6, n_kv=2, head_dim=128, n_ff=1280, n_vocab=3001,
           rope_theta=1e6, eps=1e-6, tied=True, qkv_bias=True)


@pytest.fixture(scope="module")
def E(cuda_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from taraference_b200 import engine
    return engine


def _loop_model(E, cfg, tens):
    m = E.CudaModel.load_with(cfg, tens)
    m.set_decode_path(m.PATH_LOOP)  # raises if the model does not qualify
    assert m.decode_path() == m.PATH_LOOP
    return m


@pytest.mark.parametrize("cfg", [S.TINY_DENSE, SMALL, SMALL_128, ODD], ids=["tiny", "small64", "small128", "odd"])
def test_loop_teacher_forced_layers_vs_cpu_oracle(E, oracle, cfg):
    cfg = dict(cfg, n_layer=3)
    tens = S.make_dense_model(cfg, seed=3)
    om = oracle.OracleModel(cfg, tens, 64)
    m = _loop_model(E, cfg, tens)
    kv = m.alloc_kv(64)
    le, he = teacher_forced_errors(m, kv, om.embed, om.layer_forward, om.head_forward, cfg, [5, 17, 3, 250, 9])
    assert np.median(le) < 2e-5 and np.median(he) < 2e-5, (le, he)
    assert le.max() < TF_WORST and he.max() < TF_WORST, (le, he)
    kv.free()
    m.destroy()


@pytest.mark.parametrize("cfg", [S.TINY_DENSE, SMALL_128], ids=["tiny", "small128"])
def test_loop_teacher_forced_layers_vs_reference_kernels(E, cfg):
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("reference cubin not present")
    cfg = dict(cfg, n_layer=4)
    tens = S.make_dense_model(cfg, seed=4)
    rm = ref_gpu.RefModel(cfg, tens, 64)
    m = _loop_model(E, cfg, tens)
    kv = m.alloc_kv(64)
    to_t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32).copy()).cuda()
    le, he = teacher_forced_errors(
        m, kv, lambda t: ref_gpu.embed(rm.embd, t).cpu().numpy(),
        lambda li, x, pos: rm.layer_forward(li, to_t(x), pos).cpu().numpy(),
        lambda x: rm.head_forward(to_t(x)).cpu().numpy(), cfg, [1, 2, 3, 250, 7, 9])
    assert np.median(le) < TF_TYPICAL and np.median(he) < TF_TYPICAL, (le, he)
    assert (le < 1e-5).mean() >= 0.8, le
    assert le.max() < TF_WORST and he.max() < TF_WORST, (le, he)
    kv.free()
    m.destroy()


@pytest.mark.parametrize("cfg", [SMALL, ODD], ids=["small64", "odd"])
def test_loop_burst_prompt_and_verify_agree_with_each_other(E, cfg):
    """One launch for a whole burst == one launch per token == the verification pass; prompts fed inside the
    kernel; stop ids; the cache limit.  All of it bit for bit: the schedule is deterministic."""
    tens = S.make_dense_model(cfg, seed=5)
    m = _loop_model(E, cfg, tens)
    kv = m.alloc_kv(128)
    first = m.forward_greedy([11, 12, 13], kv)
    burst = m.decode_burst(first, 24, kv)
    logits_burst = m.current_logits()
    assert len(burst) == 24 and kv.len == 27 and not m.graph_active()
    kv.len = 3
    t, single = first, []
    for _ in range(24):
        t = m.forward_greedy([t], kv)
        single.append(t)
    assert list(burst) == single
    assert np.array_equal(logits_burst, m.current_logits())
    # prompt fed token by token == prompt fed in one call
    kv2 = m.alloc_kv(128)
    for tok in [11, 12, 13]:
        f2 = m.forward_greedy([tok], kv2)
    assert f2 == first
    # verification pass: predictions after every supplied token
    kv2.len = 3
    fed = [first] + list(burst[:8])
    got = m.forward_greedy_all(fed, kv2)
    assert list(got) == list(burst[:9]) and kv2.len == 3 + 9
    # stop id and the cache limit
    kv.len = 3
    stop = int(burst[5])
    cut = m.decode_burst(first, 24, kv, stop_ids=[stop])
    k = list(burst).index(stop)
    assert list(cut) == list(burst[: k + 1]) and kv.len == 3 + k + 1
    kv.len = 120
    assert len(m.decode_burst(first, 100, kv)) == 8 and kv.len == 128
    kv.free(), kv2.free()
    m.destroy()


@pytest.mark.parametrize("cfg", [SMALL, SMALL_128], ids=["small64", "small128"])
def test_loop_vs_chained_kernels_free_running(E, oracle, cfg):
    """Both schedules against the CPU oracle: logits within the free-running drift bound, greedy tokens equal
    wherever the oracle's top-2 margin is large; and against each other at the first step, where both have
    seen identical inputs in every layer but the summation order differs."""
    tens = S.make_dense_model(cfg, seed=7)
    om = oracle.OracleModel(cfg, tens, 96)
    prompt = [5, 17, 3, 250, 9]
    for i, t in enumerate(prompt):
        ologits = om.decode_token(i, t)
    res = {}
    for path in (1, 2):
        m = E.CudaModel.load_with(cfg, tens)
        m.set_decode_path(path)
        kv = m.alloc_kv(96)
        nxt = m.forward_greedy(prompt, kv)
        logits = m.current_logits()
        toks = m.decode_burst(nxt, 40, kv)
        res[path] = (nxt, logits, toks)
        assert _rel(logits, ologits) < 5e-2
        kv.free()
        m.destroy()
    otoks, omarg, _ = om.decode_greedy(5, res[2][0], 40)
    assert margin_gated_equal(res[2][2], otoks, omarg), (res[2][2], otoks, omarg)
    assert _rel(res[1][1], res[2][1]) < 5e-2


def test_loop_longer_context_many_splits(E, oracle):
    """A context long enough for several attention splits, including the separate merge phase (more than eight
    splits): teacher-forced against the oracle at positions around 600."""
    cfg = dict(SMALL_128, n_layer=2)
    tens = S.make_dense_model(cfg, seed=9)
    m = _loop_model(E, cfg, tens)
    ref = E.CudaModel.load_with(cfg, tens)
    ref.set_decode_path(1)
    kv, kvr = m.alloc_kv(700), ref.alloc_kv(700)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg["n_vocab"], 640).tolist()
    a = m.forward_greedy(prompt, kv)
    b = ref.forward_greedy(prompt, kvr)
    la, lb = m.current_logits(), ref.current_logits()
    # free-running over 640 positions: the two schedules drift apart by activation-rounding flips only
    assert _rel(la, lb) < 5e-2, _rel(la, lb)
    # identical caches from here: one more step on both, K/V rows written by the loop equal the chained path's
    k_loop = m.debug_read("k", 640 * cfg["n_kv"] * cfg["head_dim"], np.uint16, kv=kv, layer=0)
    k_ref = ref.debug_read("k", 640 * cfg["n_kv"] * cfg["head_dim"], np.uint16, kv=kvr, layer=0)
    # layer 0 keys depend on the embedding only: the same integer dots on both schedules, another fp32 summation
    # order, so a few f16 roundings may fall the other way by one unit in the last place
    kl, kr = k_loop.view(np.float16).astype(np.float32), k_ref.view(np.float16).astype(np.float32)
    assert (k_loop != k_ref).mean() < 5e-3 and np.abs(kl - kr).max() <= 2e-3 * np.abs(kr).max()
    assert len(m.decode_burst(a, 30, kv)) == 30
    kv.free(), kvr.free()
    m.destroy(), ref.destroy()
