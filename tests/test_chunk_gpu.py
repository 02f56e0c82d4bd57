"""Prompts and verification batches in chunks (one weight pass per chunk) against the step-by-step route, the CPU
oracle and the reference's kernels, through the C ABI (needs a B200)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from taraference_b200 import synth as S  # noqa: E402
from tests.test_engine_gpu import SMALL, SMALL_128, TF_WORST, _rel, margin_gated_equal  # noqa: E402

# K = 768 gives rows of three blocks, FF = 1280 five: rows that never fill a warp's 32 blocks
ODD = dict(arch="qwen2", n_layer=2, n_embd=768, n_head=6, n_kv=2, head_dim=128, n_ff=1280, n_vocab=3001,
           rope_theta=1e6, eps=1e-6, tied=True, qkv_bias=True)
CFGS = [S.TINY_DENSE, SMALL, SMALL_128, ODD]
IDS = ["tiny", "small64", "small128", "odd"]


@pytest.fixture(scope="module")
def E(cuda_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from taraference_b200 import engine
    return engine


def _free_running(cfg):
    """One int8 flip moves a layer's output by up to TF_WORST; run freely, the flips of successive layers add up
    (the floor of test_engine_gpu.free_running_bound)."""
    return min(cfg["n_layer"], 5) * TF_WORST


def _k_rows_agree(ka, kb):
    """K rows of layer 0 from two routes of which one ran the K projection on the tensor cores: the integer sub-block
    sums are the same, the fp32 row sums differ in order, so a value now and then lands on the other side of an f16
    rounding boundary (where RoPE subtracts two close products, a few steps of a small value).  Measured on the four
    shapes: 0.1 - 0.4 % of the values move, by at most 2.1e-4 of the largest value (one f16 step of it is 4.9e-4)."""
    if np.array_equal(ka, kb):
        return True
    f = lambda a: a.view(np.float16).astype(np.float32)
    return (ka != kb).mean() < 1e-2 and _rel(f(kb), f(ka)) < 5e-4


def _margin(logits):
    top = np.sort(logits)[-2:]
    return float(top[1] - top[0])


def _cache_rows(m, kv, cfg, layer, n_pos):
    kvdim = cfg["n_kv"] * cfg["head_dim"]
    k = m.debug_read("k", n_pos * kvdim, np.uint16, kv=kv, layer=layer)
    v = m.debug_read("v", n_pos * kvdim, np.uint16, kv=kv, layer=layer)
    return k, v


@pytest.mark.parametrize("cfg", CFGS, ids=IDS)
@pytest.mark.parametrize("chunk", [5, 16, 64])
def test_chunked_prompt_equals_step_by_step(E, cfg, chunk):
    """A prompt fed in chunks leaves the cache and the next-token logits of the same prompt fed token by token.
    The projections compute the same integer sub-block sums, so layer 0 (no attention upstream) leaves the same V rows
    bit for bit and the same K rows up to an f16 step now and then; deeper layers differ by the summation order inside
    attention and the tensor-core projections (fp32 rounding level, now and then an int8 flip)."""
    tens = S.make_dense_model(cfg, seed=21)
    rng = np.random.default_rng(7)
    n = 45
    prompt = [int(t) for t in rng.integers(0, cfg["n_vocab"], n)]
    m = E.CudaModel.load_with(cfg, tens)
    kv_a, kv_b = m.alloc_kv(96), m.alloc_kv(96)
    m.set_prefill_chunk(0)
    assert m.prefill_chunk() == 0
    launches0 = m.launch_count()
    tok_a = m.forward_greedy(prompt, kv_a)
    launches_step = m.launch_count() - launches0
    logits_a = m.current_logits()
    m.set_prefill_chunk(chunk)
    assert m.prefill_chunk() == chunk
    launches0 = m.launch_count()
    tok_b = m.forward_greedy(prompt, kv_b)
    launches_chunk = m.launch_count() - launches0
    logits_b = m.current_logits()
    assert kv_a.len == kv_b.len == n
    if chunk >= 16:
        assert launches_chunk < launches_step / 2, (launches_chunk, launches_step)
    k0a, v0a = _cache_rows(m, kv_a, cfg, 0, n)
    k0b, v0b = _cache_rows(m, kv_b, cfg, 0, n)
    # layer 0 has no attention upstream: the fp32-route V rows keep the decode arithmetic bit for bit, the K rows run on
    # the tensor cores from five tokens on
    assert np.array_equal(v0a, v0b) and _k_rows_agree(k0a, k0b)
    last = cfg["n_layer"] - 1
    kla, vla = _cache_rows(m, kv_a, cfg, last, n)
    klb, vlb = _cache_rows(m, kv_b, cfg, last, n)
    f16 = lambda a: a.view(np.float16).astype(np.float32)
    assert _rel(f16(klb), f16(kla)) < _free_running(cfg) and _rel(f16(vlb), f16(vla)) < _free_running(cfg)
    # (How many f16 values move at all is not a property of either route: attention runs on the tensor cores for a
    # decode step and for chunks above 16 tokens and on CUDA cores for smaller chunks, all within 3e-7 of a float64
    # evaluation, so a rounding that falls the other way in one int8 activation moves a few per cent of the next
    # layer's cache values by one f16 step; the attribution test in test_engine_gpu.py pins such moves to their flip.)
    assert _rel(logits_b, logits_a) < _free_running(cfg)
    assert tok_a == tok_b or _margin(logits_a) <= 1e-2
    kv_a.free()
    kv_b.free()
    m.destroy()


@pytest.mark.parametrize("cfg", [SMALL, SMALL_128, ODD], ids=["small64", "small128", "odd"])
def test_long_chunked_prompt_with_key_splits(E, cfg):
    """A prompt long enough for the chunk attention to split its keys over several CTAs and merge the partials (from
    256 keys on), in chunks of 64 (the tensor-core kernel) and of 16 (the CUDA-core kernel of verification batches),
    against the same prompt fed token by token."""
    tens = S.make_dense_model(cfg, seed=24)
    rng = np.random.default_rng(10)
    n = 700
    prompt = [int(t) for t in rng.integers(0, cfg["n_vocab"], n)]
    m = E.CudaModel.load_with(cfg, tens)
    kv_a = m.alloc_kv(n + 8)
    m.set_prefill_chunk(0)
    tok_a = m.forward_greedy(prompt, kv_a)
    logits_a = m.current_logits()
    last = cfg["n_layer"] - 1
    kla, vla = _cache_rows(m, kv_a, cfg, last, n)
    f16 = lambda a: a.view(np.float16).astype(np.float32)
    for chunk in (64, 16):
        kv_b = m.alloc_kv(n + 8)
        m.set_prefill_chunk(chunk)
        tok_b = m.forward_greedy(prompt, kv_b)
        logits_b = m.current_logits()
        k0a, v0a = _cache_rows(m, kv_a, cfg, 0, n)
        k0b, v0b = _cache_rows(m, kv_b, cfg, 0, n)
        assert np.array_equal(v0a, v0b) and _k_rows_agree(k0a, k0b)  # layer 0 has no attention upstream
        klb, vlb = _cache_rows(m, kv_b, cfg, last, n)
        assert _rel(f16(klb), f16(kla)) < _free_running(cfg) and _rel(f16(vlb), f16(vla)) < _free_running(cfg), chunk
        assert _rel(logits_b, logits_a) < _free_running(cfg), chunk
        assert tok_a == tok_b or _margin(logits_a) <= 1e-2
        kv_b.free()
    kv_a.free()
    m.destroy()


@pytest.mark.parametrize("cfg", [SMALL, SMALL_128, ODD], ids=["small64", "small128", "odd"])
def test_tensor_core_projections_match_the_dp4a_projections(E, cfg, monkeypatch):
    """Prompt chunks run their Q4_K projections as int8 MMAs (k_gemm_mma_q4); TFR_GEMM_DP4A=1 keeps them on the dp4a
    kernel, which the tests above hold against the oracle and the reference.  One layer, so that what is compared is
    one pass through the projections: the integer sub-block sums are the same numbers on both routes, the fp32 sums
    differ in order (fp32 rounding level, at most an int8 flip in the layer)."""
    cfg = dict(cfg, n_layer=1)
    tens = S.make_dense_model(cfg, seed=25)
    rng = np.random.default_rng(11)
    m = E.CudaModel.load_with(cfg, tens)
    m.set_prefill_chunk(64)
    rels = []
    for n in (18, 45, 65, 130):
        prompt = [int(t) for t in rng.integers(0, cfg["n_vocab"], n)]
        kv_a, kv_b = m.alloc_kv(160), m.alloc_kv(160)
        monkeypatch.setenv("TFR_GEMM_DP4A", "1")
        tok_a = m.forward_greedy(prompt, kv_a)
        logits_a = m.current_logits()
        monkeypatch.delenv("TFR_GEMM_DP4A")
        tok_b = m.forward_greedy(prompt, kv_b)
        logits_b = m.current_logits()
        ka, va = _cache_rows(m, kv_a, cfg, 0, n)
        kb, vb = _cache_rows(m, kv_b, cfg, 0, n)
        assert np.array_equal(va, vb) and _k_rows_agree(ka, kb)  # V rows keep the decode arithmetic on both routes
        rels.append(_rel(logits_b, logits_a))
        assert rels[-1] < TF_WORST, (n, rels)
        assert tok_a == tok_b or _margin(logits_a) <= 1e-2
        kv_a.free()
        kv_b.free()
    assert np.median(rels) < 1e-4, rels  # without a flip the routes agree to fp32 rounding
    m.destroy()


def test_tensor_core_projections_on_a_wide_ffn(E, monkeypatch):
    """The tile shapes only wide matrices reach: n_ff = 11 008 gives gate / up more 64-row tiles than SMs (32-row tiles
    for a prompt chunk, 64-row tiles x 16-token tiles for a verification batch) and a down projection of 43 blocks per
    row whose k range is cut in four parts.  One layer, against the dp4a route and against feeding token by token."""
    cfg = dict(arch="qwen2", n_layer=1, n_embd=512, n_head=8, n_kv=2, head_dim=64, n_ff=11008, n_vocab=1000,
               rope_theta=1e6, eps=1e-6, tied=True, qkv_bias=True)
    tens = S.make_dense_model(cfg, seed=26)
    rng = np.random.default_rng(12)
    m = E.CudaModel.load_with(cfg, tens)
    n = 45
    prompt = [int(t) for t in rng.integers(0, cfg["n_vocab"], n)]
    kv = m.alloc_kv(64)
    m.set_prefill_chunk(0)
    tok_step = m.forward_greedy(prompt, kv)
    logits_step = m.current_logits()
    rels = []
    for chunk in (64, 16):
        m.set_prefill_chunk(chunk)
        monkeypatch.setenv("TFR_GEMM_DP4A", "1")
        kv.len = 0
        m.forward_greedy(prompt, kv)
        logits_dp4a = m.current_logits()
        monkeypatch.delenv("TFR_GEMM_DP4A")
        kv.len = 0
        tok = m.forward_greedy(prompt, kv)
        logits = m.current_logits()
        rels.append((_rel(logits, logits_dp4a), _rel(logits, logits_step)))
        assert rels[-1][0] < TF_WORST and rels[-1][1] < TF_WORST, (chunk, rels)
        assert tok == tok_step or _margin(logits_step) <= 1e-2
    assert min(r[0] for r in rels) < 1e-4, rels  # without a flip the routes agree to fp32 rounding
    # a verification batch of nine tokens (16-token tiles) against the same tokens one by one
    v = [int(t) for t in rng.integers(0, cfg["n_vocab"], 9)]
    m.set_prefill_chunk(64)
    kv.len = n
    got = m.forward_greedy_all(v, kv)
    lg = m.current_logits()
    m.set_prefill_chunk(0)
    kv.len = n
    want = m.forward_greedy_all(v, kv)
    lw = m.current_logits()
    assert _rel(lg, lw) < TF_WORST
    assert got[-1] == want[-1] or _margin(lw) <= 1e-2
    kv.free()
    m.destroy()


@pytest.mark.parametrize("cfg", CFGS, ids=IDS)
def test_chunked_prompt_vs_cpu_oracle(E, oracle, cfg):
    tens = S.make_dense_model(cfg, seed=22)
    rng = np.random.default_rng(8)
    n = 37
    prompt = [int(t) for t in rng.integers(0, cfg["n_vocab"], n)]
    om = oracle.OracleModel(cfg, tens, 64)
    ref_logits = None
    for i, t in enumerate(prompt):
        ref_logits = om.decode_token(i, t)
    m = E.CudaModel.load_with(cfg, tens)
    m.set_prefill_chunk(16)
    kv = m.alloc_kv(64)
    tok = m.forward_greedy(prompt, kv)
    got = m.current_logits()
    assert _rel(got, ref_logits) < 5e-2
    assert tok == int(np.argmax(ref_logits)) or _margin(ref_logits) <= 1e-2
    kv.free()
    m.destroy()


@pytest.mark.parametrize("cfg", [S.TINY_DENSE, SMALL_128], ids=["tiny", "small128"])
def test_chunked_prompt_vs_reference_kernels(E, cfg):
    """Against the reference's own kernels fed token by token (its decode route): the chunk kernels use that route's
    arithmetic, not the fp32-activation GEMM of the reference's prefill (kernels/gemm.cu:6-190)."""
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("reference cubin not present")
    tens = S.make_dense_model(cfg, seed=23)
    rng = np.random.default_rng(9)
    n = 29
    prompt = [int(t) for t in rng.integers(0, cfg["n_vocab"], n)]
    rm = ref_gpu.RefModel(cfg, tens, 64)
    ref_logits = None
    for i, t in enumerate(prompt):
        ref_logits = rm.decode_token(i, t).cpu().numpy()
    m = E.CudaModel.load_with(cfg, tens)
    m.set_prefill_chunk(16)
    kv = m.alloc_kv(64)
    tok = m.forward_greedy(prompt, kv)
    got = m.current_logits()
    assert _rel(got, ref_logits) < 5e-2
    assert tok == int(np.argmax(ref_logits)) or _margin(ref_logits) <= 1e-2
    kv.free()
    m.destroy()


@pytest.mark.parametrize("cfg", CFGS, ids=IDS)
def test_verification_batch_in_one_pass(E, cfg):
    """forward_greedy_all: the greedy token after every supplied position from ONE pass over the weights
    (forward.rs:268-358), equal to the step-by-step answers wherever the step-by-step margin is large."""
    tens = S.make_dense_model(cfg, seed=24)
    toks = [7, 3, 99, 250, 12, 5, 41, 8, 19]
    m = E.CudaModel.load_with(cfg, tens)
    kv = m.alloc_kv(64)
    m.set_prefill_chunk(0)
    m.forward_greedy([1, 2], kv)
    launches0 = m.launch_count()
    want, margins = [], []
    for t in toks:
        want.append(m.forward_greedy([t], kv))
        margins.append(_margin(m.current_logits()))
    launches_step = m.launch_count() - launches0
    want_logits = m.current_logits()
    kv2 = m.alloc_kv(64)
    m.forward_greedy([1, 2], kv2)
    m.set_prefill_chunk(16)
    launches0 = m.launch_count()
    got = m.forward_greedy_all(toks, kv2)
    launches_chunk = m.launch_count() - launches0
    assert kv2.len == 2 + len(toks)
    assert margin_gated_equal(list(got), want, margins)
    assert _rel(m.current_logits(), want_logits) < TF_WORST
    assert launches_chunk < launches_step / 3, (launches_chunk, launches_step)
    # accept the first four, move the length back, continue from there
    kv2.len = 2 + 4
    again = m.forward_greedy_all(toks[4:], kv2)
    assert margin_gated_equal(list(again), want[4:], margins[4:])
    # more tokens than one pass holds
    kv3 = m.alloc_kv(64)
    long_toks = [int(t) for t in np.random.default_rng(3).integers(0, cfg["n_vocab"], 40)]
    m.set_prefill_chunk(0)
    want_long = m.forward_greedy_all(long_toks, kv3)
    kv3.len = 0
    m.set_prefill_chunk(16)
    got_long = m.forward_greedy_all(long_toks, kv3)
    agree = np.mean([a == b for a, b in zip(got_long, want_long)])
    assert agree >= 0.8, agree
    with pytest.raises(E.TfrError, match="context full"):
        m.forward_greedy_all(list(range(60)), kv2)
    for k in (kv, kv2, kv3):
        k.free()
    m.destroy()


def test_hybrid_and_shortlisted_models_keep_the_step_route(E):
    cfg = S.TINY_HYBRID
    m = E.CudaModel.load_with(cfg, S.make_model(cfg, seed=2))
    assert m.prefill_chunk() == 0
    kv = m.alloc_kv(32)
    assert isinstance(m.forward_greedy([1, 2, 3, 4], kv), int)
    kv.free()
    m.destroy()
