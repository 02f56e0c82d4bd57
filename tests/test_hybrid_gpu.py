"""Hybrid (Gated-DeltaNet + gated full attention) layers through the C ABI (needs a B200).

Operator-level checks compare the fused kernels with the reference's own kernels (when the
reference cubin travels with the tree) and with the CPU restatement; model-level checks are
teacher-forced per layer, as for the dense models (see test_engine_gpu.py for why).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from taraference_b200 import synth as S  # noqa: E402
from test_engine_gpu import TF_TYPICAL, TF_WORST, _rel, margin_gated_equal, teacher_forced_errors  # noqa: E402

# head_dim 256 with four query heads per KV head and a partial rotary width, as the 4B-class hybrid
SMALL_HYBRID = dict(arch="qwen35", n_layer=4, n_embd=512, n_head=4, n_kv=1, head_dim=256, n_ff=1024, n_vocab=1000,
                    rope_theta=1e7, eps=1e-6, tied=True, qkv_bias=False, rope_dim=64, ssm_n_k=2, ssm_n_v=4,
                    ssm_state=128, conv_kernel=4, full_attention_interval=4)


@pytest.fixture(scope="module")
def E(cuda_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from taraference_b200 import engine
    return engine


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _gdn_inputs(rng, nk, nv, d, kernel):
    ch = (2 * nk + nv) * d
    conv_w = rng.uniform(-0.5, 0.5, ch * kernel).astype(np.float32)
    a = (-rng.uniform(0.5, 16.0, nv)).astype(np.float32)
    dt = np.log(np.expm1(rng.uniform(0.001, 0.1, nv))).astype(np.float32)
    norm_w = rng.uniform(0.5, 1.5, d).astype(np.float32)
    return ch, conv_w, a, dt, norm_w


def _window_from_ring(ring, steps_done, kernel, ch):
    """The reference's [kernel-1][channels] history, oldest first, out of the position-indexed ring."""
    ring = ring.reshape(kernel, ch)
    return np.stack([ring[(steps_done - (kernel - 1) + k) % kernel] for k in range(kernel - 1)])


@pytest.mark.parametrize("nk,nv,kernel", [(2, 4, 4), (16, 32, 4), (3, 3, 2), (1, 5, 3)])
def test_gdn_step_vs_oracle_and_reference(E, oracle, nk, nv, kernel):
    """Six consecutive decode steps: mixer output, recurrent state and conv history."""
    from oracle import ref_gpu
    rng = np.random.default_rng(100 + nk + nv)
    d, eps = 128, 1e-6
    ch, conv_w, a, dt, norm_w = _gdn_inputs(rng, nk, nv, d, kernel)
    vd = nv * d
    g_ring = torch.zeros(kernel * ch, device="cuda")
    g_state = torch.zeros(nv * d * d, device="cuda")
    g_out = torch.zeros(vd, device="cuda")
    o_win = np.zeros((kernel - 1) * ch, np.float32)
    o_state = np.zeros(nv * d * d, np.float32)
    use_ref = ref_gpu.available() and kernel <= 4
    if use_ref:
        r_win = torch.zeros((kernel - 1) * ch, device="cuda")
        r_state = torch.zeros(nv * d * d, device="cuda")
    dev = [_t(x) for x in (conv_w, a, dt, norm_w)]
    for step in range(6):
        proj = np.concatenate([rng.normal(0, 1.0, ch), rng.normal(0, 1.0, vd), rng.normal(0, 1.5, nv),
                               rng.normal(0, 1.5, nv)]).astype(np.float32)
        gp = _t(proj)
        E.op_gdn_step(gp, dev[0], g_ring, g_state, dev[1], dev[2], dev[3], g_out, nk, nv, d, kernel, step % kernel, eps)
        torch.cuda.synchronize()
        qkv, z, beta, alpha = proj[:ch], proj[ch:ch + vd], proj[ch + vd:ch + vd + nv], proj[ch + vd + nv:]
        oy = oracle.gdn_step(qkv, z, beta, alpha, conv_w, o_win, o_state, a, dt, norm_w, nk, nv, d, kernel, eps)
        gy = g_out.cpu().numpy()
        assert _rel(gy, oy) < 2e-5, (step, _rel(gy, oy))
        assert _rel(g_state.cpu().numpy(), o_state) < 2e-5
        win = _window_from_ring(g_ring.cpu().numpy(), step + 1, kernel, ch)
        assert np.array_equal(win.reshape(-1), o_win), "conv history must hold the raw projections bit for bit"
        if use_ref:
            rq, rk, rv = ref_gpu.gdn_conv_qkvl2(gp[:ch].contiguous(), dev[0], r_win, nk, nv, d, kernel, eps)
            ry = ref_gpu.gdn_delta_gated_d128(rq, rk, rv, gp[ch + vd + nv:].contiguous(), gp[ch + vd:ch + vd + nv].contiguous(),
                                              dev[2], dev[1], r_state, dev[3], gp[ch:ch + vd].contiguous(), nk, nv, eps)
            torch.cuda.synchronize()
            assert _rel(gy, ry.cpu().numpy()) < 5e-6, (step, _rel(gy, ry.cpu().numpy()))
            assert _rel(g_state.cpu().numpy(), r_state.cpu().numpy()) < 5e-6
            assert np.array_equal(win.reshape(-1), r_win.cpu().numpy())


@pytest.mark.parametrize("H,Hkv,hd,n_rot", [(4, 1, 256, 64), (16, 4, 256, 64), (2, 1, 128, 32), (4, 2, 64, 64)])
def test_qk_norm_rope_store_vs_oracle_and_reference(E, oracle, H, Hkv, hd, n_rot):
    from oracle import ref_gpu
    rng = np.random.default_rng(7 + H + hd)
    theta, eps, pos, max_seq = 1e7, 1e-6, 37, 64
    qn, kvn = H * hd, Hkv * hd
    raw = rng.normal(0, 1.0, 2 * qn + 2 * kvn).astype(np.float32)
    qw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    kw = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    q_out, g_out = torch.zeros(qn, device="cuda"), torch.zeros(qn, device="cuda")
    kc = torch.zeros(max_seq * kvn, dtype=torch.int16, device="cuda")
    vc = torch.zeros(max_seq * kvn, dtype=torch.int16, device="cuda")
    E.op_qk_norm_rope_store(_t(raw), _t(qw), _t(kw), q_out, g_out, kc, vc, H, Hkv, hd, n_rot, pos, theta, eps)
    torch.cuda.synchronize()
    qg = raw[:2 * qn].reshape(H, 2, hd)
    oq = oracle.qk_norm_partial_rope(qg[:, 0].reshape(-1), qw, H, hd, n_rot, pos, theta, eps)
    ok = oracle.qk_norm_partial_rope(raw[2 * qn:2 * qn + kvn], kw, Hkv, hd, n_rot, pos, theta, eps)
    assert np.array_equal(g_out.cpu().numpy(), qg[:, 1].reshape(-1))
    assert _rel(q_out.cpu().numpy(), oq) < 1e-5
    krow = kc.cpu().numpy().view(np.uint16).reshape(max_seq, kvn)
    vrow = vc.cpu().numpy().view(np.uint16).reshape(max_seq, kvn)
    assert not krow[:pos].any() and not krow[pos + 1:].any(), "only row pos may be written"
    assert _rel(oracle.half_to_float(krow[pos]), ok) < 2e-3  # f16 storage
    assert np.array_equal(vrow[pos], oracle.float_to_half_bits(raw[2 * qn + kvn:]))
    if ref_gpu.available():
        rq, rg = ref_gpu.split_q_gate(_t(raw[:2 * qn]), H, hd)
        ref_gpu.qk_norm_partial_rope(rq, _t(qw), H, hd, n_rot, pos, theta, eps)
        rk = _t(raw[2 * qn:2 * qn + kvn].copy())
        ref_gpu.qk_norm_partial_rope(rk, _t(kw), Hkv, hd, n_rot, pos, theta, eps)
        rkc = torch.zeros(max_seq * kvn, dtype=torch.int16, device="cuda")
        ref_gpu.copy_kv(rk, rkc, pos, kvn)
        torch.cuda.synchronize()
        assert _rel(q_out.cpu().numpy(), rq.cpu().numpy()) < 2e-6
        assert np.array_equal(g_out.cpu().numpy(), rg.cpu().numpy())
        same = (rkc.cpu().numpy() == kc.cpu().numpy()).mean()
        assert same > 0.995, same  # f16 bits; a last-bit difference before rounding may flip one


def test_attention_gated_matches_gate_after_attention(E):
    rng = np.random.default_rng(5)
    H, Hkv, hd, pos, max_seq = 4, 1, 256, 100, 128
    q = _t(rng.normal(0, 1, H * hd).astype(np.float32))
    gate = _t(rng.normal(0, 2, H * hd).astype(np.float32))
    kc = _t(rng.normal(0, 1, max_seq * Hkv * hd).astype(np.float16)).view(torch.int16)
    vc = _t(rng.normal(0, 1, max_seq * Hkv * hd).astype(np.float16)).view(torch.int16)
    plain, gated = torch.zeros(H * hd, device="cuda"), torch.zeros(H * hd, device="cuda")
    E.op_attention(q, kc, vc, plain, H, Hkv, hd, pos)
    E.op_attention_gated(q, kc, vc, gate, gated, H, Hkv, hd, pos)
    torch.cuda.synchronize()
    want = plain * torch.sigmoid(gate)
    assert _rel(gated.cpu().numpy(), want.cpu().numpy()) < 2e-6


@pytest.mark.parametrize("cfg", [S.TINY_HYBRID, SMALL_HYBRID], ids=["tiny", "small256"])
def test_teacher_forced_hybrid_layers_vs_reference_kernels(E, cfg):
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("reference cubin not present")
    cfg = dict(cfg, n_layer=8)
    tens = S.make_model(cfg, seed=4)
    rm = ref_gpu.RefModel(cfg, tens, 64)
    m = E.CudaModel.load_with(cfg, tens)
    kv = m.alloc_kv(64)
    to_t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32).copy()).cuda()
    le, he = teacher_forced_errors(
        m, kv, lambda t: ref_gpu.embed(rm.embd, t).cpu().numpy(),
        lambda li, x, pos: rm.layer_forward(li, to_t(x), pos).cpu().numpy(),
        lambda x: rm.head_forward(to_t(x)).cpu().numpy(), cfg, [1, 2, 3, 250, 7, 9, 11])
    assert np.median(le) < TF_TYPICAL and np.median(he) < TF_TYPICAL, (le, he)
    assert (le < 1e-5).mean() >= 0.8, le
    assert le.max() < TF_WORST and he.max() < TF_WORST, (le, he)
    # the recurrent state the two sides carried through the seven tokens
    for li in (0, 1, 2, 4):
        gs = m.debug_read("ssm_state", cfg["ssm_n_v"] * 128 * 128, kv=kv, layer=li)
        assert _rel(gs, rm.ssm[li].cpu().numpy()) < 1e-2
        ch = (2 * cfg["ssm_n_k"] + cfg["ssm_n_v"]) * 128
        gc = m.debug_read("conv_state", 3 * ch, kv=kv, layer=li)
        assert _rel(gc, rm.conv[li].cpu().numpy()) < 1e-2
    kv.free()
    m.destroy()


@pytest.mark.parametrize("cfg", [S.TINY_HYBRID, SMALL_HYBRID], ids=["tiny", "small256"])
def test_teacher_forced_hybrid_layers_vs_cpu_oracle(E, oracle, cfg):
    tens = S.make_model(cfg, seed=3)
    om = oracle.OracleModel(cfg, tens, 64)
    m = E.CudaModel.load_with(cfg, tens)
    kv = m.alloc_kv(64)
    le, he = teacher_forced_errors(m, kv, om.embed, om.layer_forward, om.head_forward, cfg, [5, 17, 3, 250, 9])
    assert np.median(le) < 2e-5 and np.median(he) < 2e-5, (le, he)
    assert le.max() < TF_WORST and he.max() < TF_WORST, (le, he)
    # move the KV length back: the recurrent state keeps everything it absorbed (the reference assigns
    # cache.len the same way) and the conv history must stay aligned although positions repeat
    kv.len = 2
    le2, he2 = teacher_forced_errors(m, kv, om.embed, om.layer_forward, om.head_forward, cfg, [8, 21, 4], pos0=2)
    assert np.median(le2) < 2e-5 and le2.max() < TF_WORST and he2.max() < TF_WORST, (le2, he2)
    kv.free()
    m.destroy()


@pytest.mark.parametrize("cfg", [S.TINY_HYBRID, SMALL_HYBRID], ids=["tiny", "small256"])
def test_free_running_hybrid_tokens_and_state_reset(E, oracle, cfg):
    tens = S.make_model(cfg, seed=6)
    om = oracle.OracleModel(cfg, tens, 64)
    m = E.CudaModel.load_with(cfg, tens)
    kv = m.alloc_kv(64)
    prompt = [5, 17, 3, 250, 9]
    nxt = m.forward_greedy(prompt, kv)
    for i, t in enumerate(prompt):
        ologits = om.decode_token(i, t)
    glogits = m.current_logits()
    from tests.test_engine_gpu import free_running_bound
    bound, self_dev = free_running_bound(cfg, tens, prompt)
    print(f"engine vs CPU oracle {_rel(glogits, ologits):.2e}; reference vs itself {self_dev}; bound {bound:.2e}")
    assert _rel(glogits, ologits) < bound, (_rel(glogits, ologits), bound, self_dev)
    toks = m.decode_burst(nxt, 20, kv)
    otoks, omarg, _ = om.decode_greedy(5, nxt, 20)
    assert len(toks) == 20 and kv.len == 25
    assert margin_gated_equal(toks, otoks, omarg), (toks, otoks, omarg)
    # a cleared cache with zeroed recurrent state reproduces the run bit for bit; without the
    # reset the old state leaks into the new sequence
    kv.clear()
    m.zero_recurrent(kv)
    assert m.forward_greedy(prompt, kv) == nxt
    assert np.array_equal(m.current_logits(), glogits)
    assert np.array_equal(m.decode_burst(nxt, 20, kv), toks)
    kv.clear()
    m.forward_greedy(prompt, kv)
    assert not np.array_equal(m.current_logits(), glogits)
    kv.free()
    m.destroy()


def test_graph_and_plain_launches_agree_hybrid(E):
    cfg = S.TINY_HYBRID
    tens = S.make_model(cfg, seed=9)
    outs = []
    for graph in (True, False):
        m = E.CudaModel.load_with(cfg, tens)
        m.set_cuda_graph(graph)
        kv = m.alloc_kv(48)
        nxt = m.forward_greedy([4, 8, 15, 16, 23, 42], kv)
        outs.append((nxt, m.decode_burst(nxt, 24, kv), m.current_logits()))
        kv.free()
        m.destroy()
    assert outs[0][0] == outs[1][0] and np.array_equal(outs[0][1], outs[1][1]) and np.array_equal(outs[0][2], outs[1][2])


def test_hybrid_config_errors(E):
    cfg = dict(S.TINY_HYBRID, ssm_state=64)
    m = E.CudaModel(0)
    with pytest.raises(E.TfrError):
        m.set_config(cfg)
    with pytest.raises(E.TfrError):
        m.set_config(dict(S.TINY_HYBRID, conv_kernel=5))
    m.destroy()
    # a linear layer without its projections fails at finalize with the tensor's name
    tens = S.make_model(S.TINY_HYBRID, seed=1)
    del tens["blk.0.ssm_beta.weight"]
    with pytest.raises(E.TfrError, match="ssm_beta"):
        E.CudaModel.load_with(S.TINY_HYBRID, tens)


def test_full_size_hybrid_4b_shapes_teacher_forced(E, oracle):
    """Four layers (three Gated-DeltaNet + one gated full attention) at the full hybrid 4B shape — 8192-channel
    conv, 32 V heads, head_dim 256, 151 936-row tied head — against the reference's kernels and the CPU oracle,
    layer by layer with identical inputs."""
    from oracle import ref_gpu
    from taraference_b200 import synth_gpu
    cfg = dict(S.QWEN35_4B, n_layer=4)
    m, host = synth_gpu.build_model(cfg, seed=0, keep_host=True)
    kv = m.alloc_kv(32)
    toks_in = [100, 2000, 30000, 151000, 7]
    to_t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32).copy()).cuda()
    if ref_gpu.available():
        rm = ref_gpu.RefModel(cfg, host, 32)
        le, he = teacher_forced_errors(
            m, kv, lambda t: ref_gpu.embed(rm.embd, t).cpu().numpy(),
            lambda li, x, pos: rm.layer_forward(li, to_t(x), pos).cpu().numpy(),
            lambda x: rm.head_forward(to_t(x)).cpu().numpy(), cfg, toks_in)
        assert np.median(le) < TF_TYPICAL and (le < 1e-5).mean() >= 0.5 and le.max() < TF_WORST, le
        assert he.max() < TF_WORST and np.median(he) < TF_TYPICAL, he
        gs = m.debug_read("ssm_state", cfg["ssm_n_v"] * 128 * 128, kv=kv, layer=1)
        assert _rel(gs, rm.ssm[1].cpu().numpy()) < 1e-2
        kv.clear()
        m.zero_recurrent(kv)
    oracle.set_threads(oracle.max_threads())
    om = oracle.OracleModel(cfg, host, 32)
    le, he = teacher_forced_errors(m, kv, om.embed, om.layer_forward, om.head_forward, cfg, toks_in[:3])
    oracle.set_threads(1)
    assert np.median(le) < 5e-5 and le.max() < TF_WORST and he.max() < TF_WORST, (le, he)
    kv.free()
    m.destroy()


def test_hybrid_with_q5_k_and_q8_0_tensors(E, oracle):
    """The tensor mix of real hybrid files: attn_qkv and ssm_out as Q5_K (converted to Q8_0 at upload, the other
    three projections stay Q4_K, so the four are launched one by one), attn_output as Q8_0."""
    cfg = S.TINY_HYBRID
    tens = S.make_model(cfg, seed=5)
    rng = np.random.default_rng(1)
    oracle_tens = dict(tens)
    for name in list(tens):
        if name.endswith("attn_qkv.weight") or name.endswith("ssm_out.weight"):
            t, K, N, _ = tens[name]
            q5 = S.random_q5_k(rng, N * (K // 256), d_sigma=0.0015).reshape(-1)
            tens[name] = (S.Q5_K, K, N, q5)
            oracle_tens[name] = (S.Q8_0, K, N, oracle.transcode_to_q8_0(S.Q5_K, q5))
        elif name.endswith("attn_output.weight"):
            t, K, N, _ = tens[name]
            q8 = S.quantize_q8_0(rng.normal(0, 0.02, (N, K)).astype(np.float32)).reshape(-1)
            tens[name] = oracle_tens[name] = (S.Q8_0, K, N, q8)
    om = oracle.OracleModel(cfg, oracle_tens, 32)
    m = E.CudaModel.load_with(cfg, tens)
    kv = m.alloc_kv(32)
    le, he = teacher_forced_errors(m, kv, om.embed, om.layer_forward, om.head_forward, cfg, [5, 17, 3, 250])
    assert np.median(le) < 2e-5 and le.max() < TF_WORST and he.max() < TF_WORST, (le, he)
    kv.free()
    m.destroy()
