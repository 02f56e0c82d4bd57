"""The CPU oracle against independent implementations and brute force (no GPU)."""
import numpy as np
import pytest

from taraference_b200 import synth as S


def brute_q4k(block: np.ndarray) -> np.ndarray:
    """Straight reading of the Q4_K layout (kernels/common.cu:40-84) in numpy."""
    d = block[0:2].view(np.float16)[0].astype(np.float32)
    dmin = block[2:4].view(np.float16)[0].astype(np.float32)
    sc = block[4:16]
    out = np.zeros(256, np.float32)
    for j in range(8):
        if j < 4:
            s, m = sc[j] & 63, sc[j + 4] & 63
        else:
            s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4)
            m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)
        t = j // 2
        qs = block[16 + 32 * t: 48 + 32 * t]
        nib = (qs >> 4) if (j & 1) else (qs & 0xF)
        out[32 * j: 32 * j + 32] = (d * np.float32(s)) * nib.astype(np.float32) - dmin * np.float32(m)
    return out


def test_block_decode_matches_gguf_py(oracle):
    gguf = pytest.importorskip("gguf")
    from gguf import GGMLQuantizationType as T, quants
    rng = np.random.default_rng(1)
    b4, b6 = S.random_q4_k(rng, 97), S.random_q6_k(rng, 97)
    r4 = quants.dequantize(b4.reshape(-1), T.Q4_K).reshape(-1)
    r6 = quants.dequantize(b6.reshape(-1), T.Q6_K).reshape(-1)
    o4 = oracle.dequant_rows(oracle.Q4_K, b4.reshape(-1), 256 * 97, 1).reshape(-1)
    o6 = oracle.dequant_rows(oracle.Q6_K, b6.reshape(-1), 256 * 97, 1).reshape(-1)
    assert np.array_equal(r4, o4)
    assert np.array_equal(r6, o6)


def test_q4k_brute_force(oracle):
    rng = np.random.default_rng(2)
    b = S.random_q4_k(rng, 5)
    o = oracle.dequant_rows(oracle.Q4_K, b.reshape(-1), 256 * 5, 1).reshape(5, 256)
    for i in range(5):
        assert np.array_equal(o[i], brute_q4k(b[i]))


def test_f16_widening_all_values(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    ours = np.array([oracle.lib().tfo_half_to_float(int(b)) for b in bits[::7]], np.float32)
    ref = bits[::7].view(np.float16).astype(np.float32)
    ok = (ours == ref) | (np.isnan(ours) & np.isnan(ref))
    assert ok.all()


def test_f16_store_rounding(oracle):
    """common.cu:9-38: like IEEE round-to-nearest except exact ties round away from zero."""
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-4, 2000), rng.normal(0, 300, 2000),
                        [0.0, -0.0, 65504.0, 65520.0, 70000.0, 1e-8, 5.9e-8, 6e-8, 1e-7, -3e-5]]).astype(np.float32)
    ours = oracle.float_to_half_bits(x)
    ieee = x.astype(np.float16).view(np.uint16)
    diff = ours.astype(np.int32) - ieee.astype(np.int32)
    # differs from RNE only on ties (by one ulp upward in magnitude) and in overflow handling
    assert (np.abs(diff) <= 1).mean() > 0.999
    # explicit tie: 1 + 2^-11 is halfway between two halfs; RNE keeps 1.0, the reference rounds up
    tie = np.array([1.0 + 2.0 ** -11], np.float32)
    assert oracle.float_to_half_bits(tie)[0] == 0x3C01
    assert tie.astype(np.float16).view(np.uint16)[0] == 0x3C00
    assert oracle.float_to_half_bits(np.array([70000.0], np.float32))[0] == 0x7C00
    assert oracle.float_to_half_bits(np.array([1e-8], np.float32))[0] == 0


def test_quantizer_definition(oracle):
    rng = np.random.default_rng(4)
    x = rng.normal(0, 1, 2048).astype(np.float32)
    x[64:96] = 0.0                      # zero group
    x[96:128] = 1e-30                   # tiny group
    q, d = oracle.quantize_q8(x)
    xr = x.reshape(-1, 32)
    amax = np.abs(xr).max(1)
    assert np.array_equal(d, (amax * np.float32(1.0 / 127.0)).astype(np.float32))
    assert (q[64:96] == 0).all() and d[2] == 0
    assert np.abs(q).max() <= 127
    with np.errstate(divide="ignore", invalid="ignore"):
        expect = np.where(amax[:, None] == 0, 0, np.rint(xr / d[:, None]))
    assert np.array_equal(q.reshape(-1, 32), expect.astype(np.int8))


@pytest.mark.parametrize("K", [256, 2048, 11008])
def test_int_dots_and_float_combine(oracle, K):
    rng = np.random.default_rng(5)
    nb = K // 256
    x = rng.normal(0, 1, K).astype(np.float32)
    q8, d8 = oracle.quantize_q8(x)
    xq = (q8.astype(np.float64).reshape(-1, 32) * d8[:, None].astype(np.float64)).reshape(-1)
    b4 = S.random_q4_k(rng, nb)
    b6 = S.random_q6_k(rng, nb)
    # integer contract against brute force
    for b in range(nb):
        I, Sm = oracle.q4k_subdots(b4[b], q8[256 * b: 256 * b + 256])
        qs = b4[b][16:144].reshape(4, 32)
        a = q8[256 * b: 256 * b + 256].astype(np.int64).reshape(4, 2, 32)
        assert np.array_equal(I[0::2], ((qs & 0xF).astype(np.int64) * a[:, 0]).sum(1))
        assert np.array_equal(I[1::2], ((qs >> 4).astype(np.int64) * a[:, 1]).sum(1))
        assert np.array_equal(Sm, a.reshape(8, 32).sum(1))
        J = oracle.q6k_groupdots(b6[b], q8[256 * b: 256 * b + 256])
        w6 = oracle.dequant_rows(oracle.Q6_K, b6[b].copy(), 256, 1).reshape(-1)
        d = b6[b][208:210].view(np.float16)[0].astype(np.float64)
        sc = b6[b][192:208].view(np.int8).astype(np.float64)
        with np.errstate(divide="ignore", invalid="ignore"):
            qv = np.where(sc.repeat(16) != 0, np.rint(w6.astype(np.float64) / (d * sc.repeat(16))), 0)
        if d > 0 and (sc != 0).all():
            assert np.array_equal(J, (qv.reshape(16, 16) * q8[256 * b: 256 * b + 256].reshape(16, 16)).sum(1))
    # float combination against float64 dequantise-and-dot on the quantised activation
    m4 = oracle.mat(oracle.Q4_K, b4.reshape(-1).copy(), K, 1)
    m6 = oracle.mat(oracle.Q6_K, b6.reshape(-1).copy(), K, 1)
    w4 = oracle.dequant_rows(oracle.Q4_K, b4.reshape(-1), K, 1).astype(np.float64)
    w6 = oracle.dequant_rows(oracle.Q6_K, b6.reshape(-1), K, 1).astype(np.float64)
    assert np.allclose(oracle.gemv(m4, x), w4 @ xq, rtol=2e-5, atol=1e-3)
    assert np.allclose(oracle.gemv(m6, x), w6 @ xq, rtol=2e-5, atol=1e-3)
    assert np.allclose(oracle.gemv(m6, x, act_mode=1), w6 @ x.astype(np.float64), rtol=2e-5, atol=1e-3)


def test_gemv_bias_residual_and_linearity(oracle):
    rng = np.random.default_rng(6)
    K, N = 512, 24
    w = S.random_q6_k(rng, N * 2).reshape(-1)
    m = oracle.mat(oracle.Q6_K, w, K, N)
    x = rng.normal(0, 1, K).astype(np.float32)
    bias = rng.normal(0, 1, N).astype(np.float32)
    base = oracle.gemv(m, x)
    assert np.allclose(oracle.gemv(m, x, bias=bias), base + bias, rtol=1e-6, atol=1e-6)
    acc = np.full(N, 3.0, np.float32)
    oracle.gemv(m, x, out=acc, use_res=2)
    assert np.allclose(acc, base + 3.0, rtol=1e-6, atol=1e-5)
    # fp32-activation route is linear in x
    y2 = oracle.gemv(m, 2 * x, act_mode=1)
    assert np.allclose(y2, 2 * oracle.gemv(m, x, act_mode=1), rtol=1e-5, atol=1e-5)


def test_rope_rms_attention_against_numpy(oracle):
    rng = np.random.default_rng(7)
    H, Hkv, hd, T = 4, 2, 64, 37
    x = rng.normal(0, 1, 256).astype(np.float32)
    w = rng.normal(1, 0.1, 256).astype(np.float32)
    ref = x * (1.0 / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-6)) * w
    assert np.allclose(oracle.rms_norm(x, w, 1e-6), ref, rtol=1e-5)
    q = rng.normal(0, 1, H * hd).astype(np.float32)
    pos, theta = 11, 1e6
    r = oracle.rope_neox(q, H, hd, pos, theta).reshape(H, hd)
    i = np.arange(hd // 2)
    ang = pos * theta ** (-2.0 * i / hd)
    qq = q.reshape(H, hd).astype(np.float64)
    exp = np.concatenate([qq[:, :32] * np.cos(ang) - qq[:, 32:] * np.sin(ang),
                          qq[:, :32] * np.sin(ang) + qq[:, 32:] * np.cos(ang)], 1)
    assert np.allclose(r, exp, rtol=1e-4, atol=1e-5)
    kc = rng.normal(0, 1, (T, Hkv * hd)).astype(np.float16)
    vc = rng.normal(0, 1, (T, Hkv * hd)).astype(np.float16)
    out = oracle.attention(q, kc.view(np.uint16), vc.view(np.uint16), H, Hkv, hd, T - 1).reshape(H, hd)
    for h in range(H):
        g = h // (H // Hkv)
        s = (kc[:, g * hd:(g + 1) * hd].astype(np.float64) @ qq[h]) / np.sqrt(hd)
        p = np.exp(s - s.max())
        p /= p.sum()
        assert np.allclose(out[h], p @ vc[:, g * hd:(g + 1) * hd].astype(np.float64), rtol=1e-4, atol=1e-5)


def test_tiny_model_deterministic_and_threaded(oracle):
    cfg = S.TINY_DENSE
    tens = S.make_dense_model(cfg, 0)
    oracle.set_threads(1)
    a = oracle.OracleModel(cfg, tens, 32)
    ta, ma, la = a.decode_greedy(0, 5, 6)
    oracle.set_threads(4)
    b = oracle.OracleModel(cfg, tens, 32)
    tb, mb, lb = b.decode_greedy(0, 5, 6)
    oracle.set_threads(1)
    assert np.array_equal(ta, tb) and np.array_equal(la, lb)
    assert np.isfinite(la).all()
    # KV rows written for exactly the decoded positions
    assert (a.kc[:, :6] != 0).any() and (a.kc[:, 6:] == 0).all()


def gdn_step_f64(qkv, z, beta, alpha, conv_w, win, S_, a, dt, norm_w, nk, nv, d, kernel, eps):
    """Gated delta rule written as matrix algebra in float64 (kernels/deltanet.cu:530-728):
    S' = g S + k (x) ((v - (g S)^T k) beta),  o = S'^T q / sqrt(d),  y = rmsnorm(o) * w * silu(z)."""
    ch = (2 * nk + nv) * d
    win = win.reshape(kernel - 1, ch).astype(np.float64)
    w = conv_w.reshape(ch, kernel).astype(np.float64)
    acc = (w[:, :kernel - 1].T * win).sum(0) + w[:, kernel - 1] * qkv
    cv = acc / (1 + np.exp(-acc))
    new_win = np.concatenate([win[1:], qkv[None].astype(np.float64)]) if kernel > 1 else win
    Q, K, V = cv[:nk * d].reshape(nk, d), cv[nk * d:2 * nk * d].reshape(nk, d), cv[2 * nk * d:].reshape(nv, d)
    Q = Q / np.sqrt((Q * Q).sum(1, keepdims=True) + eps)
    K = K / np.sqrt((K * K).sum(1, keepdims=True) + eps)
    S_ = S_.reshape(nv, d, d).astype(np.float64).copy()
    y = np.zeros((nv, d))
    for h in range(nv):
        k, q = K[h % nk], Q[h % nk]
        b = 1 / (1 + np.exp(-beta[h]))
        zz = alpha[h] + dt[h]
        g = np.exp((zz if zz > 20 else np.log1p(np.exp(zz))) * a[h])
        Sg = g * S_[h]
        delta = (V[h] - Sg.T @ k) * b
        S_[h] = Sg + np.outer(k, delta)
        o = S_[h].T @ q / np.sqrt(d)
        zz_ = z[h * d:(h + 1) * d]
        y[h] = o / np.sqrt((o * o).mean() + eps) * norm_w * (zz_ / (1 + np.exp(-zz_)))
    return y.reshape(-1), S_.reshape(-1), new_win.reshape(-1)


@pytest.mark.parametrize("nk,nv,d,kernel", [(2, 4, 128, 4), (1, 3, 32, 2), (3, 3, 16, 3)])
def test_gdn_step_matches_float64_algebra(oracle, nk, nv, d, kernel):
    rng = np.random.default_rng(nk * 10 + nv)
    ch, vd, eps = (2 * nk + nv) * d, nv * d, 1e-6
    conv_w = rng.uniform(-0.5, 0.5, ch * kernel).astype(np.float32)
    a = (-rng.uniform(0.5, 16.0, nv)).astype(np.float32)
    dt = np.log(np.expm1(rng.uniform(0.001, 0.1, nv))).astype(np.float32)
    norm_w = rng.uniform(0.5, 1.5, d).astype(np.float32)
    win, st = np.zeros((kernel - 1) * ch, np.float32), np.zeros(nv * d * d, np.float32)
    win64, st64 = win.astype(np.float64), st.astype(np.float64)
    for step in range(5):
        qkv, z = rng.normal(0, 1, ch).astype(np.float32), rng.normal(0, 1, vd).astype(np.float32)
        beta, alpha = rng.normal(0, 1.5, nv).astype(np.float32), rng.normal(0, 1.5, nv).astype(np.float32)
        y = oracle.gdn_step(qkv, z, beta, alpha, conv_w, win, st, a, dt, norm_w, nk, nv, d, kernel, eps)
        y64, st64, win64 = gdn_step_f64(qkv, z, beta, alpha, conv_w, win64, st64, a, dt, norm_w, nk, nv, d, kernel, eps)
        assert np.allclose(y, y64, rtol=2e-4, atol=2e-5), step
        assert np.allclose(st, st64, rtol=2e-4, atol=2e-6), step
        assert np.array_equal(win.astype(np.float64), win64), "the conv window holds the raw inputs"
    assert np.abs(st).max() > 0 and np.isfinite(st).all()


def test_qk_norm_partial_rope_properties(oracle):
    rng = np.random.default_rng(3)
    H, hd, n_rot, theta, eps = 3, 64, 16, 1e7, 1e-6
    x = rng.normal(0, 1, H * hd).astype(np.float32)
    w = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    y0 = oracle.qk_norm_partial_rope(x, w, H, hd, n_rot, 0, theta, eps).reshape(H, hd)
    xn = x.reshape(H, hd).astype(np.float64)
    want = xn / np.sqrt((xn * xn).mean(1, keepdims=True) + eps) * w
    assert np.allclose(y0, want, rtol=1e-5, atol=1e-6)          # position 0: rotation is the identity
    y9 = oracle.qk_norm_partial_rope(x, w, H, hd, n_rot, 9, theta, eps).reshape(H, hd)
    assert np.array_equal(y9[:, n_rot:], y0[:, n_rot:])         # dims beyond n_rot are not rotated
    half = n_rot // 2
    for i in range(half):                                       # rotation preserves each pair's norm
        n0 = y0[:, i] ** 2 + y0[:, i + half] ** 2
        n9 = y9[:, i] ** 2 + y9[:, i + half] ** 2
        assert np.allclose(n0, n9, rtol=1e-4)
    ang = 9 * theta ** (-2.0 * 1 / n_rot)
    assert np.allclose(y9[:, 1], y0[:, 1] * np.cos(ang) - y0[:, 1 + half] * np.sin(ang), rtol=1e-4, atol=1e-5)


def test_tiny_hybrid_model_layer_kinds_state_and_reset(oracle):
    cfg = S.TINY_HYBRID
    tens = S.make_model(cfg, 2)
    om = oracle.OracleModel(cfg, tens, 32)
    assert om.kinds == [oracle.LAYER_LINEAR] * 3 + [oracle.LAYER_FULL_GATED]
    toks, margins, last = om.decode_greedy(0, 5, 6)
    assert np.isfinite(last).all()
    # linear layers leave no KV rows, the full-attention layer fills exactly the decoded positions
    assert not om.kc[:3].any() and om.kc[3, :6].any() and not om.kc[3, 6:].any()
    assert om.ssm[:3].any() and not om.ssm[3].any() and om.conv[:3].any()
    om.zero_recurrent()
    t2, _, l2 = om.decode_greedy(0, 5, 6)
    assert np.array_equal(toks, t2) and np.array_equal(last, l2)
    t3, _, l3 = om.decode_greedy(0, 5, 6)  # state carried over: a different sequence state
    assert not np.array_equal(last, l3)


def test_q8_0_dot_and_transcodes_against_independent_restatements(oracle):
    """Q8_0 x Q8 dots against numpy; the loader's Q5_K / Q5_1 -> Q8_0 conversion against gguf-py's
    block decode followed by a numpy Q8_0 quantiser."""
    gguf = pytest.importorskip("gguf")
    from gguf import GGMLQuantizationType as T, quants
    rng = np.random.default_rng(9)
    K, N = 512, 5
    w = rng.normal(0, 0.05, (N, K)).astype(np.float32)
    raw = S.quantize_q8_0(w)
    assert np.array_equal(quants.dequantize(raw.reshape(-1), T.Q8_0).reshape(N, K),
                          raw[..., 0:2].copy().view(np.float16).astype(np.float32).repeat(32, -1).reshape(N, K)
                          * raw[..., 2:].view(np.int8).reshape(N, K))
    x = rng.normal(0, 1, K).astype(np.float32)
    q8, d8 = oracle.quantize_q8(x)
    m = oracle.mat(oracle.Q8_0, raw.reshape(-1), K, N)
    y = oracle.gemv(m, x)
    qw = raw[..., 2:].view(np.int8).astype(np.int64).reshape(N, K // 32, 32)
    sums = (qw * q8.astype(np.int64).reshape(K // 32, 32)).sum(-1)
    assert np.array_equal(oracle.q8_0_blockdots(raw[3].reshape(-1), K, q8), sums[3].astype(np.int32))
    dw = raw[..., 0:2].copy().view(np.float16).astype(np.float64).reshape(N, K // 32)
    assert np.allclose(y, (dw * d8 * sums).sum(-1), rtol=1e-5, atol=1e-7)
    # transcodes
    for src, blocks, gt in ((S.Q5_K, S.random_q5_k(rng, 37), T.Q5_K), (S.Q5_1, S.random_q5_1(rng, 64), T.Q5_1)):
        vals = quants.dequantize(blocks.reshape(-1), gt).reshape(-1, 32).astype(np.float32)
        want = S.quantize_q8_0(vals.reshape(1, -1)).reshape(-1, 34)
        got = oracle.transcode_to_q8_0(src, blocks).reshape(-1, 34)
        assert np.array_equal(got[:, :2], want[:, :2])                      # fp16 scales
        dq = got[:, 2:].view(np.int8).astype(np.int32) - want[:, 2:].view(np.int8).astype(np.int32)
        # gguf-py decodes with numpy broadcasting (same products, possibly another rounding of the last bit of a
        # value that sits on a rounding border): allow isolated +-1
        assert np.abs(dq).max() <= 1 and (dq != 0).mean() < 2e-3, (np.abs(dq).max(), (dq != 0).mean())
