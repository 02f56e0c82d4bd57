"""Operator-level parity of the CUDA library through the C ABI (needs a B200).

Three checkers: the CPU oracle (exact IEEE restatement), the reference's own kernels
compiled unmodified and run on the same GPU (oracle/ref_gpu.py, when its cubin travelled
with the repo), and brute-force numpy for integer quantities.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from taraference_b200 import synth as S  # noqa: E402


@pytest.fixture(scope="module")
def E(cuda_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from taraference_b200 import engine
    return engine


@pytest.fixture(scope="module")
def R():
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("reference cubin not present")
    return ref_gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def act_vectors(rng, K):
    x = rng.normal(0, 1, K).astype(np.float32)
    x[0:32] = 0.0                     # all-zero group
    x[32:64] *= 1e-20                 # tiny group
    x[64:96] *= 1e4                   # large group
    x[96] = np.abs(x[96:128]).max() * 2  # amax element positive
    return x


@pytest.mark.parametrize("K", [256, 2048, 11008, 27648])
def test_quantizer_bit_exact_vs_reference_build(E, R, oracle, K):
    rng = np.random.default_rng(K)
    mism = 0
    for rep in range(4):
        x = act_vectors(rng, K) if rep == 0 else rng.normal(0, rng.uniform(0.01, 30), K).astype(np.float32)
        xd = dev(x)
        q = torch.zeros(K, dtype=torch.int8, device="cuda")
        d = torch.zeros(K // 32, dtype=torch.float32, device="cuda")
        E.op_quantize_q8(xd, q, d)
        rq, rd = R.quantize_q8(xd)
        torch.cuda.synchronize()
        assert torch.equal(q, rq), "int8 activation differs from the reference build"
        assert torch.equal(d.view(torch.int32), rd.view(torch.int32))
        mism += int((q.cpu().numpy() != oracle.quantize_q8(x)[0]).sum())
    # the IEEE-division CPU oracle may differ by one unit on a few elements per 1e5
    assert mism <= max(2, int(4 * K * 1e-3))


def test_quantizer_vs_cpu_oracle_mismatch_rate(E, oracle):
    rng = np.random.default_rng(0)
    n = 1 << 20
    x = rng.normal(0, 1, n).astype(np.float32)
    q = torch.zeros(n, dtype=torch.int8, device="cuda")
    d = torch.zeros(n // 32, dtype=torch.float32, device="cuda")
    E.op_quantize_q8(dev(x), q, d)
    oq, od = oracle.quantize_q8(x)
    diff = q.cpu().numpy().astype(np.int32) - oq.astype(np.int32)
    assert np.array_equal(d.cpu().numpy(), od)
    assert np.abs(diff).max() <= 1
    assert (diff != 0).mean() < 2e-4, (diff != 0).mean()


@pytest.mark.parametrize("wtype,K,N", [(S.Q4_K, 256, 3), (S.Q4_K, 2048, 37), (S.Q4_K, 5120, 9), (S.Q6_K, 256, 5),
                                       (S.Q6_K, 2048, 19), (S.Q6_K, 11008, 7)])
def test_integer_sub_block_dots_bit_exact(E, oracle, wtype, K, N):
    rng = np.random.default_rng(K + N)
    nb = K // 256
    blocks = (S.random_q4_k if wtype == S.Q4_K else S.random_q6_k)(rng, N * nb)
    q8 = rng.integers(-127, 128, K, dtype=np.int8)
    d8 = np.ones(K // 32, np.float32)
    m = E.GpuMat(wtype, K, N, blocks.reshape(-1))
    if wtype == S.Q4_K:
        a = torch.zeros((N, K // 32), dtype=torch.int32, device="cuda")
        b = torch.zeros((N, K // 32), dtype=torch.int32, device="cuda")
        E.op_int_dots(m, dev(q8), dev(d8), a, b)
        a, b = a.cpu().numpy(), b.cpu().numpy()
        for r in range(N):
            for bi in range(nb):
                I, Sm = oracle.q4k_subdots(blocks[r * nb + bi], q8[256 * bi: 256 * bi + 256])
                assert np.array_equal(a[r, 8 * bi: 8 * bi + 8], I)
                assert np.array_equal(b[r, 8 * bi: 8 * bi + 8], Sm)
    else:
        a = torch.zeros((N, K // 16), dtype=torch.int32, device="cuda")
        E.op_int_dots(m, dev(q8), dev(d8), a)
        a = a.cpu().numpy()
        for r in range(N):
            for bi in range(nb):
                J = oracle.q6k_groupdots(blocks[r * nb + bi], q8[256 * bi: 256 * bi + 256])
                assert np.array_equal(a[r, 16 * bi: 16 * bi + 16], J)
    m.free()


@pytest.mark.parametrize("K,N", [(256, 3), (2048, 37), (11008, 5)])
def test_group_sums_and_int8_tapped_from_the_product_quantiser(E, oracle, K, N):
    """The fp32 vector goes through the quantiser the matrix-vector kernels run; the int8 values and the 32-group sums
    S_j are read back from the activation record the block dots use, and I_j from those dots: all bit-exact against the
    CPU restatement (the rare +-1 of the approximate division is the quantiser's own, kernels/gemv.cu:16-65)."""
    rng = np.random.default_rng(K * 7 + N)
    nb = K // 256
    blocks = S.random_q4_k(rng, N * nb)
    x = rng.normal(0, 1, K).astype(np.float32)
    x[64:96] = 0.0  # a zero group
    m = E.GpuMat(S.Q4_K, K, N, blocks.reshape(-1))
    a = torch.zeros((N, K // 32), dtype=torch.int32, device="cuda")
    b = torch.zeros((N, K // 32), dtype=torch.int32, device="cuda")
    q8_dev = torch.zeros(K, dtype=torch.int8, device="cuda")
    E.op_int_dots_x(m, dev(x), a, b, q8_dev)
    q8 = q8_dev.cpu().numpy()
    oq, _ = oracle.quantize_q8(x)
    diff = q8.astype(np.int32) - oq.astype(np.int32)
    assert np.abs(diff).max() <= 1 and (diff != 0).mean() < 2e-3
    a, b = a.cpu().numpy(), b.cpu().numpy()
    sums = q8.astype(np.int32).reshape(K // 32, 32).sum(1)
    for r in range(N):
        assert np.array_equal(b[r], sums)  # what the dots hold == the sums of the int8 they read
        for bi in range(nb):
            I, Sm = oracle.q4k_subdots(blocks[r * nb + bi], q8[256 * bi: 256 * bi + 256])
            assert np.array_equal(a[r, 8 * bi: 8 * bi + 8], I)
            assert np.array_equal(b[r, 8 * bi: 8 * bi + 8], Sm)
    m.free()


def test_kv_store_rounding_all_inputs_vs_reference_and_oracle(E, oracle):
    """Every one of the 2^32 fp32 bit patterns: the library's KV-store rounding == the reference's copy_kv_f16
    (kernels/ops.cu:471-486, kernels/common.cu:9-38, run from the reference cubin) == the CPU restatement."""
    from oracle import ref_gpu
    have_ref = ref_gpu.available()
    n = 1 << 26
    base = torch.arange(n, dtype=torch.int64, device="cuda")
    ours = torch.empty(n, dtype=torch.int16, device="cuda")
    theirs = torch.empty(n, dtype=torch.int16, device="cuda")
    for chunk in range(64):
        first = chunk << 26
        bits = (base + first)
        bits = torch.where(bits >= (1 << 31), bits - (1 << 32), bits).to(torch.int32)
        x = bits.view(torch.float32)
        E.debug_f32_to_f16(x, ours, n)
        if have_ref:
            ref_gpu.copy_kv(x, theirs, 0, n)
            assert torch.equal(ours, theirs), f"chunk {chunk}"
        host = ours.cpu().numpy().view(np.uint16)
        assert np.array_equal(host, oracle.float_to_half_bits_range(first, n)), f"chunk {chunk}"
    if not have_ref:
        pytest.skip("reference cubin not present: checked against the CPU restatement only")


def _rel(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.mark.parametrize("wtype,K,N", [(S.Q4_K, 256, 1), (S.Q4_K, 2048, 33), (S.Q4_K, 2048, 2048), (S.Q4_K, 5120, 257),
                                       (S.Q6_K, 256, 2), (S.Q6_K, 2048, 1000), (S.Q6_K, 11008, 300),
                                       (S.Q6_K, 2560, 31)])
def test_gemv_q8_route_vs_oracle_and_reference(E, oracle, wtype, K, N):
    rng = np.random.default_rng(K * 7 + N)
    nb = K // 256
    blocks = (S.random_q4_k if wtype == S.Q4_K else S.random_q6_k)(rng, N * nb).reshape(-1)
    x = act_vectors(rng, K) if K >= 128 else rng.normal(0, 1, K).astype(np.float32)
    bias = rng.normal(0, 1, N).astype(np.float32)
    m = E.GpuMat(wtype, K, N, blocks)
    out = torch.full((N,), 2.0, dtype=torch.float32, device="cuda")
    E.op_gemv(m, dev(x), out, bias=dev(bias), use_res=2)
    got = out.cpu().numpy()
    om = oracle.mat(wtype, blocks, K, N)
    want = oracle.gemv(om, x, out=np.full(N, 2.0, np.float32), bias=bias, use_res=2)
    assert _rel(got, want) < 1e-4, _rel(got, want)
    try:
        from oracle import ref_gpu
        if ref_gpu.available() and K < 4096 or (ref_gpu.available() and wtype == S.Q6_K):
            rm = ref_gpu.RefMat(wtype, K, N, blocks)
            rout = torch.full((N,), 2.0, dtype=torch.float32, device="cuda")
            ref_gpu.gemv_q8(rm, dev(x), out=rout, bias=dev(bias), use_res=2)
            assert _rel(got, rout.cpu().numpy()) < 2e-5
    finally:
        m.free()


def test_gemv_f32_route_and_fused_norm(E, oracle, R):
    rng = np.random.default_rng(11)
    K, N = 2048, 256
    blocks = S.random_q6_k(rng, N * 8).reshape(-1)
    x = rng.normal(0, 1, K).astype(np.float32)
    w = rng.normal(1, 0.1, K).astype(np.float32)
    bias = rng.normal(0, 1, N).astype(np.float32)
    m = E.GpuMat(S.Q6_K, K, N, blocks)
    out = torch.zeros(N, dtype=torch.float32, device="cuda")
    E.op_gemv(m, dev(x), out, bias=dev(bias), act_mode=1, norm_w=dev(w), eps=1e-6)
    om = oracle.mat(S.Q6_K, blocks, K, N)
    want = oracle.gemv(om, oracle.rms_norm(x, w, 1e-6), bias=bias, act_mode=1)
    assert _rel(out.cpu().numpy(), want) < 1e-4
    rm = R.RefMat(S.Q6_K, K, N, blocks)
    ref = R.gemv_q6_f32(rm, R.rms_norm(dev(x), dev(w), 1e-6), dev(bias))
    assert _rel(out.cpu().numpy(), ref.cpu().numpy()) < 2e-5
    m.free()


def test_ffn_block_config1_shape(E, oracle, R):
    """BASELINE configuration 1: gate/up 11008x2048 Q4_K, down 2048x11008 Q6_K, seed 0."""
    rng = np.random.default_rng(0)
    K, FF = 2048, 11008
    g = S.random_q4_k(rng, FF * 8).reshape(-1)
    u = S.random_q4_k(rng, FF * 8).reshape(-1)
    d = S.random_q6_k(rng, K * 43).reshape(-1)
    x = rng.normal(0, 1, K).astype(np.float32)
    mg, mu, md = E.GpuMat(S.Q4_K, K, FF, g), E.GpuMat(S.Q4_K, K, FF, u), E.GpuMat(S.Q6_K, FF, K, d)
    h = torch.zeros(FF, dtype=torch.float32, device="cuda")
    y = torch.zeros(K, dtype=torch.float32, device="cuda")
    E.op_ffn_block(mg, mu, md, dev(x), h, y)
    oracle.set_threads(8)
    oh = oracle.ffn_gate_up(oracle.mat(S.Q4_K, g, K, FF), oracle.mat(S.Q4_K, u, K, FF), x)
    assert _rel(h.cpu().numpy(), oh) < 1e-4
    # feed the GPU's own h to the oracle's down so the stage is isolated
    oy = oracle.gemv(oracle.mat(S.Q6_K, d, FF, K), h.cpu().numpy())
    oracle.set_threads(1)
    assert _rel(y.cpu().numpy(), oy) < 1e-4
    # the reference's own kernels on the same inputs
    rh = R.ffn_gate_up(R.RefMat(S.Q4_K, K, FF, g), R.RefMat(S.Q4_K, K, FF, u), dev(x))
    assert _rel(h.cpu().numpy(), rh.cpu().numpy()) < 2e-5
    ry = R.gemv_q8(R.RefMat(S.Q6_K, FF, K, d), rh)
    assert _rel(y.cpu().numpy(), ry.cpu().numpy()) < 1e-4
    # host-buffer entry point gives the same result
    yh = np.zeros(K, np.float32)
    E.ffn_block_host(mg, mu, md, x, yh)
    assert np.array_equal(yh, y.cpu().numpy())
    for m in (mg, mu, md):
        m.free()


@pytest.mark.parametrize("H,Hkv,hd,T", [(4, 2, 64, 1), (4, 2, 64, 70), (16, 2, 128, 33), (16, 2, 128, 700),
                                        (40, 8, 128, 300), (16, 4, 256, 130), (5, 1, 128, 257),
                                        # one split, a full cluster, cluster + second level, tiles of 512 keys
                                        (16, 2, 128, 64), (16, 2, 128, 65), (16, 2, 128, 512), (16, 2, 128, 513),
                                        (16, 2, 128, 4608), (16, 2, 128, 16896), (40, 8, 128, 9000), (16, 4, 256, 2500),
                                        (6, 2, 64, 5000)])
@pytest.mark.parametrize("route", ["default", "register"])
def test_flash_decode_vs_oracle_and_reference(E, oracle, H, Hkv, hd, T, route, monkeypatch):
    # default: head sizes up to 128 run scores and values on the tensor cores at every length; "register" keeps
    # short contexts on the CUDA-core register route (the library reads the variable at every call)
    if route == "register":
        monkeypatch.setenv("TFR_ATTN_REGISTER_ROUTE", "1")
    rng = np.random.default_rng(H * 1000 + T)
    q = rng.normal(0, 1, H * hd).astype(np.float32)
    kc = rng.normal(0, 1, (T + 3, Hkv * hd)).astype(np.float16).view(np.uint16)
    vc = rng.normal(0, 1, (T + 3, Hkv * hd)).astype(np.float16).view(np.uint16)
    out = torch.zeros(H * hd, dtype=torch.float32, device="cuda")
    kd, vd = dev(kc.view(np.int16)), dev(vc.view(np.int16))
    E.op_attention(dev(q), kd, vd, out, H, Hkv, hd, T - 1)
    want = oracle.attention(q, kc, vc, H, Hkv, hd, T - 1)
    assert _rel(out.cpu().numpy(), want) < 2e-5
    # second call reuses the merge counters: must give the same answer
    out2 = torch.zeros_like(out)
    E.op_attention(dev(q), kd, vd, out2, H, Hkv, hd, T - 1)
    assert torch.equal(out, out2)
    from oracle import ref_gpu
    if ref_gpu.available():
        ref = ref_gpu.attention(dev(q), kd, vd, H, Hkv, hd, T - 1)
        assert _rel(out.cpu().numpy(), ref.cpu().numpy()) < 2e-5


@pytest.mark.parametrize("pos", [0, 5, 287, 16384])
def test_qkv_rope_kv_store_vs_reference(E, oracle, R, pos):
    rng = np.random.default_rng(pos + 1)
    K, H, Hkv, hd = 2048, 16, 2, 128
    nq, nkv = H * hd, Hkv * hd
    wq = S.random_q4_k(rng, nq * 8).reshape(-1)
    wk = S.random_q4_k(rng, nkv * 8).reshape(-1)
    wv = S.random_q6_k(rng, nkv * 8).reshape(-1)
    bq, bk, bv = (rng.normal(0, 1, n).astype(np.float32) for n in (nq, nkv, nkv))
    x = rng.normal(0, 1, K).astype(np.float32)
    nw = rng.normal(1, 0.1, K).astype(np.float32)
    mq, mk, mv = E.GpuMat(S.Q4_K, K, nq, wq, hd), E.GpuMat(S.Q4_K, K, nkv, wk, hd), E.GpuMat(S.Q6_K, K, nkv, wv)
    max_seq = pos + 2
    q = torch.zeros(nq, dtype=torch.float32, device="cuda")
    kc = torch.zeros(max_seq * nkv, dtype=torch.int16, device="cuda")
    vc = torch.zeros(max_seq * nkv, dtype=torch.int16, device="cuda")
    E.op_qkv_rope_store(mq, mk, mv, dev(bq), dev(bk), dev(bv), dev(x), dev(nw), 1e-6, 1e6, hd, pos, q, kc, vc)
    # reference kernel sequence
    xb = R.rms_norm(dev(x), dev(nw), 1e-6)
    rq, rk = R.gemv_q4_pair(R.RefMat(S.Q4_K, K, nq, wq), R.RefMat(S.Q4_K, K, nkv, wk), xb, dev(bq), dev(bk))
    rv = R.gemv_q6_f32(R.RefMat(S.Q6_K, K, nkv, wv), xb, dev(bv))
    R.rope(rq, H, hd, pos, 1e6)
    R.rope(rk, Hkv, hd, pos, 1e6)
    rkc = torch.zeros_like(kc)
    rvc = torch.zeros_like(vc)
    R.copy_kv(rk, rkc, pos, nkv)
    R.copy_kv(rv, rvc, pos, nkv)
    torch.cuda.synchronize()
    assert _rel(q.cpu().numpy(), rq.cpu().numpy()) < 2e-5
    krow = kc.cpu().numpy().view(np.float16)[pos * nkv:(pos + 1) * nkv].astype(np.float32)
    rkrow = rkc.cpu().numpy().view(np.float16)[pos * nkv:(pos + 1) * nkv].astype(np.float32)
    assert _rel(krow, rkrow) < 2e-3  # one f16 ulp
    vrow = vc.cpu().numpy().view(np.float16)[pos * nkv:(pos + 1) * nkv].astype(np.float32)
    rvrow = rvc.cpu().numpy().view(np.float16)[pos * nkv:(pos + 1) * nkv].astype(np.float32)
    assert _rel(vrow, rvrow) < 2e-3
    # only row `pos` was written
    assert int((kc != 0).sum()) <= nkv and int((kc.view(-1, nkv)[pos] != 0).sum()) > nkv // 2
    # CPU oracle (accurate sin/cos): close at small positions, looser where fast-math angles drift
    xn = oracle.rms_norm(x, nw, 1e-6)
    oq = oracle.gemv(oracle.mat(S.Q4_K, wq, K, nq), xn, bias=bq)
    oq = oracle.rope_neox(oq, H, hd, pos, 1e6)
    tol = 2e-4 if pos < 1000 else 2e-2
    assert _rel(q.cpu().numpy(), oq) < tol
    for m in (mq, mk, mv):
        m.free()


def test_device_quantizer_emits_valid_blocks(E, oracle):
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    w = torch.randn((64, 1024), generator=g, device="cuda") * 0.02
    for t, tol in ((S.Q4_K, 0.09), (S.Q6_K, 0.025)):
        out = torch.zeros(64 * 4 * S.BLOCK_BYTES[t], dtype=torch.uint8, device="cuda")
        E.synth_quantize(t, w, out)
        back = oracle.dequant_rows(t, out.cpu().numpy(), 1024, 64)
        assert np.abs(back - w.cpu().numpy()).max() <= tol * float(w.abs().max())


@pytest.mark.parametrize("K,N", [(256, 40), (2048, 96), (2560, 33)])
def test_q8_0_gemv_vs_oracle_and_reference(E, oracle, K, N):
    """Q8_0 weights (what Q5_K / Q5_1 tensors become at load): integer block sums bit-exact, floats vs the
    oracle and vs the reference's gemv_q8_0_global."""
    from oracle import ref_gpu
    rng = np.random.default_rng(K + N)
    raw = S.quantize_q8_0(rng.normal(0, 0.05, (N, K)).astype(np.float32)).reshape(-1)
    x = rng.normal(0, 1, K).astype(np.float32)
    bias = rng.normal(0, 1, N).astype(np.float32)
    m = E.GpuMat(S.Q8_0, K, N, raw)
    out = torch.zeros(N, device="cuda")
    E.op_gemv(m, dev(x), out, bias=dev(bias))
    want = oracle.gemv(oracle.mat(oracle.Q8_0, raw, K, N), x, bias=bias)
    assert _rel(out.cpu().numpy(), want) < 2e-5
    q8, d8 = oracle.quantize_q8(x)
    sums = torch.zeros(N * (K // 32), dtype=torch.int32, device="cuda")
    E.op_int_dots(m, dev(q8), dev(d8), sums)
    rows = raw.reshape(N, -1)
    for r in (0, N // 2, N - 1):
        assert np.array_equal(sums.cpu().numpy().reshape(N, K // 32)[r], oracle.q8_0_blockdots(rows[r], K, q8))
    if ref_gpu.available():
        ref = ref_gpu.gemv_q8(ref_gpu.RefMat(S.Q8_0, K, N, raw), dev(x), bias=dev(bias))
        assert _rel(out.cpu().numpy(), ref.cpu().numpy()) < 5e-6
    # a Q5_K tensor handed to the library becomes the same Q8_0 matrix
    q5 = S.random_q5_k(rng, N * (K // 256)).reshape(-1)
    m5 = E.GpuMat(S.Q5_K, K, N, q5)
    out5, out8 = torch.zeros(N, device="cuda"), torch.zeros(N, device="cuda")
    E.op_gemv(m5, dev(x), out5)
    m8 = E.GpuMat(S.Q8_0, K, N, oracle.transcode_to_q8_0(S.Q5_K, q5))
    E.op_gemv(m8, dev(x), out8)
    assert torch.equal(out5, out8)
    for mm in (m, m5, m8):
        mm.free()
