#!/usr/bin/env python
"""Generates tests/golden/ref_kernels_sm100.npz: outputs of the reference's OWN kernels.

Run on a machine with a B200 and the reference checkout built by oracle/Makefile
(oracle/_ref/ref_kernels.cubin = the reference's .cu fragments, unmodified, compiled with
the reference's NVRTC options for sm_100).  Inputs are regenerated from seeds by the tests
(taraference_b200.synth + numpy default_rng), so only outputs are stored.  The CPU tests
pin the C restatement (oracle/) against these vectors; nothing here is read at run time
by the library.

    python tests/golden/make_golden.py [out.npz]
    python tests/golden/make_golden.py --hybrid [out.npz]     # ref_kernels_hybrid_sm100.npz
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from oracle import ref_gpu as R  # noqa: E402
from taraference_b200 import synth as S  # noqa: E402


def inputs():
    """Seeded inputs shared with tests/test_golden_cpu.py (keep in sync)."""
    rng = np.random.default_rng(20240611)
    d = {}
    x = rng.normal(0, 1, 2048).astype(np.float32)
    x[0:32] = 0.0
    x[32:64] *= 1e-20
    x[64:96] *= 1e4
    d["x2048"] = x
    d["x11008"] = rng.normal(0, 0.3, 11008).astype(np.float32)
    d["q4_64x2048"] = S.random_q4_k(rng, 64 * 8).reshape(-1)
    d["q6_64x2048"] = S.random_q6_k(rng, 64 * 8).reshape(-1)
    d["q6_16x11008"] = S.random_q6_k(rng, 16 * 43).reshape(-1)
    d["gate_96x2048"] = S.random_q4_k(rng, 96 * 8).reshape(-1)
    d["up_96x2048"] = S.random_q4_k(rng, 96 * 8).reshape(-1)
    d["bias64"] = rng.normal(0, 1, 64).astype(np.float32)
    d["normw"] = rng.normal(1, 0.1, 2048).astype(np.float32)
    d["q_heads"] = rng.normal(0, 1, 16 * 128).astype(np.float32)
    d["kc"] = rng.normal(0, 1, (70, 2 * 128)).astype(np.float16).view(np.uint16)
    d["vc"] = rng.normal(0, 1, (70, 2 * 128)).astype(np.float16).view(np.uint16)
    d["f16_src"] = np.concatenate([rng.normal(0, 1, 200), rng.normal(0, 1e-5, 28), [1.0 + 2.0 ** -11, 65519.0, 70000.0, 1e-8]]
                                  ).astype(np.float32)
    return d


def main(out_path):
    dev = R.dev
    inp = inputs()
    g = {}
    x = dev(inp["x2048"])
    q, d8 = R.quantize_q8(x)
    g["q8_x2048"], g["d8_x2048"] = q.cpu().numpy(), d8.cpu().numpy()
    q2, d82 = R.quantize_q8(dev(inp["x11008"]))
    g["q8_x11008"], g["d8_x11008"] = q2.cpu().numpy(), d82.cpu().numpy()
    m4 = R.RefMat(S.Q4_K, 2048, 64, inp["q4_64x2048"])
    m6 = R.RefMat(S.Q6_K, 2048, 64, inp["q6_64x2048"])
    m6t = R.RefMat(S.Q6_K, 11008, 16, inp["q6_16x11008"])
    g["gemv_q4k_q8"] = R.gemv_q8(m4, x, bias=dev(inp["bias64"])).cpu().numpy()
    g["gemv_q6k_q8"] = R.gemv_q8(m6, x).cpu().numpy()
    g["gemv_q6k_q8_8way"] = R.gemv_q8(m6t, dev(inp["x11008"])).cpu().numpy()
    g["gemv_q6k_f32"] = R.gemv_q6_f32(m6, x, dev(inp["bias64"])).cpu().numpy()
    mg, mu = R.RefMat(S.Q4_K, 2048, 96, inp["gate_96x2048"]), R.RefMat(S.Q4_K, 2048, 96, inp["up_96x2048"])
    g["ffn_mcol"] = R.ffn_gate_up(mg, mu, x).cpu().numpy()
    g["ffn_8way"] = R.ffn_gate_up_8way(mg, mu, x).cpu().numpy()
    g["rms_norm"] = R.rms_norm(x, dev(inp["normw"]), 1e-6).cpu().numpy()
    for pos in (0, 7, 300, 16384):
        g[f"rope_pos{pos}"] = R.rope(dev(inp["q_heads"]).clone(), 16, 128, pos, 1e6).cpu().numpy()
    cache = torch.zeros(2 * inp["f16_src"].size, dtype=torch.int16, device="cuda")
    R.copy_kv(dev(inp["f16_src"]), cache, 1, inp["f16_src"].size)
    g["copy_kv_bits"] = cache.cpu().numpy().view(np.uint16)[inp["f16_src"].size:]
    kc, vc = dev(inp["kc"].view(np.int16)), dev(inp["vc"].view(np.int16))
    for T in (1, 9, 70):
        g[f"attn_T{T}"] = R.attention(dev(inp["q_heads"]), kc, vc, 16, 2, 128, T - 1).cpu().numpy()
    g["embed_q6_row5"] = R.embed(m6, 5).cpu().numpy()
    g["embed_q4_row7"] = R.embed(m4, 7).cpu().numpy()
    # tiny model: free-running logits and teacher-forced layer outputs
    cfg = S.TINY_DENSE
    tens = S.make_dense_model(cfg, seed=11)
    rm = R.RefModel(cfg, tens, 16)
    toks = [3, 200, 45]
    for i, t in enumerate(toks):
        taps = {}
        logits = rm.decode_token(i, t, taps)
        g[f"tiny_logits_{i}"] = logits.cpu().numpy()
        for li in range(cfg["n_layer"]):
            g[f"tiny_x_{i}_{li}"] = taps[f"x{li}"].cpu().numpy()
    g["tiny_kc0"] = rm.kc[0].cpu().numpy().view(np.uint16)[: 3 * cfg["n_kv"] * cfg["head_dim"]]
    torch.cuda.synchronize()
    np.savez_compressed(out_path, **g)
    print("wrote", out_path, {k: v.shape for k, v in g.items()})


def hybrid_inputs():
    """Seeded inputs of the hybrid-layer kernels, shared with tests/test_golden_cpu.py."""
    rng = np.random.default_rng(20250907)
    nk, nv, d, kernel = 2, 4, 128, 4
    ch, vd = (2 * nk + nv) * d, nv * d
    h = dict(nk=nk, nv=nv, d=d, kernel=kernel, ch=ch, vd=vd)
    h["conv_w"] = rng.uniform(-0.5, 0.5, ch * kernel).astype(np.float32)
    h["a"] = (-rng.uniform(0.5, 16.0, nv)).astype(np.float32)
    h["dt"] = np.log(np.expm1(rng.uniform(0.001, 0.1, nv))).astype(np.float32)
    h["dt"][0] = 25.0  # softplus takes its linear branch (z > 20) for head 0
    h["norm_w"] = rng.uniform(0.5, 1.5, d).astype(np.float32)
    h["steps"] = [dict(qkv=rng.normal(0, 1, ch).astype(np.float32), z=rng.normal(0, 1, vd).astype(np.float32),
                       beta=rng.normal(0, 1.5, nv).astype(np.float32), alpha=rng.normal(0, 1.5, nv).astype(np.float32))
                  for _ in range(5)]
    H, Hkv, hd = 4, 1, 256
    h.update(H=H, Hkv=Hkv, hd=hd, n_rot=64, theta=1e7, eps=1e-6)
    h["qg"] = rng.normal(0, 1, 2 * H * hd).astype(np.float32)
    h["k"] = rng.normal(0, 1, Hkv * hd).astype(np.float32)
    h["qw"] = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    h["kw"] = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    h["gate"] = rng.normal(0, 2, H * hd).astype(np.float32)
    h["att"] = rng.normal(0, 1, H * hd).astype(np.float32)
    return h


def main_hybrid(out_path):
    dev = R.dev
    h = hybrid_inputs()
    g = {}
    nk, nv, d, kernel, ch = h["nk"], h["nv"], h["d"], h["kernel"], h["ch"]
    win = torch.zeros((kernel - 1) * ch, dtype=torch.float32, device="cuda")
    state = torch.zeros(nv * d * d, dtype=torch.float32, device="cuda")
    cw, a, dt, nw = dev(h["conv_w"]), dev(h["a"]), dev(h["dt"]), dev(h["norm_w"])
    for i, st in enumerate(h["steps"]):
        q, k, v = R.gdn_conv_qkvl2(dev(st["qkv"]), cw, win, nk, nv, d, kernel, h["eps"])
        y = R.gdn_delta_gated_d128(q, k, v, dev(st["alpha"]), dev(st["beta"]), dt, a, state, nw, dev(st["z"]), nk, nv, h["eps"])
        g[f"gdn_q_{i}"], g[f"gdn_k_{i}"], g[f"gdn_v_{i}"] = q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy()
        g[f"gdn_y_{i}"] = y.cpu().numpy()
    g["gdn_state"], g["gdn_window"] = state.cpu().numpy(), win.cpu().numpy()
    q, gate = R.split_q_gate(dev(h["qg"]), h["H"], h["hd"])
    g["split_q"], g["split_gate"] = q.cpu().numpy(), gate.cpu().numpy()
    for pos in (0, 5, 4000):
        qq = R.qk_norm_partial_rope(q.clone(), dev(h["qw"]), h["H"], h["hd"], h["n_rot"], pos, h["theta"], h["eps"])
        kk = R.qk_norm_partial_rope(dev(h["k"]).clone(), dev(h["kw"]), h["Hkv"], h["hd"], h["n_rot"], pos, h["theta"], h["eps"])
        g[f"qnorm_rope_pos{pos}"], g[f"knorm_rope_pos{pos}"] = qq.cpu().numpy(), kk.cpu().numpy()
    g["mul_sigmoid"] = R.mul_sigmoid(dev(h["att"]).clone(), dev(h["gate"])).cpu().numpy()
    # tiny hybrid model: teacher-forced layer outputs and free-running logits of the reference kernels
    cfg = S.TINY_HYBRID
    tens = S.make_model(cfg, seed=12)
    rm = R.RefModel(cfg, tens, 16)
    for i, t in enumerate([3, 200, 45, 17]):
        taps = {}
        logits = rm.decode_token(i, t, taps)
        g[f"tinyh_logits_{i}"] = logits.cpu().numpy()
        for li in range(cfg["n_layer"]):
            g[f"tinyh_x_{i}_{li}"] = taps[f"x{li}"].cpu().numpy()
    g["tinyh_ssm0"] = rm.ssm[0].cpu().numpy()
    torch.cuda.synchronize()
    np.savez_compressed(out_path, **g)
    print("wrote", out_path, {k: v.shape for k, v in g.items()})


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if a != "--hybrid"]
    hybrid = "--hybrid" in sys.argv[1:]
    default = "ref_kernels_hybrid_sm100.npz" if hybrid else "ref_kernels_sm100.npz"
    out = Path(args[0]) if args else ROOT / "tests" / "golden" / default
    out.parent.mkdir(parents=True, exist_ok=True)
    (main_hybrid if hybrid else main)(out)
