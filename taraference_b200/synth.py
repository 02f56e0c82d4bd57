"""Seeded synthetic GGUF-layout tensors and models (numpy, host side).

No real GGUF files are available to this project, so tests and benchmarks run on tensors
generated here: random super-blocks with the value distributions of the FFN-block
configuration, and N(0, 0.02) weights pushed through a small deterministic K-quant
quantiser for whole models.  The reference has no quantiser (crates/gguf only parses
files, crates/gguf/src/lib.rs:1-16); parity is defined downstream of the bytes, so this
one need not reproduce ggml's search — it only has to emit valid blocks
(layouts: crates/core/src/cuda/kernels/common.cu:40-84 and :164-186).
"""
from __future__ import annotations

import numpy as np

Q4_K, Q6_K, F32 = 12, 14, 0
Q8_0, Q5_K, Q5_1 = 8, 13, 7
BLOCK_BYTES = {Q4_K: 144, Q6_K: 210, Q8_0: 8 * 34}  # bytes per 256 weights


# ------------------------------------------------------------------ random blocks

def random_q4_k(rng: np.random.Generator, n_blocks: int, d_sigma: float = 0.003) -> np.ndarray:
    """n_blocks Q4_K super-blocks: fp16 d, dmin ~ |N(0, d_sigma)|, 6-bit scales/mins uniform in
    [0, 63], uniform 4-bit quants."""
    out = np.empty((n_blocks, 144), np.uint8)
    dd = np.abs(rng.normal(0.0, d_sigma, size=(n_blocks, 2))).astype(np.float16)
    out[:, 0:4] = dd.view(np.uint8).reshape(n_blocks, 4)
    sc = rng.integers(0, 64, size=(n_blocks, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(n_blocks, 8), dtype=np.uint8)
    out[:, 4:16] = pack_scales_k4(sc, mn)
    out[:, 16:144] = rng.integers(0, 256, size=(n_blocks, 128), dtype=np.uint8)
    return out


def random_q5_k(rng: np.random.Generator, n_blocks: int, d_sigma: float = 0.003) -> np.ndarray:
    """n_blocks Q5_K blocks (176 B: fp16 d, dmin, 12 scale bytes, 32 qh bytes, 128 qs bytes), uniform contents."""
    out = np.empty((n_blocks, 176), np.uint8)
    out[:, 4:] = rng.integers(0, 256, size=(n_blocks, 172), dtype=np.uint8)
    dd = np.abs(rng.normal(0, d_sigma, size=(n_blocks, 2))).astype(np.float16)
    out[:, 0:4] = dd.view(np.uint8).reshape(n_blocks, 4)
    return out


def random_q5_1(rng: np.random.Generator, n_blocks: int) -> np.ndarray:
    """n_blocks Q5_1 blocks (24 B: fp16 d, fp16 min, 4 qh bytes, 16 qs bytes)."""
    out = np.empty((n_blocks, 24), np.uint8)
    out[:, 4:] = rng.integers(0, 256, size=(n_blocks, 20), dtype=np.uint8)
    dm = np.stack([np.abs(rng.normal(0, 0.01, n_blocks)), rng.normal(0, 0.05, n_blocks)], 1).astype(np.float16)
    out[:, 0:4] = dm.view(np.uint8).reshape(n_blocks, 4)
    return out


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    """fp32 rows [N][K] -> Q8_0 bytes [N][K/32][34]: d = amax / 127 (fp16), q = round-half-away(x / d)."""
    N, K = w.shape
    g = w.reshape(N, K // 32, 32).astype(np.float32)
    amax = np.abs(g).max(-1)
    d = np.where(amax == 0, 0, amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.where(d[..., None] == 0, 0, g / d[..., None])
    q = np.clip(np.sign(r) * np.floor(np.abs(r) + 0.5), -127, 127).astype(np.int8)
    out = np.empty((N, K // 32, 34), np.uint8)
    out[..., 0:2] = d.astype(np.float16).view(np.uint8).reshape(N, K // 32, 2)
    out[..., 2:] = q.view(np.uint8)
    return out


def random_q6_k(rng: np.random.Generator, n_blocks: int, d_sigma: float = 0.002) -> np.ndarray:
    """n_blocks Q6_K blocks: uniform ql/qh bytes, int8 scales uniform in [-32, 31], fp16 d ~ |N(0, d_sigma)|."""
    out = np.empty((n_blocks, 210), np.uint8)
    out[:, 0:192] = rng.integers(0, 256, size=(n_blocks, 192), dtype=np.uint8)
    out[:, 192:208] = rng.integers(-32, 32, size=(n_blocks, 16), dtype=np.int8).view(np.uint8)
    d = np.abs(rng.normal(0.0, d_sigma, size=(n_blocks, 1))).astype(np.float16)
    out[:, 208:210] = d.view(np.uint8).reshape(n_blocks, 2)
    return out


def pack_scales_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Pack eight 6-bit scales and mins per block into the 12-byte K-quant field."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    out = np.empty(sc.shape[:-1] + (12,), np.uint8)
    out[..., 0:4] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = mn[..., 0:4] | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0xF) | ((mn[..., 4:8] & 0xF) << 4)
    return out


# ------------------------------------------------------------------ quantisers

def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    """Rows of fp32 weights (N, K) -> uint8 (N, K/256*144).  Asymmetric min/max per 32-element
    sub-block; not ggml's iterative search."""
    N, K = w.shape
    assert K % 256 == 0
    nb = K // 256
    x = w.astype(np.float32).reshape(N, nb, 8, 32)
    lo = np.minimum(x.min(-1), 0.0)
    hi = np.maximum(x.max(-1), lo)
    scale = (hi - lo) / 15.0
    mins = -lo
    d = (scale.max(-1) / 63.0).astype(np.float16)
    dmin = (mins.max(-1) / 63.0).astype(np.float16)
    df, dminf = d.astype(np.float32), dmin.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(df[..., None] > 0, np.rint(scale / df[..., None]), 0).clip(0, 63)
        mn = np.where(dminf[..., None] > 0, np.rint(mins / dminf[..., None]), 0).clip(0, 63)
        step = df[..., None] * sc
        q = np.where(step[..., None] > 0, np.rint((x + (dminf[..., None] * mn)[..., None]) / step[..., None]), 0)
    q = q.clip(0, 15).astype(np.uint8).reshape(N, nb, 4, 2, 32)
    out = np.empty((N, nb, 144), np.uint8)
    out[..., 0:2] = d.view(np.uint8).reshape(N, nb, 2)
    out[..., 2:4] = dmin.view(np.uint8).reshape(N, nb, 2)
    out[..., 4:16] = pack_scales_k4(sc.astype(np.uint8), mn.astype(np.uint8))
    out[..., 16:144] = (q[..., 0, :] | (q[..., 1, :] << 4)).reshape(N, nb, 128)
    return out.reshape(N, nb * 144)


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    """Rows of fp32 weights (N, K) -> uint8 (N, K/256*210).  Symmetric per 16-element group."""
    N, K = w.shape
    assert K % 256 == 0
    nb = K // 256
    x = w.astype(np.float32).reshape(N, nb, 16, 16)
    gscale = np.abs(x).max(-1) / 31.0
    d = (gscale.max(-1) / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(df[..., None] > 0, np.rint(gscale / df[..., None]), 0).clip(0, 127)
        step = df[..., None] * sc
        q = np.where(step[..., None] > 0, np.rint(x / step[..., None]), 0)
    L = (q.clip(-32, 31) + 32).astype(np.uint8).reshape(N, nb, 2, 4, 32)  # [half n][run j][l]
    out = np.empty((N, nb, 210), np.uint8)
    ql = np.empty((N, nb, 2, 64), np.uint8)
    ql[..., 0:32] = (L[..., 0, :] & 0xF) | ((L[..., 2, :] & 0xF) << 4)
    ql[..., 32:64] = (L[..., 1, :] & 0xF) | ((L[..., 3, :] & 0xF) << 4)
    qh = (L[..., 0, :] >> 4) | ((L[..., 1, :] >> 4) << 2) | ((L[..., 2, :] >> 4) << 4) | ((L[..., 3, :] >> 4) << 6)
    out[..., 0:128] = ql.reshape(N, nb, 128)
    out[..., 128:192] = qh.reshape(N, nb, 64)
    out[..., 192:208] = sc.astype(np.int8).view(np.uint8)
    out[..., 208:210] = d.view(np.uint8).reshape(N, nb, 2)
    return out.reshape(N, nb * 210)


def quantize(wtype: int, w: np.ndarray) -> np.ndarray:
    return quantize_q4_k(w) if wtype == Q4_K else quantize_q6_k(w)


# ------------------------------------------------------------------ models

QWEN25_3B = dict(arch="qwen2", n_layer=36, n_embd=2048, n_head=16, n_kv=2, head_dim=128, n_ff=11008,
                 n_vocab=151936, rope_theta=1e6, eps=1e-6, tied=True, qkv_bias=True)
QWEN25_32B = dict(arch="qwen2", n_layer=64, n_embd=5120, n_head=40, n_kv=8, head_dim=128, n_ff=27648,
                  n_vocab=152064, rope_theta=1e6, eps=1e-6, tied=False, qkv_bias=True)
TINY_DENSE = dict(arch="qwen2", n_layer=2, n_embd=256, n_head=4, n_kv=2, head_dim=64, n_ff=512,
                  n_vocab=320, rope_theta=1e6, eps=1e-6, tied=True, qkv_bias=True)


QWEN35_4B = dict(arch="qwen35", n_layer=32, n_embd=2560, n_head=16, n_kv=4, head_dim=256, n_ff=9216,
                 n_vocab=151936, rope_theta=1e7, eps=1e-6, tied=True, qkv_bias=False, rope_dim=64,
                 ssm_n_k=16, ssm_n_v=32, ssm_state=128, conv_kernel=4, full_attention_interval=4)
TINY_HYBRID = dict(arch="qwen35", n_layer=4, n_embd=256, n_head=2, n_kv=1, head_dim=128, n_ff=512,
                   n_vocab=320, rope_theta=1e7, eps=1e-6, tied=True, qkv_bias=False, rope_dim=32,
                   ssm_n_k=2, ssm_n_v=4, ssm_state=128, conv_kernel=4, full_attention_interval=4)


def is_hybrid(cfg: dict) -> bool:
    return cfg.get("arch") in ("qwen35", "qwen3_5")


def is_linear_layer(cfg: dict, i: int) -> bool:
    """Layer i of the hybrid architecture is a full-attention layer iff (i + 1) % interval == 0."""
    return is_hybrid(cfg) and (i + 1) % cfg.get("full_attention_interval", 4) != 0


def tensor_plan(cfg: dict) -> list[tuple[str, int, int, int]]:
    """(name, ggml_type, K, N) of every matrix in the Q4_K_M mix used by the benchmark
    configurations: Q6_K for token_embd / output, attn_v and ffn_down, Q4_K elsewhere.  Hybrid
    models: linear layers carry attn_qkv / attn_gate / ssm_beta / ssm_alpha / ssm_out, full layers
    a fused Q|gate attn_q of twice the width."""
    K, H, Hkv, hd, FF, V = (cfg[k] for k in ("n_embd", "n_head", "n_kv", "head_dim", "n_ff", "n_vocab"))
    hyb = is_hybrid(cfg)
    plan = [("token_embd.weight", Q6_K, K, V)]
    if not cfg.get("tied", True):
        plan.append(("output.weight", Q6_K, K, V))
    for i in range(cfg["n_layer"]):
        p = f"blk.{i}."
        if is_linear_layer(cfg, i):
            d, nk, nv = cfg["ssm_state"], cfg["ssm_n_k"], cfg["ssm_n_v"]
            plan += [(p + "attn_qkv.weight", Q4_K, K, (2 * nk + nv) * d), (p + "attn_gate.weight", Q4_K, K, nv * d),
                     (p + "ssm_beta.weight", Q4_K, K, nv), (p + "ssm_alpha.weight", Q4_K, K, nv),
                     (p + "ssm_out.weight", Q4_K, nv * d, K)]
        else:
            plan += [(p + "attn_q.weight", Q4_K, K, (2 if hyb else 1) * H * hd), (p + "attn_k.weight", Q4_K, K, Hkv * hd),
                     (p + "attn_v.weight", Q6_K, K, Hkv * hd), (p + "attn_output.weight", Q4_K, H * hd, K)]
        plan += [(p + "ffn_gate.weight", Q4_K, K, FF), (p + "ffn_up.weight", Q4_K, K, FF),
                 (p + "ffn_down.weight", Q6_K, FF, K)]
    return plan


def vector_plan(cfg: dict) -> list[tuple[str, int, str]]:
    """(name, length, kind) of every fp32 tensor; kind 'norm' -> ones, 'bias' -> N(0, sigma),
    'conv' -> U(-0.5, 0.5), 'a' -> -U(0.5, 16) (the GGUF stores -exp(A_log)), 'dt' -> inverse
    softplus of U(0.001, 0.1)."""
    K, H, Hkv, hd = (cfg[k] for k in ("n_embd", "n_head", "n_kv", "head_dim"))
    plan = [("output_norm.weight", K, "norm")]
    for i in range(cfg["n_layer"]):
        p = f"blk.{i}."
        plan += [(p + "attn_norm.weight", K, "norm"), (p + "ffn_norm.weight", K, "norm")]
        if is_linear_layer(cfg, i):
            d, nk, nv, ck = cfg["ssm_state"], cfg["ssm_n_k"], cfg["ssm_n_v"], cfg["conv_kernel"]
            plan += [(p + "ssm_conv1d.weight", ck * (2 * nk + nv) * d, "conv"), (p + "ssm_a", nv, "a"),
                     (p + "ssm_dt.bias", nv, "dt"), (p + "ssm_norm.weight", d, "norm")]
            continue
        if is_hybrid(cfg):
            plan += [(p + "attn_q_norm.weight", hd, "norm"), (p + "attn_k_norm.weight", hd, "norm")]
        if cfg.get("qkv_bias", False):
            plan += [(p + "attn_q.bias", H * hd, "bias"), (p + "attn_k.bias", Hkv * hd, "bias"),
                     (p + "attn_v.bias", Hkv * hd, "bias")]
    return plan


dense_tensor_plan = tensor_plan
dense_vector_plan = vector_plan


def make_vector(kind: str, n: int, rng, sigma: float) -> np.ndarray:
    if kind == "norm":
        return np.ones(n, np.float32)
    if kind == "conv":
        return rng.uniform(-0.5, 0.5, n).astype(np.float32)
    if kind == "a":
        return (-rng.uniform(0.5, 16.0, n)).astype(np.float32)
    if kind == "dt":
        return np.log(np.expm1(rng.uniform(0.001, 0.1, n))).astype(np.float32)
    return rng.normal(0, sigma, n).astype(np.float32)


def make_model(cfg: dict, seed: int = 0, sigma: float = 0.02) -> dict:
    """Whole model on the host: name -> (type, K, N, uint8 bytes) or fp32 vector.
    Only for sizes numpy handles in seconds; full-size models are generated on the GPU."""
    rng = np.random.default_rng(seed)
    tensors: dict = {}
    for name, t, K, N in tensor_plan(cfg):
        w = rng.normal(0.0, sigma, size=(N, K)).astype(np.float32)
        tensors[name] = (t, K, N, np.ascontiguousarray(quantize(t, w).reshape(-1)))
    for name, n, kind in vector_plan(cfg):
        tensors[name] = make_vector(kind, n, rng, sigma)
    return tensors


def random_model(cfg: dict, seed: int = 0, sigma: float = 0.02) -> dict:
    """Whole model on the host in the layout of make_model, but every matrix is made of random K-quant blocks
    (random_q4_k / random_q6_k) instead of quantised Gaussian weights: full-size models in seconds.  The time a
    CPU pass over the model takes does not depend on the values, so this is what the CPU baseline runs on."""
    rng = np.random.default_rng(seed)
    tensors: dict = {}
    for name, t, K, N in tensor_plan(cfg):
        n_blocks = N * (K // 256)
        blocks = random_q4_k(rng, n_blocks) if t == Q4_K else random_q6_k(rng, n_blocks)
        tensors[name] = (t, K, N, np.ascontiguousarray(blocks.reshape(-1)))
    for name, n, kind in vector_plan(cfg):
        tensors[name] = make_vector(kind, n, rng, sigma)
    return tensors


make_dense_model = make_model


def write_gguf(path, cfg: dict, tensors: dict, version_alignment: int | None = None) -> None:
    """Writes a model (layout of make_model) as a GGUF file with the tensor names of load.rs:280-417 and the
    metadata keys ModelConfig::from_gguf reads (config.rs:118-235), using gguf-py's writer."""
    import gguf
    arch = cfg["arch"]
    w = gguf.GGUFWriter(str(path), arch)
    if version_alignment:
        w.add_custom_alignment(version_alignment)
    w.add_name("synthetic " + arch)
    w.add_uint32(f"{arch}.embedding_length", cfg["n_embd"])
    w.add_uint32(f"{arch}.block_count", cfg["n_layer"])
    if "eos_token_id" in cfg:
        w.add_uint32("tokenizer.ggml.eos_token_id", cfg["eos_token_id"])
    w.add_uint32(f"{arch}.attention.head_count", cfg["n_head"])
    w.add_uint32(f"{arch}.attention.head_count_kv", cfg["n_kv"])
    w.add_uint32(f"{arch}.attention.key_length", cfg["head_dim"])
    w.add_uint32(f"{arch}.attention.value_length", cfg["head_dim"])
    w.add_uint32(f"{arch}.feed_forward_length", cfg["n_ff"])
    w.add_uint32(f"{arch}.context_length", 4096)
    w.add_uint32(f"{arch}.vocab_size", cfg["n_vocab"])
    w.add_float32(f"{arch}.rope.freq_base", float(cfg["rope_theta"]))
    w.add_float32(f"{arch}.attention.layer_norm_rms_epsilon", float(cfg["eps"]))
    if is_hybrid(cfg):
        w.add_uint32(f"{arch}.rope.dimension_count", cfg["rope_dim"])
        w.add_uint32(f"{arch}.ssm.conv_kernel", cfg["conv_kernel"])
        w.add_uint32(f"{arch}.ssm.state_size", cfg["ssm_state"])
        w.add_uint32(f"{arch}.ssm.group_count", cfg["ssm_n_k"])
        w.add_uint32(f"{arch}.ssm.time_step_rank", cfg["ssm_n_v"])
        w.add_uint32(f"{arch}.ssm.inner_size", cfg["ssm_n_v"] * cfg["ssm_state"])
        w.add_uint32(f"{arch}.full_attention_interval", cfg.get("full_attention_interval", 4))
    w.add_array("tokenizer.ggml.tokens", [f"<{i}>" for i in range(8)])  # an array the reader must step over
    qt = {Q4_K: gguf.GGMLQuantizationType.Q4_K, Q6_K: gguf.GGMLQuantizationType.Q6_K}
    for name, t in tensors.items():
        if isinstance(t, tuple):
            wt, K, N, data = t
            w.add_tensor(name, np.ascontiguousarray(data).reshape(N, (K // 256) * BLOCK_BYTES[wt]), raw_dtype=qt[wt])
        else:
            a = np.ascontiguousarray(t, dtype=np.float32)
            if name.endswith("ssm_conv1d.weight"):  # GGUF dims [kernel, channels]: numpy shape is the reverse
                a = a.reshape(-1, cfg["conv_kernel"])
            w.add_tensor(name, a)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
