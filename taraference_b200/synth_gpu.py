"""Full-size synthetic models generated on the device (torch for memory and RNG only).

Weights are drawn N(0, sigma) with torch's CUDA generator and quantised by the library's
own device quantiser (tfr_synth_quantize); norm weights are ones and biases N(0, sigma),
as the benchmark configurations specify.  The generated GGUF bytes can be copied back to
the host so that a checker sees exactly the bytes the engine was given.
"""
from __future__ import annotations

import numpy as np
import torch

from . import engine as E
from . import synth


def quantized_matrix(wtype: int, K: int, N: int, gen: torch.Generator, sigma: float = 0.02,
                     rows_per_chunk: int = 16384) -> torch.Tensor:
    """uint8 device tensor with the GGUF bytes of an N x K matrix drawn N(0, sigma)."""
    row_bytes = (K // 256) * synth.BLOCK_BYTES[wtype]
    out = torch.empty(N * row_bytes, dtype=torch.uint8, device="cuda")
    for r0 in range(0, N, rows_per_chunk):
        r1 = min(N, r0 + rows_per_chunk)
        w = torch.randn((r1 - r0, K), generator=gen, device="cuda", dtype=torch.float32) * sigma
        E.synth_quantize(wtype, w, out[r0 * row_bytes: r1 * row_bytes])
    torch.cuda.synchronize()
    return out


def build_model(cfg: dict, seed: int = 0, sigma: float = 0.02, device: int = 0, context_length: int = 4096,
                      keep_host: bool = False):
    """Dense or hybrid model.  Returns (CudaModel, host_tensors or None).  host_tensors has the layout of
    synth.make_model (name -> (type, K, N, uint8 array) / fp32 array)."""
    torch.cuda.set_device(device)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    model = E.CudaModel(device)
    model.set_config(cfg, context_length)
    host = {} if keep_host else None
    host_rng = np.random.default_rng(seed)
    for name, t, K, N in synth.tensor_plan(cfg):
        q = quantized_matrix(t, K, N, gen, sigma)
        model.upload_tensor(name, t, K, N, q)
        if keep_host:
            host[name] = (t, K, N, q.cpu().numpy())
        del q
    for name, n, kind in synth.vector_plan(cfg):
        if kind == "norm":
            v = torch.ones(n, device="cuda", dtype=torch.float32)
        elif kind == "bias":
            v = torch.randn(n, generator=gen, device="cuda", dtype=torch.float32) * sigma
        else:  # small recurrent-layer tensors: drawn on the host
            v = torch.from_numpy(synth.make_vector(kind, n, host_rng, sigma)).cuda()
        model.upload_tensor(name, E.TYPE_F32, n, 1, v)
        if keep_host:
            host[name] = v.cpu().numpy()
    model.finalize_load()
    return model, host


build_dense_model = build_model


def weight_bytes(cfg: dict) -> int:
    """Algorithmic weight bytes one decode step reads: every matrix once at GGUF density."""
    total = 0
    for _, t, K, N in synth.tensor_plan(cfg):
        total += N * (K // 256) * synth.BLOCK_BYTES[t]
    for _, n, _kind in synth.vector_plan(cfg):
        total += 4 * n
    return total


def kv_bytes_per_position(cfg: dict) -> int:
    n_full = sum(1 for i in range(cfg["n_layer"]) if not synth.is_linear_layer(cfg, i))
    return n_full * cfg["n_kv"] * cfg["head_dim"] * 2 * 2


def recurrent_state_bytes(cfg: dict) -> int:
    """fp32 state a decode step reads AND writes back once per linear layer (plus the conv history it reads)."""
    if not synth.is_hybrid(cfg):
        return 0
    n_lin = sum(1 for i in range(cfg["n_layer"]) if synth.is_linear_layer(cfg, i))
    d, nk, nv, ck = cfg["ssm_state"], cfg["ssm_n_k"], cfg["ssm_n_v"], cfg["conv_kernel"]
    return n_lin * (2 * nv * d * d * 4 + ck * (2 * nk + nv) * d * 4)
