"""Launcher for the reference's own CUDA kernels (test infrastructure, GPU box only).

oracle/Makefile compiles the reference's .cu fragments, unmodified and with the
reference's NVRTC options, into oracle/_ref/ref_kernels.cubin.  This module loads that
cubin through the CUDA driver API (ctypes on libcuda) and launches the kernels with the
reference's grid / block / shared-memory recipes (crates/core/src/cuda/matmul.rs,
layer.rs; each helper cites its recipe) on torch-allocated device buffers.  It defines
"what the reference computes" on the very same B200: the bit-exact target for the int8
activation quantiser and the tolerance target for logits.

Only tests/, the smoke check and bench.py's reference-side measurements may use it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
CUBIN = HERE / "_ref" / "ref_kernels.cubin"
Q4_K, Q6_K, Q8_0 = 12, 14, 8


def available() -> bool:
    return CUBIN.exists() and torch.cuda.is_available()


class RefKernels:
    def __init__(self):
        if not available():
            raise RuntimeError("reference cubin or GPU missing")
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make sure the primary context is current
        self.cu = C.CDLL("libcuda.so.1")
        self.mod = C.c_void_p()
        data = CUBIN.read_bytes()
        self._img = C.create_string_buffer(data, len(data))
        self._chk(self.cu.cuModuleLoadData(C.byref(self.mod), self._img), "cuModuleLoadData")
        self._fn = {}
        self.launches = 0

    def _chk(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUresult {rc}")

    def fn(self, name: str):
        if name not in self._fn:
            f = C.c_void_p()
            self._chk(self.cu.cuModuleGetFunction(C.byref(f), self.mod, name.encode()), f"cuModuleGetFunction({name})")
            self._fn[name] = f
        return self._fn[name]

    def launch(self, name, grid, block, smem, *args):
        """args: torch tensors (device pointer), python ints (int32) or floats (float32)."""
        vals = []
        for a in args:
            if isinstance(a, torch.Tensor):
                vals.append(C.c_void_p(a.data_ptr()))
            elif isinstance(a, float):
                vals.append(C.c_float(a))
            else:
                vals.append(C.c_int(int(a)))
        arr = (C.c_void_p * len(vals))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = tuple(block) + (1,) * (3 - len(block))
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._chk(self.cu.cuLaunchKernel(self.fn(name), *[C.c_uint(x) for x in g], *[C.c_uint(x) for x in b],
                                         C.c_uint(smem), stream, arr, None), f"cuLaunchKernel({name})")
        self.launches += 1


_K = None


def kernels() -> RefKernels:
    global _K
    if _K is None:
        _K = RefKernels()
    return _K


def dev(a, dtype=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def compact_q6(raw: np.ndarray, K: int, N: int) -> np.ndarray:
    """crates/core/src/cuda/load.rs:145-159: pad every 210-byte block to 212 bytes."""
    nb = K // 256
    out = np.zeros((N * nb, 212), np.uint8)
    out[:, :210] = raw.reshape(N * nb, 210)
    return out.reshape(-1)


class RefMat:
    """GpuMat as the reference loader holds it (types.rs:26-39): raw bytes, plus the 212-byte
    compact copy for Q6_K (load.rs:240-259)."""

    def __init__(self, wtype: int, K: int, N: int, raw: np.ndarray):
        self.type, self.K, self.N = wtype, K, N
        nb = K // 256
        self.col_bytes = nb * (144 if wtype == Q4_K else 272 if wtype == Q8_0 else 210)
        self.data = dev(raw)
        self.compact = dev(compact_q6(raw, K, N)) if wtype == Q6_K else None
        self.compact_col_bytes = nb * 212


# ------------------------------------------------------------------ single kernels

def quantize_q8(x: torch.Tensor):
    """quantize_q8, matmul.rs:47-70."""
    n = x.numel()
    q = torch.zeros(n, dtype=torch.int8, device="cuda")
    d = torch.zeros(n // 32, dtype=torch.float32, device="cuda")
    groups = (n + 31) // 32
    kernels().launch("quantize_q8_global", ((groups + 7) // 8,), (256,), 0, x, q, d, n)
    return q, d


def rms_norm(x, w, eps):
    """layer.rs rms_norm launch: grid n_tok x 256 (ops.cu:4-34)."""
    out = torch.empty_like(x)
    kernels().launch("rms_norm_f32", (1,), (256,), 0, x, w, out, x.numel(), 1, float(eps))
    return out


def gemv_q8(m: RefMat, x, out=None, bias=None, use_res=0, warps=16):
    """try_gemv_global_q8, matmul.rs:142-302, for K < 4096 and the tall-K 8-way Q6_K case."""
    if out is None:
        out = torch.zeros(m.N, dtype=torch.float32, device="cuda")
    q, d = quantize_q8(x)
    b = bias if bias is not None else x
    smem = m.K + (m.K // 32) * 4
    if m.type == Q8_0:
        # gemv_q8_0_global, matmul.rs:160-164 + 286-300 (K < 4096: no split)
        assert m.K < 4096, "split-K Q8_0 route not wired in the harness"
        kernels().launch("gemv_q8_0_global", ((m.N + warps - 1) // warps,), (warps * 32,), smem, m.data, q, d, out, m.K, m.N,
                         m.col_bytes, int(bias is not None), b, use_res, x)
        return out
    if m.type == Q4_K:
        if m.K >= 4096:
            # split-K route, matmul.rs:199-289: grid (N, 4) x 64, then the reduce with bias / residual
            partial = torch.zeros(4 * m.N, dtype=torch.float32, device="cuda")
            kernels().launch("gemv_q4_k_global_splitk", (m.N, 4), (64,), 0, m.data, q, d, partial, m.K, m.N, m.col_bytes, 4)
            kernels().launch("gemv_splitk_reduce", ((m.N + 255) // 256,), (256,), 0, partial, out, m.N, 4,
                             int(bias is not None), b, use_res, x)
            return out
        kernels().launch("gemv_q4_k_global", ((m.N + warps - 1) // warps,), (warps * 32,), smem, m.data, q, d, out,
                         m.K, m.N, m.col_bytes, int(bias is not None), b, use_res, x)
    elif m.K >= 4096:
        kernels().launch("gemv_q6_k_compact_global_8way", (m.N,), (256,), 0, m.compact, q, d, out, m.K, m.N,
                         m.compact_col_bytes, int(bias is not None), b, use_res, x)
    else:
        kernels().launch("gemv_q6_k_compact_global", ((m.N + warps - 1) // warps,), (warps * 32,), smem, m.compact, q,
                         d, out, m.K, m.N, m.compact_col_bytes, int(bias is not None), b, use_res, x)
    return out


def gemv_q6_f32(m: RefMat, x, bias=None):
    """gemv_baseline for Q6_K, matmul.rs:346-412 (lc_q5_gemv): fp32 activations."""
    assert m.type == Q6_K
    out = torch.zeros(m.N, dtype=torch.float32, device="cuda")
    b = bias if bias is not None else x
    if m.K >= 4096:
        # gemv_splitk, matmul.rs:414-505: four K splits (gemv_n_split), grid (ceil(N/32), 4) x 1024, then the reduce
        nb = m.K // 256
        rows_per_split = max(256, -(-nb // 4) * 256)
        partial = torch.zeros(4 * m.N, dtype=torch.float32, device="cuda")
        kernels().launch("gemv_q6_k_splitk", ((m.N + 31) // 32, 4), (1024,), rows_per_split * 4, m.data, x, partial, m.K, m.N,
                         m.col_bytes, 4)
        kernels().launch("gemv_splitk_reduce", ((m.N + 255) // 256,), (256,), 0, partial, out, m.N, 4, int(bias is not None), b, 0, x)
        return out
    kernels().launch("gemv_q6_k", ((m.N + 7) // 8,), (256,), m.K * 4, m.data, x, out, m.K, m.N, m.col_bytes,
                     int(bias is not None), b, 0, x)
    return out


def gemv_q4_pair(wa: RefMat, wb: RefMat, x, ba=None, bb=None):
    """try_gemv_q4_pair, matmul.rs:727-784."""
    q, d = quantize_q8(x)
    oa = torch.zeros(wa.N, dtype=torch.float32, device="cuda")
    ob = torch.zeros(wb.N, dtype=torch.float32, device="cuda")
    both = ba is not None and bb is not None
    kernels().launch("gemv_q4_k_pair", (wa.N + wb.N,), (64,), 0, wa.data, wb.data, q, d, oa, ob, wa.K, wa.N, wb.N,
                     wa.col_bytes, int(both), ba if both else x, bb if both else x)
    return oa, ob


def ffn_gate_up(gate: RefMat, up: RefMat, x):
    """gemv_q4_k_ffn_mcol, matmul.rs:680-725: grid ceil(ff/32) x 1024, smem K + K/8."""
    out = torch.zeros(gate.N, dtype=torch.float32, device="cuda")
    kernels().launch("gemv_q4_k_ffn_mcol", ((gate.N + 31) // 32,), (1024,), gate.K + gate.K // 8, gate.data, up.data,
                     x, out, gate.K, gate.N, gate.col_bytes)
    return out


def ffn_gate_up_8way(gate: RefMat, up: RefMat, x):
    """gemv_q4_k_ffn_8way, matmul.rs:698-725: the reference's alternative FFN kernel (8 warps split K,
    pre-quantised activation); same mathematics as the mcol kernel, different summation order."""
    q, d = quantize_q8(x)
    out = torch.zeros(gate.N, dtype=torch.float32, device="cuda")
    kernels().launch("gemv_q4_k_ffn_8way", (gate.N,), (256,), 0, gate.data, up.data, q, d, out, gate.K, gate.N,
                     gate.col_bytes)
    return out


def rope(x, n_heads, hd, pos, theta):
    """rope launch, layer.rs:~560-600: grid (heads, n_tok) x 32 (ops.cu:348-371)."""
    kernels().launch("rope_neox_f32", (n_heads, 1), (32,), 0, x, n_heads, hd, pos, 1, float(theta))
    return x


def copy_kv(src, cache, pos, stride):
    """copy_kv launch (LaunchConfig::for_num_elems: 1024-thread blocks), ops.cu:471-486."""
    kernels().launch("copy_kv_f16", ((stride + 1023) // 1024,), (1024,), 0, src, cache, pos, 1, stride)


def attention(q, kc, vc, n_head, n_kv, hd, pos):
    """launch_attn flash route, layer.rs:2040-2121: partial grid (n_head, 8) x 128, smem (hd+64)*4;
    reduce grid n_head x hd."""
    partial = torch.zeros(n_head * 8 * (2 + hd), dtype=torch.float32, device="cuda")
    out = torch.zeros(n_head * hd, dtype=torch.float32, device="cuda")
    scale = float(1.0 / np.sqrt(np.float32(hd)))
    kernels().launch("attn_flash_partial", (n_head, 8, 1), (128,), (hd + 64) * 4, q, kc, vc, partial, n_head, n_kv, hd,
                     pos, 1, 8, scale)
    kernels().launch("attn_flash_reduce", (n_head, 1), (hd,), 0, partial, out, n_head, hd, 8, 1)
    return out


def argmax(x):
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels().launch("argmax_f32", (1,), (256,), 0, x, x.numel(), out)
    return out


def embed(table: RefMat, token: int):
    out = torch.zeros(table.K, dtype=torch.float32, device="cuda")
    name = "embed_q6_k_one" if table.type == Q6_K else "embed_q4_k_one"
    kernels().launch(name, (1,), (32,), 0, table.data, out, token, table.K, table.col_bytes)
    return out


# ------------------------------------------------------------------ hybrid-layer kernels

def gdn_conv_qkvl2(qkv, conv_w, conv_state, n_k, n_v, d, kernel, eps):
    """layer.rs:845-862: grid n_k x 128 (deltanet.cu:561-622); conv_state [kernel-1][channels] is updated."""
    q = torch.zeros(n_k * d, dtype=torch.float32, device="cuda")
    k = torch.zeros(n_k * d, dtype=torch.float32, device="cuda")
    v = torch.zeros(n_v * d, dtype=torch.float32, device="cuda")
    kernels().launch("gdn_conv_qkvl2_one_f32", (n_k,), (128,), 0, qkv, conv_w, conv_state, q, k, v, n_k, n_v, d, kernel,
                     float(eps))
    return q, k, v


def gdn_delta_gated_d128(q, k, v, alpha, beta, dt, a, state, norm_w, z, n_k, n_v, eps):
    """layer.rs:863-885: grid n_v x 128 (deltanet.cu:628-728); state [n_v][128][128] is updated."""
    out = torch.zeros(n_v * 128, dtype=torch.float32, device="cuda")
    kernels().launch("gdn_delta_gated_one_d128_f32", (n_v,), (128,), 0, q, k, v, alpha, beta, dt, a, state, norm_w, z, out,
                     n_k, n_v, float(eps))
    return out


def split_q_gate(qg, n_head, hd):
    """layer.rs:386-410: grid (n_head, 1) x 128, interleaved mode (deltanet.cu:144-173)."""
    q = torch.zeros(n_head * hd, dtype=torch.float32, device="cuda")
    g = torch.zeros(n_head * hd, dtype=torch.float32, device="cuda")
    kernels().launch("split_q_gate_interleaved_f32", (n_head, 1), (128,), 0, qg, q, g, n_head, hd, 1, 0)
    return q, g


def qk_norm_partial_rope(x, w, n_heads, hd, n_rot, pos, theta, eps):
    """layer.rs:430-505: grid (heads, 1) x 128, in place (deltanet.cu:189-235)."""
    kernels().launch("qk_rms_norm_partial_rope_neox_f32", (n_heads, 1), (128,), 0, x, w, n_heads, hd, n_rot, pos, 1,
                     float(theta), float(eps))
    return x


def mul_sigmoid(x, gate):
    """layer.rs:646-659 (deltanet.cu:176-186)."""
    n = x.numel()
    kernels().launch("mul_sigmoid_f32", ((n + 1023) // 1024,), (1024,), 0, x, gate, n)
    return x


# ------------------------------------------------------------------ whole model

class RefModel:
    """The reference's n_tok = 1 schedule (layer.rs:142-709, 711-1208, 1210-1456, 2125-2259)
    assembled from its own kernels, for the Q4_K / Q6_K mix of the benchmark configurations,
    dense or hybrid."""

    def __init__(self, cfg: dict, tensors: dict, max_seq: int, alt_ffn: bool = False):
        """alt_ffn: use the reference's other FFN kernel (gemv_q4_k_ffn_8way).  Both are the
        reference; they differ only in fp32 summation order, which makes the pair a measure of
        how far the reference's logits move under reassociation alone."""
        self.cfg, self.max_seq, self.alt_ffn = cfg, max_seq, alt_ffn
        L = cfg["n_layer"]

        def m(name):
            t, K, N, data = tensors[name]
            return RefMat(t, K, N, data)

        def v(name):
            return dev(tensors[name]) if name in tensors else None

        self.embd = m("token_embd.weight")
        self.head = m("output.weight") if "output.weight" in tensors else self.embd
        self.out_norm = v("output_norm.weight")
        self.layers = []
        self.hybrid = cfg.get("arch") in ("qwen35", "qwen3_5")
        iv = cfg.get("full_attention_interval", 4)
        for i in range(L):
            p = f"blk.{i}."
            ly = dict(gate=m(p + "ffn_gate.weight"), up=m(p + "ffn_up.weight"), down=m(p + "ffn_down.weight"),
                      an=v(p + "attn_norm.weight"), fn=v(p + "ffn_norm.weight"), kind="dense")
            if self.hybrid and (i + 1) % iv != 0:
                ly.update(kind="linear", wqkv=m(p + "attn_qkv.weight"), wgate=m(p + "attn_gate.weight"),
                          wbeta=m(p + "ssm_beta.weight"), walpha=m(p + "ssm_alpha.weight"), ssm_out=m(p + "ssm_out.weight"),
                          conv=v(p + "ssm_conv1d.weight"), a=v(p + "ssm_a"), dt=v(p + "ssm_dt.bias"),
                          norm=v(p + "ssm_norm.weight"))
            else:
                ly.update(wq=m(p + "attn_q.weight"), wk=m(p + "attn_k.weight"), wv=m(p + "attn_v.weight"),
                          wo=m(p + "attn_output.weight"), bq=v(p + "attn_q.bias"), bk=v(p + "attn_k.bias"),
                          bv=v(p + "attn_v.bias"))
                if self.hybrid:
                    ly.update(kind="gated", qn=v(p + "attn_q_norm.weight"), kn=v(p + "attn_k_norm.weight"))
            self.layers.append(ly)
        if self.hybrid:
            d, nk, nv = cfg["ssm_state"], cfg["ssm_n_k"], cfg["ssm_n_v"]
            ch = (2 * nk + nv) * d
            self.ssm = [torch.zeros(nv * d * d, dtype=torch.float32, device="cuda") for _ in range(L)]
            self.conv = [torch.zeros((cfg["conv_kernel"] - 1) * ch, dtype=torch.float32, device="cuda") for _ in range(L)]
        kvn = cfg["n_kv"] * cfg["head_dim"]
        self.kc = [torch.zeros(max_seq * kvn, dtype=torch.int16, device="cuda") for _ in range(L)]
        self.vc = [torch.zeros(max_seq * kvn, dtype=torch.int16, device="cuda") for _ in range(L)]

    def layer_forward(self, li: int, x: torch.Tensor, pos: int, taps: dict | None = None) -> torch.Tensor:
        """One decoder layer applied in place to the residual stream x at position pos."""
        c = self.cfg
        H, Hkv, hd = c["n_head"], c["n_kv"], c["head_dim"]
        kvn = Hkv * hd
        L = self.layers[li]
        xb = rms_norm(x, L["an"], c["eps"])
        if L["kind"] == "linear":
            d, nk, nv = c["ssm_state"], c["ssm_n_k"], c["ssm_n_v"]
            qkv, z = gemv_q8(L["wqkv"], xb), gemv_q8(L["wgate"], xb)
            beta, alpha = gemv_q8(L["wbeta"], xb), gemv_q8(L["walpha"], xb)
            gq, gk, gv = gdn_conv_qkvl2(qkv, L["conv"], self.conv[li], nk, nv, d, c["conv_kernel"], c["eps"])
            att = gdn_delta_gated_d128(gq, gk, gv, alpha, beta, L["dt"], L["a"], self.ssm[li], L["norm"], z, nk, nv, c["eps"])
            q = gq
            gemv_q8(L["ssm_out"], att, out=x, use_res=2)
        else:
            q, k = gemv_q4_pair(L["wq"], L["wk"], xb, L["bq"], L["bk"])
            if L["wv"].type == Q6_K:
                v = gemv_q6_f32(L["wv"], xb, L["bv"])
            else:
                v = gemv_q8(L["wv"], xb, bias=L["bv"])
            if L["kind"] == "gated":
                n_rot = c["rope_dim"] if 0 < c.get("rope_dim", 0) < hd else hd
                q, g = split_q_gate(q, H, hd)
                qk_norm_partial_rope(q, L["qn"], H, hd, n_rot, pos, c["rope_theta"], c["eps"])
                qk_norm_partial_rope(k, L["kn"], Hkv, hd, n_rot, pos, c["rope_theta"], c["eps"])
            else:
                rope(q, H, hd, pos, c["rope_theta"])
                rope(k, Hkv, hd, pos, c["rope_theta"])
            copy_kv(k, self.kc[li], pos, kvn)
            copy_kv(v, self.vc[li], pos, kvn)
            att = attention(q, self.kc[li], self.vc[li], H, Hkv, hd, pos)
            if L["kind"] == "gated":
                mul_sigmoid(att, g)
            gemv_q8(L["wo"], att, out=x, use_res=2)
        xb = rms_norm(x, L["fn"], c["eps"])
        h = (ffn_gate_up_8way if self.alt_ffn else ffn_gate_up)(L["gate"], L["up"], xb)
        gemv_q8(L["down"], h, out=x, use_res=2)
        if taps is not None:
            taps[f"q{li}"], taps[f"attn{li}"], taps[f"h{li}"], taps[f"x{li}"] = q, att, h, x.clone()
        return x

    def head_forward(self, x: torch.Tensor) -> torch.Tensor:
        xb = rms_norm(x, self.out_norm, self.cfg["eps"])
        return gemv_q8(self.head, xb)

    def decode_token(self, pos: int, token: int, taps: dict | None = None) -> torch.Tensor:
        x = embed(self.embd, token)
        for li in range(len(self.layers)):
            x = self.layer_forward(li, x, pos, taps)
        if taps is not None:
            taps["x"] = x.clone()
        return self.head_forward(x)

    def decode_greedy(self, pos0: int, first: int, n: int):
        toks, margins, tok = [], [], first
        logits = None
        for s in range(n):
            logits = self.decode_token(pos0 + s, tok)
            top2 = torch.topk(logits, 2)
            tok = int(argmax(logits).item())
            toks.append(tok)
            margins.append(float(top2.values[0] - top2.values[1]))
        return np.array(toks, np.int32), np.array(margins, np.float32), logits.cpu().numpy()
