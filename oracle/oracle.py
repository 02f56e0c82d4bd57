"""ctypes binding of the CPU restatement (oracle/tfr_oracle.c).

Test infrastructure only: imported by tests/, by the smoke check and by the CPU-baseline
legs of bench.py.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"

Q4_K, Q6_K, Q8_0 = 12, 14, 8
BLOCK_BYTES = {Q4_K: 144, Q6_K: 210, Q8_0: 8 * 34}  # bytes per 256 weights


def build(force: bool = False) -> None:
    """Compile liboracle.so (and the reference cubin when the reference checkout exists)."""
    srcs = [HERE / "tfr_oracle.c", HERE / "tfr_oracle_gdn.c"]
    stale = force or not LIB_PATH.exists() or any(s.stat().st_mtime > LIB_PATH.stat().st_mtime for s in srcs)
    if stale:
        subprocess.run(["make", "-C", str(HERE), str(LIB_PATH)], check=True, capture_output=True)


class Mat(C.Structure):
    _fields_ = [("type", C.c_int32), ("K", C.c_int32), ("N", C.c_int32), ("pad_", C.c_int32),
                ("data", C.c_void_p)]


LAYER_DENSE, LAYER_LINEAR, LAYER_FULL_GATED = 0, 1, 2


class Layer(C.Structure):
    _fields_ = [(n, Mat) for n in ("wq", "wk", "wv", "wo", "gate", "up", "down")] + \
               [(n, C.c_void_p) for n in ("bq", "bk", "bv", "attn_norm", "ffn_norm")] + \
               [("kind", C.c_int32), ("pad_", C.c_int32)] + \
               [(n, Mat) for n in ("wqkv", "wgate", "wbeta", "walpha", "ssm_out")] + \
               [(n, C.c_void_p) for n in ("conv1d", "ssm_a", "ssm_dt", "ssm_norm", "q_norm", "k_norm")]


class Model(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "n_embd", "n_head", "n_kv", "head_dim", "n_ff",
                                         "n_vocab", "max_seq")] + \
               [("rope_theta", C.c_float), ("eps", C.c_float),
                ("token_embd", Mat), ("output", Mat), ("output_norm", C.c_void_p),
                ("layers", C.POINTER(Layer))] + \
               [(n, C.c_int32) for n in ("rope_dim", "ssm_n_k", "ssm_n_v", "ssm_state", "conv_kernel", "pad_")]


class Taps(C.Structure):
    _fields_ = [("x_final", C.c_void_p), ("xn_final", C.c_void_p)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(LIB_PATH))
        _lib.tfo_half_to_float.restype = C.c_float
        _lib.tfo_half_to_float.argtypes = [C.c_uint16]
        _lib.tfo_float_to_half_bits.restype = C.c_uint16
        _lib.tfo_float_to_half_bits.argtypes = [C.c_float]
        for name in ("tfo_dot_q4k_q8", "tfo_dot_q6k_q8"):
            f = getattr(_lib, name)
            f.restype = C.c_float
            f.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        for name in ("tfo_dot_q6k_f32", "tfo_dot_q4k_f32"):
            f = getattr(_lib, name)
            f.restype = C.c_float
            f.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        _lib.tfo_gemv.argtypes = [C.POINTER(Mat), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        _lib.tfo_ffn_gate_up.argtypes = [C.POINTER(Mat), C.POINTER(Mat), C.c_void_p, C.c_void_p]
        _lib.tfo_decode_token.argtypes = [C.POINTER(Model), C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                          C.c_void_p, C.POINTER(Taps), C.c_int, C.c_void_p, C.c_void_p]
        _lib.tfo_decode_greedy.argtypes = [C.POINTER(Model), C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                           C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        _lib.tfo_layer_forward.argtypes = [C.POINTER(Model), C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                           C.c_void_p, C.c_void_p]
        _lib.tfo_linear_attn_block.argtypes = [C.POINTER(Model), C.POINTER(Layer)] + [C.c_void_p] * 4
        _lib.tfo_gated_attn_block.argtypes = [C.POINTER(Model), C.POINTER(Layer)] + [C.c_void_p] * 4 + [C.c_int]
        _lib.tfo_gdn_step.argtypes = [C.c_void_p] * 11 + [C.c_int] * 4 + [C.c_float]
        _lib.tfo_qk_norm_partial_rope.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 4 + [C.c_float, C.c_float]
        _lib.tfo_head_forward.argtypes = [C.POINTER(Model), C.c_void_p, C.c_void_p, C.c_void_p]
        _lib.tfo_embed.argtypes = [C.POINTER(Model), C.c_int, C.c_void_p]
        _lib.tfo_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_float]
        _lib.tfo_float_to_half_bits_range.restype = None
        _lib.tfo_float_to_half_bits_range.argtypes = [C.c_uint32, C.c_uint64, C.c_void_p]
        _lib.tfo_set_layer_taps.restype = None
        _lib.tfo_set_layer_taps.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        _lib.tfo_rope_neox.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float]
        _lib.tfo_attention.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float]
        _lib.tfo_quantize_q8.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        _lib.tfo_dequant_row.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        _lib.tfo_q4k_subdots.argtypes = [C.c_void_p] * 4
        _lib.tfo_q6k_groupdots.argtypes = [C.c_void_p] * 3
        _lib.tfo_copy_kv_f16.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        _lib.tfo_argmax.argtypes = [C.c_void_p, C.c_int]
        _lib.tfo_set_threads.argtypes = [C.c_int]
        _lib.tfo_q8_0_blockdots.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        _lib.tfo_transcode_q5_k_to_q8_0.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        _lib.tfo_transcode_q5_1_to_q8_0.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
    return _lib


def layer_kind(cfg: dict, i: int) -> int:
    """config.rs:174-199: in the hybrid architecture layer i is a (gated) full-attention layer iff
    (i + 1) % full_attention_interval == 0, every other layer a Gated-DeltaNet mixer."""
    if cfg.get("arch") not in ("qwen35", "qwen3_5"):
        return LAYER_DENSE
    return LAYER_FULL_GATED if (i + 1) % cfg.get("full_attention_interval", 4) == 0 else LAYER_LINEAR


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def set_threads(n: int) -> None:
    lib().tfo_set_threads(int(n))


def max_threads() -> int:
    return int(lib().tfo_max_threads())


def half_to_float(bits: np.ndarray) -> np.ndarray:
    """Exact f16 -> f32 widening (numpy's own conversion is the same IEEE operation)."""
    return np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)


def float_to_half_bits(x) -> np.ndarray:
    x = _f32(x).ravel()
    out = np.empty(x.size, np.uint16)
    f = lib().tfo_float_to_half_bits
    for i, v in enumerate(x):
        out[i] = f(float(v))
    return out


def float_to_half_bits_range(first: int, count: int) -> np.ndarray:
    """f16 bits of the `count` consecutive fp32 bit patterns starting at `first` (all host threads)."""
    out = np.empty(count, np.uint16)
    lib().tfo_float_to_half_bits_range(C.c_uint32(first), C.c_uint64(count), _p(out))
    return out


def quantize_q8(x) -> tuple[np.ndarray, np.ndarray]:
    x = _f32(x)
    q = np.zeros(x.size, np.int8)
    d = np.zeros(x.size // 32, np.float32)
    lib().tfo_quantize_q8(_p(x), x.size, _p(q), _p(d))
    return q, d


def mat(wtype: int, data: np.ndarray, K: int, N: int) -> Mat:
    """Wrap raw GGUF bytes (uint8 array that the caller keeps alive) as a matrix."""
    assert data.dtype == np.uint8 and data.flags["C_CONTIGUOUS"]
    assert data.size == N * (K // 256) * BLOCK_BYTES[wtype], (data.size, N, K, wtype)
    m = Mat(wtype, K, N, 0, _p(data))
    m._keep = data  # the struct only holds the address
    return m


def dequant_rows(wtype: int, data: np.ndarray, K: int, N: int) -> np.ndarray:
    out = np.empty((N, K), np.float32)
    rb = (K // 256) * BLOCK_BYTES[wtype]
    flat = np.ascontiguousarray(data).ravel()
    for j in range(N):
        rc = lib().tfo_dequant_row(wtype, _p(flat) + j * rb, K, _p(out) + j * K * 4)
        assert rc == 0
    return out


def gemv(m: Mat, x, out=None, bias=None, use_res: int = 0, act_mode: int = 0) -> np.ndarray:
    x = _f32(x)
    if out is None:
        out = np.zeros(m.N, np.float32)
    b = _f32(bias) if bias is not None else None
    rc = lib().tfo_gemv(C.byref(m), _p(x), _p(out), _p(b) if b is not None else None, use_res, act_mode)
    assert rc == 0
    return out


def ffn_gate_up(gate: Mat, up: Mat, x) -> np.ndarray:
    x = _f32(x)
    out = np.zeros(gate.N, np.float32)
    assert lib().tfo_ffn_gate_up(C.byref(gate), C.byref(up), _p(x), _p(out)) == 0
    return out


def q4k_subdots(block: np.ndarray, q8: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    I = np.zeros(8, np.int32)
    S = np.zeros(8, np.int32)
    lib().tfo_q4k_subdots(_p(block), _p(q8), _p(I), _p(S))
    return I, S


def q6k_groupdots(block: np.ndarray, q8: np.ndarray) -> np.ndarray:
    J = np.zeros(16, np.int32)
    lib().tfo_q6k_groupdots(_p(block), _p(q8), _p(J))
    return J


def q8_0_blockdots(row: np.ndarray, K: int, q8: np.ndarray) -> np.ndarray:
    sums = np.zeros(K // 32, np.int32)
    lib().tfo_q8_0_blockdots(_p(row), K, _p(q8), _p(sums))
    return sums


def transcode_to_q8_0(src_type: int, raw: np.ndarray) -> np.ndarray:
    """Q5_K (13) or Q5_1 (7) bytes -> Q8_0 bytes, the reference loader's one-off conversion (load.rs:33-133)."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    blk, per = (176, 8) if src_type == 13 else (24, 1)
    out = np.zeros(raw.size // blk * per * 34, np.uint8)
    f = lib().tfo_transcode_q5_k_to_q8_0 if src_type == 13 else lib().tfo_transcode_q5_1_to_q8_0
    assert f(_p(raw), raw.size, _p(out)) == 0
    return out


def rms_norm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().tfo_rms_norm(_p(x), _p(w), _p(out), x.size, eps)
    return out


def rope_neox(x, n_heads: int, head_dim: int, pos: int, theta: float) -> np.ndarray:
    x = _f32(x).copy()
    lib().tfo_rope_neox(_p(x), n_heads, head_dim, pos, theta)
    return x


def attention(q, kc: np.ndarray, vc: np.ndarray, n_head: int, n_kv: int, hd: int, pos: int) -> np.ndarray:
    q = _f32(q)
    out = np.zeros(n_head * hd, np.float32)
    lib().tfo_attention(_p(q), _p(kc), _p(vc), _p(out), n_head, n_kv, hd, pos, float(1.0 / np.sqrt(np.float32(hd))))
    return out


def gdn_step(qkv, z, beta, alpha, conv_w, conv_state, ssm, ssm_a, ssm_dt, norm_w, nk: int, nv: int, d: int,
             kernel: int, eps: float) -> np.ndarray:
    """Gated-DeltaNet decode step after the projections; conv_state [kernel-1][channels] and
    ssm [nv][d][d] (float32 arrays) are updated in place."""
    args = [_f32(a) for a in (qkv, z, beta, alpha, conv_w)]
    assert conv_state.dtype == np.float32 and ssm.dtype == np.float32
    vecs = [_f32(a) for a in (ssm_a, ssm_dt, norm_w)]
    y = np.zeros(nv * d, np.float32)
    rc = lib().tfo_gdn_step(*[_p(a) for a in args], _p(conv_state), _p(ssm), *[_p(a) for a in vecs], _p(y), nk, nv, d,
                            kernel, eps)
    assert rc == 0
    return y


def qk_norm_partial_rope(x, w, n_heads: int, hd: int, n_rot: int, pos: int, theta: float, eps: float) -> np.ndarray:
    x = _f32(x).copy()
    w = _f32(w) if w is not None else None
    lib().tfo_qk_norm_partial_rope(_p(x), _p(w) if w is not None else None, n_heads, hd, n_rot, pos, theta, eps)
    return x


class OracleModel:
    """Dense or hybrid decoder held as raw GGUF tensors (dict name -> (ggml_type, K, N, uint8 array)
    for matrices, name -> float32 array for vectors), with the names of cuda/load.rs:280-417."""

    def __init__(self, cfg: dict, tensors: dict, max_seq: int):
        self.cfg, self.tensors, self.max_seq = cfg, tensors, max_seq
        L = cfg["n_layer"]
        self._keep = []
        self._layers = (Layer * L)()

        def m(name):
            t, K, N, data = tensors[name]
            return mat(t, data, K, N)

        def v(name):
            if name not in tensors:
                return None
            a = _f32(tensors[name])
            self._keep.append(a)
            return _p(a)

        self.kinds = [layer_kind(cfg, i) for i in range(L)]
        for i in range(L):
            p = f"blk.{i}."
            ly = self._layers[i]
            ly.kind = self.kinds[i]
            if ly.kind == LAYER_LINEAR:
                ly.wqkv, ly.wgate, ly.wbeta, ly.walpha, ly.ssm_out = (
                    m(p + n + ".weight") for n in ("attn_qkv", "attn_gate", "ssm_beta", "ssm_alpha", "ssm_out"))
                ly.conv1d, ly.ssm_a, ly.ssm_dt, ly.ssm_norm = (
                    v(p + n) for n in ("ssm_conv1d.weight", "ssm_a", "ssm_dt.bias", "ssm_norm.weight"))
            else:
                ly.wq, ly.wk, ly.wv, ly.wo = (m(p + n + ".weight") for n in ("attn_q", "attn_k", "attn_v", "attn_output"))
                ly.bq, ly.bk, ly.bv = v(p + "attn_q.bias"), v(p + "attn_k.bias"), v(p + "attn_v.bias")
                ly.q_norm, ly.k_norm = v(p + "attn_q_norm.weight"), v(p + "attn_k_norm.weight")
            ly.gate, ly.up, ly.down = (m(p + n + ".weight") for n in ("ffn_gate", "ffn_up", "ffn_down"))
            ly.attn_norm = v(p + "attn_norm.weight")
            ly.ffn_norm = v(p + "ffn_norm.weight") or v(p + "post_attention_norm.weight")
        self.m = Model()
        for k in ("n_layer", "n_embd", "n_head", "n_kv", "head_dim", "n_ff", "n_vocab"):
            setattr(self.m, k, cfg[k])
        self.m.max_seq = max_seq
        self.m.rope_theta, self.m.eps = cfg["rope_theta"], cfg["eps"]
        self.m.token_embd = m("token_embd.weight")
        if "output.weight" in tensors:
            self.m.output = m("output.weight")
        self.m.output_norm = v("output_norm.weight")
        self.m.layers = self._layers
        self.hybrid = any(k != LAYER_DENSE for k in self.kinds)
        if self.hybrid:
            self.m.rope_dim = cfg.get("rope_dim", 0)
            self.m.ssm_n_k, self.m.ssm_n_v = cfg["ssm_n_k"], cfg["ssm_n_v"]
            self.m.ssm_state, self.m.conv_kernel = cfg["ssm_state"], cfg["conv_kernel"]
        kvn = cfg["n_kv"] * cfg["head_dim"]
        self.kc = np.zeros((L, max_seq, kvn), np.uint16)
        self.vc = np.zeros((L, max_seq, kvn), np.uint16)
        # recurrent state of the linear layers (kv.rs:12-15): S[n_v][d][d] and the conv ring [kernel-1][channels]
        d = cfg.get("ssm_state", 0)
        ch = (2 * cfg.get("ssm_n_k", 0) + cfg.get("ssm_n_v", 0)) * d
        self.ssm = np.zeros((L, max(1, cfg.get("ssm_n_v", 0) * d * d)), np.float32)
        self.conv = np.zeros((L, max(1, (cfg.get("conv_kernel", 1) - 1) * ch)), np.float32)

    def zero_recurrent(self) -> None:
        self.ssm[:] = 0
        self.conv[:] = 0

    def _state(self):
        return (_p(self.ssm), _p(self.conv)) if self.hybrid else (None, None)

    def decode_token(self, pos: int, token: int, act_f32: bool = False, want_taps: bool = False):
        logits = np.zeros(self.cfg["n_vocab"], np.float32)
        taps = Taps()
        xf = np.zeros(self.cfg["n_embd"], np.float32)
        xn = np.zeros(self.cfg["n_embd"], np.float32)
        taps.x_final, taps.xn_final = _p(xf), _p(xn)
        rc = lib().tfo_decode_token(C.byref(self.m), _p(self.kc), _p(self.vc), pos, token, _p(logits),
                                    C.byref(taps), int(act_f32), *self._state())
        assert rc == 0, rc
        return (logits, xf, xn) if want_taps else logits

    def embed(self, token: int) -> np.ndarray:
        x = np.zeros(self.cfg["n_embd"], np.float32)
        assert lib().tfo_embed(C.byref(self.m), token, _p(x)) == 0
        return x

    def layer_forward(self, li: int, x: np.ndarray, pos: int) -> np.ndarray:
        """One layer applied to a copy of the residual stream x at position pos (writes cache row pos)."""
        x = _f32(x).copy()
        st = (_p(self.ssm[li]), _p(self.conv[li])) if self.hybrid else (None, None)
        rc = lib().tfo_layer_forward(C.byref(self.m), li, _p(x), _p(self.kc[li]), _p(self.vc[li]), pos, 0, *st)
        assert rc == 0, rc
        return x

    def layer_forward_taps(self, li: int, x: np.ndarray, pos: int):
        """layer_forward of a dense layer plus the three vectors it quantises on the way: attention output, residual
        stream after o-proj, SiLU*mul."""
        c = self.cfg
        attn = np.zeros(c["n_head"] * c["head_dim"], np.float32)
        mid = np.zeros(c["n_embd"], np.float32)
        h = np.zeros(c["n_ff"], np.float32)
        lib().tfo_set_layer_taps(_p(attn), _p(mid), _p(h))
        try:
            out = self.layer_forward(li, x, pos)
        finally:
            lib().tfo_set_layer_taps(None, None, None)
        return out, attn, mid, h

    def head_forward(self, x: np.ndarray) -> np.ndarray:
        x = _f32(x)
        logits = np.zeros(self.cfg["n_vocab"], np.float32)
        assert lib().tfo_head_forward(C.byref(self.m), _p(x), _p(logits), None) == 0
        return logits

    def decode_greedy(self, pos0: int, first: int, n: int):
        toks = np.zeros(n, np.int32)
        margins = np.zeros(n, np.float32)
        last = np.zeros(self.cfg["n_vocab"], np.float32)
        rc = lib().tfo_decode_greedy(C.byref(self.m), _p(self.kc), _p(self.vc), pos0, first, n, _p(toks),
                                     _p(margins), _p(last), *self._state())
        assert rc == 0, rc
        return toks, margins, last
