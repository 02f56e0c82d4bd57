"""Host-side mirror of the reference's device-runtime interface over the C ABI.

Names and behaviour follow crates/core/src/cuda: `CudaModel` (model.rs:18-201,
forward.rs:20-105, load.rs:166) and `CudaKv` (kv.rs:6-42).  Errors surface as
`TfrError` carrying the reference's messages ("empty tokens", "context full").
Everything here is plumbing around libtarafer_b200.so; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import ModelConfig

TYPE_F32, TYPE_Q4_K, TYPE_Q6_K = 0, 12, 14


class TfrError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code, self.msg = code, msg


def _ptr(a) -> int:
    """Address of a numpy array, a torch tensor (host or device) or a raw integer."""
    if a is None:
        return 0
    if isinstance(a, int):
        return a
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    return a.data_ptr()


def _nbytes(a) -> int:
    return a.nbytes if isinstance(a, np.ndarray) else a.numel() * a.element_size()


def model_config(cfg: dict, context_length: int = 4096) -> ModelConfig:
    c = ModelConfig()
    c.n_layer, c.n_embd, c.n_head, c.n_kv_head = cfg["n_layer"], cfg["n_embd"], cfg["n_head"], cfg["n_kv"]
    c.head_dim, c.n_ff, c.n_vocab = cfg["head_dim"], cfg["n_ff"], cfg["n_vocab"]
    c.context_length = context_length
    c.rope_theta, c.rms_eps = cfg["rope_theta"], cfg["eps"]
    # hybrid keys as ModelConfig::from_gguf reads them (config.rs:174-199): rope.dimension_count,
    # ssm.conv_kernel / state_size / group_count (K heads) / time_step_rank (V heads) / inner_size
    c.hybrid = int(cfg.get("arch") in ("qwen35", "qwen3_5"))
    if c.hybrid:
        c.rope_dim = int(cfg.get("rope_dim", 0))
        c.ssm_conv_kernel, c.ssm_state_size = int(cfg["conv_kernel"]), int(cfg["ssm_state"])
        c.ssm_group_count, c.ssm_time_step_rank = int(cfg["ssm_n_k"]), int(cfg["ssm_n_v"])
        c.ssm_inner_size = c.ssm_time_step_rank * c.ssm_state_size
        c.full_attention_interval = int(cfg.get("full_attention_interval", 4))
    c.tp_rank, c.tp_size = int(cfg.get("tp_rank", 0)), int(cfg.get("tp_size", 1))
    return c


class GgufFile:
    """crates/gguf GgufFile over the C ABI: header, metadata and tensor table of a mapped GGUF file.
    Host code only (works without a GPU)."""

    def __init__(self, path):
        h = C.c_void_p()
        err = C.create_string_buffer(512)
        rc = _lib.lib().tfr_gguf_open(str(path).encode(), C.byref(h), err, 512)
        if rc:
            raise TfrError(rc, err.value.decode())
        self._h = h.value
        self.path = str(path)

    @property
    def version(self) -> int:
        return _lib.lib().tfr_gguf_version(self._h)

    @property
    def data_offset(self) -> int:
        return int(_lib.lib().tfr_gguf_data_offset(self._h))

    def tensors(self) -> list[dict]:
        out = []
        for i in range(_lib.lib().tfr_gguf_tensor_count(self._h)):
            name, ty, nd = C.c_char_p(), C.c_int(), C.c_int()
            dims = (C.c_int64 * 4)()
            off, nb = C.c_uint64(), C.c_uint64()
            _lib.lib().tfr_gguf_tensor_info(self._h, i, C.byref(name), C.byref(ty), C.byref(nd), C.byref(dims), C.byref(off),
                                            C.byref(nb))
            out.append(dict(name=name.value.decode(), ggml_type=ty.value, dims=list(dims)[: nd.value], offset=off.value,
                            nbytes=nb.value))
        return out

    def tensor_bytes(self, name: str) -> np.ndarray:
        i = _lib.lib().tfr_gguf_find_tensor(self._h, name.encode())
        if i < 0:
            raise KeyError(name)
        nb = self.tensors()[i]["nbytes"]
        p = _lib.lib().tfr_gguf_tensor_data(self._h, i)
        return np.ctypeslib.as_array((C.c_uint8 * nb).from_address(p)).copy()

    def meta_u64(self, key: str):
        v = C.c_uint64()
        return int(v.value) if _lib.lib().tfr_gguf_meta_u64(self._h, key.encode(), C.byref(v)) == 0 else None

    def meta_f32(self, key: str):
        v = C.c_float()
        return float(v.value) if _lib.lib().tfr_gguf_meta_f32(self._h, key.encode(), C.byref(v)) == 0 else None

    def meta_str(self, key: str):
        v = C.c_char_p()
        return v.value.decode() if _lib.lib().tfr_gguf_meta_str(self._h, key.encode(), C.byref(v)) == 0 else None

    def meta_array_len(self, key: str) -> int:
        return int(_lib.lib().tfr_gguf_meta_array_len(self._h, key.encode()))

    def meta_array(self, key: str) -> list | None:
        """Items of a metadata array: bytes objects for string arrays (tokenizer.ggml.tokens / .merges), floats
        (.scores) or integers (.token_type); None when the key is missing or holds another item kind."""
        n = self.meta_array_len(key)
        if n < 0:
            return None
        l, k = _lib.lib(), key.encode()
        out: list = []
        sp, sl, fv, iv = C.c_char_p(), C.c_uint64(), C.c_float(), C.c_int64()
        for i in range(n):
            if l.tfr_gguf_meta_array_str(self._h, k, i, C.byref(sp), C.byref(sl)) == 0:
                out.append(C.string_at(sp, sl.value))
            elif l.tfr_gguf_meta_array_f32(self._h, k, i, C.byref(fv)) == 0:
                out.append(float(fv.value))
            elif l.tfr_gguf_meta_array_i64(self._h, k, i, C.byref(iv)) == 0:
                out.append(int(iv.value))
            else:
                return None
        return out

    def model_config(self) -> ModelConfig:
        c = ModelConfig()
        err = C.create_string_buffer(512)
        rc = _lib.lib().tfr_gguf_model_config(self._h, C.byref(c), err, 512)
        if rc:
            raise TfrError(rc, err.value.decode())
        return c

    def close(self) -> None:
        if self._h:
            _lib.lib().tfr_gguf_close(self._h)
            self._h = 0


class CudaKv:
    """kv.rs:6-42: append-only f16 K/V arena; `len` is assignable by the caller (session.rs:345)."""

    def __init__(self, model: "CudaModel", handle: int):
        self._model, self._h = model, handle

    @property
    def len(self) -> int:
        return _lib.lib().tfr_kv_len(self._h)

    @len.setter
    def len(self, n: int) -> None:
        rc = _lib.lib().tfr_kv_set_len(self._h, int(n))
        if rc:
            raise TfrError(rc, "kv length out of range")

    @property
    def max_seq(self) -> int:
        return _lib.lib().tfr_kv_max_seq(self._h)

    def clear(self) -> None:
        _lib.lib().tfr_kv_clear(self._h)

    def bytes_per_token(self) -> int:
        return _lib.lib().tfr_kv_bytes_per_token(self._h)

    def free(self) -> None:
        if self._h:
            _lib.lib().tfr_free_kv(self._h)
            self._h = 0


class CudaModel:
    """model.rs:18-201 / forward.rs: the decode engine for one GPU."""

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        rc = _lib.lib().tfr_create(device, C.byref(h))
        if rc:
            raise TfrError(rc, "tfr_create failed: no usable CUDA device (this library has no CPU fallback)")
        self._h = h.value
        self.cfg: dict | None = None
        name = C.create_string_buffer(256)
        maj, mnr, sms = C.c_int(), C.c_int(), C.c_int()
        _lib.lib().tfr_device_info(self._h, name, 256, C.byref(maj), C.byref(mnr), C.byref(sms))
        self.gpu_name, self.compute_major, self.compute_minor = name.value.decode(), maj.value, mnr.value
        self.sm_count = sms.value

    # -- loading (load.rs:166-609) ------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc:
            raise TfrError(rc, _lib.lib().tfr_last_error(self._h).decode())

    def set_config(self, cfg: dict, context_length: int = 4096) -> None:
        self.cfg = dict(cfg)
        c = model_config(cfg, context_length)
        self._check(_lib.lib().tfr_set_config(self._h, C.byref(c)))

    def upload_tensor(self, name: str, ggml_type: int, n_rows: int, n_cols: int, data) -> None:
        """`data`: numpy array or torch tensor (host or device) holding the raw GGUF bytes."""
        self._check(_lib.lib().tfr_upload_tensor(self._h, name.encode(), ggml_type, n_rows, n_cols, _ptr(data),
                                                 _nbytes(data)))

    def finalize_load(self) -> None:
        self._check(_lib.lib().tfr_finalize_load(self._h))

    @classmethod
    def load_with(cls, cfg: dict, tensors: dict, device: int = 0, context_length: int = 4096,
                  vocab_shortlist: tuple[int, int] | None = None) -> "CudaModel":
        """CudaModel::load_with for tensors already in memory: name -> (type, K, N, bytes) for
        matrices, name -> fp32 array for vectors.  vocab_shortlist = (limit, extra id or -1)."""
        m = cls(device)
        m.set_config(cfg, context_length)
        if vocab_shortlist:
            m.set_vocab_shortlist(*vocab_shortlist)
        for name, t in tensors.items():
            if isinstance(t, tuple):
                wt, K, N, data = t
                m.upload_tensor(name, wt, K, N, data)
            else:
                a = np.ascontiguousarray(t, dtype=np.float32) if isinstance(t, np.ndarray) else t
                m.upload_tensor(name, TYPE_F32, _nbytes(a) // 4, 1, a)
        m.finalize_load()
        return m

    @classmethod
    def load_gguf(cls, path, device: int = 0, tp_rank: int = 0, tp_size: int = 1) -> "CudaModel":
        """CudaModel::load_with(gguf): configuration and tensors straight from a GGUF file."""
        g = GgufFile(path)
        try:
            m = cls(device)
            c = g.model_config()
            m.cfg = dict(n_layer=c.n_layer, n_embd=c.n_embd, n_head=c.n_head, n_kv=c.n_kv_head, head_dim=c.head_dim,
                         n_ff=c.n_ff, n_vocab=c.n_vocab, rope_theta=c.rope_theta, eps=c.rms_eps,
                         arch=g.meta_str("general.architecture"))
            m._check(_lib.lib().tfr_load_gguf(m._h, g._h, tp_rank, tp_size))
            return m
        finally:
            g.close()

    # -- runtime ----------------------------------------------------------------------------
    def alloc_kv(self, max_seq: int) -> CudaKv:
        h = C.c_void_p()
        self._check(_lib.lib().tfr_alloc_kv(self._h, max_seq, C.byref(h)))
        return CudaKv(self, h.value)

    def zero_recurrent(self, kv: CudaKv) -> None:
        self._check(_lib.lib().tfr_zero_recurrent(self._h, kv._h))

    def set_cuda_graph(self, enabled: bool) -> None:
        self._check(_lib.lib().tfr_set_cuda_graph(self._h, int(enabled)))

    def graph_active(self) -> bool:
        return bool(_lib.lib().tfr_graph_active(self._h))

    PATH_AUTO, PATH_CHAINED, PATH_LOOP = 0, 1, 2

    def set_decode_path(self, path: int) -> None:
        """decode.rs:87-240 (backend choice): 0 = persistent loop when the model qualifies, 1 = chained kernels
        (one CUDA graph per token), 2 = persistent loop or an error."""
        self._check(_lib.lib().tfr_set_decode_path(self._h, int(path)))

    def decode_path(self) -> int:
        """The schedule the next forward call takes: 1 chained kernels, 2 persistent loop."""
        return int(_lib.lib().tfr_decode_path(self._h))

    def set_prefill_chunk(self, tokens: int) -> None:
        """forward.rs:54-65 (MAX_BATCH chunking): prompts and verification batches run in chunks of up to `tokens`
        tokens, each reading the weights once; 0 feeds every prompt token as a decode step."""
        self._check(_lib.lib().tfr_set_prefill_chunk(self._h, int(tokens)))

    def prefill_chunk(self) -> int:
        """Chunk size in effect; 0 when the model keeps the step-by-step route."""
        return int(_lib.lib().tfr_prefill_chunk(self._h))

    def set_loop_timeline(self, device_buffer, step: int, points: int) -> None:
        """Test aid: per-CTA nanosecond timestamps of decode step `step` of the persistent loop into a device
        buffer of points * sm_count uint64 (None switches it off).  Only the instrumented build has the probes:
        call _lib.use_aids_build() before anything loads the library."""
        self._check(_lib.lib().tfr_debug_set_loop_timeline(self._h, _ptr(device_buffer), int(step), int(points)))

    def forward_greedy(self, tokens, kv: CudaKv) -> int:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = C.c_uint32()
        self._check(_lib.lib().tfr_forward_greedy(self._h, kv._h, t.ctypes.data, t.size, C.byref(out)))
        return int(out.value)

    def forward_greedy_all(self, tokens, kv: CudaKv) -> np.ndarray:
        """Greedy prediction after every one of the given tokens (speculative-decoding verification)."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = np.zeros(max(t.size, 1), np.uint32)
        self._check(_lib.lib().tfr_forward_greedy_all(self._h, kv._h, t.ctypes.data, t.size, out.ctypes.data))
        return out[: t.size].copy()

    def decode_burst(self, first_token: int, max_n: int, kv: CudaKv, stop_ids=()) -> np.ndarray:
        stops = np.ascontiguousarray(stop_ids, dtype=np.uint32)
        out = np.zeros(max(max_n, 1), np.uint32)
        n = C.c_int()
        self._check(_lib.lib().tfr_decode_burst(self._h, kv._h, int(first_token), int(max_n),
                                                stops.ctypes.data if stops.size else 0, stops.size, out.ctypes.data,
                                                C.byref(n)))
        return out[: n.value].copy()

    def current_logits(self) -> np.ndarray:
        """Logits of the last decoded position.  A tensor-parallel rank gets its own vocabulary
        rows and zeros elsewhere (taraference_b200.tp.gather_logits merges the ranks).  With a
        vocabulary shortlist only the active entries come back (see active_vocab)."""
        n_active, _ = self.active_vocab()
        out = np.zeros(self.cfg["n_vocab"], np.float32)
        self._check(_lib.lib().tfr_current_logits(self._h, out.ctypes.data, out.size))
        return out[:n_active] if n_active < out.size else out

    def set_vocab_shortlist(self, limit: int, special_id: int = -1) -> None:
        """load.rs:285-352: head over ids [0, limit) plus one extra row (special_id outside the shortlist)."""
        self._check(_lib.lib().tfr_set_vocab_shortlist(self._h, int(limit), int(special_id)))

    def active_vocab(self) -> tuple[int, int]:
        """(number of logits the head produces, id behind the last one or -1)."""
        n, sid = C.c_int(0), C.c_int(-1)
        self._check(_lib.lib().tfr_active_vocab(self._h, C.byref(n), C.byref(sid)))
        return n.value, sid.value

    # -- tensor parallelism (one engine per GPU; see include/tarafer_b200.h) ---------------------------
    def tp_vocab_range(self) -> tuple[int, int]:
        a, b = C.c_int(), C.c_int()
        self._check(_lib.lib().tfr_tp_vocab_range(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def tp_ipc_handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        self._check(_lib.lib().tfr_tp_ipc_handle(self._h, buf))
        return buf.raw

    def tp_attach_ipc(self, handles: list[bytes]) -> None:
        blob = b"".join(handles)
        assert len(blob) == 64 * len(handles)
        self._check(_lib.lib().tfr_tp_attach_ipc(self._h, C.c_char_p(blob)))

    def tp_use_nccl(self, unique_id: bytes | None) -> None:
        """Comparison baseline: all-reduce through NCCL between kernels (collective call); None switches back."""
        self._check(_lib.lib().tfr_tp_use_nccl(self._h, C.c_char_p(unique_id) if unique_id else None))

    def tp_local_pointer(self) -> int:
        p = C.c_void_p()
        self._check(_lib.lib().tfr_tp_local_pointer(self._h, C.byref(p)))
        return p.value

    def tp_attach_pointers(self, bases: list[int]) -> None:
        arr = (C.c_void_p * len(bases))(*bases)
        self._check(_lib.lib().tfr_tp_attach_pointers(self._h, arr))

    def launch_count(self) -> int:
        return int(_lib.lib().tfr_launch_count(self._h))

    def last_device_ms(self) -> float:
        return float(_lib.lib().tfr_last_device_ms(self._h))

    def debug_read(self, what: str, n: int, dtype=np.float32, kv: CudaKv | None = None, layer: int = 0) -> np.ndarray:
        out = np.zeros(n, dtype)
        self._check(_lib.lib().tfr_debug_read(self._h, kv._h if kv else 0, what.encode(), layer, out.ctypes.data,
                                              out.nbytes))
        return out

    def destroy(self) -> None:
        if self._h:
            _lib.lib().tfr_destroy(self._h)
            self._h = 0


class GpuMat:
    """types.rs:26-39: one weight matrix in decode layout on the device."""

    def __init__(self, ggml_type: int, K: int, N: int, data, rope_pair_head_dim: int = 0):
        h = C.c_void_p()
        rc = _lib.lib().tfr_mat_create(ggml_type, K, N, _ptr(data), _nbytes(data), rope_pair_head_dim, C.byref(h))
        if rc:
            raise TfrError(rc, "tfr_mat_create failed")
        self._h, self.K, self.N, self.type = h.value, K, N, ggml_type

    def free(self) -> None:
        if self._h:
            _lib.lib().tfr_mat_free(self._h)
            self._h = 0


def _ok(rc: int, what: str) -> None:
    if rc:
        raise TfrError(rc, what)


# Operator-level calls on device pointers (torch tensors); thin wrappers used by tests and bench.
def op_quantize_q8(x, q8, d8, stream: int = 0) -> None:
    _ok(_lib.lib().tfr_op_quantize_q8(_ptr(x), x.numel(), _ptr(q8), _ptr(d8), stream), "quantize_q8")


def op_gemv(w: GpuMat, x, out, bias=None, use_res: int = 0, act_mode: int = 0, norm_w=None, eps: float = 0.0,
            stream: int = 0) -> None:
    _ok(_lib.lib().tfr_op_gemv(w._h, _ptr(x), _ptr(out), _ptr(bias), use_res, act_mode, _ptr(norm_w), eps, stream),
        "gemv")


def op_ffn_gate_up(gate: GpuMat, up: GpuMat, x, h, norm_w=None, eps: float = 0.0, stream: int = 0) -> None:
    _ok(_lib.lib().tfr_op_ffn_gate_up(gate._h, up._h, _ptr(x), _ptr(norm_w), eps, _ptr(h), stream), "ffn_gate_up")


def op_ffn_block(gate: GpuMat, up: GpuMat, down: GpuMat, x, h_scratch, y, use_res: int = 0, stream: int = 0) -> None:
    _ok(_lib.lib().tfr_op_ffn_block(gate._h, up._h, down._h, _ptr(x), _ptr(h_scratch), _ptr(y), use_res, stream),
        "ffn_block")


def ffn_block_host(gate: GpuMat, up: GpuMat, down: GpuMat, x: np.ndarray, y: np.ndarray) -> None:
    _ok(_lib.lib().tfr_ffn_block_host(gate._h, up._h, down._h, _ptr(x), _ptr(y)), "ffn_block_host")


def op_int_dots(w: GpuMat, q8, d8, a, b=None, stream: int = 0) -> None:
    _ok(_lib.aids().tfr_op_int_dots(w._h, _ptr(q8), _ptr(d8), _ptr(a), _ptr(b), stream), "int_dots")


def op_int_dots_x(w: GpuMat, x, a, b=None, q8_out=None, stream: int = 0) -> None:
    """Integer taps with the activation quantised by the product's own in-kernel quantiser; q8_out receives the int8
    values the block dots read, b (Q4_K) the group sums as the dots' activation record holds them."""
    _ok(_lib.aids().tfr_op_int_dots_x(w._h, _ptr(x), _ptr(a), _ptr(b), _ptr(q8_out), stream), "int_dots_x")


def debug_f32_to_f16(src, dst, n: int, stream: int = 0) -> None:
    """Test aid: the KV store's f32 -> f16 rounding over n device floats."""
    _ok(_lib.aids().tfr_debug_f32_to_f16(_ptr(src), _ptr(dst), int(n), stream), "debug_f32_to_f16")


def op_attention(q, kc, vc, out, n_head: int, n_kv: int, head_dim: int, pos: int, stream: int = 0) -> None:
    _ok(_lib.lib().tfr_op_attention(_ptr(q), _ptr(kc), _ptr(vc), _ptr(out), n_head, n_kv, head_dim, pos, stream),
        "attention")


def op_attention_noalloc(q, kc, vc, out, n_head: int, n_kv: int, head_dim: int, pos: int, stream: int = 0) -> None:
    """op_attention for callers that may not allocate: the split scratch is a fixed array inside the library
    (2 MiB, shared by all calls; larger shapes raise).  Call it once per device before any stream capture."""
    _ok(_lib.lib().tfr_op_attention_noalloc(_ptr(q), _ptr(kc), _ptr(vc), _ptr(out), n_head, n_kv, head_dim, pos,
                                            stream), "attention_noalloc: shape exceeds the built-in scratch or CUDA error")


def transcode_to_q8_0(src_type: int, raw: np.ndarray) -> np.ndarray:
    """The loader's one-off Q5_K (13) / Q5_1 (7) -> Q8_0 conversion (host code, load.rs:33-133)."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    blk, per = (176, 8) if src_type == 13 else (24, 1)
    out = np.zeros(raw.size // blk * per * 34, np.uint8)
    _ok(_lib.lib().tfr_transcode_to_q8_0(src_type, raw.ctypes.data, raw.size, out.ctypes.data), "transcode_to_q8_0")
    return out


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    _ok(_lib.lib().tfr_tp_nccl_unique_id(buf), "nccl_unique_id: libnccl.so.2 not available")
    return buf.raw


def op_attention_gated(q, kc, vc, gate, out, n_head: int, n_kv: int, head_dim: int, pos: int, stream: int = 0) -> None:
    _ok(_lib.lib().tfr_op_attention_gated(_ptr(q), _ptr(kc), _ptr(vc), _ptr(gate), _ptr(out), n_head, n_kv, head_dim,
                                          pos, stream), "attention_gated")


def op_gdn_step(proj, conv_w, conv_ring, state, ssm_a, ssm_dt, norm_w, out, n_k: int, n_v: int, state_size: int,
                kernel: int, slot: int, eps: float, stream: int = 0) -> None:
    """Gated-DeltaNet decode step (conv + SiLU + L2 + delta rule + gated RMSNorm) after the projections."""
    _ok(_lib.lib().tfr_op_gdn_step(_ptr(proj), _ptr(conv_w), _ptr(conv_ring), _ptr(state), _ptr(ssm_a), _ptr(ssm_dt),
                                   _ptr(norm_w), _ptr(out), n_k, n_v, state_size, kernel, slot, eps, stream), "gdn_step")


def op_qk_norm_rope_store(raw, q_norm, k_norm, q_out, gate_out, kc, vc, n_head: int, n_kv: int, head_dim: int,
                          n_rot: int, pos: int, theta: float, eps: float, stream: int = 0) -> None:
    _ok(_lib.lib().tfr_op_qk_norm_rope_store(_ptr(raw), _ptr(q_norm), _ptr(k_norm), _ptr(q_out), _ptr(gate_out),
                                             _ptr(kc), _ptr(vc), n_head, n_kv, head_dim, n_rot, pos, theta, eps,
                                             stream), "qk_norm_rope_store")


def op_qkv_rope_store(wq: GpuMat, wk: GpuMat, wv: GpuMat, bq, bk, bv, x, norm_w, eps: float, theta: float,
                      head_dim: int, pos: int, q_out, kc, vc, stream: int = 0) -> None:
    _ok(_lib.lib().tfr_op_qkv_rope_store(wq._h, wk._h, wv._h, _ptr(bq), _ptr(bk), _ptr(bv), _ptr(x), _ptr(norm_w),
                                         eps, theta, head_dim, pos, _ptr(q_out), _ptr(kc), _ptr(vc), stream),
        "qkv_rope_store")


def synth_quantize(ggml_type: int, w, out, stream: int = 0) -> None:
    """Quantise fp32 device rows w[N][K] into GGUF bytes on the device."""
    N, K = w.shape
    _ok(_lib.aids().tfr_synth_quantize(ggml_type, _ptr(w), K, N, _ptr(out), stream), "synth_quantize")
