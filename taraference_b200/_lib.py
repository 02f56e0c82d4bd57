"""ctypes view of libtarafer_b200.so.  There is no fallback: if the library is missing or
cannot be loaded, importing a symbol raises."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

from .build import AIDS_LIB, LIB, PKG

HEADER = PKG.parent / "include" / "tarafer_b200.h"


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "n_embd", "n_head", "n_kv_head", "head_dim", "n_ff", "n_vocab",
                                         "context_length")] + \
               [("rope_theta", C.c_float), ("rms_eps", C.c_float)] + \
               [(n, C.c_int32) for n in ("hybrid", "rope_dim", "ssm_conv_kernel", "ssm_state_size", "ssm_group_count",
                                         "ssm_time_step_rank", "ssm_inner_size", "full_attention_interval",
                                         "tp_rank", "tp_size")]


def _header_split() -> tuple[list[str], list[str]]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    aids_blocks = re.findall(r"#ifdef TFR_TEST_AIDS(.*?)#endif", text, flags=re.S)
    aids = sorted(set(re.findall(r"\b(tfr_[a-z0-9_]+)\s*\(", "\n".join(aids_blocks))))
    everything = sorted(set(re.findall(r"\b(tfr_[a-z0-9_]+)\s*\(", text)))
    return [n for n in everything if n not in aids], aids


def declared_symbols() -> list[str]:
    """Every function name the public header declares for the product library."""
    return _header_split()[0]


def declared_aid_symbols() -> list[str]:
    """The function names declared inside #ifdef TFR_TEST_AIDS: exported by the instrumented build only."""
    return _header_split()[1]


_lib = None
AID_NAMES = ("tfr_debug_set_timeline", "tfr_debug_set_loop_timeline", "tfr_debug_f32_to_f16", "tfr_op_int_dots",
             "tfr_op_int_dots_x", "tfr_synth_quantize")
_aids = None
_use_aids = False


def use_aids_build() -> None:
    """Makes lib() return the instrumented build for this process (the timeline tool: probes live inside the kernels, so
    the engine itself must come from that build).  Call before the first lib()."""
    global _use_aids
    if _lib is not None and not _use_aids:
        raise RuntimeError("use_aids_build() must be called before the library is first loaded")
    _use_aids = True


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    l = _load(AIDS_LIB if _use_aids else LIB, with_aids=_use_aids)
    _lib = l
    return l


def aids() -> C.CDLL:
    """The instrumented build, loaded beside the product library for the entry points only it has (integer taps,
    KV-store rounding operator, synthetic quantiser).  Handles of stand-alone matrices (tfr_mat) are plain data and may
    cross between the two; engines may not."""
    global _aids
    if _aids is None:
        _aids = lib() if _use_aids else _load(AIDS_LIB, with_aids=True)
    return _aids


def _load(path: Path, with_aids: bool) -> C.CDLL:
    if not path.exists():
        raise RuntimeError(f"{path} is not built; run `python -m taraference_b200.build` (needs nvcc). "
                           "There is no CPU fallback.")
    l = C.CDLL(str(path))
    vp, i32, i64, f32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
    sig = {
        "tfr_create": (i32, [i32, C.POINTER(vp)]),
        "tfr_destroy": (None, [vp]),
        "tfr_last_error": (C.c_char_p, [vp]),
        "tfr_device_info": (i32, [vp, C.c_char_p, sz, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]),
        "tfr_set_config": (i32, [vp, C.POINTER(ModelConfig)]),
        "tfr_upload_tensor": (i32, [vp, C.c_char_p, i32, i64, i64, vp, sz]),
        "tfr_finalize_load": (i32, [vp]),
        "tfr_gguf_open": (i32, [C.c_char_p, C.POINTER(vp), C.c_char_p, sz]),
        "tfr_gguf_close": (None, [vp]),
        "tfr_gguf_version": (i32, [vp]),
        "tfr_gguf_data_offset": (C.c_uint64, [vp]),
        "tfr_gguf_tensor_count": (i64, [vp]),
        "tfr_gguf_find_tensor": (i64, [vp, C.c_char_p]),
        "tfr_gguf_tensor_info": (i32, [vp, i64, C.POINTER(C.c_char_p), C.POINTER(i32), C.POINTER(i32), C.POINTER(i64 * 4),
                                       C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
        "tfr_gguf_tensor_data": (vp, [vp, i64]),
        "tfr_gguf_meta_u64": (i32, [vp, C.c_char_p, C.POINTER(C.c_uint64)]),
        "tfr_gguf_meta_f32": (i32, [vp, C.c_char_p, C.POINTER(f32)]),
        "tfr_gguf_meta_str": (i32, [vp, C.c_char_p, C.POINTER(C.c_char_p)]),
        "tfr_gguf_meta_array_len": (i64, [vp, C.c_char_p]),
        "tfr_gguf_meta_array_str": (i32, [vp, C.c_char_p, i64, C.POINTER(C.c_char_p), C.POINTER(C.c_uint64)]),
        "tfr_gguf_meta_array_f32": (i32, [vp, C.c_char_p, i64, C.POINTER(f32)]),
        "tfr_gguf_meta_array_i64": (i32, [vp, C.c_char_p, i64, C.POINTER(i64)]),
        "tfr_gguf_model_config": (i32, [vp, C.POINTER(ModelConfig), C.c_char_p, sz]),
        "tfr_load_gguf": (i32, [vp, vp, i32, i32]),
        "tfr_alloc_kv": (i32, [vp, i32, C.POINTER(vp)]),
        "tfr_free_kv": (None, [vp]),
        "tfr_kv_len": (i32, [vp]),
        "tfr_kv_max_seq": (i32, [vp]),
        "tfr_kv_set_len": (i32, [vp, i32]),
        "tfr_kv_clear": (i32, [vp]),
        "tfr_kv_bytes_per_token": (i64, [vp]),
        "tfr_zero_recurrent": (i32, [vp, vp]),
        "tfr_forward_greedy": (i32, [vp, vp, vp, i32, C.POINTER(C.c_uint32)]),
        "tfr_forward_greedy_all": (i32, [vp, vp, vp, i32, vp]),
        "tfr_decode_burst": (i32, [vp, vp, C.c_uint32, i32, vp, i32, vp, C.POINTER(i32)]),
        "tfr_current_logits": (i32, [vp, vp, i32]),
        "tfr_set_vocab_shortlist": (i32, [vp, i32, i32]),
        "tfr_active_vocab": (i32, [vp, vp, vp]),
        "tfr_tp_exchange_bytes": (i32, [vp, C.POINTER(sz)]),
        "tfr_tp_ipc_handle": (i32, [vp, vp]),
        "tfr_tp_attach_ipc": (i32, [vp, vp]),
        "tfr_tp_local_pointer": (i32, [vp, C.POINTER(vp)]),
        "tfr_tp_attach_pointers": (i32, [vp, vp]),
        "tfr_tp_vocab_range": (i32, [vp, C.POINTER(i32), C.POINTER(i32)]),
        "tfr_tp_nccl_unique_id": (i32, [vp]),
        "tfr_tp_use_nccl": (i32, [vp, vp]),
        "tfr_set_cuda_graph": (i32, [vp, i32]),
        "tfr_graph_active": (i32, [vp]),
        "tfr_set_decode_path": (i32, [vp, i32]),
        "tfr_decode_path": (i32, [vp]),
        "tfr_set_prefill_chunk": (i32, [vp, i32]),
        "tfr_prefill_chunk": (i32, [vp]),
        "tfr_debug_set_loop_timeline": (i32, [vp, vp, i32, i32]),
        "tfr_launch_count": (i64, [vp]),
        "tfr_last_device_ms": (f32, [vp]),
        "tfr_debug_read": (i32, [vp, vp, C.c_char_p, i32, vp, sz]),
        "tfr_debug_set_timeline": (i32, [vp]),
        "tfr_debug_f32_to_f16": (i32, [vp, vp, i64, vp]),
        "tfr_mat_create": (i32, [i32, i64, i64, vp, sz, i32, C.POINTER(vp)]),
        "tfr_mat_free": (None, [vp]),
        "tfr_mat_device_bytes": (i64, [vp]),
        "tfr_op_quantize_q8": (i32, [vp, i32, vp, vp, vp]),
        "tfr_op_gemv": (i32, [vp, vp, vp, vp, i32, i32, vp, f32, vp]),
        "tfr_op_ffn_gate_up": (i32, [vp, vp, vp, vp, f32, vp, vp]),
        "tfr_op_ffn_block": (i32, [vp, vp, vp, vp, vp, vp, i32, vp]),
        "tfr_ffn_block_host": (i32, [vp, vp, vp, vp, vp]),
        "tfr_op_int_dots": (i32, [vp, vp, vp, vp, vp, vp]),
        "tfr_op_int_dots_x": (i32, [vp, vp, vp, vp, vp, vp]),
        "tfr_op_attention": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
        "tfr_op_attention_noalloc": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, vp]),
        "tfr_op_qkv_rope_store": (i32, [vp] * 8 + [f32, f32, i32, i32, vp, vp, vp, vp]),
        "tfr_op_gdn_step": (i32, [vp] * 8 + [i32, i32, i32, i32, i32, f32, vp]),
        "tfr_op_qk_norm_rope_store": (i32, [vp] * 7 + [i32, i32, i32, i32, i32, f32, f32, vp]),
        "tfr_op_attention_gated": (i32, [vp] * 5 + [i32, i32, i32, i32, vp]),
        "tfr_transcode_to_q8_0": (i32, [i32, vp, sz, vp]),
        "tfr_synth_quantize": (i32, [i32, vp, i64, i64, vp, vp]),
    }
    for name, (res, args) in sig.items():
        if name in AID_NAMES and not with_aids:
            continue
        fn = getattr(l, name)
        fn.restype, fn.argtypes = res, args
    return l
