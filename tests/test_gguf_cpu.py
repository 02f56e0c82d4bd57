"""The C++ GGUF reader against gguf-py (writer and reader) on synthetic files — no GPU needed."""
import struct

import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

from taraference_b200 import synth as S  # noqa: E402


@pytest.fixture(scope="module")
def E(cuda_lib):
    from taraference_b200 import engine
    return engine


@pytest.mark.parametrize("cfg", [S.TINY_DENSE, S.TINY_HYBRID], ids=["dense", "hybrid"])
def test_reader_matches_gguf_py(E, tmp_path, cfg):
    tens = S.make_model(cfg, seed=1)
    path = tmp_path / "m.gguf"
    S.write_gguf(path, cfg, tens)
    ref = gguf.GGUFReader(str(path))
    g = E.GgufFile(path)
    assert g.version == 3
    assert g.data_offset == ref.data_offset
    mine = {t["name"]: t for t in g.tensors()}
    assert set(mine) == {t.name for t in ref.tensors} == set(tens)
    for t in ref.tensors:
        m = mine[t.name]
        assert m["ggml_type"] == int(t.tensor_type) and m["dims"] == [int(d) for d in t.shape], t.name
        assert m["nbytes"] == int(t.n_bytes) and g.data_offset + m["offset"] == int(t.data_offset)
        assert np.array_equal(g.tensor_bytes(t.name), np.asarray(t.data).view(np.uint8).reshape(-1))
    # the bytes are the model's bytes, the dims the loader's convention (dims[0] = K contiguous)
    wt, K, N, raw = tens["blk.0.ffn_gate.weight"]
    assert mine["blk.0.ffn_gate.weight"]["dims"] == [K, N] and np.array_equal(g.tensor_bytes("blk.0.ffn_gate.weight"), raw)
    arch = cfg["arch"]
    assert g.meta_str("general.architecture") == arch and g.meta_u64(f"{arch}.block_count") == cfg["n_layer"]
    assert g.meta_f32(f"{arch}.rope.freq_base") == pytest.approx(cfg["rope_theta"])
    assert g.meta_array_len("tokenizer.ggml.tokens") == 8 and g.meta_u64("tokenizer.ggml.tokens") is None
    assert g.meta_u64("no.such.key") is None and g.meta_str(f"{arch}.block_count") is None
    c = g.model_config()
    assert (c.n_layer, c.n_embd, c.n_head, c.n_kv_head, c.head_dim, c.n_ff, c.n_vocab) == tuple(
        cfg[k] for k in ("n_layer", "n_embd", "n_head", "n_kv", "head_dim", "n_ff", "n_vocab"))
    assert c.rope_theta == pytest.approx(cfg["rope_theta"]) and c.rms_eps == pytest.approx(cfg["eps"])
    assert c.hybrid == int(S.is_hybrid(cfg)) and c.context_length == 4096
    if S.is_hybrid(cfg):
        assert (c.rope_dim, c.ssm_conv_kernel, c.ssm_state_size, c.ssm_group_count, c.ssm_time_step_rank) == (
            cfg["rope_dim"], cfg["conv_kernel"], cfg["ssm_state"], cfg["ssm_n_k"], cfg["ssm_n_v"])
        assert mine["blk.0.ssm_conv1d.weight"]["dims"][0] == cfg["conv_kernel"]
    g.close()


def test_alignment_and_defaults(E, tmp_path):
    cfg = S.TINY_DENSE
    tens = S.make_model(cfg, seed=2)
    path = tmp_path / "a.gguf"
    S.write_gguf(path, cfg, tens, version_alignment=64)
    g = E.GgufFile(path)
    assert g.meta_u64("general.alignment") == 64 and g.data_offset % 64 == 0
    assert g.data_offset == gguf.GGUFReader(str(path)).data_offset
    g.close()


def _minimal(version=3, magic=b"GGUF", n_tensors=0, kv=(), tensor=b""):
    body = magic + struct.pack("<IQQ", version, n_tensors, len(kv))
    for key, ty, payload in kv:
        body += struct.pack("<Q", len(key)) + key + struct.pack("<I", ty) + payload
    return body + tensor


def test_malformed_files_are_refused_with_a_reason(E, tmp_path):
    def expect(data: bytes, text: str):
        p = tmp_path / "bad.gguf"
        p.write_bytes(data)
        with pytest.raises(E.TfrError, match=text):
            E.GgufFile(p)

    expect(_minimal(magic=b"GGML"), "bad magic")
    expect(_minimal(version=1), "unsupported GGUF version 1")
    expect(b"GGUF" + struct.pack("<I", 3), "unexpected end of file")
    expect(_minimal(n_tensors=2_000_000), "unreasonable counts")
    expect(_minimal(kv=[(b"k", 99, b"")]), "unknown metadata value type 99")
    name = b"t"
    t5 = struct.pack("<Q", 1) + name + struct.pack("<I", 5)
    expect(_minimal(n_tensors=1, tensor=t5), "n_dims=5 > 4")
    tbad = struct.pack("<Q", 1) + name + struct.pack("<IQ", 1, 32) + struct.pack("<IQ", 77, 0)
    expect(_minimal(n_tensors=1, tensor=tbad), "unknown tensor type 77")
    tbig = struct.pack("<Q", 1) + name + struct.pack("<IQ", 1, 1 << 20) + struct.pack("<IQ", 0, 0)
    expect(_minimal(n_tensors=1, tensor=tbig), "exceeds file size")
    with pytest.raises(E.TfrError, match="cannot open"):
        E.GgufFile(tmp_path / "missing.gguf")
    # a v2 file with lenient integer kinds parses: u64 where u32 is usual, f64 for a float
    kv = [(b"general.architecture", 8, struct.pack("<Q", 5) + b"qwen2"),
          (b"qwen2.block_count", 10, struct.pack("<Q", 7)), (b"qwen2.rope.freq_base", 12, struct.pack("<d", 5e5)),
          (b"qwen2.embedding_length", 5, struct.pack("<i", 512)), (b"qwen2.attention.head_count", 2, struct.pack("<H", 8)),
          (b"qwen2.feed_forward_length", 4, struct.pack("<I", 1024)), (b"qwen2.vocab_size", 4, struct.pack("<I", 99))]
    p = tmp_path / "v2.gguf"
    p.write_bytes(_minimal(version=2, kv=kv))
    g = E.GgufFile(p)
    c = g.model_config()
    assert g.version == 2 and (c.n_layer, c.n_embd, c.n_head, c.n_kv_head, c.head_dim) == (7, 512, 8, 8, 64)
    assert c.rope_theta == pytest.approx(5e5) and c.rms_eps == pytest.approx(1e-6) and c.context_length == 4096
    g.close()
    # missing keys are named
    p.write_bytes(_minimal(kv=kv[:1]))
    g = E.GgufFile(p)
    with pytest.raises(E.TfrError, match="missing qwen2.embedding_length"):
        g.model_config()
    g.close()
