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


def test_unsupported_architectures_are_refused(E, tmp_path):
    """config.rs:150 / layer.rs:417-418 (smollm3 skips RoPE on every fourth layer) and the mixture-of-experts
    families have schedules this library does not build: a header of theirs is refused, not decoded as dense."""
    def header(arch: bytes, extra=()):
        p = lambda s: arch + b"." + s
        kv = [(b"general.architecture", 8, struct.pack("<Q", len(arch)) + arch),
              (p(b"block_count"), 4, struct.pack("<I", 4)), (p(b"embedding_length"), 4, struct.pack("<I", 512)),
              (p(b"attention.head_count"), 4, struct.pack("<I", 8)), (p(b"feed_forward_length"), 4, struct.pack("<I", 1024)),
              (p(b"vocab_size"), 4, struct.pack("<I", 99))] + list(extra)
        path = tmp_path / "arch.gguf"
        path.write_bytes(_minimal(kv=kv))
        return E.GgufFile(path)

    g = header(b"smollm3")
    with pytest.raises(E.TfrError, match="smollm3 is not supported"):
        g.model_config()
    g.close()
    g = header(b"tara_moe_141")
    with pytest.raises(E.TfrError, match="mixture of experts"):
        g.model_config()
    g.close()
    g = header(b"qwen2", extra=[(b"qwen2.expert_count", 4, struct.pack("<I", 8))])
    with pytest.raises(E.TfrError, match="8 experts"):
        g.model_config()
    g.close()
    g = header(b"mistral")   # a generic dense family: accepted like the reference's OtherDense
    assert g.model_config().n_layer == 4
    g.close()


def test_tokenizer_arrays_round_trip(E, tmp_path):
    """engine.rs:130-133 needs the tokenizer arrays of the file: a byte-level vocabulary with merges, scores and
    token types written by gguf-py comes back item for item."""
    cfg = dict(S.TINY_DENSE)
    tens = S.make_model(cfg, seed=3)
    path = tmp_path / "tok.gguf"
    arch = cfg["arch"]
    w = gguf.GGUFWriter(str(path), arch)
    for k, v in (("embedding_length", cfg["n_embd"]), ("block_count", cfg["n_layer"]), ("attention.head_count", cfg["n_head"]),
                 ("feed_forward_length", cfg["n_ff"]), ("vocab_size", cfg["n_vocab"])):
        w.add_uint32(f"{arch}.{k}", v)
    tokens = [bytes([b]).decode("latin-1") for b in range(256)] + ["th", "the", "é", "中文", ""]
    merges = ["t h", "th e"]
    scores = [float(-i) * 0.5 for i in range(len(tokens))]
    types = [1] * 256 + [1, 1, 1, 1, 3]
    w.add_token_list(tokens)
    w.add_token_merges(merges)
    w.add_token_scores(scores)
    w.add_token_types(types)
    w.add_eos_token_id(260)
    w.add_tensor("token_embd.weight", np.zeros((4, 144), np.uint8), raw_dtype=gguf.GGMLQuantizationType.Q4_K)
    w.write_header_to_file(), w.write_kv_data_to_file(), w.write_tensors_to_file()
    w.close()
    g = E.GgufFile(path)
    got = g.meta_array("tokenizer.ggml.tokens")
    assert [t.decode("utf-8") for t in got] == tokens
    assert [m.decode() for m in g.meta_array("tokenizer.ggml.merges")] == merges
    assert g.meta_array("tokenizer.ggml.scores") == pytest.approx(scores)
    assert g.meta_array("tokenizer.ggml.token_type") == types
    assert g.meta_u64("tokenizer.ggml.eos_token_id") == 260
    assert g.meta_array("no.such.array") is None and g.meta_array_len("tokenizer.ggml.tokens") == len(tokens)
    g.close()


def test_reader_limits_and_fuzz(E, tmp_path):
    """Limits of the reference reader (value.rs:163-183: strings up to 64 MiB; value.rs:246-262: arrays up to 10 M
    items; reader.rs:147-158: every tensor inside the file) and a fuzz pass: truncations at every byte of the header,
    corrupted counts, lengths, types and offsets.  Every malformed file is refused with a reason; none crashes."""
    def expect(data: bytes, text: str):
        p = tmp_path / "lim.gguf"
        p.write_bytes(data)
        with pytest.raises(E.TfrError, match=text):
            E.GgufFile(p)

    big = struct.pack("<Q", 64 * 1024 * 1024 + 1)
    expect(_minimal(kv=[(b"k", 8, big)]), "string length 67108865 is unreasonably large")
    expect(b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + big, "string length 67108865 is unreasonably large")   # a key
    expect(_minimal(kv=[(b"k", 9, struct.pack("<IQ", 4, 10_000_001))]), "array length 10000001 is unreasonably large")
    expect(_minimal(kv=[(b"k", 9, struct.pack("<IQ", 4, 10_000_000))]), "unexpected end of file")             # at the limit: parsed
    expect(_minimal(kv=[(b"k", 9, struct.pack("<IQ", 13, 1))]), "malformed metadata value")                  # unknown item type
    expect(_minimal(kv=[(b"k", 8, struct.pack("<Q", 2) + b"\xff\xfe")]), "invalid UTF-8")
    expect(_minimal(kv=[(b"\xc3", 4, struct.pack("<I", 1))]), "invalid UTF-8")
    # tensor data range: offsets are relative to the aligned data section; one byte short is refused
    name = b"t"
    def one_tensor(n_elems, offset, pad):
        t = struct.pack("<Q", 1) + name + struct.pack("<IQ", 1, n_elems) + struct.pack("<IQ", 0, offset)
        body = _minimal(n_tensors=1, tensor=t)
        body += b"\0" * ((-len(body)) % 32) + b"\0" * pad
        return body
    p = tmp_path / "ok.gguf"
    p.write_bytes(one_tensor(8, 0, 32))
    E.GgufFile(p).close()
    expect(one_tensor(8, 0, 31), "exceeds file size")
    expect(one_tensor(8, 1, 32), "exceeds file size")
    expect(one_tensor(8, (1 << 64) - 16, 32), "exceeds file size")     # offset + size wraps around
    expect(one_tensor((1 << 62), 0, 32), "exceeds file size")
    # fuzz: a well-formed synthetic model file, cut at every header byte and with random byte flips
    cfg = S.TINY_DENSE
    good = tmp_path / "good.gguf"
    S.write_gguf(good, cfg, S.make_model(cfg, seed=2))
    data = good.read_bytes()
    g = E.GgufFile(good)
    header_end = g.data_offset
    g.close()
    fz = tmp_path / "fuzz.gguf"
    refused = 0
    for cut in list(range(0, 64)) + list(range(64, header_end, 7)):
        fz.write_bytes(data[:cut])
        with pytest.raises(E.TfrError):
            E.GgufFile(fz)
        refused += 1
    rng = np.random.default_rng(0)
    opened = 0
    for trial in range(300):
        b = bytearray(data[: header_end + 4096])
        for _ in range(int(rng.integers(1, 4))):
            pos = int(rng.integers(0, header_end))
            b[pos] = int(rng.integers(0, 256))
        fz.write_bytes(bytes(b))
        try:
            h = E.GgufFile(fz)
        except E.TfrError as exc:
            assert exc.msg, "a refusal carries its reason"
            refused += 1
            continue
        # still parses: every accessor must stay inside the mapping
        for t in h.tensors():
            assert h.data_offset + t["offset"] + t["nbytes"] <= len(b)
        try:
            h.model_config()
        except E.TfrError:
            pass
        h.close()
        opened += 1
    assert refused > 150 and opened + refused == 300 + 64 + len(range(64, header_end, 7))
