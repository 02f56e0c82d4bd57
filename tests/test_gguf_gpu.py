"""Loading a model from a GGUF file gives the engine the same bytes as handing it the tensors (needs a B200)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
gguf = pytest.importorskip("gguf")
pytestmark = pytest.mark.gpu

from taraference_b200 import synth as S  # noqa: E402


@pytest.mark.parametrize("cfg", [S.TINY_DENSE, S.TINY_HYBRID], ids=["dense", "hybrid"])
def test_load_gguf_equals_load_with(cuda_lib, tmp_path, cfg):
    from taraference_b200 import engine as E
    tens = S.make_model(cfg, seed=8)
    path = tmp_path / "model.gguf"
    S.write_gguf(path, cfg, tens)
    outs = []
    for load in (lambda: E.CudaModel.load_gguf(path), lambda: E.CudaModel.load_with(cfg, tens)):
        m = load()
        kv = m.alloc_kv(48)
        nxt = m.forward_greedy([4, 8, 15, 16, 23, 42], kv)
        outs.append((nxt, m.decode_burst(nxt, 16, kv), m.current_logits()))
        kv.free()
        m.destroy()
    assert outs[0][0] == outs[1][0] and np.array_equal(outs[0][1], outs[1][1]) and np.array_equal(outs[0][2], outs[1][2])


def test_load_gguf_errors_name_the_tensor(cuda_lib, tmp_path):
    from taraference_b200 import engine as E
    cfg = S.TINY_DENSE
    tens = S.make_model(cfg, seed=8)
    del tens["blk.1.ffn_down.weight"]
    path = tmp_path / "short.gguf"
    S.write_gguf(path, cfg, tens)
    with pytest.raises(E.TfrError, match="blk.1.ffn_down.weight"):
        E.CudaModel.load_gguf(path)


def test_load_gguf_applies_the_vocabulary_shortlist_rule(cuda_lib, tmp_path, monkeypatch):
    """load.rs:285-352: TARAFER_VOCAB_LIMIT shortens the head; the end-of-sequence id outside it keeps a row."""
    from taraference_b200 import engine as E
    cfg = dict(S.TINY_DENSE, n_vocab=2304, eos_token_id=2000)
    tens = S.make_model(cfg, seed=8)
    path = tmp_path / "model.gguf"
    S.write_gguf(path, cfg, tens)
    monkeypatch.delenv("TARAFER_VOCAB_LIMIT", raising=False)
    m = E.CudaModel.load_gguf(path)
    assert m.active_vocab() == (2304, -1)            # dense model, no variable: whole vocabulary
    kv = m.alloc_kv(16)
    m.forward_greedy([1, 2, 3], kv)
    full = m.current_logits()
    kv.free(); m.destroy()
    monkeypatch.setenv("TARAFER_VOCAB_LIMIT", "1024")
    m = E.CudaModel.load_gguf(path)
    assert m.active_vocab() == (1025, 2000)
    kv = m.alloc_kv(16)
    m.forward_greedy([1, 2, 3], kv)
    lg = m.current_logits()
    assert np.array_equal(lg[:1024], full[:1024]) and lg[1024] == full[2000]
    kv.free(); m.destroy()
    monkeypatch.setenv("TARAFER_VOCAB_LIMIT", "512")   # below 1024: ignored, as in the reference
    m = E.CudaModel.load_gguf(path)
    assert m.active_vocab() == (2304, -1)
    m.destroy()
