"""The allocation-free attention entry point against the regular one (needs a B200).

Collected last on purpose: if it fails in a stop-at-first-failure run, every other test has
already run.  It must pass alone in a fresh process and after the rest of the suite.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _case(rng, H, Hkv, hd, T):
    q = torch.from_numpy(rng.normal(0, 1, H * hd).astype(np.float32)).cuda()
    kc = torch.from_numpy(rng.normal(0, 1, (T, Hkv * hd)).astype(np.float16).view(np.int16)).cuda()
    vc = torch.from_numpy(rng.normal(0, 1, (T, Hkv * hd)).astype(np.float16).view(np.int16)).cuda()
    return q, kc, vc


def test_noalloc_attention_matches_regular_entry_point_twice(cuda_lib):
    """Callers that cannot allocate (capture in progress elsewhere, fixed memory budget) use the variant whose
    split scratch is a fixed array in the library.  Two calls in a row — the second sees the first one's
    leftovers in the shared array — must both equal the allocating entry point within fp32 rounding."""
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from taraference_b200 import engine as E
    rng = np.random.default_rng(7)
    for H, Hkv, hd, T in [(16, 2, 128, 700), (16, 2, 128, 33), (40, 8, 128, 300), (8, 2, 64, 130)]:
        q, kc, vc = _case(rng, H, Hkv, hd, T)
        want = torch.zeros(H * hd, device="cuda")
        E.op_attention(q, kc, vc, want, H, Hkv, hd, T - 1)
        for call in range(2):
            got = torch.full((H * hd,), float("nan"), device="cuda")
            E.op_attention_noalloc(q, kc, vc, got, H, Hkv, hd, T - 1)
            torch.cuda.synchronize()
            err = float((got - want).abs().max() / want.abs().max())
            assert err < 2e-5, (H, Hkv, hd, T, call, err)


def test_noalloc_attention_refuses_oversized_shapes(cuda_lib):
    """The built-in array is 2 MiB: 512 query heads of 256 need 512 x 8 splits x 258 floats = 4.2 MB of partials and
    are refused; so are more than 64 KV heads (the arrival counters take the first 2048 bytes)."""
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from taraference_b200 import engine as E
    rng = np.random.default_rng(8)
    for H, Hkv, hd in [(512, 64, 256), (65, 65, 64)]:
        q, kc, vc = _case(rng, H, Hkv, hd, 4)
        out = torch.zeros(H * hd, device="cuda")
        with pytest.raises(E.TfrError):
            E.op_attention_noalloc(q, kc, vc, out, H, Hkv, hd, 3)
    # a shape that fits still works after the refusals
    q, kc, vc = _case(rng, 8, 1, 256, 16)
    out = torch.full((8 * 256,), float("nan"), device="cuda")
    E.op_attention_noalloc(q, kc, vc, out, 8, 1, 256, 15)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(out).all())
