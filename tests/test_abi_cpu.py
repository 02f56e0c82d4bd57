"""The C-ABI library: loads, exports every declared symbol, fails cleanly without a GPU."""
import ctypes as C

import numpy as np
import pytest

from taraference_b200 import _lib, synth as S


def test_library_exports_every_declared_symbol(cuda_lib):
    names = _lib.declared_symbols()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(cuda_lib, n)]
    assert not missing, missing


def test_test_aids_live_in_the_instrumented_build_only(cuda_lib):
    """Timeline probes, integer taps, the rounding operator and the synthetic quantiser are compiled under
    -DTFR_TEST_AIDS: the product library must not export them, the instrumented one must export everything."""
    aid_names = _lib.declared_aid_symbols()
    assert set(aid_names) == set(_lib.AID_NAMES)
    assert not [n for n in aid_names if hasattr(cuda_lib, n)]
    aids = _lib.aids()
    assert not [n for n in aid_names + _lib.declared_symbols() if not hasattr(aids, n)]


def test_create_without_gpu_fails_cleanly(cuda_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert cuda_lib.tfr_create(0, C.byref(h)) < 0
    assert not h.value
    from taraference_b200.engine import CudaModel, TfrError
    with pytest.raises(TfrError):
        CudaModel(0)


def test_null_arguments_rejected(cuda_lib):
    assert cuda_lib.tfr_create(0, None) == -1
    assert cuda_lib.tfr_kv_len(None) == -1
    assert cuda_lib.tfr_op_quantize_q8(None, 32, None, None, None) == -1
    assert cuda_lib.tfr_mat_create(12, 256, 1, None, 144, 0, None) == -1
    assert cuda_lib.tfr_last_error(None) == b"null engine"


def test_synth_quantizers_round_trip(oracle):
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, (16, 1024)).astype(np.float32)
    for t, tol in ((S.Q4_K, 0.09), (S.Q6_K, 0.025)):
        q = S.quantize(t, w)
        assert q.shape == (16, 4 * S.BLOCK_BYTES[t])
        back = oracle.dequant_rows(t, np.ascontiguousarray(q.reshape(-1)), 1024, 16)
        assert np.abs(back - w).max() <= tol * np.abs(w).max()
    z = S.quantize(S.Q4_K, np.zeros((1, 256), np.float32))
    assert (oracle.dequant_rows(S.Q4_K, z.reshape(-1).copy(), 256, 1) == 0).all()


def test_random_blocks_have_requested_distribution():
    rng = np.random.default_rng(0)
    b = S.random_q4_k(rng, 4000)
    d = b[:, 0:4].copy().view(np.float16).astype(np.float32)
    assert 0.002 < d.mean() < 0.003 and (d >= 0).all()
    b6 = S.random_q6_k(rng, 4000)
    sc = b6[:, 192:208].view(np.int8)
    assert sc.min() == -32 and sc.max() == 31


def test_host_transcode_matches_the_oracle_byte_for_byte(cuda_lib, oracle):
    """tfr_transcode_to_q8_0 is host code: the library's Q5_K / Q5_1 -> Q8_0 conversion against the CPU oracle's."""
    import numpy as np
    from taraference_b200 import engine as E, synth as S
    rng = np.random.default_rng(4)
    for src, blocks in ((S.Q5_K, S.random_q5_k(rng, 200)), (S.Q5_1, S.random_q5_1(rng, 333))):
        assert np.array_equal(E.transcode_to_q8_0(src, blocks), oracle.transcode_to_q8_0(src, blocks))
    # all-zero blocks: scale 0, quants 0
    z = np.zeros((3, 176), np.uint8)
    assert not E.transcode_to_q8_0(S.Q5_K, z).any()
