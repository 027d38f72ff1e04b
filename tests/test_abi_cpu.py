"""CPU checks of the C-ABI boundary: the library builds/loads and exports every symbol
include/faws.h declares; host-side validation mirrors the reference's asserts."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from flash_attn_with_score_b200 import build, _lib
    build.build()
    return _lib.load()


def test_header_symbols_exported(lib):
    from flash_attn_with_score_b200 import _lib
    hdr = open(os.path.join(ROOT, "include", "faws.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(faws_[a-z0-9_]+)\s*\(", hdr))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.faws_version() == 2


def test_struct_layout_matches_header(lib):
    from flash_attn_with_score_b200 import _lib
    # 6+2 int32, float, 2 int32 = 44 bytes -> padded to 48; 4 tensors of 32; pointer;
    # backend, dropout_p, dropout_scale, reserved; philox seed and offset
    assert C.sizeof(_lib.Tensor) == 32
    assert C.sizeof(_lib.Problem) == 48 + 4 * 32 + 8 + 16 + 16
    assert _lib.Problem.philox_seed.offset == 48 + 4 * 32 + 8 + 16


def test_validation_without_gpu(lib):
    from flash_attn_with_score_b200 import _lib
    p = _lib.Problem()
    assert lib.faws_attention(C.byref(p), None) == -1  # zero shapes
    p.B, p.Hq, p.Hk, p.M, p.N, p.D = 1, 3, 2, 8, 8, 64
    assert lib.faws_attention(C.byref(p), None) == -1  # Hq % Hk
    p.Hq = 4
    p.D = 48
    assert lib.faws_attention(C.byref(p), None) == -2  # head dim
    p.D = 64
    p.m_end = 9
    assert lib.faws_attention(C.byref(p), None) == -1  # window
    assert lib.faws_workspace_bytes(3, C.byref(p), 0) == 0
    p.m_end = 8
    p.dropout_p = 1.0
    assert lib.faws_attention(C.byref(p), None) == -1  # dropout_p outside [0, 1)
    p.dropout_p = 0.5
    p.philox_offset = 2 ** 31
    assert lib.faws_attention(C.byref(p), None) == -2  # 64-bit Philox variant
    p.dropout_p = 0.0
    # scratch that is missing, too small or not on a 256-byte boundary is refused before anything is launched
    p.Hq, p.Hk, p.m_begin, p.m_end, p.sm_scale = 4, 2, 0, 8, 0.125
    for t in (p.q, p.k, p.v, p.out):  # fake addresses, never dereferenced: the checks below come first
        t.ptr, t.stride_b, t.stride_h, t.stride_s = 1 << 21, 4 * 8 * 64, 8 * 64, 64
    need = lib.faws_workspace_bytes(5, C.byref(p), 0)
    assert need > 0 and need % 256 == 0
    fake_sum, fake_ws = C.c_void_p(4096), 1 << 20  # never dereferenced: the checks come first
    assert lib.faws_attention_with_softmax_col_sum(C.byref(p), fake_sum, 0, None, need, None) == -3
    assert lib.faws_attention_with_softmax_col_sum(C.byref(p), fake_sum, 0, C.c_void_p(fake_ws), need - 1, None) == -3
    assert lib.faws_attention_with_softmax_col_sum(C.byref(p), fake_sum, 0, C.c_void_p(fake_ws + 16), need, None) == -3
    assert lib.faws_attention_with_col_sum(C.byref(p), fake_sum, 0, C.c_void_p(fake_ws + 64), 1 << 30, None) == -3
    assert b"workspace" in lib.faws_strerror(-3)
    assert lib.faws_reduce_ranks(None, 2, 4, None, None) == -1


def test_python_asserts_mirror_reference():
    import flash_attn_with_score_b200 as F
    q = torch.zeros(1, 4, 8, 64, dtype=torch.float16)
    k = torch.zeros(1, 2, 8, 64, dtype=torch.float16)
    with pytest.raises(AssertionError):
        F.attention_with_scores(q, k, torch.zeros(1, 2, 8, 32, dtype=torch.float16))
    with pytest.raises(AssertionError):
        F.attention_with_row_sum(q[:, :3], k, k)
    with pytest.raises(AssertionError):
        F.attention_cross_token_qk_sum(q, k, k, 0)
    with pytest.raises(AssertionError):
        F.attention_cross_token_softmax_sum(q, k, k, 9)
    with pytest.raises(AssertionError):
        F.attention(torch.zeros(1, 4, 8, 48, dtype=torch.float16), k, k)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        F.attention(q, k, k)
    assert set(F.__all__) >= {
        "attention", "attention_with_scores", "attention_with_col_sum", "attention_with_col_sum_sequential",
        "attention_with_softmax_col_sum", "attention_cross_token_softmax_sum",
        "attention_cross_token_softmax_sum_buffered", "attention_with_row_sum", "attention_cross_token_qk_sum"}


def test_reference_import_name():
    """The reference's own import line (its README.md:27) resolves to this implementation."""
    import flash_attention_with_scores as R
    import flash_attn_with_score_b200 as F
    from flash_attention_with_scores import attention_with_scores  # noqa: F401
    names = ["attention", "attention_with_scores", "attention_with_col_sum", "attention_with_col_sum_sequential",
             "attention_with_softmax_col_sum", "attention_cross_token_softmax_sum",
             "attention_cross_token_softmax_sum_buffered", "attention_with_row_sum", "attention_cross_token_qk_sum"]
    assert list(R.__all__) == names  # order of the reference's __init__.py:29-39
    for n in names:
        assert getattr(R, n) is getattr(F, n)
