"""Host-side checks that need no GPU: the shared library loads, exports every symbol the
header declares, rejects bad arguments before any launch, and the operators refuse CPU tensors."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from quant_flash_attn_b200 import build, _lib
    build.build()
    return _lib.load()


def test_library_exports_every_declared_symbol(lib):
    from quant_flash_attn_b200 import _lib
    header = open(os.path.join(ROOT, "include", "qfa.h")).read()
    declared = set(re.findall(r"QFA_API\s+[\w\s\*]+?\b(qfa_\w+)\s*\(", header))
    assert declared, "no declarations found in include/qfa.h"
    assert declared == set(_lib.SIGNATURES), (declared, set(_lib.SIGNATURES))
    raw = C.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), name
    assert lib.qfa_version() == 5


def test_struct_layout_matches_header():
    from quant_flash_attn_b200 import _lib
    assert C.sizeof(_lib.QfaQuantTensor) == 56
    assert _lib.QfaFwdArgs.B.offset == 16 and _lib.QfaFwdArgs.q.offset == 56
    assert _lib.QfaFwdArgs.qq.offset == 88 and _lib.QfaFwdArgs.v_hat.offset == 88 + 3 * 56
    assert C.sizeof(_lib.QfaFwdArgs) == 88 + 3 * 56 + 8 + 8 + 24 + 8 + 8 + 8 + 8 + 8
    assert _lib.QfaFwdArgs.Hkv.offset == C.sizeof(_lib.QfaFwdArgs) - 16
    assert _lib.QfaFwdArgs.k_ctr.offset == C.sizeof(_lib.QfaFwdArgs) - 8
    assert C.sizeof(_lib.QfaQuantJob) == 6 * 8 + 8 * 8 + 8 and _lib.QfaQuantJob.centered_or_null.offset == 112
    assert _lib.QfaBwdArgs.B.offset == 24 and _lib.QfaBwdArgs.qq.offset == 96


def test_strerror_and_validation_without_gpu(lib):
    from quant_flash_attn_b200 import _lib
    assert lib.qfa_strerror(0) == b"ok"
    for code in range(-9, 2):
        assert lib.qfa_strerror(code) != b"unknown qfa code"
    # every rejection below happens before any CUDA call
    assert lib.qfa_attn_fwd(None, None) == -1
    a = _lib.QfaFwdArgs(mode=7)
    assert lib.qfa_attn_fwd(C.byref(a), None) == -7
    a = _lib.QfaFwdArgs(mode=1, dtype=5)
    assert lib.qfa_attn_fwd(C.byref(a), None) == -2
    a = _lib.QfaFwdArgs(mode=1, dtype=1, B=1, H=1, Sq=0, Skv=4, D=64)
    assert lib.qfa_attn_fwd(C.byref(a), None) == -3
    a = _lib.QfaFwdArgs(mode=1, dtype=1, B=1, H=1, Sq=4, Skv=4, D=96)
    assert lib.qfa_attn_fwd(C.byref(a), None) == -4
    a = _lib.QfaFwdArgs(mode=1, dtype=1, B=1, H=1, Sq=4, Skv=4, D=64)
    assert lib.qfa_attn_fwd(C.byref(a), None) == -1          # null output
    assert lib.qfa_quant_per_token(None, None, None, None, None, 1, 1, 1, 64, 64, 64, 64, 1, 0, None) == -1
    assert lib.qfa_quant_per_token(None, None, None, None, None, 1, 1, 0, 64, 64, 64, 64, 1, 0, None) == 0  # empty
    assert lib.qfa_quant_per_token(None, None, None, None, None, 1, 1, 1, 0, 64, 64, 64, 1, 0, None) == -3
    b = _lib.QfaBwdArgs(mode=0, dtype=0, B=1, H=1, Sq=4, Skv=4, D=64)
    assert lib.qfa_attn_bwd(C.byref(b), None) == -1


def test_operators_refuse_cpu_tensors():
    import quant_flash_attn_b200 as qfa
    x = torch.zeros(1, 1, 4, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA"):
        qfa.asymmetric_quant_per_token(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        qfa.quant_attention(x, x, x, False, 0.125)
    with pytest.raises(RuntimeError, match="CUDA"):
        qfa.quant_flash_attn(x, x, (x.to(torch.int8), x[..., :1], x[..., :1].to(torch.int8)), 0.125)


def test_reference_module_names_resolve():
    import asymmetric_quant
    import quant_flash_attn
    import quant_flash_attn_b200 as qfa
    assert asymmetric_quant.asymmetric_quant_per_token is qfa.asymmetric_quant_per_token
    assert quant_flash_attn.quant_flash_attn is not None
    assert quant_flash_attn.QuantFlashAttention is qfa.QuantFlashAttention


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from quant_flash_attn_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_shard_bounds_cover_all_units():
    from quant_flash_attn_b200 import shard_bounds
    for n in (128, 32, 7, 1, 0):
        for w in (1, 2, 4, 8):
            spans = [shard_bounds(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)
