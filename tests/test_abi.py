"""The C-ABI library loads without a GPU, exports every symbol the header
declares, and the Python prototypes cover the same set. Argument checks that
fail before any CUDA call are exercised too (no kernel is launched here)."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "sparsecoder.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(sc_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from sparsify_b200 import _lib, build
    build.build()
    return _lib.lib()


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} declared in sparsecoder.h but not exported"


def test_python_prototypes_match_header(lib):
    from sparsify_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_diagnostics(lib):
    assert lib.sc_version() >= 100
    assert lib.sc_status_string(0) == b"ok"
    assert b"timed out" in lib.sc_status_string(5)


def test_argument_errors_before_any_cuda_call(lib):
    from sparsify_b200 import _lib
    # negative shape
    rc = lib.sc_csr_build(None, -1, 4, 16, None, None, None, 0, None)
    assert rc == 1 and "bad shape" in _lib.last_error()
    # N*k beyond int32
    rc = lib.sc_csr_build(1, 1 << 30, 4, 16, 1, 1, 1, 1 << 20, None)
    assert rc == 1 and "2^31" in _lib.last_error()
    # bad dtype code
    rc = lib.sc_embedding_bag_fwd(1, 1, 1, 7, None, 4, 8, 16, 2, 1, None)
    assert rc == 1
    # k above the tensor-core path's list capacity
    rc = lib.sc_encode_topk(1, 1, 1, 128, 64, 4096, 500, 1, 1, 1, 0, None, None)
    assert rc == 2
    assert lib.sc_encode_topk_workspace_bytes(16384, 4096, 131072, 32) > 0
    assert lib.sc_csr_workspace_bytes(131072) >= 2 * 131072 * 4
    with pytest.raises(_lib.SparseCoderLibError):
        _lib.call("sc_topk_rows", None, 4, 8, 16, None, None, None, None)  # k > M


def test_more_argument_errors_and_planning(lib):
    """Entry points added for groupmax, the optimisers and the SM reservation reject bad
    arguments on the host, and the encoder's workspace follows the SM reservation."""
    from sparsify_b200 import _lib
    assert lib.sc_set_reserved_sms(-1) == 1 and lib.sc_set_reserved_sms(65) == 1
    base = lib.sc_encode_topk_workspace_bytes(16384, 4096, 131072, 32)
    assert lib.sc_set_reserved_sms(4) == 0
    try:
        assert lib.sc_encode_topk_workspace_bytes(16384, 4096, 131072, 32) > 0
    finally:
        assert lib.sc_set_reserved_sms(0) == 0
    assert lib.sc_encode_topk_workspace_bytes(16384, 4096, 131072, 32) == base
    # groupmax: group size that is neither 32/64/128 nor a multiple of 256 -> unsupported (2)
    assert lib.sc_encode_groupmax(1, 1, 1, 128, 64, 4096 * 3, 32, 1, 1, None, None) == 2
    assert lib.sc_encode_groupmax(1, 1, 1, 128, 64, 1000, 3, 1, 1, None, None) == 1  # M % k != 0
    # symmetric GEMM needs A == B and a square result
    assert lib.sc_gemm_bf16_nt(16, 32, 128, 128, 64, 1.0, 0.0, None, 0, None, 0, 48, 1, 1, None, None, None) == 1
    assert "symmetric" in _lib.last_error()
    assert lib.sc_signum_schedulefree(16, 32, 48, 8, 1e-3, 1.5, 0.1, None, None) == 1  # momentum > 1
    assert lib.sc_muon_momentum(16, 32, 8, 1.0, 1, 48, 64, 80, 1 << 20, None) == 1     # beta == 1
    assert lib.sc_muon_workspace_bytes() > 0
    assert lib.sc_project_rows(None, None, -1, 4, None) == 1
