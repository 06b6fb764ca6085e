"""The allocation-free CSR entry point against the regular one.

`sc_csr_build_noalloc` exists for hosts that cannot give the library scratch
memory (they run inside someone else's memory plan, or at a point where
allocating would synchronise the device). It must produce exactly what
`sc_csr_build` produces, on consecutive calls that reuse its built-in scratch,
and refuse sizes beyond that scratch. This file sorts last on purpose: a run that
stops at the first failure has then already executed every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(lib, idx, M):
    N, k = idx.shape
    row_ptr = torch.empty(M + 1, dtype=torch.int32, device="cuda")
    entries = torch.empty(N * k, dtype=torch.int32, device="cuda")
    nbytes = lib.sc_csr_workspace_bytes(M)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    rc = lib.sc_csr_build(idx.data_ptr(), N, k, M, row_ptr.data_ptr(), entries.data_ptr(), ws.data_ptr(),
                          nbytes, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return row_ptr, entries


def _noalloc(lib, idx, M):
    N, k = idx.shape
    row_ptr = torch.empty(M + 1, dtype=torch.int32, device="cuda")
    entries = torch.empty(N * k, dtype=torch.int32, device="cuda")
    rc = lib.sc_csr_build_noalloc(idx.data_ptr(), N, k, M, row_ptr.data_ptr(), entries.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return row_ptr, entries


def test_noalloc_matches_regular_twice_in_a_row(cuda_lib):
    g = torch.Generator().manual_seed(123)
    # two different problems back to back: the second must not see the first one's counters
    for N, k, M in [(4096, 32, 16384), (1000, 8, 513)]:
        idx = torch.stack([torch.randperm(M, generator=g)[:k] for _ in range(N)]).cuda()
        want_ptr, want_entries = _regular(cuda_lib, idx, M)
        got_ptr, got_entries = _noalloc(cuda_lib, idx, M)
        torch.cuda.synchronize()
        assert torch.equal(got_ptr, want_ptr)          # integer work: exact
        assert torch.equal(got_entries, want_entries)


def test_noalloc_at_its_largest_size_and_with_no_tokens(cuda_lib):
    """M = 262144 uses the built-in scratch to its last slot (256 scan tiles); N = 0 takes the
    branch that only writes an all-zero row_ptr. A latent selected by every token exercises the
    sort of long segments, whose queue lives in the same scratch."""
    g = torch.Generator().manual_seed(124)
    M, N, k = 262144, 3000, 4
    idx = torch.randint(16, M, (N, k), generator=g)
    idx[:, 0] = M - 1
    idx[:, 1] = 7
    idx = idx.cuda()
    want_ptr, want_entries = _regular(cuda_lib, idx, M)
    got_ptr, got_entries = _noalloc(cuda_lib, idx, M)
    torch.cuda.synchronize()
    assert torch.equal(got_ptr, want_ptr) and torch.equal(got_entries, want_entries)
    assert int(got_ptr[-1]) == N * k
    seg = got_entries[int(got_ptr[7]):int(got_ptr[8])].cpu()
    assert torch.equal(seg, torch.arange(N, dtype=torch.int32) * k + 1)  # ascending flat positions
    empty = torch.zeros(0, 4, dtype=torch.int64, device="cuda")
    want_ptr, _ = _regular(cuda_lib, empty, 513)
    got_ptr, _ = _noalloc(cuda_lib, empty, 513)
    torch.cuda.synchronize()
    assert torch.equal(got_ptr, want_ptr) and int(got_ptr.abs().sum()) == 0


def test_noalloc_rejects_sizes_beyond_its_scratch(cuda_lib):
    from sparsify_b200 import _lib
    rc = cuda_lib.sc_csr_build_noalloc(None, 0, 4, 262144 + 1, 1, None, None)
    assert rc == 6 and "exceeds" in _lib.last_error()
