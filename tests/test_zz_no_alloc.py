"""The CSR builder for hosts that cannot allocate: ``e3b_csr_from_dst_static``.

Some users of this library never get to call ``cudaMalloc``: a plug-in that lives inside another
program's fixed memory arena, a control loop that cannot afford the device-wide stall of an
allocation, a thin language binding with no allocator.  For them the library carries its own work
area; this test calls that entry point straight through the C ABI (ctypes), twice in a row on
different graphs, and requires the same bits as the regular entry point that takes caller scratch.
Collected last on purpose: a failure here must not hide the results of the other tests.
"""
import ctypes

import pytest
import torch

from e3nn_b200 import _lib

pytestmark = pytest.mark.gpu


def _bind(lib):
    lib.e3b_csr_from_dst_static.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.e3b_csr_from_dst_static.restype = ctypes.c_int
    lib.e3b_csr_static_max_edges.restype = ctypes.c_int64
    lib.e3b_csr_static_max_nodes.restype = ctypes.c_int64
    return lib


def _with_scratch(lib, dst, n):
    """Existing entry point: the caller brings the scratch."""
    e, dev = dst.numel(), dst.device
    perm = torch.empty(e, dtype=torch.int64, device=dev)
    rowptr = torch.empty(n + 1, dtype=torch.int64, device=dev)
    nbytes = lib.e3b_csr_scratch_bytes(e, n)
    scratch = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.e3b_csr_from_dst(dst.data_ptr(), e, n, perm.data_ptr(), rowptr.data_ptr(), scratch.data_ptr(),
                              scratch.numel(), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.e3b_last_error()
    return perm, rowptr, status


def _no_alloc(lib, dst, n, perm, rowptr, status):
    """New entry point: only inputs and outputs are passed."""
    rc = lib.e3b_csr_from_dst_static(dst.data_ptr(), dst.numel(), n, perm.data_ptr(), rowptr.data_ptr(),
                                     status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.e3b_last_error()


def test_static_scratch_matches_regular_entry_point_twice():
    lib = _bind(_lib.core())
    dev = torch.device("cuda")
    torch.manual_seed(7)
    cases = [(200_000, 60_000), (9_001, 130)]  # a big graph first, then a small one over its leftovers
    # outputs are allocated up front: between the two calls under test nothing is allocated
    outs = [(torch.empty(e, dtype=torch.int64, device=dev), torch.empty(n + 1, dtype=torch.int64, device=dev),
             torch.ones(1, dtype=torch.int32, device=dev)) for e, n in cases]
    graphs = [torch.randint(0, n, (e,), device=dev) for e, n in cases]
    for (e, n), dst, (perm, rowptr, status) in zip(cases, graphs, outs):
        _no_alloc(lib, dst, n, perm, rowptr, status)
    torch.cuda.synchronize()
    for (e, n), dst, (perm, rowptr, status) in zip(cases, graphs, outs):
        ref_perm, ref_rowptr, ref_status = _with_scratch(lib, dst, n)
        assert torch.equal(perm, ref_perm)          # integer work: bit-exact
        assert torch.equal(rowptr, ref_rowptr)
        assert int(status.item()) == int(ref_status.item()) == 0
        assert torch.equal(rowptr.cpu()[1:], torch.cumsum(torch.bincount(dst.cpu(), minlength=n), 0))


def test_static_scratch_rejects_oversize_and_flags_bad_index():
    lib = _bind(_lib.core())
    dev = torch.device("cuda")
    max_e, max_n = lib.e3b_csr_static_max_edges(), lib.e3b_csr_static_max_nodes()
    assert (max_e, max_n) == (262144, 65536)
    dst = torch.zeros(8, dtype=torch.int64, device=dev)
    perm = torch.empty(8, dtype=torch.int64, device=dev)
    rowptr = torch.empty(16, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    s = torch.cuda.current_stream().cuda_stream
    rc = lib.e3b_csr_from_dst_static(dst.data_ptr(), max_e + 1, 4, perm.data_ptr(), rowptr.data_ptr(), status.data_ptr(), s)
    assert rc == -1 and b"at most" in lib.e3b_last_error()
    rc = lib.e3b_csr_from_dst_static(dst.data_ptr(), 8, max_n + 1, perm.data_ptr(), rowptr.data_ptr(), status.data_ptr(), s)
    assert rc == -1 and b"at most" in lib.e3b_last_error()
    bad = torch.tensor([0, 1, 9, 2, 1, 0, 3, 3], device=dev)
    rc = lib.e3b_csr_from_dst_static(bad.data_ptr(), 8, 4, perm.data_ptr(), rowptr.data_ptr(), status.data_ptr(), s)
    assert rc == 0 and int(status.item()) == 1      # out-of-range destination reported, not dereferenced
