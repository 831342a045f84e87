"""The workspace-free label sort (svoo_b200_sort_labels_static) against the regular
svoo_b200_sort_labels, through the C ABI.  Collected last on purpose: a run that stops at
the first failure has then already run every other test."""
import ctypes

import pytest
import torch


def _lib():
    from svoo_b200 import _lib
    return _lib


def test_static_sort_rejects_sizes_beyond_its_array():
    """Host-side check only: nothing is launched, so this needs no GPU."""
    L = _lib().LIB
    buf = ctypes.create_string_buffer(256)
    p = ctypes.addressof(buf)
    # 40 heads x 75,600 tokens x 500 clusters: 40 * 37 * 500 = 740,000 entries -> accepted size,
    # but with 1024 clusters it is 1,515,520 > 1,048,576 -> rejected before any CUDA call
    assert L.svoo_b200_sort_labels_static(p, 40, 75600, 1024, p, p, None) == -7
    assert L.svoo_b200_sort_labels_static(None, 1, 10, 4, p, p, None) == -1
    assert L.svoo_b200_sort_labels_static(p, 1, 10, 2000, p, p, None) == -6
    assert b"built-in scratch" in L.svoo_b200_error_string(-7)


@pytest.mark.gpu
def test_static_sort_matches_workspace_sort_on_two_calls_in_a_row():
    """Callers that cannot allocate get the same permutation and offsets, bit for bit, as
    callers that pass a workspace -- also on a second call, which finds the shared array
    full of the first call's histograms."""
    lib = _lib()
    from svoo_b200 import ops
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator("cpu").manual_seed(2024)
    for BH, N, K in ((3, 5000, 33), (40, 20000, 500)):
        lab = torch.randint(0, K, (BH, N), generator=g, dtype=torch.int32)
        lab[lab == 1] = 0                                   # an empty cluster
        lab_d = lab.to(dev)
        want_idx, want_off = ops.sort_labels(lab_d, K)       # existing entry point, caller workspace
        for call in range(2):                                # back to back on the same stream
            idx = torch.full_like(lab_d, -1)
            off = torch.full((BH, K + 1), -1, dtype=torch.int32, device=dev)
            rc = lib.LIB.svoo_b200_sort_labels_static(lab_d.data_ptr(), BH, N, K, idx.data_ptr(), off.data_ptr(),
                                                      stream)
            lib.check(rc, "sort_labels_static")
            torch.cuda.synchronize()
            assert torch.equal(off, want_off), (BH, N, K, call)
            assert torch.equal(idx, want_idx), (BH, N, K, call)
