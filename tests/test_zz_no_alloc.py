"""The arg-sort entry point whose scratch is a fixed array in the library image, called through
the C ABI and compared with the workspace-taking entry point.  Collected last by file name; it
passes on its own and after the other GPU tests (which leave the caching allocator populated)."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def _sort_with_workspace(L, keys, max_key):
    from semblo_b200._lib import ptr, stream_ptr
    heads, n = keys.shape
    order = torch.empty_like(keys)
    ws = torch.empty(int(L.semblo_layout_workspace_bytes(n, heads)), dtype=torch.uint8, device=keys.device)
    assert L.semblo_argsort_keys(ptr(keys), n, heads, max_key, ptr(order), ptr(ws), ws.numel(), stream_ptr()) == 0
    return order


def test_static_scratch_argsort_matches_and_allocates_nothing(dev):
    from semblo_b200._lib import lib, ptr, stream_ptr
    L = lib()
    cap = int(L.semblo_argsort_keys_static_max_keys())
    assert cap == 65536
    g = torch.Generator().manual_seed(11)
    cases = [(4, 8192, 2048), (1, 65536, 65536), (64, 1000, 200), (3, 1, 7), (2, 5000, 256)]
    # the first call resolves the array's address; it comes before anything is measured
    warm = torch.zeros(1, 4, dtype=torch.int32, device=dev)
    warm_out = torch.empty_like(warm)
    assert L.semblo_argsort_keys_static(ptr(warm), 4, 1, 1, ptr(warm_out), stream_ptr()) == 0
    torch.cuda.synchronize()
    assert warm_out.cpu().tolist() == [[0, 1, 2, 3]]
    for heads, n, max_key in cases:
        keys = torch.randint(0, max_key, (heads, n), generator=g, dtype=torch.int32).to(dev)
        want = _sort_with_workspace(L, keys, max_key)
        got = [torch.full_like(keys, -1), torch.full_like(keys, -1)]
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        reserved_before = torch.cuda.memory_reserved()
        for out in got:                       # two calls in a row share the array
            assert L.semblo_argsort_keys_static(ptr(keys), n, heads, max_key, ptr(out), stream_ptr()) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_reserved() == reserved_before
        assert torch.cuda.mem_get_info()[0] == free_before
        ref = torch.sort(keys.cpu().long(), dim=1, stable=True).indices.int()
        for out in got:
            assert torch.equal(out, want)
            assert torch.equal(out.cpu(), ref)
    # a different size right after a large one: stale scratch contents do not matter
    small = torch.randint(0, 16, (2, 33), generator=g, dtype=torch.int32).to(dev)
    out = torch.empty_like(small)
    assert L.semblo_argsort_keys_static(ptr(small), 33, 2, 16, ptr(out), stream_ptr()) == 0
    assert torch.equal(out, _sort_with_workspace(L, small, 16))


def test_static_scratch_argsort_refuses_what_does_not_fit(dev):
    from semblo_b200._lib import lib, ptr, stream_ptr
    L = lib()
    keys = torch.zeros(2, 40000, dtype=torch.int32, device=dev)
    out = torch.empty_like(keys)
    rc = L.semblo_argsort_keys_static(ptr(keys), 40000, 2, 8, ptr(out), stream_ptr())
    assert rc != 0
    assert b"exceed the fixed scratch" in L.semblo_last_error()
    keys = torch.zeros(65, 8, dtype=torch.int32, device=dev)
    rc = L.semblo_argsort_keys_static(ptr(keys), 8, 65, 8, ptr(torch.empty_like(keys)), stream_ptr())
    assert rc != 0 and b"heads" in L.semblo_last_error()
    # empty input is a no-op
    assert L.semblo_argsort_keys_static(None, 0, 1, 8, None, stream_ptr()) == 0
