"""The scratch-free sort entry point gives the same bytes as the regular one.

fgs_sort_pairs_static is for callers that cannot hand over a scratch buffer and are not allowed to allocate
device memory themselves (a plug-in running inside another framework's memory plan, for instance): its
scratch is a fixed array inside the library. The file name makes pytest collect it last, so a run that stops at
the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(L, n, seed, W=1920, H=1080, warm=False):
    rng = np.random.default_rng(seed)
    tiles = ((W + 15) // 16) * ((H + 15) // 16)
    keys = (rng.integers(0, tiles, n, dtype=np.uint64) << np.uint64(32)) | rng.integers(0, 1 << 32, n, dtype=np.uint64)
    ki = torch.from_numpy(keys.view(np.int64)).to(DEV)
    vi = torch.from_numpy(rng.integers(0, 1 << 31, n).astype(np.int32)).to(DEV)
    ko_a, vo_a = torch.zeros_like(ki), torch.zeros_like(vi)
    ko_b, vo_b = torch.zeros_like(ki), torch.zeros_like(vi)
    tmp = torch.zeros(L.fgs_sort_temp_bytes(n), device=DEV, dtype=torch.int8)
    if warm:
        # the first call on a device looks the array's address up, and the first launch of each kernel loads its code:
        # neither is an allocation of this entry point, both may move the driver's figure for free memory
        assert L.fgs_sort_pairs_static(n, W, H, 16, 16, ki.data_ptr(), vi.data_ptr(), ko_a.data_ptr(), vo_a.data_ptr(), None) == 0
        ko_a.zero_(); vo_a.zero_()
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]       # the driver's own count: sees a cudaMalloc inside the library, too
    st = L.fgs_sort_pairs_static(n, W, H, 16, 16, ki.data_ptr(), vi.data_ptr(), ko_a.data_ptr(), vo_a.data_ptr(), None)
    assert st == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated or freed during the call"
    st = L.fgs_sort_pairs(n, W, H, 16, 16, tmp.data_ptr(), tmp.numel(), ki.data_ptr(), vi.data_ptr(),
                          ko_b.data_ptr(), vo_b.data_ptr(), None)
    assert st == 0
    torch.cuda.synchronize()
    # integer work: exact
    assert (ko_a == ko_b).all() and (vo_a == vo_b).all()
    assert (ko_a[1:] >= ko_a[:-1]).all()


def test_static_scratch_sort_matches_regular_sort_twice():
    from flashgs_b200 import _lib
    L = _lib.load()
    cap = L.fgs_sort_static_max_pairs()
    assert cap == 1 << 18
    # two calls in a row share the array: the second must not see the first one's leftovers
    _case(L, cap, seed=1, warm=True)
    _case(L, 100003, seed=2, W=800, H=800, warm=True)
    # beyond the limit: refused with a clear status, nothing launched
    k = torch.zeros(8, device=DEV, dtype=torch.int64)
    v = torch.zeros(8, device=DEV, dtype=torch.int32)
    assert L.fgs_sort_pairs_static(cap + 1, 800, 800, 16, 16, k.data_ptr(), v.data_ptr(), k.data_ptr(), v.data_ptr(), None) == _lib.ERR_TEMP_TOO_SMALL
    assert L.fgs_sort_pairs_static(-1, 800, 800, 16, 16, k.data_ptr(), v.data_ptr(), k.data_ptr(), v.data_ptr(), None) == _lib.ERR_BAD_ARG
    assert "scratch" in _lib.status_string(_lib.ERR_TEMP_TOO_SMALL)
    assert L.fgs_device_status(1, None) == 0
