"""The allocation-free query entry point (dci_b200_query_noalloc).

It exists for callers that cannot let a query allocate device memory -- a
serving loop that must not hit the device-wide synchronisation of cudaMalloc,
or a process whose GPU memory is owned by another allocator -- and takes its
working memory from a fixed array inside the library instead.  The test calls
it through the C ABI twice in a row on the same handle and checks both answers
against the regular entry point bit for bit (ids are integers, distances use
the same fixed summation order on both paths), and checks that a problem that
cannot fit the fixed array is refused with a message instead of being attempted.
The file name makes pytest collect it last.
"""
import numpy as np
import pytest
import torch

from tests import cases

pytestmark = pytest.mark.gpu


def _make(c):
    from dciknn_cuda_b200 import DCI
    g = DCI(c["data"].shape[1], c["L"], c["S"], c["P"], c["T"], 0, proj=torch.from_numpy(c["proj"]))
    g.add(torch.from_numpy(c["data"]).cuda())
    return g


def test_noalloc_query_matches_regular_query_twice():
    c = cases.c2_shaped(n=40000, nq=300, P=4)
    g = _make(c)
    q = torch.from_numpy(c["query"]).cuda()
    want_ids, want_dists = g.query(q, c["k"], c["outer"], return_int_ids=True)
    torch.cuda.synchronize()
    ids = torch.empty_like(want_ids)
    dists = torch.empty_like(want_dists)
    g.query_noalloc(q, ids, dists, c["outer"])              # first call on the device: looks the array up
    torch.cuda.synchronize()
    assert torch.equal(ids, want_ids) and torch.equal(dists.view(torch.int32), want_dists.view(torch.int32))
    free_before = torch.cuda.mem_get_info()[0]
    ids.fill_(-7)
    dists.fill_(-1.0)
    g.query_noalloc(q, ids, dists, c["outer"])              # second call reuses the array as the first left it
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before       # nothing was allocated or freed
    assert torch.equal(ids, want_ids) and torch.equal(dists.view(torch.int32), want_dists.view(torch.int32))


def _alloc_calls():
    from dciknn_cuda_b200 import _capi
    return int(_capi.lib().dci_b200_device_alloc_calls())


def test_noalloc_query_allocates_nothing_even_on_its_first_call_with_tensor_core_projection():
    """With the tcgen05 projection selected the regular path keeps a flag word for the kernel's
    bounded waits in a buffer it creates on first use, and creates timing events when timing is on;
    the allocation-free call takes the word from the fixed array and records no timing.  The handle
    below has never projected anything when its first allocation-free call runs, and the library's
    count of cudaMalloc/cudaFree calls must not move across that call or the next."""
    from dciknn_cuda_b200 import DCI
    c = cases.c2_shaped(n=20000, nq=64, P=2)
    data = torch.from_numpy(c["data"]).cuda()
    q = torch.from_numpy(c["query"]).cuda()
    ref = DCI(128, c["L"], c["S"], c["P"], c["T"], 0, proj=torch.from_numpy(c["proj"]))
    ref.set_projection("tf32x3")
    ref.add(data)
    want_ids, want_dists = ref.query(q, c["k"], c["outer"], return_int_ids=True)
    # a second handle whose index is installed, not projected: its first projection is the call below
    g = DCI(128, c["L"], c["S"], c["P"], c["T"], 0, proj=torch.from_numpy(c["proj"]))
    g.set_projection("tf32x3")
    keys, ids_idx = ref.get_index()
    g.set_index(data, keys, ids_idx)
    g.enable_timing(True)                                   # the regular path would create events
    ids, dists = torch.empty_like(want_ids), torch.empty_like(want_dists)
    torch.cuda.synchronize()
    before = _alloc_calls()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(2):
        g.query_noalloc(q, ids, dists, c["outer"])
        torch.cuda.synchronize()
        assert _alloc_calls() == before
        assert torch.equal(ids, want_ids) and torch.equal(dists.view(torch.int32), want_dists.view(torch.int32))
    assert torch.cuda.mem_get_info()[0] == free_before


def test_noalloc_query_on_other_geometries_and_after_other_work():
    # ragged partitions (64-thread CTAs), 36 indices, k = 700, rows that are not 32-byte aligned (dim 37)
    for row in (cases.EDGE_CASES[2], cases.EDGE_CASES[6], cases.EDGE_CASES[7], cases.EDGE_CASES[14]):
        c = cases.edge_case(row)
        g = _make(c)
        q = torch.from_numpy(c["query"]).cuda()
        want_ids, want_dists = g.query(q, c["k"], c["outer"], max_num_candidates=c["max_cand"], return_int_ids=True)
        ids, dists = torch.empty_like(want_ids), torch.empty_like(want_dists)
        before = _alloc_calls()
        for _ in range(2):
            g.query_noalloc(q, ids, dists, c["outer"], max_num_candidates=c["max_cand"])
            torch.cuda.synchronize()
            assert _alloc_calls() == before, c["name"]
            assert torch.equal(ids, want_ids), c["name"]
            assert torch.equal(dists.view(torch.int32), want_dists.view(torch.int32)), c["name"]


def test_noalloc_query_refuses_what_does_not_fit():
    rng = np.random.default_rng(0)
    c = dict(data=cases.latent_linear(rng, 400000, 8, 16, 0.01), query=cases.latent_linear(rng, 32, 8, 16, 0.01),
             L=2, S=4, P=1, T=10, k=5, outer=5000, proj=cases.unit_rows(rng, 8, 16))
    g = _make(c)        # one partition of 400 000 points: the per-CTA slabs alone exceed the fixed array
    q = torch.from_numpy(c["query"]).cuda()
    ids = torch.empty((32, 5), dtype=torch.int32, device="cuda")
    dists = torch.empty((32, 5), dtype=torch.float32, device="cuda")
    with pytest.raises(NotImplementedError, match="built-in scratch"):
        g.query_noalloc(q, ids, dists)
