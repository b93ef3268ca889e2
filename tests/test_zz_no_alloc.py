"""The allocation-free search entry point (ap_search_host_static) against the regular one.

Collected last on purpose: a run that stops at the first failure has then already been through every other test.
The entry point exists for callers that cannot allocate device memory while serving -- a process whose GPU memory
belongs to another pool, or a latency-bound loop that cannot risk the device-wide synchronisation of cudaMalloc /
cudaFree -- so its batch staging lives in a fixed 8 MiB device array inside the library.  Results must be the same
bits as ap_search_host's, call after call (the array keeps the previous call's contents).
"""
import numpy as np
import pytest

import apoe
import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ds():
    return helpers.make_dataset(1500, 96, seed=31)


@pytest.fixture(scope="module")
def index(ds):
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B)
    ix.set_graph(ds.graph, ds.ep)
    yield ix
    ix.close()


def test_static_search_equals_regular_search_twice_in_a_row(ds, index):
    want_ids, want_dis, want_st = index.search(ds.QD, ds.QS, ds.QB, cands=128)
    for call in range(2):
        ids, dis, st = index.search_static(ds.QD, ds.QS, ds.QB, cands=128)
        assert np.array_equal(ids, want_ids), call
        assert np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32)), call       # bit-exact, as every search test
        assert st.expansions == want_st.expansions and st.evaluations == want_st.evaluations
    # a different batch in between must not leak into the next call through the shared array
    half = ds.queries.slice(10, 50)
    a_ids, a_dis, _ = index.search(half.dense.numpy(), half.sparse, half.bm25, cands=64, weights=(1.0, 0.0, 1.0))
    b_ids, b_dis, _ = index.search_static(half.dense.numpy(), half.sparse, half.bm25, cands=64, weights=(1.0, 0.0, 1.0))
    assert np.array_equal(a_ids, b_ids) and np.array_equal(a_dis.view(np.uint32), b_dis.view(np.uint32))
    ids, dis, _ = index.search_static(ds.QD, ds.QS, ds.QB, cands=128)
    assert np.array_equal(ids, want_ids) and np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))


def test_static_search_allocates_no_device_memory(ds, index):
    """The property the entry point exists for: once the first call on the device has looked up the array's address,
    a call leaves the device's free memory exactly as it found it (the regular call may grow its staging buffers)."""
    import torch
    index.search_static(ds.QD, ds.QS, ds.QB, cands=128)          # first call on this device: address lookup
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for cands in (128, 256, 64):                                 # sizes the regular path would have to grow buffers for
        index.search_static(ds.QD, ds.QS, ds.QB, cands=cands)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)


def test_static_search_rejects_batches_beyond_its_area(ds, index):
    reps = 30                                    # 96 x 30 queries x 4 KB of dense rows alone exceed 8 MiB
    QD = np.tile(ds.QD, (reps, 1))
    def tile(c):
        off = np.concatenate([[0], np.cumsum(np.tile(np.diff(c.off.astype(np.int64)), reps))]).astype(np.uint32)
        return helpers.orc.CsrNp(off, np.tile(c.idx, reps), np.tile(c.val, reps))
    with pytest.raises(apoe.ApoeError) as e:
        index.search_static(QD, tile(ds.QS), tile(ds.QB), cands=128)
    assert e.value.code == 4 and "static area" in str(e.value)
    ids, _, _ = index.search(QD, tile(ds.QS), tile(ds.QB), cands=32)   # the regular call takes the same batch
    assert ids.shape == (96 * reps, 32)
