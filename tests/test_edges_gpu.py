"""Edge cases of the search and build paths (empty rows, a corpus barely larger than a k-NN list, batch 1, the
largest pool) and size-independent properties at the benchmark's full size."""
import numpy as np
import pytest
import torch

import apoe
import apoe_oracle as orc
import helpers
import synth

pytestmark = pytest.mark.gpu


def _drop_rows(c: orc.CsrNp, rows):
    """The same CSR with the given rows emptied."""
    keep = np.ones(c.idx.size, dtype=bool)
    for r in rows:
        keep[int(c.off[r]):int(c.off[r + 1])] = False
    cnt = np.diff(c.off.astype(np.int64)).copy()
    cnt[list(rows)] = 0
    off = np.zeros(c.off.size, dtype=np.uint32); off[1:] = np.cumsum(cnt)
    return orc.CsrNp(off, c.idx[keep], c.val[keep])


def test_empty_rows_on_both_sides(small):
    """Documents without sparse terms, without BM25 terms or with neither, and queries likewise: every pool entry equal
    to the oracle's."""
    S = _drop_rows(small.S, range(0, small.n, 7))
    B = _drop_rows(small.B, list(range(0, small.n, 14)) + list(range(3, small.n, 11)))
    QS = _drop_rows(small.QS, [0, 5, 6])
    QB = _drop_rows(small.QB, [0, 9])
    ix = apoe.Index.from_host(small.D, S, B)
    ix.set_graph(small.graph, small.ep)
    ws, wb, wd = orc.effective_weights(small.D, S, B, small.QD, QS, QB, 1.0, 1.0, 1.0)
    qd, qs, qb = orc.scale_queries(small.QD, QS, QB, ws, wb, wd)
    want_ids, want_dis, _ = orc.search(small.Dh, S, B, orc.f2h(qd), qs, qb, small.graph, small.ep, 64, 7)
    ids, dis, st = ix.search(small.QD, QS, QB, cands=64)
    assert np.array_equal(ids, want_ids) and np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))
    ix.close()


def test_corpus_barely_larger_than_a_list():
    """70 documents: lists of 64 hold almost the whole corpus; build, rows and search stay well-formed and the search
    over the built graph equals the oracle's search over the same graph."""
    ds = helpers.make_dataset(70, 9, seed=5, with_graph=False)
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B, for_build=True)
    st = ix.build(seed=2)
    rows, ep = ix.get_graph()
    assert rows[:, :32].max() < 70 and rows[:, 32].max() <= 7 and ep.max() < 70
    assert all(i not in rows[i, :16] for i in range(70))
    eff, qdh, qs, qb, _ = helpers.scaled_queries(ds)
    want_ids, want_dis, _ = orc.search(orc.f2h(ds.D), ds.S, ds.B, qdh, qs, qb, rows, ep, 32, 7)
    ids, dis, _ = ix.search(ds.QD, ds.QS, ds.QB, cands=32)
    assert np.array_equal(ids, want_ids) and np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))
    ix.close()


@pytest.mark.parametrize("n", [3, 40])
def test_corpus_smaller_than_a_list(n):
    """Fewer documents than a k-NN list has slots: ids repeat inside the lists; the build still ends with well-formed
    rows and the search over them equals the oracle's."""
    ds = helpers.make_dataset(n, 5, seed=9, with_graph=False)
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B, for_build=True)
    ix.build(seed=4)
    rows, ep = ix.get_graph()
    assert rows[:, :32].max() < n and rows[:, 32].max() <= 7 and ep.max() < n
    eff, qdh, qs, qb, _ = helpers.scaled_queries(ds)
    want_ids, want_dis, _ = orc.search(orc.f2h(ds.D), ds.S, ds.B, qdh, qs, qb, rows, ep, 32, 7)
    ids, dis, _ = ix.search(ds.QD, ds.QS, ds.QB, cands=32)
    assert np.array_equal(ids, want_ids) and np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))
    ix.close()


def test_batch_of_one_with_the_largest_pool(small):
    ix = apoe.Index.from_host(small.D, small.S, small.B)
    ix.set_graph(small.graph, small.ep)
    eff, qdh, qs, qb, _ = helpers.scaled_queries(small)
    one = lambda c: orc.CsrNp(c.off[:2], c.idx[:int(c.off[1])], c.val[:int(c.off[1])])
    want_ids, want_dis, _ = orc.search(small.Dh, small.S, small.B, qdh[:1], one(qs), one(qb), small.graph, small.ep, 512, 7)
    q = small.queries.slice(0, 1)
    ids, dis, _ = ix.search(q.dense.numpy(), q.sparse, q.bm25, cands=512, weights=eff, flags=apoe.SEARCH_RAW_WEIGHTS)
    assert np.array_equal(ids, want_ids) and np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))
    ix.close()


def test_full_size_properties():
    """1 M documents / 10 k queries (the benchmark's configuration), checked through properties that need no oracle run:
    well-formed rows and entry points, sorted duplicate-free pools, reported distances equal to a separate evaluation
    of the same (query, document) pairs, and a second search equal to the first."""
    dev = torch.device("cuda:0")
    n, nq, cands = 1_000_000, 10_000, 128
    c = synth.make_corpus(n, device=dev)
    q = synth.make_queries(nq, c.idf, device=dev)
    ix = apoe.Index.from_device(c.dense, c.sparse, c.bm25, for_build=True)
    st = ix.build(seed=1, flags=apoe.BUILD_KEEP_KNN)
    assert st.seconds_total > 0 and st.iterations_run >= 1
    rows, ep = ix.get_graph()
    assert rows.shape == (n, 40) and rows[:, :32].max() < n and rows[:, 32].max() <= 7
    kw = rows[:, 33:][np.arange(7)[None, :] < rows[:, 32:33]]
    assert kw.size == 0 or kw.max() < n
    assert not np.any(rows[:, :16] == np.arange(n, dtype=np.uint32)[:, None])          # no self loops in the forward half
    indeg = np.bincount(rows[:, :32].reshape(-1), minlength=n)
    assert np.mean(indeg == 0) < 0.01                                                  # reverse edges reach (nearly) everyone
    _, knn_dis, norms = ix.get_knn()
    assert np.all(np.diff(knn_dis[::1000], axis=1) >= 0)
    order = np.lexsort((np.arange(n), norms))                                          # smallest norms, ties by id
    assert np.array_equal(ep, order[:32].astype(np.uint32))
    qh = synth.Queries(q.dense[:100].cpu(), q.sparse.slice_rows(0, 100).to("cpu"), q.bm25.slice_rows(0, 100).to("cpu"))
    eff = ix.effective_weights(qh.dense.numpy(), qh.sparse, qh.bm25)
    out = [(torch.empty(nq, cands, dtype=torch.int32, device=dev), torch.empty(nq, cands, dtype=torch.float32, device=dev)) for _ in range(2)]
    mq = (int((q.sparse.off[1:] - q.sparse.off[:-1]).max()), int((q.bm25.off[1:] - q.bm25.off[:-1]).max()))
    for oi, od in out:
        ix.search_device(q, oi, od, cands=cands, weights=eff, max_nnz=mq)
    torch.cuda.synchronize()
    assert torch.equal(out[0][0], out[1][0]) and torch.equal(out[0][1], out[1][1])     # same answer twice
    ids = out[0][0].cpu().numpy().view(np.uint32); dis = out[0][1].cpu().numpy()
    assert ids.max() < n                                                               # pools are full at this size
    assert np.all(np.diff(dis, axis=1) >= 0)                                           # ascending
    srt = np.sort(ids, axis=1)
    assert not np.any(srt[:, 1:] == srt[:, :-1])                                       # no document twice in a pool
    # reported distances against a separate evaluation of sampled pairs
    rng = np.random.default_rng(0)
    pq = rng.integers(0, nq, 4000).astype(np.uint32); slot = rng.integers(0, cands, 4000)
    pd = ids[pq, slot]
    qhost = synth.Queries(q.dense.cpu(), q.sparse.to("cpu"), q.bm25.to("cpu"))
    got = ix.fused_distances(qhost.dense.numpy(), qhost.sparse, qhost.bm25, pq, pd, weights=eff)
    assert np.array_equal(got.view(np.uint32), dis[pq, slot].view(np.uint32))
    ix.close()


def test_fetch_only_probe_reports_a_bandwidth():
    """The profiling hook that only fetches random records (no scoring) runs to completion, moves the bytes it reports
    and leaves the index usable."""
    ds = helpers.make_dataset(3000, 16, seed=71)
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B)
    gbs, ms, moved = ix.debug_gather_probe(batches=50)
    assert gbs > 0 and ms > 0 and moved > 50 * 2048
    ix.set_graph(ds.graph, ds.ep)
    ids, _, _ = ix.search(ds.QD, ds.QS, ds.QB, cands=64)
    assert ids.shape == (16, 64)
    ix.check_status()
    ix.close()
