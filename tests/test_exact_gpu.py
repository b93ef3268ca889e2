"""The exact device scorer (tcgen05 / TMA contraction + inverted-index sparse part + running top-k) against the CPU
oracle's exact brute force on the same rounded inputs: documents as the index stores them (dense halves), queries as
the search sees them (weights folded in, dense rounded to half).  Both accumulate in fp32 but in different orders, so
ids may differ only where two fused scores are within rounding of each other."""
import numpy as np
import pytest
import torch

import apoe
import apoe_oracle as orc
import helpers
import synth

pytestmark = pytest.mark.gpu


def _cpu_truth(ds, eff, top_k):
    qd, qs, qb = orc.scale_queries(ds.QD, ds.QS, ds.QB, *eff)
    d_stored = orc.h2f(ds.Dh)                         # what the index holds
    q_seen = orc.h2f(orc.f2h(qd))                     # what the search kernel multiplies with
    ids, dis, _ = orc.bruteforce(d_stored, ds.S, ds.B, q_seen, qs, qb, 7, top_k)
    return ids, dis


def _device_queries(ds, dev):
    q = ds.queries
    return synth.Queries(q.dense.to(dev), q.sparse.to(dev), q.bm25.to(dev))


@pytest.mark.parametrize("n,nq", [(5003, 150), (40000, 300)])
def test_exact_topk_equals_cpu_bruteforce(n, nq):
    ds = helpers.make_dataset(n, nq, seed=61, with_graph=False)
    dev = torch.device("cuda:0")
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B)
    qdev = _device_queries(ds, dev)
    for w in ((1.0, 1.0, 1.0), (0.0, 0.0, 1.0), (1.0, 0.0, 0.0), (0.5, 2.0, 1.0)):
        eff = orc.effective_weights(ds.D, ds.S, ds.B, ds.QD, ds.QS, ds.QB, *w)
        want_ids, want_dis = _cpu_truth(ds, eff, 10)
        ids, dis, st = ix.exact_topk(qdev, eff, top_k=10)
        ids, dis = ids.cpu().numpy().view(np.uint32), dis.cpu().numpy()
        assert np.all(np.diff(dis, axis=1) >= 0)
        same = float(np.mean(ids == want_ids))
        assert same >= 0.999, (w, same)
        assert np.allclose(dis, want_dis, rtol=2e-5, atol=2e-3), (w, float(np.abs(dis - want_dis).max()))
        # where an id differs the two scores are a rounding apart
        for q, j in zip(*np.nonzero(ids != want_ids)):
            assert abs(dis[q, j] - want_dis[q, j]) <= 2e-3
        assert st.dense_flops == 2 * nq * n * 1024 and st.dense_ms > 0
    # the inverted index and the dense copy are cached on the index: the second call does not rebuild them
    _, _, st2 = ix.exact_topk(qdev, eff, top_k=10)
    assert st2.seconds_index < st.seconds_total and st2.seconds_index < 0.01
    ix.exact_release()
    ids3, _, _ = ix.exact_topk(qdev, eff, top_k=16)
    assert np.array_equal(ids3.cpu().numpy().view(np.uint32)[:, :10], ids)
    with pytest.raises(apoe.ApoeError):
        ix.exact_topk(qdev, eff, top_k=17)
    ix.close()


def test_search_recall_against_the_exact_scorer(small):
    """The graph search's recall measured against the device ground truth equals the one measured against the CPU's."""
    dev = torch.device("cuda:0")
    ix = apoe.Index.from_host(small.D, small.S, small.B)
    ix.set_graph(small.graph, small.ep)
    eff = ix.effective_weights(small.QD, small.QS, small.QB)
    gt, _, _ = ix.exact_topk(_device_queries(small, dev), eff, top_k=10)
    gt = gt.cpu().numpy().view(np.uint32)
    ids, _, _ = ix.search(small.QD, small.QS, small.QB, cands=128)
    cpu_gt, _ = _cpu_truth(small, eff, 10)
    assert abs(helpers.recall_at(ids, gt) - helpers.recall_at(ids, cpu_gt)) <= 0.002
    assert helpers.recall_at(ids, gt) >= 0.85
    ix.close()
