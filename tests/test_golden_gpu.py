"""The CUDA path against the committed outputs of the reference's own kernels (tests/golden/*.npz, made by
tests/golden/make_golden.py on a B200): no oracle in between."""
import os

import numpy as np
import pytest

import apoe
import apoe_oracle as orc
import helpers
import synth
from test_oracle_golden import COMBOS, GOLD, digest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gsearch():
    g = np.load(os.path.join(GOLD, "ref_search.npz"))
    ds = helpers.make_dataset(2000, 100, seed=202, with_graph=False)
    assert digest(ds.D, ds.S.idx, ds.S.val, ds.B.idx, ds.B.val, ds.QD, ds.QS.idx, ds.QS.val, ds.QB.idx, ds.QB.val) == str(g["inputs"])
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B)
    ix.set_graph(g["graph"], g["ep"])
    yield g, ds, ix
    ix.close()


@pytest.mark.parametrize("name", list(COMBOS))
def test_search_equals_reference_kernels(gsearch, name):
    """Every pool entry (id and fused distance bits) of the reference's search kernels, all weight subsets."""
    g, ds, ix = gsearch
    w, mode, nq, cands = COMBOS[name]
    q = ds.queries.slice(0, nq)
    ids, dis, st = ix.search(q.dense.numpy(), q.sparse, q.bm25, cands=cands, weights=tuple(float(x) for x in g[name + "_eff"]),
                             flags=apoe.SEARCH_RAW_WEIGHTS)
    assert st.path == mode
    assert np.array_equal(ids, g[name + "_ids"])
    assert np.array_equal(dis.view(np.uint32), g[name + "_dis"].view(np.uint32))


def test_effective_weights_equal_oracle_values_of_the_fixture(gsearch):
    """The fixture's `*_eff` entries were written by the oracle (the reference computes them in host code that prints
    nothing); this compares the library's normalisation with those floats."""
    g, ds, ix = gsearch
    for name, (w, _, _, _) in COMBOS.items():
        eff = ix.effective_weights(ds.QD, ds.QS, ds.QB, *w)
        assert np.array_equal(np.asarray(eff, dtype=np.float32), g[name + "_eff"]), name


def test_keyword_search_top10_equals_reference(gsearch):
    g, ds, ix = gsearch
    kws = synth.make_keywords(ds.queries, seed=5)
    qb_idx = ds.QB.idx.copy()
    for q, req in enumerate(kws):       # required terms carry bit 31 (ref: src/query.cu:1828-1843)
        for j in range(int(ds.QB.off[q]), int(ds.QB.off[q + 1])):
            if int(qb_idx[j]) in req:
                qb_idx[j] |= np.uint32(0x80000000)
    ids, dis, _ = ix.search(ds.QD, ds.QS, orc.CsrNp(ds.QB.off, qb_idx, ds.QB.val), cands=128, flags=apoe.SEARCH_KEYWORD)
    assert np.array_equal(ids[:, :10], g["keyword_ids"][:, :10])
    assert np.array_equal(dis[:, :10].view(np.uint32), g["keyword_dis"][:, :10].view(np.uint32))


def test_norms_pruning_and_rows_equal_reference():
    g = np.load(os.path.join(GOLD, "ref_build.npz"))
    ds = helpers.make_dataset(1024, 8, seed=101, with_graph=False)
    assert digest(ds.D, ds.S.idx, ds.S.val, ds.B.idx, ds.B.val) == str(g["inputs"])
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B, for_build=True)
    assert np.array_equal(ix.norms().view(np.uint32), g["power"].view(np.uint32))
    new_list, kw, graph = ix.prune(g["knn"], g["knn_dis"], g["power"])
    _, ep = ix.get_graph()
    assert np.array_equal(ep, g["ep"])
    assert np.array_equal(new_list, g["new_list"])
    assert np.array_equal(kw[:, 0], g["kw"][:, 0])
    for i in range(kw.shape[0]):
        assert np.array_equal(kw[i, 1:1 + kw[i, 0]], g["kw"][i, 1:1 + kw[i, 0]])
    assert np.array_equal(graph[:, :16], g["graph"][:, :16]) and np.array_equal(graph[:, 32], g["graph"][:, 32])
    # the reverse half and the keyword slots are filled in racing-thread order by the reference: equal as sets on the
    # nodes whose reverse list its overflow rule did not touch
    calm = np.bincount(new_list.reshape(-1), minlength=new_list.shape[0]) <= 32
    for i in np.nonzero(calm)[0]:
        assert sorted(graph[i, 16:32].tolist()) == sorted(g["graph"][i, 16:32].tolist()), i
        c = int(graph[i, 32])
        assert sorted(graph[i, 33:33 + c].tolist()) == sorted(g["graph"][i, 33:33 + c].tolist()), i
    ix.close()
