"""Live parity against the reference's own CUDA kernels at the benchmark's smallest configuration.

10 000 documents / 1 000 queries (the 10k / 1k configuration of the benchmark): the graph is built by this library,
then the reference's search kernels (compiled unmodified into oracle/_ref/libapoe_ref.so) and this library's kernel
search that same graph with the same effective weights.  Every pool entry -- id and fused-distance bits -- has to be
equal for the seven weight subsets (src/query.cu:277-1268); for the keyword kernel (src/query.cu:1271-1483) the first
top_k entries (deeper slots of the reference come from memory it never initialises).  The reference's
knowledge-graph kernel is not run: it indexes shared memory with a variable that is never assigned
(src/query.cu:1559,1694).  Skipped where the reference library was not built.
"""
import os

import numpy as np
import pytest

import apoe
import apoe_oracle as orc
import apoe_ref
import helpers
import synth

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not apoe_ref.available(), reason="oracle/_ref/libapoe_ref.so is not built")]

N_DOCS, N_QUERIES, CANDS, TOP_K = 10_000, 1_000, 128, 10
MODES = {  # name -> (user weights (sparse, bm25, dense), reference kernel selector)
    "three_paths": ((1.0, 1.0, 1.0), 7), "dense": ((0.0, 0.0, 1.0), 1), "sparse": ((1.0, 0.0, 0.0), 2), "bm25": ((0.0, 1.0, 0.0), 4),
    "dense_sparse": ((1.0, 0.0, 1.0), 3), "dense_bm25": ((0.0, 1.0, 1.0), 5), "sparse_bm25": ((1.0, 1.0, 0.0), 6),
    "skewed": ((1.0, 2.0, 0.5), 7),
}
c3 = lambda c: (c.off, c.idx, c.val)


@pytest.fixture(scope="module")
def live():
    ds = helpers.make_dataset(N_DOCS, N_QUERIES, seed=20261125, with_graph=False)
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B, for_build=True)
    ix.build(seed=7)
    graph, ep = ix.get_graph()
    yield ds, ix, graph, ep
    ix.close()


@pytest.mark.parametrize("name", list(MODES))
def test_every_pool_entry_equals_the_reference_kernel(live, name):
    ds, ix, graph, ep = live
    w, mode = MODES[name]
    eff = ix.effective_weights(ds.QD, ds.QS, ds.QB, *w)
    assert eff == orc.effective_weights(ds.D, ds.S, ds.B, ds.QD, ds.QS, ds.QB, *w)
    qd, qs, qb = orc.scale_queries(ds.QD, ds.QS, ds.QB, *eff)          # src/query.cu:1871-1881, host code of the reference
    ref_ids, ref_dis, _, _ = apoe_ref.search(ds.D, c3(ds.S), c3(ds.B), qd, c3(qs), c3(qb), graph, ep, CANDS, mode)
    ids, dis, st = ix.search(ds.QD, ds.QS, ds.QB, cands=CANDS, weights=w)
    assert st.path == mode
    assert np.array_equal(ids, ref_ids), f"{name}: {np.mean(ids == ref_ids):.6f} of the ids equal"
    assert np.array_equal(dis.view(np.uint32), ref_dis.view(np.uint32)), f"{name}: {np.mean(dis.view(np.uint32) == ref_dis.view(np.uint32)):.6f} of the distances equal"


def test_keyword_top_k_equals_the_reference_kernel(live):
    ds, ix, graph, ep = live
    kws = synth.make_keywords(ds.queries, seed=5)
    qb_idx = ds.QB.idx.copy()
    for q, req in enumerate(kws):                                       # bit 31 on the required terms, src/query.cu:1828-1843
        row = qb_idx[ds.QB.off[q]:ds.QB.off[q + 1]]
        row[np.isin(row, np.asarray(req, dtype=np.uint32))] |= np.uint32(0x80000000)
    QBk = orc.CsrNp(ds.QB.off, qb_idx, ds.QB.val)
    eff = orc.effective_weights(ds.D, ds.S, ds.B, ds.QD, ds.QS, QBk, 1.0, 1.0, 1.0)
    qd, qs, qb = orc.scale_queries(ds.QD, ds.QS, QBk, *eff)
    ref_ids, ref_dis, _, _ = apoe_ref.search(ds.D, c3(ds.S), c3(ds.B), qd, c3(qs), c3(qb), graph, ep, CANDS, 7 | 8)
    ids, dis, _ = ix.search(ds.QD, ds.QS, QBk, cands=CANDS, flags=apoe.SEARCH_KEYWORD)
    assert np.array_equal(ids[:, :TOP_K], ref_ids[:, :TOP_K])
    assert np.array_equal(dis[:, :TOP_K].view(np.uint32), ref_dis[:, :TOP_K].view(np.uint32))


def test_reference_load_graph_reads_the_file_this_library_writes(live, tmp_path):
    """index.poe written by ap_index_save_graph, read back by the reference's load_graph (src/query.cu:35-62)."""
    ds, ix, graph, ep = live
    path = str(tmp_path / "index.poe")
    ix.save_graph(path)
    assert os.path.getsize(path) == 8 + 128 + N_DOCS * 164
    rows, eps = apoe_ref.load_graph(path)
    assert rows.size == N_DOCS * 40 and np.array_equal(rows.reshape(N_DOCS, 40), graph)
    assert np.array_equal(eps, ep)
