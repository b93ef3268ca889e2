"""Search parity on the GPU: the CUDA kernel against the CPU restatement of the reference, bit for bit."""
import numpy as np
import pytest

import apoe
import apoe_oracle as orc
import helpers
import synth

pytestmark = pytest.mark.gpu

PATHS = {  # name -> (weights (sparse, bm25, dense), oracle flags)
    "three": ((1.0, 1.0, 1.0), 7),
    "dense": ((0.0, 0.0, 1.0), 1),
    "sparse": ((1.0, 0.0, 0.0), 2),
    "bm25": ((0.0, 1.0, 0.0), 4),
    "dense_sparse": ((1.0, 0.0, 1.0), 3),
    "dense_bm25": ((0.0, 1.0, 1.0), 5),
    "sparse_bm25": ((1.0, 1.0, 0.0), 6),
    "skewed": ((1.0, 2.0, 0.5), 7),
}


@pytest.fixture(scope="module")
def index(small):
    ix = apoe.Index.from_host(small.D, small.S, small.B)
    ix.set_graph(small.graph, small.ep)
    yield ix
    ix.close()


def test_fused_distances_match_oracle_bitwise(small, index):
    rng = np.random.default_rng(3)
    pq = rng.integers(0, small.nq, 4000).astype(np.uint32)
    pd = rng.integers(0, small.n, 4000).astype(np.uint32)
    for name, (w, flags) in PATHS.items():
        eff, qdh, qs, qb, _ = helpers.scaled_queries(small, w, normalise=False)
        want = orc.fused_distances(small.Dh, small.S, small.B, qdh, qs, qb, pq, pd, flags)
        got = index.fused_distances(small.QD, small.QS, small.QB, pq, pd, weights=w)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name
    # the separately rounded multiply / add variant
    eff, qdh, qs, qb, _ = helpers.scaled_queries(small, (1.0, 1.0, 1.0), normalise=False)
    want = orc.fused_distances(small.Dh, small.S, small.B, qdh, qs, qb, pq, pd, 7 | orc.F_UNFUSED_DENSE)
    got = index.fused_distances(small.QD, small.QS, small.QB, pq, pd, flags=apoe.SEARCH_UNFUSED_DENSE)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name", list(PATHS))
def test_search_matches_oracle_bitwise(small, index, name):
    """Whole pool (cands ids and distances per query) equal to the oracle's, for every weight subset."""
    w, flags = PATHS[name]
    eff, qdh, qs, qb, _ = helpers.scaled_queries(small, w)
    want_ids, want_dis, cnt = orc.search(small.Dh, small.S, small.B, qdh, qs, qb, small.graph, small.ep, 128, flags)
    ids, dis, st = index.search(small.QD, small.QS, small.QB, cands=128, weights=w)
    assert np.allclose([st.eff_sparse, st.eff_bm25, st.eff_dense], eff, rtol=0, atol=0)
    assert st.path == flags
    assert np.array_equal(ids, want_ids)
    assert np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))
    assert st.expansions == int(cnt[:, 0].sum()) and st.evaluations == int(cnt[:, 1].sum())


@pytest.mark.parametrize("cands", [32, 64, 256, 512])
def test_pool_sizes(small, index, cands):
    eff, qdh, qs, qb, _ = helpers.scaled_queries(small, (1.0, 1.0, 1.0))
    sub = slice(0, 48)
    want_ids, want_dis, _ = orc.search(small.Dh, small.S, small.B, qdh[sub], orc.CsrNp(*_rows(qs, 48)), orc.CsrNp(*_rows(qb, 48)),
                                       small.graph, small.ep, cands, 7)
    q = small.queries.slice(0, 48)
    ids, dis, _ = index.search(q.dense.numpy(), q.sparse, q.bm25, cands=cands, weights=(eff[0], eff[1], eff[2]),
                               flags=apoe.SEARCH_RAW_WEIGHTS)
    assert np.array_equal(ids, want_ids)
    assert np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))


def _rows(c, k):
    e = int(c.off[k])
    return c.off[:k + 1], c.idx[:e], c.val[:e]


@pytest.mark.parametrize("arena_bytes", [8192, 12288, 17920, 65536, 200000])
def test_ring_shapes_give_same_result(small, index, arena_bytes):
    """The staging arena is a ring of slots: one record per slot and a single slot (8 KB), one record per slot and two
    slots (12 KB), two records per slot and two slots (17.5 KB), seven pair slots (64 KB), the cap of sixteen (200 KB).
    None of it may change a result."""
    ids0, dis0, _ = index.search(small.QD, small.QS, small.QB, cands=128)
    ids1, dis1, _ = index.search(small.QD, small.QS, small.QB, cands=128, arena_bytes=arena_bytes, ctas_per_sm=1)
    assert np.array_equal(ids0, ids1) and np.array_equal(dis0.view(np.uint32), dis1.view(np.uint32))


def test_both_kernel_shapes_give_the_same_pools(small, index):
    """A batch this small runs in the latency shape of the kernel (8 warps per query, pairs of records dealt through a
    shared counter); fixing the CTA count selects the throughput shape (3 warps, producer warp + round-robin
    consumers).  Plain, keyword and knowledge-graph search: same pools bit for bit (the latency-shape results are
    compared with the oracle by the tests above and below)."""
    kws = synth.make_keywords(small.queries, seed=5)
    qb_idx = small.QB.idx.copy()
    for q, req in enumerate(kws):
        row = qb_idx[small.QB.off[q]:small.QB.off[q + 1]]
        row[np.isin(row, np.asarray(list(req), dtype=np.uint32))] |= np.uint32(0x80000000)
    QBk = orc.CsrNp(small.QB.off, qb_idx, small.QB.val)
    kg = synth.make_kg(small.n, small.nq, entities=5000, seed=9)
    index.set_kg(kg.e2e_off, kg.e2e_idx, kg.e2d_off, kg.e2d_idx)
    ent = (kg.qe_off.numpy().view(np.uint32), kg.qe_idx.numpy().view(np.uint32))
    cases = {"plain": dict(qb=small.QB), "keyword": dict(qb=QBk, flags=apoe.SEARCH_KEYWORD), "kg": dict(qb=small.QB, kg_weight=40.0, ent=ent)}
    for name, kw in cases.items():
        qb = kw.pop("qb")
        for cands in (32, 128, 512):
            a_ids, a_dis, _ = index.search(small.QD, small.QS, qb, cands=cands, **kw)
            b_ids, b_dis, _ = index.search(small.QD, small.QS, qb, cands=cands, ctas_per_sm=6, **kw)
            assert np.array_equal(a_ids, b_ids), (name, cands)
            assert np.array_equal(a_dis.view(np.uint32), b_dis.view(np.uint32)), (name, cands)


def test_long_query_rows(small, index):
    """Query rows longer than 32 terms take the per-term lookup instead of the collision-free table; rows of mixed
    length in one batch take either, and both agree with the oracle bit for bit."""
    ql = synth.make_queries(48, small.corpus.idf, seed=77, nnz_sparse=70, nnz_bm25=40)
    QD = np.concatenate([ql.dense.numpy(), small.QD[:16]])
    cat = lambda a, b: orc.CsrNp(np.concatenate([a.off, b.off[1:17] + a.off[-1]]), np.concatenate([a.idx, b.idx[:int(b.off[16])]]),
                                 np.concatenate([a.val, b.val[:int(b.off[16])]]))
    QS, QB = cat(orc.CsrNp.from_torch(ql.sparse), small.QS), cat(orc.CsrNp.from_torch(ql.bm25), small.QB)
    for w, flags in (((1.0, 1.0, 1.0), 7), ((1.0, 0.0, 0.0), 2)):
        eff = orc.effective_weights(small.D, small.S, small.B, QD, QS, QB, *w)
        qd, qs, qb = orc.scale_queries(QD, QS, QB, *eff)
        want_ids, want_dis, _ = orc.search(small.Dh, small.S, small.B, orc.f2h(qd), qs, qb, small.graph, small.ep, 64, flags)
        ids, dis, _ = index.search(QD, QS, QB, cands=64, weights=w)
        assert np.array_equal(ids, want_ids)
        assert np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))


def test_recall_against_exact_bruteforce(small, index):
    eff, qdh, qs, qb, qd = helpers.scaled_queries(small, (1.0, 1.0, 1.0))
    gt, _, _ = orc.bruteforce(small.D, small.S, small.B, qd, qs, qb, 7, 10)
    ids, _, _ = index.search(small.QD, small.QS, small.QB, cands=128)
    assert helpers.recall_at(ids, gt) >= 0.85


def test_keyword_search_matches_oracle(small, index):
    kws = synth.make_keywords(small.queries, seed=5)
    qb_idx = small.QB.idx.copy()
    for q, req in enumerate(kws):
        for j in range(int(small.QB.off[q]), int(small.QB.off[q + 1])):
            if int(qb_idx[j]) in req:
                qb_idx[j] |= np.uint32(0x80000000)
    QBk = orc.CsrNp(small.QB.off, qb_idx, small.QB.val)
    ws, wb, wd = orc.effective_weights(small.D, small.S, small.B, small.QD, small.QS, QBk, 1.0, 1.0, 1.0)
    qd, qs, qb = orc.scale_queries(small.QD, small.QS, QBk, ws, wb, wd)
    want_ids, want_dis, _ = orc.search(small.Dh, small.S, small.B, orc.f2h(qd), qs, qb, small.graph, small.ep, 128,
                                       7 | orc.F_KEYWORD)
    ids, dis, st = index.search(small.QD, small.QS, QBk, cands=128, flags=apoe.SEARCH_KEYWORD)
    assert np.array_equal(ids, want_ids)
    assert np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))
    # keyword hits come first: every result before the first non-hit contains a required term
    hit = 0
    for q in range(small.nq):
        d = int(ids[q, 0])
        if d < small.n:
            terms = set(small.B.idx[small.B.off[d]:small.B.off[d + 1]].tolist())
            hit += bool(terms & set(kws[q]))
    assert hit >= small.nq // 2


def test_kg_search_matches_oracle(small, index):
    kg = synth.make_kg(small.n, small.nq, entities=5000, seed=9)
    index.set_kg(kg.e2e_off, kg.e2e_idx, kg.e2d_off, kg.e2d_idx)
    eff, qdh, qs, qb, _ = helpers.scaled_queries(small, (1.0, 1.0, 1.0))
    arrs = [t.numpy().view(np.uint32) for t in (kg.e2e_off, kg.e2e_idx, kg.e2d_off, kg.e2d_idx, kg.qe_off, kg.qe_idx)]
    want_ids, want_dis, _ = orc.search(small.Dh, small.S, small.B, qdh, qs, qb, small.graph, small.ep, 128, 7 | orc.F_KG,
                                       kg=arrs, kg_weight=40.0)
    ids, dis, st = index.search(small.QD, small.QS, small.QB, cands=128, kg_weight=40.0, ent=(arrs[4], arrs[5]))
    assert np.array_equal(ids, want_ids)
    assert np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))


def test_device_pointer_path_equals_host_path(small, index):
    import torch
    dev = torch.device("cuda:0")
    q = small.queries
    qd = synth.Queries(q.dense.to(dev), q.sparse.to(dev), q.bm25.to(dev))
    eff = index.effective_weights(small.QD, small.QS, small.QB)
    out_ids = torch.empty(small.nq, 128, dtype=torch.int32, device=dev)
    out_dis = torch.empty(small.nq, 128, dtype=torch.float32, device=dev)
    index.search_device(qd, out_ids, out_dis, cands=128, weights=eff, max_nnz=(30, 8))
    torch.cuda.synchronize()
    ids, dis, _ = index.search(small.QD, small.QS, small.QB, cands=128)
    assert np.array_equal(out_ids.cpu().numpy().view(np.uint32), ids)
    assert np.array_equal(out_dis.cpu().numpy().view(np.uint32), dis.view(np.uint32))


def test_argument_errors(small, index):
    with pytest.raises(apoe.ApoeError) as e:
        index.search(small.QD, small.QS, small.QB, cands=100)
    assert e.value.code == 1
    with pytest.raises(apoe.ApoeError):
        index.search(small.QD, small.QS, small.QB, cands=128, weights=(0.0, 0.0, 0.0))
    bad = small.graph.copy()
    bad[5, 3] = small.n + 10
    with pytest.raises(apoe.ApoeError):
        index.set_graph(bad, small.ep)
    index.set_graph(small.graph, small.ep)
    ix2 = apoe.Index.from_host(small.D[:100], helpers.orc.CsrNp(*_rows(small.S, 100)), helpers.orc.CsrNp(*_rows(small.B, 100)))
    with pytest.raises(apoe.ApoeError) as e:
        ix2.search(small.QD, small.QS, small.QB)
    assert e.value.code == 5
    ix2.close()


def test_file_level_drop_in(small, tmp_path):
    """hybrid_search-style call over the reference's file formats gives the same results as the resident index."""
    p = lambda s: str(tmp_path / s)
    synth.write_fvecs(p("d.fvecs"), small.corpus.dense)
    synth.write_fvecs(p("q.fvecs"), small.queries.dense)
    synth.write_csr(p("s.bin"), small.corpus.sparse)
    synth.write_csr(p("b.bin"), small.corpus.bm25)
    synth.write_csr(p("qs.bin"), small.queries.sparse)
    synth.write_csr(p("qb.bin"), small.queries.bm25)
    synth.write_poe(p("index.poe"), small.graph, small.ep)
    eff, qdh, qs, qb, qd = helpers.scaled_queries(small)
    gt, _, _ = orc.bruteforce(small.D, small.S, small.B, qd, qs, qb, 7, 10)
    synth.write_qrels(p("qrels.txt"), gt)
    ids, dis, ndcg, st = apoe.search_index(p("d.fvecs"), p("q.fvecs"), p("s.bin"), p("qs.bin"), p("b.bin"), p("qb.bin"), "",
                                           "", "", "", p("index.poe"), p("qrels.txt"), 10, 128, 1.0, 1.0, 1.0, 0.0)
    want_ids, want_dis, _ = orc.search(small.Dh, small.S, small.B, qdh, qs, qb, small.graph, small.ep, 128, 7)
    assert np.array_equal(ids, want_ids)
    assert 0.5 < ndcg <= 1.0
    import build as apoe_build, importlib, sys, os
    sys.path.insert(0, os.path.dirname(apoe_build.module_path()))
    hs = importlib.import_module("hybrid_search")
    hs.search_index(dense_data_path=p("d.fvecs"), dense_query_path=p("q.fvecs"), sparse_data_path=p("s.bin"),
                    sparse_query_path=p("qs.bin"), bm25_data_path=p("b.bin"), bm25_query_path=p("qb.bin"),
                    keyword_id_path="", knowledge_path="", entity2doc_path="", query_entity_path="",
                    graph_path=p("index.poe"), ground_truth_path=p("qrels.txt"), top_k=10, cands=128,
                    sparse_weight=1.0, bm25_weight=1.0, dense_weight=1.0, kg_weight=0.0)


def _write_search_files(small, p):
    synth.write_fvecs(p("d.fvecs"), small.corpus.dense)
    synth.write_fvecs(p("q.fvecs"), small.queries.dense)
    synth.write_csr(p("s.bin"), small.corpus.sparse)
    synth.write_csr(p("b.bin"), small.corpus.bm25)
    synth.write_csr(p("qs.bin"), small.queries.sparse)
    synth.write_csr(p("qb.bin"), small.queries.bm25)
    synth.write_poe(p("index.poe"), small.graph, small.ep)


def test_file_level_keyword_search_equals_in_memory_call(small, index, tmp_path):
    """keyword_id_path: the text file of required term ids is parsed (ref: load_txt, src/query.cu:65-86), bit 31 goes on
    the matching query terms (src/query.cu:1828-1843) and the keyword kernel runs -- same bits as flagging by hand."""
    p = lambda s: str(tmp_path / s)
    _write_search_files(small, p)
    kws = synth.make_keywords(small.queries, seed=5)
    synth.write_keywords(p("kw.txt"), kws)
    ids, dis, _, st = apoe.search_index(p("d.fvecs"), p("q.fvecs"), p("s.bin"), p("qs.bin"), p("b.bin"), p("qb.bin"), p("kw.txt"),
                                        "", "", "", p("index.poe"), "", 10, 128, 1.0, 1.0, 1.0, 0.0)
    qb_idx = small.QB.idx.copy()
    for q, req in enumerate(kws):
        row = qb_idx[small.QB.off[q]:small.QB.off[q + 1]]
        row[np.isin(row, np.asarray(req, dtype=np.uint32))] |= np.uint32(0x80000000)
    want_ids, want_dis, _ = index.search(small.QD, small.QS, orc.CsrNp(small.QB.off, qb_idx, small.QB.val), cands=128, flags=apoe.SEARCH_KEYWORD)
    assert np.array_equal(ids, want_ids) and np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))
    plain, _, _ = index.search(small.QD, small.QS, small.QB, cands=128)
    assert not np.array_equal(ids, plain)          # the keyword path was really taken


def test_file_level_kg_search_equals_in_memory_call(small, index, tmp_path):
    """knowledge_path / entity2doc_path / query_entity_path: the three CSR files are parsed (ref: load_kg_graph,
    src/query.cu:89-108) and the knowledge-graph kernel runs -- same bits as handing the arrays over in memory."""
    p = lambda s: str(tmp_path / s)
    _write_search_files(small, p)
    kg = synth.make_kg(small.n, small.nq, entities=5000, seed=9)
    synth.write_kg_csr(p("kg.bin"), kg.e2e_off, kg.e2e_idx)
    synth.write_kg_csr(p("e2d.bin"), kg.e2d_off, kg.e2d_idx)
    synth.write_kg_csr(p("qe.bin"), kg.qe_off, kg.qe_idx)
    ids, dis, _, st = apoe.search_index(p("d.fvecs"), p("q.fvecs"), p("s.bin"), p("qs.bin"), p("b.bin"), p("qb.bin"), "",
                                        p("kg.bin"), p("e2d.bin"), p("qe.bin"), p("index.poe"), "", 10, 128, 1.0, 1.0, 1.0, 40.0)
    index.set_kg(kg.e2e_off, kg.e2e_idx, kg.e2d_off, kg.e2d_idx)
    want_ids, want_dis, _ = index.search(small.QD, small.QS, small.QB, cands=128, kg_weight=40.0,
                                         ent=(kg.qe_off.numpy().view(np.uint32), kg.qe_idx.numpy().view(np.uint32)))
    assert np.array_equal(ids, want_ids) and np.array_equal(dis.view(np.uint32), want_dis.view(np.uint32))
    # kg_weight without the files is refused, as the reference launches nothing then (src/query.cu:2042-2047)
    with pytest.raises(apoe.ApoeError):
        apoe.search_index(p("d.fvecs"), p("q.fvecs"), p("s.bin"), p("qs.bin"), p("b.bin"), p("qb.bin"), "", "", "", "", p("index.poe"),
                          "", 10, 128, 1.0, 1.0, 1.0, 40.0)


def test_kg_bonus_lifts_entity_linked_documents(small, index):
    """Quality of the knowledge-graph path, the one check its undefined reference behaviour leaves: the documents of
    the query's own seed entities get the bonus of src/query.cu:1638 and move up the pool -- with kg_weight 40 (the
    example's value; fused scores of the best documents are around -80 here) a tenth of the top entries are such
    documents, with kg_weight 400 most of them, without the bonus hardly any."""
    kg = synth.make_kg(small.n, small.nq, entities=5000, seed=9)
    index.set_kg(kg.e2e_off, kg.e2e_idx, kg.e2d_off, kg.e2d_idx)
    qe_off, qe_idx = kg.qe_off.numpy().view(np.uint32), kg.qe_idx.numpy().view(np.uint32)
    e2d_off, e2d_idx = kg.e2d_off.numpy().view(np.uint32), kg.e2d_idx.numpy().view(np.uint32)
    ids_plain, dis_plain, _ = index.search(small.QD, small.QS, small.QB, cands=128)

    def linked_fraction(ids):
        out = []
        for q in range(small.nq):
            linked = set()
            for e in qe_idx[qe_off[q]:qe_off[q + 1]]:
                linked |= set(e2d_idx[e2d_off[e]:e2d_off[e + 1]].tolist())
            k = min(10, len(linked))
            out.append(len(linked & set(ids[q, :k].tolist())) / k)
        return float(np.mean(out))

    base = linked_fraction(ids_plain)
    ids_40, dis_40, _ = index.search(small.QD, small.QS, small.QB, cands=128, kg_weight=40.0, ent=(qe_off, qe_idx))
    ids_400, dis_400, _ = index.search(small.QD, small.QS, small.QB, cands=128, kg_weight=400.0, ent=(qe_off, qe_idx))
    assert base <= 0.02 and linked_fraction(ids_40) >= base + 0.05 and linked_fraction(ids_400) >= 0.6, \
        (base, linked_fraction(ids_40), linked_fraction(ids_400))
    assert np.all(dis_40[:, 0] <= dis_plain[:, 0]) and np.all(dis_400[:, 0] <= dis_40[:, 0])   # a bonus only lowers the best distance


def test_device_error_word_is_reported_and_cleared(small, index):
    """A bounded wait that runs out raises the error word without faulting anything; the next status check reports
    AP_ERR_DEVICE once and the index keeps working."""
    index.check_status()
    index.debug_wait_timeout(64)
    with pytest.raises(apoe.ApoeError) as e:
        index.check_status()
    assert e.value.code == 6
    index.check_status()
    ids, dis, _ = index.search(small.QD, small.QS, small.QB, cands=128)
    eff, qdh, qs, qb, _ = helpers.scaled_queries(small, (1.0, 1.0, 1.0))
    want_ids, _, _ = orc.search(small.Dh, small.S, small.B, qdh, qs, qb, small.graph, small.ep, 128, 7)
    assert np.array_equal(ids, want_ids)
    # the same through a search that passes statistics: the sticky word surfaces there
    index.debug_wait_timeout(8)
    with pytest.raises(apoe.ApoeError) as e:
        index.search(small.QD, small.QS, small.QB, cands=128)
    assert e.value.code == 6
    ids, _, _ = index.search(small.QD, small.QS, small.QB, cands=128)
    assert np.array_equal(ids, want_ids)
