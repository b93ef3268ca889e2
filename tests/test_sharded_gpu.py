"""Corpus-sharded build and search below the Python layer, on one GPU: every shard is built from its own rows of the
corpus files and written as <prefix>.<g>.poe plus a manifest; every shard then searches all queries with the weights
normalised on global documents 0..99 and ships its top-k as packed keys; the device merge gives the global top-k.
Checked against the CPU oracle shard by shard (bit for bit) and against the exact brute force (recall)."""
import os

import numpy as np
import pytest
import torch

import apoe
import apoe_oracle as orc
import dist_search
import helpers
import synth

pytestmark = pytest.mark.gpu

N_DOCS, N_QUERIES, SHARDS, TOP_K, CANDS = 3001, 64, 3, 10, 64


@pytest.fixture(scope="module")
def sharded(tmp_path_factory):
    d = tmp_path_factory.mktemp("shards")
    p = lambda s: str(d / s)
    ds = helpers.make_dataset(N_DOCS, N_QUERIES, seed=51, with_graph=False)
    synth.write_fvecs(p("d.fvecs"), ds.corpus.dense)
    synth.write_csr(p("s.bin"), ds.corpus.sparse)
    synth.write_csr(p("b.bin"), ds.corpus.bm25)
    synth.write_fvecs(p("q.fvecs"), ds.queries.dense)
    synth.write_csr(p("qs.bin"), ds.queries.sparse)
    synth.write_csr(p("qb.bin"), ds.queries.bm25)
    for g in range(SHARDS):
        apoe.build_index_shard(p("d.fvecs"), p("s.bin"), p("b.bin"), p("idx"), g, SHARDS, seed=5)
    return ds, p


def _rows(c, a, b):
    lo, hi = int(c.off[a]), int(c.off[b])
    return orc.CsrNp(c.off[a:b + 1] - c.off[a], c.idx[lo:hi], c.val[lo:hi])


def test_shard_files_and_manifest(sharded):
    ds, p = sharded
    n, shards = apoe.read_shard_manifest(p("idx.manifest"))
    assert n == N_DOCS and [(a, c) for a, c, _ in shards] == [apoe.shard_range(N_DOCS, g, SHARDS) for g in range(SHARDS)]
    for g, (a, c, name) in enumerate(shards):
        path = p(name)
        assert os.path.getsize(path) == 8 + 128 + c * 164                     # the reference's file layout, shard-local rows
        rows, ep = synth.read_poe(path)
        assert rows.shape == (c, 40) and rows[:, :32].max() < c and ep.max() < c


def test_sharded_search_equals_oracle_per_shard_and_merges_to_global_top_k(sharded):
    ds, p = sharded
    n, shards = apoe.read_shard_manifest(p("idx.manifest"))
    eff = orc.effective_weights(ds.D, ds.S, ds.B, ds.QD, ds.QS, ds.QB, 1.0, 1.0, 1.0)    # global documents 0..99
    qd, qs, qb = orc.scale_queries(ds.QD, ds.QS, ds.QB, *eff)
    all_keys, union = [], [dict() for _ in range(N_QUERIES)]
    for g, (a, c, name) in enumerate(shards):
        keys, st = apoe.search_index_shard(p("d.fvecs"), p("q.fvecs"), p("s.bin"), p("qs.bin"), p("b.bin"), p("qb.bin"), p("idx.manifest"),
                                           g, TOP_K, CANDS, 1.0, 1.0, 1.0)
        assert keys.shape == (N_QUERIES, TOP_K)
        assert (st.eff_sparse, st.eff_bm25, st.eff_dense) == tuple(np.float32(x) for x in eff)   # not the shard's own first 100 documents
        rows, ep = synth.read_poe(p(name))
        want_ids, want_dis, _ = orc.search(ds.Dh[a:a + c], _rows(ds.S, a, a + c), _rows(ds.B, a, a + c), orc.f2h(qd), qs, qb, rows, ep, CANDS, 7)
        ids, dis = apoe.unpack_shard_keys(keys)
        assert np.array_equal(ids, want_ids[:, :TOP_K] + np.uint32(a))         # global ids = local ids + the shard's first document
        assert np.array_equal(dis.view(np.uint32), want_dis[:, :TOP_K].view(np.uint32))
        all_keys.append(keys)
    g_keys = torch.from_numpy(np.stack(all_keys).view(np.int64)).cuda()
    out_ids = torch.empty(N_QUERIES, TOP_K, dtype=torch.int32, device="cuda")
    out_dis = torch.empty(N_QUERIES, TOP_K, dtype=torch.float32, device="cuda")
    apoe.merge_shard_keys(g_keys, TOP_K, out_ids, out_dis)
    torch.cuda.synchronize()
    want = dist_search.merge_keys_reference(g_keys.cpu(), TOP_K)
    want_ids, want_dis = apoe.unpack_shard_keys(want.numpy().view(np.uint64))
    got_ids = out_ids.cpu().numpy().view(np.uint32)
    assert np.array_equal(got_ids, want_ids) and np.array_equal(out_dis.cpu().numpy().view(np.uint32), want_dis.view(np.uint32))
    # the merged answer against the exact brute force over the whole corpus, and against the unsharded index
    gt, _, _ = orc.bruteforce(ds.D, ds.S, ds.B, qd, qs, qb, 7, TOP_K)
    sharded_recall = helpers.recall_at(got_ids, gt)
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B, for_build=True)
    ix.build(seed=5)
    one, _, _ = ix.search(ds.QD, ds.QS, ds.QB, cands=CANDS)
    ix.close()
    assert sharded_recall >= helpers.recall_at(one, gt) - 0.03, (sharded_recall, helpers.recall_at(one, gt))
    assert sharded_recall >= 0.8, sharded_recall


def test_range_index_equals_index_of_the_same_rows(sharded):
    """Reading rows [a, a + c) from the files gives the same records as an index made of those rows in memory."""
    ds, p = sharded
    a, c = apoe.shard_range(N_DOCS, 1, SHARDS)
    ix_f, st = apoe.Index.from_files_range(p("d.fvecs"), p("s.bin"), p("b.bin"), a, c)
    ix_m = apoe.Index.from_host(ds.D[a:a + c], _rows(ds.S, a, a + c), _rows(ds.B, a, a + c))
    assert st.rows == c and ix_f.n == c
    rng = np.random.default_rng(4)
    pq = rng.integers(0, N_QUERIES, 2000).astype(np.uint32)
    pd = rng.integers(0, c, 2000).astype(np.uint32)
    d_f = ix_f.fused_distances(ds.QD, ds.QS, ds.QB, pq, pd)
    d_m = ix_m.fused_distances(ds.QD, ds.QS, ds.QB, pq, pd)
    assert np.array_equal(d_f.view(np.uint32), d_m.view(np.uint32))
    with pytest.raises(apoe.ApoeError):
        apoe.Index.from_files_range(p("d.fvecs"), p("s.bin"), p("b.bin"), N_DOCS - 5, 10)
    ix_f.close(); ix_m.close()
