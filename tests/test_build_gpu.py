"""Build-side parity on the GPU: norms, pruning and row assembly bit-exact against the oracle; the tensor-core
join against the CUDA-core join; end-to-end build quality."""
import numpy as np
import pytest

import apoe
import apoe_oracle as orc
import helpers
import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bix(tiny):
    ix = apoe.Index.from_host(tiny.D, tiny.S, tiny.B, for_build=True)
    yield ix
    ix.close()


def test_norms_match_oracle_bitwise(tiny, bix):
    got = bix.norms()
    assert np.array_equal(got.view(np.uint32), tiny.power.view(np.uint32))


@pytest.fixture(params=["pairs", "pairs_wiped_tables", "stepwise"])
def prune_kernel(request):
    """The pruning kernels: the all-pairs one (default; its term tables numbered by pass or emptied between passes) and
    the step-wise one it falls back to; the value is the build-flag word that selects it."""
    return {"pairs": 0, "pairs_wiped_tables": apoe.BUILD_WIPE_TABLES, "stepwise": apoe.BUILD_PRUNE_STEPWISE}[request.param]


def test_prune_and_rows_match_oracle_bitwise(tiny, bix, prune_kernel):
    """Same pre-pruning k-NN lists in -> same forward lists, keyword-edge lists and 40-wide rows out."""
    new_list, kw, rows = bix.prune(tiny.knn, tiny.knn_dis, tiny.power, flags=prune_kernel)
    assert np.array_equal(new_list, tiny.new_list)
    assert np.array_equal(kw, tiny.kw_edge)
    assert np.array_equal(rows, tiny.graph)
    g, ep = bix.get_graph()
    assert np.array_equal(g, tiny.graph) and np.array_equal(ep, tiny.ep)


def test_prune_on_perturbed_lists(tiny, bix, prune_kernel):
    """Lists with repeated ids and ties (what NN-Descent can leave behind) still match the oracle."""
    rng = np.random.default_rng(1)
    knn = tiny.knn.copy()
    dis = tiny.knn_dis.copy()
    rows = rng.integers(0, tiny.n, 60)
    knn[rows, 40] = knn[rows, 10]
    dis[rows, 40] = dis[rows, 39]
    want = orc.prune(tiny.D7h, tiny.S, tiny.B, knn, dis, tiny.power)
    got = bix.prune(knn, dis, tiny.power, flags=prune_kernel)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]) and np.array_equal(got[2], want[2])


def test_prune_kernels_agree_with_long_rows():
    """A few documents with thousands of terms: nodes next to them overflow the all-pairs staging area and take the
    step-wise kernel; the result still equals the oracle's."""
    ds = helpers.make_dataset(1500, 4, seed=33, with_graph=False)
    rng = np.random.default_rng(2)
    S, B = ds.S, ds.B
    # rebuild the BM25 rows so that 6 documents carry 900 terms each
    off, idx, val = [0], [], []
    heavy = set(rng.choice(ds.n, 6, replace=False).tolist())
    for i in range(ds.n):
        a, b = int(B.off[i]), int(B.off[i + 1])
        if i in heavy:
            ids = np.sort(rng.choice(synth.BM25_VOCAB, 900, replace=False)).astype(np.uint32)
            idx.append(ids); val.append(rng.random(900, dtype=np.float32) + 0.5)
        else:
            idx.append(B.idx[a:b]); val.append(B.val[a:b])
        off.append(off[-1] + len(idx[-1]))
    B2 = orc.CsrNp(np.asarray(off, dtype=np.uint32), np.concatenate(idx).astype(np.uint32), np.concatenate(val).astype(np.float32))
    ix = apoe.Index.from_host(ds.D, S, B2, for_build=True)
    power = orc.cal_power(ds.D7h, S, B2)
    knn, dis = helpers.exact_knn(ds.D, S, B2)
    want = orc.prune(ds.D7h, S, B2, knn, dis, power)
    got = ix.prune(knn, dis, power)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]) and np.array_equal(got[2], want[2])
    # the whole build on the same corpus (wide term tables, fewer of them per join): well-formed rows, and the rows are
    # what the oracle makes of the lists the build ended with
    ix.build(flags=apoe.BUILD_KEEP_KNN, seed=5)
    ids, kdis, kpow = ix.get_knn()
    rows, ep = ix.get_graph()
    assert rows[:, :32].max() < ds.n and np.array_equal(kpow.view(np.uint32), power.view(np.uint32))
    assert np.array_equal(rows, orc.prune(ds.D7h, S, B2, ids, kdis, kpow)[2])
    ix.close()


def _join_lists(n, nodes, rng):
    plist = np.full((nodes, 64), 0xFFFFFFFF, dtype=np.uint32)
    pcnt = np.zeros((nodes, 2), dtype=np.uint32)
    for v in range(nodes):
        nn = int(rng.integers(1, 33))
        rows = nn + int(rng.integers(0, 33))
        plist[v, :rows] = rng.choice(n, size=rows, replace=False)
        pcnt[v] = (nn, rows)
    return plist, pcnt


def test_dense_join_simt_matches_numpy(tiny, bix):
    rng = np.random.default_rng(5)
    plist, pcnt = _join_lists(tiny.n, 37, rng)
    got = bix.debug_join_dense(plist, pcnt, use_tc=False)
    X = orc.h2f(tiny.D7h).astype(np.float64)
    for v in range(plist.shape[0]):
        nn, rows = pcnt[v]
        P = X[plist[v, :rows].astype(np.int64)]
        want = P @ P[:nn].T
        assert np.allclose(got[v, :rows, :nn], want, rtol=1e-5, atol=1e-4)


def test_dense_join_tensor_core_matches_simt(tiny, bix):
    """tcgen05 tiles against the CUDA-core kernel: exact half products, fp32 accumulation in both."""
    rng = np.random.default_rng(6)
    plist, pcnt = _join_lists(tiny.n, 301, rng)   # odd count: the last tile holds one node
    ref = bix.debug_join_dense(plist, pcnt, use_tc=False)
    got = bix.debug_join_dense(plist, pcnt, use_tc=True)
    for v in range(plist.shape[0]):
        nn, rows = pcnt[v]
        assert np.allclose(got[v, :rows, :nn], ref[v, :rows, :nn], rtol=1e-5, atol=2e-4), v


@pytest.mark.parametrize("simt,shared", [(True, False), (False, False), (False, True)])
def test_build_quality(simt, shared):
    """Seeded start + NN-Descent + pruning on 6 000 documents: k-NN recall against exact lists, search recall against
    brute force.  With owned pairs (the default) a true neighbour sits in the list of the end that owns the pair, so
    recall counts a document's own list together with the lists that hold it."""
    ds = helpers.make_dataset(6000, 100, seed=21, with_graph=False)
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B, for_build=True)
    flags = apoe.BUILD_KEEP_KNN | (apoe.BUILD_SIMT_JOIN if simt else 0) | (apoe.BUILD_SHARED_PAIRS if shared else 0)
    st = ix.build(flags=flags, seed=3)
    ids, dis, power = ix.get_knn()
    assert np.all(np.diff(dis, axis=1) >= 0)
    knn, _ = helpers.exact_knn(ds.D, ds.S, ds.B)
    near = [set(r.tolist()) for r in ids]
    if not shared:
        for u in range(ds.n):
            for v in ids[u]:
                assert u not in near[int(v)] or int(v) == u, "a pair sits in the lists of both of its ends"
        holders = [set() for _ in range(ds.n)]
        for u in range(ds.n):
            for v in ids[u]:
                holders[int(v)].add(u)
        near = [near[i] | holders[i] for i in range(ds.n)]
    rec = np.mean([len(near[i] & set(knn[i, :32].tolist())) / 32 for i in range(0, ds.n, 7)])
    assert rec >= 0.80, rec
    want_power = orc.cal_power(ds.D7h, ds.S, ds.B)
    assert np.array_equal(power.view(np.uint32), want_power.view(np.uint32))
    rows, ep = ix.get_graph()
    assert np.array_equal(ep, orc.entry_points(want_power))
    # the rows are what the oracle makes of the same k-NN lists
    want = orc.prune(ds.D7h, ds.S, ds.B, ids, dis, power)
    assert np.array_equal(rows, want[2])
    eff, qdh, qs, qb, qd = helpers.scaled_queries(ds)
    gt, _, _ = orc.bruteforce(ds.D, ds.S, ds.B, qd, qs, qb, 7, 10)
    got, _, _ = ix.search(ds.QD, ds.QS, ds.QB, cands=128)
    built_recall = helpers.recall_at(got, gt)
    # yardstick: the same search over the graph pruned from the *exact* k-NN lists (the synthetic corpus itself caps
    # recall well below 1: its dense component is structureless and carries a large normalised weight)
    ix.prune(knn, helpers.exact_knn(ds.D, ds.S, ds.B)[1], power)
    ref, _, _ = ix.search(ds.QD, ds.QS, ds.QB, cands=128)
    assert built_recall >= helpers.recall_at(ref, gt) - 0.05, (built_recall, helpers.recall_at(ref, gt))
    assert st.iterations_run >= 1 and st.distance_evals > 0
    ix.close()


def test_build_index_file_round_trip(tiny, tmp_path):
    p = lambda s: str(tmp_path / s)
    synth.write_fvecs(p("d.fvecs"), tiny.corpus.dense)
    synth.write_csr(p("s.bin"), tiny.corpus.sparse)
    synth.write_csr(p("b.bin"), tiny.corpus.bm25)
    st = apoe.build_index(p("d.fvecs"), p("s.bin"), p("b.bin"), p("index.poe"), seed=1)
    rows, ep = synth.read_poe(p("index.poe"))
    assert rows.shape == (tiny.n, 40) and ep.shape == (32,)
    assert rows[:, :32].max() < tiny.n and rows[:, 32].max() <= 7
    import os
    assert os.path.getsize(p("index.poe")) == 8 + 128 + tiny.n * 164
    ix = apoe.Index.from_host(tiny.D, tiny.S, tiny.B)
    ix.load_graph(p("index.poe"))
    g2, ep2 = ix.get_graph()
    assert np.array_equal(g2, rows) and np.array_equal(ep2, ep)
    ix.close()


def _graph_recall(ix, ds, gt):
    got, _, _ = ix.search(ds.QD, ds.QS, ds.QB, cands=128)
    return helpers.recall_at(got, gt)


def test_reverse_pass_and_random_start_options():
    """AP_BUILD_SHARED_PAIRS | AP_BUILD_REVERSE_PASS (the closing reverse merge, ref merge_reverse_plus
    src/index.cu:386-478) and AP_BUILD_RANDOM_START (ref initialize_graph src/index.cu:99-106): list invariants hold
    and the graphs search about as well as the default build's."""
    ds = helpers.make_dataset(5000, 100, seed=23, with_graph=False)
    eff, qdh, qs, qb, qd = helpers.scaled_queries(ds)
    gt, _, _ = orc.bruteforce(ds.D, ds.S, ds.B, qd, qs, qb, 7, 10)
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B, for_build=True)
    ix.build(flags=apoe.BUILD_KEEP_KNN, seed=3)
    base = _graph_recall(ix, ds, gt)
    knn_exact, _ = helpers.exact_knn(ds.D, ds.S, ds.B)

    def list_recall(ids):
        return float(np.mean([len(set(ids[i].tolist()) & set(knn_exact[i, :32].tolist())) / 32 for i in range(0, ds.n, 9)]))

    # classic NN-Descent without and with the closing reverse merge (deterministic builds, so that the reverse merge is
    # the only difference between the two)
    classic = apoe.BUILD_KEEP_KNN | apoe.BUILD_SHARED_PAIRS | apoe.BUILD_DETERMINISTIC
    ix.build(flags=classic, seed=3)
    ids0, dis0, _ = ix.get_knn()
    st = ix.build(flags=classic | apoe.BUILD_REVERSE_PASS, seed=3)
    ids1, dis1, power = ix.get_knn()
    assert np.all(np.diff(dis1, axis=1) >= 0) and ids1.max() < ds.n
    for i in range(0, ds.n, 11):                                  # no self loops, no repeated neighbour
        row = ids1[i][dis1[i] < 1e5]
        assert i not in row and len(set(row.tolist())) == len(row)
    # the reverse merge can only improve a list: no distance in it grows, and some lists do gain entries
    assert np.all(dis1 <= dis0) and np.mean(dis1[:, -1] < dis0[:, -1]) > 0.01
    assert list_recall(ids1) >= list_recall(ids0)
    rows, _ = ix.get_graph()
    assert np.array_equal(rows, orc.prune(ds.D7h, ds.S, ds.B, ids1, dis1, power)[2])
    assert _graph_recall(ix, ds, gt) >= base - 0.08
    # random initial lists only
    st_r = ix.build(flags=apoe.BUILD_KEEP_KNN | apoe.BUILD_RANDOM_START, seed=3, iterations=12)
    ids2, dis2, _ = ix.get_knn()
    assert np.all(np.diff(dis2, axis=1) >= 0)
    assert st_r.iterations_run >= 4                               # no head start: more rounds before the lists settle
    assert _graph_recall(ix, ds, gt) >= base - 0.08
    ix.close()


def test_deterministic_build_gives_one_graph_per_seed():
    """AP_BUILD_DETERMINISTIC: two builds with one seed give the same lists and the same graph, bit for bit (the default
    build keeps proposals in arrival order and may differ from run to run); another seed gives another graph; the
    graph searches about as well as the default one."""
    ds = helpers.make_dataset(6000, 100, seed=21, with_graph=False)
    eff, qdh, qs, qb, qd = helpers.scaled_queries(ds)
    gt, _, _ = orc.bruteforce(ds.D, ds.S, ds.B, qd, qs, qb, 7, 10)
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B, for_build=True)
    ix.build(flags=apoe.BUILD_KEEP_KNN, seed=3)
    base = _graph_recall(ix, ds, gt)
    runs = []
    for seed in (3, 3, 4):
        st = ix.build(flags=apoe.BUILD_KEEP_KNN | apoe.BUILD_DETERMINISTIC, seed=seed)
        ids, dis, _ = ix.get_knn()
        rows, ep = ix.get_graph()
        runs.append((ids.copy(), dis.copy(), rows.copy(), ep.copy(), st.distance_evals, _graph_recall(ix, ds, gt)))
        assert st.proposal_overflows == 0
    a, b, c = runs
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))
    assert np.array_equal(a[2], b[2]) and np.array_equal(a[3], b[3]) and a[4] == b[4]
    assert not np.array_equal(a[2], c[2])
    assert a[5] >= base - 0.05, (a[5], base)
    ix.close()


def test_numbered_and_wiped_term_tables_give_the_same_distances():
    """The joins either number the keys of their shared-memory term tables by pass (default where the term ids leave
    high bits free) or empty the tables between passes (AP_BUILD_WIPE_TABLES).  The numbering changes the hash slots,
    so the rare rows whose two-choice table cannot be built -- they sit one join out -- are not the same rows and the
    two builds drift apart a little: the lists have to agree almost everywhere, and a pair both hold has to carry the
    same distance up to the order of the float sums (which of the two rows was hashed and which streamed) -- a term
    product lost or added by a wrong slot would show as a difference of 0.01 and more.  (The pruning kernel is
    compared output for output by the prune_kernel fixture above.)"""
    ds = helpers.make_dataset(6000, 4, seed=22, with_graph=False)
    ix = apoe.Index.from_host(ds.D, ds.S, ds.B, for_build=True)
    out = []
    for extra in (0, apoe.BUILD_WIPE_TABLES):
        st = ix.build(flags=apoe.BUILD_KEEP_KNN | apoe.BUILD_DETERMINISTIC | extra, seed=9)
        ids, dis, _ = ix.get_knn()
        key = (np.arange(ids.shape[0], dtype=np.uint64)[:, None] << np.uint64(32)) | ids.astype(np.uint64)
        out.append((key.ravel(), dis.ravel().copy(), st.distance_evals))
    (ka, da, ea), (kb, db, eb) = out
    assert abs(int(ea) - int(eb)) <= 0.001 * ea, (ea, eb)
    common, ia, ib = np.intersect1d(ka, kb, return_indices=True)
    assert common.size >= 0.995 * ka.size, common.size / ka.size
    diff = np.abs(da[ia] - db[ib])
    assert float(diff.max()) <= 2e-4, float(diff.max())
    assert float(np.mean(diff == 0)) >= 0.98, float(np.mean(diff == 0))
    ix.close()
