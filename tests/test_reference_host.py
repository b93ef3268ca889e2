"""Host-side parity against the reference itself (no GPU needed).

The reference's file readers (include/utils.cuh:361-398, src/query.cu:35-108) and its nDCG figure (cal_precision,
src/query.cu:111-145) are plain host code; the shared library built from the reference tree under oracle/_ref/
exports them, so the library's loaders and its evaluation step are compared here with the reference's own functions,
and the oracle's restatement of cal_precision is pinned to it.  Skipped where that library was not built.  The
format fixtures are the files of the reference's example_data folder, read in place where the tree is mounted
(shapes are checked, no record is copied).
"""
import os

import numpy as np
import pytest

import apoe
import apoe_oracle as orc
import apoe_ref
import synth

REF_DATA = os.path.join(os.environ.get("APOE_REFERENCE_TREE", os.path.join(os.sep, "root", "reference")), "example_data")
needs_ref = pytest.mark.skipif(not apoe_ref.available(), reason="oracle/_ref/libapoe_ref.so is not built")
needs_data = pytest.mark.skipif(not os.path.exists(os.path.join(REF_DATA, "2wiki_kg.bin")), reason="the reference's example_data is not mounted")


def _ndcg_case(seed, nq=200, n_docs=500, top_k=10, empty_rows=False):
    """Result rows with hits at every rank, misses, relevant ids listed twice and (optionally) rows without relevant ids."""
    rng = np.random.default_rng(seed)
    results = np.stack([rng.choice(n_docs, size=16, replace=False) for _ in range(nq)]).astype(np.uint32)
    qrels = []
    for q in range(nq):
        k = int(rng.integers(1, 5))
        hits = rng.choice(results[q, :top_k], size=int(rng.integers(0, min(k, 3) + 1)), replace=False).tolist()
        miss = rng.integers(n_docs, 2 * n_docs, size=k - len(hits)).tolist()
        rel = [int(x) for x in hits + miss]
        if rel and q % 17 == 0:
            rel.append(rel[0])               # a relevant id listed twice (multiset intersection)
        rng.shuffle(rel)
        qrels.append([] if (empty_rows and q % 23 == 5) else rel)
    return results, qrels


def _as_cout(v: float) -> str:
    return "nDCG@10: %g" % np.float32(v)     # std::cout prints a float with 6 significant digits, like %g


@needs_ref
@pytest.mark.parametrize("seed", [1, 2, 3])
def test_ndcg_digits_equal_the_reference(seed):
    results, qrels = _ndcg_case(seed)
    text = apoe_ref.cal_precision_text(results, 10, qrels)          # what cal_precision prints
    assert text.startswith("nDCG@10: ")
    got = apoe.ndcg(results, 10, qrels)
    want = orc.cal_precision(results, 10, qrels)
    assert np.float32(got) == np.float32(want)                       # same float as the oracle's restatement
    assert _as_cout(got) == text and _as_cout(want) == text          # and the same printed digits as the reference
    assert 0.0 < got < 1.0


def test_ndcg_float_accumulation_and_empty_rows():
    """Without the reference library: the library equals the oracle bit for bit; rows without relevant ids are skipped
    by the library where the reference's arithmetic (restated by the oracle) yields NaN."""
    results, qrels = _ndcg_case(9)
    assert np.float32(apoe.ndcg(results, 10, qrels)) == np.float32(orc.cal_precision(results, 10, qrels))
    results, qrels = _ndcg_case(10, empty_rows=True)
    assert np.isnan(orc.cal_precision(results, 10, qrels))
    v = apoe.ndcg(results, 10, qrels)
    assert np.isfinite(v) and 0.0 < v < 1.0
    # a perfect ranking scores exactly 1
    perfect = [[int(x) for x in row[:3]] for row in results]
    assert apoe.ndcg(results, 10, perfect) == 1.0


@needs_ref
def test_written_files_are_read_alike_by_both_loaders(tmp_path):
    """Files from this repository's writers: the library's readers and the reference's readers return the same arrays."""
    c = synth.make_corpus(300, seed=41)
    q = synth.make_queries(20, c.idf, seed=42)
    kg = synth.make_kg(300, 20, entities=500, seed=43)
    p = lambda s: str(tmp_path / s)
    synth.write_fvecs(p("d.fvecs"), c.dense)
    synth.write_csr(p("s.bin"), c.sparse)
    synth.write_kg_csr(p("kg.bin"), kg.e2e_off, kg.e2e_idx)
    kws = synth.make_keywords(q, seed=44)
    synth.write_keywords(p("kw.txt"), kws)
    assert np.array_equal(apoe.read_fvecs(p("d.fvecs")), apoe_ref.load_fvecs(p("d.fvecs")))
    mine, theirs = apoe.read_csr(p("s.bin")), apoe_ref.load_csr(p("s.bin"), 300)
    assert all(np.array_equal(a, b) for a, b in zip(mine, theirs)) and mine[0].size == 301
    mine, theirs = apoe.read_kg(p("kg.bin")), apoe_ref.load_kg(p("kg.bin"))
    assert all(np.array_equal(a, b) for a, b in zip(mine, theirs))
    mine, theirs = apoe.read_id_lines(p("kw.txt"), 20), apoe_ref.load_txt(p("kw.txt"), 20)
    assert all(np.array_equal(a, b) for a, b in zip(mine, theirs))
    assert mine[1].tolist() == [t for row in kws for t in row]


@needs_data
def test_loaders_parse_the_reference_sample_files_in_place():
    """The shapes the shipped sample files are known to have (entities, rows, longest rows, id ranges)."""
    f = lambda s: os.path.join(REF_DATA, s)
    off, idx = apoe.read_kg(f("2wiki_kg.bin"))
    assert off.size == 30485 and idx.size == 60788 and off[0] == 0 and off[-1] == idx.size     # 30 484 entities + 1
    assert int(np.diff(off.astype(np.int64)).max()) == 89 and int(idx.max()) < 30484
    e_off, e_idx = apoe.read_kg(f("2wiki_entity2doc.bin"))
    assert e_off.size == off.size and e_idx.size == 39852 and int(np.diff(e_off.astype(np.int64)).max()) == 96
    assert int(e_idx.max()) < 6119                                                           # document ids of the corpus
    q_off, q_idx = apoe.read_kg(f("2wiki_query_kg.bin"))
    d = np.diff(q_off.astype(np.int64))
    assert q_off.size == 101 and d.min() == 1 and d.max() == 2 and int(q_idx.max()) < 30484
    b_off, b_idx, b_val = apoe.read_csr(f("2wiki_bm25_corpus.bin"))                          # row count from the file size
    d = np.diff(b_off.astype(np.int64))
    assert b_off.size - 1 == 6119 and d.max() == 347 and abs(d.mean() - 36.9) < 0.05 and int(b_idx.max()) < 33357
    assert all(np.all(np.diff(b_idx[b_off[r]:b_off[r + 1]].astype(np.int64)) > 0) for r in range(0, 6119, 97))   # ascending ids
    assert np.all(np.isfinite(b_val))
    for name, rows, mean, longest in (("2wiki_bm25_queries.bin", 1000, 6.8, 18), ("2wiki_sparse_queries.bin", 1000, 60.8, 98)):
        off, idx, val = apoe.read_csr(f(name))
        d = np.diff(off.astype(np.int64))
        assert off.size - 1 == rows and d.max() == longest and abs(d.mean() - mean) < 0.05
    qd = apoe.read_fvecs(f("2wiki_dense_queries.fvecs"))
    assert qd.shape == (1000, 1024) and np.allclose(np.linalg.norm(qd, axis=1), 1.0, atol=1e-3)
    r_off, r_ids = apoe.read_id_lines(f("2wiki_qrels.txt"), 1000)
    d = np.diff(r_off.astype(np.int64))
    assert d.min() == 2 and d.max() == 4 and int(r_ids.max()) < 6119


@needs_ref
@needs_data
def test_sample_files_parse_like_the_reference_parses_them():
    f = lambda s: os.path.join(REF_DATA, s)
    for name in ("2wiki_kg.bin", "2wiki_entity2doc.bin", "2wiki_query_kg.bin"):
        assert all(np.array_equal(a, b) for a, b in zip(apoe.read_kg(f(name)), apoe_ref.load_kg(f(name)))), name
    for name, rows in (("2wiki_bm25_corpus.bin", 6119), ("2wiki_bm25_queries.bin", 1000), ("2wiki_sparse_queries.bin", 1000)):
        assert all(np.array_equal(a, b) for a, b in zip(apoe.read_csr(f(name)), apoe_ref.load_csr(f(name), rows))), name
    assert np.array_equal(apoe.read_fvecs(f("2wiki_dense_queries.fvecs")), apoe_ref.load_fvecs(f("2wiki_dense_queries.fvecs")))
    assert all(np.array_equal(a, b) for a, b in zip(apoe.read_id_lines(f("2wiki_qrels.txt"), 1000), apoe_ref.load_txt(f("2wiki_qrels.txt"), 1000)))


def test_loader_errors(tmp_path):
    with pytest.raises(apoe.ApoeError) as e:
        apoe.read_kg(str(tmp_path / "missing.bin"))
    assert e.value.code == 2
    bad = tmp_path / "short.bin"
    np.array([5, 100, 0, 1], dtype=np.uint32).tofile(bad)          # header promises more than the file holds
    with pytest.raises(apoe.ApoeError) as e:
        apoe.read_kg(str(bad))
    assert e.value.code == 2
    with pytest.raises(apoe.ApoeError):
        apoe.read_csr(str(bad))
