"""BM25 input preparation on the GPU against the numpy restatement.  Integer outputs (document frequencies, the
renumbering table, the reordered ids) must be equal; float outputs within 1e-5 relative (logf and the order of
fused multiply-adds differ between the device and numpy)."""
import numpy as np
import pytest

import apoe
import apoe_oracle as orc

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def _raw_corpus(rows, vocab, seed, long_row=0):
    rng = np.random.default_rng(seed)
    cnt = rng.poisson(40, rows).clip(0, 300)
    cnt[rng.integers(0, rows, 5)] = 0          # a few empty rows
    if long_row:
        cnt[rows // 2] = long_row
    off = np.zeros(rows + 1, dtype=np.uint32); off[1:] = np.cumsum(cnt)
    idx = np.empty(int(off[-1]), dtype=np.uint32)
    p = 1.0 / np.arange(1, vocab + 1); p /= p.sum()
    for r in range(rows):
        idx[off[r]:off[r + 1]] = rng.choice(vocab, size=int(cnt[r]), replace=False, p=p if cnt[r] < 400 else None)   # unsorted
    tf = (1 + rng.geometric(0.6, idx.size)).astype(np.float32)
    return off, idx, tf


@pytest.mark.parametrize("relabel", [False, True])
def test_corpus_weights_match_oracle(relabel):
    vocab = 5000
    off, idx, tf = _raw_corpus(3000, vocab, 11, long_row=1500)
    want = orc.bm25_corpus(off, idx, tf, vocab, 1.2, 0.75, relabel_by_df=relabel)
    got = apoe.bm25_corpus(off, idx, tf, vocab, 1.2, 0.75, relabel_by_df=relabel)
    assert np.array_equal(got[2], want[2])                        # df
    assert np.allclose(got[3], want[3], rtol=RTOL, atol=1e-7)     # idf
    if relabel:
        assert np.array_equal(got[4], want[4])
    assert np.array_equal(got[0], want[0])                        # ids, renumbered and ascending per row
    assert np.allclose(got[1], want[1], rtol=RTOL, atol=1e-7)
    for r in (0, 17, 1500, 2999):
        assert np.all(np.diff(got[0][off[r]:off[r + 1]].astype(np.int64)) > 0)
    st = got[5]
    assert st.nnz == idx.size and st.rows_sorted > 0 and st.launches >= 4
    assert abs(st.avg_len - tf.sum() / 3000) < 1e-3 * st.avg_len


def test_sorted_rows_skip_the_sort_and_other_parameters():
    vocab = 2000
    off, idx, tf = _raw_corpus(500, vocab, 3)
    for r in range(500):
        idx[off[r]:off[r + 1]].sort()
    want = orc.bm25_corpus(off, idx, tf, vocab, 0.9, 0.4)
    got = apoe.bm25_corpus(off, idx, tf, vocab, 0.9, 0.4)
    assert got[5].rows_sorted == 0
    assert np.array_equal(got[0], want[0]) and np.allclose(got[1], want[1], rtol=RTOL, atol=1e-7)


def test_queries_follow_the_corpus_tables():
    vocab = 5000
    off, idx, tf = _raw_corpus(3000, vocab, 11)
    _, _, _, idf, rl, _ = apoe.bm25_corpus(off, idx, tf, vocab, relabel_by_df=True)
    qoff, qidx, qtf = _raw_corpus(200, vocab, 12)
    want = orc.bm25_queries(qoff, qidx, qtf, idf, rl)
    got = apoe.bm25_queries(qoff, qidx, qtf, idf, rl)
    assert np.array_equal(got[0], want[0]) and np.allclose(got[1], want[1], rtol=RTOL, atol=1e-7)
    got2 = apoe.bm25_queries(qoff, qidx, qtf, idf, None)
    want2 = orc.bm25_queries(qoff, qidx, qtf, idf, None)
    assert np.array_equal(got2[0], want2[0]) and np.allclose(got2[1], want2[1], rtol=RTOL, atol=1e-7)


def test_bad_inputs_are_refused():
    off = np.array([0, 2], dtype=np.uint32)
    with pytest.raises(apoe.ApoeError, match="outside the vocabulary"):
        apoe.bm25_corpus(off, np.array([1, 7], dtype=np.uint32), np.array([1, 1], dtype=np.float32), 5)
    with pytest.raises(apoe.ApoeError, match="outside the vocabulary"):
        apoe.bm25_queries(off, np.array([1, 7], dtype=np.uint32), np.array([1, 1], dtype=np.float32), np.ones(5, dtype=np.float32))
    with pytest.raises(apoe.ApoeError):
        apoe.bm25_corpus(np.array([0, 0], dtype=np.uint32), np.zeros(0, dtype=np.uint32), np.zeros(0, dtype=np.float32), 5)   # no term frequencies
