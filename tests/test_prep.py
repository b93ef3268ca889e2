"""Oracle of the BM25 input preparation against a case worked out by hand (the reference has no code for this step,
so this is the only pin: the published Okapi formula evaluated in float64 below)."""
import math

import numpy as np

import apoe_oracle as orc


def test_bm25_oracle_known_answer():
    # three documents over a vocabulary of five terms; rows deliberately not sorted by id
    off = np.array([0, 3, 5, 6], dtype=np.uint32)
    idx = np.array([4, 0, 2, 2, 1, 2], dtype=np.uint32)
    tf = np.array([2, 1, 3, 1, 4, 2], dtype=np.float32)
    k1, b, n = 1.2, 0.75, 3
    df = [1, 1, 3, 0, 1]
    idf = [math.log(1 + (n - d + 0.5) / (d + 0.5)) for d in df]
    lens = [6.0, 5.0, 2.0]
    avg = sum(lens) / n
    def w(t, f, row):
        return idf[t] * f * (k1 + 1) / (f + k1 * (1 - b + b * lens[row] / avg))
    want_idx = [0, 2, 4, 1, 2, 2]
    want_w = [w(0, 1, 0), w(2, 3, 0), w(4, 2, 0), w(1, 4, 1), w(2, 1, 1), w(2, 2, 2)]
    got_idx, got_w, got_df, got_idf, rl = orc.bm25_corpus(off, idx, tf, 5, k1, b)
    assert rl is None and got_idx.tolist() == want_idx and got_df.tolist() == df
    assert np.allclose(got_idf, idf, rtol=1e-6) and np.allclose(got_w, want_w, rtol=1e-6)
    # renumbering by descending document frequency: term 2 (df 3) -> 0, then 0, 1, 4 (df 1) by id, then 3 (df 0)
    got_idx, got_w, _, _, rl = orc.bm25_corpus(off, idx, tf, 5, k1, b, relabel_by_df=True)
    assert rl.tolist() == [1, 2, 0, 4, 3]
    assert got_idx.tolist() == [0, 1, 3, 0, 2, 0]
    assert np.allclose(got_w, [w(2, 3, 0), w(0, 1, 0), w(4, 2, 0), w(2, 1, 1), w(1, 4, 1), w(2, 2, 2)], rtol=1e-6)
    # queries: idf x tf, same renumbering
    q_idx, q_w = orc.bm25_queries(np.array([0, 2], dtype=np.uint32), np.array([4, 2], dtype=np.uint32), np.array([1, 2], dtype=np.float32), got_idf := np.asarray(idf, dtype=np.float32), rl)
    assert q_idx.tolist() == [0, 3] and np.allclose(q_w, [2 * idf[2], idf[4]], rtol=1e-6)
