"""Shared test utilities: seeded datasets, exact k-NN lists on the CPU, oracle-built graphs."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import scipy.sparse as sp

import apoe_oracle as orc
import synth


@dataclass
class Dataset:
    corpus: synth.Corpus
    queries: synth.Queries
    D: np.ndarray            # dense fp32
    S: orc.CsrNp
    B: orc.CsrNp
    QD: np.ndarray
    QS: orc.CsrNp
    QB: orc.CsrNp
    knn: np.ndarray = None
    knn_dis: np.ndarray = None
    power: np.ndarray = None
    new_list: np.ndarray = None
    kw_edge: np.ndarray = None
    graph: np.ndarray = None
    ep: np.ndarray = None
    D7h: np.ndarray = None   # half bits of 7 * dense
    Dh: np.ndarray = None    # half bits of dense

    @property
    def n(self):
        return self.D.shape[0]

    @property
    def nq(self):
        return self.QD.shape[0]


def _tosp(cs: orc.CsrNp, vocab: int):
    return sp.csr_matrix((cs.val, cs.idx.astype(np.int64), cs.off.astype(np.int64)), shape=(cs.rows, vocab))


def exact_knn(D, S, B, k=64, dense_scale=7.0):
    """Exact hybrid k-NN lists (fp32), build-time scaling of the dense part, ascending distance."""
    ip = (dense_scale * dense_scale) * (D @ D.T)
    ip += np.asarray((_tosp(S, synth.SPARSE_VOCAB) @ _tosp(S, synth.SPARSE_VOCAB).T).todense())
    ip += np.asarray((_tosp(B, synth.BM25_VOCAB) @ _tosp(B, synth.BM25_VOCAB).T).todense())
    np.fill_diagonal(ip, -np.inf)
    knn = np.argsort(-ip, axis=1, kind="stable")[:, :k].astype(np.uint32)
    dis = (1.0 - np.take_along_axis(ip, knn.astype(np.int64), axis=1)).astype(np.float32)
    return knn, dis


def make_dataset(n, nq, seed=7, with_graph=True) -> Dataset:
    c = synth.make_corpus(n, seed=seed)
    q = synth.make_queries(nq, c.idf, seed=seed + 1)
    ds = Dataset(c, q, c.dense.numpy(), orc.CsrNp.from_torch(c.sparse), orc.CsrNp.from_torch(c.bm25), q.dense.numpy(),
                 orc.CsrNp.from_torch(q.sparse), orc.CsrNp.from_torch(q.bm25))
    ds.Dh = orc.f2h(ds.D)
    ds.D7h = orc.f2h(ds.D * np.float32(7.0))
    if with_graph:
        ds.knn, ds.knn_dis = exact_knn(ds.D, ds.S, ds.B)
        ds.power = orc.cal_power(ds.D7h, ds.S, ds.B)
        ds.new_list, ds.kw_edge, ds.graph, _ = orc.prune(ds.D7h, ds.S, ds.B, ds.knn, ds.knn_dis, ds.power)
        ds.ep = orc.entry_points(ds.power)
    return ds


def scaled_queries(ds: Dataset, weights=(1.0, 1.0, 1.0), normalise=True):
    """Effective weights (sparse, bm25, dense) and the query scaled + rounded the way the search sees it."""
    ws, wb, wd = weights
    if normalise:
        ws, wb, wd = orc.effective_weights(ds.D, ds.S, ds.B, ds.QD, ds.QS, ds.QB, ws, wb, wd)
    qd, qs, qb = orc.scale_queries(ds.QD, ds.QS, ds.QB, ws, wb, wd)
    return (ws, wb, wd), orc.f2h(qd), qs, qb, qd


def recall_at(ids, gt, k=10):
    return float(np.mean([len(set(ids[i, :k].tolist()) & set(gt[i, :k].tolist())) / k for i in range(gt.shape[0])]))
