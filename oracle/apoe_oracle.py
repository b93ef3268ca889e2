"""ctypes binding of the CPU oracle (oracle/apoe_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the
benchmark's CPU-baseline leg; never by the shipped library or its Python host
layer.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

F_DENSE, F_SPARSE, F_BM25, F_KEYWORD, F_KG, F_UNFUSED_DENSE, F_NOFMA_SPARSE = 1, 2, 4, 8, 16, 32, 64


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "libapoe_oracle.so")
    src = os.path.join(_HERE, "apoe_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libapoe_oracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
    return _LIB


def _p(a, dtype):
    if a is None:
        return None
    assert a.dtype == dtype and a.flags["C_CONTIGUOUS"], (a.dtype, dtype)
    return a.ctypes.data_as(C.c_void_p)


def _u32(a):
    return None if a is None else np.ascontiguousarray(np.asarray(a).view(np.uint32) if np.asarray(a).dtype == np.int32 else np.asarray(a, dtype=np.uint32))


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


class CsrNp:
    """Host CSR triple as numpy arrays (u32 off, u32 idx, f32 val)."""

    def __init__(self, off, idx, val):
        self.off, self.idx, self.val = _u32(off), _u32(idx), _f32(val)

    @classmethod
    def from_torch(cls, csr):
        return cls(csr.off.cpu().numpy(), csr.idx.cpu().numpy(), csr.val.cpu().numpy())

    @property
    def rows(self):
        return self.off.size - 1

    def args(self):
        return [_p(self.off, np.uint32), _p(self.idx, np.uint32), _p(self.val, np.float32)]


def f2h(x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f2h(_p(x, np.float32), _p(out, np.uint16), C.c_size_t(x.size))
    return out


def h2f(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().orc_h2f(_p(x, np.uint16), _p(out, np.float32), C.c_size_t(x.size))
    return out


def effective_weights(dense, sparse: CsrNp, bm25: CsrNp, qdense, qsparse: CsrNp, qbm25: CsrNp, w_sparse, w_bm25,
                      w_dense):
    dense, qdense = _f32(dense), _f32(qdense)
    ws, wb, wd = C.c_float(w_sparse), C.c_float(w_bm25), C.c_float(w_dense)
    lib().orc_effective_weights(C.c_uint32(dense.shape[0]), _p(dense, np.float32), *sparse.args(), *bm25.args(),
                                C.c_uint32(qdense.shape[0]), _p(qdense, np.float32), *qsparse.args(), *qbm25.args(),
                                C.byref(ws), C.byref(wb), C.byref(wd))
    return ws.value, wb.value, wd.value


def scale_queries(qdense, qsparse: CsrNp, qbm25: CsrNp, w_sparse, w_bm25, w_dense):
    """Fold the effective weights into the query in fp32 (src/query.cu:1871-1881)."""
    qd = (_f32(qdense) * np.float32(w_dense)).astype(np.float32)
    qs = CsrNp(qsparse.off, qsparse.idx, (qsparse.val * np.float32(w_sparse)).astype(np.float32))
    qb = CsrNp(qbm25.off, qbm25.idx, (qbm25.val * np.float32(w_bm25)).astype(np.float32))
    return qd, qs, qb


def search(dense_h, sparse: CsrNp, bm25: CsrNp, qdense_h, qsparse: CsrNp, qbm25: CsrNp, graph, ep, cands, flags,
           kg=None, kg_weight=0.0):
    """dense_h / qdense_h: uint16 half bits.  kg: (e2e_off, e2e_idx, e2d_off, e2d_idx, qe_off, qe_idx) or None."""
    dense_h = np.ascontiguousarray(dense_h, dtype=np.uint16)
    qdense_h = np.ascontiguousarray(qdense_h, dtype=np.uint16)
    graph, ep = _u32(graph), _u32(ep)
    n, nq = dense_h.shape[0], qdense_h.shape[0]
    ids = np.empty((nq, cands), dtype=np.uint32)
    dis = np.empty((nq, cands), dtype=np.float32)
    counts = np.zeros((nq, 2), dtype=np.uint64)
    kgp = [None] * 6 if kg is None else [_p(_u32(a), np.uint32) for a in kg]
    keep = kg  # noqa: F841  (keeps converted arrays alive through the call)
    lib().orc_search(C.c_uint32(n), _p(dense_h, np.uint16), *sparse.args(), *bm25.args(), C.c_uint32(nq),
                     _p(qdense_h, np.uint16), *qsparse.args(), *qbm25.args(), _p(graph, np.uint32),
                     _p(ep, np.uint32), C.c_uint32(cands), C.c_int(flags), *kgp, C.c_float(kg_weight),
                     _p(ids, np.uint32), _p(dis, np.float32), _p(counts, np.uint64))
    return ids, dis, counts


def fused_distances(dense_h, sparse: CsrNp, bm25: CsrNp, qdense_h, qsparse: CsrNp, qbm25: CsrNp, pair_q, pair_d,
                    flags):
    dense_h = np.ascontiguousarray(dense_h, dtype=np.uint16)
    qdense_h = np.ascontiguousarray(qdense_h, dtype=np.uint16)
    pair_q, pair_d = _u32(pair_q), _u32(pair_d)
    out = np.empty(pair_q.size, dtype=np.float32)
    lib().orc_fused_distances(C.c_uint32(dense_h.shape[0]), _p(dense_h, np.uint16), *sparse.args(), *bm25.args(),
                              C.c_uint32(qdense_h.shape[0]), _p(qdense_h, np.uint16), *qsparse.args(),
                              *qbm25.args(), C.c_size_t(pair_q.size), _p(pair_q, np.uint32), _p(pair_d, np.uint32),
                              C.c_int(flags), _p(out, np.float32))
    return out


def bruteforce(dense, sparse: CsrNp, bm25: CsrNp, qdense, qsparse: CsrNp, qbm25: CsrNp, flags, topk):
    """Exact fp32 hybrid top-k; queries already weight-scaled.  Returns ids, dis, threads."""
    dense, qdense = _f32(dense), _f32(qdense)
    nq = qdense.shape[0]
    ids = np.empty((nq, topk), dtype=np.uint32)
    dis = np.empty((nq, topk), dtype=np.float32)
    thr = C.c_int(0)
    lib().orc_bruteforce(C.c_uint32(dense.shape[0]), _p(dense, np.float32), *sparse.args(), *bm25.args(),
                         C.c_uint32(nq), _p(qdense, np.float32), *qsparse.args(), *qbm25.args(), C.c_int(flags),
                         C.c_uint32(topk), _p(ids, np.uint32), _p(dis, np.float32), C.byref(thr))
    return ids, dis, thr.value


def cal_power(dense_h, sparse: CsrNp, bm25: CsrNp):
    dense_h = np.ascontiguousarray(dense_h, dtype=np.uint16)
    out = np.empty(dense_h.shape[0], dtype=np.float32)
    lib().orc_cal_power(C.c_uint32(dense_h.shape[0]), _p(dense_h, np.uint16), _p(sparse.off, np.uint32),
                        _p(sparse.val, np.float32), _p(bm25.off, np.uint32), _p(bm25.val, np.float32),
                        _p(out, np.float32))
    return out


def entry_points(power):
    power = _f32(power)
    ep = np.empty(32, dtype=np.uint32)
    lib().orc_entry_points(C.c_uint32(power.size), _p(power, np.float32), _p(ep, np.uint32))
    return ep


def prune(dense_h, sparse: CsrNp, bm25: CsrNp, knn, knn_dis, power, flags=0):
    """Returns new_list [n,32], kw_edge [n,33], graph [n,40], detour [n,32]."""
    dense_h = np.ascontiguousarray(dense_h, dtype=np.uint16)
    knn, knn_dis, power = _u32(knn), _f32(knn_dis), _f32(power)
    n = dense_h.shape[0]
    new_list = np.empty((n, 32), dtype=np.uint32)
    kw = np.empty((n, 33), dtype=np.uint32)
    graph = np.empty((n, 40), dtype=np.uint32)
    det = np.empty((n, 32), dtype=np.uint32)
    lib().orc_prune(C.c_uint32(n), _p(dense_h, np.uint16), *sparse.args(), *bm25.args(), _p(knn, np.uint32),
                    _p(knn_dis, np.float32), _p(power, np.float32), C.c_int(flags), _p(new_list, np.uint32),
                    _p(kw, np.uint32), _p(graph, np.uint32), _p(det, np.uint32))
    return new_list, kw, graph, det


def cal_precision(results, top_k, qrels) -> float:
    """nDCG@k with the reference's float arithmetic (src/query.cu:111-145); qrels: list of id lists."""
    results = _u32(results)
    off = np.zeros(len(qrels) + 1, dtype=np.uint32)
    off[1:] = np.cumsum([len(r) for r in qrels])
    flat = np.asarray([t for r in qrels for t in r], dtype=np.uint32)
    f = lib().orc_cal_precision
    f.restype = C.c_float
    return float(f(C.c_uint32(results.shape[0]), _p(results, np.uint32), C.c_uint32(results.shape[1]), C.c_uint32(top_k),
                   _p(off, np.uint32), _p(flat, np.uint32)))


def num_threads() -> int:
    return int(lib().orc_num_threads())


# ---------------------------------------------------------------------------------------------------------
# Input preparation (BM25 weighting).  PARITY UNPINNED against the reference: it has no code for this step (it
# expects pre-weighted rows, README.md:73-77); this restates the published Okapi BM25 formula in float32, step by
# step in the order the device code uses, and is pinned only by the hand-computed case in tests/test_prep.py.
# ---------------------------------------------------------------------------------------------------------
def bm25_corpus(off, idx, tf, vocab, k1=1.2, b=0.75, relabel_by_df=False):
    """Returns (idx_out, weight, df, idf, relabel): rows sorted by (renumbered) term id, float32 weights."""
    off = np.asarray(off, dtype=np.int64); idx = np.asarray(idx, dtype=np.int64); tf = np.asarray(tf, dtype=np.float32)
    rows = off.size - 1
    f32 = np.float32
    df = np.bincount(idx, minlength=vocab).astype(np.uint32)
    d = df.astype(np.float32)
    idf = np.log(f32(1.0) + (f32(rows) - d + f32(0.5)) / (d + f32(0.5))).astype(np.float32)
    cnt = np.diff(off)
    row_of = np.repeat(np.arange(rows), cnt)
    length = np.zeros(rows, dtype=np.float64)
    np.add.at(length, row_of, tf.astype(np.float64))
    avglen = f32(length.sum() / rows)
    norm = (f32(k1) * (f32(1.0) - f32(b) + f32(b) * length.astype(np.float32) / avglen)).astype(np.float32)
    w = (idf[idx] * tf * (f32(k1) + f32(1.0)) / (tf + norm[row_of])).astype(np.float32)
    relabel = None
    new_idx = idx
    if relabel_by_df:
        order = np.lexsort((np.arange(vocab), -df.astype(np.int64)))   # descending df, ties by id
        relabel = np.empty(vocab, dtype=np.uint32); relabel[order] = np.arange(vocab, dtype=np.uint32)
        new_idx = relabel[idx].astype(np.int64)
    perm = np.lexsort((new_idx, row_of))
    return new_idx[perm].astype(np.uint32), w[perm], df, idf, relabel


def bm25_queries(off, idx, tf, idf, relabel=None):
    off = np.asarray(off, dtype=np.int64); idx = np.asarray(idx, dtype=np.int64); tf = np.asarray(tf, dtype=np.float32)
    w = (np.asarray(idf, dtype=np.float32)[idx] * tf).astype(np.float32)
    new_idx = np.asarray(relabel)[idx].astype(np.int64) if relabel is not None else idx
    row_of = np.repeat(np.arange(off.size - 1), np.diff(off))
    perm = np.lexsort((new_idx, row_of))
    return new_idx[perm].astype(np.uint32), w[perm]
