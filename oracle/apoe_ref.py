"""ctypes binding of oracle/_ref/libapoe_ref.so: the reference's own CUDA kernels behind a small harness.

TEST / BASELINE INFRASTRUCTURE ONLY.  The library is compiled from the reference tree where it is mounted
(`make -C oracle ref`); on a GPU box only the prebuilt file is used.  It needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def lib_path() -> str:
    return os.path.join(_HERE, "_ref", "libapoe_ref.so")


def available() -> bool:
    return os.path.exists(lib_path())


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(lib_path())
    return _LIB


def _p(a, dt):
    a = np.ascontiguousarray(a)
    if a.dtype == np.int32 and dt == np.uint32:
        a = a.view(np.uint32)
    assert a.dtype == dt, (a.dtype, dt)
    return a, C.c_void_p(a.ctypes.data)


def build(dense, s, b):
    """dense: fp32 [n, 1024] unscaled; s, b: (off, idx, val).  Returns a dict of the reference's build state."""
    keep = []
    def arg(a, dt):
        arr, ptr = _p(a, dt); keep.append(arr); return ptr
    n = dense.shape[0]
    out = dict(knn=np.empty((n, 64), np.uint32), knn_dis=np.empty((n, 64), np.float32), power=np.empty(n, np.float32),
               new_list=np.empty((n, 32), np.uint32), kw=np.empty((n, 33), np.uint32), graph=np.empty((n, 40), np.uint32),
               ep=np.empty(32, np.uint32))
    sec = C.c_double(0)
    rc = lib().ref_build(C.c_uint(n), arg(dense, np.float32), arg(s[0], np.uint32), arg(s[1], np.uint32), arg(s[2], np.float32),
                         arg(b[0], np.uint32), arg(b[1], np.uint32), arg(b[2], np.float32),
                         *[C.c_void_p(out[k].ctypes.data) for k in ("knn", "knn_dis", "power", "new_list", "kw", "graph", "ep")],
                         C.byref(sec))
    if rc != 0:
        raise RuntimeError(f"ref_build failed with {rc}")
    out["seconds"] = sec.value
    return out


def search(dense, s, b, qdense_scaled, qs, qb, graph, ep, cands, mode):
    """Queries already scaled by the effective weights (fp32).  Returns ids, dis, seconds_total, seconds_search."""
    keep = []
    def arg(a, dt):
        arr, ptr = _p(a, dt); keep.append(arr); return ptr
    n, nq = dense.shape[0], qdense_scaled.shape[0]
    ids = np.empty((nq, cands), np.uint32)
    dis = np.empty((nq, cands), np.float32)
    t_all, t_search = C.c_double(0), C.c_double(0)
    rc = lib().ref_search(C.c_uint(n), arg(dense, np.float32), arg(s[0], np.uint32), arg(s[1], np.uint32), arg(s[2], np.float32),
                          arg(b[0], np.uint32), arg(b[1], np.uint32), arg(b[2], np.float32), C.c_uint(nq),
                          arg(qdense_scaled, np.float32), arg(qs[0], np.uint32), arg(qs[1], np.uint32), arg(qs[2], np.float32),
                          arg(qb[0], np.uint32), arg(qb[1], np.uint32), arg(qb[2], np.float32), arg(graph, np.uint32),
                          arg(ep, np.uint32), C.c_uint(cands), C.c_int(mode), C.c_void_p(ids.ctypes.data),
                          C.c_void_p(dis.ctypes.data), C.byref(t_all), C.byref(t_search))
    if rc != 0:
        raise RuntimeError(f"ref_search failed with {rc}")
    return ids, dis, t_all.value, t_search.value


def load_seconds(dense_path: str, sparse_path: str, bm25_path: str):
    """The reference's corpus loaders and uploads on three files.  Returns (rows, load seconds, load + upload seconds)."""
    rows = C.c_uint(0)
    sec = (C.c_double * 2)()
    rc = lib().ref_load(dense_path.encode(), sparse_path.encode(), bm25_path.encode(), C.byref(rows), sec)
    if rc != 0:
        raise RuntimeError(f"ref_load failed with {rc}")
    return rows.value, sec[0], sec[1]


# ---------------------------------------------------------------------------------------------------------
# Host-only calls (no GPU needed): the reference's file readers and its nDCG figure.
# ---------------------------------------------------------------------------------------------------------
def load_graph(path: str):
    """The reference's load_graph (src/query.cu:35-62) on an index.poe file.  Returns (flat rows, entry points)."""
    nw, ne = C.c_uint(0), C.c_uint(0)
    with _quiet():
        lib().ref_load_graph(path.encode(), None, C.c_size_t(0), None, C.c_uint(0), C.byref(nw), C.byref(ne))
    rows, ep = np.empty(nw.value, np.uint32), np.empty(ne.value, np.uint32)
    with _quiet():
        rc = lib().ref_load_graph(path.encode(), C.c_void_p(rows.ctypes.data), C.c_size_t(rows.size), C.c_void_p(ep.ctypes.data),
                                  C.c_uint(ep.size), C.byref(nw), C.byref(ne))
    if rc != 0:
        raise RuntimeError(f"ref_load_graph failed with {rc}")
    return rows, ep


class _quiet:
    """Sends the process's stdout (file descriptor 1: the reference prints with std::cout) to a temporary file for the
    duration of the block; `.text` holds what was printed."""

    def __enter__(self):
        import sys
        import tempfile
        sys.stdout.flush()
        self._tmp = tempfile.TemporaryFile(mode="w+b")
        self._saved = os.dup(1)
        os.dup2(self._tmp.fileno(), 1)
        return self

    def __exit__(self, *exc):
        os.dup2(self._saved, 1)
        os.close(self._saved)
        self._tmp.seek(0)
        self.text = self._tmp.read().decode(errors="replace")
        self._tmp.close()
        return False


def cal_precision_text(results, top_k: int, qrels) -> str:
    """What the reference's cal_precision (src/query.cu:111-145) prints for these results and relevant ids."""
    results = np.ascontiguousarray(results, dtype=np.uint32)
    off = np.zeros(len(qrels) + 1, dtype=np.uint32)
    off[1:] = np.cumsum([len(r) for r in qrels])
    flat = np.asarray([t for r in qrels for t in r], dtype=np.uint32)
    with _quiet() as q:
        lib().ref_cal_precision(C.c_uint(results.shape[0]), C.c_void_p(results.ctypes.data), C.c_uint(results.shape[1]), C.c_uint(top_k),
                                C.c_void_p(off.ctypes.data), C.c_void_p(flat.ctypes.data))
    return q.text.strip()


def load_kg(path: str):
    n_off, nnz = C.c_uint(0), C.c_uint(0)
    with _quiet():
        lib().ref_load_kg(path.encode(), None, C.c_size_t(0), None, C.c_size_t(0), C.byref(n_off), C.byref(nnz))
    off, idx = np.empty(n_off.value, np.uint32), np.empty(nnz.value, np.uint32)
    with _quiet():
        rc = lib().ref_load_kg(path.encode(), C.c_void_p(off.ctypes.data), C.c_size_t(off.size), C.c_void_p(idx.ctypes.data),
                               C.c_size_t(idx.size), C.byref(n_off), C.byref(nnz))
    if rc != 0:
        raise RuntimeError(f"ref_load_kg failed with {rc}")
    return off, idx


def load_txt(path: str, rows: int):
    total = C.c_uint(0)
    off = np.zeros(rows + 1, np.uint32)
    lib().ref_load_txt(path.encode(), C.c_uint(rows), C.c_void_p(off.ctypes.data), None, C.c_size_t(0), C.byref(total))
    ids = np.empty(total.value, np.uint32)
    rc = lib().ref_load_txt(path.encode(), C.c_uint(rows), C.c_void_p(off.ctypes.data), C.c_void_p(ids.ctypes.data), C.c_size_t(ids.size), C.byref(total))
    if rc != 0:
        raise RuntimeError(f"ref_load_txt failed with {rc}")
    return off, ids


def load_fvecs(path: str):
    num, dim = C.c_uint(0), C.c_uint(0)
    lib().ref_load_fvecs(path.encode(), None, C.c_size_t(0), C.byref(num), C.byref(dim))
    out = np.empty((num.value, dim.value), np.float32)
    rc = lib().ref_load_fvecs(path.encode(), C.c_void_p(out.ctypes.data), C.c_size_t(out.size), C.byref(num), C.byref(dim))
    if rc != 0:
        raise RuntimeError(f"ref_load_fvecs failed with {rc}")
    return out


def load_csr(path: str, rows: int):
    nnz = C.c_uint(0)
    with _quiet():
        lib().ref_load_csr(path.encode(), C.c_uint(rows), None, None, None, C.c_size_t(0), C.byref(nnz))
    off, idx, val = np.empty(rows + 1, np.uint32), np.empty(nnz.value, np.uint32), np.empty(nnz.value, np.float32)
    with _quiet():
        rc = lib().ref_load_csr(path.encode(), C.c_uint(rows), C.c_void_p(off.ctypes.data), C.c_void_p(idx.ctypes.data),
                                C.c_void_p(val.ctypes.data), C.c_size_t(nnz.value), C.byref(nnz))
    if rc != 0:
        raise RuntimeError(f"ref_load_csr failed with {rc}")
    return off, idx, val


class Resident:
    """The reference's search kernels over a corpus that stays on the device (see ref_open in ref_harness_query.cu):
    uploads and converts the corpus once, then searches any number of query batches, optionally over several graphs."""

    def __init__(self, dense, s, b, graph, ep):
        self._keep = []
        def arg(a, dt):
            arr, ptr = _p(a, dt); self._keep.append(arr); return ptr
        sec = C.c_double(0)
        f = lib().ref_open
        f.restype = C.c_void_p
        self.n = dense.shape[0]
        self._h = f(C.c_uint(self.n), arg(dense, np.float32), arg(s[0], np.uint32), arg(s[1], np.uint32), arg(s[2], np.float32),
                    arg(b[0], np.uint32), arg(b[1], np.uint32), arg(b[2], np.float32), arg(graph, np.uint32), arg(ep, np.uint32), C.byref(sec))
        self._keep = []
        if not self._h:
            raise RuntimeError("ref_open failed")
        self.seconds_corpus_f2h = sec.value

    def set_graph(self, graph, ep):
        g, gp = _p(graph, np.uint32)
        e, epp = _p(ep, np.uint32)
        if lib().ref_set_graph(C.c_void_p(self._h), gp, epp) != 0:
            raise RuntimeError("ref_set_graph failed")

    def search(self, qdense_scaled, qs, qb, cands, mode):
        """Queries already scaled by the effective weights.  Returns ids, dis, seconds (query f2h + search kernel)."""
        keep = []
        def arg(a, dt):
            arr, ptr = _p(a, dt); keep.append(arr); return ptr
        nq = qdense_scaled.shape[0]
        ids, dis = np.empty((nq, cands), np.uint32), np.empty((nq, cands), np.float32)
        sec = C.c_double(0)
        rc = lib().ref_search_resident(C.c_void_p(self._h), C.c_uint(nq), arg(qdense_scaled, np.float32), arg(qs[0], np.uint32), arg(qs[1], np.uint32),
                                       arg(qs[2], np.float32), arg(qb[0], np.uint32), arg(qb[1], np.uint32), arg(qb[2], np.float32), C.c_uint(cands),
                                       C.c_int(mode), C.c_void_p(ids.ctypes.data), C.c_void_p(dis.ctypes.data), C.byref(sec))
        if rc != 0:
            raise RuntimeError(f"ref_search_resident failed with {rc}")
        return ids, dis, sec.value

    def close(self):
        if self._h:
            lib().ref_close(C.c_void_p(self._h))
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
