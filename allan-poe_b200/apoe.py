"""Python host layer over the C ABI of libapoe.so (ctypes; torch only supplies device memory and streams).

`Index` is the resident index: corpus packed in device memory, graph built on the device or loaded from an
index.poe file, queries searched in batches.  There is no CPU fallback: importing works without a GPU, every
compute call needs the CUDA library and a device and raises `ApoeError` otherwise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

AP_OK = 0
CREATE_FOR_BUILD = 1
BUILD_SIMT_JOIN, BUILD_KEEP_KNN, BUILD_RANDOM_START, BUILD_SHARED_PAIRS, BUILD_REVERSE_PASS = 1, 2, 4, 8, 16
BUILD_PRUNE_STEPWISE, BUILD_TRACE, BUILD_DETERMINISTIC, BUILD_WIPE_TABLES = 32, 64, 128, 256
SEARCH_KEYWORD, SEARCH_KG, SEARCH_RAW_WEIGHTS, SEARCH_UNFUSED_DENSE = 1, 2, 4, 8
DIM, ROW, DEGREE, KNN, ENTRY_POINTS = 1024, 40, 32, 64, 32


class ApoeError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code


class _Csr(C.Structure):
    _fields_ = [("off", C.c_void_p), ("idx", C.c_void_p), ("val", C.c_void_p)]


class BuildOpts(C.Structure):
    _fields_ = [("iterations", C.c_uint32), ("seed", C.c_uint32), ("flags", C.c_uint32), ("dense_scale", C.c_float),
                ("proposals", C.c_uint32), ("seed_take", C.c_uint32), ("reserved", C.c_uint32 * 2)]


class BuildStats(C.Structure):
    _fields_ = [("seconds_total", C.c_double), ("seconds_knn", C.c_double), ("seconds_prune", C.c_double),
                ("distance_evals", C.c_uint64), ("list_updates", C.c_uint64), ("iterations_run", C.c_uint32),
                ("launches", C.c_uint32), ("proposal_overflows", C.c_uint32), ("phase_10us", C.c_uint32 * 3), ("reserved0", C.c_uint32),
                ("rows_gathered", C.c_uint64)]


class IngestStats(C.Structure):
    _fields_ = [("seconds_total", C.c_double), ("seconds_open", C.c_double), ("bytes_read", C.c_uint64),
                ("rows", C.c_uint32), ("threads", C.c_uint32), ("nnz_sparse", C.c_uint32), ("nnz_bm25", C.c_uint32),
                ("reserved", C.c_uint32 * 2)]


class Bm25Opts(C.Structure):
    _fields_ = [("k1", C.c_float), ("b", C.c_float), ("flags", C.c_uint32), ("reserved", C.c_uint32 * 5)]


class PrepStats(C.Structure):
    _fields_ = [("seconds", C.c_double), ("kernel_ms", C.c_float), ("avg_len", C.c_float), ("nnz", C.c_uint64),
                ("rows_sorted", C.c_uint32), ("launches", C.c_uint32), ("reserved", C.c_uint32 * 2)]


class SearchOpts(C.Structure):
    _fields_ = [("cands", C.c_uint32), ("flags", C.c_uint32), ("sparse_weight", C.c_float), ("bm25_weight", C.c_float),
                ("dense_weight", C.c_float), ("kg_weight", C.c_float), ("arena_bytes", C.c_uint32),
                ("ctas_per_sm", C.c_uint32), ("reserved", C.c_uint32 * 4)]


class Queries(C.Structure):
    _fields_ = [("nq", C.c_uint32), ("dense", C.c_void_p), ("sparse", _Csr), ("bm25", _Csr), ("ent_off", C.c_void_p),
                ("ent_idx", C.c_void_p), ("max_sparse_nnz", C.c_uint32), ("max_bm25_nnz", C.c_uint32)]


class ExactStats(C.Structure):
    _fields_ = [("seconds_total", C.c_double), ("seconds_index", C.c_double), ("sparse_ms", C.c_float), ("dense_ms", C.c_float),
                ("dense_flops", C.c_uint64), ("postings", C.c_uint64), ("batch_queries", C.c_uint32), ("slices", C.c_uint32),
                ("reserved", C.c_uint32 * 2)]


class SearchStats(C.Structure):
    _fields_ = [("eff_sparse", C.c_float), ("eff_bm25", C.c_float), ("eff_dense", C.c_float), ("path", C.c_uint32),
                ("kernel_ms", C.c_double), ("total_ms", C.c_double), ("expansions", C.c_uint64),
                ("evaluations", C.c_uint64), ("gathered_bytes", C.c_uint64), ("launches", C.c_uint32),
                ("h2d_bytes_lo", C.c_uint32), ("h2d_bytes_hi", C.c_uint32), ("d2h_bytes_lo", C.c_uint32),
                ("d2h_bytes_hi", C.c_uint32), ("reserved", C.c_uint32 * 3)]


def lib_path() -> str:
    return os.path.join(_HERE, "lib", "libapoe.so")


def lib() -> C.CDLL:
    """The CUDA library.  Raises if it has not been built: there is no other implementation to fall back to."""
    global _LIB
    if _LIB is None:
        p = lib_path()
        if not os.path.exists(p):
            raise ApoeError(-1, f"{p} is missing: run `python allan-poe_b200/build.py` (nvcc, sm_100a)")
        L = C.CDLL(p)
        L.ap_last_error.restype = C.c_char_p
        L.ap_ndcg.restype = C.c_double
        L.ap_index_size.restype = C.c_uint32
        _LIB = L
    return _LIB


def _check(rc: int) -> None:
    if rc != AP_OK:
        raise ApoeError(rc, lib().ap_last_error().decode(errors="replace"))


def _np(a, dtype):
    a = np.ascontiguousarray(a)
    if a.dtype == np.int32 and dtype == np.uint32:
        a = a.view(np.uint32)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


def _ptr(a) -> C.c_void_p:
    if a is None:
        return C.c_void_p(None)
    if isinstance(a, np.ndarray):
        return C.c_void_p(a.ctypes.data)
    return C.c_void_p(a.data_ptr())  # torch tensor


def _csr_np(csr):
    """(off, idx, val) in any of: tuple of arrays, object with .off/.idx/.val (numpy or CPU torch)."""
    off, idx, val = (csr.off, csr.idx, csr.val) if hasattr(csr, "off") else csr
    conv = lambda x: x.cpu().numpy() if hasattr(x, "cpu") else np.asarray(x)
    return _np(conv(off), np.uint32), _np(conv(idx), np.uint32), _np(conv(val), np.float32)


PREP_RELABEL_BY_DF = 1


def bm25_corpus(off, idx, tf, vocab: int, k1: float = 1.2, b: float = 0.75, relabel_by_df: bool = False, device: int = 0):
    """BM25 weights of a corpus from raw term frequencies (host arrays).  Returns (idx, weight, df, idf, relabel, stats)."""
    off, tf = _np(off, np.uint32), _np(tf, np.float32)
    idx = _np(idx, np.uint32).copy()
    rows = off.size - 1
    w = np.empty(idx.size, dtype=np.float32)
    df, idf = np.empty(vocab, dtype=np.uint32), np.empty(vocab, dtype=np.float32)
    rl = np.empty(vocab, dtype=np.uint32) if relabel_by_df else None
    o = Bm25Opts(k1=k1, b=b, flags=PREP_RELABEL_BY_DF if relabel_by_df else 0)
    st = PrepStats()
    _check(lib().ap_bm25_corpus_host(C.c_int(device), C.c_uint32(rows), C.c_uint32(vocab), _ptr(off), _ptr(idx), _ptr(tf), _ptr(w),
                                     _ptr(df), _ptr(idf), _ptr(rl) if rl is not None else None, C.byref(o), C.byref(st)))
    return idx, w, df, idf, rl, st


def bm25_queries(off, idx, tf, idf, relabel=None, device: int = 0):
    """BM25 query weights (idf x tf), ids renumbered with `relabel` and rows sorted.  Returns (idx, weight, stats)."""
    off, tf, idf = _np(off, np.uint32), _np(tf, np.float32), _np(idf, np.float32)
    idx = _np(idx, np.uint32).copy()
    rl = _np(relabel, np.uint32) if relabel is not None else None
    w = np.empty(idx.size, dtype=np.float32)
    st = PrepStats()
    _check(lib().ap_bm25_queries_host(C.c_int(device), C.c_uint32(off.size - 1), C.c_uint32(idf.size), _ptr(off), _ptr(idx), _ptr(tf),
                                      _ptr(w), _ptr(idf), _ptr(rl) if rl is not None else None, C.byref(st)))
    return idx, w, st


def bm25_corpus_device(off_host, off, idx, tf, weight, df, idf, relabel=None, k1: float = 1.2, b: float = 0.75, stream=None):
    """The same on CUDA tensors, in place (idx is renumbered / reordered, weight / df / idf / relabel are written)."""
    off_host = _np(off_host, np.uint32)
    o = Bm25Opts(k1=k1, b=b, flags=PREP_RELABEL_BY_DF if relabel is not None else 0)
    st = PrepStats()
    _check(lib().ap_bm25_corpus_device(C.c_int(idx.device.index or 0), C.c_uint32(off_host.size - 1), C.c_uint32(df.numel()), _ptr(off_host),
                                       _ptr(off), _ptr(idx), _ptr(tf), _ptr(weight), _ptr(df), _ptr(idf),
                                       _ptr(relabel) if relabel is not None else None, C.byref(o), C.c_void_p(stream or 0), C.byref(st)))
    return st


class Index:
    def __init__(self, handle: C.c_void_p, n: int, device: int):
        self._h, self.n, self.device = handle, n, device
        self._keep = []

    # ---- creation -------------------------------------------------------------------------------------
    @classmethod
    def from_host(cls, dense, sparse, bm25, device: int = 0, for_build: bool = False) -> "Index":
        dense = _np(dense, np.float32)
        s, b = _csr_np(sparse), _csr_np(bm25)
        h = C.c_void_p()
        _check(lib().ap_index_create_host(C.byref(h), C.c_int(device), C.c_uint32(dense.shape[0]), _ptr(dense),
                                          _Csr(*map(_ptr, s)), _Csr(*map(_ptr, b)),
                                          C.c_uint32(CREATE_FOR_BUILD if for_build else 0)))
        return cls(h, dense.shape[0], device)

    @classmethod
    def from_files(cls, dense_path: str, sparse_path: str, bm25_path: str, device: int = 0, for_build: bool = False,
                   threads: int = 0):
        """Streams the reference's corpus files into a resident index.  Returns (index, IngestStats)."""
        h = C.c_void_p()
        st = IngestStats()
        _check(lib().ap_index_create_files(C.byref(h), C.c_int(device), dense_path.encode(), sparse_path.encode(),
                                           bm25_path.encode(), C.c_uint32(CREATE_FOR_BUILD if for_build else 0),
                                           C.c_uint32(threads), C.byref(st)))
        return cls(h, int(st.rows), device), st

    @classmethod
    def from_files_range(cls, dense_path: str, sparse_path: str, bm25_path: str, row_start: int, row_count: int, device: int = 0,
                         for_build: bool = False, threads: int = 0):
        """Documents [row_start, row_start + row_count) of the corpus files only (a shard; local ids start at 0)."""
        h = C.c_void_p()
        st = IngestStats()
        _check(lib().ap_index_create_files_range(C.byref(h), C.c_int(device), dense_path.encode(), sparse_path.encode(), bm25_path.encode(),
                                                 C.c_uint32(row_start), C.c_uint32(row_count), C.c_uint32(CREATE_FOR_BUILD if for_build else 0),
                                                 C.c_uint32(threads), C.byref(st)))
        return cls(h, int(st.rows), device), st

    @classmethod
    def from_device(cls, dense, sparse, bm25, for_build: bool = False) -> "Index":
        """dense: CUDA float32 [n, 1024]; sparse / bm25: objects with CUDA int32 .off/.idx and float32 .val."""
        assert dense.is_cuda and dense.is_contiguous()
        device = dense.device.index or 0
        h = C.c_void_p()
        _check(lib().ap_index_create_device(C.byref(h), C.c_int(device), C.c_uint32(dense.shape[0]), _ptr(dense),
                                            _Csr(_ptr(sparse.off), _ptr(sparse.idx), _ptr(sparse.val)),
                                            _Csr(_ptr(bm25.off), _ptr(bm25.idx), _ptr(bm25.val)),
                                            C.c_uint32(CREATE_FOR_BUILD if for_build else 0)))
        ix = cls(h, dense.shape[0], device)
        if for_build:
            ix._keep.append(dense)  # the build may re-read the fp32 rows
        return ix

    def close(self) -> None:
        if self._h:
            lib().ap_index_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- graph ---------------------------------------------------------------------------------------
    def set_graph(self, rows, entry_points) -> None:
        rows, ep = _np(rows, np.uint32), _np(entry_points, np.uint32)
        assert rows.shape == (self.n, ROW) and ep.shape == (ENTRY_POINTS,)
        _check(lib().ap_index_set_graph(self._h, _ptr(rows), _ptr(ep)))

    def get_graph(self):
        rows = np.empty((self.n, ROW), dtype=np.uint32)
        ep = np.empty(ENTRY_POINTS, dtype=np.uint32)
        _check(lib().ap_index_get_graph(self._h, _ptr(rows), _ptr(ep)))
        return rows, ep

    def load_graph(self, path: str) -> None:
        _check(lib().ap_index_load_graph(self._h, path.encode()))

    def save_graph(self, path: str) -> None:
        _check(lib().ap_index_save_graph(self._h, path.encode()))

    def build(self, iterations: int = 0, seed: int = 0, flags: int = 0, dense_scale: float = 0.0, proposals: int = 0,
              seed_take: int = 0) -> BuildStats:
        o = BuildOpts(iterations=iterations, seed=seed, flags=flags, dense_scale=dense_scale, proposals=proposals,
                      seed_take=seed_take)
        st = BuildStats()
        _check(lib().ap_index_build(self._h, C.byref(o), C.byref(st)))
        return st

    def get_knn(self):
        ids = np.empty((self.n, KNN), dtype=np.uint32)
        dis = np.empty((self.n, KNN), dtype=np.float32)
        power = np.empty(self.n, dtype=np.float32)
        _check(lib().ap_index_get_knn(self._h, _ptr(ids), _ptr(dis), _ptr(power)))
        return ids, dis, power

    def norms(self) -> np.ndarray:
        out = np.empty(self.n, dtype=np.float32)
        _check(lib().ap_index_norms(self._h, _ptr(out)))
        return out

    def prune(self, knn_ids, knn_dis, power, flags: int = 0):
        knn_ids, knn_dis, power = _np(knn_ids, np.uint32), _np(knn_dis, np.float32), _np(power, np.float32)
        new_list = np.empty((self.n, DEGREE), dtype=np.uint32)
        kw = np.empty((self.n, 33), dtype=np.uint32)
        rows = np.empty((self.n, ROW), dtype=np.uint32)
        _check(lib().ap_index_prune(self._h, _ptr(knn_ids), _ptr(knn_dis), _ptr(power), C.c_uint32(flags), _ptr(new_list),
                                    _ptr(kw), _ptr(rows)))
        return new_list, kw, rows

    def set_kg(self, e2e_off, e2e_idx, e2d_off, e2d_idx) -> None:
        conv = lambda x: _np(x.cpu().numpy() if hasattr(x, "cpu") else x, np.uint32)
        a, b, c, d = conv(e2e_off), conv(e2e_idx), conv(e2d_off), conv(e2d_idx)
        _check(lib().ap_index_set_kg(self._h, C.c_uint32(a.size - 1), _ptr(a), _ptr(b), _ptr(c), _ptr(d)))

    def debug_join_dense(self, plist, pcnt, use_tc: bool):
        plist, pcnt = _np(plist, np.uint32), _np(pcnt, np.uint32)
        nodes = plist.shape[0]
        out = np.zeros((nodes, 64, 32), dtype=np.float32)
        _check(lib().ap_debug_join_dense(self._h, C.c_uint32(nodes), _ptr(plist), _ptr(pcnt), C.c_int(int(use_tc)),
                                         _ptr(out)))
        return out

    # ---- search --------------------------------------------------------------------------------------
    @staticmethod
    def _host_queries(qdense, qsparse, qbm25, ent=None):
        qd = _np(qdense, np.float32)
        s, b = _csr_np(qsparse), _csr_np(qbm25)
        q = Queries(nq=qd.shape[0], dense=_ptr(qd), sparse=_Csr(*map(_ptr, s)), bm25=_Csr(*map(_ptr, b)))
        keep = [qd, s, b]
        if ent is not None:
            eo, ei = _np(ent[0], np.uint32), _np(ent[1], np.uint32)
            q.ent_off, q.ent_idx = _ptr(eo), _ptr(ei)
            keep += [eo, ei]
        return q, keep

    def effective_weights(self, qdense, qsparse, qbm25, w_sparse=1.0, w_bm25=1.0, w_dense=1.0):
        q, keep = self._host_queries(qdense, qsparse, qbm25)
        ws, wb, wd = C.c_float(w_sparse), C.c_float(w_bm25), C.c_float(w_dense)
        _check(lib().ap_effective_weights(self._h, C.byref(q), C.byref(ws), C.byref(wb), C.byref(wd)))
        return ws.value, wb.value, wd.value

    def search(self, qdense, qsparse, qbm25, cands=128, weights=(1.0, 1.0, 1.0), kg_weight=0.0, flags=0, ent=None,
               arena_bytes=0, ctas_per_sm=0, out=None):
        """Host buffers in, host results out.  weights = (sparse, bm25, dense).  Returns ids, dis, SearchStats."""
        q, keep = self._host_queries(qdense, qsparse, qbm25, ent)
        o = SearchOpts(cands=cands, flags=flags, sparse_weight=weights[0], bm25_weight=weights[1],
                       dense_weight=weights[2], kg_weight=kg_weight, arena_bytes=arena_bytes, ctas_per_sm=ctas_per_sm)
        if out is None:
            ids = np.empty((q.nq, cands), dtype=np.uint32)
            dis = np.empty((q.nq, cands), dtype=np.float32)
        else:
            ids, dis = out
        st = SearchStats()
        _check(lib().ap_search_host(self._h, C.byref(q), C.byref(o), _ptr(ids), _ptr(dis), C.byref(st)))
        return ids, dis, st

    def search_static(self, qdense, qsparse, qbm25, cands=128, weights=(1.0, 1.0, 1.0), kg_weight=0.0, flags=0, ent=None):
        """`search` for callers that must not allocate device memory: the batch is staged in the library's fixed
        device array (8 MiB per GPU) and the call makes no allocation; batches that do not fit raise ApoeError(4)."""
        q, keep = self._host_queries(qdense, qsparse, qbm25, ent)
        o = SearchOpts(cands=cands, flags=flags, sparse_weight=weights[0], bm25_weight=weights[1],
                       dense_weight=weights[2], kg_weight=kg_weight)
        ids = np.empty((q.nq, cands), dtype=np.uint32)
        dis = np.empty((q.nq, cands), dtype=np.float32)
        st = SearchStats()
        _check(lib().ap_search_host_static(self._h, C.byref(q), C.byref(o), _ptr(ids), _ptr(dis), C.byref(st)))
        return ids, dis, st

    def search_shard_device(self, queries, out_keys, id_base: int, top_k: int = 10, cands=128, weights=(1.0, 1.0, 1.0), flags=0,
                            max_nnz=(0, 0), stream=None, stats=False, out_ids=None, out_dis=None):
        """This shard's part of a corpus-sharded search on device tensors: out_keys (int64 [nq, top_k]) receives the
        best top_k results of every query as (ordered distance << 32 | local id + id_base) words, written by the
        search kernel itself.  The weights must be the ones every shard uses."""
        q = Queries(nq=queries.dense.shape[0], dense=_ptr(queries.dense),
                    sparse=_Csr(_ptr(queries.sparse.off), _ptr(queries.sparse.idx), _ptr(queries.sparse.val)),
                    bm25=_Csr(_ptr(queries.bm25.off), _ptr(queries.bm25.idx), _ptr(queries.bm25.val)),
                    max_sparse_nnz=max_nnz[0], max_bm25_nnz=max_nnz[1])
        o = SearchOpts(cands=cands, flags=flags | SEARCH_RAW_WEIGHTS, sparse_weight=weights[0], bm25_weight=weights[1],
                       dense_weight=weights[2])
        st = SearchStats()
        _check(lib().ap_search_shard_device(self._h, C.byref(q), C.byref(o), C.c_uint32(id_base), C.c_uint32(top_k), _ptr(out_keys),
                                            _ptr(out_ids), _ptr(out_dis), C.c_void_p(stream or 0), C.byref(st) if stats else None))
        return st

    def search_shard(self, qdense, qsparse, qbm25, id_base: int, top_k: int = 10, cands=128, weights=(1.0, 1.0, 1.0), flags=0):
        """Host buffers in, exchange keys out (uint64 [nq, top_k]); weights are used as given."""
        q, keep = self._host_queries(qdense, qsparse, qbm25)
        o = SearchOpts(cands=cands, flags=flags | SEARCH_RAW_WEIGHTS, sparse_weight=weights[0], bm25_weight=weights[1], dense_weight=weights[2])
        keys = np.empty((q.nq, top_k), dtype=np.uint64)
        ids = np.empty((q.nq, cands), dtype=np.uint32)
        dis = np.empty((q.nq, cands), dtype=np.float32)
        st = SearchStats()
        _check(lib().ap_search_shard_host(self._h, C.byref(q), C.byref(o), C.c_uint32(id_base), C.c_uint32(top_k), _ptr(keys), _ptr(ids),
                                          _ptr(dis), C.byref(st)))
        return keys, ids, dis, st

    def search_device(self, queries, out_ids, out_dis, cands=128, weights=(1.0, 1.0, 1.0), kg_weight=0.0, flags=0,
                      ent=None, max_nnz=(0, 0), stream=None, stats=True, arena_bytes=0, ctas_per_sm=0):
        """Device tensors in and out (queries: object with CUDA .dense and .sparse/.bm25 CSRs).  The weights are
        used as given: run `effective_weights` on a host copy of the first 100 queries for the normalised ones."""
        q = Queries(nq=queries.dense.shape[0], dense=_ptr(queries.dense),
                    sparse=_Csr(_ptr(queries.sparse.off), _ptr(queries.sparse.idx), _ptr(queries.sparse.val)),
                    bm25=_Csr(_ptr(queries.bm25.off), _ptr(queries.bm25.idx), _ptr(queries.bm25.val)),
                    max_sparse_nnz=max_nnz[0], max_bm25_nnz=max_nnz[1])
        if ent is not None:
            q.ent_off, q.ent_idx = _ptr(ent[0]), _ptr(ent[1])
        o = SearchOpts(cands=cands, flags=flags | SEARCH_RAW_WEIGHTS, sparse_weight=weights[0], bm25_weight=weights[1],
                       dense_weight=weights[2], kg_weight=kg_weight, arena_bytes=arena_bytes, ctas_per_sm=ctas_per_sm)
        st = SearchStats()
        _check(lib().ap_search_device(self._h, C.byref(q), C.byref(o), _ptr(out_ids), _ptr(out_dis),
                                      C.c_void_p(stream or 0), C.byref(st) if stats else None))
        return st

    def exact_topk(self, queries, weights, top_k: int = 10, stream=None, keyword: bool = False):
        """Exact top-k of the fused score over all documents (ground truth), on device tensors.  queries: object with
        CUDA .dense and .sparse/.bm25 CSRs; weights = (sparse, bm25, dense), used as given.  Returns (ids int32
        [nq, top_k], distances float32 [nq, top_k], ExactStats) as CUDA tensors.  keyword: only documents holding one of
        the query's required BM25 terms (bit 31) are eligible."""
        import torch
        nq = queries.dense.shape[0]
        q = Queries(nq=nq, dense=_ptr(queries.dense),
                    sparse=_Csr(_ptr(queries.sparse.off), _ptr(queries.sparse.idx), _ptr(queries.sparse.val)),
                    bm25=_Csr(_ptr(queries.bm25.off), _ptr(queries.bm25.idx), _ptr(queries.bm25.val)))
        ids = torch.empty(nq, top_k, dtype=torch.int32, device=queries.dense.device)
        dis = torch.empty(nq, top_k, dtype=torch.float32, device=queries.dense.device)
        st = ExactStats()
        _check(lib().ap_exact_topk_device(self._h, C.byref(q), C.c_float(weights[0]), C.c_float(weights[1]), C.c_float(weights[2]),
                                          C.c_uint32(1 if keyword else 0), C.c_uint32(top_k), _ptr(ids), _ptr(dis), C.c_void_p(stream or 0),
                                          C.byref(st)))
        return ids, dis, st

    def exact_release(self) -> None:
        _check(lib().ap_exact_release(self._h))

    def check_status(self) -> None:
        """Raises ApoeError(6) when a kernel of an earlier asynchronous call raised its error word."""
        _check(lib().ap_index_check_status(self._h))

    def debug_wait_timeout(self, polls: int = 64) -> None:
        _check(lib().ap_debug_wait_timeout(self._h, C.c_uint32(polls)))

    def debug_gather_probe(self, batches: int = 0):
        """(GB/s, ms, bytes) of the fetch-only probe: random whole records into shared memory with the search kernel's footprint."""
        g, ms, b = C.c_double(0), C.c_double(0), C.c_ulonglong(0)
        _check(lib().ap_debug_gather_probe(self._h, C.c_uint32(batches), C.byref(g), C.byref(ms), C.byref(b)))
        return g.value, ms.value, b.value

    def debug_counters(self):
        out = np.zeros(8, dtype=np.uint64)
        _check(lib().ap_debug_counters(self._h, _ptr(out)))
        return out

    def fused_distances(self, qdense, qsparse, qbm25, pair_q, pair_d, weights=(1.0, 1.0, 1.0), flags=0):
        q, keep = self._host_queries(qdense, qsparse, qbm25)
        pq, pd = _np(pair_q, np.uint32), _np(pair_d, np.uint32)
        o = SearchOpts(cands=32, flags=flags, sparse_weight=weights[0], bm25_weight=weights[1], dense_weight=weights[2])
        out = np.empty(pq.size, dtype=np.float32)
        _check(lib().ap_fused_distances(self._h, C.byref(q), C.byref(o), C.c_size_t(pq.size), _ptr(pq), _ptr(pd),
                                        _ptr(out)))
        return out


def build_index(dense_path, sparse_path, bm25_path, out_path, device=0, iterations=0, seed=0, flags=0) -> BuildStats:
    o = BuildOpts(iterations=iterations, seed=seed, flags=flags)
    st = BuildStats()
    _check(lib().ap_build_index(dense_path.encode(), sparse_path.encode(), bm25_path.encode(), out_path.encode(),
                                C.c_int(device), C.byref(o), C.byref(st)))
    return st


def search_index(dense_data_path, dense_query_path, sparse_data_path, sparse_query_path, bm25_data_path,
                 bm25_query_path, keyword_id_path, knowledge_path, entity2doc_path, query_entity_path, graph_path,
                 ground_truth_path, top_k, cands, sparse_weight, bm25_weight, dense_weight, kg_weight, device=0,
                 max_queries=0, nq_hint=None):
    """File-level search with the results returned (the reference prints nDCG and returns nothing)."""
    import numpy as _n
    nq_cap = nq_hint if nq_hint is not None else (os.path.getsize(dense_query_path) // ((DIM + 1) * 4))
    ids = _n.empty((nq_cap, cands), dtype=_n.uint32)
    dis = _n.empty((nq_cap, cands), dtype=_n.float32)
    nq, ndcg, st = C.c_uint32(0), C.c_double(-1.0), SearchStats()
    e = lambda s: (s or "").encode()
    _check(lib().ap_search_index(e(dense_data_path), e(dense_query_path), e(sparse_data_path), e(sparse_query_path),
                                 e(bm25_data_path), e(bm25_query_path), e(keyword_id_path), e(knowledge_path),
                                 e(entity2doc_path), e(query_entity_path), e(graph_path), e(ground_truth_path),
                                 C.c_int(top_k), C.c_int(cands), C.c_float(sparse_weight), C.c_float(bm25_weight),
                                 C.c_float(dense_weight), C.c_float(kg_weight), C.c_int(device),
                                 C.c_uint32(max_queries), _ptr(ids), _ptr(dis), C.byref(nq), C.byref(ndcg), C.byref(st)))
    return ids[:nq.value], dis[:nq.value], ndcg.value, st


def read_fvecs(path: str) -> np.ndarray:
    rows = C.c_uint32(0)
    _check(lib().ap_file_read_fvecs(path.encode(), C.byref(rows), None, C.c_size_t(0)))
    out = np.empty((rows.value, DIM), dtype=np.float32)
    _check(lib().ap_file_read_fvecs(path.encode(), C.byref(rows), _ptr(out), C.c_size_t(out.shape[0])))
    return out


def read_csr(path: str, rows: int = 0):
    """(off, idx, val) of a CSR .bin file; rows = 0 derives the row count from the file size."""
    r, nnz = C.c_uint32(rows), C.c_uint32(0)
    _check(lib().ap_file_read_csr(path.encode(), C.byref(r), C.byref(nnz), None, None, None))
    off, idx, val = np.empty(r.value + 1, np.uint32), np.empty(nnz.value, np.uint32), np.empty(nnz.value, np.float32)
    _check(lib().ap_file_read_csr(path.encode(), C.byref(r), C.byref(nnz), _ptr(off), _ptr(idx), _ptr(val)))
    return off, idx, val


def read_kg(path: str):
    """(off, idx) of a knowledge-graph CSR file (entities + 1 offsets)."""
    n_off, nnz = C.c_uint32(0), C.c_uint32(0)
    _check(lib().ap_file_read_kg(path.encode(), C.byref(n_off), C.byref(nnz), None, None))
    off, idx = np.empty(n_off.value, np.uint32), np.empty(nnz.value, np.uint32)
    _check(lib().ap_file_read_kg(path.encode(), C.byref(n_off), C.byref(nnz), _ptr(off), _ptr(idx)))
    return off, idx


def read_id_lines(path: str, rows: int):
    """(off, ids): line r of a text file = the ids of row r (keyword files, relevance files)."""
    off, total = np.zeros(rows + 1, np.uint32), C.c_size_t(0)
    _check(lib().ap_file_read_id_lines(path.encode(), C.c_uint32(rows), _ptr(off), None, C.c_size_t(0), C.byref(total)))
    ids = np.empty(total.value, np.uint32)
    _check(lib().ap_file_read_id_lines(path.encode(), C.c_uint32(rows), _ptr(off), _ptr(ids), C.c_size_t(ids.size), C.byref(total)))
    return off, ids


def ndcg(results, top_k, qrels) -> float:
    results = _np(results, np.uint32)
    off = np.zeros(len(qrels) + 1, dtype=np.uint32)
    off[1:] = np.cumsum([len(r) for r in qrels])
    flat = np.asarray([t for r in qrels for t in r], dtype=np.uint32)
    return float(lib().ap_ndcg(C.c_uint32(results.shape[0]), _ptr(results), C.c_uint32(results.shape[1]),
                               C.c_uint32(top_k), _ptr(off), _ptr(flat)))


def shard_range(n: int, shard: int, shards: int):
    a, c = C.c_uint32(0), C.c_uint32(0)
    lib().ap_shard_range(C.c_uint32(n), C.c_uint32(shard), C.c_uint32(shards), C.byref(a), C.byref(c))
    return a.value, c.value


def build_index_shard(dense_path, sparse_path, bm25_path, graph_prefix, shard, shards, device=0, iterations=0, seed=0, flags=0) -> BuildStats:
    """Builds the graph of one corpus shard from its rows of the files and writes <graph_prefix>.<shard>.poe (shard 0
    also writes <graph_prefix>.manifest)."""
    o = BuildOpts(iterations=iterations, seed=seed, flags=flags)
    st = BuildStats()
    _check(lib().ap_build_index_shard(dense_path.encode(), sparse_path.encode(), bm25_path.encode(), graph_prefix.encode(),
                                      C.c_uint32(shard), C.c_uint32(shards), C.c_int(device), C.byref(o), C.byref(st)))
    return st


def write_shard_manifest(path, n_docs, shards, graph_prefix) -> None:
    _check(lib().ap_shard_manifest_write(path.encode(), C.c_uint32(n_docs), C.c_uint32(shards), graph_prefix.encode()))


def read_shard_manifest(path):
    """Returns (n_docs, [(first document, documents, graph file name), ...])."""
    n, g = C.c_uint32(0), C.c_uint32(0)
    _check(lib().ap_shard_manifest_read(path.encode(), C.byref(n), C.byref(g), None, None, None, C.c_uint32(0)))
    starts, counts = np.zeros(g.value, np.uint32), np.zeros(g.value, np.uint32)
    names = C.create_string_buffer(g.value * 256)
    _check(lib().ap_shard_manifest_read(path.encode(), C.byref(n), C.byref(g), _ptr(starts), _ptr(counts), names, C.c_uint32(g.value)))
    raw = names.raw
    return n.value, [(int(starts[i]), int(counts[i]), raw[i * 256:(i + 1) * 256].split(b"\0")[0].decode()) for i in range(g.value)]


def search_index_shard(dense_data_path, dense_query_path, sparse_data_path, sparse_query_path, bm25_data_path, bm25_query_path,
                       manifest_path, shard, top_k, cands, sparse_weight, bm25_weight, dense_weight, device=0, max_queries=0):
    """One shard's part of a file-level sharded search: exchange keys (uint64 [nq, top_k]) and the SearchStats."""
    nq_cap = os.path.getsize(dense_query_path) // ((DIM + 1) * 4)
    keys = np.empty((nq_cap, top_k), dtype=np.uint64)
    nq, st = C.c_uint32(0), SearchStats()
    _check(lib().ap_search_index_shard(dense_data_path.encode(), dense_query_path.encode(), sparse_data_path.encode(), sparse_query_path.encode(),
                                       bm25_data_path.encode(), bm25_query_path.encode(), manifest_path.encode(), C.c_uint32(shard),
                                       C.c_int(top_k), C.c_int(cands), C.c_float(sparse_weight), C.c_float(bm25_weight), C.c_float(dense_weight),
                                       C.c_int(device), C.c_uint32(max_queries), _ptr(keys), C.byref(nq), C.byref(st)))
    return keys[:nq.value], st


def merge_shard_keys(keys, top_k, out_ids, out_dis, stream=None) -> None:
    """keys: CUDA int64 tensor [shards, nq, per_shard] (the receive buffer of the all-gather); out_*: [nq, top_k]."""
    shards, nq, per = keys.shape
    _check(lib().ap_merge_shard_keys(C.c_int(keys.device.index or 0), C.c_uint32(shards), C.c_uint32(nq), C.c_uint32(per), _ptr(keys),
                                     C.c_uint32(top_k), _ptr(out_ids), _ptr(out_dis), C.c_void_p(stream or 0)))


def unpack_shard_keys(keys):
    """Exchange keys (numpy uint64) -> (global ids uint32, fused distances float32); empty slots give (0xFFFFFFFF, 1e6)."""
    keys = np.ascontiguousarray(keys, dtype=np.uint64)
    ids = (keys & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    o = (keys >> np.uint64(32)).astype(np.uint32)
    bits = np.where(o & np.uint32(0x80000000), o & np.uint32(0x7FFFFFFF), ~o)
    dis = bits.astype(np.uint32).view(np.float32).copy()
    empty = keys == np.uint64(0xFFFFFFFFFFFFFFFF)
    dis[empty] = np.float32(1e6)
    return ids, dis


def merge_shard_results(in_ids, in_dis, top_k, out_ids, out_dis, stream=None) -> None:
    """in_*: CUDA tensors [shards, nq, per_shard] (ids already global); out_*: [nq, top_k]."""
    shards, nq, per = in_ids.shape
    _check(lib().ap_merge_shard_results(C.c_int(in_ids.device.index or 0), C.c_uint32(shards), C.c_uint32(nq),
                                        C.c_uint32(per), _ptr(in_ids), _ptr(in_dis), C.c_uint32(top_k), _ptr(out_ids),
                                        _ptr(out_dis), C.c_void_p(stream or 0)))
