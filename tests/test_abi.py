"""The C-ABI library loads and exports every symbol the public header declares (no GPU needed)."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    import build as apoe_build   # allan-poe_b200/build.py
    return apoe_build.build()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "allan_poe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ap_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_drop_in_calls():
    syms = declared_symbols()
    for must in ("ap_build_index", "ap_search_index", "ap_index_create_host", "ap_search_host", "ap_search_device",
                 "ap_last_error", "ap_index_build", "ap_index_prune", "ap_merge_shard_results"):
        assert must in syms


def test_library_exports_every_declared_symbol(built):
    lib = ctypes.CDLL(built)
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing
    assert lib.ap_version() >= 100


def test_python_module_keeps_reference_signature(built):
    import importlib
    import build as apoe_build
    import sys
    sys.path.insert(0, os.path.dirname(apoe_build.module_path()))
    hs = importlib.import_module("hybrid_search")
    doc_b, doc_s = hs.build_index.__doc__, hs.search_index.__doc__
    for kw in ("dense_data_path", "sparse_data_path", "bm25_data_path", "output_graph_path"):
        assert kw in doc_b
    order = ["dense_data_path", "dense_query_path", "sparse_data_path", "sparse_query_path", "bm25_data_path",
             "bm25_query_path", "keyword_id_path", "knowledge_path", "entity2doc_path", "query_entity_path", "graph_path",
             "ground_truth_path", "top_k", "cands", "sparse_weight", "bm25_weight", "dense_weight", "kg_weight"]
    pos = [doc_s.index(k + ":") for k in order]
    assert pos == sorted(pos)


def test_errors_are_reported_not_fatal(built):
    """A missing file comes back as a status + message; the reference would exit(-1) (include/utils.cuh:344)."""
    import apoe
    with pytest.raises(apoe.ApoeError) as e:
        apoe.build_index("/nonexistent/a.fvecs", "/nonexistent/b.bin", "/nonexistent/c.bin", "/tmp/x.poe")
    assert e.value.code == 2 and "cannot open" in str(e.value)
    import numpy as np
    assert apoe.ndcg(np.array([[1, 2, 3]], dtype=np.uint32), 3, [[2, 9]]) > 0.0


def test_corpus_files_are_validated_before_any_device_work(built, tmp_path):
    """The streamed ingest reads headers and row offsets first: malformed files are refused with a message even where
    no GPU is present (what it checks: the dimension word, the CSR sizes against the row count, the last offset)."""
    import numpy as np
    import apoe
    p = lambda s: str(tmp_path / s)
    n = 5
    rows = np.zeros((n, 1025), dtype=np.float32)
    rows.view(np.uint32)[:, 0] = 1024
    rows.tofile(p("d.fvecs"))
    def csr(path, off, nnz_header=None):
        off = np.asarray(off, dtype=np.uint32)
        nnz = int(off[-1]) if nnz_header is None else nnz_header
        with open(path, "wb") as f:
            np.array([nnz], dtype=np.uint32).tofile(f); off.tofile(f)
            np.arange(int(off[-1]), dtype=np.uint32).tofile(f); np.ones(int(off[-1]), dtype=np.float32).tofile(f)
    csr(p("ok.bin"), [0, 1, 2, 3, 4, 5])
    bad = rows.copy(); bad.view(np.uint32)[0, 0] = 768; bad.tofile(p("dim.fvecs"))
    with pytest.raises(apoe.ApoeError, match="dimension 768"):
        apoe.Index.from_files(p("dim.fvecs"), p("ok.bin"), p("ok.bin"))
    csr(p("short.bin"), [0, 1, 2])            # offsets of 2 rows only
    with pytest.raises(apoe.ApoeError, match="needed for 5 rows"):
        apoe.Index.from_files(p("d.fvecs"), p("short.bin"), p("ok.bin"))
    csr(p("lying.bin"), [0, 1, 2, 3, 4, 5], nnz_header=4)   # header says 4 entries, the offsets end at 5
    with pytest.raises(apoe.ApoeError, match="last offset 5 differs from the entry count 4"):
        apoe.Index.from_files(p("d.fvecs"), p("ok.bin"), p("lying.bin"))
    with pytest.raises(apoe.ApoeError, match="cannot open"):
        apoe.Index.from_files(p("d.fvecs"), p("ok.bin"), p("missing.bin"))
