"""Streamed ingest (threaded pread -> pinned staging -> upload + pack) against the in-memory creation path."""
import os

import numpy as np
import pytest

import apoe
import helpers
import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def files(tiny, tmp_path_factory):
    d = tmp_path_factory.mktemp("corpus")
    p = lambda s: str(d / s)
    synth.write_fvecs(p("d.fvecs"), tiny.corpus.dense)
    synth.write_csr(p("s.bin"), tiny.corpus.sparse)
    synth.write_csr(p("b.bin"), tiny.corpus.bm25)
    return p


@pytest.mark.parametrize("threads", [1, 5])
def test_files_give_the_same_index_as_memory(tiny, files, threads):
    """Same records in HBM: norms, effective weights and every search result are bit-identical."""
    ix_f, st = apoe.Index.from_files(files("d.fvecs"), files("s.bin"), files("b.bin"), for_build=True, threads=threads)
    ix_m = apoe.Index.from_host(tiny.D, tiny.S, tiny.B, for_build=True)
    assert st.rows == tiny.n and st.threads == threads
    want_bytes = os.path.getsize(files("d.fvecs")) + os.path.getsize(files("s.bin")) + os.path.getsize(files("b.bin"))
    assert want_bytes - 8 <= st.bytes_read <= want_bytes + 2 * 101 * 4100 + (1 << 20)   # the first 100 rows are read twice
    assert np.array_equal(ix_f.norms().view(np.uint32), ix_m.norms().view(np.uint32))
    for ix in (ix_f, ix_m):
        ix.set_graph(tiny.graph, tiny.ep)
    a = ix_f.search(tiny.QD, tiny.QS, tiny.QB, cands=128)
    b = ix_m.search(tiny.QD, tiny.QS, tiny.QB, cands=128)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))
    ix_f.close(); ix_m.close()


def test_bad_files_are_refused(tiny, files, tmp_path):
    p = lambda s: str(tmp_path / s)
    with pytest.raises(apoe.ApoeError):
        apoe.Index.from_files(p("missing.fvecs"), files("s.bin"), files("b.bin"))
    # a row whose dimension word is wrong
    raw = np.fromfile(files("d.fvecs"), dtype=np.uint32)
    raw[7 * 1025] = 512
    raw.tofile(p("bad_dim.fvecs"))
    with pytest.raises(apoe.ApoeError, match="dimension word"):
        apoe.Index.from_files(p("bad_dim.fvecs"), files("s.bin"), files("b.bin"))
    # a truncated CSR file
    blob = open(files("s.bin"), "rb").read()
    open(p("short.bin"), "wb").write(blob[: len(blob) // 2])
    with pytest.raises(apoe.ApoeError, match="needed"):
        apoe.Index.from_files(files("d.fvecs"), p("short.bin"), files("b.bin"))
    # a dense file with fewer rows than the CSR files describe
    raw = np.fromfile(files("d.fvecs"), dtype=np.uint32)
    raw[: (tiny.n // 2) * 1025].tofile(p("half.fvecs"))
    with pytest.raises(apoe.ApoeError, match="last offset"):
        apoe.Index.from_files(p("half.fvecs"), files("s.bin"), files("b.bin"))
