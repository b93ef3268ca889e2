#!/usr/bin/env python
"""Benchmark of the hybrid graph index hot path: batched search QPS (cands = 128) and index build seconds.

Own arm (default).  Headline = the 1M-document / 10k-query configuration, weights 1/1/1, cands 128, top_k 10.  A step is
one search pass over the rank's query batch.  `value` is measured with queries and index resident in device memory,
`e2e` through the host-pointer call (pinned host query buffers in, host results out, copies inside the timed region).
On one GPU the same line also carries, measured outside the timed region: recall@10 of all queries against the exact
device scorer (and over several builds), bit-parity of the whole result pool with the reference's own kernel run over
this library's graph, the weight sweep, the cands curve, the keyword-constrained configuration (batch 1 latency through
the host call, batch 65 536 throughput, keyword-edge recycling on / off), the knowledge-graph configuration (200k
documents), the 10k-document configuration, a supplementary corpus with real neighbourhoods (QPS at recall >= 0.95),
the build's roofline figures, file ingest and BM25 preparation.

Reference arm (--impl reference): the reference's own CUDA kernels (oracle/_ref, built from the reference tree where it
is mounted) on the same corpus, queries and batch size.  `value` counts what the own arm's `value` counts -- the search
over a corpus that already lies converted on the device (query conversion + search kernel); the figure with the
reference's own timed region (whole-corpus fp32->fp16 conversion inside, src/query.cu:1999-2051) is reported beside it.

Multi-GPU (torchrun): query-parallel over a replicated index, weak scaling (every rank searches its own batch of the
same size; no collective in the data path).  Every N > 1 line also carries a `sharded` object: the same 1M documents
split N ways, every query on every shard, one NCCL all-gather of packed top-10 keys and one merge kernel per step,
checked against the torch merge and the exact scorer.  --mode sharded makes the corpus-sharded search the headline
(the 10M-document configuration: --docs 10000000 --queries 100000).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "allan-poe_b200"))

import numpy as np  # noqa: E402
import torch  # noqa: E402

DIM = 1024
METRIC = "hybrid search QPS at recall@10>=0.95 (cands=128); index build sec per 1M docs"
PRESETS = [("dense-only 1/0/0", (0.0, 0.0, 1.0), 1), ("sparse-only 0/1/0", (1.0, 0.0, 0.0), 2), ("bm25-only 0/0/1", (0.0, 1.0, 0.0), 4),
           ("1/1/1", (1.0, 1.0, 1.0), 7), ("0.5/1/2", (1.0, 2.0, 0.5), 7)]   # name (dense/sparse/bm25), weights (sparse, bm25, dense), reference kernel


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--mode", default="replicated", choices=["replicated", "sharded"])
    ap.add_argument("--docs", type=int, default=1_000_000)
    ap.add_argument("--queries", type=int, default=10_000)
    ap.add_argument("--cands", type=int, default=128)
    ap.add_argument("--cpu-queries", type=int, default=1000, help="queries of the bounded CPU brute-force sample (about 17 s on 16 cores at 1M docs)")
    ap.add_argument("--ref-queries", type=int, default=0, help="queries per step of the reference arm (0 = as the own arm)")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--quick", action="store_true", help="headline only: skip the side measurements (sweep, curve, keyword, kg, ...)")
    ap.add_argument("--ingest-docs", type=int, default=200_000, help="documents of the file-ingest measurement (0 = skip it)")
    ap.add_argument("--builds", type=int, default=3, help="builds behind the recall mean / spread")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of this rank's GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.samples, self.index, self.proc = [], index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "25"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm = [float(s[0]) for s in self.samples if len(s) >= 6 and s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if len(s) >= 6 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples if len(s) >= 6 for i in range(4) if s[2 + i] == "Active"})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def measured_peaks():
    """(HBM copy GB/s, dense bf16 TFLOP/s burst, 'measured' | 'fallback')."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            j = json.load(open(p))
            return float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 6650.0, 1590.0, "fallback"


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def host_queries(q, a=0, b=None):
    """CPU copy (pinned) of query rows [a, b)."""
    import synth
    b = q.nq if b is None else b
    s = q.slice(a, b)
    pin = lambda t: t.cpu().pin_memory() if torch.cuda.is_available() else t.cpu()
    return synth.Queries(pin(s.dense), synth.Csr(pin(s.sparse.off), pin(s.sparse.idx), pin(s.sparse.val)),
                         synth.Csr(pin(s.bm25.off), pin(s.bm25.idx), pin(s.bm25.val)))


def recall_at_10(ids, gt):
    """Mean share of the true top-10 ids found among the first 10 ids of every row (numpy arrays, uint32; 0xFFFFFFFF in the
    ground truth = fewer than 10 eligible documents)."""
    ids, gt = np.asarray(ids)[:, :10].astype(np.int64), np.asarray(gt)[:, :10].astype(np.int64)
    valid = gt != 0xFFFFFFFF
    hit = ((gt[:, :, None] == ids[:, None, :]).any(axis=2)) & valid
    return float(np.mean(hit.sum(axis=1) / np.maximum(valid.sum(axis=1), 1)))


def t2u(t):
    return t.cpu().numpy().view(np.uint32)


def oracle():
    p = os.path.join(ROOT, "oracle")
    if p not in sys.path:
        sys.path.insert(0, p)
    import apoe_oracle as orc
    return orc


def cpu_baseline(corpus_host, qsub, eff):
    """Exact OpenMP brute-force hybrid top-10 (the CPU oracle) on a bounded query sample.  Returns (dict, gt ids)."""
    orc = oracle()
    D, S, B = corpus_host
    QS, QB = orc.CsrNp.from_torch(qsub.sparse), orc.CsrNp.from_torch(qsub.bm25)
    qd, qs, qb = orc.scale_queries(qsub.dense.numpy(), QS, QB, *eff)
    t0 = time.time()
    gt, _, thr = orc.bruteforce(D, S, B, qd, qs, qb, 7, 10)
    dt = time.time() - t0
    n = qd.shape[0]
    return ({"value": n / dt, "unit": "queries/s", "cores": thr, "kind": "port",
             "sample": f"exact OpenMP brute-force hybrid top-10 of {n} queries over {D.shape[0]} docs in {dt:.1f} s "
                       f"(term-major sparse postings, blocked dense dot products)"}, gt)


# ---------------------------------------------------------------------------------------------------------
# rows next to the path: file ingest, BM25 preparation
# ---------------------------------------------------------------------------------------------------------
def ingest_files(n_docs, dev):
    """Writes a seeded synthetic corpus of n_docs documents in the reference's file formats to a temporary folder."""
    import tempfile
    import synth
    d = tempfile.mkdtemp(prefix="apoe_ingest_")
    c = synth.make_corpus(n_docs, seed=20261127, device=dev)
    paths = [os.path.join(d, f) for f in ("dense.fvecs", "sparse.bin", "bm25.bin")]
    synth.write_fvecs(paths[0], c.dense.cpu())
    synth.write_csr(paths[1], c.sparse.to("cpu"))
    synth.write_csr(paths[2], c.bm25.to("cpu"))
    return d, paths


def ingest_own(n_docs, dev):
    """File ingest of this library: files (page cache) -> resident records, best of 3."""
    import shutil
    import apoe
    d, paths = ingest_files(n_docs, dev)
    try:
        best = None
        for _ in range(3):
            ix, st = apoe.Index.from_files(*paths, device=dev.index or 0, for_build=True)
            ix.close()
            if best is None or st.seconds_total < best.seconds_total:
                best = st
        size = sum(os.path.getsize(p) for p in paths)
        return {"docs": n_docs, "file_bytes": size, "seconds": round(best.seconds_total, 4), "gb_per_s": round(size / best.seconds_total / 1e9, 2),
                "threads": int(best.threads), "what": "pread threads -> pinned staging -> H2D + pack, both record pools, files in page cache"}
    finally:
        shutil.rmtree(d, ignore_errors=True)


def ingest_reference(n_docs, dev):
    """The reference's loaders (one thread, one read per row) and uploads on the same files, best of 2."""
    import shutil
    import apoe_ref
    d, paths = ingest_files(n_docs, dev)
    try:
        best = None
        for _ in range(2):
            with apoe_ref._quiet():           # the loaders print to stdout; this program's stdout is one JSON line
                rows, t_load, t_all = apoe_ref.load_seconds(*paths)
            if best is None or t_all < best[1]:
                best = (t_load, t_all)
        size = sum(os.path.getsize(p) for p in paths)
        return {"docs": n_docs, "file_bytes": size, "seconds": round(best[1], 4), "seconds_load_only": round(best[0], 4),
                "gb_per_s": round(size / best[1] / 1e9, 2), "threads": 1, "what": "load_data + load_sparse_data x2 + cudaMemcpy of every array, files in page cache"}
    finally:
        shutil.rmtree(d, ignore_errors=True)


def prep_bench(corpus, dev, peak, with_cpu):
    """BM25 input preparation on the benchmark corpus' BM25 rows: synthetic raw term frequencies, document
    frequencies, idf, renumbering by descending df (so that nearly every row has to be re-sorted) and weights."""
    import apoe
    g = torch.Generator(device=dev); g.manual_seed(20261128)
    off, idx = corpus.bm25.off, corpus.bm25.idx.clone()
    vocab = max(int(corpus.idf.numel()), int(idx.max()) + 1)
    tf = (1 + torch.empty(idx.numel(), device=dev).geometric_(0.6, generator=g)).float()
    w = torch.empty_like(tf)
    df = torch.empty(vocab, dtype=torch.int32, device=dev); idf = torch.empty(vocab, dtype=torch.float32, device=dev)
    rl = torch.empty(vocab, dtype=torch.int32, device=dev)
    off_h = off.cpu().numpy()
    best = None
    for _ in range(3):
        idx.copy_(corpus.bm25.idx)
        st = apoe.bm25_corpus_device(off_h, off, idx, tf, w, df, idf, rl)
        if best is None or st.kernel_ms < best.kernel_ms:
            best = st
    nnz = int(best.nnz)
    algo = 24 * nnz + 8 * (off_h.size - 1) + 12 * vocab      # df pass 4, length pass 4, row pass 8 in + 8 out per posting
    out = {"postings": nnz, "rows": int(off_h.size - 1), "vocab": vocab, "kernel_ms": round(best.kernel_ms, 3), "rows_sorted": int(best.rows_sorted),
           "postings_per_s": round(nnz / (best.kernel_ms * 1e-3)), "algorithmic_gb_per_s": round(algo / (best.kernel_ms * 1e-3) / 1e9, 1),
           "frac_of_hbm_peak": round(algo / (best.kernel_ms * 1e-3) / 1e9 / peak, 4)}
    if with_cpu:
        orc = oracle()
        m = min(off_h.size - 1, 100_000)
        e = int(off_h[m])
        t0 = time.time()
        orc.bm25_corpus(off_h[:m + 1], corpus.bm25.idx[:e].cpu().numpy(), tf[:e].cpu().numpy(), vocab, relabel_by_df=True)
        out["cpu_port"] = {"postings_per_s": round(e / (time.time() - t0)), "cores": 1, "sample": f"numpy restatement on the first {m} rows ({e} postings)"}
    return out


# ---------------------------------------------------------------------------------------------------------
# pieces of the own arm
# ---------------------------------------------------------------------------------------------------------
def algorithmic_bytes(st, nq, cands, qnnz):
    """Bytes the search must move by the per-query formula: query row, entry ids, 160-byte graph rows per expansion,
    one record (2048 dense bytes + 8 bytes per stored term, as fetched) per evaluation, cands x 8 result bytes."""
    rows_fetched = st.expansions * 512                       # the kernel's own count includes 512-byte locator rows
    records = st.gathered_bytes - rows_fetched
    return records + st.expansions * 160 + nq * (2 * DIM + 8 * qnnz + 128 + 8 * cands)


def max_nnz(q):
    return (int((q.sparse.off[1:] - q.sparse.off[:-1]).max()), int((q.bm25.off[1:] - q.bm25.off[:-1]).max()))


class Searcher:
    """Device-resident searches of one index with reusable output buffers; kernel time from the library's events."""

    def __init__(self, ix, dev):
        self.ix, self.dev, self.stream = ix, dev, torch.cuda.current_stream().cuda_stream
        self.bufs = {}

    def out(self, nq, cands):
        key = (nq, cands)
        if key not in self.bufs:
            self.bufs[key] = (torch.empty(nq, cands, dtype=torch.int32, device=self.dev), torch.empty(nq, cands, dtype=torch.float32, device=self.dev))
        return self.bufs[key]

    def run(self, q, cands, weights, repeat=2, **kw):
        oi, od = self.out(q.nq, cands)
        st = None
        for _ in range(repeat):
            st = self.ix.search_device(q, oi, od, cands=cands, weights=weights, max_nnz=max_nnz(q), stream=self.stream, **kw)
        return oi, st


def flag_keywords(queries_host, synth, seed=20261128):
    """Query BM25 ids with bit 31 set on the required terms (ref: src/query.cu:1828-1843), as a numpy array, and the
    required-term lists."""
    kws = synth.make_keywords(queries_host, seed=seed)
    off = queries_host.bm25.off.numpy().astype(np.int64)
    idx = queries_host.bm25.idx.numpy().astype(np.uint32)
    for q, req in enumerate(kws):
        row = idx[off[q]:off[q + 1]]
        row[np.isin(row, np.asarray(req, dtype=np.uint32))] |= np.uint32(0x80000000)
    return idx, kws


def keyword_hit_rate(ids, kws, corpus_bm25_host):
    """Share of the valid top-10 results that hold at least one of the query's required terms."""
    off, idx = corpus_bm25_host
    good = total = 0
    for q in range(ids.shape[0]):
        req = set(kws[q])
        for d in ids[q, :10]:
            if d < off.size - 1:
                total += 1
                good += bool(req & set(idx[off[d]:off[d + 1]].tolist()))
    return good / max(total, 1)


def section_keyword(ix, sr, corpus, eff, dev, n, cands):
    """The keyword-constrained configuration: 1-4 required BM25 terms per query; batch 1 latency through the
    host-pointer call, batch 65 536 throughput, and the index with keyword-edge recycling against the same index with the
    keyword-edge count (slot 32 of every row) zeroed."""
    import apoe
    import synth
    out = {}
    big = synth.make_queries(65_536, corpus.idf, seed=20261131, device=dev)
    bh = host_queries(big)
    kidx, kws = flag_keywords(bh, synth)
    kq = synth.Queries(big.dense, big.sparse, synth.Csr(big.bm25.off, torch.from_numpy(kidx.view(np.int32)).to(dev), big.bm25.val))
    oi, st = sr.run(kq, cands, eff, flags=apoe.SEARCH_KEYWORD)
    out["batch_65536"] = {"qps": round(kq.nq / st.kernel_ms * 1e3, 1), "kernel_ms": round(st.kernel_ms, 3), "cands": cands,
                          "evaluations_per_query": round(st.evaluations / kq.nq, 1)}
    # quality on the first 10 000 of them: constrained ground truth = exact top-10 among the documents that hold a required term
    m = 10_000
    sub = kq.slice(0, m)
    gt, _, _ = ix.exact_topk(sub, eff, top_k=10, keyword=True)
    gt = t2u(gt)
    bm25_host = (corpus.bm25.off.cpu().numpy().astype(np.int64), corpus.bm25.idx.cpu().numpy())
    graph, ep = ix.get_graph()
    res = {}
    for name in ("with_recycling", "without_recycling"):
        if name == "without_recycling":
            g2 = graph.copy()
            g2[:, 32] = 0
            ix.set_graph(g2, ep)
        oi, st = sr.run(sub, cands, eff, flags=apoe.SEARCH_KEYWORD)
        ids = t2u(oi)
        res[name] = {"constrained_recall_at_10": round(recall_at_10(ids, gt), 4), "hit_rate_at_10": round(keyword_hit_rate(ids[:2000], kws[:2000], bm25_host), 4),
                     "qps": round(m / st.kernel_ms * 1e3, 1)}
    ix.set_graph(graph, ep)
    res["keyword_edges_per_row"] = round(float(graph[:, 32].mean()), 3)
    res["what"] = ("10 000 queries; ground truth = exact top-10 among the documents holding a required term (device scorer); 'without' = the same "
                   "index with slot 32 (keyword-edge count) of every row zeroed; hit rate on the first 2 000 queries")
    out["recycling"] = res
    # batch 1: one query per call through ap_search_host (host buffers in and out), 1 000 different queries
    one = []
    qd = bh.dense.numpy()
    so, si, sv = bh.sparse.off.numpy(), bh.sparse.idx.numpy(), bh.sparse.val.numpy()
    bo, bv = bh.bm25.off.numpy(), bh.bm25.val.numpy()
    oi1 = (np.empty((1, cands), dtype=np.uint32), np.empty((1, cands), dtype=np.float32))
    for i in range(1100):
        s = (np.array([0, so[i + 1] - so[i]], dtype=np.uint32), si[so[i]:so[i + 1]], sv[so[i]:so[i + 1]])
        b = (np.array([0, bo[i + 1] - bo[i]], dtype=np.uint32), kidx[bo[i]:bo[i + 1]], bv[bo[i]:bo[i + 1]])
        t0 = time.perf_counter()
        ix.search(qd[i:i + 1], s, b, cands=cands, weights=eff, flags=apoe.SEARCH_RAW_WEIGHTS | apoe.SEARCH_KEYWORD, out=oi1)
        one.append((time.perf_counter() - t0) * 1e3)
    one = np.asarray(one[100:])
    out["batch_1"] = {"p50_ms": round(float(np.percentile(one, 50)), 4), "p99_ms": round(float(np.percentile(one, 99)), 4), "calls": int(one.size),
                      "what": "ap_search_host, one query per call, host buffers in and out, keyword kernel"}
    return out


def section_kg(dev, cands):
    """The knowledge-graph configuration: 200k documents, 500k entities (power-law degree, mean 4), 1-5 documents per
    entity, 1-3 seed entities per query.  The reference's KG kernel is not run (it indexes shared memory with a variable
    that is never assigned, src/query.cu:1559,1694): own arm only, judged by quality -- recall against the exact fused
    top-10 and nDCG@10 with the seed entities' documents as the relevant ones, KG bonus on (40) and off."""
    import apoe
    import synth
    n, nq = 200_000, 10_000
    corpus = synth.make_corpus(n, seed=20261140, device=dev)
    queries = synth.make_queries(nq, corpus.idf, seed=20261141, device=dev)
    ix = apoe.Index.from_device(corpus.dense, corpus.sparse, corpus.bm25, for_build=True)
    bst = ix.build(seed=20261125)
    q100 = host_queries(queries, 0, 100)
    eff = ix.effective_weights(q100.dense.numpy(), q100.sparse, q100.bm25)
    kg = synth.make_kg(n, nq, device=dev)
    ix.set_kg(kg.e2e_off, kg.e2e_idx, kg.e2d_off, kg.e2d_idx)
    sr = Searcher(ix, dev)
    gt, _, _ = ix.exact_topk(queries, eff, top_k=10)
    gt = t2u(gt)
    qe_off, qe_idx = kg.qe_off.cpu().numpy().astype(np.int64), kg.qe_idx.cpu().numpy().astype(np.int64)
    e2d_off, e2d_idx = kg.e2d_off.cpu().numpy().astype(np.int64), kg.e2d_idx.cpu().numpy()
    qrels = []
    for q in range(nq):
        rel = set()
        for e in qe_idx[qe_off[q]:qe_off[q + 1]]:
            rel.update(e2d_idx[e2d_off[e]:e2d_off[e + 1]].tolist())
        qrels.append(sorted(rel))
    out = {"docs": n, "queries": nq, "entities": int(kg.e2e_off.numel() - 1), "build_seconds": round(bst.seconds_total, 3), "cands": cands}
    for name, kw in (("kg_weight_40", 40.0), ("kg_weight_0", 0.0)):
        if kw > 0:
            oi, st = sr.run(queries, cands, eff, kg_weight=kw, ent=(kg.qe_off, kg.qe_idx))
        else:
            oi, st = sr.run(queries, cands, eff)
        ids = t2u(oi)
        out[name] = {"qps": round(nq / st.kernel_ms * 1e3, 1), "recall_at_10_vs_exact_fused": round(recall_at_10(ids, gt), 4),
                     "ndcg_at_10_seed_entity_docs": round(apoe.ndcg(np.ascontiguousarray(ids[:, :10]), 10, qrels), 4)}
    out["what"] = "relevance for nDCG = the documents of the query's own seed entities; recall against the exact fused top-10 (no KG bonus)"
    ix.close()
    return out


def section_config0(dev, cands, with_cpu):
    """The 10k-document / 1k-query configuration: build, search, recall, parity with the reference's kernel, CPU brute force in full."""
    import apoe
    import synth
    n, nq = 10_000, 1_000
    corpus = synth.make_corpus(n, seed=20261150, device=dev)
    queries = synth.make_queries(nq, corpus.idf, seed=20261151, device=dev)
    ix = apoe.Index.from_device(corpus.dense, corpus.sparse, corpus.bm25, for_build=True)
    bst = ix.build(seed=20261125)
    hq = host_queries(queries)
    eff = ix.effective_weights(hq.dense.numpy()[:100], hq.sparse.slice_rows(0, 100), hq.bm25.slice_rows(0, 100))
    sr = Searcher(ix, dev)
    oi, st = sr.run(queries, cands, eff, repeat=3)
    ids = t2u(oi)
    gt, _, _ = ix.exact_topk(queries, eff, top_k=10)
    out = {"docs": n, "queries": nq, "cands": cands, "build_seconds": round(bst.seconds_total, 4), "qps": round(nq / st.kernel_ms * 1e3, 1),
           "recall_at_10": round(recall_at_10(ids, t2u(gt)), 4)}
    graph, ep = ix.get_graph()
    par = reference_parity(corpus, queries, eff, graph, ep, sr, cands, nq)
    if par:
        out["parity"] = par
    if with_cpu:
        orc = oracle()
        cpu, cgt = cpu_baseline((corpus.dense.cpu().numpy(), orc.CsrNp.from_torch(corpus.sparse), orc.CsrNp.from_torch(corpus.bm25)), hq, eff)
        out["cpu_bruteforce_qps"] = round(cpu["value"], 1)
        out["cpu_cores"] = cpu["cores"]
        out["device_gt_equals_cpu_gt"] = round(float(np.mean(t2u(gt) == cgt)), 5)
    ix.close()
    return out


def reference_parity(corpus, queries, eff, graph, ep, sr, cands, nq_check):
    """The reference's own search_with_three_paths kernel over THIS library's graph, same effective weights, against this
    library's result pools: share of equal ids and of equal fused-distance bit patterns over all pool entries.
    A checker, outside every timed region.  None where the reference library was not built."""
    p = os.path.join(ROOT, "oracle")
    if p not in sys.path:
        sys.path.insert(0, p)
    import apoe_ref
    if not apoe_ref.available():
        return None
    orc = oracle()
    nq_check = min(nq_check, queries.nq)
    sub = queries.slice(0, nq_check)
    QD = sub.dense.cpu().numpy()
    QS, QB = orc.CsrNp.from_torch(sub.sparse), orc.CsrNp.from_torch(sub.bm25)
    qd, qs, qb = orc.scale_queries(QD, QS, QB, *eff)
    S, B = orc.CsrNp.from_torch(corpus.sparse), orc.CsrNp.from_torch(corpus.bm25)
    resident = apoe_ref.Resident(corpus.dense.cpu().numpy(), (S.off, S.idx, S.val), (B.off, B.idx, B.val), graph, ep)
    ref_ids, ref_dis, _ = resident.search(qd, (qs.off, qs.idx, qs.val), (qb.off, qb.idx, qb.val), cands, 7)
    resident.close()
    oi, od = sr.out(nq_check, cands)
    sr.ix.search_device(sub, oi, od, cands=cands, weights=eff, max_nnz=max_nnz(sub), stream=sr.stream)
    ids, dis = t2u(oi), od.cpu().numpy()
    return {"ids_equal_frac": float(np.mean(ids == ref_ids)), "dis_bits_equal_frac": float(np.mean(dis.view(np.uint32) == ref_dis.view(np.uint32))),
            "queries": int(nq_check), "pool_entries": int(ids.size),
            "against": "the reference's search_with_three_paths kernel (oracle/_ref) over this library's graph, same effective weights"}


def recall_search(sr, queries, eff, gt, cands_list):
    out = []
    for c in cands_list:
        oi, st = sr.run(queries, c, eff)
        out.append({"cands": c, "qps": round(queries.nq / st.kernel_ms * 1e3, 1), "recall_at_10": round(recall_at_10(t2u(oi), gt), 4),
                    "evaluations_per_query": round(st.evaluations / queries.nq, 1)})
    return out


def first_reaching(curve, target=0.95):
    for row in curve:
        if row["recall_at_10"] >= target:
            return {"cands": row["cands"], "qps": row["qps"], "recall_at_10": row["recall_at_10"]}
    return None


SUPPLEMENTARY_LABEL = ("{n} docs in topics of ~100, topics in groups of ~100 (mixture: dense = topic centre + noise, topic centre = group centre + noise, "
                       "60 % of the sparse / BM25 terms from the topic's term list, half of which is the group's), {nq} queries = perturbed documents; "
                       "supplementary corpus, not the prescribed generator")


def section_supplementary(dev, n, nq):
    """Supplementary corpus, clearly not the prescribed one: documents drawn from a mixture, queries = perturbed
    documents; everything else (shapes, value distributions, row lengths, index parameters) is unchanged.  On the
    prescribed i.i.d. dense vectors no graph reaches recall 0.95; here the metric's own qualifier -- QPS at recall@10
    >= 0.95 -- can be reported: the smallest cands that reaches it, and the QPS there."""
    import apoe
    import synth
    corpus = synth.make_clustered_corpus(n, device=dev)
    queries = synth.make_clustered_queries(nq, corpus)
    ix = apoe.Index.from_device(corpus.dense, corpus.sparse, corpus.bm25, for_build=True)
    bst = ix.build(seed=20261125)
    q100 = host_queries(queries, 0, 100)
    eff = ix.effective_weights(q100.dense.numpy(), q100.sparse, q100.bm25)
    gt, _, _ = ix.exact_topk(queries, eff, top_k=10)
    sr = Searcher(ix, dev)
    curve = recall_search(sr, queries, eff, t2u(gt), (32, 64, 128, 256, 512))
    # the sweep's dense-only preset over the same graph: the one preset whose exact top-10 this corpus lets a graph reach
    eff_d = ix.effective_weights(q100.dense.numpy(), q100.sparse, q100.bm25, 0.0, 0.0, 1.0)
    gt_d, _, _ = ix.exact_topk(queries, eff_d, top_k=10)
    curve_d = recall_search(sr, queries, eff_d, t2u(gt_d), (32, 64, 96, 128, 256, 512))
    ix.close()
    return {"corpus": SUPPLEMENTARY_LABEL.format(n=n, nq=nq), "build_seconds": round(bst.seconds_total, 3), "curve": curve,
            "qps_at_recall_0.95": first_reaching(curve), "qps_at_recall_0.90": first_reaching(curve, 0.90), "qps_at_recall_0.75": first_reaching(curve, 0.75),
            "effective_weights": {"sparse": eff[0], "bm25": eff[1], "dense": eff[2]},
            "dense_only": {"weights_dense_sparse_bm25": "1/0/0", "graph": "the same hybrid graph", "curve": curve_d, "qps_at_recall_0.95": first_reaching(curve_d)}}


def build_roofline(bst, corpus, n, hbm_peak, tc_peak, peak_kind):
    """Roofline figures of the build.  A local join stages the record of each of its (up to 64) participants once --
    dense halves for the tensor-core tile, 8 bytes per stored term for the sparse part -- and evaluates up to 32 distances
    per staged record, so the bytes the k-NN phase gathers are `rows_gathered` records, not one record per distance; the
    per-distance formula (one ~3.5 KB record per evaluated distance) is reported beside it.  The dense half of the joins
    is 2 x 1024 flops per evaluated pair on the tensor pipe."""
    nnz = int(corpus.sparse.off[-1]) + int(corpus.bm25.off[-1])
    rec_bytes = 2 * DIM + 8.0 * nnz / n
    evals, rows = int(bst.distance_evals), int(bst.rows_gathered)
    gathered = rows * rec_bytes
    hbm = gathered / max(bst.seconds_knn, 1e-9) / 1e9
    per_distance = evals * rec_bytes / max(bst.seconds_knn, 1e-9) / 1e9
    batches = (n + (1 << 18) - 1) // (1 << 18)          # the dense-tile phase timer covers the first node batch of every round
    dense_s = bst.phase_10us[0] * 1e-5 * batches
    tf = evals * 2.0 * DIM / max(dense_s, 1e-9) / 1e12
    return {"knn": {"bound": "hbm", "achieved": round(hbm, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(hbm / hbm_peak, 4),
                    "algorithmic_bytes": int(gathered), "records_gathered": rows, "mean_record_bytes": round(rec_bytes, 1),
                    "distances_per_gathered_record": round(evals / max(rows, 1), 2), "seconds": round(bst.seconds_knn, 3),
                    "by_per_distance_formula": {"gb_per_s": round(per_distance, 1), "frac": round(per_distance / hbm_peak, 4),
                                                "what": "one record per evaluated distance; above the copy peak because a staged record serves many distances"},
                    "limiter": "shared-memory data pipe of the term-probing kernels (ncu: LSU pipe 81 % / 61 %, DRAM 3 %; profiles/build_kernels_200k_docs.md), not HBM"},
            "dense_join": {"bound": "tensor", "achieved": round(tf, 1), "peak": tc_peak, "unit": "TFLOP/s", "frac": round(tf / tc_peak, 4),
                           "useful_flops": int(evals * 2.0 * DIM), "seconds": round(dense_s, 4),
                           "limiter": "row gather (the kernel runs at the rate its operand rows arrive), not the tensor pipe"},
            "peak_kind": f"of {peak_kind}"}


def pack_keys_torch(ids, dis, base):
    """(ordered distance << 32 | id + base) as int64 bit patterns, the exchange word of the sharded search (torch)."""
    b = dis.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    o = torch.where((b & 0x80000000) != 0, (~b) & 0xFFFFFFFF, b | 0x80000000)
    lid = ids.to(torch.int64) & 0xFFFFFFFF
    k = (o << 32) | (lid + base)
    return torch.where(lid == 0xFFFFFFFF, torch.full_like(k, -1), k)


def section_sharded(args, ix_full, corpus, eff, dev, rank, world, steps=5):
    """The same corpus split over the ranks: per-shard graphs, every query on every shard, one all-gather of packed
    top-10 keys + one merge kernel per step.  Checked on the GPUs: the device merge against the torch merge of the gathered
    keys, and the merged top-10 against the exact scorer over the whole corpus."""
    import apoe
    import dist_search
    import synth
    import torch.distributed as dist
    n, nq, cands, top_k = corpus.n, args.queries, args.cands, 10
    a, b = dist_search.shard_range(n, rank, world)
    queries = synth.make_queries(nq, corpus.idf, seed=20261126, device=dev)      # the same batch on every rank
    ix = apoe.Index.from_device(corpus.dense[a:b].contiguous(), corpus.sparse.slice_rows(a, b), corpus.bm25.slice_rows(a, b), for_build=True)
    bst = ix.build(seed=20261125)
    mq = max_nnz(queries)
    stream = torch.cuda.current_stream().cuda_stream
    g_keys = torch.empty(world, nq, top_k, dtype=torch.int64, device=dev)
    m_ids = torch.empty(nq, top_k, dtype=torch.int32, device=dev)
    m_dis = torch.empty(nq, top_k, dtype=torch.float32, device=dev)

    def step():
        ix.search_shard_device(queries, g_keys[rank], a, top_k=top_k, cands=cands, weights=eff, max_nnz=mq, stream=stream)
        dist_search.exchange_and_merge(g_keys, rank, m_ids, m_dis, top_k)

    for _ in range(3):
        step()
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize(); dist.barrier()
    ms = e0.elapsed_time(e1)
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(steps):
        dist.all_gather_into_tensor(g_keys.view(-1), g_keys[rank].view(-1))
    c1.record()
    torch.cuda.synchronize()
    t = torch.tensor([ms, c0.elapsed_time(c1), bst.seconds_total], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    want = dist_search.merge_keys_reference(g_keys, top_k)
    w_ids = torch.where(want == -1, torch.full_like(want, -1), want & 0xFFFFFFFF).to(torch.int32)
    flag = torch.tensor([1 if bool(torch.equal(w_ids, m_ids)) else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    out = None
    if rank == 0:
        gt, _, est = ix_full.exact_topk(queries, eff, top_k=top_k)
        out = {"docs": n, "shards": world, "queries": nq, "cands": cands, "top_k": top_k, "steps": steps,
               "qps": round(nq * steps / (float(t[0]) * 1e-3), 1), "ms_per_step": round(float(t[0]) / steps, 3),
               "build_seconds_max_over_shards": round(float(t[2]), 3),
               "all_gather_bytes_per_rank": int(world * nq * top_k * 8), "all_gather_ms": round(float(t[1]) / steps, 4),
               "merge_equals_reference": bool(int(flag[0])), "recall_at_10_vs_exact": round(recall_at_10(t2u(m_ids), t2u(gt)), 4),
               "exchange": "one NCCL all-gather of packed (distance, global id) top-10 keys written by the search kernel, one merge kernel"}
        ix_full.exact_release()
    dist.barrier()
    ix.close()
    return out


# ---------------------------------------------------------------------------------------------------------
# own arm
# ---------------------------------------------------------------------------------------------------------
def bench_config(n, nq, cands):
    """The workload, named identically by both arms."""
    return {"workload": f"{n} docs / {nq} queries per step, weights 1/1/1, top_k 10, cands {cands}", "docs": n, "queries_per_step": nq,
            "cands": cands, "top_k": 10, "l2": "inputs larger than L2 (records pool %.1f GB, random gathers)" % (n * 3.5e-6)}


# DRAM bytes / algorithmic bytes of the search kernel: dram__bytes_read.sum + dram__bytes_write.sum of one launch over the
# kernel's counted bytes in the 3-metric ncu capture summarised under profiles/ (the full-size launch is too large to
# capture; both grow with the number of fused distances, the L2-served share shrinks with the corpus)
TRAFFIC = {"ratio": 0.9565, "from": "ncu capture of the 500k-doc / 4k-query case (records pool 1.75 GB), profiles/search_kernel_traffic_500k_docs_4k_queries.md"}


def traffic_ratio():
    return TRAFFIC


def run_own(args):
    import apoe
    import synth
    rank, world, local = dist_env()
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    n, nq, cands = args.docs, args.queries, args.cands
    sharded = args.mode == "sharded" and world > 1
    hbm_peak, tc_peak, peak_kind = measured_peaks()

    t0 = time.time()
    if sharded:
        import dist_search
        a, b = dist_search.shard_range(n, rank, world)
        full = synth.make_corpus(n, device=dev)
        corpus = synth.Corpus(full.dense[a:b].contiguous(), full.sparse.slice_rows(a, b), full.bm25.slice_rows(a, b), full.idf)
        sample = synth.Corpus(full.dense[:100].contiguous(), full.sparse.slice_rows(0, 100), full.bm25.slice_rows(0, 100), full.idf)
        del full
        queries = synth.make_queries(nq, corpus.idf, device=dev)
    else:
        corpus = synth.make_corpus(n, device=dev)
        queries = synth.make_queries(nq, corpus.idf, seed=20261126 + rank, device=dev)
    torch.cuda.synchronize()
    t_gen = time.time() - t0

    # page the library's kernels in (a fresh machine reads them from disk at first launch) before the timed build
    warm = synth.make_corpus(4096, seed=1, device=dev)
    ixw = apoe.Index.from_device(warm.dense, warm.sparse, warm.bm25, for_build=True)
    ixw.build(seed=1)
    ixw.close()
    del warm
    ix = apoe.Index.from_device(corpus.dense, corpus.sparse, corpus.bm25, for_build=True)
    bst = ix.build(seed=20261125)
    torch.cuda.synchronize()

    # effective weights: first 100 docs x first 100 queries on the host (global docs 0..99 in sharded mode)
    q100 = host_queries(queries, 0, min(100, nq))
    if sharded:
        tmp = apoe.Index.from_device(sample.dense, sample.sparse, sample.bm25)
        eff = tmp.effective_weights(q100.dense.numpy(), q100.sparse, q100.bm25)
        tmp.close()
    else:
        eff = ix.effective_weights(q100.dense.numpy(), q100.sparse, q100.bm25)

    out_ids = torch.empty(nq, cands, dtype=torch.int32, device=dev)
    out_dis = torch.empty(nq, cands, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    mq = max_nnz(queries)
    top_k = 10

    if sharded:
        import dist_search
        a, _ = dist_search.shard_range(n, rank, world)
        g_keys = torch.empty(world, nq, top_k, dtype=torch.int64, device=dev)
        m_ids = torch.empty(nq, top_k, dtype=torch.int32, device=dev)
        m_dis = torch.empty(nq, top_k, dtype=torch.float32, device=dev)

        def step():
            ix.search_shard_device(queries, g_keys[rank], a, top_k=top_k, cands=cands, weights=eff, max_nnz=mq, stream=stream)
            dist_search.exchange_and_merge(g_keys, rank, m_ids, m_dis, top_k)
    else:
        def step():
            ix.search_device(queries, out_ids, out_dis, cands=cands, weights=eff, max_nnz=mq, stream=stream, stats=False)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # kernel-only duration and byte counts of one more pass (events on the launch stream inside the library)
    st = ix.search_device(queries, out_ids, out_dis, cands=cands, weights=eff, max_nnz=mq, stream=stream, stats=True)
    clocks = sampler.stop()
    # what the memory system gives this access pattern when the records are only fetched (same CTAs, same shared memory)
    probe = max(ix.debug_gather_probe()[0] for _ in range(3))

    # end to end through the host-pointer call: pinned host queries in, host results out
    hq = host_queries(queries)
    h_ids = np.empty((nq, cands), dtype=np.uint32)
    h_dis = np.empty((nq, cands), dtype=np.float32)
    for _ in range(2):
        _, _, est = ix.search(hq.dense.numpy(), hq.sparse, hq.bm25, cands=cands, weights=eff, flags=apoe.SEARCH_RAW_WEIGHTS, out=(h_ids, h_dis))
    barrier()
    t0 = time.time()
    for _ in range(args.steps):
        _, _, est = ix.search(hq.dense.numpy(), hq.sparse, hq.bm25, cands=cands, weights=eff, flags=apoe.SEARCH_RAW_WEIGHTS, out=(h_ids, h_dis))
    torch.cuda.synchronize()
    e2e_s = time.time() - t0
    h2d = est.h2d_bytes_lo + (est.h2d_bytes_hi << 32)
    d2h = est.d2h_bytes_lo + (est.d2h_bytes_hi << 32)

    times = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_max, e2e_ms_max = float(times[0]), float(times[1])
    total_q = nq * (1 if sharded else world)

    # sharded mode: global ground truth = per-shard exact top-10, all-gathered and merged like the results themselves
    sharded_recall = None
    if sharded:
        import dist_search
        import torch.distributed as dist
        gt_ids, gt_dis, _ = ix.exact_topk(queries, eff, top_k=top_k)
        gk = torch.empty(world, nq, top_k, dtype=torch.int64, device=dev)
        gk[rank] = pack_keys_torch(gt_ids, gt_dis, a)
        dist.all_gather_into_tensor(gk.view(-1), gk[rank].clone().view(-1))
        gt_glob = (dist_search.merge_keys_reference(gk, top_k) & 0xFFFFFFFF).to(torch.int32)
        sharded_recall = recall_at_10(t2u(m_ids), t2u(gt_glob))
        ix.exact_release()

    line = None
    shard_obj = None
    if world > 1 and not sharded and not args.quick:
        shard_obj = section_sharded(args, ix, corpus, eff, dev, rank, world)
    if rank == 0:
        algo = algorithmic_bytes(st, nq, cands, mq[0] + mq[1])
        achieved = algo / (st.kernel_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(achieved / hbm_peak, 4),
                "traffic": None, "peak_kind": f"of {peak_kind}",
                "kernel": "search_kernel<dense|sparse|bm25>", "kernel_ms": round(st.kernel_ms, 3),
                "algorithmic_bytes_per_launch": int(algo), "expansions_per_query": round(st.expansions / nq, 1),
                "evaluations_per_query": round(st.evaluations / nq, 1)}
        roof["fetch_only_probe"] = {"gb_per_s": round(probe, 1), "frac_of_copy_peak": round(probe / hbm_peak, 4), "search_frac_of_probe": round(achieved / probe, 4),
                                    "what": "whole records of random documents brought into shared memory by bulk copies with the search kernel's CTA count and "
                                            "shared-memory budget, every staging buffer refilled the moment it has landed and nothing computed: what the memory "
                                            "system gives this access pattern when the whole arena is in flight (the search holds the records it is scoring)"}
        tr = traffic_ratio()
        if tr:
            roof["traffic"] = round(tr["ratio"] * algo)
            roof["traffic_from"] = tr["from"]
        line = {
            "metric": METRIC, "value": round(total_q * args.steps / (ms_max * 1e-3), 1), "unit": "queries/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(ms_max / args.steps, 3), "higher_is_better": True,
            "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "f16 storage, f16 dense accumulate + f32 sparse (as the reference)",
            "data": "synthetic (seeded generators with the benchmark's shapes and value distributions)",
            "config": bench_config(n, nq, cands),
            "details": {"mode": args.mode if world > 1 else "single", "queries_timed_per_step": total_q,
                        "parallelism": (f"corpus-sharded x{world}: {n} docs split over the GPUs, every query on every shard" if sharded
                                        else f"query-parallel replicas x{world}: {n} docs and {nq} queries per GPU")},
            "e2e": {"value": round(total_q * args.steps / (e2e_ms_max * 1e-3), 1), "unit": "queries/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": args.steps * (2 if sharded else 1),
            "clocks": clocks, "roofline": roof, "cpu_baseline": None,
            "effective_weights": {"sparse": eff[0], "bm25": eff[1], "dense": eff[2]},
            "build": {"seconds": round(bst.seconds_total, 3), "seconds_per_1M_docs": round(bst.seconds_total * 1e6 / (corpus.n), 3),
                      "knn_seconds": round(bst.seconds_knn, 3), "prune_seconds": round(bst.seconds_prune, 3),
                      "iterations": bst.iterations_run, "distance_evals": int(bst.distance_evals),
                      "timer": "norms + k-NN rounds + pruning + rows + entry points; the fp32->fp16 packing of the corpus (about 1 ms per 1M docs on this GPU, "
                               "inside the reference's own timer) happens when the index is created",
                      "roofline": build_roofline(bst, corpus, corpus.n, hbm_peak, tc_peak, peak_kind)},
            "setup_seconds": {"generate": round(t_gen, 2)},
        }
        if sharded:
            line["recall"] = {"at_10": round(sharded_recall, 4), "queries": nq, "ground_truth": "per-shard exact device scorer, all-gathered and merged"}
            line["recall_at_10"] = line["recall"]["at_10"]
        if shard_obj:
            line["sharded"] = shard_obj
        if world == 1:
            own_sections(args, line, ix, corpus, queries, hq, eff, out_ids, dev, hbm_peak, tc_peak, peak_kind)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def own_sections(args, line, ix, corpus, queries, hq, eff, out_ids, dev, hbm_peak, tc_peak, peak_kind):
    """Single-GPU side measurements, all outside the timed region."""
    import apoe
    import synth
    n, nq, cands = corpus.n, queries.nq, args.cands
    sr = Searcher(ix, dev)
    # ground truth for every query from the exact device scorer
    gt_t, _, est = ix.exact_topk(queries, eff, top_k=10)
    _, _, est2 = ix.exact_topk(queries, eff, top_k=10)
    gt = t2u(gt_t)
    ids_main = t2u(out_ids)
    line["recall"] = {"at_10": round(recall_at_10(ids_main, gt), 4), "queries": nq, "ground_truth": "exact device scorer over all queries"}
    line["recall_at_10"] = line["recall"]["at_10"]
    tfl = est2.dense_flops / (est2.dense_ms * 1e-3) / 1e12
    line["exact_scorer"] = {"queries": nq, "docs": n, "index_seconds": round(est.seconds_index, 3), "sparse_ms": round(est2.sparse_ms, 2),
                            "dense_ms": round(est2.dense_ms, 2), "seconds_total": round(est2.seconds_total, 3),
                            "roofline": {"bound": "tensor", "achieved": round(tfl, 1), "peak": tc_peak, "unit": "TFLOP/s", "frac": round(tfl / tc_peak, 4),
                                         "peak_kind": f"of {peak_kind}", "kernel": "exact_dense_topk_kernel (tcgen05.mma kind::f16, TMA-fed, top-k epilogue)"},
                            "postings": int(est.postings), "batch_queries": int(est.batch_queries), "slices": int(est.slices)}
    if not args.skip_cpu:
        orc = oracle()
        D = corpus.dense.cpu().numpy()
        S, B = orc.CsrNp.from_torch(corpus.sparse), orc.CsrNp.from_torch(corpus.bm25)
        qsub = host_queries(queries, 0, min(nq, args.cpu_queries))
        cpu, cgt = cpu_baseline((D, S, B), synth.Queries(qsub.dense, qsub.sparse, qsub.bm25), eff)
        line["cpu_baseline"] = cpu
        line["recall"]["device_gt_equals_cpu_gt"] = round(float(np.mean(gt[:cgt.shape[0]] == cgt)), 5)
        line["recall"]["at_10_cpu_sample"] = round(recall_at_10(ids_main[:cgt.shape[0]], cgt), 4)
        del D, S, B
    if args.quick:
        return
    graph, ep = ix.get_graph()
    par = reference_parity(corpus, queries, eff, graph, ep, sr, cands, nq)
    if par:
        line["parity"] = par
    # pool-size curve and weight sweep over the one index
    line["curve"] = recall_search(sr, queries, eff, gt, (32, 64, 128, 256))
    sweep = []
    for name, w, _ in PRESETS:
        e = ix.effective_weights(hq.dense.numpy()[:100], hq.sparse.slice_rows(0, 100), hq.bm25.slice_rows(0, 100), *w)
        g, _, _ = ix.exact_topk(queries, e, top_k=10)
        oi, st = sr.run(queries, cands, e)
        sweep.append({"weights_dense_sparse_bm25": name, "path": int(st.path), "qps": round(nq / st.kernel_ms * 1e3, 1),
                      "recall_at_10": round(recall_at_10(t2u(oi), t2u(g)), 4), "evaluations_per_query": round(st.evaluations / nq, 1)})
    line["sweep"] = sweep
    line["keyword"] = section_keyword(ix, sr, corpus, eff, dev, n, cands)
    # batch 1 through the host call, plain three-path search
    lat, kern = [], []
    qd = hq.dense.numpy()
    so, si, sv = hq.sparse.off.numpy(), hq.sparse.idx.numpy(), hq.sparse.val.numpy()
    bo, bi, bv = hq.bm25.off.numpy(), hq.bm25.idx.numpy(), hq.bm25.val.numpy()
    o1 = (np.empty((1, cands), dtype=np.uint32), np.empty((1, cands), dtype=np.float32))
    for i in range(min(600, nq)):
        s = (np.array([0, so[i + 1] - so[i]], dtype=np.uint32), si[so[i]:so[i + 1]], sv[so[i]:so[i + 1]])
        b = (np.array([0, bo[i + 1] - bo[i]], dtype=np.uint32), bi[bo[i]:bo[i + 1]], bv[bo[i]:bo[i + 1]])
        t0 = time.perf_counter()
        _, _, s1 = ix.search(qd[i:i + 1], s, b, cands=cands, weights=eff, flags=apoe.SEARCH_RAW_WEIGHTS, out=o1)
        lat.append((time.perf_counter() - t0) * 1e3)
        kern.append(s1.kernel_ms)
    lat = np.asarray(lat[100:])
    line["latency_batch1"] = {"p50_ms": round(float(np.percentile(lat, 50)), 4), "p99_ms": round(float(np.percentile(lat, 99)), 4),
                              "kernel_p50_ms": round(float(np.median(kern[100:])), 4), "calls": int(lat.size), "what": "ap_search_host, host buffers in and out"}
    line["latency_batch1_ms"] = line["latency_batch1"]["kernel_p50_ms"]
    # small batches through the same host call: up to 2 x SMs queries run in the latency shape of the kernel (8 warps per
    # query), larger ones in the throughput shape
    small = []
    for bsz in (8, 64, 296, 297, 1000):
        if bsz > nq:
            break
        s = (so[:bsz + 1].astype(np.uint32), si[:so[bsz]], sv[:so[bsz]])
        b = (bo[:bsz + 1].astype(np.uint32), bi[:bo[bsz]], bv[:bo[bsz]])
        ob = (np.empty((bsz, cands), dtype=np.uint32), np.empty((bsz, cands), dtype=np.float32))
        lt, kn = [], []
        for _ in range(40):
            t0 = time.perf_counter()
            _, _, s1 = ix.search(qd[:bsz], s, b, cands=cands, weights=eff, flags=apoe.SEARCH_RAW_WEIGHTS, out=ob)
            lt.append((time.perf_counter() - t0) * 1e3)
            kn.append(s1.kernel_ms)
        small.append({"batch": bsz, "host_p50_ms": round(float(np.median(lt[10:])), 4), "kernel_p50_ms": round(float(np.median(kn[10:])), 4)})
    line["latency_small_batches"] = small
    # recall over several builds (the default build keeps proposals in arrival order), and what the deterministic build costs
    ix.exact_release()
    rec, secs = [line["recall"]["at_10"]], [line["build"]["seconds"]]
    for i in range(max(0, args.builds - 1)):
        ixb = apoe.Index.from_device(corpus.dense, corpus.sparse, corpus.bm25, for_build=True)
        b2 = ixb.build(seed=20261125 + 17 * (i + 1))
        oi, _ = Searcher(ixb, dev).run(queries, cands, eff, repeat=1)
        rec.append(round(recall_at_10(t2u(oi), gt), 4)); secs.append(round(b2.seconds_total, 3))
        ixb.close()
    line["recall"]["over_builds"] = {"values": rec, "mean": round(float(np.mean(rec)), 4), "min": min(rec), "max": max(rec), "build_seconds": secs}
    det = []
    for _ in range(2):
        ixb = apoe.Index.from_device(corpus.dense, corpus.sparse, corpus.bm25, for_build=True)
        b2 = ixb.build(seed=20261125, flags=apoe.BUILD_DETERMINISTIC)
        oi, _ = Searcher(ixb, dev).run(queries, cands, eff, repeat=1)
        det.append((ixb.get_graph()[0], round(b2.seconds_total, 3), round(recall_at_10(t2u(oi), gt), 4)))
        ixb.close()
    line["build"]["deterministic"] = {"seconds": det[0][1], "recall_at_10": det[0][2], "two_builds_identical": bool(np.array_equal(det[0][0], det[1][0])),
                                      "what": "AP_BUILD_DETERMINISTIC: proposals and reverse samples kept by key instead of by arrival"}
    del det
    ix.close()   # the remaining measurements want the memory and the copy engines to themselves
    line["kg"] = section_kg(dev, cands)
    line["config0"] = section_config0(dev, cands, not args.skip_cpu)
    if args.ingest_docs > 0:
        line["ingest"] = ingest_own(min(args.ingest_docs, n), dev)
        line["prep"] = prep_bench(corpus, dev, hbm_peak, not args.skip_cpu)
    del corpus
    torch.cuda.empty_cache()
    line["supplementary"] = section_supplementary(dev, n, nq)


# ---------------------------------------------------------------------------------------------------------
# reference arm
# ---------------------------------------------------------------------------------------------------------
def run_reference(args):
    """The reference's own CUDA kernels on the same corpus, queries and batch size; rank 0 only."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    if world > 1:   # the launcher pins every rank to one OpenMP thread; this arm works on rank 0 alone and may use the host
        os.environ["OMP_NUM_THREADS"] = str(min(32, os.cpu_count() or 1))
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import apoe_ref
    if not apoe_ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libapoe_ref.so is not built (the reference tree was not mounted at build time)"}))
        return
    orc = oracle()
    import synth
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    n, cands = min(args.docs, 1_000_000), args.cands     # the reference's static arrays hold 1M points (src/index.cu:10)
    nq = min(args.queries, args.ref_queries) if args.ref_queries else args.queries
    quick = args.quick or world > 1
    corpus = synth.make_corpus(n, device=dev)
    queries = synth.make_queries(args.queries, corpus.idf, device=dev).slice(0, nq)
    c3 = lambda c: (c.off, c.idx, c.val)

    def host(corpus, queries):
        return (corpus.dense.cpu().numpy(), orc.CsrNp.from_torch(corpus.sparse), orc.CsrNp.from_torch(corpus.bm25),
                queries.dense.cpu().numpy(), orc.CsrNp.from_torch(queries.sparse), orc.CsrNp.from_torch(queries.bm25))

    def clean(graph):
        g = graph.copy()   # keyword slots beyond the row's count are never written by the reference: stale memory
        g[:, 33:] = np.where(np.arange(33, 40)[None, :] - 33 < g[:, 32:33], g[:, 33:], 0)
        return g

    def exact_gt(corpus, queries, eff, keyword=False):
        """Ground truth from this repository's exact device scorer, used as a checker outside every timed region."""
        import apoe
        ixg = apoe.Index.from_device(corpus.dense, corpus.sparse, corpus.bm25)
        try:
            return t2u(ixg.exact_topk(queries, eff, top_k=10, keyword=keyword)[0])
        finally:
            ixg.close()

    D, S, B, QD, QS, QB = host(corpus, queries)
    built = apoe_ref.build(D, c3(S), c3(B))
    graph = clean(built["graph"])
    eff = orc.effective_weights(D, S, B, QD, QS, QB, 1.0, 1.0, 1.0)
    qd, qs, qb = orc.scale_queries(QD, QS, QB, *eff)
    res = apoe_ref.Resident(D, c3(S), c3(B), graph, built["ep"])
    warmup = max(args.warmup, 1)
    sampler = ClockSampler(local)
    secs = []
    for i in range(warmup + args.steps):
        if i == warmup:
            sampler.start()
        ids, dis, t = res.search(qd, c3(qs), c3(qb), cands, 7)
        if i >= warmup:
            secs.append(t)
    clocks = sampler.stop()
    total = float(np.sum(secs))
    qps = nq * args.steps / total
    qps_own_region = nq * args.steps / (total + args.steps * res.seconds_corpus_f2h)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(qps, 1), "unit": "queries/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(total / args.steps * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 storage, f16 dense accumulate + f32 sparse", "data": "synthetic (same generators and seeds as the own arm)",
        "config": bench_config(n, nq, cands),
        "details": {"timed_region": "query fp32->fp16 conversion + the reference's search_with_three_paths kernel over a corpus already converted on the device "
                                    "(what the own arm's value counts); the reference's own timed region also converts the whole corpus in every call "
                                    "(src/query.cu:1999-2051): see qps_with_corpus_conversion",
                    "graph": "the reference's own 25-round build"},
        "qps_with_corpus_conversion": round(qps_own_region, 1), "corpus_f2h_seconds": round(res.seconds_corpus_f2h, 4),
        "e2e": {"value": round(qps, 1), "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "cpu_baseline": {"value": round(qps, 1), "unit": "queries/s", "cores": 0, "kind": "reference",
                         "sample": f"the reference's CUDA kernels (oracle/_ref) on GPU {local}: {nq} queries per step; it has no CPU path"},
        "clocks": clocks, "gpu_launches": 0,
        "build": {"seconds": round(built["seconds"], 3), "seconds_per_1M_docs": round(built["seconds"] * 1e6 / n, 3)},
        "effective_weights": {"sparse": eff[0], "bm25": eff[1], "dense": eff[2]},
    }
    gt = None
    try:
        gt = exact_gt(corpus, queries, eff)
        line["recall"] = {"at_10": round(recall_at_10(ids, gt), 4), "queries": nq, "ground_truth": "exact device scorer over all queries (a checker, outside the timed region)"}
    except Exception as e:   # noqa: BLE001
        if not args.skip_cpu:
            m = min(nq, args.cpu_queries)
            sub = lambda c: orc.CsrNp(c.off[:m + 1], c.idx[:int(c.off[m])], c.val[:int(c.off[m])])
            cgt, _, _ = orc.bruteforce(D, S, B, qd[:m], sub(qs), sub(qb), 7, 10)
            line["recall"] = {"at_10": round(recall_at_10(ids[:m], cgt), 4), "queries": m, "ground_truth": f"CPU brute force on a sample ({e})"}
    if "recall" in line:
        line["recall_at_10"] = line["recall"]["at_10"]
    if not quick and gt is not None:
        curve = []
        for cc in (32, 64, 128, 256):
            i_c, _, t_c = res.search(qd, c3(qs), c3(qb), cc, 7)
            curve.append({"cands": cc, "qps": round(nq / t_c, 1), "recall_at_10": round(recall_at_10(i_c, gt), 4)})
        line["curve"] = curve
        sweep = []
        for name, w, mode in PRESETS:
            e = orc.effective_weights(D, S, B, QD, QS, QB, *w)
            q1, q2, q3 = orc.scale_queries(QD, QS, QB, *e)
            i_s, _, t_s = res.search(q1, c3(q2), c3(q3), cands, mode)
            sweep.append({"weights_dense_sparse_bm25": name, "path": mode, "qps": round(nq / t_s, 1),
                          "recall_at_10": round(recall_at_10(i_s, exact_gt(corpus, queries, e)), 4)})
        line["sweep"] = sweep
    if not quick:
        # keyword kernel: batch 65 536, recycling on / off, single queries (device time: query conversion + kernel)
        big = synth.make_queries(65_536, corpus.idf, seed=20261131, device=dev)
        bh = host_queries(big)
        kidx, kws = flag_keywords(bh, synth)
        BQS, BQB = orc.CsrNp.from_torch(bh.sparse), orc.CsrNp(bh.bm25.off.numpy(), kidx, bh.bm25.val.numpy())
        k1, k2, k3 = orc.scale_queries(bh.dense.numpy(), BQS, BQB, *eff)
        for _ in range(2):
            i_k, _, t_k = res.search(k1, c3(k2), c3(k3), cands, 15)
        kw = {"batch_65536": {"qps": round(65_536 / t_k, 1), "cands": cands}}
        m = 10_000
        cut = lambda c: (c.off[:m + 1], c.idx[:int(c.off[m])], c.val[:int(c.off[m])])
        try:
            e_b = int(bh.bm25.off[m])
            subq = synth.Queries(big.dense[:m].contiguous(), big.sparse.slice_rows(0, m),
                                 synth.Csr(big.bm25.off[:m + 1].contiguous(), torch.from_numpy(kidx[:e_b].view(np.int32)).to(dev), big.bm25.val[:e_b].contiguous()))
            gk = exact_gt(corpus, subq, eff, keyword=True)
            bm25_host = (B.off.astype(np.int64), B.idx)
            rc = {}
            for name in ("with_recycling", "without_recycling"):
                if name == "without_recycling":
                    g2 = graph.copy(); g2[:, 32] = 0
                    res.set_graph(g2, built["ep"])
                i_r, _, t_r = res.search(k1[:m], cut(k2), cut(k3), cands, 15)
                rc[name] = {"constrained_recall_at_10": round(recall_at_10(i_r, gk), 4),
                            "hit_rate_at_10": round(keyword_hit_rate(i_r[:2000], kws[:2000], bm25_host), 4), "qps": round(m / t_r, 1)}
            res.set_graph(graph, built["ep"])
            rc["keyword_edges_per_row"] = round(float(graph[:, 32].mean()), 3)
            kw["recycling"] = rc
        except Exception as e:   # noqa: BLE001
            kw["recycling"] = {"error": str(e)}
        one = []
        for i in range(300):
            cut1 = lambda c: (c.off[i:i + 2] - c.off[i], c.idx[int(c.off[i]):int(c.off[i + 1])], c.val[int(c.off[i]):int(c.off[i + 1])])
            _, _, t1 = res.search(k1[i:i + 1], cut1(k2), cut1(k3), cands, 15)
            one.append(t1 * 1e3)
        kw["batch_1"] = {"p50_ms": round(float(np.percentile(one[50:], 50)), 4), "p99_ms": round(float(np.percentile(one[50:], 99)), 4), "calls": len(one) - 50,
                         "what": "query conversion + keyword kernel, device time of one call (copies and allocations of the harness not counted)"}
        line["keyword"] = kw
        lat1 = []
        for qi in range(120):
            cut1 = lambda c: (c.off[qi:qi + 2] - c.off[qi], c.idx[int(c.off[qi]):int(c.off[qi + 1])], c.val[int(c.off[qi]):int(c.off[qi + 1])])
            _, _, t1 = res.search(qd[qi:qi + 1], cut1(qs), cut1(qb), cands, 7)
            lat1.append(t1 * 1e3)
        line["latency_batch1_ms"] = round(float(np.median(lat1[20:])), 4)
    res.close()
    if not quick:
        del D, S, B, corpus
        torch.cuda.empty_cache()
        # the 10k-document configuration
        c0 = synth.make_corpus(10_000, seed=20261150, device=dev)
        q0 = synth.make_queries(1_000, c0.idf, seed=20261151, device=dev)
        D0, S0, B0, QD0, QS0, QB0 = host(c0, q0)
        b0 = apoe_ref.build(D0, c3(S0), c3(B0))
        e0 = orc.effective_weights(D0, S0, B0, QD0, QS0, QB0, 1.0, 1.0, 1.0)
        a1, a2, a3 = orc.scale_queries(QD0, QS0, QB0, *e0)
        r0 = apoe_ref.Resident(D0, c3(S0), c3(B0), clean(b0["graph"]), b0["ep"])
        for _ in range(3):
            i0, _, t0 = r0.search(a1, c3(a2), c3(a3), cands, 7)
        r0.close()
        cfg0 = {"docs": 10_000, "queries": 1_000, "cands": cands, "build_seconds": round(b0["seconds"], 4), "qps": round(1_000 / t0, 1)}
        try:
            cfg0["recall_at_10"] = round(recall_at_10(i0, exact_gt(c0, q0, e0)), 4)
        except Exception:   # noqa: BLE001
            pass
        line["config0"] = cfg0
        if args.ingest_docs > 0:
            line["ingest"] = ingest_reference(min(args.ingest_docs, n), dev)
        # supplementary corpus with neighbourhoods (see section_supplementary)
        cs = synth.make_clustered_corpus(n, device=dev)
        qs_ = synth.make_clustered_queries(nq, cs)
        Ds, Ss, Bs, QDs, QSs, QBs = host(cs, qs_)
        bs = apoe_ref.build(Ds, c3(Ss), c3(Bs))
        es = orc.effective_weights(Ds, Ss, Bs, QDs, QSs, QBs, 1.0, 1.0, 1.0)
        s1, s2, s3 = orc.scale_queries(QDs, QSs, QBs, *es)
        sup = {"corpus": SUPPLEMENTARY_LABEL.format(n=n, nq=nq), "build_seconds": round(bs["seconds"], 3)}
        try:
            gs = exact_gt(cs, qs_, es)
            rs = apoe_ref.Resident(Ds, c3(Ss), c3(Bs), clean(bs["graph"]), bs["ep"])
            curve = []
            for cc in (32, 64, 128, 256, 512):
                i_c, _, t_c = rs.search(s1, c3(s2), c3(s3), cc, 7)
                curve.append({"cands": cc, "qps": round(nq / t_c, 1), "recall_at_10": round(recall_at_10(i_c, gs), 4)})
            ed = orc.effective_weights(Ds, Ss, Bs, QDs, QSs, QBs, 0.0, 0.0, 1.0)
            d1, d2, d3 = orc.scale_queries(QDs, QSs, QBs, *ed)
            gd = exact_gt(cs, qs_, ed)
            curve_d = []
            for cc in (32, 64, 96, 128, 256, 512):
                i_c, _, t_c = rs.search(d1, c3(d2), c3(d3), cc, 1)
                curve_d.append({"cands": cc, "qps": round(nq / t_c, 1), "recall_at_10": round(recall_at_10(i_c, gd), 4)})
            sup["dense_only"] = {"weights_dense_sparse_bm25": "1/0/0", "graph": "the same hybrid graph", "curve": curve_d, "qps_at_recall_0.95": first_reaching(curve_d)}
            rs.close()
            sup["curve"] = curve
            sup["qps_at_recall_0.95"] = first_reaching(curve)
            sup["qps_at_recall_0.90"] = first_reaching(curve, 0.90)
            sup["qps_at_recall_0.75"] = first_reaching(curve, 0.75)
        except Exception as e:   # noqa: BLE001
            sup["error"] = str(e)
        line["supplementary"] = sup
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: this benchmark has no CPU path"}))
        sys.exit(1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
