#!/usr/bin/env python
"""Benchmark of the hybrid graph index hot path: batched search QPS (cands = 128) and index build seconds.

Own arm (default): 1M synthetic documents / 10k queries per GPU, weights 1/1/1, cands 128, top_k 10.  A step is one
search pass over the rank's query batch.  `value` is measured with queries and index resident in device memory,
`e2e` through the host-pointer call (pinned host query buffers in, host results out, copies inside the timed region).
Reference arm (--impl reference): the reference's own CUDA kernels (oracle/_ref, built from the reference tree
where it is mounted) on the same corpus, its own timed region (corpus + query fp16 conversion and the search kernel).

Multi-GPU (torchrun): query-parallel over a replicated index, weak scaling (every rank searches its own batch of the
same size); no collective in the data path.  --mode sharded runs the corpus-sharded variant instead (each rank owns
1/N of the corpus and builds its own graph; per-query shard results are all-gathered over NCCL and merged on device).
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
# DRAM bytes / algorithmic bytes of the search kernel (dram__bytes_read.sum + dram__bytes_write.sum of one launch over
# the kernel's counted bytes), from the ncu capture of the 200k-document case summarised under profiles/; the full-size
# launch is scaled by this ratio (both grow with the number of fused distances)
TRAFFIC_RATIO = 0.864


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
    ap.add_argument("--cpu-queries", type=int, default=256, help="queries of the bounded CPU brute-force sample")
    ap.add_argument("--ref-queries", type=int, default=2000, help="queries per step of the reference arm")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--ingest-docs", type=int, default=200_000, help="documents of the file-ingest measurement (0 = skip it)")
    ap.add_argument("--curve", action="store_true", help="also sweep cands in {32,64,128,256} and the weight presets")
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


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def host_queries(q, a=0, b=None):
    """CPU copy (pinned) of query rows [a, b)."""
    import synth
    b = q.nq if b is None else b
    s = q.slice(a, b)
    pin = lambda t: t.cpu().pin_memory() if torch.cuda.is_available() else t.cpu()
    return synth.Queries(pin(s.dense), synth.Csr(pin(s.sparse.off), pin(s.sparse.idx), pin(s.sparse.val)),
                         synth.Csr(pin(s.bm25.off), pin(s.bm25.idx), pin(s.bm25.val)))


def recall_at_10(ids, gt):
    return float(np.mean([len(set(ids[i, :10].tolist()) & set(gt[i, :10].tolist())) / 10.0 for i in range(gt.shape[0])]))


def cpu_baseline(corpus_host, qsub, eff, threads_note=True):
    """Exact OpenMP brute-force hybrid top-10 (the CPU oracle) on a bounded query sample.  Returns (dict, gt ids)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import apoe_oracle as orc
    D, S, B = corpus_host
    ws, wb, wd = eff
    QS, QB = orc.CsrNp.from_torch(qsub.sparse), orc.CsrNp.from_torch(qsub.bm25)
    qd, qs, qb = orc.scale_queries(qsub.dense.numpy(), QS, QB, ws, wb, wd)
    t0 = time.time()
    gt, _, thr = orc.bruteforce(D, S, B, qd, qs, qb, 7, 10)
    dt = time.time() - t0
    n = qd.shape[0]
    return ({"value": n / dt, "unit": "queries/s", "cores": thr, "kind": "port",
             "sample": f"exact OpenMP brute-force hybrid top-10 of {n} queries over {D.shape[0]} docs in {dt:.1f} s "
                       f"(term-major sparse postings, blocked dense dot products)"}, gt)


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
            sys.stdout.flush()
            saved = os.dup(1)           # the reference's loaders print to stdout; this program's stdout is one JSON line
            null = os.open(os.devnull, os.O_WRONLY)
            os.dup2(null, 1)
            try:
                rows, t_load, t_all = apoe_ref.load_seconds(*paths)
            finally:
                os.dup2(saved, 1); os.close(saved); os.close(null)
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
    vocab = int(corpus.idf.numel()) if hasattr(corpus.idf, "numel") else int(idx.max()) + 1
    vocab = max(vocab, int(idx.max()) + 1)
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
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import apoe_oracle as orc
        m = min(off_h.size - 1, 100_000)
        e = int(off_h[m])
        t0 = time.time()
        orc.bm25_corpus(off_h[:m + 1], corpus.bm25.idx[:e].cpu().numpy(), tf[:e].cpu().numpy(), vocab, relabel_by_df=True)
        out["cpu_port"] = {"postings_per_s": round(e / (time.time() - t0)), "cores": 1, "sample": f"numpy restatement on the first {m} rows ({e} postings)"}
    return out


def algorithmic_bytes(st, nq, cands, qnnz):
    """Bytes the search must move by the per-query formula: query row, entry ids, 160-byte graph rows per expansion,
    one record (2048 dense bytes + 8 bytes per stored term, as fetched) per evaluation, cands x 8 result bytes."""
    rows_fetched = st.expansions * 512                       # the kernel's own count includes 512-byte locator rows
    records = st.gathered_bytes - rows_fetched
    return records + st.expansions * 160 + nq * (2 * DIM + 8 * qnnz + 128 + 8 * cands)


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
    mq = (int((queries.sparse.off[1:] - queries.sparse.off[:-1]).max()), int((queries.bm25.off[1:] - queries.bm25.off[:-1]).max()))

    if sharded:
        import dist_search
        top_k = 10
        a, _ = dist_search.shard_range(n, rank, world)
        g_ids = torch.empty(world, nq, cands, dtype=torch.int32, device=dev)
        g_dis = torch.empty(world, nq, cands, dtype=torch.float32, device=dev)
        m_ids = torch.empty(nq, top_k, dtype=torch.int32, device=dev)
        m_dis = torch.empty(nq, top_k, dtype=torch.float32, device=dev)

        def step():
            ix.search_device(queries, out_ids, out_dis, cands=cands, weights=eff, max_nnz=mq, stream=stream, stats=False)
            dist_search.gather_and_merge(out_ids, out_dis, a, g_ids, g_dis, m_ids, m_dis, top_k)
    else:
        def step():
            ix.search_device(queries, out_ids, out_dis, cands=cands, weights=eff, max_nnz=mq, stream=stream, stats=False)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
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

    line = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        algo = algorithmic_bytes(st, nq, cands, mq[0] + mq[1])
        achieved = algo / (st.kernel_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                "traffic": (round(TRAFFIC_RATIO * algo) if TRAFFIC_RATIO else None), "peak_kind": f"of {peak_kind}",
                "kernel": "search_kernel<dense|sparse|bm25>", "kernel_ms": round(st.kernel_ms, 3),
                "algorithmic_bytes_per_launch": int(algo), "expansions_per_query": round(st.expansions / nq, 1),
                "evaluations_per_query": round(st.evaluations / nq, 1)}
        cpu, recall = None, None
        if not args.skip_cpu and not sharded and world == 1:
            D = corpus.dense.cpu().numpy()
            sys.path.insert(0, os.path.join(ROOT, "oracle"))
            import apoe_oracle as orc
            S, B = orc.CsrNp.from_torch(corpus.sparse), orc.CsrNp.from_torch(corpus.bm25)
            qsub = host_queries(queries, 0, min(nq, args.cpu_queries))
            cpu, gt = cpu_baseline((D, S, B), synth.Queries(qsub.dense, qsub.sparse, qsub.bm25), eff)
            recall = recall_at_10(out_ids[:gt.shape[0]].cpu().numpy().view(np.uint32), gt)
        line = {
            "metric": "hybrid search QPS at recall@10>=0.95 (cands=128); index build sec per 1M docs",
            "value": round(total_q * args.steps / (ms_max * 1e-3), 1), "unit": "queries/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_max / args.steps, 3), "higher_is_better": True,
            "scaling": "strong" if sharded else "weak", "vs_baseline": None, "dtype": "f16 storage, f16 dense accumulate + f32 sparse (as the reference)",
            "data": "synthetic (seeded generators with the benchmark's shapes and value distributions)",
            "config": {"workload": f"{n} docs / {nq} queries per GPU, weights 1/1/1, top_k 10, cands {cands}", "docs": n,
                       "queries_per_gpu": nq, "cands": cands, "mode": args.mode if world > 1 else "single",
                       "l2": "inputs larger than L2 (records pool %.1f GB, random gathers)" % (n * 3.5e-6),
                       "parallelism": f"{'corpus-sharded' if sharded else 'query-parallel replicas'} x{world}"},
            "e2e": {"value": round(total_q * args.steps / (e2e_ms_max * 1e-3), 1), "unit": "queries/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h)},
            "gpu_launches": args.steps * (2 if sharded else 1),
            "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
            "recall_at_10": recall, "effective_weights": {"sparse": eff[0], "bm25": eff[1], "dense": eff[2]},
            "build": {"seconds": round(bst.seconds_total, 3), "seconds_per_1M_docs": round(bst.seconds_total * 1e6 / (corpus.n), 3),
                      "knn_seconds": round(bst.seconds_knn, 3), "prune_seconds": round(bst.seconds_prune, 3),
                      "iterations": bst.iterations_run, "distance_evals": int(bst.distance_evals)},
            "setup_seconds": {"generate": round(t_gen, 2)},
        }
        if args.curve and not sharded:
            line["curve"] = curve(ix, queries, eff, mq, gt if cpu else None, dev, stream)
            line["variants"] = variants(ix, queries, eff, mq, dev, stream, n, cands)
        # single-query latency (kernel time by CUDA events, device-resident query), median of 30 different queries
        lat = []
        o1 = torch.empty(1, cands, dtype=torch.int32, device=dev); d1 = torch.empty(1, cands, dtype=torch.float32, device=dev)
        for qi in range(min(30, nq)):
            st1 = ix.search_device(queries.slice(qi, qi + 1), o1, d1, cands=cands, weights=eff, max_nnz=mq, stream=stream, stats=True)
            lat.append(st1.kernel_ms)
        line["latency_batch1_ms"] = round(float(np.median(lat)), 4)
        if world == 1 and args.ingest_docs > 0:
            ix.close()   # the measurement wants the memory and the copy engines to itself
            line["ingest"] = ingest_own(min(args.ingest_docs, n), dev)
            line["prep"] = prep_bench(corpus, dev, peak, not args.skip_cpu)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def curve(ix, queries, eff, mq, gt, dev, stream):
    out = []
    nq = queries.nq
    for cands in (32, 64, 128, 256):
        oi = torch.empty(nq, cands, dtype=torch.int32, device=dev)
        od = torch.empty(nq, cands, dtype=torch.float32, device=dev)
        for _ in range(2):
            st = ix.search_device(queries, oi, od, cands=cands, weights=eff, max_nnz=mq, stream=stream)
        rec = recall_at_10(oi[:gt.shape[0]].cpu().numpy().view(np.uint32), gt) if gt is not None else None
        out.append({"cands": cands, "qps": round(nq / st.kernel_ms * 1e3, 1), "recall_at_10": rec})
    return out


def flag_keywords(queries_host, synth):
    """Query BM25 ids with bit 31 set on the required terms (ref: src/query.cu:1828-1843), as a numpy array."""
    kws = synth.make_keywords(queries_host)
    off = queries_host.bm25.off.numpy().astype(np.int64)
    idx = queries_host.bm25.idx.numpy().astype(np.uint32)
    for q, req in enumerate(kws):
        row = idx[off[q]:off[q + 1]]
        row[np.isin(row, np.asarray(req, dtype=np.uint32))] |= np.uint32(0x80000000)
    return idx


def variants(ix, queries, eff, mq, dev, stream, n, cands):
    """The keyword-constrained and the knowledge-graph searches on the benchmark corpus (kernel time, resident queries)."""
    import apoe
    import synth
    nq = queries.nq
    out = {}
    oi = torch.empty(nq, cands, dtype=torch.int32, device=dev); od = torch.empty(nq, cands, dtype=torch.float32, device=dev)
    qh = host_queries(queries)
    kq = synth.Queries(queries.dense, queries.sparse, synth.Csr(queries.bm25.off, torch.from_numpy(flag_keywords(qh, synth).view(np.int32)).to(dev), queries.bm25.val))
    for _ in range(2):
        st = ix.search_device(kq, oi, od, cands=cands, weights=eff, max_nnz=mq, stream=stream, flags=apoe.SEARCH_KEYWORD)
    out["keyword"] = {"qps": round(nq / st.kernel_ms * 1e3, 1), "cands": cands, "queries": nq, "what": "1-4 required BM25 terms per query, keyword-edge recycling on"}
    kg = synth.make_kg(n, nq, device=dev)
    ix.set_kg(kg.e2e_off, kg.e2e_idx, kg.e2d_off, kg.e2d_idx)
    for _ in range(2):
        st = ix.search_device(queries, oi, od, cands=cands, weights=eff, max_nnz=mq, stream=stream, kg_weight=40.0, ent=(kg.qe_off, kg.qe_idx))
    out["kg"] = {"qps": round(nq / st.kernel_ms * 1e3, 1), "cands": cands, "queries": nq, "what": "500 k entities, 1-3 seed entities per query, kg_weight 40"}
    return out


def run_reference(args):
    """The reference's own CUDA kernels on the same corpus and queries; rank 0 only."""
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
    import apoe_oracle as orc
    import synth
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    n, cands = min(args.docs, 1_000_000), args.cands     # the reference's static arrays hold 1M points (src/index.cu:10)
    nq = min(args.queries, args.ref_queries)
    corpus = synth.make_corpus(n, device=dev)
    queries = synth.make_queries(args.queries, corpus.idf, device=dev)
    D = corpus.dense.cpu().numpy()
    S, B = orc.CsrNp.from_torch(corpus.sparse), orc.CsrNp.from_torch(corpus.bm25)
    QD = queries.dense.cpu().numpy()
    QS, QB = orc.CsrNp.from_torch(queries.sparse), orc.CsrNp.from_torch(queries.bm25)
    del corpus
    torch.cuda.empty_cache()
    c3 = lambda c: (c.off, c.idx, c.val)
    built = apoe_ref.build(D, c3(S), c3(B))
    graph = built["graph"].copy()
    graph[:, 33:] = np.where(np.arange(33, 40)[None, :] - 33 < graph[:, 32:33], graph[:, 33:], 0)
    eff = orc.effective_weights(D, S, B, QD, QS, QB, 1.0, 1.0, 1.0)
    qd, qs, qb = orc.scale_queries(QD, QS, QB, *eff)
    sub = lambda c: (c.off[:nq + 1], c.idx[:int(c.off[nq])], c.val[:int(c.off[nq])])
    sampler = ClockSampler(local)
    secs, secs_k = [], []
    for i in range(max(args.warmup, 1) + args.steps):
        if i == max(args.warmup, 1):
            sampler.start()
        ids, dis, t_all, t_search = apoe_ref.search(D, c3(S), c3(B), qd[:nq], sub(qs), sub(qb), graph, built["ep"], cands, 7)
        if i >= max(args.warmup, 1):
            secs.append(t_all)
            secs_k.append(t_search)
    clocks = sampler.stop()
    total = float(np.sum(secs))
    recall = None
    if not args.skip_cpu:
        m = min(nq, args.cpu_queries)
        gt, _, _ = orc.bruteforce(D, S, B, qd[:m], orc.CsrNp(*sub(qs)), orc.CsrNp(*sub(qb)), 7, 10)
        recall = recall_at_10(ids[:m], gt[:m])
    qps = nq * args.steps / total
    ref_curve = None
    if args.curve:   # the reference's kernels over its own graph at the other pool sizes (kernel-only time)
        ref_curve = []
        m = min(nq, args.cpu_queries)
        gt_c = None if args.skip_cpu else orc.bruteforce(D, S, B, qd[:m], orc.CsrNp(*sub(qs)), orc.CsrNp(*sub(qb)), 7, 10)[0]
        for cc in (32, 64, 128, 256):
            for _ in range(2):
                ids_c, _, t_all_c, t_search_c = apoe_ref.search(D, c3(S), c3(B), qd[:nq], sub(qs), sub(qb), graph, built["ep"], cc, 7)
            ref_curve.append({"cands": cc, "qps_kernel_only": round(nq / t_search_c, 1), "qps": round(nq / t_all_c, 1),
                              "recall_at_10": recall_at_10(ids_c[:m], gt_c[:m]) if gt_c is not None else None})
    ref_variants = None
    if args.curve:   # the reference's keyword kernel on the same flagged queries (its KG kernel is not run: it reads an unset index)
        class _Q:   # host queries in the shape flag_keywords expects
            pass
        qh = _Q(); qh.bm25 = _Q(); qh.nq = nq
        qh.bm25.off = torch.from_numpy(QB.off[:nq + 1].astype(np.int64)); qh.bm25.idx = torch.from_numpy(QB.idx[:int(QB.off[nq])].astype(np.int64))
        kidx = flag_keywords(qh, synth)
        for _ in range(2):
            _, _, t_all_k, t_search_k = apoe_ref.search(D, c3(S), c3(B), qd[:nq], sub(qs), (qb.off[:nq + 1], kidx, qb.val[:int(qb.off[nq])]), graph, built["ep"], cands, 7 | 8)
        ref_variants = {"keyword": {"qps_kernel_only": round(nq / t_search_k, 1), "qps": round(nq / t_all_k, 1), "cands": cands, "queries": nq}}
    lat1 = []
    one = lambda c, i: (c.off[i:i + 2] - c.off[i], c.idx[int(c.off[i]):int(c.off[i + 1])], c.val[int(c.off[i]):int(c.off[i + 1])])
    for qi in range(min(10, nq)):
        _, _, _, t1 = apoe_ref.search(D, c3(S), c3(B), qd[qi:qi + 1], one(qs, qi), one(qb, qi), graph, built["ep"], cands, 7)
        lat1.append(t1 * 1e3)
    ingest = ingest_reference(min(args.ingest_docs, n), torch.device("cuda", local)) if args.ingest_docs > 0 else None
    print(json.dumps({
        "ingest": ingest, "curve": ref_curve, "variants": ref_variants, "latency_batch1_ms": round(float(np.median(lat1)), 4),
        "impl": "reference", "metric": "hybrid search QPS at recall@10>=0.95 (cands=128); index build sec per 1M docs",
        "value": round(qps, 1), "unit": "queries/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 1),
        "ms_per_step": round(total / args.steps * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 storage, f16 dense accumulate + f32 sparse", "data": "synthetic (same generators and seeds as the own arm)",
        "config": {"workload": f"{n} docs / {nq} queries per step, weights 1/1/1, top_k 10, cands {cands}", "docs": n,
                   "queries_per_step": nq, "cands": cands,
                   "timed_region": "the reference's own: fp32->fp16 conversion of corpus and queries + search kernel (src/query.cu:1999-2051)"},
        "e2e": {"value": round(qps, 1), "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "cpu_baseline": {"value": round(qps, 1), "unit": "queries/s", "cores": 0, "kind": "reference",
                         "sample": f"the reference's CUDA kernels (oracle/_ref) on GPU {local}: {nq} queries per step; it has no CPU path"},
        "search_kernel_only_qps": round(nq * args.steps / float(np.sum(secs_k)), 1),
        "recall_at_10": recall, "clocks": clocks, "gpu_launches": 0,
        "build": {"seconds": round(built["seconds"], 3), "seconds_per_1M_docs": round(built["seconds"] * 1e6 / n, 3)},
    }), flush=True)


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
