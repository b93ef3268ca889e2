"""Generates the golden fixtures of tests/golden/ by running the reference's own CUDA kernels (oracle/_ref) on a
GPU, on seeded synthetic inputs that the tests regenerate from the same seeds.

Run on a CUDA machine, from the repository root, after `make -C oracle ref` has been run where the reference
tree is mounted:   python tests/golden/make_golden.py <output directory>
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
for p in ("allan-poe_b200", "oracle", "tests"):
    sys.path.insert(0, os.path.join(ROOT, p))
import apoe_oracle as orc  # noqa: E402
import apoe_ref  # noqa: E402
import helpers  # noqa: E402
import synth  # noqa: E402

BUILD_N, BUILD_SEED = 1024, 101
SEARCH_N, SEARCH_Q, SEARCH_SEED = 2000, 100, 202


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def csr3(c):
    return (c.off, c.idx, c.val)


def main(outdir):
    os.makedirs(outdir, exist_ok=True)
    # ---- build state of the reference on a small corpus -----------------------------------------------
    ds = helpers.make_dataset(BUILD_N, 8, seed=BUILD_SEED, with_graph=False)
    st = apoe_ref.build(ds.D, csr3(ds.S), csr3(ds.B))
    np.savez_compressed(os.path.join(outdir, "ref_build.npz"), inputs=digest(ds.D, ds.S.idx, ds.S.val, ds.B.idx, ds.B.val),
                        knn=st["knn"], knn_dis=st["knn_dis"], power=st["power"], new_list=st["new_list"], kw=st["kw"],
                        graph=st["graph"], ep=st["ep"])
    print("build fixture: seconds", st["seconds"])

    # ---- search results of the reference on its own graph -----------------------------------------------
    ds = helpers.make_dataset(SEARCH_N, SEARCH_Q, seed=SEARCH_SEED, with_graph=False)
    st = apoe_ref.build(ds.D, csr3(ds.S), csr3(ds.B))
    graph, ep = st["graph"].copy(), st["ep"]
    graph[:, 33:] = np.where(np.arange(33, 40)[None, :] - 33 < graph[:, 32:33], graph[:, 33:], 0)  # unwritten slots are stale memory
    out = dict(inputs=digest(ds.D, ds.S.idx, ds.S.val, ds.B.idx, ds.B.val, ds.QD, ds.QS.idx, ds.QS.val, ds.QB.idx, ds.QB.val),
               graph=graph, ep=ep)
    combos = {"three": ((1.0, 1.0, 1.0), 7, SEARCH_Q, 128), "dense": ((0.0, 0.0, 1.0), 1, 32, 64), "sparse": ((1.0, 0.0, 0.0), 2, 32, 64),
              "bm25": ((0.0, 1.0, 0.0), 4, 32, 64), "dense_sparse": ((1.0, 0.0, 1.0), 3, 32, 64), "dense_bm25": ((0.0, 1.0, 1.0), 5, 32, 64),
              "sparse_bm25": ((1.0, 1.0, 0.0), 6, 32, 64), "skewed": ((1.0, 2.0, 0.5), 7, 32, 256)}
    verdict = {}
    for name, (w, mode, nq, cands) in combos.items():
        eff = orc.effective_weights(ds.D, ds.S, ds.B, ds.QD, ds.QS, ds.QB, *w)
        qd, qs, qb = orc.scale_queries(ds.QD, ds.QS, ds.QB, *eff)
        sub = lambda c: (c.off[:nq + 1], c.idx[:int(c.off[nq])], c.val[:int(c.off[nq])])
        ids, dis, _, _ = apoe_ref.search(ds.D, csr3(ds.S), csr3(ds.B), qd[:nq], sub(qs), sub(qb), graph, ep, cands, mode)
        out[name + "_ids"], out[name + "_dis"] = ids, dis
        out[name + "_eff"] = np.asarray(eff, dtype=np.float32)
        # which arithmetic does the oracle need to reproduce this bit for bit?
        for flags, tag in ((0, "hfma2+ffma"), (orc.F_UNFUSED_DENSE, "hmul2/hadd2+ffma"), (orc.F_NOFMA_SPARSE, "hfma2+fmul/fadd"),
                           (orc.F_UNFUSED_DENSE | orc.F_NOFMA_SPARSE, "hmul2/hadd2+fmul/fadd")):
            oi, od, _ = orc.search(ds.Dh, ds.S, ds.B, orc.f2h(qd[:nq]), orc.CsrNp(*sub(qs)), orc.CsrNp(*sub(qb)), graph, ep, cands, mode | flags)
            same_ids = float(np.mean(oi == ids))
            same_dis = float(np.mean(od.view(np.uint32) == dis.view(np.uint32)))
            verdict.setdefault(tag, []).append((name, same_ids, same_dis))
            print(f"{name:13s} {tag:24s} ids equal {same_ids:.4f} dis equal {same_dis:.4f}", flush=True)
    # keyword kernel
    kws = synth.make_keywords(ds.queries, seed=5)
    qb_idx = ds.QB.idx.copy()
    for q, req in enumerate(kws):
        for j in range(int(ds.QB.off[q]), int(ds.QB.off[q + 1])):
            if int(qb_idx[j]) in req:
                qb_idx[j] |= np.uint32(0x80000000)
    QBk = orc.CsrNp(ds.QB.off, qb_idx, ds.QB.val)
    eff = orc.effective_weights(ds.D, ds.S, ds.B, ds.QD, ds.QS, QBk, 1.0, 1.0, 1.0)
    qd, qs, qb = orc.scale_queries(ds.QD, ds.QS, QBk, *eff)
    ids, dis, _, _ = apoe_ref.search(ds.D, csr3(ds.S), csr3(ds.B), qd, csr3(qs), csr3(qb), graph, ep, 128, 15)
    out["keyword_ids"], out["keyword_dis"], out["keyword_eff"] = ids, dis, np.asarray(eff, dtype=np.float32)
    oi, od, _ = orc.search(ds.Dh, ds.S, ds.B, orc.f2h(qd), qs, qb, graph, ep, 128, 7 | orc.F_KEYWORD)
    print("keyword: top-10 ids equal", float(np.mean(oi[:, :10] == ids[:, :10])), "all", float(np.mean(oi == ids)))
    np.savez_compressed(os.path.join(outdir, "ref_search.npz"), **out)
    for tag, rows in verdict.items():
        print(tag, "mean ids", np.mean([r[1] for r in rows]), "mean dis", np.mean([r[2] for r in rows]))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden"))
