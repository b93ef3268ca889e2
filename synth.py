"""Seeded synthetic corpora, queries, knowledge graphs and keyword files.

The generators follow the shapes and value distributions of the benchmark
configurations (dense 1024-d unit vectors; learned-sparse rows over a 30 522
term vocabulary with Zipf(1.1) term ids and log-normal values; BM25 rows over a
100 000 term vocabulary with Zipf(1.0) ids, tf = 1 + Geometric(0.6) and
k1 = 1.2, b = 0.75 weights) and write them in the byte formats the reference
loaders read (include/utils.cuh:361-398, src/query.cu:35-108).

Everything is torch code that runs on CPU (tests) or on a GPU (benchmark), so a
1M-document corpus can be produced directly in device memory.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch

DIM = 1024
SPARSE_VOCAB = 30522
BM25_VOCAB = 100000
MAX_SPARSE = 550   # row capacities of the reference kernels (src/query.cu:13-14)
MAX_BM25 = 780


@dataclass
class Csr:
    off: torch.Tensor   # int32 (bit pattern of u32), rows + 1
    idx: torch.Tensor   # int32
    val: torch.Tensor   # float32

    @property
    def rows(self) -> int:
        return self.off.numel() - 1

    def to(self, device) -> "Csr":
        return Csr(self.off.to(device), self.idx.to(device), self.val.to(device))

    def slice_rows(self, a: int, b: int) -> "Csr":
        lo, hi = int(self.off[a]), int(self.off[b])
        return Csr((self.off[a:b + 1] - lo).contiguous(), self.idx[lo:hi].contiguous(), self.val[lo:hi].contiguous())


@dataclass
class Corpus:
    dense: torch.Tensor          # [n, 1024] float32, unit rows
    sparse: Csr
    bm25: Csr
    idf: torch.Tensor            # [BM25_VOCAB] float32 (for query weights)
    extra: dict = field(default_factory=dict)

    @property
    def n(self) -> int:
        return self.dense.shape[0]


@dataclass
class Queries:
    dense: torch.Tensor
    sparse: Csr
    bm25: Csr

    @property
    def nq(self) -> int:
        return self.dense.shape[0]

    def slice(self, a: int, b: int) -> "Queries":
        return Queries(self.dense[a:b].contiguous(), self.sparse.slice_rows(a, b), self.bm25.slice_rows(a, b))


def _zipf_cdf(vocab: int, s: float, device) -> torch.Tensor:
    r = torch.arange(1, vocab + 1, dtype=torch.float64, device=device)
    p = r.pow(-s)
    return (p.cumsum(0) / p.sum()).to(torch.float64)


def _zipf_rows(counts: torch.Tensor, vocab: int, s: float, gen: torch.Generator, oversample: float = 2.5):
    """Per row, `counts[i]` distinct Zipf-distributed term ids in ascending order.

    Draws `oversample * count + 8` ids with replacement, removes duplicates and
    keeps a random subset of the requested size (fewer if the draws held fewer
    distinct ids).  Returns (row_offsets int64 [rows+1], term ids int64).
    """
    device = counts.device
    rows = counts.numel()
    cdf = _zipf_cdf(vocab, s, device)
    draws = (counts.to(torch.float64) * oversample).ceil().to(torch.int64) + 8
    total = int(draws.sum())
    row_of = torch.repeat_interleave(torch.arange(rows, device=device), draws)
    u = torch.rand(total, generator=gen, device=device, dtype=torch.float64)
    term = torch.searchsorted(cdf, u).clamp_(max=vocab - 1)
    key = torch.unique(row_of * vocab + term)           # sorted (row, term), duplicates removed
    row_u = key // vocab
    n_u = torch.bincount(row_u, minlength=rows)
    # random priority inside each row; keep the `counts[row]` smallest
    pr = torch.rand(key.numel(), generator=gen, device=device, dtype=torch.float64)
    order = torch.argsort(row_u.to(torch.float64) + pr * 0.999999)
    start = torch.cumsum(n_u, 0) - n_u
    rank = torch.empty_like(order)
    rank[order] = torch.arange(key.numel(), device=device) - start[row_u[order]]
    keep = rank < counts[row_u]
    key = key[keep]
    row_k = key // vocab
    n_k = torch.bincount(row_k, minlength=rows)
    off = torch.zeros(rows + 1, dtype=torch.int64, device=device)
    off[1:] = torch.cumsum(n_k, 0)
    return off, key % vocab


def _chunks(n: int, step: int):
    for a in range(0, n, step):
        yield a, min(n, a + step)


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def make_corpus(n: int, seed: int = 20261125, device="cpu", mean_sparse: float = 120.0, mean_bm25: float = 60.0,
                chunk: int = 100_000) -> Corpus:
    device = torch.device(device)
    g = _gen(seed, device)
    dense = torch.empty(n, DIM, dtype=torch.float32, device=device)
    for a, b in _chunks(n, chunk):
        x = torch.randn(b - a, DIM, generator=g, device=device, dtype=torch.float32)
        dense[a:b] = x / x.norm(dim=1, keepdim=True)

    def rows(mean, vocab, s, cap):
        offs, idxs = [], []
        base = 0
        for a, b in _chunks(n, chunk):
            cnt = torch.poisson(torch.full((b - a,), mean, device=device), generator=g).to(torch.int64).clamp_(1, cap)
            off, idx = _zipf_rows(cnt, vocab, s, g)
            offs.append(off[:-1] + base)
            base += int(off[-1])
            idxs.append(idx)
        off = torch.cat(offs + [torch.tensor([base], device=device)])
        return off, torch.cat(idxs)

    s_off, s_idx = rows(mean_sparse, SPARSE_VOCAB, 1.1, MAX_SPARSE)
    s_val = torch.exp(torch.randn(s_idx.numel(), generator=g, device=device) * 0.8 - 1.0).to(torch.float32)
    b_off, b_idx = rows(mean_bm25, BM25_VOCAB, 1.0, MAX_BM25)
    # tf = 1 + Geometric(0.6) failures-before-success
    uu = torch.rand(b_idx.numel(), generator=g, device=device, dtype=torch.float64).clamp_(min=1e-12)
    tf = 1.0 + torch.floor(torch.log(uu) / math.log(1.0 - 0.6))
    row_of = torch.repeat_interleave(torch.arange(n, device=device), (b_off[1:] - b_off[:-1]))
    length = torch.zeros(n, dtype=torch.float64, device=device).index_add_(0, row_of, tf)
    avglen = length.mean()
    df = torch.bincount(b_idx, minlength=BM25_VOCAB).to(torch.float64)
    idf = torch.log(1.0 + (n - df + 0.5) / (df + 0.5))
    k1, bb = 1.2, 0.75
    w = idf[b_idx] * tf * (k1 + 1.0) / (tf + k1 * (1.0 - bb + bb * length[row_of] / avglen))
    return Corpus(dense,
                  Csr(s_off.to(torch.int32), s_idx.to(torch.int32), s_val),
                  Csr(b_off.to(torch.int32), b_idx.to(torch.int32), w.to(torch.float32)),
                  idf.to(torch.float32))


def make_queries(nq: int, corpus_idf: torch.Tensor, seed: int = 20261126, device="cpu", nnz_sparse: int = 30,
                 nnz_bm25: int = 8) -> Queries:
    device = torch.device(device)
    g = _gen(seed, device)
    x = torch.randn(nq, DIM, generator=g, device=device, dtype=torch.float32)
    dense = x / x.norm(dim=1, keepdim=True)
    s_off, s_idx = _zipf_rows(torch.full((nq,), nnz_sparse, dtype=torch.int64, device=device), SPARSE_VOCAB, 1.1, g, 4.0)
    s_val = torch.exp(torch.randn(s_idx.numel(), generator=g, device=device) * 0.8 - 1.0).to(torch.float32)
    b_off, b_idx = _zipf_rows(torch.full((nq,), nnz_bm25, dtype=torch.int64, device=device), BM25_VOCAB, 1.0, g, 4.0)
    b_val = corpus_idf.to(device)[b_idx].to(torch.float32)
    return Queries(dense, Csr(s_off.to(torch.int32), s_idx.to(torch.int32), s_val),
                   Csr(b_off.to(torch.int32), b_idx.to(torch.int32), b_val))


# ---------------------------------------------------------------------------
# Supplementary corpus with neighbourhoods.  The benchmark's prescribed dense vectors are i.i.d. points on the unit
# sphere: no document has real neighbours, and no graph index reaches a high recall on them.  This generator keeps
# every shape and value distribution of the prescribed one (unit 1024-d dense rows; Zipf term ids, log-normal sparse
# values, BM25 weights from tf / df with k1 = 1.2, b = 0.75; the same row lengths) but draws documents from a mixture:
# a document belongs to one of n / cluster_size topics, its dense row is the topic's centre plus noise, and a share of
# its sparse and BM25 terms comes from the topic's own term list.  Queries are perturbed documents: the dense row of
# a random document plus noise, 30 of its sparse terms and 8 of its BM25 terms.
# ---------------------------------------------------------------------------
def _subsample_rows(row_of: torch.Tensor, rows: int, keep: torch.Tensor, gen: torch.Generator) -> torch.Tensor:
    """Boolean mask over items (grouped by `row_of`, ascending) that keeps `keep[row]` random items of every row."""
    device = row_of.device
    n_items = torch.bincount(row_of, minlength=rows)
    pr = torch.rand(row_of.numel(), generator=gen, device=device, dtype=torch.float64)
    order = torch.argsort(row_of.to(torch.float64) + pr * 0.999999)
    start = torch.cumsum(n_items, 0) - n_items
    rank = torch.empty_like(order)
    rank[order] = torch.arange(row_of.numel(), device=device) - start[row_of[order]]
    return rank < keep[row_of]


def _topic_rows(counts, topic_of_row, topic_terms, share, vocab, s, gen, oversample=2.5, second_topic=None, second_share=0.0):
    """Like _zipf_rows, but a `share` of every row's draws comes from its topic's term list (a `second_share` of those
    from the list of the row's second topic, when it has one)."""
    device = counts.device
    rows = counts.numel()
    cdf = _zipf_cdf(vocab, s, device)
    draws = (counts.to(torch.float64) * oversample).ceil().to(torch.int64) + 8
    total = int(draws.sum())
    row_of = torch.repeat_interleave(torch.arange(rows, device=device), draws)
    u = torch.rand(total, generator=gen, device=device, dtype=torch.float64)
    term = torch.searchsorted(cdf, u).clamp_(max=vocab - 1)
    from_topic = torch.rand(total, generator=gen, device=device) < share
    pick = torch.randint(0, topic_terms.shape[1], (total,), generator=gen, device=device)
    which = topic_of_row[row_of]
    if second_topic is not None and second_share > 0:
        which = torch.where(torch.rand(total, generator=gen, device=device) < second_share, second_topic[row_of], which)
    term = torch.where(from_topic, topic_terms[which, pick], term)
    key = torch.unique(row_of * vocab + term)
    row_u = key // vocab
    keep = _subsample_rows(row_u, rows, counts, gen)
    key = key[keep]
    n_k = torch.bincount(key // vocab, minlength=rows)
    off = torch.zeros(rows + 1, dtype=torch.int64, device=device)
    off[1:] = torch.cumsum(n_k, 0)
    return off, key % vocab


def make_clustered_corpus(n: int, seed: int = 20261201, device="cpu", cluster_size: int = 100, dense_noise: float = 0.6,
                          topic_share: float = 0.6, topic_terms: int = 256, mean_sparse: float = 120.0, mean_bm25: float = 60.0,
                          chunk: int = 100_000, group_size: int = 10_000, group_noise: float = 0.7, group_share: float = 0.5,
                          latent_dim: int = 0, mix: float = 0.0) -> Corpus:
    """mix > 0: every document also belongs, with that weight, to a second topic (a sibling of its group when topics are
    grouped): its dense row is centre + mix x second centre + noise and a share mix / (1 + mix) of its topic terms comes
    from the second topic's list.  Documents that span two topics are what ties the neighbourhoods of a real
    collection together; without them every topic is an island in the k-NN graph.
    latent_dim > 0: documents lie near a low-dimensional manifold instead of around isolated centres -- a latent
    point z ~ N(0, I) of that dimension is mapped into the 1024-d space by a fixed random matrix and perturbed by
    `dense_noise`; a document's topic is the nearest of n / cluster_size anchor points in the latent space and topics
    are grouped by the nearest of n / group_size coarser anchors, so neighbouring topics are neighbours in the dense
    space too (neighbourhoods overlap, as they do in real collections).
    group_size > 0 adds a level: topics come in groups of group_size / cluster_size siblings whose centres are a group
    centre plus noise and whose term lists share `group_share` of their terms with the group's list (a hierarchy, as
    real collections have: it is what lets a greedy search descend from far away)."""
    device = torch.device(device)
    g = _gen(seed, device)
    topics = max(1, n // cluster_size)
    centres = torch.randn(topics, DIM, generator=g, device=device)
    centres = centres / centres.norm(dim=1, keepdim=True)
    groups, group_of_topic = 0, None
    if group_size > 0:
        groups = max(1, n // group_size)
        gc = torch.randn(groups, DIM, generator=g, device=device)
        gc = gc / gc.norm(dim=1, keepdim=True)
        group_of_topic = torch.randint(0, groups, (topics,), generator=g, device=device)
        centres = gc[group_of_topic] + group_noise * centres
        centres = centres / centres.norm(dim=1, keepdim=True)
    topic_of = torch.randint(0, topics, (n,), generator=g, device=device)
    second_of = None
    dense = torch.empty(n, DIM, dtype=torch.float32, device=device)
    if latent_dim > 0:
        lift = torch.randn(latent_dim, DIM, generator=g, device=device) / math.sqrt(DIM)
        anchors = torch.randn(topics, latent_dim, generator=g, device=device)
        anchors = anchors / anchors.norm(dim=1, keepdim=True)
        if group_size > 0:
            coarse = torch.randn(groups, latent_dim, generator=g, device=device)
            group_of_topic = torch.argmax(anchors @ (coarse / coarse.norm(dim=1, keepdim=True)).T, dim=1)
        for a, b in _chunks(n, min(chunk, 20_000)):
            z = torch.randn(b - a, latent_dim, generator=g, device=device)
            zn = z / z.norm(dim=1, keepdim=True)
            topic_of[a:b] = torch.argmax(zn @ anchors.T, dim=1)
            x = zn @ lift
            x = x / x.norm(dim=1, keepdim=True)
            e = torch.randn(b - a, DIM, generator=g, device=device)
            x = x + dense_noise * e / e.norm(dim=1, keepdim=True)
            dense[a:b] = x / x.norm(dim=1, keepdim=True)
    else:
        if mix > 0:
            if groups:   # a sibling: a random topic of the same group (topics sorted by group, one draw inside the group's span)
                order = torch.argsort(group_of_topic)
                gcount = torch.bincount(group_of_topic, minlength=groups)
                gstart = torch.cumsum(gcount, 0) - gcount
                gt = group_of_topic[topic_of]
                r = (torch.rand(n, generator=g, device=device) * gcount[gt].to(torch.float32)).to(torch.int64).clamp_(max=int(gcount.max()) - 1)
                second_of = order[gstart[gt] + torch.minimum(r, gcount[gt] - 1)]
            else:
                second_of = torch.randint(0, topics, (n,), generator=g, device=device)
        for a, b in _chunks(n, chunk):
            e = torch.randn(b - a, DIM, generator=g, device=device)
            x = centres[topic_of[a:b]] + dense_noise * e / e.norm(dim=1, keepdim=True)
            if second_of is not None:
                x = x + mix * centres[second_of[a:b]]
            dense[a:b] = x / x.norm(dim=1, keepdim=True)

    def rows(mean, vocab, s, cap):
        draw = lambda r: torch.searchsorted(_zipf_cdf(vocab, s, device), torch.rand(r, topic_terms, generator=g, device=device, dtype=torch.float64)).clamp_(max=vocab - 1)
        tt = draw(topics)
        if groups:
            shared = torch.rand(topics, topic_terms, generator=g, device=device) < group_share
            tt = torch.where(shared, draw(groups)[group_of_topic], tt)
        offs, idxs, base = [], [], 0
        for a, b in _chunks(n, chunk):
            cnt = torch.poisson(torch.full((b - a,), mean, device=device), generator=g).to(torch.int64).clamp_(1, cap)
            off, idx = _topic_rows(cnt, topic_of[a:b], tt, topic_share, vocab, s, g,
                                   second_topic=None if second_of is None else second_of[a:b], second_share=mix / (1.0 + mix))
            offs.append(off[:-1] + base)
            base += int(off[-1])
            idxs.append(idx)
        return torch.cat(offs + [torch.tensor([base], device=device)]), torch.cat(idxs)

    s_off, s_idx = rows(mean_sparse, SPARSE_VOCAB, 1.1, MAX_SPARSE)
    s_val = torch.exp(torch.randn(s_idx.numel(), generator=g, device=device) * 0.8 - 1.0).to(torch.float32)
    b_off, b_idx = rows(mean_bm25, BM25_VOCAB, 1.0, MAX_BM25)
    uu = torch.rand(b_idx.numel(), generator=g, device=device, dtype=torch.float64).clamp_(min=1e-12)
    tf = 1.0 + torch.floor(torch.log(uu) / math.log(1.0 - 0.6))
    row_of = torch.repeat_interleave(torch.arange(n, device=device), (b_off[1:] - b_off[:-1]))
    length = torch.zeros(n, dtype=torch.float64, device=device).index_add_(0, row_of, tf)
    df = torch.bincount(b_idx, minlength=BM25_VOCAB).to(torch.float64)
    idf = torch.log(1.0 + (n - df + 0.5) / (df + 0.5))
    k1, bb = 1.2, 0.75
    w = idf[b_idx] * tf * (k1 + 1.0) / (tf + k1 * (1.0 - bb + bb * length[row_of] / length.mean()))
    return Corpus(dense, Csr(s_off.to(torch.int32), s_idx.to(torch.int32), s_val),
                  Csr(b_off.to(torch.int32), b_idx.to(torch.int32), w.to(torch.float32)), idf.to(torch.float32),
                  extra={"topic_of": topic_of, "topics": topics})


def make_clustered_queries(nq: int, corpus: Corpus, seed: int = 20261202, device=None, nnz_sparse: int = 30, nnz_bm25: int = 8,
                           dense_noise: float = 0.3) -> Queries:
    """Queries as perturbed documents of `corpus` (see make_clustered_corpus)."""
    device = corpus.dense.device if device is None else torch.device(device)
    g = _gen(seed, device)
    src = torch.randint(0, corpus.n, (nq,), generator=g, device=device)
    e = torch.randn(nq, DIM, generator=g, device=device)
    x = corpus.dense[src] + dense_noise * e / e.norm(dim=1, keepdim=True)
    dense = x / x.norm(dim=1, keepdim=True)

    def take(csr: Csr, k: int, values):
        off = csr.off.to(torch.int64)
        lens = off[src + 1] - off[src]
        row_of = torch.repeat_interleave(torch.arange(nq, device=device), lens)
        pos = torch.arange(int(lens.sum()), device=device) - torch.repeat_interleave(torch.cumsum(lens, 0) - lens, lens) + off[src][row_of]
        keep = _subsample_rows(row_of, nq, torch.full((nq,), k, dtype=torch.int64, device=device), g)
        pos, row_k = pos[keep], row_of[keep]
        n_k = torch.bincount(row_k, minlength=nq)
        qoff = torch.zeros(nq + 1, dtype=torch.int64, device=device)
        qoff[1:] = torch.cumsum(n_k, 0)
        idx = csr.idx[pos]
        return Csr(qoff.to(torch.int32), idx.contiguous(), values(pos, idx).to(torch.float32).contiguous())

    sparse = take(corpus.sparse, nnz_sparse, lambda pos, idx: corpus.sparse.val[pos])
    bm25 = take(corpus.bm25, nnz_bm25, lambda pos, idx: corpus.idf.to(device)[idx.to(torch.int64)])
    return Queries(dense, sparse, bm25)


@dataclass
class KnowledgeGraph:
    e2e_off: torch.Tensor   # int32 [entities + 1]
    e2e_idx: torch.Tensor
    e2d_off: torch.Tensor
    e2d_idx: torch.Tensor
    qe_off: torch.Tensor    # int32 [nq + 1]
    qe_idx: torch.Tensor


def make_kg(n_docs: int, nq: int, entities: int = 500_000, seed: int = 20261127, device="cpu",
            mean_degree: float = 4.0, alpha: float = 2.1) -> KnowledgeGraph:
    """Entity graph with power-law out-degree (Pareto tail `alpha`, rescaled to the
    requested mean), 1-5 uniformly drawn docs per entity, 1-3 seed entities per query."""
    device = torch.device(device)
    g = _gen(seed, device)
    u = torch.rand(entities, generator=g, device=device, dtype=torch.float64).clamp_(min=1e-12)
    raw = u.pow(-1.0 / (alpha - 1.0))                      # Pareto, x_min = 1
    deg = torch.floor(raw * (mean_degree / float(raw.clamp(max=1000.0).mean()))).clamp_(0, 1000).to(torch.int64)
    e2e_off = torch.zeros(entities + 1, dtype=torch.int64, device=device)
    e2e_off[1:] = torch.cumsum(deg, 0)
    e2e_idx = torch.randint(0, entities, (int(e2e_off[-1]),), generator=g, device=device)
    nd = torch.randint(1, 6, (entities,), generator=g, device=device)
    e2d_off = torch.zeros(entities + 1, dtype=torch.int64, device=device)
    e2d_off[1:] = torch.cumsum(nd, 0)
    e2d_idx = torch.randint(0, n_docs, (int(e2d_off[-1]),), generator=g, device=device)
    ne = torch.randint(1, 4, (nq,), generator=g, device=device)
    qe_off = torch.zeros(nq + 1, dtype=torch.int64, device=device)
    qe_off[1:] = torch.cumsum(ne, 0)
    qe_idx = torch.randint(0, entities, (int(qe_off[-1]),), generator=g, device=device)
    i32 = lambda t: t.to(torch.int32)
    return KnowledgeGraph(i32(e2e_off), i32(e2e_idx), i32(e2d_off), i32(e2d_idx), i32(qe_off), i32(qe_idx))


def make_keywords(queries: Queries, seed: int = 20261128) -> list[list[int]]:
    """1-4 required term ids per query, drawn from the query's own BM25 terms."""
    rng = np.random.default_rng(seed)
    off = queries.bm25.off.cpu().numpy().astype(np.int64)
    idx = queries.bm25.idx.cpu().numpy().astype(np.int64)
    out = []
    for q in range(queries.nq):
        row = idx[off[q]:off[q + 1]]
        k = int(min(len(row), rng.integers(1, 5)))
        out.append(sorted(int(t) for t in rng.choice(row, size=k, replace=False)))
    return out


# ---------------------------------------------------------------------------
# File formats of the reference loaders
# ---------------------------------------------------------------------------
def write_fvecs(path: str, dense: torch.Tensor) -> None:
    """Each row: int32 dim, then dim float32 (include/utils.cuh:361-378)."""
    x = dense.detach().cpu().numpy().astype(np.float32)
    n, d = x.shape
    out = np.empty((n, d + 1), dtype=np.float32)
    out[:, 0] = np.array([d], dtype=np.int32).view(np.float32)[0]
    out[:, 1:] = x
    out.tofile(path)


def read_fvecs(path: str) -> np.ndarray:
    raw = np.fromfile(path, dtype=np.float32)
    d = int(raw[:1].view(np.int32)[0])
    return raw.reshape(-1, d + 1)[:, 1:].copy()


def write_csr(path: str, csr: Csr) -> None:
    """u32 nnz | u32 off[rows+1] | u32 idx[nnz] | f32 val[nnz] (include/utils.cuh:380-398)."""
    off = csr.off.cpu().numpy().astype(np.uint32)
    with open(path, "wb") as f:
        np.array([off[-1]], dtype=np.uint32).tofile(f)
        off.tofile(f)
        csr.idx.cpu().numpy().astype(np.uint32).tofile(f)
        csr.val.cpu().numpy().astype(np.float32).tofile(f)


def read_csr(path: str, rows: int) -> Csr:
    raw = np.fromfile(path, dtype=np.uint32)
    nnz = int(raw[0])
    off = raw[1:rows + 2]
    idx = raw[rows + 2:rows + 2 + nnz]
    val = raw[rows + 2 + nnz:rows + 2 + 2 * nnz].view(np.float32)
    t = lambda a, dt: torch.from_numpy(a.astype(dt))
    return Csr(t(off, np.int32), t(idx, np.int32), torch.from_numpy(val.copy()))


def write_kg_csr(path: str, off: torch.Tensor, idx: torch.Tensor) -> None:
    """u32 n_off | u32 nnz | u32 off[n_off] | u32 idx[nnz] (src/query.cu:89-108)."""
    o = off.cpu().numpy().astype(np.uint32)
    with open(path, "wb") as f:
        np.array([o.size, int(o[-1])], dtype=np.uint32).tofile(f)
        o.tofile(f)
        idx.cpu().numpy().astype(np.uint32).tofile(f)


def write_keywords(path: str, kws: list[list[int]]) -> None:
    with open(path, "w") as f:
        for row in kws:
            f.write(" ".join(str(t) for t in row) + "\n")


def write_qrels(path: str, ids: np.ndarray) -> None:
    with open(path, "w") as f:
        for row in ids:
            f.write(" ".join(str(int(t)) for t in row) + "\n")


def write_poe(path: str, graph: np.ndarray, ep: np.ndarray) -> None:
    """u32 width | u32 n_ep | u32 ep[n_ep] | n x (u32 width | u32 row[width]) (src/index.cu:928-939)."""
    n, w = graph.shape
    rows = np.empty((n, w + 1), dtype=np.uint32)
    rows[:, 0] = w
    rows[:, 1:] = graph
    with open(path, "wb") as f:
        np.array([w, ep.size], dtype=np.uint32).tofile(f)
        ep.astype(np.uint32).tofile(f)
        rows.tofile(f)


def read_poe(path: str):
    """Reader with the tolerance of src/query.cu:35-62."""
    raw = np.fromfile(path, dtype=np.uint32)
    w, n_ep = int(raw[0]), int(raw[1])
    ep = raw[2:2 + n_ep].copy()
    n = (raw.size - (n_ep + 1)) // (w + 1)   # the reference's own arithmetic (one header word is not subtracted)
    body = raw[2 + n_ep:2 + n_ep + n * (w + 1)].reshape(n, w + 1)
    return body[:, 1:].copy(), ep
