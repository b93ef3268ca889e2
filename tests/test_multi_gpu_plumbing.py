"""Host-side logic of the multi-GPU modes, exercised as two gloo ranks on CPU (no GPU needed): document / query
partitioning, local -> global id mapping, the all-gather of per-shard result lists and the merge order."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import dist_search


def test_partitions_cover_everything_once():
    for n, w in ((10, 3), (1_000_000, 8), (7, 8), (64, 2)):
        spans = [dist_search.shard_range(n, r, w) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    assert dist_search.query_range(10_000, 3, 4) == (7500, 10000)


def test_global_ids_keep_empty_slots_empty():
    ids = torch.tensor([[0, 5, 0x7FFFFFFF, 99]], dtype=torch.int32)
    out = dist_search.to_global_ids(ids, 1000, 100)
    assert out.tolist() == [[1000, 1005, -1, 1099]]


def test_merge_reference_orders_by_distance_then_id():
    g_ids = torch.tensor([[[4, 9, -1]], [[7, 2, 30]]], dtype=torch.int32)          # 2 shards x 1 query x 3
    g_dis = torch.tensor([[[0.5, 0.7, 1e6]], [[0.5, 0.1, 0.9]]], dtype=torch.float32)
    ids, dis = dist_search.merge_topk_reference(g_ids, g_dis, 4)
    assert ids.tolist() == [[2, 4, 7, 9]]
    assert np.allclose(dis.numpy(), [[0.1, 0.5, 0.5, 0.7]])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_docs, nq, per, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a, b = dist_search.shard_range(n_docs, rank, world)
        rng = np.random.default_rng(100 + rank)
        # a shard's local result lists: ascending distances, distinct local ids, a few empty tails
        local = np.stack([rng.choice(b - a, size=per, replace=False) for _ in range(nq)]).astype(np.int32)
        dis = np.sort(rng.random((nq, per)).astype(np.float32), axis=1)
        local[:, -2:] = 0x7FFFFFFF
        dis[:, -2:] = 1e6
        gids = dist_search.to_global_ids(torch.from_numpy(local), a, b - a)
        g_ids = torch.empty(world, nq, per, dtype=torch.int32)
        g_dis = torch.empty(world, nq, per, dtype=torch.float32)
        dist_search.gather_results(gids, torch.from_numpy(dis), g_ids, g_dis)
        ids, d = dist_search.merge_topk_reference(g_ids, g_dis, 10)
        # every rank must hold the same merged answer
        ref = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(ref, ids)
        same = all(torch.equal(ref[0], r) for r in ref)
        if rank == 0:
            torch.save({"ids": ids, "dis": d, "g_ids": g_ids, "g_dis": g_dis, "same": same, "span": (a, b)}, out)
    finally:
        dist.destroy_process_group()


def test_sharded_exchange_two_ranks(tmp_path):
    out = str(tmp_path / "r0.pt")
    n_docs, nq, per = 1001, 17, 16
    mp.spawn(_worker, args=(2, _free_port(), n_docs, nq, per, out), nprocs=2, join=True)
    r = torch.load(out)
    assert r["same"]
    g_ids, g_dis = r["g_ids"], r["g_dis"]
    # rank 0's rows hold ids of its own range, rank 1's rows ids of the other range
    a0, b0 = dist_search.shard_range(n_docs, 0, 2)
    v0 = g_ids[0][g_ids[0] >= 0]
    v1 = g_ids[1][g_ids[1] >= 0]
    assert int(v0.min()) >= a0 and int(v0.max()) < b0 and int(v1.min()) >= b0 and int(v1.max()) < n_docs
    # the merged list is the global top-10 of the union, ascending
    for q in range(nq):
        pairs = sorted((float(g_dis[s, q, j]), int(g_ids[s, q, j])) for s in range(2) for j in range(per) if int(g_ids[s, q, j]) >= 0)
        assert [p[1] for p in pairs[:10]] == r["ids"][q].tolist()
    assert torch.all(r["dis"][:, 1:] >= r["dis"][:, :-1])


@pytest.mark.gpu
def test_device_merge_kernel_matches_reference_merge():
    import apoe
    torch.manual_seed(0)
    shards, nq, per = 8, 333, 128
    dev = torch.device("cuda:0")
    g_ids = torch.stack([torch.stack([torch.randperm(100000)[:per] + s * 100000 for _ in range(nq)]) for s in range(shards)]).to(torch.int32)
    g_dis = torch.sort(torch.rand(shards, nq, per), dim=2).values
    g_ids[:, :, -3:] = -1
    g_dis[:, :, -3:] = 1e6
    want_ids, want_dis = dist_search.merge_topk_reference(g_ids, g_dis, 10)
    out_ids = torch.empty(nq, 10, dtype=torch.int32, device=dev)
    out_dis = torch.empty(nq, 10, dtype=torch.float32, device=dev)
    apoe.merge_shard_results(g_ids.to(dev), g_dis.to(dev), 10, out_ids, out_dis)
    torch.cuda.synchronize()
    assert torch.equal(out_ids.cpu(), want_ids) and torch.equal(out_dis.cpu(), want_dis)
