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


# ---------------------------------------------------------------------------------------------------------
# shards on disk: ranges and the manifest (host code of the library; no GPU needed)
# ---------------------------------------------------------------------------------------------------------
def test_library_shard_ranges_equal_the_python_ones():
    import apoe
    for n, w in ((10, 3), (1_000_000, 8), (10_000_000, 8), (64, 2), (1001, 7)):
        for r in range(w):
            a, b = dist_search.shard_range(n, r, w)
            assert apoe.shard_range(n, r, w) == (a, b - a)


def test_shard_manifest_round_trip_and_validation(tmp_path):
    import apoe
    path = str(tmp_path / "idx.manifest")
    apoe.write_shard_manifest(path, 1001, 4, str(tmp_path / "idx"))
    n, shards = apoe.read_shard_manifest(path)
    assert n == 1001 and len(shards) == 4
    assert [(a, c) for a, c, _ in shards] == [apoe.shard_range(1001, g, 4) for g in range(4)]
    assert [name for _, _, name in shards] == [f"idx.{g}.poe" for g in range(4)]
    text = open(path).read().splitlines()
    assert text[0] == "allan-poe-shards 1" and text[1] == "docs 1001 shards 4"
    # a manifest whose ranges leave a gap, and a file that is no manifest at all
    broken = text[:]
    broken[3] = "1 300 250 idx.1.poe"
    open(path, "w").write("\n".join(broken) + "\n")
    with pytest.raises(apoe.ApoeError) as e:
        apoe.read_shard_manifest(path)
    assert e.value.code == 2
    open(path, "w").write("something else\n")
    with pytest.raises(apoe.ApoeError):
        apoe.read_shard_manifest(path)
    with pytest.raises(apoe.ApoeError):
        apoe.read_shard_manifest(str(tmp_path / "missing.manifest"))


def _pack_keys(dis: np.ndarray, gids: np.ndarray) -> np.ndarray:
    """The exchange word of the sharded search: order-preserving distance bits << 32 | global id (empty: all ones)."""
    b = dis.astype(np.float32).view(np.uint32)
    o = np.where(b & np.uint32(0x80000000), ~b, b | np.uint32(0x80000000)).astype(np.uint64)
    k = (o << np.uint64(32)) | gids.astype(np.uint64)
    k[gids < 0] = np.uint64(0xFFFFFFFFFFFFFFFF)
    return k


def _key_worker(rank, world, port, manifest, nq, top_k, out):
    import apoe
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, shards = apoe.read_shard_manifest(manifest)          # every rank learns its document range from the manifest
        a, c, _ = shards[rank]
        rng = np.random.default_rng(200 + rank)
        local = np.stack([rng.choice(c, size=top_k, replace=False) for _ in range(nq)]).astype(np.int64)
        dis = np.sort(rng.normal(size=(nq, top_k)).astype(np.float32) * 50.0, axis=1)       # fused distances are mostly negative
        gids = local + a
        gids[:, -1] = np.where(np.arange(nq) % 5 == rank, -1, gids[:, -1])                 # some lists are one short
        g_keys = torch.zeros(world, nq, top_k, dtype=torch.int64)
        g_keys[rank] = torch.from_numpy(_pack_keys(dis, gids).view(np.int64))
        dist.all_gather_into_tensor(g_keys.view(-1), g_keys[rank].clone().view(-1))         # one collective, as on the GPUs
        merged = dist_search.merge_keys_reference(g_keys, top_k)
        ref = [torch.empty_like(merged) for _ in range(world)]
        dist.all_gather(ref, merged)
        if rank == 0:
            torch.save({"merged": merged, "g_keys": g_keys, "same": all(torch.equal(ref[0], r) for r in ref), "shards": shards}, out)
    finally:
        dist.destroy_process_group()


def test_key_exchange_two_ranks_from_a_manifest(tmp_path):
    import apoe
    manifest, out = str(tmp_path / "idx.manifest"), str(tmp_path / "r0.pt")
    apoe.write_shard_manifest(manifest, 1001, 2, str(tmp_path / "idx"))
    nq, top_k = 23, 10
    mp.spawn(_key_worker, args=(2, _free_port(), manifest, nq, top_k, out), nprocs=2, join=True)
    r = torch.load(out)
    assert r["same"]
    keys = r["g_keys"].numpy().view(np.uint64)
    ids, dis = apoe.unpack_shard_keys(r["merged"].numpy().view(np.uint64))
    for q in range(nq):
        allk = np.sort(keys[:, q, :].reshape(-1))
        assert np.array_equal(r["merged"][q].numpy().view(np.uint64), allk[:top_k])
    assert np.all(np.diff(dis, axis=1) >= 0)
    (a0, c0, _), (a1, c1, _) = r["shards"]
    valid = ids != 0xFFFFFFFF
    assert np.all(ids[valid] < a1 + c1)


def _leaving_worker(rank, world, port, out):
    """Rank 1 leaves between two steps without joining the next collective; rank 0 learns of it on the host -- the short
    process-group timeout ends its next collective with an error -- and finishes the step alone."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    x = torch.full((4,), float(rank + 1))
    dist.all_reduce(x)                     # step 1: both ranks take part
    if rank == 1:
        os._exit(0)                        # leaves between steps, nothing in flight
    failed = False
    try:
        y = torch.ones(4)
        dist.all_reduce(y)                 # step 2: the peer is gone
    except Exception:
        failed = True
    torch.save({"step1": x, "failed": failed}, out)
    os._exit(0)


def test_rank_leaving_between_steps_is_noticed_on_the_host(tmp_path):
    out = str(tmp_path / "r0.pt")
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive()
    r = torch.load(out)
    assert torch.equal(r["step1"], torch.full((4,), 3.0))
    assert r["failed"], "the collective after the peer left must end with an error, not hang"


@pytest.mark.gpu
def test_device_key_merge_matches_reference_merge():
    import apoe
    rng = np.random.default_rng(3)
    shards, nq, per = 8, 517, 10
    dev = torch.device("cuda:0")
    dis = np.sort(rng.normal(size=(shards, nq, per)).astype(np.float32) * 100.0, axis=2)
    gids = np.stack([np.stack([rng.choice(100000, size=per, replace=False) + s * 100000 for _ in range(nq)]) for s in range(shards)]).astype(np.int64)
    gids[:, ::7, -2:] = -1
    dis[0, 5, 3] = dis[1, 5, 2]                                  # equal distances in two shards: the lower id goes first
    g_keys = torch.from_numpy(_pack_keys(dis, gids).view(np.int64))
    want = dist_search.merge_keys_reference(g_keys, 10)
    want_ids, want_dis = apoe.unpack_shard_keys(want.numpy().view(np.uint64))
    out_ids = torch.empty(nq, 10, dtype=torch.int32, device=dev)
    out_dis = torch.empty(nq, 10, dtype=torch.float32, device=dev)
    apoe.merge_shard_keys(g_keys.to(dev), 10, out_ids, out_dis)
    torch.cuda.synchronize()
    assert np.array_equal(out_ids.cpu().numpy().view(np.uint32), want_ids)
    assert np.array_equal(out_dis.cpu().numpy().view(np.uint32), want_dis.view(np.uint32))
