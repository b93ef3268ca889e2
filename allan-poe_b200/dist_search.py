"""Multi-GPU plumbing (one process per GPU, torch.distributed).

Two ways to use one 8-GPU box:
  * query-parallel: every rank holds the whole index and searches a contiguous slice of the query batch; queries are
    independent, so there is no collective on the data path (results can be gathered once at the end);
  * corpus-sharded: rank r owns documents [r*n/W, (r+1)*n/W) with local ids and its own graph; every rank searches all
    queries on its shard with the same effective weights, the per-shard (distance, global id) lists are
    all-gathered (NCCL over NVLink on GPUs) and each rank merges them to the global top-k with a device kernel.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n: int, rank: int, world: int) -> tuple[int, int]:
    """Documents of `rank`: contiguous, sizes differ by at most one."""
    base, rem = divmod(n, world)
    a = rank * base + min(rank, rem)
    return a, a + base + (1 if rank < rem else 0)


def query_range(nq: int, rank: int, world: int) -> tuple[int, int]:
    return shard_range(nq, rank, world)


def to_global_ids(local_ids: torch.Tensor, shard_start: int, shard_size: int) -> torch.Tensor:
    """Local document ids of a shard -> corpus-wide ids; empty slots (0x7FFFFFFF or beyond the shard) stay empty (-1)."""
    ids = local_ids.to(torch.int64)
    valid = (ids >= 0) & (ids < shard_size)
    return torch.where(valid, ids + shard_start, torch.full_like(ids, -1)).to(torch.int32)


def gather_results(ids: torch.Tensor, dis: torch.Tensor, g_ids: torch.Tensor, g_dis: torch.Tensor, group=None) -> None:
    """all_gather of [nq, per] result lists into [world, nq, per] buffers."""
    dist.all_gather_into_tensor(g_ids.view(-1), ids.contiguous().view(-1), group=group)
    dist.all_gather_into_tensor(g_dis.view(-1), dis.contiguous().view(-1), group=group)


def merge_topk_reference(g_ids: torch.Tensor, g_dis: torch.Tensor, top_k: int):
    """Plain torch restatement of the merge (used to check the device kernel and in CPU tests of the plumbing):
    ascending (distance, id), empty slots (id < 0) last."""
    w, nq, per = g_ids.shape
    ids = g_ids.permute(1, 0, 2).reshape(nq, w * per).to(torch.int64)
    dis = g_dis.permute(1, 0, 2).reshape(nq, w * per).to(torch.float64)
    dis = torch.where(ids < 0, torch.full_like(dis, float("inf")), dis)
    key_order = torch.argsort(ids, dim=1, stable=True)
    ids_s, dis_s = torch.gather(ids, 1, key_order), torch.gather(dis, 1, key_order)
    order = torch.argsort(dis_s, dim=1, stable=True)[:, :top_k]
    return torch.gather(ids_s, 1, order).to(torch.int32), torch.gather(dis_s, 1, order).to(torch.float32)


def exchange_and_merge(g_keys: torch.Tensor, rank: int, out_ids: torch.Tensor, out_dis: torch.Tensor, top_k: int, group=None) -> None:
    """The exchange step of the sharded search on packed keys.  g_keys: int64 [world, nq, per]; slice `rank` already
    holds this shard's keys (the search kernel wrote them there).  One all-gather in place, then one merge kernel."""
    import apoe
    dist.all_gather_into_tensor(g_keys.view(-1), g_keys[rank].view(-1), group=group)
    apoe.merge_shard_keys(g_keys, top_k, out_ids, out_dis, torch.cuda.current_stream().cuda_stream)


def merge_keys_reference(g_keys: torch.Tensor, top_k: int):
    """Plain torch restatement of the key merge: the top_k smallest keys of every query as unsigned 64-bit words (int64
    tensors hold them; flipping the sign bit makes the signed order the unsigned one).  Returns the merged keys
    [nq, top_k] as int64 bit patterns."""
    w, nq, per = g_keys.shape
    flat = g_keys.permute(1, 0, 2).reshape(nq, w * per)
    flipped = flat ^ torch.iinfo(torch.int64).min
    return (torch.sort(flipped, dim=1).values[:, :top_k]) ^ torch.iinfo(torch.int64).min


def gather_and_merge(local_ids, local_dis, shard_start, g_ids, g_dis, out_ids, out_dis, top_k, shard_size=None, group=None):
    """One exchange step of the sharded search, on device tensors."""
    import apoe
    size = shard_size if shard_size is not None else (1 << 31) - 2
    gids = to_global_ids(local_ids, shard_start, size)
    gather_results(gids, local_dis, g_ids, g_dis, group)
    apoe.merge_shard_results(g_ids, g_dis, top_k, out_ids, out_dis, torch.cuda.current_stream().cuda_stream)
