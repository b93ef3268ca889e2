"""Host-side helpers of bench.py (no GPU needed): the recall measure and the torch form of the shard exchange key."""
import numpy as np
import torch

import apoe
import bench


def test_recall_counts_true_ids_found_and_ignores_missing_truth():
    gt = np.array([[1, 2, 3, 4, 5, 6, 7, 8, 9, 10], [1, 2, 3, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF]], dtype=np.uint32)
    ids = np.array([[10, 9, 99, 98, 97, 96, 95, 94, 93, 1, 2], [3, 0x3FFFFFFF, 1, 50, 51, 52, 53, 54, 55, 56, 2]], dtype=np.uint32)
    # row 0: 3 of 10 found in the first ten (the eleventh does not count); row 1: 2 of its 3 eligible documents
    assert abs(bench.recall_at_10(ids, gt) - (0.3 + 2 / 3) / 2) < 1e-12
    assert bench.recall_at_10(gt, gt) == 1.0


def test_torch_keys_equal_the_library_decoder():
    rng = np.random.default_rng(1)
    ids = rng.integers(0, 1_000_000, (50, 10)).astype(np.int32)
    dis = (rng.normal(size=(50, 10)) * 300).astype(np.float32)
    ids[3, 7:] = -1
    keys = bench.pack_keys_torch(torch.from_numpy(ids), torch.from_numpy(dis), 5_000_000).numpy().view(np.uint64)
    got_ids, got_dis = apoe.unpack_shard_keys(keys)
    valid = ids != -1
    assert np.array_equal(got_ids[valid], (ids[valid].astype(np.int64) + 5_000_000).astype(np.uint32))
    assert np.array_equal(got_dis[valid].view(np.uint32), dis[valid].view(np.uint32))
    assert np.all(got_ids[~valid] == 0xFFFFFFFF)
    # the unsigned order of the keys is the order of (distance, id)
    order = np.argsort(keys[0])
    assert np.all(np.diff(dis[0][order]) >= 0)


def test_both_arms_name_the_workload_alike():
    assert bench.bench_config(1_000_000, 10_000, 128) == bench.bench_config(1_000_000, 10_000, 128)
    assert "queries_per_step" in bench.bench_config(10, 5, 32)
