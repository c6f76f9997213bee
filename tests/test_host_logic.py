"""Host-side decisions that need no GPU: key-split counts, pull-stage grouping, descriptor layouts."""

import ctypes

import pytest


def test_key_split_counts_follow_the_wave_model(monkeypatch):
    from chitudiffusion_b200 import ops

    monkeypatch.delenv("CHITU_B200_KEY_SPLITS", raising=False)
    assert ops.NUM_SMS == 148
    # Flux1-dev joint attention (4608 rows, 24 heads) on 1, 2, 4 and 8 GPUs: only the 54-CTA grid is split
    assert [ops.auto_key_splits(1, 4608, 4608, h) for h in (24, 12, 6, 3)] == [1, 1, 1, 2]
    # large grids are never split: the parked rows would not stay in L2
    assert ops.auto_key_splits(1, 75600, 75600, 40) == 1
    assert ops.auto_key_splits(1, 9450, 75600, 40) == 1
    assert ops.auto_key_splits(1, 32760, 32760, 12) == 1
    # a single key tile cannot be split; tiny grids stay whole when the split saves less than it costs
    assert ops.auto_key_splits(1, 256, 128, 1) == 1
    assert ops.auto_key_splits(1, 1024, 1024, 2) == 1
    monkeypatch.setenv("CHITU_B200_KEY_SPLITS", "3")
    assert ops.auto_key_splits(1, 4608, 4608, 24) == 3
    assert ops.auto_key_splits(1, 256, 256, 1) == 2  # clamped to the number of key tiles


def test_owner_runs_of_the_all_gather_stages():
    from chitudiffusion_b200.peer import _runs

    assert _runs([7, 0, 1, 2]) == [(0, 3), (7, 1)]
    assert _runs([3]) == [(3, 1)]
    assert _runs([4, 5, 6]) == [(4, 3)]
    assert _runs([]) == []
    # rank 6 of 8: own block, then four peers (wrapping), then three
    order = [(6 + t) % 8 for t in range(8)]
    stages = [order[:1], order[1:5], order[5:]]
    assert [_runs(s) for s in stages] == [[(6, 1)], [(0, 3), (7, 1)], [(3, 3)]]


def test_descriptor_layouts_match_the_header():
    from chitudiffusion_b200 import _lib

    # chitu_b200_push: three staging pointers, three pointer-to-pointer arrays, one int64
    assert ctypes.sizeof(_lib.PushDesc) == 3 * 8 + 3 * 8 + 8
    desc, keep = _lib.push_desc([0, 4096, 8192], [[16, 32], [48, 64], [80, 96]], 1 << 20)
    assert desc.stage[0] is None and desc.stage[1] == 4096 and desc.block_bytes == 1 << 20
    assert [int(keep[2][i]) for i in range(2)] == [80, 96]
    # chitu_b200_peer_sync: pointer array, rank, world
    assert ctypes.sizeof(_lib.PeerSyncDesc) == 16
    sync = _lib.peer_sync_desc([256, 512, 768], 1)
    assert sync[0].rank == 1 and sync[0].world == 3


def test_cached_ring_refuses_bad_plans():
    from chitudiffusion_b200.cached_ring import CachedRingAttention

    class Group:
        group_size, rank_in_group = 4, 1

    ring = CachedRingAttention(lambda *a, **k: None, Group(), merger_factory=object)
    with pytest.raises(ValueError):
        ring(None, None, None, plan=[True, True])  # one entry per rank
    with pytest.raises(ValueError):
        ring(None, None, None, plan=[False, True, True, True])  # the local block is always computed
    with pytest.raises(RuntimeError):
        ring(None, None, None, plan=[True, False, True, True])  # nothing kept yet for offset 1
