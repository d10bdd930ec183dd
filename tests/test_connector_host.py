"""The host-slot free list of the connector, on the CPU: runs are preferred, freed slots merge, and a
seeded random sequence of requests never hands a slot out twice."""
import random

import pytest
import torch

from heterofusedkernels_b200.connector import HostSlotPool


def test_requests_are_served_from_runs_and_holes_are_reused_best_fit():
    p = HostSlotPool(100)
    a = p.alloc(10)
    b = p.alloc(30)
    c = p.alloc(5)
    assert a.tolist() == list(range(10)) and b.tolist() == list(range(10, 40)) and c.tolist() == list(range(40, 45))
    assert a.dtype == torch.int64 and p.free_count == 55 and p.largest_run() == 55
    p.free(b)
    assert p.runs() == [(10, 30), (45, 55)]
    assert p.alloc(20).tolist() == list(range(10, 30))          # the smallest run that fits
    assert p.alloc(40).tolist() == list(range(45, 85))
    assert p.runs() == [(30, 10), (85, 15)]
    got = p.alloc(22)                                             # no single run: longest first
    assert got.tolist() == list(range(85, 100)) + list(range(30, 37))
    assert p.free_count == 3 and p.runs() == [(37, 3)]
    with pytest.raises(RuntimeError, match="exhausted"):
        p.alloc(4)
    assert p.alloc(0).numel() == 0


def test_freed_slots_merge_with_both_neighbours_and_double_frees_are_refused():
    p = HostSlotPool(16)
    s = p.alloc(16)
    p.free(s[[0, 1, 2]])
    p.free(s[[6, 7]])
    assert p.runs() == [(0, 3), (6, 2)]
    p.free([3, 4, 5])                                             # bridges the two runs
    assert p.runs() == [(0, 8)] and p.free_count == 8
    with pytest.raises(ValueError, match="already free"):
        p.free([7])
    with pytest.raises(ValueError, match="outside"):
        p.free([16])
    p.free(torch.tensor([15, 9, 12]))                             # unsorted, scattered
    assert p.runs() == [(0, 8), (9, 1), (12, 1), (15, 1)] and p.free_count == 11


def test_random_requests_never_share_a_slot():
    rng = random.Random(7)
    p = HostSlotPool(500)
    held = []
    in_use = set()
    for _ in range(2000):
        if held and (rng.random() < 0.45 or p.free_count < 40):
            s = held.pop(rng.randrange(len(held)))
            p.free(s)
            in_use -= set(s.tolist())
        else:
            n = rng.randint(1, 40)
            s = p.alloc(n)
            assert s.numel() == n == len(set(s.tolist())) and not (set(s.tolist()) & in_use)
            assert 0 <= min(s.tolist()) and max(s.tolist()) < 500
            in_use |= set(s.tolist())
            held.append(s)
        assert p.free_count == 500 - len(in_use) == sum(n for _, n in p.runs())
        runs = p.runs()
        assert all(runs[i][0] + runs[i][1] < runs[i + 1][0] for i in range(len(runs) - 1))   # sorted, never adjacent


def test_the_connector_takes_the_staged_mover_only_for_host_resident_slot_lists_made_of_runs():
    from heterofusedkernels_b200.connector import PagedKVCache

    c = PagedKVCache.__new__(PagedKVCache)       # the choice needs no device state
    c.pool_layout = "slot_major"
    c.slot_bytes = 2 << 20
    assert c._pick_mover(torch.arange(100, 612)) == "staged"                       # one run
    assert c._pick_mover(list(range(5, 13)) + list(range(40, 48))) == "staged"     # two runs of 8
    scattered = torch.randperm(40000, generator=torch.Generator().manual_seed(0))[:512]
    assert c._pick_mover(scattered) == "hybrid"                                    # 1 GiB of scattered 2 MiB slots
    assert c._pick_mover(scattered[:32]) is None                                   # 64 MiB: not worth two movers
    assert c._pick_mover(scattered.to(torch.int64).tolist()[:10]) is None
    assert c._pick_mover(torch.tensor([0, 1, 2, 3, 10, 11, 12, 13, 20, 22])) is None   # mean run below 4, small
    assert c._pick_mover([1, 2, 3]) is None                                        # too few to matter
    c.pool_layout = "layer_major"                                                  # slots are not contiguous there
    assert c._pick_mover(torch.arange(64)) is None
