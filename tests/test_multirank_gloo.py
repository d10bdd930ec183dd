"""The N>1 host logic on CPU: two gloo ranks exercise the barrier, the max-over-ranks reduction,
the per-rank id lists and the aggregate — the same RankContext bench.py uses with NCCL."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from heterofusedkernels_b200 import ranks


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    ctx = ranks.RankContext.from_env().init("gloo")
    ctx.barrier()
    local_ms = 10.0 + 5.0 * rank          # rank 1 is the slow one
    worst = ctx.max_over_ranks(local_ms)
    sets = ranks.rank_id_sets(rank, 3, 8, 64, 32)
    per_rank = ctx.gather_floats([rank, local_ms])
    assert per_rank == [[0.0, 10.0], [1.0, 15.0]]
    ctx.barrier()
    q.put((rank, worst, [tuple(t.tolist() for t in s) for s in sets]))
    ctx.close()


def test_two_ranks_take_the_max_time_and_disjoint_seeds():
    world, port = 2, _free_port()
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    procs = [ctxm.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [g[1] for g in got] == [15.0, 15.0]            # both ranks see the slowest rank's time
    assert got[0][2] != got[1][2]                          # ranks do not share id lists
    for _, _, sets in got:
        for out_ids, slots, in_ids in sets:
            assert len(set(out_ids)) == 8 and len(set(slots)) == 8 and len(set(in_ids)) == 8
            assert max(out_ids) < 64 and max(slots) < 32
    # whole-job throughput: all ranks' bytes over the slowest rank's time
    assert ranks.aggregate_gbs(10**9, 2, 15.0) == pytest.approx(2 * 10**9 / 15e-3 / 1e9)


def test_single_rank_context_needs_no_process_group():
    ctx = ranks.RankContext(0, 0, 1).init("gloo")
    ctx.barrier()
    assert ctx.max_over_ranks(3.5) == 3.5 and ctx.dist is None
    assert ctx.gather_floats([1, 2.5]) == [[1.0, 2.5]]


def test_host_pool_is_shrunk_per_rank_but_never_below_the_transferred_set():
    slot = 2 << 20
    assert ranks.host_pool_slots(40000, slot, 512, 1, 200 << 30) == (40000, "")
    slots, note = ranks.host_pool_slots(40000, slot, 512, 8, 200 << 30)
    assert slots == int((200 << 30) * 0.6 / 8) // slot and "shrunk" in note
    assert ranks.host_pool_slots(40000, slot, 512, 8, 1 << 30)[0] == 1024


def test_ranks_are_spread_over_the_visible_gpus():
    assert [ranks.spread_device_index(r, 2, 8) for r in range(2)] == [0, 4]
    assert [ranks.spread_device_index(r, 4, 8) for r in range(4)] == [0, 2, 4, 6]
    assert [ranks.spread_device_index(r, 8, 8) for r in range(8)] == list(range(8))
    assert [ranks.spread_device_index(r, 2, 2) for r in range(2)] == [0, 1]
    assert ranks.spread_device_index(0, 1, 8) == 0 and ranks.spread_device_index(3, 4, 1) == 0


def test_id_sets_let_a_step_read_the_previous_steps_slots_while_it_writes_its_own():
    sets = ranks.rank_id_sets(3, 6, 50, 200, 120)
    prev = None
    for out_ids, slots, in_ids in sets:
        assert not set(out_ids.tolist()) & set(in_ids.tolist())          # blocks come back to OTHER blocks
        assert len(set(slots.tolist())) == 50 == slots.numel()
        if prev is not None:
            assert not set(slots.tolist()) & prev                         # consecutive steps: disjoint slots
        prev = set(slots.tolist())
    with pytest.raises(AssertionError):
        ranks.rank_id_sets(0, 2, 50, 99, 120)                             # cache too small for disjoint lists


def test_issue_orders_of_a_step_per_rank():
    """How each rank issues a step under every variant of the benchmark (no GPU: only the plan)."""
    import sys
    from pathlib import Path
    from types import SimpleNamespace as NS

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench

    def plan(rank, world, variant):
        sb = bench.SwapBench.__new__(bench.SwapBench)
        sb.ctx = NS(rank=rank, world=world)
        return sb.plan(variant)

    assert plan(0, 1, "sequential") == ("own", "out_first", 1, False)
    assert plan(1, 2, "sequential") == ("own", "out_first", 1, False)
    assert plan(0, 2, "stagger") == ("own", "out_first", 1, False)
    assert plan(1, 2, "stagger") == ("prev", "in_first", 1, False)        # odd ranks swap in first
    assert plan(0, 8, "bidir") == plan(5, 8, "bidir") == ("prev", "out_first", 1, True)
    assert plan(3, 4, "bidir_paced") == plan(0, 8, "bidir")                 # the same order; only the swap-out is paced
    assert plan(2, 4, "interleave:4") == ("own", "out_first", 4, False)
    assert plan(3, 4, "interleave:4") == ("prev", "in_first", 4, False)
    assert plan(1, 1, "stagger") == ("own", "out_first", 1, False)        # a single rank has nobody to stagger with
    with pytest.raises(ValueError):
        plan(0, 2, "nonsense")
    assert set(bench.MULTI_GPU_VARIANTS) <= set(bench.VARIANT_TEXT)
