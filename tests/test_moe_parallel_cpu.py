"""Expert-parallel exchange logic on CPU: index math alone, then two gloo ranks end to end."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO / "ascend-ops_b200"))

import moe_parallel  # noqa: E402


def _fake_expert_rows(rows, expert_of_row):
    """Stand-in expert e: x -> x * (e + 1) + e  (distinguishes experts, exact in fp32)."""
    e = expert_of_row.to(rows.dtype)[:, None]
    return rows * (e + 1) + e


def _reference_output(x, ids, wts):
    y = torch.zeros_like(x)
    for k in range(ids.shape[1]):
        y += wts[:, k:k + 1] * _fake_expert_rows(x, ids[:, k])
    return y


def test_sort_by_expert_and_owner():
    ids = torch.tensor([[3, 0], [1, 3], [0, 2]])
    order, counts = moe_parallel.sort_by_expert(ids, 4)
    assert counts.tolist() == [2, 1, 1, 2]
    assert ids.reshape(-1)[order].tolist() == [0, 0, 1, 2, 3, 3]
    assert (order // 2).tolist() == [0, 2, 1, 2, 0, 1]
    assert moe_parallel.expert_owner(8, 4).tolist() == [0, 0, 1, 1, 2, 2, 3, 3]
    assert moe_parallel.expert_owner(8, 3).tolist() == [0, 0, 0, 1, 1, 1, 2, 2]
    assert moe_parallel.local_experts(8, 8, 5).tolist() == [5]


def test_exchange_plan_is_consistent():
    g = torch.Generator().manual_seed(0)
    world, experts = 4, 8
    counts = torch.randint(0, 6, (world, experts), generator=g)
    counts[2] = 0  # a rank that routes nothing
    counts[:, 3] = 0  # an expert nobody uses
    owner = moe_parallel.expert_owner(experts, world)
    plans = [moe_parallel.make_exchange_plan(counts, r, owner) for r in range(world)]
    for r, p in enumerate(plans):
        assert sum(p.send_splits) == int(counts[r].sum())
        for s in range(world):
            assert p.send_splits[s] == plans[s].recv_splits[r]
        assert sorted(p.recv_to_grouped.tolist()) == list(range(p.num_local_rows))
        mine = torch.nonzero(owner == r).flatten()
        assert p.group_list.tolist() == counts[:, mine].sum(0).cumsum(0).tolist()


def _single_process_local_mlp(rows, group_list):
    ends = group_list.tolist()
    e_of_row = torch.cat([torch.full((e - (ends[i - 1] if i else 0),), i) for i, e in enumerate(ends)])
    return _fake_expert_rows(rows, e_of_row)


def test_single_process_path_matches_reference():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(13, 8, generator=g)
    ids = torch.stack([torch.randperm(4, generator=g)[:2] for _ in range(13)])
    wts = torch.rand(13, 2, generator=g)
    y = moe_parallel.expert_parallel_mlp(x, ids, wts, 4, _single_process_local_mlp)
    torch.testing.assert_close(y, _reference_output(x, ids, wts))


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        experts = 4
        g = torch.Generator().manual_seed(100 + rank)
        t = 9 if rank == 0 else 5  # ragged token counts across ranks
        x = torch.randn(t, 6, generator=g)
        ids = torch.stack([torch.randperm(experts, generator=g)[:2] for _ in range(t)])
        if rank == 1:
            ids[:] = torch.tensor([0, 1])  # rank 1 sends everything to rank 0's experts
        wts = torch.rand(t, 2, generator=g)
        mine = moe_parallel.local_experts(experts, world, rank)

        def local_mlp(rows, group_list):
            ends = group_list.tolist()
            parts = [torch.full((e - (ends[i - 1] if i else 0),), int(mine[i])) for i, e in enumerate(ends)]
            e_of_row = torch.cat(parts) if parts else torch.zeros(0, dtype=torch.long)
            return _fake_expert_rows(rows, e_of_row)

        y = moe_parallel.expert_parallel_mlp(x, ids, wts, experts, local_mlp)
        results[rank] = bool(torch.allclose(y, _reference_output(x, ids, wts), atol=1e-5))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_dispatch_and_combine():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(results) == {0: True, 1: True}


def test_balanced_placement_replicates_hot_experts():
    load = [99, 512, 3881, 990, 1329, 287, 98, 996]  # the benchmark's routing skew
    plain = moe_parallel.balanced_placement(load, 8, 1)
    assert sorted(plain.slot_expert.tolist()) == list(range(8))
    assert moe_parallel.placement_balance(load, plain, 8) < 0.3  # one expert per GPU: the hot one dominates
    p = moe_parallel.balanced_placement(load, 8, 3)
    assert p.num_slots == 24 and int(p.num_replicas.sum()) == 24 and int(p.num_replicas.min()) >= 1
    assert int(p.num_replicas[2]) == int(p.num_replicas.max())
    assert moe_parallel.placement_balance(load, p, 8) > 0.85
    for e in range(8):  # the slot table lists exactly the slots that hold the expert
        assert set(p.expert_slots[e].tolist()) == set(torch.nonzero(p.slot_expert == e).flatten().tolist())
    # fewer ranks than experts
    p2 = moe_parallel.balanced_placement(load, 2, 6)
    assert moe_parallel.placement_balance(load, p2, 2) > 0.9


def test_slot_ids_keep_the_expert_and_spread_over_replicas():
    load = [10, 1000, 10, 10]
    p = moe_parallel.balanced_placement(load, 4, 2)
    g = torch.Generator().manual_seed(0)
    ids = torch.stack([torch.randperm(4, generator=g)[:2] for _ in range(4000)]).int()
    slots = moe_parallel.to_slot_ids(ids, p)
    assert torch.equal(p.slot_expert[slots.long()], ids.long())  # a slot always holds the routed expert
    hot = slots[ids == 1].long()
    used = torch.bincount(hot, minlength=p.num_slots)
    reps = int(p.num_replicas[1])
    assert reps > 1 and int((used > 0).sum()) == reps and int(used.max()) < 1.25 * int(used[used > 0].min())
    assert (slots[:, 0] != slots[:, 1]).all()  # top-k experts differ, so their slots differ
