"""Expert-parallel token exchange for the MoE grouped GEMM (host-side index logic).

The reference has no multi-device code; its grouped_matmul expects rows already sorted by
expert with cumulative group ends (csrc/opdev/op_kernel/grouped_mat_mul_ex.cpp:29-38).
Sharding that op over G GPUs therefore needs exactly one exchange before it (send each
routed row to the rank that owns its expert) and one after it (send results back):

    route (local)  ->  dispatch all-to-all  ->  local grouped GEMMs  ->  combine all-to-all
                                                                     ->  weighted sum (local)

Every function here works on index tensors only and runs on CPU (gloo) as well as CUDA
(NCCL), which is how the world_size-2 tests exercise it without GPUs.  The exchange itself
is `torch.distributed.all_to_all_single` with split sizes derived from one all-gather of
the per-expert counts; payload rows land in local memory before any kernel reads them.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def expert_owner(num_experts: int, world: int) -> torch.Tensor:
    """Contiguous placement: expert e lives on rank e // ceil(E / world)."""
    per = -(-num_experts // world)
    return torch.arange(num_experts) // per


def local_experts(num_experts: int, world: int, rank: int) -> torch.Tensor:
    return torch.nonzero(expert_owner(num_experts, world) == rank).flatten()


def sort_by_expert(expert_ids: torch.Tensor, num_experts: int):
    """Routing on one rank: flat (token, k) slots sorted by expert, stable.

    Returns (order, counts): `order[i]` = flat slot that supplies sorted row i (its token is
    order[i] // top_k); counts[e] = rows routed to expert e.
    """
    flat = expert_ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    return order, counts


@dataclass
class ExchangePlan:
    send_splits: list          # rows this rank sends to each rank (sorted-by-expert order)
    recv_splits: list          # rows this rank receives from each rank
    recv_to_grouped: torch.Tensor  # gather index: grouped row i comes from received row [i]
    group_list: torch.Tensor   # int64 cumulative ends over this rank's experts
    num_local_rows: int


def make_exchange_plan(all_counts: torch.Tensor, rank: int, owner: torch.Tensor) -> ExchangePlan:
    """all_counts[r, e] = rows rank r routes to expert e (identical on every rank).

    Rows travel sorted by expert, and experts are placed contiguously, so the rows a rank
    sends to one peer are a contiguous slice.  Received rows arrive ordered (source rank,
    expert); the grouped GEMM wants (expert, source rank): `recv_to_grouped` is that
    permutation.
    """
    world, num_experts = all_counts.shape
    owner = owner.to(all_counts.device)
    mine = torch.nonzero(owner == rank).flatten()
    send_splits = [int(all_counts[rank, owner == r].sum()) for r in range(world)]
    recv_mat = all_counts[:, mine]  # [world, local experts]
    recv_splits = [int(v) for v in recv_mat.sum(1)]
    # offset of block (source r, local expert j) in the receive buffer (source-major)
    flat = recv_mat.reshape(-1)
    starts = torch.cumsum(flat, 0) - flat
    starts = starts.reshape(world, -1)
    pieces = []
    for j in range(mine.numel()):
        for r in range(world):
            n = int(recv_mat[r, j])
            if n:
                s = int(starts[r, j])
                pieces.append(torch.arange(s, s + n, device=all_counts.device))
    total = int(flat.sum())
    recv_to_grouped = (torch.cat(pieces) if pieces else
                       torch.zeros(0, dtype=torch.long, device=all_counts.device))
    group_list = torch.cumsum(recv_mat.sum(0), 0).to(torch.int64)
    return ExchangePlan(send_splits, recv_splits, recv_to_grouped, group_list, total)


def gather_counts(counts: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather the per-expert counts of every rank -> [world, E]."""
    world = dist.get_world_size(group)
    out = torch.empty(world * counts.numel(), dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(out, counts.contiguous(), group=group)
    return out.view(world, counts.numel())


def exchange(rows: torch.Tensor, send_splits, recv_splits, group=None) -> torch.Tensor:
    out = rows.new_empty((sum(recv_splits),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_splits),
                           input_split_sizes=list(send_splits), group=group)
    return out


def expert_parallel_mlp(x, expert_ids, expert_weights, num_experts, local_mlp, group=None):
    """Run the routed expert MLP for this rank's tokens with experts sharded over the group.

    x [T, H]; expert_ids, expert_weights [T, top_k]; local_mlp(rows [R, H], group_list) ->
    [R, H_out] applies this rank's experts to rows sorted by (local) expert.  Returns
    y [T, H_out] = sum_k weight[t, k] * expert_{ids[t, k]}(x[t]).
    With no process group (single GPU) the exchange steps vanish.
    """
    top_k = expert_ids.shape[1]
    order, counts = sort_by_expert(expert_ids, num_experts)
    tokens = order // top_k
    rows = x.index_select(0, tokens)
    distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    if not distributed:
        out_rows = local_mlp(rows, torch.cumsum(counts, 0).to(torch.int64))
    else:
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        all_counts = gather_counts(counts, group).cpu()  # split sizes are host integers
        plan = make_exchange_plan(all_counts, rank, expert_owner(num_experts, world))
        recv = exchange(rows, plan.send_splits, plan.recv_splits, group)
        idx = plan.recv_to_grouped.to(recv.device)
        grouped = recv.index_select(0, idx)
        res = local_mlp(grouped, plan.group_list.to(recv.device))
        back = torch.empty_like(res)
        back.index_copy_(0, idx, res)  # back to (source rank, expert) order
        out_rows = exchange(back, plan.recv_splits, plan.send_splits, group)
    w = expert_weights.reshape(-1).index_select(0, order).to(torch.float32)
    y = torch.zeros(x.shape[0], out_rows.shape[1], dtype=torch.float32, device=x.device)
    y.index_add_(0, tokens, out_rows.to(torch.float32) * w[:, None])
    return y.to(x.dtype)


def expert_parallel_mlp_device(moe, x, expert_ids, expert_weights, num_experts, local_mlp, group=None,
                               segment_rows=None, overflow_out=None, local=False):
    """Same contract as expert_parallel_mlp, built from the library's own glue kernels
    (`ascend910a_extras.moe`) with every piece of metadata on the device: no host
    synchronisation anywhere in the step.

    expert_ids int32 [T, top_k], expert_weights float32 [T, top_k] (from moe.route_topk).
    Across ranks the exchange is an equal-split all-to-all of fixed-capacity segments:
    every rank sends `segment_rows` rows to every peer (default T*top_k, the most one peer
    can be owed), of which only the leading rows are meaningful; the per-expert counts
    travel in a small all-gather and stay on the device, where `moe.ep_plan` turns them into
    the grouped order and the group ends grouped_matmul reads.  All ranks must pass the same
    `segment_rows`.  A capacity below T*top_k can overflow: rows that do not fit are left out of
    the result and counted in a device int32 that is appended to `overflow_out` (a list) for the
    caller to inspect later -- reading it here would be the host sync this path exists to avoid.
    `local=True` runs the single-GPU form whatever process group exists (this rank then needs
    every expert's weights behind `local_mlp`).
    """
    t, top_k = expert_ids.shape
    slots, hidden = t * top_k, x.shape[1]
    distributed = (not local and dist.is_available() and dist.is_initialized()
                   and dist.get_world_size(group) > 1)
    if not distributed:
        pos, _, group_list, _ = moe.permute(expert_ids, num_experts, 1, 0)
        rows = x.new_empty(slots, hidden)
        moe.copy_rows(rows, x, dst_index=pos, src_div=top_k, n_max=slots)
        return moe.finalize(local_mlp(rows, group_list), pos, expert_weights)
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    cap = slots if segment_rows is None else int(segment_rows)
    pos, counts, _, overflow = moe.permute(expert_ids, num_experts, world, cap)
    if overflow_out is not None:
        overflow_out.append(overflow)
    send = x.new_empty(world * cap, hidden)
    moe.copy_rows(send, x, dst_index=pos, src_div=top_k, n_max=slots)
    all_counts = counts.new_empty(world * num_experts)
    dist.all_gather_into_tensor(all_counts, counts, group=group)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    grouped_to_received, group_list, total = moe.ep_plan(all_counts.view(world, num_experts), rank, cap)
    grouped = x.new_empty(world * cap, hidden)
    moe.copy_rows(grouped, recv, src_index=grouped_to_received, n_valid=total, n_max=world * cap)
    res = local_mlp(grouped, group_list)
    back = res.new_empty(world * cap, res.shape[1])
    moe.copy_rows(back, res, dst_index=grouped_to_received, n_valid=total, n_max=world * cap)
    returned = torch.empty_like(back)
    dist.all_to_all_single(returned, back, group=group)
    return moe.finalize(returned, pos, expert_weights)


# --------------------------------------------------------------------------- balanced placement
@dataclass
class Placement:
    """Which expert each slot holds.  Slots are placed contiguously on ranks
    (`slots_per_rank` each), so a slot id is used as the expert id of the exchange; an expert
    with several slots is replicated and its rows are spread over the replicas."""
    slot_expert: torch.Tensor    # [num_slots] expert held by each slot
    expert_slots: torch.Tensor   # [E, max_replicas] slots of each expert, padded by repeating
    num_replicas: torch.Tensor   # [E]
    slots_per_rank: int

    @property
    def num_slots(self):
        return int(self.slot_expert.numel())

    def local_slot_experts(self, rank):
        s = self.slots_per_rank
        return self.slot_expert[rank * s:(rank + 1) * s].tolist()

    def to(self, device):
        """The tables on `device` (also as the int32 tensors `moe.dispatch` reads)."""
        self.expert_slots = self.expert_slots.to(device)
        self.num_replicas = self.num_replicas.to(device)
        self.expert_slots_i32 = self.expert_slots.to(torch.int32).contiguous()
        self.num_replicas_i32 = self.num_replicas.to(torch.int32).contiguous()
        return self


def balanced_placement(load, world: int, slots_per_rank: int) -> Placement:
    """Replicate heavily loaded experts and pack the replicas onto ranks so that every rank
    gets about the same number of rows.

    `load[e]` = expected rows of expert e (a routing histogram).  With one slot per expert a
    skewed router leaves most GPUs idle: the busiest expert bounds the step.  Here the
    world*slots_per_rank slots go first one to each expert, then one at a time to the expert
    with the largest load per replica; the replicas (each worth load/replicas rows) are then
    assigned largest-first to the rank with the least load that still has a free slot.
    """
    load = [float(v) for v in load]
    num_experts = len(load)
    num_slots = world * slots_per_rank
    assert num_slots >= num_experts, "need at least one slot per expert"
    replicas = [1] * num_experts
    for _ in range(num_slots - num_experts):
        e = max(range(num_experts), key=lambda i: (load[i] / replicas[i], -i))
        replicas[e] += 1
    items = sorted(((load[e] / replicas[e], e) for e in range(num_experts) for _ in range(replicas[e])),
                   key=lambda t: (-t[0], t[1]))
    rank_load = [0.0] * world
    rank_slots = [[] for _ in range(world)]
    for share, e in items:
        r = min((r for r in range(world) if len(rank_slots[r]) < slots_per_rank),
                key=lambda r: (rank_load[r], r))
        rank_slots[r].append(e)
        rank_load[r] += share
    slot_expert = torch.tensor([e for r in range(world) for e in sorted(rank_slots[r])], dtype=torch.long)
    max_rep = max(replicas)
    table = torch.zeros(num_experts, max_rep, dtype=torch.long)
    for e in range(num_experts):
        mine = torch.nonzero(slot_expert == e).flatten()
        table[e] = mine[torch.arange(max_rep) % mine.numel()]
    return Placement(slot_expert, table, torch.tensor(replicas, dtype=torch.long), slots_per_rank)


def to_slot_ids(expert_ids: torch.Tensor, placement: Placement, token_offset: int = 0) -> torch.Tensor:
    """Replace expert ids [T, top_k] by slot ids: replica (token index mod replicas) of the
    expert, which spreads an expert's rows evenly over its replicas without any counting."""
    dev = expert_ids.device
    ids = expert_ids.long()
    t = torch.arange(token_offset, token_offset + ids.shape[0], device=dev)[:, None]
    which = t % placement.num_replicas.to(dev)[ids]
    return placement.expert_slots.to(dev)[ids, which].to(expert_ids.dtype)


def placement_balance(load, placement: Placement, world: int) -> float:
    """mean / max rows per rank under the placement (1.0 = perfectly even)."""
    per_rank = [0.0] * world
    for s, e in enumerate(placement.slot_expert.tolist()):
        per_rank[s // placement.slots_per_rank] += float(load[e]) / int(placement.num_replicas[e])
    return sum(per_rank) / (world * max(per_rank)) if max(per_rank) > 0 else 1.0


# --------------------------------------------------------------------------- peer-memory exchange
class PeerExchange:
    """Expert-parallel dispatch/combine over NVLink peer memory instead of NCCL collectives.

    Each rank holds, in symmetric memory its peers have mapped, a receive buffer and a return
    buffer, a table of count words and a flag array.  A step is three launches around the two
    expert GEMMs (`moe.dispatch`, `moe.gather`, `moe.combine`):

    * dispatch routes every token (or takes the given expert ids), claims a row of the
      (this rank, slot) sub-segment in the slot owner's receive buffer and stores the token's row
      there through the peer mapping; its last CTA sends the counts, tagged with the step number;
    * gather waits (bounded) for every source's counts of the step and compacts the received rows into
      expert-major order for `grouped_matmul`;
    * the down projection stores its result rows straight into the owners' return buffers
      (`moe.grouped_matmul_scatter`), and combine announces "returned", waits (bounded) for the
      peers and forms the weighted sum.

    `slots_per_rank` slots live on every rank (an expert, or a replica of a replicated expert: pass
    a `Placement` to `mlp`); a (source, slot) sub-segment holds `segment_rows` rows; rows that do
    not fit are left out and counted in `overflow` (device int32 [2]: at dispatch, at gather).

    Buffer reuse across steps needs no extra synchronisation: a rank starts dispatching step
    n+1 only after its combine of step n, which waited for every peer's "returned" of step n, and
    a peer sends that only after its own gather of step n has read its receive buffer; a peer's
    down projection of step n+1 writes into this rank's return buffer only after that peer's
    gather of step n+1, which waited for this rank's dispatch of step n+1, which its stream issues
    after the combine of step n.  All ranks must construct the object together and call `mlp` the
    same number of times.
    """

    def __init__(self, moe, group, device, segment_rows, hidden, hidden_out, num_slots, max_rows=None):
        import torch.distributed._symmetric_memory as symm

        self.moe, self.group = moe, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.cap, self.num_slots = int(segment_rows), int(num_slots)
        assert self.num_slots % self.world == 0, "slots must divide evenly over ranks"
        self.spr = self.num_slots // self.world
        rows = self.num_slots * self.cap  # world * spr * cap, both for receiving and for returning
        self.max_rows = rows if max_rows is None else min(int(max_rows), rows)
        align = lambda n: (n + 255) // 256 * 256
        o_recv = 0
        o_ret = o_recv + align(rows * hidden * 2)
        o_counts = o_ret + align(rows * hidden_out * 2)
        o_flags_r = o_counts + align(self.world * self.spr * 4)
        total = o_flags_r + align(self.world * 4)
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buf, group.group_name)
        self.buf.zero_()
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.peer_recv = [p + o_recv for p in ptrs]
        self.peer_ret = [p + o_ret for p in ptrs]
        self.peer_counts = [p + o_counts for p in ptrs]
        self.peer_flags_r = [p + o_flags_r for p in ptrs]
        self.recv = self.buf[o_recv:o_recv + rows * hidden * 2].view(torch.float16).view(rows, hidden)
        self.ret = self.buf[o_ret:o_ret + rows * hidden_out * 2].view(torch.float16).view(rows, hidden_out)
        self.counts = self.buf[o_counts:o_counts + self.world * self.spr * 4].view(torch.int32).view(
            self.world, self.spr)
        self.flags_r = self.buf[o_flags_r:o_flags_r + self.world * 4].view(torch.int32)
        self.cursor = torch.zeros(self.num_slots, dtype=torch.int32, device=device)
        self.state = torch.zeros(8, dtype=torch.int32, device=device)
        self.overflow = torch.zeros(2, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # everyone's flags are zero before anyone announces

    def barrier_error(self) -> int:
        """0, or 100 + the rank whose announcement did not arrive within the time limit (synchronises)."""
        return int(self.state[1].item())

    def mlp(self, x, expert_ids, expert_weights, local_mlp, overflow_out=None, local_mlp_scatter=None,
            router_weight=None, top_k=None, placement=None, token_offset=0, num_experts=None,
            return_routing=False):
        """Same contract as expert_parallel_mlp_device for world > 1.

        Either `expert_ids` [T, top_k] int32 with `expert_weights` [T, top_k] float32, or
        `router_weight` [E, H] with `top_k` (the routing then happens inside the dispatch launch).
        `placement` (a `Placement` whose tables are on the device) maps experts to slots.
        `local_mlp_scatter(rows, group_list, scatter)`, if given, replaces `local_mlp` plus the
        return push: it must end in `moe.grouped_matmul_scatter(..., *scatter)`, whose epilogue
        stores the result rows into the peers' return buffers itself."""
        moe, rank = self.moe, self.rank
        if num_experts is None:
            num_experts = router_weight.shape[0] if router_weight is not None else (
                placement.num_replicas.numel() if placement is not None else self.num_slots)
        k = top_k if router_weight is not None else expert_ids.shape[1]
        slots_tab = placement.expert_slots_i32 if placement is not None else None
        reps_tab = placement.num_replicas_i32 if placement is not None else None
        pos, ids, wts = moe.dispatch(x, router_weight, None if router_weight is not None else expert_ids, k,
                                     slots_tab, reps_tab, token_offset, self.peer_recv, self.peer_counts,
                                     self.cursor, self.state, self.overflow, num_experts, self.cap, rank)
        if router_weight is None:
            wts = expert_weights
        if overflow_out is not None:
            overflow_out.append(self.overflow)
        grouped, to_received, group_list, total = moe.gather(self.recv, self.counts, self.state, self.overflow,
                                                             self.cap, self.max_rows)
        seg = self.spr * self.cap  # rows one source owns in a receive buffer
        if local_mlp_scatter is not None:
            local_mlp_scatter(grouped, group_list, (to_received, self.peer_ret, seg, rank))
        else:
            res = local_mlp(grouped, group_list)
            moe.push_rows(res, to_received, 1, total, self.max_rows, self.peer_ret, seg, rank)
        y = moe.combine(self.ret, pos, wts, self.peer_flags_r, self.flags_r, self.state, rank)
        if return_routing:
            return y, ids, wts
        return y
