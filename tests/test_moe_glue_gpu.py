"""MoE glue kernels through the C ABI against straightforward torch formulations."""
import ctypes

import pytest
import torch

from conftest import knob

import moe_parallel

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("tokens,hidden,experts,top_k", [(256, 4096, 8, 2), (7, 512, 64, 4), (1, 64, 3, 1),
                                                         (33, 1024, 256, 8)])
def test_route_topk(cabi, tokens, hidden, experts, top_k):
    g = torch.Generator().manual_seed(tokens + experts)
    x = torch.randn(tokens, hidden, generator=g).half()
    w = (torch.randn(experts, hidden, generator=g) * 0.05).half()
    ids = torch.full((tokens, top_k), -1, dtype=torch.int32, device=DEV)
    wts = torch.zeros(tokens, top_k, device=DEV)
    xd, wd = x.to(DEV), w.to(DEV)
    cabi.check(cabi.load().b200ops_moe_route_topk(p(xd), p(wd), p(ids), p(wts), tokens, hidden, experts, top_k,
                                                  stream()))
    torch.cuda.synchronize()
    logits = (x.float() @ w.float().T).half().float()
    prob = torch.softmax(logits, -1)
    ew, ei = torch.topk(prob, top_k, -1)
    got_w, got_i = wts.cpu(), ids.cpu().long()
    torch.testing.assert_close(got_w, ew, rtol=2e-3, atol=1e-5)
    # expert choices may differ only where two probabilities are within rounding of each other
    differs = got_i != ei
    if differs.any():
        gap = (prob.gather(1, got_i) - prob.gather(1, ei)).abs()
        assert float(gap[differs].max()) < 2e-3
    assert (got_i.sort(1).values[:, 1:] != got_i.sort(1).values[:, :-1]).all() or top_k == 1


@pytest.mark.parametrize("tokens,top_k,experts,world", [(256, 2, 8, 1), (256, 2, 8, 4), (1000, 4, 64, 8),
                                                        (3, 1, 5, 1), (40000, 2, 16, 2)])
def test_permute_is_the_stable_sort(cabi, tokens, top_k, experts, world):
    g = torch.Generator().manual_seed(tokens)
    ids = torch.randint(0, experts, (tokens, top_k), generator=g, dtype=torch.int32)
    slots = tokens * top_k
    cap = slots
    idd = ids.to(DEV)
    pos = torch.full((slots,), -5, dtype=torch.int32, device=DEV)
    counts = torch.zeros(experts, dtype=torch.int32, device=DEV)
    gl = torch.zeros(experts, dtype=torch.int64, device=DEV)
    cabi.check(cabi.load().b200ops_moe_permute(p(idd), p(pos), p(counts), p(gl), None, slots, experts, world,
                                               cap, stream()))
    torch.cuda.synchronize()
    flat = ids.reshape(-1).long()
    want_counts = torch.bincount(flat, minlength=experts)
    assert counts.cpu().tolist() == want_counts.tolist()
    assert gl.cpu().tolist() == want_counts.cumsum(0).tolist()
    order = torch.argsort(flat, stable=True)
    want_pos = torch.empty(slots, dtype=torch.long)
    if world == 1:
        want_pos[order] = torch.arange(slots)
    else:
        per = experts // world
        dest = flat[order] // per
        start_of_dest = torch.zeros(world, dtype=torch.long)
        cnt_dest = torch.bincount(dest, minlength=world)
        start_sorted = torch.cumsum(cnt_dest, 0) - cnt_dest
        want_pos[order] = dest * cap + (torch.arange(slots) - start_sorted[dest])
    assert torch.equal(pos.cpu().long(), want_pos)


@pytest.mark.parametrize("world,experts", [(2, 8), (8, 8), (4, 64)])
def test_ep_plan_matches_host_plan(cabi, world, experts):
    g = torch.Generator().manual_seed(world * experts)
    all_counts = torch.randint(0, 9, (world, experts), generator=g, dtype=torch.int32)
    cap = 9 * (experts // world)  # a segment must hold the most one source can send one rank
    all_counts[:, 1] = 0
    local = experts // world
    owner = moe_parallel.expert_owner(experts, world)
    for rank in (0, world - 1):
        host = moe_parallel.make_exchange_plan(all_counts.long(), rank, owner)
        m = torch.full((world * cap,), -1, dtype=torch.int32, device=DEV)
        gl = torch.zeros(local, dtype=torch.int64, device=DEV)
        total = torch.zeros(1, dtype=torch.int32, device=DEV)
        acd = all_counts.to(DEV)
        cabi.check(cabi.load().b200ops_moe_ep_plan(p(acd), p(m), p(gl), p(total), world, experts, rank, cap,
                                                   stream()))
        torch.cuda.synchronize()
        n = int(total)
        assert n == host.num_local_rows and gl.cpu().tolist() == host.group_list.tolist()
        # host plan indexes a densely packed receive buffer; the device plan indexes fixed segments
        recv_counts = all_counts[:, rank * local:(rank + 1) * local].sum(1).long()
        dense_start = torch.cumsum(recv_counts, 0) - recv_counts
        src_rank = torch.bucketize(host.recv_to_grouped, torch.cumsum(recv_counts, 0), right=True)
        want = src_rank * cap + (host.recv_to_grouped - dense_start[src_rank])
        assert torch.equal(m[:n].cpu().long(), want)


def test_copy_rows_and_finalize(cabi):
    g = torch.Generator().manual_seed(9)
    t, k, h = 50, 2, 256
    x = torch.randn(t, h, generator=g).half().to(DEV)
    ids = torch.randint(0, 4, (t, k), generator=g, dtype=torch.int32).to(DEV)
    wts = torch.rand(t, k, generator=g).to(DEV)
    lib = cabi.load()
    pos = torch.empty(t * k, dtype=torch.int32, device=DEV)
    counts = torch.empty(4, dtype=torch.int32, device=DEV)
    gl = torch.empty(4, dtype=torch.int64, device=DEV)
    cabi.check(lib.b200ops_moe_permute(p(ids), p(pos), p(counts), p(gl), None, t * k, 4, 1, 0, stream()))
    rows = torch.zeros(t * k, h, dtype=torch.float16, device=DEV)
    cabi.check(lib.b200ops_moe_copy_rows(p(rows), p(x), p(pos), None, k, None, t * k, h, stream()))
    torch.cuda.synchronize()
    want_rows = torch.empty_like(rows)
    want_rows[pos.long()] = x.repeat_interleave(k, 0)
    assert torch.equal(rows, want_rows)
    # n_valid limits the copy; a negative index skips its row
    idx = torch.arange(t * k, dtype=torch.int32, device=DEV)
    idx[3] = -1
    dst = torch.zeros_like(rows)
    nvalid = torch.tensor([10], dtype=torch.int32, device=DEV)
    cabi.check(lib.b200ops_moe_copy_rows(p(dst), p(rows), None, p(idx), 1, p(nvalid), t * k, h, stream()))
    torch.cuda.synchronize()
    assert torch.equal(dst[:3], rows[:3]) and not dst[3].any() and torch.equal(dst[4:10], rows[4:10])
    assert not dst[10:].any()
    y = torch.empty(t, h, dtype=torch.float16, device=DEV)
    cabi.check(lib.b200ops_moe_finalize(p(rows), p(pos), p(wts), p(y), t, k, h, stream()))
    torch.cuda.synchronize()
    want = (rows[pos.long()].float().view(t, k, h) * wts[:, :, None]).sum(1)
    torch.testing.assert_close(y.float(), want, rtol=1e-2, atol=1e-3)


def test_permute_bounded_capacity_drops_and_reports(cabi):
    """Two ranks, two experts each, capacity 5 rows per destination: 9 rows want rank 0."""
    ids = torch.tensor([0, 1, 0, 0, 3, 1, 1, 0, 2, 0, 1, 3], dtype=torch.int32, device=DEV)  # e0 x5, e1 x4, e2 x1, e3 x2
    pos = torch.empty(12, dtype=torch.int32, device=DEV)
    counts = torch.empty(4, dtype=torch.int32, device=DEV)
    gl = torch.empty(4, dtype=torch.int64, device=DEV)
    ov = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    cabi.check(cabi.load().b200ops_moe_permute(p(ids), p(pos), p(counts), p(gl), p(ov), 12, 4, 2, 5, stream()))
    torch.cuda.synchronize()
    assert counts.cpu().tolist() == [5, 0, 1, 2]  # expert 1's four rows do not fit behind expert 0's five
    assert int(ov) == 4
    got = pos.cpu().tolist()
    assert [got[i] for i in (0, 2, 3, 7, 9)] == [0, 1, 2, 3, 4]  # expert 0, stable order, segment 0
    assert [got[i] for i in (1, 5, 6, 10)] == [-1] * 4             # dropped
    assert got[8] == 5 and [got[4], got[11]] == [6, 7]             # segment 1 starts at row 5
    # ample capacity: nothing dropped
    cabi.check(cabi.load().b200ops_moe_permute(p(ids), p(pos), p(counts), p(gl), p(ov), 12, 4, 2, 12, stream()))
    torch.cuda.synchronize()
    assert int(ov) == 0 and counts.cpu().tolist() == [5, 4, 1, 2] and (pos >= 0).all()


def _ptr_array(addresses):
    arr = (ctypes.c_void_p * len(addresses))(*addresses)
    return arr


def test_push_rows_two_emulated_ranks_on_one_gpu(cabi):
    """Both 'ranks' live on this GPU (their buffers are ordinary tensors), pushed one after the
    other: checks the addressing of rows and count tables without any cross-GPU wait."""
    lib = cabi.load()
    world, cap, h, experts, top_k, t = 2, 16, 64, 4, 2, 6
    g = torch.Generator().manual_seed(5)
    recv = [torch.zeros(world * cap, h, dtype=torch.float16, device=DEV) for _ in range(world)]
    tables = [torch.full((world, experts), -1, dtype=torch.int32, device=DEV) for _ in range(world)]
    rows_ptrs = _ptr_array([b.data_ptr() for b in recv])
    table_ptrs = _ptr_array([b.data_ptr() for b in tables])
    xs, poss, cnts = [], [], []
    for rank in range(world):
        x = torch.randn(t, h, generator=g).half().to(DEV)
        ids = torch.randint(0, experts, (t, top_k), generator=g, dtype=torch.int32).to(DEV)
        pos = torch.empty(t * top_k, dtype=torch.int32, device=DEV)
        counts = torch.empty(experts, dtype=torch.int32, device=DEV)
        gl = torch.empty(experts, dtype=torch.int64, device=DEV)
        cabi.check(lib.b200ops_moe_permute(p(ids), p(pos), p(counts), p(gl), None, t * top_k, experts, world, cap,
                                           stream()))
        cabi.check(lib.b200ops_moe_push_rows(p(x), p(pos), top_k, None, t * top_k, rows_ptrs, world, cap, rank, h,
                                             p(counts), experts, table_ptrs, stream()))
        xs.append(x), poss.append(pos), cnts.append(counts)
    torch.cuda.synchronize()
    for rank in range(world):
        for dest in range(world):
            assert tables[dest][rank].cpu().tolist() == cnts[rank].cpu().tolist()
        for s, idx in enumerate(poss[rank].cpu().tolist()):
            dest, off = divmod(idx, cap)
            assert torch.equal(recv[dest][rank * cap + off], xs[rank][s // top_k])
    total = sum(int(c.sum()) for c in cnts)
    assert sum(int((b.abs().sum(1) > 0).sum()) for b in recv) == total


def test_peer_barrier_passes_when_peers_arrived_and_gives_up_when_not(cabi):
    """The barrier's wait is bounded.  Flags of a second, emulated rank are set by hand: with the
    flag in place the barrier returns at once and counts the step; without it the kernel gives
    up after its time limit, records which peer was missing, and the context stays usable."""
    import time

    lib = cabi.load()
    flags = torch.zeros(2, dtype=torch.int32, device=DEV)       # this rank's flag array
    other = torch.zeros(2, dtype=torch.int32, device=DEV)       # the emulated peer's flag array
    state = torch.zeros(2, dtype=torch.int32, device=DEV)
    ptrs = _ptr_array([flags.data_ptr(), other.data_ptr()])
    flags[1] = 1  # "rank 1 has reached step 1"
    cabi.check(lib.b200ops_peer_barrier(ptrs, p(flags), p(state), 2, 0, stream()))
    torch.cuda.synchronize()
    assert state.cpu().tolist() == [1, 0]
    assert flags.cpu().tolist() == [1, 1] and other.cpu().tolist() == [1, 0]  # own arrival announced to both
    t0 = time.perf_counter()
    cabi.check(lib.b200ops_peer_barrier(ptrs, p(flags), p(state), 2, 0, stream()))  # nobody sets step 2
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert state.cpu().tolist() == [2, 101]  # peer 1 never arrived
    assert 1.0 < waited < 10.0
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0  # the device still answers


@pytest.mark.parametrize("pair_mode", ["0", "2"])  # single-CTA kernel / CTA-pair kernel
@pytest.mark.parametrize("counts,k,n", [([40, 3, 0, 21], 256, 192), ([70], 8192, 256),  # second: split-K path
                                        ([300, 129, 0, 60], 512, 320)])
def test_grouped_matmul_scatter_equals_matmul_then_push(cabi, monkeypatch, counts, k, n, pair_mode):
    """The GEMM whose epilogue stores into the (emulated) peers' return buffers must leave
    exactly what grouped_matmul followed by push_rows leaves."""
    knob(monkeypatch, "B200OPS_GMM_PAIR", pair_mode)
    lib = cabi.load()
    world, rank, cap = 2, 1, 256
    g = torch.Generator().manual_seed(sum(counts) + k)
    m = sum(counts)
    x = torch.randn(m, k, generator=g).half().to(DEV)
    w = (torch.randn(len(counts), n, k, generator=g) * 0.05).half().to(DEV)
    gl = torch.tensor(counts).cumsum(0).to(torch.int64).to(DEV)
    # every grouped row returns to a distinct (peer, offset); a few rows are dropped (-1)
    idx = torch.randperm(world * cap, generator=g)[:m].int()
    idx[::9] = -1
    idx = idx.to(DEV)
    nbytes = cabi.grouped_matmul_workspace_size(m, k, len(counts), n)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
    fused = [torch.zeros(world * cap, n, dtype=torch.float16, device=DEV) for _ in range(world)]
    cabi.check(lib.b200ops_grouped_matmul_scatter(p(x), p(w), p(gl), m, k, len(counts), n,
                                                  p(ws) if nbytes else None, nbytes, p(idx),
                                                  _ptr_array([b.data_ptr() for b in fused]), world, cap, rank,
                                                  stream()))
    y = torch.empty(m, n, dtype=torch.float16, device=DEV)
    cabi.grouped_matmul(x, w, gl, y, ws if nbytes else None)
    plain = [torch.zeros(world * cap, n, dtype=torch.float16, device=DEV) for _ in range(world)]
    cabi.check(lib.b200ops_moe_push_rows(p(y), p(idx), 1, None, m, _ptr_array([b.data_ptr() for b in plain]),
                                         world, cap, rank, n, None, 0, None, stream()))
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    for a, b in zip(fused, plain):
        assert torch.equal(a, b)
    assert sum(int((b.abs().sum(1) > 0).sum()) for b in fused) == int((idx >= 0).sum())


# ---------------------------------------------------------------------------------------
# The fused expert-parallel step (dispatch / gather / combine), all ranks emulated on this GPU.
# The launches run one after the other on one stream, so every announcement a kernel waits for
# was made by a launch that has already completed: no kernel ever waits for a later launch.
class EmulatedRanks:
    def __init__(self, world, spr, cap, hidden, hidden_out, max_rows=None):
        self.world, self.spr, self.cap, self.h, self.ho = world, spr, cap, hidden, hidden_out
        self.slots = world * spr
        rows = self.slots * cap
        self.max_rows = rows if max_rows is None else max_rows
        z = lambda *s, dt=torch.int32: torch.zeros(*s, dtype=dt, device=DEV)
        self.recv = [z(rows, hidden, dt=torch.float16) for _ in range(world)]
        self.ret = [z(rows, hidden_out, dt=torch.float16) for _ in range(world)]
        self.counts = [z(world, spr) for _ in range(world)]
        self.flags_r = [z(world) for _ in range(world)]
        self.cursor = [z(self.slots) for _ in range(world)]
        self.state = [z(8) for _ in range(world)]
        self.overflow = [z(2) for _ in range(world)]
        arr = lambda bufs: _ptr_array([b.data_ptr() for b in bufs])
        self.p_recv, self.p_ret, self.p_counts = arr(self.recv), arr(self.ret), arr(self.counts)
        self.p_flags_r = arr(self.flags_r)

    def step(self, cabi, xs, ids, wts, weights, router=None, top_k=None, tables=None, offsets=None):
        """One exchange step of all ranks.  weights[r] = [spr, n, k] f16 of rank r's slots (a plain
        grouped_matmul per rank stands for the expert MLP).  Returns (y per rank, pos per rank,
        ids per rank, wts per rank)."""
        lib = cabi.load()
        w_, spr, cap = self.world, self.spr, self.cap
        pos, out_ids, out_w = [], [], []
        for r in range(w_):
            t = xs[r].shape[0]
            k = top_k if router is not None else ids[r].shape[1]
            pr = torch.full((t * k,), -7, dtype=torch.int32, device=DEV)
            oi = torch.full((t, k), -1, dtype=torch.int32, device=DEV)
            ow = torch.zeros(t, k, device=DEV)
            cabi.check(lib.b200ops_moe_dispatch(
                p(xs[r]), p(router), None if router is not None else p(ids[r]),
                p(oi) if router is not None else None, p(ow) if router is not None else None,
                p(tables[0]) if tables else None, p(tables[1]) if tables else None,
                tables[0].shape[1] if tables else 0, offsets[r] if offsets else 0, p(pr), self.p_recv,
                self.p_counts, p(self.cursor[r]), p(self.state[r]), p(self.overflow[r]), t,
                self.h, router.shape[0] if router is not None else (tables[1].numel() if tables else self.slots),
                k, self.slots, w_, cap, r, stream()))
            pos.append(pr)
            out_ids.append(oi if router is not None else ids[r])
            out_w.append(ow if router is not None else wts[r])
        ys = []
        for r in range(w_):
            grouped = torch.full((self.max_rows, self.h), float("nan"), dtype=torch.float16, device=DEV)
            back = torch.full((self.max_rows,), -9, dtype=torch.int32, device=DEV)
            gl = torch.zeros(spr, dtype=torch.int64, device=DEV)
            total = torch.zeros(1, dtype=torch.int32, device=DEV)
            cabi.check(lib.b200ops_moe_gather(p(self.recv[r]), p(self.counts[r]),
                                              p(self.state[r]), p(self.overflow[r]), p(grouped), p(back), p(gl),
                                              p(total), self.h, w_, spr, cap, self.max_rows, stream()))
            n = weights[r].shape[1]
            nbytes = cabi.grouped_matmul_workspace_size(self.max_rows, self.h, spr, n)
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
            cabi.check(lib.b200ops_grouped_matmul_scatter(p(grouped), p(weights[r]), p(gl), self.max_rows, self.h,
                                                          spr, n, p(ws) if nbytes else None, nbytes, p(back),
                                                          self.p_ret, w_, spr * cap, r, stream()))
        for r in range(w_):
            # the peers' "returned" announcements come from their combine launches, which in
            # this one-stream emulation run later: set them by hand (their GEMMs have completed)
            step_no = self.state[r][0:1].clone()
            for peer in range(w_):
                if peer != r:
                    self.flags_r[r][peer:peer + 1] = step_no
            t, k = out_w[r].shape
            y = torch.full((t, self.ho), float("nan"), dtype=torch.float16, device=DEV)
            cabi.check(lib.b200ops_moe_combine(p(self.ret[r]), p(pos[r]), p(out_w[r]), p(y), self.p_flags_r,
                                               p(self.flags_r[r]), p(self.state[r]), t, k, self.ho, w_, r, stream()))
            ys.append(y)
        torch.cuda.synchronize()
        return ys, pos, out_ids, out_w


def _mlp_reference(x, ids, wts, slot_of, slot_weights, pos):
    """y[t] = sum_k w[t,k] * (x[t] @ W[slot(t,k)]^T) over the slots that were placed (pos >= 0)."""
    y = torch.zeros(x.shape[0], slot_weights[0].shape[0])
    for t in range(x.shape[0]):
        for k in range(ids.shape[1]):
            if pos[t * ids.shape[1] + k] < 0:
                continue
            s = slot_of(t, int(ids[t, k]))
            y[t] += float(wts[t, k]) * (x[t].float() @ slot_weights[s].float().T).half().float()
    return y


@pytest.mark.parametrize("world,spr,tokens", [(2, 2, 37), (4, 1, 16), (1, 3, 50)])
def test_fused_expert_parallel_step_emulated_ranks(cabi, world, spr, tokens):
    """Given expert ids, ample capacity, two steps in a row (the second with other inputs, so
    cursors, counts and step numbers must have been left ready by the first)."""
    h, n, top_k = 128, 192, 2
    slots = world * spr
    g = torch.Generator().manual_seed(world * 100 + spr)
    em = EmulatedRanks(world, spr, cap=tokens * top_k, hidden=h, hidden_out=n)
    slot_w = [(torch.randn(n, h, generator=g) * 0.1).half() for _ in range(slots)]
    weights = [torch.stack(slot_w[r * spr:(r + 1) * spr]).to(DEV) for r in range(world)]
    for step in (1, 2):
        xs = [torch.randn(tokens, h, generator=g).half() for _ in range(world)]
        ids = [torch.randint(0, slots, (tokens, top_k), generator=g, dtype=torch.int32) for _ in range(world)]
        for r in range(world):
            ids[r][0, 0] = -1          # an invalid id: left out
            ids[r][1, 1] = slots + 5   # another
        wts = [torch.rand(tokens, top_k, generator=g) for _ in range(world)]
        ys, pos, _, _ = em.step(cabi, [x.to(DEV) for x in xs], [i.to(DEV) for i in ids],
                                [w.to(DEV) for w in wts], weights)
        for r in range(world):
            assert em.state[r].cpu().tolist()[:5] == [step, 0, 0, 0, 0]
            assert em.overflow[r].cpu().tolist() == [0, 0] and em.cursor[r].abs().sum() == 0
            pr = pos[r].cpu().tolist()
            assert pr[0] == -1 and pr[top_k + 1] == -1 and sum(v < 0 for v in pr) == 2
            want = _mlp_reference(xs[r], ids[r], wts[r], lambda t, e: e, slot_w, pr)
            torch.testing.assert_close(ys[r].cpu().float(), want, rtol=1e-2, atol=2e-3)
        assert cabi.pipeline_status() == 0


def test_fused_dispatch_routes_like_route_topk_and_spreads_replicas(cabi):
    """Router inside the dispatch launch (same choices and probabilities as moe_route_topk), and an
    expert-to-slot table with a replicated expert: replica = (token_offset + t) mod replicas."""
    lib = cabi.load()
    world, spr, tokens, h, n, experts, top_k = 2, 3, 41, 256, 64, 4, 2
    g = torch.Generator().manual_seed(9)
    router = (torch.randn(experts, h, generator=g) * 0.05).half().to(DEV)
    # six slots: expert 0 three times (slots 0, 2, 5), experts 1, 2, 3 once (slots 1, 3, 4)
    slot_expert = [0, 1, 0, 2, 3, 0]
    table = torch.tensor([[0, 2, 5], [1, 1, 1], [3, 3, 3], [4, 4, 4]], dtype=torch.int32, device=DEV)
    reps = torch.tensor([3, 1, 1, 1], dtype=torch.int32, device=DEV)
    expert_w = [(torch.randn(n, h, generator=g) * 0.1).half() for _ in range(experts)]
    slot_w = [expert_w[e] for e in slot_expert]
    weights = [torch.stack(slot_w[r * spr:(r + 1) * spr]).to(DEV) for r in range(world)]
    em = EmulatedRanks(world, spr, cap=tokens * top_k, hidden=h, hidden_out=n)
    xs = [torch.randn(tokens, h, generator=g).half() for _ in range(world)]
    offsets = [0, tokens]
    ys, pos, ids, wts = em.step(cabi, [x.to(DEV) for x in xs], None, None, weights, router=router, top_k=top_k,
                                tables=(table, reps), offsets=offsets)
    for r in range(world):
        want_ids = torch.full((tokens, top_k), -1, dtype=torch.int32, device=DEV)
        want_w = torch.zeros(tokens, top_k, device=DEV)
        cabi.check(lib.b200ops_moe_route_topk(p(xs[r].to(DEV)), p(router), p(want_ids), p(want_w), tokens, h,
                                              experts, top_k, stream()))
        torch.cuda.synchronize()
        assert torch.equal(ids[r], want_ids) and torch.equal(wts[r], want_w)
        pr = pos[r].cpu().tolist()
        cap = tokens * top_k
        for t in range(tokens):
            for k in range(top_k):
                e = int(ids[r][t, k])
                want_slot = int(table[e, (offsets[r] + t) % int(reps[e])])
                assert pr[t * top_k + k] // cap == want_slot
        want = _mlp_reference(xs[r], ids[r].cpu(), wts[r].cpu(),
                              lambda t, e, r=r: int(table[e, (offsets[r] + t) % int(reps[e])]), slot_w, pr)
        torch.testing.assert_close(ys[r].cpu().float(), want, rtol=1e-2, atol=2e-3)


def test_fused_step_counts_rows_that_do_not_fit(cabi):
    """A sub-segment too small for the rows routed to it, and a grouped buffer too small for the
    rows received: the rows left out are counted, the others come back right."""
    world, spr, tokens, h, n, top_k = 2, 1, 24, 64, 64, 1
    g = torch.Generator().manual_seed(4)
    slot_w = [(torch.randn(n, h, generator=g) * 0.1).half() for _ in range(world)]
    weights = [w[None].to(DEV) for w in slot_w]
    xs = [torch.randn(tokens, h, generator=g).half() for _ in range(world)]
    ids = [torch.zeros(tokens, 1, dtype=torch.int32) for _ in range(world)]  # everything to slot 0
    wts = [torch.ones(tokens, 1) for _ in range(world)]
    em = EmulatedRanks(world, spr, cap=16, hidden=h, hidden_out=n)  # 24 rows into segments of 16
    ys, pos, _, _ = em.step(cabi, [x.to(DEV) for x in xs], [i.to(DEV) for i in ids], [w.to(DEV) for w in wts],
                            weights)
    for r in range(world):
        assert em.overflow[r].cpu().tolist()[0] == 8
        pr = pos[r].cpu().tolist()
        assert sum(v < 0 for v in pr) == 8
        want = _mlp_reference(xs[r], ids[r], wts[r], lambda t, e: e, slot_w, pr)
        torch.testing.assert_close(ys[r].cpu().float(), want, rtol=1e-2, atol=2e-3)
    # second form: ample sub-segments, but the receiving rank keeps only 40 of its 48 rows
    em = EmulatedRanks(world, spr, cap=32, hidden=h, hidden_out=n, max_rows=40)
    em.step(cabi, [x.to(DEV) for x in xs], [i.to(DEV) for i in ids], [w.to(DEV) for w in wts], weights)
    assert em.overflow[0].cpu().tolist() == [0, 8] and em.overflow[1].cpu().tolist() == [0, 0]


def test_fused_gather_gives_up_when_a_peer_never_announces(cabi):
    """The wait inside the gather launch is bounded like the barrier's: with one source's count
    words missing it records 100 + source, carries on, and the context stays usable."""
    import time

    lib = cabi.load()
    em = EmulatedRanks(2, 1, cap=4, hidden=64, hidden_out=64)
    x = torch.randn(3, 64, device=DEV, dtype=torch.float16)
    ids = torch.zeros(3, 1, dtype=torch.int32, device=DEV)
    pos = torch.empty(3, dtype=torch.int32, device=DEV)
    cabi.check(lib.b200ops_moe_dispatch(p(x), None, p(ids), None, None, None, None, 0, 0, p(pos), em.p_recv,
                                        em.p_counts, p(em.cursor[0]), p(em.state[0]), None, 3, 64, 2,
                                        1, 2, 2, 4, 0, stream()))  # rank 0 only: rank 1 never dispatches
    grouped = torch.zeros(8, 64, dtype=torch.float16, device=DEV)
    back = torch.zeros(8, dtype=torch.int32, device=DEV)
    gl = torch.zeros(1, dtype=torch.int64, device=DEV)
    total = torch.zeros(1, dtype=torch.int32, device=DEV)
    t0 = time.perf_counter()
    cabi.check(lib.b200ops_moe_gather(p(em.recv[0]), p(em.counts[0]), p(em.state[0]), None,
                                      p(grouped), p(back), p(gl), p(total), 64, 2, 1, 4, 8, stream()))
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert em.state[0].cpu().tolist()[:2] == [1, 101]
    assert 1.0 < waited < 10.0
    assert int(total) == 3  # its own rows arrived all the same (in the order the CTAs claimed them)
    order = lambda t: t[torch.argsort(t[:, 0].float())]
    assert torch.equal(order(grouped[:3]), order(x))
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0
