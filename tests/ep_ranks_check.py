"""Child program of test_layer_gpu.py: run under torchrun, one rank per GPU (2, 4 or 8 ranks).

Checks the expert-parallel paths against the single-GPU path on the same inputs:
  1. the decode layer with the NCCL exchange (experts placed contiguously),
  2. the same layer with the NVLink peer-memory exchange (fused dispatch / gather / combine, the
     down projection storing into the peers' return buffers), three steps in a row so that the
     buffers, cursors and step numbers are reused, and once more with the separate return push,
  3. the MoE MLP with a skewed routing histogram and replicated experts (balanced placement,
     bounded sub-segments) through the peer exchange,
each rank comparing its own rows with what ONE GPU holding every expert computes for them.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO / "ascend-ops_b200"))

import ascend910a_extras.moe as moe  # noqa: E402
import ascend910a_extras.ops as ops  # noqa: E402
import moe_decode_layer as mdl  # noqa: E402
import moe_parallel  # noqa: E402

TOL = dict(rtol=1e-2, atol=2e-3)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    cfg = mdl.LayerConfig(hidden=512, heads=8, kv_heads=2, head_dim=128, intermediate=256, experts=8)
    per = 6
    full = mdl.make_weights(cfg, seed=3, std=0.05)
    pos = mdl.draw_positions(per * world, 3, 900, seed=5)
    b = mdl.make_decode_batch(cfg, positions=pos[rank * per:(rank + 1) * per], seed=20 + rank)
    g = torch.Generator().manual_seed(30 + rank)
    kc = torch.randn(b["cache_shape"], generator=g).half()
    vc = torch.randn(b["cache_shape"], generator=g).half()
    args = [b[n].to(dev) for n in ("x", "residual", "positions", "slots", "block_tables", "context_lens")]

    # ---- what one GPU with every expert computes for this rank's sequences ----
    solo = mdl.MoEDecodeLayer(cfg, full, dev, ops, group=None)
    solo.local_only = True
    y_solo, res_solo = solo.forward(*args, kc.to(dev), vc.to(dev))

    # ---- 1. NCCL exchange ----
    mine = moe_parallel.local_experts(cfg.experts, world, rank).tolist()
    part = mdl.make_weights(cfg, seed=3, std=0.05, experts=mine)
    ep = mdl.MoEDecodeLayer(cfg, part, dev, ops, group=group, segment_rows=per * cfg.top_k)
    y_ep, res_ep = ep.forward(*args, kc.to(dev), vc.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(res_ep, res_solo)
    torch.testing.assert_close(y_ep.float(), y_solo.float(), **TOL)

    # ---- 2. peer-memory exchange, fused launches ----
    ex = moe_parallel.PeerExchange(moe, group, dev, per * cfg.top_k, cfg.hidden, cfg.hidden, cfg.experts)
    peer = mdl.MoEDecodeLayer(cfg, part, dev, ops, group=group, segment_rows=per * cfg.top_k, exchange=ex)
    for _ in range(3):
        y_peer, res_peer = peer.forward(*args, kc.to(dev), vc.to(dev))
    torch.cuda.synchronize()
    assert ex.barrier_error() == 0, f"a peer announcement timed out: {ex.barrier_error()}"
    assert ex.overflow.cpu().tolist() == [0, 0]
    assert torch.equal(res_peer, res_solo)
    torch.testing.assert_close(y_peer.float(), y_solo.float(), **TOL)
    peer.fuse_return = False  # separate push_rows launch instead of the GEMM's scatter epilogue
    y_unfused, _ = peer.forward(*args, kc.to(dev), vc.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(y_unfused, y_peer)
    # the same step replayed from a CUDA graph
    peer.fuse_return = True
    step = mdl.CapturedDecodeStep(peer, b, kc.to(dev), vc.to(dev))
    for _ in range(3):
        y_graph, res_graph = step.run()
    torch.cuda.synchronize()
    assert ex.barrier_error() == 0
    assert torch.equal(y_graph, y_peer) and torch.equal(res_graph, res_solo)

    # ---- 3. MoE MLP, skewed routing, replicated experts, bounded sub-segments ----
    tokens, top_k = 96, 2
    gi = torch.Generator().manual_seed(77)
    prob = torch.softmax(2.0 * torch.randn(cfg.experts, generator=gi), 0)
    ids_all = torch.multinomial(prob, tokens * world * top_k, replacement=True, generator=gi).view(-1, top_k).int()
    load = torch.bincount(ids_all.flatten().long(), minlength=cfg.experts).tolist()
    spr = cfg.experts // world + 2
    placement = moe_parallel.balanced_placement(load, world, spr).to(dev)
    assert int(placement.num_replicas.max()) >= 2  # a replicated expert is part of the case
    my_ids = ids_all[rank * tokens:(rank + 1) * tokens].contiguous().to(dev)
    gx = torch.Generator(device=dev).manual_seed(50 + rank)
    x = torch.randn(tokens, cfg.hidden, generator=gx, device=dev, dtype=torch.float16)
    wts = torch.rand(tokens, top_k, generator=gx, device=dev)
    w_slots = mdl.make_weights(cfg, seed=3, std=0.05, experts=placement.local_slot_experts(rank), device="cpu")
    s_gu, s_dn = w_slots["w_gate_up"].to(dev).transpose(1, 2), w_slots["w_down"].to(dev).transpose(1, 2)
    a_gu, a_dn = full["w_gate_up"].to(dev).transpose(1, 2), full["w_down"].to(dev).transpose(1, 2)

    def mlp(gu, dn):
        return lambda rows, gl: ops.grouped_matmul(moe.grouped_matmul_swiglu(rows, gu, gl), dn, gl)

    def mlp_scatter(rows, gl, scatter):
        moe.grouped_matmul_scatter(moe.grouped_matmul_swiglu(rows, s_gu, gl), s_dn, gl, *scatter)

    want = moe_parallel.expert_parallel_mlp_device(moe, x, my_ids, wts, cfg.experts, mlp(a_gu, a_dn), local=True)
    ex2 = moe_parallel.PeerExchange(moe, group, dev, tokens * top_k, cfg.hidden, cfg.hidden, placement.num_slots,
                                    max_rows=tokens * top_k * world)
    for _ in range(2):
        got = ex2.mlp(x, my_ids, wts, mlp(s_gu, s_dn), local_mlp_scatter=mlp_scatter, placement=placement,
                      token_offset=rank * tokens, num_experts=cfg.experts)
    torch.cuda.synchronize()
    assert ex2.barrier_error() == 0 and ex2.overflow.cpu().tolist() == [0, 0]
    torch.testing.assert_close(got.float(), want.float(), **TOL)
    assert float(want.float().abs().max()) > 0

    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} of {world} EP_CHECK_OK", flush=True)


if __name__ == "__main__":
    main()
