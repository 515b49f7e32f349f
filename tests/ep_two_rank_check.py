"""Child program of test_layer_gpu.py: run under torchrun with two ranks (one GPU each)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO / "ascend-ops_b200"))

import ascend910a_extras.ops as ops  # noqa: E402
import moe_decode_layer as mdl  # noqa: E402
import moe_parallel  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    cfg = mdl.LayerConfig(hidden=512, heads=8, kv_heads=2, head_dim=128, intermediate=256, experts=4)
    full = mdl.make_weights(cfg, seed=3, std=0.05)
    pos = mdl.draw_positions(12, 3, 900, seed=5)
    per = 12 // world
    b = mdl.make_decode_batch(cfg, positions=pos[rank * per:(rank + 1) * per], seed=20 + rank)
    g = torch.Generator().manual_seed(30 + rank)
    kc = torch.randn(b["cache_shape"], generator=g).half()
    vc = torch.randn(b["cache_shape"], generator=g).half()
    args = [b[n].to(dev) for n in ("x", "residual", "positions", "slots", "block_tables", "context_lens")]
    # single-GPU layer with all experts, no process group
    solo = mdl.MoEDecodeLayer(cfg, full, dev, ops, group=None)
    # expert_parallel_mlp looks at the default group, so run the solo layer's MLP explicitly local
    h_y, h_res, ids, wts = None, None, None, None
    mine = moe_parallel.local_experts(cfg.experts, world, rank).tolist()
    part = mdl.make_weights(cfg, seed=3, std=0.05, experts=mine)
    ep = mdl.MoEDecodeLayer(cfg, part, dev, ops, group=dist.group.WORLD, segment_rows=per * cfg.top_k)
    y_ep, res_ep = ep.forward(*args, kc.to(dev), vc.to(dev))
    torch.cuda.synchronize()
    # the same layer with the NVLink peer-memory exchange instead of NCCL: identical rows move,
    # so the output must be bit-identical; run it three times to cross the buffer-reuse path
    import ascend910a_extras.moe as moe
    ex = moe_parallel.PeerExchange(moe, dist.group.WORLD, dev, per * cfg.top_k, cfg.hidden, cfg.hidden,
                                   cfg.experts)
    peer = mdl.MoEDecodeLayer(cfg, part, dev, ops, group=dist.group.WORLD, segment_rows=per * cfg.top_k,
                              exchange=ex)
    for _ in range(3):
        y_peer, res_peer = peer.forward(*args, kc.to(dev), vc.to(dev))
    torch.cuda.synchronize()
    assert ex.barrier_error() == 0, f"peer barrier gave up waiting: {ex.barrier_error()}"
    assert torch.equal(y_peer, y_ep) and torch.equal(res_peer, res_ep)
    peer.fuse_return = False  # separate push_rows launch instead of the fused GEMM epilogue
    y_unfused, _ = peer.forward(*args, kc.to(dev), vc.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(y_unfused, y_ep)
    dist.barrier()
    dist.destroy_process_group()  # from here on expert_parallel_mlp sees no group: local path
    y_solo, res_solo = solo.forward(*args, kc.to(dev), vc.to(dev))
    torch.cuda.synchronize()
    torch.testing.assert_close(res_ep.float(), res_solo.float(), rtol=0, atol=0)
    torch.testing.assert_close(y_ep.float(), y_solo.float(), rtol=1e-2, atol=2e-3)
    print(f"rank {rank} EP_CHECK_OK", flush=True)


if __name__ == "__main__":
    main()
