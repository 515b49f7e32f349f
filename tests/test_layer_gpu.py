"""The MoE decoder layer (decode step) on the GPU against the CPU oracle's layer, stage by
stage, at a reduced size; the expert-parallel paths on every visible GPU when there are at least
two; and a step at the benchmark's full dimensions against the oracle on sampled sequences."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import moe_decode_layer as mdl
from oracle import decode_ops_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REPO = Path(__file__).resolve().parent.parent


def small_case(batch=12, seed=3):
    cfg = mdl.LayerConfig(hidden=512, heads=8, kv_heads=2, head_dim=128, intermediate=256, experts=4)
    w = mdl.make_weights(cfg, seed=seed, std=0.05)
    b = mdl.make_decode_batch(cfg, batch=batch, min_pos=3, max_pos=900, seed=seed + 1)
    g = torch.Generator().manual_seed(seed + 2)
    kc = torch.randn(b["cache_shape"], generator=g).half()
    vc = torch.randn(b["cache_shape"], generator=g).half()
    return cfg, w, b, kc, vc


def test_layer_matches_oracle_stage_by_stage(ops):
    cfg, w, b, kc, vc = small_case()
    layer = mdl.MoEDecodeLayer(cfg, w, DEV, ops)
    kd, vd = kc.to(DEV), vc.to(DEV)
    y, res, ids, wts = layer.forward(*(b[n].to(DEV) for n in ("x", "residual", "positions", "slots",
                                                              "block_tables", "context_lens")),
                                     kd, vd, return_routing=True)
    torch.cuda.synchronize()
    cos, sin = oracle.cos_sin_cache(16385, cfg.head_dim, cfg.rope_theta)
    kw = dict(heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, experts=cfg.experts,
              top_k=cfg.top_k, eps=cfg.eps, cos_cache=cos, sin_cache=sin)
    kc_o, vc_o = kc.clone(), vc.clone()
    ey, eres, eids, ewts, st = oracle.moe_decode_layer(w, b, kc_o, vc_o, expert_ids=ids.cpu(),
                                                       expert_weights=wts.cpu(), **kw)
    # the scatter touched exactly the slots of the new tokens, with the rotated keys
    slots = b["slots"].long()
    flat_k = kd.cpu().view(-1, cfg.kv_heads, cfg.head_dim)
    torch.testing.assert_close(flat_k[slots].float(), st["k_rot"].float(), rtol=1e-2, atol=2e-3)
    untouched = torch.ones(flat_k.shape[0], dtype=torch.bool)
    untouched[slots] = False
    assert torch.equal(flat_k[untouched], kc.view(-1, cfg.kv_heads, cfg.head_dim)[untouched])
    # routing agrees except where the router's top-2 is a near tie
    same = (ids.cpu().sort(1).values == st["own_ids"].sort(1).values).all(1).float().mean()
    assert same >= 0.9
    torch.testing.assert_close(res.cpu().float(), eres.float(), rtol=1e-2, atol=2e-3)
    torch.testing.assert_close(y.cpu().float(), ey.float(), rtol=2e-2, atol=3e-3)


def test_layer_is_deterministic_and_cache_update_is_idempotent(ops):
    cfg, w, b, kc, vc = small_case(batch=5, seed=11)
    layer = mdl.MoEDecodeLayer(cfg, w, DEV, ops)
    kd, vd = kc.to(DEV), vc.to(DEV)
    args = [b[n].to(DEV) for n in ("x", "residual", "positions", "slots", "block_tables", "context_lens")]
    y1, r1 = layer.forward(*args, kd, vd)
    k_after = kd.clone()
    y2, r2 = layer.forward(*args, kd, vd)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and torch.equal(r1, r2) and torch.equal(k_after, kd)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_expert_parallel_ranks_match_single_gpu(tmp_path):
    """One rank per visible GPU (2, 4 or 8): the layer over the NCCL exchange and over the fused
    peer-memory exchange, and the MoE MLP with replicated experts, each rank's rows against the
    single-GPU path (tests/ep_ranks_check.py).  NVLS stays off: a rank that died while bound to an
    NVLink multicast object would fault its peers."""
    n = torch.cuda.device_count()
    ranks = 8 if n >= 8 else (4 if n >= 4 else 2)
    script = Path(__file__).with_name("ep_ranks_check.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
                        "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("EP_CHECK_OK") == ranks


@pytest.mark.parametrize("nz", [False, True])
def test_fused_rope_cache_equals_the_two_operators(ops, nz):
    import ascend910a_extras.moe as moe
    import decode_workloads as wl

    g = torch.Generator().manual_seed(4)
    t, hq, hkv, d, pages, p = 37, 8, 2, 128, 9, 16
    qkv = torch.randn(t, (hq + 2 * hkv) * d, generator=g).half().to(DEV)
    r = wl.rope_inputs(t, hq, hkv, d, 0, 200, seed=3)
    pos, cos, sin = (r[n].to(DEV) for n in ("position_ids", "cos_cache", "sin_cache"))
    pos[2] = 5000  # outside the table: zeros, as in ops.rope
    slots = torch.randperm(pages * p, generator=g)[:t].int().to(DEV)
    slots[5] = -1
    shape = (pages, hkv * d // 16, p, 16) if nz else (pages, p, hkv, d)
    base = torch.randn(shape, generator=g).half()
    kc1, vc1, kc2, vc2 = (base.to(DEV).clone() for _ in range(4))
    q1 = moe.fused_qkv_rope_cache(qkv, pos, cos, sin, slots, kc1, vc1, hq, hkv)
    q = qkv[:, : hq * d].contiguous().view(t, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].contiguous().view(t, hkv, d)
    v = qkv[:, (hq + hkv) * d:].contiguous().view(t, hkv, d)
    q2, k2 = ops.rope(q, k, pos, cos, sin)
    ops.reshape_and_cache(k2, v, kc2, vc2, slots)
    torch.cuda.synchronize()
    assert torch.equal(q1, q2) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert not torch.equal(kc1.cpu(), base)


def test_captured_step_equals_eager_step(ops):
    cfg, w, b, kc, vc = small_case(batch=9, seed=21)
    layer = mdl.MoEDecodeLayer(cfg, w, DEV, ops)
    kd, vd = kc.to(DEV), vc.to(DEV)
    args = [b[n].to(DEV) for n in mdl.CapturedDecodeStep.NAMES]
    y_eager, r_eager = layer.forward(*args, kd, vd)
    step = mdl.CapturedDecodeStep(layer, b, kd, vd)
    step.load({n: b[n].pin_memory() for n in step.NAMES})
    y, r = step.run()
    torch.cuda.synchronize()
    assert torch.equal(y, y_eager) and torch.equal(r, r_eager)
    # new inputs through the same graph
    b2 = dict(b)
    b2["x"] = (b["x"].float() * 0.5).half()
    step.load(b2)
    y2, _ = step.run()
    y2_eager, _ = layer.forward(b2["x"].to(DEV), *args[1:], kd, vd)
    torch.cuda.synchronize()
    assert torch.equal(y2, y2_eager) and not torch.equal(y2, y_eager)


def test_host_to_host_step_equals_eager_step(ops):
    """The recording that includes the copies (inputs up from pinned host memory, residual_out
    down early on a side stream, y down at the end) must return what the eager step returns,
    also for new contents of the host buffers."""
    cfg, w, b, kc, vc = small_case(batch=9, seed=22)
    layer = mdl.MoEDecodeLayer(cfg, w, DEV, ops)
    kd, vd = kc.to(DEV), vc.to(DEV)
    args = [b[n].to(DEV) for n in mdl.CapturedDecodeStep.NAMES]
    y_eager, r_eager = layer.forward(*args, kd, vd)
    step = mdl.CapturedDecodeStep(layer, b, kd, vd, host_io=True)
    y, r = step.run_host()
    torch.cuda.synchronize()
    assert torch.equal(y, y_eager.cpu()) and torch.equal(r, r_eager.cpu())
    step.host_in["x"].copy_((b["x"].float() * 0.25).half())
    step.host_in["residual"].copy_((b["residual"].float() - 1.0).half())
    y2, r2 = step.run_host()
    torch.cuda.synchronize()
    y2_eager, r2_eager = layer.forward(step.host_in["x"].to(DEV), step.host_in["residual"].to(DEV), *args[2:], kd, vd)
    torch.cuda.synchronize()
    assert torch.equal(y2, y2_eager.cpu()) and torch.equal(r2, r2_eager.cpu())
    assert not torch.equal(y2, y_eager.cpu())
    with pytest.raises(RuntimeError):
        mdl.CapturedDecodeStep(layer, b, kd, vd).run_host()


def test_layer_with_per_head_qk_norm_matches_oracle_and_unfused_operators(ops):
    """Qwen3-style layer: RMSNorm over head_dim on q and k between the split and rope.  The
    fused kernel (norm + rope + cache scatter in one launch) against the oracle, and against the
    stand-alone operators (add_rms_norm with a zero residual, rope, reshape_and_cache)."""
    cfg = mdl.LayerConfig(hidden=512, heads=8, kv_heads=2, head_dim=128, intermediate=256, experts=4, qk_norm=True)
    w = mdl.make_weights(cfg, seed=31, std=0.05)
    b = mdl.make_decode_batch(cfg, batch=11, min_pos=3, max_pos=900, seed=32)
    g = torch.Generator().manual_seed(33)
    kc = torch.randn(b["cache_shape"], generator=g).half()
    vc = torch.randn(b["cache_shape"], generator=g).half()
    names = ("x", "residual", "positions", "slots", "block_tables", "context_lens")
    layer = mdl.MoEDecodeLayer(cfg, w, DEV, ops)
    kd, vd = kc.to(DEV), vc.to(DEV)
    y, res, ids, wts = layer.forward(*(b[n].to(DEV) for n in names), kd, vd, return_routing=True)
    layer.fuse_rope_cache = False
    kd2, vd2 = kc.to(DEV), vc.to(DEV)
    y2, res2 = layer.forward(*(b[n].to(DEV) for n in names), kd2, vd2)
    torch.cuda.synchronize()
    torch.testing.assert_close(kd.float(), kd2.float(), rtol=1e-2, atol=2e-3)
    assert torch.equal(vd, vd2)
    torch.testing.assert_close(y.float(), y2.float(), rtol=2e-2, atol=3e-3)
    cos, sin = oracle.cos_sin_cache(16385, cfg.head_dim, cfg.rope_theta)
    kc_o, vc_o = kc.clone(), vc.clone()
    ey, eres, _, _, st = oracle.moe_decode_layer(
        w, b, kc_o, vc_o, expert_ids=ids.cpu(), expert_weights=wts.cpu(), heads=cfg.heads, kv_heads=cfg.kv_heads,
        head_dim=cfg.head_dim, experts=cfg.experts, top_k=cfg.top_k, eps=cfg.eps, cos_cache=cos, sin_cache=sin)
    slots = b["slots"].long()
    flat_k = kd.cpu().view(-1, cfg.kv_heads, cfg.head_dim)
    torch.testing.assert_close(flat_k[slots].float(), st["k_rot"].float(), rtol=1e-2, atol=2e-3)
    assert float(st["k_rot"].float().pow(2).mean().sqrt()) > 0.5  # normalised keys: unit scale, not 0.05-ish
    torch.testing.assert_close(res.cpu().float(), eres.float(), rtol=1e-2, atol=2e-3)
    torch.testing.assert_close(y.cpu().float(), ey.float(), rtol=2e-2, atol=3e-3)


@pytest.mark.parametrize("head_dim,heads,kv_heads", [(64, 5, 1), (128, 4, 4), (256, 3, 1), (32, 7, 2)])
def test_fused_qk_norm_head_sizes(head_dim, heads, kv_heads):
    """The in-kernel head reduction for every supported head size, including head counts that
    leave a warp's last lanes past the end of the work."""
    import ascend910a_extras.moe as moe

    g = torch.Generator().manual_seed(head_dim + heads)
    t = 9
    qkv = torch.randn(t, (heads + 2 * kv_heads) * head_dim, generator=g).half()
    qw = (1 + 0.1 * torch.randn(head_dim, generator=g)).half()
    kw = (1 + 0.1 * torch.randn(head_dim, generator=g)).half()
    pos = torch.randint(0, 50, (t,), generator=g, dtype=torch.int32)
    cos, sin = oracle.cos_sin_cache(64, head_dim, 1e4)
    slots = torch.randperm(32, generator=g)[:t].int()
    kc = torch.zeros(2, 16, kv_heads, head_dim, dtype=torch.float16, device=DEV)
    vc = torch.zeros_like(kc)
    q = moe.fused_qkv_rope_cache(qkv.to(DEV), pos.to(DEV), cos.to(DEV), sin.to(DEV), slots.to(DEV), kc, vc,
                                 heads, kv_heads, qw.to(DEV), kw.to(DEV), 1e-6).cpu()
    nq, nkv = heads * head_dim, kv_heads * head_dim
    q_ref = oracle.head_rms_norm(qkv[:, :nq].reshape(t, heads, head_dim), qw, 1e-6)
    k_ref = oracle.head_rms_norm(qkv[:, nq:nq + nkv].reshape(t, kv_heads, head_dim), kw, 1e-6)
    q_ref, k_ref = oracle.rope(q_ref, k_ref, pos, cos, sin)
    torch.testing.assert_close(q.float(), q_ref.float(), rtol=1e-2, atol=2e-3)
    flat_k = kc.cpu().view(-1, kv_heads, head_dim)
    torch.testing.assert_close(flat_k[slots.long()].float(), k_ref.float(), rtol=1e-2, atol=2e-3)
    flat_v = vc.cpu().view(-1, kv_heads, head_dim)
    assert torch.equal(flat_v[slots.long()], qkv[:, nq + nkv:].reshape(t, kv_heads, head_dim))


def test_layer_step_at_benchmark_dimensions_on_sampled_sequences(ops):
    """The step the benchmark reports (batch 256, hidden 4096, 32 q / 8 kv heads, positions
    U[1024, 16384], 8 experts of 14336) against the CPU oracle on eight of its sequences, the
    longest and the shortest among them.  Every operator of the layer acts on a sequence by
    itself, so the oracle runs on just those sequences: their pages are gathered out of the
    9 GB cache (as it was before the step) into a small cache with a renumbered block table."""
    cfg = mdl.LayerConfig()
    w = mdl.make_weights(cfg, seed=7, device=DEV)
    batch = mdl.make_decode_batch(cfg, seed=8)
    g = torch.Generator(device=DEV).manual_seed(90)
    k_cache = torch.randn(batch["cache_shape"], generator=g, device=DEV, dtype=torch.float16)
    v_cache = torch.randn(batch["cache_shape"], generator=g, device=DEV, dtype=torch.float16)
    lens = batch["context_lens"].long()
    sample = sorted({0, 17, 101, 200, 255, int(lens.argmax()), int(lens.argmin()), 128})
    bs = cfg.block_size
    # the sampled sequences' pages, before the step writes the new tokens into them
    tables, new_slots, page_ids, o = [], [], [], 0
    for b in sample:
        n = int((lens[b] + bs - 1) // bs)
        ids = batch["block_tables"][b, :n].long()
        page_ids.append(ids)
        row = torch.zeros(batch["block_tables"].shape[1], dtype=torch.int32)
        row[:n] = torch.arange(o, o + n, dtype=torch.int32)
        tables.append(row)
        p = int(batch["positions"][b])
        new_slots.append((o + p // bs) * bs + p % bs)
        o += n
    gather = torch.cat(page_ids).to(DEV)
    k_small, v_small = k_cache[gather].cpu(), v_cache[gather].cpu()
    layer = mdl.MoEDecodeLayer(cfg, w, DEV, ops)
    names = ("x", "residual", "positions", "slots", "block_tables", "context_lens")
    y, res, ids, wts = layer.forward(*(batch[n].to(DEV) for n in names), k_cache, v_cache, return_routing=True)
    torch.cuda.synchronize()
    from ascend910a_extras import cabi
    assert cabi.pipeline_status() == 0
    sub = {"x": batch["x"][sample], "residual": batch["residual"][sample], "positions": batch["positions"][sample],
           "context_lens": batch["context_lens"][sample], "block_tables": torch.stack(tables),
           "slots": torch.tensor(new_slots, dtype=torch.int32)}
    w_cpu = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in w.items()}
    cos, sin = oracle.cos_sin_cache(16385, cfg.head_dim, cfg.rope_theta)
    ey, eres, _, _, st = oracle.moe_decode_layer(
        w_cpu, sub, k_small, v_small, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim,
        experts=cfg.experts, top_k=cfg.top_k, eps=cfg.eps, cos_cache=cos, sin_cache=sin,
        expert_ids=ids[sample].cpu().long(), expert_weights=wts[sample].cpu())
    # the new tokens' rotated keys landed in the right cache rows
    flat_k = k_cache.view(-1, cfg.kv_heads, cfg.head_dim)
    got_k = flat_k[batch["slots"][sample].long().to(DEV)].cpu()
    torch.testing.assert_close(got_k.float(), st["k_rot"].float(), rtol=1e-2, atol=2e-3)
    # routing: the same experts, except where two probabilities are within rounding of each other
    prob = torch.softmax(st["logits"].float(), -1)
    mine, theirs = ids[sample].cpu().long(), st["own_ids"]
    differs = mine.sort(1).values != theirs.sort(1).values
    if differs.any():
        gap = (prob.gather(1, mine).sort(1).values - prob.gather(1, theirs).sort(1).values).abs()
        assert float(gap.max()) < 5e-3
    torch.testing.assert_close(res[sample].cpu().float(), eres.float(), rtol=1e-2, atol=2e-3)
    torch.testing.assert_close(y[sample].cpu().float(), ey.float(), rtol=2e-2, atol=3e-3)
