"""Benchmark of the B200 decode operator set.

    python bench.py --gpus N --steps K --warmup W          this implementation (GPU)
    python bench.py --impl reference ...                    the CPU golden path, for the ratio

Prints ONE JSON line on rank 0: `value` is device-timed with inputs resident in HBM, `e2e` goes
through the public `ascend910a_extras.ops` API from pinned host buffers with the copies inside
the timed region, `roofline` is the dominant kernel against the measured peak, `cpu_baseline`
times the CPU oracle's layer step, `ep_check` (more than one GPU) compares the exchanged result
with the single-GPU path, and `per_op` holds one short row per operator (columns in
`per_op_cols`: device time, achieved rate, fraction of the measured peak, the CPU oracle's time
on all host threads, and the GPU result's error against it).  Shapes, byte counts and the other
details of every row go to bench_detail_n<N>.json in the side-file directory (OUT_DIR).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO / "ascend-ops_b200"))
sys.path.insert(0, str(REPO))

import torch  # noqa: E402

import decode_workloads as wl  # noqa: E402

# DRAM traffic of the attention kernel relative to its algorithmic bytes (dram read + write over
# algorithmic bytes in an ncu capture of a 16-sequence case; the traffic grows in proportion to
# the context tokens, so the ratio carries over to the full batch).
ATTENTION_TRAFFIC_RATIO = 1.05

# Side files (row details, timelines) go here; the printed line never depends on them.
OUT_DIR = REPO / "gpurun_out"

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_BYTES = 126 * 1024 * 1024


def load_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d} | {"source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS) | {"source": "fallback"}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------- timing
def time_launches(launch, n_sets, steps, warmup, device, repeats=3):
    """Device time of one launch, in microseconds.

    `launch(i)` enqueues the operator on buffer set i (0 <= i < n_sets); the caller sizes the
    sets so that together (or each by itself) they exceed L2.  `steps` launches are enqueued
    back to back between two CUDA events on the launching stream, so the GPU never waits for
    the host's per-call work (argument checks, output allocation, descriptor encoding) and
    the figure is kernel time including the gaps between an operator's own kernels.  The
    median over `repeats` such batches is returned together with the raw list.
    """
    stream = torch.cuda.current_stream(device)
    for i in range(warmup):
        launch(i % n_sets)
    torch.cuda.synchronize(device)
    times = []
    for r in range(repeats):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            launch(i % n_sets)
        e1.record(stream)
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / steps)
    return statistics.median(times), times


def time_graph(launch, n_sets, reps, steps, warmup, device):
    """For kernels of a few microseconds: capture `reps` launches over rotating buffer sets in
    one CUDA graph so that CPU launch gaps do not dominate, and time graph replays.
    Returns microseconds per launch."""
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream(device)
    with torch.cuda.stream(s):
        for i in range(min(n_sets, 3)):
            launch(i)
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            for i in range(reps):
                launch(i % n_sets)
    torch.cuda.synchronize(device)
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize(device)
    times = []
    stream = torch.cuda.current_stream(device)
    for _ in range(steps):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        g.replay()
        e1.record(stream)
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / reps)
    return statistics.median(times), times


def sets_for(bytes_per_set, minimum=2, maximum=16):
    """How many rotating buffer sets make the combined footprint exceed twice the L2."""
    n = max(minimum, -(-2 * L2_BYTES // max(bytes_per_set, 1)))
    return int(min(n, maximum))


# --------------------------------------------------------------------------- per-op cases
# Every case returns one row: device time and roofline fraction of the operator at its benchmark
# size, and beside it the CPU oracle on the same tensors -- its time on all host threads and the
# error of the GPU result against it (max |got - want|, and the largest |got - want| /
# (atol + rtol * |want|) with the operator's tolerance rtol 1e-2 / atol 1e-3: <= 1 passes).
RTOL, ATOL = 1e-2, 1e-3


def _oracle():
    from oracle import decode_ops_oracle as oracle

    torch.set_num_threads(len(os.sched_getaffinity(0)))
    return oracle


def cpu_run(fn, repeats=1):
    best, out = None, None
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = fn()
        dt = (time.perf_counter() - t0) * 1e6
        best = dt if best is None else min(best, dt)
    return out, best


def errors(got, want, magnitude=None, atol=ATOL):
    """`magnitude` replaces |want| in the tolerance where `want` is a sum whose terms cancel (the
    error of such a sum scales with the terms, not with what is left of them)."""
    d = (got.float() - want.float()).abs()
    ref = want.float().abs() if magnitude is None else magnitude.float()
    return float(d.max()), float((d / (atol + RTOL * ref)).max())


def op_record(name, us, work, peaks, bound, cpu_us=None, err=None, launches=1, cpu_sample=None, **detail):
    if bound == "hbm":
        achieved, unit, peak = work / us / 1e3, "GB/s", peaks["hbm_gbs"]
    else:
        achieved, unit, peak = work / us / 1e6, "TFLOP/s", peaks["bf16_tflops"]
    rec = {"op": name, "us": round(us, 2), "achieved": round(achieved, 1), "unit": unit, "peak": peak,
           "frac": round(achieved / peak, 4), "bound": bound, "launches": launches,
           "work": int(work), "cpu_us": None if cpu_us is None else round(cpu_us, 1),
           "max_abs_err": None if err is None else float(f"{err[0]:.3g}"),
           "err_over_tol": None if err is None else float(f"{err[1]:.3g}")}
    if cpu_sample is not None:
        rec["cpu_sample"] = cpu_sample
    rec.update(detail)
    return rec


def case_add_rms_norm(ops, dev, steps, warmup, peaks):
    d = wl.add_rms_norm_inputs()
    t, h = d["x"].shape
    nbytes = 8 * t * h + 2 * h
    n = sets_for(nbytes)
    xs = [d["x"].to(dev).clone() for _ in range(n)]
    rs = [d["residual"].to(dev).clone() for _ in range(n)]
    w = d["weight"].to(dev)
    us, _ = time_graph(lambda i: ops.add_rms_norm(xs[i], rs[i], w, d["eps"]), n, 2 * n, steps, warmup, dev)
    y, res = ops.add_rms_norm(xs[0], rs[0], w, d["eps"])
    oracle = _oracle()
    (ey, eres), cpu_us = cpu_run(lambda: oracle.add_rms_norm(d["x"], d["residual"], d["weight"], d["eps"]), 2)
    err = errors(y.cpu(), ey)
    if not torch.equal(res.cpu(), eres):
        err = (float("inf"), float("inf"))  # residual_out is a bit-exact contract
    return op_record("add_rms_norm", us, nbytes, peaks, "hbm", cpu_us, err, shape=f"[{t},{h}] f16")


def case_swiglu(ops, dev, steps, warmup, peaks):
    t, dd = 8192, 14336
    xc = wl.swiglu_inputs(t, dd)["x"]
    x = xc.to(dev)
    nbytes = 6 * t * dd
    us, _ = time_launches(lambda i: ops.swiglu(x), 1, steps, warmup, dev)
    oracle = _oracle()
    want, cpu_us = cpu_run(lambda: oracle.swiglu(xc))
    return op_record("swiglu", us, nbytes, peaks, "hbm", cpu_us, errors(ops.swiglu(x).cpu(), want),
                     shape=f"[{t},{2 * dd}] f16")


def case_rope(ops, dev, steps, warmup, peaks):
    r = wl.rope_inputs()
    t, hq, d = r["q"].shape
    hkv = r["k"].shape[1]
    nbytes = 2 * t * (hq + hkv) * d * 2 + t * d * 2 + 4 * t
    n = sets_for(nbytes)
    qs = [r["q"].to(dev).clone() for _ in range(n)]
    ks = [r["k"].to(dev).clone() for _ in range(n)]
    pos, cos, sin = r["position_ids"].to(dev), r["cos_cache"].to(dev), r["sin_cache"].to(dev)
    us, _ = time_graph(lambda i: ops.rope(qs[i], ks[i], pos, cos, sin), n, 2 * n, steps, warmup, dev)
    oq, ok = ops.rope(qs[0], ks[0], pos, cos, sin)
    oracle = _oracle()
    (eq, ek), cpu_us = cpu_run(lambda: oracle.rope(r["q"], r["k"], r["position_ids"], r["cos_cache"],
                                                   r["sin_cache"]), 2)
    e1, e2 = errors(oq.cpu(), eq), errors(ok.cpu(), ek)
    return op_record("rope", us, nbytes, peaks, "hbm", cpu_us, (max(e1[0], e2[0]), max(e1[1], e2[1])),
                     shape=f"q[{t},{hq},{d}] k[{t},{hkv},{d}] f16")


def case_reshape_and_cache(ops, dev, steps, warmup, peaks, layout=wl.KV_LAYOUT_NHD, tokens=2048):
    c = wl.reshape_and_cache_inputs(tokens=tokens, layout=layout)
    t, hkv, d = c["key"].shape
    nbytes = 2 * (t * hkv * d * 2) * 2 + 4 * t
    n = 16 if tokens <= 4096 else 3
    g = torch.Generator().manual_seed(77)
    keys = [c["key"].to(dev).clone() for _ in range(n)]
    vals = [c["value"].to(dev).clone() for _ in range(n)]
    total_slots = c["cache_shape"][0] * (c["cache_shape"][1] if layout == wl.KV_LAYOUT_NHD else c["cache_shape"][2])
    slots = [torch.randperm(total_slots, generator=g)[:t].int().to(dev) for _ in range(n)]
    kc = torch.zeros(c["cache_shape"], dtype=torch.float16, device=dev)
    vc = torch.zeros(c["cache_shape"], dtype=torch.float16, device=dev)
    us, _ = time_graph(lambda i: ops.reshape_and_cache(keys[i], vals[i], kc, vc, slots[i]), n, 2 * n,
                       steps, warmup, dev)
    name = "reshape_and_cache" + ("" if layout == wl.KV_LAYOUT_NHD else "_nz") + (
        "" if tokens == 2048 else f"_{tokens}tok")
    cpu_us, err = None, None
    if tokens == 2048:  # the benchmark size: bit-exact against the oracle on fresh caches
        kc.zero_()
        vc.zero_()
        ops.reshape_and_cache(keys[0], vals[0], kc, vc, c["slot_indices"].to(dev))
        oracle = _oracle()
        ekc = torch.zeros(c["cache_shape"], dtype=torch.float16)
        evc = torch.zeros(c["cache_shape"], dtype=torch.float16)
        _, cpu_us = cpu_run(lambda: oracle.reshape_and_cache(c["key"], ekc, c["slot_indices"], c["value"], evc))
        same = torch.equal(kc.cpu(), ekc) and torch.equal(vc.cpu(), evc)
        err = (0.0, 0.0) if same else (float("inf"), float("inf"))
    return op_record(name, us, nbytes, peaks, "hbm", cpu_us, err,
                     shape=f"{t} tokens -> cache {list(c['cache_shape'])} f16")


def case_paged_attention(ops, dev, steps, warmup, peaks, layout=wl.KV_LAYOUT_NHD):
    a = wl.paged_attention_inputs(layout=layout)
    nbytes = wl.paged_attention_bytes(a["context_lens"], 4, 128, 28, 128)
    q, kc, vc = a["q"].to(dev), a["key_cache"].to(dev), a["value_cache"].to(dev)
    bt, cl = a["block_tables"].to(dev), a["context_lens"].to(dev)
    us, _ = time_launches(lambda i: ops.paged_attention(q, kc, vc, bt, cl), 1, steps, warmup, dev)
    nz = layout == wl.KV_LAYOUT_NZ
    oracle = _oracle()
    want, cpu_us = cpu_run(lambda: oracle.paged_attention(a["q"], a["key_cache"], a["value_cache"],
                                                          a["block_tables"], a["context_lens"]))
    return op_record("paged_attention_nz" if nz else "paged_attention", us, nbytes, peaks, "hbm", cpu_us,
                     errors(ops.paged_attention(q, kc, vc, bt, cl).cpu(), want),
                     shape="B=64 28q/4kv D=128 L~U[512,8192] page 128" + (", cache [blocks, 32, 128, 16]" if nz else ""),
                     sum_context=int(a["context_lens"].sum()))


def case_grouped_matmul(ops, dev, steps, warmup, peaks, which="gate_up"):
    k, n = (4096, 28672) if which == "gate_up" else (14336, 4096)
    w = wl.grouped_matmul_inputs(rows=8192, k=k, n=n, seed=4 if which == "gate_up" else 5)
    x, ws, gl = w["x"].to(dev), w["w_storage"].to(dev), w["group_list"].to(dev)
    wv = ws.transpose(1, 2)
    flops = 2 * 8192 * k * n
    us, _ = time_launches(lambda i: ops.grouped_matmul(x, wv, gl), 1, steps, warmup, dev)
    # CPU oracle on every 4th row of every group (the full product is about ten seconds of host
    # time per shape); its time is scaled by 4 and the errors are those of the sampled rows.
    y = ops.grouped_matmul(x, wv, gl)
    ends = w["group_list"].tolist()
    rows, sample_ends, lo = [], [], 0
    for e in ends:
        rows.extend(range(lo, e, 4))
        sample_ends.append(len(rows))
        lo = e
    idx = torch.tensor(rows, dtype=torch.long)
    oracle = _oracle()
    want, cpu_us = cpu_run(lambda: oracle.grouped_matmul(w["x"][idx], w["w_storage"].transpose(1, 2),
                                                         torch.tensor(sample_ends, dtype=torch.int64)))
    rec = op_record(f"grouped_matmul_{which}", us, flops, peaks, "tensor", cpu_us * 4,
                    errors(y[idx.to(dev)].cpu(), want), cpu_sample="every 4th row of each group, time x4",
                    shape=f"8 experts, 8192 rows, {k}->{n} f16",
                    group_rows=torch.diff(w["group_list"], prepend=torch.zeros(1, dtype=torch.int64)).tolist())
    rec["frac_of_sustained"] = round(rec["achieved"] / peaks.get("bf16_tflops_sustained", rec["peak"]), 4)
    return rec


def case_dense_projection(ops, dev, steps, warmup, peaks, rows=256, k=4096, n=6144):
    """The QKV projection of the layer's decode batch as the layer calls it (a one-group
    grouped_matmul): weights stream from HBM once, so the bound is HBM."""
    nbytes = 2 * (n * k + rows * k + rows * n)
    sets = sets_for(nbytes)
    g = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn(rows, k, generator=g, device=dev, dtype=torch.float16)
    ws = [(0.02 * torch.randn(1, n, k, generator=g, device=dev, dtype=torch.float16)).transpose(1, 2)
          for _ in range(sets)]
    gl = torch.tensor([rows], dtype=torch.int64, device=dev)
    us, _ = time_graph(lambda i: ops.grouped_matmul(x, ws[i], gl), sets, 2 * sets, steps, warmup, dev)
    oracle = _oracle()
    xc, wc = x.cpu(), ws[0].cpu()
    want, cpu_us = cpu_run(lambda: oracle.grouped_matmul(xc, wc, gl.cpu()), 2)
    return op_record("dense_projection_qkv", us, nbytes, peaks, "hbm", cpu_us,
                     errors(ops.grouped_matmul(x, ws[0], gl).cpu(), want), shape=f"[{rows},{k}] x [{k},{n}] f16")


# --------------------------------------------------------------------------- the layer step
LAYER_WORKLOAD = ("MoE decoder layer, decode step: batch 256, hidden 4096, 32q/8kv heads, D 128, "
                  "positions U[1024,16384], block 128, 8 experts top-2, intermediate 14336")


EXCHANGE = "peer"  # "peer": NVLink peer-memory pushes (moe_parallel.PeerExchange); "nccl": collectives


def make_exchange(group, dev, segment_rows, hidden, hidden_out, num_slots, max_rows=None):
    """The expert-parallel exchange object for this run (None = NCCL collectives or 1 GPU)."""
    if group is None or EXCHANGE != "peer":
        return None
    import ascend910a_extras.moe as moe
    import moe_parallel

    return moe_parallel.PeerExchange(moe, group, dev, segment_rows, hidden, hidden_out, num_slots, max_rows)


def balanced_sequence_shard(positions, world, rank):
    """Which sequences of the batch this rank serves.  Attention time is proportional to a
    rank's total context, and every rank waits for the slowest at the expert exchange, so the
    sequences are dealt out longest-first in snake order (0..G-1, G-1..0, ...): equal counts and
    nearly equal total context per rank.  A contiguous split of this batch leaves up to 15 %
    imbalance."""
    order = torch.argsort(positions, descending=True).tolist()
    mine = []
    for i, seq in enumerate(order):
        lap, k = divmod(i, world)
        if (k if lap % 2 == 0 else world - 1 - k) == rank:
            mine.append(seq)
    return torch.tensor(sorted(mine), dtype=torch.long)


def build_layer(ops, dev, rank, world, group):
    """This rank's share of the layer: all dense weights, its experts, its sequences and
    their KV pages (filled with N(0,1) on the device)."""
    import moe_decode_layer as mdl
    import moe_parallel

    cfg = mdl.LayerConfig()
    mine = moe_parallel.local_experts(cfg.experts, world, rank).tolist()
    weights = mdl.make_weights(cfg, seed=7, experts=mine, device=dev)
    per = 256 // world
    # a rank can receive at most every routed row of the batch: the bound the GEMMs are sized by
    exchange = make_exchange(group, dev, per * cfg.top_k, cfg.hidden, cfg.hidden, cfg.experts,
                             max_rows=256 * cfg.top_k)
    layer = mdl.MoEDecodeLayer(cfg, weights, dev, ops, group, segment_rows=per * cfg.top_k, exchange=exchange)
    pos = mdl.draw_positions(256)
    mine_seq = balanced_sequence_shard(pos, world, rank)
    batch = mdl.make_decode_batch(cfg, positions=pos[mine_seq], seed=80 + rank)
    g = torch.Generator(device=dev).manual_seed(90 + rank)
    k_cache = torch.randn(batch["cache_shape"], generator=g, device=dev, dtype=torch.float16)
    v_cache = torch.randn(batch["cache_shape"], generator=g, device=dev, dtype=torch.float16)
    return cfg, layer, batch, k_cache, v_cache, int(pos.long().sum()) + 256


def gather_check(ok, max_err, rows, group, dev):
    """Combine the ranks' value checks: all must pass; the largest error and the row total."""
    t = torch.tensor([0.0 if ok else 1.0, max_err, float(rows)], device=dev, dtype=torch.float64)
    if group is not None:
        worst = t[:2].clone()
        torch.distributed.all_reduce(worst, op=torch.distributed.ReduceOp.MAX, group=group)
        total = t[2:].clone()
        torch.distributed.all_reduce(total, op=torch.distributed.ReduceOp.SUM, group=group)
        t = torch.cat([worst, total])
    return {"ok": bool(t[0] == 0), "max_abs_err": float(f"{float(t[1]):.3g}"), "rows": int(t[2])}


def check_layer_against_single_gpu(ops, dev, layer, inp, k_cache, v_cache, y_ep, res_ep, group):
    """Value check of the expert-parallel step that was just timed: the same layer with ALL
    experts on this GPU and no exchange (the single-GPU path) runs this rank's sequences, and its
    output must match the exchanged result (residual bit for bit; y within the operators'
    tolerance, since the GEMM kernels chosen for the local row counts differ)."""
    import moe_decode_layer as mdl

    cfg = layer.cfg
    w_all = mdl.make_weights(cfg, seed=7, device=dev)
    solo = mdl.MoEDecodeLayer(cfg, w_all, dev, ops, group=None)
    solo.local_only = True
    y, res = solo.forward(inp["x"], inp["residual"], inp["positions"], inp["slots"], inp["block_tables"],
                          inp["context_lens"], k_cache, v_cache)
    torch.cuda.synchronize(dev)
    d = (y.float() - y_ep.float()).abs()
    ok = bool(torch.equal(res, res_ep)) and bool((d <= 2e-3 + 1e-2 * y.float().abs()).all())
    out = gather_check(ok, float(d.max()), y.shape[0], group, dev)
    del solo, w_all
    torch.cuda.empty_cache()
    return out


def run_layer(ops, dev, rank, world, group, steps, warmup, peaks):
    import moe_decode_layer as mdl

    cfg, layer, batch, k_cache, v_cache, total_context = build_layer(ops, dev, rank, world, group)
    names = ("x", "residual", "positions", "slots", "block_tables", "context_lens")
    host = {n: batch[n].pin_memory() for n in names}
    devt = {n: batch[n].to(dev) for n in names}
    h2d = sum(host[n].numel() * host[n].element_size() for n in names)

    def step(inp, events=None):
        return layer.forward(inp["x"], inp["residual"], inp["positions"], inp["slots"],
                             inp["block_tables"], inp["context_lens"], k_cache, v_cache,
                             attention_events=events)

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            torch.distributed.barrier(group)
            torch.cuda.synchronize(dev)

    def max_over_ranks(ms):
        t = torch.tensor([ms], device=dev)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group)
        return float(t)

    # ---- eager launches with events around the attention operator (roofline of the dominant
    #      kernel, measured inside the step) ----
    for _ in range(warmup):
        step(devt)
    sync_all()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(steps):
        step(devt, ev[i])
    t1.record()
    sync_all()
    eager_us = max_over_ranks(t0.elapsed_time(t1)) * 1e3 / steps
    attn_us = statistics.mean(a.elapsed_time(b) for a, b in ev) * 1e3

    # ---- the step as the library runs it in production: recorded once in a CUDA graph ----
    captured = mdl.CapturedDecodeStep(layer, batch, k_cache, v_cache, warmup=warmup)
    for _ in range(warmup):
        captured.run()
    sync_all()
    t0.record()
    for _ in range(steps):
        captured.run()
    t1.record()
    sync_all()
    layer_us = max_over_ranks(t0.elapsed_time(t1)) * 1e3 / steps

    # ---- end to end: host buffers in, result out, copies inside the timed region ----
    # The library's host-to-host step: inputs sit in pinned host memory, every step copies
    # them up, runs the layer and copies both results down (residual_out as soon as it is final).
    hosted = mdl.CapturedDecodeStep(layer, batch, k_cache, v_cache, warmup=warmup, host_io=True)
    for n in names:
        hosted.host_in[n].copy_(host[n])
    d2h = hosted.host_y.numel() * 2 + hosted.host_res.numel() * 2

    for _ in range(warmup):
        hosted.run_host()
    sync_all()
    t0.record()
    for _ in range(steps):
        hosted.run_host()
    t1.record()
    sync_all()
    e2e_us = max_over_ranks(t0.elapsed_time(t1)) * 1e3 / steps
    y_dev, res_dev = captured.run()
    torch.cuda.synchronize(dev)
    if not (torch.equal(hosted.host_y, y_dev.cpu()) and torch.equal(hosted.host_res, res_dev.cpu())):
        raise RuntimeError("host-to-host step and device-resident step disagree")
    ep_check = None
    if world > 1:
        sync_all()
        if layer.exchange is not None and layer.exchange.barrier_error() != 0:
            raise RuntimeError(f"a peer announcement timed out: {layer.exchange.barrier_error()}")
        ep_check = check_layer_against_single_gpu(ops, dev, layer, devt, k_cache, v_cache, y_dev, res_dev, group)

    local_ctx = int(batch["context_lens"].long().sum())
    attn_bytes = wl.paged_attention_bytes(batch["context_lens"], cfg.kv_heads, cfg.head_dim, cfg.heads,
                                          cfg.block_size)
    gbs = attn_bytes / attn_us / 1e3
    return {
        "layer_us": layer_us, "eager_us": eager_us, "e2e_us": e2e_us, "h2d": h2d, "d2h": d2h,
        "attention": {"us": attn_us, "bytes": attn_bytes, "gbs": gbs, "local_context": local_ctx},
        "launches": 3 * steps * (layer.KERNEL_LAUNCHES if world == 1 else layer.KERNEL_LAUNCHES_EP),
        "total_context": total_context, "ep_check": ep_check,
    }


# --------------------------------------------------------------------------- expert-parallel MoE MLP
def run_moe_mlp(ops, dev, rank, world, group, steps, warmup, peaks):
    """The grouped-GEMM benchmark config as a whole MoE MLP: 4096 tokens, top-2 of 8 experts with
    softmax(N(0,1)) routing skew (8192 routed rows), gate_up [4096 -> 2*14336], swiglu, down
    [14336 -> 4096].  Tokens are sharded over ranks.  Experts are placed by load: every rank has
    ceil(E/G) + 2 slots, hot experts are replicated into the spare slots and their rows spread
    over the replicas (moe_parallel.balanced_placement), because with one expert per GPU the
    busiest expert (47 % of the rows here) would bound the step.  Rows travel through bounded
    sub-segments (twice the expected rows per source and slot) into a bounded row buffer (1.25
    times a rank's expected rows); an overflow is detected on the device and the measurement
    repeated at full capacity.  Reports whole-job TFLOP/s of the two GEMMs (everything else in
    the step is overhead counted against them).  At more than one GPU the result of a sample
    of every rank's tokens is checked against the single-GPU path with all experts local."""
    import ascend910a_extras.moe as moe
    import moe_decode_layer as mdl
    import moe_parallel

    cfg = mdl.LayerConfig()
    tokens, top_k = 4096, 2
    _, ids_flat = wl.moe_group_list(rows=tokens * top_k, experts=cfg.experts, seed=4)
    ids = ids_flat.view(tokens, top_k).int()
    load = torch.bincount(ids_flat, minlength=cfg.experts).tolist()
    per = tokens // world
    spr = -(-cfg.experts // world) + (2 if world > 1 else 0)
    placement = moe_parallel.balanced_placement(load, world, spr).to(dev)
    my_ids = ids[rank * per:(rank + 1) * per].contiguous().to(dev)
    g = torch.Generator(device=dev).manual_seed(40 + rank)
    x = torch.randn(per, cfg.hidden, generator=g, device=dev, dtype=torch.float16)
    wts = torch.full((per, top_k), 0.5, device=dev)
    w = mdl.make_weights(cfg, seed=7, experts=placement.local_slot_experts(rank), device=dev)
    w_gu, w_dn = w["w_gate_up"].transpose(1, 2), w["w_down"].transpose(1, 2)
    full_cap = per * top_k
    up = lambda v, m: -(-int(v) // m) * m
    slot_rows = [load[e] / int(placement.num_replicas[e]) for e in placement.slot_expert.tolist()]
    rank_rows = [sum(slot_rows[r * spr:(r + 1) * spr]) for r in range(world)]
    if world > 1 and EXCHANGE == "peer":  # rows of one (source, slot) sub-segment; rows of the grouped buffer
        cap = min(full_cap, up(2 * max(slot_rows) / world, 64))
        max_rows = up(1.25 * max(rank_rows), 128)
    elif world > 1:  # NCCL form: one segment per peer, twice the balanced share
        cap, max_rows = min(full_cap, up(2 * full_cap / world, 64)), None
    else:
        cap, max_rows = full_cap, None

    def local_mlp(rows, gl):
        return ops.grouped_matmul(moe.grouped_matmul_swiglu(rows, w_gu, gl), w_dn, gl)

    def local_mlp_scatter(rows, gl, scatter):
        moe.grouped_matmul_scatter(moe.grouped_matmul_swiglu(rows, w_gu, gl), w_dn, gl, *scatter)

    def make_step(capacity, rows_bound, flags):
        exchange = make_exchange(group, dev, capacity, cfg.hidden, cfg.hidden, placement.num_slots, rows_bound)

        def step():
            if exchange is not None:
                return exchange.mlp(x, my_ids, wts, local_mlp, overflow_out=flags,
                                    local_mlp_scatter=local_mlp_scatter, placement=placement,
                                    token_offset=rank * per, num_experts=cfg.experts)
            slot_ids = moe_parallel.to_slot_ids(my_ids, placement, rank * per)
            return moe_parallel.expert_parallel_mlp_device(moe, x, slot_ids, wts, placement.num_slots, local_mlp,
                                                           group, capacity, overflow_out=flags)

        return step, exchange

    if steps == 0:  # for a per-kernel timeline: hand back the eager step at the bounded capacity
        return make_step(cap, max_rows, [])[0]

    def measure(capacity, rows_bound):
        flags = []
        step, exchange = make_step(capacity, rows_bound, flags)

        # Recorded once into a CUDA graph (fixed shapes, no host sync, NCCL included), like the
        # layer step: at 8 GPUs the step is shorter than the host time to launch it op by op.
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                step()
        side.synchronize()
        del flags[:]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            y_graph = step()
        torch.cuda.current_stream(dev).wait_stream(side)
        for _ in range(warmup):
            graph.replay()
        torch.cuda.synchronize(dev)
        if world > 1:
            torch.distributed.barrier(group)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            graph.replay()
        t1.record()
        torch.cuda.synchronize(dev)
        dropped = float(flags[-1].sum().item()) if flags else 0.0
        t = torch.tensor([t0.elapsed_time(t1), dropped], device=dev)
        if world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group)
        if exchange is not None and exchange.barrier_error() != 0:
            raise RuntimeError(f"a peer announcement timed out: {exchange.barrier_error()}")
        return float(t[0]) * 1e3 / steps, int(t[1]), y_graph

    us, dropped, y_ep = measure(cap, max_rows)
    used_cap, used_rows = cap, max_rows
    if dropped > 0:
        us, dropped, y_ep = measure(full_cap, None)
        used_cap, used_rows = full_cap, None
    ep_check = None
    if world > 1:  # the first 64 tokens of every rank through the single-GPU path, all experts local
        n = min(64, per)
        w_all = mdl.make_weights(cfg, seed=7, device=dev)
        a_gu, a_dn = w_all["w_gate_up"].transpose(1, 2), w_all["w_down"].transpose(1, 2)
        want = moe_parallel.expert_parallel_mlp_device(
            moe, x[:n].contiguous(), my_ids[:n].contiguous(), wts[:n].contiguous(), cfg.experts,
            lambda rows, gl: ops.grouped_matmul(moe.grouped_matmul_swiglu(rows, a_gu, gl), a_dn, gl), local=True)
        torch.cuda.synchronize(dev)
        d = (want.float() - y_ep[:n].float()).abs()
        ok = bool((d <= 2e-3 + 1e-2 * want.float().abs()).all()) and bool(want.float().abs().max() > 0)
        ep_check = gather_check(ok, float(d.max()), n, group, dev)
        del w_all, a_gu, a_dn
        torch.cuda.empty_cache()
    err = None
    if world == 1:  # the first 32 tokens through the CPU oracle's operators, expert by expert
        oracle = _oracle()
        n = 32
        xc, idc, wc = x[:n].cpu(), my_ids[:n].cpu().long(), wts[:n].cpu()
        want, terms = torch.zeros(n, cfg.hidden), torch.zeros(n, cfg.hidden)
        for e in idc.unique().tolist():
            tok, kth = (idc == e).nonzero(as_tuple=True)
            gl = torch.tensor([tok.numel()], dtype=torch.int64)
            i = w["experts"].index(e)  # the (only) slot that holds this expert
            act = oracle.swiglu(oracle.grouped_matmul(xc[tok], w["w_gate_up"][i:i + 1].cpu().transpose(1, 2), gl))
            dn = oracle.grouped_matmul(act, w["w_down"][i:i + 1].cpu().transpose(1, 2), gl)
            want.index_add_(0, tok, dn.float() * wc[tok, kth].float()[:, None])
            terms.index_add_(0, tok, dn.float().abs() * wc[tok, kth].float()[:, None])
        # y is a sum of two experts' rows, each the end of two chained GEMMs with an fp16
        # intermediate: about 3 % of the intermediate's elements round the other way on the two
        # machines (fp32 sums in a different order), which moves an output by 2e-4 rms and up to
        # 1e-3 among 131 072 outputs, whatever its size; hence twice the operators' atol.
        err = errors(y_ep[:n].cpu(), want.half(), magnitude=terms, atol=2 * ATOL)
    flops = 2 * tokens * top_k * cfg.hidden * 3 * cfg.intermediate
    rec = op_record("moe_mlp_expert_parallel", us, flops, {"bf16_tflops": peaks["bf16_tflops"] * world}, "tensor",
                    err=err, launches=5 if (world == 1 or EXCHANGE == "peer") else 8,
                    shape="4096 tokens top-2 of 8 experts, 4096->2x14336->4096 f16", rows_per_expert=load,
                    slots_per_rank=spr, replicas_per_expert=placement.num_replicas.tolist(),
                    balance=round(moe_parallel.placement_balance(load, placement, world), 3),
                    one_expert_per_slot_balance=round(sum(load) / (cfg.experts * max(load)), 3),
                    segment_rows=used_cap, row_bound=used_rows, dropped_rows=dropped,
                    includes="slot choice, dispatch, SwiGLU (in the gate/up GEMM's epilogue) and (for >1 GPU) gather/combine")
    rec["ep_check"] = ep_check
    return rec


# --------------------------------------------------------------------------- CPU baseline
def cpu_layer_sample(seqs=32, repeats=1, warmup=0, budget_s=None):
    """The CPU oracle's layer on a bounded sample: the first `seqs` of the 256 sequences with
    the full weights.  `warmup` untimed passes, then `repeats` timed ones; with `budget_s` both
    stop early once that many seconds have gone (a slow host), and the passes done are returned.
    Returns (microseconds scaled to 256 sequences, seconds per pass, sequences[, passes, warm-ups])."""
    import moe_decode_layer as mdl
    from oracle import decode_ops_oracle as oracle

    torch.set_num_threads(len(os.sched_getaffinity(0)))
    cfg = mdl.LayerConfig()
    w = mdl.make_weights(cfg, seed=7)
    seqs = max(1, min(seqs, 256))
    pos = mdl.draw_positions(256)[:seqs]
    batch = mdl.make_decode_batch(cfg, positions=pos, seed=80)
    block = torch.randn(64, *batch["cache_shape"][1:], generator=torch.Generator().manual_seed(1)).half()
    reps = -(-batch["cache_shape"][0] // 64)
    k_cache = block.repeat(reps, 1, 1, 1)[: batch["cache_shape"][0]].contiguous()
    v_cache = k_cache.flip(0).contiguous()
    cos, sin = oracle.cos_sin_cache(16385, cfg.head_dim, cfg.rope_theta)
    def one_pass():
        t0 = time.perf_counter()
        oracle.moe_decode_layer(w, batch, k_cache, v_cache, heads=cfg.heads, kv_heads=cfg.kv_heads,
                                head_dim=cfg.head_dim, experts=cfg.experts, top_k=cfg.top_k, eps=cfg.eps,
                                cos_cache=cos, sin_cache=sin)
        return time.perf_counter() - t0

    start = time.perf_counter()
    warmed = 0
    for _ in range(warmup):
        if budget_s is not None and warmed >= 1 and time.perf_counter() - start > budget_s / 4:
            break
        one_pass()
        warmed += 1
    times = []
    for _ in range(repeats):
        if budget_s is not None and times and time.perf_counter() - start > budget_s:
            break
        times.append(one_pass())
    if budget_s is None:
        dt = statistics.median(times)
        return dt * 1e6 * (256 / seqs), dt, seqs
    dt = sum(times) / len(times)  # the timed passes back to back, as the GPU arm's steps are
    return dt * 1e6 * (256 / seqs), dt, seqs, len(times), warmed


def cpu_sample_text(seqs, dt):
    if seqs >= 256:
        return f"the whole step (all 256 sequences, all weights), one pass of {dt:.2f} s; KV cache values tiled from 64 random pages"
    return (f"first {seqs} of 256 sequences with all weights; {dt:.2f} s per pass, scaled x{256 / seqs:g} to the "
            "full batch (an over-estimate: the weight-bound part does not shrink with the sample)")


# --------------------------------------------------------------------------- profiling cases
def profile_case(name, ops, dev):
    """A small, self-ending run of one operator for `ncu` captures: inputs larger than L2 but
    at most a few hundred MB, one warm-up launch and three profiled-size launches."""
    if name in ("paged_attention", "paged_attention_full", "paged_attention_layer_shard"):
        if name == "paged_attention_full":
            a = wl.paged_attention_inputs()
        elif name == "paged_attention_layer_shard":  # one rank's share of the layer batch at 8 GPUs
            a = wl.paged_attention_inputs(bs=32, heads=32, kv_heads=8, min_len=1025, max_len=16385,
                                          blocks=32 * 129, seed=8)
        else:
            a = wl.paged_attention_inputs(bs=16, blocks=16 * 64, seed=3)
        args = [a[n].to(dev) for n in ("q", "key_cache", "value_cache", "block_tables", "context_lens")]
        fn = lambda: ops.paged_attention(*args)
        info = {"bytes": wl.paged_attention_bytes(a["context_lens"], a["kv_heads"], 128, a["q"].shape[1], 128)}
    elif name == "grouped_matmul":
        w = wl.grouped_matmul_inputs(rows=2048, k=4096, n=4096, seed=4)
        x, ws, gl = w["x"].to(dev), w["w_storage"].to(dev).transpose(1, 2), w["group_list"].to(dev)
        fn = lambda: ops.grouped_matmul(x, ws, gl)
        info = {"flops": 2 * 2048 * 4096 * 4096}
    elif name == "grouped_matmul_pairs":  # 4096 rows: the CTA-pair kernel
        w = wl.grouped_matmul_inputs(rows=4096, k=4096, n=4096, seed=4)
        x, ws, gl = w["x"].to(dev), w["w_storage"].to(dev).transpose(1, 2), w["group_list"].to(dev)
        fn = lambda: ops.grouped_matmul(x, ws, gl)
        info = {"flops": 2 * 4096 * 4096 * 4096}
    elif name == "grouped_matmul_swiglu":  # gate/up projection with SwiGLU epilogue, CTA pairs
        import ascend910a_extras.moe as moe

        w = wl.grouped_matmul_inputs(rows=4096, k=4096, n=4096, seed=4)
        x, ws, gl = w["x"].to(dev), w["w_storage"].to(dev).transpose(1, 2), w["group_list"].to(dev)
        fn = lambda: moe.grouped_matmul_swiglu(x, ws, gl)
        info = {"flops": 2 * 4096 * 4096 * 4096}
    elif name == "grouped_matmul_balanced":  # one rank's down projection of the 4096-token MoE MLP at 8 GPUs
        counts = [350, 340, 410]
        g = torch.Generator(device=dev).manual_seed(4)
        x = torch.randn(1408, 14336, generator=g, device=dev, dtype=torch.float16)  # rows past 1100 belong to no group
        ws = (0.02 * torch.randn(3, 4096, 14336, generator=g, device=dev, dtype=torch.float16)).transpose(1, 2)
        gl = torch.tensor(counts, device=dev).cumsum(0).to(torch.int64)
        fn = lambda: ops.grouped_matmul(x, ws, gl)
        info = {"flops": 2 * sum(counts) * 14336 * 4096, "tiles": 160}
    elif name == "grouped_matmul_decode":  # the layer's expert gate/up projection: 8 experts x 64 rows, SwiGLU epilogue
        import ascend910a_extras.moe as moe

        counts = [64] * 8
        g = torch.Generator(device=dev).manual_seed(4)
        x = torch.randn(512, 4096, generator=g, device=dev, dtype=torch.float16)
        ws = (0.02 * torch.randn(8, 28672, 4096, generator=g, device=dev, dtype=torch.float16)).transpose(1, 2)
        gl = torch.tensor(counts, device=dev).cumsum(0).to(torch.int64)
        fn = lambda: moe.grouped_matmul_swiglu(x, ws, gl)
        info = {"bytes": 2 * (8 * 28672 * 4096 + 512 * 4096 + 512 * 14336), "tiles": 896}
    elif name == "moe_exchange":  # the three exchange launches with one rank (its own peer): latency only
        import ascend910a_extras.moe as moe

        t, h, e, k, cap = 256, 4096, 8, 2, 512
        g = torch.Generator(device=dev).manual_seed(4)
        x = torch.randn(t, h, generator=g, device=dev, dtype=torch.float16)
        wr = 0.02 * torch.randn(e, h, generator=g, device=dev, dtype=torch.float16)
        z = lambda *shape, dt=torch.int32: torch.zeros(*shape, dtype=dt, device=dev)
        recv, ret = z(e * cap, h, dt=torch.float16), z(e * cap, h, dt=torch.float16)
        counts, flags, cursor, state, over = z(1, e), z(1), z(e), z(8), z(2)

        def fn():
            pos, ids, wts = moe.dispatch(x, wr, None, k, None, None, 0, [recv.data_ptr()], [counts.data_ptr()], cursor,
                                         state, over, e, cap, 0)
            grouped, back, gl, total = moe.gather(recv, counts, state, over, cap, t * k)
            moe.push_rows(grouped, back, 1, total, t * k, [ret.data_ptr()], e * cap, 0)
            return moe.combine(ret, pos, wts, [flags.data_ptr()], flags, state, 0)
        info = {"tokens": t, "rows": t * k}
    elif name == "dense_projection":  # QKV projection of a 256-row decode batch: cluster split-K
        g = torch.Generator().manual_seed(4)
        x = torch.randn(256, 4096, generator=g).half().to(dev)
        ws = (torch.randn(1, 6144, 4096, generator=g) * 0.02).half().to(dev).transpose(1, 2)
        gl = torch.tensor([256], dtype=torch.int64, device=dev)
        fn = lambda: ops.grouped_matmul(x, ws, gl)
        info = {"bytes": 2 * (6144 * 4096 + 256 * 4096 + 256 * 6144)}
    elif name == "add_rms_norm":
        d = wl.add_rms_norm_inputs()
        x, r, wt = d["x"].to(dev), d["residual"].to(dev), d["weight"].to(dev)
        fn = lambda: ops.add_rms_norm(x, r, wt, d["eps"])
        info = {"bytes": 8 * 4096 * 4096 + 2 * 4096}
    elif name == "swiglu":
        x = wl.swiglu_inputs(2048, 14336)["x"].to(dev)
        fn = lambda: ops.swiglu(x)
        info = {"bytes": 6 * 2048 * 14336}
    elif name == "rope":
        r = wl.rope_inputs()
        args = [r[n].to(dev) for n in ("q", "k", "position_ids", "cos_cache", "sin_cache")]
        fn = lambda: ops.rope(*args)
        info = {"bytes": 2 * 4096 * 40 * 128 * 2 + 4096 * 128 * 2 + 4 * 4096}
    elif name in ("reshape_and_cache", "reshape_and_cache_nz"):
        layout = wl.KV_LAYOUT_NHD if name == "reshape_and_cache" else wl.KV_LAYOUT_NZ
        c = wl.reshape_and_cache_inputs(blocks=1024, layout=layout)
        kc = torch.zeros(c["cache_shape"], dtype=torch.float16, device=dev)
        vc = torch.zeros(c["cache_shape"], dtype=torch.float16, device=dev)
        args = [c["key"].to(dev), c["value"].to(dev), kc, vc, c["slot_indices"].to(dev)]
        fn = lambda: ops.reshape_and_cache(*args)
        info = {"bytes": 2 * 2 * 2048 * 8 * 128 * 2 + 4 * 2048}
    else:
        raise SystemExit(f"unknown profile case {name}")
    flush = torch.empty(L2_BYTES * 2, dtype=torch.uint8, device=dev)
    for _ in range(4):
        flush.zero_()  # evict the operator's lines so each launch starts from DRAM
        fn()
    torch.cuda.synchronize(dev)
    print(json.dumps({"profile_case": name, **info}))


# --------------------------------------------------------------------------- per-kernel timeline
def timeline(which, ops, dev, rank, world, group):
    """Per-kernel timeline of one step on every rank (torch profiler; the step launched op by op,
    so kernel durations are clean but the gaps are host launch gaps, not the graph's).  Rank r
    writes timeline_<which>_n<N>_r<r>.txt into OUT_DIR: start offset, duration, kernel name."""
    from torch.profiler import ProfilerActivity, profile

    if which == "layer":
        cfg, layer, batch, k_cache, v_cache, _ = build_layer(ops, dev, rank, world, group)
        names = ("x", "residual", "positions", "slots", "block_tables", "context_lens")
        d = {n: batch[n].to(dev) for n in names}
        step = lambda: layer.forward(*(d[n] for n in names), k_cache, v_cache)
    else:
        step = run_moe_mlp(ops, dev, rank, world, group, 0, 3, load_peaks())
    for _ in range(5):
        step()
    torch.cuda.synchronize(dev)
    if world > 1:
        torch.distributed.barrier(group)
    reps = 4
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(reps):
            step()
        torch.cuda.synchronize(dev)
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                 key=lambda e: e.time_range.start)
    last = evs[-(len(evs) // reps):]
    t0 = last[0].time_range.start
    out = OUT_DIR
    out.mkdir(exist_ok=True)
    with open(out / f"timeline_{which}_n{world}_r{rank}.txt", "w") as f:
        f.write(f"# {which} step, {world} GPUs, rank {rank}, exchange {EXCHANGE}, "
                f"B200OPS_PDL={os.environ.get('B200OPS_PDL', '1')}\n")
        for e in last:
            f.write(f"{e.time_range.start - t0:9.1f} +{e.time_range.elapsed_us():8.1f} us  {e.name[:110]}\n")
        f.write(f"step span us: {last[-1].time_range.end - t0:.1f}\n")
    if world > 1:
        torch.distributed.barrier(group)


# --------------------------------------------------------------------------- main
PER_OP_COLS = ["us", "achieved", "frac_of_peak", "cpu_us", "max_abs_err", "err_over_tol"]


def compact(rec):
    """One per-op row of the printed line, in the order of PER_OP_COLS (the full rows go to the
    detail file)."""
    return [rec["us"], rec["achieved"], rec["frac"], rec["cpu_us"], rec["max_abs_err"], rec["err_over_tol"]]


def write_detail(n_gpus, detail):
    """Everything the printed line leaves out (shapes, byte counts, group sizes, placement), as
    bench_detail_n<N>.json in OUT_DIR, if that directory can be written."""
    try:
        out = OUT_DIR
        out.mkdir(exist_ok=True)
        path = out / f"bench_detail_n{n_gpus}.json"
        path.write_text(json.dumps(detail, indent=1))
        return str(path.relative_to(REPO))
    except OSError:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--ops", default="auto",
                    help="per-op cases: comma list, 'all', 'none', or 'auto' (all at 1 GPU, none otherwise)")
    ap.add_argument("--no-layer", action="store_true", help="skip the layer step (per-op cases only)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline of the layer step")
    ap.add_argument("--cpu-seqs", type=int, default=256,
                    help="sequences in the CPU-baseline sample (256 = the whole batch, no extrapolation)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel exchange: NVLink peer-memory pushes, or NCCL collectives")
    ap.add_argument("--profile-case", default=None,
                    help="run a small case of one operator (for ncu) and exit")
    ap.add_argument("--timeline", default=None, choices=["layer", "mlp"],
                    help="write a per-kernel timeline of one step per rank (torch profiler) and exit")
    ns = ap.parse_args()
    global EXCHANGE
    EXCHANGE = ns.exchange
    ns.warmup = max(ns.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    peaks = load_peaks()
    cores = len(os.sched_getaffinity(0))
    base = {
        "metric": "moe_decode_layer_latency", "unit": "us", "n_gpus": ns.gpus, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": LAYER_WORKLOAD, "parallelism": f"ep{ns.gpus}+batch-sharded attention",
                   "exchange": ("none" if ns.gpus == 1 else
                                "NVLink peer pushes, flag waits in the kernels" if ns.exchange == "peer" else
                                "NCCL all-gather + all-to-all"),
                   "execution": "CUDA graph replay (eager_us: op by op)",
                   "l2": "inputs larger than L2 (GBs of KV cache and expert weights per step)"},
    }

    if ns.impl == "reference":
        # The reference's kernels need Ascend hardware and the CANN toolchain; what can run
        # here is the CPU golden path, timed with every host thread on a bounded sample.
        if rank != 0:
            return
        # K timed passes after W untimed ones, as asked; a host so slow that this would run for
        # more than about three minutes stops early and reports the passes it made.
        us, dt, seqs, done, warmed = cpu_layer_sample(ns.cpu_seqs, repeats=max(1, ns.steps), warmup=ns.warmup,
                                                      budget_s=180.0)
        line = dict(base)
        line.update({
            "impl": "reference", "value": round(us, 1), "steps": done, "warmup": warmed,
            "ms_per_step": round(us / 1e3, 3),
            "cpu_baseline": {"value": round(us, 1), "unit": "us", "cores": cores, "kind": "port",
                             "sample": cpu_sample_text(seqs, dt)},
            "e2e": {"value": round(us, 1), "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        })
        print(json.dumps(line))
        return

    import ascend910a_extras.ops as ops

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    if ns.profile_case:
        profile_case(ns.profile_case, ops, dev)
        return
    if ns.timeline:
        timeline(ns.timeline, ops, dev, rank, world, group)
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    layer = None if ns.no_layer else run_layer(ops, dev, rank, world, group, ns.steps, ns.warmup, peaks)
    mlp = None if ns.no_layer else run_moe_mlp(ops, dev, rank, world, group, max(3, ns.steps // 2), ns.warmup, peaks)
    clocks = sampler.stop() if rank == 0 else None
    torch.cuda.empty_cache()

    cases = {
        "add_rms_norm": case_add_rms_norm, "reshape_and_cache": case_reshape_and_cache,
        "reshape_and_cache_nz": lambda *a: case_reshape_and_cache(*a, layout=wl.KV_LAYOUT_NZ),
        # same kernel on a prefill-size batch: shows its streaming rate once the launch is not
        # a single DRAM round trip
        "reshape_and_cache_32768tok": lambda *a: case_reshape_and_cache(*a, tokens=32768),
        "rope": case_rope, "swiglu": case_swiglu, "paged_attention": case_paged_attention,
        # the same batch on the reference's own cache layout
        "paged_attention_nz": lambda *a: case_paged_attention(*a, layout=wl.KV_LAYOUT_NZ),
        "grouped_matmul_gate_up": lambda *a: case_grouped_matmul(*a, which="gate_up"),
        "grouped_matmul_down": lambda *a: case_grouped_matmul(*a, which="down"),
        "dense_projection_qkv": case_dense_projection,
    }
    if ns.ops == "auto":
        want = list(cases) if world == 1 else []
    elif ns.ops == "all":
        want = list(cases)
    else:
        want = [c for c in ns.ops.split(",") if c and c != "none"]
    per_op = [mlp] if mlp is not None else []
    if rank == 0:
        for name in want:
            if name not in cases:
                raise SystemExit(f"--ops: unknown case {name!r}; choose from {', '.join(cases)}")
            per_op.append(cases[name](ops, dev, max(5, ns.steps // 2), ns.warmup, peaks))
            torch.cuda.empty_cache()
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    if rank != 0:
        return

    # Key order: the contract's keys first, the per-op table last (a reader that keeps only the
    # end of a long line still sees every operator's row).
    line = dict(base)
    line.update({"steps": ns.steps, "warmup": ns.warmup, "clocks": clocks})
    launches = sum(r["launches"] * max(5, ns.steps // 2) for r in per_op)
    if layer is not None:
        att = layer["attention"]
        line.update({
            "value": round(layer["layer_us"], 1), "ms_per_step": round(layer["layer_us"] / 1e3, 4),
            "tokens_per_s": round(256 / layer["layer_us"] * 1e6, 1),
            "eager_us": round(layer["eager_us"], 1),
            "e2e": {"value": round(layer["e2e_us"], 1), "unit": "us",
                    "h2d_bytes_per_step": layer["h2d"], "d2h_bytes_per_step": layer["d2h"]},
            "roofline": {"bound": "hbm", "kernel": "paged_attention_fast_kernel inside the step",
                         "achieved": round(att["gbs"], 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(att["gbs"] / peaks["hbm_gbs"], 4),
                         "traffic": int(att["bytes"] * ATTENTION_TRAFFIC_RATIO),
                         "us": round(att["us"], 1), "bytes": att["bytes"], "peak_source": peaks["source"]},
        })
        launches += layer["launches"]
        if not ns.no_cpu:
            us, dt, seqs = cpu_layer_sample(ns.cpu_seqs)
            line["cpu_baseline"] = {"value": round(us, 1), "unit": "us", "cores": cores, "kind": "port",
                                    "sample": cpu_sample_text(seqs, dt)}
        if layer["ep_check"] is not None:
            line["ep_check"] = {"layer": layer["ep_check"], "moe_mlp": mlp["ep_check"] if mlp else None,
                                "against": "single-GPU path, all experts local"}
            if not (layer["ep_check"]["ok"] and (mlp is None or mlp["ep_check"]["ok"])):
                print(json.dumps(line))
                raise SystemExit("expert-parallel result differs from the single-GPU path")
    line["gpu_launches"] = launches
    line["detail_file"] = write_detail(ns.gpus, {"per_op": per_op, "layer": layer})
    line["per_op_cols"] = PER_OP_COLS
    line["per_op"] = {r["op"]: compact(r) for r in per_op}
    print(json.dumps(line))
    wrong = [r["op"] for r in per_op if r["err_over_tol"] is not None and not r["err_over_tol"] <= 1.0]
    if wrong:
        raise SystemExit(f"outside the tolerance against the CPU oracle: {', '.join(wrong)}")


if __name__ == "__main__":
    main()
