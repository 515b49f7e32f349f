"""One MoE decoder layer, decode step, composed from the `ascend910a_extras.ops` operators.

Operator order follows the decoder layer the reference assembles in its graph builder
(csrc/ffi/graph.cpp:145-283: norm+residual -> QKV linear -> split -> rope -> reshape_and_cache
-> paged attention -> output linear -> norm+residual -> MLP), with the dense MLP replaced by
a top-2-of-E routed expert MLP (grouped_matmul gate_up -> swiglu -> grouped_matmul down) and
without Qwen3's per-head q/k norms:

    add_rms_norm -> QKV GEMM -> rope -> reshape_and_cache -> paged_attention -> o_proj
    -> add_rms_norm -> router top-k -> [dispatch] grouped_matmul -> swiglu -> grouped_matmul
    [combine] -> weighted sum

The dense projections run on the same tcgen05 grouped GEMM with a single group (an NT GEMM,
like the reference's legacy `matmul`, _csrc/kernels/matmul.cpp:3-28).  Router top-k, the
token permutation and the weighted sum are the library's MoE glue kernels
(`ascend910a_extras.moe`).  Sequences (and their
KV pages) are sharded over ranks with no collective; only the expert MLP exchanges rows
(moe_parallel.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

import moe_parallel


@dataclass
class LayerConfig:
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 14336
    experts: int = 8
    top_k: int = 2
    rope_theta: float = 1e6
    eps: float = 1e-6
    block_size: int = 128
    qk_norm: bool = False  # per-head RMSNorm of q and k before rope (Qwen3; csrc/ffi/graph.cpp:252-255)


def make_weights(cfg: LayerConfig, seed=7, experts=None, std=0.02, device="cpu"):
    """Random-init fp16 weights ~ N(0, std); norm weights ~ N(1, 0.1).  All matrices are
    stored [out, in] (K contiguous), the layout the grouped GEMM reads.  `experts` selects
    which expert matrices to materialise (all by default; a rank's own under EP).  Each
    expert draws from its own seeded stream, so a rank that holds a subset sees the same
    values as a rank that holds all.  `device` chooses where the numbers are drawn (CPU for
    parity tests, the GPU for full-size benchmark weights)."""
    def gen(s):
        return torch.Generator(device=device).manual_seed(s)

    def mat(n, k, g):
        return (std * torch.randn(n, k, generator=g, device=device)).half()

    g = gen(seed)
    qkv_out = (cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim
    w = {
        "ln1": (1 + 0.1 * torch.randn(cfg.hidden, generator=g, device=device)).half(),
        "ln2": (1 + 0.1 * torch.randn(cfg.hidden, generator=g, device=device)).half(),
        "wqkv": mat(qkv_out, cfg.hidden, g),
        "wo": mat(cfg.hidden, cfg.heads * cfg.head_dim, g),
        "wrouter": mat(cfg.experts, cfg.hidden, g),
    }
    if cfg.qk_norm:
        gn = gen(seed + 500)
        w["q_norm"] = (1 + 0.1 * torch.randn(cfg.head_dim, generator=gn, device=device)).half()
        w["k_norm"] = (1 + 0.1 * torch.randn(cfg.head_dim, generator=gn, device=device)).half()
    keep = list(range(cfg.experts)) if experts is None else [int(e) for e in experts]
    gu = torch.empty(len(keep), 2 * cfg.intermediate, cfg.hidden, dtype=torch.float16, device=device)
    dn = torch.empty(len(keep), cfg.hidden, cfg.intermediate, dtype=torch.float16, device=device)
    for i, e in enumerate(keep):
        ge = gen(seed * 1000 + e)
        gu[i] = mat(2 * cfg.intermediate, cfg.hidden, ge)
        dn[i] = mat(cfg.hidden, cfg.intermediate, ge)
    w["w_gate_up"], w["w_down"], w["experts"] = gu, dn, keep
    return w


def route(logits: torch.Tensor, top_k: int):
    """softmax over experts in fp32, then top-k (weights not renormalised)."""
    p = torch.softmax(logits.float(), dim=-1)
    wts, ids = torch.topk(p, top_k, dim=-1)
    return ids, wts


class MoEDecodeLayer:
    """Device-resident weights + the decode-step forward.  `ops` is ascend910a_extras.ops."""

    def __init__(self, cfg: LayerConfig, weights: dict, device, ops, group=None, segment_rows=None,
                 exchange=None):
        import ascend910a_extras.moe as moe

        self.cfg, self.ops, self.device, self.group, self.moe = cfg, ops, device, group, moe
        self.segment_rows = segment_rows  # rows each rank sends each peer under expert parallelism
        self.exchange = exchange  # a moe_parallel.PeerExchange: NVLink peer-memory dispatch/combine
        self.local_only = False  # True: all experts are here; ignore any process group
        self.fuse_return = True  # down projection stores into the peers' buffers in its epilogue
        self.fuse_rope_cache = True  # False: split + ops.rope + ops.reshape_and_cache separately
        self.fuse_swiglu = True  # False: ops.grouped_matmul then ops.swiglu
        d = lambda t: t.to(device)
        self.ln1, self.ln2 = d(weights["ln1"]), d(weights["ln2"])
        self.q_norm = d(weights["q_norm"]) if cfg.qk_norm else None
        self.k_norm = d(weights["k_norm"]) if cfg.qk_norm else None
        # NT-GEMM weights as single-group stacks [1, N, K]; the op takes the [1, K, N] view.
        self.wqkv = d(weights["wqkv"])[None].transpose(1, 2)
        self.wo = d(weights["wo"])[None].transpose(1, 2)
        self.wrouter = d(weights["wrouter"]).contiguous()
        self.w_gate_up = d(weights["w_gate_up"]).transpose(1, 2)
        self.w_down = d(weights["w_down"]).transpose(1, 2)
        max_pos = 16385
        inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2).float() / cfg.head_dim))
        freqs = torch.einsum("i,j->ij", torch.arange(max_pos, dtype=torch.float), inv_freq)
        self.cos, self.sin = d(freqs.cos().half().contiguous()), d(freqs.sin().half().contiguous())
        self._one_group = {}

    def _dense(self, x, w):
        """x [T, K] @ w^T as a one-group grouped GEMM."""
        t = x.shape[0]
        gl = self._one_group.get(t)
        if gl is None:
            gl = torch.tensor([t], dtype=torch.int64, device=self.device)
            self._one_group[t] = gl
        return self.ops.grouped_matmul(x, w, gl)

    def _gate_up(self, rows, group_list):
        """silu(gate) * up of the routed rows: one kernel, or the reference's two operators."""
        if self.fuse_swiglu:
            return self.moe.grouped_matmul_swiglu(rows, self.w_gate_up, group_list)
        return self.ops.swiglu(self.ops.grouped_matmul(rows, self.w_gate_up, group_list))

    def _local_mlp(self, rows, group_list):
        if rows.shape[0] == 0:
            return rows.new_zeros(0, self.cfg.hidden)
        return self.ops.grouped_matmul(self._gate_up(rows, group_list), self.w_down, group_list)

    def _local_mlp_scatter(self, rows, group_list, scatter):
        """Expert MLP whose down projection stores its rows into the peers' return buffers."""
        self.moe.grouped_matmul_scatter(self._gate_up(rows, group_list), self.w_down, group_list, *scatter)

    def forward(self, x, residual, positions, slots, block_tables, context_lens, k_cache, v_cache,
                return_routing=False, attention_events=None, on_residual=None):
        """`attention_events`, if given, is a pair of CUDA events recorded right before and
        after the attention operator on the current stream (used by the benchmark to time the
        dominant kernel inside the step).  `on_residual(residual_out)` is called as soon as the
        launch that produces the step's second output has been enqueued, well before the expert
        MLP: a caller that ships results to the host can start that copy early."""
        cfg, ops = self.cfg, self.ops
        t = x.shape[0]
        h1, res1 = ops.add_rms_norm(x, residual, self.ln1, cfg.eps)
        qkv = self._dense(h1, self.wqkv)
        nq = cfg.heads * cfg.head_dim
        if self.fuse_rope_cache:
            q = self.moe.fused_qkv_rope_cache(qkv, positions, self.cos, self.sin, slots, k_cache, v_cache,
                                              cfg.heads, cfg.kv_heads, self.q_norm, self.k_norm, cfg.eps)
        else:
            nkv = cfg.kv_heads * cfg.head_dim
            q = qkv[:, :nq].contiguous().view(t, cfg.heads, cfg.head_dim)
            k = qkv[:, nq:nq + nkv].contiguous().view(t, cfg.kv_heads, cfg.head_dim)
            v = qkv[:, nq + nkv:].contiguous().view(t, cfg.kv_heads, cfg.head_dim)
            if cfg.qk_norm:  # the stand-alone operator, one head per row and a zero residual
                zq, zk = torch.zeros_like(q), torch.zeros_like(k)
                q = ops.add_rms_norm(q.view(-1, cfg.head_dim), zq.view(-1, cfg.head_dim), self.q_norm,
                                     cfg.eps)[0].view_as(q)
                k = ops.add_rms_norm(k.view(-1, cfg.head_dim), zk.view(-1, cfg.head_dim), self.k_norm,
                                     cfg.eps)[0].view_as(k)
            q, k = ops.rope(q, k, positions, self.cos, self.sin)
            ops.reshape_and_cache(k, v, k_cache, v_cache, slots)
        if attention_events is not None:
            attention_events[0].record()
        attn = ops.paged_attention(q, k_cache, v_cache, block_tables, context_lens)
        if attention_events is not None:
            attention_events[1].record()
        o = self._dense(attn.view(t, nq), self.wo)
        h2, res2 = ops.add_rms_norm(o, res1, self.ln2, cfg.eps)
        if on_residual is not None:
            on_residual(res2)
        if self.exchange is not None:  # the router runs inside the dispatch launch
            y, ids, wts = self.exchange.mlp(h2, None, None, self._local_mlp,
                                            local_mlp_scatter=self._local_mlp_scatter if self.fuse_return else None,
                                            router_weight=self.wrouter, top_k=cfg.top_k, return_routing=True)
        else:
            ids, wts = self.moe.route_topk(h2, self.wrouter, cfg.top_k)
            y = moe_parallel.expert_parallel_mlp_device(self.moe, h2, ids, wts, cfg.experts, self._local_mlp,
                                                        self.group, self.segment_rows, local=self.local_only)
        if return_routing:
            return y, res2, ids, wts
        return y, res2

    # number of this library's kernels one single-GPU forward launches (for the benchmark's
    # accounting): 2 add_rms_norm, 2 dense GEMMs, fused rope+cache, attention (one kernel: the
    # chunk merge is fused), route, permute, copy_rows, gate/up GEMM with SwiGLU epilogue, down GEMM,
    # finalize.  Under expert parallelism with the peer-memory exchange the MoE part is dispatch
    # (router inside), gather, gate/up GEMM with SwiGLU epilogue, down GEMM with scatter epilogue,
    # combine.
    KERNEL_LAUNCHES = 12
    KERNEL_LAUNCHES_EP = 11


class CapturedDecodeStep:
    """The layer's decode step recorded once into a CUDA graph and replayed.

    Counterpart of the reference's two-phase graph execution (csrc/ffi/adaptor.h:57-89 `Setup`
    then `Execute`; csrc/ffi/graph.cpp `Context.setup` / `Context.run`): set-up fixes shapes,
    allocates every intermediate once and records the launches; a run only refreshes the
    input buffers and replays.  Possible because no step of the layer synchronises with the
    host (routing metadata stays on the device, the expert-parallel exchange has fixed
    shapes).  Under expert parallelism every rank must construct and run it together.
    """

    NAMES = ("x", "residual", "positions", "slots", "block_tables", "context_lens")

    def __init__(self, layer: MoEDecodeLayer, example: dict, k_cache, v_cache, warmup=3, host_io=False):
        self.layer, self.k_cache, self.v_cache = layer, k_cache, v_cache
        dev = layer.device
        self.inputs = {n: example[n].to(dev).clone() for n in self.NAMES}
        # x and residual share one allocation so that a host caller can send both with one copy
        self._act = torch.stack([self.inputs["x"], self.inputs["residual"]])
        self.inputs["x"], self.inputs["residual"] = self._act[0], self._act[1]
        self.stream = torch.cuda.Stream(dev)
        self.stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):  # first-call set-up (function attributes, NCCL channels) happens here
                self._forward()
        self.stream.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.stream):
            self.y, self.res = self._forward()
        torch.cuda.current_stream(dev).wait_stream(self.stream)
        self.graph_host = None
        if host_io:
            self._capture_host_io(example)

    def _forward(self, on_residual=None):
        i = self.inputs
        return self.layer.forward(i["x"], i["residual"], i["positions"], i["slots"], i["block_tables"],
                                  i["context_lens"], self.k_cache, self.v_cache, on_residual=on_residual)

    def _capture_host_io(self, example):
        """A second graph for callers whose inputs and results live in host memory: the step's
        copies are part of the recording.  The two activation tensors go up in one transfer on the
        main stream while the small integer tensors go up on a side stream; `residual_out` starts down on
        the side stream as soon as the launch producing it is enqueued (it is final before the
        expert MLP, which is a quarter of the step), `y` follows at the end."""
        dev = self.layer.device
        self.host_in = {n: example[n].clone().pin_memory() for n in self.NAMES if n not in ("x", "residual")}
        self._act_host = torch.stack([example["x"], example["residual"]]).pin_memory()
        self.host_in["x"], self.host_in["residual"] = self._act_host[0], self._act_host[1]
        self.host_y = torch.empty(self.y.shape, dtype=self.y.dtype).pin_memory()
        self.host_res = torch.empty(self.res.shape, dtype=self.res.dtype).pin_memory()
        self.side = torch.cuda.Stream(dev)
        big = ("x", "residual")

        def record():
            self.side.wait_stream(self.stream)
            with torch.cuda.stream(self.side):
                for n in self.NAMES:
                    if n not in big:
                        self.inputs[n].copy_(self.host_in[n], non_blocking=True)
            self._act.copy_(self._act_host, non_blocking=True)  # x and residual in one transfer
            self.stream.wait_stream(self.side)

            def ship_residual(res):
                self.side.wait_stream(self.stream)
                with torch.cuda.stream(self.side):
                    self.host_res.copy_(res, non_blocking=True)

            y, _ = self._forward(on_residual=ship_residual)
            self.host_y.copy_(y, non_blocking=True)
            self.stream.wait_stream(self.side)

        self.stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(self.stream):
            record()  # once outside capture, so that errors surface eagerly
        self.stream.synchronize()
        self.side.synchronize()
        self.graph_host = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph_host, stream=self.stream):
            record()
        torch.cuda.current_stream(dev).wait_stream(self.stream)

    def run_host(self):
        """Replay the host-to-host step: reads `host_in` (pinned; fill it before the call), leaves
        the results in `host_y` / `host_res` (valid once the current stream has been synchronised)."""
        if self.graph_host is None:
            raise RuntimeError("CapturedDecodeStep was built without host_io=True")
        self.graph_host.replay()
        return self.host_y, self.host_res

    def load(self, batch: dict, non_blocking=True):
        """Copy a step's inputs (host or device tensors) into the graph's input buffers."""
        for n in self.NAMES:
            self.inputs[n].copy_(batch[n], non_blocking=non_blocking)

    def run(self):
        """Replay on the current stream; returns the graph's output tensors (overwritten by the
        next run)."""
        self.graph.replay()
        return self.y, self.res


def draw_positions(batch=256, min_pos=1024, max_pos=16384, seed=8):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(min_pos, max_pos + 1, (batch,), generator=g, dtype=torch.int32)


def make_decode_batch(cfg: LayerConfig, batch=256, min_pos=1024, max_pos=16384, seed=8,
                      spare_blocks=8, positions=None):
    """Decode-step inputs: hidden states ~ N(0,1), positions uniform in [min_pos, max_pos],
    context_len = position + 1, distinct random physical blocks per sequence, the new token's
    slot = its position inside its last block.  The KV cache itself (shape returned) is
    filled on the device by the caller.  `positions` overrides the draw (a rank's share of a
    global batch from draw_positions)."""
    g = torch.Generator().manual_seed(seed)
    if positions is not None:  # a rank's slice of a global batch
        pos = torch.as_tensor(positions, dtype=torch.int32)
        batch = pos.numel()
    x = torch.randn(batch, cfg.hidden, generator=g).half()
    residual = torch.randn(batch, cfg.hidden, generator=g).half()
    if positions is None:
        pos = torch.randint(min_pos, max_pos + 1, (batch,), generator=g, dtype=torch.int32)
    lens = pos + 1
    bs = cfg.block_size
    pages = (lens.long() + bs - 1) // bs
    total = int(pages.sum())
    blocks = total + spare_blocks
    ids = torch.randperm(blocks, generator=g)[:total].int()
    max_pages = int(pages.max())
    table = torch.zeros(batch, max_pages, dtype=torch.int32)
    slots = torch.empty(batch, dtype=torch.int32)
    o = 0
    for b in range(batch):
        n = int(pages[b])
        table[b, :n] = ids[o:o + n]
        o += n
        slots[b] = int(table[b, int(pos[b]) // bs]) * bs + int(pos[b]) % bs
    return {"x": x, "residual": residual, "positions": pos, "context_lens": lens.int(),
            "block_tables": table, "slots": slots, "num_blocks": blocks,
            "cache_shape": (blocks, bs, cfg.kv_heads, cfg.head_dim)}


def layer_floor_bytes(cfg: LayerConfig, context_lens, experts_touched=None):
    """HBM bytes one decode step cannot avoid: the KV of every context token and every
    weight matrix once (activations are negligible)."""
    kv = int(torch.as_tensor(context_lens).long().sum()) * cfg.kv_heads * cfg.head_dim * 2 * 2
    dense = ((cfg.heads + 2 * cfg.kv_heads) * cfg.head_dim * cfg.hidden + cfg.hidden * cfg.heads * cfg.head_dim) * 2
    e = cfg.experts if experts_touched is None else experts_touched
    experts = e * 3 * cfg.intermediate * cfg.hidden * 2
    return kv, dense + experts


def attention_scale(cfg):
    return 1.0 / math.sqrt(cfg.head_dim)
