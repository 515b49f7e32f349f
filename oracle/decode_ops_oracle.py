"""CPU oracle for the decode operator set.  TEST INFRASTRUCTURE ONLY.

This file restates, on CPU with torch, the golden formulas the reference checks its
kernels against.  It exists to CHECK the CUDA kernels (tests/, the smoke check, and the
CPU-baseline leg of the benchmark).  The product never imports it and has no CPU path.

Pinning (how each function is tied to the reference), verified by tests/test_oracle.py
against fixtures under tests/golden/ that were produced by running the reference's own
golden code (tests/golden/make_golden.py):
  add_rms_norm       reference golden `add_rms_norm_cpu`   benchmark/test_add_rms_norm.py:6-10
  swiglu             reference golden `swiglu_cpu`         benchmark/test_swiglu.py:6-12
  grouped_matmul     reference golden `grouped_matmul_ref` benchmark/test_grouped_matmul.py:6-23
                     (restated with an fp32 upcast: fp32 accumulation, one rounding)
  rope               reference golden `fn_naive`           benchmark/test_graph.py:347-367
                     (restated in fp32 with one rounding; the reference evaluates it in fp16)
  reshape_and_cache  reference golden `reference_reshape_and_cache`
                                                           benchmark/test_reshape_and_cache.py:6-25
                     plus the kernel's skip rule for invalid slots
                     csrc/opdev/op_kernel/reshape_and_cache_ex.cpp:50; the [pages, P, Hkv, D]
                     layout is the same scatter with the standard index formula
  paged_attention    PARITY UNPINNED.  The reference has no golden for it: its kernel is
                     unfinished (csrc/opdev/op_kernel/paged_attention_ex.cpp:137-152) and its
                     only check calls a third-party library, torch_npu._npu_paged_attention
                     (torch-npu 2.5.1.post1.dev20250619, benchmark/test_graph.py:545-555),
                     whose source is not part of the reference.  What is restated here is the
                     published definition of decode attention, with the reference's GQA head
                     mapping (paged_attention_ex.cpp:91-95) and scale 1/sqrt(head_dim)
                     (csrc/opdev/op_host/paged_attention_ex.cpp:26).
"""
from __future__ import annotations

import math

import torch

KV_LAYOUT_NZ = 0
KV_LAYOUT_NHD = 1


def add_rms_norm(x, residual, weight, epsilon):
    """benchmark/test_add_rms_norm.py:6-10.  fp16 add, fp32 mean of squares, one rounding."""
    y = x + residual
    rms = torch.sqrt((y.float() ** 2).mean(-1, keepdim=True) + epsilon)
    out = y / rms * weight
    return out.to(x.dtype), y.to(x.dtype)


def head_rms_norm(x, weight, epsilon):
    """RMSNorm over the last dimension without a residual: the per-head q / k normalisation the
    reference's graph builder inserts before rope (csrc/ffi/graph.cpp:252-255), with the
    arithmetic of `add_rms_norm` above (fp32 mean of squares, one rounding)."""
    rms = torch.sqrt((x.float() ** 2).mean(-1, keepdim=True) + epsilon)
    return (x / rms * weight).to(x.dtype)


def swiglu(x):
    """benchmark/test_swiglu.py:6-12 (`swiglu_cpu`): silu(first half) * second half in fp32."""
    x1, x2 = x.chunk(2, -1)
    x1_f32, x2_f32 = x1.to(torch.float32), x2.to(torch.float32)
    out = (x1_f32 * x1_f32.sigmoid()) * x2_f32
    return out.to(x.dtype)


def grouped_matmul(x, weight, group_list):
    """benchmark/test_grouped_matmul.py:6-23 with fp32 accumulation.

    `weight` is the torch-level view [E, K, N]; group_list holds inclusive cumulative row
    ends; rows outside every group are left as zeros here (the kernel does not write them).
    Empty groups are skipped (csrc/opdev/op_kernel/grouped_mat_mul_ex.cpp:40).
    """
    num_experts = weight.shape[0]
    out = torch.zeros(x.shape[0], weight.shape[2], dtype=x.dtype)
    assert group_list.shape[0] == num_experts
    gl = group_list.tolist()
    for ei in range(num_experts):
        start = 0 if ei == 0 else gl[ei - 1]
        end = gl[ei]
        if end - start <= 0:
            continue
        out[start:end, :] = torch.matmul(x[start:end, :].float(), weight[ei].float()).to(x.dtype)
    return out


def rope(q, k, position_ids, cos_cache, sin_cache):
    """benchmark/test_graph.py:347-367 (`fn_naive`), evaluated in fp32 and rounded once."""
    pos = position_ids.long()
    cos = cos_cache[pos].float()[:, None, :]
    sin = sin_cache[pos].float()[:, None, :]

    def rot(t):
        x, y = t.float().chunk(2, -1)
        return torch.cat([x * cos - y * sin, y * cos + x * sin], dim=-1).to(t.dtype)

    return rot(q), rot(k)


def cos_sin_cache(max_pos, rotary_dim, theta=1000000.0, dtype=torch.float16):
    """cos/sin tables as the reference's test builds them (benchmark/test_graph.py:299-317)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2).float() / rotary_dim))
    t = torch.arange(max_pos, dtype=torch.float)
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    return freqs.cos().to(dtype).contiguous(), freqs.sin().to(dtype).contiguous()


def reshape_and_cache(key, key_cache, slot_indices, value=None, value_cache=None, layout=None):
    """In-place scatter; vectorised form of benchmark/test_reshape_and_cache.py:6-25.

    NZ  cache [pages, C, P, 16]:  cache[s//P, c, s%P, j] = flat(key[t])[c*16+j]
    NHD cache [pages, P, Hkv, D]: cache[s//P, s%P, h, d] = key[t, h, d]
    Slots outside [0, pages*P) are skipped (reshape_and_cache_ex.cpp:50).  Values are only
    written when both value and value_cache are given (reshape_and_cache_ex.cpp:24-25).
    """
    if layout is None:
        layout = KV_LAYOUT_NHD if tuple(key_cache.shape[2:]) == tuple(key.shape[1:]) else KV_LAYOUT_NZ
    num_tokens = key.shape[0]
    row = key.shape[1] * key.shape[2]
    slots = slot_indices.long()
    if layout == KV_LAYOUT_NHD:
        pages, page_size = key_cache.shape[0], key_cache.shape[1]
    else:
        pages, chunks, page_size, sixteen = key_cache.shape
        assert sixteen == 16
    ok = (slots >= 0) & (slots < pages * page_size)
    toks = torch.nonzero(ok).flatten()
    s = slots[toks]
    page, off = s // page_size, s % page_size

    def scatter(src, cache):
        flat = src.reshape(num_tokens, row)[toks]
        if layout == KV_LAYOUT_NHD:
            cache.view(pages, page_size, row)[page, off] = flat
        else:
            n = min(chunks * 16, row)
            full, rem = n // 16, n % 16
            if full:
                cache[page, :full, off, :] = flat[:, : full * 16].reshape(-1, full, 16)
            if rem:
                cache[page, full, off, :rem] = flat[:, full * 16 : n]

    scatter(key, key_cache)
    if value is not None and value_cache is not None:
        scatter(value, value_cache)


def _gather_kv(cache, pages, head, num_kv_heads, head_dim, layout):
    """All tokens of the listed pages for one kv head, as [len(pages)*P, D] fp32."""
    if layout == KV_LAYOUT_NHD:
        return cache[pages, :, head, :].reshape(-1, head_dim).float()
    c0 = head * head_dim // 16
    blk = cache[pages, c0 : c0 + head_dim // 16]  # [n, D/16, P, 16]
    return blk.permute(0, 2, 1, 3).reshape(-1, head_dim).float()


def paged_attention(q, key_cache, value_cache, block_tables, context_lens, layout=None):
    """Decode attention over a paged KV cache, fp32 math, fp16 result.  See module docstring."""
    bs, num_heads, head_dim = q.shape
    if layout is None:
        layout = KV_LAYOUT_NHD if key_cache.shape[3] == head_dim else KV_LAYOUT_NZ
    if layout == KV_LAYOUT_NHD:
        page_size, num_kv_heads = key_cache.shape[1], key_cache.shape[2]
    else:
        num_kv_heads, page_size = key_cache.shape[1] * 16 // head_dim, key_cache.shape[2]
    group = num_heads // num_kv_heads
    scale = 1.0 / math.sqrt(head_dim)
    out = torch.zeros_like(q)
    cap = block_tables.shape[1] * page_size
    for b in range(bs):
        L = min(int(context_lens[b]), cap)
        if L <= 0:
            continue
        pages = block_tables[b, : (L + page_size - 1) // page_size].long()
        for h in range(num_kv_heads):
            k = _gather_kv(key_cache, pages, h, num_kv_heads, head_dim, layout)[:L]
            v = _gather_kv(value_cache, pages, h, num_kv_heads, head_dim, layout)[:L]
            qh = q[b, h * group : (h + 1) * group].float()
            p = torch.softmax(qh @ k.T * scale, dim=-1)
            out[b, h * group : (h + 1) * group] = (p @ v).to(q.dtype)
    return out


def moe_decode_layer(w, batch, k_cache, v_cache, *, heads, kv_heads, head_dim, experts, top_k, eps,
                     cos_cache, sin_cache, expert_ids=None, expert_weights=None):
    """One MoE decoder layer (decode step) from the operator goldens above, in the operator
    order of the reference's decoder layer (csrc/ffi/graph.cpp:145-283) with a routed expert
    MLP in place of the dense one.  Dense projections use fp32 accumulation and one rounding,
    like grouped_matmul.  `w` holds [out, in] matrices: wqkv, wo, wrouter, w_gate_up [E, 2I, H],
    w_down [E, H, I], and the two norm weights.  The caches are updated in place.
    If `expert_ids`/`expert_weights` are given they replace the oracle's own routing (used to
    compare outputs when a near-tie in the router flips between fp16 implementations).
    Returns (y, residual_out, ids, weights, stages) where `stages` keeps intermediates.
    """
    x, residual = batch["x"], batch["residual"]
    t = x.shape[0]
    lin = lambda a, m: (a.float() @ m.float().T).to(a.dtype)
    h1, res1 = add_rms_norm(x, residual, w["ln1"], eps)
    qkv = lin(h1, w["wqkv"])
    nq, nkv = heads * head_dim, kv_heads * head_dim
    q = qkv[:, :nq].reshape(t, heads, head_dim)
    k = qkv[:, nq:nq + nkv].reshape(t, kv_heads, head_dim)
    v = qkv[:, nq + nkv:].reshape(t, kv_heads, head_dim)
    if "q_norm" in w:  # Qwen3-style per-head normalisation of q and k
        q = head_rms_norm(q, w["q_norm"], eps)
        k = head_rms_norm(k, w["k_norm"], eps)
    q, k = rope(q, k, batch["positions"], cos_cache, sin_cache)
    reshape_and_cache(k, k_cache, batch["slots"], v, v_cache)
    attn = paged_attention(q, k_cache, v_cache, batch["block_tables"], batch["context_lens"])
    o = lin(attn.reshape(t, nq), w["wo"])
    h2, res2 = add_rms_norm(o, res1, w["ln2"], eps)
    logits = lin(h2, w["wrouter"])
    p = torch.softmax(logits.float(), dim=-1)
    own_w, own_ids = torch.topk(p, top_k, dim=-1)
    ids = own_ids if expert_ids is None else expert_ids
    wts = own_w if expert_weights is None else expert_weights
    flat = ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=experts)
    tokens = order // top_k
    rows = h2[tokens]
    gl = counts.cumsum(0).to(torch.int64)
    gu = grouped_matmul(rows, w["w_gate_up"].transpose(1, 2), gl)
    act = swiglu(gu)
    dn = grouped_matmul(act, w["w_down"].transpose(1, 2), gl)
    y = torch.zeros(t, dn.shape[1], dtype=torch.float32)
    y.index_add_(0, tokens, dn.float() * wts.reshape(-1)[order].float()[:, None])
    stages = {"h1": h1, "qkv": qkv, "q_rot": q, "k_rot": k, "attn": attn, "o": o, "h2": h2,
              "logits": logits, "own_ids": own_ids, "own_weights": own_w}
    return y.to(x.dtype), res2, ids, wts, stages
