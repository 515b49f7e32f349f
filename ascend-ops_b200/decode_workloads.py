"""Seeded synthetic inputs for the decode operator benchmarks and parity tests.

The reference measures on no dataset (its scripts draw random tensors,
benchmark/test_*.py), so every workload here is synthetic with the shapes, dtypes and value
distributions of the benchmark configurations.  Tensors are created on CPU from a seeded
generator, so the CPU oracle and the GPU kernels see identical bits.
`scale` < 1 shrinks the token/sequence counts for quick checks; 1.0 is the full size.
"""
from __future__ import annotations

import math

import torch

KV_LAYOUT_NZ = 0
KV_LAYOUT_NHD = 1


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def add_rms_norm_inputs(tokens=4096, hidden=4096, seed=1):
    """x, residual ~ N(0,1); weight ~ N(1, 0.1); eps 1e-6."""
    g = _gen(seed)
    return {
        "x": torch.randn(tokens, hidden, generator=g).half(),
        "residual": torch.randn(tokens, hidden, generator=g).half(),
        "weight": (1 + 0.1 * torch.randn(hidden, generator=g)).half(),
        "eps": 1e-6,
    }


def reshape_and_cache_inputs(tokens=2048, kv_heads=8, head_dim=128, blocks=4096, block_size=128,
                             layout=KV_LAYOUT_NHD, seed=2):
    """K/V rows ~ N(0,1) and distinct random slots in [0, blocks*block_size)."""
    g = _gen(seed)
    key = torch.randn(tokens, kv_heads, head_dim, generator=g).half()
    value = torch.randn(tokens, kv_heads, head_dim, generator=g).half()
    slots = torch.randperm(blocks * block_size, generator=g)[:tokens].int()
    if layout == KV_LAYOUT_NHD:
        shape = (blocks, block_size, kv_heads, head_dim)
    else:
        shape = (blocks, kv_heads * head_dim // 16, block_size, 16)
    return {"key": key, "value": value, "slot_indices": slots, "cache_shape": shape, "layout": layout}


def paged_attention_inputs(bs=64, heads=28, kv_heads=4, head_dim=128, min_len=512, max_len=8192,
                           block_size=128, blocks=8192, layout=KV_LAYOUT_NHD, seed=3,
                           context_lens=None):
    """GQA decode batch: lengths uniform in [min_len, max_len], distinct random physical blocks."""
    g = _gen(seed)
    if context_lens is None:
        context_lens = torch.randint(min_len, max_len + 1, (bs,), generator=g, dtype=torch.int32)
    else:
        context_lens = torch.as_tensor(context_lens, dtype=torch.int32)
        bs = context_lens.numel()
    pages = (context_lens.long() + block_size - 1) // block_size
    total = int(pages.sum())
    assert total <= blocks, f"cache of {blocks} blocks too small for {total} pages"
    max_pages = max(int(pages.max()), 1)
    ids = torch.randperm(blocks, generator=g)[:total].int()
    table = torch.zeros(bs, max_pages, dtype=torch.int32)
    o = 0
    for b in range(bs):
        n = int(pages[b])
        table[b, :n] = ids[o:o + n]
        o += n
    if layout == KV_LAYOUT_NHD:
        shape = (blocks, block_size, kv_heads, head_dim)
    else:
        shape = (blocks, kv_heads * head_dim // 16, block_size, 16)
    k_cache = torch.randn(shape, generator=g).half()
    v_cache = torch.randn(shape, generator=g).half()
    q = torch.randn(bs, heads, head_dim, generator=g).half()
    return {"q": q, "key_cache": k_cache, "value_cache": v_cache, "block_tables": table,
            "context_lens": context_lens, "layout": layout, "kv_heads": kv_heads,
            "block_size": block_size}


def paged_attention_bytes(context_lens, kv_heads, head_dim, heads, block_size):
    """Algorithmic HBM bytes of one decode-attention call: K and V of every context token
    once, q and o once, the block-table entries and the lengths."""
    lens = torch.as_tensor(context_lens).long()
    bs = lens.numel()
    kv = int(lens.sum()) * kv_heads * head_dim * 2 * 2
    qo = 2 * bs * heads * head_dim * 2
    tables = 4 * int(((lens + block_size - 1) // block_size).sum()) + 4 * bs
    return kv + qo + tables


def moe_group_list(rows=8192, experts=8, seed=4):
    """Rows per expert: multinomial with softmax(N(0,1)) expert probabilities; returns the
    inclusive cumulative ends (int64) the grouped GEMM takes, and the per-row expert ids."""
    g = _gen(seed)
    p = torch.softmax(torch.randn(experts, generator=g), 0)
    ids = torch.multinomial(p, rows, replacement=True, generator=g)
    counts = torch.bincount(ids, minlength=experts)
    return counts.cumsum(0).to(torch.int64), ids


def grouped_matmul_inputs(rows=8192, k=4096, n=28672, experts=8, seed=4, w_std=0.02):
    """x ~ N(0,1) [rows, k]; w ~ N(0, w_std) stored [E, n, k] (the op takes its transpose view)."""
    g = _gen(seed + 1000)
    gl, ids = moe_group_list(rows, experts, seed)
    x = torch.randn(rows, k, generator=g).half()
    w_storage = torch.empty(experts, n, k, dtype=torch.float16)
    for e in range(experts):  # chunked to bound the fp32 temporary
        w_storage[e] = (w_std * torch.randn(n, k, generator=g)).half()
    return {"x": x, "w_storage": w_storage, "group_list": gl, "expert_ids": ids}


def rope_inputs(tokens=4096, heads=32, kv_heads=8, head_dim=128, min_pos=1024, max_pos=16384,
                theta=1e6, seed=5):
    g = _gen(seed)
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    freqs = torch.einsum("i,j->ij", torch.arange(max_pos + 1, dtype=torch.float), inv_freq)
    return {
        "q": torch.randn(tokens, heads, head_dim, generator=g).half(),
        "k": torch.randn(tokens, kv_heads, head_dim, generator=g).half(),
        "position_ids": torch.randint(min_pos, max_pos + 1, (tokens,), generator=g, dtype=torch.int32),
        "cos_cache": freqs.cos().half().contiguous(),
        "sin_cache": freqs.sin().half().contiguous(),
    }


def swiglu_inputs(tokens=8192, d=14336, seed=6):
    g = _gen(seed)
    return {"x": torch.randn(tokens, 2 * d, generator=g).half()}


def attention_scale(head_dim):
    return 1.0 / math.sqrt(head_dim)
