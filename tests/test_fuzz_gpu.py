"""Seeded random-shape sweeps of the two pipelined operators against the CPU oracle: shapes no
hand-written case names (odd group mixes, tails in every dimension, every kernel-selection
branch the shape rules can reach)."""
import random

import pytest
import torch

import decode_workloads as wl
from oracle import decode_ops_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def close(got, want, rtol=1e-2, atol=1e-3):
    torch.testing.assert_close(got.float(), want.float(), rtol=rtol, atol=atol)


@pytest.mark.parametrize("seed", range(24))
def test_grouped_matmul_random_shapes(cabi, seed):
    rnd = random.Random(1000 + seed)
    experts = rnd.choice([1, 1, 2, 3, 5, 8, 17])
    k = 64 * rnd.choice([1, 2, 3, 8, 17, 64, 130])
    n = 64 * rnd.choice([1, 2, 3, 4, 5, 9, 16, 33])
    kinds = [lambda: 0, lambda: rnd.randint(1, 40), lambda: rnd.randint(100, 300), lambda: 128, lambda: 256,
             lambda: rnd.randint(300, 700)]
    counts = [rnd.choice(kinds)() for _ in range(experts)]
    if sum(counts) == 0:
        counts[-1] = 7
    if k * n * experts > 40_000_000:  # keep the oracle fast
        n = 64 * 3
    slack = rnd.choice([0, 0, 5, 200])  # rows of x beyond the last group
    g = torch.Generator().manual_seed(seed)
    m = sum(counts) + slack
    x = torch.randn(m, k, generator=g).half()
    w_storage = (torch.randn(experts, n, k, generator=g) * (0.5 / k ** 0.5)).half()
    gl = torch.tensor(counts).cumsum(0).to(torch.int64)
    want = oracle.grouped_matmul(x[: sum(counts)], w_storage.transpose(1, 2), gl)
    y = torch.full((m, n), 5.0, dtype=torch.float16, device=DEV)
    nbytes = cabi.grouped_matmul_workspace_size(m, k, experts, n)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
    cabi.grouped_matmul(x.to(DEV), w_storage.to(DEV), gl.to(DEV), y, ws if nbytes else None)
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    y = y.cpu()
    close(y[: sum(counts)], want)
    assert (y[sum(counts):] == 5.0).all()
    if n % 128 == 0:  # the same shape through the SwiGLU epilogue
        act = torch.full((m, n // 2), 5.0, dtype=torch.float16, device=DEV)
        cabi.grouped_matmul_swiglu(x.to(DEV), w_storage.to(DEV), gl.to(DEV), act)
        torch.cuda.synchronize()
        assert cabi.pipeline_status() == 0
        close(act.cpu()[: sum(counts)], oracle.swiglu(want))
        assert (act.cpu()[sum(counts):] == 5.0).all()


@pytest.mark.parametrize("seed", range(16))
def test_paged_attention_random_shapes(cabi, seed):
    rnd = random.Random(2000 + seed)
    head_dim = rnd.choice([128, 128, 128, 64, 256])
    kv_heads = rnd.choice([1, 2, 4, 8])
    group = rnd.choice([1, 2, 4, 7, 8, 16]) if head_dim == 128 else rnd.choice([1, 4])
    page = rnd.choice([16, 64, 128, 256]) if head_dim == 128 else rnd.choice([16, 32])
    layout = rnd.choice([wl.KV_LAYOUT_NHD, wl.KV_LAYOUT_NHD, wl.KV_LAYOUT_NZ])
    bs = rnd.randint(1, 12)
    lens = [rnd.choice([0, 1, page - 1, page, page + 1, rnd.randint(2, 3000), rnd.randint(2, 600)]) for _ in range(bs)]
    lens = [max(l, 0) for l in lens]
    blocks = sum((l + page - 1) // page for l in lens) + 2
    w = wl.paged_attention_inputs(heads=kv_heads * group, kv_heads=kv_heads, head_dim=head_dim, block_size=page,
                                  blocks=blocks, layout=layout, context_lens=lens, seed=seed)
    want = oracle.paged_attention(w["q"], w["key_cache"], w["value_cache"], w["block_tables"], w["context_lens"])
    q = w["q"].to(DEV)
    out = torch.full_like(q, float("nan"))
    nbytes = cabi.paged_attention_workspace_size(bs, q.shape[1], kv_heads, head_dim, page, w["block_tables"].shape[1])
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
    cabi.paged_attention(q, w["key_cache"].to(DEV), w["value_cache"].to(DEV), w["block_tables"].to(DEV),
                         w["context_lens"].to(DEV), out, kv_heads, page, layout, ws if nbytes else None)
    torch.cuda.synchronize()
    assert cabi.pipeline_status() == 0
    close(out.cpu(), want)
