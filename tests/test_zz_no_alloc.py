"""The allocation-free decode-attention entry point, b200ops_paged_attention_static.

It serves hosts that cannot get device memory at call time (all HBM already handed to the
host's own arena, or cudaMalloc banned on the request path), so its split-context scratch
is an array inside the library.  The check: through the C ABI, its output must equal what
the workspace-taking entry point produces on the same inputs, on two calls in a row.  The
second call uses shorter contexts than the first, so the shared array still holds the first
call's records when the second runs; a correct kernel never reads them.
"""
import ctypes

import pytest
import torch

import decode_workloads as wl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _both_entry_points(cabi, w):
    q = w["q"].to(DEV)
    kc, vc = w["key_cache"].to(DEV), w["value_cache"].to(DEV)
    bt, cl = w["block_tables"].to(DEV), w["context_lens"].to(DEV)
    n = cabi.paged_attention_workspace_size(q.shape[0], q.shape[1], w["kv_heads"], q.shape[2],
                                            w["block_size"], bt.shape[1])
    assert n > 0, "the case must need scratch, otherwise it proves nothing"
    ws = torch.empty(n, dtype=torch.uint8, device=DEV)
    want = torch.full_like(q, float("nan"))
    got = torch.full_like(q, float("nan"))
    cabi.paged_attention(q, kc, vc, bt, cl, want, w["kv_heads"], w["block_size"], w["layout"], ws)
    cabi.paged_attention_static(q, kc, vc, bt, cl, got, w["kv_heads"], w["block_size"], w["layout"])
    torch.cuda.synchronize()
    return got.cpu(), want.cpu()


def test_static_scratch_entry_matches_workspace_entry_twice(cabi):
    first = wl.paged_attention_inputs(bs=6, blocks=6 * 64, min_len=4000, max_len=8192, seed=71)
    second = wl.paged_attention_inputs(bs=6, blocks=6 * 64, context_lens=[300, 2500, 1, 8192, 0, 2049],
                                       seed=72)
    for w in (first, second):
        got, want = _both_entry_points(cabi, w)
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-3)
    assert cabi.pipeline_status() == 0


def test_static_scratch_entry_allocates_nothing(cabi):
    """What the name promises: once the warm-up call has made the runtime load the library's
    device code (its documented first call), further calls leave the device's free memory
    exactly where it was -- including memory torch's allocator holds, which is read with it."""
    w = wl.paged_attention_inputs(bs=6, blocks=6 * 64, min_len=4000, max_len=8192, seed=73)
    q = w["q"].to(DEV)
    kc, vc = w["key_cache"].to(DEV), w["value_cache"].to(DEV)
    bt, cl = w["block_tables"].to(DEV), w["context_lens"].to(DEV)
    out = torch.empty_like(q)
    call = lambda: cabi.paged_attention_static(q, kc, vc, bt, cl, out, w["kv_heads"], w["block_size"], w["layout"])
    call()  # warm-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    assert torch.isfinite(out.float()).all()


def test_static_scratch_entry_rejects_shapes_beyond_its_array(cabi):
    lib = cabi.load()
    null = ctypes.c_void_p(None)
    # 4096 sequences x 64 heads x 4 chunks of partial records is far more than the array holds
    rc = lib.b200ops_paged_attention_static(null, null, null, null, null, null, 4096, 64, 8, 128,
                                            1 << 20, 128, 64, cabi.KV_LAYOUT_NHD, null)
    assert rc == cabi.EWORKSPACE
    assert "built-in array" in cabi.last_error()
