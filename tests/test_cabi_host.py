"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol the
header declares, and rejects bad arguments before touching CUDA; the torch extension
mirrors the reference FFI's argument checks."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (REPO / "include" / "b200ops.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200ops_\w+)\s*\(", text)))


def test_header_declares_the_six_operators():
    names = declared_symbols()
    for op in ("add_rms_norm", "swiglu", "rope", "reshape_and_cache", "paged_attention", "grouped_matmul"):
        assert f"b200ops_{op}" in names


def test_library_exports_every_declared_symbol(cabi):
    lib = cabi.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/b200ops.h but not exported"
    assert sorted(cabi.SIGNATURES) == declared_symbols()
    assert lib.b200ops_version() >= 100
    assert cabi.last_error() is not None


def test_argument_checks_run_before_any_cuda_call(cabi):
    lib = cabi.load()
    null = ctypes.c_void_p(None)
    one = ctypes.c_void_p(16)  # never dereferenced: every call below fails validation first
    assert lib.b200ops_add_rms_norm(one, one, one, 1e-6, one, one, 4, 100, null) == cabi.EINVAL
    assert "multiple of 64" in cabi.last_error()
    assert lib.b200ops_add_rms_norm(null, one, one, 1e-6, one, one, 4, 128, null) == cabi.EINVAL
    assert lib.b200ops_swiglu(one, one, 4, 32, null) == cabi.EINVAL
    assert lib.b200ops_swiglu(one, one, 4, 96, null) == cabi.EINVAL
    assert lib.b200ops_rope(one, one, one, one, one, one, one, 2, 4, 1, 24, 16, null) == cabi.EINVAL
    dims = (ctypes.c_int64 * 4)(4, 8, 2, 31)
    assert lib.b200ops_reshape_and_cache(one, one, one, one, one, 2, 2, 32, dims, cabi.KV_LAYOUT_NHD,
                                         null) == cabi.EINVAL
    dims = (ctypes.c_int64 * 4)(4, 4, 8, 8)
    assert lib.b200ops_reshape_and_cache(one, one, one, one, one, 2, 2, 32, dims, cabi.KV_LAYOUT_NZ,
                                         null) == cabi.EINVAL
    assert lib.b200ops_grouped_matmul(one, one, one, one, 8, 100, 2, 64, null, 0, null) == cabi.EINVAL
    assert lib.b200ops_grouped_matmul(one, one, one, one, 8, 64, 2, 96, null, 0, null) == cabi.EINVAL
    assert lib.b200ops_paged_attention(one, one, one, one, one, one, 2, 6, 4, 128, 8, 16, 4,
                                       cabi.KV_LAYOUT_NHD, null, 0, null) == cabi.EINVAL
    assert "multiple of num_kv_heads" in cabi.last_error()
    assert lib.b200ops_paged_attention(one, one, one, one, one, one, 2, 8, 4, 48, 8, 16, 4,
                                       cabi.KV_LAYOUT_NHD, null, 0, null) == cabi.EINVAL
    assert lib.b200ops_matmul(one, one, one, 4, 0, 64, null) == cabi.EINVAL
    assert lib.b200ops_matmul(null, one, one, 4, 64, 64, null) == cabi.EINVAL
    assert lib.b200ops_matmul(null, null, null, 0, 64, 64, null) == cabi.OK
    # the fused expert-parallel launches: geometry is checked before anything is dereferenced
    peers = (ctypes.c_void_p * 2)(256, 512)
    assert lib.b200ops_moe_dispatch(one, None, one, None, None, None, None, 0, 0, one, peers, peers, one, one,
                                    None, 4, 64, 8, 2, 7, 2, 16, 0, null) == cabi.EINVAL  # 7 slots over 2 ranks
    assert "geometry" in cabi.last_error()
    assert lib.b200ops_moe_dispatch(one, None, None, None, None, None, None, 0, 0, one, peers, peers, one, one,
                                    None, 4, 64, 8, 2, 8, 2, 16, 0, null) == cabi.EINVAL  # neither router nor ids
    assert lib.b200ops_moe_gather(one, one, one, None, one, one, one, one, 60, 2, 4, 16, 128, null) == cabi.EINVAL
    assert lib.b200ops_moe_combine(one, one, one, one, peers, one, one, 4, 2, 64, 2, 2, null) == cabi.EINVAL
    # zero-size problems succeed without a device
    assert lib.b200ops_swiglu(null, null, 0, 64, null) == cabi.OK
    assert lib.b200ops_add_rms_norm(null, null, null, 1e-6, null, null, 0, 64, null) == cabi.OK


def test_workspace_queries(cabi):
    lib = cabi.load()
    assert lib.b200ops_grouped_matmul_workspace_size(8192, 4096, 8, 28672) == 0  # plenty of tiles
    assert lib.b200ops_grouped_matmul_workspace_size(64, 14336, 1, 4096) > 0  # few tiles: split-K
    assert lib.b200ops_grouped_matmul_workspace_size(1100, 14336, 3, 4096) > 0  # a ragged second wave
    assert lib.b200ops_grouped_matmul_workspace_size(256, 512, 1, 6144) == 0  # k too short to cut
    assert lib.b200ops_paged_attention_workspace_size(4, 8, 2, 128, 128, 2) == 0  # one chunk per sequence
    small = lib.b200ops_paged_attention_workspace_size(4, 8, 2, 128, 128, 16)
    n = lib.b200ops_paged_attention_workspace_size(64, 28, 4, 128, 128, 64)
    assert 0 < small < n
    # grows with the batch, covers the chunk partials of the split-context path
    assert n >= 64 * 28 * 4 * 130 * 4
    assert lib.b200ops_paged_attention_workspace_size(128, 28, 4, 128, 128, 64) > n
    assert lib.b200ops_paged_attention_workspace_size(0, 28, 4, 128, 128, 64) == 0


def test_torch_extension_mirrors_reference_checks(ops):
    h = torch.float16
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.swiglu(torch.zeros(4, 64, dtype=h))
    with pytest.raises(RuntimeError, match="must be 2D"):
        ops.swiglu(torch.zeros(4, 4, 64, dtype=h))
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops.swiglu(torch.zeros(4, 96, dtype=h))
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops.add_rms_norm(torch.zeros(2, 96, dtype=h), torch.zeros(2, 96, dtype=h), torch.zeros(96, dtype=h))
    with pytest.raises(RuntimeError, match="same shape"):
        ops.add_rms_norm(torch.zeros(2, 64, dtype=h), torch.zeros(3, 64, dtype=h), torch.zeros(64, dtype=h))
    with pytest.raises(RuntimeError, match="K-major"):
        ops.grouped_matmul(torch.zeros(8, 64, dtype=h), torch.zeros(2, 64, 64, dtype=h),
                           torch.zeros(2, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="same batch size"):
        ops.rope(torch.zeros(2, 4, 64, dtype=h), torch.zeros(2, 1, 64, dtype=h),
                 torch.zeros(3, dtype=torch.int32), torch.zeros(8, 32, dtype=h), torch.zeros(8, 32, dtype=h))
    with pytest.raises(RuntimeError, match="key must be 3D"):
        ops.reshape_and_cache(torch.zeros(2, 64, dtype=h), None, torch.zeros(2, 2, 2, 16, dtype=h), None,
                              torch.zeros(2, dtype=torch.int32))


def test_ops_module_keeps_the_reference_signatures(ops):
    import inspect
    expect = {
        "rope": ["q", "k", "position_ids", "cos_cache", "sin_cache"],
        "swiglu": ["x"],
        "grouped_matmul": ["x", "w", "group_list"],
        "add_rms_norm": ["x", "residual", "weight", "epsilon"],
        "reshape_and_cache": ["key", "value", "key_cache", "value_cache", "slot_indices"],
        "paged_attention": ["q", "key_cache", "value_cache", "block_tables", "context_lens"],
        "print_info": [],
    }
    for name, params in expect.items():
        assert list(inspect.signature(getattr(ops, name)).parameters) == params
    assert inspect.signature(ops.add_rms_norm).parameters["epsilon"].default == 1e-5


def test_matmul_of_the_earlier_interface_is_exposed(ops):
    """ops.matmul(x, w) and the dispatcher registration of the reference's earlier interface
    (TORCH_LIBRARY(ascend910a, ...), _csrc/ffi.cpp:473-482), with its argument checks (:409-414)."""
    import inspect
    assert list(inspect.signature(ops.matmul).parameters) == ["x", "w"]
    for name in ("swiglu", "grouped_matmul", "matmul"):
        assert hasattr(torch.ops.ascend910a, name)
    h = torch.float16
    with pytest.raises(RuntimeError, match="must be 2D"):
        ops.matmul(torch.zeros(4, 4, 64, dtype=h), torch.zeros(8, 64, dtype=h))
    with pytest.raises(RuntimeError, match="last dimension of x must match"):
        ops.matmul(torch.zeros(4, 64, dtype=h), torch.zeros(8, 32, dtype=h))
    with pytest.raises(RuntimeError, match="only float16"):
        ops.matmul(torch.zeros(4, 64), torch.zeros(8, 64))
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.matmul(torch.zeros(4, 64, dtype=h), torch.zeros(8, 64, dtype=h))


def test_tuning_variables_are_read_once_and_can_be_reloaded(cabi, monkeypatch):
    """Launch-time knobs come from the environment at first use only; reload_options() is the
    hook that makes a changed variable visible (what conftest.knob calls)."""
    lib = cabi.load()
    monkeypatch.setenv("B200OPS_PA_CHUNK_TOKENS", "4096")
    cabi.reload_options()
    big = lib.b200ops_paged_attention_workspace_size(64, 28, 4, 128, 128, 64)
    monkeypatch.setenv("B200OPS_PA_CHUNK_TOKENS", "256")
    unchanged = lib.b200ops_paged_attention_workspace_size(64, 28, 4, 128, 128, 64)
    assert unchanged == big  # not re-read
    cabi.reload_options()
    small_chunks = lib.b200ops_paged_attention_workspace_size(64, 28, 4, 128, 128, 64)
    assert small_chunks > big  # shorter chunks, more partial records
