"""ctypes binding of the C ABI in include/b200ops.h (libb200ops.so).

This is the binding a non-torch host (a C++ graph runner, a Go/Rust service through cgo/FFI)
would write; here it lets tests and benchmarks call the library exactly as such a host
does: raw device pointers, sizes and a stream handle, an int status back.  Nothing in this
file computes, and nothing falls back anywhere if the library is missing.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "lib", "libb200ops.so")

KV_LAYOUT_NZ = 0
KV_LAYOUT_NHD = 1

OK = 0
EINVAL = -1
ECUDA = -2
EWORKSPACE = -3
EUNSUPPORTED = -4

# name -> (restype, argtypes); one entry per declaration in include/b200ops.h
SIGNATURES = {
    "b200ops_version": (c_int, []),
    "b200ops_last_error": (c_char_p, []),
    "b200ops_print_info": (c_int, [c_int, c_void_p, c_size_t]),
    "b200ops_add_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                     c_int64, c_int64, c_void_p]),
    "b200ops_swiglu": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "b200ops_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "b200ops_reshape_and_cache": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int64, c_int64, c_int64, ctypes.POINTER(c_int64),
                                          c_int, c_void_p]),
    "b200ops_paged_attention_workspace_size": (c_size_t, [c_int64] * 6),
    "b200ops_paged_attention": (c_int, [c_void_p] * 6 + [c_int64] * 7 + [c_int, c_void_p,
                                                                         c_size_t, c_void_p]),
    "b200ops_paged_attention_static": (c_int, [c_void_p] * 6 + [c_int64] * 7 + [c_int, c_void_p]),
    "b200ops_grouped_matmul_workspace_size": (c_size_t, [c_int64] * 4),
    "b200ops_grouped_matmul": (c_int, [c_void_p] * 4 + [c_int64] * 4 + [c_void_p, c_size_t,
                                                                        c_void_p]),
    "b200ops_grouped_matmul_swiglu": (c_int, [c_void_p] * 4 + [c_int64] * 4 + [c_void_p, c_size_t, c_void_p]),
    "b200ops_fused_qkv_rope_cache": (c_int, [c_void_p] * 8 + [c_int64] * 5 + [ctypes.POINTER(c_int64), c_int,
                                                                              c_void_p]),
    "b200ops_fused_qkv_norm_rope_cache": (c_int, [c_void_p] * 3 + [c_float] + [c_void_p] * 7 + [c_int64] * 5 +
                                          [ctypes.POINTER(c_int64), c_int, c_void_p]),
    "b200ops_moe_route_topk": (c_int, [c_void_p] * 4 + [c_int64] * 4 + [c_void_p]),
    "b200ops_moe_permute": (c_int, [c_void_p] * 5 + [c_int64] * 4 + [c_void_p]),
    "b200ops_moe_ep_plan": (c_int, [c_void_p] * 4 + [c_int64] * 4 + [c_void_p]),
    "b200ops_moe_copy_rows": (c_int, [c_void_p] * 4 + [c_int64, c_void_p, c_int64, c_int64, c_void_p]),
    "b200ops_moe_finalize": (c_int, [c_void_p] * 4 + [c_int64] * 3 + [c_void_p]),
    "b200ops_grouped_matmul_scatter": (c_int, [c_void_p] * 3 + [c_int64] * 4 + [c_void_p, c_size_t, c_void_p,
                                                                                 c_void_p, c_int64, c_int64,
                                                                                 c_int64, c_void_p]),
    "b200ops_moe_push_rows": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64,
                                      c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p]),
    "b200ops_peer_barrier": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "b200ops_pipeline_status": (c_int, [ctypes.POINTER(c_int)]),
    "b200ops_reload_options": (None, []),
    "b200ops_matmul": (c_int, [c_void_p] * 3 + [c_int64] * 3 + [c_void_p]),
    "b200ops_moe_dispatch": (c_int, [c_void_p] * 7 + [c_int64] * 2 + [c_void_p] * 6 + [c_int64] * 8 + [c_void_p]),
    "b200ops_moe_gather": (c_int, [c_void_p] * 8 + [c_int64] * 5 + [c_void_p]),
    "b200ops_moe_combine": (c_int, [c_void_p] * 7 + [c_int64] * 5 + [c_void_p]),
}

_lib = None


class B200OpsError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"b200ops error {code}: {message}")
        self.code = code
        self.message = message


def load() -> ctypes.CDLL:
    """dlopen libb200ops.so and attach the prototypes.  Raises if the library is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} is not built; run ascend-ops_b200/build.py")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().b200ops_last_error().decode()


def check(rc: int) -> None:
    if rc != OK:
        raise B200OpsError(rc, last_error())


def _ptr(t):
    """Device (or host) address of a torch tensor, or None."""
    return None if t is None else c_void_p(t.data_ptr())


def _stream(stream):
    if stream is None:
        import torch

        stream = torch.cuda.current_stream().cuda_stream
    return c_void_p(stream)


# Thin helpers: every argument is passed straight through; outputs are caller-allocated.
def add_rms_norm(x, residual, weight, eps, y, residual_out, stream=None):
    check(load().b200ops_add_rms_norm(_ptr(x), _ptr(residual), _ptr(weight), eps, _ptr(y),
                                      _ptr(residual_out), x.shape[0], x.shape[1], _stream(stream)))


def swiglu(x, y, stream=None):
    check(load().b200ops_swiglu(_ptr(x), _ptr(y), x.shape[0], x.shape[1], _stream(stream)))


def rope(q, k, position_ids, cos_cache, sin_cache, out_q, out_k, stream=None):
    check(load().b200ops_rope(_ptr(q), _ptr(k), _ptr(position_ids), _ptr(cos_cache),
                              _ptr(sin_cache), _ptr(out_q), _ptr(out_k), q.shape[0], q.shape[1],
                              k.shape[1], q.shape[2], cos_cache.shape[0], _stream(stream)))


def reshape_and_cache(key, value, key_cache, value_cache, slot_indices, layout, stream=None):
    dims = (c_int64 * 4)(*key_cache.shape)
    check(load().b200ops_reshape_and_cache(_ptr(key), _ptr(value), _ptr(key_cache),
                                           _ptr(value_cache), _ptr(slot_indices), key.shape[0],
                                           key.shape[1], key.shape[2], dims, layout,
                                           _stream(stream)))


def paged_attention_workspace_size(bs, num_heads, num_kv_heads, head_dim, page_size,
                                   max_pages_per_seq) -> int:
    return load().b200ops_paged_attention_workspace_size(bs, num_heads, num_kv_heads, head_dim,
                                                         page_size, max_pages_per_seq)


def paged_attention(q, key_cache, value_cache, block_tables, context_lens, out, num_kv_heads,
                    page_size, layout, workspace, stream=None):
    ws_size = 0 if workspace is None else workspace.numel() * workspace.element_size()
    check(load().b200ops_paged_attention(_ptr(q), _ptr(key_cache), _ptr(value_cache),
                                         _ptr(block_tables), _ptr(context_lens), _ptr(out),
                                         q.shape[0], q.shape[1], num_kv_heads, q.shape[2],
                                         key_cache.shape[0], page_size, block_tables.shape[1],
                                         layout, _ptr(workspace), ws_size, _stream(stream)))


def paged_attention_static(q, key_cache, value_cache, block_tables, context_lens, out, num_kv_heads,
                           page_size, layout, stream=None):
    """Same as paged_attention, with the scratch inside the library (nothing is allocated)."""
    check(load().b200ops_paged_attention_static(_ptr(q), _ptr(key_cache), _ptr(value_cache),
                                                _ptr(block_tables), _ptr(context_lens), _ptr(out),
                                                q.shape[0], q.shape[1], num_kv_heads, q.shape[2],
                                                key_cache.shape[0], page_size,
                                                block_tables.shape[1], layout, _stream(stream)))


def grouped_matmul_workspace_size(num_tokens, k, num_experts, n) -> int:
    return load().b200ops_grouped_matmul_workspace_size(num_tokens, k, num_experts, n)


def grouped_matmul(x, w_storage, group_list, y, workspace=None, stream=None):
    """`w_storage` is the [E, N, K] storage tensor (the torch-level view is its transpose).
    `workspace` (uint8 tensor of grouped_matmul_workspace_size bytes) enables split-K."""
    e, n, k = w_storage.shape
    ws_size = 0 if workspace is None else workspace.numel() * workspace.element_size()
    check(load().b200ops_grouped_matmul(_ptr(x), _ptr(w_storage), _ptr(group_list), _ptr(y),
                                        x.shape[0], k, e, n, _ptr(workspace), ws_size, _stream(stream)))


def grouped_matmul_swiglu(x, w_storage, group_list, y, workspace=None, stream=None):
    """`w_storage` [E, 2*d, K]: gate rows then up rows; y [M, d] = swiglu(x @ w).  `workspace` as
    for grouped_matmul (size from grouped_matmul_workspace_size with n = 2*d)."""
    e, n, k = w_storage.shape
    ws_size = 0 if workspace is None else workspace.numel() * workspace.element_size()
    check(load().b200ops_grouped_matmul_swiglu(_ptr(x), _ptr(w_storage), _ptr(group_list), _ptr(y),
                                               x.shape[0], k, e, n, _ptr(workspace), ws_size, _stream(stream)))


def matmul(x, w, y, stream=None):
    """y [m, n] = x [m, k] . w [n, k]^T (any m, n, k)."""
    check(load().b200ops_matmul(_ptr(x), _ptr(w), _ptr(y), x.shape[0], w.shape[0], x.shape[1], _stream(stream)))


def reload_options() -> None:
    """Make the library read its B200OPS_* tuning variables from the environment again."""
    load().b200ops_reload_options()


def set_option(name: str, value) -> None:
    """Set (or with value None, unset) a B200OPS_* tuning variable for this process."""
    if value is None:
        os.environ.pop(name, None)
    else:
        os.environ[name] = str(value)
    reload_options()


def pipeline_status() -> int:
    v = c_int(0)
    check(load().b200ops_pipeline_status(ctypes.byref(v)))
    return v.value
