"""Decode-layer glue around the six operators: fused split+rope+cache, and MoE routing glue around `ops.grouped_matmul`: router top-k, permutation by expert, the
plan of the expert-parallel exchange, row gather/scatter and the weighted recombination.

The reference's operator API stops at grouped_matmul (rows must arrive sorted by expert,
csrc/opdev/op_kernel/grouped_mat_mul_ex.cpp:29-38); these are the steps its caller performs
around it.  Each function forwards to one sm_100a kernel of the C ABI (`b200ops_moe_*`) on
the current CUDA stream; all metadata stays on the device.
"""
import ascend910a_extras.ascend910a_extras_C as _C

route_topk = _C.moe.route_topk
permute = _C.moe.permute
ep_plan = _C.moe.ep_plan
copy_rows = _C.moe.copy_rows
finalize = _C.moe.finalize
fused_qkv_rope_cache = _C.moe.fused_qkv_rope_cache
push_rows = _C.moe.push_rows
peer_barrier = _C.moe.peer_barrier
grouped_matmul_scatter = _C.moe.grouped_matmul_scatter
grouped_matmul_swiglu = _C.moe.grouped_matmul_swiglu
dispatch = _C.moe.dispatch
gather = _C.moe.gather
combine = _C.moe.combine
