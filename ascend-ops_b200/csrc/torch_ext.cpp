// Torch-facing layer: module `ascend910a_extras_C` with the same layout as the reference's
// pybind module (csrc/ffi/bind.cpp:56-61): `print_info` plus submodule `ops` holding
// rope, swiglu, grouped_matmul, add_rms_norm, reshape_and_cache, paged_attention
// (csrc/ffi/ops.cpp:484-491).  Each function checks its arguments under the same
// conditions as the reference FFI, allocates the outputs and the scratch tensor, and
// calls the C ABI of libb200ops.so on the current CUDA stream.  Nothing here computes.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <tuple>
#include <vector>

#include "b200ops.h"

namespace native {

namespace {

void check_status(int rc, const char* op) {
  if (rc == B200OPS_OK) return;
  if (rc == B200OPS_EINVAL) {
    TORCH_CHECK(false, b200ops_last_error());
  }
  throw std::runtime_error(std::string("Failed to execute ") + op + ": " + b200ops_last_error());
}

void check_f16_cuda(const at::Tensor& t, const char* op, const char* name) {
  TORCH_CHECK(t.is_cuda(), op, ": ", name, " must be a CUDA tensor (there is no CPU path)");
  TORCH_CHECK(t.scalar_type() == at::kHalf, op, ": ", name, " must be float16, got ", t.scalar_type());
}

void check_same_device(const at::Tensor& a, const at::Tensor& b, const char* op) {
  TORCH_CHECK(a.device() == b.device(), op, ": all tensors must be on the same device");
}

void* current_stream() { return static_cast<void*>(at::cuda::getCurrentCUDAStream().stream()); }

}  // namespace

// Mirrors native::rope (csrc/ffi/ops.cpp:13-108).
std::vector<at::Tensor> rope(at::Tensor q, at::Tensor k, at::Tensor position_ids,
                             at::Tensor cos_cache, at::Tensor sin_cache) {
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && position_ids.dim() == 1 && cos_cache.dim() == 2 &&
                  sin_cache.dim() == 2,
              "rope: input tensors must be 3D, 3D, 1D, 2D, and 2D, got ", q.dim(), "D, ", k.dim(),
              "D, ", position_ids.dim(), "D, ", cos_cache.dim(), "D, ", sin_cache.dim(), "D");
  TORCH_CHECK(position_ids.size(0) == q.size(0),
              "rope: position_ids must have the same batch size as q, got ", position_ids.size(0),
              " and ", q.size(0));
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && position_ids.is_contiguous() &&
                  cos_cache.is_contiguous() && sin_cache.is_contiguous(),
              "rope: all input tensors must be contiguous");
  check_f16_cuda(q, "rope", "q");
  check_f16_cuda(k, "rope", "k");
  check_f16_cuda(cos_cache, "rope", "cos_cache");
  check_f16_cuda(sin_cache, "rope", "sin_cache");
  TORCH_CHECK(position_ids.is_cuda() && position_ids.scalar_type() == at::kInt,
              "rope: position_ids must be a CUDA int32 tensor, got ", position_ids.scalar_type());
  check_same_device(q, k, "rope");
  check_same_device(q, position_ids, "rope");
  check_same_device(q, cos_cache, "rope");
  check_same_device(q, sin_cache, "rope");
  TORCH_CHECK(k.size(0) == q.size(0) && k.size(2) == q.size(2),
              "rope: q and k must agree in batch size and head_dim, got ", q.sizes(), " and ", k.sizes());
  TORCH_CHECK(cos_cache.size(1) * 2 == q.size(2) && sin_cache.sizes() == cos_cache.sizes(),
              "rope: cos_cache and sin_cache must be [max_pos, head_dim/2], got ", cos_cache.sizes(),
              " and ", sin_cache.sizes(), " for head_dim ", q.size(2));

  const c10::cuda::CUDAGuard guard(q.device());
  at::Tensor out_q = at::empty_like(q);
  at::Tensor out_k = at::empty_like(k);
  check_status(b200ops_rope(q.data_ptr(), k.data_ptr(), position_ids.data_ptr<int32_t>(),
                            cos_cache.data_ptr(), sin_cache.data_ptr(), out_q.data_ptr(),
                            out_k.data_ptr(), q.size(0), q.size(1), k.size(1), q.size(2),
                            cos_cache.size(0), current_stream()),
               "rope");
  return {out_q, out_k};
}

// Mirrors native::swiglu (csrc/ffi/ops.cpp:110-154).
at::Tensor swiglu(at::Tensor x) {
  TORCH_CHECK(x.dim() == 2, "swiglu: input tensor must be 2D, got ", x.dim(), "D tensor");
  TORCH_CHECK(x.size(-1) >= 64 && x.size(-1) % 64 == 0,
              "swiglu: last dimension must be a multiple of 64, got ", x.size(-1));
  TORCH_CHECK(x.is_contiguous(), "swiglu: input tensor must be contiguous");
  check_f16_cuda(x, "swiglu", "x");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({x.size(0), x.size(1) / 2}, x.options());
  check_status(b200ops_swiglu(x.data_ptr(), y.data_ptr(), x.size(0), x.size(1), current_stream()),
               "swiglu");
  return y;
}

// Mirrors native::grouped_matmul (csrc/ffi/ops.cpp:157-233).
at::Tensor grouped_matmul(at::Tensor x, at::Tensor w, at::Tensor group_list) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && group_list.dim() == 1,
              "grouped_matmul: input tensors must be 2D and group_list must be 1D");
  const int64_t num_tokens = x.size(0);
  const int64_t dim = x.size(1);
  const int64_t num_experts = w.size(0);
  const int64_t inner_dim = w.size(2);
  TORCH_CHECK(dim == w.size(1),
              "grouped_matmul: last dimension of x must match second dimension of w, got ", dim,
              " and ", w.size(1));
  TORCH_CHECK(x.is_contiguous() && group_list.is_contiguous(),
              "grouped_matmul: x and group_list must be contiguous tensors");
  TORCH_CHECK(w.stride(1) == 1 && w.stride(2) == dim,
              "grouped_matmul: w must be K-major order, got strides ", w.strides());
  TORCH_CHECK(w.size(1) % 64 == 0 && w.size(2) % 64 == 0,
              "grouped_matmul: second and third dimensions of w must be multiples of 64, got ",
              w.size(1), " and ", w.size(2));
  TORCH_CHECK(num_experts <= 1 || w.stride(0) == dim * inner_dim,
              "grouped_matmul: experts of w must be densely packed, got strides ", w.strides());
  TORCH_CHECK(group_list.size(0) == num_experts,
              "grouped_matmul: group_list must have one entry per expert, got ", group_list.size(0),
              " and ", num_experts);
  check_f16_cuda(x, "grouped_matmul", "x");
  check_f16_cuda(w, "grouped_matmul", "w");
  TORCH_CHECK(group_list.is_cuda() && group_list.scalar_type() == at::kLong,
              "grouped_matmul: group_list must be a CUDA int64 tensor, got ", group_list.scalar_type());
  check_same_device(x, w, "grouped_matmul");
  check_same_device(x, group_list, "grouped_matmul");

  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({num_tokens, inner_dim}, x.options());
  const size_t ws = b200ops_grouped_matmul_workspace_size(num_tokens, dim, num_experts, inner_dim);
  at::Tensor workspace = at::empty({static_cast<int64_t>(ws)}, x.options().dtype(at::kByte));
  check_status(b200ops_grouped_matmul(x.data_ptr(), w.data_ptr(), group_list.data_ptr<int64_t>(),
                                      y.data_ptr(), num_tokens, dim, num_experts, inner_dim,
                                      ws ? workspace.data_ptr() : nullptr, ws, current_stream()),
               "grouped_matmul");
  return y;
}

// Mirrors native::add_rms_norm (csrc/ffi/ops.cpp:236-333).
std::tuple<at::Tensor, at::Tensor> add_rms_norm(at::Tensor x, at::Tensor residual,
                                                at::Tensor weight, float epsilon) {
  TORCH_CHECK(x.dim() == 2 && residual.dim() == 2 && weight.dim() == 1,
              "add_rms_norm: x and residual must be 2D, weight must be 1D");
  TORCH_CHECK(x.size(1) == weight.size(0),
              "add_rms_norm: last dimension of x must match weight size, got ", x.size(1), " and ",
              weight.size(0));
  TORCH_CHECK(x.size(0) == residual.size(0) && x.size(1) == residual.size(1),
              "add_rms_norm: x and residual must have the same shape, got ", x.sizes(), " and ",
              residual.sizes());
  TORCH_CHECK(x.is_contiguous() && residual.is_contiguous() && weight.is_contiguous(),
              "add_rms_norm: all input tensors must be contiguous");
  TORCH_CHECK(x.size(1) % 64 == 0, "add_rms_norm: last dimension must be a multiple of 64, got ",
              x.size(1));
  check_f16_cuda(x, "add_rms_norm", "x");
  check_f16_cuda(residual, "add_rms_norm", "residual");
  check_f16_cuda(weight, "add_rms_norm", "weight");
  check_same_device(x, residual, "add_rms_norm");
  check_same_device(x, weight, "add_rms_norm");

  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({x.size(0), x.size(1)}, x.options());
  at::Tensor residual_output = at::empty({x.size(0), x.size(1)}, x.options());
  check_status(b200ops_add_rms_norm(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), epsilon,
                                    y.data_ptr(), residual_output.data_ptr(), x.size(0), x.size(1),
                                    current_stream()),
               "add_rms_norm");
  return std::make_tuple(y, residual_output);
}

namespace {

// NHD if the cache's trailing sizes repeat the key's [Hkv, D]; else NZ if the last size is 16.
int cache_layout_for_key(const at::Tensor& cache, int64_t num_kv_heads, int64_t head_size,
                         const char* op) {
  if (cache.size(2) == num_kv_heads && cache.size(3) == head_size) return B200OPS_KV_LAYOUT_NHD;
  TORCH_CHECK(cache.size(3) == 16, op,
              ": cache must be [pages, Hkv*D/16, page_size, 16] or [pages, page_size, Hkv, D], got ",
              cache.sizes());
  return B200OPS_KV_LAYOUT_NZ;
}

}  // namespace

// Mirrors native::reshape_and_cache (csrc/ffi/ops.cpp:336-405).
void reshape_and_cache(at::Tensor key, at::Tensor value, at::Tensor key_cache,
                       at::Tensor value_cache, at::Tensor slot_indices) {
  TORCH_CHECK(key.dim() == 3 && key_cache.dim() == 4 && slot_indices.dim() == 1,
              "reshape_and_cache: key must be 3D, key_cache must be 4D, slot_indices must be 1D");
  TORCH_CHECK(key.is_contiguous() && key_cache.is_contiguous() && slot_indices.is_contiguous(),
              "reshape_and_cache: key, key_cache, slot_indices must be contiguous tensors");
  if (value.numel() > 0) {
    TORCH_CHECK(value.dim() == 3 && value.is_contiguous(),
                "reshape_and_cache: value must be 3D and contiguous if not None");
    TORCH_CHECK(value.sizes() == key.sizes(), "reshape_and_cache: value must have key's shape, got ",
                value.sizes(), " and ", key.sizes());
    check_f16_cuda(value, "reshape_and_cache", "value");
  }
  if (value_cache.numel() > 0) {
    TORCH_CHECK(value_cache.dim() == 4 && value_cache.is_contiguous(),
                "reshape_and_cache: value_cache must be 4D and contiguous if not None");
    TORCH_CHECK(value_cache.sizes() == key_cache.sizes(),
                "reshape_and_cache: value_cache must have key_cache's shape, got ",
                value_cache.sizes(), " and ", key_cache.sizes());
    check_f16_cuda(value_cache, "reshape_and_cache", "value_cache");
  }
  // The reference's host tiling fails the launch when the lengths differ
  // (csrc/opdev/op_host/reshape_and_cache_ex.cpp:33-36).
  TORCH_CHECK(slot_indices.size(0) == key.size(0),
              "reshape_and_cache: slot_indices must have one entry per token, got ",
              slot_indices.size(0), " and ", key.size(0));
  check_f16_cuda(key, "reshape_and_cache", "key");
  check_f16_cuda(key_cache, "reshape_and_cache", "key_cache");
  TORCH_CHECK(slot_indices.is_cuda() && slot_indices.scalar_type() == at::kInt,
              "reshape_and_cache: slot_indices must be a CUDA int32 tensor, got ",
              slot_indices.scalar_type());
  check_same_device(key, key_cache, "reshape_and_cache");
  check_same_device(key, slot_indices, "reshape_and_cache");

  const int layout = cache_layout_for_key(key_cache, key.size(1), key.size(2), "reshape_and_cache");
  const int64_t dims[4] = {key_cache.size(0), key_cache.size(1), key_cache.size(2), key_cache.size(3)};
  const c10::cuda::CUDAGuard guard(key.device());
  check_status(b200ops_reshape_and_cache(
                   key.data_ptr(), value.numel() > 0 ? value.data_ptr() : nullptr,
                   key_cache.data_ptr(), value_cache.numel() > 0 ? value_cache.data_ptr() : nullptr,
                   slot_indices.data_ptr<int32_t>(), key.size(0), key.size(1), key.size(2), dims,
                   layout, current_stream()),
               "reshape_and_cache");
}

// Mirrors native::paged_attention (csrc/ffi/ops.cpp:408-482).  The reference validates
// nothing here; these checks are what the kernels rely on.
at::Tensor paged_attention(at::Tensor q, at::Tensor key_cache, at::Tensor value_cache,
                           at::Tensor block_tables, at::Tensor context_lens) {
  TORCH_CHECK(q.dim() == 3 && key_cache.dim() == 4 && value_cache.dim() == 4 &&
                  block_tables.dim() == 2 && context_lens.dim() == 1,
              "paged_attention: q must be 3D, caches 4D, block_tables 2D, context_lens 1D");
  TORCH_CHECK(q.is_contiguous() && key_cache.is_contiguous() && value_cache.is_contiguous() &&
                  block_tables.is_contiguous() && context_lens.is_contiguous(),
              "paged_attention: all input tensors must be contiguous");
  check_f16_cuda(q, "paged_attention", "q");
  check_f16_cuda(key_cache, "paged_attention", "key_cache");
  check_f16_cuda(value_cache, "paged_attention", "value_cache");
  TORCH_CHECK(block_tables.is_cuda() && block_tables.scalar_type() == at::kInt &&
                  context_lens.is_cuda() && context_lens.scalar_type() == at::kInt,
              "paged_attention: block_tables and context_lens must be CUDA int32 tensors");
  TORCH_CHECK(value_cache.sizes() == key_cache.sizes(),
              "paged_attention: key_cache and value_cache must have the same shape, got ",
              key_cache.sizes(), " and ", value_cache.sizes());
  TORCH_CHECK(block_tables.size(0) == q.size(0) && context_lens.size(0) == q.size(0),
              "paged_attention: block_tables and context_lens must have one row per sequence");
  check_same_device(q, key_cache, "paged_attention");
  check_same_device(q, value_cache, "paged_attention");
  check_same_device(q, block_tables, "paged_attention");
  check_same_device(q, context_lens, "paged_attention");

  const int64_t bs = q.size(0), num_heads = q.size(1), head_dim = q.size(2);
  int layout;
  int64_t num_kv_heads, page_size;
  if (key_cache.size(3) == head_dim) {
    // [pages, page_size, num_kv_heads, head_dim]
    layout = B200OPS_KV_LAYOUT_NHD;
    page_size = key_cache.size(1);
    num_kv_heads = key_cache.size(2);
  } else {
    // kvcache: [num_pages, num_kv_heads * head_dim / 16, page_size, 16] (csrc/ffi/ops.cpp:412-415)
    TORCH_CHECK(key_cache.size(3) == 16 && (key_cache.size(1) * 16) % head_dim == 0,
                "paged_attention: cache must be [pages, Hkv*D/16, page_size, 16] or "
                "[pages, page_size, Hkv, D], got ", key_cache.sizes());
    layout = B200OPS_KV_LAYOUT_NZ;
    num_kv_heads = key_cache.size(1) * 16 / head_dim;
    page_size = key_cache.size(2);
  }
  TORCH_CHECK(num_kv_heads > 0 && num_heads % num_kv_heads == 0,
              "paged_attention: num_heads ", num_heads, " is not a multiple of num_kv_heads ",
              num_kv_heads);

  const c10::cuda::CUDAGuard guard(q.device());
  at::Tensor y = at::empty_like(q);
  if (bs == 0) return y;
  const size_t ws = b200ops_paged_attention_workspace_size(bs, num_heads, num_kv_heads, head_dim,
                                                           page_size, block_tables.size(1));
  at::Tensor workspace = at::empty({static_cast<int64_t>(ws)}, q.options().dtype(at::kByte));
  check_status(b200ops_paged_attention(q.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(),
                                       block_tables.data_ptr<int32_t>(),
                                       context_lens.data_ptr<int32_t>(), y.data_ptr(), bs, num_heads,
                                       num_kv_heads, head_dim, key_cache.size(0), page_size,
                                       block_tables.size(1), layout,
                                       ws ? workspace.data_ptr() : nullptr, ws, current_stream()),
               "paged_attention");
  return y;
}

// Mirrors native::matmul of the reference's earlier interface (_csrc/ffi.cpp:408-442): the same
// three argument checks and messages, float16 only, output allocated here.
at::Tensor matmul(const at::Tensor& x, const at::Tensor& w) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2, "matmul: input tensors must be 2D");
  TORCH_CHECK(x.size(1) == w.size(1), "matmul: last dimension of x must match last dimension of w, got ",
              x.size(1), " and ", w.size(1));
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous(), "matmul: x and w must be contiguous tensors");
  TORCH_CHECK(x.scalar_type() == at::kHalf && w.scalar_type() == at::kHalf,
              "matmul: only float16 is supported, got ", x.scalar_type());
  TORCH_CHECK(x.is_cuda() && w.is_cuda(), "matmul: x and w must be CUDA tensors (there is no CPU path)");
  check_same_device(x, w, "matmul");
  TORCH_CHECK(w.size(0) > 0 && x.size(1) > 0, "matmul: empty weight");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({x.size(0), w.size(0)}, x.options());
  check_status(b200ops_matmul(x.data_ptr(), w.data_ptr(), y.data_ptr(), x.size(0), w.size(0), x.size(1),
                              current_stream()),
               "matmul");
  return y;
}

int print_info(int device_id) {
  check_status(b200ops_print_info(device_id, nullptr, 0), "print_info");
  return 0;
}

// ---- MoE routing glue (no counterpart in the reference FFI; see include/b200ops.h) ----
namespace {
void check_i32_cuda(const at::Tensor& t, const char* op, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(), op, ": ", name,
              " must be a contiguous CUDA int32 tensor");
}
}  // namespace

std::tuple<at::Tensor, at::Tensor> moe_route_topk(at::Tensor x, at::Tensor router_weight, int64_t top_k) {
  TORCH_CHECK(x.dim() == 2 && router_weight.dim() == 2 && x.size(1) == router_weight.size(1),
              "moe_route_topk: x must be [T, H] and router_weight [E, H], got ", x.sizes(), " and ",
              router_weight.sizes());
  TORCH_CHECK(x.is_contiguous() && router_weight.is_contiguous(), "moe_route_topk: tensors must be contiguous");
  check_f16_cuda(x, "moe_route_topk", "x");
  check_f16_cuda(router_weight, "moe_route_topk", "router_weight");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor ids = at::empty({x.size(0), top_k}, x.options().dtype(at::kInt));
  at::Tensor wts = at::empty({x.size(0), top_k}, x.options().dtype(at::kFloat));
  check_status(b200ops_moe_route_topk(x.data_ptr(), router_weight.data_ptr(), ids.data_ptr<int32_t>(),
                                      wts.data_ptr<float>(), x.size(0), x.size(1), router_weight.size(0),
                                      top_k, current_stream()),
               "moe_route_topk");
  return {ids, wts};
}

// Returns (slot_to_row, counts, group_list, overflow[1]).
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> moe_permute(at::Tensor expert_ids,
                                                                       int64_t num_experts, int64_t world,
                                                                       int64_t segment_rows) {
  check_i32_cuda(expert_ids, "moe_permute", "expert_ids");
  const c10::cuda::CUDAGuard guard(expert_ids.device());
  const int64_t slots = expert_ids.numel();
  at::Tensor pos = at::empty({slots}, expert_ids.options());
  at::Tensor counts = at::empty({num_experts}, expert_ids.options());
  at::Tensor gl = at::empty({num_experts}, expert_ids.options().dtype(at::kLong));
  at::Tensor overflow = at::empty({1}, expert_ids.options());
  check_status(b200ops_moe_permute(expert_ids.data_ptr<int32_t>(), pos.data_ptr<int32_t>(),
                                   counts.data_ptr<int32_t>(), gl.data_ptr<int64_t>(),
                                   overflow.data_ptr<int32_t>(), slots, num_experts, world, segment_rows,
                                   current_stream()),
               "moe_permute");
  return {pos, counts, gl, overflow};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_ep_plan(at::Tensor all_counts, int64_t rank,
                                                           int64_t segment_rows) {
  check_i32_cuda(all_counts, "moe_ep_plan", "all_counts");
  TORCH_CHECK(all_counts.dim() == 2, "moe_ep_plan: all_counts must be [world, experts]");
  const c10::cuda::CUDAGuard guard(all_counts.device());
  const int64_t world = all_counts.size(0), experts = all_counts.size(1);
  at::Tensor map = at::empty({world * segment_rows}, all_counts.options());
  at::Tensor gl = at::empty({experts / std::max<int64_t>(world, 1)}, all_counts.options().dtype(at::kLong));
  at::Tensor total = at::empty({1}, all_counts.options());
  check_status(b200ops_moe_ep_plan(all_counts.data_ptr<int32_t>(), map.data_ptr<int32_t>(),
                                   gl.data_ptr<int64_t>(), total.data_ptr<int32_t>(), world, experts, rank,
                                   segment_rows, current_stream()),
               "moe_ep_plan");
  return {map, gl, total};
}

void moe_copy_rows(at::Tensor dst, at::Tensor src, c10::optional<at::Tensor> dst_index,
                   c10::optional<at::Tensor> src_index, int64_t src_div, c10::optional<at::Tensor> n_valid,
                   int64_t n_max) {
  TORCH_CHECK(dst.dim() == 2 && src.dim() == 2 && dst.size(1) == src.size(1) && dst.is_contiguous() &&
                  src.is_contiguous(),
              "moe_copy_rows: dst and src must be contiguous [rows, H] with the same H");
  check_f16_cuda(dst, "moe_copy_rows", "dst");
  check_f16_cuda(src, "moe_copy_rows", "src");
  if (dst_index) check_i32_cuda(*dst_index, "moe_copy_rows", "dst_index");
  if (src_index) check_i32_cuda(*src_index, "moe_copy_rows", "src_index");
  if (n_valid) check_i32_cuda(*n_valid, "moe_copy_rows", "n_valid");
  TORCH_CHECK((!dst_index || dst_index->numel() >= n_max) && (!src_index || src_index->numel() >= n_max),
              "moe_copy_rows: index tensors shorter than n_max");
  TORCH_CHECK((dst_index || n_max <= dst.size(0)) && (src_index || n_max <= src.size(0) * src_div),
              "moe_copy_rows: n_max exceeds the tensor rows");
  const c10::cuda::CUDAGuard guard(dst.device());
  check_status(b200ops_moe_copy_rows(dst.data_ptr(), src.data_ptr(),
                                     dst_index ? dst_index->data_ptr<int32_t>() : nullptr,
                                     src_index ? src_index->data_ptr<int32_t>() : nullptr, src_div,
                                     n_valid ? n_valid->data_ptr<int32_t>() : nullptr, n_max, dst.size(1),
                                     current_stream()),
               "moe_copy_rows");
}

at::Tensor moe_finalize(at::Tensor rows, at::Tensor slot_to_row, at::Tensor expert_weights) {
  TORCH_CHECK(rows.dim() == 2 && rows.is_contiguous() && expert_weights.dim() == 2 &&
                  expert_weights.is_contiguous() && slot_to_row.numel() == expert_weights.numel(),
              "moe_finalize: rows [R, H], expert_weights [T, k], slot_to_row [T*k]");
  check_f16_cuda(rows, "moe_finalize", "rows");
  check_i32_cuda(slot_to_row, "moe_finalize", "slot_to_row");
  TORCH_CHECK(expert_weights.is_cuda() && expert_weights.scalar_type() == at::kFloat,
              "moe_finalize: expert_weights must be a CUDA float32 tensor");
  const c10::cuda::CUDAGuard guard(rows.device());
  at::Tensor y = at::empty({expert_weights.size(0), rows.size(1)}, rows.options());
  check_status(b200ops_moe_finalize(rows.data_ptr(), slot_to_row.data_ptr<int32_t>(),
                                    expert_weights.data_ptr<float>(), y.data_ptr(), expert_weights.size(0),
                                    expert_weights.size(1), rows.size(1), current_stream()),
               "moe_finalize");
  return y;
}

// q_out = rope(q part of qkv); rope(k) and v go into the caches.  See b200ops_fused_qkv_rope_cache.
// q_norm_weight / k_norm_weight ([head_dim] f16, optional): per-head RMSNorm before the rotation.
at::Tensor fused_qkv_rope_cache(at::Tensor qkv, at::Tensor position_ids, at::Tensor cos_cache,
                                at::Tensor sin_cache, at::Tensor slot_indices, at::Tensor key_cache,
                                at::Tensor value_cache, int64_t num_heads, int64_t num_kv_heads,
                                c10::optional<at::Tensor> q_norm_weight, c10::optional<at::Tensor> k_norm_weight,
                                double epsilon) {
  TORCH_CHECK(qkv.dim() == 2 && qkv.is_contiguous() && qkv.size(1) % (num_heads + 2 * num_kv_heads) == 0,
              "fused_qkv_rope_cache: qkv must be contiguous [T, (Hq + 2*Hkv) * D], got ", qkv.sizes());
  const int64_t head_dim = qkv.size(1) / (num_heads + 2 * num_kv_heads);
  TORCH_CHECK(key_cache.dim() == 4 && key_cache.is_contiguous() && value_cache.is_contiguous() &&
                  value_cache.sizes() == key_cache.sizes(),
              "fused_qkv_rope_cache: caches must be contiguous 4D tensors of the same shape");
  TORCH_CHECK(cos_cache.dim() == 2 && cos_cache.size(1) * 2 == head_dim && cos_cache.is_contiguous() &&
                  sin_cache.is_contiguous() && sin_cache.sizes() == cos_cache.sizes(),
              "fused_qkv_rope_cache: cos_cache and sin_cache must be [max_pos, head_dim/2]");
  TORCH_CHECK(position_ids.numel() == qkv.size(0) && slot_indices.numel() == qkv.size(0),
              "fused_qkv_rope_cache: one position and one slot per token");
  check_f16_cuda(qkv, "fused_qkv_rope_cache", "qkv");
  check_f16_cuda(key_cache, "fused_qkv_rope_cache", "key_cache");
  check_f16_cuda(value_cache, "fused_qkv_rope_cache", "value_cache");
  check_f16_cuda(cos_cache, "fused_qkv_rope_cache", "cos_cache");
  check_f16_cuda(sin_cache, "fused_qkv_rope_cache", "sin_cache");
  check_i32_cuda(position_ids, "fused_qkv_rope_cache", "position_ids");
  check_i32_cuda(slot_indices, "fused_qkv_rope_cache", "slot_indices");
  for (const auto* w : {&q_norm_weight, &k_norm_weight}) {
    if (!w->has_value()) continue;
    TORCH_CHECK((*w)->dim() == 1 && (*w)->size(0) == head_dim && (*w)->is_contiguous(),
                "fused_qkv_rope_cache: a norm weight must be a contiguous [head_dim] tensor");
    check_f16_cuda(**w, "fused_qkv_rope_cache", "norm weight");
    check_same_device(qkv, **w, "fused_qkv_rope_cache");
  }
  const int layout = cache_layout_for_key(key_cache, num_kv_heads, head_dim, "fused_qkv_rope_cache");
  const int64_t dims[4] = {key_cache.size(0), key_cache.size(1), key_cache.size(2), key_cache.size(3)};
  const c10::cuda::CUDAGuard guard(qkv.device());
  at::Tensor q_out = at::empty({qkv.size(0), num_heads, head_dim}, qkv.options());
  check_status(b200ops_fused_qkv_norm_rope_cache(qkv.data_ptr(),
                                            q_norm_weight ? q_norm_weight->data_ptr() : nullptr,
                                            k_norm_weight ? k_norm_weight->data_ptr() : nullptr,
                                            static_cast<float>(epsilon), position_ids.data_ptr<int32_t>(),
                                            cos_cache.data_ptr(), sin_cache.data_ptr(),
                                            slot_indices.data_ptr<int32_t>(), q_out.data_ptr(),
                                            key_cache.data_ptr(), value_cache.data_ptr(), qkv.size(0),
                                            num_heads, num_kv_heads, head_dim, cos_cache.size(0), dims,
                                            layout, current_stream()),
               "fused_qkv_rope_cache");
  return q_out;
}

// Peer-memory exchange (see b200ops_moe_push_rows / b200ops_peer_barrier).  Peer addresses are
// passed as Python ints (what torch's symmetric-memory handle reports as buffer_ptrs).
void moe_push_rows(at::Tensor src, at::Tensor index, int64_t src_div, c10::optional<at::Tensor> n_valid,
                   int64_t n_max, std::vector<int64_t> peer_rows, int64_t cap, int64_t my_rank,
                   c10::optional<at::Tensor> counts, std::vector<int64_t> peer_counts) {
  TORCH_CHECK(src.dim() == 2 && src.is_contiguous(), "moe_push_rows: src must be contiguous [rows, H]");
  check_f16_cuda(src, "moe_push_rows", "src");
  check_i32_cuda(index, "moe_push_rows", "index");
  TORCH_CHECK(index.numel() >= n_max, "moe_push_rows: index shorter than n_max");
  TORCH_CHECK(n_max <= src.size(0) * src_div, "moe_push_rows: n_max exceeds the source rows");
  if (n_valid) check_i32_cuda(*n_valid, "moe_push_rows", "n_valid");
  if (counts) {
    check_i32_cuda(*counts, "moe_push_rows", "counts");
    TORCH_CHECK(peer_counts.size() == peer_rows.size(), "moe_push_rows: one count table per peer");
  }
  std::vector<void*> rows(peer_rows.size()), cnts(peer_counts.size());
  for (size_t i = 0; i < peer_rows.size(); ++i) rows[i] = reinterpret_cast<void*>(peer_rows[i]);
  for (size_t i = 0; i < peer_counts.size(); ++i) cnts[i] = reinterpret_cast<void*>(peer_counts[i]);
  const c10::cuda::CUDAGuard guard(src.device());
  check_status(b200ops_moe_push_rows(src.data_ptr(), index.data_ptr<int32_t>(), src_div,
                                     n_valid ? n_valid->data_ptr<int32_t>() : nullptr, n_max, rows.data(),
                                     static_cast<int64_t>(rows.size()), cap, my_rank, src.size(1),
                                     counts ? counts->data_ptr<int32_t>() : nullptr,
                                     counts ? counts->numel() : 0, counts ? cnts.data() : nullptr,
                                     current_stream()),
               "moe_push_rows");
}

// grouped_matmul with the result rows stored straight into the peers' return buffers.
void grouped_matmul_scatter(at::Tensor x, at::Tensor w, at::Tensor group_list, at::Tensor row_index,
                            std::vector<int64_t> peer_out, int64_t cap, int64_t my_rank) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && group_list.dim() == 1 && x.size(1) == w.size(1),
              "grouped_matmul_scatter: x [M, K], w [E, K, N], group_list [E]");
  TORCH_CHECK(x.is_contiguous() && group_list.is_contiguous() && w.stride(1) == 1 && w.stride(2) == x.size(1),
              "grouped_matmul_scatter: x must be contiguous and w K-major");
  TORCH_CHECK(w.size(1) % 64 == 0 && w.size(2) % 64 == 0 && group_list.size(0) == w.size(0),
              "grouped_matmul_scatter: K and N must be multiples of 64, one group end per expert");
  check_f16_cuda(x, "grouped_matmul_scatter", "x");
  check_f16_cuda(w, "grouped_matmul_scatter", "w");
  check_i32_cuda(row_index, "grouped_matmul_scatter", "row_index");
  TORCH_CHECK(group_list.is_cuda() && group_list.scalar_type() == at::kLong && row_index.numel() >= x.size(0),
              "grouped_matmul_scatter: group_list must be CUDA int64, row_index must cover every row");
  std::vector<void*> peers(peer_out.size());
  for (size_t i = 0; i < peer_out.size(); ++i) peers[i] = reinterpret_cast<void*>(peer_out[i]);
  const c10::cuda::CUDAGuard guard(x.device());
  const size_t ws = b200ops_grouped_matmul_workspace_size(x.size(0), x.size(1), w.size(0), w.size(2));
  at::Tensor workspace = at::empty({static_cast<int64_t>(ws)}, x.options().dtype(at::kByte));
  check_status(b200ops_grouped_matmul_scatter(x.data_ptr(), w.data_ptr(), group_list.data_ptr<int64_t>(),
                                              x.size(0), x.size(1), w.size(0), w.size(2),
                                              ws ? workspace.data_ptr() : nullptr, ws,
                                              row_index.data_ptr<int32_t>(), peers.data(),
                                              static_cast<int64_t>(peers.size()), cap, my_rank, current_stream()),
               "grouped_matmul_scatter");
}

// Gate/up projection with SwiGLU in the GEMM's epilogue: w [E, K, 2*d] (the first d output
// columns are the gate, the rest the up projection) -> [M, d], bit-identical to
// ops.swiglu(ops.grouped_matmul(x, w, group_list)).
at::Tensor grouped_matmul_swiglu(at::Tensor x, at::Tensor w, at::Tensor group_list) {
  TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && group_list.dim() == 1 && x.size(1) == w.size(1),
              "grouped_matmul_swiglu: x [M, K], w [E, K, 2*d], group_list [E]");
  TORCH_CHECK(x.is_contiguous() && group_list.is_contiguous() && w.stride(1) == 1 && w.stride(2) == x.size(1),
              "grouped_matmul_swiglu: x must be contiguous and w K-major");
  TORCH_CHECK(w.size(0) <= 1 || w.stride(0) == w.size(1) * w.size(2),
              "grouped_matmul_swiglu: experts of w must be densely packed");
  TORCH_CHECK(w.size(1) % 64 == 0 && w.size(2) % 128 == 0 && group_list.size(0) == w.size(0),
              "grouped_matmul_swiglu: K must be a multiple of 64 and 2*d of 128, one group end per expert");
  check_f16_cuda(x, "grouped_matmul_swiglu", "x");
  check_f16_cuda(w, "grouped_matmul_swiglu", "w");
  TORCH_CHECK(group_list.is_cuda() && group_list.scalar_type() == at::kLong,
              "grouped_matmul_swiglu: group_list must be a CUDA int64 tensor");
  check_same_device(x, w, "grouped_matmul_swiglu");
  check_same_device(x, group_list, "grouped_matmul_swiglu");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({x.size(0), w.size(2) / 2}, x.options());
  const size_t ws = b200ops_grouped_matmul_workspace_size(x.size(0), x.size(1), w.size(0), w.size(2));
  at::Tensor workspace = at::empty({static_cast<int64_t>(ws)}, x.options().dtype(at::kByte));
  check_status(b200ops_grouped_matmul_swiglu(x.data_ptr(), w.data_ptr(), group_list.data_ptr<int64_t>(),
                                             y.data_ptr(), x.size(0), x.size(1), w.size(0), w.size(2),
                                             ws ? workspace.data_ptr() : nullptr, ws, current_stream()),
               "grouped_matmul_swiglu");
  return y;
}

void peer_barrier(std::vector<int64_t> peer_flags, at::Tensor my_flags, at::Tensor state, int64_t my_rank) {
  TORCH_CHECK(my_flags.is_cuda() && state.is_cuda() && state.numel() >= 2 &&
                  my_flags.numel() >= static_cast<int64_t>(peer_flags.size()) &&
                  my_flags.element_size() == 4 && state.element_size() == 4,
              "peer_barrier: flags [world] and state [2] must be 32-bit CUDA tensors");
  std::vector<void*> flags(peer_flags.size());
  for (size_t i = 0; i < peer_flags.size(); ++i) flags[i] = reinterpret_cast<void*>(peer_flags[i]);
  const c10::cuda::CUDAGuard guard(state.device());
  check_status(b200ops_peer_barrier(flags.data(), my_flags.data_ptr(), state.data_ptr(),
                                    static_cast<int64_t>(flags.size()), my_rank, current_stream()),
               "peer_barrier");
}

namespace {
std::vector<void*> as_pointers(const std::vector<int64_t>& v) {
  std::vector<void*> out(v.size());
  for (size_t i = 0; i < v.size(); ++i) out[i] = reinterpret_cast<void*>(v[i]);
  return out;
}
}  // namespace

// Fused dispatch of the expert-parallel step (see b200ops_moe_dispatch).  Routes with
// router_weight, or takes expert_ids (then returns them unchanged with an empty weight tensor).
// Returns (slot_to_row, expert_ids, expert_weights).
std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_dispatch(
    at::Tensor x, c10::optional<at::Tensor> router_weight, c10::optional<at::Tensor> expert_ids, int64_t top_k,
    c10::optional<at::Tensor> expert_slots, c10::optional<at::Tensor> num_replicas, int64_t token_offset,
    std::vector<int64_t> peer_recv, std::vector<int64_t> peer_counts, at::Tensor cursor, at::Tensor state, c10::optional<at::Tensor> overflow, int64_t num_experts, int64_t cap,
    int64_t my_rank) {
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous(), "moe_dispatch: x must be contiguous [T, H]");
  check_f16_cuda(x, "moe_dispatch", "x");
  TORCH_CHECK(router_weight.has_value() != expert_ids.has_value(),
              "moe_dispatch: give either router_weight or expert_ids");
  check_i32_cuda(cursor, "moe_dispatch", "cursor");
  TORCH_CHECK(state.is_cuda() && state.element_size() == 4 && state.numel() >= 5 && state.is_contiguous(),
              "moe_dispatch: state must be a contiguous 32-bit CUDA tensor of at least 5 elements");
  TORCH_CHECK(peer_recv.size() == peer_counts.size(), "moe_dispatch: one receive buffer and count table per rank");
  const int64_t world = static_cast<int64_t>(peer_recv.size());
  const int64_t num_slots = cursor.numel();
  const int64_t tokens = x.size(0);
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor pos = at::empty({tokens * top_k}, x.options().dtype(at::kInt));
  at::Tensor ids, wts;
  if (router_weight) {
    TORCH_CHECK(router_weight->dim() == 2 && router_weight->size(1) == x.size(1) && router_weight->is_contiguous(),
                "moe_dispatch: router_weight must be contiguous [E, H]");
    check_f16_cuda(*router_weight, "moe_dispatch", "router_weight");
    TORCH_CHECK(router_weight->size(0) == num_experts, "moe_dispatch: router_weight rows must equal num_experts");
    ids = at::empty({tokens, top_k}, x.options().dtype(at::kInt));
    wts = at::empty({tokens, top_k}, x.options().dtype(at::kFloat));
  } else {
    check_i32_cuda(*expert_ids, "moe_dispatch", "expert_ids");
    TORCH_CHECK(expert_ids->numel() == tokens * top_k, "moe_dispatch: expert_ids must be [T, top_k]");
    ids = *expert_ids;
    wts = at::empty({0}, x.options().dtype(at::kFloat));
  }
  int64_t max_rep = 0;
  if (expert_slots) {
    TORCH_CHECK(num_replicas.has_value(), "moe_dispatch: expert_slots needs num_replicas");
    check_i32_cuda(*expert_slots, "moe_dispatch", "expert_slots");
    check_i32_cuda(*num_replicas, "moe_dispatch", "num_replicas");
    TORCH_CHECK(expert_slots->dim() == 2 && expert_slots->size(0) == num_experts &&
                    num_replicas->numel() == num_experts,
                "moe_dispatch: expert_slots [E, max_replicas], num_replicas [E]");
    max_rep = expert_slots->size(1);
  }
  if (overflow) {
    check_i32_cuda(*overflow, "moe_dispatch", "overflow");
    TORCH_CHECK(overflow->numel() >= 2, "moe_dispatch: overflow must hold 2 counters");
  }
  if (tokens == 0) return {pos, ids, wts};
  auto recv = as_pointers(peer_recv), cnt = as_pointers(peer_counts);
  check_status(b200ops_moe_dispatch(
                   x.data_ptr(), router_weight ? router_weight->data_ptr() : nullptr,
                   router_weight ? nullptr : ids.data_ptr<int32_t>(),
                   router_weight ? ids.data_ptr<int32_t>() : nullptr, router_weight ? wts.data_ptr<float>() : nullptr,
                   expert_slots ? expert_slots->data_ptr<int32_t>() : nullptr,
                   num_replicas ? num_replicas->data_ptr<int32_t>() : nullptr, max_rep, token_offset,
                   pos.data_ptr<int32_t>(), recv.data(), cnt.data(), cursor.data_ptr<int32_t>(),
                   state.data_ptr(), overflow ? overflow->data_ptr<int32_t>() : nullptr, tokens, x.size(1),
                   num_experts, top_k, num_slots, world, cap, my_rank, current_stream()),
               "moe_dispatch");
  return {pos, ids, wts};
}

// Receiving side of the fused step (see b200ops_moe_gather): returns (grouped rows [max_rows, H],
// grouped_to_received [max_rows], group_list [slots_per_rank], total [1]).
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> moe_gather(at::Tensor recv, at::Tensor counts,
                                                                     at::Tensor state,
                                                                     c10::optional<at::Tensor> overflow,
                                                                     int64_t cap, int64_t max_rows) {
  TORCH_CHECK(recv.dim() == 2 && recv.is_contiguous(), "moe_gather: recv must be contiguous [rows, H]");
  check_f16_cuda(recv, "moe_gather", "recv");
  check_i32_cuda(counts, "moe_gather", "counts");
  TORCH_CHECK(counts.dim() == 2, "moe_gather: counts must be [world, slots_per_rank]");
  TORCH_CHECK(state.is_cuda() && state.element_size() == 4 && state.numel() >= 5,
              "moe_gather: state [5] must be a 32-bit CUDA tensor");
  const int64_t world = counts.size(0), spr = counts.size(1);
  TORCH_CHECK(recv.size(0) >= world * spr * cap, "moe_gather: recv holds fewer than world * slots * cap rows");
  const c10::cuda::CUDAGuard guard(recv.device());
  at::Tensor grouped = at::empty({max_rows, recv.size(1)}, recv.options());
  at::Tensor map = at::empty({max_rows}, recv.options().dtype(at::kInt));
  at::Tensor gl = at::empty({spr}, recv.options().dtype(at::kLong));
  at::Tensor total = at::empty({1}, recv.options().dtype(at::kInt));
  check_status(b200ops_moe_gather(recv.data_ptr(), counts.data_ptr(), state.data_ptr(),
                                  overflow ? overflow->data_ptr<int32_t>() : nullptr, grouped.data_ptr(),
                                  map.data_ptr<int32_t>(), gl.data_ptr<int64_t>(), total.data_ptr<int32_t>(),
                                  recv.size(1), world, spr, cap, max_rows, current_stream()),
               "moe_gather");
  return {grouped, map, gl, total};
}

// Last launch of the fused step (see b200ops_moe_combine).
at::Tensor moe_combine(at::Tensor returned, at::Tensor slot_to_row, at::Tensor expert_weights,
                       std::vector<int64_t> peer_flags, at::Tensor my_flags, at::Tensor state, int64_t my_rank) {
  TORCH_CHECK(returned.dim() == 2 && returned.is_contiguous() && expert_weights.dim() == 2 &&
                  expert_weights.is_contiguous() && slot_to_row.numel() == expert_weights.numel(),
              "moe_combine: returned [R, H], expert_weights [T, k], slot_to_row [T*k]");
  check_f16_cuda(returned, "moe_combine", "returned");
  check_i32_cuda(slot_to_row, "moe_combine", "slot_to_row");
  TORCH_CHECK(expert_weights.is_cuda() && expert_weights.scalar_type() == at::kFloat,
              "moe_combine: expert_weights must be a CUDA float32 tensor");
  TORCH_CHECK(my_flags.is_cuda() && my_flags.element_size() == 4 &&
                  my_flags.numel() >= static_cast<int64_t>(peer_flags.size()) && state.is_cuda() &&
                  state.element_size() == 4 && state.numel() >= 5,
              "moe_combine: flags [world] and state [5] must be 32-bit CUDA tensors");
  const c10::cuda::CUDAGuard guard(returned.device());
  at::Tensor y = at::empty({expert_weights.size(0), returned.size(1)}, returned.options());
  if (expert_weights.size(0) == 0) return y;
  auto flg = as_pointers(peer_flags);
  check_status(b200ops_moe_combine(returned.data_ptr(), slot_to_row.data_ptr<int32_t>(),
                                   expert_weights.data_ptr<float>(), y.data_ptr(), flg.data(), my_flags.data_ptr(),
                                   state.data_ptr(), expert_weights.size(0), expert_weights.size(1),
                                   returned.size(1), static_cast<int64_t>(flg.size()), my_rank, current_stream()),
               "moe_combine");
  return y;
}

void init_ffi_moe(py::module_&& m) {
  m.def("dispatch", &moe_dispatch, py::arg("x"), py::arg("router_weight"), py::arg("expert_ids"), py::arg("top_k"),
        py::arg("expert_slots"), py::arg("num_replicas"), py::arg("token_offset"), py::arg("peer_recv"),
        py::arg("peer_counts"), py::arg("cursor"), py::arg("state"), py::arg("overflow"),
        py::arg("num_experts"), py::arg("cap"), py::arg("my_rank"));
  m.def("gather", &moe_gather, py::arg("recv"), py::arg("counts"), py::arg("state"),
        py::arg("overflow"), py::arg("cap"), py::arg("max_rows"));
  m.def("combine", &moe_combine);
  m.def("push_rows", &moe_push_rows, py::arg("src"), py::arg("index"), py::arg("src_div"),
        py::arg("n_valid"), py::arg("n_max"), py::arg("peer_rows"), py::arg("cap"), py::arg("my_rank"),
        py::arg("counts") = py::none(), py::arg("peer_counts") = std::vector<int64_t>());
  m.def("peer_barrier", &peer_barrier);
  m.def("grouped_matmul_scatter", &grouped_matmul_scatter);
  m.def("grouped_matmul_swiglu", &grouped_matmul_swiglu);
  m.def("fused_qkv_rope_cache", &fused_qkv_rope_cache, py::arg("qkv"), py::arg("position_ids"),
        py::arg("cos_cache"), py::arg("sin_cache"), py::arg("slot_indices"), py::arg("key_cache"),
        py::arg("value_cache"), py::arg("num_heads"), py::arg("num_kv_heads"),
        py::arg("q_norm_weight") = py::none(), py::arg("k_norm_weight") = py::none(),
        py::arg("epsilon") = 1e-6);
  m.def("route_topk", &moe_route_topk);
  m.def("permute", &moe_permute);
  m.def("ep_plan", &moe_ep_plan);
  m.def("copy_rows", &moe_copy_rows, py::arg("dst"), py::arg("src"), py::arg("dst_index") = py::none(),
        py::arg("src_index") = py::none(), py::arg("src_div") = 1, py::arg("n_valid") = py::none(),
        py::arg("n_max") = 0);
  m.def("finalize", &moe_finalize);
}

void init_ffi_ops(py::module_&& m) {
  m.def("rope", &rope, "Rope");
  m.def("swiglu", &swiglu, "Swiglu");
  m.def("grouped_matmul", &grouped_matmul, "GroupedMatMul");
  m.def("add_rms_norm", &add_rms_norm, "AddRMSNorm");
  m.def("reshape_and_cache", &reshape_and_cache, "ReshapeAndCache");
  m.def("paged_attention", &paged_attention, "PagedAttention");
  m.def("matmul", &matmul, "MatMul (dense NT product of the reference's earlier interface)");
}

}  // namespace native

// The reference's earlier interface also registers its operators with the dispatcher
// (TORCH_LIBRARY(ascend910a, ...), _csrc/ffi.cpp:473-482): torch.ops.ascend910a.{swiglu,
// grouped_matmul, matmul}.  Same schemas here, bound to the CUDA key.
TORCH_LIBRARY(ascend910a, m) {
  m.def("swiglu(Tensor x) -> Tensor");
  m.def("grouped_matmul(Tensor x, Tensor w, Tensor group_list) -> Tensor");
  m.def("matmul(Tensor x, Tensor w) -> Tensor");
}

TORCH_LIBRARY_IMPL(ascend910a, CUDA, m) {
  m.impl("swiglu", &native::swiglu);
  m.impl("grouped_matmul", &native::grouped_matmul);
  m.impl("matmul", &native::matmul);
}

PYBIND11_MODULE(ascend910a_extras_C, m) {
  m.def("print_info", &native::print_info, "Print info about the device");
  native::init_ffi_ops(m.def_submodule("ops"));
  native::init_ffi_moe(m.def_submodule("moe"));
}
