// Fused split + rotary embedding + KV-cache scatter for the decode step.
//
// The reference's decoder layer runs these as separate graph nodes after the QKV projection:
// Split, RopeEx, ReshapeAndCache (csrc/ffi/graph.cpp:207-283).  Done separately on a GPU they
// cost three strided copies (to make q, k, v contiguous) and two more launches that each move
// only a few hundred KB at decode batch sizes.  This kernel reads the projection output
// qkv [T, (Hq + 2*Hkv) * D] once and
//   - writes the rotated q to a contiguous [T, Hq, D] tensor,
//   - writes the rotated k and the untouched v straight into the paged caches at each
//     token's slot (either cache layout).
// Arithmetic and rounding are those of rope.cu followed by reshape_and_cache.cu, so the
// result is bit-identical to calling the two operators in sequence.
#include "common.cuh"

namespace b200ops {
namespace {

constexpr int kThreads = 256;

struct FusedParams {
  const __half* qkv;
  const int32_t* positions;
  const __half* cos_cache;
  const __half* sin_cache;
  const int32_t* slots;
  __half* q_out;
  __half* k_cache;
  __half* v_cache;
  uint32_t total_items, items_per_token, vecs_per_half;
  uint32_t num_heads, num_kv_heads;
  int max_pos;
  int64_t num_slots;
  uint32_t page_size, chunks;
  int layout;
};

// Vector (16 B) index inside a cache of the token's row element `e` (= head * D + d, d % 8 == 0).
__device__ __forceinline__ size_t cache_vec(const FusedParams& p, int64_t slot, uint32_t e,
                                            uint32_t row_elems) {
  if (p.layout == B200OPS_KV_LAYOUT_NHD) return (static_cast<size_t>(slot) * row_elems + e) >> 3;
  const uint32_t page = static_cast<uint32_t>(slot / p.page_size);
  const uint32_t off = static_cast<uint32_t>(slot - static_cast<int64_t>(page) * p.page_size);
  const uint32_t c = e >> 4;
  return ((static_cast<size_t>(page) * p.chunks + c) * p.page_size + off) * 2 + ((e >> 3) & 1u);
}

__global__ void __launch_bounds__(kThreads) fused_qkv_rope_cache_kernel(FusedParams p) {
  const uint32_t item = blockIdx.x * kThreads + threadIdx.x;
  if (item >= p.total_items) return;
  const uint32_t token = item / p.items_per_token;
  const uint32_t rem = item - token * p.items_per_token;
  const uint32_t head = rem / p.vecs_per_half;  // index over Hq + 2*Hkv heads of the qkv row
  const uint32_t j = rem - head * p.vecs_per_half;
  const uint32_t vecs_per_head = 2 * p.vecs_per_half;
  const uint32_t total_heads = p.num_heads + 2 * p.num_kv_heads;
  const uint4* in = reinterpret_cast<const uint4*>(p.qkv) +
                    (static_cast<size_t>(token) * total_heads + head) * vecs_per_head;
  uint4 xv = ld_stream(in + j);
  uint4 yv = ld_stream(in + j + p.vecs_per_half);
  const bool is_q = head < p.num_heads;
  const bool is_k = !is_q && head < p.num_heads + p.num_kv_heads;
  if (is_q || is_k) {
    const int pos = p.positions[token];
    if (pos < 0 || pos >= p.max_pos) {
      xv = make_uint4(0, 0, 0, 0);
      yv = make_uint4(0, 0, 0, 0);
    } else {
      const size_t cs = static_cast<size_t>(pos) * p.vecs_per_half + j;
      const uint4 cv = __ldg(reinterpret_cast<const uint4*>(p.cos_cache) + cs);
      const uint4 sv = __ldg(reinterpret_cast<const uint4*>(p.sin_cache) + cs);
      uint32_t* xs = reinterpret_cast<uint32_t*>(&xv);
      uint32_t* ys = reinterpret_cast<uint32_t*>(&yv);
      const uint32_t* c32 = reinterpret_cast<const uint32_t*>(&cv);
      const uint32_t* s32 = reinterpret_cast<const uint32_t*>(&sv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 xf = h2_to_f2(xs[i]);
        const float2 yf = h2_to_f2(ys[i]);
        const float2 cf = h2_to_f2(c32[i]);
        const float2 sf = h2_to_f2(s32[i]);
        xs[i] = f2_to_h2(xf.x * cf.x - yf.x * sf.x, xf.y * cf.y - yf.y * sf.y);
        ys[i] = f2_to_h2(yf.x * cf.x + xf.x * sf.x, yf.y * cf.y + xf.y * sf.y);
      }
    }
  }
  if (is_q) {
    uint4* out = reinterpret_cast<uint4*>(p.q_out) +
                 (static_cast<size_t>(token) * p.num_heads + head) * vecs_per_head;
    out[j] = xv;
    out[j + p.vecs_per_half] = yv;
    return;
  }
  const int64_t slot = p.slots[token];
  if (slot < 0 || slot >= p.num_slots) return;
  const uint32_t kvh = is_k ? head - p.num_heads : head - p.num_heads - p.num_kv_heads;
  const uint32_t head_dim = vecs_per_head * 8;
  const uint32_t row_elems = p.num_kv_heads * head_dim;
  uint4* cache = reinterpret_cast<uint4*>(is_k ? p.k_cache : p.v_cache);
  const uint32_t e0 = kvh * head_dim + j * 8;
  cache[cache_vec(p, slot, e0, row_elems)] = xv;
  cache[cache_vec(p, slot, e0 + head_dim / 2, row_elems)] = yv;
}

}  // namespace
}  // namespace b200ops

extern "C" int b200ops_fused_qkv_rope_cache(const void* qkv, const int32_t* position_ids,
                                            const void* cos_cache, const void* sin_cache,
                                            const int32_t* slot_indices, void* q_out, void* key_cache,
                                            void* value_cache, int64_t num_tokens, int64_t num_heads,
                                            int64_t num_kv_heads, int64_t head_dim, int64_t max_pos,
                                            const int64_t cache_dims[4], int layout, void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0 && head_dim > 0 && max_pos >= 0,
                  "fused_qkv_rope_cache: bad shape tokens=%lld heads=%lld kv_heads=%lld head_dim=%lld",
                  (long long)num_tokens, (long long)num_heads, (long long)num_kv_heads, (long long)head_dim);
  B200OPS_REQUIRE(head_dim % 16 == 0, "fused_qkv_rope_cache: head_dim must be a multiple of 16, got %lld",
                  (long long)head_dim);
  B200OPS_REQUIRE(cache_dims != nullptr, "fused_qkv_rope_cache: cache_dims is null");
  B200OPS_REQUIRE(layout == B200OPS_KV_LAYOUT_NZ || layout == B200OPS_KV_LAYOUT_NHD,
                  "fused_qkv_rope_cache: unknown cache layout %d", layout);
  int64_t page_size, chunks = 0;
  if (layout == B200OPS_KV_LAYOUT_NZ) {
    B200OPS_REQUIRE(cache_dims[3] == 16 && cache_dims[1] * 16 == num_kv_heads * head_dim,
                    "fused_qkv_rope_cache: NZ cache must be [pages, Hkv*D/16, page_size, 16]");
    chunks = cache_dims[1];
    page_size = cache_dims[2];
  } else {
    B200OPS_REQUIRE(cache_dims[2] == num_kv_heads && cache_dims[3] == head_dim,
                    "fused_qkv_rope_cache: NHD cache must be [pages, page_size, Hkv, D]");
    page_size = cache_dims[1];
  }
  B200OPS_REQUIRE(cache_dims[0] > 0 && page_size > 0 && page_size < (1LL << 31) && max_pos < (1LL << 31),
                  "fused_qkv_rope_cache: bad cache shape");
  if (num_tokens == 0) return B200OPS_OK;
  B200OPS_REQUIRE(qkv && position_ids && cos_cache && sin_cache && slot_indices && q_out && key_cache && value_cache,
                  "fused_qkv_rope_cache: null pointer");
  B200OPS_REQUIRE(aligned16(qkv) && aligned16(cos_cache) && aligned16(sin_cache) && aligned16(q_out) &&
                      aligned16(key_cache) && aligned16(value_cache),
                  "fused_qkv_rope_cache: pointers must be 16-byte aligned");
  FusedParams p;
  p.qkv = static_cast<const __half*>(qkv);
  p.positions = position_ids;
  p.cos_cache = static_cast<const __half*>(cos_cache);
  p.sin_cache = static_cast<const __half*>(sin_cache);
  p.slots = slot_indices;
  p.q_out = static_cast<__half*>(q_out);
  p.k_cache = static_cast<__half*>(key_cache);
  p.v_cache = static_cast<__half*>(value_cache);
  p.vecs_per_half = static_cast<uint32_t>(head_dim / 16);
  p.num_heads = static_cast<uint32_t>(num_heads);
  p.num_kv_heads = static_cast<uint32_t>(num_kv_heads);
  p.items_per_token = static_cast<uint32_t>((num_heads + 2 * num_kv_heads) * p.vecs_per_half);
  const int64_t total = num_tokens * p.items_per_token;
  B200OPS_REQUIRE(total < 0x7fffff00LL, "fused_qkv_rope_cache: tensor too large");
  p.total_items = static_cast<uint32_t>(total);
  p.max_pos = static_cast<int>(max_pos);
  p.num_slots = cache_dims[0] * page_size;
  p.page_size = static_cast<uint32_t>(page_size);
  p.chunks = static_cast<uint32_t>(chunks);
  p.layout = layout;
  const unsigned grid = static_cast<unsigned>((total + kThreads - 1) / kThreads);
  fused_qkv_rope_cache_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  B200OPS_LAUNCH_CHECK("fused_qkv_rope_cache");
  return B200OPS_OK;
}
