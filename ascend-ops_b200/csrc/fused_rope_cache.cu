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
//
// Optionally the per-head RMSNorm that Qwen3-style layers apply to q and k between the split
// and the rotary embedding (csrc/ffi/graph.cpp:252-255: add_rmsnorm on q [T, Hq, D] and
// k [T, Hkv, D] with a [D] weight, then add_rope) is applied on the way: the D/16 threads that
// hold one head reduce its sum of squares with shuffles, and the normalised values are rounded
// to fp16 before the rotation, as the stand-alone operator would have stored them.
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
  const __half* q_norm_w;  // [D] or nullptr: RMSNorm weights of the query / key heads
  const __half* k_norm_w;
  float eps, inv_dim;
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
  // No early return: with the norm switched on, the lanes of a head reduce with shuffles, so
  // every lane of the warp stays (threads past the end work on the last item and store nothing).
  pdl_trigger();
  pdl_wait();
  const uint32_t raw_item = blockIdx.x * kThreads + threadIdx.x;
  const bool valid = raw_item < p.total_items;
  const uint32_t item = valid ? raw_item : p.total_items - 1;
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
  if (p.q_norm_w != nullptr || p.k_norm_w != nullptr) {
    // vecs_per_half is a power of two <= 32 here (host check) and heads start at multiples of
    // it, so the lanes of one head are an aligned group of the warp.
    uint32_t* xs = reinterpret_cast<uint32_t*>(&xv);
    uint32_t* ys = reinterpret_cast<uint32_t*>(&yv);
    float sumsq = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 xf = h2_to_f2(xs[i]);
      const float2 yf = h2_to_f2(ys[i]);
      sumsq += xf.x * xf.x + xf.y * xf.y + yf.x * yf.x + yf.y * yf.y;
    }
    for (uint32_t m = p.vecs_per_half >> 1; m > 0; m >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, m);
    const __half* w = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
    if (w != nullptr) {
      const float inv_rms = 1.0f / sqrtf(sumsq * p.inv_dim + p.eps);
      const uint4 wx = __ldg(reinterpret_cast<const uint4*>(w) + j);
      const uint4 wy = __ldg(reinterpret_cast<const uint4*>(w) + j + p.vecs_per_half);
      const uint32_t* wxs = reinterpret_cast<const uint32_t*>(&wx);
      const uint32_t* wys = reinterpret_cast<const uint32_t*>(&wy);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 xf = h2_to_f2(xs[i]), yf = h2_to_f2(ys[i]);
        const float2 wxf = h2_to_f2(wxs[i]), wyf = h2_to_f2(wys[i]);
        xs[i] = f2_to_h2(xf.x * inv_rms * wxf.x, xf.y * inv_rms * wxf.y);
        ys[i] = f2_to_h2(yf.x * inv_rms * wyf.x, yf.y * inv_rms * wyf.y);
      }
    }
  }
  if (!valid) return;
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
  return b200ops_fused_qkv_norm_rope_cache(qkv, nullptr, nullptr, 0.f, position_ids, cos_cache, sin_cache,
                                           slot_indices, q_out, key_cache, value_cache, num_tokens, num_heads,
                                           num_kv_heads, head_dim, max_pos, cache_dims, layout, stream);
}

extern "C" int b200ops_fused_qkv_norm_rope_cache(const void* qkv, const void* q_norm_weight,
                                                 const void* k_norm_weight, float eps,
                                                 const int32_t* position_ids, const void* cos_cache,
                                                 const void* sin_cache, const int32_t* slot_indices,
                                                 void* q_out, void* key_cache, void* value_cache,
                                                 int64_t num_tokens, int64_t num_heads, int64_t num_kv_heads,
                                                 int64_t head_dim, int64_t max_pos, const int64_t cache_dims[4],
                                                 int layout, void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0 && head_dim > 0 && max_pos >= 0,
                  "fused_qkv_rope_cache: bad shape tokens=%lld heads=%lld kv_heads=%lld head_dim=%lld",
                  (long long)num_tokens, (long long)num_heads, (long long)num_kv_heads, (long long)head_dim);
  B200OPS_REQUIRE(head_dim % 16 == 0, "fused_qkv_rope_cache: head_dim must be a multiple of 16, got %lld",
                  (long long)head_dim);
  if (q_norm_weight != nullptr || k_norm_weight != nullptr) {
    const int64_t v = head_dim / 16;
    B200OPS_REQUIRE(v <= 32 && (v & (v - 1)) == 0,
                    "fused_qkv_rope_cache: the q/k norm needs head_dim in {16, 32, 64, 128, 256, 512}, got %lld",
                    (long long)head_dim);
    B200OPS_REQUIRE((!q_norm_weight || aligned16(q_norm_weight)) && (!k_norm_weight || aligned16(k_norm_weight)),
                    "fused_qkv_rope_cache: norm weights must be 16-byte aligned");
  }
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
  p.q_norm_w = static_cast<const __half*>(q_norm_weight);
  p.k_norm_w = static_cast<const __half*>(k_norm_weight);
  p.eps = eps;
  p.inv_dim = 1.0f / static_cast<float>(head_dim);
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
  B200OPS_CUDA(launch_kernel(fused_qkv_rope_cache_kernel, dim3(grid), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), p));
  return B200OPS_OK;
}
