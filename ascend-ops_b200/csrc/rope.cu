// Rotary position embedding (half-split / "neox" form) for sm_100a, q and k in one launch.
//
// Per head h = [x | y] (two halves of head_dim/2):  out_x = x*cos - y*sin,  out_y = y*cos + x*sin
// with cos/sin = cache[position] -- the arithmetic of the reference kernel
// (csrc/opdev/op_kernel/rope_ex.cpp:88-108) and of its golden `fn_naive`
// (benchmark/test_graph.py:347-367).  The reference evaluates this in fp16 vector ops
// (three roundings); here the products and the sum are fp32 and the result is rounded once.
// HBM-bound: 4*T*(Hq+Hkv)*D bytes of q/k traffic plus one cos and one sin row per token.
#include "common.cuh"

namespace b200ops {
namespace {

constexpr int kThreads = 256;

// One work item = one 128-bit vector of the x half and the matching vector of the y half
// of one head of one token.
__global__ void __launch_bounds__(kThreads)
rope_kernel(const __half* __restrict__ q, const __half* __restrict__ k,
            const int32_t* __restrict__ position_ids, const __half* __restrict__ cos_cache,
            const __half* __restrict__ sin_cache, __half* __restrict__ out_q,
            __half* __restrict__ out_k, uint32_t total_items, uint32_t items_per_token,
            uint32_t vecs_per_half, uint32_t num_heads, uint32_t num_kv_heads, int max_pos) {
  pdl_trigger();
  pdl_wait();
  const uint32_t item = blockIdx.x * kThreads + threadIdx.x;
  if (item >= total_items) return;
  const uint32_t token = item / items_per_token;
  const uint32_t rem = item - token * items_per_token;
  const uint32_t head = rem / vecs_per_half;
  const uint32_t j = rem - head * vecs_per_half;

  const bool is_q = head < num_heads;
  const uint32_t vecs_per_head = 2 * vecs_per_half;
  const size_t head_vec =
      is_q ? (static_cast<size_t>(token) * num_heads + head) * vecs_per_head
           : (static_cast<size_t>(token) * num_kv_heads + (head - num_heads)) * vecs_per_head;
  const uint4* in = reinterpret_cast<const uint4*>(is_q ? q : k) + head_vec;
  uint4* out = reinterpret_cast<uint4*>(is_q ? out_q : out_k) + head_vec;

  const int pos = position_ids[token];
  if (pos < 0 || pos >= max_pos) {
    out[j] = make_uint4(0, 0, 0, 0);
    out[j + vecs_per_half] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4 xv = ld_stream(in + j);
  const uint4 yv = ld_stream(in + j + vecs_per_half);
  const size_t cs = static_cast<size_t>(pos) * vecs_per_half + j;
  const uint4 cv = __ldg(reinterpret_cast<const uint4*>(cos_cache) + cs);
  const uint4 sv = __ldg(reinterpret_cast<const uint4*>(sin_cache) + cs);

  const uint32_t* xs = reinterpret_cast<const uint32_t*>(&xv);
  const uint32_t* ys = reinterpret_cast<const uint32_t*>(&yv);
  const uint32_t* cs32 = reinterpret_cast<const uint32_t*>(&cv);
  const uint32_t* ss32 = reinterpret_cast<const uint32_t*>(&sv);
  uint4 ox, oy;
  uint32_t* oxs = reinterpret_cast<uint32_t*>(&ox);
  uint32_t* oys = reinterpret_cast<uint32_t*>(&oy);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 xf = h2_to_f2(xs[i]);
    const float2 yf = h2_to_f2(ys[i]);
    const float2 cf = h2_to_f2(cs32[i]);
    const float2 sf = h2_to_f2(ss32[i]);
    oxs[i] = f2_to_h2(xf.x * cf.x - yf.x * sf.x, xf.y * cf.y - yf.y * sf.y);
    oys[i] = f2_to_h2(yf.x * cf.x + xf.x * sf.x, yf.y * cf.y + xf.y * sf.y);
  }
  st_stream(out + j, ox);
  st_stream(out + j + vecs_per_half, oy);
}

}  // namespace
}  // namespace b200ops

extern "C" int b200ops_rope(const void* q, const void* k, const int32_t* position_ids,
                            const void* cos_cache, const void* sin_cache, void* out_q,
                            void* out_k, int64_t bs, int64_t num_heads, int64_t num_kv_heads,
                            int64_t head_dim, int64_t max_pos, void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(bs >= 0 && num_heads >= 0 && num_kv_heads >= 0 && head_dim > 0 && max_pos >= 0,
                  "rope: bad shape bs=%lld heads=%lld kv_heads=%lld head_dim=%lld max_pos=%lld",
                  (long long)bs, (long long)num_heads, (long long)num_kv_heads,
                  (long long)head_dim, (long long)max_pos);
  B200OPS_REQUIRE(head_dim % 16 == 0, "rope: head_dim must be a multiple of 16, got %lld",
                  (long long)head_dim);
  if (bs == 0 || num_heads + num_kv_heads == 0) return B200OPS_OK;
  B200OPS_REQUIRE(position_ids && cos_cache && sin_cache, "rope: null pointer");
  B200OPS_REQUIRE((num_heads == 0 || (q && out_q)) && (num_kv_heads == 0 || (k && out_k)),
                  "rope: null pointer");
  B200OPS_REQUIRE(aligned16(q) && aligned16(k) && aligned16(cos_cache) && aligned16(sin_cache) &&
                      aligned16(out_q) && aligned16(out_k),
                  "rope: pointers must be 16-byte aligned");
  B200OPS_REQUIRE(max_pos <= 0x7fffffffLL, "rope: cache too long");

  const int64_t vecs_per_half = head_dim / 16;
  const int64_t items_per_token = (num_heads + num_kv_heads) * vecs_per_half;
  const int64_t total = bs * items_per_token;
  B200OPS_REQUIRE(total < 0x7fffff00LL, "rope: tensor too large");
  const unsigned grid = static_cast<unsigned>((total + kThreads - 1) / kThreads);
  B200OPS_CUDA(launch_kernel(rope_kernel, dim3(grid), dim3(kThreads), 0, static_cast<cudaStream_t>(stream),
                      static_cast<const __half*>(q), static_cast<const __half*>(k), position_ids,
                      static_cast<const __half*>(cos_cache), static_cast<const __half*>(sin_cache),
                      static_cast<__half*>(out_q), static_cast<__half*>(out_k), static_cast<uint32_t>(total),
                      static_cast<uint32_t>(items_per_token), static_cast<uint32_t>(vecs_per_half),
                      static_cast<uint32_t>(num_heads), static_cast<uint32_t>(num_kv_heads),
                      static_cast<int>(max_pos)));
  return B200OPS_OK;
}
