// Paged-attention decode for sm_100a: C-ABI entry, split-context plan, the general kernel
// (any cache layout, head_dim in {32,64,128,256}, any GQA ratio) and the combine kernel.
//
// Semantics (the reference's kernel is unfinished, so these come from its interface and
// tiling code): one query token per sequence; query head h reads kv head h / (Hq/Hkv)
// (csrc/opdev/op_kernel/paged_attention_ex.cpp:91-95); scale = 1/sqrt(head_dim) and the
// exponentials are taken base 2 with scale*log2(e) folded in
// (csrc/opdev/op_host/paged_attention_ex.cpp:26-27); pages are found through
// block_tables[b, i] (paged_attention_ex.cpp:129-137); only the first context_lens[b]
// tokens count.  Scores, softmax and the PV sum are fp32; the output is rounded once.
#include "paged_attention.cuh"

#include <atomic>
#include <cmath>

namespace b200ops {
namespace pa {
namespace {

constexpr int kWarps = 4;
constexpr int kHeadTile = 8;   // query heads of one kv head handled per CTA
constexpr int kTokUnroll = 4;  // tokens whose K/V loads are in flight per warp

template <int N>
struct HalfVec;
template <>
struct HalfVec<1> { unsigned short v; };
template <>
struct HalfVec<2> { uint32_t v; };
template <>
struct HalfVec<4> { uint2 v; };
template <>
struct HalfVec<8> { uint4 v; };

template <int DPL>
__device__ __forceinline__ void unpack(const HalfVec<DPL>& in, float* out) {
  const __half* h = reinterpret_cast<const __half*>(&in);
#pragma unroll
  for (int i = 0; i < DPL; ++i) out[i] = __half2float(h[i]);
}

// Element offset of (page, off, kv head, d) in either cache layout.
__device__ __forceinline__ size_t kv_offset(int layout, int page, int off, int head, int d,
                                            int page_size, int num_kv_heads, int head_dim) {
  if (layout == B200OPS_KV_LAYOUT_NHD) {
    return ((static_cast<size_t>(page) * page_size + off) * num_kv_heads + head) * head_dim + d;
  }
  const int e = head * head_dim + d;
  const size_t chunks = static_cast<size_t>(num_kv_heads) * head_dim / 16;
  return ((static_cast<size_t>(page) * chunks + (e >> 4)) * page_size + off) * 16 + (e & 15);
}

// General kernel: a warp owns whole tokens, lane i owns DPL = head_dim/32 consecutive
// channels.  grid = (max_chunks, num_kv_heads * head_tiles, bs).
template <int DPL>
__global__ void __launch_bounds__(kWarps * 32) paged_attention_general_kernel(Args a) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int D = a.head_dim;
  const int chunk = blockIdx.x;
  const int group = a.num_heads / a.num_kv_heads;
  const int head_tiles = (group + kHeadTile - 1) / kHeadTile;
  const int kvh = blockIdx.y / head_tiles;
  const int tile = blockIdx.y - kvh * head_tiles;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  int L = a.context_lens[b];
  const int cap = a.max_pages_per_seq * a.page_size;
  if (L > cap) L = cap;
  const int h0 = kvh * group + tile * kHeadTile;           // first query head of this CTA
  const int nh = min(kHeadTile, group - tile * kHeadTile);  // query heads of this CTA
  if (L <= 0) {
    if (chunk == 0)
      for (int i = threadIdx.x; i < nh * D; i += blockDim.x)
        a.out[(static_cast<size_t>(b) * a.num_heads + h0) * D + i] = __float2half(0.f);
    return;
  }
  const int ct = seq_chunk_tokens(a.chunk_tokens, a.max_chunks, a.chunk_align, L);
  const int start = chunk * ct;
  if (start >= L) return;
  const int end = min(L, start + ct);
  const int n_chunks = (L + ct - 1) / ct;

  float qf[kHeadTile][DPL];
#pragma unroll
  for (int g = 0; g < kHeadTile; ++g) {
#pragma unroll
    for (int i = 0; i < DPL; ++i)
      qf[g][i] = (g < nh) ? __half2float(a.q[(static_cast<size_t>(b) * a.num_heads + h0 + g) * D +
                                              lane * DPL + i]) * a.scale_log2
                          : 0.f;
  }
  float m[kHeadTile], l[kHeadTile], acc[kHeadTile][DPL];
#pragma unroll
  for (int g = 0; g < kHeadTile; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
  }

  const int32_t* table = a.block_tables + static_cast<size_t>(b) * a.max_pages_per_seq;
  for (int t0 = start + warp * kTokUnroll; t0 < end; t0 += kWarps * kTokUnroll) {
    HalfVec<DPL> kv[kTokUnroll], vv[kTokUnroll];
    bool ok[kTokUnroll];
#pragma unroll
    for (int j = 0; j < kTokUnroll; ++j) {
      const int t = t0 + j;
      ok[j] = t < end;
      if (ok[j]) {
        const int page = table[t / a.page_size];
        ok[j] = page >= 0 && page < a.num_pages;
        if (ok[j]) {
          const size_t o = kv_offset(a.layout, page, t % a.page_size, kvh, lane * DPL,
                                     a.page_size, a.num_kv_heads, D);
          kv[j] = *reinterpret_cast<const HalfVec<DPL>*>(a.k_cache + o);
          vv[j] = *reinterpret_cast<const HalfVec<DPL>*>(a.v_cache + o);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kTokUnroll; ++j) {
      if (!ok[j]) continue;  // warp-uniform
      float kf[DPL], vf[DPL];
      unpack<DPL>(kv[j], kf);
      unpack<DPL>(vv[j], vf);
#pragma unroll
      for (int g = 0; g < kHeadTile; ++g) {
        if (g >= nh) break;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) s = fmaf(qf[g][i], kf[i], s);
        s = warp_sum(s);
        const float m_new = fmaxf(m[g], s);
        const float alpha = exp2f(m[g] - m_new);  // exp2(-inf) = 0 on the first token
        const float p = exp2f(s - m_new);
        l[g] = l[g] * alpha + p;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] = fmaf(p, vf[i], acc[g][i] * alpha);
        m[g] = m_new;
      }
    }
  }

  // Merge the four warps through shared memory: [warp][head][D + 2].
  const int rec = D + 2;
#pragma unroll
  for (int g = 0; g < kHeadTile; ++g) {
    float* r = smem + (warp * kHeadTile + g) * rec;
#pragma unroll
    for (int i = 0; i < DPL; ++i) r[lane * DPL + i] = acc[g][i];
    if (lane == 0) {
      r[D] = m[g];
      r[D + 1] = l[g];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nh * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, smem[(w * kHeadTile + g) * rec + D]);
    float o = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float* r = smem + (w * kHeadTile + g) * rec;
      const float f = (r[D] == -INFINITY) ? 0.f : exp2f(r[D] - mm);
      o += r[d] * f;
      ll += r[D + 1] * f;
    }
    const int h = h0 + g;
    if (n_chunks == 1) {
      a.out[(static_cast<size_t>(b) * a.num_heads + h) * D + d] =
          __float2half(ll > 0.f ? o / ll : 0.f);
    } else {
      float* pr = a.partials +
                  ((static_cast<size_t>(b) * a.num_heads + h) * a.max_chunks + chunk) * rec;
      pr[d] = o;
      if (d == 0) {
        pr[D] = mm;
        pr[D + 1] = ll;
      }
    }
  }
}

// Combine: one warp per (sequence, query head) merges the chunk partials of sequences that
// were split.  Lanes first take one chunk each for the maximum and the normaliser, then every
// lane sums its channels (lane, lane + 32, ...) over the chunks.
constexpr int kCombineWarps = 4;

__global__ void __launch_bounds__(kCombineWarps * 32) paged_attention_combine_kernel(Args a) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
  if (item >= a.bs * a.num_heads) return;
  const int b = item / a.num_heads;
  int L = a.context_lens[b];
  const int cap = a.max_pages_per_seq * a.page_size;
  if (L > cap) L = cap;
  if (L <= 0) return;
  const int ct = seq_chunk_tokens(a.chunk_tokens, a.max_chunks, a.chunk_align, L);
  const int n_chunks = (L + ct - 1) / ct;
  if (n_chunks <= 1) return;
  combine_head(a, b, item - b * a.num_heads, n_chunks, lane);
}

}  // namespace

// Chunk partials, then one int per (sequence, kv head) for the fused merge.
size_t chunk_partial_bytes(int64_t bs, int64_t num_heads, int64_t head_dim, int max_chunks) {
  if (max_chunks <= 1) return 0;
  const size_t n = static_cast<size_t>(bs) * num_heads * max_chunks * partial_stride((int)head_dim) * sizeof(float);
  return (n + 255) & ~static_cast<size_t>(255);
}

size_t chunk_workspace_bytes(int64_t bs, int64_t num_heads, int64_t num_kv_heads, int64_t head_dim,
                             int max_chunks) {
  const size_t partials = chunk_partial_bytes(bs, num_heads, head_dim, max_chunks);
  return partials == 0 ? 0 : partials + static_cast<size_t>(bs) * num_kv_heads * sizeof(int);
}

Plan make_plan(int64_t bs, int64_t num_kv_heads, int64_t page_size, int64_t max_pages_per_seq) {
  // Chunk length.  Each CTA pays a fixed start-up (barrier set-up, first TMA round trip) and
  // a merge at the end, so long chunks stream best: measured on B200 at 256 (sequence, head)
  // pairs, 2048-token chunks reach 5.1 TB/s where 256-token chunks reach 3.7 TB/s.  Short
  // batches need more, smaller chunks to occupy the SMs.  Lengths are device data, so the
  // capacity of the block table stands in for them: aim at about 4 CTAs per resident slot
  // (148 SMs x 2 CTAs) and clamp to [256, 2048] tokens.
  const int64_t pairs = bs * num_kv_heads;
  const int64_t cap_tokens = max_pages_per_seq * page_size;
  int64_t chunk = (pairs * cap_tokens + 1183) / 1184;
  chunk = chunk < 256 ? 256 : (chunk > 2048 ? 2048 : chunk);
  if (const int v = knob(kKnobPaChunkTokens, 0); v > 0) chunk = v;
  // Chunk lengths are whole pages, so that a chunk never starts inside a page, and (for the TMA
  // path) whole 64-token tiles.
  int64_t align = page_size;
  while (align % 64 != 0 && align < 64 * page_size) align += page_size;
  chunk = (chunk + align - 1) / align * align;
  const int64_t cap = (max_pages_per_seq * page_size + align - 1) / align * align;
  if (chunk > cap && cap > 0) chunk = cap;
  // Chunks per sequence: what the capacity asks for, but no more than keeps about eight CTAs
  // per resident slot busy (and at least 8) -- see the note on block-table capacity in the header
  // -- and no fewer than keeps the longest possible chunk within kMaxChunkPages pages.
  int64_t max_chunks = cap > 0 ? (cap + chunk - 1) / chunk : 1;
  int64_t limit = (2368 + pairs - 1) / (pairs > 0 ? pairs : 1);
  if (limit < 8) limit = 8;
  if (max_chunks > limit) max_chunks = limit;
  while (((cap + max_chunks - 1) / max_chunks + align - 1) / align * align > kMaxChunkPages * page_size) ++max_chunks;
  Plan p;
  p.chunk_tokens = static_cast<int>(chunk);
  p.max_chunks = static_cast<int>(max_chunks);
  p.chunk_align = static_cast<int>(align);
  return p;
}

int launch_general(const Args& a, cudaStream_t st) {
  const int group = a.num_heads / a.num_kv_heads;
  const int head_tiles = (group + kHeadTile - 1) / kHeadTile;
  const dim3 grid(a.max_chunks, a.num_kv_heads * head_tiles, a.bs);
  const size_t smem = static_cast<size_t>(kWarps) * kHeadTile * (a.head_dim + 2) * sizeof(float);
  B200OPS_REQUIRE(grid.y <= 65535 && grid.z <= 65535,
                  "paged_attention: batch or head count too large for one launch");
  const dim3 block(kWarps * 32);
  switch (a.head_dim / 32) {
    case 1: B200OPS_CUDA(launch_kernel(paged_attention_general_kernel<1>, grid, block, smem, st, a)); break;
    case 2: B200OPS_CUDA(launch_kernel(paged_attention_general_kernel<2>, grid, block, smem, st, a)); break;
    case 4: B200OPS_CUDA(launch_kernel(paged_attention_general_kernel<4>, grid, block, smem, st, a)); break;
    case 8: B200OPS_CUDA(launch_kernel(paged_attention_general_kernel<8>, grid, block, smem, st, a)); break;
    default:
      return fail(B200OPS_EUNSUPPORTED, "paged_attention: head_dim %d not in {32,64,128,256}",
                  a.head_dim);
  }
  return B200OPS_OK;
}

int launch_combine(const Args& a, cudaStream_t st) {
  if (a.max_chunks <= 1) return B200OPS_OK;
  const int items = a.bs * a.num_heads;
  B200OPS_CUDA(launch_kernel(paged_attention_combine_kernel, dim3((items + kCombineWarps - 1) / kCombineWarps),
                      dim3(kCombineWarps * 32), 0, st, a));
  return B200OPS_OK;
}

}  // namespace pa
}  // namespace b200ops

extern "C" size_t b200ops_paged_attention_workspace_size(int64_t bs, int64_t num_heads,
                                                         int64_t num_kv_heads, int64_t head_dim,
                                                         int64_t page_size,
                                                         int64_t max_pages_per_seq) {
  using namespace b200ops;
  if (bs <= 0 || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || page_size <= 0 ||
      max_pages_per_seq <= 0)
    return 0;
  // Chunk partials plus one counter per (sequence, kv head); 0 when no sequence can be split.
  const pa::Plan p = pa::make_plan(bs, num_kv_heads, page_size, max_pages_per_seq);
  return pa::chunk_workspace_bytes(bs, num_heads, num_kv_heads, head_dim, p.max_chunks);
}

extern "C" int b200ops_paged_attention(const void* q, const void* key_cache,
                                       const void* value_cache, const int32_t* block_tables,
                                       const int32_t* context_lens, void* out, int64_t bs,
                                       int64_t num_heads, int64_t num_kv_heads, int64_t head_dim,
                                       int64_t num_pages, int64_t page_size,
                                       int64_t max_pages_per_seq, int layout, void* workspace,
                                       size_t workspace_size, void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(bs >= 0 && num_heads > 0 && num_kv_heads > 0 && head_dim > 0,
                  "paged_attention: bad q shape [%lld, %lld, %lld]", (long long)bs,
                  (long long)num_heads, (long long)head_dim);
  B200OPS_REQUIRE(num_heads % num_kv_heads == 0,
                  "paged_attention: num_heads %lld is not a multiple of num_kv_heads %lld",
                  (long long)num_heads, (long long)num_kv_heads);
  B200OPS_REQUIRE(num_pages > 0 && page_size > 0 && max_pages_per_seq > 0,
                  "paged_attention: bad cache shape pages=%lld page_size=%lld max_pages_per_seq=%lld",
                  (long long)num_pages, (long long)page_size, (long long)max_pages_per_seq);
  B200OPS_REQUIRE(layout == B200OPS_KV_LAYOUT_NZ || layout == B200OPS_KV_LAYOUT_NHD,
                  "paged_attention: unknown cache layout %d", layout);
  B200OPS_REQUIRE(head_dim % 32 == 0 && head_dim <= 256,
                  "paged_attention: head_dim must be 32, 64, 128 or 256, got %lld",
                  (long long)head_dim);
  B200OPS_REQUIRE(bs <= 65535 && num_heads <= 4096 && num_pages <= 0x7fffffffLL &&
                      page_size <= (1 << 20) && max_pages_per_seq <= (1 << 24) &&
                      max_pages_per_seq * page_size <= 0x7fffffffLL,
                  "paged_attention: shape too large");
  if (bs == 0) return B200OPS_OK;
  B200OPS_REQUIRE(q && key_cache && value_cache && block_tables && context_lens && out,
                  "paged_attention: null pointer");
  B200OPS_REQUIRE(aligned16(q) && aligned16(key_cache) && aligned16(value_cache) && aligned16(out),
                  "paged_attention: pointers must be 16-byte aligned");

  const pa::Plan plan = pa::make_plan(bs, num_kv_heads, page_size, max_pages_per_seq);
  const size_t need = b200ops_paged_attention_workspace_size(bs, num_heads, num_kv_heads,
                                                             head_dim, page_size,
                                                             max_pages_per_seq);
  if (need > 0 && (workspace == nullptr || workspace_size < need))
    return fail(B200OPS_EWORKSPACE, "paged_attention: workspace of %zu bytes needed, got %zu",
                need, workspace ? workspace_size : (size_t)0);

  pa::Args a;
  a.q = static_cast<const __half*>(q);
  a.k_cache = static_cast<const __half*>(key_cache);
  a.v_cache = static_cast<const __half*>(value_cache);
  a.block_tables = block_tables;
  a.context_lens = context_lens;
  a.out = static_cast<__half*>(out);
  a.partials = static_cast<float*>(workspace);
  a.bs = (int)bs;
  a.num_heads = (int)num_heads;
  a.num_kv_heads = (int)num_kv_heads;
  a.head_dim = (int)head_dim;
  a.num_pages = (int)num_pages;
  a.page_size = (int)page_size;
  a.max_pages_per_seq = (int)max_pages_per_seq;
  a.layout = layout;
  a.chunk_tokens = plan.chunk_tokens;
  a.max_chunks = plan.max_chunks;
  a.chunk_align = plan.chunk_align;
  a.scale_log2 = (1.0f / std::sqrt(static_cast<float>(head_dim))) * 1.44269504088896340736f;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  a.pair_counters = nullptr;
  if (pa::fast_path_supported(a)) {
    // The split-context TMA kernel merges a pair's chunks itself: the CTA that finishes the
    // pair's last outstanding chunk (a counter per pair, zeroed here) does the merge, so no
    // second launch follows.
    if (a.max_chunks > 1) {
      a.pair_counters = reinterpret_cast<int*>(
          static_cast<char*>(workspace) + pa::chunk_partial_bytes(bs, num_heads, head_dim, a.max_chunks));
      B200OPS_CUDA(cudaMemsetAsync(a.pair_counters, 0, static_cast<size_t>(bs) * num_kv_heads * sizeof(int), st));
    }
    return pa::launch_fast(a, st);
  }
  const int rc = pa::launch_general(a, st);
  if (rc != B200OPS_OK) return rc;
  return pa::launch_combine(a, st);
}

// ---------------------------------------------------------------------------------------
// Decode attention for hosts that cannot allocate device memory.
//
// Some embedders hand every byte of HBM to their own arena at start-up (a serving engine
// that sizes its KV cache to "whatever is left after the weights"), or forbid cudaMalloc on
// the request path because it synchronises the device and may fail once memory is
// exhausted.  Such a host has nowhere to get the split-context scratch that
// b200ops_paged_attention() asks for.  This entry point takes the same inputs and outputs
// but keeps the scratch in an array that is part of the library image itself.
namespace b200ops {
namespace pa {
namespace {

constexpr size_t kStaticScratchBytes = B200OPS_PAGED_ATTENTION_STATIC_SCRATCH_BYTES;

// Lives in every CUDA context that loads this library, from load until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// `g_static_scratch` named in host code is only the host-side handle of the symbol, never
// a device address; the address on the current device comes from the runtime, once per device.
// Host threads may race to be first: they look up the same address, and the slot is atomic.
int static_scratch_address(void** out) {
  static std::atomic<void*> address[64];
  int dev = -1;
  B200OPS_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200OPS_EUNSUPPORTED, "paged_attention_static: device index %d", dev);
  void* p = address[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    B200OPS_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    if (p == nullptr) return fail(B200OPS_ECUDA, "paged_attention_static: scratch symbol has no device address");
    address[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return B200OPS_OK;
}

}  // namespace
}  // namespace pa
}  // namespace b200ops

extern "C" int b200ops_paged_attention_static(const void* q, const void* key_cache,
                                              const void* value_cache, const int32_t* block_tables,
                                              const int32_t* context_lens, void* out, int64_t bs,
                                              int64_t num_heads, int64_t num_kv_heads,
                                              int64_t head_dim, int64_t num_pages,
                                              int64_t page_size, int64_t max_pages_per_seq,
                                              int layout, void* stream) {
  using namespace b200ops;
  const size_t need = b200ops_paged_attention_workspace_size(bs, num_heads, num_kv_heads, head_dim,
                                                             page_size, max_pages_per_seq);
  if (need > pa::kStaticScratchBytes)
    return fail(B200OPS_EWORKSPACE,
                "paged_attention_static: this shape needs %zu bytes of scratch but the built-in "
                "array holds %zu; use b200ops_paged_attention with a caller-owned workspace",
                need, pa::kStaticScratchBytes);
  // Looked up on every call, also for shapes that need no scratch: the first call on a device is
  // the documented warm-up that makes the runtime load this module (and claim the array's memory).
  void* scratch = nullptr;
  const int rc = pa::static_scratch_address(&scratch);
  if (rc != B200OPS_OK) return rc;
  // The partial records are fully written by the attention kernel before the combine
  // kernel reads them, so nothing in the array has to start at zero.
  return b200ops_paged_attention(q, key_cache, value_cache, block_tables, context_lens, out, bs,
                                 num_heads, num_kv_heads, head_dim, num_pages, page_size,
                                 max_pages_per_seq, layout, scratch, need > 0 ? pa::kStaticScratchBytes : 0,
                                 stream);
}
