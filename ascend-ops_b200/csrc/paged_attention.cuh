// Shared definitions of the paged-attention decode kernels (split-context plan, partial
// record layout, combine step).
#pragma once

#include "common.cuh"

namespace b200ops {
namespace pa {

// How one launch cuts the work.  A sequence's context is cut into chunks of
// `chunk_tokens`; one CTA handles one (sequence, kv head, chunk).  Chunk c of sequence b
// exists iff c*chunk_tokens < context_len[b]; CTAs of absent chunks exit at once.
// The block table's width is only a capacity (a host that replays CUDA graphs pads it to the
// longest context the model allows), so the chunk count per sequence is capped at
// `max_chunks` whatever the capacity: a sequence that would need more takes proportionally
// longer chunks (seq_chunk_tokens).  Absent-chunk CTAs cost about 0.7 us of an SM slot each; a
// grid sized for a 131072-token capacity made a 104 us call take 142 us.
// When a sequence has a single chunk its CTA writes the final fp16 output directly;
// otherwise every chunk writes a partial record and the combine kernel merges them.
struct Plan {
  int chunk_tokens;  // base chunk length: multiple of chunk_align, > 0
  int max_chunks;    // chunks per sequence never exceed this (= grid extent, record stride)
  int chunk_align;   // chunk lengths are multiples of this: of the page size and of the 64-token tile
};

// Partial record of one (sequence, query head, chunk), fp32:
//   acc[head_dim]  un-normalised sum_t exp2(s_t - m) * v_t
//   m              running maximum of s_t = q.k_t * scale * log2(e)   (-inf if chunk empty)
//   l              sum_t exp2(s_t - m)
// stored at ((b*num_heads + h)*max_chunks + c) * (head_dim + 2) floats.
__host__ __device__ inline size_t partial_stride(int head_dim) { return static_cast<size_t>(head_dim) + 2; }

struct Args {
  const __half* q;
  const __half* k_cache;
  const __half* v_cache;
  const int32_t* block_tables;
  const int32_t* context_lens;
  __half* out;
  float* partials;
  int* pair_counters;  // [bs * num_kv_heads] finished chunks per pair; non-null = the last chunk merges
  int bs, num_heads, num_kv_heads, head_dim;
  int num_pages, page_size, max_pages_per_seq;
  int layout;
  int chunk_tokens, max_chunks, chunk_align;
  float scale_log2;  // 1/sqrt(head_dim) * log2(e)
};

// Block-table entries of one chunk that the TMA kernel keeps in shared memory; the plan makes
// no chunk longer than this many pages.
constexpr int kMaxChunkPages = 1024;

// Chunk length of a sequence of L tokens: the base length, or the shortest multiple of
// chunk_align that covers L in max_chunks chunks.
__host__ __device__ inline int seq_chunk_tokens(int chunk_tokens, int max_chunks, int chunk_align, int L) {
  if (static_cast<long long>(chunk_tokens) * max_chunks >= L) return chunk_tokens;
  const int need = (L + max_chunks - 1) / max_chunks;
  return (need + chunk_align - 1) / chunk_align * chunk_align;
}

#ifdef __CUDACC__
// Merge the n_chunks partial records of (sequence b, query head h) and write the fp16 row.
// One warp.  Lane c keeps the maximum and normaliser of chunk c (further chunks of a very
// long context are folded in by loops); then every lane sums its channels (lane, lane + 32,
// ...) over the chunks, eight chunks per batch so that their loads are all in flight before
// the first one is used: the merge is a chain of L2 round trips, not of bandwidth.  Records
// are read with ld.global.cg because in the fused form other SMs of the same launch wrote them.
// kStaticD is the head dimension when the caller knows it at compile time (0 = read it from
// the arguments, up to 256): a known 128 halves the registers per chunk and doubles the batch.
template <int kStaticD = 0>
__device__ __forceinline__ void combine_head(const Args& a, int b, int h, int n_chunks, int lane) {
  constexpr int kPerLane = kStaticD > 0 ? kStaticD / 32 : 8;
  constexpr int kBatch = 64 / kPerLane;
  const int D = kStaticD > 0 ? kStaticD : a.head_dim;
  const size_t rec = partial_stride(D);
  const size_t item = static_cast<size_t>(b) * a.num_heads + h;
  const float* base = a.partials + item * a.max_chunks * rec;
  float m0 = -INFINITY, l0 = 0.f;
  if (lane < n_chunks) {
    m0 = __ldcg(base + lane * rec + D);
    l0 = __ldcg(base + lane * rec + D + 1);
  }
  float mm = m0;
  for (int c = lane + 32; c < n_chunks; c += 32) mm = fmaxf(mm, __ldcg(base + c * rec + D));
  mm = warp_max(mm);
  float ll = (m0 == -INFINITY) ? 0.f : l0 * exp2f(m0 - mm);
  for (int c = lane + 32; c < n_chunks; c += 32) {
    const float mc = __ldcg(base + c * rec + D);
    if (mc != -INFINITY) ll += __ldcg(base + c * rec + D + 1) * exp2f(mc - mm);
  }
  ll = warp_sum(ll);
  const float inv = ll > 0.f ? 1.0f / ll : 0.f;
  float acc[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) acc[i] = 0.f;
  for (int c0 = 0; c0 < n_chunks; c0 += 32) {
    const int mine = c0 + lane;
    float w = 0.f;
    if (mine < n_chunks) {
      const float mc = c0 == 0 ? m0 : __ldcg(base + mine * rec + D);
      w = (mc == -INFINITY) ? 0.f : exp2f(mc - mm);
    }
    const int n = min(32, n_chunks - c0);
    for (int j0 = 0; j0 < n; j0 += kBatch) {
      float v[kBatch][kPerLane];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const float* p = base + static_cast<size_t>(c0 + min(j0 + u, n - 1)) * rec;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
          const int d = lane + i * 32;
          v[u][i] = d < D ? __ldcg(p + d) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        float wu = __shfl_sync(0xffffffffu, w, (j0 + u) & 31);
        if (j0 + u >= n) wu = 0.f;
        // A chunk of weight zero may hold anything (an empty chunk's sums): select, not multiply.
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) acc[i] = fmaf(wu, wu != 0.f ? v[u][i] : 0.f, acc[i]);
      }
    }
  }
  __half* out = a.out + item * D;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int d = lane + i * 32;
    if (d < D) out[d] = __float2half(acc[i] * inv);
  }
}
#endif

Plan make_plan(int64_t bs, int64_t num_kv_heads, int64_t page_size, int64_t max_pages_per_seq);
size_t chunk_partial_bytes(int64_t bs, int64_t num_heads, int64_t head_dim, int max_chunks);
size_t chunk_workspace_bytes(int64_t bs, int64_t num_heads, int64_t num_kv_heads, int64_t head_dim,
                             int max_chunks);

// Launchers implemented in the .cu files.  Each returns a B200OPS_* code.
int launch_general(const Args& a, cudaStream_t st);
bool fast_path_supported(const Args& a);
int launch_fast(const Args& a, cudaStream_t st);
int launch_combine(const Args& a, cudaStream_t st);

}  // namespace pa
}  // namespace b200ops
