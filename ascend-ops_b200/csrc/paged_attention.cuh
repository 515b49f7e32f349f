// Shared definitions of the paged-attention decode kernels (split-context plan, partial
// record layout, combine step).
#pragma once

#include "common.cuh"

namespace b200ops {
namespace pa {

// How one launch cuts the work.  A sequence's context is cut into chunks of
// `chunk_tokens`; one CTA handles one (sequence, kv head, chunk).  Chunk c of sequence b
// exists iff c*chunk_tokens < context_len[b]; CTAs of absent chunks exit at once.
// When a sequence has a single chunk its CTA writes the final fp16 output directly;
// otherwise every chunk writes a partial record and the combine kernel merges them.
struct Plan {
  int chunk_tokens;  // multiple of page_size (or of the tile size), > 0
  int max_chunks;    // ceil(max_pages_per_seq * page_size / chunk_tokens)
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
  int bs, num_heads, num_kv_heads, head_dim;
  int num_pages, page_size, max_pages_per_seq;
  int layout;
  int chunk_tokens, max_chunks;
  float scale_log2;  // 1/sqrt(head_dim) * log2(e)
};

Plan make_plan(int64_t bs, int64_t num_kv_heads, int64_t page_size, int64_t max_pages_per_seq);

// Launchers implemented in the .cu files.  Each returns a B200OPS_* code.
int launch_general(const Args& a, cudaStream_t st);
bool fast_path_supported(const Args& a);
int launch_fast(const Args& a, cudaStream_t st);
int launch_combine(const Args& a, cudaStream_t st);

// Persistent tile-balanced path (paged_attention_stream.cu): plan + main + combine in one call.
bool stream_path_supported(const Args& a);
size_t stream_workspace_bytes(int64_t bs, int64_t num_heads, int64_t num_kv_heads, int64_t head_dim);
int launch_stream(const Args& a, void* workspace, cudaStream_t st);

}  // namespace pa
}  // namespace b200ops
