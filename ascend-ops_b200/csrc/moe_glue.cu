// MoE routing glue for sm_100a: the steps on either side of grouped_matmul.
//
// The reference's grouped_matmul takes rows already sorted by expert plus cumulative group
// ends (csrc/opdev/op_kernel/grouped_mat_mul_ex.cpp:29-38); producing that order, and
// undoing it afterwards, is left to its caller (the companion vLLM plugin named in the
// reference's README.md:3, not part of its tree).  These kernels are that caller's work,
// written so that a decode step needs no host synchronisation:
//
//   moe_route_topk     logits = x . Wr^T (fp32 accumulate, rounded to fp16 like a GEMM output),
//                      softmax in fp32, top-k experts and their probabilities per token
//   moe_permute        stable counting sort of the (token, k) slots by expert: destination row
//                      of every slot, per-expert counts, cumulative group ends.  With
//                      `world` > 1 the destination is laid out as one fixed-capacity segment
//                      per destination rank (experts placed contiguously on ranks), the form
//                      an equal-split all-to-all sends
//   moe_ep_plan        on the receiving rank: from every rank's counts, the map from grouped
//                      (expert-major) rows to rows of the received segments, and the local
//                      cumulative group ends
//   moe_copy_rows      dst[di(i)] = src[si(i)] for i < n, the row gather/scatter all of the
//                      above feed
//   moe_finalize       y[t] = sum_k weight[t,k] * rows[pos[t,k]]  (fp32 accumulate, no atomics)
//
// All are bandwidth- or latency-trivial next to the GEMMs; the point is launch count (four
// launches replace about twenty framework index kernels) and device-resident metadata.
#include "common.cuh"

namespace b200ops {
namespace moe {
namespace {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;

// Routing of one token by one CTA, one warp per expert (warps loop when there are more experts
// than warps): every warp forms its expert's dot product with 128-bit loads and kBatch
// independent accumulators, so even a handful of tokens keeps hundreds of loads in flight.
// kBatch 16-byte loads of x and of w are in flight per lane: with 16, a hidden size of 4096 is
// one batch, i.e. one memory round trip per expert, but that needs 128 registers for the loads
// alone, so it is the variant for up to 8 experts (a CTA of at most 256 threads).
// Leaves logits[e] (rounded to fp16 like a GEMM output, clamped to the finite fp16 range so that
// an overflowing dot product or a NaN input cannot turn every probability into NaN) in shared
// memory; the caller synchronises the CTA before route_select.
template <int kBatch>
__device__ __forceinline__ void route_logits(const __half* __restrict__ x, const __half* __restrict__ wr,
                                             float* logits, int token, int hidden, int num_experts) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int vecs = hidden >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(token) * hidden);
  for (int e = warp; e < num_experts; e += warps) {
    const uint4* w = reinterpret_cast<const uint4*>(wr + static_cast<size_t>(e) * hidden);
    float acc[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) acc[u] = 0.f;
    for (int v0 = lane; v0 < vecs; v0 += 32 * kBatch) {
      uint4 a[kBatch], b[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int v = v0 + u * 32;
        if (v < vecs) {
          a[u] = __ldg(xr + v);
          b[u] = __ldg(w + v);
        } else {
          a[u] = make_uint4(0, 0, 0, 0);
          b[u] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const uint32_t* as = reinterpret_cast<const uint32_t*>(&a[u]);
        const uint32_t* bs = reinterpret_cast<const uint32_t*>(&b[u]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = h2_to_f2(as[j]);
          const float2 fb = h2_to_f2(bs[j]);
          acc[u] = fmaf(fa.x, fb.x, acc[u]);
          acc[u] = fmaf(fa.y, fb.y, acc[u]);
        }
      }
    }
    float part = 0.f;
#pragma unroll
    for (int u = 0; u < kBatch; u += 4) part += (acc[u] + acc[u + 1]) + (acc[u + 2] + acc[u + 3]);
    const float dot = warp_sum(part);
    if (lane == 0) {
      float v = fminf(fmaxf(dot, -65504.f), 65504.f);  // fmaxf / fminf drop a NaN operand
      if (!(dot == dot)) v = -65504.f;
      logits[e] = __half2float(__float2half_rn(v));
    }
  }
}

// One warp: softmax over the experts in fp32, then top-k by repeated arg-max (ties go to the
// lower expert index).  Lane 0 stores the choices.
__device__ __forceinline__ void route_select(float* logits, int32_t* __restrict__ ids, float* __restrict__ weights,
                                             int num_experts, int top_k) {
  const int lane = threadIdx.x & 31;
  float mx = -INFINITY;
  for (int e = lane; e < num_experts; e += 32) mx = fmaxf(mx, logits[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < num_experts; e += 32) sum += expf(logits[e] - mx);
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  __syncwarp();
  for (int e = lane; e < num_experts; e += 32) logits[e] = expf(logits[e] - mx) * inv;
  __syncwarp();
  for (int k = 0; k < top_k; ++k) {
    float best = -1.f;
    int best_e = 0x7fffffff;
    for (int e = lane; e < num_experts; e += 32) {
      const float p = logits[e];
      if (p > best) {
        best = p;
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if (best_e >= num_experts) {  // nothing compared greater than -1 (cannot happen with finite logits)
      best_e = k;
      best = 0.f;
    }
    if (lane == 0) {
      ids[k] = best_e;
      weights[k] = best;
      logits[best_e] = -2.f;  // remove from the next round
    }
    __syncwarp();
  }
}

template <int kBatch, int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads)
route_topk_kernel(const __half* __restrict__ x, const __half* __restrict__ wr, int32_t* __restrict__ ids,
                  float* __restrict__ weights, int hidden, int num_experts, int top_k) {
  __shared__ float logits[kMaxExperts];
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  route_logits<kBatch>(x, wr, logits, token, hidden, num_experts);
  __syncthreads();
  if (threadIdx.x >= 32) return;
  route_select(logits, ids + static_cast<size_t>(token) * top_k, weights + static_cast<size_t>(token) * top_k,
               num_experts, top_k);
}

// Single CTA.  Warps own contiguous slices of the flat slot array; a slot's rank inside its
// expert is (slots of lower warps) + (earlier slots of this warp), so the order is the
// stable sort order and does not depend on scheduling.
constexpr int kPermuteThreads = 1024;
constexpr int kPermuteWarps = kPermuteThreads / 32;

__global__ void __launch_bounds__(kPermuteThreads)
permute_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ pos, int32_t* __restrict__ counts,
               int64_t* __restrict__ group_list, int32_t* __restrict__ overflow, int num_slots,
               int num_experts, int experts_per_rank, int segment_rows) {
  extern __shared__ int hist[];  // [kPermuteWarps][num_experts], then base[num_experts], limit[num_experts]
  pdl_trigger();
  pdl_wait();
  int* base = hist + kPermuteWarps * num_experts;
  int* limit = base + num_experts;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kPermuteWarps * num_experts; i += kPermuteThreads) hist[i] = 0;
  __syncthreads();
  const int per_warp = (num_slots + kPermuteWarps - 1) / kPermuteWarps;
  const int lo = min(num_slots, warp * per_warp), hi = min(num_slots, lo + per_warp);
  int* my = hist + warp * num_experts;
  for (int s = lo + lane; s < hi; s += 32) {
    const int e = ids[s];
    if (e >= 0 && e < num_experts) atomicAdd(&my[e], 1);
  }
  __syncthreads();
  // per expert: exclusive scan over warps; totals; segment bases
  for (int e = threadIdx.x; e < num_experts; e += kPermuteThreads) {
    int run = 0;
    for (int w = 0; w < kPermuteWarps; ++w) {
      const int c = hist[w * num_experts + e];
      hist[w * num_experts + e] = run;
      run += c;
    }
    base[e] = run;  // total of expert e for now
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // A destination rank's segment holds at most segment_rows rows (segment_rows == 0: one
    // unbounded segment).  Rows that do not fit are dropped: their slot maps to -1, the count
    // sent to the peers is clamped, and the overflow flag is raised for the caller to act on.
    long long cum = 0;
    int in_segment = 0, dropped = 0;
    for (int e = 0; e < num_experts; ++e) {
      const int c = base[e];
      if (e % experts_per_rank == 0) in_segment = 0;
      int keep = c;
      if (segment_rows > 0) keep = min(c, max(0, segment_rows - in_segment));
      dropped += c - keep;
      base[e] = (e / experts_per_rank) * segment_rows + in_segment;
      limit[e] = base[e] + keep;
      counts[e] = keep;
      in_segment += keep;
      cum += keep;
      group_list[e] = cum;
    }
    if (overflow != nullptr) *overflow = dropped;
  }
  __syncthreads();
  for (int s0 = lo; s0 < hi; s0 += 32) {
    const int s = s0 + lane;
    const bool ok = s < hi;
    int e = ok ? ids[s] : -1;
    if (e < 0 || e >= num_experts) e = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int before = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0) {
      const int p = base[e] + my[e] + before;
      pos[s] = p < limit[e] ? p : -1;
    } else if (ok) {
      pos[s] = -1;
    }
    __syncwarp();
    if (e >= 0 && before == 0) my[e] += __popc(peers);  // leader advances the warp's cursor
    __syncwarp();
  }
}

// Receiving side of the fixed-capacity exchange.  all_counts[r][e] = rows rank r routed to
// expert e.  Rows from rank r arrive in segment r, sorted by (local) expert.  The grouped GEMM
// wants expert-major order: map[d] = received row that supplies grouped row d.
__global__ void __launch_bounds__(256)
ep_plan_kernel(const int32_t* __restrict__ all_counts, int32_t* __restrict__ map,
               int64_t* __restrict__ group_list, int32_t* __restrict__ total_rows, int world,
               int num_experts, int first_expert, int local_experts, int segment_rows) {
  __shared__ int dst_base[64 * 64];  // [local expert][source rank] start in grouped order
  __shared__ int src_base[64 * 64];  // same block's start inside the received buffer
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) {
    int d = 0;
    for (int j = 0; j < local_experts; ++j) {
      for (int r = 0; r < world; ++r) {
        dst_base[j * world + r] = d;
        d += all_counts[r * num_experts + first_expert + j];
      }
      group_list[j] = d;
    }
    *total_rows = d;
    for (int r = 0; r < world; ++r) {
      int s = r * segment_rows;
      for (int j = 0; j < local_experts; ++j) {
        src_base[j * world + r] = s;
        s += all_counts[r * num_experts + first_expert + j];
      }
    }
  }
  __syncthreads();
  for (int blk = 0; blk < local_experts * world; ++blk) {
    const int j = blk / world, r = blk - j * world;
    const int n = all_counts[r * num_experts + first_expert + j];
    for (int i = threadIdx.x; i < n; i += blockDim.x) map[dst_base[blk] + i] = src_base[blk] + i;
  }
}

// dst[di] = src[si] for logical rows i < *n_valid (or n_max if n_valid is null), where
//   si = src_index ? src_index[i] : i, divided by src_div (token = slot / top_k)
//   di = dst_index ? dst_index[i] : i
// Negative indices skip the row.  One CTA per row, 128-bit copies.
__global__ void __launch_bounds__(128)
copy_rows_kernel(__half* __restrict__ dst, const __half* __restrict__ src,
                 const int32_t* __restrict__ dst_index, const int32_t* __restrict__ src_index,
                 int src_div, const int32_t* __restrict__ n_valid, int row_vecs) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  if (n_valid != nullptr && i >= *n_valid) return;
  int si = src_index ? src_index[i] : i;
  const int di = dst_index ? dst_index[i] : i;
  if (si < 0 || di < 0) return;
  si /= src_div;
  const uint4* s = reinterpret_cast<const uint4*>(src) + static_cast<size_t>(si) * row_vecs;
  uint4* d = reinterpret_cast<uint4*>(dst) + static_cast<size_t>(di) * row_vecs;
  for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) d[v] = s[v];
}

__global__ void __launch_bounds__(128)
finalize_kernel(const __half* __restrict__ rows, const int32_t* __restrict__ pos,
                const float* __restrict__ weights, __half* __restrict__ y, int top_k, int row_vecs) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top_k; ++k) {
      const int p = pos[t * top_k + k];
      if (p < 0) continue;
      const float w = weights[t * top_k + k];
      const uint4 r = reinterpret_cast<const uint4*>(rows)[static_cast<size_t>(p) * row_vecs + v];
      const uint32_t* rs = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = h2_to_f2(rs[j]);
        acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
      }
    }
    uint4 o;
    o.x = f2_to_h2(acc[0], acc[1]);
    o.y = f2_to_h2(acc[2], acc[3]);
    o.z = f2_to_h2(acc[4], acc[5]);
    o.w = f2_to_h2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(y)[static_cast<size_t>(t) * row_vecs + v] = o;
  }
}

}  // namespace
}  // namespace moe
}  // namespace b200ops

using namespace b200ops;

extern "C" int b200ops_moe_route_topk(const void* x, const void* router_weight, int32_t* expert_ids,
                                      float* expert_weights, int64_t num_tokens, int64_t hidden,
                                      int64_t num_experts, int64_t top_k, void* stream) {
  B200OPS_REQUIRE(num_tokens >= 0 && hidden > 0 && hidden % 8 == 0, "moe_route_topk: bad shape [%lld, %lld]",
                  (long long)num_tokens, (long long)hidden);
  B200OPS_REQUIRE(num_experts >= 1 && num_experts <= moe::kMaxExperts, "moe_route_topk: 1..%d experts, got %lld",
                  moe::kMaxExperts, (long long)num_experts);
  B200OPS_REQUIRE(top_k >= 1 && top_k <= moe::kMaxTopK && top_k <= num_experts,
                  "moe_route_topk: top_k must be in 1..min(%d, experts), got %lld", moe::kMaxTopK, (long long)top_k);
  if (num_tokens == 0) return B200OPS_OK;
  B200OPS_REQUIRE(num_tokens < (1LL << 31), "moe_route_topk: too many tokens");
  B200OPS_REQUIRE(x && router_weight && expert_ids && expert_weights, "moe_route_topk: null pointer");
  B200OPS_REQUIRE(aligned16(x) && aligned16(router_weight), "moe_route_topk: pointers must be 16-byte aligned");
  const int warps = static_cast<int>(num_experts < 32 ? num_experts : 32);
  auto kern = warps <= 8 ? moe::route_topk_kernel<16, 256> : moe::route_topk_kernel<8, 1024>;
  B200OPS_CUDA(launch_kernel(kern, dim3(static_cast<unsigned>(num_tokens)), dim3(warps * 32), 0,
                      static_cast<cudaStream_t>(stream), static_cast<const __half*>(x),
                      static_cast<const __half*>(router_weight), expert_ids, expert_weights,
                      static_cast<int>(hidden), static_cast<int>(num_experts), static_cast<int>(top_k)));
  return B200OPS_OK;
}

extern "C" int b200ops_moe_permute(const int32_t* expert_ids, int32_t* slot_to_row, int32_t* counts,
                                   int64_t* group_list, int32_t* overflow, int64_t num_slots,
                                   int64_t num_experts, int64_t world, int64_t segment_rows,
                                   void* stream) {
  B200OPS_REQUIRE(num_slots >= 0 && num_slots < (1LL << 30), "moe_permute: bad slot count %lld", (long long)num_slots);
  B200OPS_REQUIRE(num_experts >= 1 && num_experts <= moe::kMaxExperts, "moe_permute: 1..%d experts, got %lld",
                  moe::kMaxExperts, (long long)num_experts);
  B200OPS_REQUIRE(world >= 1 && num_experts % world == 0,
                  "moe_permute: experts (%lld) must divide evenly over ranks (%lld)", (long long)num_experts,
                  (long long)world);
  B200OPS_REQUIRE(world == 1 || (segment_rows > 0 && segment_rows * world < (1LL << 31)),
                  "moe_permute: bad segment capacity %lld", (long long)segment_rows);
  B200OPS_REQUIRE(slot_to_row && counts && group_list && (expert_ids || num_slots == 0), "moe_permute: null pointer");
  const size_t smem = (static_cast<size_t>(moe::kPermuteWarps) + 2) * num_experts * sizeof(int);
  B200OPS_CUDA(launch_kernel(moe::permute_kernel, dim3(1), dim3(moe::kPermuteThreads), smem,
                      static_cast<cudaStream_t>(stream), expert_ids, slot_to_row, counts, group_list, overflow,
                      static_cast<int>(num_slots), static_cast<int>(num_experts),
                      static_cast<int>(num_experts / world), static_cast<int>(world == 1 ? 0 : segment_rows)));
  return B200OPS_OK;
}

extern "C" int b200ops_moe_ep_plan(const int32_t* all_counts, int32_t* grouped_to_received,
                                   int64_t* group_list, int32_t* total_rows, int64_t world,
                                   int64_t num_experts, int64_t rank, int64_t segment_rows, void* stream) {
  B200OPS_REQUIRE(world >= 1 && world <= 64 && num_experts >= 1 && num_experts % world == 0 &&
                      num_experts / world <= 64 && rank >= 0 && rank < world,
                  "moe_ep_plan: bad geometry world=%lld experts=%lld rank=%lld", (long long)world,
                  (long long)num_experts, (long long)rank);
  B200OPS_REQUIRE(all_counts && grouped_to_received && group_list && total_rows, "moe_ep_plan: null pointer");
  const int local = static_cast<int>(num_experts / world);
  B200OPS_CUDA(launch_kernel(moe::ep_plan_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), all_counts,
                      grouped_to_received, group_list, total_rows, static_cast<int>(world),
                      static_cast<int>(num_experts), static_cast<int>(rank) * local, local,
                      static_cast<int>(segment_rows)));
  return B200OPS_OK;
}

extern "C" int b200ops_moe_copy_rows(void* dst, const void* src, const int32_t* dst_index,
                                     const int32_t* src_index, int64_t src_div, const int32_t* n_valid,
                                     int64_t n_max, int64_t row_elems, void* stream) {
  B200OPS_REQUIRE(n_max >= 0 && n_max < (1LL << 31) && row_elems > 0 && row_elems % 8 == 0 && src_div >= 1,
                  "moe_copy_rows: bad shape n=%lld row=%lld div=%lld", (long long)n_max, (long long)row_elems,
                  (long long)src_div);
  if (n_max == 0) return B200OPS_OK;
  B200OPS_REQUIRE(dst && src && aligned16(dst) && aligned16(src), "moe_copy_rows: null or misaligned pointer");
  B200OPS_CUDA(launch_kernel(moe::copy_rows_kernel, dim3(static_cast<unsigned>(n_max)), dim3(128), 0,
                      static_cast<cudaStream_t>(stream), static_cast<__half*>(dst), static_cast<const __half*>(src),
                      dst_index, src_index, static_cast<int>(src_div), n_valid, static_cast<int>(row_elems / 8)));
  return B200OPS_OK;
}

extern "C" int b200ops_moe_finalize(const void* rows, const int32_t* slot_to_row, const float* expert_weights,
                                    void* y, int64_t num_tokens, int64_t top_k, int64_t row_elems,
                                    void* stream) {
  B200OPS_REQUIRE(num_tokens >= 0 && num_tokens < (1LL << 31) && top_k >= 1 && row_elems > 0 && row_elems % 8 == 0,
                  "moe_finalize: bad shape tokens=%lld top_k=%lld row=%lld", (long long)num_tokens,
                  (long long)top_k, (long long)row_elems);
  if (num_tokens == 0) return B200OPS_OK;
  B200OPS_REQUIRE(rows && slot_to_row && expert_weights && y && aligned16(rows) && aligned16(y),
                  "moe_finalize: null or misaligned pointer");
  B200OPS_CUDA(launch_kernel(moe::finalize_kernel, dim3(static_cast<unsigned>(num_tokens)), dim3(128), 0,
                      static_cast<cudaStream_t>(stream), static_cast<const __half*>(rows), slot_to_row,
                      expert_weights, static_cast<__half*>(y), static_cast<int>(top_k),
                      static_cast<int>(row_elems / 8)));
  return B200OPS_OK;
}

// ---------------------------------------------------------------------------------------
// Expert-parallel exchange over peer memory (NVLink / NVSwitch), in place of NCCL.
//
// Every rank owns a receive buffer of `world` segments of `cap` rows in memory that its peers
// have mapped (symmetric memory).  A sender does not stage rows in a send buffer and hand them
// to a collective: the kernel that gathers the routed rows stores each row directly into the
// destination rank's segment (plain 16-byte stores through the peer mapping), and writes its
// per-expert counts into every peer's count table in the same launch.  A second, one-CTA
// kernel is the barrier: a system-scope release of "I have pushed step n" into every peer's
// flag array, then a bounded wait until every peer has said the same.  The wait gives up after
// two seconds, records an error code and returns, so a missing peer cannot hang the GPU.
// Flags carry a step number kept on the device, never reset, so the same launches can be
// replayed from a CUDA graph.
namespace b200ops {
namespace moe {
namespace {

// Logical row i (i < *n_valid, or n_max) of `src` (row i / src_div) goes to peer idx / cap,
// row my_rank * cap + idx % cap of that peer's buffer, where idx = index[i] (negative: skip).
// CTA 0 additionally copies `counts` into row my_rank of every peer's count table.
__global__ void __launch_bounds__(128)
push_rows_kernel(const __half* __restrict__ src, const int32_t* __restrict__ index, int src_div,
                 const int32_t* __restrict__ n_valid, PeerTable rows, int cap, int my_rank, int row_vecs,
                 const int32_t* __restrict__ counts, int num_counts, PeerTable count_tables, int world) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  if (i == 0 && counts != nullptr) {
    for (int t = threadIdx.x; t < num_counts * world; t += blockDim.x) {
      const int peer = t / num_counts, e = t - peer * num_counts;
      static_cast<int32_t*>(count_tables.base[peer])[my_rank * num_counts + e] = counts[e];
    }
  }
  if (n_valid != nullptr && i >= *n_valid) return;
  const int idx = index[i];
  if (idx < 0) return;
  const int peer = idx / cap, off = idx - peer * cap;
  if (peer >= world) return;  // an index outside the exchange's geometry names no buffer
  const uint4* s = reinterpret_cast<const uint4*>(src) + static_cast<size_t>(i / src_div) * row_vecs;
  uint4* d = static_cast<uint4*>(rows.base[peer]) + (static_cast<size_t>(my_rank) * cap + off) * row_vecs;
  for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) d[v] = s[v];
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One CTA, thread t talks to peer t.  `state[0]` = this rank's step counter, `state[1]` = error
// word (0 ok, otherwise 100 + the peer that never arrived).  flags[r] on a rank = last step
// rank r announced.  The preceding kernel on the stream has completed, so its peer stores are
// ordered before the release below.
__global__ void __launch_bounds__(kMaxPeers)
peer_barrier_kernel(PeerTable flag_arrays, uint32_t* __restrict__ my_flags, uint32_t* __restrict__ state,
                    int world, int my_rank) {
  __shared__ uint32_t step_s;
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0) step_s = state[0] + 1;
  __syncthreads();
  const uint32_t step = step_s;
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(flag_arrays.base[t]) + my_rank, step);
    const uint64_t t0 = [] {
      uint64_t x;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(x));
      return x;
    }();
    uint32_t spins = 0;
    // step numbers only grow; compare with wrap-around in mind
    while (static_cast<int32_t>(ld_acquire_sys(my_flags + t) - step) < 0) {
      if ((++spins & 0xffu) == 0) {
        uint64_t now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (now - t0 > 2000000000ull) {
          atomicCAS(reinterpret_cast<unsigned int*>(state + 1), 0u, 100u + static_cast<unsigned>(t));
          break;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) state[0] = step;
}

}  // namespace
}  // namespace moe
}  // namespace b200ops

extern "C" int b200ops_moe_push_rows(const void* src, const int32_t* index, int64_t src_div,
                                     const int32_t* n_valid, int64_t n_max, void* const* peer_rows,
                                     int64_t world, int64_t cap, int64_t my_rank, int64_t row_elems,
                                     const int32_t* counts, int64_t num_counts, void* const* peer_counts,
                                     void* stream) {
  B200OPS_REQUIRE(world >= 1 && world <= kMaxPeers && my_rank >= 0 && my_rank < world && cap > 0 &&
                      cap * world < (1LL << 31),
                  "moe_push_rows: bad geometry world=%lld rank=%lld cap=%lld", (long long)world,
                  (long long)my_rank, (long long)cap);
  B200OPS_REQUIRE(n_max >= 0 && n_max < (1LL << 31) && row_elems > 0 && row_elems % 8 == 0 && src_div >= 1,
                  "moe_push_rows: bad shape n=%lld row=%lld div=%lld", (long long)n_max, (long long)row_elems,
                  (long long)src_div);
  B200OPS_REQUIRE(peer_rows != nullptr && (counts == nullptr || (peer_counts != nullptr && num_counts > 0)),
                  "moe_push_rows: null peer table");
  B200OPS_REQUIRE(n_max == 0 || (src && index && aligned16(src)), "moe_push_rows: null or misaligned pointer");
  PeerTable rows, cnt;
  for (int r = 0; r < kMaxPeers; ++r) {
    rows.base[r] = r < world ? peer_rows[r] : nullptr;
    cnt.base[r] = (counts != nullptr && r < world) ? peer_counts[r] : nullptr;
    B200OPS_REQUIRE(r >= world || (rows.base[r] != nullptr && aligned16(rows.base[r])),
                    "moe_push_rows: peer %d has no buffer", r);
  }
  const unsigned grid = static_cast<unsigned>(n_max > 0 ? n_max : 1);
  B200OPS_CUDA(launch_kernel(moe::push_rows_kernel, dim3(grid), dim3(128), 0, static_cast<cudaStream_t>(stream),
                      static_cast<const __half*>(src), index, static_cast<int>(src_div),
                      n_max > 0 ? n_valid : nullptr, rows, static_cast<int>(cap), static_cast<int>(my_rank),
                      static_cast<int>(row_elems / 8), counts, static_cast<int>(num_counts), cnt,
                      static_cast<int>(world)));
  return B200OPS_OK;
}

extern "C" int b200ops_peer_barrier(void* const* peer_flags, void* my_flags, void* state, int64_t world,
                                    int64_t my_rank, void* stream) {
  B200OPS_REQUIRE(world >= 1 && world <= kMaxPeers && my_rank >= 0 && my_rank < world,
                  "peer_barrier: bad geometry world=%lld rank=%lld", (long long)world, (long long)my_rank);
  B200OPS_REQUIRE(peer_flags && my_flags && state, "peer_barrier: null pointer");
  PeerTable flags;
  for (int r = 0; r < kMaxPeers; ++r) {
    flags.base[r] = r < world ? peer_flags[r] : nullptr;
    B200OPS_REQUIRE(r >= world || flags.base[r] != nullptr, "peer_barrier: peer %d has no flag array", r);
  }
  B200OPS_CUDA(launch_kernel(moe::peer_barrier_kernel, dim3(1), dim3(kMaxPeers), 0, static_cast<cudaStream_t>(stream), flags,
                      static_cast<uint32_t*>(my_flags), static_cast<uint32_t*>(state), static_cast<int>(world),
                      static_cast<int>(my_rank)));
  return B200OPS_OK;
}

// ---------------------------------------------------------------------------------------
// Fused expert-parallel step: three launches around the two expert GEMMs instead of eight.
//
//   moe_dispatch   one CTA per token: route it (or take the given expert ids), pick the slot
//                  that holds the expert (a replica by token index when an expert has several),
//                  claim a row of the (this rank, slot) sub-segment in the owner's receive buffer
//                  with an atomic cursor, store the token's row there through the peer mapping
//                  and remember where the result will come back.  The last CTA to finish sends
//                  each peer the row counts of that peer's slots; a count word carries the step
//                  number in its upper bits, so the counts ARE the announcement "step n
//                  dispatched" (one NVLink round trip instead of counts, fence, flags).
//   moe_gather     every CTA waits (bounded) until the count words of all sources carry step n,
//                  derives the expert-major order from the counts, and the CTAs together copy the
//                  received rows into that order (the input of grouped_matmul) with the map back.
//   moe_combine    runs after the down projection whose epilogue stored the result rows into
//                  the peers' return buffers: the first CTA to run announces "step n returned"
//                  to every peer, every CTA waits (bounded) for all peers' announcements, then
//                  forms y[t] = sum_k weight[t,k] * returned_row(t,k).
//
// Layout.  Slots are placed contiguously on ranks, `spr` per rank.  Rank d's receive buffer is
// [world sources][spr slots][cap rows]; rank s's return buffer is [world*spr slots][cap rows]: the
// row claimed as number p of (source s, slot e) travels to row (s*spr + e%spr)*cap + p of rank
// e/spr and its result comes back to row e*cap + p of rank s.  A sub-segment holds `cap` rows;
// rows that do not fit are left out of the result and counted.
//
// Waiting.  A kernel only ever waits for announcements made by kernels of OTHER GPUs, which wait
// for nothing themselves before announcing; each wait gives up after two seconds, records
// 100 + peer in the state's error word and carries on, so a missing peer cannot hang the GPU.
// Step numbers only grow and live on the device, so the launches replay from a CUDA graph.
//
// state (uint32, local memory, zero-initialised once): [0] step, [1] error word, [2] CTAs of
// the running dispatch that have finished, [3] CTAs of the running combine that have started,
// [4] ... that have finished.  overflow (int32 [2], may be NULL): [0] rows dispatch could not
// place, [1] rows gather could not fit.
namespace b200ops {
namespace moe {
namespace {

constexpr int kMaxFusedBlocks = 1024;  // world * slots per rank
constexpr uint64_t kPeerWaitNs = 2000000000ull;
// A count word: rows in the low kCountBits bits, the step number (mod 2^12) above them.  A
// source's word for step n replaces its word for step n - 1 and no source can be a step ahead
// (it waits for this rank's "returned" of step n first), so equality of the tag is the test.
constexpr int kCountBits = 20;
constexpr uint32_t kCountMask = (1u << kCountBits) - 1u;
__device__ __forceinline__ uint32_t step_tag(uint32_t step) { return (step & 0xfffu) << kCountBits; }

struct DispatchParams {
  const __half* x;
  const __half* router_weight;     // null: expert ids and weights are given
  const int32_t* ids_in;           // [T, top_k] when router_weight is null
  int32_t* ids_out;                // [T, top_k] when routing here
  float* weights_out;              // [T, top_k] when routing here
  const int32_t* expert_slots;     // [E, max_replicas] slots of each expert, or null (slot = expert)
  const int32_t* num_replicas;     // [E]
  int32_t* pos;                    // [T * top_k] row of the return buffer, -1 = left out
  int32_t* cursor;                 // [num_slots] rows claimed so far (zero between launches)
  uint32_t* state;
  int32_t* overflow;
  PeerTable recv, counts;
  int hidden, num_experts, top_k, max_replicas, token_offset;
  int num_slots, spr, cap, world, my_rank;
};

__device__ __forceinline__ bool wait_for_peer(const uint32_t* flag, uint32_t step) {
  // step numbers only grow; compare with wrap-around in mind
  if (static_cast<int32_t>(ld_acquire_sys(flag) - step) >= 0) return true;
  uint64_t t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - step) < 0) {
    if ((++spins & 0xffu) == 0) {
      uint64_t now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (now - t0 > kPeerWaitNs) return false;
    }
  }
  return true;
}

// Waits until the count word carries `tag`; `word` receives it (0 rows if the wait ran out).
__device__ __forceinline__ bool wait_for_count(const uint32_t* p, uint32_t tag, uint32_t& word) {
  word = ld_acquire_sys(p);
  if ((word & ~kCountMask) == tag) return true;
  uint64_t t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  uint32_t spins = 0;
  while (true) {
    word = ld_acquire_sys(p);
    if ((word & ~kCountMask) == tag) return true;
    if ((++spins & 0xffu) == 0) {
      uint64_t now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (now - t0 > kPeerWaitNs) {
        word = 0;
        return false;
      }
    }
  }
}

// kBatch > 0: route here (route_logits<kBatch>); kBatch == 0: the expert ids are given, and the
// kernel needs a fraction of the registers, so that a large batch's CTAs are all resident at once.
template <int kBatch>
__global__ void __launch_bounds__(256) moe_dispatch_kernel(const DispatchParams p) {
  __shared__ float logits[kBatch > 0 ? kMaxExperts : 1];
  __shared__ int32_t chosen[kMaxTopK];
  __shared__ float chosen_w[kMaxTopK];
  __shared__ int dest_peer[kMaxTopK];
  __shared__ int dest_row[kMaxTopK];
  __shared__ int is_last, dropped;
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const int tid = threadIdx.x;
  if (tid == 0) dropped = 0;
  if constexpr (kBatch > 0) {
    route_logits<kBatch>(p.x, p.router_weight, logits, token, p.hidden, p.num_experts);
    __syncthreads();
    if (tid < 32) {
      route_select(logits, chosen, chosen_w, p.num_experts, p.top_k);
      __syncwarp();
      if (tid < p.top_k) {
        p.ids_out[static_cast<size_t>(token) * p.top_k + tid] = chosen[tid];
        p.weights_out[static_cast<size_t>(token) * p.top_k + tid] = chosen_w[tid];
      }
    }
  } else if (tid < p.top_k) {
    chosen[tid] = p.ids_in[static_cast<size_t>(token) * p.top_k + tid];
  }
  __syncthreads();
  if (tid < p.top_k) {
    const int e = chosen[tid];
    int slot = -1;
    if (e >= 0 && e < p.num_experts) {
      slot = e;
      if (p.expert_slots != nullptr) {
        const int reps = max(p.num_replicas[e], 1);
        slot = p.expert_slots[e * p.max_replicas + (p.token_offset + token) % reps];
      }
    }
    int row = -1, peer = 0, back = -1;
    if (slot >= 0 && slot < p.num_slots) {
      const int claimed = atomicAdd(&p.cursor[slot], 1);
      if (claimed < p.cap) {
        peer = slot / p.spr;
        row = (p.my_rank * p.spr + (slot - peer * p.spr)) * p.cap + claimed;
        back = slot * p.cap + claimed;
      }
    }
    p.pos[static_cast<size_t>(token) * p.top_k + tid] = back;
    dest_peer[tid] = peer;
    dest_row[tid] = row;
  }
  __syncthreads();
  const int row_vecs = p.hidden >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(p.x) + static_cast<size_t>(token) * row_vecs;
  for (int v = tid; v < row_vecs; v += blockDim.x) {
    const uint4 val = __ldg(src + v);
    for (int k = 0; k < p.top_k; ++k) {
      if (dest_row[k] < 0) continue;
      uint4* dst = static_cast<uint4*>(p.recv.base[dest_peer[k]]) + static_cast<size_t>(dest_row[k]) * row_vecs;
      dst[v] = val;
    }
  }
  // Publish: this CTA's stores (ordered before thread 0's fence by the CTA barrier), then its
  // arrival; the CTA that finds all others arrived finishes the step for the rank.  One thread
  // fences: a system-scope fence waits for the peer stores to be acknowledged over NVLink, and
  // 256 threads doing so one after the other cost tens of microseconds.
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    is_last = atomicAdd(&p.state[2], 1u) == gridDim.x - 1;
    if (is_last) __threadfence();  // acquire the other CTAs' arrivals; the count words below release at system scope
  }
  __syncthreads();
  if (!is_last) return;
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(p.state) + 1u;
  int lost = 0;
  for (int slot = tid; slot < p.num_slots; slot += blockDim.x) {
    const int claimed = atomicExch(&p.cursor[slot], 0);  // read at L2 and reset for the next launch
    const int kept = min(claimed, p.cap);
    lost += claimed - kept;
    const int peer = slot / p.spr;
    // thread 0's fence above ordered every CTA's row stores before this point; the release makes
    // them visible to whoever sees the word
    st_release_sys(static_cast<uint32_t*>(p.counts.base[peer]) + p.my_rank * p.spr + (slot - peer * p.spr),
                   step_tag(step) | static_cast<uint32_t>(kept));
  }
  if (lost) atomicAdd(&dropped, lost);
  __syncthreads();
  if (tid == 0) {
    if (p.overflow != nullptr) p.overflow[0] = dropped;
    p.state[0] = step;
    p.state[2] = 0;
  }
}

struct GatherParams {
  const __half* recv;        // [world][spr][cap][hidden], local
  const uint32_t* counts;    // [world][spr] count words, local, written by the peers
  uint32_t* state;
  int32_t* overflow;
  __half* grouped;           // [max_rows][hidden]
  int32_t* map;              // [max_rows] grouped row -> received row
  int64_t* group_list;       // [spr]
  int32_t* total;            // [1]
  int hidden, world, spr, cap, max_rows;
};

// Exclusive prefix sums of n <= kMaxFusedBlocks values held in shared memory, by one CTA of 256
// threads; returns the total.  `v` is overwritten with the prefix, v[n] receives the total.
__device__ __forceinline__ int block_exclusive_scan(int* v, int n, int* warp_sums) {
  constexpr int kPer = kMaxFusedBlocks / 256;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int local[kPer], sum = 0;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int idx = tid * kPer + i;
    local[i] = idx < n ? v[idx] : 0;
    sum += local[i];
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  int base = 0, total = 0;
  for (int w = 0; w < 8; ++w) {
    const int ws = warp_sums[w];
    if (w < warp) base += ws;
    total += ws;
  }
  int run = base + incl - sum;
#pragma unroll
  for (int i = 0; i < kPer; ++i) {
    const int idx = tid * kPer + i;
    if (idx < n) v[idx] = run;
    run += local[i];
  }
  if (tid == 0) v[n] = total;
  __syncthreads();
  return total;
}

__global__ void __launch_bounds__(256) moe_gather_kernel(const GatherParams p) {
  __shared__ int dst_base[kMaxFusedBlocks + 1];  // [slot j][source r] start in grouped order; [n] = total
  __shared__ int warp_sums[8];
  pdl_trigger();
  pdl_wait();
  const int tid = threadIdx.x;
  const uint32_t tag = step_tag(*reinterpret_cast<volatile uint32_t*>(p.state));
  const int blocks = p.world * p.spr;
  for (int blk = tid; blk < blocks; blk += blockDim.x) {
    const int j = blk / p.world, r = blk - j * p.world;
    uint32_t word = 0;
    if (!wait_for_count(p.counts + r * p.spr + j, tag, word))
      atomicCAS(reinterpret_cast<unsigned int*>(p.state + 1), 0u, 100u + static_cast<unsigned>(r));
    const int n = static_cast<int>(word & kCountMask);
    dst_base[blk] = n > p.cap ? p.cap : n;
  }
  __syncthreads();
  const int all_rows = block_exclusive_scan(dst_base, blocks, warp_sums);
  const int total = min(all_rows, p.max_rows);
  if (blockIdx.x == 0) {
    for (int j = tid; j < p.spr; j += blockDim.x) p.group_list[j] = min(dst_base[(j + 1) * p.world], p.max_rows);
    if (tid == 0) {
      *p.total = total;
      if (p.overflow != nullptr) p.overflow[1] = all_rows - total;
    }
  }
  const int row_vecs = p.hidden >> 3;
  for (int d = blockIdx.x; d < total; d += gridDim.x) {
    int lo = 0, hi = blocks - 1;  // last block whose start is <= d (empty blocks share a start)
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (dst_base[mid] <= d) lo = mid; else hi = mid - 1;
    }
    const int j = lo / p.world, r = lo - j * p.world;
    const int src_row = (r * p.spr + j) * p.cap + (d - dst_base[lo]);
    if (tid == 0) p.map[d] = src_row;
    const uint4* s = reinterpret_cast<const uint4*>(p.recv) + static_cast<size_t>(src_row) * row_vecs;
    uint4* o = reinterpret_cast<uint4*>(p.grouped) + static_cast<size_t>(d) * row_vecs;
    for (int v = tid; v < row_vecs; v += blockDim.x) o[v] = __ldcg(s + v);
  }
}

struct CombineParams {
  const __half* ret;         // [world*spr][cap][hidden_out], local, written by the peers
  const int32_t* pos;
  const float* weights;
  __half* y;
  uint32_t* my_flags;        // [world] return announcements, local
  uint32_t* state;
  PeerTable flags;
  int top_k, row_vecs, world, my_rank;
};

__global__ void __launch_bounds__(128) moe_combine_kernel(const CombineParams p) {
  __shared__ unsigned ticket;
  pdl_trigger();
  pdl_wait();  // the down projection before this kernel has completed: its peer stores are done
  const int tid = threadIdx.x;
  const uint32_t step = *reinterpret_cast<volatile uint32_t*>(p.state);
  if (tid == 0) ticket = atomicAdd(&p.state[3], 1u);
  __syncthreads();
  if (ticket == 0 && tid < p.world)  // the release orders the completed down projection's stores before the flag
    st_release_sys(static_cast<uint32_t*>(p.flags.base[tid]) + p.my_rank, step);
  if (tid < p.world && !wait_for_peer(p.my_flags + tid, step))
    atomicCAS(reinterpret_cast<unsigned int*>(p.state + 1), 0u, 100u + static_cast<unsigned>(tid));
  __syncthreads();
  const int t = blockIdx.x;
  for (int v = tid; v < p.row_vecs; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < p.top_k; ++k) {
      const int row = p.pos[t * p.top_k + k];
      if (row < 0) continue;
      const float w = p.weights[t * p.top_k + k];
      const uint4 r = __ldcg(reinterpret_cast<const uint4*>(p.ret) + static_cast<size_t>(row) * p.row_vecs + v);
      const uint32_t* rs = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = h2_to_f2(rs[j]);
        acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
      }
    }
    uint4 o;
    o.x = f2_to_h2(acc[0], acc[1]);
    o.y = f2_to_h2(acc[2], acc[3]);
    o.z = f2_to_h2(acc[4], acc[5]);
    o.w = f2_to_h2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(p.y)[static_cast<size_t>(t) * p.row_vecs + v] = o;
  }
  __syncthreads();
  if (tid == 0 && atomicAdd(&p.state[4], 1u) == gridDim.x - 1) {  // every CTA has its ticket by now
    p.state[3] = 0;
    p.state[4] = 0;
  }
}

int fill_peers(PeerTable& t, void* const* ptrs, int64_t world, const char* what) {
  for (int r = 0; r < kMaxPeers; ++r) {
    t.base[r] = (ptrs != nullptr && r < world) ? ptrs[r] : nullptr;
    B200OPS_REQUIRE(r >= world || (t.base[r] != nullptr && aligned16(t.base[r])), "%s: peer %d has no buffer", what, r);
  }
  return B200OPS_OK;
}

}  // namespace
}  // namespace moe
}  // namespace b200ops

extern "C" int b200ops_moe_dispatch(const void* x, const void* router_weight, const int32_t* expert_ids_in,
                                    int32_t* expert_ids_out, float* expert_weights_out,
                                    const int32_t* expert_slots, const int32_t* num_replicas,
                                    int64_t max_replicas, int64_t token_offset, int32_t* slot_to_row,
                                    void* const* peer_recv, void* const* peer_counts,
                                    int32_t* cursor, void* state, int32_t* overflow, int64_t num_tokens,
                                    int64_t hidden, int64_t num_experts, int64_t top_k, int64_t num_slots,
                                    int64_t world, int64_t cap, int64_t my_rank, void* stream) {
  B200OPS_REQUIRE(num_tokens > 0 && num_tokens < (1LL << 30) && hidden > 0 && hidden % 8 == 0,
                  "moe_dispatch: bad shape [%lld, %lld]", (long long)num_tokens, (long long)hidden);
  B200OPS_REQUIRE(num_experts >= 1 && num_experts <= moe::kMaxExperts && top_k >= 1 && top_k <= moe::kMaxTopK &&
                      top_k <= num_experts,
                  "moe_dispatch: 1..%d experts and top_k in 1..min(%d, experts), got %lld and %lld",
                  moe::kMaxExperts, moe::kMaxTopK, (long long)num_experts, (long long)top_k);
  B200OPS_REQUIRE(world >= 1 && world <= kMaxPeers && my_rank >= 0 && my_rank < world && num_slots >= 1 &&
                      num_slots % world == 0 && num_slots <= moe::kMaxFusedBlocks && cap > 0 &&
                      cap <= moe::kCountMask && num_slots * cap < (1LL << 31),
                  "moe_dispatch: bad geometry world=%lld rank=%lld slots=%lld cap=%lld", (long long)world,
                  (long long)my_rank, (long long)num_slots, (long long)cap);
  B200OPS_REQUIRE(x && slot_to_row && cursor && state && aligned16(x), "moe_dispatch: null or misaligned pointer");
  B200OPS_REQUIRE(router_weight ? (expert_ids_out && expert_weights_out && aligned16(router_weight))
                                : expert_ids_in != nullptr,
                  "moe_dispatch: give router_weight with the two outputs, or expert_ids_in");
  B200OPS_REQUIRE(expert_slots == nullptr || (num_replicas != nullptr && max_replicas >= 1),
                  "moe_dispatch: expert_slots needs num_replicas");
  moe::DispatchParams p;
  p.x = static_cast<const __half*>(x);
  p.router_weight = static_cast<const __half*>(router_weight);
  p.ids_in = expert_ids_in;
  p.ids_out = expert_ids_out;
  p.weights_out = expert_weights_out;
  p.expert_slots = expert_slots;
  p.num_replicas = num_replicas;
  p.pos = slot_to_row;
  p.cursor = cursor;
  p.state = static_cast<uint32_t*>(state);
  p.overflow = overflow;
  int rc = moe::fill_peers(p.recv, peer_recv, world, "moe_dispatch(recv)");
  if (rc == B200OPS_OK) rc = moe::fill_peers(p.counts, peer_counts, world, "moe_dispatch(counts)");
  if (rc != B200OPS_OK) return rc;
  p.hidden = static_cast<int>(hidden);
  p.num_experts = static_cast<int>(num_experts);
  p.top_k = static_cast<int>(top_k);
  p.max_replicas = static_cast<int>(max_replicas);
  p.token_offset = static_cast<int>(token_offset);
  p.num_slots = static_cast<int>(num_slots);
  p.spr = static_cast<int>(num_slots / world);
  p.cap = static_cast<int>(cap);
  p.world = static_cast<int>(world);
  p.my_rank = static_cast<int>(my_rank);
  auto kern = router_weight == nullptr ? moe::moe_dispatch_kernel<0>
              : num_experts <= 8       ? moe::moe_dispatch_kernel<16>
                                       : moe::moe_dispatch_kernel<8>;
  B200OPS_CUDA(launch_kernel(kern, dim3(static_cast<unsigned>(num_tokens)), dim3(256), 0, static_cast<cudaStream_t>(stream), p));
  return B200OPS_OK;
}

extern "C" int b200ops_moe_gather(const void* recv, const void* counts, void* state, int32_t* overflow, void* grouped, int32_t* grouped_to_received,
                                  int64_t* group_list, int32_t* total_rows, int64_t hidden, int64_t world,
                                  int64_t slots_per_rank, int64_t cap, int64_t max_rows, void* stream) {
  B200OPS_REQUIRE(world >= 1 && world <= kMaxPeers && slots_per_rank >= 1 &&
                      world * slots_per_rank <= moe::kMaxFusedBlocks && cap > 0 && max_rows > 0 &&
                      world * slots_per_rank * cap < (1LL << 31) && max_rows < (1LL << 31),
                  "moe_gather: bad geometry world=%lld slots=%lld cap=%lld rows=%lld", (long long)world,
                  (long long)slots_per_rank, (long long)cap, (long long)max_rows);
  B200OPS_REQUIRE(hidden > 0 && hidden % 8 == 0, "moe_gather: bad row length %lld", (long long)hidden);
  B200OPS_REQUIRE(recv && counts && state && grouped && grouped_to_received && group_list && total_rows &&
                      aligned16(recv) && aligned16(grouped),
                  "moe_gather: null or misaligned pointer");
  moe::GatherParams p;
  p.recv = static_cast<const __half*>(recv);
  p.counts = static_cast<const uint32_t*>(counts);
  p.state = static_cast<uint32_t*>(state);
  p.overflow = overflow;
  p.grouped = static_cast<__half*>(grouped);
  p.map = grouped_to_received;
  p.group_list = group_list;
  p.total = total_rows;
  p.hidden = static_cast<int>(hidden);
  p.world = static_cast<int>(world);
  p.spr = static_cast<int>(slots_per_rank);
  p.cap = static_cast<int>(cap);
  p.max_rows = static_cast<int>(max_rows);
  const int64_t ctas = 4LL * sm_count();
  const unsigned grid = static_cast<unsigned>(max_rows < ctas ? max_rows : ctas);
  B200OPS_CUDA(launch_kernel(moe::moe_gather_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), p));
  return B200OPS_OK;
}

extern "C" int b200ops_moe_combine(const void* returned, const int32_t* slot_to_row, const float* expert_weights,
                                   void* y, void* const* peer_flags, void* my_flags, void* state,
                                   int64_t num_tokens, int64_t top_k, int64_t row_elems, int64_t world,
                                   int64_t my_rank, void* stream) {
  B200OPS_REQUIRE(num_tokens > 0 && num_tokens < (1LL << 31) && top_k >= 1 && row_elems > 0 && row_elems % 8 == 0,
                  "moe_combine: bad shape tokens=%lld top_k=%lld row=%lld", (long long)num_tokens,
                  (long long)top_k, (long long)row_elems);
  B200OPS_REQUIRE(world >= 1 && world <= kMaxPeers && my_rank >= 0 && my_rank < world,
                  "moe_combine: bad geometry world=%lld rank=%lld", (long long)world, (long long)my_rank);
  B200OPS_REQUIRE(returned && slot_to_row && expert_weights && y && my_flags && state && aligned16(returned) &&
                      aligned16(y),
                  "moe_combine: null or misaligned pointer");
  moe::CombineParams p;
  p.ret = static_cast<const __half*>(returned);
  p.pos = slot_to_row;
  p.weights = expert_weights;
  p.y = static_cast<__half*>(y);
  p.my_flags = static_cast<uint32_t*>(my_flags);
  p.state = static_cast<uint32_t*>(state);
  const int rc = moe::fill_peers(p.flags, peer_flags, world, "moe_combine(flags)");
  if (rc != B200OPS_OK) return rc;
  p.top_k = static_cast<int>(top_k);
  p.row_vecs = static_cast<int>(row_elems / 8);
  p.world = static_cast<int>(world);
  p.my_rank = static_cast<int>(my_rank);
  B200OPS_CUDA(launch_kernel(moe::moe_combine_kernel, dim3(static_cast<unsigned>(num_tokens)), dim3(128), 0,
                      static_cast<cudaStream_t>(stream), p));
  return B200OPS_OK;
}
