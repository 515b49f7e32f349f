// Paged-attention decode, persistent tile-balanced kernel for sm_100a
// ([pages, P, Hkv, 128] caches, P % 64 == 0, GQA group <= 16).
//
// The context of every sequence is a run of 64-token tiles.  Laid end to end in sequence
// order they form one global tile sequence whose length is known only on the device (it
// depends on context_lens).  A one-CTA plan kernel writes the per-sequence tile prefix sums;
// the main kernel is launched with a fixed grid of about two CTAs per SM, arranged as
// `shares` x `kv heads`: the global sequence is cut into equal shares, and the Hkv CTAs with
// adjacent block ids take the same share, one kv head each.  They run side by side, so the
// bytes of one token row ([Hkv, D] contiguous in the cache) are fetched by neighbouring CTAs
// at about the same time -- the DRAM-page locality a per-head walk would lose.  A share may
// start and end inside a sequence, so each maximal run of tiles that lies in one sequence and
// one share (a "segment") produces partial softmax records; the combine kernel merges the
// records of a sequence.  Every SM streams the same number of K/V bytes however ragged the
// lengths are, and a single long sequence is spread over the whole GPU.
//
// Inside a CTA the pipeline never drains between segments: the producer warp issues the
// next segment's Q block (cp.async.bulk) and K/V tiles (TMA through the block table) while
// the consumer warps are still on the previous segment.  Each consumer warp owns 16 tokens
// of every tile (paged_attention_tile.cuh) and writes its own record at the end of a
// segment, so consumer warps never synchronise with each other.
//
// Segment ids: segment (sequence b, share s) is stored at record slot b + s.  Along the global
// tile sequence consecutive segments advance b or s (or both), so b + s is strictly
// increasing and the slots are unique and bounded by sequences + shares.
#include "paged_attention.cuh"
#include "paged_attention_tile.cuh"
#include "tma_host.cuh"

#include <cstdlib>

namespace b200ops {
namespace pa {
namespace {

using namespace tile;

constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kStages = 3;
constexpr int kPageBatch = 64;          // block-table entries staged in shared memory at a time
constexpr int kQBytes = 16 * kD * 2;    // one Q block: up to 16 heads x 128 channels
constexpr int kErrProducerWait = 13;
constexpr int kErrConsumerWait = 14;
constexpr int kErrQWait = 15;

constexpr int kMaxInlineBatch = 512;    // batches up to this size are planned inside the main kernel

constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kStageBytes + 2 * kQBytes +
                              (2 * kStages + 4) * 8 + kPageBatch * 4 + 16 +
                              (kMaxInlineBatch + 1 + kThreads) * 4;

__device__ int g_stream_status = 0;

// tile_prefix[b] = tiles of sequences 0..b-1; tile_prefix[bs] = total per kv head.
__global__ void __launch_bounds__(1024)
stream_plan_kernel(const int32_t* __restrict__ context_lens, int bs, int cap,
                   int32_t* __restrict__ tile_prefix) {
  __shared__ int partial[1024];
  const int per = (bs + 1023) / 1024;
  const int lo = min(bs, static_cast<int>(threadIdx.x) * per), hi = min(bs, lo + per);
  int sum = 0;
  for (int b = lo; b < hi; ++b) {
    int L = context_lens[b];
    L = L < 0 ? 0 : (L > cap ? cap : L);
    sum += (L + kTile - 1) / kTile;
  }
  partial[threadIdx.x] = sum;
  __syncthreads();
  // Hillis-Steele inclusive scan over 1024 partial sums
  for (int o = 1; o < 1024; o <<= 1) {
    const int v = threadIdx.x >= o ? partial[threadIdx.x - o] : 0;
    __syncthreads();
    partial[threadIdx.x] += v;
    __syncthreads();
  }
  int run = partial[threadIdx.x] - sum;  // exclusive
  if (threadIdx.x == 0) tile_prefix[0] = 0;
  for (int b = lo; b < hi; ++b) {
    int L = context_lens[b];
    L = L < 0 ? 0 : (L > cap ? cap : L);
    run += (L + kTile - 1) / kTile;
    tile_prefix[b + 1] = run;
  }
}

// Largest b in [0, bs) whose tile range starts at or before global tile g: tile_prefix[b] <= g.
// (Sequences with no tiles share a start; the callers skip them.)
__device__ __forceinline__ int find_sequence(const int32_t* __restrict__ tile_prefix, int bs, int g) {
  int lo = 0, hi = bs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tile_prefix[mid] <= g) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// kInlinePlan: the batch is small enough that every CTA computes the tile prefix sums itself
// (into shared memory; CTA 0 also publishes them for the combine kernel), which saves the
// separate plan launch.  Otherwise `tile_prefix_global` was filled by stream_plan_kernel.
template <bool kUpper, bool kInlinePlan>
__global__ void __launch_bounds__(kThreads)
paged_attention_stream_kernel(const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v, Args a,
                              int32_t* __restrict__ tile_prefix_global, float* __restrict__ records) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem + kStages * kStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(q_smem + 2 * kQBytes);
  uint64_t* empty = full + kStages;
  uint64_t* qfull = empty + kStages;
  uint64_t* qempty = qfull + 2;
  int* page_ids = reinterpret_cast<int*>(qempty + 2);
  int* abort_flag = page_ids + kPageBatch;
  int* prefix_s = abort_flag + 4;                      // [kMaxInlineBatch + 1]
  int* scan_s = prefix_s + kMaxInlineBatch + 1;        // [kThreads]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hkv = a.num_kv_heads;
  const int32_t* tile_prefix = tile_prefix_global;
  if (kInlinePlan) {
    const int cap_tokens = a.max_pages_per_seq * a.page_size;
    const int per = (a.bs + kThreads - 1) / kThreads;
    const int lo = min(a.bs, static_cast<int>(threadIdx.x) * per), hi = min(a.bs, lo + per);
    int sum = 0;
    for (int i = lo; i < hi; ++i) {
      int L = a.context_lens[i];
      L = L < 0 ? 0 : (L > cap_tokens ? cap_tokens : L);
      const int n = (L + kTile - 1) / kTile;
      prefix_s[i + 1] = n;
      sum += n;
    }
    scan_s[threadIdx.x] = sum;
    __syncthreads();
    int run = 0;
    for (int t = 0; t < static_cast<int>(threadIdx.x); ++t) run += scan_s[t];
    if (threadIdx.x == 0) prefix_s[0] = 0;
    for (int i = lo; i < hi; ++i) {
      run += prefix_s[i + 1];
      prefix_s[i + 1] = run;
    }
    __syncthreads();
    if (blockIdx.x == 0)
      for (int i = threadIdx.x; i <= a.bs; i += kThreads) tile_prefix_global[i] = prefix_s[i];
    tile_prefix = prefix_s;
  }
  const int group = a.num_heads / hkv;
  const int n_shares = gridDim.x / hkv;
  const int my_share = blockIdx.x / hkv;
  const int h = blockIdx.x - my_share * hkv;  // this CTA's kv head
  if (my_share >= n_shares) return;
  const int total = tile_prefix[a.bs];
  const int share = (total + n_shares - 1) / n_shares;
  const int g0 = my_share * share;
  const int g1 = min(total, g0 + share);
  if (g0 >= g1) return;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], kConsumerWarps);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&qfull[s], 1);
      ptx::mbar_init(&qempty[s], kConsumerWarps);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();

  int g = g0;
  int b = find_sequence(tile_prefix, a.bs, g);
  int stage = 0, seg = 0;
  uint32_t phase = 0;

  if (warp == kConsumerWarps) {
    // ---------------- producer warp (all lanes walk the segments; lane 0 issues) ----------------
    if (lane == 0) {
      ptx::prefetch_tensormap(&map_k);
      ptx::prefetch_tensormap(&map_v);
    }
    int ok = 1;
    while (g < g1 && ok) {
      const int nb = tile_prefix[b + 1] - tile_prefix[b];
      if (nb == 0) {
        ++b;
        continue;
      }
      const int t0 = g - tile_prefix[b];
      const int nseg = min(nb - t0, g1 - g);
      const int qs = seg & 1;
      if (lane == 0) {
        if (!ptx::mbar_wait(&qempty[qs], ((seg >> 1) & 1) ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_stream_status, 0, kErrQWait);
          ok = 0;
        } else {
          const uint32_t bytes = static_cast<uint32_t>(group) * kD * 2;
          ptx::mbar_arrive_expect_tx(&qfull[qs], bytes);
          const __half* src = a.q + (static_cast<size_t>(b) * a.num_heads + static_cast<size_t>(h) * group) * kD;
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                  ptx::smem_u32(q_smem + qs * kQBytes)),
              "l"(src), "r"(bytes), "r"(ptx::smem_u32(&qfull[qs]))
              : "memory");
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      const int32_t* table = a.block_tables + static_cast<size_t>(b) * a.max_pages_per_seq;
      int cached_first = -(1 << 30);
      for (int i = 0; i < nseg && ok; ++i) {
        const int tok = (t0 + i) * kTile;
        const int pidx = tok / a.page_size;
        const int off = tok - pidx * a.page_size;
        if (pidx < cached_first || pidx >= cached_first + kPageBatch) {
          __syncwarp();
          cached_first = pidx;
          for (int j = lane; j < kPageBatch; j += 32) {
            const int pi = cached_first + j;
            int pg = pi < a.max_pages_per_seq ? table[pi] : 0;
            pg = pg < 0 ? 0 : (pg >= a.num_pages ? a.num_pages - 1 : pg);
            page_ids[j] = pg;
          }
          __syncwarp();
        }
        if (lane == 0) {
          if (!ptx::mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(&g_stream_status, 0, kErrProducerWait);
            ok = 0;
          } else {
            const int pg = page_ids[pidx - cached_first];
            uint8_t* st = smem + stage * kStageBytes;
            ptx::mbar_arrive_expect_tx(&full[stage], kStageBytes);
            ptx::tma_load_4d(st, &map_k, &full[stage], 0, h, off, pg);
            ptx::tma_load_4d(st + kSubTileBytes, &map_k, &full[stage], 64, h, off, pg);
            ptx::tma_load_4d(st + kTensorTileBytes, &map_v, &full[stage], 0, h, off, pg);
            ptx::tma_load_4d(st + kTensorTileBytes + kSubTileBytes, &map_v, &full[stage], 64, h, off, pg);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      g += nseg;
      ++seg;
      if (t0 + nseg == nb) ++b;
    }
  } else {
    // ---------------- consumer warps ----------------
    const int gq = lane >> 2, t4 = lane & 3;
    const int row0 = warp * 16;
    const int cap = a.max_pages_per_seq * a.page_size;
    bool ok = true;
    while (g < g1 && ok) {
      const int nb = tile_prefix[b + 1] - tile_prefix[b];
      if (nb == 0) {
        ++b;
        continue;
      }
      const int t0 = g - tile_prefix[b];
      const int nseg = min(nb - t0, g1 - g);
      const bool has_last_tile = t0 + nseg == nb;
      // Only the sequence's last tile can be partial; the length is needed just for that one.
      int seq_len = 0x7fffffff;
      if (has_last_tile) {
        seq_len = a.context_lens[b];
        seq_len = seq_len > cap ? cap : seq_len;
      }
      const int qs = seg & 1;
      if (!ptx::mbar_wait(&qfull[qs], (seg >> 1) & 1, abort_flag)) {
        *abort_flag = 1;
        atomicCAS(&g_stream_status, 0, kErrQWait);
        break;
      }
      uint32_t qa[kD / 16][4];
      load_q_fragments<kUpper>(qa, reinterpret_cast<const __half*>(q_smem + qs * kQBytes), group, lane);
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&qempty[qs]);
      WarpState st;
      st.reset();
      for (int i = 0; i < nseg; ++i) {
        if (!ptx::mbar_wait(&full[stage], phase, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_stream_status, 0, kErrConsumerWait);
          ok = false;
          break;
        }
        const int end = (has_last_tile && i == nseg - 1) ? seq_len : 0x7fffffff;
        consume_slice<kUpper>(st, qa, smem + stage * kStageBytes, row0, (t0 + i) * kTile + row0, end, lane,
                              a.scale_log2);
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&empty[stage]);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (!ok) break;
      st.finish_sums();
      // This warp's record of the segment: [group][D + 2] floats.
      const size_t slot = static_cast<size_t>(b) + my_share;
      float* rec = records + (((slot * hkv + h) * kConsumerWarps + warp) * group) * (kD + 2);
      if (gq < group) {
#pragma unroll
        for (int i = 0; i < kD / 8; ++i)
          *reinterpret_cast<float2*>(rec + gq * (kD + 2) + i * 8 + 2 * t4) = make_float2(st.o[i][0], st.o[i][1]);
        if (t4 == 0) {
          rec[gq * (kD + 2) + kD] = st.m_lo;
          rec[gq * (kD + 2) + kD + 1] = st.l_lo;
        }
      }
      if (kUpper && gq + 8 < group) {
#pragma unroll
        for (int i = 0; i < kD / 8; ++i)
          *reinterpret_cast<float2*>(rec + (gq + 8) * (kD + 2) + i * 8 + 2 * t4) =
              make_float2(st.o[i][2], st.o[i][3]);
        if (t4 == 0) {
          rec[(gq + 8) * (kD + 2) + kD] = st.m_hi;
          rec[(gq + 8) * (kD + 2) + kD + 1] = st.l_hi;
        }
      }
      g += nseg;
      ++seg;
      if (has_last_tile) ++b;
    }
  }
}

// One warp per (sequence, query head): lanes first take one record each to find the global
// maximum and the normaliser, then every lane sums its four channels over the records.
constexpr int kCombineWarps = 4;

__global__ void __launch_bounds__(kCombineWarps * 32)
stream_combine_kernel(Args a, const int32_t* __restrict__ tile_prefix, const float* __restrict__ records,
                      int num_ctas) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * kCombineWarps + (threadIdx.x >> 5);
  if (item >= a.bs * a.num_heads) return;
  const int b = item / a.num_heads, hq = item - b * a.num_heads;
  const int hkv = a.num_kv_heads, group = a.num_heads / hkv;
  const int h = hq / group, r = hq - h * group;
  __half* out = a.out + static_cast<size_t>(item) * kD;
  const int nb = tile_prefix[b + 1] - tile_prefix[b];
  if (nb == 0) {
    *reinterpret_cast<uint2*>(out + lane * 4) = make_uint2(0u, 0u);
    return;
  }
  const int n_shares = num_ctas / hkv;
  const int total = tile_prefix[a.bs];
  const int share = (total + n_shares - 1) / n_shares;
  const int first_tile = tile_prefix[b];
  const int c_first = first_tile / share;
  const int c_last = (first_tile + nb - 1) / share;
  const int n_rec = (c_last - c_first + 1) * kConsumerWarps;
  auto record = [&](int i) {
    const size_t slot = static_cast<size_t>(b) + c_first + i / kConsumerWarps;
    return records + (((slot * hkv + h) * kConsumerWarps + (i % kConsumerWarps)) * group + r) * (kD + 2);
  };
  float mm = -INFINITY;
  for (int i = lane; i < n_rec; i += 32) mm = fmaxf(mm, record(i)[kD]);
  mm = warp_max(mm);
  float ll = 0.f;
  for (int i = lane; i < n_rec; i += 32) {
    const float* p = record(i);
    if (p[kD] != -INFINITY) ll += p[kD + 1] * exp2f(p[kD] - mm);
  }
  ll = warp_sum(ll);
  const float inv = ll > 0.f ? 1.0f / ll : 0.f;
  float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
  for (int i0 = 0; i0 < n_rec; i0 += 32) {
    // lane j of this batch holds the weight of record i0 + j
    const int mine = i0 + lane;
    float w = 0.f;
    if (mine < n_rec) {
      const float m = record(mine)[kD];
      w = (m == -INFINITY) ? 0.f : exp2f(m - mm);
    }
    const int n = min(32, n_rec - i0);
    for (int j = 0; j < n; ++j) {
      const float wj = __shfl_sync(0xffffffffu, w, j);
      if (wj != 0.f) {
        const float2* p = reinterpret_cast<const float2*>(record(i0 + j) + lane * 4);
        const float2 x = p[0], y = p[1];
        o0 = fmaf(wj, x.x, o0);
        o1 = fmaf(wj, x.y, o1);
        o2 = fmaf(wj, y.x, o2);
        o3 = fmaf(wj, y.y, o3);
      }
    }
  }
  uint2 packed;
  packed.x = f2_to_h2(o0 * inv, o1 * inv);
  packed.y = f2_to_h2(o2 * inv, o3 * inv);
  *reinterpret_cast<uint2*>(out + lane * 4) = packed;
}

int env_int(const char* name, int fallback) {
  const char* s = std::getenv(name);
  return (s && *s) ? std::atoi(s) : fallback;
}

size_t align256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

}  // namespace

// Grid: as many whole groups of Hkv CTAs as fit in two CTAs per SM (at least one group).
int stream_num_ctas(int64_t num_kv_heads) {
  const int64_t fit = 2 * sm_count() / num_kv_heads;
  return static_cast<int>((fit > 0 ? fit : 1) * num_kv_heads);
}

size_t stream_workspace_bytes(int64_t bs, int64_t num_heads, int64_t num_kv_heads, int64_t head_dim) {
  const size_t slots = static_cast<size_t>(bs) + stream_num_ctas(num_kv_heads) / num_kv_heads;
  return align256(static_cast<size_t>(bs + 1) * sizeof(int32_t)) +
         slots * kConsumerWarps * num_heads * (head_dim + 2) * sizeof(float);
}

bool stream_path_supported(const Args& a) {
  // Opt-in (B200OPS_PA_MODE=3).  Measured on B200 the main kernel matches the split-context
  // kernel (both at the measured HBM peak on a 1.25 GB batch), but its combine step reads four
  // records per segment and the whole operator came out 3-6 % slower on large batches and
  // clearly slower on small ones, so the split-context path stays the default.
  if (env_int("B200OPS_PA_MODE", 0) != 3) return false;
  const int group = a.num_heads / a.num_kv_heads;
  return a.layout == B200OPS_KV_LAYOUT_NHD && a.head_dim == kD && a.page_size % kTile == 0 && group <= 16 &&
         a.page_size <= 256 * kTile && a.num_kv_heads <= 2 * sm_count() &&
         static_cast<long long>(a.bs) * (a.max_pages_per_seq * a.page_size / kTile + 1) < 0x7fffffffLL;
}

int launch_stream(const Args& a, void* workspace, cudaStream_t st) {
  int32_t* tile_prefix = static_cast<int32_t*>(workspace);
  float* records = reinterpret_cast<float*>(static_cast<char*>(workspace) +
                                            align256(static_cast<size_t>(a.bs + 1) * sizeof(int32_t)));
  CUtensorMap mk, mv;
  const uint64_t dims[4] = {static_cast<uint64_t>(kD), static_cast<uint64_t>(a.num_kv_heads),
                            static_cast<uint64_t>(a.page_size), static_cast<uint64_t>(a.num_pages)};
  const uint64_t strides[3] = {static_cast<uint64_t>(kD) * 2, static_cast<uint64_t>(a.num_kv_heads) * kD * 2,
                               static_cast<uint64_t>(a.page_size) * a.num_kv_heads * kD * 2};
  const uint32_t box[4] = {64, 1, kTile, 1};
  int rc = encode_f16_map(&mk, a.k_cache, 4, dims, strides, box, "paged_attention(key_cache)");
  if (rc != B200OPS_OK) return rc;
  rc = encode_f16_map(&mv, a.v_cache, 4, dims, strides, box, "paged_attention(value_cache)");
  if (rc != B200OPS_OK) return rc;

  const bool upper = a.num_heads / a.num_kv_heads > 8;
  const bool inline_plan = a.bs <= kMaxInlineBatch;
  auto kern = upper ? (inline_plan ? paged_attention_stream_kernel<true, true>
                                   : paged_attention_stream_kernel<true, false>)
                    : (inline_plan ? paged_attention_stream_kernel<false, true>
                                   : paged_attention_stream_kernel<false, false>);
  static bool attr_set[4][64] = {{false}};
  const int variant = (upper ? 2 : 0) + (inline_plan ? 1 : 0);
  int dev = 0;
  B200OPS_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[variant][dev]) {
    B200OPS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(kSmemBytes)));
    attr_set[variant][dev] = true;
  }
  if (!inline_plan) {
    const int cap = a.max_pages_per_seq * a.page_size;
    stream_plan_kernel<<<1, 1024, 0, st>>>(a.context_lens, a.bs, cap, tile_prefix);
    B200OPS_LAUNCH_CHECK("paged_attention plan");
  }
  const int ctas = stream_num_ctas(a.num_kv_heads);
  kern<<<ctas, kThreads, kSmemBytes, st>>>(mk, mv, a, tile_prefix, records);
  B200OPS_LAUNCH_CHECK("paged_attention");
  const int items = a.bs * a.num_heads;
  stream_combine_kernel<<<(items + kCombineWarps - 1) / kCombineWarps, kCombineWarps * 32, 0, st>>>(
      a, tile_prefix, records, ctas);
  B200OPS_LAUNCH_CHECK("paged_attention combine");
  return B200OPS_OK;
}

int stream_status_take() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
  }
  return v;
}

}  // namespace pa
}  // namespace b200ops
