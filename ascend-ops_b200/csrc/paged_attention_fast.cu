// Paged-attention decode, fast path for sm_100a: head_dim 128, GQA group <= 16; caches
// [pages, P, Hkv, 128] (NHD; P a multiple of 64, or 16 or 32) or [pages, Hkv*8, P, 16] (NZ, the
// reference's layout; P a multiple of 64).
//
// One CTA = one (sequence, kv head, context chunk).  A producer warp walks the chunk's pages
// through the block table and streams 64-token K and V tiles into a ring of 128B-swizzled
// shared-memory stages with TMA (cp.async.bulk.tensor.4d; NHD: the cache viewed as
// [pages][P][Hkv][D], two 64-channel boxes per tile and tensor; NZ: the cache viewed as
// [pages][Hkv*8][P/16][256], one box of 8 chunks x 64 tokens per tile and tensor).  Four consumer warps each own
// 16 tokens of every tile: S = Q.K^T and O += P.V run on warp-level tensor-core MMAs
// (m16n8k16, query heads padded to the 16-row operand, fp32 accumulation), the online
// softmax is fp32 with exp2 and scale*log2(e) folded in.  Every K/V byte crosses HBM -> smem
// once and is shared by all query heads of the group; the kernel is HBM-bound (about 28
// flop per KV byte at group 7).  Warps merge their (max, sum, O) through shared memory and
// the CTA writes either the final fp16 rows (single-chunk sequence) or a partial record; the
// CTA that completes a pair's last outstanding chunk (an atomic counter, nobody waits) then
// merges the pair's records into the output, so the operator is a single kernel.
//
// Cache bytes past a sequence's length are never trusted: scores of such tokens are
// replaced by -inf and their V rows are zeroed in shared memory before the PV product, so
// uninitialised cache memory (NaN patterns) cannot leak into the output.
#include "paged_attention.cuh"
#include "paged_attention_tile.cuh"
#include "tma_host.cuh"

#include <atomic>

namespace b200ops {
namespace pa {
namespace {

using namespace tile;

constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kErrProducerWait = 11;
constexpr int kErrConsumerWait = 12;

template <int kStages>
struct Smem {
  static constexpr size_t kTiles = static_cast<size_t>(kStages) * kStageBytes;
  static constexpr size_t kMerge = static_cast<size_t>(kConsumerWarps) * 16 * (kD + 2) * 4;
  static constexpr size_t kData = kTiles > kMerge ? kTiles : kMerge;
  static constexpr size_t kBytes = 1024 + kData + 2 * kStages * 8 + kMaxChunkPages * 4 + 16;
};

__device__ int g_pa_status = 0;

// kUpper: the GQA group has more than 8 query heads, so MMA rows 8..15 carry data.
template <int kStages, bool kUpper, bool kNz>
__global__ void __launch_bounds__(kThreads, 2)
paged_attention_fast_kernel(const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Smem<kStages>::kData);
  uint64_t* empty = full + kStages;
  int* page_ids = reinterpret_cast<int*>(empty + kStages);
  int* abort_flag = page_ids + kMaxChunkPages;

  // Dispatch order: the chunks of one (sequence, kv head) first, then the kv heads, then the
  // sequences.  (kv head fastest and chunk slowest -- neighbouring bytes side by side, the
  // longest sequences' last chunks at the end -- was measured and is 3 % slower on the
  // 64-sequence batch, equal elsewhere: every merge then falls into the kernel's tail.)
  const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = a.num_heads / a.num_kv_heads;
  const int h0 = kvh * group;

  // The producer warp starts the chunk's block-table reads before the sequence length is
  // known (entries that name no page -- past the sequence's end, or invalid inside it -- are
  // fetched from page 0 and their tokens left out, as the general kernel leaves them out), and its
  // first lane sets up the barriers: three dependent global round trips (length, table, data)
  // become two, and the first tiles are on their way before the CTA-wide barrier.  The reads
  // assume the base chunk length; a sequence long enough to take longer chunks reads again.
  const int32_t* table = a.block_tables + static_cast<size_t>(b) * a.max_pages_per_seq;
  auto load_page_ids = [&](int chunk_tokens) {
    const int pages_per_chunk = chunk_tokens / a.page_size;
    const int first_page = chunk * pages_per_chunk;
    for (int i = lane; i < pages_per_chunk; i += 32) {
      const int pg = first_page + i < a.max_pages_per_seq ? table[first_page + i] : 0;
      page_ids[i] = (pg < 0 || pg >= a.num_pages) ? -1 : pg;  // -1: loaded from page 0, never used
    }
  };
  pdl_trigger();
  if (warp == kConsumerWarps && lane == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], kConsumerWarps);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
  }
  pdl_wait();  // everything below reads what earlier kernels wrote (the cache, the tables)
  if (warp == kConsumerWarps) load_page_ids(a.chunk_tokens);

  int L = a.context_lens[b];
  const int cap = a.max_pages_per_seq * a.page_size;
  if (L > cap) L = cap;
  if (L <= 0) {
    if (chunk == 0)
      for (int i = threadIdx.x; i < group * kD; i += kThreads)
        a.out[(static_cast<size_t>(b) * a.num_heads + h0) * kD + i] = __float2half(0.f);
    return;
  }
  const int ct = seq_chunk_tokens(a.chunk_tokens, a.max_chunks, a.chunk_align, L);
  const int start = chunk * ct;
  if (start >= L) return;
  const int end = min(L, start + ct);
  const int n_tiles = (end - start + kTile - 1) / kTile;
  const int n_chunks = (L + ct - 1) / ct;
  if (ct != a.chunk_tokens && warp == kConsumerWarps) {
    __syncwarp();
    load_page_ids(ct);
  }

  // One tile = K and V of 64 tokens of this kv head: four boxes of 64 channels.
  auto issue_tile = [&](int t, int stage) {
    const int tok = t * kTile;  // relative to the chunk start (a page boundary)
    const int pg = max(page_ids[tok / a.page_size], 0);
    const int off = tok % a.page_size;
    uint8_t* st = smem + stage * kStageBytes;
    ptx::mbar_arrive_expect_tx(&full[stage], kStageBytes);
    if (kNz) {  // {256 halfs = 16 tokens, 4 such rows, the head's 8 chunks, 1 page}
      ptx::tma_load_4d(st, &map_k, &full[stage], 0, off / 16, kvh * (kD / 16), pg);
      ptx::tma_load_4d(st + kTensorTileBytes, &map_v, &full[stage], 0, off / 16, kvh * (kD / 16), pg);
    } else if (a.page_size >= kTile) {  // {64 channels, 1 head, 64 tokens, 1 page}, twice
      ptx::tma_load_4d(st, &map_k, &full[stage], 0, kvh, off, pg);
      ptx::tma_load_4d(st + kSubTileBytes, &map_k, &full[stage], 64, kvh, off, pg);
      ptx::tma_load_4d(st + kTensorTileBytes, &map_v, &full[stage], 0, kvh, off, pg);
      ptx::tma_load_4d(st + kTensorTileBytes + kSubTileBytes, &map_v, &full[stage], 64, kvh, off, pg);
    } else {  // pages of 16 or 32 tokens: the tile is 4 or 2 pages, one set of boxes per page
      for (int j = 0; j < kTile / a.page_size; ++j) {
        const int pj = max(page_ids[tok / a.page_size + j], 0);
        uint8_t* dst = st + j * a.page_size * 128;  // whole 8-row swizzle groups: the pattern is kept
        ptx::tma_load_4d(dst, &map_k, &full[stage], 0, kvh, 0, pj);
        ptx::tma_load_4d(dst + kSubTileBytes, &map_k, &full[stage], 64, kvh, 0, pj);
        ptx::tma_load_4d(dst + kTensorTileBytes, &map_v, &full[stage], 0, kvh, 0, pj);
        ptx::tma_load_4d(dst + kTensorTileBytes + kSubTileBytes, &map_v, &full[stage], 64, kvh, 0, pj);
      }
    }
  };
  const int prefill = min(kStages, n_tiles);
  if (warp == kConsumerWarps) {
    __syncwarp();  // page_ids of all lanes are in shared memory
    if (lane == 0)
      for (int t = 0; t < prefill; ++t) issue_tile(t, t);  // a fresh ring: nothing to wait for
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ---------------- producer warp: the rest of the chunk ----------------
    if (lane == 0) {
      int stage = prefill == kStages ? 0 : prefill;
      uint32_t phase = prefill == kStages ? 1u : 0u;
      for (int t = prefill; t < n_tiles; ++t) {
        if (!ptx::mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_pa_status, 0, kErrProducerWait);
          break;
        }
        issue_tile(t, stage);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else {
    // ---------------- consumer warps ----------------
    const int g = lane >> 2, t4 = lane & 3;
    uint32_t qa[kD / 16][4];
    load_q_fragments<kUpper>(qa, a.q + (static_cast<size_t>(b) * a.num_heads + h0) * kD, group, lane);
    WarpState st;
    st.reset();
    int stage = 0;
    uint32_t phase = 0;
    const int row0 = warp * 16;  // this warp's token rows inside a tile
    for (int t = 0; t < n_tiles; ++t) {
      if (!ptx::mbar_wait(&full[stage], phase, abort_flag)) {
        *abort_flag = 1;
        atomicCAS(&g_pa_status, 0, kErrConsumerWait);
        break;
      }
      // A warp's 16 tokens lie inside one page (pages hold a multiple of 16 tokens).
      if (page_ids[(t * kTile + row0) / a.page_size] >= 0)
        consume_slice<kUpper, kNz>(st, qa, smem + stage * kStageBytes, row0, start + t * kTile + row0, end, lane,
                                   a.scale_log2);
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty[stage]);
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    st.finish_sums();
    float (&o)[kD / 8][4] = st.o;
    const float m_lo = st.m_lo, m_hi = st.m_hi, l_lo = st.l_lo, l_hi = st.l_hi;

    // All tiles of this CTA have landed and been read: reuse the stage memory for the merge.
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32));
    float* rec = reinterpret_cast<float*>(smem) + static_cast<size_t>(warp) * 16 * (kD + 2);
#pragma unroll
    for (int i = 0; i < kD / 8; ++i) {
      const int d = i * 8 + 2 * t4;
      *reinterpret_cast<float2*>(rec + g * (kD + 2) + d) = make_float2(o[i][0], o[i][1]);
      if (kUpper)
        *reinterpret_cast<float2*>(rec + (g + 8) * (kD + 2) + d) = make_float2(o[i][2], o[i][3]);
    }
    if (t4 == 0) {
      rec[g * (kD + 2) + kD] = m_lo;
      rec[g * (kD + 2) + kD + 1] = l_lo;
      if (kUpper) {
        rec[(g + 8) * (kD + 2) + kD] = m_hi;
        rec[(g + 8) * (kD + 2) + kD + 1] = l_hi;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32));
    const float* all = reinterpret_cast<const float*>(smem);
    for (int idx = threadIdx.x; idx < group * kD; idx += kConsumerWarps * 32) {
      const int r = idx >> 7, d = idx & (kD - 1);
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w)
        mm = fmaxf(mm, all[(w * 16 + r) * (kD + 2) + kD]);
      float acc = 0.f, ll = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float* rr = all + (w * 16 + r) * (kD + 2);
        const float f = (rr[kD] == -INFINITY) ? 0.f : exp2f(rr[kD] - mm);
        acc += rr[d] * f;
        ll += rr[kD + 1] * f;
      }
      const int h = h0 + r;
      if (n_chunks == 1) {
        a.out[(static_cast<size_t>(b) * a.num_heads + h) * kD + d] =
            __float2half(ll > 0.f ? acc / ll : 0.f);
      } else {
        float* pr = a.partials +
                    ((static_cast<size_t>(b) * a.num_heads + h) * a.max_chunks + chunk) * (kD + 2);
        pr[d] = acc;
        if (d == 0) {
          pr[kD] = mm;
          pr[kD + 1] = ll;
        }
      }
    }
    if (n_chunks > 1 && a.pair_counters != nullptr) {
      // Publish this chunk, then see whether it was the pair's last one; if so merge all of
      // the pair's chunks here (one warp per query head).  No CTA waits for another.
      int* arrival = abort_flag + 1;
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32));
      if (threadIdx.x == 0) *arrival = atomicAdd(&a.pair_counters[b * a.num_kv_heads + kvh], 1);
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32));
      if (*arrival == n_chunks - 1) {
        __threadfence();
        for (int r = warp; r < group; r += kConsumerWarps) combine_head<kD>(a, b, h0 + r, n_chunks, lane);
      }
    }
  }
}

template <int kStages, bool kUpper, bool kNz>
int launch_variant(const CUtensorMap& mk, const CUtensorMap& mv, const Args& a, dim3 grid, cudaStream_t st) {
  auto kern = paged_attention_fast_kernel<kStages, kUpper, kNz>;
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  B200OPS_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    B200OPS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(Smem<kStages>::kBytes)));
    attr_set[dev].store(true, std::memory_order_release);
  }
  B200OPS_CUDA(launch_kernel(kern, grid, dim3(kThreads), Smem<kStages>::kBytes, st, mk, mv, a));
  return B200OPS_OK;
}

template <int kStages>
int launch_with_stages(const CUtensorMap& mk, const CUtensorMap& mv, const Args& a, dim3 grid,
                       cudaStream_t st) {
  const bool upper = a.num_heads / a.num_kv_heads > 8;
  const bool nz = a.layout == B200OPS_KV_LAYOUT_NZ;
  if (nz) return upper ? launch_variant<kStages, true, true>(mk, mv, a, grid, st)
                       : launch_variant<kStages, false, true>(mk, mv, a, grid, st);
  return upper ? launch_variant<kStages, true, false>(mk, mv, a, grid, st)
               : launch_variant<kStages, false, false>(mk, mv, a, grid, st);
}

}  // namespace

bool fast_path_supported(const Args& a) {
  // B200OPS_PA_MODE: 2 = general kernel, anything else = this split-context TMA path.
  if (knob(kKnobPaMode, 0) == 2) return false;
  const int group = a.num_heads / a.num_kv_heads;
  const bool page_ok = a.page_size % kTile == 0 ||
                       (a.layout == B200OPS_KV_LAYOUT_NHD && (a.page_size == 16 || a.page_size == 32) &&
                        a.chunk_tokens % kTile == 0);
  return a.head_dim == kD && page_ok &&
         group <= 16 && a.chunk_tokens % a.page_size == 0 &&
         a.chunk_tokens / a.page_size <= kMaxChunkPages && a.page_size <= 256 * kTile;
}

int launch_fast(const Args& a, cudaStream_t st) {
  CUtensorMap mk, mv;
  int rc;
  if (a.layout == B200OPS_KV_LAYOUT_NZ) {
    // [pages][Hkv*8 chunks][P/16][16 tokens x 16 halfs]: a tile is the head's 8 chunks x 64 tokens
    const uint64_t chunks = static_cast<uint64_t>(a.num_kv_heads) * (kD / 16);
    const uint64_t dims[4] = {256, static_cast<uint64_t>(a.page_size) / 16, chunks, static_cast<uint64_t>(a.num_pages)};
    const uint64_t strides[3] = {512, static_cast<uint64_t>(a.page_size) * 32,
                                 chunks * static_cast<uint64_t>(a.page_size) * 32};
    const uint32_t box[4] = {256, kTile / 16, kD / 16, 1};
    rc = encode_f16_map(&mk, a.k_cache, 4, dims, strides, box, "paged_attention(key_cache)",
                        CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != B200OPS_OK) return rc;
    rc = encode_f16_map(&mv, a.v_cache, 4, dims, strides, box, "paged_attention(value_cache)",
                        CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != B200OPS_OK) return rc;
  } else {
    const uint64_t dims[4] = {static_cast<uint64_t>(kD), static_cast<uint64_t>(a.num_kv_heads),
                              static_cast<uint64_t>(a.page_size), static_cast<uint64_t>(a.num_pages)};
    const uint64_t strides[3] = {static_cast<uint64_t>(kD) * 2,
                                 static_cast<uint64_t>(a.num_kv_heads) * kD * 2,
                                 static_cast<uint64_t>(a.page_size) * a.num_kv_heads * kD * 2};
    const uint32_t box[4] = {64, 1, static_cast<uint32_t>(a.page_size < kTile ? a.page_size : kTile), 1};
    rc = encode_f16_map(&mk, a.k_cache, 4, dims, strides, box, "paged_attention(key_cache)");
    if (rc != B200OPS_OK) return rc;
    rc = encode_f16_map(&mv, a.v_cache, 4, dims, strides, box, "paged_attention(value_cache)");
    if (rc != B200OPS_OK) return rc;
  }
  const dim3 grid(a.max_chunks, a.num_kv_heads, a.bs);
  B200OPS_REQUIRE(grid.y <= 65535 && grid.z <= 65535,
                  "paged_attention: batch or head count too large for one launch");
  switch (knob(kKnobPaStages, 3)) {
    case 2: return launch_with_stages<2>(mk, mv, a, grid, st);
    case 4: return launch_with_stages<4>(mk, mv, a, grid, st);
    case 6: return launch_with_stages<6>(mk, mv, a, grid, st);
    default: return launch_with_stages<3>(mk, mv, a, grid, st);
  }
}

int fast_path_status_take() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_pa_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_pa_status, &zero, sizeof(int));
  }
  return v;
}

}  // namespace pa
}  // namespace b200ops
