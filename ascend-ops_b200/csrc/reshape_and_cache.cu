// reshape_and_cache for sm_100a: scatter this step's K/V rows into the paged KV cache.
//
// Pure address arithmetic plus 128-bit copies; results are bit-exact.  Two cache layouts:
//   NZ  [pages, C, P, 16] : cache[s/P, c, s%P, j] = flat(key[t])[c*16 + j]   (reference-native;
//        golden benchmark/test_reshape_and_cache.py:6-25, kernel
//        csrc/opdev/op_kernel/reshape_and_cache_ex.cpp:47-69)
//   NHD [pages, P, Hkv, D]: cache[s/P, s%P, h, d] = key[t, h, d]             (vLLM standard)
// Slots outside [0, pages*P) are skipped, as the reference kernel does (:50).  Where the
// reference lets every core copy all tokens element by element, here a warp moves one token's
// K and V rows in 32-byte pieces (rows of whole sectors), or each thread one 16-byte vector of
// K and the matching vector of V (other rows that are multiples of 8), or single elements.
//
// A slot named by two tokens: the reference walks the tokens in order, so the later token's
// row stays (:47-61).  Batches of up to kDedupMaxTokens tokens (every decode step) reproduce
// that: a token is skipped when a later token of the batch names its slot.  Larger batches do
// not pay for the check; there one of the rows that name the slot ends up in it, whole for the
// row-per-warp kernel (callers never do this: a slot is one cache position).
#include "common.cuh"

namespace b200ops {
namespace {

constexpr int kThreads = 256;

struct ScatterParams {
  const __half* key;
  const __half* value;
  __half* key_cache;
  __half* value_cache;
  const int32_t* slots;
  uint32_t num_tokens;
  uint32_t row_elems;   // Hkv * D
  uint32_t items_per_token;
  int64_t num_slots;    // pages * P
  uint32_t page_size;   // P
  uint32_t chunks;      // NZ: C
  bool dedup;           // small batch: a token whose slot a later token names again is skipped
  bool slots_vec;       // the slot array is 16-byte aligned
};

// The per-thread form of the check for the fallback kernels (odd row sizes; never on a hot path).
__device__ __forceinline__ bool thread_named_again(const int32_t* __restrict__ slots, uint32_t token,
                                                   uint32_t num_tokens, int32_t slot) {
  for (uint32_t t = token + 1; t < num_tokens; ++t)
    if (__ldg(slots + t) == slot) return true;
  return false;
}

// NHD: a token's destination is one contiguous row of row_elems halfs at slot * row_elems.
__global__ void __launch_bounds__(kThreads) scatter_nhd_vec_kernel(ScatterParams p) {
  pdl_trigger();
  pdl_wait();
  const uint32_t item = blockIdx.x * kThreads + threadIdx.x;
  const uint32_t token = item / p.items_per_token;
  if (token >= p.num_tokens) return;
  const uint32_t v = item - token * p.items_per_token;
  const int64_t slot = p.slots[token];
  if (slot < 0 || slot >= p.num_slots) return;
  if (p.dedup && thread_named_again(p.slots, token, p.num_tokens, static_cast<int32_t>(slot))) return;
  const size_t src = static_cast<size_t>(token) * p.items_per_token + v;
  const size_t dst = static_cast<size_t>(slot) * p.items_per_token + v;
  const uint4 kv = ld_stream(reinterpret_cast<const uint4*>(p.key) + src);
  if (p.value != nullptr) {
    const uint4 vv = ld_stream(reinterpret_cast<const uint4*>(p.value) + src);
    reinterpret_cast<uint4*>(p.value_cache)[dst] = vv;
  }
  reinterpret_cast<uint4*>(p.key_cache)[dst] = kv;
}

// NZ: vector v of the flat row belongs to chunk c = v/2 (16 halfs = two vectors per chunk).
__global__ void __launch_bounds__(kThreads) scatter_nz_vec_kernel(ScatterParams p) {
  pdl_trigger();
  pdl_wait();
  const uint32_t item = blockIdx.x * kThreads + threadIdx.x;
  const uint32_t token = item / p.items_per_token;
  if (token >= p.num_tokens) return;
  const uint32_t v = item - token * p.items_per_token;
  const uint32_t c = v >> 1;
  if (c >= p.chunks) return;
  const int64_t slot = p.slots[token];
  if (slot < 0 || slot >= p.num_slots) return;
  if (p.dedup && thread_named_again(p.slots, token, p.num_tokens, static_cast<int32_t>(slot))) return;
  const uint32_t page = static_cast<uint32_t>(slot / p.page_size);
  const uint32_t off = static_cast<uint32_t>(slot - static_cast<int64_t>(page) * p.page_size);
  const size_t src = static_cast<size_t>(token) * p.items_per_token + v;
  const size_t dst =
      ((static_cast<size_t>(page) * p.chunks + c) * p.page_size + off) * 2 + (v & 1u);
  const uint4 kv = ld_stream(reinterpret_cast<const uint4*>(p.key) + src);
  if (p.value != nullptr) {
    const uint4 vv = ld_stream(reinterpret_cast<const uint4*>(p.value) + src);
    reinterpret_cast<uint4*>(p.value_cache)[dst] = vv;
  }
  reinterpret_cast<uint4*>(p.key_cache)[dst] = kv;
}

// The repeated-slot check of one warp: is the token's slot named again by a later token?  The
// warp scans the rest of the batch's slots, four per load and kScanBatch loads per lane in
// flight, while the token's own rows are still on their way from DRAM.  The price is the extra
// load traffic (every warp reads up to the whole slot array through L1): about 1 us on a decode
// batch of 2048 tokens, 0.4 us on the NZ layout.  Issuing the scan loads before the slot is known
// does not help (measured), the volume is what costs.  `vec_ok`: the slot array is 16-byte
// aligned (otherwise single loads).
constexpr int kScanBatch = 8;

__device__ __forceinline__ bool named_again(const int32_t* __restrict__ slots, uint32_t token,
                                            uint32_t num_tokens, int32_t slot, uint32_t lane, bool vec_ok) {
  bool later = false;
  if (!vec_ok) {
#pragma unroll 4
    for (uint32_t t = token + 1 + lane; t < num_tokens; t += 32) later |= (__ldg(slots + t) == slot);
    return __any_sync(0xffffffffu, later);
  }
  const uint32_t full = num_tokens >> 2;  // complete groups of four slots
  const int4* s4 = reinterpret_cast<const int4*>(slots);
#pragma unroll 1
  for (uint32_t base = (token + 1) >> 2; base < full; base += 32 * kScanBatch) {
    int4 v[kScanBatch];
#pragma unroll
    for (int i = 0; i < kScanBatch; ++i) {
      const uint32_t g = base + lane + 32 * i;
      v[i] = g < full ? __ldg(s4 + g) : make_int4(-1, -1, -1, -1);  // -1 equals no valid slot
    }
#pragma unroll
    for (int i = 0; i < kScanBatch; ++i) {
      const uint32_t idx = (base + lane + 32 * i) << 2;  // only the first group can hold earlier tokens
      later |= (v[i].x == slot && idx > token) | (v[i].y == slot && idx + 1 > token) |
               (v[i].z == slot && idx + 2 > token) | (v[i].w == slot && idx + 3 > token);
    }
  }
  const uint32_t tail = (full << 2) + lane;  // the last one to three slots
  if (lane < (num_tokens & 3u) && tail > token) later |= (__ldg(slots + tail) == slot);
  return __any_sync(0xffffffffu, later);
}

constexpr int kDedupMaxTokens = 4096;

// Row-per-warp kernel for rows that are whole 32-byte sectors (row_elems % 16 == 0): a warp
// owns one token, every lane moves 32-byte pieces of the K row and of the V row.  All loads
// (including the slot) are issued before anything depends on them, so one DRAM round trip
// covers them; stores are one full sector each.  kMaxPieces bounds the
// pieces a lane holds.  (Giving a token's K row and V row to separate warps, and CTAs of 2, 8 or
// 16 warps, were measured: slower or equal at a decode batch of 2048 tokens.)
constexpr int kRowWarps = 4;
constexpr int kMaxPieces = 4;  // 32 lanes x 4 pieces x 32 B = rows up to 4 KB

template <bool kNz, bool kDedup>
__global__ void __launch_bounds__(kRowWarps * 32) scatter_rows_kernel(ScatterParams p) {
  pdl_trigger();
  pdl_wait();
  const uint32_t token = blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (token >= p.num_tokens) return;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t pieces = p.row_elems >> 4;  // 32-byte pieces (= NZ chunks) per row
  const char* ks = reinterpret_cast<const char*>(p.key) + static_cast<size_t>(token) * p.row_elems * 2;
  const char* vs = reinterpret_cast<const char*>(p.value) + static_cast<size_t>(token) * p.row_elems * 2;
  const int32_t slot32 = p.slots[token];
  Vec256 kb[kMaxPieces], vb[kMaxPieces];
#pragma unroll
  for (int i = 0; i < kMaxPieces; ++i) {
    const uint32_t c = lane + i * 32;
    if (c < pieces) {
      kb[i] = ld_stream256(ks + c * 32);
      if (p.value != nullptr) vb[i] = ld_stream256(vs + c * 32);
    }
  }
  const int64_t slot = slot32;
  if (slot < 0 || slot >= p.num_slots) return;
  if (kDedup && named_again(p.slots, token, p.num_tokens, slot32, lane, p.slots_vec)) return;
  size_t base, stride;  // byte offset of piece 0 and distance between pieces in the cache
  uint32_t limit = pieces;
  if (kNz) {
    const uint64_t page = static_cast<uint64_t>(slot) / p.page_size;
    const uint64_t off = static_cast<uint64_t>(slot) - page * p.page_size;
    base = (page * p.chunks * p.page_size + off) * 32;
    stride = static_cast<size_t>(p.page_size) * 32;
    limit = min(pieces, p.chunks);
  } else {
    base = static_cast<size_t>(slot) * p.row_elems * 2;
    stride = 32;
  }
  char* kc = reinterpret_cast<char*>(p.key_cache) + base;
  char* vc = reinterpret_cast<char*>(p.value_cache) + base;
#pragma unroll
  for (int i = 0; i < kMaxPieces; ++i) {
    const uint32_t c = lane + i * 32;
    if (c < limit) {
      st256(kc + c * stride, kb[i]);
      if (p.value != nullptr) st256(vc + c * stride, vb[i]);
    }
  }
}

// Any shape / alignment: one 16-bit element per item.
template <bool kNz>
__global__ void __launch_bounds__(kThreads) scatter_scalar_kernel(ScatterParams p) {
  pdl_trigger();
  pdl_wait();
  const uint64_t item = static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x;
  const uint64_t token = item / p.row_elems;
  if (token >= p.num_tokens) return;
  const uint32_t e = static_cast<uint32_t>(item - token * p.row_elems);
  const int64_t slot = p.slots[token];
  if (slot < 0 || slot >= p.num_slots) return;
  if (p.dedup && thread_named_again(p.slots, static_cast<uint32_t>(token), p.num_tokens, static_cast<int32_t>(slot)))
    return;
  size_t dst;
  if (kNz) {
    const uint32_t c = e >> 4;
    if (c >= p.chunks) return;
    const uint64_t page = static_cast<uint64_t>(slot) / p.page_size;
    const uint64_t off = static_cast<uint64_t>(slot) - page * p.page_size;
    dst = ((page * p.chunks + c) * p.page_size + off) * 16 + (e & 15u);
  } else {
    dst = static_cast<size_t>(slot) * p.row_elems + e;
  }
  const unsigned short* ks = reinterpret_cast<const unsigned short*>(p.key);
  reinterpret_cast<unsigned short*>(p.key_cache)[dst] = ks[item];
  if (p.value != nullptr) {
    const unsigned short* vs = reinterpret_cast<const unsigned short*>(p.value);
    reinterpret_cast<unsigned short*>(p.value_cache)[dst] = vs[item];
  }
}

}  // namespace
}  // namespace b200ops

extern "C" int b200ops_reshape_and_cache(const void* key, const void* value, void* key_cache,
                                         void* value_cache, const int32_t* slot_indices,
                                         int64_t num_tokens, int64_t num_kv_heads,
                                         int64_t head_size, const int64_t cache_dims[4],
                                         int layout, void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(num_tokens >= 0 && num_kv_heads > 0 && head_size > 0,
                  "reshape_and_cache: bad key shape [%lld, %lld, %lld]", (long long)num_tokens,
                  (long long)num_kv_heads, (long long)head_size);
  B200OPS_REQUIRE(cache_dims != nullptr, "reshape_and_cache: cache_dims is null");
  B200OPS_REQUIRE(layout == B200OPS_KV_LAYOUT_NZ || layout == B200OPS_KV_LAYOUT_NHD,
                  "reshape_and_cache: unknown cache layout %d", layout);
  for (int i = 0; i < 4; ++i)
    B200OPS_REQUIRE(cache_dims[i] > 0, "reshape_and_cache: key_cache must be 4D with positive sizes");
  const int64_t row_elems = num_kv_heads * head_size;
  B200OPS_REQUIRE(row_elems <= 0x7fffffffLL && num_tokens <= 0x7fffffffLL,
                  "reshape_and_cache: key too large");

  ScatterParams p;
  int64_t pages = cache_dims[0], page_size, chunks = 0;
  if (layout == B200OPS_KV_LAYOUT_NZ) {
    B200OPS_REQUIRE(cache_dims[3] == 16,
                    "reshape_and_cache: NZ cache must be [pages, chunks, page_size, 16], last size is %lld",
                    (long long)cache_dims[3]);
    chunks = cache_dims[1];
    page_size = cache_dims[2];
  } else {
    page_size = cache_dims[1];
    B200OPS_REQUIRE(cache_dims[2] == num_kv_heads && cache_dims[3] == head_size,
                    "reshape_and_cache: NHD cache must be [pages, page_size, %lld, %lld], got [.., .., %lld, %lld]",
                    (long long)num_kv_heads, (long long)head_size, (long long)cache_dims[2],
                    (long long)cache_dims[3]);
  }
  B200OPS_REQUIRE(page_size <= 0x7fffffffLL && chunks <= 0x7fffffffLL,
                  "reshape_and_cache: cache too large");
  if (num_tokens == 0) return B200OPS_OK;
  B200OPS_REQUIRE(key && key_cache && slot_indices, "reshape_and_cache: null pointer");

  const bool with_value = value != nullptr && value_cache != nullptr;
  p.key = static_cast<const __half*>(key);
  p.value = with_value ? static_cast<const __half*>(value) : nullptr;
  p.key_cache = static_cast<__half*>(key_cache);
  p.value_cache = with_value ? static_cast<__half*>(value_cache) : nullptr;
  p.slots = slot_indices;
  p.num_tokens = static_cast<uint32_t>(num_tokens);
  p.row_elems = static_cast<uint32_t>(row_elems);
  p.num_slots = pages * page_size;
  p.page_size = static_cast<uint32_t>(page_size);
  p.chunks = static_cast<uint32_t>(chunks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const bool aligned32 = ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(key_cache) |
                           (with_value ? reinterpret_cast<uintptr_t>(value) |
                                             reinterpret_cast<uintptr_t>(value_cache)
                                       : 0)) & 31u) == 0;
  p.dedup = num_tokens <= kDedupMaxTokens && knob(kKnobRacDedup, 1) != 0;
  p.slots_vec = aligned16(slot_indices);
  if (row_elems % 16 == 0 && row_elems <= 16 * 32 * kMaxPieces && aligned32) {
    const unsigned grid = static_cast<unsigned>((num_tokens + kRowWarps - 1) / kRowWarps);
    const bool nz = layout == B200OPS_KV_LAYOUT_NZ;
    auto kern = nz ? (p.dedup ? scatter_rows_kernel<true, true> : scatter_rows_kernel<true, false>)
                   : (p.dedup ? scatter_rows_kernel<false, true> : scatter_rows_kernel<false, false>);
    B200OPS_CUDA(launch_kernel(kern, dim3(grid), dim3(kRowWarps * 32), 0, st, p));
    return B200OPS_OK;
  }
  const bool vec_ok = row_elems % 8 == 0 && aligned16(key) && aligned16(key_cache) &&
                      (!with_value || (aligned16(value) && aligned16(value_cache)));
  const int64_t vec_items = num_tokens * (row_elems / 8);
  if (vec_ok && vec_items < 0x7fffff00LL) {
    p.items_per_token = static_cast<uint32_t>(row_elems / 8);
    const unsigned grid = static_cast<unsigned>((vec_items + kThreads - 1) / kThreads);
    B200OPS_CUDA(launch_kernel(layout == B200OPS_KV_LAYOUT_NZ ? scatter_nz_vec_kernel : scatter_nhd_vec_kernel, dim3(grid),
                        dim3(kThreads), 0, st, p));
    return B200OPS_OK;
  } else {
    p.items_per_token = 0;
    const int64_t items = num_tokens * row_elems;
    const int64_t grid = (items + kThreads - 1) / kThreads;
    B200OPS_REQUIRE(grid <= 0x7fffffffLL, "reshape_and_cache: key too large");
    B200OPS_CUDA(launch_kernel(layout == B200OPS_KV_LAYOUT_NZ ? scatter_scalar_kernel<true> : scatter_scalar_kernel<false>,
                        dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0, st, p));
  }
  return B200OPS_OK;
}
