// NT GEMM for decode-size dense projections: split-K over a thread-block cluster.
//
// Included by grouped_matmul.cu (inside namespace b200ops::gmm, after the shared definitions).
// A projection of a decode batch (a few hundred rows at most, K = 4096, N = 4096..6144) has
// only 16-48 output tiles of 128 x 256, and one CTA cannot pull more than about 120 GB/s through
// its shared memory: with a CTA per tile the weights stream at 1.4 TB/s.  Here the s CTAs of a
// cluster (s <= 8, chosen by the host so that tiles x s fills the SMs) share ONE output tile:
// CTA r multiplies k-slice r into its own TMEM accumulator, copies the fp32 tile into its
// shared memory (the operand ring, idle by then), and after a cluster barrier reduces the rows
// r, r + s, ... by reading all s copies through distributed shared memory, in rank order, so
// the result does not depend on timing.  The hardware co-schedules a cluster, so the barrier
// is a hardware one and there is no workspace, no counter and no spin.
// Single group only: the tile grid follows from the host's row bound; clusters whose rows do
// not exist leave at once.
#pragma once

constexpr int kSplitBN = kWideBN;
constexpr int kSplitStages = 4;
constexpr int kSplitBBytes = kSplitBN * BK * 2;
constexpr int kSplitStageBytes = kABytes + kSplitBBytes;
// With at most kShortRows rows the ring holds kShortStages stages of a short activation tile and
// the weight tile (see kShortRows): more weight bytes in flight per CTA.
constexpr int kSplitShortStageBytes = kShortABytes + kSplitBBytes;
constexpr int kSplitRingBytes = kShortStages * kSplitShortStageBytes > kSplitStages * kSplitStageBytes
                                    ? kShortStages * kSplitShortStageBytes
                                    : kSplitStages * kSplitStageBytes;
constexpr int kSplitTmemCols = kSplitBN;                       // one accumulator
constexpr int kSplitRowBytes = kSplitBN * 4;                   // an fp32 row of the partial tile
constexpr size_t kSplitSmemBytes = 1024 + kSplitRingBytes + sizeof(Control);
constexpr int kMaxClusterSplit = 8;                            // portable cluster size
static_assert(BM * kSplitRowBytes <= kSplitStages * kSplitStageBytes, "partial tile must fit the ring");
static_assert(kSplitSmemBytes <= 227 * 1024, "shared memory per CTA");
// How the launch chooses the activation tile's height: the host knows (rows <= kShortRows by its
// bound, or not), or the kernel reads the row count first (a loose bound: an expert-parallel
// receive buffer), which costs a load's latency before the first TMA.
constexpr int kSplitTilesFull = 0, kSplitTilesShort = 1, kSplitTilesByRowCount = 2;

__device__ __forceinline__ uint32_t cluster_size_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(r));
  return r;
}

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

// Byte offset of 16-byte chunk c4 of `row` in the partial tile.  The XOR spreads the 32 rows a
// warp writes at once (one row per lane, same chunk) over all banks.
__device__ __forceinline__ uint32_t partial_offset(int row, int c4) {
  return static_cast<uint32_t>(row) * kSplitRowBytes + static_cast<uint32_t>((c4 ^ (row & 31)) * 16);
}

// Sum rows rank, rank + s, ... of the cluster's s partial tiles (in rank order) and store them.
// All 192 threads: a thread owns one 16-byte chunk (4 output columns) of kRows rows per iteration
// and has all of their kPeers x kRows remote loads in flight before the first add: the step is a
// chain of distributed-shared-memory round trips of about 0.3 us otherwise.
template <int kPeers, int kRows>
__device__ __forceinline__ void reduce_rows(uint8_t* smem, int rank, int splits, int rows_here,
                                            const TileCoord& tc, __half* y, int N, const RowScatter& scatter) {
  const int t = threadIdx.x;               // 0..191
  const int c4 = t & 63;                   // 16-byte chunk = 4 output columns
  const bool col_ok = tc.n0 + c4 * 4 < N;  // N is a multiple of 64: chunks are all-or-nothing
  uint32_t peer_base[kPeers];
#pragma unroll
  for (int p = 0; p < kPeers; ++p) peer_base[p] = ptx::map_to_cta(smem, p < splits ? p : 0);
  const int step = (kThreads / 64) * splits;  // the three groups of 64 threads take owned rows in turn
  for (int row0 = rank + splits * (t >> 6); row0 < rows_here; row0 += kRows * step) {
    float4 v[kRows][kPeers];
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      const int row = min(row0 + j * step, BM - 1);
      const uint32_t off = partial_offset(row, c4);
#pragma unroll
      for (int p = 0; p < kPeers; ++p)
        v[j][p] = p < splits ? ld_cluster_f4(peer_base[p] + off) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      const int row = row0 + j * step;
      float4 acc = v[j][0];
#pragma unroll
      for (int p = 1; p < kPeers; ++p) {
        acc.x += v[j][p].x;
        acc.y += v[j][p].y;
        acc.z += v[j][p].z;
        acc.w += v[j][p].w;
      }
      bool row_ok = row < rows_here;
      __half* out_row = output_row(scatter, y, tc.row0 + row, N, row_ok);
      if (row_ok && col_ok) {
        uint2 o;
        o.x = f2_to_h2(acc.x, acc.y);
        o.y = f2_to_h2(acc.z, acc.w);
        *reinterpret_cast<uint2*>(out_row + tc.n0 + c4 * 4) = o;
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
grouped_matmul_ksplit_kernel(const __grid_constant__ CUtensorMap map_x,
                             const __grid_constant__ CUtensorMap map_x_short,
                             const __grid_constant__ CUtensorMap map_w,
                             const int64_t* __restrict__ group_list, __half* __restrict__ y, int M, int N,
                             int K, int E, const RowScatter scatter, const int tile_choice) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* a_tiles = smem;
  Control* ctl = reinterpret_cast<Control*>(smem + kSplitRingBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(ptx::cluster_ctarank());
  const int splits = static_cast<int>(cluster_size_x());
  const int tile = static_cast<int>(ptx::cluster_id_x());
  const int n_tiles = (N + kSplitBN - 1) / kSplitBN;
  const int k_blocks = K / BK;
  const int kb0 = static_cast<int>(static_cast<long long>(rank) * k_blocks / splits);
  const int kb1 = static_cast<int>(static_cast<long long>(rank + 1) * k_blocks / splits);

  // One group only (the host checks): tile -> (m-tile, n-tile) needs no table.  Tiles are
  // numbered m-tile by m-tile, so the clusters of the first m-tile are scheduled first.  They
  // always run, even before the row count is known (rows past the group's end are computed from
  // whatever x holds there and never stored).  Clusters of further m-tiles first read the row
  // count and leave if their rows do not exist: the host's row bound can be far above the rows
  // present (an expert-parallel receive buffer), and idle clusters must cost next to nothing.
  const int m_tiles = (M + BM - 1) / BM;
  const int m_tile = tile / n_tiles;
  pdl_trigger();
  TileCoord tc;
  tc.group = 0;
  tc.n0 = (tile - m_tile * n_tiles) * kSplitBN;
  tc.row0 = m_tile * BM;
  tc.row_end = 0;  // first m-tile: read after the first loads are on their way
  // splits <= k_blocks gives every rank at least one k-block; the host never asks otherwise.
  const bool may_run = splits <= k_blocks && tile < m_tiles * n_tiles;
  // Set-up that needs no input runs before the wait for the previous kernel, so that it overlaps
  // that kernel's tail: the barriers, and the TMEM allocation (warp 1, in parallel).
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&map_x);
    ptx::prefetch_tensormap(&map_x_short);
    ptx::prefetch_tensormap(&map_w);
    for (int s = 0; s < kShortStages; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    ptx::mbar_init(&ctl->tmem_full[0], 1);
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
  }
  if (may_run && warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, kSplitTmemCols);
    ptx::tmem_relinquish_alloc_permit();
  }
  pdl_wait();  // the row count and the loads below are inputs
  bool active = may_run;
  bool short_tiles = tile_choice == kSplitTilesShort;
  if (m_tile > 0 || tile_choice == kSplitTilesByRowCount) {
    long long rows = group_list ? group_list[0] : M;
    rows = rows > M ? M : rows;
    if (m_tile > 0) active = active && tc.row0 < rows;
    if (tile_choice == kSplitTilesByRowCount) short_tiles = rows <= kShortRows;  // the same in every CTA
  }
  // Ring geometry of this launch.
  const int stages = short_tiles ? kShortStages : kSplitStages;
  const int a_bytes = short_tiles ? kShortABytes : kABytes;
  const uint32_t stage_tx = static_cast<uint32_t>(a_bytes + kSplitBBytes);
  uint8_t* b_tiles = smem + stages * a_bytes;
  const CUtensorMap* x_map = short_tiles ? &map_x_short : &map_x;
  const int prefill = active ? min(stages, kb1 - kb0) : 0;
  if (threadIdx.x == 0) {
    // The first ring-full of loads needs nobody else: issue it before the CTA-wide barrier so
    // that its latency (about 2 us from HBM) overlaps it.
    for (int i = 0; i < prefill; ++i) {
      ptx::mbar_arrive_expect_tx(&ctl->full[i], stage_tx);
      ptx::tma_load_2d(a_tiles + i * a_bytes, x_map, &ctl->full[i], (kb0 + i) * BK, tc.row0);
      ptx::tma_load_3d(b_tiles + i * kSplitBBytes, &map_w, &ctl->full[i], (kb0 + i) * BK, tc.n0, 0);
    }
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();

  const uint32_t tmem_base = may_run ? ctl->tmem_base : 0u;
  volatile int* abort_flag = &ctl->abort_flag;
  {
    long long rows = group_list ? group_list[0] : M;
    rows = rows < 0 ? 0 : (rows > M ? M : rows);
    tc.row_end = static_cast<int>(rows);
  }

  if (active && warp == 0) {
    // ---------------- TMA producer (the rest of the k-slice) ----------------
    if (lane == 0) {
      int stage = prefill == stages ? 0 : prefill;
      uint32_t phase = prefill == stages ? 1u : 0u;
      for (int kb = kb0 + prefill; kb < kb1; ++kb) {
        if (!ptx::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_pipeline_status, 0, kErrProducerWait);
          break;
        }
        ptx::mbar_arrive_expect_tx(&ctl->full[stage], stage_tx);
        ptx::tma_load_2d(a_tiles + stage * a_bytes, x_map, &ctl->full[stage], kb * BK, tc.row0);
        ptx::tma_load_3d(b_tiles + stage * kSplitBBytes, &map_w, &ctl->full[stage], kb * BK, tc.n0, 0);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (active && warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_f16_idesc(BM, kSplitBN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!ptx::mbar_wait(&ctl->full[stage], phase, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_pipeline_status, 0, kErrMmaWaitFull);
          ok = false;
          break;
        }
        ptx::tcgen05_fence_after();
        const uint32_t a_addr = ptx::smem_u32(a_tiles + stage * a_bytes);
        const uint32_t b_addr = ptx::smem_u32(b_tiles + stage * kSplitBBytes);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint64_t a_desc = ptx::make_sw128_kmajor_desc(a_addr + k * UMMA_K * 2);
          const uint64_t b_desc = ptx::make_sw128_kmajor_desc(b_addr + k * UMMA_K * 2);
          ptx::umma_f16(tmem_base, a_desc, b_desc, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
        }
        ptx::umma_commit(&ctl->empty[stage]);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) ptx::umma_commit(&ctl->tmem_full[0]);
    }
  } else if (active) {
    // ---------------- accumulator -> shared memory (warps 2..5) ----------------
    // Once tmem_full completes, every load of this CTA has landed and every MMA has read its
    // operands: the ring is free to hold the fp32 tile.
    const int quarter = warp & 3;
    if (ptx::mbar_wait(&ctl->tmem_full[0], 0, abort_flag)) {
      ptx::tcgen05_fence_after();
      const int row = quarter * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < kSplitBN / 32; ++c) {
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 8; ++v)
          *reinterpret_cast<uint4*>(smem + partial_offset(row, c * 8 + v)) =
              make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
      }
    } else {
      *abort_flag = 1;
      atomicCAS(&g_pipeline_status, 0, kErrEpilogueWait);
    }
  }

  // All partial tiles of the cluster are in place (or the cluster has no tile at all).
  ptx::tcgen05_fence_before();
  __syncthreads();  // reconverges the single-lane roles before the warp-aligned cluster barrier
  ptx::cluster_sync();

  if (active) {
    const int rows_here = min(BM, tc.row_end - tc.row0);
    if (splits <= 2)
      reduce_rows<2, 8>(smem, rank, splits, rows_here, tc, y, N, scatter);
    else if (splits <= 4)
      reduce_rows<4, 4>(smem, rank, splits, rows_here, tc, y, N, scatter);
    else if (splits <= 6)
      reduce_rows<6, 3>(smem, rank, splits, rows_here, tc, y, N, scatter);
    else
      reduce_rows<kMaxClusterSplit, 2>(smem, rank, splits, rows_here, tc, y, N, scatter);
  }

  // Nobody leaves (and frees its shared memory) while a peer may still be reading it.
  __syncthreads();
  ptx::cluster_sync();
  if (may_run && warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kSplitTmemCols);
  }
}
