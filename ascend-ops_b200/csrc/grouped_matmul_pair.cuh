// Grouped NT GEMM, CTA-pair form: clusters of two CTAs run one tcgen05.mma of 256 x 256 x 16.
//
// Included by grouped_matmul.cu (inside namespace b200ops::gmm, after the shared definitions).
// Same semantics and output as grouped_matmul_kernel; used for problems bound by the tensor
// pipe (several waves of output tiles), where a single CTA's 128 x 256 tile has to pull 48 KB
// per k-block through L2 and shared memory.  In a pair each CTA loads only 32 KB per k-block
// for the same tensor work: its own 128 rows of x, and HALF of the 256-row w tile, which the
// tensor cores of both SMs read.
//
//   item        (group, n-tile of 256 columns, pair of m-tiles): CTA r of the cluster owns m-tile
//               2p + r.  A group with an odd number of m-tiles leaves CTA 1 of its last pair a
//               tile past the group's end: it multiplies whatever rows lie there and stores nothing.
//   warp 0      TMA producer in BOTH CTAs (own x rows, own half of w); completion is counted on
//               the even CTA's `full` barrier, which expects the bytes of both
//   warp 1      even CTA: MMA issuer for the pair; commits signal `empty` / `tmem_full` in both
//               CTAs.  Both CTAs: TMEM allocation (a pair-wide operation)
//   warps 2-5   epilogue in both CTAs, each on its own 128 accumulator rows; releases the
//               accumulator by arriving on the even CTA's `tmem_empty` (8 arrivals)
#pragma once

constexpr int kPairStages = 6;
constexpr int kPairBN = 256;
constexpr int kPairBHalfBytes = (kPairBN / 2) * BK * 2;            // this CTA's half of the w tile
constexpr int kPairStageBytes = kABytes + kPairBHalfBytes;         // 32 KB per CTA and k-block
constexpr int kPairTmemCols = 2 * kPairBN;
constexpr size_t kPairSmemBytes = 1024 + kPairStages * kPairStageBytes + sizeof(Control);

// Items of one group are numbered m-pair fastest, like the tiles of the single-CTA kernel.
__device__ __forceinline__ TileCoord locate_pair_item(const Control* c, int item, int& g, int rank, int out_bn) {
  while (item >= c->tile_prefix[g + 1]) ++g;
  const int local = item - c->tile_prefix[g];
  const int rows = c->row_end[g] - c->row_start[g];
  const int m_pairs = ((rows + BM - 1) / BM + 1) / 2;
  const int n_tile = local / m_pairs;
  const int m_pair = local - n_tile * m_pairs;
  TileCoord t;
  t.group = g;
  t.row0 = c->row_start[g] + (2 * m_pair + rank) * BM;
  t.row_end = c->row_end[g];
  t.n0 = n_tile * out_bn;
  return t;
}

// kGlu: the fused gate/up projection (see Cfg::kGlu): the even CTA's half of the w tile is the
// 128 gate rows, the odd CTA's half the 128 up rows of the same outputs, and each CTA's
// epilogue applies SwiGLU to its own 128 rows.
template <bool kGlu>
__global__ void __launch_bounds__(kThreads, 1)
grouped_matmul_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                           const __grid_constant__ CUtensorMap map_w,
                           const int64_t* __restrict__ group_list, __half* __restrict__ y, int M, int N,
                           int K, int E, const RowScatter scatter) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* a_tiles = smem;
  uint8_t* b_tiles = smem + kPairStages * kABytes;
  Control* ctl = reinterpret_cast<Control*>(smem + kPairStages * kPairStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(ptx::cluster_ctarank());
  const int cluster = static_cast<int>(ptx::cluster_id_x());
  const int n_clusters = static_cast<int>(ptx::num_clusters_x());
  constexpr int kOutBN = kGlu ? kPairBN / 2 : kPairBN;
  const int n_out = kGlu ? N / 2 : N;
  const int n_tiles = (n_out + kOutBN - 1) / kOutBN;
  const int k_blocks = K / BK;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      ptx::mbar_init(&ctl->full[s], 1);   // used in the even CTA: its producer's expect_tx
      ptx::mbar_init(&ctl->empty[s], 1);  // one commit arrival per CTA
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->tmem_full[i], 1);
      ptx::mbar_init(&ctl->tmem_empty[i], 8);  // used in the even CTA: 4 epilogue warps x 2 CTAs
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_x);
    ptx::prefetch_tensormap(&map_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(&ctl->tmem_base, kPairTmemCols);
    ptx::tmem_relinquish_alloc_permit_pair();
  }
  pdl_wait();  // set-up done; from here on the kernel reads its inputs
  for (int e = threadIdx.x; e < E; e += kThreads) {
    long long s = (e && group_list) ? group_list[e - 1] : 0;
    long long t = group_list ? group_list[e] : M;
    s = s < 0 ? 0 : (s > M ? M : s);
    t = t < s ? s : (t > M ? M : t);
    ctl->row_start[e] = static_cast<int>(s);
    ctl->row_end[e] = static_cast<int>(t);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    ctl->tile_prefix[0] = 0;
    for (int e = 0; e < E; ++e) {
      const int rows = ctl->row_end[e] - ctl->row_start[e];
      acc += (((rows + BM - 1) / BM + 1) / 2) * n_tiles;
      ctl->tile_prefix[e + 1] = acc;
    }
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // the peer's barriers are initialised before anything signals them
  ptx::tcgen05_fence_after();

  const int total_items = ctl->tile_prefix[E];
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0, g = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = cluster; ok && item < total_items; item += n_clusters) {
        const TileCoord tc = locate_pair_item(ctl, item, g, rank, kOutBN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ptx::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(&g_pipeline_status, 0, kErrProducerWait);
            ok = false;
            break;
          }
          const uint32_t lead_full = ptx::map_to_cta(&ctl->full[stage], 0);
          if (rank == 0) ptx::mbar_arrive_expect_tx(&ctl->full[stage], 2 * kPairStageBytes);
          ptx::tma_load_2d_pair(a_tiles + stage * kABytes, &map_x, lead_full, kb * BK, tc.row0);
          ptx::tma_load_3d_pair(b_tiles + stage * kPairBHalfBytes, &map_w, lead_full, kb * BK,
                                kGlu ? rank * n_out + tc.n0 : tc.n0 + rank * (kPairBN / 2), tc.group);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (rank == 0 && lane == 0) {
      constexpr uint32_t idesc = ptx::make_f16_idesc(2 * BM, kPairBN);
      constexpr uint16_t kBoth = 0x3;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int iter = 0;
      for (int item = cluster; ok && item < total_items; item += n_clusters, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!ptx::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_pipeline_status, 0, kErrMmaWaitTmem);
          break;
        }
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairBN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!ptx::mbar_wait(&ctl->full[stage], phase, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(&g_pipeline_status, 0, kErrMmaWaitFull);
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint32_t a_addr = ptx::smem_u32(a_tiles + stage * kABytes);
          const uint32_t b_addr = ptx::smem_u32(b_tiles + stage * kPairBHalfBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = ptx::make_sw128_kmajor_desc(a_addr + k * UMMA_K * 2);
            const uint64_t b_desc = ptx::make_sw128_kmajor_desc(b_addr + k * UMMA_K * 2);
            ptx::umma_f16_pair(d_tmem, a_desc, b_desc, idesc, (kb != 0 || k != 0) ? 1u : 0u);
          }
          ptx::umma_commit_pair(&ctl->empty[stage], kBoth);  // frees the stage in both CTAs
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) ptx::umma_commit_pair(&ctl->tmem_full[acc], kBoth);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5, both CTAs) ----------------
    const int quarter = warp & 3;
    int g = 0, iter = 0;
    for (int item = cluster; item < total_items; item += n_clusters, ++iter) {
      const TileCoord tc = locate_pair_item(ctl, item, g, rank, kOutBN);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!ptx::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag)) {
        *abort_flag = 1;
        atomicCAS(&g_pipeline_status, 0, kErrEpilogueWait);
        break;
      }
      ptx::tcgen05_fence_after();
      const int row = tc.row0 + quarter * 32 + lane;
      bool row_ok = row < tc.row_end;
      __half* yrow = output_row(scatter, y, row, n_out, row_ok) + tc.n0;
      const uint32_t taddr = tmem_base + acc * kPairBN + (static_cast<uint32_t>(quarter * 32) << 16);
      if constexpr (kGlu) glu_epilogue<kOutBN>(taddr, yrow, row_ok, tc.n0, n_out);
#pragma unroll 1
      for (int c = 0; !kGlu && c < kPairBN / 32; ++c) {
        if (tc.n0 + c * 32 >= N) break;
        uint32_t r[32];
        ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
        ptx::tmem_ld_wait();
        if (!row_ok) continue;
        uint4* dst = reinterpret_cast<uint4*>(yrow + c * 32);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 o;
          o.x = f2_to_h2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
          o.y = f2_to_h2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
          o.z = f2_to_h2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
          o.w = f2_to_h2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
          dst[v] = o;
        }
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(&ctl->tmem_empty[acc], 0));
    }
  }

  // Neither CTA may free its TMEM or leave while the pair's MMAs can still touch it.
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::cluster_sync();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, kPairTmemCols);
  }
}
