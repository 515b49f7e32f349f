// Grouped (per-expert) NT GEMM for sm_100a on the 5th-generation tensor cores.
//
//   y[gl[e-1]:gl[e], :] = x[gl[e-1]:gl[e], :] @ w[e],   w[e] stored [N, K] (K contiguous)
//
// Semantics follow the reference kernel (csrc/opdev/op_kernel/grouped_mat_mul_ex.cpp:29-44:
// inclusive cumulative ends, empty groups skipped) and its tile engine MatMulNT
// (csrc/opdev/op_kernel/matmul_core.h:43-68: fp16 operands, fp32 accumulation, fp16 result).
// The reference gives one core per expert and walks 64x64x64 tiles serially; this kernel
// is a persistent, warp-specialised pipeline over all SMs:
//
//   warp 0      TMA producer: x tile [128 x 64] and w tile [256 x 64] per k-block into a
//               4-stage ring of 128B-swizzled shared memory (48 KB per stage)
//   warp 1      MMA issuer: tcgen05.mma 128x256x16 (kind::f16), fp32 accumulators in TMEM,
//               two accumulator buffers (2 x 256 columns) so the epilogue of tile i overlaps
//               the main loop of tile i+1
//   warps 2-5   epilogue: tcgen05.ld of their TMEM lane quarter, fp32 -> fp16 (RNE), stores
//               predicated on the group's row end (an M-tail tile never writes into the next
//               group's rows; reading them is harmless)
//
// Balanced schedule.  Tiles handed out whole leave a ragged last wave (160 tiles of a long k on
// 148 SMs take two waves), and a problem with fewer tiles than SMs leaves SMs idle while each
// busy CTA streams its operands at the rate one SM can ingest.  If the caller passes a
// workspace, every CTA derives the same decision from the tile count it computed on the device:
// the full waves are handed out tile by tile as before, and the (tile, k-block) units of the
// ragged last wave are cut into one contiguous range per CTA.  The parts of a cut tile go to the
// workspace as fp32 partial tiles; a counter per tile identifies the last CTA to publish a part,
// and it alone sums the parts in CTA order and writes the fp16 rows (with SwiGLU applied for the
// fused gate/up form).  Nobody waits on another CTA.
//
// CTA pairs.  Problems of a wave of tiles or more run grouped_matmul_pair_kernel instead
// (grouped_matmul_pair.cuh): clusters of two CTAs issue one 256 x 256 x 16 MMA (cta_group::2), each
// CTA loading its own rows of x and half of the w tile.
//
// Cluster split-K.  A single group of at most 256 rows (the dense projections of a decode batch)
// runs grouped_matmul_ksplit_kernel (grouped_matmul_ksplit.cuh): the CTAs of a cluster share one
// output tile and reduce their k-slices through distributed shared memory, without a workspace.
//
// Short activation tiles.  When no group has more than 80 rows (a decode batch) the x tile is
// loaded 80 rows high and the ring has five stages of 42 KB: such problems are bound by the
// weight bytes a CTA has in flight (see kShortRows).
//
// SwiGLU epilogue.  Cfg<.., true> and grouped_matmul_pair_kernel<true> compute the gate/up
// projection of a gated MLP and apply SwiGLU before storing (b200ops_grouped_matmul_swiglu).
//
// Tiles are enumerated group by group, m-tile fastest, so that CTAs running at the same
// time share the same w tile (read from HBM once, then from L2) while the group's x rows
// stay L2-resident.  Work is 2*M*K*N flops; at the sizes of interest the kernel is bound by
// the tensor pipe, at decode sizes (few rows per expert) by streaming w from HBM once.
#include <atomic>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace b200ops {
namespace gmm {

constexpr int BM = 128;
constexpr int kWideBN = 256;    // output tile width of the throughput configuration
constexpr int kNarrowBN = 64;   // single m-tile problems: four times as many CTAs stream the weights
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kMaxStages = 8;
constexpr int kThreads = 192;
constexpr int kMaxExperts = 1024;

constexpr int kABytes = BM * BK * 2;

// Error codes left in the device status word.
constexpr int kErrProducerWait = 1;
constexpr int kErrMmaWaitFull = 2;
constexpr int kErrMmaWaitTmem = 3;
constexpr int kErrEpilogueWait = 4;
constexpr int kMinKBlocksPerSplit = 4;  // keep every k-slice long enough to fill the ring
constexpr int kMaxPartsSplitK = 8;      // parts of one tile: few rows per tile, small partial tiles
constexpr int kMaxPartsEvenOut = 4;     // parts of one tile when tiles are full (128 KB per part)
constexpr int kEvenOutMinSavedKBlocks = 80;  // cut the last wave only if it saves more tensor time than this

// Workspace layout (used by the balanced schedule): one counter per tile, then two fp32 partial
// tiles of BM x BN per CTA (a CTA's range has at most two incomplete tiles, see partial_slot).
constexpr int kMaxGrid = 256;
constexpr int kBalancedWaves = 16;  // the host offers the workspace below this many waves of tiles (by its row bound)
constexpr size_t kPartialTileBytes = static_cast<size_t>(BM) * kWideBN * sizeof(float);
constexpr size_t kCounterBytes = static_cast<size_t>(kBalancedWaves) * kMaxGrid * sizeof(int);

// A k range shorter than this does not amortise the publish-and-sum tail of split-K proper
// (fewer tiles than half the CTAs).
constexpr int64_t kMinSplitK = 8192;

// Narrow tiles: one m-tile of rows at most, wide tiles would occupy under a quarter of the SMs,
// and K too short for split-K (which wins where both apply).
inline bool use_narrow_tiles(int64_t num_tokens, int64_t k, int64_t n, int sms) {
  return num_tokens <= BM && ((n + kWideBN - 1) / kWideBN) * 4 <= sms && k < kMinSplitK;
}

// CTA pairs (grouped_matmul_pair.cuh): for problems bound by the tensor pipe and not by streaming
// the weights once -- at least one wave of 128 x 256 output tiles, and two m-tiles per expert on
// average (with one m-tile per expert the second CTA of every pair would multiply nothing useful).
// The row count the host sees is only a bound (an expert-parallel receive buffer holds a fraction
// of it at decode time, where the pair kernel is slower than the single-CTA one), hence also an
// absolute floor on it.  B200OPS_GMM_PAIR: 0 = never, 2 = always (tests), otherwise this rule.
constexpr int64_t kMinRowsForPairs = 2048;
inline int pair_mode() { return knob(kKnobGmmPair, 1); }

inline bool use_cta_pairs(int64_t num_tokens, int64_t num_experts, int64_t n, int sms) {
  const int mode = pair_mode();
  if (mode == 0) return false;
  if (mode == 2) return true;
  const int64_t n_tiles = (n + kWideBN - 1) / kWideBN;
  const int64_t min_tiles = ((num_tokens + BM - 1) / BM) * n_tiles;
  return min_tiles >= sms && num_tokens >= 2 * BM * num_experts && num_tokens >= kMinRowsForPairs;
}

// Cluster split-K (grouped_matmul_ksplit.cuh), single group only.  Two cases:
//  * at most 256 rows (a dense projection of a decode batch, whose row count the host knows)
//    and so few output tiles that at least two CTAs can share each;
//  * a row BOUND of up to 1024 with K >= 8192 (the down projection of a rank that hosts one
//    expert: the bound is the receive buffer, the rows present are about a tile's worth): the
//    cluster size is chosen for the tiles of the first m-tile, further m-tiles run as extra waves.
// Returns the wanted cluster size (0 = not this path) and the tile count that must be resident.
// B200OPS_GMM_KSPLIT=0 disables the path.
constexpr int kMaxClusterSplitRows = 256;
constexpr int kMaxClusterSplitRowBound = 1024;
constexpr int kMaxClusterSplitHost = 8;

inline int cluster_split_factor(int64_t num_tokens, int64_t k, int64_t num_experts, int64_t n, int sms,
                                int64_t* resident_tiles) {
  if (knob(kKnobGmmKsplit, 1) == 0) return 0;
  if (num_experts != 1) return 0;
  const int64_t n_tiles = (n + kWideBN - 1) / kWideBN;
  int64_t tiles;
  if (num_tokens <= kMaxClusterSplitRows)
    tiles = ((num_tokens + BM - 1) / BM) * n_tiles;
  else if (num_tokens <= kMaxClusterSplitRowBound && k >= kMinSplitK)
    tiles = n_tiles;
  else
    return 0;
  int64_t s = sms / tiles;
  if (s > kMaxClusterSplitHost) s = kMaxClusterSplitHost;
  if (s > (k / BK) / kMinKBlocksPerSplit) s = (k / BK) / kMinKBlocksPerSplit;
  *resident_tiles = tiles;
  return s >= 2 ? static_cast<int>(s) : 0;
}

inline int launch_sms() { return sm_count() < kMaxGrid ? sm_count() : kMaxGrid; }

inline size_t workspace_bytes() { return kCounterBytes + 2 * static_cast<size_t>(launch_sms()) * kPartialTileBytes; }

// Host-side gate of the balanced schedule, shared by the size query and the launch: a workspace
// is worth having when the tile count (by the host's row bound, an upper bound of the real
// one) is within kBalancedWaves waves.  The kernel decides with the real count.
inline bool balanced_possible(int64_t num_tokens, int64_t k, int64_t num_experts, int64_t n, int sms) {
  const int64_t n_tiles = (n + kWideBN - 1) / kWideBN;
  const int64_t max_tiles = ((num_tokens + BM - 1) / BM + num_experts) * n_tiles;
  return k >= 1024 && max_tiles < static_cast<int64_t>(kBalancedWaves) * sms;
}

// Short activation tiles.  When no group has more than kShortRows rows (a decode batch: one
// m-tile per expert, mostly half empty) the 256-column kernels load only kShortRows rows of x per
// k-block and use the room for a fifth stage.  Such a problem streams its weights once and is
// bound by the bytes a CTA has in flight (about 3 us pass between a load's issue and the release
// of its stage): with 48 KB stages a third of them are the activation tile, an L2 hit, and the
// weights stream at 6.0 TB/s; with 10 + 32 KB stages, five of them, 160 KB of weights are in
// flight instead of 128.  The MMA still multiplies 128 rows: rows past the box are whatever the
// next stage holds, and are never stored.  Decided on the device from the real group sizes.
constexpr int kShortRows = 80;
constexpr int kShortABytes = kShortRows * BK * 2;
constexpr int kShortStages = 5;

struct Control {
  int short_tiles;  // this launch runs with short activation tiles
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int split_rank;  // arrival order of this CTA among the parts of its tile
  int live_groups;  // groups that hold rows
  int part_slot[kMaxGrid];  // workspace slots of a tile's parts, in CTA order (reducing CTA only)
  int tile_prefix[kMaxExperts + 1];  // first tile id of each group; [E] = total tiles
  int row_start[kMaxExperts];
  int row_end[kMaxExperts];
};

// Tile configuration: BM x BN_ output tile, STAGES_-deep ring of (A 16 KB + B BN_*128 B) stages,
// two fp32 accumulators of BN_ TMEM columns.  <256, 4> is the throughput shape (48 KB stages).
// <64, 8> (24 KB stages, the same 192 KB in flight) is for problems whose rows fit ONE m-tile and
// whose wide tiles would occupy under a quarter of the SMs (decode-size dense projections): a
// CTA can only pull about 100 GB/s through its ring, so four times as many CTAs stream the
// weights four times as fast.  With more than one m-tile the narrow shape loses (two thirds of
// every stage is the re-read activation tile), so it is not used there.
template <int BN_, int STAGES_, bool GLU_ = false>
struct Cfg {
  static constexpr int BN = BN_;
  static constexpr int kStages = STAGES_;
  // GLU_: the gate/up projection with SwiGLU in the epilogue.  The 256 accumulator columns of a
  // tile are 128 gate columns and the 128 up columns of the SAME outputs (two 128-row boxes of
  // w, at n0 and at d + n0); the epilogue rounds both to fp16, as the unfused GEMM would have
  // stored them, applies (g * sigmoid(g)) * u and writes 128 columns.
  static constexpr bool kGlu = GLU_;
  static constexpr int kOutBN = GLU_ ? BN_ / 2 : BN_;
  static constexpr int kBBytes = BN_ * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN_ < 32 ? 32 : 2 * BN_;  // a power of two >= 32
  static constexpr bool kShortCapable = BN_ == kWideBN;  // the narrow shape's stages are small already
  static constexpr int kShortStageBytes = kShortABytes + kBBytes;
  static constexpr int kRingBytes = (kShortCapable && kShortStages * kShortStageBytes > STAGES_ * kStageBytes)
                                        ? kShortStages * kShortStageBytes
                                        : STAGES_ * kStageBytes;
  static constexpr size_t kSmemBytes = 1024 /* alignment slack */ + kRingBytes + sizeof(Control);
  static_assert(kSmemBytes <= 227 * 1024, "shared memory per CTA");
};
using WideCfg = Cfg<kWideBN, 4>;
using NarrowCfg = Cfg<kNarrowBN, 8>;
using GluCfg = Cfg<kWideBN, 4, true>;

// Sticky per-device status of the pipeline kernels (0 = no failure).
__device__ int g_pipeline_status = 0;

struct TileCoord {
  int group, row0, row_end, n0;
};

// Optional output redirection: row r of the result is not written to y[r] but into the buffer
// of rank index[r] / cap, at row my_rank * cap + index[r] % cap -- the return leg of the
// expert-parallel exchange fused into the GEMM's epilogue (plain stores through the NVLink
// peer mapping).  index == nullptr: ordinary output.
struct RowScatter {
  const int32_t* index;
  PeerTable peers;
  int cap, my_rank, world;
};

__device__ __forceinline__ __half* output_row(const RowScatter& sc, __half* y, int row, int N, bool& ok) {
  if (sc.index == nullptr) return y + static_cast<size_t>(row) * N;
  const int idx = ok ? sc.index[row] : -1;
  if (idx < 0) {
    ok = false;
    return y;
  }
  const int peer = idx / sc.cap, off = idx - peer * sc.cap;
  if (peer >= sc.world) {  // an index outside the exchange's geometry names no buffer
    ok = false;
    return y;
  }
  return static_cast<__half*>(sc.peers.base[peer]) + (static_cast<size_t>(sc.my_rank) * sc.cap + off) * N;
}

// Work decomposition.  Tiles are numbered as locate_tile numbers them; a unit is one k-block
// of one tile.  Two schedules:
//   by tiles    CTA c takes tiles c, c + G, ... whole (no workspace needed).  CTAs that run at the
//               same time work on neighbouring tiles, which share weight tiles through L2.
//   balanced    the full waves of G tiles are handed out as above; the tiles of the ragged last
//               wave are cut, as (tile, k-block) units, into equal contiguous ranges, one per CTA.
//               A range covers the end of one tile and/or the start of the next: both are parts
//               that go through the workspace (see the epilogue).  160 tiles of a long k on 148
//               SMs are two waves by tiles, 1.08 balanced.  With fewer tiles than CTAs this is
//               split-K.  Ranges are kept at least kMinKBlocksPerSplit k-blocks long.
//               (Cutting ALL units into one range per CTA balances as well but lets every CTA walk
//               its own stretch of the tile sequence: 148 weight tiles are then live at once,
//               more than L2 holds, and the re-reads by a weight tile's other m-tiles go to HBM --
//               measured 1.7 times slower on three experts of 350 rows.)
struct Segment {
  int tile, kb0, kb1;
};

struct Schedule {
  int k_blocks, total_tiles, grid;
  int whole_tiles;       // tiles [0, whole_tiles) are handed out whole, round-robin
  long long tail_units;  // balanced: units of the tiles [whole_tiles, total_tiles)
  int tail_ctas;         // balanced: CTAs that take a range of them
  bool balanced;
  // Ranges of the tail, in units counted from the first tail tile.
  __device__ __forceinline__ long long first_unit(int c) const { return tail_units * c / tail_ctas; }
  // The CTA whose range holds unit u: the largest c with first_unit(c) <= u.
  __device__ __forceinline__ int cta_of(long long u) const {
    return static_cast<int>(((u + 1) * tail_ctas + tail_units - 1) / tail_units) - 1;
  }
};

__device__ __forceinline__ Schedule make_schedule(int total_tiles, int k_blocks, int grid, bool have_workspace,
                                                  int weight_tiles) {
  Schedule s;
  s.k_blocks = k_blocks;
  s.total_tiles = total_tiles;
  s.grid = grid;
  s.whole_tiles = total_tiles;
  s.tail_units = 0;
  s.tail_ctas = 0;
  const int tail = total_tiles % grid;
  // Fewer tiles than half the CTAs is split-K proper, whose publish-and-sum tail only pays for a
  // long k (kMinSplitK).  With more tiles, cutting the last wave pays when (a) CTAs run at their
  // own pace, i.e. the tensor pipe is the limit: every weight tile (`weight_tiles` of them: one per
  // group with rows and column block) is used by two m-tiles or more on average -- with one
  // m-tile per weight tile (decode batches) the kernel streams weights at the HBM rate, the CTAs
  // of a ragged last wave simply run faster, and cutting tiles only adds traffic -- and (b) the
  // k-blocks saved exceed the price of summing a cut tile: the CTA that sums reads every part
  // (128 KB each) at the rate of a chain of L2 round trips, about 4 us per part or 10 k-blocks'
  // worth of tensor time.  Hence also the cap on the parts of a tile.
  const bool split_k = 2 * total_tiles <= grid && k_blocks * BK >= kMinSplitK;
  const int parts_cap = split_k ? kMaxPartsSplitK : kMaxPartsEvenOut;
  const long long want = static_cast<long long>(tail) * parts_cap;
  int ctas = want < grid ? static_cast<int>(want) : grid;
  const long long most = static_cast<long long>(tail) * k_blocks / kMinKBlocksPerSplit;
  if (most < ctas) ctas = most < 1 ? 1 : static_cast<int>(most);
  const int range = ctas > 0 ? static_cast<int>((static_cast<long long>(tail) * k_blocks + ctas - 1) / ctas) : k_blocks;
  const bool even_out = 2 * total_tiles > grid && total_tiles < 8 * grid && total_tiles >= 2 * weight_tiles &&
                        k_blocks - range > kEvenOutMinSavedKBlocks;
  s.balanced = have_workspace && tail != 0 && (split_k || even_out);
  if (s.balanced) {
    s.whole_tiles = total_tiles - tail;
    s.tail_units = static_cast<long long>(tail) * k_blocks;
    s.tail_ctas = ctas;
  }
  return s;
}

// Workspace slot of a part: a CTA's range has at most one part that starts inside a tile (its
// first segment) and at most one that starts a tile without finishing it (its last).
__device__ __forceinline__ int partial_slot(int cta, int kb0) { return 2 * cta + (kb0 == 0 ? 1 : 0); }

struct Walk {
  const Schedule& s;
  int tile;          // next whole tile of this CTA
  long long lo, hi;  // remaining units of its tail range
  __device__ __forceinline__ Walk(const Schedule& sched, int cta) : s(sched), tile(cta), lo(0), hi(0) {
    if (s.balanced && cta < s.tail_ctas) {
      lo = s.first_unit(cta);
      hi = s.first_unit(cta + 1);
    }
  }
  __device__ __forceinline__ bool next(Segment& g) {
    if (tile < s.whole_tiles) {
      g.tile = tile;
      g.kb0 = 0;
      g.kb1 = s.k_blocks;
      tile += s.grid;
      return true;
    }
    if (lo >= hi) return false;
    const int t = static_cast<int>(lo / s.k_blocks);
    const long long t0 = static_cast<long long>(t) * s.k_blocks;
    const long long end = hi < t0 + s.k_blocks ? hi : t0 + s.k_blocks;
    g.tile = s.whole_tiles + t;
    g.kb0 = static_cast<int>(lo - t0);
    g.kb1 = static_cast<int>(end - t0);
    lo = end;
    return true;
  }
};

// Tiles of one group are numbered m-fastest.  `g` is carried between calls: tile ids only
// grow within a CTA, so the search is amortised O(1).
__device__ __forceinline__ TileCoord locate_tile(const Control* c, int tile, int& g, int bn) {
  while (tile >= c->tile_prefix[g + 1]) ++g;
  const int local = tile - c->tile_prefix[g];
  const int rows = c->row_end[g] - c->row_start[g];
  const int m_tiles = (rows + BM - 1) / BM;
  const int n_tile = local / m_tiles;
  const int m_tile = local - n_tile * m_tiles;
  TileCoord t;
  t.group = g;
  t.row0 = c->row_start[g] + m_tile * BM;
  t.row_end = c->row_end[g];
  t.n0 = n_tile * bn;
  return t;
}

// Epilogue of the fused gate/up projection: this thread's accumulator row holds kOut gate columns
// followed by the kOut up columns of the same outputs.  Both are rounded to fp16 first -- the
// values the unfused GEMM would have stored and SwiGLU would have read -- so the result is
// bit-identical to grouped_matmul followed by swiglu.
template <int kOut>
__device__ __forceinline__ void glu_epilogue(uint32_t taddr, __half* yrow, bool row_ok, int n0, int n_out) {
#pragma unroll 1
  for (int c = 0; c < kOut / 32; ++c) {
    if (n0 + c * 32 >= n_out) break;  // n_out is a multiple of 32: chunks are all-or-nothing
    uint32_t g[32], u[32];
    ptx::tmem_ld_32x32b_x32(taddr + c * 32, g);
    ptx::tmem_ld_32x32b_x32(taddr + kOut + c * 32, u);
    ptx::tmem_ld_wait();
    if (!row_ok) continue;
    uint4* dst = reinterpret_cast<uint4*>(yrow + c * 32);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = v * 8 + j * 2;
        const float2 gf = h2_to_f2(f2_to_h2(__uint_as_float(g[i]), __uint_as_float(g[i + 1])));
        const float2 uf = h2_to_f2(f2_to_h2(__uint_as_float(u[i]), __uint_as_float(u[i + 1])));
        o[j] = f2_to_h2(silu_mul(gf.x, uf.x), silu_mul(gf.y, uf.y));
      }
      dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Sum the parts of one output tile (fp32 partial tiles in the workspace, `slots` in CTA order) and
// store its rows.  Run by the 128 epilogue threads of the CTA that published the tile's last
// part.  Warp `quarter` takes rows quarter, quarter + 4, ...; a row is read and written by one
// warp, coalesced.  Four rows and two parts are loaded before anything is added, so each lane
// keeps sixteen 16-byte loads in flight: the step is a chain of L2 round trips otherwise.
// kGlu: the tile's first BN / 2 columns are gate columns, the rest the up columns of the same
// outputs; sums are rounded to fp16 and SwiGLU applied as in glu_epilogue.
template <int BN, bool kGlu>
__device__ __forceinline__ void reduce_parts(const float* __restrict__ partials, const int* slots, int parts,
                                             int rows_here, int quarter, int lane, const TileCoord& tc,
                                             __half* y, int y_cols, const RowScatter& scatter) {
  constexpr int kPerLane = kGlu ? 4 : 8;           // accumulator columns per lane and operand half
  constexpr int kHalves = kGlu ? 2 : 1;            // gate + up, or one run of columns
  constexpr int kVecs = kPerLane / 4;              // float4 loads per half
  const int col = lane * kPerLane;
  if (col >= (kGlu ? BN / 2 : BN) || tc.n0 + col >= y_cols) return;  // widths are multiples of 64
  for (int r0 = quarter; r0 < rows_here; r0 += 16) {
    float acc[4][kHalves][kPerLane];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int h = 0; h < kHalves; ++h)
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) acc[j][h][i] = 0.f;
    for (int s0 = 0; s0 < parts; s0 += 2) {
      float4 v[2][4][kHalves][kVecs];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int rr = r0 + 4 * j;
          const bool live = s0 + u < parts && rr < rows_here;
          const float* base =
              live ? partials + static_cast<size_t>(slots[s0 + u]) * (BM * BN) + rr * BN + col : nullptr;
#pragma unroll
          for (int h = 0; h < kHalves; ++h)
#pragma unroll
            for (int q = 0; q < kVecs; ++q)
              v[u][j][h][q] = live ? __ldcg(reinterpret_cast<const float4*>(base + h * (BN / 2)) + q)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int h = 0; h < kHalves; ++h)
#pragma unroll
            for (int q = 0; q < kVecs; ++q) {
              acc[j][h][4 * q + 0] += v[u][j][h][q].x;
              acc[j][h][4 * q + 1] += v[u][j][h][q].y;
              acc[j][h][4 * q + 2] += v[u][j][h][q].z;
              acc[j][h][4 * q + 3] += v[u][j][h][q].w;
            }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int rr = r0 + 4 * j;
      bool out_ok = rr < rows_here;
      __half* out_row = output_row(scatter, y, tc.row0 + rr, y_cols, out_ok);
      if (!out_ok) continue;
      if constexpr (kGlu) {
        uint32_t o[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const float2 gf = h2_to_f2(f2_to_h2(acc[j][0][2 * q], acc[j][0][2 * q + 1]));
          const float2 uf = h2_to_f2(f2_to_h2(acc[j][1][2 * q], acc[j][1][2 * q + 1]));
          o[q] = f2_to_h2(silu_mul(gf.x, uf.x), silu_mul(gf.y, uf.y));
        }
        *reinterpret_cast<uint2*>(out_row + tc.n0 + col) = make_uint2(o[0], o[1]);
      } else {
        uint4 o;
        o.x = f2_to_h2(acc[j][0][0], acc[j][0][1]);
        o.y = f2_to_h2(acc[j][0][2], acc[j][0][3]);
        o.z = f2_to_h2(acc[j][0][4], acc[j][0][5]);
        o.w = f2_to_h2(acc[j][0][6], acc[j][0][7]);
        *reinterpret_cast<uint4*>(out_row + tc.n0 + col) = o;
      }
    }
  }
}

#include "grouped_matmul_pair.cuh"
#include "grouped_matmul_ksplit.cuh"

template <class C>
__global__ void __launch_bounds__(kThreads, 1)
grouped_matmul_kernel(const __grid_constant__ CUtensorMap map_x,
                      const __grid_constant__ CUtensorMap map_x_short,
                      const __grid_constant__ CUtensorMap map_w,
                      const int64_t* __restrict__ group_list, __half* __restrict__ y, int M, int N,
                      int K, int E, int* __restrict__ tile_counters, float* __restrict__ partials,
                      const RowScatter scatter, const int allow_short) {
  constexpr int BN = C::BN;
  constexpr int kStages = C::kStages;
  constexpr int kBBytes = C::kBBytes;
  constexpr int kTmemCols = C::kTmemCols;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* a_tiles = smem;
  Control* ctl = reinterpret_cast<Control*>(smem + C::kRingBytes);

  constexpr bool kGlu = C::kGlu;
  constexpr int kOutBN = C::kOutBN;  // output columns per tile
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_out = kGlu ? N / 2 : N;  // columns of y (N counts the rows of w)
  const int n_tiles = (n_out + kOutBN - 1) / kOutBN;
  const int k_blocks = K / BK;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < (kStages > kShortStages ? kStages : kShortStages); ++s) {
      ptx::mbar_init(&ctl->full[s], 1);
      ptx::mbar_init(&ctl->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&ctl->tmem_full[i], 1);
      ptx::mbar_init(&ctl->tmem_empty[i], 4);  // one arrival per epilogue warp
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_x);
    ptx::prefetch_tensormap(&map_x_short);
    ptx::prefetch_tensormap(&map_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&ctl->tmem_base, kTmemCols);
    ptx::tmem_relinquish_alloc_permit();
  }
  pdl_wait();  // set-up done; from here on the kernel reads its inputs
  // Group table: clamp the cumulative ends into [0, M] and count m-tiles per group.
  for (int e = threadIdx.x; e < E; e += kThreads) {
    long long s = (e && group_list) ? group_list[e - 1] : 0;
    long long t = group_list ? group_list[e] : M;  // no group list: one group of all M rows
    s = s < 0 ? 0 : (s > M ? M : s);
    t = t < s ? s : (t > M ? M : t);
    ctl->row_start[e] = static_cast<int>(s);
    ctl->row_end[e] = static_cast<int>(t);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, live = 0, most = 0;
    ctl->tile_prefix[0] = 0;
    for (int e = 0; e < E; ++e) {
      const int rows = ctl->row_end[e] - ctl->row_start[e];
      acc += ((rows + BM - 1) / BM) * n_tiles;
      live += rows > 0;
      most = rows > most ? rows : most;
      ctl->tile_prefix[e + 1] = acc;
    }
    ctl->live_groups = live;
    ctl->short_tiles = C::kShortCapable && allow_short != 0 && most <= kShortRows;
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();

  const int total_tiles = ctl->tile_prefix[E];
  // Ring geometry of this launch (the same in every CTA: it follows from the group sizes).
  const bool short_tiles = ctl->short_tiles != 0;
  const int stages = short_tiles ? kShortStages : kStages;
  const int a_bytes = short_tiles ? kShortABytes : kABytes;
  const uint32_t stage_tx = static_cast<uint32_t>(a_bytes + kBBytes);
  uint8_t* b_tiles = smem + stages * a_bytes;
  const CUtensorMap* x_map = short_tiles ? &map_x_short : &map_x;
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  // Every role walks the same sequence of segments (tile, k-blocks [kb0, kb1)); the schedule
  // depends only on the tile count, so all CTAs agree on it.
  const Schedule sched = make_schedule(total_tiles, k_blocks, static_cast<int>(gridDim.x), partials != nullptr,
                                       n_tiles * ctl->live_groups);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0, g = 0;
      uint32_t phase = 0;
      bool ok = true;
      Walk walk(sched, static_cast<int>(blockIdx.x));
      Segment sg;
      while (ok && walk.next(sg)) {
        const TileCoord tc = locate_tile(ctl, sg.tile, g, kOutBN);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!ptx::mbar_wait(&ctl->empty[stage], phase ^ 1u, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(&g_pipeline_status, 0, kErrProducerWait);
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(&ctl->full[stage], stage_tx);
          ptx::tma_load_2d(a_tiles + stage * a_bytes, x_map, &ctl->full[stage], kb * BK, tc.row0);
          if (kGlu) {  // gate rows, then the up rows of the same outputs (boxes of BN / 2 rows)
            ptx::tma_load_3d(b_tiles + stage * kBBytes, &map_w, &ctl->full[stage], kb * BK, tc.n0, tc.group);
            ptx::tma_load_3d(b_tiles + stage * kBBytes + kBBytes / 2, &map_w, &ctl->full[stage], kb * BK,
                             n_out + tc.n0, tc.group);
          } else
          ptx::tma_load_3d(b_tiles + stage * kBBytes, &map_w, &ctl->full[stage], kb * BK, tc.n0,
                           tc.group);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_f16_idesc(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int iter = 0;
      Walk walk(sched, static_cast<int>(blockIdx.x));
      Segment sg;
      for (; ok && walk.next(sg); ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!ptx::mbar_wait(&ctl->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
          *abort_flag = 1;
          atomicCAS(&g_pipeline_status, 0, kErrMmaWaitTmem);
          break;
        }
        ptx::tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!ptx::mbar_wait(&ctl->full[stage], phase, abort_flag)) {
            *abort_flag = 1;
            atomicCAS(&g_pipeline_status, 0, kErrMmaWaitFull);
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after();
          const uint32_t a_addr = ptx::smem_u32(a_tiles + stage * a_bytes);
          const uint32_t b_addr = ptx::smem_u32(b_tiles + stage * kBBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // Inside a 128-byte swizzle row the k-th 16-element slice starts 32 bytes on.
            const uint64_t a_desc = ptx::make_sw128_kmajor_desc(a_addr + k * UMMA_K * 2);
            const uint64_t b_desc = ptx::make_sw128_kmajor_desc(b_addr + k * UMMA_K * 2);
            ptx::umma_f16(d_tmem, a_desc, b_desc, idesc, (kb != sg.kb0 || k != 0) ? 1u : 0u);
          }
          ptx::umma_commit(&ctl->empty[stage]);  // frees the stage once these MMAs retire
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) ptx::umma_commit(&ctl->tmem_full[acc]);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32)
    int g = 0, iter = 0;
    Walk walk(sched, static_cast<int>(blockIdx.x));
    Segment sg;
    for (; walk.next(sg); ++iter) {
      const TileCoord tc = locate_tile(ctl, sg.tile, g, kOutBN);
      const bool whole = sg.kb0 == 0 && sg.kb1 == k_blocks;
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!ptx::mbar_wait(&ctl->tmem_full[acc], acc_phase, abort_flag)) {
        *abort_flag = 1;
        atomicCAS(&g_pipeline_status, 0, kErrEpilogueWait);
        break;
      }
      ptx::tcgen05_fence_after();
      const int tile_row = quarter * 32 + lane;
      const int row = tc.row0 + tile_row;
      bool row_ok = row < tc.row_end;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      if (whole) {
        __half* yrow = output_row(scatter, y, row, n_out, row_ok) + tc.n0;
        if constexpr (kGlu) {
          glu_epilogue<kOutBN>(taddr, yrow, row_ok, tc.n0, n_out);
        } else {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            if (tc.n0 + c * 32 >= N) break;  // N is a multiple of 64, so chunks are all-or-nothing
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
        }
      } else {
        // Part of a tile's k range: the fp32 accumulator goes to this CTA's slot of the workspace.
        float* prow = partials + static_cast<size_t>(partial_slot(blockIdx.x, sg.kb0)) * (BM * BN) + tile_row * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32b_x32(taddr + c * 32, r);
          ptx::tmem_ld_wait();
          if (!row_ok) continue;
          uint4* dst = reinterpret_cast<uint4*>(prow + c * 32);
#pragma unroll
          for (int v = 0; v < 8; ++v) dst[v] = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
        }
      }
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&ctl->tmem_empty[acc]);
      if (!whole) {
        // Publish this part; the CTA that finds all other parts of the tile already published
        // sums them (in CTA order, so the result does not depend on timing) and writes the rows.
        // Counters were zeroed by the host before the launch.  Nobody waits.
        const long long tile_unit0 = static_cast<long long>(sg.tile - sched.whole_tiles) * k_blocks;
        const int c_first = sched.cta_of(tile_unit0);
        const int c_last = sched.cta_of(tile_unit0 + k_blocks - 1);
        const int parts = c_last - c_first + 1;
        __threadfence();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (threadIdx.x == 64) ctl->split_rank = atomicAdd(&tile_counters[sg.tile], 1);
        for (int i = threadIdx.x - 64; i < parts; i += 128) {
          const long long begin = sched.first_unit(c_first + i) - tile_unit0;
          ctl->part_slot[i] = partial_slot(c_first + i, begin > 0 ? static_cast<int>(begin) : 0);
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (ctl->split_rank == parts - 1) {
          __threadfence();
          const int rows_here = min(BM, tc.row_end - tc.row0);
          reduce_parts<BN, kGlu>(partials, ctl->part_slot, parts, rows_here, quarter, lane, tc, y, kGlu ? n_out : N,
                                 scatter);
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");  // part_slot is reused by the next segment
      }
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tcgen05_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace gmm
}  // namespace b200ops

// The workspace enables split-K for problems with few output tiles (0 = split-K cannot help
// this shape).  Without a workspace (NULL) the kernel always runs without split-K.
extern "C" size_t b200ops_grouped_matmul_workspace_size(int64_t num_tokens, int64_t k, int64_t num_experts,
                                                        int64_t n) {
  using namespace b200ops;
  if (num_tokens <= 0 || k <= 0 || num_experts <= 0 || n <= 0) return 0;
  return gmm::balanced_possible(num_tokens, k, num_experts, n, gmm::launch_sms()) ? gmm::workspace_bytes() : 0;
}

namespace b200ops {
namespace gmm {
int launch(const void* x, const void* w, const int64_t* group_list, void* y, int64_t num_tokens, int64_t k,
           int64_t num_experts, int64_t n, void* workspace, size_t workspace_size, const RowScatter& scatter,
           bool glu, void* stream);
}
}  // namespace b200ops

extern "C" int b200ops_grouped_matmul(const void* x, const void* w, const int64_t* group_list,
                                      void* y, int64_t num_tokens, int64_t k, int64_t num_experts,
                                      int64_t n, void* workspace, size_t workspace_size, void* stream) {
  b200ops::gmm::RowScatter none;
  none.index = nullptr;
  none.cap = 1;
  none.my_rank = 0;
  none.world = 0;
  for (int r = 0; r < b200ops::kMaxPeers; ++r) none.peers.base[r] = nullptr;
  B200OPS_REQUIRE(num_tokens <= 0 || y != nullptr, "grouped_matmul: null pointer");
  return b200ops::gmm::launch(x, w, group_list, y, num_tokens, k, num_experts, n, workspace, workspace_size,
                              none, false, stream);
}

extern "C" int b200ops_grouped_matmul_swiglu(const void* x, const void* w, const int64_t* group_list, void* y,
                                             int64_t num_tokens, int64_t k, int64_t num_experts, int64_t two_d,
                                             void* workspace, size_t workspace_size, void* stream) {
  b200ops::gmm::RowScatter none;
  none.index = nullptr;
  none.cap = 1;
  none.my_rank = 0;
  none.world = 0;
  for (int r = 0; r < b200ops::kMaxPeers; ++r) none.peers.base[r] = nullptr;
  B200OPS_REQUIRE(num_tokens <= 0 || y != nullptr, "grouped_matmul_swiglu: null pointer");
  return b200ops::gmm::launch(x, w, group_list, y, num_tokens, k, num_experts, two_d, workspace, workspace_size,
                              none, true, stream);
}

extern "C" int b200ops_grouped_matmul_scatter(const void* x, const void* w, const int64_t* group_list,
                                              int64_t num_tokens, int64_t k, int64_t num_experts, int64_t n,
                                              void* workspace, size_t workspace_size,
                                              const int32_t* row_index, void* const* peer_out, int64_t world,
                                              int64_t cap, int64_t my_rank, void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(world >= 1 && world <= kMaxPeers && my_rank >= 0 && my_rank < world && cap > 0 &&
                      cap * world < (1LL << 31),
                  "grouped_matmul_scatter: bad geometry world=%lld rank=%lld cap=%lld", (long long)world,
                  (long long)my_rank, (long long)cap);
  B200OPS_REQUIRE(row_index != nullptr && peer_out != nullptr, "grouped_matmul_scatter: null pointer");
  gmm::RowScatter sc;
  sc.index = row_index;
  sc.cap = static_cast<int>(cap);
  sc.my_rank = static_cast<int>(my_rank);
  sc.world = static_cast<int>(world);
  for (int r = 0; r < kMaxPeers; ++r) {
    sc.peers.base[r] = r < world ? peer_out[r] : nullptr;
    B200OPS_REQUIRE(r >= world || (sc.peers.base[r] != nullptr && aligned16(sc.peers.base[r])),
                    "grouped_matmul_scatter: peer %d has no buffer", r);
  }
  return gmm::launch(x, w, group_list, sc.peers.base[my_rank], num_tokens, k, num_experts, n, workspace,
                     workspace_size, sc, false, stream);
}

namespace b200ops {
namespace gmm {
// y = x . w^T for shapes the tensor-core kernels do not take (k or n not a multiple of 64, or
// pointers that are not 16-byte aligned): 64 x 64 output tiles, 16 x 16 threads with a 4 x 4
// block each, operands staged through shared memory as fp32, element-wise bounds checks.  Same
// arithmetic contract: fp16 products summed in fp32, one rounding.
constexpr int kGenTile = 64, kGenK = 16;

__global__ void __launch_bounds__(256) matmul_nt_general_kernel(const __half* __restrict__ x,
                                                                const __half* __restrict__ w,
                                                                __half* __restrict__ y, int m, int n, int k) {
  __shared__ float xs[kGenK][kGenTile + 1];
  __shared__ float ws[kGenK][kGenTile + 1];
  pdl_trigger();
  pdl_wait();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int row0 = blockIdx.y * kGenTile, col0 = blockIdx.x * kGenTile;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += kGenK) {
    for (int i = threadIdx.x; i < kGenTile * kGenK; i += 256) {
      const int r = i / kGenK, c = i - r * kGenK;
      const bool kin = k0 + c < k;
      xs[c][r] = (kin && row0 + r < m) ? __half2float(x[static_cast<size_t>(row0 + r) * k + k0 + c]) : 0.f;
      ws[c][r] = (kin && col0 + r < n) ? __half2float(w[static_cast<size_t>(col0 + r) * k + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < kGenK; ++c) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = xs[c][ty * 4 + i];
        b[i] = ws[c][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = row0 + ty * 4 + i, c = col0 + tx * 4 + j;
      if (r < m && c < n) y[static_cast<size_t>(r) * n + c] = __float2half_rn(acc[i][j]);
    }
}
}  // namespace gmm
}  // namespace b200ops

extern "C" int b200ops_matmul(const void* x, const void* w, void* y, int64_t m, int64_t n, int64_t k,
                              void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(m >= 0 && n > 0 && k > 0 && m < (1LL << 30) && n < (1LL << 30) && k < (1LL << 30),
                  "matmul: bad shape m=%lld n=%lld k=%lld", (long long)m, (long long)n, (long long)k);
  if (m == 0) return B200OPS_OK;
  B200OPS_REQUIRE(x && w && y, "matmul: null pointer");
  if (k % 64 == 0 && n % 64 == 0 && aligned16(x) && aligned16(w) && aligned16(y)) {
    gmm::RowScatter none;
    none.index = nullptr;
    none.cap = 1;
    none.my_rank = 0;
    none.world = 0;
    for (int r = 0; r < kMaxPeers; ++r) none.peers.base[r] = nullptr;
    return gmm::launch(x, w, nullptr, y, m, k, 1, n, nullptr, 0, none, false, stream);
  }
  const dim3 grid(static_cast<unsigned>((n + gmm::kGenTile - 1) / gmm::kGenTile),
                  static_cast<unsigned>((m + gmm::kGenTile - 1) / gmm::kGenTile));
  B200OPS_REQUIRE(grid.y <= 65535, "matmul: too many rows for the general kernel (%lld)", (long long)m);
  B200OPS_CUDA(launch_kernel(gmm::matmul_nt_general_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream),
                      static_cast<const __half*>(x), static_cast<const __half*>(w), static_cast<__half*>(y),
                      static_cast<int>(m), static_cast<int>(n), static_cast<int>(k)));
  return B200OPS_OK;
}

namespace b200ops {
namespace gmm {
// Clusters of two CTAs that the device can keep resident at once (cached per device).
static int resident_pairs(int dev, int sms) {
  static std::atomic<int> cached[64];
  if (dev >= 0 && dev < 64 && cached[dev].load(std::memory_order_relaxed) > 0)
    return cached[dev].load(std::memory_order_relaxed);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(sms / 2 * 2));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, grouped_matmul_pair_kernel<false>, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = sms / 2;
  }
  if (n > sms / 2) n = sms / 2;
  if (dev >= 0 && dev < 64) cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

// Clusters of `splits` CTAs of the split-K kernel that the device keeps resident at once.
static int resident_split_clusters(int dev, int splits) {
  static std::atomic<int> cached[64][kMaxClusterSplitHost + 1];
  if (dev >= 0 && dev < 64 && cached[dev][splits].load(std::memory_order_relaxed) != 0)
    return cached[dev][splits].load(std::memory_order_relaxed);
  // The query counts against the function's shared-memory limit, so raise that first.
  if (cudaFuncSetAttribute(grouped_matmul_ksplit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kSplitSmemBytes)) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(static_cast<unsigned>(launch_sms() / splits * splits));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSplitSmemBytes;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, grouped_matmul_ksplit_kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  if (n <= 0) n = -1;  // cached as "none fit"
  if (dev >= 0 && dev < 64) cached[dev][splits].store(n, std::memory_order_relaxed);
  return n;
}

// All clusters must be resident at once: a cluster that has to wait for a free slot starts
// when the others end and doubles the time.  Clusters are placed within a GPC, so fewer fit
// than SMs / s: the largest s <= `splits` whose clusters all fit, 0 if none of two or more does.
static int fit_split_to_device(int splits, int64_t tiles) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  while (splits > 1 && resident_split_clusters(dev, splits) < tiles) --splits;
  return splits >= 2 ? splits : 0;
}

static int launch_ksplit(const CUtensorMap& map_x, const CUtensorMap& map_x_short, const void* w,
                         const int64_t* group_list, void* y,
                         int64_t num_tokens, int64_t k, int64_t num_experts, int64_t n, int splits,
                         const RowScatter& scatter, cudaStream_t st) {
  CUtensorMap map_w;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                              static_cast<uint64_t>(num_experts)};
    const uint64_t strides[2] = {static_cast<uint64_t>(k) * 2, static_cast<uint64_t>(k) * n * 2};
    const uint32_t box[3] = {BK, kSplitBN, 1};
    const int rc = encode_f16_map(&map_w, w, 3, dims, strides, box, "grouped_matmul(w)");
    if (rc != B200OPS_OK) return rc;
  }
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  B200OPS_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    B200OPS_CUDA(cudaFuncSetAttribute(grouped_matmul_ksplit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(kSplitSmemBytes)));
    attr_set[dev].store(true, std::memory_order_release);
  }
  static_assert(kMaxClusterSplitHost == kMaxClusterSplit, "host and device agree on the cluster limit");
  const int64_t tiles = ((num_tokens + BM - 1) / BM) * ((n + kSplitBN - 1) / kSplitBN);
  int tile_choice = kSplitTilesFull;
  if (knob(kKnobGmmShort, 1) != 0) {
    if (num_tokens <= kShortRows) tile_choice = kSplitTilesShort;
    else if (num_tokens > kMaxClusterSplitRows && group_list != nullptr) tile_choice = kSplitTilesByRowCount;
  }
  B200OPS_CUDA(launch_cluster(grouped_matmul_ksplit_kernel, dim3(static_cast<unsigned>(tiles * splits)),
                              dim3(kThreads), kSplitSmemBytes, st, static_cast<unsigned>(splits), map_x, map_x_short,
                              map_w, group_list, static_cast<__half*>(y), static_cast<int>(num_tokens),
                              static_cast<int>(n), static_cast<int>(k), static_cast<int>(num_experts), scatter,
                              tile_choice));
  return B200OPS_OK;
}

static int launch_pairs(const CUtensorMap& map_x, const void* w, const int64_t* group_list, void* y,
                        int64_t num_tokens, int64_t k, int64_t num_experts, int64_t n, bool glu,
                        const RowScatter& scatter, cudaStream_t st) {
  CUtensorMap map_w;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                              static_cast<uint64_t>(num_experts)};
    const uint64_t strides[2] = {static_cast<uint64_t>(k) * 2, static_cast<uint64_t>(k) * n * 2};
    const uint32_t box[3] = {BK, kPairBN / 2, 1};
    const int rc = encode_f16_map(&map_w, w, 3, dims, strides, box, "grouped_matmul(w)");
    if (rc != B200OPS_OK) return rc;
  }
  auto kern = glu ? grouped_matmul_pair_kernel<true> : grouped_matmul_pair_kernel<false>;
  static std::atomic<bool> attr_set[2][64];
  int dev = 0;
  B200OPS_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[glu][dev].load(std::memory_order_acquire)) {
    B200OPS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(kPairSmemBytes)));
    attr_set[glu][dev].store(true, std::memory_order_release);
  }
  const int64_t n_tiles = (n + kPairBN - 1) / kPairBN;  // the same count with and without SwiGLU
  const int64_t max_items = (((num_tokens + BM - 1) / BM + 1) / 2 + num_experts) * n_tiles;
  const int64_t resident = resident_pairs(dev, launch_sms());
  const int pairs = static_cast<int>(max_items < resident ? max_items : resident);
  B200OPS_CUDA(launch_cluster(kern, dim3(static_cast<unsigned>(2 * pairs)), dim3(kThreads), kPairSmemBytes, st, 2u,
                              map_x, map_w, group_list, static_cast<__half*>(y), static_cast<int>(num_tokens),
                              static_cast<int>(n), static_cast<int>(k), static_cast<int>(num_experts), scatter));
  return B200OPS_OK;
}
}  // namespace gmm
}  // namespace b200ops

int b200ops::gmm::launch(const void* x, const void* w, const int64_t* group_list, void* y, int64_t num_tokens,
                         int64_t k, int64_t num_experts, int64_t n, void* workspace, size_t workspace_size,
                         const RowScatter& scatter, bool glu, void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(num_tokens >= 0 && k > 0 && n > 0 && num_experts > 0,
                  "grouped_matmul: bad shape tokens=%lld k=%lld experts=%lld n=%lld",
                  (long long)num_tokens, (long long)k, (long long)num_experts, (long long)n);
  B200OPS_REQUIRE(k % 64 == 0 && n % 64 == 0,
                  "grouped_matmul: second and third dimensions of w must be multiples of 64, got %lld and %lld",
                  (long long)k, (long long)n);
  B200OPS_REQUIRE(num_experts <= gmm::kMaxExperts, "grouped_matmul: at most %d experts, got %lld",
                  gmm::kMaxExperts, (long long)num_experts);
  B200OPS_REQUIRE(num_tokens < (1LL << 30) && k < (1LL << 30) && n < (1LL << 30),
                  "grouped_matmul: dimension too large");
  B200OPS_REQUIRE(!glu || n % 128 == 0,
                  "grouped_matmul_swiglu: w must have 2*d rows with d a multiple of 64, got %lld", (long long)n);
  if (num_tokens == 0) return B200OPS_OK;
  B200OPS_REQUIRE(x && w && y && (group_list || num_experts == 1), "grouped_matmul: null pointer");
  B200OPS_REQUIRE(aligned16(x) && aligned16(w) && aligned16(y),
                  "grouped_matmul: pointers must be 16-byte aligned");

  CUtensorMap map_x, map_w;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(num_tokens)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k) * 2};
    const uint32_t box[2] = {gmm::BK, gmm::BM};
    const int rc = encode_f16_map(&map_x, x, 2, dims, strides, box, "grouped_matmul(x)");
    if (rc != B200OPS_OK) return rc;
  }
  CUtensorMap map_x_short;  // the same rows in boxes of kShortRows (decode-size problems)
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(num_tokens)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k) * 2};
    const uint32_t box[2] = {gmm::BK, gmm::kShortRows};
    const int rc = encode_f16_map(&map_x_short, x, 2, dims, strides, box, "grouped_matmul(x, short tiles)");
    if (rc != B200OPS_OK) return rc;
  }
  const int sms = gmm::launch_sms();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The fused gate/up form exists in the two throughput kernels only (its shapes have thousands
  // of output columns and a short K: neither split-K nor narrow tiles apply).
  int64_t resident_tiles = 0;
  int s = glu ? 0 : gmm::cluster_split_factor(num_tokens, k, num_experts, n, sms, &resident_tiles);
  if (s) s = gmm::fit_split_to_device(s, resident_tiles);
  if (s)
    return gmm::launch_ksplit(map_x, map_x_short, w, group_list, y, num_tokens, k, num_experts, n, s, scatter, st);
  if (gmm::use_cta_pairs(num_tokens, num_experts, n, sms))
    return gmm::launch_pairs(map_x, w, group_list, y, num_tokens, k, num_experts, n, glu, scatter, st);
  const bool narrow = !glu && gmm::use_narrow_tiles(num_tokens, k, n, sms);
  const int bn = narrow ? gmm::kNarrowBN : gmm::kWideBN;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                              static_cast<uint64_t>(num_experts)};
    const uint64_t strides[2] = {static_cast<uint64_t>(k) * 2, static_cast<uint64_t>(k) * n * 2};
    const uint32_t box[3] = {gmm::BK, static_cast<uint32_t>(glu ? bn / 2 : bn), 1};  // glu: gate and up boxes
    const int rc = encode_f16_map(&map_w, w, 3, dims, strides, box, "grouped_matmul(w)");
    if (rc != B200OPS_OK) return rc;
  }

  auto kern = glu      ? gmm::grouped_matmul_kernel<gmm::GluCfg>
              : narrow ? gmm::grouped_matmul_kernel<gmm::NarrowCfg>
                       : gmm::grouped_matmul_kernel<gmm::WideCfg>;
  const size_t smem = narrow ? gmm::NarrowCfg::kSmemBytes : gmm::WideCfg::kSmemBytes;
  static_assert(gmm::WideCfg::kSmemBytes == gmm::GluCfg::kSmemBytes, "the gate/up form shares the wide shape's ring");
  const int variant = glu ? 2 : (narrow ? 1 : 0);
  static std::atomic<bool> attr_set[3][64];
  int dev = 0;
  B200OPS_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[variant][dev].load(std::memory_order_acquire)) {
    B200OPS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
    attr_set[variant][dev].store(true, std::memory_order_release);
  }
  const int64_t n_tiles = (n + bn - 1) / bn;  // glu: n / 2 columns in tiles of bn / 2, the same count
  const int64_t max_tiles = ((num_tokens + gmm::BM - 1) / gmm::BM + num_experts) * n_tiles;
  int* counters = nullptr;
  float* partials = nullptr;
  int grid = static_cast<int>(max_tiles < sms ? max_tiles : sms);
  if (!narrow && workspace != nullptr && gmm::balanced_possible(num_tokens, k, num_experts, n, sms)) {
    if (workspace_size < gmm::workspace_bytes())
      return fail(B200OPS_EWORKSPACE, "grouped_matmul: workspace of %zu bytes needed, got %zu",
                  gmm::workspace_bytes(), workspace_size);
    B200OPS_REQUIRE(aligned16(workspace), "grouped_matmul: workspace must be 16-byte aligned");
    counters = static_cast<int*>(workspace);
    partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + gmm::kCounterBytes);
    B200OPS_CUDA(cudaMemsetAsync(counters, 0, gmm::kCounterBytes, st));
    grid = sms;  // the schedule cuts the work into one range per SM; CTAs without one exit
  }
  const int allow_short = knob(kKnobGmmShort, 1) != 0 ? 1 : 0;
  B200OPS_CUDA(launch_kernel(kern, dim3(grid), dim3(gmm::kThreads), smem, st, map_x, map_x_short, map_w, group_list,
                      static_cast<__half*>(y), static_cast<int>(num_tokens), static_cast<int>(n),
                      static_cast<int>(k), static_cast<int>(num_experts), counters, partials, scatter,
                      allow_short));
  return B200OPS_OK;
}

namespace b200ops {
namespace gmm {
// Reads and clears this translation unit's status word (the device must be idle).
int status_take() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_pipeline_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_pipeline_status, &zero, sizeof(int));
  }
  return v;
}
}  // namespace gmm
}  // namespace b200ops
