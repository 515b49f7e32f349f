// Warp-level building blocks shared by the TMA-staged paged-attention kernels: one warp
// consumes its 16-token slice of a 64-token K/V tile held in swizzled shared memory.
//
// Two tile layouts, following the two cache layouts:
//   NHD cache  a tensor's tile is two sub-tiles [64 tokens][64 channels] (128-byte rows,
//              128-byte swizzle), one per half of head_dim;
//   NZ cache   a tensor's tile is eight sub-tiles [64 tokens][16 channels] (32-byte rows, no
//              swizzle), one per 16-channel chunk of the head -- the cache's own
//              [chunk][token][16] order, so one TMA box fetches the whole tile.  The box is
//              declared with 512-byte rows (16 tokens x 16 halfs are contiguous in the cache):
//              with 32-byte rows the copy engine had 1024 row requests per tile to issue and
//              the kernel ran 18 % slower.  Unswizzled 32-byte rows cost ldmatrix a two-way
//              bank conflict, which this HBM-bound kernel does not notice.
#pragma once

#include "paged_attention.cuh"
#include "sm100_ptx.cuh"

namespace b200ops {
namespace pa {
namespace tile {

constexpr int kD = 128;
constexpr int kTile = 64;                            // tokens per pipeline stage
constexpr int kConsumerWarps = 4;                    // each owns 16 tokens of a tile
constexpr int kSubTileBytes = kTile * 128;           // 64 tokens x 64 halfs
constexpr int kTensorTileBytes = 2 * kSubTileBytes;  // both halves of D
constexpr int kStageBytes = 2 * kTensorTileBytes;    // K and V

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte offset of 16-byte chunk `c` (0..7) of row `r` inside a 128B-swizzled sub-tile.
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return static_cast<uint32_t>(r * 128 + ((c ^ (r & 7)) << 4));
}

constexpr int kNzSubTileBytes = kTile * 32;  // 64 tokens x 16 halfs

// Byte offset inside a tensor's tile of the 8 channels starting at 8*c (c = 0..15) of token row
// `r`.  NHD: sub-tile c/8, 128-byte swizzle.  NZ: sub-tile c/2 (a 16-channel chunk), plain rows.
template <bool kNz>
__device__ __forceinline__ uint32_t tile_offset(int r, int c) {
  if (kNz) return static_cast<uint32_t>((c >> 1) * kNzSubTileBytes + r * 32 + ((c & 1) << 4));
  return static_cast<uint32_t>((c >> 3) * kSubTileBytes) + swz(r, c & 7);
}

// Running softmax state of one warp: rows g (lo) and g+8 (hi) of the 16-row MMA operand.
struct WarpState {
  float o[kD / 8][4];
  float m_lo, m_hi, l_lo, l_hi;
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int i = 0; i < kD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    m_lo = m_hi = -INFINITY;
    l_lo = l_hi = 0.f;
  }
  // Row sums are kept per thread while streaming; finish them across the quad.
  __device__ __forceinline__ void finish_sums() {
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  }
};

// One warp's 16 tokens of one tile: S = Q.K^T (two n-blocks of 8 tokens), online softmax in
// base 2, O += P.V.  `stage` is the generic address of the stage (K sub-tiles then V
// sub-tiles); `tok0` the sequence position of the warp's first token; tokens >= `end` are
// masked and their V rows zeroed first so that 0 * garbage cannot become NaN.
// kUpper: the GQA group has more than 8 query heads, so MMA rows 8..15 carry data.
template <bool kUpper, bool kNz = false>
__device__ __forceinline__ void consume_slice(WarpState& st, const uint32_t (&qa)[kD / 16][4],
                                              uint8_t* stage, int row0, int tok0, int end, int lane,
                                              float scale_log2) {
  const int t4 = lane & 3;
  const uint32_t kbase = ptx::smem_u32(stage);
  const uint32_t vbase = kbase + kTensorTileBytes;
  // ldmatrix row/chunk selectors of this lane
  const int k_row = row0 + ((lane >> 4) << 3) + (lane & 7);  // K: matrices 2,3 are tokens +8
  const int k_csel = (lane >> 3) & 1;                        //    matrices 1,3 are chunk +1
  const int v_row = row0 + (((lane >> 3) & 1) << 3) + (lane & 7);  // V: matrices 1,3 tokens +8
  const int v_csel = lane >> 4;                                    //    matrices 2,3 chunk +1
  const bool tail = tok0 + 16 > end;  // warp-uniform
  if (tail) {
    uint8_t* vt = stage + kTensorTileBytes;
    for (int i = lane; i < 16 * 16; i += 32) {
      const int r = row0 + (i >> 4), c = i & 15;
      if (tok0 + (i >> 4) >= end)  // the whole row goes to zero, so the swizzle does not matter
        *reinterpret_cast<uint4*>(vt + (kNz ? (c >> 1) * kNzSubTileBytes + r * 32 + ((c & 1) << 4)
                                            : (c >> 3) * kSubTileBytes + r * 128 + ((c & 7) << 4))) =
            make_uint4(0, 0, 0, 0);
    }
    __syncwarp();
  }
  float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
  for (int ks = 0; ks < kD / 16; ++ks) {
    uint32_t kb[4];
    ldmatrix_x4(kb, kbase + tile_offset<kNz>(k_row, ks * 2 + k_csel));
    mma_16816(s[0], qa[ks], kb[0], kb[1]);
    mma_16816(s[1], qa[ks], kb[2], kb[3]);
  }
#pragma unroll
  for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int tok = tok0 + nb * 8 + 2 * t4 + (j & 1);
      s[nb][j] = (!tail || tok < end) ? s[nb][j] * scale_log2 : -INFINITY;
    }
  }
  uint32_t pa_frag[4];
  {
    float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(st.m_lo, mx);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = exp2f(st.m_lo - m_use);
    const float p0 = exp2f(s[0][0] - m_use), p1 = exp2f(s[0][1] - m_use);
    const float p2 = exp2f(s[1][0] - m_use), p3 = exp2f(s[1][1] - m_use);
    st.l_lo = st.l_lo * alpha + (p0 + p1 + p2 + p3);
    st.m_lo = m_new;
    pa_frag[0] = f2_to_h2(p0, p1);
    pa_frag[2] = f2_to_h2(p2, p3);
#pragma unroll
    for (int i = 0; i < kD / 8; ++i) {
      st.o[i][0] *= alpha;
      st.o[i][1] *= alpha;
    }
  }
  if (kUpper) {
    float mx = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(st.m_hi, mx);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = exp2f(st.m_hi - m_use);
    const float p0 = exp2f(s[0][2] - m_use), p1 = exp2f(s[0][3] - m_use);
    const float p2 = exp2f(s[1][2] - m_use), p3 = exp2f(s[1][3] - m_use);
    st.l_hi = st.l_hi * alpha + (p0 + p1 + p2 + p3);
    st.m_hi = m_new;
    pa_frag[1] = f2_to_h2(p0, p1);
    pa_frag[3] = f2_to_h2(p2, p3);
#pragma unroll
    for (int i = 0; i < kD / 8; ++i) {
      st.o[i][2] *= alpha;
      st.o[i][3] *= alpha;
    }
  } else {
    pa_frag[1] = 0u;
    pa_frag[3] = 0u;
  }
#pragma unroll
  for (int cc = 0; cc < kD / 8; cc += 2) {
    uint32_t vb[4];
    const int c = cc + v_csel;
    ldmatrix_x4_trans(vb, vbase + tile_offset<kNz>(v_row, c));
    mma_16816(st.o[cc], pa_frag, vb[0], vb[1]);
    mma_16816(st.o[cc + 1], pa_frag, vb[2], vb[3]);
  }
  if (tail) ptx::fence_proxy_async();
}

// Q fragments (A operand, 16 heads x 16 channels per k-step) from a [group, 128] f16 block
// in global or shared memory; rows >= group are zero.
template <bool kUpper>
__device__ __forceinline__ void load_q_fragments(uint32_t (&qa)[kD / 16][4], const __half* qb, int group,
                                                 int lane) {
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int ks = 0; ks < kD / 16; ++ks) {
    const int c = ks * 16 + 2 * t4;
    qa[ks][0] = (g < group) ? *reinterpret_cast<const uint32_t*>(qb + g * kD + c) : 0u;
    qa[ks][2] = (g < group) ? *reinterpret_cast<const uint32_t*>(qb + g * kD + c + 8) : 0u;
    if (kUpper) {
      qa[ks][1] = (g + 8 < group) ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * kD + c) : 0u;
      qa[ks][3] = (g + 8 < group) ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * kD + c + 8) : 0u;
    } else {
      qa[ks][1] = 0u;
      qa[ks][3] = 0u;
    }
  }
}

}  // namespace tile
}  // namespace pa
}  // namespace b200ops
