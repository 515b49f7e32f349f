// SwiGLU for sm_100a: y[t, j] = silu(x[t, j]) * x[t, d + j], fp32 math, one RNE rounding.
//
// Formula and operand order follow the reference's torch golden `swiglu_cpu`
// (benchmark/test_swiglu.py:6-12) and kernel (csrc/opdev/op_kernel/swi_glu_ex.cpp:52-57):
// (x0 * sigmoid(x0)) * x1.  HBM-bound: 6*T*d bytes (read 2d, write d halfs per row).
#include "common.cuh"

namespace b200ops {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;  // 128-bit vector pairs in flight per thread

template <typename index_t>
__global__ void __launch_bounds__(kThreads)
swiglu_kernel(const __half* __restrict__ x, __half* __restrict__ y, index_t total_vecs,
              index_t vecs_per_row) {
  pdl_trigger();
  pdl_wait();
  const uint4* xin = reinterpret_cast<const uint4*>(x);
  uint4* yout = reinterpret_cast<uint4*>(y);
  const index_t base = static_cast<index_t>(blockIdx.x) * (kThreads * kUnroll) + threadIdx.x;

  uint4 g[kUnroll], u[kUnroll];
#pragma unroll
  for (int i = 0; i < kUnroll; ++i) {
    const index_t v = base + static_cast<index_t>(i) * kThreads;
    if (v < total_vecs) {
      const index_t row = v / vecs_per_row;
      const index_t col = v - row * vecs_per_row;
      const index_t in = row * (2 * vecs_per_row) + col;
      g[i] = ld_stream(xin + in);
      u[i] = ld_stream(xin + in + vecs_per_row);
    }
  }
#pragma unroll
  for (int i = 0; i < kUnroll; ++i) {
    const index_t v = base + static_cast<index_t>(i) * kThreads;
    if (v < total_vecs) {
      const uint32_t* gs = reinterpret_cast<const uint32_t*>(&g[i]);
      const uint32_t* us = reinterpret_cast<const uint32_t*>(&u[i]);
      uint4 o;
      uint32_t* os = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gf = h2_to_f2(gs[j]);
        const float2 uf = h2_to_f2(us[j]);
        os[j] = f2_to_h2(silu_mul(gf.x, uf.x), silu_mul(gf.y, uf.y));
      }
      st_stream(yout + v, o);
    }
  }
}

}  // namespace
}  // namespace b200ops

extern "C" int b200ops_swiglu(const void* x, void* y, int64_t num_tokens, int64_t two_d,
                              void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(num_tokens >= 0, "swiglu: bad row count %lld", (long long)num_tokens);
  B200OPS_REQUIRE(two_d >= 64 && two_d % 64 == 0,
                  "swiglu: last dimension must be a multiple of 64, got %lld", (long long)two_d);
  if (num_tokens == 0) return B200OPS_OK;
  B200OPS_REQUIRE(x && y, "swiglu: null pointer");
  B200OPS_REQUIRE(aligned16(x) && aligned16(y), "swiglu: pointers must be 16-byte aligned");

  const int64_t vecs_per_row = two_d / 16;  // output vectors (8 halfs) per row
  const int64_t total = num_tokens * vecs_per_row;
  const int64_t per_cta = static_cast<int64_t>(kThreads) * kUnroll;
  const int64_t grid = (total + per_cta - 1) / per_cta;
  B200OPS_REQUIRE(grid <= 0x7fffffffLL, "swiglu: tensor too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half* xp = static_cast<const __half*>(x);
  __half* yp = static_cast<__half*>(y);
  // Input vector indices reach 2*total: stay in 32-bit arithmetic when that fits.
  if (2 * total + per_cta < 0x7fffffffLL) {
    B200OPS_CUDA(launch_kernel(swiglu_kernel<uint32_t>, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0, st, xp, yp,
                        static_cast<uint32_t>(total), static_cast<uint32_t>(vecs_per_row)));
  } else {
    B200OPS_CUDA(launch_kernel(swiglu_kernel<unsigned long long>, dim3(static_cast<unsigned>(grid)), dim3(kThreads), 0, st,
                        xp, yp, static_cast<unsigned long long>(total),
                        static_cast<unsigned long long>(vecs_per_row)));
  }
  return B200OPS_OK;
}
