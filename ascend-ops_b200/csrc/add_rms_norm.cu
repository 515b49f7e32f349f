// Fused residual add + RMSNorm for sm_100a.
//
// One pass over HBM: every thread keeps its slice of the row in registers between the
// sum-of-squares reduction and the normalisation, so x and residual are read once and
// y / residual_out written once (8*T*H + 2*H bytes in total).  The reference kernel
// (csrc/opdev/op_kernel/add_rms_norm_ex.cpp:52-121) reads x and residual twice.
//
// Arithmetic follows the reference's torch golden (benchmark/test_add_rms_norm.py:6-10):
// s = f16(x + r) (one rounding of the exact fp32 sum), rms = sqrt(mean(float(s)^2) + eps),
// y = f16(float(s) / rms * float(w)), residual_out = s.
#include "common.cuh"

#include <cstdlib>

namespace b200ops {
namespace {

constexpr int kMaxVecPerThread = 8;

// A CTA holds `rows_per_cta` rows; each row is owned by `warps_per_row` whole warps.
// VPT = 128-bit vectors (8 halfs) per thread per tensor.
template <int VPT>
__global__ void __launch_bounds__(1024)
add_rms_norm_kernel(const __half* __restrict__ x, const __half* __restrict__ residual,
                    const __half* __restrict__ weight, __half* __restrict__ y,
                    __half* __restrict__ residual_out, int64_t num_tokens, int dim,
                    int warps_per_row, float eps, float inv_dim) {
  __shared__ float partial[32];
  pdl_trigger();
  pdl_wait();

  const int threads_per_row = warps_per_row * 32;
  const int rows_per_cta = blockDim.x / threads_per_row;
  const int row_in_cta = threadIdx.x / threads_per_row;
  const int t_in_row = threadIdx.x - row_in_cta * threads_per_row;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * rows_per_cta + row_in_cta;
  const bool row_ok = row < num_tokens;
  const int vecs = dim >> 3;

  const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
  const uint4* rr = reinterpret_cast<const uint4*>(residual + row * dim);
  uint4* yr = reinterpret_cast<uint4*>(y + row * dim);
  uint4* sr = reinterpret_cast<uint4*>(residual_out + row * dim);
  const uint4* wr = reinterpret_cast<const uint4*>(weight);

  uint4 xv[VPT], rv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t_in_row + i * threads_per_row;
    if (row_ok && v < vecs) {
      xv[i] = ld_stream(xr + v);
      rv[i] = ld_stream(rr + v);
    } else {
      xv[i] = make_uint4(0, 0, 0, 0);
      rv[i] = make_uint4(0, 0, 0, 0);
    }
  }

  // s = f16(x + r), kept packed in xv; sum of squares of the ROUNDED s in fp32.
  float sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    uint32_t* xs = reinterpret_cast<uint32_t*>(&xv[i]);
    const uint32_t* rs = reinterpret_cast<const uint32_t*>(&rv[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = h2_to_f2(xs[j]);
      const float2 b = h2_to_f2(rs[j]);
      const uint32_t s = f2_to_h2(a.x + b.x, a.y + b.y);
      const float2 sf = h2_to_f2(s);
      sumsq = fmaf(sf.x, sf.x, sumsq);
      sumsq = fmaf(sf.y, sf.y, sumsq);
      xs[j] = s;
    }
    const int v = t_in_row + i * threads_per_row;
    if (row_ok && v < vecs) st_stream(sr + v, xv[i]);
  }

  // Weight loads are issued before the reduction so their latency hides behind it.
  uint4 wv[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t_in_row + i * threads_per_row;
    wv[i] = (v < vecs) ? __ldg(wr + v) : make_uint4(0, 0, 0, 0);
  }

  sumsq = warp_sum(sumsq);
  if (warps_per_row > 1) {
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) partial[warp] = sumsq;
    __syncthreads();
    const int first = row_in_cta * warps_per_row;
    float tot = 0.f;
    for (int i = 0; i < warps_per_row; ++i) tot += partial[first + i];
    sumsq = tot;
  }
  const float inv_rms = 1.0f / sqrtf(sumsq * inv_dim + eps);

#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = t_in_row + i * threads_per_row;
    if (row_ok && v < vecs) {
      const uint32_t* ss = reinterpret_cast<const uint32_t*>(&xv[i]);
      const uint32_t* ws = reinterpret_cast<const uint32_t*>(&wv[i]);
      uint4 o;
      uint32_t* os = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 sf = h2_to_f2(ss[j]);
        const float2 wf = h2_to_f2(ws[j]);
        os[j] = f2_to_h2(sf.x * inv_rms * wf.x, sf.y * inv_rms * wf.y);
      }
      st_stream(yr + v, o);
    }
  }
}

// Rows too long for the register-resident kernel: the rounded sum s is written to
// residual_out in pass one and read back (from L2 for any sane row length) in pass two.
__global__ void __launch_bounds__(1024)
add_rms_norm_long_row_kernel(const __half* __restrict__ x, const __half* __restrict__ residual,
                             const __half* __restrict__ weight, __half* __restrict__ y,
                             __half* __restrict__ residual_out, int dim, float eps,
                             float inv_dim) {
  __shared__ float partial[32];
  __shared__ float total;
  pdl_trigger();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int vecs = dim >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
  const uint4* rr = reinterpret_cast<const uint4*>(residual + row * dim);
  uint4* yr = reinterpret_cast<uint4*>(y + row * dim);
  uint4* sr = reinterpret_cast<uint4*>(residual_out + row * dim);
  const uint4* wr = reinterpret_cast<const uint4*>(weight);

  float sumsq = 0.f;
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    uint4 a = ld_stream(xr + v);
    const uint4 b = ld_stream(rr + v);
    uint32_t* as = reinterpret_cast<uint32_t*>(&a);
    const uint32_t* bs = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = h2_to_f2(as[j]);
      const float2 fb = h2_to_f2(bs[j]);
      const uint32_t s = f2_to_h2(fa.x + fb.x, fa.y + fb.y);
      const float2 sf = h2_to_f2(s);
      sumsq = fmaf(sf.x, sf.x, sumsq);
      sumsq = fmaf(sf.y, sf.y, sumsq);
      as[j] = s;
    }
    sr[v] = a;
  }
  sumsq = warp_sum(sumsq);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sumsq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) tot += partial[i];
    total = tot;
  }
  __syncthreads();
  const float inv_rms = 1.0f / sqrtf(total * inv_dim + eps);
  // Each thread re-reads exactly the vectors it wrote itself, so no fence is needed.
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    const uint4 s = sr[v];
    const uint4 w = __ldg(wr + v);
    const uint32_t* ss = reinterpret_cast<const uint32_t*>(&s);
    const uint32_t* ws = reinterpret_cast<const uint32_t*>(&w);
    uint4 o;
    uint32_t* os = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 sf = h2_to_f2(ss[j]);
      const float2 wf = h2_to_f2(ws[j]);
      os[j] = f2_to_h2(sf.x * inv_rms * wf.x, sf.y * inv_rms * wf.y);
    }
    st_stream(yr + v, o);
  }
}

}  // namespace
}  // namespace b200ops

extern "C" int b200ops_add_rms_norm(const void* x, const void* residual, const void* weight,
                                    float eps, void* y, void* residual_out, int64_t num_tokens,
                                    int64_t dim, void* stream) {
  using namespace b200ops;
  B200OPS_REQUIRE(num_tokens >= 0 && dim > 0, "add_rms_norm: bad shape [%lld, %lld]",
                  (long long)num_tokens, (long long)dim);
  B200OPS_REQUIRE(dim % 64 == 0, "add_rms_norm: last dimension must be a multiple of 64, got %lld",
                  (long long)dim);
  B200OPS_REQUIRE(dim <= (1 << 24), "add_rms_norm: last dimension too large: %lld", (long long)dim);
  if (num_tokens == 0) return B200OPS_OK;
  B200OPS_REQUIRE(x && residual && weight && y && residual_out, "add_rms_norm: null pointer");
  B200OPS_REQUIRE(aligned16(x) && aligned16(residual) && aligned16(weight) && aligned16(y) &&
                      aligned16(residual_out),
                  "add_rms_norm: pointers must be 16-byte aligned");

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half* xp = static_cast<const __half*>(x);
  const __half* rp = static_cast<const __half*>(residual);
  const __half* wp = static_cast<const __half*>(weight);
  __half* yp = static_cast<__half*>(y);
  __half* sp = static_cast<__half*>(residual_out);
  const int d = static_cast<int>(dim);
  const int vecs = d / 8;
  const float inv_dim = 1.0f / static_cast<float>(d);

  if (vecs > 1024 * kMaxVecPerThread) {
    B200OPS_CUDA(launch_kernel(add_rms_norm_long_row_kernel, dim3(static_cast<unsigned>(num_tokens)), dim3(1024), 0, st,
                        xp, rp, wp, yp, sp, d, eps, inv_dim));
    return B200OPS_OK;
  }

  // Two vectors per thread and tensor keep 64 B per thread in flight; rows shorter than a
  // warp's worth share a CTA so that small hidden sizes still fill the SMs.
  int vpt = knob(kKnobRmsnormVpt, 2);
  if (vpt != 1 && vpt != 2 && vpt != 4 && vpt != 8) vpt = 2;
  int warps_per_row = (vecs + 32 * vpt - 1) / (32 * vpt);
  while (warps_per_row > 32) {
    vpt *= 2;
    warps_per_row = (vecs + 32 * vpt - 1) / (32 * vpt);
  }
  const int cta_warps_target = knob(kKnobRmsnormCtaWarps, 8);
  int rows_per_cta = cta_warps_target / warps_per_row;
  if (rows_per_cta < 1) rows_per_cta = 1;
  const int threads = rows_per_cta * warps_per_row * 32;
  const int64_t grid = (num_tokens + rows_per_cta - 1) / rows_per_cta;
  B200OPS_REQUIRE(grid <= 0x7fffffffLL, "add_rms_norm: too many rows");

#define LAUNCH(V)                                                                             \
  launch_kernel(add_rms_norm_kernel<V>, dim3(static_cast<unsigned>(grid)), dim3(threads), 0, st, xp, \
         rp, wp, yp, sp, num_tokens, d, warps_per_row, eps, inv_dim)
  cudaError_t err;
  switch (vpt) {
    case 1: err = LAUNCH(1); break;
    case 2: err = LAUNCH(2); break;
    case 4: err = LAUNCH(4); break;
    default: err = LAUNCH(8); break;
  }
#undef LAUNCH
  B200OPS_CUDA(err);
  return B200OPS_OK;
}
