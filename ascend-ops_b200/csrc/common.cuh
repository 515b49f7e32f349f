// Shared host/device helpers for the sm_100a decode operator kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <utility>

#include "b200ops.h"

namespace b200ops {

// ---- host-side error reporting -------------------------------------------------------
// One message buffer per host thread; b200ops_last_error() returns it.
char* last_error_buffer();
constexpr size_t kLastErrorLen = 512;

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), kLastErrorLen, fmt, ap);
  va_end(ap);
  return code;
}

#define B200OPS_REQUIRE(cond, ...)                         \
  do {                                                     \
    if (!(cond)) return ::b200ops::fail(B200OPS_EINVAL, __VA_ARGS__); \
  } while (0)

#define B200OPS_CUDA(expr)                                                          \
  do {                                                                              \
    cudaError_t err__ = (expr);                                                     \
    if (err__ != cudaSuccess) {                                                     \
      (void)cudaGetLastError(); /* do not leave the error for an unrelated later launch check */ \
      return ::b200ops::fail(B200OPS_ECUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
    }                                                                               \
  } while (0)

// Launch check: reports configuration errors of the launch just made without
// synchronising (asynchronous faults surface at the caller's next sync, as with any stream work).
#define B200OPS_LAUNCH_CHECK(name)                                                        \
  do {                                                                                    \
    cudaError_t err__ = cudaGetLastError();                                               \
    if (err__ != cudaSuccess)                                                             \
      return ::b200ops::fail(B200OPS_ECUDA, "%s launch failed: %s", name, cudaGetErrorString(err__)); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Addresses, valid on this device, of one buffer per rank (peer-mapped memory); passed to
// kernels by value.
constexpr int kMaxPeers = 64;
struct PeerTable {
  void* base[kMaxPeers];
};

// Number of SMs of the current device (cached per device).
int sm_count();

// Tuning knobs.  Each is an environment variable read ONCE per process, at its first use (a
// launch never calls getenv again); b200ops_reload_options() forgets what was read so that the
// next use looks at the environment again.  `knob` returns `fallback` for an unset variable.
enum Knob {
  kKnobGmmPair,         // B200OPS_GMM_PAIR: 0 never use CTA pairs, 2 always, otherwise by shape
  kKnobGmmKsplit,       // B200OPS_GMM_KSPLIT: 0 disables the cluster split-K kernel
  kKnobGmmShort,        // B200OPS_GMM_SHORT: 0 never loads short activation tiles (decode-size grouped GEMMs)
  kKnobPaMode,          // B200OPS_PA_MODE: 2 forces the general attention kernel
  kKnobPaStages,        // B200OPS_PA_STAGES: ring depth of the TMA attention kernel (2, 3, 4, 6)
  kKnobPaChunkTokens,   // B200OPS_PA_CHUNK_TOKENS: base chunk length of the split context
  kKnobRmsnormVpt,      // B200OPS_RMSNORM_VPT: 16-byte vectors per thread
  kKnobRmsnormCtaWarps, // B200OPS_RMSNORM_CTA_WARPS: warps per CTA
  kKnobRacDedup,        // B200OPS_RAC_DEDUP: 0 = skip the repeated-slot check (measurement only)
  kKnobPdl,             // B200OPS_PDL: 0 = plain stream-ordered launches (no programmatic dependent launch)
  kKnobCount
};
int knob(Knob k, int fallback);

// ---- kernel launch ---------------------------------------------------------------------
// Every kernel of the library is launched through launch_kernel() / launch_cluster(), which ask for
// programmatic dependent launch: the kernel may become resident while its predecessor on the
// stream is still draining, so that its launch latency and its set-up (barrier initialisation,
// TMEM allocation, descriptor prefetch) overlap the predecessor's tail.  The contract that makes
// this safe: every kernel executes pdl_wait() before its first access to global memory that an
// earlier kernel may have written or may still read -- in practice before its first global
// access of any kind except L2 prefetches -- and pdl_trigger() as early as it likes.  Launched
// without the attribute (B200OPS_PDL=0, or a predecessor that is not a kernel) both are no-ops
// and the launch is an ordinary stream-ordered one.  Works under stream capture: the edges
// become programmatic dependencies of the CUDA graph.
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (knob(kKnobPdl, 1) != 0) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                          Args&&... args) {
  return launch_cluster(kern, grid, block, smem, st, 1u, std::forward<Args>(args)...);
}
#endif

// ---- device helpers --------------------------------------------------------------------
#ifdef __CUDACC__

// See launch_kernel() above.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 128-bit global loads/stores with cache hints.  Streaming data that is touched once is
// loaded without L1 allocation and stored with an evict-first policy so that it does not
// push reusable lines (weights, cos/sin rows) out of L2.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st_stream(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// 256-bit global accesses (sm_100): one instruction per 32-byte sector.
struct Vec256 {
  uint32_t r[8];
};

__device__ __forceinline__ Vec256 ld_stream256(const void* p) {
  Vec256 v;
  asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]),
                 "=r"(v.r[6]), "=r"(v.r[7])
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st256(void* p, const Vec256& v) {
  asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.r[0]), "r"(v.r[1]),
               "r"(v.r[2]), "r"(v.r[3]), "r"(v.r[4]), "r"(v.r[5]), "r"(v.r[6]), "r"(v.r[7])
               : "memory");
}

__device__ __forceinline__ float2 h2_to_f2(uint32_t u) {
  return __half22float2(*reinterpret_cast<const __half2*>(&u));
}

__device__ __forceinline__ uint32_t f2_to_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// SwiGLU element: (g * sigmoid(g)) * u in fp32, the operand order of the reference's golden
// (benchmark/test_swiglu.py:6-12) and kernel (csrc/opdev/op_kernel/swi_glu_ex.cpp:52-57).
__device__ __forceinline__ float silu_mul(float g, float u) {
  const float sig = __fdividef(1.0f, 1.0f + __expf(-g));
  return (g * sig) * u;
}

#endif  // __CUDACC__

}  // namespace b200ops
