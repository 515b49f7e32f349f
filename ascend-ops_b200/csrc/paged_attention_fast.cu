// Placeholder translation unit: the TMA/mma fast path is not wired yet.
#include "paged_attention.cuh"
namespace b200ops { namespace pa {
bool fast_path_supported(const Args&) { return false; }
int launch_fast(const Args&, cudaStream_t) { return fail(B200OPS_EUNSUPPORTED, "paged_attention: fast path not built"); }
}}
