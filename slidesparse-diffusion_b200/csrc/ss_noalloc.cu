// ss_projection_static: the complete projection for callers that must not allocate.
//
// Who needs this: a host that embeds the library inside a memory plan it does not own -- a
// serving engine whose device memory was carved up front (every byte of HBM handed to a pool
// with no headroom left), a real-time or safety-reviewed loop in which cudaMalloc / cudaFree
// are forbidden because they take driver locks, can block on other streams and can fail at an
// arbitrary moment, or a plug-in that may be called from a context where the framework's
// caching allocator is not reachable.  Such a caller still owns its inputs and outputs, but has
// nowhere to put the projection's intermediate (the quantised, slide-expanded activations and
// the per-token scales that travel from the front-end kernel to the GEMM kernel).
//
// Here that intermediate lives in one file-scope device array that is part of the library
// image: every GPU that loads the library holds kStaticScratchBytes of it until the process
// exits, and nothing is ever allocated or freed at run time.
#include "ss_common.cuh"
#include <mutex>

namespace ss {
namespace {

// 32 MiB: enough for, e.g., 1536 tokens x 18432 lifted columns (FLUX MLP fc2 in 6:8 mode) or
// 8192 tokens x 3328 (SD3.5-Large QKV in 4:6 mode).  Larger problems are rejected.
constexpr size_t kStaticScratchBytes = 32u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_address[kMaxDevices] = {};

// The array's name is only a host-side handle; the device address has to be asked for, once per
// device, while that device is current.
int static_scratch(unsigned char** out) {
  int dev = 0;
  SS_CUDA(cudaGetDevice(&dev));
  SS_REQUIRE(dev >= 0 && dev < kMaxDevices, SS_E_LIMIT, "projection_static: device index %d beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_address[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    SS_REQUIRE(e == cudaSuccess && p, SS_E_CUDA, "projection_static: cudaGetSymbolAddress failed: %s",
               cudaGetErrorString(e));
    g_scratch_address[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_address[dev];
  return SS_OK;
}

}  // namespace
}  // namespace ss

using namespace ss;

extern "C" int ss_projection_static(const void* x, int64_t sx, int64_t m, int64_t k, int group,
                                    const int8_t* packed, const int32_t* meta, const float* sw,
                                    const float* bias, int64_t n, int64_t pn, void* out,
                                    int64_t out_stride, void* stream) {
  SS_REQUIRE(mode_ok(group), SS_E_ARG, "projection_static: group must be 4, 6 or 8 (got %d)", group);
  SS_REQUIRE(m > 0 && k > 0 && n > 0, SS_E_ARG, "projection_static: positive m, k, n required");
  SS_REQUIRE(pn % 32 == 0 && pn >= n, SS_E_ARG, "projection_static: pn must be a multiple of 32 and >= n");
  int64_t valid = 0, pk = 0;
  ss_lifted_k(k, group, &valid, &pk);
  const int64_t pm = ceil_to(m, 32);
  const int64_t sa_bytes = ceil_to(pm * static_cast<int64_t>(sizeof(float)), 256);
  const int64_t need = sa_bytes + pm * pk;
  SS_REQUIRE(need <= static_cast<int64_t>(kStaticScratchBytes), SS_E_LIMIT,
             "projection_static: %lld tokens x %lld lifted columns need %lld bytes of scratch, the "
             "built-in scratch holds %lld; use ss_projection with caller scratch instead",
             (long long)pm, (long long)pk, (long long)need, (long long)kStaticScratchBytes);
  unsigned char* base = nullptr;
  if (int rc = static_scratch(&base)) return rc;
  float* sa = reinterpret_cast<float*>(base);
  int8_t* q = reinterpret_cast<int8_t*>(base + sa_bytes);
  // Nothing has to be cleared: the front-end writes every byte of q[pm,pk] and sa[pm] that the
  // GEMM of this call reads, so whatever an earlier call left in the array is never consumed.
  auto s = static_cast<cudaStream_t>(stream);
  if (int rc = launch_quantize_lift(x, sx, m, k, group, q, sa, s)) return rc;
  GemmArgs a{q, packed, meta, sa, sw, bias, nullptr, 0, out, out_stride, m, n, pm, pn, pk, false};
  a.overlap_prologue = true;
  a.allow_split = false;          // the split schedule's tile sums live in memory the library allocates      // same launch pair as ss_projection: the GEMM sets up under the front-end's tail
  return launch_gemm(a, s);
}
