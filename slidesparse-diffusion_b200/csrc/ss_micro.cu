// Micro-benchmark behind the statement that a sparse INT8 tcgen05.mma is bound by shared-memory
// operand reads, not by the tensor pipe: one CTA issues back-to-back MMAs of 128 x N (sparse: K = 64
// lifted columns, dense: K = 32) whose operands rotate through four shared-memory slots, and the
// cycles per instruction are compared with the tensor-pipe time of that instruction.  No global
// memory traffic, no TMA: only the instruction stream and the operand reads.  Diagnostic only; no
// part of the projection calls it.
#include "ss_common.cuh"

namespace ss {
namespace {

__device__ __forceinline__ uint64_t micro_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  uint64_t d = static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= 1ull << 46;
  d |= static_cast<uint64_t>(layout) << 61;
  return d;
}

__device__ __forceinline__ void micro_mma_dense_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(1));
}

template <int NT, int SPARSE>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(long long* cycles, uint32_t* status, int iters, int with_cp) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  // any bit pattern is a valid operand; 0x44 nibbles are valid index pairs for the metadata
  for (int i = threadIdx.x; i < 200 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x44444444u;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::fence_barrier_init();
  }
  if (threadIdx.x < 32) {
    ptx::tmem_alloc(&slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = slot;
  constexpr uint32_t idesc = (static_cast<uint32_t>(SPARSE) << 2) | (2u << 4) | (1u << 7) | (1u << 10) |
                             (static_cast<uint32_t>(NT >> 3) << 17) | (8u << 24);
  if (threadIdx.x == 0) {
    const uint32_t base = ptx::smem_u32(smem);
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      const uint32_t s = i % 4;
      const uint32_t a = base + s * 8192, b = base + 32768 + s * 32768, e = base + 163840 + s * 2048;
      const uint32_t e_tmem = tmem + 256 + s * 4;
      if (with_cp) ptx::tc_cp_128x128b(e_tmem, micro_desc(e, 128, 128, 0));
      for (int j = 0; j < 2; ++j) {
        if (SPARSE)
          ptx::tc_mma_sp_i8(tmem, micro_desc(a + j * 32, 16, 512, 4), micro_desc(b + j * 64, 16, 1024, 2), e_tmem + 2 * j, idesc, 1);
        else
          micro_mma_dense_i8(tmem, micro_desc(a + j * 32, 16, 512, 4), micro_desc(b + j * 32, 16, 1024, 2), idesc);
      }
    }
    ptx::tc_commit(&bar);
    if (!ptx::mbar_wait(&bar, 0)) atomicOr(status, kStatusMmaTimeout);     // bounded (about two seconds)
    cycles[0] = clock64() - t0;
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

template <int NT, int SPARSE>
int run_rate(int iters, int with_cp, double* cycles_per_mma) {
  const int smem = 212 * 1024;
  long long* d_cycles = nullptr;
  SS_CUDA(cudaFuncSetAttribute(mma_rate_kernel<NT, SPARSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  SS_CUDA(cudaMalloc(&d_cycles, sizeof(long long)));
  uint32_t* status = device_status_ptr();
  int rc = SS_OK;
  long long host = 0;
  for (int rep = 0; rep < 2 && rc == SS_OK; ++rep) {            // first launch warms up
    mma_rate_kernel<NT, SPARSE><<<1, 128, smem>>>(d_cycles, status, iters, with_cp);
    if (cudaDeviceSynchronize() != cudaSuccess) rc = SS_E_CUDA;
  }
  if (rc == SS_OK && cudaMemcpy(&host, d_cycles, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) rc = SS_E_CUDA;
  cudaFree(d_cycles);
  if (rc != SS_OK) {
    set_error("mma rate micro-benchmark: %s", cudaGetErrorString(cudaGetLastError()));
    return rc;
  }
  *cycles_per_mma = static_cast<double>(host) / iters / 2.0;
  return SS_OK;
}

}  // namespace
}  // namespace ss

namespace ss {
namespace {

// One warp waits, with the given limit, on an mbarrier that nothing ever arrives on.  The wait
// must run out, the kernel must record that in the device status word and return normally.
__global__ void wait_limit_kernel(unsigned long long limit_ns, uint32_t* status, unsigned long long* elapsed_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&bar, 1);
    ptx::fence_barrier_init();
    const uint64_t t0 = ptx::globaltimer_ns();
    const bool arrived = ptx::mbar_wait(&bar, 0, limit_ns);
    elapsed_ns[0] = ptx::globaltimer_ns() - t0;
    if (!arrived) atomicOr(status, kStatusProbeTimeout);
  }
}

}  // namespace
}  // namespace ss

extern "C" int ss_micro_wait_limit(int64_t limit_ns, int64_t* elapsed_ns) {
  using namespace ss;
  SS_REQUIRE(elapsed_ns, SS_E_ARG, "wait limit probe: result pointer required");
  SS_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ll, SS_E_ARG,
             "wait limit probe: limit must be between 1 ns and 100 ms (got %lld)", (long long)limit_ns);
  uint32_t* status = device_status_ptr();
  SS_REQUIRE(status, SS_E_CUDA, "device status word unavailable");
  unsigned long long* d_elapsed = nullptr;
  SS_CUDA(cudaMalloc(&d_elapsed, sizeof(unsigned long long)));
  wait_limit_kernel<<<1, 32>>>(static_cast<unsigned long long>(limit_ns), status, d_elapsed);
  unsigned long long host = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(&host, d_elapsed, sizeof(host), cudaMemcpyDeviceToHost);
  cudaFree(d_elapsed);
  SS_REQUIRE(e == cudaSuccess, SS_E_CUDA, "wait limit probe: %s", cudaGetErrorString(e));
  *elapsed_ns = static_cast<int64_t>(host);
  return SS_OK;
}

extern "C" int ss_micro_pair_rate(int64_t m, int64_t n, int64_t pk, int token_tile, int flags,
                                  double* cycles_per_stage, int64_t* stages) {
  using namespace ss;
  SS_REQUIRE(cycles_per_stage && stages, SS_E_ARG, "pair rate: result pointers required");
  SS_REQUIRE(m > 0 && n > 0 && pk > 0 && pk % 128 == 0 && m <= 65536 && n <= 65536 && pk <= 65536, SS_E_ARG,
             "pair rate: sizes must be positive, pk a multiple of 128, each at most 65536");
  SS_REQUIRE((flags & ~15) == 0, SS_E_ARG, "pair rate: flags are bits 0..3 (no MMAs, no epilogue, no TMA stores, TMEM loads only)");
  const int64_t pm = ceil_to(m, 32), pn = ceil_to(n, 32);
  const size_t q_bytes = static_cast<size_t>(pm) * pk, a_bytes = static_cast<size_t>(pn) * pk / 2;
  const size_t e_bytes = static_cast<size_t>(pn) * pk / 8, o_bytes = static_cast<size_t>(m) * pn * 2;
  unsigned char* base = nullptr;
  const size_t v_bytes = static_cast<size_t>(pm + 2 * pn) * sizeof(float);
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  const size_t total = up(q_bytes) + up(a_bytes) + up(e_bytes) + up(o_bytes) + up(v_bytes) + 256;
  SS_CUDA(cudaMalloc(&base, total));
  unsigned char* q = base;
  unsigned char* packed = q + up(q_bytes);
  unsigned char* meta = packed + up(a_bytes);
  unsigned char* out = meta + up(e_bytes);
  float* vec = reinterpret_cast<float*>(out + up(o_bytes));
  unsigned long long* probe = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(vec) + up(v_bytes));
  int rc = SS_OK;
  // any bytes are valid operands; 0x44 nibbles are valid index pairs for the metadata
  if (cudaMemset(q, 1, q_bytes) != cudaSuccess || cudaMemset(packed, 1, a_bytes) != cudaSuccess ||
      cudaMemset(meta, 0x44, e_bytes) != cudaSuccess || cudaMemset(vec, 0, v_bytes) != cudaSuccess ||
      cudaMemset(probe, 0, 16) != cudaSuccess)
    rc = SS_E_CUDA;
  Options& opt = options();
  const int saved_tile = opt.token_tile, saved_resident = opt.resident;
  opt.token_tile = token_tile;
  GemmArgs a{reinterpret_cast<const int8_t*>(q), reinterpret_cast<const int8_t*>(packed),
             reinterpret_cast<const int32_t*>(meta), vec, vec + pm, vec + pm + pn, nullptr, 0, out, pn,
             m, n, pm, pn, pk, false};
  a.debug = flags;
  a.probe = probe;
  a.allow_split = false;          // the rate is that of the whole-tile schedule
  for (int rep = 0; rep < 3 && rc == SS_OK; ++rep) {          // the first launches warm up
    rc = launch_gemm(a, nullptr);
    if (rc == SS_OK && cudaDeviceSynchronize() != cudaSuccess) rc = SS_E_CUDA;
  }
  opt.token_tile = saved_tile;
  opt.resident = saved_resident;
  unsigned long long host[2] = {0, 0};
  if (rc == SS_OK && cudaMemcpy(host, probe, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) rc = SS_E_CUDA;
  if (rc == SS_E_CUDA) set_error("pair rate micro-benchmark: %s", cudaGetErrorString(cudaGetLastError()));
  cudaFree(base);
  if (rc != SS_OK) return rc;
  SS_REQUIRE(host[1] > 0, SS_E_CUDA, "pair rate micro-benchmark: the kernel reported no stages");
  *cycles_per_stage = static_cast<double>(host[0]) / static_cast<double>(host[1]);
  *stages = static_cast<int64_t>(host[1]);
  return SS_OK;
}

extern "C" int ss_micro_mma_rate(int token_tile, int sparse, int with_metadata_copy, int iterations,
                                 double* cycles_per_mma) {
  using namespace ss;
  SS_REQUIRE(cycles_per_mma && iterations > 0 && iterations <= (1 << 20), SS_E_ARG, "mma rate: bad arguments");
  SS_REQUIRE(device_status_ptr(), SS_E_CUDA, "device status word unavailable");
#define SS_RATE(NT)                                                                           \
  if (token_tile == NT)                                                                       \
    return sparse ? run_rate<NT, 1>(iterations, with_metadata_copy, cycles_per_mma)            \
                  : run_rate<NT, 0>(iterations, 0, cycles_per_mma)
  SS_RATE(64);
  SS_RATE(128);
  SS_RATE(192);
  SS_RATE(256);
#undef SS_RATE
  set_error("mma rate: token tile must be 64, 128, 192 or 256 (got %d)", token_tile);
  return SS_E_ARG;
}
