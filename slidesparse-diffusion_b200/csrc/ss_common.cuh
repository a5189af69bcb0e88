// Shared host/device helpers of the sm_100a sparse W8A8 projection library.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include "../../include/slidesparse_b200.h"

namespace ss {

// ---- host-side error plumbing -----------------------------------------------------------
void set_error(const char* fmt, ...);
#define SS_REQUIRE(cond, code, ...)                \
  do {                                             \
    if (!(cond)) {                                 \
      ::ss::set_error(__VA_ARGS__);                \
      return (code);                               \
    }                                              \
  } while (0)
#define SS_CUDA(call)                                                                   \
  do {                                                                                  \
    cudaError_t e__ = (call);                                                           \
    if (e__ != cudaSuccess) {                                                           \
      ::ss::set_error("%s failed: %s", #call, cudaGetErrorString(e__));                 \
      return SS_E_CUDA;                                                                 \
    }                                                                                   \
  } while (0)

inline int64_t ceil_to(int64_t v, int64_t a) { return (v + a - 1) / a * a; }
inline bool mode_ok(int group) { return group == 4 || group == 6 || group == 8; }

// Device status word: a kernel that gives up on a bounded wait ORs a code into it.
enum : uint32_t {
  kStatusProducerTimeout = 1u,
  kStatusMmaTimeout = 2u,
  kStatusEpilogueTimeout = 4u,
  kStatusProbeTimeout = 8u,      // the wait-limit diagnostic (ss_micro_wait_limit)
};
uint32_t* device_status_ptr();   // address of the status word on the current device (or nullptr)
constexpr unsigned long long kDefaultWaitNs = 2000000000ull;   // limit of every mbarrier wait

// Tuning switches.  Read from the environment ONCE, when the library is first used (SS_TOKEN_TILE,
// SS_WIDE_CP, SS_META_WARP, SS_STORE, SS_RESIDENT, SS_PDL, SS_WAIT_NS), and changeable afterwards
// through ss_set_option; the launch path itself never calls getenv.
struct Options {
  int token_tile = 0;     // 0 = chosen per problem; 128 / 192 / 224 / 256 force a tile
  int wide_cp = 1;        // one tcgen05.cp.128x256b per stage instead of two 128x128b
  int meta_warp = -1;     // -1 = by pipeline depth; 0 / 1 force the metadata-copy warp off / on
  int store = 1;          // 1 = TMA-store epilogue where alignment allows, 0 = direct stores
  int resident = 1;       // weights-resident form where applicable
  int pdl = 1;            // programmatic dependent launch between front-end and GEMM
  int split = -1;         // split schedule of the GEMM: -1 = where the cost model prefers it, 0 never, 1 wherever eligible
  unsigned long long wait_ns = kDefaultWaitNs;
};
Options& options();

// cuTensorMapEncodeTiled behind a per-process cache keyed by everything the descriptor encodes
// (address, type, extents, pitches, box, swizzle): a descriptor is pure geometry, so one built for
// an address stays valid for as long as that geometry is wanted there.  Weights and the scratch of a
// prepared plan hit the cache on every launch after the first.
struct MapKey {
  const void* base;
  int type, rank, swizzle;
  unsigned long long dims[3], strides[2];
  unsigned box[3];
};
int encode_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base,
               const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
               CUtensorMapSwizzle swizzle);

// ---- entry points implemented per kernel file -------------------------------------------
int launch_quantize_lift(const void* x, int64_t sx, int64_t m, int64_t k, int group,
                         int8_t* q, float* sa, cudaStream_t stream);
int launch_quantize_lift_fused(const void* x, int64_t sx, int64_t m, int64_t k, int group, int prologue,
                               const void* shift, const void* scale, int64_t mod_stride,
                               int64_t rows_per_batch, float eps, int8_t* q, float* sa, cudaStream_t stream);

struct GemmArgs {
  const int8_t* q;
  const int8_t* packed;
  const int32_t* meta;
  const float* sa;
  const float* sw;
  const float* bias;
  const void* addend;
  int64_t addend_stride;
  void* out;            // bf16 or int32
  int64_t out_stride;
  int64_t m, n, pm, pn, pk;
  bool int32_out;
  // the launch directly follows the front-end that produces q and sa in the same stream: the
  // kernel may start (set-up, weight prefetch) before that grid has finished and waits on the
  // device before it touches q, sa or out
  bool overlap_prologue = false;
  // gated accumulation (an extension): out[t, c] += bf16(gate[t / rows_per_batch, c] * y[t, c])
  // instead of out[t, c] = bf16(y[t, c]); gate is BF16 with gate_stride elements between batches
  const void* gate = nullptr;
  int64_t gate_stride = 0;
  int64_t rows_per_batch = 0;
  // tensor-parallel form (an extension): the BF16 result is stored to peer_count destinations
  // (this GPU's and its peers' copies of the gathered output, each pointer already at this rank's
  // first column) instead of `out`; all share out_stride
  const void* peer_out[8] = {};
  int peer_count = 0;
  // diagnostics (ss_micro.cu): wait limit of this launch (0 = the library's), kernel parts switched
  // off (bit 0 the MMAs, 1 the epilogue work, 2 its TMA stores, 3 all but its TMEM loads), and where
  // cluster 0 reports {cycles, stages}
  unsigned long long wait_ns = 0;
  int debug = 0;
  unsigned long long* probe = nullptr;
  // false: the launch may not use the library's own device memory beyond the status word (the
  // split schedule sums shared tiles in an area the library allocates on first use)
  bool allow_split = true;
};
constexpr int kMaxPeers = 8;
struct GemmResources {
  int threads, smem, regs, local, ctas_per_sm, token_tile, stages, tmem_cols;
};
int launch_gemm(const GemmArgs& a, cudaStream_t stream);
// Zeroes the split schedule's tile-sum area of the current device (after a launch that gave up on a wait).
int reset_split_workspace();
// GEMM launches of this process that took the split schedule (read-only "split_launches" of ss_get_option).
long long split_launch_count();
int gemm_resources(int64_t m, int64_t n, int64_t pk, GemmResources* r);

}  // namespace ss

// ---- device-side PTX wrappers -------------------------------------------------------------
#if defined(__CUDACC__)
namespace ss { namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after limit_ns of wall time (two seconds unless the launch says
// otherwise) and returns false.  The clock is looked at every 64 polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          unsigned long long limit_ns = kDefaultWaitNs) {
  if (mbar_test(bar, parity)) return true;
  uint64_t deadline = 0;
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_test(bar, parity)) return true;
    if ((spin & 0x3fu) == 0) {
      uint64_t now = globaltimer_ns();
      if (deadline == 0) deadline = now + limit_ns;
      else if (now > deadline) return false;
    }
  }
}

// TMA tiled loads (no multicast anywhere in this library).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// tcgen05 / tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_slot)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar))
               : "memory");
}
// 128 lanes x 128 bit from shared memory (matrix descriptor) into 4 TMEM columns.
__device__ __forceinline__ void tc_cp_128x128b(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// D[tmem] (+)= A_sparse[smem] * B[smem], 2:4 metadata in TMEM, INT8 x INT8 -> INT32.
__device__ __forceinline__ void tc_mma_sp_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                             uint32_t e_tmem, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.sp.cta_group::1.kind::i8 [%0], %1, %2, [%3], %4, p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread.
__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 16 lanes x 32 columns in the matrix-fragment layout: for each group of 8 columns g, thread t
// holds r[4g+0], r[4g+1] = lane t/4, columns 8g + 2(t%4) and +1; r[4g+2], r[4g+3] = lane t/4 + 8,
// same columns.  The lane field of taddr selects which 16 lanes of the warp's quadrant.
__device__ __forceinline__ void tc_ld_16x256b_x4(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Four 8x8 matrices of 16-bit elements, transposed on the way: thread t's register i carries, for
// matrix i, the elements of memory rows 2(t%4) (low half) and 2(t%4)+1 (high half) at position t/4;
// thread t supplies the address of row t%8 of matrix t/8 (16 bytes per row).
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};"
               ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
// Programmatic dependent launch: a kernel launched with programmatic stream serialization may
// start once every CTA of the preceding kernel has called grid_dep_launch (or exited); it must
// call grid_dep_wait before touching anything that kernel writes.  Both are no-ops otherwise.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// TMA tiled store of a shared-memory tile (bulk async-group completion, issuing thread only).
// TMA tiled reduction: global[tile] += shared[tile], element-wise in the tensor map's type.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
// The same store with an L2 eviction-priority hint: evict_first, for outputs far larger than L2,
// whose lines would otherwise push the operands out while they wait for their write-back.
__device__ __forceinline__ void tma_store_2d_evict_first(const CUtensorMap* map, const void* src, int x, int y) {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;"
               ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's bulk groups still have to read their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- CTA-pair (cta_group::2) variants.  A pair is the two CTAs of a 2-CTA cluster; rank 0
// issues the MMAs for both.  Shared-memory addresses of the two CTAs differ only in bit 24 of
// their shared::cluster form, so clearing that bit names the same object in rank 0.
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_rank0(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPeerMask) : "memory");
}
// Loads issued by either CTA of the pair; completion bytes are credited to rank 0's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* bar,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & kPeerMask), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint64_t* bar,
                                                 int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar) & kPeerMask), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_slot)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
// Arrives on the barrier at this shared-memory offset in every CTA of `mask` once all earlier
// tcgen05 operations of the issuing thread have completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}
__device__ __forceinline__ void tc_cp_128x128b_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// 128 lanes x 256 bit: two 16-byte column blocks of the source (leading-dimension offset apart)
// land in 8 consecutive TMEM columns.
__device__ __forceinline__ void tc_cp_128x256b_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.128x256b [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_sp_i8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                  uint32_t e_tmem, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.sp.cta_group::2.kind::i8 [%0], %1, %2, [%3], %4, p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(e_tmem), "r"(idesc), "r"(accumulate)
      : "memory");
}

}}  // namespace ss::ptx
#endif
