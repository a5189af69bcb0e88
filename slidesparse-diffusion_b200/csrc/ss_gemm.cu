// 2:4 sparse INT8 GEMM for sm_100a: tcgen05.mma.sp (kind::i8) with TMA-fed shared-memory
// stages, INT32 accumulators in tensor memory and a fused dequant / bias / addend / BF16 epilogue.
//
//   acc[ch, tok] = sum_c  W_lifted[ch, c] * q[tok, c]          (exact int32)
//   out[tok, ch] = bf16( fma(float(acc), sa[tok]*sw[ch], bias[ch]) [+ float(addend[tok,ch])] )
//
// The 2:4-compressed weights are the sparse A operand (UMMA M = 128 output channels per tile),
// the quantised activations are B (UMMA N = token tile), so the accumulator lanes are channels
// and its columns are tokens, as in the reference (csrc/dualscale_sm80.cu:189-204).
//
// One persistent CTA per SM, 6 warps:
//   warp 0     TMA producer: per 128-wide lifted-K block one load each of A (128 x 64 B, 64B
//              swizzle), B (NT x 128 B, 128B swizzle) and the metadata block (128 x 16 B)
//   warp 1     owns tensor memory; one lane copies the metadata block to TMEM (tcgen05.cp) and
//              issues two K=64 tcgen05.mma.sp per stage, commits to the stage's empty barrier
//   warps 2-5  epilogue: tcgen05.ld of their 32-lane quadrant, dequantise, store BF16
// Accumulators are double-buffered in TMEM when the token tile leaves room (NT <= 192), so the
// epilogue of tile i overlaps the main loop of tile i+1.  Every mbarrier wait is bounded; a
// wait that runs out records a code in the device status word and the CTA winds down.
#include "ss_common.cuh"
#include <cuda_bf16.h>
#include <mutex>
#include <unordered_map>
#include <vector>
#include <string>
#include <cstdlib>
#include <cstring>

namespace ss {
namespace {

constexpr int kThreads = 192;
constexpr int kTileCh = 128;                     // UMMA M
constexpr int kTileK = 128;                      // lifted K per stage
constexpr int kABytes = kTileCh * kTileK / 2;    // compressed weights per stage
constexpr int kEBytes = kTileCh * kTileK / 8;    // metadata per stage
constexpr int kTmemCols = 512;
constexpr int kMetaColsPerStage = 4;

template <int NT>
struct Tile {
  static constexpr int kBBytes = NT * kTileK;
  static constexpr int kStageBytes = kABytes + kBBytes + kEBytes;
  static constexpr int kStagesRaw = (214 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kAccBufs = (kTmemCols - kStages * kMetaColsPerStage) / NT >= 2 ? 2 : 1;
  static constexpr int kMetaCol = kAccBufs * NT;             // first metadata column
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kOffA + kStages * kABytes;
  static constexpr int kOffE = kOffB + kStages * kBBytes;
  static constexpr int kOffBar = kOffE + kStages * kEBytes;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;    // + barrier block + alignment slack
  static_assert(kMetaCol + kStages * kMetaColsPerStage <= kTmemCols, "TMEM budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  static_assert(NT % 32 == 0 && NT >= 32 && NT <= 256, "token tile");
};

struct KernelArgs {
  const float* sa;
  const float* sw;
  const float* bias;
  const __nv_bfloat16* addend;
  long long addend_stride;
  void* out;
  long long out_stride;
  int m, n;
  int tiles_ch, tiles_tok, num_kb;
  uint32_t* status;
};

__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;
  d |= 1ull << 46;                                   // descriptor version of this architecture
  d |= static_cast<uint64_t>(layout_type) << 61;     // 0 none, 2 128B, 4 64B swizzle
  return d;
}

template <int NT, bool INT32_OUT, bool HAS_ADDEND>
__global__ void __launch_bounds__(kThreads, 1)
sparse_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                   const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_e, const KernelArgs args) {
  using T = Tile<NT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(smem + T::kOffBar);
  uint64_t* bar_empty = bar_full + T::kStages;
  uint64_t* bar_acc_full = bar_empty + T::kStages;
  uint64_t* bar_acc_empty = bar_acc_full + T::kAccBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_acc_empty + T::kAccBufs);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = args.tiles_ch * args.tiles_tok;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      ptx::mbar_init(&bar_full[s], 1);
      ptx::mbar_init(&bar_empty[s], 1);
    }
    for (int b = 0; b < T::kAccBufs; ++b) {
      ptx::mbar_init(&bar_acc_full[b], 1);
      ptx::mbar_init(&bar_acc_empty[b], 4);
    }
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    ptx::prefetch_tensormap(&map_e);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int ch0 = (tile % args.tiles_ch) * kTileCh;
        const int tok0 = (tile / args.tiles_ch) * NT;
        for (int kb = 0; kb < args.num_kb; ++kb, ++issued) {
          const uint32_t s = issued % T::kStages, use = issued / T::kStages;
          if (!ptx::mbar_wait(&bar_empty[s], (use & 1u) ^ 1u)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(&bar_full[s], T::kStageBytes);
          ptx::tma_load_2d(smem + T::kOffA + s * kABytes, &map_a, &bar_full[s], kb * (kTileK / 2), ch0);
          ptx::tma_load_2d(smem + T::kOffB + s * T::kBBytes, &map_b, &bar_full[s], kb * kTileK, tok0);
          ptx::tma_load_3d(smem + T::kOffE + s * kEBytes, &map_e, &bar_full[s], 0, kb, ch0 >> 5);
        }
      }
      if (!ok) {
        atomicOr(args.status, kStatusProducerTimeout);
        // let the copies already in flight land before the CTA's shared memory is released
        for (uint32_t s = 0; s < static_cast<uint32_t>(T::kStages) && s < issued; ++s) {
          const uint32_t fills = (issued - s + T::kStages - 1) / T::kStages;
          ptx::mbar_wait(&bar_full[s], (fills - 1) & 1u);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 2)                 // sparse A
                                 | (2u << 4)               // D format: S32
                                 | (1u << 7) | (1u << 10)  // A, B format: signed 8-bit
                                 | (static_cast<uint32_t>(NT >> 3) << 17) |
                                 (static_cast<uint32_t>(kTileCh >> 4) << 24);
      uint32_t consumed = 0, acc_it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
        const uint32_t buf = acc_it % T::kAccBufs, acc_use = acc_it / T::kAccBufs;
        if (!ptx::mbar_wait(&bar_acc_empty[buf], (acc_use & 1u) ^ 1u)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * NT;
        for (int kb = 0; kb < args.num_kb; ++kb, ++consumed) {
          const uint32_t s = consumed % T::kStages, use = consumed / T::kStages;
          if (!ptx::mbar_wait(&bar_full[s], use & 1u)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_addr = ptx::smem_u32(smem + T::kOffA + s * kABytes);
          const uint32_t b_addr = ptx::smem_u32(smem + T::kOffB + s * T::kBBytes);
          const uint32_t e_addr = ptx::smem_u32(smem + T::kOffE + s * kEBytes);
          const uint32_t e_tmem = tmem_base + T::kMetaCol + s * kMetaColsPerStage;
          ptx::tc_cp_128x128b(e_tmem, smem_desc(e_addr, 128, 128, 0));
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            // K = 64 lifted columns per instruction: 32 B of compressed A, 64 B of B per row
            const uint64_t adesc = smem_desc(a_addr + j * 32, 16, 512, 4);
            const uint64_t bdesc = smem_desc(b_addr + j * 64, 16, 1024, 2);
            ptx::tc_mma_sp_i8(d_tmem, adesc, bdesc, e_tmem + j * 2, idesc, (kb | j) != 0 ? 1u : 0u);
          }
          ptx::tc_commit(&bar_empty[s]);
        }
        if (ok) ptx::tc_commit(&bar_acc_full[buf]);
      }
      if (!ok) atomicOr(args.status, kStatusMmaTimeout);
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
    uint32_t acc_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
      const uint32_t buf = acc_it % T::kAccBufs, acc_use = acc_it / T::kAccBufs;
      const int ch = (tile % args.tiles_ch) * kTileCh + quad * 32 + lane;
      const int tok0 = (tile / args.tiles_ch) * NT;
      const bool ch_ok = ch < args.n;
      float sw = 1.f, bias = 0.f;
      if constexpr (!INT32_OUT) {
        if (ch_ok) {
          sw = __ldg(args.sw + ch);
          if (args.bias) bias = __ldg(args.bias + ch);
        }
      }
      if (!ptx::mbar_wait(&bar_acc_full[buf], acc_use & 1u)) { ok = false; break; }
      ptx::tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < NT / 32; ++c) {
        const int tok_base = tok0 + c * 32;
        if (tok_base >= args.m) break;
        uint32_t r[32];
        ptx::tc_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * NT + c * 32, r);
        ptx::tc_wait_ld();
        if constexpr (INT32_OUT) {
          int32_t* out = static_cast<int32_t*>(args.out);
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (ch_ok && tok_base + j < args.m)
              out[static_cast<long long>(tok_base + j) * args.out_stride + ch] = static_cast<int32_t>(r[j]);
        } else {
          __nv_bfloat16* out = static_cast<__nv_bfloat16*>(args.out);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 s4 = __ldg(reinterpret_cast<const float4*>(args.sa + tok_base) + j4);
            const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const int j = j4 * 4 + jj, tok = tok_base + j;
              float y = __fmaf_rn(__int2float_rn(static_cast<int32_t>(r[j])), __fmul_rn(sv[jj], sw), bias);
              if (ch_ok && tok < args.m) {
                if constexpr (HAS_ADDEND)
                  y = __fadd_rn(y, __bfloat162float(args.addend[static_cast<long long>(tok) * args.addend_stride + ch]));
                out[static_cast<long long>(tok) * args.out_stride + ch] = __float2bfloat16_rn(y);
              }
            }
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bar_acc_empty[buf]);
    }
    if (!ok && lane == 0) atomicOr(args.status, kStatusEpilogueTimeout);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side -----------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

int encode(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base,
           const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
           CUtensorMapSwizzle swizzle) {
  EncodeFn fn = encode_fn();
  SS_REQUIRE(fn, SS_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint32_t ones[3] = {1, 1, 1};
  CUresult r = fn(map, type, rank, const_cast<void*>(base), dims, strides, box, ones,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SS_REQUIRE(r == CUDA_SUCCESS, SS_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return SS_OK;
}

struct DeviceInfo { int sms = 0; bool configured[4][2][2] = {}; };
DeviceInfo* device_info() {
  static std::mutex mu;
  static std::unordered_map<int, DeviceInfo> table;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  DeviceInfo& d = table[dev];
  if (d.sms == 0) {
    if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
  }
  return &d;
}

int pick_token_tile(int64_t m, int64_t pn, int64_t pk, int sms) {
  if (const char* env = std::getenv("SS_TOKEN_TILE")) {
    const int v = std::atoi(env);
    if (v == 64 || v == 128 || v == 192 || v == 256) return v;
  }
  const int64_t tiles_ch = (pn + kTileCh - 1) / kTileCh;
  const double num_kb = static_cast<double>(pk / kTileK);
  const int cand[4] = {256, 192, 128, 64};
  // shared-memory operand traffic per MMA relative to the 256-token tile
  const double feed[4] = {1.0, 1.0625, 1.2, 1.6};
  double best = 0;
  int best_nt = 128;
  for (int i = 0; i < 4; ++i) {
    const int nt = cand[i];
    const int64_t tiles = tiles_ch * ((m + nt - 1) / nt);
    const int64_t waves = (tiles + sms - 1) / sms;
    const bool overlapped = nt <= 192;
    // per-tile time in "k-block units": main loop plus the part of the epilogue that is exposed
    const double epilogue = 6.0 * nt / 256.0;
    const double main = num_kb * feed[i] * nt / 256.0;
    const double tile_time = overlapped ? (main > epilogue ? main : epilogue) + 0.5 : main + epilogue + 0.5;
    const double cost = waves * tile_time;
    if (best == 0 || cost < best) { best = cost; best_nt = nt; }
  }
  return best_nt;
}

template <int NT, bool I32, bool ADD>
int launch_t(const GemmArgs& a, DeviceInfo* dev, int cfg_index, cudaStream_t stream) {
  using T = Tile<NT>;
  auto kernel = sparse_gemm_kernel<NT, I32, ADD>;
  if (!dev->configured[cfg_index][I32][ADD]) {
    SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes));
    dev->configured[cfg_index][I32][ADD] = true;
  }
  CUtensorMap map_a, map_b, map_e;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.pk / 2), static_cast<cuuint64_t>(a.pn)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.pk / 2)};
    const cuuint32_t box[2] = {kTileK / 2, kTileCh};
    int rc = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.packed, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
  }
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.pk), static_cast<cuuint64_t>(a.pm)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.pk)};
    const cuuint32_t box[2] = {kTileK, NT};
    int rc = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    const cuuint64_t kblocks = static_cast<cuuint64_t>(a.pk / kTileK);
    const cuuint64_t dims[3] = {128, kblocks, static_cast<cuuint64_t>(a.pn / 32)};
    const cuuint64_t strides[2] = {512, kblocks * 512};
    const cuuint32_t box[3] = {128, 1, 4};
    int rc = encode(&map_e, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, a.meta, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  KernelArgs k;
  k.sa = a.sa; k.sw = a.sw; k.bias = a.bias;
  k.addend = static_cast<const __nv_bfloat16*>(a.addend);
  k.addend_stride = a.addend_stride;
  k.out = a.out; k.out_stride = a.out_stride;
  k.m = static_cast<int>(a.m); k.n = static_cast<int>(a.n);
  k.tiles_ch = static_cast<int>((a.pn + kTileCh - 1) / kTileCh);
  k.tiles_tok = static_cast<int>((a.m + NT - 1) / NT);
  k.num_kb = static_cast<int>(a.pk / kTileK);
  k.status = device_status_ptr();
  SS_REQUIRE(k.status, SS_E_CUDA, "device status word unavailable");
  const int64_t tiles = static_cast<int64_t>(k.tiles_ch) * k.tiles_tok;
  const unsigned grid = static_cast<unsigned>(tiles < dev->sms ? tiles : dev->sms);
  kernel<<<grid, kThreads, T::kSmemBytes, stream>>>(map_a, map_b, map_e, k);
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}

template <int NT>
int launch_nt(const GemmArgs& a, DeviceInfo* dev, int cfg_index, cudaStream_t stream) {
  if (a.int32_out) return launch_t<NT, true, false>(a, dev, cfg_index, stream);
  if (a.addend) return launch_t<NT, false, true>(a, dev, cfg_index, stream);
  return launch_t<NT, false, false>(a, dev, cfg_index, stream);
}

int check_args(const GemmArgs& a) {
  SS_REQUIRE(a.q && a.packed && a.meta && a.out, SS_E_ARG, "gemm: null pointer");
  SS_REQUIRE(a.int32_out || (a.sa && a.sw), SS_E_ARG, "gemm: scales required");
  SS_REQUIRE(a.pk > 0 && a.pk % 128 == 0 && a.pm > 0 && a.pm % 32 == 0 && a.pn > 0 && a.pn % 32 == 0,
             SS_E_ARG, "gemm: padding mismatch (pm=%lld pn=%lld pk=%lld)", (long long)a.pm, (long long)a.pn, (long long)a.pk);
  SS_REQUIRE(a.pk <= 131008, SS_E_ARG, "gemm: INT32 worst-case bound exceeded (pk=%lld)", (long long)a.pk);
  SS_REQUIRE(a.m > 0 && a.m <= a.pm && a.n > 0 && a.n <= a.pn, SS_E_ARG,
             "gemm: original dimensions exceed the padded ones (m=%lld n=%lld)", (long long)a.m, (long long)a.n);
  SS_REQUIRE(a.pm < (1ll << 31) && a.pn < (1ll << 31), SS_E_ARG, "gemm: dimension too large");
  SS_REQUIRE(a.out_stride >= a.n, SS_E_ARG, "gemm: output row stride smaller than n");
  SS_REQUIRE((reinterpret_cast<uintptr_t>(a.q) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.packed) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(a.meta) & 15) == 0,
             SS_E_ARG, "gemm: q, packed and metadata must be 16-byte aligned");
  SS_REQUIRE(a.int32_out || (reinterpret_cast<uintptr_t>(a.sa) & 15) == 0, SS_E_ARG,
             "gemm: token scales must be 16-byte aligned");
  SS_REQUIRE(!a.addend || a.addend_stride >= a.n, SS_E_ARG, "gemm: addend row stride smaller than n");
  return SS_OK;
}

}  // namespace

int launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (int rc = check_args(a)) return rc;
  DeviceInfo* dev = device_info();
  SS_REQUIRE(dev, SS_E_CUDA, "gemm: no current CUDA device");
  switch (pick_token_tile(a.m, a.pn, a.pk, dev->sms)) {
    case 256: return launch_nt<256>(a, dev, 0, stream);
    case 192: return launch_nt<192>(a, dev, 1, stream);
    case 128: return launch_nt<128>(a, dev, 2, stream);
    default:  return launch_nt<64>(a, dev, 3, stream);
  }
}

template <int NT>
static int resources_t(GemmResources* r) {
  using T = Tile<NT>;
  auto kernel = sparse_gemm_kernel<NT, false, false>;
  cudaFuncAttributes attr;
  SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes));
  SS_CUDA(cudaFuncGetAttributes(&attr, kernel));
  int blocks = 0;
  SS_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kThreads, T::kSmemBytes));
  r->threads = kThreads; r->smem = T::kSmemBytes; r->regs = attr.numRegs;
  r->local = static_cast<int>(attr.localSizeBytes); r->ctas_per_sm = blocks;
  r->token_tile = NT; r->stages = T::kStages; r->tmem_cols = kTmemCols;
  return SS_OK;
}

int gemm_resources(int64_t m, int64_t n, int64_t pk, GemmResources* r) {
  DeviceInfo* dev = device_info();
  SS_REQUIRE(dev, SS_E_CUDA, "gemm: no current CUDA device");
  switch (pick_token_tile(m, ceil_to(n, 32), pk, dev->sms)) {
    case 256: return resources_t<256>(r);
    case 192: return resources_t<192>(r);
    case 128: return resources_t<128>(r);
    default:  return resources_t<64>(r);
  }
}

}  // namespace ss
