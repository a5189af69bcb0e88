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
//   warp 0     TMA producer.  A pipeline stage holds KB blocks of 128 lifted columns (KB = 2
//              wherever shared memory allows): one load of A (128 rows x 64*KB bytes), and per
//              block one load of B (NT rows x 128 B, 128B swizzle) and of metadata (128 x 16 B)
//   warp 1     owns tensor memory; one lane copies the metadata blocks to TMEM (tcgen05.cp),
//              issues 2*KB tcgen05.mma.sp (K = 64 each) per stage and commits to the stage's
//              empty barrier.  The tensor pipe accepts little work ahead of what it executes,
//              so everything else this lane does between two MMAs (barrier wait, commit) leaves
//              the pipe idle: stages are as large as they can be and the next stage's barrier
//              is tested before the current stage's MMAs are issued.
//   warps 2-5  epilogue: token scales of the tile are staged in shared memory before the
//              accumulator is ready; tcgen05.ld of the warp's 32-lane quadrant is double
//              buffered, the TMEM buffer is handed back as soon as the last load has landed.
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
#include <type_traits>

namespace ss {
namespace {

constexpr int kThreads = 192;
constexpr int kTileCh = 128;                     // UMMA M
constexpr int kBlockK = 128;                     // lifted columns per metadata / B block
constexpr int kTmemCols = 512;

template <int NT, int KB>
struct Tile {
  static constexpr int kABytes = kTileCh * (kBlockK / 2) * KB;   // compressed weights per stage
  static constexpr int kBBlock = NT * kBlockK;                    // one B block
  static constexpr int kBBytes = kBBlock * KB;
  static constexpr int kEBlock = kTileCh * kBlockK / 8;           // one metadata block (2 KB)
  static constexpr int kEBytes = kEBlock * KB;
  static constexpr int kStageBytes = kABytes + kBBytes + kEBytes;
  static constexpr int kStagesRaw = (212 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kMetaColsPerStage = 4 * KB;
  static constexpr int kAccBufs = (kTmemCols - kStages * kMetaColsPerStage) / NT >= 2 ? 2 : 1;
  static constexpr int kMetaCol = kAccBufs * NT;             // first metadata column
  static constexpr int kOffA = 0;
  static constexpr int kOffB = kOffA + kStages * kABytes;
  static constexpr int kOffE = kOffB + kStages * kBBytes;
  static constexpr int kOffSa = kOffE + kStages * kEBytes;   // 4 warps x NT token scales
  static constexpr int kOffBar = kOffSa + 4 * NT * 4;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;    // + barrier block + alignment slack
  static_assert(kStages >= 2, "pipeline depth");
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
  int wide_cp;          // CTA-pair kernel: copy a stage's two metadata blocks with one tcgen05.cp
  int meta_warp;        // CTA-pair kernel: a dedicated warp issues the metadata copies
  const __nv_bfloat16* gate;   // gated accumulation: BF16 [batches, n], rows gate_stride apart
  long long gate_stride;
  int rows_per_batch;
  int res_stages;       // weights-resident form: activation pipeline stages
  int peer_count;       // tensor-parallel form: number of destination tensor maps
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

__device__ __forceinline__ bool mbar_peek(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(ptx::smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Dequantise one 32-token chunk held in registers (lane = channel) and store it.
template <bool INT32_OUT, bool HAS_ADDEND>
__device__ __forceinline__ void store_chunk(const uint32_t (&r)[32], const KernelArgs& args,
                                            const float* sa_chunk, int tok_base, int ch, bool ch_ok,
                                            float sw, float bias) {
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
      const float4 s4 = reinterpret_cast<const float4*>(sa_chunk)[j4];
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

template <int NT, int KB, bool INT32_OUT, bool HAS_ADDEND>
__global__ void __launch_bounds__(kThreads, 1)
sparse_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                   const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_e, const KernelArgs args) {
  using T = Tile<NT, KB>;
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
  const int num_st = (args.num_kb + KB - 1) / KB;          // pipeline stages per tile

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
        for (int st = 0; st < num_st; ++st, ++issued) {
          const uint32_t s = issued % T::kStages, use = issued / T::kStages;
          const int kb0 = st * KB;
          const int nkb = args.num_kb - kb0 < KB ? args.num_kb - kb0 : KB;
          if (!ptx::mbar_wait(&bar_empty[s], (use & 1u) ^ 1u)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(&bar_full[s], T::kABytes + nkb * (T::kBBlock + T::kEBlock));
          // the A box always spans KB blocks; columns past the row end arrive as zeros
          ptx::tma_load_2d(smem + T::kOffA + s * T::kABytes, &map_a, &bar_full[s], kb0 * (kBlockK / 2), ch0);
          for (int h = 0; h < nkb; ++h) {
            ptx::tma_load_2d(smem + T::kOffB + s * T::kBBytes + h * T::kBBlock, &map_b, &bar_full[s],
                             (kb0 + h) * kBlockK, tok0);
            ptx::tma_load_3d(smem + T::kOffE + s * T::kEBytes + h * T::kEBlock, &map_e, &bar_full[s], 0,
                             kb0 + h, ch0 >> 5);
          }
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
      // A rows are 64*KB bytes: 64B swizzle (8 rows = 512 B) or 128B swizzle (8 rows = 1024 B)
      constexpr uint32_t a_layout = KB == 2 ? 2u : 4u, a_sbo = KB == 2 ? 1024u : 512u;
      uint32_t consumed = 0, acc_it = 0;
      bool ok = true, ready = false;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
        const uint32_t buf = acc_it % T::kAccBufs, acc_use = acc_it / T::kAccBufs;
        if (!ptx::mbar_wait(&bar_acc_empty[buf], (acc_use & 1u) ^ 1u)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * NT;
        for (int st = 0; st < num_st; ++st, ++consumed) {
          const uint32_t s = consumed % T::kStages, use = consumed / T::kStages;
          const int kb0 = st * KB;
          const int nkb = args.num_kb - kb0 < KB ? args.num_kb - kb0 : KB;
          if (!ready && !ptx::mbar_wait(&bar_full[s], use & 1u)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_addr = ptx::smem_u32(smem + T::kOffA + s * T::kABytes);
          const uint32_t b_addr = ptx::smem_u32(smem + T::kOffB + s * T::kBBytes);
          const uint32_t e_addr = ptx::smem_u32(smem + T::kOffE + s * T::kEBytes);
          const uint32_t e_tmem = tmem_base + T::kMetaCol + s * T::kMetaColsPerStage;
          for (int h = 0; h < nkb; ++h)
            ptx::tc_cp_128x128b(e_tmem + 4 * h, smem_desc(e_addr + h * T::kEBlock, 128, 128, 0));
          {  // look at the next stage's barrier while the pipe is still busy
            const uint32_t s2 = (consumed + 1) % T::kStages, use2 = (consumed + 1) / T::kStages;
            ready = mbar_peek(&bar_full[s2], use2 & 1u);
          }
          for (int j = 0; j < 2 * nkb; ++j) {
            // K = 64 lifted columns per instruction: 32 B of compressed A, 64 B of B per row
            const uint64_t adesc = smem_desc(a_addr + j * 32, 16, a_sbo, a_layout);
            const uint64_t bdesc = smem_desc(b_addr + (j >> 1) * T::kBBlock + (j & 1) * 64, 16, 1024, 2);
            ptx::tc_mma_sp_i8(d_tmem, adesc, bdesc, e_tmem + j * 2, idesc, (st | j) != 0 ? 1u : 0u);
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
    float* sa_s = reinterpret_cast<float*>(smem + T::kOffSa) + (warp - 2) * NT;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++acc_it) {
      const uint32_t buf = acc_it % T::kAccBufs, acc_use = acc_it / T::kAccBufs;
      const int ch = (tile % args.tiles_ch) * kTileCh + quad * 32 + lane;
      const int tok0 = (tile / args.tiles_ch) * NT;
      const bool ch_ok = ch < args.n;
      float sw = 1.f, bias = 0.f;
      if constexpr (!INT32_OUT) {
        // stage this tile's token scales while the main loop is still running
        __syncwarp();
        for (int i = lane; i < NT; i += 32) sa_s[i] = tok0 + i < args.m ? __ldg(args.sa + tok0 + i) : 1.f;
        if (ch_ok) {
          sw = __ldg(args.sw + ch);
          if (args.bias) bias = __ldg(args.bias + ch);
        }
        __syncwarp();
      }
      int chunks = (args.m - tok0 + 31) / 32;
      chunks = chunks < NT / 32 ? chunks : NT / 32;
      if (!ptx::mbar_wait(&bar_acc_full[buf], acc_use & 1u)) { ok = false; break; }
      ptx::tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * NT;
      auto release = [&]() {                         // every load has landed: hand the buffer back
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&bar_acc_empty[buf]);
      };
      uint32_t r0[32], r1[32];
      ptx::tc_ld_32x32b_x32(t_addr, r0);
#pragma unroll 1
      for (int c = 0; c < chunks; c += 2) {
        ptx::tc_wait_ld();
        if (c + 1 < chunks) ptx::tc_ld_32x32b_x32(t_addr + (c + 1) * 32, r1); else release();
        store_chunk<INT32_OUT, HAS_ADDEND>(r0, args, sa_s + c * 32, tok0 + c * 32, ch, ch_ok, sw, bias);
        if (c + 1 < chunks) {
          ptx::tc_wait_ld();
          if (c + 2 < chunks) ptx::tc_ld_32x32b_x32(t_addr + (c + 2) * 32, r0); else release();
          store_chunk<INT32_OUT, HAS_ADDEND>(r1, args, sa_s + (c + 1) * 32, tok0 + (c + 1) * 32, ch, ch_ok, sw, bias);
        }
      }
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

#include "ss_gemm_pair.cuh"

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

struct DeviceInfo { int sms = 0; bool configured[5][2][2] = {}; bool pair_configured[4][6][2] = {}; };
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
  const double num_kb = static_cast<double>(pk / kBlockK);
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

// Token tile of the CTA-pair kernel (256 channels x NT tokens per pair): the candidate with the
// smallest rounds x cost-per-tile; ties go to the smaller tile.
int pick_pair_token_tile(int64_t m, int64_t pn, int64_t pk, int sms) {
  if (const char* env = std::getenv("SS_TOKEN_TILE")) {
    const int v = std::atoi(env);
    if (v == 128 || v == 192 || v == 224 || v == 256) return v;
  }
  const int64_t tiles_ch2 = (pn + 2 * kTileCh - 1) / (2 * kTileCh);
  const double num_kb = static_cast<double>(pk / kBlockK);
  const int64_t pairs = sms / 2 > 0 ? sms / 2 : 1;
  // Cost of one tile in cycles = blocks of 128 lifted columns x per-block cost + per-tile cost,
  // both fitted per token tile to measured kernel times (graph replay) over the benchmark shapes
  // (a long-K and a short-K shape each): 330 / 348 / 343 / 472 cycles per block and 2300 / 2650 /
  // 3400 / 4800 per tile for token tiles of 128 / 192 / 224 / 256 (256 has one pipeline stage less
  // and no metadata warp; the per-tile part is the epilogue tail and the barrier round trips).
  // Over the eleven shapes of the fit the model's choice costs 0.2 % more than the best tile.
  const int cand[4] = {128, 192, 224, 256};
  const double per_block[4] = {330.0, 348.0, 343.0, 472.0};
  const double per_tile[4] = {2300.0, 2650.0, 3400.0, 4800.0};
  double best = 0;
  int best_nt = 224;
  for (int i = 0; i < 4; ++i) {
    const int nt = cand[i];
    const int64_t tiles = tiles_ch2 * ((m + nt - 1) / nt);
    const int64_t rounds = (tiles + pairs - 1) / pairs;
    const double cost = static_cast<double>(rounds) * (num_kb * per_block[i] + per_tile[i]);
    if (best == 0 || cost < best * 0.999) { best = cost; best_nt = nt; }
  }
  return best_nt;
}

template <int NT, int KB, bool I32, bool ADD>
int launch_t(const GemmArgs& a, DeviceInfo* dev, int cfg_index, cudaStream_t stream) {
  using T = Tile<NT, KB>;
  auto kernel = sparse_gemm_kernel<NT, KB, I32, ADD>;
  if (!dev->configured[cfg_index][I32][ADD]) {
    SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes));
    dev->configured[cfg_index][I32][ADD] = true;
  }
  CUtensorMap map_a, map_b, map_e;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.pk / 2), static_cast<cuuint64_t>(a.pn)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.pk / 2)};
    const cuuint32_t box[2] = {kBlockK / 2 * KB, kTileCh};
    int rc = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.packed, dims, strides, box,
                    KB == 2 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
  }
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.pk), static_cast<cuuint64_t>(a.pm)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.pk)};
    const cuuint32_t box[2] = {kBlockK, NT};
    int rc = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    const cuuint64_t kblocks = static_cast<cuuint64_t>(a.pk / kBlockK);
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
  k.num_kb = static_cast<int>(a.pk / kBlockK);
  k.status = device_status_ptr();
  k.wide_cp = 0;
  k.meta_warp = 0;
  k.gate = nullptr; k.gate_stride = 0; k.rows_per_batch = 0;
  k.res_stages = 0;
  k.peer_count = 0;
  SS_REQUIRE(k.status, SS_E_CUDA, "device status word unavailable");
  const int64_t tiles = static_cast<int64_t>(k.tiles_ch) * k.tiles_tok;
  const unsigned grid = static_cast<unsigned>(tiles < dev->sms ? tiles : dev->sms);
  kernel<<<grid, kThreads, T::kSmemBytes, stream>>>(map_a, map_b, map_e, k);
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}

template <int NT, int KB>
int launch_nt(const GemmArgs& a, DeviceInfo* dev, int cfg_index, cudaStream_t stream) {
  if (a.int32_out) return launch_t<NT, KB, true, false>(a, dev, cfg_index, stream);
  if (a.addend) return launch_t<NT, KB, false, true>(a, dev, cfg_index, stream);
  return launch_t<NT, KB, false, false>(a, dev, cfg_index, stream);
}

// SS_PDL=0 switches the overlapped GEMM prologue off (plain stream order).
bool pdl_enabled() {
  const char* env = std::getenv("SS_PDL");
  return !(env && std::atoi(env) == 0);
}

// ---- CTA-pair launcher -----------------------------------------------------------------------
// RES: weights-resident form (see PairResident); res_stages = its activation pipeline depth.
template <int NT, int KB, int MODE, bool RES = false>
int launch_pair_t(const GemmArgs& a, DeviceInfo* dev, int cfg_index, cudaStream_t stream, int res_stages = 0) {
  using T = PairTile<NT, KB>;
  using Peers = std::conditional_t<MODE == kOutBf16TmaPeers, PeerMaps, NoPeers>;
  auto kernel = sparse_gemm_pair_kernel<NT, KB, MODE, RES, Peers>;
  if (!dev->pair_configured[cfg_index][MODE][RES]) {
    SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 RES ? 227 * 1024 : T::kSmemBytes));
    dev->pair_configured[cfg_index][MODE][RES] = true;
  }
  CUtensorMap map_a, map_b, map_e, map_out;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.pk / 2), static_cast<cuuint64_t>(a.pn)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.pk / 2)};
    const cuuint32_t box[2] = {kBlockK / 2 * KB, kTileCh};
    int rc = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.packed, dims, strides, box,
                    KB == 2 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
  }
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.pk), static_cast<cuuint64_t>(a.pm)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.pk)};
    const cuuint32_t box[2] = {kBlockK, T::kHalf};          // each CTA loads half of the token rows
    int rc = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.q, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    const cuuint64_t kblocks = static_cast<cuuint64_t>(a.pk / kBlockK);
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
  k.num_kb = static_cast<int>(a.pk / kBlockK);
  k.status = device_status_ptr();
  SS_REQUIRE(k.status, SS_E_CUDA, "device status word unavailable");
  k.gate = static_cast<const __nv_bfloat16*>(a.gate);
  k.gate_stride = a.gate_stride;
  k.rows_per_batch = static_cast<int>(a.rows_per_batch);
  { const char* env = std::getenv("SS_WIDE_CP"); k.wide_cp = env ? std::atoi(env) : 1; }
  { const char* env = std::getenv("SS_META_WARP"); k.meta_warp = env ? std::atoi(env) : (T::kStages >= 4 ? 1 : 0); }
  k.res_stages = res_stages;
  const int64_t tiles_ch2 = (k.tiles_ch + 1) / 2;
  const int64_t tiles = tiles_ch2 * k.tiles_tok;
  const int64_t pairs = dev->sms / 2;
  unsigned grid = 2u * static_cast<unsigned>(tiles < pairs ? tiles : pairs);
  int smem_bytes = T::kSmemBytes;
  if constexpr (RES) {
    // a whole number of clusters per channel tile, so that a cluster never changes its weights
    int64_t group = pairs / tiles_ch2;
    if (group > k.tiles_tok) group = k.tiles_tok;
    SS_REQUIRE(group >= 1 && res_stages >= 3, SS_E_ARG, "gemm: resident form not applicable");
    grid = 2u * static_cast<unsigned>(group * tiles_ch2);
    smem_bytes = PairResident<NT, KB>::smem_bytes((k.num_kb + KB - 1) / KB, res_stages);
  }
  if constexpr (MODE == kOutBf16Tma || MODE == kOutBf16GateAdd) {
    // out[m, n] BF16, row pitch out_stride: one 32-channel x 32-token box per epilogue warp and chunk
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.n), static_cast<cuuint64_t>(a.m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.out_stride) * 2};
    const cuuint32_t box[2] = {32, 32};
    // the epilogue writes its 64-byte rows with the 16-byte pieces XOR-swizzled (bank-conflict-free stmatrix)
    int rc = encode(&map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
  } else {
    map_out = map_a;       // unused by the direct-store epilogues
  }
  Peers peers{};
  if constexpr (MODE == kOutBf16TmaPeers) {
    SS_REQUIRE(a.peer_count >= 1 && a.peer_count <= kMaxPeers, SS_E_ARG, "gemm: 1..%d destinations", kMaxPeers);
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.n), static_cast<cuuint64_t>(a.m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.out_stride) * 2};
    const cuuint32_t box[2] = {32, 32};
    for (int g = 0; g < a.peer_count; ++g) {
      SS_REQUIRE(a.peer_out[g] && (reinterpret_cast<uintptr_t>(a.peer_out[g]) & 15) == 0, SS_E_ARG,
                 "gemm: destination %d must be a 16-byte aligned pointer", g);
      int rc = encode(&peers.m[g], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.peer_out[g]), dims, strides,
                      box, CU_TENSOR_MAP_SWIZZLE_64B);
      if (rc) return rc;
    }
    k.peer_count = a.peer_count;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.overlap_prologue && pdl_enabled() ? 1 : 0;
  SS_CUDA(cudaLaunchKernelEx(&cfg, kernel, map_a, map_b, map_e, map_out, k, peers));
  SS_CUDA(cudaGetLastError());
  return SS_OK;
}

// Weights-resident form: applicable when the K extent's metadata fits the TMEM columns left beside
// two accumulators and there are no more channel tiles than clusters; worth using (measured) only
// when at least four activation stages fit next to the weights (lifted K up to about 1300: with
// three the pipeline is too shallow, 6:8 at K = 1152 ran 30 % slower) and a cluster sees at least
// four token tiles (the weights are fetched before the first MMA; with two tiles that start-up
// costs more than the re-use saves).  Returns the activation pipeline depth, 0 if not applicable.
template <int NT>
int resident_stages(const GemmArgs& a, int sms) {
  using R = PairResident<NT, 2>;
  const int64_t num_kb = a.pk / kBlockK, slabs = (num_kb + 1) / 2;
  const int64_t tiles_ch2 = (a.pn + 2 * kTileCh - 1) / (2 * kTileCh), tiles_tok = (a.m + NT - 1) / NT;
  const int64_t pairs = sms / 2;
  if (slabs > R::kMaxStagesK || tiles_ch2 > pairs) return 0;
  const int stages = R::b_stages(static_cast<int>(slabs));
  if (stages < 4 || num_kb * R::T::kEBlock > static_cast<int64_t>(stages) * R::T::kBBytes) return 0;
  const int64_t group = pairs / tiles_ch2;
  if (tiles_tok < 4 * group) return 0;
  return stages;
}

template <int NT, int KB>
int launch_pair_nt(const GemmArgs& a, DeviceInfo* dev, int cfg_index, cudaStream_t stream, int res_stages = 0) {
  if (a.int32_out) return launch_pair_t<NT, KB, kOutInt32>(a, dev, cfg_index, stream);
  if (a.addend) return launch_pair_t<NT, KB, kOutBf16Addend>(a, dev, cfg_index, stream);
  if constexpr (KB == 2 && NT <= 224) {
    if (res_stages > 0) {
      const bool aligned = (reinterpret_cast<uintptr_t>(a.out) & 15) == 0 && a.out_stride % 8 == 0;
      if (aligned && a.gate) return launch_pair_t<NT, KB, kOutBf16GateAdd, true>(a, dev, cfg_index, stream, res_stages);
      if (aligned) return launch_pair_t<NT, KB, kOutBf16Tma, true>(a, dev, cfg_index, stream, res_stages);
    }
  }
  // TMA stores need a 16-byte aligned base and row pitch
  const bool tma_ok = (reinterpret_cast<uintptr_t>(a.out) & 15) == 0 && a.out_stride % 8 == 0;
  if (a.gate) {
    SS_REQUIRE(tma_ok, SS_E_ARG, "gated accumulation needs a 16-byte aligned output and row pitch");
    return launch_pair_t<NT, KB, kOutBf16GateAdd>(a, dev, cfg_index, stream);
  }
  if (a.peer_count > 0) {
    SS_REQUIRE(a.out_stride % 8 == 0, SS_E_ARG, "tensor-parallel stores need a row pitch that is a multiple of 8");
    return launch_pair_t<NT, KB, kOutBf16TmaPeers>(a, dev, cfg_index, stream);
  }
  const char* env = std::getenv("SS_STORE");          // 0 direct stores, 1 TMA stores (default)
  const int store = env ? std::atoi(env) : 1;
  if (tma_ok && store == 1) return launch_pair_t<NT, KB, kOutBf16Tma>(a, dev, cfg_index, stream);
  return launch_pair_t<NT, KB, kOutBf16>(a, dev, cfg_index, stream);
}

// Blocks of 128 lifted columns per pipeline stage: 2 wherever at least 3 stages still fit.
int stage_blocks(int nt) {
  if (nt != 256) return 2;
  const char* env = std::getenv("SS_STAGE_BLOCKS");
  return env && std::atoi(env) == 2 ? 2 : 1;
}

int check_args(const GemmArgs& a) {
  SS_REQUIRE(a.q && a.packed && a.meta && (a.out || a.peer_count > 0), SS_E_ARG, "gemm: null pointer");
  SS_REQUIRE(a.peer_count == 0 || (!a.int32_out && !a.addend && !a.gate), SS_E_ARG,
             "gemm: the tensor-parallel form excludes addend, gate and the INT32 dump");
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
  if (a.gate) {
    SS_REQUIRE(!a.int32_out && !a.addend, SS_E_ARG, "gemm: gated accumulation excludes the addend and the INT32 dump");
    SS_REQUIRE(a.rows_per_batch > 0 && a.rows_per_batch % 32 == 0 && a.rows_per_batch < (1ll << 31), SS_E_ARG,
               "gemm: gated accumulation needs rows_per_batch to be a positive multiple of 32 (got %lld)",
               (long long)a.rows_per_batch);
    SS_REQUIRE(a.gate_stride >= a.n, SS_E_ARG, "gemm: gate row stride smaller than n");
  }
  return SS_OK;
}

}  // namespace

int launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (int rc = check_args(a)) return rc;
  DeviceInfo* dev = device_info();
  SS_REQUIRE(dev, SS_E_CUDA, "gemm: no current CUDA device");
  // The CTA-pair kernel is the default; SS_PAIR=0 selects the single-CTA kernel (kept for
  // comparison and for token tiles of 64).
  const char* pair_env = std::getenv("SS_PAIR");
  if (!pair_env || std::atoi(pair_env) != 0) {
    // SS_RESIDENT=0 switches the weights-resident form off
    const char* res_env = std::getenv("SS_RESIDENT");
    const bool token_tile_forced = std::getenv("SS_TOKEN_TILE") != nullptr;
    if (!(res_env && std::atoi(res_env) == 0) && !a.int32_out && !a.addend && a.peer_count == 0 && !token_tile_forced) {
      // prefer the token tile that needs fewer rounds of the clusters that share a channel tile
      const int s224 = resident_stages<224>(a, dev->sms), s192 = resident_stages<192>(a, dev->sms);
      const int64_t tiles_ch2 = (a.pn + 2 * kTileCh - 1) / (2 * kTileCh), group = (dev->sms / 2) / (tiles_ch2 ? tiles_ch2 : 1);
      auto rounds = [&](int nt) { const int64_t t = (a.m + nt - 1) / nt; return (t + group - 1) / group; };
      if (s224 && (!s192 || rounds(224) * 224 <= rounds(192) * 192)) return launch_pair_nt<224, 2>(a, dev, 2, stream, s224);
      if (s192) return launch_pair_nt<192, 2>(a, dev, 1, stream, s192);
    }
    switch (pick_pair_token_tile(a.m, a.pn, a.pk, dev->sms)) {
      case 128: return launch_pair_nt<128, 2>(a, dev, 0, stream);
      case 192: return launch_pair_nt<192, 2>(a, dev, 1, stream);
      case 224: return launch_pair_nt<224, 2>(a, dev, 2, stream);
      default:  return launch_pair_nt<256, 2>(a, dev, 3, stream);
    }
  }
  SS_REQUIRE(!a.gate && a.peer_count == 0, SS_E_ARG,
             "gemm: gated accumulation and the tensor-parallel form are implemented by the CTA-pair kernel only");
  const int nt = pick_token_tile(a.m, a.pn, a.pk, dev->sms);
  switch (nt) {
    case 256: return stage_blocks(nt) == 2 ? launch_nt<256, 2>(a, dev, 4, stream) : launch_nt<256, 1>(a, dev, 0, stream);
    case 192: return launch_nt<192, 2>(a, dev, 1, stream);
    case 128: return launch_nt<128, 2>(a, dev, 2, stream);
    default:  return launch_nt<64, 2>(a, dev, 3, stream);
  }
}

template <int NT, int KB>
static int resources_t(GemmResources* r) {
  using T = Tile<NT, KB>;
  auto kernel = sparse_gemm_kernel<NT, KB, false, false>;
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

template <int NT, int KB>
static int pair_resources_t(GemmResources* r) {
  using T = PairTile<NT, KB>;
  auto kernel = sparse_gemm_pair_kernel<NT, KB, kOutBf16Tma>;
  cudaFuncAttributes attr;
  SS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes));
  SS_CUDA(cudaFuncGetAttributes(&attr, kernel));
  r->threads = kPairThreads; r->smem = T::kSmemBytes; r->regs = attr.numRegs;
  r->local = static_cast<int>(attr.localSizeBytes); r->ctas_per_sm = 1;
  r->token_tile = NT; r->stages = T::kStages; r->tmem_cols = kTmemCols;
  return SS_OK;
}

int gemm_resources(int64_t m, int64_t n, int64_t pk, GemmResources* r) {
  DeviceInfo* dev = device_info();
  SS_REQUIRE(dev, SS_E_CUDA, "gemm: no current CUDA device");
  const char* pair_env = std::getenv("SS_PAIR");
  if (!pair_env || std::atoi(pair_env) != 0) {
    switch (pick_pair_token_tile(m, ceil_to(n, 32), pk, dev->sms)) {
      case 128: return pair_resources_t<128, 2>(r);
      case 192: return pair_resources_t<192, 2>(r);
      case 224: return pair_resources_t<224, 2>(r);
      default:  return pair_resources_t<256, 2>(r);
    }
  }
  const int nt = pick_token_tile(m, ceil_to(n, 32), pk, dev->sms);
  switch (nt) {
    case 256: return stage_blocks(nt) == 2 ? resources_t<256, 2>(r) : resources_t<256, 1>(r);
    case 192: return resources_t<192, 2>(r);
    case 128: return resources_t<128, 2>(r);
    default:  return resources_t<64, 2>(r);
  }
}

}  // namespace ss
